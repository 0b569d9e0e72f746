"""Continuous batching with chunked prefill under a token budget.

Each step: requests that already run come first, oldest first — each gets its
next decoded token or the next portion of its prompt, cut to the budget that is
left; then waiting requests are admitted in order while the budget, the request
cap and the cache allow.  (src/dli/engine/scheduler.py:151-214.)

When pages run out: the request that needs a page takes it from the *newest*
running request not yet in this step's batch, which is preempted by recompute —
its pages are freed, its tokens are kept, and it goes to the front of the
waiting queue; when it is admitted again, prompt and generated tokens are run
as a prompt, without sampling, up to the last known token.  If nobody else can
yield, the requester itself is preempted.  A step that preempted admits nobody.
A request whose prompt plus ``max_tokens`` can never fit in the pool is finished
at once with reason ``capacity``, so the oldest running request can always
finish and the engine cannot livelock.  (src/dli/engine/scheduler.py:102-120,255-267.)
One case the reference leaves open is closed here: a request that fits the pool but
not the pool less its watermark is admitted when nobody runs (the reference would
keep it waiting for ever).

Who is served first among equals in need (classes of service with aging, tenants'
weighted shares) is decided by ``ordering.ServiceOrder``.

The scheduler is the only place that decides what a step holds.  That includes the step the
engine launches *ahead* (``schedule_ahead``): the decode step behind one whose sampled ids are
still on the device.  It is offered only when there is nothing to decide — every running request
decodes, nobody waits, pages are there — and is counted and charged like any other step.
"""

from __future__ import annotations

from collections import deque
from collections.abc import Mapping
from dataclasses import dataclass, field

from ..cache import UNKNOWN_TOKEN, CacheManager, OutOfPages
from .ordering import ServiceOrder
from .request import FinishReason, Request, RequestStatus


@dataclass(frozen=True)
class SchedulerConfig:
    max_num_seqs: int = 64  # requests holding pages at once
    max_num_batched_tokens: int = 512  # tokens per step, prompt portions and decoded tokens together
    namespace: bytes = b""  # scope of prefix reuse (identity of model and weights)
    tenant_weights: Mapping[str, float] = field(default_factory=dict)  # share of a tenant (default 1.0): weight 2 gets about twice the tokens
    aging_steps: int = 200  # a request this many steps in the system counts as INTERACTIVE

    def __post_init__(self) -> None:
        if self.max_num_seqs < 1 or self.max_num_batched_tokens < 1:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be >= 1")
        if self.aging_steps < 1:
            raise ValueError("aging_steps must be >= 1")
        if any(not w > 0 for w in self.tenant_weights.values()):
            raise ValueError("tenant weights must be positive")


@dataclass(frozen=True)
class ScheduledChunk:
    """Run ``num_tokens`` tokens of ``request`` from position ``start``; ``needs_logits`` when
    the chunk reaches the request's last known token, so a new one is sampled."""

    request: Request
    start: int
    num_tokens: int
    needs_logits: bool


@dataclass
class SchedulerOutput:
    chunks: list[ScheduledChunk] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)
    admitted: list[Request] = field(default_factory=list)
    copies: list = field(default_factory=list)  # cache.PageCopy: to carry out before the step runs
    # of a step planned ahead only: for each chunk the row of the step in flight whose sampled id is its token,
    # and request -> position that was given a slot without an id (the engine names it once the id is read)
    token_rows: list[int] | None = None
    unknown: dict[str, int] = field(default_factory=dict)

    @property
    def num_batched_tokens(self) -> int:
        return sum(c.num_tokens for c in self.chunks)


@dataclass
class _Step:
    """A step while it is put together: what has been decided, the tokens still to give out, who is in."""

    out: SchedulerOutput
    budget: int
    served: set[str] = field(default_factory=set)

    def give(self, req: Request, n: int) -> None:
        """``req`` runs its next ``n`` tokens in this step."""
        start = req.num_computed_tokens
        self.out.chunks.append(ScheduledChunk(req, start, n, start + n == req.num_tokens))
        self.served.add(req.request_id)
        self.budget -= n


class Scheduler:
    def __init__(self, config: SchedulerConfig, manager: CacheManager) -> None:
        self.config = config
        self.manager = manager
        self.order = ServiceOrder(config.tenant_weights, config.aging_steps)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []  # kept in service order by every schedule()
        self._known: dict[str, Request] = {}

    # ------------------------------------------------------------ life of a request

    def add(self, req: Request) -> bool:
        """Queue a request; False (finished with ``capacity``) if it could never fit."""
        if req.request_id in self._known:
            raise ValueError(f"duplicate request id {req.request_id!r}")
        if not self.manager.fits_at_all(len(req.prompt_ids) + req.params.max_tokens):
            req.status, req.finish_reason = RequestStatus.FINISHED, FinishReason.CAPACITY
            return False
        self._known[req.request_id] = req
        req.arrival_step = self.order.steps
        self.order.arrive(req.tenant, (r.tenant for r in (*self.waiting, *self.running)))
        self.waiting.append(req)
        return True

    def finish(self, req: Request, reason: FinishReason) -> None:
        if req.status is RequestStatus.RUNNING:
            self.manager.free(req.request_id)
            self.running.remove(req)
        elif req.status is RequestStatus.WAITING:
            self.waiting.remove(req)
        req.status, req.finish_reason = RequestStatus.FINISHED, reason
        self._known.pop(req.request_id, None)

    def abort(self, request_id: str) -> Request | None:
        """Cancel a waiting or running request; None for unknown or finished ids."""
        req = self._known.get(request_id)
        if req is not None:
            self.finish(req, FinishReason.ABORTED)
        return req

    @property
    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    @property
    def num_steps(self) -> int:
        return self.order.steps

    def tenant_clock(self, tenant: str) -> float:
        return self.order.clock(tenant)

    # ------------------------------------------------------------ one step's batch

    def schedule(self) -> SchedulerOutput:
        """Decide the next step from what the host knows (every sampled id has been read)."""
        step = _Step(SchedulerOutput(), self.config.max_num_batched_tokens)
        self.running.sort(key=self.order.running_key)
        for req in tuple(self.running):
            if step.budget == 0:
                break
            # (a request earlier in this loop may have taken this one's pages: it waits again)
            if req.status is RequestStatus.RUNNING and req.num_tokens > req.num_computed_tokens:
                self._continue(req, step)
        if not step.out.preempted:  # a step that had to take pages away gives none out
            self._admit(step)
        self.order.tick()
        return step.out

    def schedule_ahead(self, in_flight: list[Request]) -> SchedulerOutput:
        """The decode step behind a step that is still running.  ``in_flight``: the requests that step samples
        a token for, in the order of its sampled rows; their ids are on the device, so each request's next
        token is named by its row.  The plan has chunks only if there is nothing to decide first: nobody
        waits, every running request is among those sampling (no prompt in portions, nobody aborted), and
        every request that goes on gets its slot.  A request that ends by length with the token in flight is
        left out.  Slots taken for tokens without an id are reported in ``unknown`` whether or not the step
        comes about (they are kept, and named when the ids arrive); so are page copies."""
        plan = SchedulerOutput(token_rows=[])
        if self.waiting or not in_flight or len(in_flight) != len(self.running):
            return plan
        going_on = [(row, r) for row, r in enumerate(in_flight)
                    if not r.is_finished and len(r.output_ids) + 1 < r.params.max_tokens]  # the others end with the token in flight
        if not going_on or len(going_on) > self.config.max_num_batched_tokens:
            return plan
        try:
            for _, req in going_on:
                position = req.num_tokens  # of the token in flight
                if self.manager.num_tokens(req.request_id) <= position:
                    plan.copies.extend(self.manager.append_slots(req.request_id, [UNKNOWN_TOKEN]) or ())
                    plan.unknown[req.request_id] = position
        except OutOfPages:
            return plan  # schedule() will decide who yields
        for row, req in going_on:
            plan.chunks.append(ScheduledChunk(req, req.num_computed_tokens, 1, True))
            plan.token_rows.append(row)
            self.order.charge(req.tenant, 1)
        self.order.tick()
        return plan

    # ------------------------------------------------------------ internals

    def _continue(self, req: Request, step: _Step) -> None:
        """A running request's next token, or the next portion of its prompt cut to the budget.  Pages it lacks
        are taken from whoever ``_who_yields`` names, one request at a time, until its slots are there (or it
        has given up its own)."""
        while not self._has_slots(req, step.out):
            victim = self._who_yields(req, step.served)
            self._send_back(victim)
            step.out.preempted.append(victim)
            if victim is req:
                return
        n = min(req.num_tokens - req.num_computed_tokens, step.budget)
        step.give(req, n)
        self.order.charge(req.tenant, n)

    def _who_yields(self, needy: Request, served: set[str]) -> Request:
        """The last request in service order that is not yet in the step's batch; the needy one itself if there is none."""
        for c in reversed(self.running):
            if c is not needy and c.request_id not in served:
                return c
        return needy

    def _admit(self, step: _Step) -> None:
        """Waiting requests, the most deserving first, while budget, request cap and pages allow."""
        while self.waiting and step.budget > 0 and len(self.running) < self.config.max_num_seqs:
            req = min(self.waiting, key=self.order.admission_key)
            tokens = req.all_token_ids
            # The pages held back by the watermark are room for running requests to grow into.
            # With nobody running there is nobody to keep them for, and a request that needs
            # them would otherwise wait for ever (it passed the capacity check, so it fits alone).
            hold_back = bool(self.running)
            if not self.manager.can_allocate(tokens, self.config.namespace, hold_back):
                return  # the head of the queue waits for memory; nobody jumps past it
            found = self.manager.allocate(req.request_id, tokens, namespace=self.config.namespace, respect_watermark=hold_back)
            self.waiting.remove(req)
            self.running.append(req)
            req.status, req.num_computed_tokens = RequestStatus.RUNNING, found.num_cached_tokens
            step.out.admitted.append(req)
            n = min(len(tokens) - found.num_cached_tokens, step.budget)
            step.give(req, n)
            self.order.charge(req.tenant, n)

    def _has_slots(self, req: Request, out: SchedulerOutput) -> bool:
        """Make sure every token the request knows has a slot (the newly sampled one may not); False if pages ran out."""
        have = self.manager.num_tokens(req.request_id)
        if have >= req.num_tokens:
            return True
        try:
            out.copies.extend(self.manager.append_slots(req.request_id, req.token_slice(have, req.num_tokens)) or ())
        except OutOfPages:
            return False
        return True

    def _send_back(self, req: Request) -> None:
        """Preemption by recompute: the pages go, the tokens stay, the request is first in the queue again."""
        self.manager.free(req.request_id)
        self.running.remove(req)
        self.waiting.appendleft(req)
        req.status, req.num_computed_tokens = RequestStatus.WAITING, 0
        req.num_preemptions += 1
