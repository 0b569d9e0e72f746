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
"""

from __future__ import annotations

from collections import deque
from collections.abc import Mapping
from dataclasses import dataclass, field

from ..cache import CacheManager, OutOfPages
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

    @property
    def num_batched_tokens(self) -> int:
        return sum(c.num_tokens for c in self.chunks)


class Scheduler:
    def __init__(self, config: SchedulerConfig, manager: CacheManager) -> None:
        self.config = config
        self.manager = manager
        self.order = ServiceOrder(config.tenant_weights, config.aging_steps)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
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
        out = SchedulerOutput()
        left = self._serve_running(out, self.config.max_num_batched_tokens)
        if not out.preempted:  # a step that had to take pages away gives none out
            self._admit_waiting(out, left)
        self.order.tick()
        return out

    def step_launched_ahead(self, reqs) -> None:
        """A decode step of ``reqs`` that the engine launched without asking ``schedule``: it
        counts as a step and its tokens are charged, as if it had been scheduled."""
        for req in reqs:
            self.order.charge(req.tenant, 1)
        self.order.tick()

    def _serve_running(self, out: SchedulerOutput, budget: int) -> int:
        """Every running request's next token or next portion, in service order; returns the budget left."""
        in_batch: set[str] = set()
        self.running.sort(key=self.order.running_key)
        for req in list(self.running):
            if budget == 0:
                break
            if req.status is not RequestStatus.RUNNING:
                continue  # taken as a victim earlier in this loop
            total = len(req.prompt_ids) + len(req.output_ids)
            n = min(total - req.num_computed_tokens, budget)
            if n <= 0:
                continue
            while not self._reserve(req, total, out):
                victim = next((c for c in reversed(self.running) if c.request_id not in in_batch and c is not req), None)
                if victim is None:
                    victim = req  # nobody else can yield
                self._preempt(victim)
                out.preempted.append(victim)
                if victim is req:
                    break
            if req.status is not RequestStatus.RUNNING:
                continue
            start = req.num_computed_tokens
            out.chunks.append(ScheduledChunk(req, start, n, start + n == total))
            in_batch.add(req.request_id)
            self.order.charge(req.tenant, n)
            budget -= n
        return budget

    def _admit_waiting(self, out: SchedulerOutput, budget: int) -> None:
        """Waiting requests, the most deserving first, while budget, request cap and pages allow."""
        while self.waiting and budget > 0 and len(self.running) < self.config.max_num_seqs:
            req = min(self.waiting, key=self.order.admission_key)
            tokens = req.all_token_ids
            # The pages held back by the watermark are room for running requests to grow into.
            # With nobody running there is nobody to keep them for, and a request that needs
            # them would otherwise wait for ever (it passed the capacity check, so it fits alone).
            hold_back = bool(self.running)
            if not self.manager.can_allocate(tokens, self.config.namespace, hold_back):
                break  # the head of the queue waits for memory; nobody jumps past it
            alloc = self.manager.allocate(req.request_id, tokens, namespace=self.config.namespace, respect_watermark=hold_back)
            self.waiting.remove(req)
            req.status = RequestStatus.RUNNING
            req.num_computed_tokens = alloc.num_cached_tokens
            self.running.append(req)
            out.admitted.append(req)
            n = min(len(tokens) - alloc.num_cached_tokens, budget)
            out.chunks.append(ScheduledChunk(req, req.num_computed_tokens, n, req.num_computed_tokens + n == len(tokens)))
            self.order.charge(req.tenant, n)
            budget -= n

    # ------------------------------------------------------------ internals

    def _reserve(self, req: Request, total: int, out: SchedulerOutput) -> bool:
        """Slots for tokens the cache manager has not seen yet (the newly sampled one)."""
        missing = total - self.manager.num_tokens(req.request_id)
        if missing <= 0:
            return True
        try:
            out.copies.extend(self.manager.append_slots(req.request_id, req.token_slice(total - missing, total)) or ())
            return True
        except OutOfPages:
            return False

    def _preempt(self, req: Request) -> None:
        self.manager.free(req.request_id)
        self.running.remove(req)
        req.status = RequestStatus.WAITING
        req.num_computed_tokens = 0
        req.num_preemptions += 1
        self.waiting.appendleft(req)
