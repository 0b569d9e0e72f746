"""Who is served first: classes of service with aging, and weighted shares for tenants.

The rules are the reference's (src/dli/engine/scheduler.py:218-242); they live in one object that
the scheduler consults, so that the batching loop does not know how the order comes about.

* Class.  INTERACTIVE before BATCH.  A request that has been in the system for ``aging_steps``
  scheduling steps is treated as INTERACTIVE whatever it was submitted as, which bounds how long
  BATCH work can sit behind a steady interactive stream.
* Among running requests: class, then arrival.  Preemption takes its victims from the far end
  of that order, so the request at its front always makes progress.
* Among waiting requests: class; then a request that was preempted (it already held pages once)
  before one that never ran; then the tenant whose virtual clock is furthest behind; then arrival.
* Virtual clocks (weighted fair queuing).  A tenant's clock advances by tokens / weight for every
  token scheduled for it, so a tenant of weight 2 is given about twice the tokens of a tenant of
  weight 1 while both have work.  A tenant that arrives (again) is set to the smallest clock among
  the tenants that have work: an idle spell earns no credit to spend later.
"""

from __future__ import annotations

from collections.abc import Iterable, Mapping

from .request import Priority, Request


class ServiceOrder:
    def __init__(self, tenant_weights: Mapping[str, float] | None = None, aging_steps: int = 200) -> None:
        self.weights = dict(tenant_weights or {})
        self.aging_steps = aging_steps
        self.steps = 0  # scheduling steps so far; ages are differences of this count
        self._clocks: dict[str, float] = {}

    # ---- time

    def tick(self) -> None:
        """One more step has been decided."""
        self.steps += 1

    def service_class(self, req: Request) -> int:
        """The request's class after aging (0 is served first)."""
        aged = self.steps - req.arrival_step >= self.aging_steps
        return int(Priority.INTERACTIVE) if aged else int(req.priority)

    # ---- sort keys

    def running_key(self, req: Request) -> tuple[int, int]:
        return self.service_class(req), req.arrival

    def admission_key(self, req: Request) -> tuple[int, int, float, int]:
        never_ran = 0 if req.num_preemptions else 1
        return self.service_class(req), never_ran, self.clock(req.tenant), req.arrival

    # ---- tenants

    def clock(self, tenant: str) -> float:
        return self._clocks.get(tenant, 0.0)

    def charge(self, tenant: str, tokens: int) -> None:
        self._clocks[tenant] = self.clock(tenant) + tokens / self.weights.get(tenant, 1.0)

    def arrive(self, tenant: str, tenants_with_work: Iterable[str]) -> None:
        """``tenant`` submits a request; ``tenants_with_work`` are those with requests waiting or running."""
        floor = min((self.clock(t) for t in set(tenants_with_work) - {tenant}), default=0.0)
        self._clocks[tenant] = max(self.clock(tenant), floor)
