"""One token per logits row, on the device.

A request's random stream is a counter-based generator keyed by its seed; the
draw for its i-th generated token uses counter i.  So the numbers a request
sees depend only on its seed and on how many tokens it has generated, never on
its neighbours in the batch, on preemption or on recomputation
(src/dli/sampling.py:3-7 reaches the same with one torch.Generator per request).
"""

from __future__ import annotations

from typing import Sequence

import torch

from ..kernels import ops
from .params import SamplingParams


class PendingTokens:
    """Token ids that a step sampled: on the device at once (``device_ids``, int32, for a step that is
    launched before the host reads them), on the host after ``result()`` (which waits for the copy)."""

    def __init__(self, device_ids: torch.Tensor, host_ids: torch.Tensor, copied: torch.cuda.Event) -> None:
        self.device_ids, self._host, self._copied = device_ids, host_ids, copied
        self._list: list[int] | None = None

    def result(self) -> list[int]:
        if self._list is None:
            self._copied.synchronize()
            self._list = self._host.tolist()
        return self._list


class SamplerState:
    """The sampler's share of a request's state slot, on the device: for every slot the request's temperature,
    top-k, top-p, seed and the number of draws it has made.  A request's values are written once, when it is
    given its slot (``bind``: one small copy from pinned memory; a request that comes back after a preemption is
    bound again, with the number of tokens it has generated as its draw count, so its stream goes on where it
    stopped).  The sampling kernel reads a row's values by its slot and advances the draw count itself, so a
    step passes only the slots of its rows.  Greedy requests are bound too (temperature 0): a slot never keeps
    the values of the request that held it before."""

    def __init__(self, max_requests: int, device: torch.device) -> None:
        self.size = max_requests
        self.temperature = torch.zeros(max_requests, dtype=torch.float32, device=device)
        self.top_p = torch.ones(max_requests, dtype=torch.float32, device=device)
        self.top_k = torch.full((max_requests,), -1, dtype=torch.int32, device=device)
        self.seed = torch.zeros(max_requests, dtype=torch.int64, device=device)
        self.draws = torch.zeros(max_requests, dtype=torch.int64, device=device)
        # pinned staging for one step's admissions: [slot, top_k] int32, [temperature, top_p] float32, [seed, draws] int64
        self._i = torch.empty((max_requests, 2), dtype=torch.int32).pin_memory()
        self._f = torch.empty((max_requests, 2), dtype=torch.float32).pin_memory()
        self._l = torch.empty((max_requests, 2), dtype=torch.int64).pin_memory()
        self._staged = 0
        self._copied: torch.cuda.Event | None = None
        self.binds = 0

    def bind(self, slot: int, params: SamplingParams, seed: int, draws: int) -> None:
        """Stage a request's values for its slot; they reach the device with the next ``flush``."""
        if not 0 <= slot < self.size:
            raise ValueError(f"state slot {slot} outside [0, {self.size})")
        if self._staged == self.size:
            self.flush()
        if self._staged == 0 and self._copied is not None:
            self._copied.synchronize()  # the staging buffers are free again once the last copy has read them
        n = self._staged
        self._i[n, 0], self._i[n, 1] = slot, params.top_k
        self._f[n, 0], self._f[n, 1] = (0.0 if params.greedy else params.temperature), params.top_p
        self._l[n, 0], self._l[n, 1] = seed & 0x7FFFFFFFFFFFFFFF, draws
        self._staged = n + 1
        self.binds += 1

    def flush(self) -> None:
        """Write what was staged into the tables (behind the kernels already launched on the stream)."""
        n = self._staged
        if n == 0:
            return
        dev = self.temperature.device
        i, f, l = (t[:n].to(dev, non_blocking=True) for t in (self._i, self._f, self._l))
        self._copied = torch.cuda.Event()
        self._copied.record()
        at = i[:, 0].long()
        self.top_k.index_copy_(0, at, i[:, 1].contiguous())
        self.temperature.index_copy_(0, at, f[:, 0].contiguous())
        self.top_p.index_copy_(0, at, f[:, 1].contiguous())
        self.seed.index_copy_(0, at, l[:, 0].contiguous())
        self.draws.index_copy_(0, at, l[:, 1].contiguous())
        self._staged = 0


class Sampler:
    RING = 4  # output buffers in turn: ids of a step stay readable while the next steps are launched

    def __init__(self, device: torch.device | str, max_requests: int = 0) -> None:
        self.device = torch.device(device)
        self._out: torch.Tensor | None = None
        self._ring: list[tuple[torch.Tensor, torch.Tensor]] = []
        self._turn = 0
        # with a slot table (an engine gives its number of state slots) requests are bound to slots and sampled by slot
        self.state = SamplerState(max_requests, self.device) if max_requests > 0 else None
        self._slot_ring: list[tuple[torch.Tensor, torch.Tensor, torch.cuda.Event | None]] = []
        self._slot_turn = 0

    # ---- by state slot (the engine's way)

    def bind(self, slot: int, params: SamplingParams, seed: int, draws: int) -> None:
        """A request was given state slot ``slot``: its parameters, its seed and the draws it has made so far."""
        if self.state is None:
            raise ValueError("this sampler was built without a slot table")
        self.state.bind(slot, params, seed, draws)

    def sample_slots_async(self, logits: torch.Tensor, slots: Sequence[int], all_greedy: bool) -> PendingTokens:
        """One token per row for the requests bound to ``slots`` (one per row): parameters, seed and draw count are
        read from the slot table on the device, and the kernel advances the draw count of every stochastic row.
        ``all_greedy``: the caller knows that every row is an argmax (nothing is read from the table then)."""
        rows = logits.shape[0]
        if self.state is None or len(slots) != rows or rows == 0:
            raise ValueError("one bound slot per row (at least one row)")
        self.state.flush()
        dev, host, copied = self._output(rows)
        if all_greedy:
            ops.sample(dev, logits)
        else:
            if not self._slot_ring:
                self._slot_ring = [(torch.empty(max(256, self.state.size), dtype=torch.int32, device=self.device),
                                    torch.empty(max(256, self.state.size), dtype=torch.int32).pin_memory(), None) for _ in range(self.RING)]
            d_slots, h_slots, busy = self._slot_ring[self._slot_turn]
            if rows > h_slots.numel():
                raise ValueError(f"{rows} rows, but the slot table has {self.state.size} slots")
            if busy is not None:
                busy.synchronize()
            h_slots[:rows] = torch.as_tensor(list(slots), dtype=torch.int32)
            d_slots[:rows].copy_(h_slots[:rows], non_blocking=True)
            done = torch.cuda.Event()
            done.record()
            self._slot_ring[self._slot_turn] = (d_slots, h_slots, done)
            self._slot_turn = (self._slot_turn + 1) % self.RING
            st = self.state
            ops.sample(dev, logits, st.temperature, st.top_k, st.top_p, st.seed, st.draws, slots=d_slots[:rows])
        host.copy_(dev, non_blocking=True)
        copied.record()
        return PendingTokens(dev, host, copied)

    def _output(self, rows: int):
        if not self._ring or self._ring[0][0].numel() < rows:
            size = max(rows, 256)
            self._ring = [(torch.empty(size, dtype=torch.int32, device=self.device), torch.empty(size, dtype=torch.int32).pin_memory())
                          for _ in range(self.RING)]
        dev, host = self._ring[self._turn]
        self._turn = (self._turn + 1) % self.RING
        return dev[:rows], host[:rows], torch.cuda.Event()

    # ---- with explicit values per row

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int], draws: Sequence[int]) -> PendingTokens:
        """As ``sample``, without waiting: the ids stay on the device and travel to pinned host memory
        behind the kernels already launched."""
        dev, host, copied = self._output(logits.shape[0])
        self._launch(dev, logits, params, seeds, draws)
        host.copy_(dev, non_blocking=True)
        copied.record()
        return PendingTokens(dev, host, copied)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int], draws: Sequence[int]) -> list[int]:
        """logits [rows, vocab] float32 on the device; seeds[r] and draws[r] identify the
        row's draw.  Returns one token id per row (one device-to-host read)."""
        rows = logits.shape[0]
        if not (len(params) == len(seeds) == len(draws) == rows):
            raise ValueError("logits, params, seeds and draws must have one entry per row")
        if rows == 0:
            return []
        if self._out is None or self._out.numel() < rows:
            self._out = torch.empty(max(rows, 256), dtype=torch.int32, device=self.device)
        out = self._out[:rows]
        self._launch(out, logits, params, seeds, draws)
        return out.tolist()

    def _launch(self, out: torch.Tensor, logits: torch.Tensor, params, seeds, draws) -> None:
        rows = logits.shape[0]
        if not (len(params) == len(seeds) == len(draws) == rows) or rows == 0:
            raise ValueError("logits, params, seeds and draws must have one entry per row (at least one)")
        if all(p.greedy for p in params):
            ops.sample(out, logits)
            return
        f = torch.tensor([[p.temperature if not p.greedy else 0.0, p.top_p] for p in params], dtype=torch.float32).pin_memory()
        k = torch.tensor([p.top_k for p in params], dtype=torch.int32).pin_memory()
        sd = torch.tensor([[s & 0x7FFFFFFFFFFFFFFF, d] for s, d in zip(seeds, draws)], dtype=torch.int64).pin_memory()
        f, k, sd = (t.to(self.device, non_blocking=True) for t in (f, k, sd))
        ops.sample(out, logits, f[:, 0].contiguous(), k, f[:, 1].contiguous(), sd[:, 0].contiguous(), sd[:, 1].contiguous())
