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


class Sampler:
    RING = 4  # output buffers in turn: ids of a step stay readable while the next steps are launched

    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)
        self._out: torch.Tensor | None = None
        self._ring: list[tuple[torch.Tensor, torch.Tensor]] = []
        self._turn = 0

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int], draws: Sequence[int]) -> PendingTokens:
        """As ``sample``, without waiting: the ids stay on the device and travel to pinned host memory
        behind the kernels already launched."""
        rows = logits.shape[0]
        if not self._ring or self._ring[0][0].numel() < rows:
            size = max(rows, 256)
            self._ring = [(torch.empty(size, dtype=torch.int32, device=self.device), torch.empty(size, dtype=torch.int32).pin_memory())
                          for _ in range(self.RING)]
        dev, host = self._ring[self._turn]
        self._turn = (self._turn + 1) % self.RING
        self._launch(dev[:rows], logits, params, seeds, draws)
        host[:rows].copy_(dev[:rows], non_blocking=True)
        copied = torch.cuda.Event()
        copied.record()
        return PendingTokens(dev[:rows], host[:rows], copied)

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
