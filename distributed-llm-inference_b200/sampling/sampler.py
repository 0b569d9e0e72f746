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


class Sampler:
    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)
        self._out: torch.Tensor | None = None

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
        if all(p.greedy for p in params):
            ops.sample(out, logits)
            return out.tolist()
        f = torch.tensor([[p.temperature if not p.greedy else 0.0, p.top_p] for p in params], dtype=torch.float32).pin_memory()
        k = torch.tensor([p.top_k for p in params], dtype=torch.int32).pin_memory()
        sd = torch.tensor([[s & 0x7FFFFFFFFFFFFFFF, d] for s, d in zip(seeds, draws)], dtype=torch.int64).pin_memory()
        f, k, sd = (t.to(self.device, non_blocking=True) for t in (f, k, sd))
        ops.sample(out, logits, f[:, 0].contiguous(), k, f[:, 1].contiguous(), sd[:, 0].contiguous(), sd[:, 1].contiguous())
        return out.tolist()
