"""Per-request generation settings.

This class is the reference's API schema restated: the same seven fields with the same defaults, the same
four checks with the same messages, and the same ``greedy`` property as ``SamplingParams`` in
src/dli/sampling.py:22-56, so that code written against the reference's engine passes its parameters
unchanged.  Nothing here is this engine's own design; what the engine does with the fields is
(``sampling/sampler.py``, ``csrc/sampling.cu``)."""

from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    """max_tokens: most generated tokens.  temperature: 0 selects argmax (lowest id on ties).
    top_k: keep the k most likely tokens, -1 disables.  top_p: keep tokens until the mass of
    the strictly more likely ones reaches top_p.  seed: of this request's random stream; None
    lets the engine draw one.  stop_token_ids: stop after emitting one (it is part of the
    output).  ignore_eos: do not stop at the engine's end-of-sequence tokens."""

    max_tokens: int = 16
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    seed: int | None = None
    stop_token_ids: tuple[int, ...] = ()
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if math.isnan(self.temperature) or not 0.0 <= self.temperature <= 2.0:
            raise ValueError("temperature must be in [0, 2]")
        if self.top_k == 0 or self.top_k < -1:
            raise ValueError("top_k must be -1 (disabled) or >= 1")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1
