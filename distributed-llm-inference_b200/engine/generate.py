"""Greedy generation for one prompt, without scheduler or sampler state: the plain entry point
(src/dli/generate.py:22-87), on the engine's own step function, cache and kernels."""

from __future__ import annotations

from typing import Collection, Sequence

from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .runner import ModelRunner


def greedy_generate(model, prompt_ids: Sequence[int], max_new_tokens: int, *, eos_token_ids: Collection[int] = (),
                    use_cache: bool = True, page_size: int = 16) -> list[int]:
    """Up to ``max_new_tokens`` ids, each the argmax of the logits after everything before it (lowest
    id on ties); generation stops after an id of ``eos_token_ids``, which is part of the result.
    ``use_cache=False`` runs the whole sequence again for every token, from an empty cache: slow, and
    a check of the cached path that shares nothing with it but the kernels."""
    prompt = [int(t) for t in prompt_ids]
    if not prompt:
        raise ValueError("prompt_ids must be non-empty")
    if max_new_tokens <= 0:
        return []
    pages = -(-(len(prompt) + max_new_tokens) // page_size) + 1
    runner = ModelRunner(model, num_pages=pages, page_size=page_size, max_requests=1, enable_prefix_caching=False, watermark=0.0)
    sampler, greedy, eos = Sampler(model.device), [SamplingParams()], set(eos_token_ids)
    out: list[int] = []
    if use_cache:
        runner.manager.allocate("g", prompt)
        feed = prompt
    while len(out) < max_new_tokens:
        if use_cache:
            logits = runner.step([StepEntry("g", feed, [len(feed) - 1])])
        else:
            tokens = prompt + out
            runner.manager.allocate("g", tokens)
            logits = runner.step([StepEntry("g", tokens, [len(tokens) - 1])])
            runner.manager.free("g")
        token = sampler.sample(logits, greedy, [0], [0])[0]
        out.append(token)
        if token in eos:
            break
        if use_cache and len(out) < max_new_tokens:
            runner.manager.append_slots("g", [token])
            feed = [token]
    return out
