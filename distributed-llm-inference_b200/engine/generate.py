"""Generation for one request without the scheduler: ``greedy_generate``, the plain entry point
(src/dli/generate.py:22-87), and ``PagedSequence`` / ``paged_greedy_generate``, one request stepped
by hand on a shared runner (src/dli/generate.py:98-174) — all on the engine's own step function,
cache and kernels."""

from __future__ import annotations

from dataclasses import dataclass
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


class PagedSequence:
    """One request stepped by hand on a runner that other requests may share: ``prefill`` runs the
    part of the prompt that the prefix index did not supply, ``feed`` appends one token (sampled or
    forced) and runs it; both return the float32 logits [vocab] after the last token they ran.
    The request must hold pages already (``runner.manager.allocate`` or ``fork``).
    (src/dli/generate.py:98-138: the reference's closest thing to a replay primitive.)"""

    def __init__(self, runner, request_id) -> None:
        if not runner.manager.has_request(request_id):
            raise KeyError(f"unknown request {request_id!r}: allocate or fork it first")
        self.runner, self.manager, self.request_id = runner, runner.manager, request_id

    def prefill(self, prompt_ids: Sequence[int]):
        start = self.manager.num_computed_tokens(self.request_id)
        if self.manager.num_tokens(self.request_id) != len(prompt_ids):
            raise ValueError("the prompt's length does not match the allocation")
        rest = [int(t) for t in prompt_ids[start:]]
        return self.runner.step([StepEntry(self.request_id, rest, [len(rest) - 1])])[0]

    def feed(self, token: int):
        copies = self.manager.append_slots(self.request_id, [int(token)])
        if copies:
            self.runner.copy_pages(copies)
        return self.runner.step([StepEntry(self.request_id, [int(token)], [0])])[0]


@dataclass(frozen=True)
class PagedGeneration:
    tokens: list[int]
    num_cached_prompt_tokens: int


def paged_greedy_generate(runner, request_id, prompt_ids: Sequence[int], max_new_tokens: int, *,
                          eos_token_ids: Collection[int] = (), namespace: bytes = b"", release: bool = True, pick=None) -> PagedGeneration:
    """Greedy generation for one request on a shared runner, reusing whatever prefix of the prompt
    the index holds (src/dli/generate.py:141-174).  Tokens as ``greedy_generate`` gives them.  With
    ``release`` the request is freed at the end, its full pages staying in the index for later ones.
    ``pick`` turns a row of logits into an id (default: the engine's sampling kernel, greedy)."""
    if pick is None:
        sampler, greedy = Sampler(runner.model.device), [SamplingParams()]

        def pick(row):
            return sampler.sample(row.reshape(1, -1), greedy, [0], [0])[0]

    prompt = [int(t) for t in prompt_ids]
    alloc = runner.manager.allocate(request_id, prompt, namespace=namespace)
    runner.start_request(request_id, alloc.state_slot)
    seq, eos, out = PagedSequence(runner, request_id), set(eos_token_ids), []
    try:
        logits = seq.prefill(prompt)
        for i in range(max_new_tokens):
            token = int(pick(logits))  # the lowest id among equal maxima
            out.append(token)
            if token in eos or i == max_new_tokens - 1:
                break
            logits = seq.feed(token)
    finally:
        if release:
            runner.manager.free(request_id)
    return PagedGeneration(out, alloc.num_cached_tokens)
