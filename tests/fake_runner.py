"""A model without tensors for scheduler tests: the next token is a hash of the whole history,
so a dropped, repeated or reordered token, or lost progress, changes the output
(the idea of the reference's tests/unit/engine/fake.py:21-56)."""

import hashlib

from dli_b200.cache import CacheManager, GroupSpec
from dli_b200.engine import LLMEngine, SchedulerConfig


def next_token(history) -> int:
    return int.from_bytes(hashlib.blake2b(repr(list(history)).encode(), digest_size=4).digest(), "little") % 50


def sequential(prompt, max_tokens, stop=()):
    hist, out = list(prompt), []
    for _ in range(max_tokens):
        t = next_token(hist)
        hist.append(t)
        out.append(t)
        if t in stop:
            break
    return out


class FakeRunner:
    def __init__(self, num_pages, page_size, max_requests=64, prefix_caching=True, watermark=0.01):
        self.manager = CacheManager([GroupSpec(num_pages)], page_size, max_requests,
                                    enable_prefix_caching=prefix_caching, watermark=watermark)
        self.started = []
        self.steps = []

    def start_request(self, request_id, slot):
        self.started.append(request_id)

    def execute(self, chunks):
        rows = []
        self.steps.append([(c.request.request_id, c.start, c.num_tokens, c.needs_logits) for c in chunks])
        for c in chunks:
            rid = c.request.request_id
            assert self.manager.num_computed_tokens(rid) == c.start, "a chunk does not start where the cache ends"
            assert self.manager.num_tokens(rid) >= c.start + c.num_tokens, "tokens without reserved slots"
            self.manager.mark_computed(rid, c.start + c.num_tokens)
            if c.needs_logits:
                rows.append(next_token(c.request.all_token_ids[: c.start + c.num_tokens]))
        self.manager.check_invariants()
        return rows


class FakeSampler:
    def sample(self, logits, params, seeds, draws):
        return list(logits)


def fake_engine(num_pages=64, page_size=4, max_num_seqs=8, budget=32, **kw):
    runner = FakeRunner(num_pages, page_size, max_requests=max_num_seqs, **kw)
    return LLMEngine(runner, SchedulerConfig(max_num_seqs, budget), sampler=FakeSampler()), runner
