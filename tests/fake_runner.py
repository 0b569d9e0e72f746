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
    def __init__(self, num_pages, page_size, max_requests=64, prefix_caching=True, watermark=0.01, eviction_policy="lru"):
        self.manager = CacheManager([GroupSpec(num_pages)], page_size, max_requests,
                                    enable_prefix_caching=prefix_caching, watermark=watermark, eviction_policy=eviction_policy)
        self.started = []
        self.steps = []
        self.prompts, self.histories, self.stepped = {}, {}, []

    def start_request(self, request_id, slot):
        self.started.append(request_id)

    def copy_pages(self, copies):
        self.copied = getattr(self, "copied", []) + list(copies)

    def execute(self, chunks, token_source=None, token_rows=None):
        rows = []
        self.steps.append([(c.request.request_id, c.start, c.num_tokens, c.needs_logits) for c in chunks])
        for i, c in enumerate(chunks):
            rid = c.request.request_id
            assert self.manager.num_computed_tokens(rid) == c.start, "a chunk does not start where the cache ends"
            assert self.manager.num_tokens(rid) >= c.start + c.num_tokens, "tokens without reserved slots"
            self.manager.mark_computed(rid, c.start + c.num_tokens)
            history = c.request.all_token_ids[: c.start + c.num_tokens]
            if token_rows is not None and token_rows[i] >= 0:  # the token the host has not read: the step before left it
                assert c.num_tokens == 1 and c.start == len(history), "a token from the device is the one after the known ones"
                history = history + [token_source.device_ids[token_rows[i]]]
            if c.needs_logits:
                rows.append(next_token(history))
        self.manager.check_invariants()
        return rows


    def step(self, entries):
        """The step function's side of the fake: rows of 50 "logits" whose maximum is the hash of the
        history up to the wanted token.  ``self.prompts[rid]`` must hold the request's prompt, so that
        tokens served by the prefix index (which a step never sees) are part of the history."""
        import numpy as np

        rows = []
        for e in entries:
            rid = e.request_id
            done = self.manager.num_computed_tokens(rid)
            hist = self.histories.setdefault(rid, list(self.prompts[rid][:done]))
            assert len(hist) == done, "a step does not start where the cache ends"
            assert self.manager.num_tokens(rid) >= done + len(e.token_ids), "tokens without reserved slots"
            for w in e.want:
                row = np.zeros(50, dtype=np.float32)
                row[next_token(hist + list(e.token_ids[: w + 1]))] = 1.0
                rows.append(row)
            hist.extend(e.token_ids)
            self.manager.mark_computed(rid, done + len(e.token_ids))
            self.stepped.append((rid, done, len(e.token_ids)))
        self.manager.check_invariants()
        return np.stack(rows) if rows else np.zeros((0, 50), dtype=np.float32)


class AheadRunner(FakeRunner):
    """Takes a step's tokens from what the step before sampled, as the real runner does on the device."""

    takes_token_source = True


class FakeSampler:
    def sample(self, logits, params, seeds, draws):
        return list(logits)


class FakeTokens:
    def __init__(self, ids):
        self.device_ids = list(ids)
        self.reads = 0

    def result(self):
        self.reads += 1
        return self.device_ids


class AheadSampler(FakeSampler):
    def sample_async(self, logits, params, seeds, draws):
        return FakeTokens(logits)


def fake_engine(num_pages=64, page_size=4, max_num_seqs=8, budget=32, ahead=False, tenant_weights=None, aging_steps=200, **kw):
    runner = (AheadRunner if ahead else FakeRunner)(num_pages, page_size, max_requests=max_num_seqs, **kw)
    config = SchedulerConfig(max_num_seqs, budget, tenant_weights=tenant_weights or {}, aging_steps=aging_steps)
    return LLMEngine(runner, config, sampler=AheadSampler() if ahead else FakeSampler()), runner
