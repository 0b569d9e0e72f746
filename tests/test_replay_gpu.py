"""Trace replay against the plain implementation: the same requests whole, with the last 32
tokens decoded one by one, in portions of changing size, and mixed with other requests in a
pool so small that pages are used again — in float32 and in bfloat16."""

import numpy as np
import pytest

from tests.plain import llama_plain as plain
from tests.tiny_configs import TINY
from tests.util import TOL, TraceRun, make_model_dir, plain_weights_for, random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [100, 37, 81, 64, 120, 49], "tiny_b": [90, 130, 65, 33, 150, 71], "tiny_c": [70, 96, 41, 111, 58, 80]}


@pytest.fixture(scope="module", params=[(n, d) for n in sorted(TINY) for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    name, dtype = request.param
    path = tmp_path_factory.mktemp(f"{name}_{dtype}")
    cfg, weights, page = make_model_dir(path, name, sharpen=6.0)
    reqs = {f"r{i}": random_tokens(cfg["vocab_size"], n, seed=10 * i + 1) for i, n in enumerate(LENGTHS[name])}
    w = plain_weights_for(weights, dtype)
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    return dict(name=name, dtype=dtype, path=path, cfg=cfg, page=page, reqs=reqs, ref=ref, tmp=tmp_path_factory)


def check(case, got: dict, what: str):
    """got: request -> logits [n, vocab] for all its positions."""
    tol = TOL[case["dtype"]]
    for rid, logits in got.items():
        ref = case["ref"][rid]
        assert logits.shape == ref.shape
        err = np.abs(logits - ref).max(axis=1)
        bad = np.nonzero(err > tol)[0]
        assert bad.size == 0, f"{what}: request {rid}: first wrong position {bad[0]} of {len(err)} (error {err[bad[0]]:.3g}, tolerance {tol})"


def rounded(n, page):
    unit = max(64, page)
    return -(-n // unit) * unit


def test_whole_and_last_32_one_by_one(case):
    reqs = case["reqs"]
    longest = max(len(t) for t in reqs.values())
    run = TraceRun(case["path"], case["dtype"], case["tmp"].mktemp("out"), rounded(longest, case["page"]), case["page"])
    whole, decoded = {}, {}
    for rid, toks in reqs.items():
        whole[rid] = run.step([(rid, toks, range(len(toks)))], end=[rid])
    for rid, toks in reqs.items():
        cut = max(1, len(toks) - 32)
        parts = [run.step([(rid + "d", toks[:cut], range(cut))])]
        for i in range(cut, len(toks)):
            parts.append(run.step([(rid + "d", [toks[i]], [0])], end=[rid + "d"] if i == len(toks) - 1 else []))
        decoded[rid] = np.concatenate(parts)
    assert run.close() == 0
    check(case, whole, "whole")
    check(case, decoded, "last 32 decoded")


def test_portions_of_changing_size(case):
    reqs = case["reqs"]
    longest = max(len(t) for t in reqs.values())
    run = TraceRun(case["path"], case["dtype"], case["tmp"].mktemp("out"), rounded(longest, case["page"]), case["page"])
    got = {}
    sizes = [2, 17, 3, 2, 31, 5, 16, 2, 9, 64, 4, 1, 2]
    for k, (rid, toks) in enumerate(reqs.items()):
        parts, pos, j = [], 0, k
        while pos < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - pos)
            j += 1
            out = run.step([(rid, toks[pos : pos + n], range(n))], end=[rid] if pos + n == len(toks) else [])
            parts.append(out)
            pos += n
        got[rid] = np.concatenate(parts)
    assert run.close() == 0
    check(case, got, "portions")


def test_mixed_requests_in_a_pool_that_reuses_pages(case):
    """Up to four live requests; portions of some beside decoded tokens of others; a request
    is sometimes left out of a step; the pool holds exactly the most that is ever live."""
    reqs = case["reqs"]
    rng = np.random.default_rng(7)
    page = case["page"]
    # plan first (to know the pool size), then replay
    waiting = list(reqs)
    live: dict[str, int] = {}
    plan, peak = [], 0
    while waiting or live:
        while waiting and len(live) < 4 and (not live or rng.random() < 0.6):
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue  # left out of this step
            toks, pos = reqs[rid], live[rid]
            n = 1 if pos >= len(toks) - 32 and pos > 0 else int(min(rng.integers(2, 24), len(toks) - pos))
            entries.append((rid, pos, n))
            live[rid] = pos + n
        peak = max(peak, sum(rounded(p, page) for p in live.values()))
        for rid in list(live):
            if live[rid] == len(reqs[rid]):
                end.append(rid)
                del live[rid]
        if entries:
            plan.append((entries, end))
    run = TraceRun(case["path"], case["dtype"], case["tmp"].mktemp("out"), peak, page)
    parts = {rid: [] for rid in reqs}
    saw_mixed = False
    for entries, end in plan:
        saw_mixed |= any(n == 1 for _, _, n in entries) and any(n > 1 for _, _, n in entries)
        out = run.step([(rid, reqs[rid][pos : pos + n], range(n)) for rid, pos, n in entries], end=end)
        row = 0
        for rid, pos, n in entries:
            parts[rid].append(out[row : row + n])
            row += n
    assert run.close() == 0
    assert saw_mixed
    total = sum(rounded(len(t), page) for t in reqs.values())
    assert peak < total, "the pool is as large as all requests together: no page is used again"
    check(case, {rid: np.concatenate(p) for rid, p in parts.items()}, "mixed")


def test_want_may_be_empty_and_partial(case):
    rid, toks = next(iter(case["reqs"].items()))
    run = TraceRun(case["path"], case["dtype"], case["tmp"].mktemp("out"), rounded(len(toks), case["page"]), case["page"])
    assert run.step([(rid, toks[:40], [])]) is None
    out = run.step([(rid, toks[40:60], [19, 0, 7])])
    tail = run.step([(rid, toks[60:], [len(toks) - 61])], end=[rid])
    assert run.close() == 0
    ref = case["ref"][rid]
    tol = TOL[case["dtype"]]
    assert np.abs(out - ref[[59, 40, 47]]).max() < tol and np.abs(tail - ref[-1:]).max() < tol


def test_prefix_hits_change_nothing(case):
    """The prefix index on: requests that begin like an earlier one (ended, its pages idle in the index; or live,
    its pages shared) skip the shared pages, in a pool so small that idle pages are evicted and used again; the
    logits at every place computed are those of the plain implementation."""
    cfg, page = case["cfg"], case["page"]
    tol = TOL[case["dtype"]]
    w = plain_weights_for(plain.read_safetensors(case["path"] / "model.safetensors"), case["dtype"])
    stem = random_tokens(cfg["vocab_size"], 70, seed=501)
    seqs = {k: stem[:n] + random_tokens(cfg["vocab_size"], m, seed=502 + i) for i, (k, n, m) in
            enumerate((("a", 70, 12), ("b", 70, 25), ("c", 45, 30), ("d", 0, 126), ("e", 70, 5)))}
    ref = {k: plain.forward(cfg, w, v) for k, v in seqs.items()}
    run = TraceRun(case["path"], case["dtype"], case["tmp"].mktemp("out"), 2 * rounded(100, page), page, prefix_caching=True)
    got = {}
    got["a"] = (0, run.step([("a", seqs["a"], range(len(seqs["a"])))], end=["a"]))
    b = seqs["b"]
    first = run.step([("b", b[:80], range(70, 80))])  # the stem's full pages are idle in the index
    c = seqs["c"]
    both = run.step([("c", c, range(45, len(c))), ("b", b[80:], range(len(b) - 80))], end=["c"])  # c shares pages with the live b
    got["b"] = (70, np.concatenate([first, both[len(c) - 45:]]))
    got["c"] = (45, both[: len(c) - 45])
    d = seqs["d"]
    got["d"] = (0, run.step([("d", d, range(len(d)))], end=["d", "b"]))  # more pages than are free: idle ones are evicted for it
    e = seqs["e"]
    got["e"] = (70, run.step([("e", e, range(70, len(e)))], end=["e"]))
    assert run.close() == 0
    found = run.found_in_cache()
    assert found.get("b") == 70 // page * page and found.get("c") == 45 // page * page, found
    for rid, (start, logits) in got.items():
        err = np.abs(logits - ref[rid][start:]).max(axis=1)
        assert err.max() < tol, f"request {rid}: first wrong position {start + int(np.argmax(err > tol))} (error {err.max():.3g})"
