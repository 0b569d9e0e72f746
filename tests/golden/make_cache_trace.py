"""Makes tests/golden/cache_trace.json from the reference's own block manager.

Run once, on the CPU, with the reference's sources importable:

    PYTHONPATH=<reference checkout>/src python tests/golden/make_cache_trace.py

Random sequences of operations (prompts that share stems, growth token by token, partial and full
computation, forks, frees, resets; pools small enough that idle pages are evicted and admissions
fail) are run through ``dli.kv.block_manager.BlockManager``; every operation is stored with what
the reference answered and with the pool's counters after it.  tests/test_cache_vs_golden.py runs
the same operations through this repository's cache manager and compares.
"""

import json
import random
from pathlib import Path

from dli.kv.block_manager import BlockManager, NoFreeBlocksError  # the reference


def observe(bm, probes):
    """free, idle, used pages; evictions; prompt tokens queried, hit; copies; duplicate registrations; pages
    obtainable; then for every probe prompt whether it would be admitted and how many new pages it would take."""
    s = bm.stats()
    row = [s.free_blocks, s.cached_idle_blocks, s.used_blocks, s.evictions, s.prompt_tokens_queried, s.prompt_tokens_hit,
           s.cow_copies, s.duplicate_registrations, bm.num_available_blocks]
    for p in probes:
        row += [int(bm.can_allocate(p)), bm.blocks_needed_for_prompt(p)]
    return row


def scenario(seed, policy, num_blocks, block_size, watermark, steps):
    rng = random.Random(seed)
    bm = BlockManager(num_blocks, block_size, eviction_policy=policy, watermark=watermark)
    stems = [[rng.randrange(1000) for _ in range(rng.randrange(1, 5) * block_size + rng.randrange(block_size))] for _ in range(4)]
    probes = [stems[0] + [1, 2, 3], stems[1][: block_size + 1], [7] * (2 * block_size)]
    live, ops, counter = {}, [], 0  # live: id -> token list
    for _ in range(steps):
        kind = rng.choices(["allocate", "append", "compute", "free", "fork", "reset"], [5, 6, 6, 3, 1, 0.2])[0]
        rec = None
        if kind == "allocate":
            stem = rng.choice(stems)
            toks = stem[: rng.randrange(1, len(stem) + 1)] + [rng.randrange(1000) for _ in range(rng.randrange(0, 2 * block_size))]
            sid = f"s{counter}"
            counter += 1
            rec = {"op": "allocate", "id": sid, "tokens": toks, "respect_watermark": rng.random() < 0.8}
            try:
                alloc = bm.allocate(sid, toks, respect_watermark=rec["respect_watermark"])
                rec["cached"] = alloc.num_cached_tokens
                rec["table"] = list(alloc.block_table)
                live[sid] = list(toks)
            except NoFreeBlocksError:
                rec["fails"] = True
        elif kind == "append" and live:
            sid = rng.choice(sorted(live))
            toks = [rng.randrange(1000) for _ in range(rng.choice([1, 1, 1, 2, block_size]))]
            rec = {"op": "append", "id": sid, "tokens": toks}
            try:
                rec["copies"] = [[c.src, c.dst] for c in bm.append_slots(sid, toks)]
                live[sid] += toks
            except NoFreeBlocksError:
                rec["fails"] = True
        elif kind == "compute" and live:
            sid = rng.choice(sorted(live))
            lo, hi = bm.num_computed_tokens(sid), bm.num_tokens(sid)
            n = rng.choice([hi, rng.randrange(lo, hi + 1)])
            bm.mark_computed(sid, n)
            rec = {"op": "compute", "id": sid, "n": n}
        elif kind == "free" and live:
            sid = rng.choice(sorted(live))
            bm.free(sid)
            del live[sid]
            rec = {"op": "free", "id": sid}
        elif kind == "fork" and live:
            parent = rng.choice(sorted(live))
            child = f"s{counter}"
            counter += 1
            bm.fork(parent, child)
            live[child] = list(live[parent])
            rec = {"op": "fork", "parent": parent, "child": child}
        elif kind == "reset":
            rec = {"op": "reset", "evicted": bm.reset_prefix_cache()}
        if rec is None:
            continue
        bm.check_invariants()
        rec["after"] = observe(bm, probes)
        if len(ops) % 6 == 0 or rec["op"] == "fork":  # every table now and then (the file stays small)
            rec["tables"] = {sid: list(bm.block_table(sid)) for sid in sorted(live)}
        ops.append(rec)
    return {"seed": seed, "policy": policy, "num_blocks": num_blocks, "block_size": block_size, "watermark": watermark,
            "probes": probes, "ops": ops}


def main():
    cases = [scenario(1, "lru", 24, 4, 0.0, 260), scenario(2, "lru", 40, 8, 0.1, 260), scenario(3, "cost", 24, 4, 0.0, 260),
             scenario(4, "cost", 32, 2, 0.05, 260), scenario(5, "lru", 12, 4, 0.0, 200)]
    out = Path(__file__).resolve().parent / "cache_trace.json"
    out.write_text(json.dumps(cases, separators=(",", ":")))
    for c in cases:
        fails = sum(1 for o in c["ops"] if o.get("fails"))
        print(c["seed"], c["policy"], len(c["ops"]), "ops,", fails, "refused,", c["ops"][-1]["after"][3], "evictions,",
              c["ops"][-1]["after"][5], "tokens hit,", c["ops"][-1]["after"][6], "copies")
    print(out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
