"""Makes tests/golden/schedule_trace.json from the reference's own scheduler and engine loop.

Run once, on the CPU, with the reference's sources and its tests importable:

    PYTHONPATH=<reference checkout>/src:<reference checkout> python tests/golden/make_schedule_trace.py

Scenarios of arrivals (prompts that share stems, classes of service, tenants with weights, stop ids),
cancellations and small pools are run through ``dli.engine.LLMEngine`` with the reference's fake model
(``tests/unit/engine/fake.py``: the next token is a hash of the whole history).  For every step the
file holds what was submitted and cancelled before it, the batch the scheduler chose (request, start,
tokens, whether a token is sampled), who was preempted, and the tokens and finish reasons that came
out.  tests/test_schedule_vs_golden.py runs the same events through this repository's engine.
"""

import json
import random
from pathlib import Path

from dli.engine import LLMEngine, Priority, SchedulerConfig
from dli.kv.block_manager import BlockManager
from dli.sampling import SamplingParams
from tests.unit.engine.fake import FakeRunner


def scenario(seed, *, num_blocks, block_size, max_num_seqs, budget, watermark, policy="lru", prefix_caching=True,
             tenant_weights=None, aging_steps=200, requests=18, max_steps=400):
    rng = random.Random(seed)
    bm = BlockManager(num_blocks, block_size, eviction_policy=policy, enable_prefix_caching=prefix_caching, watermark=watermark)
    runner = FakeRunner(bm)
    config = SchedulerConfig(max_num_seqs, budget, tenant_weights=tenant_weights or {}, aging_steps=aging_steps)
    eng = LLMEngine(runner, bm, config)
    stems = [[rng.randrange(50) for _ in range(rng.randrange(0, 3 * block_size + 2))] for _ in range(3)]
    pending = []
    for i in range(requests):
        prompt = rng.choice(stems) + [rng.randrange(50) for _ in range(rng.randrange(1, 2 * block_size + 3))]
        max_tokens = rng.randrange(1, 14)
        limit = (num_blocks - int(watermark * num_blocks)) * block_size  # the reference would keep a larger one waiting for ever
        if len(prompt) + max_tokens > limit:
            prompt = prompt[: max(1, limit - max_tokens)]
        pending.append({"id": f"r{i}", "prompt": prompt, "max_tokens": max_tokens,
                        "priority": rng.choice([0, 0, 1]), "tenant": rng.choice(["t0", "t1", "t2"]),
                        "stop": [rng.randrange(50)] if rng.random() < 0.3 else []})
    steps, live = [], []
    while (pending or eng.has_unfinished()) and len(steps) < max_steps:
        added, aborted = [], []
        while pending and rng.random() < 0.45:
            r = pending.pop(0)
            eng.add_request(r["id"], r["prompt"], SamplingParams(max_tokens=r["max_tokens"], stop_token_ids=tuple(r["stop"])),
                            priority=Priority(r["priority"]), tenant=r["tenant"])
            added.append(r)
            live.append(r["id"])
        if live and rng.random() < 0.04:
            rid = rng.choice(live)
            if eng.abort(rid):
                aborted.append(rid)
        before = len(runner.calls)
        outs = eng.step()
        sched = runner.calls[-1] if len(runner.calls) > before else None
        steps.append({
            "add": added, "abort": aborted,
            "chunks": [[c.request.request_id, c.start, c.num_tokens, int(c.needs_logits)] for c in sched.chunks] if sched else [],
            "preempted": eng.stats.steps[-1].num_preempted,
            "out": [[o.request_id, o.new_token_ids[0], o.finish_reason.value if o.finish_reason else None] for o in outs],
        })
        bm.check_invariants()
    assert not pending and not eng.has_unfinished(), "the scenario did not finish"
    return {"seed": seed, "num_blocks": num_blocks, "block_size": block_size, "max_num_seqs": max_num_seqs, "budget": budget,
            "watermark": watermark, "policy": policy, "prefix_caching": prefix_caching, "tenant_weights": tenant_weights or {},
            "aging_steps": aging_steps, "steps": steps}


def main():
    cases = [
        scenario(1, num_blocks=40, block_size=4, max_num_seqs=4, budget=16, watermark=0.0),
        scenario(2, num_blocks=14, block_size=4, max_num_seqs=5, budget=24, watermark=0.0),
        scenario(3, num_blocks=24, block_size=2, max_num_seqs=3, budget=8, watermark=0.1, tenant_weights={"t1": 2.0}, aging_steps=5),
        scenario(4, num_blocks=12, block_size=8, max_num_seqs=6, budget=12, watermark=0.0, policy="cost", aging_steps=3),
        scenario(5, num_blocks=30, block_size=4, max_num_seqs=2, budget=5, watermark=0.0, prefix_caching=False, tenant_weights={"t0": 3.0, "t2": 0.5}),
        scenario(6, num_blocks=10, block_size=4, max_num_seqs=8, budget=64, watermark=0.0, requests=24),
    ]
    out = Path(__file__).resolve().parent / "schedule_trace.json"
    out.write_text(json.dumps(cases, separators=(",", ":")))
    for c in cases:
        print(c["seed"], len(c["steps"]), "steps,", sum(s["preempted"] for s in c["steps"]), "preemptions,",
              sum(len(s["abort"]) for s in c["steps"]), "cancelled,", sum(1 for s in c["steps"] for o in s["out"] if o[2] == "stop"), "stopped by id")
    print(out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
