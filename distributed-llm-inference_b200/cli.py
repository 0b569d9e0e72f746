"""Command line of the engine: ``dli generate``, ``dli init``, ``dli bench``, ``dli workload``, ``dli env``, ``dli replay``.

Option names and meanings are those of the reference's only command line, its
server (src/dli/server/__main__.py:65-124): --model, --device, --dtype,
--num-blocks | --kv-cache-gb, --block-size, --no-prefix-caching, --max-num-seqs,
--max-num-batched-tokens.  Sampling options carry the names of SamplingParams
(src/dli/sampling.py:22-56).  Token ids in, token ids out: there is no tokenizer.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def _engine_options(p: argparse.ArgumentParser, model_required: bool = True) -> None:
    p.add_argument("--model", required=model_required, default=None, help="model folder (config.json + *.safetensors)")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--dtype", default="auto", choices=["auto", "float32", "bfloat16"], help="auto = bfloat16")
    kv = p.add_mutually_exclusive_group()
    kv.add_argument("--num-blocks", type=int, default=None, help="cache pages in the pool")
    kv.add_argument("--kv-cache-gb", type=float, default=None, help="cache pool size in GiB (default 1.0)")
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--no-prefix-caching", action="store_true", help="do not reuse cached prefixes across requests")
    p.add_argument("--max-num-seqs", type=int, default=64)
    p.add_argument("--max-num-batched-tokens", type=int, default=512)
    p.add_argument("--seed", type=int, default=0, help="engine seed (draws the seeds of requests that give none)")
    p.add_argument("--eos-token-ids", type=str, default="", help="comma-separated end-of-sequence ids")


def _ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def cmd_generate(args) -> int:
    from . import LLMEngine, SamplingParams, SchedulerConfig

    engine = LLMEngine.from_model_dir(
        args.model, dtype=args.dtype, device=args.device, num_blocks=args.num_blocks, kv_cache_gb=args.kv_cache_gb,
        block_size=args.block_size, enable_prefix_caching=not args.no_prefix_caching,
        config=SchedulerConfig(args.max_num_seqs, args.max_num_batched_tokens), eos_token_ids=_ids(args.eos_token_ids), seed=args.seed,
    )
    prompts = [_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        prompts += [_ids(line) for line in Path(args.prompt_file).read_text().splitlines() if line.strip()]
    if not prompts:
        raise SystemExit("give --prompt-ids (repeatable) or --prompt-file")
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            seed=args.sampling_seed, stop_token_ids=tuple(_ids(args.stop_token_ids)), ignore_eos=args.ignore_eos)
    reqs = [engine.add_request(f"cli-{i}", p, params) for i, p in enumerate(prompts)]
    while engine.has_unfinished():
        engine.step()
    for r in reqs:
        print(json.dumps({"request_id": r.request_id, "prompt_ids": r.prompt_ids, "output_ids": r.output_ids,
                          "finish_reason": r.finish_reason.value if r.finish_reason else None}))
    return 0


def cmd_bench(args) -> int:
    """Steady decode steps of ``--batch`` requests through the engine, as a user would drive it
    (the measurement of benchmarks/scripts/engine_profile.py:36-117: random prompts, warm-up past the
    prompts, timed steps, the split of a step, and the floor that memory bandwidth sets)."""
    import statistics
    import time

    import torch

    from . import LLMEngine, SamplingParams, SchedulerConfig

    model = _model_for(args)
    total = args.input_len + args.output_len
    blocks = args.num_blocks or args.batch * (-(-total // args.block_size) + 1)
    # no pages are held back: the pool is sized so that all requests run at once, to their last token
    eng = LLMEngine.for_model(model, num_blocks=blocks, block_size=args.block_size, enable_prefix_caching=not args.no_prefix_caching,
                              config=SchedulerConfig(args.batch, max(args.max_num_batched_tokens, args.batch)), seed=args.seed, watermark=0.0)
    g = torch.Generator().manual_seed(0)
    for i in range(args.batch):
        ids = torch.randint(min(1000, model.spec.vocab_size - 1), model.spec.vocab_size, (args.input_len,), generator=g).tolist()
        eng.add_request(f"r{i}", ids, SamplingParams(max_tokens=args.output_len, ignore_eos=True))
    while any(r.num_computed_tokens < args.input_len for r in eng.scheduler.running + list(eng.scheduler.waiting)):
        eng.step()
        if eng.stats.steps[-1].num_batched_tokens == 0:
            raise SystemExit("the prompts make no progress: the pool (--num-blocks) is too small for one of them")
    if len(eng.scheduler.running) != args.batch:
        raise SystemExit(f"only {len(eng.scheduler.running)} of {args.batch} requests run at once: the steps timed would not be steps of the whole batch")
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    first = len(eng.stats.steps)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        eng.step()
    torch.cuda.synchronize()
    step_ms = (time.perf_counter() - t0) / args.steps * 1e3
    if len(eng.scheduler.running) != args.batch:
        raise SystemExit(f"the batch did not stay whole for {args.warmup} + {args.steps} steps: requests ended (raise --output-len, now "
                         f"{args.output_len}) or were preempted (raise --num-blocks)")
    st = eng.stats.steps[first:]
    weights = sum(t.numel() * t.element_size() for t in {id(t): t for part in model.parts() for t in vars(part).values() if isinstance(t, torch.Tensor)}.values())
    ctx = statistics.mean(r.num_computed_tokens for r in eng.scheduler.running) if eng.scheduler.running else 0
    kv = args.batch * ctx * sum(eng.runner.pools.bytes_per_page(model.cache_needs(), model.spec.run_order, args.block_size, model.dtype)) / args.block_size
    print(json.dumps({
        "batch": args.batch, "input_len": args.input_len, "steps": args.steps, "step_ms": step_ms, "tokens_per_s": args.batch / step_ms * 1e3,
        "schedule_ms_mean": statistics.mean(s.schedule_s for s in st) * 1e3, "forward_ms_mean": statistics.mean(s.forward_s for s in st) * 1e3,
        "postprocess_ms_mean": statistics.mean(s.postprocess_s for s in st) * 1e3, "steps_launched_ahead": eng.steps_ahead,
        "graph_steps": eng.runner.graph_steps, "mixed_graph_steps": eng.runner.mixed_graph_steps, "weight_bytes": weights, "kv_bytes_read_per_step": kv,
        "bandwidth_floor_ms": (weights + kv) / (args.bandwidth_gbs * 1e9) * 1e3, "bandwidth_gbs": args.bandwidth_gbs,
        "max_memory_allocated_mib": torch.cuda.max_memory_allocated() >> 20,
    }))
    _note_env(args)
    return 0


SHAPES = Path(__file__).resolve().parent / "config" / "shapes"  # config.json files of the models that benchmarks name


def shape_config(name_or_path: str) -> dict:
    """A config.json given as a path, or as the name of one of the shapes kept with the package."""
    path = Path(name_or_path)
    if not path.exists():
        path = SHAPES / f"{name_or_path}.json"
    if not path.exists():
        known = ", ".join(sorted(p.stem for p in SHAPES.glob("*.json")))
        raise SystemExit(f"{name_or_path!r} is neither a config.json nor one of the shapes {known}")
    return json.loads(path.read_text())


def _model_for(args):
    from . import load_model, random_model

    if not args.random_config and not args.model:
        raise SystemExit("give --model DIR or --random-config JSON")
    dtype = "bfloat16" if args.dtype == "auto" else args.dtype
    if args.random_config:
        return random_model(shape_config(args.random_config), args.seed, dtype, args.device)
    return load_model(args.model, dtype, args.device)


def cmd_workload(args) -> int:
    """A closed set of requests run to the end through the engine, all queued at the start or
    --concurrency of them in flight (the next is submitted when one finishes):
    prompts of seeded random ids with lengths uniform in [--min-input, --max-input], a share of
    them opening with the same --shared-prefix-len ids, --output-len tokens generated for each
    (end-of-sequence ignored, temperature 0, as the reference's load generator sends them:
    benchmarks/methodology.md:55-67).  Prompt portions and decoded tokens share the steps."""
    import random
    import statistics

    import torch

    from . import LLMEngine, SamplingParams, SchedulerConfig
    from .engine import percentile, run_closed_loop

    model = _model_for(args)
    rng = random.Random(args.seed)
    vocab = model.spec.vocab_size
    low = min(1000, vocab - 1)
    stem = [rng.randrange(low, vocab) for _ in range(args.shared_prefix_len)]
    prompts = []
    for i in range(args.num_requests):
        n = rng.randint(args.min_input, args.max_input)
        shared = args.shared_prefix_len > 0 and rng.random() < args.shared_fraction
        head = stem[:n] if shared else []
        prompts.append(head + [rng.randrange(low, vocab) for _ in range(n - len(head))])
    longest = max(len(p) for p in prompts) + args.output_len
    per_request = -(-longest // args.block_size) + 1
    blocks = args.num_blocks or (None if args.kv_cache_gb else args.max_num_seqs * per_request)
    eng = LLMEngine.for_model(model, num_blocks=blocks, kv_cache_gb=args.kv_cache_gb, block_size=args.block_size,
                              enable_prefix_caching=not args.no_prefix_caching,
                              config=SchedulerConfig(args.max_num_seqs, args.max_num_batched_tokens), seed=args.seed)
    params = SamplingParams(max_tokens=args.output_len, ignore_eos=True)
    for rep in range(args.warmup_runs + 1):  # warm-up runs compile nothing new later: same lengths, other ids
        if rep:
            eng.manager.reset_prefix_cache()
        timed = rep == args.warmup_runs
        run_prompts = prompts if timed else [[(t + 1 + rep) % vocab for t in p] for p in prompts]
        first_step = len(eng.stats.steps)
        hit_before = eng.manager.stats.prompt_tokens_hit
        run = run_closed_loop(eng, run_prompts, params, concurrency=args.concurrency, name=f"w{rep}", synchronize=torch.cuda.synchronize)
    st = eng.stats.steps[first_step:]
    reqs, seconds = run.requests, run.seconds
    generated = sum(len(r.output_ids) for r in reqs)
    prompt_tokens = sum(len(p) for p in prompts)
    ttft, tpot = run.time_to_first_token(), run.time_per_output_token()
    print(json.dumps({
        "requests": len(reqs), "concurrency": args.concurrency or len(reqs), "prompt_tokens": prompt_tokens, "generated_tokens": generated,
        "seconds": seconds, "generated_tokens_per_s": generated / seconds, "total_tokens_per_s": (prompt_tokens + generated) / seconds,
        "steps": len(st), "prefill_tokens_run": sum(s.num_prefill_tokens for s in st), "decode_tokens_run": sum(s.num_decode_tokens for s in st),
        "prompt_tokens_reused": eng.manager.stats.prompt_tokens_hit - hit_before,
        "preemptions": sum(s.num_preempted for s in st), "mean_batched_tokens": statistics.mean(s.num_batched_tokens for s in st),
        "first_token_s_median": percentile(ttft, 0.5), "first_token_s_p99": percentile(ttft, 0.99), "first_token_s_max": ttft[-1] if ttft else None,
        "per_output_token_s_median": percentile(tpot, 0.5), "per_output_token_s_p99": percentile(tpot, 0.99),
        "schedule_ms_mean": statistics.mean(s.schedule_s for s in st) * 1e3, "forward_ms_mean": statistics.mean(s.forward_s for s in st) * 1e3,
        "steps_launched_ahead": eng.steps_ahead, "graph_steps": eng.runner.graph_steps, "mixed_graph_steps": eng.runner.mixed_graph_steps,
        "mixed_graph_captures": getattr(getattr(eng.runner, "graphs", None), "mixed_captures", 0),
        "mixed_graph_capture_s": round(getattr(getattr(eng.runner, "graphs", None), "mixed_capture_seconds", 0.0), 3),
        "pages": eng.manager.groups[0].num_pages, "max_memory_allocated_mib": torch.cuda.max_memory_allocated() >> 20,
    }))
    _note_env(args)
    return 0


def cmd_env(args) -> int:
    from . import envinfo

    return envinfo.main([args.out] if args.out else [])


def _note_env(args) -> None:
    """``--env-json PATH``: the machine and the code a result came from, written beside it."""
    if getattr(args, "env_json", None):
        from . import envinfo

        envinfo.write(args.env_json)


def cmd_init(args) -> int:
    import torch

    from .weights import write_model_dir

    cfg = json.loads(Path(args.config).read_text())
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.storage_dtype]
    write_model_dir(args.out, cfg, args.seed, dtype)
    print(f"wrote {args.out}/config.json and model.safetensors (seed {args.seed})")
    return 0


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="dli", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate token ids for prompts given as token ids")
    _engine_options(g)
    g.add_argument("--prompt-ids", action="append", default=[], help="one prompt as comma- or space-separated ids; repeatable")
    g.add_argument("--prompt-file", default=None, help="file with one prompt (ids) per line")
    g.add_argument("--max-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=-1)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--sampling-seed", type=int, default=None, help="seed of each request's random stream")
    g.add_argument("--stop-token-ids", type=str, default="")
    g.add_argument("--ignore-eos", action="store_true")
    g.set_defaults(fn=cmd_generate)

    i = sub.add_parser("init", help="write a random-weights model folder from a config.json and a seed")
    i.add_argument("--config", required=True, help="a config.json of a registered architecture")
    i.add_argument("--seed", type=int, default=0)
    i.add_argument("--out", required=True)
    i.add_argument("--storage-dtype", default="float32", choices=["float32", "bfloat16"])
    i.set_defaults(fn=cmd_init)

    b = sub.add_parser("bench", help="time steady decode steps of a batch through the engine")
    _engine_options(b, model_required=False)
    b.add_argument("--random-config", default=None, help="a config.json, or the name of a shape kept with the package (llama-3.2-1b, smollm2-1.7b, llama-3.2-3b): run with seeded random weights instead of --model")
    b.add_argument("--batch", type=int, default=8)
    b.add_argument("--input-len", type=int, default=256)
    b.add_argument("--output-len", type=int, default=128)
    b.add_argument("--steps", type=int, default=20)
    b.add_argument("--warmup", type=int, default=8)
    b.add_argument("--bandwidth-gbs", type=float, default=6650.0, help="memory bandwidth for the floor, GB/s")
    b.add_argument("--env-json", default=None, help="also write what the run ran on (hardware, driver, libraries, revision) to this file")
    b.set_defaults(fn=cmd_bench)

    w = sub.add_parser("workload", help="run a closed set of requests of mixed lengths, part of them sharing a prefix, to the end")
    _engine_options(w, model_required=False)
    w.add_argument("--random-config", default=None, help="a config.json, or the name of a shape kept with the package (llama-3.2-1b, smollm2-1.7b, llama-3.2-3b): run with seeded random weights instead of --model")
    w.add_argument("--num-requests", type=int, default=64)
    w.add_argument("--min-input", type=int, default=128)
    w.add_argument("--max-input", type=int, default=2048)
    w.add_argument("--output-len", type=int, default=256)
    w.add_argument("--shared-prefix-len", type=int, default=512, help="ids that the sharing requests open with (0: nobody shares)")
    w.add_argument("--shared-fraction", type=float, default=0.5, help="share of the requests that open with the shared ids")
    w.add_argument("--warmup-runs", type=int, default=1, help="untimed runs of the same lengths before the timed one")
    w.add_argument("--concurrency", type=int, default=None, help="requests in flight: the next is submitted when one finishes (default: all are queued at the start)")
    w.add_argument("--env-json", default=None, help="also write what the run ran on (hardware, driver, libraries, revision) to this file")
    w.set_defaults(fn=cmd_workload)

    e = sub.add_parser("env", help="print what a measurement would run on: hardware, driver, libraries, revision of the code")
    e.add_argument("--out", default=None, help="write it to this file instead")
    e.set_defaults(fn=cmd_env)

    r = sub.add_parser("replay", help="trace replay (see bin/trace_run)", add_help=False)
    r.set_defaults(fn=None)

    if argv is None:
        argv = sys.argv[1:]
    if argv[:1] == ["replay"]:
        from . import replay

        return replay.main(argv[1:])
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
