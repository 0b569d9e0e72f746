"""Command line of the engine: ``dli generate``, ``dli init``, ``dli replay``.

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


def _engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", required=True, help="model folder (config.json + *.safetensors)")
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

    r = sub.add_parser("replay", help="trace replay (see bin/trace_run)", add_help=False)
    r.set_defaults(fn=None)

    if argv is None:
        argv = sys.argv[1:]
    if argv[:1] == ["replay"]:
        import runpy

        sys.argv = ["trace_run", *argv[1:]]
        runpy.run_path(str(Path(__file__).resolve().parents[1] / "bin" / "trace_run"), run_name="__main__")
        return 0
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
