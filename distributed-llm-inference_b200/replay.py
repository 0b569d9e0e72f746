"""Trace replay (the program ``bin/trace_run``; also ``dli replay``): feeds given token ids through a model step by step and writes logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch through the engine's own model, step
function, cache manager and kernels (nothing is sampled).  For a step in which
logits are wanted, ``DIR/<step>.f32`` holds them as little-endian float32
[wanted, vocab], in the order of the entries and of ``want``.  After every
step a line ``done <step>`` is printed.  The cache pool holds ``--max-tokens``
tokens (in pages of ``--page-size``), so pages of finished requests are used
again.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (default 16)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    print("[trace_run] loading the engine ...", file=sys.stderr, flush=True)
    import numpy as np

    from .engine import ModelRunner, StepEntry, load_model

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    model = load_model(args.model, args.dtype, args.device)
    pages = max(1, -(-args.max_tokens // args.page_size))
    runner = ModelRunner(model, num_pages=pages, page_size=args.page_size, max_requests=8,
                         enable_prefix_caching=False, watermark=0.0)
    manager = runner.manager
    print(f"[trace_run] ready: {pages} pages of {args.page_size} tokens", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = []
        for e in rec.get("entries", []):
            rid, tokens = e["id"], [int(t) for t in e["tokens"]]
            if manager.has_request(rid):
                manager.append_slots(rid, tokens)
            else:
                alloc = manager.allocate(rid, tokens, respect_watermark=False)
                runner.start_request(rid, alloc.state_slot)
            entries.append(StepEntry(rid, tokens, [int(w) for w in e.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                logits.cpu().numpy().astype("<f4").tofile(out_dir / f"{rec['step']}.f32")
        for rid in rec.get("end", []):
            if manager.has_request(rid):
                manager.free(rid)
        print(f"done {rec['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
