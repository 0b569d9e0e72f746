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

With ``--prefix-caching`` the cache manager's prefix index is on: full pages of a finished (or live)
request stay findable by the hash chain of their tokens, and a new request whose tokens begin the
same way is not run over them again.  Only pages that lie wholly before the first place whose logits
the request's first entry wants are taken from the index, so every wanted place is still computed;
a line on standard error says how many tokens of a request were found.
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
    ap.add_argument("--prefix-caching", action="store_true", help="reuse indexed pages of earlier requests that begin with the same tokens")
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
                         enable_prefix_caching=args.prefix_caching, watermark=0.0)
    manager = runner.manager
    print(f"[trace_run] ready: {pages} pages of {args.page_size} tokens", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = []
        for e in rec.get("entries", []):
            rid, tokens, want = e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]
            if manager.has_request(rid):
                manager.append_slots(rid, tokens)
            else:
                # the index is asked about the tokens up to the first wanted place only (a hit never covers the
                # page of the last token it is asked about), so that place and all behind it are computed
                head = min(want) + 1 if want and args.prefix_caching else len(tokens)
                alloc = manager.allocate(rid, tokens[:head], respect_watermark=False)
                if head < len(tokens):
                    manager.append_slots(rid, tokens[head:])
                runner.start_request(rid, alloc.state_slot)
                found = alloc.num_cached_tokens
                if found:
                    print(f"[trace_run] request {rid}: {found} tokens found in the cache", file=sys.stderr, flush=True)
                    tokens, want = tokens[found:], [w - found for w in want]
            entries.append(StepEntry(rid, tokens, want))
        if entries:
            logits = runner.step(entries)
            host = logits.cpu().numpy() if logits.shape[0] else None
            runner.check_device_errors()  # the copy above waited for the step's kernels
            if host is not None:
                host.astype("<f4").tofile(out_dir / f"{rec['step']}.f32")
        for rid in rec.get("end", []):
            if manager.has_request(rid):
                manager.free(rid)
        print(f"done {rec['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
