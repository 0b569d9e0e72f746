"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]

The default run has the layer sizes of Llama-3.2-1B with random bfloat16 weights, 8 sequences
prefilled to 2,048 tokens each and then decoded (pool sized for a context of 4,096).  A step
is one decode step.  One JSON line is printed:

  value        decoded tokens a second, device-timed over exactly K steps (CUDA events)
  e2e          the same through LLMEngine.step(): host token ids in (pinned, copied every step),
               sampled token ids out (read back every step)
  prefill      one 2,048-token prompt in one step: tokens a second, ms, fraction of the bf16 peak
  roofline     bytes the decode step must read (every weight once + the live cache) / its time
  points       decoded tokens a second at batch 1 and 64
  clocks       SM clock and throttle reasons sampled while the timed steps ran

Each timed step reads all weights (2.5 GB), far more than the 126 MB L2, so no flush is needed.
For --gpus > 1 it prints one line saying so and exits with 2.
"""

import argparse
import json
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA_3_2_1B = json.loads((ROOT / "distributed-llm-inference_b200" / "config" / "shapes" / "llama-3.2-1b.json").read_text())
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
        except Exception:
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """nvidia-smi in the background while timed steps run; settings are only read."""

    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        self.lines += [line for line in out.splitlines() if line.strip()]
        self.proc = None

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            try:
                sm.append(float(f[0])), mx.append(float(f[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes(model):
    """Bytes of every tensor a decode step reads once (the embedding matrix counts once: it is
    the head; the few embedding rows gathered are negligible)."""
    seen, total = set(), 0
    for part in model.parts():
        for t in vars(part).values():
            if hasattr(t, "data_ptr") and hasattr(t, "numel") and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
    return total


def cache_bytes_per_token(model):
    from dli_b200.cache import PagedKVNeed

    return sum(2 * n.num_kv_heads * n.head_dim * model.dtype.itemsize for n in model.cache_needs() if isinstance(n, PagedKVNeed))


def prefill_flops(cfg, layers, tokens):
    H, I, d, nh, nkv, V = (cfg[k] for k in ("hidden_size", "intermediate_size", "head_dim", "num_attention_heads", "num_key_value_heads", "vocab_size"))
    per_token = 2 * (H * (nh + 2 * nkv) * d + nh * d * H + 3 * H * I)
    attention = 2 * tokens * tokens * d * nh  # QK^T and PV over the causal half
    return layers * (tokens * per_token + attention) + 2 * H * V


def make_engine(model, batch, steps_total):
    from dli_b200 import LLMEngine, SchedulerConfig

    pages = batch * (CONTEXT // PAGE) + 8
    return LLMEngine.for_model(model, num_blocks=pages, block_size=PAGE, config=SchedulerConfig(max(batch, 1), PROMPT_LEN),
                               enable_prefix_caching=False, watermark=0.0)


def decode_device_timed(model, batch, steps, warmup, sampler_clock=None, graphs=True):
    """K decode steps timed on the device: step function plus greedy sampling.  Each step runs on
    the ids the step before sampled, taken on the device; the host reads every step's ids, one
    step late (the engine's own way of stepping)."""
    import torch

    from dli_b200.cache import UNKNOWN_TOKEN
    from dli_b200.engine import ModelRunner, StepEntry
    from dli_b200.kernels import ops
    from dli_b200.sampling import Sampler, SamplingParams

    runner = ModelRunner(model, num_pages=batch * (CONTEXT // PAGE) + 8, page_size=PAGE, max_requests=batch,
                         enable_prefix_caching=False, watermark=0.0, cuda_graphs=graphs)
    sampler = Sampler(model.device)
    g = torch.Generator().manual_seed(1)
    vocab = model.spec.vocab_size
    params = [SamplingParams()] * batch
    tokens = []
    for b in range(batch):
        prompt = torch.randint(1000, vocab, (PROMPT_LEN,), generator=g).tolist()
        runner.manager.allocate(b, prompt)
        logits = runner.step([StepEntry(b, prompt, [PROMPT_LEN - 1])])
        tokens.append(sampler.sample(logits, params[:1], [0], [0])[0])

    def launch(prev):
        """One decode step of every request, launched on the ids the step before left on the device
        (``prev``: PendingTokens), as LLMEngine.step does; the host reads those ids afterwards."""
        entries = []
        for b in range(batch):
            runner.manager.append_slots(b, [UNKNOWN_TOKEN])  # no prefix index in this run: the id is never needed
            entries.append(StepEntry(b, [0], [0], token_src=b))
        logits = runner.step(entries, borrow=True, token_source=prev.device_ids)
        return sampler.sample_async(logits, params, [0] * batch, [0] * batch)

    # the first step runs on ids the host knows
    for b in range(batch):
        runner.manager.append_slots(b, [tokens[b]])
    flight = sampler.sample_async(runner.step([StepEntry(b, [tokens[b]], [0]) for b in range(batch)], borrow=True),
                                  params, [0] * batch, [0] * batch)

    def one_step(flight):
        ahead = launch(flight)
        ids = flight.result()  # this step's tokens reach the host while the next step runs
        assert len(ids) == batch
        return ahead

    for _ in range(warmup):
        flight = one_step(flight)
    flight.result()
    ctx_start = runner.manager.num_tokens(0)
    torch.cuda.synchronize()
    if sampler_clock:
        sampler_clock.start()
    launches = ops.launch_count
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        flight = one_step(flight)
    end.record()
    torch.cuda.synchronize()
    flight.result()
    if sampler_clock:
        sampler_clock.stop()
    ms = start.elapsed_time(end) / steps
    mean_ctx = ctx_start + steps / 2
    for b in range(batch):
        runner.manager.free(b)
    del runner
    torch.cuda.empty_cache()
    return {"ms": ms, "tok_s": batch * 1000.0 / ms, "launches": ops.launch_count - launches, "mean_ctx": mean_ctx}


def decode_end_to_end(model, batch, steps, warmup):
    """K steps of LLMEngine.step(): every step copies its token ids and tables from pinned host
    memory to the device and reads the sampled ids back."""
    import torch

    from dli_b200 import SamplingParams

    eng = make_engine(model, batch, steps + warmup)
    g = torch.Generator().manual_seed(2)
    for b in range(batch):
        eng.add_request(f"r{b}", torch.randint(1000, model.spec.vocab_size, (PROMPT_LEN,), generator=g).tolist(),
                        SamplingParams(max_tokens=CONTEXT - PROMPT_LEN, ignore_eos=True))
    while any(r.num_computed_tokens < PROMPT_LEN for r in eng.scheduler.running + list(eng.scheduler.waiting)):
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        out = eng.step()
        assert len(out) == batch
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = eng.runner.uploader.bytes_last  # what the last step copied from pinned memory: token ids, positions, lengths, slots, block tables
    while eng.has_unfinished():
        for rid in [r.request_id for r in eng.scheduler.running]:
            eng.abort(rid)
    return {"value": batch * steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch, "ms_per_step": dt / steps * 1e3}


def prefill_timed(model, cfg, layers, peak_tflops, reps=5, warmup=3):
    import torch

    from dli_b200.engine import ModelRunner, StepEntry

    runner = ModelRunner(model, num_pages=PROMPT_LEN // PAGE + 8, page_size=PAGE, max_requests=2, enable_prefix_caching=False, watermark=0.0)
    g = torch.Generator().manual_seed(3)
    times = []
    for i in range(warmup + reps):
        prompt = torch.randint(1000, model.spec.vocab_size, (PROMPT_LEN,), generator=g).tolist()
        runner.manager.allocate("p", prompt)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry("p", prompt, [PROMPT_LEN - 1])])
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(end))
        runner.manager.free("p")
    ms = statistics.median(times)
    flops = prefill_flops(cfg, layers, PROMPT_LEN)
    return {"value": PROMPT_LEN * 1000.0 / ms, "tokens": PROMPT_LEN, "ms": ms, "frac": flops / (ms * 1e-3) / (peak_tflops * 1e12),
            "flops": flops, "unit": "tokens/s"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=LLAMA_3_2_1B["num_hidden_layers"], help="fewer layers than the model has, if memory or time needs it")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the main batch size (for profiling runs)")
    ap.add_argument("--phase", default="all", choices=["all", "decode", "prefill"],
                    help="profiling runs: only the device-timed decode steps, or only the prefill step (prints a short line)")
    ap.add_argument("--no-graphs", action="store_true", help="profiling runs: launch the decode step's kernels one by one")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference's build backend (hatchling) is neither installed nor in the offline wheelhouse, so pip cannot build it here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch

    import dli_b200
    from dli_b200.kernels import ops  # noqa: F401

    cfg = dict(LLAMA_3_2_1B, num_hidden_layers=args.layers)
    pk = peaks()
    model = dli_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    clocks = ClockSampler()
    if args.phase == "decode":
        run = decode_device_timed(model, args.batch, args.steps, args.warmup, graphs=not args.no_graphs)
        print(json.dumps({"phase": "decode", "batch": args.batch, "layers": args.layers, **run}))
        return 0
    if args.phase == "prefill":
        print(json.dumps({"phase": "prefill", "layers": args.layers, **prefill_timed(model, cfg, args.layers, pk["bf16_tflops"], reps=args.steps)}))
        return 0
    main_run = decode_device_timed(model, args.batch, args.steps, args.warmup, clocks)
    clocks.start()  # the end-to-end steps are timed too: keep sampling
    e2e = decode_end_to_end(model, args.batch, args.steps, args.warmup)
    clocks.stop()
    prefill = prefill_timed(model, cfg, args.layers, pk["bf16_tflops"])
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(decode_device_timed(model, b, args.steps, args.warmup)["tok_s"], 1)

    step_bytes = weight_bytes(model) + args.batch * main_run["mean_ctx"] * cache_bytes_per_token(model)
    achieved = step_bytes / (main_run["ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B shape, random bf16 weights, context 2048..4096)",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, seeded random weights", "impl": "ours",
        "config": {
            "model": "Llama-3.2-1B shape", "layers": args.layers, "layers_full": LLAMA_3_2_1B["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": args.batch, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "block_size": PAGE,
            "rope": "llama3 factor 32", "tied_embeddings": True, "parallelism": "1 GPU",
            "l2": "each step reads 2.5 GB of weights (> 126 MB L2); no flush", "peaks": pk["source"],
        },
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main_run["launches"],
        "prefill": {k: (round(v, 4) if isinstance(v, float) else v) for k, v in prefill.items()},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
