"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]

The default run has the layer sizes of Llama-3.2-1B with random bfloat16 weights, 8 sequences
prefilled to 2,048 tokens each and then decoded (pool sized for a context of 4,096).  A step
is one decode step.  After W warm-up steps, blocks of exactly K steps are timed (up to five, as
many as the context leaves room for) and the median block is reported.  One JSON line is printed:

  value        decoded tokens a second, device-timed over exactly K steps (CUDA events)
  e2e          the same through LLMEngine.step(): host token ids in (pinned, copied every step),
               sampled token ids out (read back every step)
  prefill      one 2,048-token prompt in one step: tokens a second, ms, fraction of the bf16 peak
  roofline     bytes the decode step must read (every weight once + the live cache) / its time
  points       decode at batch 1 and 64: tokens a second, ms, bytes a step, fraction of the HBM peak
  more         other shapes and contexts (decode at 16 K and 32 K tokens; Llama-3.2-3B sizes: a prompt
               of 8,000 tokens, decode behind it, 64 sequences at 2 K); left out with --skip-more
  clocks       SM clock and throttle reasons sampled while the timed steps ran

Each timed step reads all weights (2.5 GB), far more than the 126 MB L2, so no flush is needed.
For --gpus > 1 it prints one line saying so and exits with 2.

``--impl reference`` times the reference's own engine (its unmodified package, looked for under
baseline/_ref, through its LLMEngine.for_model / add_request / step) on the same shape, batch, steps
and warm-up and prints the same line with "impl": "reference"; nothing of this package is imported
on that path.  Where the package is not there, or does not run, it prints why in one line.
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

SHAPES = ROOT / "distributed-llm-inference_b200" / "config" / "shapes"
LLAMA_3_2_1B = json.loads((SHAPES / "llama-3.2-1b.json").read_text())
LLAMA_3_2_3B = json.loads((SHAPES / "llama-3.2-3b.json").read_text())
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE = 16
BLOCKS = 5  # timed blocks of --steps steps each; the median block is reported
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

    def __init__(self, gpu: str = "0"):
        self.proc = None
        self.lines = []
        self.gpu = gpu  # what nvidia-smi -i takes: an index, or the UUID of the device this process computes on

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
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


def device_id_for_smi() -> str:
    """The UUID of torch's device 0 (CUDA_VISIBLE_DEVICES may map it to any physical GPU of a shared
    machine; nvidia-smi counts physical ones), or "0" where torch does not tell."""
    import torch

    try:
        return "GPU-" + str(torch.cuda.get_device_properties(0).uuid)
    except Exception:
        return "0"


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
    from dli_b200.cache.needs import paged_need_of

    paged = [paged_need_of(n) for n in model.cache_needs()]
    return sum(2 * n.num_kv_heads * n.head_dim * model.dtype.itemsize for n in paged if n is not None)


def prefill_flops(cfg, layers, tokens):
    H, I, d, nh, nkv, V = (cfg[k] for k in ("hidden_size", "intermediate_size", "head_dim", "num_attention_heads", "num_key_value_heads", "vocab_size"))
    per_token = 2 * (H * (nh + 2 * nkv) * d + nh * d * H + 3 * H * I)
    attention = 2 * tokens * tokens * d * nh  # QK^T and PV over the causal half
    return layers * (tokens * per_token + attention) + 2 * H * V


def timed_blocks(steps: int, warmup: int, room: int) -> int:
    """How many blocks of ``steps`` steps fit into ``room`` more tokens of context after the warm-up."""
    return max(1, min(BLOCKS, (room - warmup - 2) // max(1, steps)))


def make_engine(model, batch, prompt_len=PROMPT_LEN, context=CONTEXT):
    from dli_b200 import LLMEngine, SchedulerConfig

    pages = batch * (context // PAGE) + 8
    return LLMEngine.for_model(model, num_blocks=pages, block_size=PAGE, config=SchedulerConfig(max(batch, 1), min(prompt_len, 8192)),
                               enable_prefix_caching=False, watermark=0.0)


def decode_device_timed(model, batch, steps, warmup, sampler_clock=None, graphs=True, prompt_len=PROMPT_LEN, context=CONTEXT,
                        portion=2048, blocks=None, sampling=None):
    """Blocks of K decode steps timed on the device: step function plus sampling (greedy, or with ``sampling``:
    SamplingParams that every request gets, bound to its state slot as the engine binds them).  Each step runs
    on the ids the step before sampled, taken on the device; the host reads every step's ids, one
    step late (the engine's own way of stepping).  Prompts are prefilled in portions of ``portion``."""
    import torch

    from dli_b200.cache import UNKNOWN_TOKEN
    from dli_b200.engine import ModelRunner, StepEntry
    from dli_b200.kernels import ops
    from dli_b200.sampling import Sampler, SamplingParams

    runner = ModelRunner(model, num_pages=batch * (context // PAGE) + 8, page_size=PAGE, max_requests=batch,
                         enable_prefix_caching=False, watermark=0.0, cuda_graphs=graphs)
    sampler = Sampler(model.device, max_requests=batch if sampling else 0)
    g = torch.Generator().manual_seed(1)
    vocab = model.spec.vocab_size
    params = [SamplingParams()] * batch
    for b in range(batch if sampling else 0):
        sampler.bind(b, sampling, (sampling.seed or 0) + b, 0)

    def sample_rows(logits):
        if sampling:
            return sampler.sample_slots_async(logits, list(range(batch)), all_greedy=False)
        return sampler.sample_async(logits, params, [0] * batch, [0] * batch)

    tokens = []
    for b in range(batch):
        prompt = torch.randint(1000, vocab, (prompt_len,), generator=g).tolist()
        runner.manager.allocate(b, prompt)
        for at in range(0, prompt_len, portion):
            part = prompt[at : at + portion]
            logits = runner.step([StepEntry(b, part, [len(part) - 1] if at + portion >= prompt_len else [])])
        tokens.append(sampler.sample(logits, params[:1], [0], [0])[0])

    def launch(prev):
        """One decode step of every request, launched on the ids the step before left on the device
        (``prev``: PendingTokens), as LLMEngine.step does; the host reads those ids afterwards."""
        entries = []
        for b in range(batch):
            runner.manager.append_slots(b, [UNKNOWN_TOKEN])  # no prefix index in this run: the id is never needed
            entries.append(StepEntry(b, [0], [0], token_src=b))
        return sample_rows(runner.step(entries, borrow=True, token_source=prev.device_ids))

    # the first step runs on ids the host knows
    for b in range(batch):
        runner.manager.append_slots(b, [tokens[b]])
    flight = sample_rows(runner.step([StepEntry(b, [tokens[b]], [0]) for b in range(batch)], borrow=True))

    def one_step(flight):
        ahead = launch(flight)
        ids = flight.result()  # this step's tokens reach the host while the next step runs
        assert len(ids) == batch
        return ahead

    for _ in range(warmup):
        flight = one_step(flight)
    flight.result()
    torch.cuda.synchronize()
    if sampler_clock:
        sampler_clock.start()
    runs = []
    for _ in range(blocks or timed_blocks(steps, warmup, context - prompt_len)):
        ctx_start = runner.manager.num_tokens(0)
        launches = ops.launch_count
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            flight = one_step(flight)
        end.record()
        torch.cuda.synchronize()
        runs.append({"ms": start.elapsed_time(end) / steps, "launches": ops.launch_count - launches, "mean_ctx": ctx_start + steps / 2})
    flight.result()
    if sampler_clock:
        sampler_clock.stop()
    for b in range(batch):
        runner.manager.free(b)
    del runner
    torch.cuda.empty_cache()
    runs.sort(key=lambda r: r["ms"])
    mid = runs[len(runs) // 2]
    return {**mid, "tok_s": batch * 1000.0 / mid["ms"], "blocks": len(runs), "block_ms": [round(r["ms"], 4) for r in runs]}


def decode_end_to_end(model, batch, steps, warmup):
    """Blocks of K steps of LLMEngine.step(): every step copies its token ids and tables from pinned
    host memory to the device and reads the sampled ids back.  The median block is reported."""
    import torch

    from dli_b200 import SamplingParams

    eng = make_engine(model, batch)
    g = torch.Generator().manual_seed(2)
    for b in range(batch):
        eng.add_request(f"r{b}", torch.randint(1000, model.spec.vocab_size, (PROMPT_LEN,), generator=g).tolist(),
                        SamplingParams(max_tokens=CONTEXT - PROMPT_LEN, ignore_eos=True))
    while any(r.num_computed_tokens < PROMPT_LEN for r in eng.scheduler.running + list(eng.scheduler.waiting)):
        eng.step()
    for _ in range(warmup):
        eng.step()
    times = []
    for _ in range(timed_blocks(steps, warmup, CONTEXT - PROMPT_LEN)):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            out = eng.step()
            assert len(out) == batch
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    h2d = eng.runner.uploader.bytes_last  # what the last step copied from pinned memory: token ids, positions, lengths, slots, block tables
    while eng.has_unfinished():
        for rid in [r.request_id for r in eng.scheduler.running]:
            eng.abort(rid)
    return {"value": batch * steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch, "ms_per_step": dt / steps * 1e3}


def prefill_timed(model, cfg, layers, peak_tflops, reps=5, warmup=3, tokens=PROMPT_LEN, graphs=True):
    import torch

    from dli_b200.engine import ModelRunner, StepEntry

    runner = ModelRunner(model, num_pages=tokens // PAGE + 8, page_size=PAGE, max_requests=2, enable_prefix_caching=False, watermark=0.0,
                         cuda_graphs=graphs)
    g = torch.Generator().manual_seed(3)
    times = []
    for i in range(warmup + reps):
        prompt = torch.randint(1000, model.spec.vocab_size, (tokens,), generator=g).tolist()
        runner.manager.allocate("p", prompt)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry("p", prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(end))
        runner.manager.free("p")
    del runner
    torch.cuda.empty_cache()
    ms = statistics.median(times)
    flops = prefill_flops(cfg, layers, tokens)
    return {"value": tokens * 1000.0 / ms, "tokens": tokens, "ms": ms, "frac": flops / (ms * 1e-3) / (peak_tflops * 1e12),
            "flops": flops, "unit": "tokens/s"}


def sampling_timed(vocab, reps=5, per_graph=8):
    """Microseconds of the sampling kernel alone, by what the rows ask for, at 1, 8 and 64 rows of ``vocab`` logits:
    a graph of ``per_graph`` launches, replayed ``reps`` times between two events."""
    import torch

    from dli_b200.kernels import ops

    dev = "cuda:0"
    modes = {"greedy": None, "temperature": (0.8, -1, 1.0), "top_k_50": (0.8, 50, 1.0), "top_p_0.9": (0.8, -1, 0.9), "top_k_50_top_p_0.9": (0.8, 50, 0.9)}
    out = {}
    for rows in (1, 8, 64):
        g = torch.Generator().manual_seed(rows)
        logits = (torch.randn(rows, vocab, generator=g) * 3).to(dev)
        ids = torch.empty(rows, dtype=torch.int32, device=dev)
        seed, draw = torch.arange(rows, dtype=torch.int64, device=dev), torch.zeros(rows, dtype=torch.int64, device=dev)
        for name, mode in modes.items():
            if mode is None:
                fn = lambda: ops.sample(ids, logits)
            else:
                t, k, p = (torch.full((rows,), mode[0], device=dev), torch.full((rows,), mode[1], dtype=torch.int32, device=dev),
                           torch.full((rows,), mode[2], device=dev))
                fn = lambda t=t, k=k, p=p: ops.sample(ids, logits, t, k, p, seed, draw)
            fn()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(per_graph):
                    fn()
            graph.replay()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(reps):
                graph.replay()
            end.record()
            torch.cuda.synchronize()
            out[f"rows{rows}_{name}"] = round(start.elapsed_time(end) * 1000.0 / reps / per_graph, 1)
    return out


def decode_point(model, batch, steps, warmup, hbm_gbs, **kw):
    """A decode measurement as a record: tokens a second, ms a step, the bytes a step has to read
    (every weight once and the live cache at the block's mean context) and their share of the HBM peak."""
    run = decode_device_timed(model, batch, steps, warmup, **kw)
    step_bytes = weight_bytes(model) + batch * run["mean_ctx"] * cache_bytes_per_token(model)
    gbs = step_bytes / (run["ms"] * 1e-3) / 1e9
    return {"tok_s": round(run["tok_s"], 1), "ms": round(run["ms"], 4), "bytes_per_step": int(step_bytes), "gb_s": round(gbs, 1),
            "frac": round(gbs / hbm_gbs, 4), "mean_ctx": run["mean_ctx"]}


def more_points(model_1b, steps, warmup, pk):
    """Beyond the headline: longer contexts at the 1B sizes, and the Llama-3.2-3B sizes (a prompt of 8,000
    tokens in one step, decode behind it, 64 sequences at a context of 2 K)."""
    import torch

    import dli_b200

    from dli_b200.sampling import SamplingParams

    steps = min(steps, 32)
    out = {}
    # the headline step with every request sampling at temperature 0.8 among the 50 likeliest tokens and 0.9 of their mass
    out["decode_b8_sampled"] = decode_point(model_1b, 8, steps, warmup, pk["hbm_gbs"], blocks=1,
                                            sampling=SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=1))
    # a short prompt in one step: launched kernel by kernel the host needs 2.3 ms for it; once the shape has come
    # often enough the step is replayed from a graph (engine/graphs.py, MixedGraph)
    short = prefill_timed(model_1b, LLAMA_3_2_1B, LLAMA_3_2_1B["num_hidden_layers"], pk["bf16_tflops"], reps=5, warmup=40, tokens=256)
    out["prefill_256"] = {"tok_s": round(short["value"], 1), "ms": round(short["ms"], 4), "frac": round(short["frac"], 4)}
    for name, batch, ctx in (("decode_b8_ctx16k", 8, 16384), ("decode_b1_ctx32k", 1, 32768), ("decode_b8_ctx32k", 8, 32768)):
        out[name] = decode_point(model_1b, batch, steps, warmup, pk["hbm_gbs"], prompt_len=ctx, context=ctx + 512, blocks=1)
    cfg = LLAMA_3_2_3B
    model = dli_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    pre = prefill_timed(model, cfg, cfg["num_hidden_layers"], pk["bf16_tflops"], reps=3, warmup=2, tokens=8000)
    out["3b_prefill_8000"] = {"tok_s": round(pre["value"], 1), "ms": round(pre["ms"], 3), "tflops": round(pre["flops"] / pre["ms"] / 1e9, 1),
                              "frac": round(pre["frac"], 4)}
    out["3b_decode_b1_ctx8k"] = decode_point(model, 1, steps, warmup, pk["hbm_gbs"], prompt_len=8000, context=8192 + 512, blocks=1)
    out["3b_decode_b8_ctx8k"] = decode_point(model, 8, steps, warmup, pk["hbm_gbs"], prompt_len=8000, context=8192 + 512, blocks=1)
    out["3b_decode_b64_ctx2k"] = decode_point(model, 64, steps, warmup, pk["hbm_gbs"], prompt_len=2048, context=2048 + 512, blocks=1)
    return out


def config_record(cfg, layers, batch, source, extra=None):
    rec = {
        "model": "Llama-3.2-1B shape", "layers": layers, "layers_full": LLAMA_3_2_1B["num_hidden_layers"],
        "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
        "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
        "global_batch": batch, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "block_size": PAGE,
        "rope": "llama3 factor 32", "tied_embeddings": True, "parallelism": "1 GPU",
        "l2": "each step reads 2.5 GB of weights (> 126 MB L2); no flush", "peaks": source,
    }
    rec.update(extra or {})
    return rec


METRIC = "decode tok/s at batch {batch} (Llama-3.2-1B shape, random bf16 weights, context 2048..4096)"


# ----------------------------------------------------------------------------------------------
# The reference arm: the reference's own package and engine, nothing of this repository's.

def reference_unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def reference_engine(model, batch, attention):
    """The reference's engine as its own server builds it: LLMEngine.for_model with its graph shapes for the
    resolved decode kernel (src/dli/engine/engine.py:92-145, src/dli/server/__main__.py:138-175)."""
    from dli.engine import LLMEngine, SchedulerConfig
    from dli.engine.cuda_graph import default_shapes
    from dli.model import paged_attention

    kernel = paged_attention.resolve(attention, "cuda")
    pages = batch * (CONTEXT // PAGE) + 8
    pages += pages // 100 + 2  # its block manager holds one page in a hundred back at admission
    eng = LLMEngine.for_model(model, num_blocks=pages, block_size=PAGE, config=SchedulerConfig(max_num_seqs=max(batch, 1), max_num_batched_tokens=PROMPT_LEN),
                              enable_prefix_caching=False, cuda_graphs=default_shapes(kernel), decode_attention=kernel)
    return eng, kernel


def reference_decode(model, batch, steps, warmup, attention, clock=None):
    """Method of benchmarks/scripts/engine_profile.py:49-70 of the reference: requests of random ids
    ``randint(1000, vocab)``, steps until every prompt is computed, warm-up steps, then timed ``eng.step()`` loops
    around a synchronize; here in blocks of K steps, once by CUDA events and once by the host's clock."""
    import torch

    from dli.sampling import SamplingParams

    eng, kernel = reference_engine(model, batch, attention)
    vocab = model.config.vocab_size
    g = torch.Generator().manual_seed(2)
    for b in range(batch):
        eng.add_request(f"r{b}", torch.randint(1000, vocab, (PROMPT_LEN,), generator=g).tolist(),
                        SamplingParams(max_tokens=CONTEXT - PROMPT_LEN, ignore_eos=True))
    while any(r.num_computed_tokens < PROMPT_LEN for r in eng.scheduler.running + list(eng.scheduler.waiting)):
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    blocks = max(1, timed_blocks(steps, warmup, 2560 - PROMPT_LEN) // 2)  # its widest graph holds 2,560 tokens
    if clock:
        clock.start()
    device_ms, host_ms = [], []
    for _ in range(blocks):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            assert len(eng.step()) == batch
        end.record()
        torch.cuda.synchronize()
        device_ms.append(start.elapsed_time(end) / steps)
    for _ in range(blocks):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            assert len(eng.step()) == batch
        torch.cuda.synchronize()
        host_ms.append((time.perf_counter() - t0) / steps * 1e3)
    if clock:
        clock.stop()
    ctx = statistics.mean(r.num_computed_tokens for r in eng.scheduler.running)
    graphs = getattr(eng.runner, "decode_graphs", None)
    summary = graphs.summary() if graphs is not None else None
    rows = next((g["batch"] for g in (summary or {}).get("graphs", []) if g["replays"]), batch)
    width = next((g["width_blocks"] for g in (summary or {}).get("graphs", []) if g["replays"]), -(-int(ctx) // PAGE))
    for rid in [r.request_id for r in eng.scheduler.running]:
        eng.abort(rid)
    del eng
    torch.cuda.empty_cache()
    return {"ms": statistics.median(device_ms), "host_ms": statistics.median(host_ms), "kernel": kernel, "mean_ctx": ctx,
            "graphs": None if summary is None else {"status": summary["status"], "replays": summary["replays"], "fallbacks": summary["fallbacks"]},
            "h2d": 8 * (4 * rows + rows * width), "d2h": 8 * batch}


def reference_prefill(model, attention, reps=3, warmup=2):
    """One prompt of 2,048 tokens as one step of the reference's engine (a pure prefill step as in
    benchmarks/scripts/pipeline_profile.py:60-103 of the reference)."""
    import torch

    from dli.sampling import SamplingParams

    eng, _ = reference_engine(model, 1, attention)
    g = torch.Generator().manual_seed(3)
    times = []
    for i in range(warmup + reps):
        eng.add_request(f"p{i}", torch.randint(1000, model.config.vocab_size, (PROMPT_LEN,), generator=g).tolist(), SamplingParams(max_tokens=1, ignore_eos=True))
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = eng.step()
        end.record()
        torch.cuda.synchronize()
        assert len(out) == 1 and out[0].finished
        if i >= warmup:
            times.append(start.elapsed_time(end))
    del eng
    torch.cuda.empty_cache()
    return statistics.median(times)


def reference_arm(args) -> int:
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "dli" / "engine" / "engine.py").exists():
        return reference_unavailable("no copy of the reference's package under baseline/_ref (its build backend, hatchling, is not installed, so pip "
                                     "cannot build it; a copy of its src/dli is what its pure wheel would install)")
    sys.path[:] = [p for p in sys.path if Path(p or ".").resolve() != ROOT]
    sys.path.insert(0, str(ref))
    try:
        import torch

        from dli.model.config import ModelConfig
        from dli.model.llama import LlamaForCausalLM
    except Exception as exc:
        return reference_unavailable(f"the reference's package does not import here: {type(exc).__name__}: {exc}")
    if not torch.cuda.is_available():
        return reference_unavailable("no CUDA device")
    cfg = dict(LLAMA_3_2_1B, num_hidden_layers=args.layers)
    pk = peaks()
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = LlamaForCausalLM(ModelConfig.from_hf_dict(cfg)).to(torch.bfloat16).eval()
    model.reset_rope(torch.device("cuda"))
    clocks = ClockSampler(device_id_for_smi())
    errors = []
    for attention in ("auto", "sdpa"):  # its Triton kernel first; should that not build or run on this GPU, its library attention
        try:
            with torch.inference_mode():
                main_run = reference_decode(model, args.batch, args.steps, args.warmup, attention, clocks)
                prefill_ms = reference_prefill(model, attention)
                points = {}
                if not args.skip_points:
                    for b in (1, 64):
                        run = reference_decode(model, b, args.steps, args.warmup, attention)
                        points[f"decode_b{b}"] = {"tok_s": round(b * 1000.0 / run["ms"], 1), "ms": round(run["ms"], 4),
                                                  "e2e_tok_s": round(b * 1000.0 / run["host_ms"], 1), "graphs": run["graphs"]}
            break
        except Exception as exc:  # noqa: BLE001 - whatever stops the reference is reported, not raised
            errors.append(f"decode_attention={attention}: {type(exc).__name__}: {exc}")
            clocks.stop()
            torch.cuda.synchronize()
    else:
        return reference_unavailable("the reference's engine does not run on this GPU: " + " | ".join(errors))
    weights = sum(p.numel() * p.element_size() for p in model.parameters())
    kv_token = 2 * args.layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    step_bytes = weights + args.batch * main_run["mean_ctx"] * kv_token
    achieved = step_bytes / (main_run["ms"] * 1e-3) / 1e9
    flops = prefill_flops(cfg, args.layers, PROMPT_LEN)
    line = {
        "metric": METRIC.format(batch=args.batch), "value": round(args.batch * 1000.0 / main_run["ms"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights (torch's default initialisation)",
        "impl": "reference",
        "config": config_record(cfg, args.layers, args.batch, pk["source"]),
        "e2e": {"value": round(args.batch * 1000.0 / main_run["host_ms"], 2), "unit": "tokens/s", "h2d_bytes_per_step": main_run["h2d"],
                "d2h_bytes_per_step": main_run["d2h"], "ms_per_step": round(main_run["host_ms"], 4)},
        "prefill": {"value": round(PROMPT_LEN * 1000.0 / prefill_ms, 1), "tokens": PROMPT_LEN, "ms": round(prefill_ms, 4),
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "flops": flops, "unit": "tokens/s"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
        "reference": {"decode_attention": main_run["kernel"], "cuda_graphs": main_run["graphs"], "earlier_errors": errors,
                      "path": "LLMEngine.for_model / add_request / step of the unmodified package under baseline/_ref"},
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=LLAMA_3_2_1B["num_hidden_layers"], help="fewer layers than the model has, if memory or time needs it")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the main batch size (for profiling runs)")
    ap.add_argument("--skip-more", action="store_true", help="leave out the other shapes and contexts (the \"more\" key)")
    ap.add_argument("--phase", default="all", choices=["all", "decode", "prefill", "sample"],
                    help="profiling runs: only the device-timed decode steps, only the prefill step, or only the sampling kernel (prints a short line)")
    ap.add_argument("--no-graphs", action="store_true", help="profiling runs: launch the step's kernels one by one")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN,
                    help="profiling runs: the context at which decoding starts (--phase decode), the prompt's length (--phase prefill)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return reference_arm(args)

    import torch

    import dli_b200
    from dli_b200.kernels import ops  # noqa: F401

    cfg = dict(LLAMA_3_2_1B, num_hidden_layers=args.layers)
    pk = peaks()
    if args.phase == "sample":
        print(json.dumps({"phase": "sample", "vocab": cfg["vocab_size"], "unit": "us", **sampling_timed(cfg["vocab_size"])}))
        return 0
    model = dli_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    clocks = ClockSampler(device_id_for_smi())
    if args.phase == "decode":
        run = decode_device_timed(model, args.batch, args.steps, args.warmup, graphs=not args.no_graphs, blocks=1, prompt_len=args.prompt_len,
                                  context=max(CONTEXT, args.prompt_len + 512))
        print(json.dumps({"phase": "decode", "batch": args.batch, "layers": args.layers, "prompt_len": args.prompt_len, **run}))
        return 0
    if args.phase == "prefill":
        print(json.dumps({"phase": "prefill", "layers": args.layers, "graphs": not args.no_graphs,
                          **prefill_timed(model, cfg, args.layers, pk["bf16_tflops"], reps=args.steps, warmup=args.warmup, tokens=args.prompt_len,
                                          graphs=not args.no_graphs)}))
        return 0
    main_run = decode_device_timed(model, args.batch, args.steps, args.warmup, clocks)
    clocks.start()  # the end-to-end steps are timed too: keep sampling
    e2e = decode_end_to_end(model, args.batch, args.steps, args.warmup)
    clocks.stop()
    prefill = prefill_timed(model, cfg, args.layers, pk["bf16_tflops"])
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = decode_point(model, b, args.steps, args.warmup, pk["hbm_gbs"])

    step_bytes = weight_bytes(model) + args.batch * main_run["mean_ctx"] * cache_bytes_per_token(model)
    achieved = step_bytes / (main_run["ms"] * 1e-3) / 1e9
    line = {
        "metric": METRIC.format(batch=args.batch),
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, seeded random weights", "impl": "ours",
        "config": config_record(cfg, args.layers, args.batch, pk["source"]),
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main_run["launches"],
        "timed_blocks": {"blocks": main_run["blocks"], "ms_per_step": main_run["block_ms"], "reported": "median"},
        "prefill": {k: (round(v, 4) if isinstance(v, float) else v) for k, v in prefill.items()},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
        "clocks": clocks.summary(),
    }
    if not args.skip_more and args.layers == LLAMA_3_2_1B["num_hidden_layers"]:
        line["more"] = more_points(model, args.steps, args.warmup, pk)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
