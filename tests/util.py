"""Helpers of the GPU tests: tiny model folders, plain logits, and a driver for bin/trace_run."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

import dli_b200
from dli_b200.weights import write_safetensors
from tests.plain import llama_plain as plain
from tests.tiny_configs import TINY

ROOT = Path(__file__).resolve().parents[1]

# logits of the tiny models are of order 1
TOL = {"float32": 1e-4, "bfloat16": 5e-2}


def make_model_dir(path: Path, name: str, sharpen: float = 1.0):
    """A random-weights folder of a tiny configuration.  ``sharpen`` scales the query and key
    projections, so attention weights are far from uniform and one wrong or missing key
    changes the logits visibly (with N(0, 0.02) weights attention is almost an average)."""
    cfg, seed, page = TINY[name]
    dli_b200.write_model_dir(path, cfg, seed)
    if sharpen != 1.0:
        w = {k: torch.from_numpy(v.copy()) for k, v in plain.read_safetensors(path / "model.safetensors").items()}
        for k in w:
            if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
                w[k] = w[k] * sharpen
        write_safetensors(path / "model.safetensors", w)
    weights = plain.read_safetensors(path / "model.safetensors")
    return cfg, weights, page


def plain_weights_for(weights, dtype: str):
    """What the engine computes with: matrices rounded to bfloat16 in that mode, vectors kept."""
    if dtype == "float32":
        return weights
    return {k: (plain.round_to_bfloat16(v) if v.ndim == 2 else v) for k, v in weights.items()}


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


class TraceRun:
    """bin/trace_run as a child process, fed one step at a time."""

    def __init__(self, model_dir, dtype: str, out_dir, max_tokens: int, page_size: int | None = None, cwd=None, env=None,
                 prefix_caching: bool = False):
        self.out_dir = Path(out_dir)
        cmd = [str((Path(cwd) if cwd else ROOT) / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
               "--out", str(out_dir), "--max-tokens", str(max_tokens)]
        if page_size:
            cmd += ["--page-size", str(page_size)]
        self.err_path = None
        stderr = None
        if prefix_caching:
            cmd.append("--prefix-caching")
            self.err_path = Path(out_dir) / "stderr.txt"  # where trace_run says what it found in the cache
            stderr = open(self.err_path, "w")
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=stderr, text=True, cwd=cwd, env=env)
        if stderr is not None:
            stderr.close()
        self.step_no = 0

    def step(self, entries, end=()):
        """entries: [(id, tokens, want)].  Returns logits [wanted, vocab] or None."""
        rec = {"step": self.step_no, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries], "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {self.step_no}":
            raise RuntimeError(f"trace_run answered {line!r} (exit code {self.proc.poll()})")
        path = self.out_dir / f"{self.step_no}.f32"
        self.step_no += 1
        wanted = sum(len(w) for _, _, w in entries)
        if not wanted:
            assert not path.exists()
            return None
        return np.fromfile(path, dtype="<f4").reshape(wanted, -1)

    def close(self) -> int:
        self.proc.stdin.close()
        return self.proc.wait(timeout=120)

    def found_in_cache(self) -> dict[str, int]:
        """request -> tokens that trace_run reported as found in the prefix index (after close)."""
        out = {}
        for line in self.err_path.read_text().splitlines():
            if "tokens found in the cache" in line:
                words = line.split()
                out[words[2].rstrip(":")] = int(words[3])
        return out
