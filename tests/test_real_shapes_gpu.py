"""Replay at the layer sizes of the benchmark models (few layers, random weights): the kernels
that tiny models never reach — 64-wide heads on the tcgen05 and TMA paths, 128-wide heads,
thousands of features per product, a six-digit vocabulary — against the plain implementation."""

import numpy as np
import pytest
import torch

import dli_b200
from dli_b200.engine import ModelRunner, StepEntry
from dli_b200.weights import write_safetensors
from tests.plain import llama_plain as plain
from tests.util import plain_weights_for, random_tokens

pytestmark = pytest.mark.gpu

LLAMA_1B_2L = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "rms_norm_eps": 1e-5,
}
LLAMA_3B_1L = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 1, "hidden_size": 3072,
    "num_attention_heads": 24, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 8192, "vocab_size": 32000,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "rms_norm_eps": 1e-5,
}
SMOLLM2_1L = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 1, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 49152,
    "rope_theta": 130000.0, "tie_word_embeddings": True, "rms_norm_eps": 1e-5,
}


@pytest.fixture(scope="module", params=["llama_1b", "llama_3b", "smollm2"])
def case(request, tmp_path_factory):
    cfg = {"llama_1b": LLAMA_1B_2L, "llama_3b": LLAMA_3B_1L, "smollm2": SMOLLM2_1L}[request.param]
    path = tmp_path_factory.mktemp(request.param)
    dli_b200.write_model_dir(path, cfg, seed=7)
    # sharpen attention as the tiny-model tests do
    w = {k: torch.from_numpy(v.copy()) for k, v in plain.read_safetensors(path / "model.safetensors").items()}
    for k in w:
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            w[k] = w[k] * 3.0
    write_safetensors(path / "model.safetensors", w)
    weights = {k: v.numpy() for k, v in w.items()}
    tokens = random_tokens(cfg["vocab_size"], 300, seed=3)
    return cfg, path, weights, tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_decode_and_batch_at_real_sizes(case, dtype):
    cfg, path, weights, tokens = case
    want = plain.forward(cfg, plain_weights_for(weights, dtype), tokens)
    scale = float(np.abs(want).max())
    tol = (2e-4 if dtype == "float32" else 5e-2) * max(1.0, scale)
    model = dli_b200.load_model(path, dtype)
    r = ModelRunner(model, num_pages=48, page_size=16, max_requests=4, enable_prefix_caching=False, watermark=0.0)

    def run(rid, cuts, want_rows):
        """Feed ``tokens`` in the given portions; logits of every position."""
        pos, parts = 0, []
        for n in cuts:
            piece = tokens[pos : pos + n]
            if r.manager.has_request(rid):
                r.manager.append_slots(rid, piece)
            else:
                r.manager.allocate(rid, piece)
            parts.append(r.step([StepEntry(rid, piece, range(n))]))
            pos += n
        r.manager.free(rid)
        return torch.cat(parts).cpu().numpy()

    whole = run("w", [300], None)
    err = np.abs(whole - want).max(axis=1)
    assert err.max() <= tol, f"whole: first wrong position {int(np.argmax(err > tol))} (error {err.max():.3g}, tolerance {tol:.3g})"
    cut = run("c", [129, 2, 64, 5, 70] + [1] * 30, None)
    err = np.abs(cut - want).max(axis=1)
    assert err.max() <= tol, f"portions + decode: first wrong position {int(np.argmax(err > tol))} (error {err.max():.3g})"

    # two requests side by side: a decoded token of one beside a portion of the other
    r.manager.allocate("a", tokens[:200])
    r.step([StepEntry("a", tokens[:200], [])])
    r.manager.allocate("b", tokens[:150])
    r.manager.append_slots("a", tokens[200:201])
    out = r.step([StepEntry("b", tokens[:150], [149]), StepEntry("a", tokens[200:201], [0])]).cpu().numpy()
    assert np.abs(out[0] - want[149]).max() <= tol and np.abs(out[1] - want[200]).max() <= tol
    # both decode together (the replayed graph)
    r.manager.append_slots("a", tokens[201:202])
    r.manager.append_slots("b", tokens[150:151])
    out = r.step([StepEntry("a", tokens[201:202], [0]), StepEntry("b", tokens[150:151], [0])]).cpu().numpy()
    assert np.abs(out[0] - want[201]).max() <= tol and np.abs(out[1] - want[150]).max() <= tol
    r.manager.check_invariants()
