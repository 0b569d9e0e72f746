"""The same question as tests/test_mutants.py, for the Python that wires the model together: one-line
faults in the parts, the model's loop over the run order, the cache pools and the weights' layout must show
in the logits that the engine computes on the CPU stand-ins (tests/cpu_ops.py), whole, in portions and token by
token, in float32 and in bfloat16.  No GPU."""

import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import dli_b200
from dli_b200.engine import ModelRunner, StepEntry
from dli_b200.parts import block as block_mod
from dli_b200.parts import mlp as mlp_mod
from dli_b200.parts import model as model_mod
from dli_b200.parts import rotary as rotary_mod
from dli_b200.parts.attention import GQAttention
from dli_b200.parts.base import ResidualStream
from tests import cpu_ops
from tests.plain import llama_plain as plain
from tests.test_mutants import mutate
from tests.util import make_model_dir, plain_weights_for, random_tokens

TOLS = {"float32": 2e-4, "bfloat16": 5e-2}


def logits_every_way(name: str, dtype: str) -> None:
    """Raises when the engine's logits differ from the plain ones, whole or cut."""
    with tempfile.TemporaryDirectory() as tmp, cpu_ops.patched():
        cfg, weights, page = make_model_dir(Path(tmp), name, sharpen=6.0)
        w = plain_weights_for(weights, dtype)
        model = dli_b200.load_model(tmp, dtype, "cpu")
        toks = random_tokens(cfg["vocab_size"], 41, seed=6)
        want = plain.forward(cfg, w, toks)
        runner = ModelRunner(model, num_pages=14, page_size=page, cuda_graphs=False, enable_prefix_caching=False, watermark=0.0)
        runner.manager.allocate("x", toks)
        got = runner.step([StepEntry("x", toks, list(range(len(toks))))]).numpy()
        np.testing.assert_allclose(got, want, atol=TOLS[dtype])
        runner.manager.free("x")
        runner.manager.allocate("y", toks[:30])
        rows, at = [], 0
        for n in (9, 2, 12, 4, 3):
            rows.append(runner.step([StepEntry("y", toks[at : at + n], list(range(n)))]))
            at += n
        for t in toks[30:]:
            runner.manager.append_slots("y", [t])
            rows.append(runner.step([StepEntry("y", [t], [0])]))
        np.testing.assert_allclose(torch.cat(rows).numpy(), want, atol=TOLS[dtype])


def detect():
    for name in ("tiny_a", "tiny_b", "tiny_c"):
        for dtype in ("float32", "bfloat16"):
            logits_every_way(name, dtype)


MUTANTS = {
    "llama3 scaling leaves the long wavelengths alone": (rotary_mod, "inverse_frequencies", "torch.where(wavelen > old / low, inv / factor, inv)", "torch.where(wavelen > old / low, inv, inv)"),
    "linear scaling multiplies": (rotary_mod, "inverse_frequencies", "return inv / float(params[\"factor\"])", "return inv * float(params[\"factor\"])"),
    "the feed-forward's output of the layer before is forgotten": (block_mod.PreNormBlock, "forward", "stream.take_pending(), self.mixer)", "None, self.mixer)"),
    "the mixer's output is not added": (block_mod.PreNormBlock, "forward", "normed_input(self.ffn_norm, stream.h, a, self.ffn)", "normed_input(self.ffn_norm, stream.h, None, self.ffn)"),
    "every layer writes into the first layer's cache": (model_mod.DecoderModel, "forward", "forward(stream, batch, caches[i])", "forward(stream, batch, caches[0])"),
    "the last layer's output misses the final norm": (model_mod.DecoderModel, "forward", "stream.take_pending(), self.head, rows=rows)", "None, self.head, rows=rows)"),
    "gate and up change places": (mlp_mod.SwiGLU, "load", 'gate, up = tensors[px + "gate_proj.weight"], tensors[px + "up_proj.weight"]', 'up, gate = tensors[px + "gate_proj.weight"], tensors[px + "up_proj.weight"]'),
    "keys and values change places at load": (GQAttention, "load", 'tensors[px + "k_proj.weight"], tensors[px + "v_proj.weight"]], 0)', 'tensors[px + "v_proj.weight"], tensors[px + "k_proj.weight"]], 0)'),
    "the scale of the scores is lost": (GQAttention, "forward", "self.nh, self.scale, self.window,", "self.nh, 1.0, self.window,"),
    "a pending product is dropped instead of computed": (ResidualStream, "take_pending", "return self._pending", "return None if type(self._pending).__name__ == 'PendingProduct' else self._pending"),
}


@pytest.mark.timeout(300)
@pytest.mark.parametrize("name", list(MUTANTS), ids=lambda n: n.replace(" ", "_"))
def test_model_mutant_is_noticed(name, monkeypatch):
    owner, method, old, new = MUTANTS[name]
    mutate(monkeypatch, owner, method, old, new)
    with pytest.raises(AssertionError):
        detect()


def test_without_a_mutant_the_logits_agree():
    detect()
