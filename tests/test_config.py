"""Typed configuration and the architecture registry (no GPU)."""

import copy

import numpy as np
import pytest

from dli_b200.config import (Architecture, LlamaConfig, UnsupportedModelError, llama_model_spec, register_architecture,
                             resolve_architecture, unregister_architecture)
from dli_b200.config.spec import ModelSpec, RunStep
from tests.tiny_configs import TINY_A, TINY_B, TINY_C


def test_tiny_configs_parse_and_differ():
    a, b, c = (LlamaConfig.from_hf_dict(x) for x in (TINY_A, TINY_B, TINY_C))
    assert (a.num_layers, a.hidden_size, a.num_heads, a.num_kv_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (b.num_layers, b.hidden_size, b.num_heads, b.num_kv_heads, b.head_dim) == (3, 96, 3, 1, 32)
    assert b.rope.rope_type == "llama3" and b.rope.factor == 8.0 and b.rope.original_max_position_embeddings == 64
    assert a.rope.rope_type == "default" and a.tie_word_embeddings and not b.tie_word_embeddings
    for key in ("num_layers", "hidden_size", "num_heads", "num_kv_heads", "head_dim", "intermediate_size", "vocab_size", "rms_norm_eps"):
        assert len({getattr(x, key) for x in (a, b, c)}) == 3 or key == "num_kv_heads"


def test_defaults_follow_the_reference():
    cfg = {"model_type": "llama", "vocab_size": 10, "hidden_size": 32, "intermediate_size": 8, "num_hidden_layers": 1,
           "num_attention_heads": 4, "rms_norm_eps": 1e-5}
    c = LlamaConfig.from_hf_dict(cfg)
    assert c.num_kv_heads == 4 and c.head_dim == 8 and c.max_position_embeddings == 4096
    assert c.rope.theta == 10000.0 and c.rope.rope_type == "default" and not c.tie_word_embeddings


def test_rms_norm_eps_is_required():
    cfg = dict(TINY_A)
    del cfg["rms_norm_eps"]
    with pytest.raises(KeyError):
        LlamaConfig.from_hf_dict(cfg)


def test_rope_parameters_win_and_legacy_type_key():
    cfg = copy.deepcopy(TINY_B)
    cfg["rope_parameters"] = {"rope_type": "llama3", "factor": 4.0, "rope_theta": 1234.0}
    c = LlamaConfig.from_hf_dict(cfg)
    assert c.rope.factor == 4.0 and c.rope.theta == 1234.0 and c.rope.original_max_position_embeddings == 64
    cfg = copy.deepcopy(TINY_B)
    cfg["rope_scaling"] = {"type": "llama3", "factor": 2.0}
    c = LlamaConfig.from_hf_dict(cfg)
    assert c.rope.rope_type == "llama3" and c.rope.original_max_position_embeddings == 256  # falls back to max_position_embeddings
    cfg["rope_scaling"] = {"type": "llama3"}
    with pytest.raises(KeyError):
        LlamaConfig.from_hf_dict(cfg)


@pytest.mark.parametrize("override, word", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"use_sliding_window": True}, "sliding"),
    ({"layer_types": ["full_attention", "sliding_attention"]}, "sliding"),
    ({"pretraining_tp": 2}, "pretraining_tp"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type"),
    ({"rope_scaling": {"rope_type": "dynamic", "factor": 2.0}}, "rope_type"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"head_dim": 15}, "head_dim"),
    ({"model_type": "qwen2"}, "model_type"),
])
def test_unsupported_features_name_their_key(override, word):
    with pytest.raises(UnsupportedModelError, match=word):
        LlamaConfig.from_hf_dict({**TINY_A, **override})


def test_round_trip_through_config_json():
    for cfg in (TINY_A, TINY_B, TINY_C):
        c = LlamaConfig.from_hf_dict(cfg)
        assert LlamaConfig.from_hf_dict(c.to_hf_dict()) == c


def test_registry_by_architecture_then_model_type():
    assert resolve_architecture(TINY_A).name == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(UnsupportedModelError, match="MysteryLM"):
        resolve_architecture({"architectures": ["MysteryLM"]})
    with pytest.raises(UnsupportedModelError, match="model_type"):
        resolve_architecture({"model_type": "mystery"})
    register_architecture(Architecture("MysteryLM", LlamaConfig.from_hf_dict, llama_model_spec))
    try:
        assert resolve_architecture({"architectures": ["MysteryLM"]}).name == "MysteryLM"
    finally:
        unregister_architecture("MysteryLM")


def test_spec_carries_every_size_and_the_run_order():
    spec = llama_model_spec(LlamaConfig.from_hf_dict(TINY_B))
    assert len(spec.layers) == 3 and [s.layer for s in spec.run_order] == [0, 1, 2]
    mixer = spec.layers[1].parts["mixer"]
    assert mixer.kind == "gqa_attention" and mixer.params["num_kv_heads"] == 1 and mixer.params["head_dim"] == 32
    assert mixer.params["position"].params["scaling"] == "llama3"
    assert mixer.prefix == "model.layers.1.self_attn."
    assert spec.head.params["tied_to"] is None
    assert llama_model_spec(LlamaConfig.from_hf_dict(TINY_A)).head.params["tied_to"] == "model.embed_tokens.weight"


def test_run_order_is_validated():
    spec = llama_model_spec(LlamaConfig.from_hf_dict(TINY_A))
    with pytest.raises(ValueError, match="names layer"):
        ModelSpec(spec.hidden_size, spec.vocab_size, spec.embedding, spec.layers, (RunStep(5),), spec.final_norm, spec.head)
    with pytest.raises(ValueError, match="earlier"):
        ModelSpec(spec.hidden_size, spec.vocab_size, spec.embedding, spec.layers, (RunStep(0, cache_of=0),), spec.final_norm, spec.head)
    ok = ModelSpec(spec.hidden_size, spec.vocab_size, spec.embedding, spec.layers,
                   (RunStep(0), RunStep(1), RunStep(0), RunStep(1, cache_of=1)), spec.final_norm, spec.head)
    assert len(ok.run_order) == 4


def test_linear_rope_scaling_divides_every_frequency():
    from tests.plain import llama_plain as plain
    from tests.tiny_configs import TINY_C

    c = LlamaConfig.from_hf_dict(TINY_C)
    assert c.rope.rope_type == "linear" and c.rope.factor == 2.5
    position = llama_model_spec(c).layers[0].parts["mixer"].params["position"]
    assert position.params["scaling"] == "linear" and position.params["factor"] == 2.5
    pc = plain.read_config(TINY_C)
    base = plain.inverse_frequencies({**pc, "rope_type": "default"})
    assert np.allclose(plain.inverse_frequencies(pc), base / np.float32(2.5), rtol=1e-7)
    with pytest.raises(KeyError):
        LlamaConfig.from_hf_dict({**TINY_C, "rope_scaling": {"type": "linear"}})
    assert LlamaConfig.from_hf_dict(c.to_hf_dict()).rope == c.rope  # survives the round trip through config.json


def test_same_outcomes_as_the_reference_parser():
    """tests/golden/config_and_hash.json (made by tests/golden/make_config_hash_golden.py from the reference's
    ModelConfig.from_hf_dict): every config.json there parses to the same fields here, or is refused in the
    same way (a key that is missing, a feature that is not supported)."""
    import dataclasses
    import json
    from pathlib import Path

    golden = json.loads((Path(__file__).parent / "golden" / "config_and_hash.json").read_text())
    for i, case in enumerate(golden["configs"]):
        cfg, outcome = case["config"], case["outcome"]
        try:
            parsed = LlamaConfig.from_hf_dict(cfg)
        except UnsupportedModelError:
            assert outcome == {"error": "unsupported"}, f"config {i}: refused here, the reference gives {outcome}"
            continue
        except KeyError:
            assert outcome == {"error": "missing key"}, f"config {i}: a key is missed here, the reference gives {outcome}"
            continue
        assert "ok" in outcome, f"config {i}: parsed here, the reference gives {outcome}"
        want = outcome["ok"]
        got = dataclasses.asdict(parsed)
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_layers", "num_heads", "num_kv_heads", "head_dim",
                    "max_position_embeddings", "tie_word_embeddings"):
            assert got[key] == want[key], f"config {i}: {key}"
        assert got["rms_norm_eps"] == pytest.approx(want["rms_norm_eps"])
        for key in ("theta", "rope_type", "factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings"):
            assert got["rope"][key] == want["rope"][key], f"config {i}: rope.{key}"
