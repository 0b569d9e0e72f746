"""Strict loading by tensor name and the random-weights mode (no GPU)."""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

import dli_b200
from dli_b200.config import resolve_architecture
from dli_b200.parts import declared_tensors
from dli_b200.weights import CheckpointError, SafetensorsFile, load_tensors, random_tensors, write_safetensors
from tests.plain import llama_plain as plain
from tests.tiny_configs import TINY_A, TINY_B


def _declared(cfg):
    arch = resolve_architecture(cfg)
    return declared_tensors(arch.model_spec(arch.parse_config(cfg)))


def test_written_folder_reads_back(tmp_path):
    dli_b200.write_model_dir(tmp_path, TINY_B, seed=1)
    assert json.loads((tmp_path / "config.json").read_text())["num_hidden_layers"] == 3
    decl = _declared(TINY_B)
    got = load_tensors(tmp_path, decl, torch.float32, "cpu")
    theirs = plain.read_safetensors(tmp_path / "model.safetensors")
    assert set(got) == set(theirs) == {n for n, d in decl.items() if not d.optional_alias_of}
    for name, t in got.items():
        np.testing.assert_array_equal(t.numpy(), theirs[name])
    w = got["model.layers.0.self_attn.q_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002
    n = got["model.norm.weight"]
    assert float(n.min()) >= 0.9 and float(n.max()) <= 1.1 and float(n.std()) > 0.01


def test_seed_and_name_decide_the_values():
    decl = _declared(TINY_A)
    a, b, c = random_tensors(decl, 0), random_tensors(decl, 0), random_tensors(decl, 1)
    name = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(a[name], b[name]) and not torch.equal(a[name], c[name])
    alone = random_tensors({name: decl[name]}, 0)
    assert torch.equal(alone[name], a[name])  # a tensor's stream does not depend on the others


def test_precision_kinds(tmp_path):
    dli_b200.write_model_dir(tmp_path, TINY_A, seed=0, storage_dtype=torch.bfloat16)
    f = SafetensorsFile(tmp_path / "model.safetensors")
    assert f.entries["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert f.entries["model.norm.weight"].dtype == torch.float32  # stored in 32-bit, stays so
    got = load_tensors(tmp_path, _declared(TINY_A), torch.bfloat16, "cpu")
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert got["model.norm.weight"].dtype == torch.float32
    from dli_b200.weights import TensorDecl
    write_safetensors(tmp_path / "t.safetensors", {"table": torch.arange(6, dtype=torch.int64).view(2, 3)})
    (tmp_path / "model.safetensors").unlink()
    got = load_tensors(tmp_path, {"table": TensorDecl((2, 3), "int")}, torch.bfloat16, "cpu")
    assert got["table"].dtype == torch.int32 and got["table"].tolist() == [[0, 1, 2], [3, 4, 5]]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    decl = _declared(TINY_A)
    tensors = random_tensors(decl, 0)
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.extra.weight"] = torch.zeros(2)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(5, 7)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(CheckpointError) as err:
        load_tensors(tmp_path, decl, torch.float32, "cpu")
    msg = str(err.value)
    assert "model.layers.0.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "model.layers.0.mlp.extra.weight" in msg
    assert "model.layers.1.self_attn.k_proj.weight: file [5, 7], model [32, 64]" in msg


def test_only_safetensors_is_read(tmp_path):
    with pytest.raises(CheckpointError, match="no \\*.safetensors"):
        load_tensors(tmp_path, {}, torch.float32, "cpu")
    (tmp_path / "pytorch_model.bin").write_bytes(b"x")
    with pytest.raises(CheckpointError, match="pickle"):
        load_tensors(tmp_path, {}, torch.float32, "cpu")


def test_tied_head_stored_anyway(tmp_path):
    decl = _declared(TINY_A)
    tensors = random_tensors(decl, 0)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(tmp_path / "model.safetensors", tensors)
    got = load_tensors(tmp_path, decl, torch.float32, "cpu")
    assert "lm_head.weight" not in got
    tensors["lm_head.weight"][3, 4] += 1.0
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(CheckpointError, match="tied"):
        load_tensors(tmp_path, decl, torch.float32, "cpu")


def test_shards_are_merged(tmp_path):
    decl = _declared(TINY_A)
    tensors = random_tensors(decl, 0)
    names = sorted(tensors)
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {n: tensors[n] for n in names[::2]})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {n: tensors[n] for n in names[1::2]})
    got = load_tensors(tmp_path, decl, torch.float32, "cpu")
    assert all(torch.equal(got[n], tensors[n]) for n in names)


def test_broken_header_is_refused(tmp_path):
    (tmp_path / "model.safetensors").write_bytes(b"\xff" * 8 + b"{}")
    with pytest.raises(ValueError, match="header length"):
        load_tensors(tmp_path, {}, torch.float32, "cpu")


def test_engine_refuses_the_cpu(tmp_path):
    dli_b200.write_model_dir(tmp_path, TINY_A, seed=0)
    with pytest.raises(RuntimeError, match="CUDA"):
        dli_b200.load_model(tmp_path, "float32", "cpu")
