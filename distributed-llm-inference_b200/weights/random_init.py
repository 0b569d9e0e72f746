"""Random-weights mode: a model from a configuration and a seed.

Matrices and the embedding are N(0, 0.02); norm weights are 1 + U(-0.1, 0.1),
so that a norm whose weight is ignored shows.  Each tensor has its own stream,
keyed by the seed and the tensor's name, so a tensor's values do not depend on
which other tensors exist.  ``write_model_dir`` writes a folder (config.json,
model.safetensors) that the loader — and the reference's loader — can read.
"""

from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Any

import torch

from .loader import TensorDecl
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str, device: torch.device | str) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((seed * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensors(
    expected: dict[str, TensorDecl],
    seed: int,
    dtype: torch.dtype = torch.float32,
    device: torch.device | str = "cpu",
) -> dict[str, torch.Tensor]:
    """Values drawn in float32 on ``device`` and rounded once to the target dtype.
    (Streams differ between CPU and CUDA generators; a folder is always written from the CPU.)"""
    out: dict[str, torch.Tensor] = {}
    for name, decl in sorted(expected.items()):
        if decl.optional_alias_of:
            continue
        g = _generator(seed, name, device)
        if decl.kind == "matrix":
            t = torch.empty(decl.shape, dtype=torch.float32, device=device).normal_(0.0, 0.02, generator=g).to(dtype)
        elif decl.kind == "vector32":
            t = 1.0 + torch.empty(decl.shape, dtype=torch.float32, device=device).uniform_(-0.1, 0.1, generator=g)
        else:
            t = torch.randint(0, 2**15, decl.shape, dtype=torch.int32, device=device, generator=g)
        out[name] = t
    return out


def write_model_dir(
    model_dir: str | Path,
    config_json: dict[str, Any],
    seed: int,
    storage_dtype: torch.dtype = torch.float32,
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for the architecture the config names."""
    from ..config.registry import resolve_architecture
    from ..parts.model import declared_tensors

    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    arch = resolve_architecture(config_json)
    spec = arch.model_spec(arch.parse_config(config_json))
    tensors = random_tensors(declared_tensors(spec), seed, dtype=storage_dtype)
    (model_dir / "config.json").write_text(json.dumps(config_json, indent=2) + "\n")
    write_safetensors(model_dir / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return model_dir
