"""Strict loading of a model folder's tensors by name.

Only safetensors is read; names and shapes must equal what the model's parts
declare (src/dli/model/loader.py:26-35,70-89).  Unlike the reference, which
raises on the first kind of mismatch, one error lists everything: missing
tensors, unexpected tensors and wrong shapes.

Precision on the device: a ``matrix`` tensor takes the engine's dtype
(bfloat16 or float32); a ``vector32`` tensor (norm weights and other small
tables the kernels read as float) is float32 whatever the file holds;
an ``int`` tensor becomes int32.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import torch

from .safetensors_io import SafetensorsFile


class CheckpointError(ValueError):
    """The model folder is unusable: format, missing or unexpected tensors, shapes."""


@dataclass(frozen=True)
class TensorDecl:
    shape: tuple[int, ...]
    kind: str = "matrix"  # "matrix" | "vector32" | "int"
    # name of another declared tensor this one must equal if the file stores it anyway
    # (a tied head some checkpoints serialise): the duplicate is checked and dropped
    optional_alias_of: str | None = None


def safetensor_files(model_dir: Path) -> list[Path]:
    files = sorted(model_dir.glob("*.safetensors"))
    if files:
        return files
    if any(model_dir.glob("*.bin")) or any(model_dir.glob("*.pt")):
        raise CheckpointError(f"{model_dir} only has pickle-based weights (.bin/.pt); refusing to load them")
    raise CheckpointError(f"no *.safetensors files in {model_dir}")


def _target_dtype(decl: TensorDecl, dtype: torch.dtype) -> torch.dtype:
    if decl.kind == "matrix":
        return dtype
    if decl.kind == "vector32":
        return torch.float32
    if decl.kind == "int":
        return torch.int32
    raise ValueError(f"unknown tensor kind {decl.kind!r}")


def load_tensors(
    model_dir: str | Path,
    expected: dict[str, TensorDecl],
    dtype: torch.dtype,
    device: torch.device | str,
) -> dict[str, torch.Tensor]:
    """Read ``expected`` from the folder's safetensors files onto ``device``."""
    model_dir = Path(model_dir)
    files = [SafetensorsFile(f) for f in safetensor_files(model_dir)]
    where: dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.entries:
            where[name] = f  # a later shard wins, as a merged dict would

    aliases = {n: d.optional_alias_of for n, d in expected.items() if d.optional_alias_of}
    required = {n for n in expected if n not in aliases}
    missing = sorted(required - where.keys())
    unexpected = sorted(where.keys() - expected.keys())
    wrong = []
    for name in sorted(expected.keys() & where.keys()):
        got = where[name].entries[name].shape
        if tuple(got) != tuple(expected[name].shape):
            wrong.append(f"{name}: file {list(got)}, model {list(expected[name].shape)}")
    if missing or unexpected or wrong:
        raise CheckpointError(
            f"{model_dir}: missing tensors: {missing}; unexpected tensors: {unexpected}; wrong shapes: {wrong}"
        )
    for name, target in aliases.items():
        if name in where and not torch.equal(where[name].tensor(name), where[target].tensor(target)):
            raise CheckpointError(f"{model_dir}: {name} is stored but differs from {target}, to which it is tied")

    out: dict[str, torch.Tensor] = {}
    for name in sorted(required):
        src = where[name].tensor(name)
        out[name] = src.to(device=device, dtype=_target_dtype(expected[name], dtype)).contiguous()
    for f in files:
        f.close()
    return out
