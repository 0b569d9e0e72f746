"""One registry from an architecture's name to its configuration and model.

The name is ``config.json["architectures"][0]``; a file without that key is
looked up by ``model_type``.  (The reference has no registry: it keys on
``model_type`` alone, src/dli/model/config.py:91-93.)
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .llama import LlamaConfig, UnsupportedModelError, llama_model_spec
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict[str, Any]], Any]  # config.json dict -> typed configuration
    model_spec: Callable[[Any], ModelSpec]  # typed configuration -> parts and run order
    model_types: tuple[str, ...] = ()  # model_type values that also select it


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def resolve_architecture(cfg: dict[str, Any]) -> Architecture:
    names = cfg.get("architectures") or []
    if names:
        if names[0] in _ARCHITECTURES:
            return _ARCHITECTURES[names[0]]
        raise UnsupportedModelError(f"architectures[0]={names[0]!r} is not registered (known: {sorted(_ARCHITECTURES)})")
    model_type = cfg.get("model_type")
    for arch in _ARCHITECTURES.values():
        if model_type in arch.model_types:
            return arch
    raise UnsupportedModelError(f"model_type={model_type!r} is not registered (known: {sorted(_ARCHITECTURES)})")


def load_config(model_dir: str | Path) -> tuple[Architecture, Any]:
    """Parse ``config.json`` of a model folder (src/dli/model/loader.py:38-40)."""
    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    arch = resolve_architecture(cfg)
    return arch, arch.parse_config(cfg)


register_architecture(
    Architecture("LlamaForCausalLM", LlamaConfig.from_hf_dict, llama_model_spec, model_types=("llama",))
)
