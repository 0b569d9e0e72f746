"""Typed configuration of the Llama 3.2 / SmolLM2 dense GQA decoder.

Parsed strictly from the architecture's own ``config.json`` keys, with the
defaults and the rejections of the reference (src/dli/model/config.py:80-150).
No size or constant that config.json gives appears anywhere else in code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .spec import LayerSpec, ModelSpec, PartSpec, RunStep


class UnsupportedModelError(ValueError):
    """The configuration asks for a feature this engine does not implement."""


@dataclass(frozen=True)
class RopeConfig:
    """Rotary embedding constants (src/dli/model/config.py:22-39)."""

    theta: float
    rope_type: str = "default"  # "default" | "linear" | "llama3"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    rms_norm_eps: float
    max_position_embeddings: int
    rope: RopeConfig
    tie_word_embeddings: bool

    def __post_init__(self) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_layers", "num_heads", "num_kv_heads", "head_dim"):
            if getattr(self, key) < 1:
                raise UnsupportedModelError(f"{key}={getattr(self, key)} must be positive")
        if self.num_heads % self.num_kv_heads:
            raise UnsupportedModelError(
                f"num_attention_heads={self.num_heads} is not a multiple of num_key_value_heads={self.num_kv_heads}"
            )
        if self.head_dim % 2:
            raise UnsupportedModelError(f"head_dim={self.head_dim} must be even for rotary embeddings")

    @classmethod
    def from_hf_dict(cls, cfg: dict[str, Any]) -> "LlamaConfig":
        """Both spellings are read: hub (``rope_theta`` + ``rope_scaling``, legacy key
        ``type``) and ``rope_parameters``, which wins (src/dli/model/config.py:130-136)."""
        model_type = cfg.get("model_type", "llama")
        if model_type != "llama":
            raise UnsupportedModelError(f"model_type={model_type!r} is not the llama decoder")
        act = cfg.get("hidden_act", "silu")
        if act != "silu":
            raise UnsupportedModelError(f"hidden_act={act!r} (only 'silu' / SwiGLU is supported)")
        if cfg.get("use_sliding_window") or any(t != "full_attention" for t in cfg.get("layer_types") or []):
            raise UnsupportedModelError("use_sliding_window / layer_types: sliding-window attention is not part of this architecture")
        if cfg.get("pretraining_tp", 1) not in (1, None):
            raise UnsupportedModelError("pretraining_tp > 1 changes numerics and is not supported")
        for key in ("attention_bias", "mlp_bias"):
            if cfg.get(key, False):
                raise UnsupportedModelError(f"{key}=true: biased projections are not part of this architecture")
        heads = int(cfg["num_attention_heads"])
        hidden = int(cfg["hidden_size"])
        return cls(
            vocab_size=int(cfg["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(cfg["intermediate_size"]),
            num_layers=int(cfg["num_hidden_layers"]),
            num_heads=heads,
            num_kv_heads=int(cfg.get("num_key_value_heads") or heads),
            head_dim=int(cfg.get("head_dim") or hidden // heads),
            rms_norm_eps=float(cfg["rms_norm_eps"]),
            max_position_embeddings=int(cfg.get("max_position_embeddings", 4096)),
            rope=_parse_rope(cfg),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        )

    def to_hf_dict(self) -> dict[str, Any]:
        """A config.json that parses back to this configuration."""
        out: dict[str, Any] = {
            "architectures": ["LlamaForCausalLM"],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope.theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "torch_dtype": "float32",
        }
        if self.rope.rope_type != "default":
            out["rope_scaling"] = {
                "rope_type": self.rope.rope_type,
                "factor": self.rope.factor,
                "low_freq_factor": self.rope.low_freq_factor,
                "high_freq_factor": self.rope.high_freq_factor,
                "original_max_position_embeddings": self.rope.original_max_position_embeddings,
            }
        return out


def _parse_rope(cfg: dict[str, Any]) -> RopeConfig:
    merged = {**dict(cfg.get("rope_scaling") or {}), **dict(cfg.get("rope_parameters") or {})}
    theta = float(merged.get("rope_theta", cfg.get("rope_theta", 10000.0)))
    rope_type = merged.get("rope_type", merged.get("type", "default"))
    if rope_type not in ("default", "linear", "llama3"):
        raise UnsupportedModelError(f"rope_type={rope_type!r} is not supported (default, linear, llama3)")
    if rope_type == "default":
        return RopeConfig(theta=theta)
    if "factor" not in merged:
        raise KeyError("rope_scaling.factor")
    return RopeConfig(
        theta=theta,
        rope_type=rope_type,
        factor=float(merged["factor"]),
        low_freq_factor=float(merged.get("low_freq_factor", 1.0)),
        high_freq_factor=float(merged.get("high_freq_factor", 4.0)),
        original_max_position_embeddings=int(
            merged.get("original_max_position_embeddings", cfg.get("max_position_embeddings", 8192))
        ),
    )


def llama_model_spec(cfg: LlamaConfig) -> ModelSpec:
    """The decoder as parts: L identical pre-norm layers of GQA attention with
    rotary position encoding and a SwiGLU feed-forward, each run once and in
    order (src/dli/model/llama.py:194-223); tensor names as in the checkpoint
    (src/dli/model/llama.py:56-59,185-187,201-202,221-223,238-240)."""
    position = PartSpec(
        "rotary",
        {
            "head_dim": cfg.head_dim,
            "rotary_dim": cfg.head_dim,
            "theta": cfg.rope.theta,
            "scaling": cfg.rope.rope_type,
            "factor": cfg.rope.factor,
            "low_freq_factor": cfg.rope.low_freq_factor,
            "high_freq_factor": cfg.rope.high_freq_factor,
            "original_max_position_embeddings": cfg.rope.original_max_position_embeddings,
        },
    )
    layers = []
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        norm = {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}
        layers.append(
            LayerSpec(
                "prenorm",
                {
                    "mixer_norm": PartSpec("rmsnorm", norm, p + "input_layernorm."),
                    "mixer": PartSpec(
                        "gqa_attention",
                        {
                            "hidden_size": cfg.hidden_size,
                            "num_heads": cfg.num_heads,
                            "num_kv_heads": cfg.num_kv_heads,
                            "head_dim": cfg.head_dim,
                            "scale": cfg.head_dim**-0.5,
                            "window": None,
                            "position": position,
                        },
                        p + "self_attn.",
                    ),
                    "ffn_norm": PartSpec("rmsnorm", norm, p + "post_attention_layernorm."),
                    "ffn": PartSpec(
                        "swiglu",
                        {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size},
                        p + "mlp.",
                    ),
                },
            )
        )
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}, "model.embed_tokens."),
        layers=tuple(layers),
        run_order=tuple(RunStep(i) for i in range(cfg.num_layers)),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, "model.norm."),
        head=PartSpec(
            "lm_head",
            {
                "vocab_size": cfg.vocab_size,
                "hidden_size": cfg.hidden_size,
                "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None,
            },
            "lm_head.",
        ),
    )
