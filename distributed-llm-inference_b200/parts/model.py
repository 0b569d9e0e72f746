"""The decoder: embedding, layers in run order, final norm, head — built from a ModelSpec."""

from __future__ import annotations

import torch

from ..config.spec import ModelSpec
from ..kernels import ops
from ..kernels.gemm import SKINNY_MAX_TOKENS_HEAD, linear, project
from ..weights.loader import TensorDecl
from .base import BuildEnv, Part, ResidualStream, build_part, can_fuse, normed_input, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """h = table[token_ids], no scale (src/dli/model/llama.py:291).  params: vocab_size, hidden_size."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.weight: torch.Tensor | None = None

    def declare(self):
        return {self.spec.prefix + "weight": TensorDecl((self.vocab, self.hidden))}

    def load(self, tensors):
        self.weight = tensors[self.spec.prefix + "weight"]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        h = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        ops.embedding(h, self.weight, token_ids)
        return h


@register_part("head", "lm_head")
class LMHead(Part):
    """logits = y W^T in float32, W the embedding matrix when ``tied_to`` names it
    (src/dli/model/llama.py:304-305).  A tied checkpoint that stores the head anyway is
    accepted if both are equal (src/dli/model/loader.py:75-80).
    params: vocab_size, hidden_size, tied_to."""

    graph_capturable = True
    takes_scaled_rows = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.tied_to = spec.params.get("tied_to")
        self.weight: torch.Tensor | None = None

    def declare(self):
        return {self.spec.prefix + "weight": TensorDecl((self.vocab, self.hidden), optional_alias_of=self.tied_to)}

    def load(self, tensors):
        self.weight = tensors[self.tied_to or self.spec.prefix + "weight"]

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        return project(y, self.weight, out_dtype=torch.float32, max_tokens=SKINNY_MAX_TOKENS_HEAD)


def _walk(part) -> list[Part]:
    out = [part]
    for c in part.children():
        out.extend(_walk(c))
    return out


class DecoderModel:
    """Runs the tokens of one step through the layers, in the order ``spec.run_order`` gives."""

    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str) -> None:
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not supported (bfloat16, float32)")
        self.spec = spec
        self.env = BuildEnv(dtype, torch.device(device))
        self.embedding = build_part("embedding", spec.embedding, self.env)
        self.layers = [build_part("arrangement", layer, self.env) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, self.env)
        self.head = build_part("head", spec.head, self.env)
        self._wire_deferred_products()

    def _wire_deferred_products(self) -> None:
        """A layer may leave its last product to the norm of whatever runs after it, if every
        successor it has in the run order (or the final norm and the head) can take it."""
        order = [step.layer for step in self.spec.run_order]
        ok: dict[int, bool] = {}
        for i, layer in enumerate(order):
            if i + 1 < len(order):
                first = getattr(self.layers[order[i + 1]], "first_consumer", None)
                able = first is not None and can_fuse(*first())
            else:
                able = can_fuse(self.final_norm, self.head)
            ok[layer] = ok.get(layer, True) and able
        for layer, able in ok.items():
            defer = getattr(self.layers[layer], "defer_last_product", None)
            if defer is not None:
                defer(able)

    @property
    def dtype(self) -> torch.dtype:
        return self.env.dtype

    @property
    def device(self) -> torch.device:
        return self.env.device

    def parts(self) -> list[Part]:
        out: list[Part] = []
        for top in (self.embedding, *self.layers, self.final_norm, self.head):
            out.extend(_walk(top))
        return out

    def declared_tensors(self) -> dict[str, TensorDecl]:
        out: dict[str, TensorDecl] = {}
        for part in self.parts():
            for name, decl in part.declare().items():
                if name in out and out[name] != decl:
                    raise ValueError(f"tensor {name!r} is declared twice with different shapes")
                out[name] = decl
        return out

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(tensors)

    def cache_needs(self) -> list:
        """What each run step asks of the cache manager, as its arrangement answers ``cache_need()``: None, one
        need, or several (pages and a fixed-size state side by side).  None for a step that reads another
        step's cache.  An arrangement without that method is asked through its attribute ``mixer``."""
        needs = []
        for step in self.spec.run_order:
            layer = self.layers[step.layer]
            ask = getattr(layer, "cache_need", None) or getattr(getattr(layer, "mixer", None), "cache_need", None)
            needs.append(ask() if ask is not None and step.cache_of is None else None)
        return needs

    def forward(self, batch, caches) -> torch.Tensor:
        """Logits [k, vocab] (float32) at ``batch.logit_rows``; every token's cache entries are written."""
        batch.scratch.clear()
        stream = ResidualStream(self.embedding.forward(batch.token_ids))
        for i, step in enumerate(self.spec.run_order):
            self.layers[step.layer].forward(stream, batch, caches[i])
        if batch.logit_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        rows = None if getattr(batch, "logits_all_rows", False) else batch.logit_rows
        y = normed_input(self.final_norm, stream.h, stream.take_pending(), self.head, rows=rows)
        return self.head.forward(y)


def declared_tensors(spec: ModelSpec) -> dict[str, TensorDecl]:
    """Names, shapes and kinds of a spec's tensors, without touching a device."""
    return DecoderModel(spec, torch.float32, "meta").declared_tensors()
