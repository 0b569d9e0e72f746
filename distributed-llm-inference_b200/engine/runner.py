"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.step`` runs only the tokens it is given, as one batch, against the
cache that earlier steps left, and returns the logits at the wanted places.
Portions of prompts and single decoded tokens, cut anywhere, take the same path
(the reference has three: src/dli/engine/runner.py:57-61).
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Sequence

import numpy as np
import torch

from ..cache import CacheManager, CachePools, GroupSpec
from ..cache.needs import paged_need_of, state_needs_of
from ..config.registry import load_config, resolve_architecture
from ..kernels import ops
from ..parts import DecoderModel
from ..weights import load_tensors, random_tensors
from .batch import StepEntry, Uploader, build_batch, gather_host, gather_single_tokens
from .graphs import PORTION_BUCKETS, SEQ_BUCKETS, TOKEN_BUCKETS, DecodeGraphs

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def resolve_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    if dtype == "auto":
        return torch.bfloat16
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not supported (bfloat16, float32)") from None


def _require_cuda(device: torch.device) -> None:
    if device.type != "cuda":
        raise RuntimeError(f"device {device} is not a CUDA device: the engine's kernels run on the GPU only")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available: the engine has no CPU path")


def load_model(model_dir: str | Path, dtype: str | torch.dtype = "bfloat16", device: str | torch.device = "cuda:0") -> DecoderModel:
    """Build the model config.json names and load its tensors strictly by name
    (src/dli/model/loader.py:43-93)."""
    device = torch.device(device)
    _require_cuda(device)
    arch, cfg = load_config(model_dir)
    model = DecoderModel(arch.model_spec(cfg), resolve_dtype(dtype), device)
    model.load(load_tensors(model_dir, model.declared_tensors(), model.dtype, device))
    model.config = cfg
    return model


def random_model(config_json: dict[str, Any], seed: int, dtype: str | torch.dtype = "bfloat16",
                 device: str | torch.device = "cuda:0") -> DecoderModel:
    """A model with seeded random weights drawn on the device (no folder is written)."""
    device = torch.device(device)
    _require_cuda(device)
    arch = resolve_architecture(config_json)
    cfg = arch.parse_config(config_json)
    model = DecoderModel(arch.model_spec(cfg), resolve_dtype(dtype), device)
    model.load(random_tensors(model.declared_tensors(), seed, dtype=model.dtype, device=device))
    model.config = cfg
    return model


class ModelRunner:
    """A model with its cache pools and cache manager."""

    def __init__(self, model: DecoderModel, *, num_pages: int | Sequence[int], page_size: int = 16, max_requests: int = 64,
                 enable_prefix_caching: bool = True, watermark: float = 0.01, cuda_graphs: bool = True,
                 eviction_policy: str = "lru") -> None:
        self.model = model
        needs = model.cache_needs()
        order = model.spec.run_order
        n_groups = len({paged_need_of(n) for n in needs} - {None})
        pages = [num_pages] * n_groups if isinstance(num_pages, int) else list(num_pages)
        self.pools = CachePools(needs, order, pages, page_size, max_requests, model.dtype, model.device)
        self.manager = CacheManager(
            [GroupSpec(p, need.window) for p, need in zip(pages, self.pools.group_needs)],
            page_size, max_requests, enable_prefix_caching=enable_prefix_caching,
            has_state=any(state_needs_of(n) for n in needs), watermark=watermark, eviction_policy=eviction_policy,
        )
        self.page_size = page_size
        self.uploader = Uploader(model.device)
        # graphs replay padding rows through every mixer: not with per-request state, which they would touch
        capturable = all(getattr(part, "graph_capturable", False) for part in model.parts())
        self.graphs = DecodeGraphs(model, self.pools, page_size) if cuda_graphs and capturable and not self.pools.has_state else None
        self.graph_steps = 0  # pure-decode steps replayed from a graph
        self.mixed_graph_steps = 0  # small steps with prompt portions replayed from a graph

    @staticmethod
    def pages_for_budget(model: DecoderModel, budget_bytes: float, page_size: int) -> int:
        """Pages per group that ``budget_bytes`` buys, every group getting the same count
        (src/dli/kv/paged_store.py:78-89)."""
        per_page = sum(CachePools.bytes_per_page(model.cache_needs(), model.spec.run_order, page_size, model.dtype))
        return max(1, int(budget_bytes // max(1, per_page)))

    def start_request(self, request_id, slot: int) -> None:
        if self.pools.has_state:
            self.pools.reset_state(slot)

    def copy_pages(self, copies) -> None:
        """Carry out the cache manager's page copies (``append_slots`` of a forked request) in every
        layer of their groups, before the step that writes the appended tokens."""
        for c in copies:
            ops.copy_page(self.pools.k[c.group], c.src, c.dst)
            ops.copy_page(self.pools.v[c.group], c.src, c.dst)

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], borrow: bool = False, token_source: torch.Tensor | None = None) -> torch.Tensor:
        """Logits [wanted, vocab] float32 on the device, in the order of ``entries`` and of
        each entry's ``want``.  Afterwards every entry's tokens count as computed.
        With ``borrow`` the result may be a view of a buffer the next step overwrites.
        ``token_source``: int32 ids on the device (what the step before sampled); entries with
        ``token_src >= 0`` take their token from that row of it, so a step can be launched before
        the host has read the ids it runs on."""
        if token_source is None and any(e.token_src >= 0 for e in entries):
            raise ValueError("entries name rows of a token source, but none was given")
        logits = None
        if self.graphs is not None and all(len(e.token_ids) == 1 for e in entries):
            logits = self._replay_decode(entries, token_source)
            if logits is not None and not borrow:
                logits = logits.clone()
        gathered = None
        if logits is None and self.graphs is not None and self._small_mixed_step(entries):
            gathered = gather_host(entries, self.manager, self.model.spec.vocab_size)
            logits = self._replay_mixed(gathered, token_source)
            if logits is not None and not borrow:
                logits = logits.clone()
        if logits is None:
            batch, _ = build_batch(entries, self.manager, self.model.device, self.model.spec.vocab_size, self.uploader, gathered)
            if batch.token_src is not None:
                ops.patch_tokens(batch.token_ids, token_source, batch.token_src)
            logits = self.model.forward(batch, self.pools.layer_caches)
        manager = self.manager
        for e in entries:
            manager.mark_computed(e.request_id, manager.progress(e.request_id)[0] + len(e.token_ids))
        return logits

    def _replay_decode(self, entries: Sequence[StepEntry], token_source: torch.Tensor | None = None) -> torch.Tensor | None:
        """A step of single tokens through a captured graph; None if no graph takes its shape."""
        h = gather_single_tokens(entries, self.manager, self.model.spec.vocab_size)
        graph = self.graphs.lookup(h["S"], h["width"], int(h["kv_len"].max()))
        if graph is None:
            return None
        self.uploader.upload(graph.fill(h), out=graph.ints)
        logits = graph.replay(token_source if h["token_src"] is not None else None)
        self.graph_steps += 1
        rows = h["logit_rows"]
        if rows.size == h["S"] and (rows == np.arange(h["S"])).all():
            return logits[: h["S"]]
        return logits[torch.from_numpy(rows).to(logits.device)]

    @staticmethod
    def _small_mixed_step(entries: Sequence[StepEntry]) -> bool:
        """Whether a step with longer portions is small enough that launching it kernel by kernel would take the host
        longer than the GPU needs for it (the buckets of engine.graphs end there)."""
        portions = tokens = 0
        for e in entries:
            if len(e.token_ids) > 1:
                portions += 1
                tokens += len(e.token_ids)
        return 0 < portions <= PORTION_BUCKETS[-1] and tokens <= TOKEN_BUCKETS[-1] and len(entries) - portions <= SEQ_BUCKETS[-1]

    def _replay_mixed(self, h: dict, token_source: torch.Tensor | None = None) -> torch.Tensor | None:
        """A small step with prompt portions through a captured graph; None if no graph takes its shape (yet)."""
        singles = int((h["q_lens"] == 1).sum())
        graph = self.graphs.lookup_mixed(singles, h["S"] - singles, h["n"] - singles, h["width"], h["logit_rows"].size)
        if graph is None:
            return None
        self.uploader.upload(graph.fill(h), out=graph.ints)
        logits = graph.replay(token_source if h["token_src"] is not None else None)
        self.mixed_graph_steps += 1
        return logits[: h["logit_rows"].size]

    def check_device_errors(self) -> None:
        """Raise if a bounded wait inside one of the kernels gave up since this was last asked: what
        such a step computed is not to be trusted.  Call it once the step's results are on the host."""
        errors = ops.device_wait_errors()
        if errors:
            raise ops.KernelError("a device-side wait ran out; the step's results are invalid: "
                                  + ", ".join(f"{lib} code {code}" for lib, code in sorted(errors.items())))

    takes_token_source = True  # execute() accepts chunks whose token is still on the device

    def execute(self, chunks, token_source=None, token_rows: Sequence[int] | None = None) -> torch.Tensor:
        """The engine's view of ``step``: one entry per scheduled chunk, logits at the last
        token of the chunks that sample (src/dli/engine/runner.py:53-80).  ``token_rows[i] >= 0``:
        chunk i is one token that the host has not read yet, row token_rows[i] of ``token_source``
        (sampling.PendingTokens)."""
        entries = []
        for i, ch in enumerate(chunks):
            src = token_rows[i] if token_rows is not None else -1
            tokens = [0] if src >= 0 else ch.request.token_slice(ch.start, ch.start + ch.num_tokens)
            entries.append(StepEntry(ch.request.request_id, tokens, [ch.num_tokens - 1] if ch.needs_logits else [], src))
        return self.step(entries, borrow=True, token_source=None if token_source is None else token_source.device_ids)
