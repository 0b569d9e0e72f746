"""CUDA graphs of the pure-decode step.

A step in which every sequence brings one token has the same kernels whatever the tokens
are, so its launches are captured once per shape and replayed: shapes are buckets of
(sequences, block-table width, what the model's parts say changes their launches).  The step's integers are copied into a static
device buffer before the replay; rows beyond the real sequences are padding that reads and
writes a scratch page no request owns.  (The reference replays its decode forward the same
way, src/dli/engine/cuda_graph.py:83-237, to hide the launch cost of its eager kernels; here
it removes the Python time between this engine's launches.)
"""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .batch import GroupView, StepBatch

SEQ_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
WIDTH_STEP = 64  # block-table widths are rounded up to a multiple of this many pages


def bucket_seqs(n: int) -> int | None:
    return next((b for b in SEQ_BUCKETS if b >= n), None)


class DecodeGraph:
    """One captured shape: ``seqs`` rows, tables ``width`` pages wide."""

    def __init__(self, model, caches, num_groups: int, scratch_pages: list[int], page_size: int, seqs: int, width: int,
                 launch_keys: dict) -> None:
        self.seqs, self.width, self.num_groups = seqs, width, num_groups
        dev = model.device
        per_group = seqs + seqs * width
        self.src_base = 4 * seqs + num_groups * per_group  # behind the groups: each row's place in the token source, or -1
        self.size = self.src_base + seqs
        self.ints = torch.zeros(self.size, dtype=torch.int32, device=dev)
        pad = self.padding(scratch_pages, page_size)
        self.ints.copy_(torch.from_numpy(pad))
        arange = torch.arange(seqs + 1, dtype=torch.int32, device=dev)
        views = []
        for g in range(num_groups):
            base = 4 * seqs + g * per_group
            views.append(GroupView(self.ints[base + seqs : base + per_group].view(seqs, width), self.ints[base : base + seqs]))
        self.batch = StepBatch(
            n=seqs, num_seqs=seqs, num_single=seqs, token_ids=self.ints[0:seqs], positions=self.ints[seqs : 2 * seqs],
            seq_of_token=arange[:seqs], q_start=arange, kv_len=self.ints[2 * seqs : 3 * seqs], state_slot=self.ints[3 * seqs : 4 * seqs],
            logit_rows=arange[:seqs], groups=views, q_lens=[1] * seqs, starts=[0] * seqs, state_slots=[0] * seqs, max_q_len=1,
            max_kv_len=width * page_size, max_kv_len_single=width * page_size, launch_keys=launch_keys,
            logits_all_rows=True,
        )
        self._pad = pad
        # run eagerly first (kernels set their attributes, libraries pick their algorithms), then capture
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                model.forward(self.batch, caches)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        before = ops.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = model.forward(self.batch, caches)
        self.kernels = ops.launch_count - before

    def padding(self, scratch_pages: list[int], page_size: int) -> np.ndarray:
        """Integers of a step whose every row is padding: token 0 at position 0 of a
        one-token sequence that lives in the scratch page."""
        seqs, width = self.seqs, self.width
        flat = np.zeros(self.size, dtype=np.int32)
        flat[2 * seqs : 3 * seqs] = 1  # kv_len
        per_group = seqs + seqs * width
        for g, page in enumerate(scratch_pages):
            base = 4 * seqs + g * per_group
            flat[base : base + seqs] = page * page_size
            flat[base + seqs : base + per_group] = page
        flat[self.src_base :] = -1
        return flat

    def fill(self, h: dict) -> np.ndarray:
        """The static buffer's contents for a gathered step of at most ``seqs`` sequences."""
        seqs, width, S = self.seqs, self.width, h["S"]
        flat = self._pad.copy()
        flat[0:S] = h["token_ids"]
        flat[seqs : seqs + S] = h["positions"]
        flat[2 * seqs : 2 * seqs + S] = h["kv_len"]
        flat[3 * seqs : 3 * seqs + S] = h["state_slot"]
        per_group = seqs + seqs * width
        for g in range(self.num_groups):
            base = 4 * seqs + g * per_group
            flat[base : base + S] = h["slots"][g]
            tables = flat[base + seqs : base + per_group].reshape(seqs, width)
            tables[:S, : h["width"]] = h["tables"][g]
        if h.get("token_src") is not None:
            flat[self.src_base : self.src_base + S] = h["token_src"]
        return flat

    def replay(self, token_source: torch.Tensor | None = None) -> torch.Tensor:
        """Run the step whose integers are in ``ints``.  With ``token_source`` (ids sampled on the device
        by the step before), rows that name a place in it take their token id from there first."""
        if token_source is not None:
            ops.patch_tokens(self.ints[0 : self.seqs], token_source, self.ints[self.src_base : self.size])
        self.graph.replay()
        ops.launch_count += self.kernels
        return self.logits


class DecodeGraphs:
    """Graphs by shape, captured at first use."""

    def __init__(self, model, pools, page_size: int) -> None:
        self.model, self.pools, self.page_size = model, pools, page_size
        self.graphs: dict[tuple, DecodeGraph] = {}  # (sequences, width, the parts' launch keys) -> graph, oldest use first
        self.max_graphs = 32  # at the cap the graph that was used least recently makes room
        self.failure: str | None = None
        self._asked: dict[tuple[int, int], dict] = {}  # (sequences, width) -> the parts' answers (they depend on nothing else)

    def launch_keys(self, seqs: int, max_kv_len: int) -> dict:
        """id(part) -> the part's answer, for every part of the model that has one (``Part.decode_launch_key``)."""
        keys = {}
        for part in self.model.parts():
            ask = getattr(part, "decode_launch_key", None)
            key = ask(seqs, max_kv_len, self.page_size) if ask is not None else None
            if key is not None:
                keys[id(part)] = key
        return keys

    def lookup(self, num_seqs: int, width: int, max_kv_len: int) -> DecodeGraph | None:
        seqs = bucket_seqs(num_seqs)
        if seqs is None:
            return None
        width = -(-width // WIDTH_STEP) * WIDTH_STEP
        launch = self._asked.get((seqs, width))
        if launch is None:
            launch = self._asked[(seqs, width)] = self.launch_keys(seqs, width * self.page_size)
        key = (seqs, width, tuple(launch.values()))  # (parts are walked in a fixed order)
        graph = self.graphs.pop(key, None)
        if graph is not None:
            self.graphs[key] = graph  # most recently used: last
        else:
            if self.max_graphs == 0:
                return None
            while len(self.graphs) >= self.max_graphs:
                del self.graphs[next(iter(self.graphs))]  # shapes drift in a long run: the stalest graph goes
            try:
                graph = self.graphs[key] = DecodeGraph(self.model, self.pools.layer_caches, len(self.pools.group_needs),
                                                       self.pools.scratch_pages, self.page_size, seqs, width, launch)
            except RuntimeError as exc:  # a part turned out not to be capturable after all: run step by step from now on
                self.max_graphs = 0
                self.failure = str(exc)
                torch.cuda.synchronize(self.model.device)
                return None
        return graph
