"""CUDA graphs of the pure-decode step, and of small steps that mix prompt portions with decoded tokens.

A step in which every sequence brings one token has the same kernels whatever the tokens
are, so its launches are captured once per shape and replayed: shapes are buckets of
(sequences, block-table width, what the model's parts say changes their launches).  The step's integers are copied into a static
device buffer before the replay; rows beyond the real sequences are padding that reads and
writes a scratch page no request owns.  (The reference replays its decode forward the same
way, src/dli/engine/cuda_graph.py:83-237, to hide the launch cost of its eager kernels; here
it removes the Python time between this engine's launches.)

A step with prompt portions launches some 130 kernels, which the host issues in about 2.3 ms whatever their size;
the GPU needs less than that for up to about a thousand tokens.  Such steps are captured too (``MixedGraph``),
by (single-token sequences, longer portions, the portions' tokens together, width), each rounded up to a bucket: the
attention kernels take each sequence's first row and length from device arrays and size their grids for the longest
portion the bucket allows, so a shorter step runs in the same launches and the surplus CTAs return at once.
"""

from __future__ import annotations

import time

import numpy as np
import torch

from ..kernels import ops
from .batch import GroupView, StepBatch

SEQ_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
WIDTH_STEP = 64  # block-table widths are rounded up to a multiple of this many pages
# Buckets of a mixed step: a capture costs what some twenty steps launched one by one cost (47 ms at Llama-3.2-1B
# sizes), so there are few shapes.  Padding is cheap: an empty portion's CTAs return at once, a padding single-token
# row reads one key, and below a few hundred tokens a step's time is the weights'.
PORTION_BUCKETS = (4,)  # sequences of a mixed step that bring more than one token
TOKEN_BUCKETS = (32, 128, 256, 512, 1024)  # their tokens together
MIXED_SINGLE_BUCKETS = (0, 8, 16, 32, 64, 128, 256)


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


def _bucket(n: int, buckets) -> int | None:
    return next((b for b in buckets if b >= n), None)


class MixedGraph:
    """One captured shape of a step with prompt portions: ``singles`` single-token sequences, then ``portions`` longer
    ones with ``tokens`` tokens together, then one empty sequence in the scratch page, which the token rows that no
    request fills name as theirs (a kernel that walks tokens, not sequences, finds one key for them).  Token rows:
    the singles' first, then the portions' back to back, then padding."""

    def __init__(self, model, caches, num_groups: int, scratch_pages: list[int], page_size: int, singles: int, portions: int,
                 tokens: int, width: int, launch_keys: dict, pool=None) -> None:
        self.set_layout(singles, portions, tokens, width, num_groups)
        dev = model.device
        self._pad = self.padding(scratch_pages, page_size)
        self.ints = torch.zeros(self.size, dtype=torch.int32, device=dev)
        self.ints.copy_(torch.from_numpy(self._pad))
        n, S, o = self.n, self.S, self.offsets
        views = []
        for g in range(num_groups):
            base = o["groups"] + g * self.per_group
            views.append(GroupView(self.ints[base + n : base + self.per_group].view(S, width), self.ints[base : base + n]))
        self.batch = StepBatch(
            n=n, num_seqs=S, num_single=singles, token_ids=self.ints[0:n], positions=self.ints[o["positions"] : o["positions"] + n],
            seq_of_token=self.ints[o["seq_of_token"] : o["seq_of_token"] + n], q_start=self.ints[o["q_start"] : o["q_start"] + S + 1],
            kv_len=self.ints[o["kv_len"] : o["kv_len"] + S], state_slot=self.ints[o["state_slot"] : o["state_slot"] + S],
            logit_rows=self.ints[o["logit_rows"] : o["logit_rows"] + S - 1], groups=views, q_lens=[1] * singles + [0] * (portions + 1),
            starts=[0] * S, state_slots=[0] * S, max_q_len=tokens, max_kv_len=width * page_size, max_kv_len_single=width * page_size,
            launch_keys=launch_keys, logits_all_rows=False,
        )
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                model.forward(self.batch, caches)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        before = ops.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=pool):
            self.logits = model.forward(self.batch, caches)
        self.kernels = ops.launch_count - before

    def set_layout(self, singles: int, portions: int, tokens: int, width: int, num_groups: int) -> None:
        self.singles, self.portions, self.tokens, self.width, self.num_groups = singles, portions, tokens, width, num_groups
        n, S = singles + tokens, singles + portions + 1
        self.n, self.S = n, S
        self.per_group = n + S * width
        o, at = {}, 0
        for name, count in (("token_ids", n), ("positions", n), ("seq_of_token", n), ("q_start", S + 1), ("kv_len", S), ("state_slot", S),
                            ("logit_rows", S - 1), ("groups", num_groups * self.per_group), ("token_src", n)):
            o[name] = at
            at += count
        self.offsets, self.size = o, at

    def padding(self, scratch_pages: list[int], page_size: int) -> np.ndarray:
        """Integers of a step whose every row is padding: the singles are one-token sequences in the scratch page, the
        portions are empty, every token row beyond the singles names the empty last sequence."""
        n, S, o, singles = self.n, self.S, self.offsets, self.singles
        flat = np.zeros(self.size, dtype=np.int32)
        flat[o["seq_of_token"] : o["seq_of_token"] + singles] = np.arange(singles)
        flat[o["seq_of_token"] + singles : o["seq_of_token"] + n] = S - 1
        flat[o["q_start"] : o["q_start"] + singles + 1] = np.arange(singles + 1)
        flat[o["q_start"] + singles + 1 : o["q_start"] + S + 1] = singles
        flat[o["kv_len"] : o["kv_len"] + S] = 1
        for g, page in enumerate(scratch_pages):
            base = o["groups"] + g * self.per_group
            flat[base : base + n] = page * page_size
            flat[base + n : base + self.per_group] = page
        flat[o["token_src"] : o["token_src"] + n] = -1
        return flat

    def fill(self, h: dict) -> np.ndarray:
        """The static buffer's contents for a gathered step (engine.batch.gather_host) that fits this shape: its S1
        single-token sequences come first in ``h``, then its longer portions."""
        n, S, o, singles, width = self.n, self.S, self.offsets, self.singles, self.width
        q_lens = h["q_lens"]
        S1 = int((q_lens == 1).sum())
        S2, Q = h["S"] - S1, h["n"] - S1
        flat = self._pad.copy()

        def rows(name: str, values) -> None:  # per token: the singles' rows, then the portions' behind the padding singles
            at = o[name]
            flat[at : at + S1] = values[:S1]
            flat[at + singles : at + singles + Q] = values[S1:]

        rows("token_ids", h["token_ids"])
        rows("positions", h["positions"])
        flat[o["seq_of_token"] + singles : o["seq_of_token"] + singles + Q] = h["seq_of_token"][S1:] - S1 + singles
        ends = singles + np.cumsum(q_lens[S1:])
        flat[o["q_start"] + singles + 1 : o["q_start"] + singles + 1 + S2] = ends
        flat[o["q_start"] + singles + 1 + S2 : o["q_start"] + S + 1] = singles + Q
        for name in ("kv_len", "state_slot"):
            at = o[name]
            flat[at : at + S1] = h[name][:S1]
            flat[at + singles : at + singles + S2] = h[name][S1:]
        wanted = h["logit_rows"]  # token rows in the gathered step's numbering, caller's order: logits[:len(wanted)] answers the step
        flat[o["logit_rows"] : o["logit_rows"] + wanted.size] = np.where(wanted < S1, wanted, wanted - S1 + singles)
        for g in range(self.num_groups):
            base = o["groups"] + g * self.per_group
            flat[base : base + S1] = h["slots"][g][:S1]
            flat[base + singles : base + singles + Q] = h["slots"][g][S1:]
            tables = flat[base + n : base + self.per_group].reshape(S, width)
            tables[:S1, : h["width"]] = h["tables"][g][:S1]
            tables[singles : singles + S2, : h["width"]] = h["tables"][g][S1:]
        if h.get("token_src") is not None:
            rows("token_src", h["token_src"])
        return flat

    @property
    def max_logit_rows(self) -> int:
        return self.S - 1

    def replay(self, token_source: torch.Tensor | None = None) -> torch.Tensor:
        if token_source is not None:
            o = self.offsets
            ops.patch_tokens(self.ints[0 : self.n], token_source, self.ints[o["token_src"] : o["token_src"] + self.n])
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
        self.mixed: dict[tuple, MixedGraph] = {}  # (singles, portions, tokens, width, launch keys) -> graph, oldest use first
        self.max_mixed = 32
        # a capture pays for itself after some fifty replays (and the first one of a process, which also loads the
        # library's kernels for the new row count, takes up to half a second), so a shape is captured only when it
        # keeps coming
        self.mixed_after = 32
        self.mixed_failure: str | None = None
        self._sightings: dict[tuple, int] = {}
        self._needed: dict[tuple, int] = {}  # sightings a shape needs: doubled each time its graph had to make room
        self._pool = None  # the mixed graphs share one memory pool: they never run at the same time
        self.mixed_captures, self.mixed_capture_seconds = 0, 0.0

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

    def lookup_mixed(self, singles: int, portions: int, tokens: int, width: int, logit_rows: int) -> MixedGraph | None:
        """The graph for a step of ``singles`` single-token sequences and ``portions`` longer ones of ``tokens`` tokens
        together; None if the shape is outside the buckets, wants more logits than a graph returns, or has not
        come often enough to be captured."""
        sb, pb, tb = _bucket(singles, MIXED_SINGLE_BUCKETS), _bucket(portions, PORTION_BUCKETS), _bucket(tokens, TOKEN_BUCKETS)
        if sb is None or pb is None or tb is None or logit_rows > sb + pb or self.max_graphs == 0 or self.max_mixed == 0:
            return None
        wb = WIDTH_STEP
        while wb < width:  # widths double: few shapes
            wb *= 2
        launch = {}
        if sb:
            launch = self._asked.get((sb, wb))
            if launch is None:
                launch = self._asked[(sb, wb)] = self.launch_keys(sb, wb * self.page_size)
        key = (sb, pb, tb, wb, tuple(launch.values()))
        graph = self.mixed.pop(key, None)
        if graph is not None:
            self.mixed[key] = graph
            return graph
        seen = self._sightings[key] = self._sightings.get(key, 0) + 1
        if seen < self._needed.get(key, self.mixed_after):
            return None
        while len(self.mixed) >= self.max_mixed:
            stale = next(iter(self.mixed))
            del self.mixed[stale]
            # a shape that keeps coming back after it made room has to come twice as often before it is captured again
            self._needed[stale], self._sightings[stale] = 2 * self._needed.get(stale, self.mixed_after), 0
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        began = time.perf_counter()
        try:
            graph = self.mixed[key] = MixedGraph(self.model, self.pools.layer_caches, len(self.pools.group_needs), self.pools.scratch_pages,
                                                 self.page_size, sb, pb, tb, wb, launch, self._pool)
            self.mixed_captures += 1
            self.mixed_capture_seconds += time.perf_counter() - began
        except RuntimeError as exc:  # no memory for it, or a part that cannot be captured with longer portions: these steps stay uncaptured
            self.max_mixed = 0
            self.mixed_failure = str(exc)
            self.mixed.clear()
            torch.cuda.synchronize(self.model.device)
            return None
        return graph
