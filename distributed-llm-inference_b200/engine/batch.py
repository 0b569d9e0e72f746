"""The device-side description of one step's batch.

A step is a list of entries (request, its next tokens, the places whose logits
are wanted).  All entries are flattened into one token vector; entries of a
single token come first, longer portions after them (attention kernels launch
once per kind), and ``logit_rows`` restores the caller's order.  Every integer
array of a step is laid out in one host array and travels to the device in one
copy from pinned memory.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
import torch


@dataclass(frozen=True)
class StepEntry:
    request_id: Hashable
    token_ids: Sequence[int]  # the request's next tokens, at positions start .. start + len - 1
    want: Sequence[int] = ()  # indices into token_ids whose logits are returned
    # >= 0: the entry brings one token whose id the host does not know yet; it is this row of the
    # step's token source (ids sampled on the device by the step before), and token_ids[0] is ignored
    token_src: int = -1


@dataclass
class GroupView:
    block_tables: torch.Tensor  # [num_seqs, max_blocks] int32; -1 where a page was given back
    slots: torch.Tensor  # [n] int32: page * page_size + offset of each token's own key/value


@dataclass
class StepBatch:
    n: int  # tokens in this step
    num_seqs: int
    num_single: int  # sequences with exactly one token this step; they come first
    token_ids: torch.Tensor  # [n] int32
    positions: torch.Tensor  # [n] int32, absolute
    seq_of_token: torch.Tensor  # [n] int32
    q_start: torch.Tensor  # [num_seqs + 1] int32: first token row of each sequence
    kv_len: torch.Tensor  # [num_seqs] int32: tokens of the sequence in the cache after this step
    state_slot: torch.Tensor  # [num_seqs] int32
    logit_rows: torch.Tensor  # [k] int32: token rows whose logits are wanted, caller's order
    groups: list[GroupView]
    # host copies, for launch decisions only
    q_lens: list[int] = field(default_factory=list)
    starts: list[int] = field(default_factory=list)
    state_slots: list[int] = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    max_kv_len_single: int = 0  # longest context among the single-token sequences
    # id(part) -> what that part answered to ``decode_launch_key`` when this step's shape was fixed ahead of its
    # data (a captured graph); a part not named here decides its launches from the step itself
    launch_keys: dict = field(default_factory=dict)
    token_src: torch.Tensor | None = None  # [n] int32: row of the token source per token, -1 where token_ids holds the id
    logits_all_rows: bool = False  # logit_rows is 0, 1, .., n - 1: the final norm's output needs no gather
    scratch: dict = field(default_factory=dict)  # per-step results that parts share across layers; cleared by each forward

    def group(self, index: int) -> GroupView:
        return self.groups[index]


class Uploader:
    """Host-to-device copies of a step's integers through pinned memory.

    Two pinned buffers alternate; before one is written again, the copy that last read it
    has finished (an event is recorded after each copy)."""

    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self._bufs: list[torch.Tensor | None] = [None, None]
        self._events: list[torch.cuda.Event | None] = [None, None]
        self._turn = 0
        self.bytes_last = 0

    def stage(self, flat: np.ndarray) -> torch.Tensor:
        """A pinned int32 tensor holding ``flat`` (a plain tensor without a CUDA device)."""
        if not self.cuda:
            return torch.from_numpy(flat)
        i = self._turn
        self._turn ^= 1
        if self._events[i] is not None:
            self._events[i].synchronize()
        buf = self._bufs[i]
        if buf is None or buf.numel() < flat.size:
            buf = self._bufs[i] = torch.empty(max(4096, 2 * flat.size), dtype=torch.int32).pin_memory()
        view = buf[: flat.size]
        view.numpy()[:] = flat
        self._pending = i
        return view

    def upload(self, flat: np.ndarray, out: torch.Tensor | None = None) -> torch.Tensor:
        src = self.stage(flat)
        self.bytes_last = flat.size * 4
        if out is None:
            out = torch.empty(flat.size, dtype=torch.int32, device=self.device)
        out[: flat.size].copy_(src, non_blocking=True)
        if self.cuda:
            ev = self._events[self._pending] or torch.cuda.Event()
            ev.record()
            self._events[self._pending] = ev
        return out


def _check_entries(entries: Sequence[StepEntry], vocab_size: int) -> list[np.ndarray]:
    if not entries:
        raise ValueError("a step needs at least one entry")
    seen = set()
    arrays = []
    for e in entries:
        if e.request_id in seen:
            raise ValueError(f"request {e.request_id!r} appears twice in one step")
        seen.add(e.request_id)
        a = np.asarray(e.token_ids, dtype=np.int64)
        if a.ndim != 1 or a.size == 0:
            raise ValueError(f"request {e.request_id!r} brings no tokens")
        if e.token_src >= 0:
            if a.size != 1:
                raise ValueError(f"request {e.request_id!r}: a token from the device comes alone")
            a = np.zeros(1, dtype=np.int64)
        if a.min() < 0 or a.max() >= vocab_size:
            bad = int(a[(a < 0) | (a >= vocab_size)][0])
            raise ValueError(f"token id {bad} of request {e.request_id!r} is outside the vocabulary [0, {vocab_size})")
        for w in e.want:
            if not 0 <= w < a.size:
                raise ValueError(f"want index {w} of request {e.request_id!r} is outside its {a.size} tokens")
        arrays.append(a)
    return arrays


def gather_host(entries: Sequence[StepEntry], manager, vocab_size: int):
    """The step's integer arrays on the host.  Returns a dict of int32 arrays and lists."""
    arrays = _check_entries(entries, vocab_size)
    order = sorted(range(len(entries)), key=lambda i: (arrays[i].size != 1, i))
    place = [0] * len(entries)
    for new, old in enumerate(order):
        place[old] = new
    S = len(order)
    q_lens = np.empty(S, dtype=np.int64)
    starts = np.empty(S, dtype=np.int64)
    rows = np.empty(S, dtype=np.int64)
    for s, old in enumerate(order):
        rid = entries[old].request_id
        q_lens[s] = arrays[old].size
        starts[s] = manager.num_computed_tokens(rid)
        rows[s] = manager.state_slot(rid)
        if starts[s] + q_lens[s] > manager.num_tokens(rid):
            raise ValueError(f"request {rid!r}: tokens up to {starts[s] + q_lens[s]} have no slots reserved")
    q_start = np.zeros(S + 1, dtype=np.int64)
    np.cumsum(q_lens, out=q_start[1:])
    n = int(q_start[-1])
    seq_of_token = np.repeat(np.arange(S), q_lens)
    positions = np.arange(n) - q_start[seq_of_token] + starts[seq_of_token]
    kv_len = starts + q_lens
    ps = manager.page_size
    width = int(-(-kv_len.max() // ps))
    slots, tables = [], []
    for g in range(len(manager.pools)):
        table = manager.table_array(g)
        pages = table[rows[seq_of_token], positions // ps].astype(np.int64)
        if (pages < 0).any():
            raise ValueError("a token's position lies in a page the window has given back")
        slots.append(pages * ps + positions % ps)
        tables.append(table[rows, :width])
    logit_rows = [int(q_start[place[i]]) + w for i, e in enumerate(entries) for w in e.want]
    token_src = None
    if any(e.token_src >= 0 for e in entries):
        token_src = np.full(n, -1, dtype=np.int64)
        for i, e in enumerate(entries):
            if e.token_src >= 0:
                token_src[q_start[place[i]]] = e.token_src
    return dict(
        token_src=token_src,
        token_ids=np.concatenate([arrays[old] for old in order]), positions=positions, seq_of_token=seq_of_token,
        q_start=q_start, kv_len=kv_len, state_slot=rows, logit_rows=np.asarray(logit_rows, dtype=np.int64),
        slots=slots, tables=tables, q_lens=q_lens, starts=starts, n=n, S=S, width=width, place=place,
    )


def gather_single_tokens(entries: Sequence[StepEntry], manager, vocab_size: int):
    """gather_host for a step in which every entry brings exactly one token (the decode step):
    the same arrays, built with far fewer operations."""
    S = len(entries)
    if S == 0:
        raise ValueError("a step needs at least one entry")
    tokens = np.empty(S, dtype=np.int64)
    src = np.empty(S, dtype=np.int64)
    starts = np.empty(S, dtype=np.int64)
    rows = np.empty(S, dtype=np.int64)
    seen = set()
    logit_rows = []
    for s, e in enumerate(entries):
        rid = e.request_id
        if rid in seen:
            raise ValueError(f"request {rid!r} appears twice in one step")
        seen.add(rid)
        tok = e.token_ids[0] if e.token_src < 0 else 0
        src[s] = e.token_src
        if not 0 <= tok < vocab_size:
            raise ValueError(f"token id {tok} of request {rid!r} is outside the vocabulary [0, {vocab_size})")
        for w in e.want:
            if w != 0:
                raise ValueError(f"want index {w} of request {rid!r} is outside its 1 tokens")
            logit_rows.append(s)
        computed, reserved, slot = manager.progress(rid)
        if computed + 1 > reserved:
            raise ValueError(f"request {rid!r}: tokens up to {computed + 1} have no slots reserved")
        tokens[s] = tok
        starts[s] = computed
        rows[s] = slot
    ps = manager.page_size
    kv_len = starts + 1
    width = int(starts.max()) // ps + 1
    slots, tables = [], []
    blocks = starts // ps
    offsets = starts - blocks * ps
    for g in range(len(manager.pools)):
        table = manager.table_array(g)
        pages = table[rows, blocks].astype(np.int64)
        if (pages < 0).any():
            raise ValueError("a token's position lies in a page the window has given back")
        slots.append(pages * ps + offsets)
        tables.append(table[rows, :width])
    return dict(token_ids=tokens, positions=starts, kv_len=kv_len, state_slot=rows, logit_rows=np.asarray(logit_rows, dtype=np.int64),
                slots=slots, tables=tables, S=S, width=width, token_src=src if (src >= 0).any() else None)


def build_batch(entries: Sequence[StepEntry], manager, device, vocab_size: int, uploader: Uploader | None = None,
                gathered: dict | None = None) -> tuple[StepBatch, list[int]]:
    """Flatten ``entries`` against the cache manager's tables.

    Each request's tokens must already have slots (allocate / append_slots); its first token
    sits at the position the manager has computed up to.  Returns the batch and, for each
    entry in the caller's order, its index in the batch's sequence order.  ``gathered``: what
    gather_host made of these entries, if the caller has it already.
    """
    h = gathered if gathered is not None else gather_host(entries, manager, vocab_size)
    n, S, width = h["n"], h["S"], h["width"]
    pieces = [h["token_ids"], h["positions"], h["seq_of_token"], h["q_start"], h["kv_len"], h["state_slot"], h["logit_rows"]]
    for g in range(len(manager.pools)):
        pieces += [h["slots"][g], h["tables"][g].reshape(-1)]
    if h["token_src"] is not None:
        pieces.append(h["token_src"])
    flat = np.concatenate([np.asarray(p).reshape(-1) for p in pieces]).astype(np.int32)
    dev = (uploader or Uploader(device)).upload(flat)
    cut = 0

    def take(count: int) -> torch.Tensor:
        nonlocal cut
        out = dev[cut : cut + count]
        cut += count
        return out

    b_tokens, b_pos, b_seq = take(n), take(n), take(n)
    b_qstart, b_kvlen, b_slot, b_rows = take(S + 1), take(S), take(S), take(h["logit_rows"].size)
    views = []
    for g in range(len(manager.pools)):
        gs = take(n)
        views.append(GroupView(take(S * width).view(S, width), gs))
    b_src = take(n) if h["token_src"] is not None else None
    q_lens = h["q_lens"].tolist()
    kv = h["kv_len"].tolist()
    batch = StepBatch(
        n=n, num_seqs=S, num_single=sum(1 for q in q_lens if q == 1), token_ids=b_tokens, positions=b_pos,
        seq_of_token=b_seq, q_start=b_qstart, kv_len=b_kvlen, state_slot=b_slot, logit_rows=b_rows, groups=views,
        q_lens=q_lens, starts=h["starts"].tolist(), state_slots=h["state_slot"].tolist(), max_q_len=max(q_lens), max_kv_len=max(kv),
        max_kv_len_single=max((k for k, q in zip(kv, q_lens) if q == 1), default=0),
        logits_all_rows=h["logit_rows"].size == n and bool((h["logit_rows"] == np.arange(n)).all()),
        token_src=b_src,
    )
    return batch, h["place"]
