"""The device-side description of one step's batch.

A step is a list of entries (request, its next tokens, the places whose logits
are wanted).  All entries are flattened into one token vector; entries of a
single token come first, longer portions after them (attention kernels launch
once per kind), and ``logit_rows`` restores the caller's order.  Every integer
array of a step travels to the device in one pinned copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import torch


@dataclass(frozen=True)
class StepEntry:
    request_id: Hashable
    token_ids: Sequence[int]  # the request's next tokens, at positions start .. start + len - 1
    want: Sequence[int] = ()  # indices into token_ids whose logits are returned


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
    forced_splits: int = 0  # key splits of decode attention fixed by the caller (0: chosen per step)

    def group(self, index: int) -> GroupView:
        return self.groups[index]


def build_batch(entries: Sequence[StepEntry], manager, device, vocab_size: int) -> tuple[StepBatch, list[int]]:
    """Flatten ``entries`` against the cache manager's tables.

    Each request's tokens must already have slots (allocate / append_slots); its first token
    sits at the position the manager has computed up to.  Returns the batch and, for each
    entry in the caller's order, its index in the batch's sequence order.
    """
    if not entries:
        raise ValueError("a step needs at least one entry")
    seen = set()
    for e in entries:
        if e.request_id in seen:
            raise ValueError(f"request {e.request_id!r} appears twice in one step")
        seen.add(e.request_id)
        if len(e.token_ids) == 0:
            raise ValueError(f"request {e.request_id!r} brings no tokens")
        for t in e.token_ids:
            if not 0 <= t < vocab_size:
                raise ValueError(f"token id {t} of request {e.request_id!r} is outside the vocabulary [0, {vocab_size})")
        for w in e.want:
            if not 0 <= w < len(e.token_ids):
                raise ValueError(f"want index {w} of request {e.request_id!r} is outside its {len(e.token_ids)} tokens")
    order = sorted(range(len(entries)), key=lambda i: (len(entries[i].token_ids) != 1, i))
    place = [0] * len(entries)
    for new, old in enumerate(order):
        place[old] = new

    token_ids: list[int] = []
    positions: list[int] = []
    seq_of_token: list[int] = []
    q_start = [0]
    kv_len: list[int] = []
    state_slot: list[int] = []
    starts: list[int] = []
    num_groups = len(manager.pools)
    slots: list[list[int]] = [[] for _ in range(num_groups)]
    tables: list[list[list[int]]] = [[] for _ in range(num_groups)]
    for s, old in enumerate(order):
        e = entries[old]
        start = manager.num_computed_tokens(e.request_id)
        end = start + len(e.token_ids)
        if end > manager.num_tokens(e.request_id):
            raise ValueError(f"request {e.request_id!r}: tokens up to {end} have no slots reserved")
        token_ids.extend(e.token_ids)
        positions.extend(range(start, end))
        seq_of_token.extend([s] * len(e.token_ids))
        q_start.append(len(token_ids))
        kv_len.append(end)
        starts.append(start)
        state_slot.append(manager.state_slot(e.request_id))
        for g in range(num_groups):
            slots[g].extend(manager.slot_mapping(e.request_id, g, start, end))
            tables[g].append(manager.block_table(e.request_id, g))
    logit_rows = [q_start[place[i]] + w for i, e in enumerate(entries) for w in e.want]

    n, S = len(token_ids), len(order)
    widths = [max(1, max(len(t) for t in tables[g])) for g in range(num_groups)]
    flat: list[int] = []
    flat += token_ids + positions + seq_of_token + q_start + kv_len + state_slot + logit_rows
    for g in range(num_groups):
        flat += slots[g]
        for t in tables[g]:
            flat += t + [-1] * (widths[g] - len(t))
    host = torch.tensor(flat, dtype=torch.int32)
    if torch.device(device).type == "cuda":
        host = host.pin_memory()
    dev = host.to(device, non_blocking=True)
    cut = 0

    def take(count: int) -> torch.Tensor:
        nonlocal cut
        out = dev[cut : cut + count]
        cut += count
        return out

    b_tokens, b_pos, b_seq = take(n), take(n), take(n)
    b_qstart, b_kvlen, b_slot, b_rows = take(S + 1), take(S), take(S), take(len(logit_rows))
    views = []
    for g in range(num_groups):
        gs = take(n)
        views.append(GroupView(take(S * widths[g]).view(S, widths[g]), gs))
    q_lens = [q_start[i + 1] - q_start[i] for i in range(S)]
    batch = StepBatch(
        n=n, num_seqs=S, num_single=sum(1 for q in q_lens if q == 1), token_ids=b_tokens, positions=b_pos,
        seq_of_token=b_seq, q_start=b_qstart, kv_len=b_kvlen, state_slot=b_slot, logit_rows=b_rows, groups=views,
        q_lens=q_lens, starts=starts, state_slots=state_slot, max_q_len=max(q_lens), max_kv_len=max(kv_len),
        max_kv_len_single=max((k for k, q in zip(kv_len, q_lens) if q == 1), default=0),
    )
    return batch, place
