"""Python wrappers of the hand-written CUDA kernels.

Every wrapper checks device, dtype, shape and contiguity, then launches on the
current CUDA stream through the compiled library's C entry point.  There is no
CPU or library fallback: a tensor that is not on a CUDA device, or a library
that cannot be built, raises.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..csrc.build import ExtensionError, load_library

DT_CODE = {torch.float32: 0, torch.bfloat16: 1}

# number of this package's kernels launched since import (a graph replay adds its node count)
launch_count = 0
DECODE_TMA_CLUSTER_SPLITS = 16  # CLUSTER_SPLITS_MAX of csrc/attention_tc.cu


class KernelError(RuntimeError):
    pass


_ERRORS = {1001: "size or option not supported by this kernel"}


def _check(code: int, what: str) -> None:
    global launch_count
    if code != 0:
        detail = _ERRORS.get(code)
        if detail is None:
            try:
                detail = torch.cuda.cudart().cudaGetErrorString(code)  # type: ignore[attr-defined]
            except Exception:
                detail = f"CUDA error {code}"
        raise KernelError(f"{what}: {detail} (code {code})")
    launch_count += 1


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: the engine has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")


_fns: dict[str, ctypes._CFuncPtr] = {}


def _fn(source: str, name: str, argtypes: list, defines: dict | None = None):
    key = f"{source}:{name}:{sorted((defines or {}).items())}"
    f = _fns.get(key)
    if f is None:
        lib = load_library(source, defines)
        try:
            f = getattr(lib, name)
        except AttributeError as exc:
            raise ExtensionError(f"{name} missing from {source}") from exc
        f.argtypes = argtypes
        f.restype = c_int
        _fns[key] = f
    return f


# ------------------------------------------------------------------ elementwise


def embedding(h: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    """h[t] = float32(table[ids[t]]); h is the float32 residual stream [n, H]."""
    _need(h, "h", torch.float32), _need(table, "table"), _need(ids, "ids", torch.int32)
    n, H = h.shape
    if table.shape[1] != H or ids.numel() != n or table.dtype not in DT_CODE:
        raise KernelError("embedding: shapes or dtype do not agree")
    f = _fn("elementwise.cu", "dli_embedding", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(table), _ptr(ids), n, H, DT_CODE[table.dtype], _stream()), "embedding")


def patch_tokens(ids: torch.Tensor, source: torch.Tensor, src: torch.Tensor) -> None:
    """ids[i] = source[src[i]] wherever src[i] >= 0: the token ids of a step that were sampled on
    the device by the step before and have not been read by the host."""
    _need(ids, "ids", torch.int32), _need(source, "source", torch.int32), _need(src, "src", torch.int32)
    if src.numel() != ids.numel():
        raise KernelError("patch_tokens: one source row per token")
    f = _fn("elementwise.cu", "dli_patch_tokens", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(source), _ptr(src), ids.numel(), _stream()), "patch_tokens")


def copy_page(pool: torch.Tensor, src: int, dst: int) -> None:
    """pool[:, dst] = pool[:, src] for a cache pool [layers, pages, ...] (copy-on-write of a forked
    request's last page)."""
    _need(pool, "pool")
    if pool.dim() < 2 or not (0 <= src < pool.shape[1] and 0 <= dst < pool.shape[1]):
        raise KernelError("copy_page: pool must be [layers, pages, ...] and the pages inside it")
    page_bytes = pool[0, 0].numel() * pool.element_size()
    f = _fn("elementwise.cu", "dli_copy_page", [c_void_p, c_longlong, c_longlong, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(pool), pool.shape[1] * page_bytes, page_bytes, pool.shape[0], src, dst, _stream()), "copy_page")


def add_rmsnorm(
    y: torch.Tensor,
    h: torch.Tensor,
    delta: torch.Tensor | None,
    weight: torch.Tensor,
    eps: float,
    rows: torch.Tensor | None = None,
) -> None:
    """y[r] = rmsnorm(h[s] + delta[s]) * weight with s = rows[r] (or r).

    Without ``rows`` the sum is written back to ``h`` (the residual stream moves on);
    with ``rows`` only the selected rows are read and ``h`` is left alone.
    """
    _need(y, "y"), _need(h, "h", torch.float32), _need(weight, "weight", torch.float32)
    H = h.shape[1]
    n_rows = y.shape[0]
    if y.dtype not in DT_CODE or y.shape[1] != H or weight.numel() != H:
        raise KernelError("add_rmsnorm: shapes or dtype do not agree")
    if delta is not None:
        _need(delta, "delta", y.dtype)
        if delta.shape != h.shape:
            raise KernelError("add_rmsnorm: delta and h differ in shape")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() != n_rows:
            raise KernelError("add_rmsnorm: one output row per entry of rows")
    elif n_rows != h.shape[0]:
        raise KernelError("add_rmsnorm: y and h differ in rows")
    f = _fn(
        "elementwise.cu", "dli_add_rmsnorm",
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    )
    _check(f(_ptr(y), _ptr(h), _ptr(delta), _ptr(weight), _ptr(rows), n_rows, H, eps, DT_CODE[y.dtype], _stream()), "add_rmsnorm")


def rotary_store(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    inv_freq: torch.Tensor | None,
    slots: torch.Tensor | None,
    k_pool: torch.Tensor | None,
    v_pool: torch.Tensor | None,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rotary_dim: int,
    page_size: int,
    write_kv: bool = True,
    table: torch.Tensor | None = None,
) -> None:
    """Rotate q and k heads of qkv [n, (nh + 2 nkv) d] by position; q in place, k and v into
    one layer's pools [pages, nkv, page_size, d] at ``slots`` (page * page_size + offset).
    ``table`` [n, rotary_dim] (from rotary_table) spares the kernel the sines and cosines."""
    _need(qkv, "qkv"), _need(positions, "positions", torch.int32)
    n = qkv.shape[0]
    if qkv.dtype not in DT_CODE or qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or positions.numel() != n:
        raise KernelError("rotary_store: shapes or dtype do not agree")
    if rotary_dim:
        if inv_freq is None:
            raise KernelError("rotary_store: inv_freq is needed when rotary_dim > 0")
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("rotary_store: inv_freq must have rotary_dim / 2 entries")
    if write_kv:
        if slots is None or k_pool is None or v_pool is None:
            raise KernelError("rotary_store: slots and pools are needed to write keys and values")
        _need(slots, "slots", torch.int32), _need(k_pool, "k_pool", qkv.dtype), _need(v_pool, "v_pool", qkv.dtype)
        if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, head_dim) or k_pool.shape != v_pool.shape or slots.numel() != n:
            raise KernelError("rotary_store: pool layout must be [pages, kv_heads, page_size, head_dim]")
    if table is not None:
        _need(table, "table", torch.float32)
        if tuple(table.shape) != (n, rotary_dim):
            raise KernelError("rotary_store: table must be [n, rotary_dim]")
    f = _fn(
        "elementwise.cu", "dli_rotary_store",
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 8 + [c_void_p],
    )
    _check(
        f(_ptr(qkv), _ptr(positions), _ptr(inv_freq), _ptr(table), _ptr(slots), _ptr(k_pool), _ptr(v_pool), n, num_heads, num_kv_heads,
          head_dim, rotary_dim, page_size, int(write_kv), DT_CODE[qkv.dtype], _stream()),
        "rotary_store",
    )


def rotary_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """cos | sin of float32(position) * inv_freq for every token: float32 [n, 2 * len(inv_freq)]."""
    _need(positions, "positions", torch.int32), _need(inv_freq, "inv_freq", torch.float32)
    n, rot = positions.numel(), 2 * inv_freq.numel()
    table = torch.empty((n, rot), dtype=torch.float32, device=positions.device)
    f = _fn("elementwise.cu", "dli_rotary_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(table), _ptr(positions), _ptr(inv_freq), n, rot, _stream()), "rotary_table")
    return table


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor, tiled: bool = False) -> None:
    """out[n, I] = silu(gate) * up.  gate_up [n, 2 I] holds gate | up side by side, or, ``tiled``
    (I a multiple of 64), blocks of 128 columns: 64 gate features, then the same 64 up features."""
    _need(out, "out"), _need(gate_up, "gate_up", out.dtype)
    n, I = out.shape
    if out.dtype not in DT_CODE or tuple(gate_up.shape) != (n, 2 * I) or (tiled and I % 64):
        raise KernelError("silu_mul: shapes or dtype do not agree")
    f = _fn("elementwise.cu", "dli_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(gate_up), n, I, int(tiled), DT_CODE[out.dtype], _stream()), "silu_mul")


# ------------------------------------------------------------------ attention


def paged_attention_simt(
    out: torch.Tensor,
    qkv: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_tables: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    num_heads: int,
    scale: float,
    window: int | None = None,
) -> None:
    """Causal attention of every token over its sequence's pages, on CUDA cores.

    out [n, nh * d]; queries are the first nh * d columns of qkv; pools [pages, nkv, page_size, d];
    block_tables [seqs, max_blocks]; a token at position p reads keys max(0, p - window + 1) .. p.
    """
    _need(out, "out"), _need(qkv, "qkv", out.dtype), _need(k_pool, "k_pool", out.dtype), _need(v_pool, "v_pool", out.dtype)
    _need(block_tables, "block_tables", torch.int32), _need(seq_of_token, "seq_of_token", torch.int32)
    _need(positions, "positions", torch.int32)
    n = out.shape[0]
    _, nkv, page_size, d = k_pool.shape
    if out.dtype not in DT_CODE or out.shape[1] != num_heads * d or qkv.shape[0] != n or qkv.shape[1] < num_heads * d:
        raise KernelError("paged_attention_simt: shapes or dtype do not agree")
    if d > 256 or num_heads % nkv:
        raise KernelError(f"paged_attention_simt: head_dim {d} (<= 256) / heads {num_heads} per kv head {nkv} not supported")
    f = _fn(
        "attention_simt.cu", "dli_paged_attention_simt",
        [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 6 + [c_float, c_int, c_void_p],
    )
    _check(
        f(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), block_tables.shape[1],
          _ptr(seq_of_token), _ptr(positions), n, num_heads, nkv, d, page_size, int(window or 0), scale, DT_CODE[out.dtype], _stream()),
        "paged_attention_simt",
    )


def prefill_tc_supported(head_dim: int, page_size: int) -> bool:
    return head_dim in (64, 128) and page_size in (8, 16, 32, 64, 128)


def paged_prefill_tc(
    out: torch.Tensor,
    qkv: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_tables: torch.Tensor,
    q_start: torch.Tensor,
    kv_len: torch.Tensor,
    seq0: int,
    num_seqs: int,
    max_q_len: int,
    num_heads: int,
    scale: float,
    window: int | None = None,
    query_tiles: int = 0,
) -> None:
    """bfloat16 attention for prompt portions on tcgen05 tensor cores with TMA-fed pages
    (head size 64 or 128; page sizes 8, 16, 32, 64, 128).  Arguments as paged_attention_mma.
    ``query_tiles`` (head size 64): 1 or 2 tiles of 128 (token, head) rows per CTA; 0 lets the launcher choose (two
    when a sequence brings more tokens than one tile holds)."""
    for t, name in ((out, "out"), (qkv, "qkv"), (k_pool, "k_pool"), (v_pool, "v_pool")):
        _need(t, name, torch.bfloat16)
    _need(block_tables, "block_tables", torch.int32), _need(q_start, "q_start", torch.int32), _need(kv_len, "kv_len", torch.int32)
    pages, nkv, page_size, d = k_pool.shape
    if not prefill_tc_supported(d, page_size):
        raise KernelError(f"paged_prefill_tc: head_dim {d} (64 or 128) or page size {page_size} (8..128, dividing 128) not supported")
    if out.shape[1] != num_heads * d or qkv.shape[0] != out.shape[0] or qkv.shape[1] < num_heads * d or num_heads % nkv or k_pool.shape != v_pool.shape:
        raise KernelError("paged_prefill_tc: shapes do not agree")
    if seq0 + num_seqs > kv_len.numel() or q_start.numel() != kv_len.numel() + 1:
        raise KernelError("paged_prefill_tc: sequence range outside the batch")
    f = _fn(
        "attention_tc.cu", "dli_paged_prefill_tc",
        [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 8 + [c_float, c_int, c_void_p],
    )
    if query_tiles not in (0, 1, 2):
        raise KernelError("paged_prefill_tc: query_tiles is 0 (choose), 1 or 2")
    _check(
        f(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), pages, _ptr(block_tables), block_tables.shape[1],
          _ptr(q_start), _ptr(kv_len), seq0, num_seqs, max_q_len, num_heads, nkv, d, page_size, int(window or 0), scale, query_tiles, _stream()),
        "paged_prefill_tc",
    )


def decode_tma_supported(head_dim: int, page_size: int) -> bool:
    return head_dim in (64, 128) and page_size % 8 == 0 and (page_size == 8 or page_size % 16 == 0) and page_size <= 256


def paged_decode_tma(
    out: torch.Tensor,
    qkv: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_tables: torch.Tensor,
    q_start: torch.Tensor,
    kv_len: torch.Tensor,
    seq0: int,
    num_seqs: int,
    first_row: int,
    num_heads: int,
    scale: float,
    window: int | None = None,
    splits: int = 1,
    scratch: tuple[torch.Tensor, torch.Tensor] | None = None,
    max_kv_len: int = 0,
) -> None:
    """bfloat16 attention of single-token sequences whose keys and values arrive by TMA (head size
    64 or 128; page sizes 8, 16, 32, ...).  Arguments as paged_attention_mma with max_q_len = 1.
    ``max_kv_len``: the longest sequence, if the host knows it (a hint: with few CTAs and long runs of keys
    the launcher gives a CTA eight warps instead of four); 0 if not."""
    for t, name in ((out, "out"), (qkv, "qkv"), (k_pool, "k_pool"), (v_pool, "v_pool")):
        _need(t, name, torch.bfloat16)
    _need(block_tables, "block_tables", torch.int32), _need(q_start, "q_start", torch.int32), _need(kv_len, "kv_len", torch.int32)
    pages, nkv, page_size, d = k_pool.shape
    if not decode_tma_supported(d, page_size):
        raise KernelError(f"paged_decode_tma: head_dim {d} (64 or 128) or page size {page_size} not supported")
    if out.shape[1] != num_heads * d or qkv.shape[0] != out.shape[0] or qkv.shape[1] < num_heads * d or num_heads % nkv or k_pool.shape != v_pool.shape:
        raise KernelError("paged_decode_tma: shapes do not agree")
    if seq0 + num_seqs > kv_len.numel() or q_start.numel() != kv_len.numel() + 1:
        raise KernelError("paged_decode_tma: sequence range outside the batch")
    acc = ml = None
    if splits > 1:
        if scratch is None:
            raise KernelError("paged_decode_tma: split keys need scratch")
        acc, ml = scratch
        _need(acc, "scratch[0]", torch.float32), _need(ml, "scratch[1]", torch.float32)
        rows = (first_row + num_seqs) * num_heads
        if acc.numel() < rows * splits * d or ml.numel() < rows * splits * 2:
            raise KernelError("paged_decode_tma: scratch too small")
    f = _fn(
        "attention_tc.cu", "dli_paged_decode_tma",
        [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 8
        + [c_float, c_int, c_void_p, c_void_p, c_int, c_void_p],
    )
    _check(
        f(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), pages, _ptr(block_tables), block_tables.shape[1],
          _ptr(q_start), _ptr(kv_len), seq0, num_seqs, first_row, num_heads, nkv, d, page_size, int(window or 0), scale, splits,
          _ptr(acc), _ptr(ml), int(max_kv_len), _stream()),
        "paged_decode_tma",
    )
    global launch_count
    if splits > 1 and not _fn("attention_tc.cu", "dli_decode_tma_merges_in_cluster", [c_int, c_int, c_int])(num_heads, nkv, splits):
        launch_count += 1  # the merge kernel; otherwise the splits merge inside the kernel, as one cluster


def paged_prefill_tc_error() -> int:
    """0, or which bounded wait of the tcgen05 / TMA attention kernels ran out since the library was loaded
    (or since the code was last cleared)."""
    return _fn("attention_tc.cu", "dli_paged_prefill_tc_error", [])()


def _library_in_use(source: str) -> bool:
    return any(key.startswith(source + ":") for key in _fns)


def device_wait_errors(clear: bool = True) -> dict[str, int]:
    """Bounded device waits that ran out: {library: code} for the libraries this process has used
    (a library nobody called has recorded nothing and is not built for the question).  The flags live
    in mapped host memory, so reading them costs no copy; read them once the step's results have
    reached the host.  With ``clear`` a code that was read is forgotten."""
    found = {}
    for source, read, forget in (("skinny_gemm.cu", "dli_skinny_gemm_error", "dli_skinny_gemm_clear_error"),
                                 ("dense_gemm.cu", "dli_dense_gemm_error", "dli_dense_gemm_clear_error"),
                                 ("attention_tc.cu", "dli_paged_prefill_tc_error", "dli_paged_prefill_tc_clear_error")):
        if not _library_in_use(source):
            continue
        code = _fn(source, read, [])()
        if code:
            found[source] = int(code)
            if clear:
                _fn(source, forget, [])()
    return found


# ------------------------------------------------------------------ sampling


# A stochastic row's logits are kept in the shared memory of a cluster of 8 CTAs, 47 K floats each
SAMPLE_MAX_VOCAB_STOCHASTIC = 8 * 47 * 1024


def sample(
    out: torch.Tensor,
    logits: torch.Tensor,
    temperature: torch.Tensor | None = None,
    top_k: torch.Tensor | None = None,
    top_p: torch.Tensor | None = None,
    seed: torch.Tensor | None = None,
    draw: torch.Tensor | None = None,
    slots: torch.Tensor | None = None,
) -> None:
    """out[r] = token of row r of float32 logits [rows, V]; all-greedy when temperature is None.
    seed and draw are int64 tensors read as unsigned 64-bit.  With ``slots`` (int32, one per row) the five
    parameter tensors are tables indexed by slots[r] instead of r (the requests' state slots), and the draw
    count of every stochastic row's slot is advanced by one on the device."""
    _need(out, "out", torch.int32), _need(logits, "logits", torch.float32)
    rows, V = logits.shape
    if out.numel() != rows:
        raise KernelError("sample: one output per row")
    if temperature is not None:
        if top_k is None or top_p is None or seed is None or draw is None:
            raise KernelError("sample: stochastic rows need top_k, top_p, seed and draw")
        if V > SAMPLE_MAX_VOCAB_STOCHASTIC:
            raise KernelError(f"sample: temperature sampling takes vocabularies of up to {SAMPLE_MAX_VOCAB_STOCHASTIC} tokens, not {V} "
                              "(greedy rows alone, passed without parameters, take any)")
        _need(temperature, "temperature", torch.float32), _need(top_k, "top_k", torch.int32), _need(top_p, "top_p", torch.float32)
        _need(seed, "seed", torch.int64), _need(draw, "draw", torch.int64)
        entries = rows if slots is None else temperature.numel()
        if not (temperature.numel() == top_k.numel() == top_p.numel() == seed.numel() == draw.numel() == entries):
            raise KernelError("sample: one parameter per row (or, with slots, tables of one length)")
    if slots is not None:
        _need(slots, "slots", torch.int32)
        if temperature is None or slots.numel() != rows:
            raise KernelError("sample: slots go with parameter tables and name one slot per row")
    f = _fn(
        "sampling.cu", "dli_sample",
        [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    )
    _check(
        f(_ptr(out), _ptr(logits), logits.stride(0), rows, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(seed), _ptr(draw), _ptr(slots),
          _stream()),
        "sample",
    )


def mma_head_dim_supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def paged_attention_mma(
    out: torch.Tensor,
    qkv: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_tables: torch.Tensor,
    q_start: torch.Tensor,
    kv_len: torch.Tensor,
    seq0: int,
    num_seqs: int,
    max_q_len: int,
    first_row: int,
    num_heads: int,
    scale: float,
    window: int | None = None,
    splits: int = 1,
    scratch: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> None:
    """bfloat16 tensor-core attention for the sequences [seq0, seq0 + num_seqs) of a batch.

    Queries are the first nh * d columns of qkv; a sequence's tokens sit in rows
    q_start[s] .. q_start[s + 1] at positions kv_len[s] - q_len .. kv_len[s] - 1.  With
    ``splits`` > 1 (single-token sequences only) the keys are cut into that many runs;
    ``scratch`` = (float32 [rows * splits * d], float32 [rows * splits * 2]) with
    rows = (first_row + num_seqs) * nh holds the partial results.
    """
    for t, name in ((out, "out"), (qkv, "qkv"), (k_pool, "k_pool"), (v_pool, "v_pool")):
        _need(t, name, torch.bfloat16)
    _need(block_tables, "block_tables", torch.int32), _need(q_start, "q_start", torch.int32), _need(kv_len, "kv_len", torch.int32)
    _, nkv, page_size, d = k_pool.shape
    if not mma_head_dim_supported(d):
        raise KernelError(f"paged_attention_mma: head_dim {d} is not a multiple of 16 in [16, 256]")
    if out.shape[1] != num_heads * d or qkv.shape[0] != out.shape[0] or qkv.shape[1] < num_heads * d or num_heads % nkv:
        raise KernelError("paged_attention_mma: shapes do not agree")
    if seq0 + num_seqs > kv_len.numel() or q_start.numel() != kv_len.numel() + 1:
        raise KernelError("paged_attention_mma: sequence range outside the batch")
    acc = ml = None
    if splits > 1:
        if max_q_len != 1 or scratch is None:
            raise KernelError("paged_attention_mma: split keys need single-token sequences and scratch")
        acc, ml = scratch
        _need(acc, "scratch[0]", torch.float32), _need(ml, "scratch[1]", torch.float32)
        rows = (first_row + num_seqs) * num_heads
        if acc.numel() < rows * splits * d or ml.numel() < rows * splits * 2:
            raise KernelError("paged_attention_mma: scratch too small")
    f = _fn(
        "attention_mma.cu", "dli_paged_attention_mma",
        [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        + [c_int] * 8 + [c_float, c_int, c_void_p, c_void_p, c_void_p],
        {"HEAD_DIM": d},
    )
    _check(
        f(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), block_tables.shape[1],
          _ptr(q_start), _ptr(kv_len), seq0, num_seqs, max_q_len, first_row, num_heads, nkv, page_size, int(window or 0),
          scale, splits, _ptr(acc), _ptr(ml), _stream()),
        "paged_attention_mma",
    )
    global launch_count
    if splits > 1:
        launch_count += 1  # the merge kernel


# ------------------------------------------------------------------ decode matrix product


def skinny_gemm_supported(tokens: int, in_features: int) -> bool:
    return 1 <= tokens <= 256 and in_features >= 8 and in_features % 8 == 0


class ScaledRows:
    """Activations whose rows still lack a factor: ``x`` [n, size] holds bfloat16(h * gain) of a
    residual stream h, ``ssq`` [n, tiles] float32 the sums of h^2 over tiles of 128 features, and
    the finished RMS norm is x[t] * rsqrt(sum(ssq[t]) / size + eps).  A factor per row commutes
    with a matrix product, so the decode products take this as their input and apply the factor
    to their float32 sums (``skinny_gemm*``); ``skinny_gemm_residual`` makes it."""

    __slots__ = ("x", "ssq", "eps")

    def __init__(self, x: torch.Tensor, ssq: torch.Tensor, eps: float) -> None:
        self.x, self.ssq, self.eps = x, ssq, float(eps)

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device


def _row_scale(x, name: str):
    """(activations, the four row-scaling arguments of the kernel) for a tensor or ScaledRows."""
    if not isinstance(x, ScaledRows):
        return x, (None, 0, 0.0, 0)
    _need(x.ssq, name + ".ssq", torch.float32)
    n, size = x.x.shape
    if x.ssq.dim() != 2 or x.ssq.shape[0] != n or n > 64:
        raise KernelError(f"{name}: row sums of squares must be [tokens <= 64, tiles]")
    return x.x, (_ptr(x.ssq), x.ssq.shape[1], x.eps, size)


_ROW_SCALE_ARGS = [c_void_p, c_int, c_float, c_int]
_slices_cache: dict[tuple[int, int, int], int] = {}


def skinny_gemm_slices(tokens: int, features: int, in_features: int) -> int:
    """K slices the kernel's launcher recommends for these sizes."""
    key = (tokens, features, in_features)
    n = _slices_cache.get(key)
    if n is None:
        n = _slices_cache[key] = _fn("skinny_gemm.cu", "dli_skinny_gemm_slices", [c_int, c_int, c_int])(*key)
    return n


def skinny_gemm(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, slices: int | None = None,
                out: torch.Tensor | None = None, max_stages: int = 0) -> torch.Tensor:
    """x [tokens <= 256, K] times weight [features, K] transposed, bfloat16 in, on tcgen05 tensor
    cores fed by TMA; returns [tokens, features] in bfloat16 or float32.  ``slices`` (1..16) cuts K
    across the CTAs of a cluster, which add their partial sums through distributed shared memory."""
    x, scale = _row_scale(x, "skinny_gemm")
    _need(x, "x", torch.bfloat16), _need(weight, "weight", torch.bfloat16)
    tokens, K = x.shape
    features = weight.shape[0]
    if weight.shape[1] != K or not skinny_gemm_supported(tokens, K) or out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"skinny_gemm: tokens {tokens} (1..256), K {K} (a multiple of 8) or output {out_dtype} not supported")
    if slices is not None and not 1 <= slices <= 16:
        raise KernelError("skinny_gemm: 1 to 16 K slices")
    if slices is None:
        slices = skinny_gemm_slices(tokens, features, K)
    if out is None:
        out = torch.empty((tokens, features), dtype=out_dtype, device=x.device)
    else:
        _need(out, "out", out_dtype)
        if tuple(out.shape) != (tokens, features):
            raise KernelError("skinny_gemm: out has the wrong shape")
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int] + _ROW_SCALE_ARGS + [c_void_p])
    _check(f(_ptr(out), int(out_dtype == torch.float32), _ptr(x), _ptr(weight), tokens, features, K, slices, max_stages, *scale, _stream()), "skinny_gemm")
    return out


def skinny_gemm_wait_test(x: torch.Tensor, weight: torch.Tensor, slices: int, wait_limit: int, skip_tile: int) -> torch.Tensor:
    """For the test of the kernel's bounded waits: the plain product in float32, except that the copies of k tile
    ``skip_tile`` (64 columns of K each) are left out and every wait gives up after ``wait_limit`` polls.  The
    kernel then records code 2 (``skinny_gemm_error``), stores what it has and returns; nothing hangs or
    faults.  ``skip_tile`` must be the last tile of its slice and K / 64 / slices at most 8.  Not used by the engine."""
    _need(x, "x", torch.bfloat16), _need(weight, "weight", torch.bfloat16)
    tokens, K = x.shape
    features = weight.shape[0]
    per = -(-(-(-K // 64)) // slices)
    if weight.shape[1] != K or not 1 <= slices <= 16 or per > 8 or skip_tile < 0 or (skip_tile + 1) % per:
        raise KernelError("skinny_gemm_wait_test: the tile left out must be the last one of a slice of at most 8 tiles")
    out = torch.zeros((tokens, features), dtype=torch.float32, device=x.device)
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm_wait_test", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, ctypes.c_uint, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(weight), tokens, features, K, slices, wait_limit, skip_tile, _stream()), "skinny_gemm_wait_test")
    return out


def skinny_gemm_residual(x, weight: torch.Tensor, h: torch.Tensor, gain: torch.Tensor, eps: float, slices: int | None = None) -> ScaledRows:
    """h += x W^T (float32, in place) and the first half of the RMS norm that follows, in the
    product's epilogue: returns ScaledRows(bfloat16(h * gain), sums of h^2 per 128 features, eps).
    x [tokens <= 64, K] may itself be ScaledRows."""
    x, scale = _row_scale(x, "skinny_gemm_residual")
    _need(x, "x", torch.bfloat16), _need(weight, "weight", torch.bfloat16), _need(h, "h", torch.float32), _need(gain, "gain", torch.float32)
    tokens, K = x.shape
    features = weight.shape[0]
    if weight.shape[1] != K or not skinny_gemm_supported(tokens, K) or tokens > 64:
        raise KernelError(f"skinny_gemm_residual: tokens {tokens} (1..64) or K {K} (a multiple of 8) not supported")
    if tuple(h.shape) != (tokens, features) or gain.numel() != features:
        raise KernelError("skinny_gemm_residual: h must be [tokens, features] and gain [features]")
    if slices is None:
        slices = skinny_gemm_slices(tokens, features, K)
    out = torch.empty((tokens, features), dtype=torch.bfloat16, device=x.device)
    ssq = torch.empty((tokens, (features + 127) // 128), dtype=torch.float32, device=x.device)
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm_residual",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int] + _ROW_SCALE_ARGS + [c_void_p])
    _check(f(_ptr(out), _ptr(h), _ptr(gain), _ptr(ssq), _ptr(x), _ptr(weight), tokens, features, K, slices, *scale, _stream()), "skinny_gemm_residual")
    return ScaledRows(out, ssq, eps)


def skinny_gemm_swiglu(x: torch.Tensor, weight_tiled: torch.Tensor) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) in one kernel: the decode matrix product with the activation in its
    epilogue.  weight_tiled [2 I, K]: rows in blocks of 128 — 64 gate rows, then the 64 up rows of
    the same features.  Returns bfloat16 [tokens, I]."""
    x, scale = _row_scale(x, "skinny_gemm_swiglu")
    _need(x, "x", torch.bfloat16), _need(weight_tiled, "weight", torch.bfloat16)
    tokens, K = x.shape
    features = weight_tiled.shape[0]
    if weight_tiled.shape[1] != K or features % 128 or not skinny_gemm_supported(tokens, K):
        raise KernelError("skinny_gemm_swiglu: sizes not supported")
    out = torch.empty((tokens, features // 2), dtype=torch.bfloat16, device=x.device)
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm_swiglu", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int] + _ROW_SCALE_ARGS + [c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(weight_tiled), tokens, features, K, skinny_gemm_slices(tokens, features, K), *scale, _stream()), "skinny_gemm_swiglu")
    return out


def skinny_rotary_supported(head_dim: int) -> bool:
    return head_dim >= 2 and 128 % head_dim == 0


def skinny_gemm_rotary(x, wqkv, positions, inv_freq, slots, k_pool, v_pool, num_heads: int, num_kv_heads: int, head_dim: int,
                       rotary_dim: int, page_size: int, write_kv: bool) -> torch.Tensor:
    """q | k | v = x Wqkv^T with the rotary embedding and the write of keys and values into the
    cache pages done in the product's epilogue; returns the rotated queries [tokens, nh * d]."""
    x, scale = _row_scale(x, "skinny_gemm_rotary")
    _need(x, "x", torch.bfloat16), _need(wqkv, "wqkv", torch.bfloat16), _need(positions, "positions", torch.int32)
    tokens, K = x.shape
    features = (num_heads + 2 * num_kv_heads) * head_dim
    if tuple(wqkv.shape) != (features, K) or not skinny_gemm_supported(tokens, K) or not skinny_rotary_supported(head_dim):
        raise KernelError("skinny_gemm_rotary: sizes not supported")
    if rotary_dim:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("skinny_gemm_rotary: inv_freq must have rotary_dim / 2 entries")
    if write_kv:
        _need(slots, "slots", torch.int32), _need(k_pool, "k_pool", torch.bfloat16), _need(v_pool, "v_pool", torch.bfloat16)
        if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, head_dim) or k_pool.shape != v_pool.shape or slots.numel() != tokens:
            raise KernelError("skinny_gemm_rotary: pool layout must be [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((tokens, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm_rotary",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 6
            + _ROW_SCALE_ARGS + [c_void_p])
    _check(f(_ptr(q), _ptr(x), _ptr(wqkv), tokens, K, skinny_gemm_slices(tokens, features, K), _ptr(positions),
             _ptr(inv_freq if rotary_dim else None), _ptr(slots if write_kv else None), _ptr(k_pool if write_kv else None),
             _ptr(v_pool if write_kv else None), num_heads, num_kv_heads, head_dim, rotary_dim, page_size, int(write_kv), *scale, _stream()),
           "skinny_gemm_rotary")
    return q


# ------------------------------------------------------------------ matrix product of many tokens
# A portion of a prompt: tokens are the 128-row side of the tensor-core instruction, a thread of the epilogue holds
# one token's row of a tile, and the elementwise step behind the product is done on the sums before they are stored.


def dense_gemm_supported(in_features: int, features: int) -> bool:
    return in_features >= 8 and in_features % 8 == 0 and features >= 8 and features % 8 == 0


def dense_rotary_supported(head_dim: int, rotary_dim: int) -> bool:
    return head_dim in (64, 128) and rotary_dim in (0, 64, 128) and rotary_dim <= head_dim


def _dense_sizes(x: torch.Tensor, weight: torch.Tensor, name: str):
    _need(x, "x", torch.bfloat16), _need(weight, "weight", torch.bfloat16)
    tokens, K = x.shape
    features = weight.shape[0]
    if weight.shape[1] != K or tokens < 1 or not dense_gemm_supported(K, features):
        raise KernelError(f"{name}: K {K} and features {features} must be multiples of 8 and the shapes agree")
    return tokens, features, K


def dense_gemm(x, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [tokens, K] times weight [features, K] transposed, bfloat16 in and out, float32 sums, on tcgen05 tensor
    cores fed by TMA: persistent pairs of CTAs (cta_group::2) over tiles of 256 tokens x 256 features, two
    accumulators in each CTA's tensor memory."""
    tokens, features, K = _dense_sizes(x, weight, "dense_gemm")
    if out is None:
        out = torch.empty((tokens, features), dtype=torch.bfloat16, device=x.device)
    else:
        _need(out, "out", torch.bfloat16)
        if tuple(out.shape) != (tokens, features):
            raise KernelError("dense_gemm: out has the wrong shape")
    f = _fn("dense_gemm.cu", "dli_dense_gemm", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(weight), tokens, features, K, _stream()), "dense_gemm")
    return out


def dense_gemm_swiglu(x, weight_tiled: torch.Tensor) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) in the product's epilogue.  weight_tiled [2 I, K]: rows in blocks of 128 — 64 gate
    rows, then the 64 up rows of the same features.  Returns bfloat16 [tokens, I]."""
    tokens, features, K = _dense_sizes(x, weight_tiled, "dense_gemm_swiglu")
    if features % 128:
        raise KernelError("dense_gemm_swiglu: the interleaved layout needs an intermediate size that is a multiple of 64")
    act = torch.empty((tokens, features // 2), dtype=torch.bfloat16, device=x.device)
    f = _fn("dense_gemm.cu", "dli_dense_gemm_swiglu", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(act), _ptr(x), _ptr(weight_tiled), tokens, features, K, _stream()), "dense_gemm_swiglu")
    return act


def dense_gemm_rotary(x, wqkv, table, slots, k_pool, v_pool, num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int,
                      page_size: int, write_kv: bool) -> torch.Tensor:
    """q | k | v = x Wqkv^T with the rotary embedding (``table`` [tokens, rotary_dim]: cos | sin of every token's
    angles, as ``rotary_table`` makes it) and the write of keys and values into the cache pages done in the
    product's epilogue; returns the rotated queries [tokens, nh * d]."""
    features = (num_heads + 2 * num_kv_heads) * head_dim
    tokens, _, K = _dense_sizes(x, wqkv, "dense_gemm_rotary")
    if wqkv.shape[0] != features or not dense_rotary_supported(head_dim, rotary_dim):
        raise KernelError("dense_gemm_rotary: sizes not supported")
    if rotary_dim:
        _need(table, "table", torch.float32)
        if tuple(table.shape) != (tokens, rotary_dim):
            raise KernelError("dense_gemm_rotary: table must be [tokens, rotary_dim]")
    if write_kv:
        _need(slots, "slots", torch.int32), _need(k_pool, "k_pool", torch.bfloat16), _need(v_pool, "v_pool", torch.bfloat16)
        if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, head_dim) or k_pool.shape != v_pool.shape or slots.numel() != tokens:
            raise KernelError("dense_gemm_rotary: pool layout must be [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((tokens, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    f = _fn("dense_gemm.cu", "dli_dense_gemm_rotary",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 6 + [c_void_p])
    _check(f(_ptr(q), _ptr(x), _ptr(wqkv), tokens, K, _ptr(table if rotary_dim else None), _ptr(slots if write_kv else None),
             _ptr(k_pool if write_kv else None), _ptr(v_pool if write_kv else None), num_heads, num_kv_heads, head_dim, rotary_dim,
             page_size, int(write_kv), _stream()), "dense_gemm_rotary")
    return q


def dense_gemm_wait_test(x: torch.Tensor, weight: torch.Tensor, wait_limit: int) -> torch.Tensor:
    """For the test of the kernel's bounded waits: the product of one tile (tokens <= 256, features <= 256, K <= 384)
    in which neither CTA of the pair issues the copies of the last k step and every wait gives up after
    ``wait_limit`` polls.  The kernel records a code (``dense_gemm_error``: 3, the wait for operands, or 4, the wait
    for the accumulator that depends on them), both CTAs end together and free their tensor memory; nothing hangs or
    faults.  Not used by the engine."""
    tokens, features, K = _dense_sizes(x, weight, "dense_gemm_wait_test")
    out = torch.zeros((tokens, features), dtype=torch.bfloat16, device=x.device)
    f = _fn("dense_gemm.cu", "dli_dense_gemm_wait_test", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, ctypes.c_uint, c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(weight), tokens, features, K, int(wait_limit), _stream()), "dense_gemm_wait_test")
    return out


def dense_gemm_error() -> int:
    """0, or which bounded wait of the many-token product ran out (1 copies, 2 and 3 products, 4 epilogue)."""
    return _fn("dense_gemm.cu", "dli_dense_gemm_error", [])()


def skinny_gemm_error() -> int:
    """0, or which bounded wait of the decode matrix product ran out since the library was loaded."""
    return _fn("skinny_gemm.cu", "dli_skinny_gemm_error", [])()
