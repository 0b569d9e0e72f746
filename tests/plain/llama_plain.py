"""Plain, slow implementation of the Llama 3.2 / SmolLM2 decoder in numpy.

Whole sequences, no cache, one function per part.  It shares no code with the
engine: it reads config.json keys itself, has its own safetensors reader and
its own random-number generator for sampling.  Every function cites the file
and lines of zshabb/distributed-llm-inference whose formula it restates.

A comparison of this file with the reference's own model code (run once on the
CPU on tiny random models) lives in ``tests/golden/``: ``make_golden.py`` made
the committed arrays, ``tests/test_plain_vs_golden.py`` checks them.

All arithmetic is float32 unless ``dtype=np.float64`` is asked for.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np

# --------------------------------------------------------------------------- config


def read_config(cfg: dict) -> dict:
    """The keys the decoder needs, with the reference's defaults.

    src/dli/model/config.py:80-127 (from_hf_dict) and :130-150 (_parse_rope).
    """
    heads = int(cfg["num_attention_heads"])
    hidden = int(cfg["hidden_size"])
    merged = {**dict(cfg.get("rope_scaling") or {}), **dict(cfg.get("rope_parameters") or {})}
    rope_type = merged.get("rope_type", merged.get("type", "default"))
    out = {
        "vocab": int(cfg["vocab_size"]),
        "hidden": hidden,
        "inter": int(cfg["intermediate_size"]),
        "layers": int(cfg["num_hidden_layers"]),
        "heads": heads,
        "kv_heads": int(cfg.get("num_key_value_heads") or heads),
        "head_dim": int(cfg.get("head_dim") or hidden // heads),
        "eps": float(cfg["rms_norm_eps"]),
        "tied": bool(cfg.get("tie_word_embeddings", False)),
        "theta": float(merged.get("rope_theta", cfg.get("rope_theta", 10000.0))),
        "rope_type": rope_type,
    }
    if rope_type != "default":
        out["factor"] = float(merged["factor"])
        out["low"] = float(merged.get("low_freq_factor", 1.0))
        out["high"] = float(merged.get("high_freq_factor", 4.0))
        out["old_ctx"] = int(
            merged.get("original_max_position_embeddings", cfg.get("max_position_embeddings", 8192))
        )
    return out


# --------------------------------------------------------------------------- weights


def read_safetensors(path: str | Path) -> dict[str, np.ndarray]:
    """Read every tensor of one safetensors file as float32 arrays.

    File layout: 8-byte little-endian header length, JSON header
    ``{name: {dtype, shape, data_offsets}}``, raw little-endian data.
    (The reference reads through the safetensors package, src/dli/model/loader.py:70-73.)
    """
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = raw[base + lo : base + hi]
        if info["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4")
        elif info["dtype"] == "BF16":
            arr = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        else:
            raise ValueError(f"plain reader: dtype {info['dtype']} of {name}")
        out[name] = arr.reshape(info["shape"]).astype(np.float32)
    return out


def round_to_bfloat16(x: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16 (ties to even), returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    # 32-bit arithmetic: the sum wraps only for bit patterns above 0xFFFF8000, which are NaNs (put back below)
    out = (bits + (np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1)))) & np.uint32(0xFFFF0000)
    out = out.view(np.float32).reshape(x.shape)
    nan = np.isnan(x)
    if nan.any():
        out[nan] = np.nan
    return out


# --------------------------------------------------------------------------- parts


def inverse_frequencies(c: dict) -> np.ndarray:
    """Per-pair inverse frequencies [head_dim/2], float32.  src/dli/model/rope.py:21-47."""
    d = c["head_dim"]
    f32 = np.float32
    exponents = np.arange(0, d, 2, dtype=np.int64).astype(f32) / f32(d)
    inv = (f32(1.0) / np.power(f32(c["theta"]), exponents, dtype=f32)).astype(f32)
    if c["rope_type"] == "default":
        return inv
    if c["rope_type"] == "linear":
        return (inv / f32(c["factor"])).astype(f32)
    if c["rope_type"] != "llama3":
        raise ValueError(c["rope_type"])
    old = c["old_ctx"]
    low_wl = old / c["low"]
    high_wl = old / c["high"]
    wavelen = (f32(2 * math.pi) / inv).astype(f32)
    scaled = np.where(wavelen > f32(low_wl), inv / f32(c["factor"]), inv).astype(f32)
    smooth = ((f32(old) / wavelen - f32(c["low"])) / f32(c["high"] - c["low"])).astype(f32)
    smoothed = ((f32(1) - smooth) * scaled / f32(c["factor"]) + smooth * scaled).astype(f32)
    medium = ~(wavelen < f32(high_wl)) & ~(wavelen > f32(low_wl))
    return np.where(medium, smoothed, scaled).astype(f32)


def rope_cos_sin(inv_freq: np.ndarray, positions: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """cos/sin tables [n, head_dim]; angles in float32.  src/dli/model/rope.py:50-60."""
    angles = positions.astype(np.float32)[:, None] * inv_freq.astype(np.float32)[None, :]
    emb = np.concatenate([angles, angles], axis=-1).astype(np.float32)
    # cos/sin of a float32 angle, evaluated in double and rounded once
    return np.cos(emb.astype(np.float64)).astype(np.float32), np.sin(emb.astype(np.float64)).astype(np.float32)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Rotate-half rotation of x [heads, n, d].  src/dli/model/rope.py:63-70."""
    half = x.shape[-1] // 2
    rot = np.concatenate([-x[..., half:], x[..., :half]], axis=-1)
    return x * cos + rot * sin


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """x * rsqrt(mean(x^2) + eps) * w.  src/dli/model/llama.py:41-44."""
    x = x.astype(w.dtype)
    var = np.mean(x * x, axis=-1, keepdims=True)
    return w * (x / np.sqrt(var + w.dtype.type(eps)))


def _same(x):
    return x


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: int | None = None, rnd=_same) -> np.ndarray:
    """softmax(q k^T / sqrt(d) + causal mask) v for one whole sequence.

    q [heads, n, d]; k, v [kv_heads, n, d]; query head h reads kv head h // (heads/kv_heads).
    src/dli/model/llama.py:147-177 (expansion :158-163, causal case :169).
    ``window`` (keys u with p - u < window) is not part of the reference's architecture;
    it exists so that the engine's generic attention part can be checked with one.
    ``rnd`` (identity, or round_to_bfloat16): applied to the unnormalised probabilities before the product
    with v, as a bfloat16 tensor-core kernel must (src/dli/model/paged_attention.py:167 does the same);
    the row sums stay float32.
    """
    heads, n, d = q.shape
    fan = heads // k.shape[0]
    qi = np.arange(n)[:, None]
    ki = np.arange(n)[None, :]
    mask = ki <= qi
    if window is not None:
        mask &= (qi - ki) < window
    out = np.empty_like(q)
    for h in range(heads):  # head by head: a square of scores at a time, however long the sequence
        s = (q[h] @ k[h // fan].T) / q.dtype.type(math.sqrt(d))
        s = np.where(mask, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        out[h] = (rnd(p) @ v[h // fan]) / p.sum(axis=-1, keepdims=True)
    return out


def attention_block(x, w, prefix, c, cos, sin, rnd=_same):
    """q/k/v projections, RoPE on q and k, attention, output projection.

    src/dli/model/llama.py:72-76 (projections, rope), :94-95 (merge heads, o_proj).
    ``rnd``: rounding of every tensor that a bfloat16 model holds in bfloat16 (identity for float32).
    """
    n = x.shape[0]
    d = c["head_dim"]
    q = rnd(x @ w[prefix + "q_proj.weight"].T).reshape(n, c["heads"], d).transpose(1, 0, 2)
    k = rnd(x @ w[prefix + "k_proj.weight"].T).reshape(n, c["kv_heads"], d).transpose(1, 0, 2)
    v = rnd(x @ w[prefix + "v_proj.weight"].T).reshape(n, c["kv_heads"], d).transpose(1, 0, 2)
    q = rnd(apply_rope(q, cos, sin))
    k = rnd(apply_rope(k, cos, sin))
    o = rnd(causal_attention(q, k, v, rnd=rnd))
    merged = o.transpose(1, 0, 2).reshape(n, c["heads"] * d)
    return rnd(merged @ w[prefix + "o_proj.weight"].T)


def silu(z: np.ndarray) -> np.ndarray:
    return z / (1 + np.exp(-z))


def swiglu_mlp(x, w, prefix, rnd=_same):
    """down(silu(gate(x)) * up(x)).  src/dli/model/llama.py:189-191."""
    g = rnd(x @ w[prefix + "gate_proj.weight"].T)
    u = rnd(x @ w[prefix + "up_proj.weight"].T)
    return rnd(rnd(silu(g) * u) @ w[prefix + "down_proj.weight"].T)


def decoder_layer(x, w, i, c, cos, sin, rnd=_same):
    """x + attn(norm(x)), then x + mlp(norm(x)).  src/dli/model/llama.py:211-212."""
    p = f"model.layers.{i}."
    x = x + attention_block(rnd(rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])), w, p + "self_attn.", c, cos, sin, rnd)
    return x + swiglu_mlp(rnd(rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"])), w, p + "mlp.", rnd)


def forward(config: dict, weights: dict[str, np.ndarray], token_ids, dtype=np.float32, rows=None, bf16_activations=False) -> np.ndarray:
    """Logits [n, vocab] of one whole sequence at positions 0..n-1 (with ``rows``: only at those positions,
    [len(rows), vocab]; every position still goes through the layers).

    ``bf16_activations``: a bfloat16 model as the reference runs one (src/dli/model/loader.py:46 casts the
    weights; every module output is then bfloat16): the outputs of the products, of the norms, of rope, of the
    attention (and its probabilities) and of SiLU * up are rounded to bfloat16; the arithmetic between
    roundings, the residual sum and the logits stay float32.  With it off (and weights rounded by the
    caller) only the weights are bfloat16.

    src/dli/model/llama.py:291-305: embed, rope tables, layers, final norm, head
    (tied head uses the embedding matrix, :304).
    """
    c = read_config(config)
    w = {k: v.astype(dtype) for k, v in weights.items()}
    ids = np.asarray(token_ids, dtype=np.int64)
    h = w["model.embed_tokens.weight"][ids]
    cos, sin = rope_cos_sin(inverse_frequencies(c), np.arange(len(ids)))
    cos, sin = cos.astype(dtype), sin.astype(dtype)
    rnd = round_to_bfloat16 if bf16_activations else _same
    for i in range(c["layers"]):
        h = decoder_layer(h, w, i, c, cos, sin, rnd)
    if rows is not None:
        h = h[np.asarray(rows, dtype=np.int64)]
    h = rnd(rms_norm(h, w["model.norm.weight"], c["eps"]))
    head = w["model.embed_tokens.weight"] if c["tied"] else w["lm_head.weight"]
    return (h @ head.T).astype(np.float32)


def greedy_generate(config: dict, weights: dict[str, np.ndarray], prompt, max_new_tokens: int) -> list[int]:
    """Argmax decoding that recomputes the whole sequence each step.

    src/dli/generate.py:21-87 with use_cache=False; ties go to the lowest id (:44-46).
    """
    tokens = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        nxt = int(np.argmax(forward(config, weights, tokens)[-1]))
        out.append(nxt)
        tokens.append(nxt)
    return out


# --------------------------------------------------------------------------- sampling


def _mulhilo32(a: int, b: int) -> tuple[int, int]:
    p = a * b
    return (p >> 32) & 0xFFFFFFFF, p & 0xFFFFFFFF


def philox4x32(counter: tuple[int, int, int, int], key: tuple[int, int], rounds: int = 10):
    """Philox-4x32-10 (Salmon et al. 2011), the counter-based generator the engine's
    sampling kernel uses; restated here from the paper's constants."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(rounds):
        hi0, lo0 = _mulhilo32(0xD2511F53, c0)
        hi1, lo1 = _mulhilo32(0xCD9E8D57, c2)
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & 0xFFFFFFFF, lo1, (hi0 ^ c3 ^ k1) & 0xFFFFFFFF, lo0
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return c0, c1, c2, c3


def uniform_for_draw(seed: int, draw: int) -> float:
    """The uniform number in [0, 1) of a request's ``draw``-th sampled token.

    One draw per sampled token, from the request's own stream, so it does not
    depend on the batch (src/dli/sampling.py:3-7).
    """
    r = philox4x32((draw & 0xFFFFFFFF, (draw >> 32) & 0xFFFFFFFF, 0, 0), (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    return float(np.float32(r[0] >> 8) * np.float32(1.0 / 16777216.0))


def filtered_probabilities(logits: np.ndarray, temperature: float, top_k: int = -1, top_p: float = 1.0) -> np.ndarray:
    """Probabilities after temperature, top-k and top-p, in token order (float64).

    src/dli/sampling.py:92-110: divide by temperature; keep the k largest; softmax;
    drop a token when the mass of the strictly more likely ones reaches top_p; softmax again.
    """
    x = logits.astype(np.float64) / temperature
    order = np.argsort(-x, kind="stable")
    sx = x[order]
    if top_k > 0:
        sx[top_k:] = -np.inf
    p = np.exp(sx - sx.max())
    p /= p.sum()
    preceding = np.cumsum(p) - p
    sx[preceding >= top_p] = -np.inf
    p = np.exp(sx - sx.max())
    p /= p.sum()
    out = np.zeros_like(p)
    out[order] = p
    return out


def sample_token(logits: np.ndarray, temperature: float, top_k: int, top_p: float, seed: int, draw: int) -> int:
    """One token: argmax when greedy (src/dli/sampling.py:57-58, :84), else the first
    token in id order whose cumulative probability exceeds the request's uniform number."""
    if temperature == 0.0 or top_k == 1:
        return int(np.argmax(logits))
    p = filtered_probabilities(logits, temperature, top_k, top_p)
    u = uniform_for_draw(seed, draw)
    cdf = np.cumsum(p)
    idx = int(np.searchsorted(cdf, u * cdf[-1], side="right"))
    kept = np.nonzero(p > 0)[0]
    return int(min(idx, kept[-1]))
