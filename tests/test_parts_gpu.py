"""Each part alone against its plain restatement, and the generality of the assembly: a layer
run twice, a layer that reads another layer's cache, a windowed layer with pages of its own,
other position encodings, and a toy mixer with state of its own that is defined here and
registered, built and stepped without touching the package's files."""

import dataclasses
import math

import numpy as np
import pytest
import torch

from dli_b200.cache import StateNeed
from dli_b200.config import Architecture, LlamaConfig, llama_model_spec, register_architecture, unregister_architecture
from dli_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunStep
from dli_b200.engine import ModelRunner, StepEntry, random_model
from dli_b200.kernels import ops
from dli_b200.parts import BuildEnv, DecoderModel, Part, build_part, register_part, unregister_part
from dli_b200.parts.base import ResidualStream
from dli_b200.weights import TensorDecl, random_tensors
from tests.plain import llama_plain as plain
from tests.tiny_configs import TINY_A, TINY_B, TINY_C

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 1e-4, torch.bfloat16: 5e-2}


def env(dtype):
    return BuildEnv(dtype, DEV)


def np32(t):
    return t.float().cpu().numpy()


def weights_as_plain(model_tensors, dtype):
    """The tensors the model was loaded with, as the float32 arrays the plain code takes."""
    return {k: np32(v) for k, v in model_tensors.items()}


def build(spec, dtype, seed, sharpen=6.0):
    model = DecoderModel(spec, dtype, DEV)
    tensors = random_tensors(model.declared_tensors(), seed, dtype=dtype, device=DEV)
    for k in tensors:
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            tensors[k] = (tensors[k].float() * sharpen).to(dtype)
    model.load(tensors)
    return model, weights_as_plain(tensors, dtype)


# ------------------------------------------------------------------ parts alone


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    torch.manual_seed(11)  # the inputs below come from the global generator: the same ones in every order of tests
    part = build_part("norm", PartSpec("rmsnorm", {"size": 72, "eps": 2e-5}, "n."), env(dtype))
    assert part.declare() == {"n.weight": TensorDecl((72,), "vector32")}
    w = torch.rand(72, device=DEV) + 0.5
    part.load({"n.weight": w})
    h = torch.randn(5, 72, device=DEV)
    d = torch.randn(5, 72, device=DEV).to(dtype)
    want = plain.rms_norm(np32(h) + np32(d), np32(w), 2e-5)
    y = part.add_norm(h, d)
    np.testing.assert_allclose(np32(y), want, atol=TOL[dtype])


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C], ids=["default", "llama3", "linear48"])
def test_rotary_part_frequencies(cfg):
    spec = llama_model_spec(LlamaConfig.from_hf_dict(cfg))
    pos = build_part("position", spec.layers[0].parts["mixer"].params["position"], env(torch.float32))
    want = plain.inverse_frequencies(plain.read_config(cfg))
    np.testing.assert_allclose(np32(pos.inv_freq), want, rtol=2e-7, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    torch.manual_seed(12)
    part = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": 40, "intermediate_size": 72}, "m."), env(dtype))
    t = random_tensors(part.declare(), 3, dtype=dtype, device=DEV)
    t = {k: (v.float() * 10).to(dtype) for k, v in t.items()}
    part.load(t)
    x = torch.randn(9, 40, device=DEV).to(dtype)
    want = plain.swiglu_mlp(np32(x), weights_as_plain(t, dtype), "m.")
    np.testing.assert_allclose(np32(part.forward(x)), want, atol=TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tied", [True, False])
def test_embedding_and_head_parts(dtype, tied):
    torch.manual_seed(13)
    e = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 130, "hidden_size": 24}, "emb."), env(dtype))
    hd = build_part("head", PartSpec("lm_head", {"vocab_size": 130, "hidden_size": 24, "tied_to": "emb.weight" if tied else None}, "head."), env(dtype))
    decl = {**e.declare(), **hd.declare()}
    assert decl["head.weight"].optional_alias_of == ("emb.weight" if tied else None)
    t = random_tensors(decl, 1, dtype=dtype, device=DEV)
    assert ("head.weight" in t) == (not tied)
    e.load(t), hd.load(t)
    ids = torch.tensor([3, 129, 0], dtype=torch.int32, device=DEV)
    h = e.forward(ids)
    assert h.dtype == torch.float32 and torch.equal(h, t["emb.weight"].float()[ids.long()])
    y = torch.randn(4, 24, device=DEV).to(dtype)
    logits = hd.forward(y)
    assert logits.dtype == torch.float32
    wname = "emb.weight" if tied else "head.weight"
    np.testing.assert_allclose(np32(logits), np32(y) @ np32(t[wname]).T, atol=TOL[dtype])


def one_layer_model(cfg_json, dtype, seed=5, **mixer_overrides):
    cfg = LlamaConfig.from_hf_dict({**cfg_json, "num_hidden_layers": 1})
    spec = llama_model_spec(cfg)
    if mixer_overrides:
        layer = spec.layers[0]
        mixer = layer.parts["mixer"]
        mixer = dataclasses.replace(mixer, params={**mixer.params, **mixer_overrides})
        spec = dataclasses.replace(spec, layers=(LayerSpec(layer.arrangement, {**layer.parts, "mixer": mixer}),))
    return spec, *build(spec, dtype, seed)


def run_whole_and_cut(model, tokens, page, cuts):
    """Logits of one request run whole, and run in the given portions; [n, vocab] each.  Both want every
    position, so their steps are launched kernel by kernel.  Where the model's parts can be recorded, the
    portions run a third time wanting only each portion's last position: those steps replay graphs captured at
    their first coming (engine.graphs.MixedGraph: padded shapes, an empty sequence for the rows nobody fills),
    and their logits must be the whole run's at those positions."""
    out = []
    for portions in ([len(tokens)], cuts):
        r = ModelRunner(model, num_pages=64, page_size=page, max_requests=4, enable_prefix_caching=False, watermark=0.0)
        alloc = r.manager.allocate("x", tokens)
        r.start_request("x", alloc.state_slot)
        pos, parts = 0, []
        for n in portions:
            parts.append(r.step([StepEntry("x", tokens[pos : pos + n], range(n))]))
            pos += n
        assert pos == len(tokens)
        out.append(np32(torch.cat(parts)))
        r.manager.free("x")
        r.manager.check_invariants()
    r = ModelRunner(model, num_pages=64, page_size=page, max_requests=4, enable_prefix_caching=False, watermark=0.0)
    if r.graphs is not None and DEV.type == "cuda":
        r.graphs.mixed_after = 1
        r.manager.allocate("x", tokens)
        pos = 0
        for n in cuts:
            got = np32(r.step([StepEntry("x", tokens[pos : pos + n], [n - 1])]))[0]
            pos += n
            np.testing.assert_allclose(got, out[0][pos - 1], atol=TOL[model.dtype], err_msg=f"from a graph: position {pos - 1}")
        assert r.mixed_graph_steps == sum(n > 1 for n in cuts), r.graphs.mixed_failure
        r.manager.free("x")
        r.manager.check_invariants()
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C], ids=["a", "b", "c"])
def test_block_of_parts_equals_plain_layer(dtype, cfg):
    """mixer (attention with rotary), norms, feed-forward and their arrangement, as one layer."""
    spec, model, w = one_layer_model(cfg, dtype)
    tokens = np.random.default_rng(1).integers(0, cfg["vocab_size"], 50).tolist()
    want = plain.forward({**cfg, "num_hidden_layers": 1}, w, tokens)
    whole, cut = run_whole_and_cut(model, tokens, 8, [13, 2, 1, 30, 4])
    np.testing.assert_allclose(whole, want, atol=TOL[dtype])
    np.testing.assert_allclose(cut, want, atol=TOL[dtype])


def plain_layer(x, w, i, c, cos, sin, window=None, kv_from=None, rot=None):
    """plain.decoder_layer with a window, with keys/values taken from another layer's
    projections of that layer's own input (``kv_from`` = (layer index, its normed input)),
    and with rotation of the first ``rot`` elements only."""
    p = f"model.layers.{i}."
    n, d = x.shape[0], c["head_dim"]
    y = plain.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
    q = (y @ w[p + "self_attn.q_proj.weight"].T).reshape(n, c["heads"], d).transpose(1, 0, 2)
    src, ysrc = (i, y) if kv_from is None else kv_from
    ps = f"model.layers.{src}.self_attn."
    k = (ysrc @ w[ps + "k_proj.weight"].T).reshape(n, c["kv_heads"], d).transpose(1, 0, 2)
    v = (ysrc @ w[ps + "v_proj.weight"].T).reshape(n, c["kv_heads"], d).transpose(1, 0, 2)
    rot = d if rot is None else rot
    if rot:
        rope = lambda t: np.concatenate([plain.apply_rope(t[..., :rot], cos, sin), t[..., rot:]], axis=-1)
        q, k = rope(q), rope(k)
    o = plain.causal_attention(q, k, v, window).transpose(1, 0, 2).reshape(n, c["heads"] * d)
    x = x + o @ w[p + "self_attn.o_proj.weight"].T
    return x + plain.swiglu_mlp(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"]), w, p + "mlp."), y


def plain_variant(cfg, w, tokens, run_order, windows=None, rot=None):
    c = plain.read_config(cfg)
    x = w["model.embed_tokens.weight"][np.asarray(tokens)]
    rc = dict(c, head_dim=rot) if rot else c
    cos = sin = None
    if rot is None or rot:
        cos, sin = plain.rope_cos_sin(plain.inverse_frequencies(rc), np.arange(len(tokens)))
    normed = {}
    for j, step in enumerate(run_order):
        kv_from = None if step.cache_of is None else (run_order[step.cache_of].layer, normed[step.cache_of])
        x, normed[j] = plain_layer(x, w, step.layer, c, cos, sin, (windows or {}).get(step.layer), kv_from, rot)
    x = plain.rms_norm(x, w["model.norm.weight"], c["eps"])
    head = w["model.embed_tokens.weight"] if c["tied"] else w["lm_head.weight"]
    return x @ head.T


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rotary_dim", [0, 16])
def test_other_position_encodings(dtype, rotary_dim):
    """No position encoding at all, and rotation of a part of each head."""
    base = llama_model_spec(LlamaConfig.from_hf_dict({**TINY_B, "num_hidden_layers": 1}))
    pos = base.layers[0].parts["mixer"].params["position"]
    new_pos = PartSpec("none", {"head_dim": 32}) if rotary_dim == 0 else dataclasses.replace(pos, params={**pos.params, "rotary_dim": rotary_dim})
    spec, model, w = one_layer_model(TINY_B, dtype, position=new_pos)
    tokens = np.random.default_rng(2).integers(0, 1000, 45).tolist()
    want = plain_variant({**TINY_B, "num_hidden_layers": 1}, w, tokens, [RunStep(0)], rot=rotary_dim)
    whole, cut = run_whole_and_cut(model, tokens, 16, [20, 1, 1, 23])
    np.testing.assert_allclose(whole, want, atol=TOL[dtype])
    np.testing.assert_allclose(cut, want, atol=TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
def test_run_order_names_a_layer_twice_and_shares_a_cache(dtype):
    """Order 0, 1, 0, then layer 1 again reading the cache its first run wrote: four run steps,
    two layers' weights, three caches."""
    base = llama_model_spec(LlamaConfig.from_hf_dict(TINY_A))
    order = (RunStep(0), RunStep(1), RunStep(0), RunStep(1, cache_of=1))
    spec = dataclasses.replace(base, run_order=order)
    model, w = build(spec, dtype, seed=8)
    assert [n is not None for n in model.cache_needs()] == [True, True, True, False]
    tokens = np.random.default_rng(3).integers(0, 256, 41).tolist()
    want = plain_variant(TINY_A, w, tokens, order)
    whole, cut = run_whole_and_cut(model, tokens, 4, [7, 30, 1, 1, 2])
    np.testing.assert_allclose(whole, want, atol=TOL[dtype])
    np.testing.assert_allclose(cut, want, atol=TOL[dtype])
    r = ModelRunner(model, num_pages=8, page_size=4)
    assert r.pools.k[0].shape[0] == 3  # one group, three owned caches
    assert r.pools.layer_caches[3].k.data_ptr() == r.pools.layer_caches[1].k.data_ptr() and not r.pools.layer_caches[3].writes


@pytest.mark.parametrize("dtype", DTYPES)
def test_windowed_layer_has_pages_of_its_own_and_gives_them_back(dtype):
    """Layer 1 sees a window of 9 keys: two cache groups, and the windowed group's pages go
    back to its pool while the request is still running."""
    base = llama_model_spec(LlamaConfig.from_hf_dict(TINY_C | {"num_hidden_layers": 2}))
    layers = list(base.layers)
    mixer = layers[1].parts["mixer"]
    layers[1] = LayerSpec("prenorm", {**layers[1].parts, "mixer": dataclasses.replace(mixer, params={**mixer.params, "window": 9})})
    spec = dataclasses.replace(base, layers=tuple(layers))
    model, w = build(spec, dtype, seed=9)
    tokens = np.random.default_rng(4).integers(0, 517, 60).tolist()
    want = plain_variant(TINY_C | {"num_hidden_layers": 2}, w, tokens, spec.run_order, windows={1: 9})
    r = ModelRunner(model, num_pages=[16, 16], page_size=4, max_requests=2, watermark=0.0)
    assert len(r.pools.k) == 2 and not r.manager.prefix_caching
    r.manager.allocate("x", tokens[:30])
    parts = [r.step([StepEntry("x", tokens[:30], range(30))])]
    assert r.manager.block_table("x", 1)[:5] == [-1] * 5 and r.manager.pools[1].available == 16 - 8 + 5
    for t in tokens[30:]:
        r.manager.append_slots("x", [t])
        parts.append(r.step([StepEntry("x", [t], [0])]))
        r.manager.check_invariants()
    assert r.manager.pools[1].available >= 16 - 4 and r.manager.pools[0].available == 1
    np.testing.assert_allclose(np32(torch.cat(parts)), want, atol=TOL[dtype])


# ------------------------------------------------------------------ a toy mixer with state


class RunningMean(Part):
    """out_t = W mean(x_0 .. x_t): per-request state (the sum so far and the count) in a slot."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = spec.params["hidden_size"]
        self.w = None

    def declare(self):
        return {self.spec.prefix + "mix.weight": TensorDecl((self.hidden, self.hidden))}

    def load(self, tensors):
        self.w = tensors[self.spec.prefix + "mix.weight"]

    def cache_need(self):
        return StateNeed((self.hidden + 1,), torch.float32)

    def forward(self, x, batch, cache):
        out = torch.empty_like(x)
        a = 0
        for q_len, slot in zip(batch.q_lens, batch.state_slots):
            state = cache.state[slot]
            sums = state[: self.hidden] + torch.cumsum(x[a : a + q_len].float(), 0)
            counts = state[self.hidden] + torch.arange(1, q_len + 1, device=x.device)
            out[a : a + q_len] = ((sums / counts[:, None]).to(x.dtype) @ self.w.t())
            state[: self.hidden] = sums[-1]
            state[self.hidden] = counts[-1]
            a += q_len
        return out


def toy_spec(cfg):
    """The llama layers, with the mixer of every odd layer replaced by the toy one."""
    base = llama_model_spec(LlamaConfig.from_hf_dict(cfg))
    layers = []
    for i, layer in enumerate(base.layers):
        if i % 2:
            toy = PartSpec("toy_running_mean", {"hidden_size": base.hidden_size}, f"model.layers.{i}.toy.")
            layer = LayerSpec("prenorm", {**layer.parts, "mixer": toy})
        layers.append(layer)
    return dataclasses.replace(base, layers=tuple(layers))


def plain_toy_forward(cfg, w, tokens):
    c = plain.read_config(cfg)
    x = w["model.embed_tokens.weight"][np.asarray(tokens)]
    cos, sin = plain.rope_cos_sin(plain.inverse_frequencies(c), np.arange(len(tokens)))
    for i in range(c["layers"]):
        if i % 2 == 0:
            x, _ = plain_layer(x, w, i, c, cos, sin)
            continue
        p = f"model.layers.{i}."
        y = plain.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
        mean = np.cumsum(y, axis=0) / np.arange(1, len(tokens) + 1)[:, None]
        x = x + mean @ w[p + "toy.mix.weight"].T
        x = x + plain.swiglu_mlp(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"]), w, p + "mlp.")
    x = plain.rms_norm(x, w["model.norm.weight"], c["eps"])
    return x @ w["lm_head.weight"].T


@pytest.fixture
def toy_architecture():
    register_part("mixer", "toy_running_mean")(RunningMean)
    register_architecture(Architecture("ToyStateLM", LlamaConfig.from_hf_dict, lambda cfg: toy_spec(cfg.to_hf_dict())))
    yield {**TINY_B, "architectures": ["ToyStateLM"]}
    unregister_architecture("ToyStateLM")
    unregister_part("mixer", "toy_running_mean")


def test_toy_mixer_with_state_is_registered_built_and_stepped(toy_architecture):
    cfg = toy_architecture
    model = random_model(cfg, seed=4, dtype="float32")
    assert [type(n).__name__ for n in model.cache_needs()] == ["PagedKVNeed", "StateNeed", "PagedKVNeed"]
    w = {}
    for part in model.parts():
        for name in part.declare():
            pass
    # the plain code needs the tensors by name: take them from the parts that hold them
    tensors = random_tensors(model.declared_tensors(), 4, dtype=torch.float32, device=DEV)
    w = weights_as_plain(tensors, torch.float32)
    reqs = {rid: np.random.default_rng(k).integers(0, 1000, n).tolist() for k, (rid, n) in enumerate([("p", 50), ("q", 33), ("r", 47)])}
    want = {rid: plain_toy_forward(cfg, w, t) for rid, t in reqs.items()}
    r = ModelRunner(model, num_pages=8, page_size=16, max_requests=2, watermark=0.0)  # 2 slots, 3 requests: a slot is used again
    assert not r.manager.prefix_caching  # pages alone would not restore a request's state
    got = {rid: [] for rid in reqs}

    def feed(entries):
        batch = []
        for rid, lo, hi in entries:
            toks = reqs[rid][lo:hi]
            if r.manager.has_request(rid):
                r.manager.append_slots(rid, toks)
            else:
                r.start_request(rid, r.manager.allocate(rid, toks).state_slot)
            batch.append(StepEntry(rid, toks, range(hi - lo)))
        out = r.step(batch)
        row = 0
        for rid, lo, hi in entries:
            got[rid].append(out[row : row + hi - lo])
            row += hi - lo

    feed([("p", 0, 20)])
    feed([("p", 20, 21), ("q", 0, 30)])  # a decoded token of one beside a portion of another
    feed([("q", 30, 33), ("p", 21, 50)])
    r.manager.free("p")
    feed([("r", 0, 2)])  # takes over the slot p left; its state must start from nothing
    feed([("r", 2, 47)])
    r.manager.free("q"), r.manager.free("r")
    r.manager.check_invariants()
    for rid in reqs:
        np.testing.assert_allclose(np32(torch.cat(got[rid])), want[rid], atol=1e-4, err_msg=rid)


# ------------------------------------------------------------------ a toy layer that keeps pages AND a state slot


class HybridBlock(Part):
    """x = x + attention(norm(x)) + running_mean(norm(x)); x = x + ffn(norm(x)): two mixers side by side in one
    layer, one with keys and values in pages, one with state of fixed size.  The arrangement declares both
    needs; both mixers get the run step's one LayerCache.  Defined here only."""

    def __init__(self, spec, env):
        self.spec, self.env = spec, env
        self.mixer_norm = build_part("norm", spec.parts["mixer_norm"], env)
        self.attention = build_part("mixer", spec.parts["mixer"], env)
        self.mean = build_part("mixer", spec.parts["second_mixer"], env)
        self.ffn_norm = build_part("norm", spec.parts["ffn_norm"], env)
        self.ffn = build_part("feed_forward", spec.parts["ffn"], env)

    def children(self):
        return [self.mixer_norm, self.attention, self.mean, self.ffn_norm, self.ffn]

    def cache_need(self):
        return (self.attention.cache_need(), self.mean.cache_need())

    def forward(self, stream, batch, cache):
        y = self.mixer_norm.add_norm(stream.h, stream.pending)
        delta = self.attention.forward(y, batch, cache) + self.mean.forward(y, batch, cache)
        y = self.ffn_norm.add_norm(stream.h, delta)
        stream.pending = self.ffn.forward(y)


def test_a_layer_may_keep_pages_and_a_state_slot():
    """Layer 1 of tiny-B becomes the hybrid arrangement: the cache manager gives its run step pages and a slot,
    requests are cut into portions beside one another, a slot is used again, and the logits are those of a
    numpy restatement."""
    register_part("mixer", "toy_running_mean")(RunningMean)
    register_part("arrangement", "toy_hybrid")(HybridBlock)
    try:
        base = llama_model_spec(LlamaConfig.from_hf_dict(TINY_B))
        layers = list(base.layers)
        mean = PartSpec("toy_running_mean", {"hidden_size": base.hidden_size}, "model.layers.1.toy.")
        layers[1] = LayerSpec("toy_hybrid", {**layers[1].parts, "second_mixer": mean})
        spec = dataclasses.replace(base, layers=tuple(layers))
        model, w = build(spec, torch.float32, seed=21)
        needs = model.cache_needs()
        assert [type(n).__name__ for n in needs] == ["PagedKVNeed", "tuple", "PagedKVNeed"]
        assert [type(n).__name__ for n in needs[1]] == ["PagedKVNeed", "StateNeed"]

        def want_for(tokens):
            c = plain.read_config(TINY_B)
            x = w["model.embed_tokens.weight"][np.asarray(tokens)]
            cos, sin = plain.rope_cos_sin(plain.inverse_frequencies(c), np.arange(len(tokens)))
            for i in range(c["layers"]):
                if i != 1:
                    x, _ = plain_layer(x, w, i, c, cos, sin)
                    continue
                p = "model.layers.1."
                y = plain.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
                mean_y = np.cumsum(y, axis=0) / np.arange(1, len(tokens) + 1)[:, None]
                x = x + plain.attention_block(y, w, p + "self_attn.", c, cos, sin) + mean_y @ w[p + "toy.mix.weight"].T
                x = x + plain.swiglu_mlp(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"]), w, p + "mlp.")
            return plain.rms_norm(x, w["model.norm.weight"], c["eps"]) @ w["lm_head.weight"].T

        reqs = {rid: np.random.default_rng(30 + k).integers(0, 1000, n).tolist() for k, (rid, n) in enumerate([("p", 41), ("q", 30), ("r", 37)])}
        r = ModelRunner(model, num_pages=8, page_size=16, max_requests=2, watermark=0.0)
        assert r.pools.layer_caches[1].k is not None and len(r.pools.layer_caches[1].states) == 1 and r.graphs is None
        assert not r.manager.prefix_caching  # pages alone would not bring a request's state back
        got = {rid: [] for rid in reqs}

        def feed(entries):
            batch = []
            for rid, lo, hi in entries:
                toks = reqs[rid][lo:hi]
                if r.manager.has_request(rid):
                    r.manager.append_slots(rid, toks)
                else:
                    r.start_request(rid, r.manager.allocate(rid, toks).state_slot)
                batch.append(StepEntry(rid, toks, range(hi - lo)))
            out = r.step(batch)
            row = 0
            for rid, lo, hi in entries:
                got[rid].append(out[row : row + hi - lo])
                row += hi - lo

        feed([("p", 0, 18)])
        feed([("p", 18, 19), ("q", 0, 28)])
        feed([("q", 28, 30), ("p", 19, 41)])
        r.manager.free("p")
        feed([("r", 0, 3)])  # p's slot and pages, used again
        feed([("r", 3, 37)])
        r.manager.free("q"), r.manager.free("r")
        r.manager.check_invariants()
        for rid, tokens in reqs.items():
            np.testing.assert_allclose(np32(torch.cat(got[rid])), want_for(tokens), atol=1e-4, err_msg=rid)
    finally:
        unregister_part("arrangement", "toy_hybrid")
        unregister_part("mixer", "toy_running_mean")


# ------------------------------------------------------------------ a toy mixer whose launches depend on the step's shape


class ChunkedLinearMixer(Part):
    """out = x W^T, computed in one product or in two halves of the width added up, as it sees fit from the number
    of sequences: a stand-in for a mixer with a launch policy of its own.  It tells the step function what its
    policy depends on (``decode_launch_key``) and is handed its answer back for steps replayed from a graph."""

    graph_capturable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = spec.params["hidden_size"]
        self.w = None
        self.keys_seen = []  # what forward was handed, call by call (graph captures included)

    def declare(self):
        return {self.spec.prefix + "mix.weight": TensorDecl((self.hidden, self.hidden))}

    def load(self, tensors):
        self.w = tensors[self.spec.prefix + "mix.weight"]

    def cache_need(self):
        return None

    def decode_launch_key(self, num_seqs, max_kv_len, page_size):
        return ("halves", 2 if num_seqs <= 2 else 1)

    def forward(self, x, batch, cache):
        key = batch.launch_keys.get(id(self))
        self.keys_seen.append(key)
        halves = key[1] if key is not None else 1
        if halves == 1:
            return x @ self.w.t()
        mid = self.hidden // 2
        return x[:, :mid] @ self.w[:, :mid].t() + x[:, mid:] @ self.w[:, mid:].t()


def test_a_toy_mixer_with_its_own_launch_key_decodes_through_graphs():
    """The graph layer knows nothing of the toy: it asks every part, keys its graphs by the answers and hands each
    part its own answer back.  One and two sequences decode through a graph recorded with two halves, four
    sequences through one recorded with one product; the logits are right either way."""
    register_part("mixer", "toy_chunked_linear")(ChunkedLinearMixer)
    try:
        base = llama_model_spec(LlamaConfig.from_hf_dict(TINY_B))
        layers = list(base.layers)
        toy = PartSpec("toy_chunked_linear", {"hidden_size": base.hidden_size}, "model.layers.1.toy.")
        layers[1] = LayerSpec("prenorm", {**layers[1].parts, "mixer": toy})
        spec = dataclasses.replace(base, layers=tuple(layers))
        model, w = build(spec, torch.float32, seed=22)
        mixer = model.layers[1].mixer

        def want_for(tokens):
            c = plain.read_config(TINY_B)
            x = w["model.embed_tokens.weight"][np.asarray(tokens)]
            cos, sin = plain.rope_cos_sin(plain.inverse_frequencies(c), np.arange(len(tokens)))
            for i in range(c["layers"]):
                if i != 1:
                    x, _ = plain_layer(x, w, i, c, cos, sin)
                    continue
                p = "model.layers.1."
                x = x + plain.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"]) @ w[p + "toy.mix.weight"].T
                x = x + plain.swiglu_mlp(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"]), w, p + "mlp.")
            return plain.rms_norm(x, w["model.norm.weight"], c["eps"]) @ w["lm_head.weight"].T

        reqs = {f"s{i}": np.random.default_rng(50 + i).integers(0, 1000, 20 + 3 * i).tolist() for i in range(4)}
        want = {rid: want_for(t) for rid, t in reqs.items()}
        r = ModelRunner(model, num_pages=16, page_size=16, max_requests=4, watermark=0.0, enable_prefix_caching=False)
        assert r.graphs is not None
        for rid, toks in reqs.items():
            r.manager.allocate(rid, toks[:-6])
            r.step([StepEntry(rid, toks[:-6], [])])

        at = {rid: len(toks) - 6 for rid, toks in reqs.items()}  # each request's next position

        def decode(ids):
            for rid in ids:
                r.manager.append_slots(rid, [reqs[rid][at[rid]]])
            out = np32(r.step([StepEntry(rid, [reqs[rid][at[rid]]], [0]) for rid in ids]))
            for j, rid in enumerate(ids):
                np.testing.assert_allclose(out[j], want[rid][at[rid]], atol=1e-4, err_msg=f"{rid} at {at[rid]}")
                at[rid] += 1

        if DEV.type != "cuda":  # (on the stand-ins there is nothing to record; the toy still runs step by step)
            decode(list(reqs))
            return
        decode(["s0"])
        decode(["s0", "s1"])
        assert r.graph_steps == 2 and ("halves", 2) in mixer.keys_seen
        decode(list(reqs))
        assert r.graph_steps == 3 and ("halves", 1) in mixer.keys_seen
        assert any(("halves", 2) in key[2] for key in r.graphs.graphs) and any(("halves", 1) in key[2] for key in r.graphs.graphs), sorted(r.graphs.graphs)
        calls = len(mixer.keys_seen)
        decode(list(reqs))  # replayed: the toy's Python does not run again
        assert r.graph_steps == 4 and len(mixer.keys_seen) == calls
    finally:
        unregister_part("mixer", "toy_chunked_linear")


def test_unknown_part_kind_is_named():
    with pytest.raises(ValueError, match="no mixer part of kind 'nonesuch'"):
        build_part("mixer", PartSpec("nonesuch"), env(torch.float32))


# ------------------------------------------------------------------ a toy feed-forward with routing


class RoutedFFN(Part):
    """Three small SwiGLU experts, top-1 routing by float32 router logits; defined here only."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.inter, self.experts = spec.params["hidden_size"], spec.params["intermediate_size"], spec.params["experts"]

    def declare(self):
        px = self.spec.prefix
        out = {px + "router.weight": TensorDecl((self.experts, self.hidden))}
        for e in range(self.experts):
            out[px + f"experts.{e}.gate_up.weight"] = TensorDecl((2 * self.inter, self.hidden))
            out[px + f"experts.{e}.down.weight"] = TensorDecl((self.hidden, self.inter))
        return out

    def load(self, tensors):
        px = self.spec.prefix
        self.router = tensors[px + "router.weight"]
        self.gate_up = [tensors[px + f"experts.{e}.gate_up.weight"] for e in range(self.experts)]
        self.down = [tensors[px + f"experts.{e}.down.weight"] for e in range(self.experts)]

    def forward(self, x):
        choice = (x.float() @ self.router.float().t()).argmax(-1)  # router logits in float32
        out = torch.zeros_like(x)
        for e in range(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                gu = x[rows] @ self.gate_up[e].t()
                act = torch.nn.functional.silu(gu[:, : self.inter].float()) * gu[:, self.inter :].float()
                out[rows] = (act.to(x.dtype) @ self.down[e].t())
        return out


def test_toy_routed_feed_forward_is_registered_and_stepped():
    """One model, different feed-forwards in different layers: layer 0 keeps SwiGLU, layer 1
    routes among experts.  Float32, cut into portions, against a numpy restatement."""
    register_part("feed_forward", "toy_routed")(RoutedFFN)
    try:
        base = llama_model_spec(LlamaConfig.from_hf_dict(TINY_A))
        layers = list(base.layers)
        routed = PartSpec("toy_routed", {"hidden_size": 64, "intermediate_size": 24, "experts": 3}, "model.layers.1.moe.")
        layers[1] = LayerSpec("prenorm", {**layers[1].parts, "ffn": routed})
        spec = dataclasses.replace(base, layers=tuple(layers))
        model, w = build(spec, torch.float32, seed=12)
        for k in list(w):  # make routing decisive: no near ties between experts
            if k.endswith("router.weight"):
                w[k] = w[k] * 50
        model.load({k: torch.from_numpy(v).to(DEV) for k, v in w.items()})
        tokens = np.random.default_rng(6).integers(0, 256, 40).tolist()

        c = plain.read_config(TINY_A)
        x = w["model.embed_tokens.weight"][np.asarray(tokens)]
        cos, sin = plain.rope_cos_sin(plain.inverse_frequencies(c), np.arange(len(tokens)))
        x, _ = plain_layer(x, w, 0, c, cos, sin)
        p = "model.layers.1."
        y = plain.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
        n, d = len(tokens), c["head_dim"]
        q = (y @ w[p + "self_attn.q_proj.weight"].T).reshape(n, c["heads"], d).transpose(1, 0, 2)
        k = (y @ w[p + "self_attn.k_proj.weight"].T).reshape(n, c["kv_heads"], d).transpose(1, 0, 2)
        v = (y @ w[p + "self_attn.v_proj.weight"].T).reshape(n, c["kv_heads"], d).transpose(1, 0, 2)
        o = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v).transpose(1, 0, 2).reshape(n, -1)
        x = x + o @ w[p + "self_attn.o_proj.weight"].T
        y = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
        choice = (y @ w[p + "moe.router.weight"].T).argmax(-1)
        delta = np.zeros_like(y)
        for t, e in enumerate(choice):
            gu = y[t] @ w[p + f"moe.experts.{e}.gate_up.weight"].T
            delta[t] = (plain.silu(gu[:24]) * gu[24:]) @ w[p + f"moe.experts.{e}.down.weight"].T
        x = plain.rms_norm(x + delta, w["model.norm.weight"], c["eps"])
        want = x @ w["model.embed_tokens.weight"].T
        assert len(set(choice.tolist())) > 1, "the router sent every token to one expert"

        whole, cut = run_whole_and_cut(model, tokens, 4, [9, 1, 1, 27, 2])
        np.testing.assert_allclose(whole, want, atol=1e-4)
        np.testing.assert_allclose(cut, want, atol=1e-4)
    finally:
        unregister_part("feed_forward", "toy_routed")


# ------------------------------------------------------------------ a toy position encoding with a table of its own


class LearnedOffsets(Part):
    """Adds a learned row offsets[position] to every q and k head before the scores are taken
    (absolute positions, no rotation); defined here only.  It has a tensor of its own, and it
    offers ``rotate_and_store`` alone, so the mixer makes the q | k | v product itself."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim, self.max_positions = int(spec.params["head_dim"]), int(spec.params["max_positions"])

    def declare(self):
        return {self.spec.prefix + "offsets.weight": TensorDecl((self.max_positions, self.head_dim))}

    def load(self, tensors):
        self.offsets = tensors[self.spec.prefix + "offsets.weight"]

    def rotate_and_store(self, qkv, batch, cache, num_heads, num_kv_heads, write_kv):
        n, d = qkv.shape[0], self.head_dim
        rows = self.offsets[batch.positions.long()].float()  # [n, d]
        heads = qkv[:, : (num_heads + num_kv_heads) * d].view(n, num_heads + num_kv_heads, d)
        heads.copy_((heads.float() + rows[:, None, :]).to(qkv.dtype))
        slots = batch.group(cache.group).slots
        ops.rotary_store(qkv, batch.positions, None, slots if write_kv else None, cache.k if write_kv else None,
                         cache.v if write_kv else None, num_heads, num_kv_heads, d, 0, cache.page_size, write_kv)
        return qkv


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_position_encoding_with_a_table_is_registered_and_stepped(dtype):
    """Layer 0 keeps its rotary encoding, layer 1 takes the toy one: its table is declared, loaded by
    name and indexed by the positions of the step, whole and in portions down to single tokens."""
    register_part("position", "toy_learned_offsets")(LearnedOffsets)
    try:
        base = llama_model_spec(LlamaConfig.from_hf_dict(TINY_A))
        c = plain.read_config(TINY_A)
        layers = list(base.layers)
        mixer = layers[1].parts["mixer"]
        toy = PartSpec("toy_learned_offsets", {"head_dim": c["head_dim"], "max_positions": 64}, "model.layers.1.self_attn.position.")
        layers[1] = LayerSpec(layers[1].arrangement, {**layers[1].parts, "mixer": dataclasses.replace(mixer, params={**mixer.params, "position": toy})})
        spec = dataclasses.replace(base, layers=tuple(layers))
        model = DecoderModel(spec, dtype, DEV)
        tensors = random_tensors(model.declared_tensors(), 21, dtype=dtype, device=DEV)
        table = "model.layers.1.self_attn.position.offsets.weight"
        tensors[table] = tensors[table] * 32  # a power of two, exact in bfloat16 too: the offsets move the scores visibly
        model.load(tensors)
        w = weights_as_plain(tensors, dtype)
        tokens = np.random.default_rng(9).integers(0, 256, 43).tolist()

        x = w["model.embed_tokens.weight"][np.asarray(tokens)]
        cos, sin = plain.rope_cos_sin(plain.inverse_frequencies(c), np.arange(len(tokens)))
        x, _ = plain_layer(x, w, 0, c, cos, sin)
        p = "model.layers.1."
        n, d = len(tokens), c["head_dim"]
        y = plain.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
        rows = w[p + "self_attn.position.offsets.weight"][:n]
        q = (y @ w[p + "self_attn.q_proj.weight"].T).reshape(n, c["heads"], d) + rows[:, None, :]
        k = (y @ w[p + "self_attn.k_proj.weight"].T).reshape(n, c["kv_heads"], d) + rows[:, None, :]
        v = (y @ w[p + "self_attn.v_proj.weight"].T).reshape(n, c["kv_heads"], d)
        o = plain.causal_attention(q.transpose(1, 0, 2), k.transpose(1, 0, 2), v.transpose(1, 0, 2)).transpose(1, 0, 2).reshape(n, -1)
        x = x + o @ w[p + "self_attn.o_proj.weight"].T
        x = x + plain.swiglu_mlp(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"]), w, p + "mlp.")
        want = plain.rms_norm(x, w["model.norm.weight"], c["eps"]) @ w["model.embed_tokens.weight"].T

        # the table matters: it moves the scores by far more than the tolerance
        with_rows = np.einsum("nhd,mhd->hnm", q, k[:, : 1].repeat(c["heads"], 1))
        without = np.einsum("nhd,mhd->hnm", q - rows[:, None, :], (k - rows[:, None, :])[:, : 1].repeat(c["heads"], 1))
        assert np.abs(with_rows - without).max() > 1.0, "the offsets are too small to show a fault"

        whole, cut = run_whole_and_cut(model, tokens, 4, [9, 1, 1, 2, 28, 1, 1])
        np.testing.assert_allclose(whole, want, atol=TOL[dtype])
        np.testing.assert_allclose(cut, want, atol=TOL[dtype])
    finally:
        unregister_part("position", "toy_learned_offsets")
