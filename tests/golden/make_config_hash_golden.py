"""Makes tests/golden/config_and_hash.json from the reference's own configuration parser and page hashing.

Run once, on the CPU, with the reference's sources importable:

    PYTHONPATH=<reference checkout>/src python tests/golden/make_config_hash_golden.py

For a list of config.json dictionaries (complete, with keys left out so that defaults apply, with both
spellings of the rope keys, and with values the reference refuses) it stores what
``dli.model.config.ModelConfig.from_hf_dict`` makes of each: the parsed fields, or the kind of error.  For a few
(namespace, tokens, page size) it stores the chain of page hashes of ``dli.kv.hashing.chain_hashes``.
tests/test_config.py and tests/test_cache_manager.py compare this repository's parser and hashing with them.
"""

import copy
import dataclasses
import json
import random
from pathlib import Path

from dli.kv.hashing import chain_hashes  # the reference
from dli.model.config import ModelConfig, UnsupportedModelError  # the reference

BASE = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 200, "vocab_size": 1000, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "tie_word_embeddings": False, "rms_norm_eps": 1e-5, "max_position_embeddings": 256, "hidden_act": "silu",
}


def variants():
    def without(*keys):
        d = copy.deepcopy(BASE)
        for k in keys:
            d.pop(k)
        return d

    def with_(**kw):
        d = copy.deepcopy(BASE)
        d.update(kw)
        return d

    return [
        BASE,
        without("head_dim"), without("num_key_value_heads"), without("rope_scaling"), without("rope_theta", "rope_scaling"),
        without("tie_word_embeddings"), without("max_position_embeddings"), without("hidden_act"), without("rms_norm_eps"),
        without("vocab_size"), without("num_hidden_layers"),
        with_(rope_scaling=None), with_(rope_scaling={"type": "llama3", "factor": 2.0}), with_(rope_scaling={"rope_type": "llama3"}),
        with_(rope_scaling={"rope_type": "linear", "factor": 4.0}), with_(rope_scaling={"type": "linear"}),
        with_(rope_scaling={"rope_type": "yarn", "factor": 2.0}), with_(rope_scaling={"rope_type": "default"}),
        with_(rope_parameters={"rope_type": "llama3", "factor": 4.0, "rope_theta": 1234.0}),
        with_(rope_parameters={"rope_theta": 777.0}, rope_scaling=None),
        with_(hidden_act="gelu"), with_(model_type="mistral"), with_(pretraining_tp=2), with_(pretraining_tp=1), with_(pretraining_tp=None),
        with_(use_sliding_window=True), with_(layer_types=["full_attention"] * 3), with_(layer_types=["sliding_attention"] * 3),
        with_(num_attention_heads=4, num_key_value_heads=3), with_(head_dim=31), with_(num_key_value_heads=None, head_dim=None),
        with_(torch_dtype="bfloat16", bos_token_id=1, eos_token_id=[2, 3], use_cache=True, attention_dropout=0.0, mlp_bias=False, attention_bias=False),
    ]


def main():
    configs = []
    for cfg in variants():
        try:
            parsed = ModelConfig.from_hf_dict(cfg)
            fields = dataclasses.asdict(parsed)
            outcome = {"ok": {k: fields[k] for k in ("vocab_size", "hidden_size", "intermediate_size", "num_layers", "num_heads", "num_kv_heads",
                                                     "head_dim", "rms_norm_eps", "max_position_embeddings", "rope", "tie_word_embeddings")}}
        except UnsupportedModelError:
            outcome = {"error": "unsupported"}
        except KeyError:
            outcome = {"error": "missing key"}
        configs.append({"config": cfg, "outcome": outcome})
    rng = random.Random(3)
    hashes = []
    for ns, n, ps in ((b"", 9, 4), (b"model-a", 16, 4), (b"model-a", 16, 8), (b"\x00\xff", 33, 16), (b"", 3, 4)):
        toks = [rng.randrange(200000) for _ in range(n)]
        hashes.append({"namespace": ns.hex(), "tokens": toks, "page_size": ps, "chain": [h.hex() for h in chain_hashes(ns, toks, ps)]})
    out = Path(__file__).resolve().parent / "config_and_hash.json"
    out.write_text(json.dumps({"configs": configs, "hashes": hashes}, indent=0))
    print(len(configs), "configs:", sum(1 for c in configs if "ok" in c["outcome"]), "parsed;", len(hashes), "hash chains ->", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
