"""Tiny configurations of the architecture, as config.json dictionaries.

They differ in every size and option: head counts and groups (GQA 4/2, MQA 3/1,
MHA 5/5), head sizes 16/32/48, widths and vocabularies that are no power of
two, number of layers, eps, rope (default / llama3 with all three frequency
bands inside 256 positions / linear), tied and untied heads, and the KV page size the
tests pair with each.
"""

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "intermediate_size": 128,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "tie_word_embeddings": True,
    "rms_norm_eps": 1e-6,
    "max_position_embeddings": 128,
    "hidden_act": "silu",
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 3,
    "hidden_size": 96,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "head_dim": 32,
    "intermediate_size": 200,
    "vocab_size": 1000,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64,
    },
    "tie_word_embeddings": False,
    "rms_norm_eps": 1e-5,
    "max_position_embeddings": 256,
    "hidden_act": "silu",
}

# A third one: MHA, head_dim 48 (a multiple of 16 that is no power of two),
# head_dim * heads != hidden, odd vocabulary, linear rope scaling (legacy spelling of the key).
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 1,
    "hidden_size": 80,
    "num_attention_heads": 5,
    "num_key_value_heads": 5,
    "head_dim": 48,
    "intermediate_size": 144,
    "vocab_size": 517,
    "rope_theta": 130000.0,
    "rope_scaling": {"type": "linear", "factor": 2.5},
    "tie_word_embeddings": True,
    "rms_norm_eps": 3e-6,
    "max_position_embeddings": 512,
    "hidden_act": "silu",
}

# name -> (config, weight seed, KV page size)
TINY = {"tiny_a": (TINY_A, 0, 4), "tiny_b": (TINY_B, 1, 16), "tiny_c": (TINY_C, 2, 8)}
