"""
Tiny Llama configurations for the tests, as the config.json dictionaries a model folder would hold.
They differ from one another in every size and option: layers, width, heads and groups, head size
(left out of A so the hidden_size // heads default is used; not equal to that default in C),
feed-forward width, vocabulary, rope base and scaling (absent / top-level rope_scaling /
rope_parameters spelling), norm eps, tied or untied head, and table length.
"""

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 512,
    "hidden_size": 64,
    "intermediate_size": 176,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "hidden_act": "silu",
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "max_position_embeddings": 256,
    "tie_word_embeddings": True,
    "eos_token_id": 3,
}
PAGE_A = 16

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 1000,
    "hidden_size": 192,
    "intermediate_size": 512,
    "num_hidden_layers": 3,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "hidden_act": "silu",
    "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64,
    },
    "max_position_embeddings": 512,
    "tie_word_embeddings": False,
    "eos_token_id": [7, 9],
}
PAGE_B = 32

TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 777,
    "hidden_size": 120,
    "intermediate_size": 200,
    "num_hidden_layers": 2,
    "num_attention_heads": 5,
    "num_key_value_heads": 1,
    "head_dim": 48,
    "hidden_act": "silu",
    "rms_norm_eps": 1e-4,
    "rope_parameters": {
        "rope_type": "llama3",
        "rope_theta": 1000000.0,
        "factor": 4.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 2.0,
        "original_max_position_embeddings": 32,
    },
    "max_position_embeddings": 320,
    "tie_word_embeddings": False,
}
PAGE_C = 64

# Head size 64 and a page size the replay program uses (64): the sizes the bfloat16 tensor-core
# attention kernels take; three query heads per kv head.
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 640,
    "hidden_size": 160,
    "intermediate_size": 336,
    "num_hidden_layers": 2,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "hidden_act": "silu",
    "rms_norm_eps": 1e-5,
    "rope_theta": 50000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 2.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 256},
    "max_position_embeddings": 1100,
    "tie_word_embeddings": True,
}
PAGE_D = 64

# Seeds and spreads of the random weights the tests and the golden files use.  Norm weights spread
# widely (1 + N(0, 0.25)) so that a norm weight left out or misplaced changes the logits visibly.
WEIGHTS = {"std": 0.05, "unit_std": 0.25}
SEED_A, SEED_B, SEED_C, SEED_D = 11, 22, 33, 44
