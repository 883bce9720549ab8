"""Two tiny Qwen3 configurations for tests; they differ in every size and option."""

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 192, "vocab_size": 512, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": True,
    "max_position_embeddings": 256, "eos_token_id": 7,
}

# heads * head_dim = 192 != hidden; sizes that are no power of two; biases; untied head; a window
# on two of the three layers; two stop tokens.
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 32, "intermediate_size": 160, "vocab_size": 1000, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "attention_bias": True, "tie_word_embeddings": False,
    "max_position_embeddings": 512, "eos_token_id": [3, 11],
    "use_sliding_window": True, "sliding_window": 40,
    "layer_types": ["sliding_attention", "full_attention", "sliding_attention"],
}

# A third shape for spot checks: one kv head, a wider head, partial rotation.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 1, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 1,
    "head_dim": 48, "intermediate_size": 112, "vocab_size": 301, "rope_theta": 50000.0,
    "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": False,
    "partial_rotary_factor": 0.5, "max_position_embeddings": 1024,
}

# Heads of 128 as the released models have (few of them, a narrow model): the shapes at which the
# tensor-core attention kernels, the streaming decode attention and the fused q/k/v product apply.
# A window on one layer, biases, a vocabulary that is no multiple of anything.
SMALL_128 = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 384, "vocab_size": 1003, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": False,
    "max_position_embeddings": 2048, "eos_token_id": 5,
    "use_sliding_window": True, "sliding_window": 200,
    "layer_types": ["full_attention", "sliding_attention"],
}

# Heads of 64: the other head size that the tensor-core prompt attention and the streaming decode
# attention take (three query heads to a kv head, no biases, a tied head).
SMALL_64 = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 320, "vocab_size": 777, "rope_theta": 500000.0,
    "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": True,
    "max_position_embeddings": 2048, "eos_token_id": 5,
    "use_sliding_window": True, "sliding_window": 130,
    "layer_types": ["sliding_attention", "full_attention"],
}

# How far the bfloat16 engine may be from the float64 plain implementation on the same
# (bfloat16-valued) weights, as a fraction of the largest logit.  Measured on a B200 over three
# weight seeds, sequences of 9 to 740 tokens, whole and with the last 32 tokens one by one: at
# most 2.8e-3 (Tiny A), 5.1e-3 (Tiny B), 6.0e-3 (heads of 128); the bound is twice that.  The
# logits' standard deviation is 0.11 to 0.23 of the largest logit, so a dropped key, a wrong page
# or a tensor rounded in the wrong place shows; a single wrong low bit does not, and is what the
# kernel tests are for (2^-7 to 2^-8 of the result against float32, with planted far keys).
TOL_BF16 = {"A": 6e-3, "B": 1e-2, "S128": 1.2e-2}
