"""Tiny Qwen3 configurations for the tests.  They differ in every size and option:
layers, width, head counts, group size, head size (a power of two or not, equal to
width/heads or not), feed-forward width, vocabulary (a power of two or not), rope
base, eps, tied or untied head, and sliding window."""
from __future__ import annotations

import copy

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "hidden_size": 64,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "intermediate_size": 128,
    "vocab_size": 256,
    "max_position_embeddings": 128,
    "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0,
    "tie_word_embeddings": True,
    "use_sliding_window": False,
    "hidden_act": "silu",
    "attention_bias": False,
    "torch_dtype": "bfloat16",
    "eos_token_id": 255,
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "hidden_size": 96,
    "num_hidden_layers": 3,
    "num_attention_heads": 6,
    "num_key_value_heads": 3,
    "head_dim": 32,
    "intermediate_size": 224,
    "vocab_size": 384,
    "max_position_embeddings": 256,
    "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0,
    "tie_word_embeddings": False,
    "use_sliding_window": False,
    "sliding_window": None,
    "max_window_layers": 3,
    "hidden_act": "silu",
    "attention_bias": False,
    "torch_dtype": "bfloat16",
    "eos_token_id": [382, 383],
}

# Odd sizes: one kv head for five query heads, a head size that is no power of two,
# an odd vocabulary, and a window on the layers from index 1 on.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "hidden_size": 80,
    "num_hidden_layers": 4,
    "num_attention_heads": 5,
    "num_key_value_heads": 1,
    "head_dim": 48,
    "intermediate_size": 176,
    "vocab_size": 515,
    "max_position_embeddings": 1024,
    "rms_norm_eps": 3e-6,
    "rope_theta": 500000.0,
    "tie_word_embeddings": False,
    "use_sliding_window": True,
    "sliding_window": 40,
    "max_window_layers": 1,
    "hidden_act": "silu",
    "attention_bias": False,
    "torch_dtype": "bfloat16",
}

# Head size 64, which in bfloat16 takes prompt portions through the tcgen05 attention
# kernel: three query heads per kv head, a window on the second layer only.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "hidden_size": 112,
    "num_hidden_layers": 2,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "intermediate_size": 144,
    "vocab_size": 300,
    "max_position_embeddings": 2048,
    "rms_norm_eps": 2e-6,
    "rope_theta": 20000.0,
    "tie_word_embeddings": True,
    "use_sliding_window": True,
    "sliding_window": 150,
    "max_window_layers": 1,
    "hidden_act": "silu",
    "attention_bias": False,
    "torch_dtype": "bfloat16",
}

ALL = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_d": TINY_D}


def get(name: str) -> dict:
    return copy.deepcopy(ALL[name])
