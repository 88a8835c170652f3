"""Tiny Llama4 configurations for the tests: two that differ in every size and option, one that
stays inside what the reference's own engine computes, and helpers that write model folders."""
from __future__ import annotations

import copy
import tempfile

import torch

# A: all layers MoE, top-1, llama3-scaled RoPE, QK norm, temperature tuning, untied head.
TINY_A = {
    "architectures": ["Llama4ForCausalLM"],
    "num_hidden_layers": 4, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "intermediate_size_mlp": 256,
    "num_local_experts": 4, "num_experts_per_tok": 1, "interleave_moe_layer_step": 1,
    "vocab_size": 512, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "nope_layer_interval": 4, "attention_chunk_size": 32, "use_qk_norm": True,
    "attn_temperature_tuning": True, "floor_scale": 32, "attn_scale": 0.1,
    "tie_word_embeddings": False, "max_position_embeddings": 1024, "initializer_range": 0.02,
    "eos_token_id": [3, 5],
}

# B: differs from A in every size and option; nested text_config under the multimodal architecture.
TINY_B = {
    "architectures": ["Llama4ForConditionalGeneration"],
    "text_config": {
        "num_hidden_layers": 6, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 3,
        "head_dim": 32, "intermediate_size": 64, "intermediate_size_mlp": 192,
        "num_local_experts": 8, "num_experts_per_tok": 2, "interleave_moe_layer_step": 2,
        "vocab_size": 1000, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "rope_scaling": None,
        "nope_layer_interval": 3, "attention_chunk_size": 16, "use_qk_norm": False,
        "attn_temperature_tuning": False, "floor_scale": 8192, "attn_scale": 0.1,
        "max_position_embeddings": 512, "initializer_range": 0.05,
        "rope_pairing": "interleaved", "router_gate": "sigmoid_output",
        "eos_token_id": 7,
    },
    "tie_word_embeddings": True,
}

# R: only what the reference's engine computes (src/engine/llama4_cpu_engine.cpp): every layer RoPE and
# MoE, top-1 without a gate, weightless QK norm before RoPE, full causal attention, Q width == hidden.
TINY_R = {
    "architectures": ["Llama4ForConditionalGeneration"],
    "text_config": {
        "num_hidden_layers": 3, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
        "head_dim": 16, "intermediate_size": 128, "intermediate_size_mlp": 128,
        "num_local_experts": 4, "num_experts_per_tok": 1, "interleave_moe_layer_step": 1,
        "vocab_size": 512, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
        "nope_layer_interval": 0, "attention_chunk_size": 0, "use_qk_norm": True,
        "attn_temperature_tuning": False, "max_position_embeddings": 1024, "initializer_range": 0.02,
        "qk_norm_order": "before_rope", "qk_norm_scope": "all_layers", "router_gate": "none",
    },
    "tie_word_embeddings": False,
}

# C: head size 64 and widths that are multiples of 8, so that the bfloat16 path runs on the tensor-core
# kernels (GEMM, prefill and decode attention); chunk and temperature floor inside a few hundred tokens.
TINY_C = {
    "architectures": ["Llama4ForCausalLM"],
    "num_hidden_layers": 4, "hidden_size": 136, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 200, "intermediate_size_mlp": 264,
    "num_local_experts": 5, "num_experts_per_tok": 2, "interleave_moe_layer_step": 2,
    "vocab_size": 777, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 128},
    "nope_layer_interval": 2, "attention_chunk_size": 160, "use_qk_norm": True,
    "attn_temperature_tuning": True, "floor_scale": 100, "attn_scale": 0.2,
    "tie_word_embeddings": False, "max_position_embeddings": 4096, "initializer_range": 0.03,
}

# R2: a second point inside what the reference's engine computes, other in every size it lets one choose:
# flat config, wider, more heads in groups of two, fewer layers, three experts of a width that is no power of
# two, another vocabulary, another RoPE base, factor and band edges, a short original context.
TINY_R2 = {
    "architectures": ["Llama4ForConditionalGeneration"],
    "text_config": {
        "num_hidden_layers": 2, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 3,
        "head_dim": 16, "intermediate_size": 80, "intermediate_size_mlp": 80,
        "num_local_experts": 3, "num_experts_per_tok": 1, "interleave_moe_layer_step": 1,
        "vocab_size": 300, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 2.0,
                         "high_freq_factor": 6.0, "original_max_position_embeddings": 32},
        "nope_layer_interval": 0, "attention_chunk_size": 0, "use_qk_norm": True,
        "attn_temperature_tuning": False, "max_position_embeddings": 1024, "initializer_range": 0.05,
        "qk_norm_order": "before_rope", "qk_norm_scope": "all_layers", "router_gate": "none",
    },
    "tie_word_embeddings": False,
}

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "R": (TINY_R, 2), "C": (TINY_C, 3), "R2": (TINY_R2, 4)}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name][0])


def make_model_dir(name_or_config, seed=None, root=None, dtype=torch.bfloat16) -> str:
    """Writes config.json and model.safetensors into a fresh temporary folder; returns its path."""
    from cpi_b200.weights import write_random_model
    if isinstance(name_or_config, str):
        cfg, default_seed = config(name_or_config), CONFIGS[name_or_config][1]
    else:
        cfg, default_seed = copy.deepcopy(name_or_config), 0
    d = tempfile.mkdtemp(prefix="cpi_tiny_", dir=root)
    write_random_model(d, cfg, default_seed if seed is None else seed, dtype)
    return d


def random_tokens(n: int, vocab: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
