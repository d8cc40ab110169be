"""The two tiny Falcon-H1 configurations of the test-suite (config.json dicts).  They
differ in every size and option: layers, widths that are no power of two, head counts and
groups, head sizes, vocabulary, eps, theta, d_state/d_conv/n_groups/chunk size, biases,
gated norm, multipliers, tied or untied head."""
from __future__ import annotations

import copy
import random

TINY_A = {
    "model_type": "falcon_h1", "architectures": ["FalconH1ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "vocab_size": 256, "intermediate_size": 128,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "rope_theta": 10000.0,
    "attention_bias": False, "attention_dropout": 0.0, "mlp_bias": False,
    "mamba_d_ssm": 128, "mamba_n_heads": 8, "mamba_d_head": 16, "mamba_d_state": 16,
    "mamba_n_groups": 1, "mamba_d_conv": 4, "mamba_chunk_size": 32,
    "mamba_conv_bias": False, "mamba_proj_bias": False, "mamba_rms_norm": True,
    "mamba_norm_before_gate": False, "rms_norm_eps": 1e-5, "hidden_act": "silu",
    "embedding_multiplier": 1.0, "lm_head_multiplier": 1.0, "attention_in_multiplier": 1.0,
    "attention_out_multiplier": 1.0, "key_multiplier": 1.0, "ssm_in_multiplier": 1.0,
    "ssm_out_multiplier": 1.0, "ssm_multipliers": [1.0, 1.0, 1.0, 1.0, 1.0],
    "mlp_multipliers": [1.0, 1.0], "tie_word_embeddings": True,
    "bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0,
}

TINY_B = {
    "model_type": "falcon_h1", "architectures": ["FalconH1ForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 96, "vocab_size": 384, "intermediate_size": 160,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "rope_theta": 1e11,
    "attention_bias": False, "attention_dropout": 0.0, "mlp_bias": False,
    "mamba_d_ssm": 192, "mamba_n_heads": 6, "mamba_d_head": 32, "mamba_d_state": 32,
    "mamba_n_groups": 2, "mamba_d_conv": 3, "mamba_chunk_size": 16,
    "mamba_conv_bias": True, "mamba_proj_bias": True, "mamba_rms_norm": False,
    "mamba_norm_before_gate": False, "rms_norm_eps": 1e-6, "hidden_act": "silu",
    "embedding_multiplier": 5.0, "lm_head_multiplier": 0.5, "attention_in_multiplier": 0.8,
    "attention_out_multiplier": 0.9, "key_multiplier": 0.7, "ssm_in_multiplier": 1.2,
    "ssm_out_multiplier": 0.6, "ssm_multipliers": [0.5, 1.1, 0.9, 1.3, 0.7],
    "mlp_multipliers": [1.5, 0.4], "tie_word_embeddings": False,
    "bos_token_id": 1, "eos_token_id": 3, "pad_token_id": 0,
}

# (seed, prompt lengths, decode steps)
TINY_WORKLOADS = {"A": (0, (7, 19, 33), 8), "B": (1, (1, 16, 17, 50), 12)}
TINY = {"A": TINY_A, "B": TINY_B}


def tiny_config(which: str) -> dict:
    return copy.deepcopy(TINY[which])


def token_sequences(which: str, extra: int = 0):
    """The workload's sequences: prompt + forced decode tokens, uniform ids from the seed."""
    seed, lens, n_dec = TINY_WORKLOADS[which]
    rng = random.Random(seed)
    vocab = TINY[which]["vocab_size"]
    return [[rng.randrange(vocab) for _ in range(n + n_dec + extra)] for n in lens]
