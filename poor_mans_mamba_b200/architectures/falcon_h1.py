"""Falcon-H1 hybrid: every layer runs a Mamba2 mixer and a GQA RoPE attention in parallel
on one RMS-normed input, adds both (scaled) to the residual stream, then a SwiGLU
feed-forward (reference src/runtime/runner/falconh1_runner.cpp:20-127).

This module only *describes* the model: it turns a FalconH1Config into a ModelSpec (parts
by name with their constants, tensor-name prefixes from src/model/falconh1_loader.cpp:27-58,
and the order of layers).  The parts themselves do not know this architecture.
"""
from __future__ import annotations

from ..config.falcon_h1 import FalconH1Config
from ..parts.base import LayerCall, ModelSpec, PartSpec
from ..parts.block import prenorm_layer


def model_spec(cfg: FalconH1Config) -> ModelSpec:
    a, m, s = cfg.attention, cfg.mamba, cfg.multipliers
    norm = {"eps": cfg.rms_norm_eps}
    layers = []
    for i in range(cfg.num_hidden_layers):
        mamba = PartSpec("mamba2", "mamba", {
            "n_heads": m.n_heads, "d_head": m.d_head, "d_state": m.d_state, "d_conv": m.d_conv,
            "n_groups": m.n_groups, "chunk_size": m.chunk_size, "conv_bias": m.conv_bias,
            "proj_bias": m.proj_bias, "gated_norm": m.rms_norm, "norm_before_gate": m.norm_before_gate,
            "norm_eps": cfg.rms_norm_eps, "in_multiplier": s.ssm_in, "out_multiplier": s.ssm_out,
            "chunk_multipliers": tuple(s.ssm),
        })
        attn = PartSpec("paged_attention", "self_attn", {
            "num_heads": a.num_heads, "num_kv_heads": a.num_kv_heads, "head_dim": a.head_dim,
            "position_encoding": {"kind": "rotary", "theta": a.rope_theta},
            "in_multiplier": s.attention_in, "out_multiplier": s.attention_out,
            "key_multiplier": s.key,
        })
        ffn = PartSpec("swiglu", "feed_forward", {
            "intermediate_size": cfg.intermediate_size, "gate_multiplier": s.mlp[0],
            "down_multiplier": s.mlp[1],
        })
        layers.append(prenorm_layer(
            prefix=f"model.layers.{i}.",
            mixer_norm=PartSpec("rmsnorm", "input_layernorm", dict(norm)),
            mixers=(mamba, attn),  # joined in this order: (h + mamba) + attention
            ffn_norm=PartSpec("rmsnorm", "pre_ff_layernorm", dict(norm)),
            ffn=ffn,
        ))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding_name="model.embed_tokens.weight",
        embedding_multiplier=s.embedding,
        layers=tuple(layers),
        order=tuple(LayerCall(i, i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", "model.final_layernorm", dict(norm)),
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        head_multiplier=s.lm_head,
        eos_token_id=cfg.eos_token_id,
        bos_token_id=cfg.bos_token_id,
    )
