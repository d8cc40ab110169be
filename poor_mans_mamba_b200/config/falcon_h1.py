"""Typed configuration of the Falcon-H1 hybrid architecture, read from its own
config.json keys.

Key names and validation rules follow the reference parser
(src/io/config_parser.cpp:10-34, :80-162; struct in include/io/config.h:9-71).
Differences, on purpose: sizes are required but multipliers, bias switches, eps,
theta and the chunk size fall back to neutral defaults when a checkpoint omits
them; ``mamba_norm_before_gate`` (never read by the reference) is understood;
``attention_bias`` / ``mlp_bias`` set to true are refused instead of silently
ignored (the reference parses them at :108/:152 and never applies a bias).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Tuple

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class AttentionConfig:
    num_heads: int
    num_kv_heads: int
    head_dim: int
    rope_theta: float
    bias: bool = False
    dropout: float = 0.0


@dataclass(frozen=True)
class Mamba2Config:
    n_heads: int
    d_head: int
    d_state: int
    d_conv: int
    d_ssm: int
    n_groups: int
    chunk_size: int
    conv_bias: bool
    proj_bias: bool
    rms_norm: bool
    norm_before_gate: bool

    @property
    def conv_dim(self) -> int:
        return self.d_ssm + 2 * self.n_groups * self.d_state

    @property
    def proj_dim(self) -> int:
        return self.d_ssm + self.conv_dim + self.n_heads


@dataclass(frozen=True)
class Multipliers:
    """The muP scale factors; order of ``ssm`` is z, x, B, C, dt; of ``mlp`` gate, down."""
    embedding: float = 1.0
    lm_head: float = 1.0
    attention_in: float = 1.0
    attention_out: float = 1.0
    key: float = 1.0
    ssm_in: float = 1.0
    ssm_out: float = 1.0
    ssm: Tuple[float, float, float, float, float] = (1.0, 1.0, 1.0, 1.0, 1.0)
    mlp: Tuple[float, float] = (1.0, 1.0)


@dataclass(frozen=True)
class FalconH1Config:
    model_type: str
    hidden_size: int
    vocab_size: int
    num_hidden_layers: int
    intermediate_size: int
    tie_word_embeddings: bool
    rms_norm_eps: float
    hidden_act: str
    bos_token_id: int
    eos_token_id: int
    pad_token_id: int
    mlp_bias: bool
    attention: AttentionConfig
    mamba: Mamba2Config
    multipliers: Multipliers
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    MODEL_TYPE = "falcon_h1"

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "FalconH1Config":
        r = KeyReader(data)
        model_type = r.str("model_type")
        if model_type != cls.MODEL_TYPE:
            raise ConfigError(f"expected model_type {cls.MODEL_TYPE}, got {model_type}")
        hidden = r.int("hidden_size")
        n_heads = r.int("num_attention_heads")
        if n_heads <= 0:
            raise ConfigError("config field 'num_attention_heads': must be positive")
        head_dim = r.optional_int("head_dim")
        if head_dim is None:
            if hidden % n_heads:
                raise ConfigError("config field 'head_dim': missing and hidden_size is not a "
                                  "multiple of num_attention_heads")
            head_dim = hidden // n_heads
        attn = AttentionConfig(
            num_heads=n_heads,
            num_kv_heads=r.int("num_key_value_heads", n_heads),
            head_dim=head_dim,
            rope_theta=r.float("rope_theta", 10000.0),
            bias=r.bool("attention_bias", False),
            dropout=r.float("attention_dropout", 0.0),
        )
        mamba = Mamba2Config(
            n_heads=r.int("mamba_n_heads"),
            d_head=r.int("mamba_d_head"),
            d_state=r.int("mamba_d_state"),
            d_conv=r.int("mamba_d_conv"),
            d_ssm=r.int("mamba_d_ssm"),
            n_groups=r.int("mamba_n_groups"),
            chunk_size=r.int("mamba_chunk_size", 128),
            conv_bias=r.bool("mamba_conv_bias", True),
            proj_bias=r.bool("mamba_proj_bias", False),
            rms_norm=r.bool("mamba_rms_norm", False),
            norm_before_gate=cls._norm_before_gate(r),
        )
        mult = Multipliers(
            embedding=r.float("embedding_multiplier", 1.0),
            lm_head=r.float("lm_head_multiplier", 1.0),
            attention_in=r.float("attention_in_multiplier", 1.0),
            attention_out=r.float("attention_out_multiplier", 1.0),
            key=r.float("key_multiplier", 1.0),
            ssm_in=r.float("ssm_in_multiplier", 1.0),
            ssm_out=r.float("ssm_out_multiplier", 1.0),
            ssm=r.float_list("ssm_multipliers", 5, (1.0,) * 5),
            mlp=r.float_list("mlp_multipliers", 2, (1.0, 1.0)),
        )
        cfg = cls(
            model_type=model_type,
            hidden_size=hidden,
            vocab_size=r.int("vocab_size"),
            num_hidden_layers=r.int("num_hidden_layers"),
            intermediate_size=r.int("intermediate_size"),
            tie_word_embeddings=r.bool("tie_word_embeddings", False),
            rms_norm_eps=r.float("rms_norm_eps", 1e-5),
            hidden_act=r.str("hidden_act", "silu"),
            bos_token_id=r.int("bos_token_id", 0),
            eos_token_id=r.int("eos_token_id", -1),
            pad_token_id=r.int("pad_token_id", 0),
            mlp_bias=r.bool("mlp_bias", False),
            attention=attn,
            mamba=mamba,
            multipliers=mult,
            raw=dict(data),
        )
        cfg.validate()
        return cfg

    @staticmethod
    def _norm_before_gate(r: KeyReader) -> bool:
        """``mamba_norm_before_gate``.  The order of gate and norm changes the result, the
        reference never reads the key (its gated norm is gate first, then norm,
        src/ops/cpu_backend.cpp:286-304), and writers of configurations disagree on what an absent
        key means.  So with the gated norm on the key must be there; with it off the key has no
        effect and defaults to false."""
        if r.bool("mamba_rms_norm", False) and "mamba_norm_before_gate" not in r.data:
            raise ConfigError("config field 'mamba_norm_before_gate': required when mamba_rms_norm is true "
                              "(false: gate, then norm, as the reference computes it; true: norm, then gate)")
        return r.bool("mamba_norm_before_gate", False)

    def validate(self) -> None:
        a, m = self.attention, self.mamba
        for name, val in (("hidden_size", self.hidden_size), ("vocab_size", self.vocab_size),
                          ("num_hidden_layers", self.num_hidden_layers),
                          ("intermediate_size", self.intermediate_size),
                          ("num_key_value_heads", a.num_kv_heads), ("head_dim", a.head_dim)):
            if val <= 0:
                raise ConfigError(f"config field '{name}': must be positive, got {val}")
        if a.num_heads % a.num_kv_heads:
            raise ConfigError("invalid attention head config: num_attention_heads must be a "
                              "multiple of num_key_value_heads")
        if a.head_dim % 2:
            raise ConfigError("config field 'head_dim': rotate-half RoPE needs an even head_dim")
        if a.rope_theta <= 0:
            raise ConfigError("config field 'rope_theta': must be positive")
        # src/io/config_parser.cpp:22-34
        if (m.n_heads <= 0 or m.d_head <= 0 or m.d_state <= 0 or m.d_conv <= 1 or m.d_ssm <= 0
                or m.n_groups <= 0 or m.chunk_size <= 0):
            raise ConfigError("invalid ssm dimensions")
        if m.n_heads % m.n_groups:
            raise ConfigError("n_heads must be divisible by n_groups")
        if m.d_ssm != m.n_heads * m.d_head:
            raise ConfigError("d_inner must equal n_heads * d_head")
        if m.rms_norm and m.d_ssm % m.n_groups:
            raise ConfigError("mamba_d_ssm must be divisible by mamba_n_groups for the gated norm")
        if self.hidden_act != "silu":
            raise ConfigError(f"config field 'hidden_act': only 'silu' is implemented, got "
                              f"{self.hidden_act!r}")
        if a.bias:
            raise ConfigError("config field 'attention_bias': true is not supported (no bias "
                              "tensor is ever applied to the attention projections)")
        if self.mlp_bias:
            raise ConfigError("config field 'mlp_bias': true is not supported (no bias tensor is "
                              "ever applied to the feed-forward projections)")
        if self.rms_norm_eps <= 0:
            raise ConfigError("config field 'rms_norm_eps': must be positive")

    def to_dict(self) -> Dict[str, Any]:
        """The config.json form of this configuration (round-trips through from_dict)."""
        a, m, s = self.attention, self.mamba, self.multipliers
        return {
            "model_type": self.model_type,
            "architectures": ["FalconH1ForCausalLM"],
            "hidden_size": self.hidden_size,
            "vocab_size": self.vocab_size,
            "num_hidden_layers": self.num_hidden_layers,
            "intermediate_size": self.intermediate_size,
            "tie_word_embeddings": self.tie_word_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "hidden_act": self.hidden_act,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": self.eos_token_id,
            "pad_token_id": self.pad_token_id,
            "mlp_bias": self.mlp_bias,
            "num_attention_heads": a.num_heads,
            "num_key_value_heads": a.num_kv_heads,
            "head_dim": a.head_dim,
            "rope_theta": a.rope_theta,
            "attention_bias": a.bias,
            "attention_dropout": a.dropout,
            "mamba_n_heads": m.n_heads,
            "mamba_d_head": m.d_head,
            "mamba_d_state": m.d_state,
            "mamba_d_conv": m.d_conv,
            "mamba_d_ssm": m.d_ssm,
            "mamba_n_groups": m.n_groups,
            "mamba_chunk_size": m.chunk_size,
            "mamba_conv_bias": m.conv_bias,
            "mamba_proj_bias": m.proj_bias,
            "mamba_rms_norm": m.rms_norm,
            "mamba_norm_before_gate": m.norm_before_gate,
            "embedding_multiplier": s.embedding,
            "lm_head_multiplier": s.lm_head,
            "attention_in_multiplier": s.attention_in,
            "attention_out_multiplier": s.attention_out,
            "key_multiplier": s.key,
            "ssm_in_multiplier": s.ssm_in,
            "ssm_out_multiplier": s.ssm_out,
            "ssm_multipliers": list(s.ssm),
            "mlp_multipliers": list(s.mlp),
        }
