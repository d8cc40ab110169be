"""Configuration and registry (no GPU)."""
import json
import os

import pytest

from tiny_configs import tiny_config

from poor_mans_mamba_b200 import architectures  # noqa: F401
from poor_mans_mamba_b200.architectures.falcon_h1 import model_spec
from poor_mans_mamba_b200.config import (ConfigError, FalconH1Config, load_config_json, open_model_dir,
                                         registered_architectures, resolve_architecture)


def test_tiny_configs_parse_and_differ():
    a = FalconH1Config.from_dict(tiny_config("A"))
    b = FalconH1Config.from_dict(tiny_config("B"))
    assert (a.hidden_size, a.vocab_size, a.num_hidden_layers) == (64, 256, 2)
    assert (b.attention.num_heads, b.attention.num_kv_heads, b.attention.head_dim) == (3, 1, 32)
    assert a.mamba.conv_dim == 128 + 2 * 16 and a.mamba.proj_dim == 128 + 160 + 8
    assert b.mamba.conv_dim == 192 + 2 * 2 * 32
    assert b.multipliers.ssm == (0.5, 1.1, 0.9, 1.3, 0.7) and b.multipliers.mlp == (1.5, 0.4)
    for fa, fb in ((a.hidden_size, b.hidden_size), (a.attention.head_dim, b.attention.head_dim),
                   (a.mamba.d_state, b.mamba.d_state), (a.mamba.d_conv, b.mamba.d_conv),
                   (a.mamba.n_groups, b.mamba.n_groups), (a.rms_norm_eps, b.rms_norm_eps),
                   (a.tie_word_embeddings, b.tie_word_embeddings), (a.mamba.rms_norm, b.mamba.rms_norm)):
        assert fa != fb


def test_round_trip_through_dict():
    b = FalconH1Config.from_dict(tiny_config("B"))
    assert FalconH1Config.from_dict(b.to_dict()) == b


def test_defaults_for_optional_keys():
    d = tiny_config("A")
    for k in ("ssm_multipliers", "mlp_multipliers", "key_multiplier", "embedding_multiplier",
              "mamba_rms_norm", "mamba_conv_bias", "rms_norm_eps", "rope_theta", "head_dim",
              "mamba_chunk_size", "tie_word_embeddings", "mamba_norm_before_gate"):
        d.pop(k)
    c = FalconH1Config.from_dict(d)
    assert c.multipliers.ssm == (1.0,) * 5 and c.multipliers.key == 1.0
    assert c.mamba.rms_norm is False and c.mamba.conv_bias is True
    assert c.attention.head_dim == 64 // 4 and c.attention.rope_theta == 10000.0
    assert c.rms_norm_eps == 1e-5 and c.mamba.chunk_size == 128 and not c.tie_word_embeddings


@pytest.mark.parametrize("key", ["hidden_size", "vocab_size", "num_hidden_layers", "intermediate_size",
                                 "num_attention_heads", "mamba_n_heads", "mamba_d_head", "mamba_d_state",
                                 "mamba_d_conv", "mamba_d_ssm", "mamba_n_groups", "model_type"])
def test_missing_size_names_the_key(key):
    d = tiny_config("B")
    d.pop(key)
    with pytest.raises(ConfigError, match=key):
        if key == "model_type":
            d.pop("architectures")
            resolve_architecture(d)
        else:
            FalconH1Config.from_dict(d)


@pytest.mark.parametrize("patch,msg", [
    ({"ssm_multipliers": [1, 2, 3]}, "length 5"),
    ({"mlp_multipliers": [1.0]}, "length 2"),
    ({"mamba_d_conv": 1}, "invalid ssm dimensions"),
    ({"mamba_n_groups": 4}, "divisible by n_groups"),
    ({"mamba_d_ssm": 100}, "n_heads \\* d_head"),
    ({"num_key_value_heads": 2}, "multiple of num_key_value_heads"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"hidden_size": "96"}, "hidden_size"),
    ({"head_dim": 31}, "head_dim"),
    ({"vocab_size": 0}, "vocab_size"),
])
def test_validation_rules(patch, msg):
    d = tiny_config("B")
    d.update(patch)
    with pytest.raises(ConfigError, match=msg):
        FalconH1Config.from_dict(d)


def test_registry_by_model_type_and_architectures():
    assert "falcon_h1" in registered_architectures()
    assert resolve_architecture({"model_type": "falcon_h1"}).name == "falcon_h1"
    assert resolve_architecture({"model_type": "x", "architectures": ["FalconH1ForCausalLM"]}).name == "falcon_h1"
    with pytest.raises(ConfigError, match="unsupported model_type: llama"):
        resolve_architecture({"model_type": "llama"})


def test_config_json_with_non_json_numbers(tmp_path):
    d = tiny_config("A")
    text = json.dumps(d).replace('"rope_theta": 10000.0', '"rope_theta": 10000.0, "x_inf": Infinity, '
                                                          '"x_ninf": -Infinity, "x_nan": NaN')
    (tmp_path / "config.json").write_text(text)
    data = load_config_json(str(tmp_path))
    assert data["x_inf"] == 1e308 and data["x_ninf"] == -1e308 and data["x_nan"] is None
    arch, cfg = open_model_dir(str(tmp_path))
    assert arch.name == "falcon_h1" and cfg.hidden_size == 64
    with pytest.raises(ConfigError, match="cannot read"):
        load_config_json(str(tmp_path / "nope"))


def test_model_spec_is_data_taken_from_the_config():
    cfg = FalconH1Config.from_dict(tiny_config("B"))
    spec = model_spec(cfg)
    assert len(spec.layers) == 3 and [c.layer for c in spec.order] == [0, 1, 2]
    assert spec.head_name == "lm_head.weight" and spec.head_multiplier == 0.5
    layer = spec.layers[1]
    mixers = layer.part("mixers")
    assert layer.arrangement == "parallel_prenorm" and set(layer.parts) == {"mixer_norm", "mixers", "ffn_norm", "ffn"}
    assert layer.prefix == "model.layers.1." and [m.kind for m in mixers] == ["mamba2", "paged_attention"]
    assert mixers[0].params["chunk_multipliers"] == (0.5, 1.1, 0.9, 1.3, 0.7)
    assert mixers[1].params["position_encoding"] == {"kind": "rotary", "theta": 1e11}
    assert layer.part("mixer_norm").params["eps"] == 1e-6 and layer.part("ffn").kind == "swiglu"
    assert model_spec(FalconH1Config.from_dict(tiny_config("A"))).head_name is None


def test_parts_are_built_from_specs_by_name():
    from poor_mans_mamba_b200.parts import PartSpec, build_part, registered
    assert {"mamba2", "paged_attention"} <= set(registered("mixer"))
    assert {"rotary", "none"} <= set(registered("position_encoding"))
    plain = build_part("mixer", PartSpec("paged_attention", "attn", {"num_heads": 4, "num_kv_heads": 2, "head_dim": 32}),
                       hidden_size=64)
    assert plain.position_encoding.inv_freq is None and plain.input_rows() == (4 + 2 * 2) * 32
    assert [s.name for s in plain.state_specs()] == ["kv"] and plain.state_specs()[0].width == 64
    shared = build_part("mixer", PartSpec("paged_attention", "attn", {"num_heads": 4, "num_kv_heads": 2, "head_dim": 32,
                                                                      "shared_kv": True}), hidden_size=64)
    assert shared.state_specs() == [] and [p.name for p in shared.param_specs()] == ["q_proj.weight", "o_proj.weight"]
    with pytest.raises(KeyError, match="unknown mixer"):
        build_part("mixer", PartSpec("nope", "x", {}), hidden_size=8)


def test_gate_and_norm_order_must_be_stated_when_the_gated_norm_is_on():
    from poor_mans_mamba_b200.config import ConfigError
    from poor_mans_mamba_b200.config.falcon_h1 import FalconH1Config
    from tiny_configs import tiny_config
    a = tiny_config("A")            # gated norm on
    del a["mamba_norm_before_gate"]
    with pytest.raises(ConfigError, match="mamba_norm_before_gate"):
        FalconH1Config.from_dict(a)
    a["mamba_norm_before_gate"] = True
    assert FalconH1Config.from_dict(a).mamba.norm_before_gate is True
    b = tiny_config("B")            # gated norm off: the key has no effect and may be absent
    del b["mamba_norm_before_gate"]
    assert FalconH1Config.from_dict(b).mamba.norm_before_gate is False
