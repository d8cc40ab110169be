"""Safetensors reading/writing, by-name loading and its one error, random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

from tiny_configs import tiny_config

from poor_mans_mamba_b200.config import open_model_dir
from poor_mans_mamba_b200.engine.model import Model
from poor_mans_mamba_b200.weights import (ModelFiles, SafetensorsError, SafetensorsFile, WeightsError,
                                          load_tensors, save_file, write_random_model)


def _model_for(d):
    arch, cfg = open_model_dir(d)
    return Model(arch.model_spec(cfg))


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b.c": torch.randn(7).to(torch.bfloat16), "i": torch.arange(6, dtype=torch.int32),
         "e": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p, {"k": "v"})
    f = SafetensorsFile(p)
    assert sorted(f.keys()) == sorted(t) and f.metadata == {"k": "v"}
    for k, v in t.items():
        assert f.info(k)[1] == tuple(v.shape)
        assert torch.equal(f.tensor(k), v)
    f.close()


def test_own_reader_agrees_with_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"w": torch.randn(4, 6).to(torch.bfloat16), "v": torch.randn(9)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p)
    other = st.load_file(p)
    assert all(torch.equal(other[k], t[k]) for k in t)
    st.save_file(t, str(tmp_path / "y.safetensors"))
    f = SafetensorsFile(str(tmp_path / "y.safetensors"))
    assert all(torch.equal(f.tensor(k), t[k]) for k in t)
    f.close()


def test_corrupt_files_are_refused(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x05")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError, match="neither"):
        ModelFiles(str(tmp_path))


@pytest.mark.parametrize("which", ["A", "B"])
def test_random_model_has_exactly_the_declared_tensors(tmp_path, which):
    d = write_random_model(tiny_config(which), seed=3, out_dir=str(tmp_path / "m"))
    model = _model_for(d)
    specs = model.param_specs()
    files = ModelFiles(d)
    assert sorted(files.keys()) == sorted(specs)
    cfg = tiny_config(which)
    assert ("lm_head.weight" in specs) == (not cfg["tie_word_embeddings"])
    assert ("model.layers.0.mamba.conv1d.bias" in specs) == cfg["mamba_conv_bias"]
    assert ("model.layers.0.mamba.in_proj.bias" in specs) == cfg["mamba_proj_bias"]
    assert ("model.layers.0.mamba.norm.weight" in specs) == cfg["mamba_rms_norm"]
    assert files.info("model.layers.0.mamba.conv1d.weight")[1][1] == 1  # stored [C, 1, K]
    assert files.info("model.embed_tokens.weight")[0] == "BF16"
    assert files.info("model.layers.0.mamba.A_log")[0] == "F32"
    a_log = files.tensor("model.layers.0.mamba.A_log")
    assert a_log.min() >= 0.0 and a_log.max() <= 2.78  # log of U[1, 16]
    dt = torch.nn.functional.softplus(files.tensor("model.layers.0.mamba.dt_bias"))
    assert dt.min() > 9e-4 and dt.max() < 0.11
    assert torch.all(files.tensor("model.layers.0.mamba.D") == 1)
    assert abs(files.tensor("model.embed_tokens.weight").float().std().item() - 0.02) < 2e-3
    files.close()


def test_random_model_is_reproducible_and_seeded(tmp_path):
    d1 = write_random_model(tiny_config("A"), 0, str(tmp_path / "a"))
    d2 = write_random_model(tiny_config("A"), 0, str(tmp_path / "b"))
    d3 = write_random_model(tiny_config("A"), 1, str(tmp_path / "c"))
    d4 = write_random_model(tiny_config("A"), 0, str(tmp_path / "d"), store_dtype="float32")
    b = lambda d: open(os.path.join(d, "model.safetensors"), "rb").read()
    assert b(d1) == b(d2) and b(d1) != b(d3)
    f1, f4 = ModelFiles(d1), ModelFiles(d4)
    for k in f1.keys():  # same values whichever way they are stored
        assert torch.equal(f1.tensor(k).float(), f4.tensor(k).float())
    assert f4.info("model.embed_tokens.weight")[0] == "F32"
    f1.close(), f4.close()
    assert json.load(open(os.path.join(d1, "config.json")))["hidden_size"] == 64


def test_loading_types(tmp_path):
    d = write_random_model(tiny_config("B"), 1, str(tmp_path / "m"))
    model = _model_for(d)
    for dtype in (torch.bfloat16, torch.float32):
        t = load_tensors(d, model.param_specs(), model.ignored_names(), dtype, torch.device("cpu"))
        assert t["model.layers.0.self_attn.q_proj.weight"].dtype == dtype
        assert t["model.layers.0.mamba.A_log"].dtype == torch.float32
        assert t["model.layers.0.input_layernorm.weight"].dtype == torch.float32
        assert t["model.layers.0.mamba.conv1d.weight"].shape == (320, 3)


def test_one_error_lists_everything_wrong(tmp_path):
    d = write_random_model(tiny_config("B"), 1, str(tmp_path / "m"))
    files = ModelFiles(d)
    tensors = {k: files.tensor(k) for k in files.keys()}
    files.close()
    del tensors["model.layers.1.mamba.A_log"]
    del tensors["lm_head.weight"]
    tensors["model.layers.2.bogus.weight"] = torch.zeros(3)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 95, dtype=torch.bfloat16)
    tensors["model.layers.0.mamba.D"] = torch.zeros(6, dtype=torch.int32)
    save_file(tensors, os.path.join(d, "model.safetensors"))
    model = _model_for(d)
    with pytest.raises(WeightsError) as ei:
        load_tensors(d, model.param_specs(), model.ignored_names(), torch.float32, torch.device("cpu"))
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.mamba.A_log"]
    assert e.unexpected == ["model.layers.2.bogus.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 95), (32, 96))]
    assert e.wrong_dtype == [("model.layers.0.mamba.D", "I32")]
    msg = str(e)
    for s in ("missing (2)", "unexpected (1)", "wrong shape (1)", "is [32, 95], expected [32, 96]", "unusable dtype"):
        assert s in msg


def test_tensors_of_switched_off_options_are_tolerated(tmp_path):
    d = write_random_model(tiny_config("B"), 1, str(tmp_path / "m"))  # B: gated norm off
    files = ModelFiles(d)
    tensors = {k: files.tensor(k) for k in files.keys()}
    files.close()
    tensors["model.layers.0.mamba.norm.weight"] = torch.ones(192)
    save_file(tensors, os.path.join(d, "model.safetensors"))
    model = _model_for(d)
    load_tensors(d, model.param_specs(), model.ignored_names(), torch.float32, torch.device("cpu"))


def test_missing_weight_file(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(tiny_config("A")))
    model = _model_for(str(d))
    with pytest.raises(WeightsError, match="no readable weights"):
        load_tensors(str(d), model.param_specs(), [], torch.float32, torch.device("cpu"))


def test_tensors_nobody_asked_for_are_listed_not_refused(tmp_path, capsys):
    """The reference loads by name and never looks at the rest (src/model/falconh1_loader.cpp:27-58):
    a tied checkpoint that still carries lm_head.weight, or an exporter's extra buffer, loads."""
    cfg = tiny_config("A")  # tied embeddings
    d = write_random_model(cfg, 0, str(tmp_path / "m"))
    files = ModelFiles(d)
    tensors = {k: files.tensor(k) for k in files.keys()}
    files.close()
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    save_file(tensors, os.path.join(d, "model.safetensors"))
    model = _model_for(d)
    out = load_tensors(d, model.param_specs(), model.ignored_names(), torch.float32, torch.device("cpu"))
    assert "lm_head.weight" not in out and len(out) == len(model.param_specs())
    err = capsys.readouterr().err
    assert "2 tensors" in err and "lm_head.weight" in err and "rotary_emb.inv_freq" in err
    with pytest.raises(WeightsError) as ei:
        load_tensors(d, model.param_specs(), model.ignored_names(), torch.float32, torch.device("cpu"), strict=True)
    assert ei.value.unexpected == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert not ei.value.missing
