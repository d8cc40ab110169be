"""The plain implementation against independent restatements of each formula (no GPU)."""
import json
import math
import os
import tempfile

import pytest
import torch
import torch.nn.functional as F

from plain import falcon_h1_plain as P
from tiny_configs import TINY_WORKLOADS, tiny_config, token_sequences

from poor_mans_mamba_b200.weights import ModelFiles, write_random_model

torch.manual_seed(0)
D64 = torch.float64


def test_elementwise_helpers():
    x = torch.linspace(-30, 30, 121, dtype=D64)
    assert torch.allclose(P.silu(x), F.silu(x), atol=1e-12)
    assert torch.allclose(P.softplus(x), F.softplus(x), atol=3e-9)  # the branches at |v|>20 cost ~2e-9
    assert P.softplus(torch.tensor([25.0], dtype=D64)).item() == 25.0


def test_rms_norm():
    x, w = torch.randn(5, 12, dtype=D64), torch.randn(12, dtype=D64)
    ref = x / torch.sqrt((x ** 2).mean(-1, keepdim=True) + 1e-3) * w
    assert torch.allclose(P.rms_norm(x, w, 1e-3), ref, atol=1e-12)


def test_embedding_checks_ids():
    table = torch.randn(7, 3, dtype=D64)
    assert torch.equal(P.embedding([2, 6], table, 2.0), table[[2, 6]] * 2.0)
    with pytest.raises(ValueError, match="out of range"):
        P.embedding([7], table, 1.0)


def test_conv_matches_library_conv():
    x, w, b = torch.randn(11, 6, dtype=D64), torch.randn(6, 1, 4, dtype=D64), torch.randn(6, dtype=D64)
    ref = F.silu(F.conv1d(F.pad(x.t()[None], (3, 0)), w, b, groups=6)[0].t())
    assert torch.allclose(P.causal_conv1d_silu(x, w, b), ref, atol=1e-12)
    assert torch.allclose(P.causal_conv1d_silu(x, w.reshape(6, 4), None),
                          F.silu(F.conv1d(F.pad(x.t()[None], (3, 0)), w, None, groups=6)[0].t()), atol=1e-12)


def test_attention_matches_library_attention():
    t, hq, hkv, dh = 9, 6, 2, 8
    q, k, v = torch.randn(t, hq, dh, dtype=D64), torch.randn(t, hkv, dh, dtype=D64), torch.randn(t, hkv, dh, dtype=D64)
    kk, vv = k.repeat_interleave(3, dim=1), v.repeat_interleave(3, dim=1)
    ref = F.scaled_dot_product_attention(q.transpose(0, 1), kk.transpose(0, 1), vv.transpose(0, 1), is_causal=True)
    assert torch.allclose(P.causal_attention(q, k, v, 3), ref.transpose(0, 1), atol=1e-12)


def test_rope_is_a_rotation_that_depends_on_relative_position():
    dh = 16
    q, k = torch.randn(1, 1, dh, dtype=D64), torch.randn(1, 1, dh, dtype=D64)

    def dot(pq, pk):
        a = P.rope_rotate_half(q, torch.tensor([pq]), dh, 1e4)
        b = P.rope_rotate_half(k, torch.tensor([pk]), dh, 1e4)
        return float((a * b).sum())

    assert abs(dot(5, 2) - dot(40, 37)) < 1e-4  # float32 angles
    r = P.rope_rotate_half(q, torch.tensor([9]), dh, 1e4)
    assert abs(float(r.norm()) - float(q.norm())) < 1e-12
    assert torch.equal(P.rope_rotate_half(q, torch.tensor([0]), dh, 1e4), q)
    # element i pairs with i + Dh/2 and turns by pos * theta^(-2i/Dh)
    ang = 3 * 1e4 ** (-2 * 2 / dh)
    r3 = P.rope_rotate_half(q, torch.tensor([3]), dh, 1e4)[0, 0]
    assert abs(float(r3[2]) - float(q[0, 0, 2] * math.cos(ang) - q[0, 0, 10] * math.sin(ang))) < 1e-6


def test_recurrence_matches_the_chunked_closed_form():
    t, h, p, g, n = 13, 4, 3, 2, 5
    x, b, c = torch.randn(t, h, p, dtype=D64), torch.randn(t, g, n, dtype=D64), torch.randn(t, g, n, dtype=D64)
    dt, a_log, d, dtb = torch.randn(t, h, dtype=D64), torch.rand(h, dtype=D64), torch.randn(h, dtype=D64), torch.randn(h, dtype=D64)
    y = P.ssm_recurrence(x, b, c, dt, a_log, d, dtb)
    delta = F.softplus(dt + dtb)
    a = delta * -torch.exp(a_log)  # [T, H]
    cs = torch.cumsum(a, 0)
    ref = torch.zeros_like(y)
    for hh in range(h):
        gg = hh // (h // g)
        decay = torch.exp(cs[:, None, hh] - cs[None, :, hh]).tril()  # [t, s]
        m = (c[:, gg] @ b[:, gg].t()) * decay * delta[None, :, hh]
        ref[:, hh] = m @ x[:, hh] + d[hh] * x[:, hh]
    assert torch.allclose(y, ref, atol=1e-10)


def test_gate_and_norm_variants():
    y, z, w = torch.randn(4, 12, dtype=D64), torch.randn(4, 12, dtype=D64), torch.randn(12, dtype=D64)
    assert torch.allclose(P.gate_and_norm(y, z, None, 1e-5, 1, False), y * F.silu(z))
    v = y * F.silu(z)
    one = v / torch.sqrt((v ** 2).mean(-1, keepdim=True) + 1e-5) * w
    assert torch.allclose(P.gate_and_norm(y, z, w, 1e-5, 1, False), one)
    vg = v.view(4, 3, 4)
    grp = (vg / torch.sqrt((vg ** 2).mean(-1, keepdim=True) + 1e-5)).view(4, 12) * w
    assert torch.allclose(P.gate_and_norm(y, z, w, 1e-5, 3, False), grp)
    yg = y.view(4, 3, 4)
    before = (yg / torch.sqrt((yg ** 2).mean(-1, keepdim=True) + 1e-5)).view(4, 12) * w * F.silu(z)
    assert torch.allclose(P.gate_and_norm(y, z, w, 1e-5, 3, True), before)


def _weights(which):
    cfg = tiny_config(which)
    with tempfile.TemporaryDirectory() as d:
        write_random_model(cfg, TINY_WORKLOADS[which][0], d)
        files = ModelFiles(d)
        w = {k: files.tensor(k).float() for k in files.keys()}
        files.close()
    return cfg, w


@pytest.mark.parametrize("which", ["A", "B"])
def test_whole_model_is_causal_and_matches_its_golden_numbers(which):
    cfg, w = _weights(which)
    gold = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "plain_tiny.json")))[which]
    seq = token_sequences(which)[-1]
    assert seq == gold["tokens"]
    full = P.forward_logits(seq, w, cfg, D64)
    half = P.forward_logits(seq[:len(seq) // 2 + 1], w, cfg, D64)
    assert torch.allclose(full[:len(seq) // 2 + 1], half, atol=1e-12)  # later tokens change nothing earlier
    for p, row in zip(gold["positions"], gold["first8"]):
        assert torch.allclose(full[p, :8], torch.tensor(row, dtype=D64), atol=1e-7)
    assert [int(full[p].argmax()) for p in range(len(seq))] == gold["argmax"]
    f32 = P.forward_logits(seq, w, cfg, torch.float32)
    assert (f32.double() - full).abs().max() < 2e-5


def test_multipliers_and_biases_act_where_the_formulas_say():
    cfg, w = _weights("B")
    seq = token_sequences("B")[1]
    base = P.forward_logits(seq, w, cfg, D64)
    c2 = dict(cfg, lm_head_multiplier=cfg["lm_head_multiplier"] * 2)
    assert torch.allclose(P.forward_logits(seq, w, c2, D64), base * 2, atol=1e-12)
    for key in ("key_multiplier", "ssm_in_multiplier", "attention_out_multiplier", "embedding_multiplier"):
        c3 = dict(cfg, **{key: cfg[key] * 1.5})
        assert (P.forward_logits(seq, w, c3, D64) - base).abs().max() > 1e-6, key
    for i in range(5):
        m = list(cfg["ssm_multipliers"]); m[i] *= 1.5
        assert (P.forward_logits(seq, w, dict(cfg, ssm_multipliers=m), D64) - base).abs().max() > 1e-10, i
    w2 = dict(w); w2["model.layers.0.mamba.in_proj.bias"] = w["model.layers.0.mamba.in_proj.bias"] + 0.1
    assert (P.forward_logits(seq, w2, cfg, D64) - base).abs().max() > 1e-6


def test_greedy_generation_extends_the_sequence():
    cfg, w = _weights("A")
    out = P.greedy_generate([3, 9, 27], 4, w, cfg, D64)
    seq = [3, 9, 27]
    for t in out:
        assert t == int(P.forward_logits(seq, w, cfg, D64)[-1].argmax())
        seq.append(t)
