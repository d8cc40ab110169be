"""Plain, slow Falcon-H1 forward pass: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the package: it
reads ``config.json`` keys from a plain dict, takes weights as a ``name -> tensor``
dict, and runs every formula directly on the CPU in one floating-point type
(float64 by default, float32 on request).

It is written from the formulas of AlterHoodie/poor_mans_mamba (file:line cited at every
function, paths inside that project).  That project's CPU model code cannot be compiled
offline (it needs Eigen, nlohmann_json and safetensors-cpp, fetched from the network by its
CMake build), but its CUDA path needs only nvcc and cuBLAS: tests/golden/reference_cuda_tiny.json
holds logits computed by that unmodified code on a B200 (tests/golden/make_reference_golden.py),
tests/test_reference_golden.py compares this file with them on the CPU, and
tests/test_gpu_reference_anchor.py runs the reference's binaries again on the GPU.  The
reference's Falcon-H1 runner has neither projection biases nor the gated mixer norm; for those
two options the definition written here is the one the engine is held to.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------- helpers
def silu(x: Tensor) -> Tensor:
    """x / (1 + exp(-x)) -- include/ops/cpu/element_wise.h:86."""
    return x / (1.0 + torch.exp(-x))


def softplus(x: Tensor) -> Tensor:
    """v if v>20; exp(v) if v<-20; log1p(exp(v)) -- include/ops/cpu/element_wise.h:88-94."""
    mid = torch.log1p(torch.exp(torch.clamp(x, -20.0, 20.0)))
    return torch.where(x > 20.0, x, torch.where(x < -20.0, torch.exp(x), mid))


def linear(x: Tensor, w: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """y = x W^T with W stored [out, in] -- src/ops/cpu/linear.cpp:30-42 (no bias there)."""
    y = x @ w.t()
    return y if bias is None else y + bias


# --------------------------------------------------------------------------- parts
def embedding(tokens: Sequence[int], table: Tensor, multiplier: float) -> Tensor:
    """h[t] = multiplier * E[tok[t]] -- src/runtime/runner/falconh1_runner.cpp:129-152,
    src/ops/gpu/embed.cu:5-16.  Ids outside [0, V) are an error (cuda_backend.cu:205-209)."""
    v = table.shape[0]
    for t in tokens:
        if not 0 <= int(t) < v:
            raise ValueError("token id out of range")
    idx = torch.tensor(list(tokens), dtype=torch.long)
    return table[idx] * multiplier


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """x * 1/sqrt(mean(x^2) + eps) * w, mean over the last dim, eps inside the root --
    src/ops/cpu/rms_norm.cpp:11-16."""
    mean_sq = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(mean_sq + eps)) * weight


def rope_rotate_half(x: Tensor, positions: Tensor, head_dim: int, theta: float) -> Tensor:
    """Rotate-half RoPE on x[T, heads, Dh] at absolute positions --
    src/ops/cpu_backend.cpp:14-46.  inv_freq and the angle are float32 values there
    (theta is parsed as float32, the position is converted to float32); the same
    float32 rounding of inv_freq and of the angle is reproduced here and only then
    widened, so the angles are the reference's."""
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    theta32 = torch.tensor(theta, dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(theta32, (2.0 * i) / float(head_dim))  # float32
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]  # float32 [T, half]
    c = torch.cos(ang.to(x.dtype))[:, None, :]
    s = torch.sin(ang.to(x.dtype))[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def causal_attention(q: Tensor, k: Tensor, v: Tensor, n_rep: int) -> Tensor:
    """q[T,Hq,Dh], k/v[T,Hkv,Dh] (whole sequence from position 0): for query t and keys
    s <= t, sc = (q.k)/sqrt(Dh); p = exp(sc-max)/sum; o = sum p v; query head hq uses kv
    head hq // n_rep -- src/ops/cpu_backend.cpp:145-195."""
    t_len, hq, dh = q.shape
    scale = 1.0 / math.sqrt(float(dh))
    out = torch.zeros_like(q)
    for h in range(hq):
        hk = h // n_rep
        sc = (q[:, h, :] @ k[:, hk, :].t()) * scale  # [T, T]
        mask = torch.ones(t_len, t_len, dtype=torch.bool).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        m = sc.max(dim=-1, keepdim=True).values
        e = torch.exp(sc - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, hk, :]
    return out


def attention_mixer(n: Tensor, w: Dict[str, Tensor], prefix: str, cfg: dict) -> Tensor:
    """GQA attention with RoPE over a whole sequence starting at position 0 --
    src/ops/cpu_backend.cpp:48-202 and src/runtime/runner/falconh1_runner.cpp:66-101:
    a_in = n*attention_in_multiplier; Q,K,V projections; K *= key_multiplier (before
    RoPE); RoPE on Q and K; causal softmax attention; o_proj; * attention_out_multiplier."""
    hq, hkv, dh = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    t_len = n.shape[0]
    a_in = n * cfg.get("attention_in_multiplier", 1.0)
    q = linear(a_in, w[prefix + "q_proj.weight"]).view(t_len, hq, dh)
    k = linear(a_in, w[prefix + "k_proj.weight"]).view(t_len, hkv, dh)
    v = linear(a_in, w[prefix + "v_proj.weight"]).view(t_len, hkv, dh)
    k = k * cfg.get("key_multiplier", 1.0)
    pos = torch.arange(t_len)
    theta = cfg.get("rope_theta", 10000.0)
    q = rope_rotate_half(q, pos, dh, theta)
    k = rope_rotate_half(k, pos, dh, theta)
    o = causal_attention(q, k, v, hq // hkv).reshape(t_len, hq * dh)
    return linear(o, w[prefix + "o_proj.weight"]) * cfg.get("attention_out_multiplier", 1.0)


def causal_conv1d_silu(x: Tensor, weight: Tensor, bias: Optional[Tensor]) -> Tensor:
    """Depthwise causal conv over time with a zero history, then SiLU:
    a[t,c] = bias[c] + sum_k w[c,k] * x[t-(K-1)+k, c]; y = silu(a) --
    src/ops/cpu_backend.cpp:250-284 (window = previous K-1 inputs, oldest first)."""
    t_len, c = x.shape
    k = weight.shape[-1]
    w = weight.reshape(c, k)
    xp = torch.cat([torch.zeros(k - 1, c, dtype=x.dtype), x], dim=0)
    acc = torch.zeros(t_len, c, dtype=x.dtype) if bias is None else bias.expand(t_len, c).clone()
    for j in range(k):
        acc = acc + xp[j:j + t_len, :] * w[:, j]
    return silu(acc)


def ssm_recurrence(x: Tensor, b: Tensor, c: Tensor, dt: Tensor, a_log: Tensor, d_skip: Tensor,
                   dt_bias: Tensor) -> Tensor:
    """The Mamba2 recurrence, token by token, zero initial state --
    src/ops/cpu_backend.cpp:204-248.  x[T,H,P], b/c[T,G,N], dt[T,H].
    delta = softplus(dt + dt_bias); dA = exp(delta * -exp(A_log));
    s = s*dA + delta*B*x; y = sum_n s*C + D*x (y uses the updated state);
    head h reads group h // (H/G)."""
    t_len, h, p = x.shape
    g, n = b.shape[1], b.shape[2]
    hpg = h // g
    state = torch.zeros(h, p, n, dtype=x.dtype)
    y = torch.zeros_like(x)
    a = -torch.exp(a_log)  # [H]
    grp = torch.arange(h) // hpg
    for t in range(t_len):
        delta = softplus(dt[t] + dt_bias)  # [H]
        da = torch.exp(delta * a)  # [H]
        bt = b[t][grp]  # [H, N]
        ct = c[t][grp]
        state = state * da[:, None, None] + (delta[:, None, None] * bt[:, None, :]) * x[t][:, :, None]
        y[t] = (state * ct[:, None, :]).sum(-1) + d_skip[:, None] * x[t]
    return y


def gate_and_norm(y: Tensor, z: Tensor, norm_weight: Optional[Tensor], eps: float, n_groups: int,
                  norm_before_gate: bool) -> Tensor:
    """Without a norm weight: y * silu(z) (src/ops/cpu_backend.cpp:475-481).  With one:
    rmsnorm(y * silu(z)) (src/ops/cpu_backend.cpp:286-304), or rmsnorm(y) * silu(z) when
    norm_before_gate.  The norm runs over each of the n_groups groups of I/G channels;
    with one group that is the reference's whole-row norm."""
    if norm_weight is None:
        return y * silu(z)
    t_len, width = y.shape

    def grouped(vv: Tensor) -> Tensor:
        vg = vv.view(t_len, n_groups, width // n_groups)
        ms = (vg * vg).mean(dim=-1, keepdim=True)
        return (vg * (1.0 / torch.sqrt(ms + eps))).view(t_len, width) * norm_weight

    if norm_before_gate:
        return grouped(y) * silu(z)
    return grouped(y * silu(z))


def mamba2_mixer(n: Tensor, w: Dict[str, Tensor], prefix: str, cfg: dict) -> Tensor:
    """Mamba2 mixer over a whole sequence -- src/ops/cpu_backend.cpp:306-492 and
    src/runtime/runner/falconh1_runner.cpp:50-64.  u = n*ssm_in_multiplier;
    Pj = u W_in^T (+ in_proj.bias when mamba_proj_bias); columns [z:I][x:I][B:GN][C:GN][dt:H]
    times ssm_multipliers[0..4]; conv+SiLU over [x,B,C]; recurrence; gate/norm;
    out_proj (+ out_proj.bias); * ssm_out_multiplier."""
    i_dim = cfg["mamba_d_ssm"]
    g, st, h, p = cfg["mamba_n_groups"], cfg["mamba_d_state"], cfg["mamba_n_heads"], cfg["mamba_d_head"]
    gn = g * st
    t_len = n.shape[0]
    m = cfg.get("ssm_multipliers", [1.0] * 5)
    proj_bias = cfg.get("mamba_proj_bias", False)
    u = n * cfg.get("ssm_in_multiplier", 1.0)
    pj = linear(u, w[prefix + "in_proj.weight"], w[prefix + "in_proj.bias"] if proj_bias else None)
    z = pj[:, :i_dim] * m[0]
    xbc = torch.cat([pj[:, i_dim:2 * i_dim] * m[1],
                     pj[:, 2 * i_dim:2 * i_dim + gn] * m[2],
                     pj[:, 2 * i_dim + gn:2 * i_dim + 2 * gn] * m[3]], dim=-1)
    dt = pj[:, 2 * i_dim + 2 * gn:] * m[4]
    conv_bias = w[prefix + "conv1d.bias"] if cfg.get("mamba_conv_bias", True) else None
    xbc = causal_conv1d_silu(xbc, w[prefix + "conv1d.weight"], conv_bias)
    x = xbc[:, :i_dim].reshape(t_len, h, p)
    b = xbc[:, i_dim:i_dim + gn].reshape(t_len, g, st)
    c = xbc[:, i_dim + gn:].reshape(t_len, g, st)
    y = ssm_recurrence(x, b, c, dt, w[prefix + "A_log"], w[prefix + "D"], w[prefix + "dt_bias"])
    y = y.reshape(t_len, i_dim)
    norm_w = w[prefix + "norm.weight"] if cfg.get("mamba_rms_norm", False) else None
    y = gate_and_norm(y, z, norm_w, cfg.get("rms_norm_eps", 1e-5), g,
                      cfg.get("mamba_norm_before_gate", False))
    out = linear(y, w[prefix + "out_proj.weight"], w[prefix + "out_proj.bias"] if proj_bias else None)
    return out * cfg.get("ssm_out_multiplier", 1.0)


def swiglu_mlp(f: Tensor, w: Dict[str, Tensor], prefix: str, cfg: dict) -> Tensor:
    """g = (f Wg^T)*mlp_multipliers[0]; u = f Wu^T; ((silu(g)*u) Wd^T)*mlp_multipliers[1] --
    src/ops/cpu_backend.cpp:494-531."""
    mm = cfg.get("mlp_multipliers", [1.0, 1.0])
    gate = linear(f, w[prefix + "gate_proj.weight"]) * mm[0]
    up = linear(f, w[prefix + "up_proj.weight"])
    return linear(silu(gate) * up, w[prefix + "down_proj.weight"]) * mm[1]


def decoder_block(h: Tensor, w: Dict[str, Tensor], layer: int, cfg: dict) -> Tensor:
    """One parallel-hybrid block -- src/runtime/runner/falconh1_runner.cpp:20-127: one
    pre-norm feeds the mixer and the attention; h = (h + mamba) + attn; then
    h += mlp(rmsnorm(h))."""
    pre = f"model.layers.{layer}."
    eps = cfg.get("rms_norm_eps", 1e-5)
    n = rms_norm(h, w[pre + "input_layernorm.weight"], eps)
    m_out = mamba2_mixer(n, w, pre + "mamba.", cfg)
    a_out = attention_mixer(n, w, pre + "self_attn.", cfg)
    h = (h + m_out) + a_out
    f = rms_norm(h, w[pre + "pre_ff_layernorm.weight"], eps)
    return h + swiglu_mlp(f, w, pre + "feed_forward.", cfg)


def forward_logits(tokens: Sequence[int], weights: Dict[str, Tensor], cfg: dict,
                   dtype: torch.dtype = torch.float64) -> Tensor:
    """Logits [T, V] at every position of one whole sequence --
    src/runtime/runner/falconh1_runner.cpp:202-228 (which keeps only the last row):
    embed, L blocks, final norm, lm_head (the embedding table when tied), * lm_head_multiplier."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    h = embedding(tokens, w["model.embed_tokens.weight"], cfg.get("embedding_multiplier", 1.0))
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_block(h, w, layer, cfg)
    h = rms_norm(h, w["model.final_layernorm.weight"], cfg.get("rms_norm_eps", 1e-5))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(h, head) * cfg.get("lm_head_multiplier", 1.0)


def forward_logits_at(tokens: Sequence[int], weights: Dict[str, Tensor], cfg: dict, rows: Sequence[int],
                      dtype: torch.dtype = torch.float64) -> Tensor:
    """The rows ``rows`` of `forward_logits` without forming the others: the same blocks over the
    whole sequence, final norm and head on the chosen positions only (the reference keeps one row,
    src/runtime/runner/falconh1_runner.cpp:154-214).  For vocabularies where [T, V] is too large."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    h = embedding(tokens, w["model.embed_tokens.weight"], cfg.get("embedding_multiplier", 1.0))
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_block(h, w, layer, cfg)
    h = rms_norm(h[torch.tensor(list(rows), dtype=torch.long)], w["model.final_layernorm.weight"],
                 cfg.get("rms_norm_eps", 1e-5))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(h, head) * cfg.get("lm_head_multiplier", 1.0)


def greedy_generate(prompt: Sequence[int], n_new: int, weights: Dict[str, Tensor], cfg: dict,
                    dtype: torch.dtype = torch.float64) -> List[int]:
    """Greedy continuation by re-running the whole sequence each step; the first index wins
    ties -- src/runtime/worker.cpp:30-59."""
    seq = list(prompt)
    out: List[int] = []
    for _ in range(n_new):
        logits = forward_logits(seq, weights, cfg, dtype)[-1]
        tok = int(torch.argmax(logits).item())  # torch.argmax returns the first maximal index on CPU
        out.append(tok)
        seq.append(tok)
    return out
