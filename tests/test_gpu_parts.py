"""Each part alone against the plain formulas, and the framework's openness: a toy mixer
with state of its own, another position encoding, layers run twice and layers that read
another layer's cache, all defined here without touching the framework's files (GPU)."""
import math

import pytest
import torch

import gpu_harness as H
from model_dirs import make_model_dir
from plain import falcon_h1_plain as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _runner_for(model, dtype, page_size=16, num_pages=32, num_slots=3):
    from poor_mans_mamba_b200.cache import CacheManager
    from poor_mans_mamba_b200.engine import ModelRunner
    cache = CacheManager(model.state_specs(), page_size=page_size, num_pages=num_pages, num_slots=num_slots,
                         dtype=dtype, device=DEV)
    return ModelRunner(model, cache)


def _random_tensors(model, seed, dtype, scale=None):
    """name -> device tensor for every declared parameter, by the random-weights rules."""
    from poor_mans_mamba_b200.weights.random_init import make_tensor
    out, plain = {}, {}
    for name, spec in model.param_specs().items():
        t = make_tensor(spec, seed, name).reshape(spec.shape)
        if scale and spec.kind == "matrix" and "embed" not in name:
            t = t * scale
        plain[name] = t.clone()
        out[name] = t.to(dtype if spec.kind == "matrix" else torch.float32).to(DEV)
    return out, plain


def _single_layer_model(mixers, ffn=None, hidden=48, vocab=50, order=None, n_layers=1, layer_specs=None):
    from poor_mans_mamba_b200.engine.model import Model
    from poor_mans_mamba_b200.parts import LayerCall, ModelSpec, PartSpec, prenorm_layer
    norm = PartSpec("rmsnorm", "norm1", {"eps": 1e-5})
    layers = layer_specs or [prenorm_layer(f"layers.{i}.", norm, tuple(mixers),
                                       PartSpec("rmsnorm", "norm2", {"eps": 1e-5}) if ffn else None, ffn)
                             for i in range(n_layers)]
    spec = ModelSpec(hidden_size=hidden, vocab_size=vocab, embedding_name="embed.weight", embedding_multiplier=1.0,
                     layers=tuple(layers), order=tuple(order or [LayerCall(i, i) for i in range(len(layers))]),
                     final_norm=PartSpec("rmsnorm", "final_norm", {"eps": 1e-5}), head_name="head.weight",
                     head_multiplier=1.0)
    return Model(spec)


def _plain_shell(tokens, w, layer_fn, n_layers=1):
    """embedding -> layers given by layer_fn(h, i) -> final norm -> head, in float64."""
    h = w["embed.weight"].double()[torch.tensor(tokens)]
    for i in range(n_layers):
        h = layer_fn(h, i)
    h = P.rms_norm(h, w["final_norm.weight"].double(), 1e-5)
    return h @ w["head.weight"].double().t()


def _two_cuttings(runner, tokens):
    from poor_mans_mamba_b200.engine import StepEntry
    n = len(tokens)
    whole = runner.step([StepEntry("w", tokens, list(range(n)))]).cpu().clone()
    runner.finish("w")
    parts, p = [], 0
    for c in [3, 1, 1, 7, 2, 1, n]:
        c = min(c, n - p)
        if c <= 0:
            break
        parts.append(runner.step([StepEntry("c", tokens[p:p + c], list(range(c)))]).cpu().clone())
        p += c
    runner.finish("c")
    return whole, torch.cat(parts)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_alone(dtype):
    """GQA with 6/3 heads of 48, theta 500, non-unit multipliers, inside a bare layer."""
    from poor_mans_mamba_b200.parts import PartSpec
    params = {"num_heads": 6, "num_kv_heads": 3, "head_dim": 48, "position_encoding": {"kind": "rotary", "theta": 500.0},
              "in_multiplier": 0.9, "out_multiplier": 1.1, "key_multiplier": 0.8}
    model = _single_layer_model([PartSpec("paged_attention", "attn", params)])
    dev, w = _random_tensors(model, 3, dtype, scale=8.0)
    model.bind(dev, dtype, DEV)
    cfg = {"num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48, "rope_theta": 500.0,
           "attention_in_multiplier": 0.9, "attention_out_multiplier": 1.1, "key_multiplier": 0.8}
    w64 = {k: v.double() for k, v in w.items()}

    def layer(h, i):
        n = P.rms_norm(h, w64["layers.0.norm1.weight"], 1e-5)
        return h + P.attention_mixer(n, w64, "layers.0.attn.", cfg)

    tokens = [int(t) for t in torch.randint(0, 50, (40,), generator=torch.Generator().manual_seed(1))]
    ref = _plain_shell(tokens, w, layer)
    whole, cut = _two_cuttings(_runner_for(model, dtype), tokens)
    name = "float32" if dtype == torch.float32 else "bfloat16"
    H.check_rows(whole, ref, name, "attention part whole")
    H.check_rows(cut, ref, name, "attention part in portions")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("variant", ["gated_groups", "norm_first_bias"])
def test_mamba2_part_alone(dtype, variant):
    from poor_mans_mamba_b200.parts import PartSpec
    gated = {"gated_groups": dict(gated_norm=True, norm_before_gate=False, proj_bias=False, conv_bias=False),
             "norm_first_bias": dict(gated_norm=True, norm_before_gate=True, proj_bias=True, conv_bias=True)}[variant]
    params = dict(n_heads=6, d_head=20, d_state=24, d_conv=5, n_groups=3, chunk_size=8, norm_eps=1e-4,
                  in_multiplier=1.2, out_multiplier=0.7, chunk_multipliers=(0.5, 1.1, 0.9, 1.3, 0.7), **gated)
    model = _single_layer_model([PartSpec("mamba2", "ssm", params)])
    dev, w = _random_tensors(model, 4, dtype, scale=8.0)
    model.bind(dev, dtype, DEV)
    cfg = {"mamba_d_ssm": 120, "mamba_n_groups": 3, "mamba_d_state": 24, "mamba_n_heads": 6, "mamba_d_head": 20,
           "ssm_multipliers": [0.5, 1.1, 0.9, 1.3, 0.7], "mamba_proj_bias": gated["proj_bias"],
           "mamba_conv_bias": gated["conv_bias"], "mamba_rms_norm": True, "rms_norm_eps": 1e-4,
           "mamba_norm_before_gate": gated["norm_before_gate"], "ssm_in_multiplier": 1.2, "ssm_out_multiplier": 0.7}
    w64 = {k: v.double() for k, v in w.items()}

    def layer(h, i):
        n = P.rms_norm(h, w64["layers.0.norm1.weight"], 1e-5)
        return h + P.mamba2_mixer(n, w64, "layers.0.ssm.", cfg)

    tokens = [int(t) for t in torch.randint(0, 50, (37,), generator=torch.Generator().manual_seed(2))]
    ref = _plain_shell(tokens, w, layer)
    whole, cut = _two_cuttings(_runner_for(model, dtype), tokens)
    name = "float32" if dtype == torch.float32 else "bfloat16"
    H.check_rows(whole, ref, name, f"mamba2 part {variant} whole")
    H.check_rows(cut, ref, name, f"mamba2 part {variant} in portions")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_and_norm_parts_alone(dtype):
    from poor_mans_mamba_b200.parts import PartSpec, build_part
    ffn = build_part("feed_forward", PartSpec("swiglu", "ff", {"intermediate_size": 112, "gate_multiplier": 1.5,
                                                               "down_multiplier": 0.4}), hidden_size=48)
    g = torch.Generator().manual_seed(5)
    w = {s.name: torch.randn(s.shape, generator=g) * 0.3 for s in ffn.param_specs()}
    ffn.bind({k: v.to(dtype).to(DEV) for k, v in w.items()})
    x = torch.randn(9, 48, generator=g).to(dtype)

    class Ctx:
        pass
    from poor_mans_mamba_b200.engine import Workspace
    ctx = Ctx()
    ctx.workspace = Workspace(DEV)
    out = torch.empty(9, 48, dtype=dtype, device=DEV)
    ffn.forward(x.to(DEV), ctx, out)
    w64 = {"ff." + k: v.to(dtype).double() for k, v in w.items()}
    ref = P.swiglu_mlp(x.double(), w64, "ff.", {"mlp_multipliers": [1.5, 1.0]})
    assert ffn.out_scale == 0.4
    err = float((out.double().cpu() - ref).abs().max())
    assert err <= (2e-5 if dtype == torch.float32 else 0.03 * float(ref.abs().max())), err

    norm = build_part("norm", PartSpec("rmsnorm", "n", {"eps": 1e-3}), width=48)
    wn = torch.randn(48, generator=g)
    norm.bind({"weight": wn.to(DEV)})
    h = torch.randn(9, 48, generator=g)
    hd, o = h.clone().to(DEV), torch.empty(9, 48, dtype=dtype, device=DEV)
    norm.forward(hd, [(out, 0.4)], o, None, ctx)
    hs = h.double() + 0.4 * out.double().cpu()
    assert float((hd.double().cpu() - hs).abs().max()) < 1e-5
    refn = P.rms_norm(hs, wn.double(), 1e-3)
    assert float((o.double().cpu() - refn).abs().max()) <= (1e-5 if dtype == torch.float32 else 0.03)


def test_rotary_table_matches_the_plain_angles():
    from poor_mans_mamba_b200.parts import PartSpec, build_part
    pe = build_part("position_encoding", PartSpec("rotary", "", {"theta": 1e11}), head_dim=64)
    pe.finalize(torch.float32, DEV)
    i = torch.arange(32, dtype=torch.float32)
    want = 1.0 / torch.pow(torch.tensor(1e11, dtype=torch.float32), 2.0 * i / 64.0)
    assert torch.equal(pe.inv_freq.cpu(), want)


# ----------------------------------------------------------------------------- openness
class RunningMeanMixer:
    """A toy mixer with per-request state of its own: the running mean of a projection of
    all tokens so far.  state = (sum [W], count [1]); out_t = (sum_{s<=t} x_s W^T) / (t+1)."""

    def __new__(cls, *a, **k):
        from poor_mans_mamba_b200.parts import Mixer

        class _Impl(Mixer):
            def __init__(self, hidden_size, width):
                self.hidden_size, self.width, self.out_scale = hidden_size, width, 0.5

            def param_specs(self):
                from poor_mans_mamba_b200.parts import ParamSpec
                return [ParamSpec("w.weight", (self.width, self.hidden_size)),
                        ParamSpec("o.weight", (self.hidden_size, self.width))]

            def state_specs(self):
                from poor_mans_mamba_b200.parts import StateSpec
                return [StateSpec.fixed("sum", (self.width,), "float32"), StateSpec.fixed("count", (1,), "float32")]

            def bind(self, params):
                self.w, self.o = params["w.weight"], params["o.weight"]

            def forward(self, x, ctx, cache, out):
                ssum, cnt = cache.fixed(f"{self.name}.sum"), cache.fixed(f"{self.name}.count")
                proj = x.float() @ self.w.float().t()
                slots = ctx.slots.tolist()
                t0 = 0
                for s, n in enumerate(ctx.new_lens):
                    run = ssum[slots[s]] + torch.cumsum(proj[t0:t0 + n], 0)
                    k = cnt[slots[s]] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                    out[t0:t0 + n] = ((run / k[:, None]) @ self.o.float().t()).to(out.dtype)
                    ssum[slots[s]] = run[-1]
                    cnt[slots[s]] += n
                    t0 += n

        return _Impl(*a, **k)


class AlibiLikeEncoding:
    """Another position encoding, applied through the generic (unfused) path: scales queries
    and keys by a position-dependent factor."""

    def __new__(cls, *a, **k):
        from poor_mans_mamba_b200.parts import PositionEncoding

        class _Impl(PositionEncoding):
            def __init__(self, head_dim, rate):
                self.rate = rate

            def apply(self, q, k, positions):
                f = (1.0 + self.rate * positions.float())[:, None, None]
                q.copy_((q.float() * f).to(q.dtype))
                if k is not None:
                    k.copy_((k.float() / f).to(k.dtype))

        return _Impl(*a, **k)


@pytest.fixture(scope="module")
def toy_registered():
    from poor_mans_mamba_b200.parts import register_mixer, register_position_encoding
    register_mixer("test_running_mean", RunningMeanMixer)
    register_position_encoding("test_scaling", AlibiLikeEncoding)


def test_toy_mixer_with_its_own_state_is_registered_built_and_stepped(toy_registered):
    from poor_mans_mamba_b200.parts import PartSpec, registered
    assert "test_running_mean" in registered("mixer")
    dtype = torch.float32
    mixers = [PartSpec("test_running_mean", "toy", {"width": 20}),
              PartSpec("paged_attention", "attn", {"num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                                   "position_encoding": {"kind": "test_scaling", "rate": 0.01}})]
    ffn = PartSpec("swiglu", "ff", {"intermediate_size": 64})
    model = _single_layer_model(mixers, ffn, n_layers=2)
    assert sorted(n for n, _ in model.state_specs()[0]) == ["attn.kv", "toy.count", "toy.sum"]
    dev, w = _random_tensors(model, 6, dtype, scale=8.0)
    model.bind(dev, dtype, DEV)
    w64 = {k: v.double() for k, v in w.items()}

    def layer(h, i):
        pre = f"layers.{i}."
        n = P.rms_norm(h, w64[pre + "norm1.weight"], 1e-5)
        t = n.shape[0]
        mean = torch.cumsum(n @ w64[pre + "toy.w.weight"].t(), 0) / torch.arange(1, t + 1, dtype=torch.float64)[:, None]
        toy = mean @ w64[pre + "toy.o.weight"].t()
        f = (1.0 + 0.01 * torch.arange(t, dtype=torch.float64))[:, None, None]
        q = (n @ w64[pre + "attn.q_proj.weight"].t()).view(t, 2, 16) * f
        k = (n @ w64[pre + "attn.k_proj.weight"].t()).view(t, 1, 16) / f
        v = (n @ w64[pre + "attn.v_proj.weight"].t()).view(t, 1, 16)
        att = P.causal_attention(q, k, v, 2).reshape(t, 32) @ w64[pre + "attn.o_proj.weight"].t()
        h = (h + 0.5 * toy) + att
        return h + P.swiglu_mlp(P.rms_norm(h, w64[pre + "norm2.weight"], 1e-5), w64, pre + "ff.", {})

    tokens = [int(t) for t in torch.randint(0, 50, (33,), generator=torch.Generator().manual_seed(7))]
    ref = _plain_shell(tokens, w, layer, n_layers=2)
    whole, cut = _two_cuttings(_runner_for(model, dtype), tokens)
    H.check_rows(whole, ref, "float32", "toy model whole")
    H.check_rows(cut, ref, "float32", "toy model in portions")


class Top1RoutedFeedForward:
    """A toy feed-forward with routing: a float32 router picks one of E small two-matrix experts
    per token; out_t = gate_t * W2[e_t] relu(W1[e_t] x_t), gate_t the softmax weight of the pick."""

    def __new__(cls, *a, **k):
        from poor_mans_mamba_b200.parts import FeedForward

        class _Impl(FeedForward):
            def __init__(self, hidden_size, experts, width):
                self.hidden_size, self.experts, self.width, self.out_scale = hidden_size, experts, width, 1.0

            def param_specs(self):
                from poor_mans_mamba_b200.parts import ParamSpec
                specs = [ParamSpec("router.weight", (self.experts, self.hidden_size))]
                for e in range(self.experts):
                    specs += [ParamSpec(f"experts.{e}.w1.weight", (self.width, self.hidden_size)),
                              ParamSpec(f"experts.{e}.w2.weight", (self.hidden_size, self.width))]
                return specs

            def bind(self, params):
                self.router = params["router.weight"]
                self.w1 = [params[f"experts.{e}.w1.weight"] for e in range(self.experts)]
                self.w2 = [params[f"experts.{e}.w2.weight"] for e in range(self.experts)]

            def forward(self, x, ctx, out):
                xf = x.float()
                prob = torch.softmax(xf @ self.router.float().t(), -1)
                gate, pick = prob.max(-1)
                res = torch.zeros_like(xf)
                for e in range(self.experts):
                    rows = (pick == e).nonzero().flatten()
                    if rows.numel():
                        hid = torch.relu(xf[rows] @ self.w1[e].float().t())
                        res[rows] = gate[rows, None] * (hid @ self.w2[e].float().t())
                out.copy_(res.to(out.dtype))

        return _Impl(*a, **k)


def test_toy_routed_feed_forward_in_one_layer_and_a_dense_one_in_the_next():
    """Feed-forwards are chosen layer by layer: a routed toy in layer 0, the dense SwiGLU in layer 1."""
    from poor_mans_mamba_b200.parts import PartSpec, prenorm_layer, register_feed_forward, registered
    register_feed_forward("test_top1_routed", Top1RoutedFeedForward)
    assert "test_top1_routed" in registered("feed_forward")
    dtype = torch.float32
    attn = PartSpec("paged_attention", "attn", {"num_heads": 3, "num_kv_heads": 1, "head_dim": 16,
                                                "position_encoding": {"kind": "rotary", "theta": 100.0}})
    norm1, norm2 = PartSpec("rmsnorm", "norm1", {"eps": 1e-5}), PartSpec("rmsnorm", "norm2", {"eps": 1e-5})
    layers = [prenorm_layer("layers.0.", norm1, (attn,), norm2,
                        PartSpec("test_top1_routed", "moe", {"experts": 3, "width": 24})),
              prenorm_layer("layers.1.", norm1, (attn,), norm2,
                        PartSpec("swiglu", "ff", {"intermediate_size": 40}))]
    model = _single_layer_model(None, layer_specs=layers)
    names = set(model.param_specs())
    assert "layers.0.moe.experts.2.w2.weight" in names and "layers.1.ff.down_proj.weight" in names
    dev, w = _random_tensors(model, 11, dtype, scale=6.0)
    model.bind(dev, dtype, DEV)
    w64 = {k: v.double() for k, v in w.items()}

    cfg = {"num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16, "rope_theta": 100.0}

    def attention(n, pre):
        return P.attention_mixer(n, w64, pre + "attn.", cfg)

    picks = []

    def layer(h, i):
        pre = f"layers.{i}."
        h = h + attention(P.rms_norm(h, w64[pre + "norm1.weight"], 1e-5), pre)
        n = P.rms_norm(h, w64[pre + "norm2.weight"], 1e-5)
        if i == 1:
            return h + P.swiglu_mlp(n, w64, pre + "ff.", {})
        prob = torch.softmax(n @ w64[pre + "moe.router.weight"].t(), -1)
        gate, pick = prob.max(-1)
        picks.append(pick)
        res = torch.zeros_like(n)
        for t in range(n.shape[0]):
            e = int(pick[t])
            hid = torch.relu(w64[pre + f"moe.experts.{e}.w1.weight"] @ n[t])
            res[t] = gate[t] * (w64[pre + f"moe.experts.{e}.w2.weight"] @ hid)
        return h + res

    tokens = [int(t) for t in torch.randint(0, 50, (29,), generator=torch.Generator().manual_seed(3))]
    ref = _plain_shell(tokens, w, layer, n_layers=2)
    assert len(set(picks[0].tolist())) >= 2, "the routing is trivial for these weights"
    whole, cut = _two_cuttings(_runner_for(model, dtype), tokens)
    H.check_rows(whole, ref, "float32", "routed toy whole")
    H.check_rows(cut, ref, "float32", "routed toy in portions")


def test_order_may_run_a_layer_twice_and_share_a_cache():
    """Order [L0 on cache 0, L1 reading cache 0's keys/values, L0 again on cache 2]."""
    from poor_mans_mamba_b200.parts import LayerCall, PartSpec, prenorm_layer
    dtype = torch.float32
    rot = {"kind": "rotary", "theta": 100.0}
    attn = {"num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "position_encoding": rot}
    n1 = PartSpec("rmsnorm", "norm1", {"eps": 1e-5})
    l0 = prenorm_layer("layers.0.", n1, (PartSpec("paged_attention", "attn", attn),))
    l1 = prenorm_layer("layers.1.", n1,
                   (PartSpec("paged_attention", "attn", dict(attn, shared_kv=True)),))
    model = _single_layer_model(None, layer_specs=[l0, l1],
                                order=[LayerCall(0, 0), LayerCall(1, 0), LayerCall(0, 2)])
    specs = model.state_specs()
    assert sorted(specs) == [0, 2] and [n for n, _ in specs[0]] == ["attn.kv"] == [n for n, _ in specs[2]]
    assert "layers.1.attn.k_proj.weight" not in model.param_specs()
    dev, w = _random_tensors(model, 8, dtype, scale=8.0)
    model.bind(dev, dtype, DEV)
    w64 = {k: v.double() for k, v in w.items()}
    tokens = [int(t) for t in torch.randint(0, 50, (29,), generator=torch.Generator().manual_seed(8))]
    t = len(tokens)
    pos = torch.arange(t)

    def attn_layer(h, pre, kv_from=None):
        n = P.rms_norm(h, w64[pre + "norm1.weight"], 1e-5)
        q = P.rope_rotate_half((n @ w64[pre + "attn.q_proj.weight"].t()).view(t, 4, 16), pos, 16, 100.0)
        if kv_from is None:
            k = P.rope_rotate_half((n @ w64[pre + "attn.k_proj.weight"].t()).view(t, 2, 16), pos, 16, 100.0)
            v = (n @ w64[pre + "attn.v_proj.weight"].t()).view(t, 2, 16)
        else:
            k, v = kv_from
        o = P.causal_attention(q, k, v, 2).reshape(t, 64) @ w64[pre + "attn.o_proj.weight"].t()
        return h + o, (k, v)

    h = w64["embed.weight"][torch.tensor(tokens)]
    h, kv0 = attn_layer(h, "layers.0.")
    h, _ = attn_layer(h, "layers.1.", kv_from=kv0)
    h, _ = attn_layer(h, "layers.0.")
    ref = P.rms_norm(h, w64["final_norm.weight"], 1e-5) @ w64["head.weight"].t()
    whole, cut = _two_cuttings(_runner_for(model, dtype), tokens)
    H.check_rows(whole, ref, "float32", "reordered layers whole")
    H.check_rows(cut, ref, "float32", "reordered layers in portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sliding_window_layers_give_pages_back(dtype, tmp_path):
    """A model whose second layer attends to a window: its pages are of a group of their own
    and return to the pool while the sequence goes on; logits match a windowed plain model."""
    from poor_mans_mamba_b200.parts import PartSpec, prenorm_layer
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    rot = {"kind": "rotary", "theta": 1000.0}
    base = {"num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "position_encoding": rot}
    n1 = PartSpec("rmsnorm", "norm1", {"eps": 1e-5})
    layers = [prenorm_layer("layers.0.", n1, (PartSpec("paged_attention", "attn", base),)),
              prenorm_layer("layers.1.", n1, (PartSpec("paged_attention", "attn", dict(base, window=20)),))]
    model = _single_layer_model(None, layer_specs=layers)
    dev, w = _random_tensors(model, 9, tdt, scale=8.0)
    model.bind(dev, tdt, DEV)
    w64 = {k: v.double() for k, v in w.items()}
    tokens = [int(t) for t in torch.randint(0, 50, (90,), generator=torch.Generator().manual_seed(9))]
    t = len(tokens)
    pos = torch.arange(t)
    h = w64["embed.weight"][torch.tensor(tokens)]
    for i, window in ((0, 0), (1, 20)):
        pre = f"layers.{i}."
        n = P.rms_norm(h, w64[pre + "norm1.weight"], 1e-5)
        q = P.rope_rotate_half((n @ w64[pre + "attn.q_proj.weight"].t()).view(t, 4, 16), pos, 16, 1000.0)
        k = P.rope_rotate_half((n @ w64[pre + "attn.k_proj.weight"].t()).view(t, 2, 16), pos, 16, 1000.0)
        v = (n @ w64[pre + "attn.v_proj.weight"].t()).view(t, 2, 16)
        if window:
            o = torch.stack([P.causal_attention(q[max(0, j - window + 1):j + 1], k[max(0, j - window + 1):j + 1],
                                                v[max(0, j - window + 1):j + 1], 2)[-1] for j in range(t)])
        else:
            o = P.causal_attention(q, k, v, 2)
        h = h + o.reshape(t, 64) @ w64[pre + "attn.o_proj.weight"].t()
    ref = P.rms_norm(h, w64["final_norm.weight"], 1e-5) @ w64["head.weight"].t()
    runner = _runner_for(model, tdt, page_size=16, num_pages=8)
    assert len(runner.cache.groups) == 2
    from poor_mans_mamba_b200.engine import StepEntry
    rows, p = [], 0
    for c in [30, 1, 1, 25, 1, 1, 1, 30]:
        rows.append(runner.step([StepEntry("r", tokens[p:p + c], list(range(c)))]).cpu().clone())
        p += c
        runner.cache.check()
    win = runner.cache.groups[(2, 32, 20)]
    assert win.pool.n_held <= 3 and runner.cache.groups[(2, 32, 0)].pool.n_held == 6
    H.check_rows(torch.cat(rows), ref, dtype, "windowed layers")


# ----------------------------------------------------------------------------- another arrangement, another feed-forward
def _squared_relu_feed_forward(*a, **k):
    """out = relu(x W1^T)^2 W2^T: not SwiGLU, with a few-token path of its own built from the
    weight-streaming operations that the framework offers to parts."""
    from poor_mans_mamba_b200.kernels import ops as K
    from poor_mans_mamba_b200.parts import FeedForward, ParamSpec, streaming

    class _Impl(FeedForward):
        def __init__(self, hidden_size, width, out_multiplier=1.0):
            self.hidden_size, self.width, self.out_scale = hidden_size, width, float(out_multiplier)

        def param_specs(self):
            return [ParamSpec("w1.weight", (self.width, self.hidden_size)),
                    ParamSpec("w2.weight", (self.hidden_size, self.width))]

        def bind(self, params):
            self.w1, self.w2 = params["w1.weight"].contiguous(), params["w2.weight"].contiguous()

        def forward(self, x, ctx, out):
            mid = ctx.workspace.alloc((x.shape[0], self.width), x.dtype)
            K.linear(x, self.w1, mid)
            mid.copy_(torch.relu(mid.float()).square().to(mid.dtype))
            K.linear(mid, self.w2, out)

        def forward_few_tokens(self, h, norm, ctx):
            if not streaming.eligible(ctx, self.hidden_size):
                return False
            _squared_relu_feed_forward.few_token_calls += 1
            mid = ctx.workspace.alloc((h.shape[0], self.width), ctx.dtype)
            streaming.normed_linear(h, norm, self.w1, mid, ctx)
            mid.copy_(torch.relu(mid.float()).square().to(mid.dtype))
            streaming.add_products(h, [(mid, self.w2, self.out_scale)], ctx)
            return True

        def streamed_weights(self):
            return [self.w1, self.w2]

    return _Impl(*a, **k)


_squared_relu_feed_forward.few_token_calls = 0


def _centered_norm(*a, **k):
    """y = (x - mean) / sqrt(var + eps) * w: a norm the streaming products cannot take into their
    prologue (rms_prologue stays None), so it is launched on its own."""
    from poor_mans_mamba_b200.parts import Norm, ParamSpec
    from poor_mans_mamba_b200.parts.norm import fold_branches

    class _Impl(Norm):
        def __init__(self, width, eps):
            self.width, self.eps = width, eps

        def param_specs(self):
            return [ParamSpec("weight", (self.width,), kind="vector", init=("ones",))]

        def bind(self, params):
            self.weight = params["weight"]

        def forward(self, h, pending, out, rows, ctx):
            if rows is None:
                fold_branches(h, pending)
                x = h
            else:
                x = h.index_select(0, rows.long())
                for branch, scale in pending:
                    x = x + scale * branch.index_select(0, rows.long()).float()
            c = x - x.mean(-1, keepdim=True)
            out.copy_((c * torch.rsqrt(c.square().mean(-1, keepdim=True) + self.eps) * self.weight).to(out.dtype))

    return _Impl(*a, **k)


def _plain_centered_norm(x, w, eps):
    c = x - x.mean(-1, keepdim=True)
    return c / torch.sqrt(c.square().mean(-1, keepdim=True) + eps) * w


def test_another_feed_forward_and_norm_take_the_few_token_path():
    """A feed-forward that is not SwiGLU, behind a norm that is not RMSNorm, in a layer of two
    parallel attention mixers: bfloat16 decode steps run it through its own few-token path (the
    arrangement asks the part, it does not test for a class), prompt portions through `forward`."""
    from poor_mans_mamba_b200.engine import StepEntry
    from poor_mans_mamba_b200.parts import PartSpec, prenorm_layer, register_feed_forward, register_norm
    register_feed_forward("test_squared_relu", _squared_relu_feed_forward)
    register_norm("test_centered", _centered_norm)
    dtype = torch.bfloat16
    attn = {"num_heads": 2, "num_kv_heads": 1, "head_dim": 32, "position_encoding": {"kind": "rotary", "theta": 100.0}}
    layers = [prenorm_layer(f"layers.{i}.", PartSpec("rmsnorm", "norm1", {"eps": 1e-5}),
                            (PartSpec("paged_attention", "attn_a", attn), PartSpec("paged_attention", "attn_b", attn)),
                            PartSpec("test_centered", "norm2", {"eps": 1e-4}),
                            PartSpec("test_squared_relu", "ff", {"width": 72, "out_multiplier": 0.5}))
              for i in range(2)]
    model = _single_layer_model(None, hidden=64, layer_specs=layers)
    dev, w = _random_tensors(model, 21, dtype, scale=6.0)
    model.bind(dev, dtype, DEV)
    w64 = {k: v.double() for k, v in w.items()}
    cfg = {"num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 32, "rope_theta": 100.0}

    def layer(h, i):
        pre = f"layers.{i}."
        n = P.rms_norm(h, w64[pre + "norm1.weight"], 1e-5)
        h = (h + P.attention_mixer(n, w64, pre + "attn_a.", cfg)) + P.attention_mixer(n, w64, pre + "attn_b.", cfg)
        f = _plain_centered_norm(h, w64[pre + "norm2.weight"], 1e-4)
        return h + 0.5 * (torch.relu(f @ w64[pre + "ff.w1.weight"].t()).square() @ w64[pre + "ff.w2.weight"].t())

    tokens = [int(t) for t in torch.randint(0, 50, (37,), generator=torch.Generator().manual_seed(5))]
    ref = _plain_shell(tokens, w, layer, n_layers=2)
    runner = _runner_for(model, dtype)
    impl = _squared_relu_feed_forward
    whole = runner.step([StepEntry("w", tokens, list(range(len(tokens))))]).cpu().clone()   # 37 tokens: also few
    runner.finish("w")
    before = impl.few_token_calls
    rows = [runner.step([StepEntry("c", tokens[:20], list(range(20)))]).cpu().clone()]
    rows += [runner.step([StepEntry("c", [t], [0])]).cpu().clone() for t in tokens[20:]]
    assert impl.few_token_calls - before == 2 * (1 + len(tokens) - 20)
    H.check_rows(whole, ref, "bfloat16", "other feed-forward whole")
    H.check_rows(torch.cat(rows), ref, "bfloat16", "other feed-forward token by token")


def _post_norm_block(spec, hidden_size):
    """h <- norm_a(h + mixer(h)); h <- norm_b(h + ffn(h)): the norms come after the residual sums.
    Described by a LayerSpec with part names of its own; nothing of the framework knows them."""
    from poor_mans_mamba_b200.parts import Part, build_part

    class _Impl(Part):
        def __init__(self):
            self.prefix = spec.prefix
            self.mixer = build_part("mixer", spec.part("mixer"), hidden_size=hidden_size)
            self.norm_a = build_part("norm", spec.part("after_mixer"), width=hidden_size)
            self.ffn = build_part("feed_forward", spec.part("ffn"), hidden_size=hidden_size)
            self.norm_b = build_part("norm", spec.part("after_ffn"), width=hidden_size)

        def parts(self):
            return [self.mixer, self.norm_a, self.ffn, self.norm_b]

        def branch_buffers_needed(self):
            return 1

        def state_specs(self):
            return [(f"{self.mixer.name}.{s.name}", s) for s in self.mixer.state_specs()]

        def finalize(self, dtype, device):
            for p in self.parts():
                p.finalize(dtype, device)

        def forward(self, stream, ctx, cache):
            for part, norm in ((self.mixer, self.norm_a), (self.ffn, self.norm_b)):
                h = stream.flush()
                out = stream.take_branch()
                x = h.to(ctx.dtype)
                if part is self.mixer:
                    part.forward(x, ctx, cache, out)
                else:
                    part.forward(x, ctx, out)
                stream.add(out, part.out_scale)
                h.copy_(stream.normed(norm))   # folds the branch in, then the stream goes on from the norm

    return _Impl()


@pytest.mark.parametrize("dtype", [torch.float32])
def test_post_norm_arrangement_described_by_named_parts(dtype):
    from poor_mans_mamba_b200.parts import LayerSpec, PartSpec, register_arrangement, registered
    register_arrangement("test_post_norm", _post_norm_block)
    assert "test_post_norm" in registered("arrangement")
    attn = {"num_heads": 3, "num_kv_heads": 3, "head_dim": 16, "position_encoding": {"kind": "rotary", "theta": 50.0}}
    layers = [LayerSpec("test_post_norm", f"layers.{i}.", {
        "mixer": PartSpec("paged_attention", "attn", attn), "after_mixer": PartSpec("rmsnorm", "ln_a", {"eps": 1e-5}),
        "ffn": PartSpec("swiglu", "ff", {"intermediate_size": 56}), "after_ffn": PartSpec("rmsnorm", "ln_b", {"eps": 1e-5})})
        for i in range(2)]
    model = _single_layer_model(None, layer_specs=layers)
    assert "layers.1.ln_b.weight" in model.param_specs()
    dev, w = _random_tensors(model, 31, dtype, scale=6.0)
    model.bind(dev, dtype, DEV)
    w64 = {k: v.double() for k, v in w.items()}
    cfg = {"num_attention_heads": 3, "num_key_value_heads": 3, "head_dim": 16, "rope_theta": 50.0}

    def layer(h, i):
        pre = f"layers.{i}."
        h = P.rms_norm(h + P.attention_mixer(h, w64, pre + "attn.", cfg), w64[pre + "ln_a.weight"], 1e-5)
        return P.rms_norm(h + P.swiglu_mlp(h, w64, pre + "ff.", {}), w64[pre + "ln_b.weight"], 1e-5)

    tokens = [int(t) for t in torch.randint(0, 50, (33,), generator=torch.Generator().manual_seed(8))]
    ref = _plain_shell(tokens, w, layer, n_layers=2)
    whole, cut = _two_cuttings(_runner_for(model, dtype), tokens)
    H.check_rows(whole, ref, "float32", "post-norm arrangement whole")
    H.check_rows(cut, ref, "float32", "post-norm arrangement in portions")
