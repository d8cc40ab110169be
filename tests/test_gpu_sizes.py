"""One layer each of the larger published layer shapes (head size 128, state size 256, SSM heads
of 64 and of 128, widths of 1280 and 3072), with a small odd vocabulary, against the plain
implementation: whole, with a decoded tail, and in portions (GPU).  The tiny configurations
cannot show a kernel that refuses or mishandles these shapes."""
import copy
import random

import pytest
import torch

import gpu_harness as H
from tiny_configs import TINY_B

from poor_mans_mamba_b200.weights import ModelFiles, write_random_model

pytestmark = pytest.mark.gpu


def _shape(**kw):
    cfg = copy.deepcopy(TINY_B)   # non-unit multipliers, untied head
    cfg.update({"mamba_conv_bias": True, "mamba_proj_bias": False, "mamba_rms_norm": False, "num_hidden_layers": 1,
                "rope_theta": 1e11, "rms_norm_eps": 1e-5})
    cfg.update(kw)
    return cfg


SHAPES = {
    # Falcon-H1-1.5B-Deep layer sizes
    "deep": _shape(hidden_size=1280, num_attention_heads=6, num_key_value_heads=2, head_dim=128, intermediate_size=3072,
                   vocab_size=2003, mamba_d_ssm=2560, mamba_n_heads=40, mamba_d_head=64, mamba_d_state=256,
                   mamba_n_groups=1, mamba_d_conv=4, mamba_chunk_size=256),
    # Falcon-H1-7B layer sizes
    "wide": _shape(hidden_size=3072, num_attention_heads=12, num_key_value_heads=2, head_dim=128, intermediate_size=12288,
                   vocab_size=3001, mamba_d_ssm=6144, mamba_n_heads=48, mamba_d_head=128, mamba_d_state=256,
                   mamba_n_groups=1, mamba_d_conv=4, mamba_chunk_size=256),
}


@pytest.fixture(scope="module", params=list(SHAPES))
def shaped(request, tmp_path_factory):
    name = request.param
    cfg = SHAPES[name]
    d = str(tmp_path_factory.mktemp(f"shape_{name}"))
    write_random_model(cfg, 11, d)
    from model_dirs import make_loud
    make_loud(d, hidden_size=cfg["hidden_size"])  # so that a lost state, a wrong page or rotation moves the logits
    files = ModelFiles(d)
    weights = {k: files.tensor(k).float() for k in files.keys()}
    files.close()
    rng = random.Random(5)
    seqs = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (150, 41)]
    refs = H.reference_logits(seqs, weights, cfg)
    # the comparison below can fail: without the state-space branch, or without the attention branch,
    # the logits move by far more than the bfloat16 tolerance
    tol = H.BF16_FRAC * float(refs[1].abs().max())
    for suffix in ("mamba.out_proj.weight", "self_attn.o_proj.weight"):
        broken = {k: (torch.zeros_like(v) if k.endswith(suffix) else v) for k, v in weights.items()}
        assert float((H.reference_logits(seqs[1:], broken, cfg)[0] - refs[1]).abs().max()) > 3 * tol, suffix
    return name, d, cfg, seqs, refs


@pytest.mark.parametrize("dtype,cutting", [("bfloat16", "whole"), ("bfloat16", "tail"), ("bfloat16", "portions"),
                                           ("float32", "tail")])
def test_larger_layer_shapes_agree_with_plain(shaped, dtype, cutting):
    name, d, cfg, seqs, refs = shaped
    runner = H.make_runner(d, dtype, page_size=64, num_pages=8, num_slots=2)
    script = {"whole": H.script_whole, "portions": H.script_portions,
              "tail": lambda s: H.script_tail_one_by_one(s, tail=12)}[cutting](seqs)
    out = H.run_script(runner, seqs, script)
    for i, ref in enumerate(refs):
        # float32: products over 3,072 to 12,288 terms and loud weights; the bound is 2e-5 of the largest logit
        H.check_rows(out[i], ref, dtype, f"{name} {dtype} {cutting} seq {i}", f32_frac=2e-5)


def test_decode_graph_at_larger_shapes(shaped):
    """The fused decode path (weight-streaming products, attention from the projections) and its
    CUDA graph at these widths: the logits of 12 decoded tokens, two requests a step, row by row
    against the plain implementation."""
    name, d, cfg, seqs, refs = shaped
    from poor_mans_mamba_b200.engine import StepEntry
    runner = H.make_runner(d, "bfloat16", page_size=64, num_pages=8, num_slots=2)
    runner.enable_graphs(max_seq_len=256)
    starts = [len(s) - 12 for s in seqs]
    reqs = [("r", i) for i in range(len(seqs))]
    for r, s, a in zip(reqs, seqs, starts):
        got = runner.step([StepEntry(r, s[:a], [a - 1])])
        H.check_rows(got, refs[r[1]][a - 1:a], "bfloat16", f"{name} prompt of request {r[1]}")
    for j in range(12):
        runner.decode_tokens(reqs, [s[a + j] for s, a in zip(seqs, starts)])
        logits = runner.graphs.last_logits(len(reqs)).cpu()
        for i, a in enumerate(starts):
            H.check_rows(logits[i:i + 1], refs[i][a + j:a + j + 1], "bfloat16", f"{name} decode step {j} request {i}")
    assert runner.graphs.replays == 12


def test_rounded_step_graphs_at_larger_shapes(shaped):
    """Steps recorded under a rounded shape at these widths (head size 128, state size 256): four
    rounds cut the two prompts differently into two steps each; all eight steps round to (256 tokens,
    4 sequences), so the shape is issued twice launch by launch, recorded at its third coming and
    replayed five times.  Three rows of every portion against the plain implementation."""
    name, d, cfg, seqs, refs = shaped
    from poor_mans_mamba_b200.engine import StepEntry
    runner = H.make_runner(d, "bfloat16", page_size=64, num_pages=8, num_slots=2)
    runner.enable_graphs(max_seq_len=256)
    assert runner.model.accepts_length_bounds(64)
    for rnd in range(4):
        a, b = 60 + rnd, 20 - rnd
        for what, cuts in (("first", ((0, a), (0, b))), ("second", ((a, len(seqs[0]) - a), (b, len(seqs[1]) - b)))):
            wants = [[0, n // 2, n - 1] for _, n in cuts]
            logits = runner.step([StepEntry(("r", i, rnd), seqs[i][p:p + n], w)
                                  for i, ((p, n), w) in enumerate(zip(cuts, wants))]).float().cpu()
            r = 0
            for i, ((p, n), w) in enumerate(zip(cuts, wants)):
                for k in w:
                    H.check_rows(logits[r:r + 1], refs[i][p + k:p + k + 1], "bfloat16",
                                 f"{name} round {rnd} {what} step, request {i} at {p + k}")
                    r += 1
        for i in range(2):
            runner.finish(("r", i, rnd))
        runner.cache.check()
    runner.check_kernels(wait=True)
    assert ("rounded", 256, 4, 8, 256) in runner._step_graphs, list(runner._step_graphs)
    assert runner._step_kernels_replayed > 0


# ---------------------------------------------------------------------------------------------
# A small model whose attention takes the tcgen05 kernel (head size 64, pages of 64 tokens, steps
# of 256 tokens and more).
H64 = _shape(hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=256,
             vocab_size=301, mamba_d_ssm=128, mamba_n_heads=2, mamba_d_head=64, mamba_d_state=128, mamba_n_groups=1,
             mamba_d_conv=4, mamba_chunk_size=64, num_hidden_layers=2)


@pytest.fixture(scope="module")
def h64(tmp_path_factory):
    from model_dirs import make_loud
    d = str(tmp_path_factory.mktemp("shape_h64"))
    write_random_model(H64, 13, d)
    make_loud(d)  # so that a wrong key, page or rotation moves the logits
    files = ModelFiles(d)
    weights = {k: files.tensor(k).float() for k in files.keys()}
    files.close()
    rng = random.Random(7)
    seqs = [[rng.randrange(H64["vocab_size"]) for _ in range(n)] for n in (700, 300, 521)]
    return d, seqs, H.reference_logits(seqs, weights, H64)


@pytest.mark.parametrize("cutting", ["whole", "two portions", "three requests in one step", "prefix then long portion"])
def test_prompt_steps_through_the_tcgen05_attention(h64, cutting, monkeypatch):
    d, seqs, refs = h64
    from poor_mans_mamba_b200.kernels import ops as K
    calls = []
    original = K.attention_tc
    monkeypatch.setattr(K, "attention_tc", lambda *a, **k: (calls.append(1), original(*a, **k))[1])
    runner = H.make_runner(d, "bfloat16", page_size=64, num_pages=40, num_slots=4)
    if cutting == "whole":
        script = H.script_whole(seqs)
    elif cutting == "two portions":
        script = []
        for i, s in enumerate(seqs):
            cut = min(len(s), 290 + 7 * i)
            script.append(([(i, 0, cut)], [] if cut < len(s) else [i]))
            if cut < len(s):
                script.append(([(i, cut, len(s) - cut)], [i]))
    elif cutting == "three requests in one step":
        script = [([(0, 0, 260), (1, 0, 300), (2, 0, 270)], [1]), ([(0, 260, 440), (2, 270, 251)], [0, 2])]
    else:
        script = [([(0, 0, 70)], []), ([(0, 70, 630)], [0]), ([(1, 0, 3)], []), ([(1, 3, 297)], [1]),
                  ([(2, 0, 129)], []), ([(2, 129, 392)], [2])]
    out = H.run_script(runner, seqs, script)
    for i, ref in enumerate(refs):
        H.check_rows(out[i], ref, "bfloat16", f"h64 {cutting} seq {i}")
    assert K.tc_gemm_status("cuda:0") == 0 and len(calls) >= 2 * 2  # two layers, at least two long steps


def test_steps_of_33_to_64_tokens_take_the_tcgen05_products(h64, monkeypatch):
    """Portions and mixed steps of 33..64 tokens run their SwiGLU and residual products on the
    tcgen05 weight-streaming kernel; the logits match the plain implementation all the same."""
    d, seqs, refs = h64
    from poor_mans_mamba_b200.kernels import ops as K
    calls = {"swiglu": 0, "residual": 0}
    for name in calls:
        original = getattr(K, f"skinny_tc_{name}")
        monkeypatch.setattr(K, f"skinny_tc_{name}",
                            lambda *a, _o=original, _n=name, **k: (calls.__setitem__(_n, calls[_n] + 1), _o(*a, **k))[1])
    runner = H.make_runner(d, "bfloat16", page_size=64, num_pages=40, num_slots=4)
    script = [([(0, 0, 48)], []), ([(0, 48, 64)], []), ([(0, 112, 33)], []), ([(1, 0, 30), (2, 0, 20)], []),
              ([(0, 145, 555)], [0]), ([(1, 30, 40), (2, 20, 24)], []), ([(1, 70, 230)], [1]), ([(2, 44, 477)], [2])]
    out = H.run_script(runner, seqs, script)
    for i, ref in enumerate(refs):
        H.check_rows(out[i], ref, "bfloat16", f"h64 steps of 33..64 tokens seq {i}")
    assert K.tc_gemm_status("cuda:0") == 0
    assert calls["swiglu"] == 5 * 2 and calls["residual"] == 5 * 2 * 2  # five such steps, two layers
