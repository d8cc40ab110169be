"""The benchmark's own layer sizes and schedule against the plain implementation (GPU).

bench.py times Falcon-H1-0.5B layer sizes: a 2,048-token prompt step from a recorded graph,
decode at batch 8 from CUDA graphs with contexts up to 4,096, key ranges planned per context
bucket, the next layer's weights fetched ahead, the two mixers of a layer on two streams, the
tcgen05 attention and the tcgen05 gate/up product.  The tiny configurations reach none of these
at these sizes.  Here: the same layer sizes (two layers, a 4,099-word vocabulary that is no
power of two), weights made loud so that a wrong key range, a wrong page or a lost state moves
the logits, every compared row against float64.
"""
import copy
import random

import pytest
import torch

import parity_at_sizes
from model_dirs import make_loud
from plain.falcon_h1_plain import forward_logits

from poor_mans_mamba_b200.weights import ModelFiles, write_random_model

pytestmark = pytest.mark.gpu

SIZES_05B = {
    "model_type": "falcon_h1", "architectures": ["FalconH1ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 1024, "vocab_size": 4099, "intermediate_size": 2048,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64, "rope_theta": 1e11,
    "attention_bias": False, "attention_dropout": 0.0, "mlp_bias": False,
    "mamba_d_ssm": 1536, "mamba_n_heads": 24, "mamba_d_head": 64, "mamba_d_state": 128,
    "mamba_n_groups": 1, "mamba_d_conv": 4, "mamba_chunk_size": 128, "mamba_conv_bias": True,
    "mamba_proj_bias": False, "mamba_rms_norm": False, "mamba_norm_before_gate": False,
    "rms_norm_eps": 1e-5, "hidden_act": "silu", "tie_word_embeddings": False,
    "embedding_multiplier": 1.0, "lm_head_multiplier": 1.0, "attention_in_multiplier": 1.0,
    "attention_out_multiplier": 1.0, "key_multiplier": 1.0, "ssm_in_multiplier": 1.0,
    "ssm_out_multiplier": 1.0, "ssm_multipliers": [1.0] * 5, "mlp_multipliers": [1.0, 1.0],
    "bos_token_id": 1, "eos_token_id": 11, "pad_token_id": 0,
}


@pytest.fixture(scope="module")
def model_05b(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("sizes_05b"))
    cfg = copy.deepcopy(SIZES_05B)
    write_random_model(cfg, 2, d)
    make_loud(d, hidden_size=cfg["hidden_size"])
    files = ModelFiles(d)
    weights = {k: files.tensor(k).float() for k in files.keys()}
    files.close()
    return d, cfg, weights


def test_the_weights_are_loud_enough_to_show_a_fault(model_05b):
    """Losing the state-space branch, the attention branch, or the far half of the keys each moves
    the logits by more than the bfloat16 tolerance: a comparison at that tolerance can fail."""
    d, cfg, weights = model_05b
    rng = random.Random(0)
    seq = [rng.randrange(cfg["vocab_size"]) for _ in range(600)]
    ref = forward_logits(seq, weights, cfg, torch.float64)
    tol = parity_at_sizes.BF16_FRAC * float(ref.abs().max())
    for name in ("mamba.out_proj.weight", "self_attn.o_proj.weight"):
        broken = {k: (torch.zeros_like(v) if k.endswith("layers.1." + name) else v) for k, v in weights.items()}
        moved = float((forward_logits(seq, broken, cfg, torch.float64) - ref).abs().max())
        assert moved > 2 * tol, f"{name}: {moved:.3f} against a tolerance of {tol:.3f}"
    near = forward_logits(seq[300:], weights, cfg, torch.float64)   # the same last tokens without their far context
    assert float((near[-1] - ref[-1]).abs().max()) > 2 * tol


def test_bfloat16_schedule_of_the_benchmark(model_05b, monkeypatch):
    d, cfg, weights = model_05b
    from poor_mans_mamba_b200.kernels import ops as K
    calls = {"attention_tc": 0, "tc_gemm_swiglu": 0, "flash_decode_attention": 0, "l2_prefetch": 0}
    for name in calls:
        original = getattr(K, name)
        monkeypatch.setattr(K, name, lambda *a, _o=original, _n=name, **k: (calls.__setitem__(_n, calls[_n] + 1), _o(*a, **k))[1])
    summary = parity_at_sizes.run_parity(d, cfg, weights, "bfloat16")
    assert summary["rows"] >= 2 * 23 + 8 + 6 * 8
    # the prompt steps ran on the tcgen05 kernels (plain launches once, recorded once; two layers each) ...
    assert calls["attention_tc"] >= 4 and calls["tc_gemm_swiglu"] >= 4
    # ... and the decode steps on the fused decode attention with the next layer's weights fetched ahead
    assert calls["flash_decode_attention"] > 0 and calls["l2_prefetch"] > 0
    assert K.tc_gemm_status("cuda:0") == 0


def test_float32_check_path_at_the_same_sizes(model_05b):
    d, cfg, weights = model_05b
    summary = parity_at_sizes.run_parity(d, cfg, weights, "float32", prompt_len=512, contexts=(300, 517, 700, 1100),
                                         decode_steps=16, max_seq_len=1216)
    assert summary["rows"] >= 2 * 7 + 4 + 16 * 4


def test_bfloat16_agrees_with_the_float32_engine(model_05b):
    """Beside the 3 % bound against float64: the two engine paths against each other, over a
    prompt and a decoded tail.  No logit differs by more than 1.5 % of the largest one (measured:
    1.04 %), and on average they differ by less than a quarter of a percent."""
    d, cfg, weights = model_05b
    from poor_mans_mamba_b200.engine.runner import StepEntry
    from gpu_harness import make_runner
    rng = random.Random(4)
    seq = [rng.randrange(cfg["vocab_size"]) for _ in range(700)]
    outs = {}
    for dtype in ("float32", "bfloat16"):
        runner = make_runner(d, dtype, page_size=64, num_pages=16, num_slots=2)
        rows = [runner.step([StepEntry("r", seq[:680], [100, 400, 679])]).cpu().clone()]
        rows += [runner.step([StepEntry("r", [t], [0])]).cpu().clone() for t in seq[680:]]
        outs[dtype] = torch.cat(rows).double()
        runner.finish("r")
    scale = float(outs["float32"].abs().max())
    diff = (outs["bfloat16"] - outs["float32"]).abs()
    assert float(diff.max()) <= 0.015 * scale and float(diff.mean()) <= 0.0025 * scale


def test_rounded_step_graphs_serve_different_cuts(model_05b):
    """Large steps are recorded under a rounded shape (sequences padded to a power of two, tokens to
    a multiple of 64, lengths given to the parts as bounds) and replayed for every cut that rounds
    to it.  Four rounds cut the same three prompts differently; their first steps all round to
    (512 tokens, 4 sequences), their second steps (two continued prompts beside a decoding request,
    447 tokens) to (512, 4) with other rows and key bound: each shape is issued twice launch by launch (exact, then padded),
    recorded in the third round and replayed in the fourth.  Two short prompts in two portions each
    (71 and 80 tokens a step) round up to 256 tokens the same way.  Every wanted row of every round
    against float64, and the padding leaves no trace in the cache's accounting."""
    d, cfg, weights = model_05b
    from poor_mans_mamba_b200.engine.runner import StepEntry
    from gpu_harness import check_rows, make_runner
    rng = random.Random(11)
    V = cfg["vocab_size"]
    seqs = {k: [rng.randrange(V) for _ in range(n)] for k, n in (("A", 700), ("B", 520), ("C", 300), ("D", 140), ("S", 90), ("U", 61))}
    ref = {k: forward_logits(s, weights, cfg, torch.float64) for k, s in seqs.items()}
    runner = make_runner(d, "bfloat16", page_size=64, num_pages=40, num_slots=7)
    runner.enable_graphs(1024)
    assert runner.model.accepts_length_bounds(64)
    compared = 0

    def step(portions, what):
        """portions: [(name, request id, start, count, wanted places)]"""
        nonlocal compared
        entries = [StepEntry(rid, seqs[k][a:a + n], want) for k, rid, a, n, want in portions]
        logits = runner.step(entries).float().cpu()
        r = 0
        for k, rid, a, n, want in portions:
            for w in want:
                check_rows(logits[r:r + 1], ref[k][a + w:a + w + 1], "bfloat16", f"{what}: {k} at {a + w}")
                r += 1
                compared += 1
        assert r == logits.shape[0]

    runner.step([StepEntry("d", seqs["D"][:130], [])])
    cuts = [(200, 150, 120), (180, 200, 100), (250, 130, 110), (170, 170, 160)]
    for rnd, (a, b, c) in enumerate(cuts):
        ids = {k: (k, rnd) for k in "ABC"}
        want_c = [0, c // 2, c - 1] + ([7] if rnd % 2 else [])       # 9 or 10 rows: both round to 16
        step([("A", ids["A"], 0, a, [0, a // 2, a - 1]), ("B", ids["B"], 0, b, [1, b - 2, b - 1]),
              ("C", ids["C"], 0, c, want_c)], f"round {rnd} first step")
        a2, b2 = 256 + rnd, 190 - rnd
        step([("A", ids["A"], a, a2, [0, 63, a2 - 1]), ("B", ids["B"], b, b2, [b2 - 1]),
              ("D", "d", 130 + 2 * rnd, 1, [0])], f"round {rnd} second step")
        step([("A", ids["A"], a + a2, 700 - a - a2, [700 - a - a2 - 1]), ("B", ids["B"], b + b2, 520 - b - b2, [0]),
              ("C", ids["C"], c, 300 - c, [300 - c - 1])], f"round {rnd} last step")
        # short steps round up to 256 tokens: two short prompts in two portions each, the first beside the decoding request
        s1, u1 = 40 + rnd, 30 - rnd
        step([("S", ("S", rnd), 0, s1, [0, s1 - 1]), ("U", ("U", rnd), 0, u1, [u1 - 1]), ("D", "d", 131 + 2 * rnd, 1, [0])],
             f"round {rnd} short step")
        step([("S", ("S", rnd), s1, 90 - s1, [90 - s1 - 1]), ("U", ("U", rnd), u1, 61 - u1, [0, 61 - u1 - 1])],
             f"round {rnd} second short step")
        for rid in list(ids.values()) + [("S", rnd), ("U", rnd)]:
            runner.finish(rid)
        runner.cache.check()
    runner.finish("d")
    runner.check_kernels(wait=True)
    recorded = {k: v.get("graph") is not None for k, v in runner._step_graphs.items() if k[0] == "rounded"}
    # (the second steps' 448 tokens are rounded on to 512: below the largest step seen, sizes go in steps of 256)
    assert recorded.get(("rounded", 512, 4, 16, 256)) and recorded.get(("rounded", 512, 4, 8, 512)), recorded
    assert recorded.get(("rounded", 256, 4, 4, 256)), recorded
    assert runner._step_kernels_replayed > 0
    assert compared == 70 + 4 * 7
    assert runner.cache.min_free_pages() == 40 and runner.cache.free_slots == 7
