"""The engine against the plain implementation at the benchmark's own layer sizes and schedule.

Used twice: by tests/test_gpu_bench_sizes.py and by `bench.py --check`, which runs it on the first
layers of the benchmark's model before it times anything.  The schedule is the benchmark's: a
2,048-token prompt as one step, twice (the second time the step is recorded into a CUDA graph
and replayed: tcgen05 attention, tcgen05 gate/up product, the mixers on two streams), then
decode steps of a batch whose requests sit at contexts spread up to the longest the engine
allows, through the decode graphs (key ranges planned per context bucket, the next layer's
weights fetched ahead, sampling on the device).  Every compared row is a row of float64 logits of
the plain implementation run over the whole sequence.
"""
from __future__ import annotations

import random
from typing import Dict, List, Sequence

import torch

from plain.falcon_h1_plain import forward_logits_at

BF16_FRAC = 0.03   # of the sequence's largest logit, as everywhere in the GPU tests
F32_FRAC = 2e-5    # float32: rows of 1,024..2,048 products, accumulated in a different order than the plain sum


def _tolerance(dtype: str, ref: torch.Tensor) -> float:
    return (BF16_FRAC if dtype == "bfloat16" else F32_FRAC) * max(1.0, float(ref.abs().max()))


def _compare(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, tol: float, worst: List[float]) -> None:
    got = got.detach().double().cpu()
    if got.shape != ref.shape:
        raise AssertionError(f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}")
    if not torch.isfinite(got).all():
        raise AssertionError(f"{what}: non-finite logits")
    err = float((got - ref).abs().max())
    worst.append(err / tol)
    if err > tol:
        row = int((got - ref).abs().max(dim=1).values.argmax())
        raise AssertionError(f"{what}: |engine - plain| = {err:.3e} > {tol:.3e} (row {row} of {ref.shape[0]})")


def run_parity(model_dir: str, cfg: dict, weights: Dict[str, torch.Tensor], dtype: str = "bfloat16",
               prompt_len: int = 2048, contexts: Sequence[int] = (300, 517, 1000, 1290, 2049, 2300, 3100, 4090),
               decode_steps: int = 6, max_seq_len: int = 4160, seed: int = 3) -> dict:
    """Raises AssertionError at the first row that differs beyond the tolerance; returns a summary."""
    from poor_mans_mamba_b200.engine.runner import StepEntry
    from poor_mans_mamba_b200.entry import Engine

    rng = random.Random(seed)
    vocab = cfg["vocab_size"]
    worst: List[float] = []
    rows_compared = 0
    eng = Engine(model_dir, dtype=dtype, max_tokens=(len(contexts) + 1) * (max_seq_len + 64), max_seqs=len(contexts) + 1,
                 page_size=64, max_batched_tokens=8192, max_seq_len=max_seq_len)
    runner = eng.runner

    # 1. the prompt step, twice (plain launches, then recorded and replayed)
    if prompt_len > 0:
        prompt = [rng.randrange(vocab) for _ in range(prompt_len)]
        want = sorted(set(range(0, prompt_len, 97)) | {prompt_len - 1})
        ref = forward_logits_at(prompt, weights, cfg, want, torch.float64)
        tol = _tolerance(dtype, ref)
        for turn in range(2):
            got = runner.step([StepEntry(("prompt", turn), prompt, want)])
            _compare(got, ref, dtype, f"{prompt_len}-token prompt step, turn {turn}", tol, worst)
            runner.check_kernels()
            runner.finish(("prompt", turn))
            rows_compared += len(want)

    # 2. a batch at spread contexts: prompts in one step each, then decode steps through the graphs
    seqs = [[rng.randrange(vocab) for _ in range(c + decode_steps)] for c in contexts]
    # rows c-1 .. c+decode_steps-1 of each sequence: the prompt's last position and every decoded one
    refs = [forward_logits_at(s, weights, cfg, range(c - 1, c + decode_steps), torch.float64)
            for s, c in zip(seqs, contexts)]
    tols = [_tolerance(dtype, r) for r in refs]
    reqs = [("batch", i) for i in range(len(seqs))]
    for i, (s, c) in enumerate(zip(seqs, contexts)):
        got = runner.step([StepEntry(reqs[i], s[:c], [c - 1])])
        _compare(got, refs[i][0:1], dtype, f"prompt of {c} tokens, last row", tols[i], worst)
        rows_compared += 1
    replays_before = runner.graphs.replays if runner.graphs is not None else 0
    for j in range(decode_steps):
        runner.decode_tokens(reqs, [s[c + j] for s, c in zip(seqs, contexts)])
        logits = runner.graphs.last_logits(len(reqs))
        for i, c in enumerate(contexts):
            _compare(logits[i:i + 1], refs[i][j + 1:j + 2], dtype, f"decode step {j}, request at context {c + j}",
                     tols[i], worst)
            rows_compared += 1
    runner.check_kernels(wait=True)
    if runner.graphs.replays - replays_before != decode_steps:
        raise AssertionError("the decode steps did not go through the CUDA graphs")
    for r in reqs:
        runner.finish(r)
    return {"rows": rows_compared, "worst_error_over_tolerance": round(max(worst), 4), "dtype": dtype,
            "contexts": list(contexts), "prompt_len": prompt_len, "decode_steps": decode_steps}
