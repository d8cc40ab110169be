"""Helpers of the GPU tests: building a runner, replaying scripts of steps in the ways
the engine must be indifferent to, and comparing with the plain implementation."""
from __future__ import annotations

import random
from typing import Dict, Hashable, List, Sequence, Tuple

import torch

from plain.falcon_h1_plain import forward_logits

from poor_mans_mamba_b200.cache import CacheManager
from poor_mans_mamba_b200.engine import ModelRunner, StepEntry, load_model

# Largest allowed |engine - plain(float64)| on a logit.  float32: absolute.  bfloat16: as a
# fraction of the largest reference logit of the sequence (bfloat16 carries 8 bits).
F32_ATOL = 1e-5
BF16_FRAC = 0.03


def make_runner(model_dir: str, dtype: str, page_size: int = 16, num_pages: int = 64, num_slots: int = 4):
    model, cfg = load_model(model_dir, dtype, "cuda:0")
    cache = CacheManager(model.state_specs(), page_size=page_size, num_pages=num_pages, num_slots=num_slots,
                         dtype=model.dtype, device="cuda:0")
    return ModelRunner(model, cache)


def reference_logits(seqs: Sequence[Sequence[int]], weights, cfg) -> List[torch.Tensor]:
    return [forward_logits(s, weights, cfg, torch.float64) for s in seqs]


def check_rows(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, f32_frac: float = 0.0) -> float:
    """``f32_frac`` > 0 (models with rows of thousands of products, whose float32 sums differ from
    the float64 ones by more than the tiny models' absolute bound): the float32 bound is that
    fraction of the largest logit instead."""
    got = got.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    err = (got - ref).abs()
    tol = F32_ATOL if dtype == "float32" else BF16_FRAC * float(ref.abs().max())
    if dtype == "float32" and f32_frac > 0.0:
        tol = f32_frac * max(1.0, float(ref.abs().max()))
    worst = float(err.max())
    if worst > tol:
        r, c = divmod(int(err.argmax()), err.shape[1])
        first_bad = int((err.max(dim=1).values > tol).nonzero()[0])
        raise AssertionError(f"{what}: |engine - plain| = {worst:.3e} > {tol:.3e} at row {r} col {c}; "
                             f"first wrong row {first_bad} of {err.shape[0]}")
    return worst


Step = Tuple[List[Tuple[Hashable, int, int]], List[Hashable]]  # ([(seq index, start, count)], [ended seq indices])


def run_script(runner: ModelRunner, seqs: Sequence[Sequence[int]], script: Sequence[Step]) -> Dict[int, torch.Tensor]:
    """Feeds the script; wants logits at every position; returns seq index -> [len, V] logits."""
    vocab = runner.model.vocab_size
    out = {i: torch.full((len(s), vocab), float("nan"), dtype=torch.float32) for i, s in enumerate(seqs)}
    for portions, ended in script:
        if portions:
            entries = [StepEntry(("req", i), seqs[i][a:a + n], list(range(n))) for i, a, n in portions]
            logits = runner.step(entries).cpu()
            r = 0
            for i, a, n in portions:
                out[i][a:a + n] = logits[r:r + n]
                r += n
        for i in ended:
            runner.finish(("req", i))
        runner.cache.check()
    return out


# ----------------------------------------------------------------------------- ways of cutting
def script_whole(seqs) -> List[Step]:
    """Each request alone and whole."""
    return [([(i, 0, len(s))], [i]) for i, s in enumerate(seqs)]


def script_tail_one_by_one(seqs, tail: int = 32) -> List[Step]:
    """Most of it in one step, the last ``tail`` tokens one by one."""
    script: List[Step] = []
    for i, s in enumerate(seqs):
        head = max(len(s) - tail, 0)
        if head:
            script.append(([(i, 0, head)], []))
        for p in range(head, len(s)):
            script.append(([(i, p, 1)], [i] if p == len(s) - 1 else []))
    return script


def script_portions(seqs, seed: int = 0) -> List[Step]:
    """Each request alone, in portions of changing size, down to two tokens."""
    rng = random.Random(seed)
    script: List[Step] = []
    for i, s in enumerate(seqs):
        p = 0
        while p < len(s):
            n = min(len(s) - p, rng.choice([2, 2, 3, 5, 7, 13, 16, 17, 31, 33]))
            script.append(([(i, p, n)], [i] if p + n == len(s) else []))
            p += n
    return script


def script_mixed(seqs, max_live: int = 4, seed: int = 0, budget_pages=None, page_size: int = 16) -> List[Step]:
    """Up to ``max_live`` live requests; every step mixes portions of some with single tokens
    of others; some requests sit out a step.  Requests start when a slot frees, so with a
    small pool the pages (and slots) of finished requests are used again."""
    rng = random.Random(seed)
    pos = {i: 0 for i in range(len(seqs))}
    waiting = list(range(len(seqs)))
    live: List[int] = []
    script: List[Step] = []

    def pages(n):
        return (n + page_size - 1) // page_size

    if budget_pages is not None:
        assert all(pages(len(s)) <= budget_pages for s in seqs), "a sequence alone exceeds the pool"
    while waiting or live:
        # a request starts only when the pool can hold all of it beside the live ones, so the
        # script can always go on; the pool is still far smaller than all requests together
        while waiting and len(live) < max_live and (
                budget_pages is None
                or sum(pages(len(seqs[i])) for i in live) + pages(len(seqs[waiting[0]])) <= budget_pages):
            live.append(waiting.pop(0))
        portions, ended = [], []
        for i in list(live):
            if len(live) > 1 and len(portions) > 0 and rng.random() < 0.25:
                continue  # sits this step out
            rem = len(seqs[i]) - pos[i]
            # prompts advance in portions, the last quarter of every sequence token by token
            n = 1 if rem <= max(len(seqs[i]) // 4, 1) else min(rem, rng.choice([2, 3, 6, 11, 19, 40]))
            portions.append((i, pos[i], n))
            pos[i] += n
            if pos[i] == len(seqs[i]):
                ended.append(i)
                live.remove(i)
        script.append((portions, ended))
    return script
