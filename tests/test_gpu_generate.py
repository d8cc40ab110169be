"""Generation through the Python entry point and the command line (GPU)."""
import os
import subprocess
import sys

import pytest
import torch

from model_dirs import make_model_dir
from plain.falcon_h1_plain import forward_logits, greedy_generate
from tiny_configs import token_sequences

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module", params=["A", "B"])
def case(request, tmp_path_factory):
    which = request.param
    d, cfg, weights = make_model_dir(which, str(tmp_path_factory.mktemp(f"gen{which}")))
    return which, d, cfg, weights


def prompts_of(which):
    from tiny_configs import TINY_WORKLOADS
    _, lens, n_dec = TINY_WORKLOADS[which]
    return [s[:n] for s, n in zip(token_sequences(which), lens)], n_dec


def test_greedy_generation_matches_plain(case):
    from poor_mans_mamba_b200.entry import Engine
    which, d, cfg, weights = case
    prompts, n_dec = prompts_of(which)
    want = [greedy_generate(p, n_dec, weights, cfg) for p in prompts]
    eng = Engine(d, dtype="float32", max_tokens=1024, max_seqs=4, page_size=16, max_batched_tokens=24)
    got = eng.generate(prompts, max_new_tokens=n_dec, eos_token_id=-1)
    assert got == want
    assert eng.cache.free_slots == 4 and eng.cache.min_free_pages() == 64
    # bfloat16: same tokens except where the two best logits are closer than its rounding
    eng16 = Engine(d, dtype="bfloat16", max_tokens=1024, max_seqs=4, page_size=16, max_batched_tokens=24)
    got16 = eng16.generate(prompts, max_new_tokens=n_dec, eos_token_id=-1)
    for p, g16, w in zip(prompts, got16, want):
        for j, (a, b) in enumerate(zip(g16, w)):
            if a != b:
                logits = forward_logits(p + w[:j], weights, cfg)[-1]
                top = torch.topk(logits, 2).values
                assert float(top[0] - top[1]) < 0.03 * float(logits.abs().max()), (which, j, a, b)
                break


def test_stop_token_and_poll(case):
    from poor_mans_mamba_b200.engine.scheduler import SamplingParams
    from poor_mans_mamba_b200.entry import Engine
    which, d, cfg, weights = case
    prompts, _ = prompts_of(which)
    want = greedy_generate(prompts[1], 6, weights, cfg)
    eng = Engine(d, dtype="float32", max_tokens=512, max_seqs=2, page_size=16)
    rid = eng.submit(prompts[1], SamplingParams(max_new_tokens=20, eos_id=want[3]))
    assert eng.poll(rid).done is False
    while eng.has_work():
        eng.step()
    r = eng.poll(rid)
    stop = want.index(want[3])
    assert r.done and r.status == "done" and r.tokens == want[:stop + 1]  # the stop token is kept
    with pytest.raises(ValueError, match="out of range"):
        eng.submit([cfg["vocab_size"] + 1])


def test_preemption_on_the_device_gives_the_same_tokens(case):
    """A pool too small for all requests at once: some are preempted and recomputed."""
    from poor_mans_mamba_b200.entry import Engine
    which, d, cfg, weights = case
    prompts, _ = prompts_of(which)
    prompts = prompts[:3]
    n_new = 40
    calm = Engine(d, dtype="float32", max_tokens=4096, max_seqs=4, page_size=16).generate(
        prompts, max_new_tokens=n_new, eos_token_id=-1)
    tight = Engine(d, dtype="float32", max_tokens=16 * 8, max_seqs=4, page_size=16)
    got = tight.generate(prompts, max_new_tokens=n_new, eos_token_id=-1)
    assert tight.scheduler.counters["preemptions"] > 0
    assert got == calm
    tight.cache.check()


def test_temperature_sampling_is_seeded_and_independent_of_batching(case):
    from poor_mans_mamba_b200.entry import Engine
    which, d, cfg, weights = case
    prompts, _ = prompts_of(which)
    eng = Engine(d, dtype="float32", max_tokens=1024, max_seqs=4, page_size=16)
    a = eng.generate(prompts, max_new_tokens=10, temperature=1.5, seed=7, eos_token_id=-1)
    b = eng.generate(prompts, max_new_tokens=10, temperature=1.5, seed=7, eos_token_id=-1)
    c = eng.generate(prompts, max_new_tokens=10, temperature=1.5, seed=8, eos_token_id=-1)
    alone = eng.generate(prompts[:1], max_new_tokens=10, temperature=1.5, seed=7, eos_token_id=-1)
    greedy = eng.generate(prompts, max_new_tokens=10, temperature=0.0, eos_token_id=-1)
    assert a == b and a != c and a != greedy and alone[0] == a[0]


def test_command_line(case):
    which, d, cfg, weights = case
    want = greedy_generate([5, 9, 2], 5, weights, cfg)
    proc = subprocess.run([sys.executable, "-m", "poor_mans_mamba_b200", d, "256", "GPU", "1", "2", "5",
                           "--dtype", "float32", "--prompt-ids", "5,9,2"], cwd=ROOT, capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("req_id=")]
    assert len(lines) == 2 and all(f"tokens={want}" in l for l in lines), proc.stdout
    # the cache geometry from the command line: a pool of 4 pages of 16 tokens, one request alive at
    # a time, at most 6 tokens of context each (3 prompt tokens + 3 fed back: 4 tokens come out)
    proc = subprocess.run([sys.executable, "-m", "poor_mans_mamba_b200", d, "256", "GPU", "1", "2", "5",
                           "--dtype", "float32", "--prompt-ids", "5,9,2", "--page-size", "16", "--num-pages", "4",
                           "--max-seqs", "1", "--max-seq-len", "6", "--max-batched-tokens", "2"], cwd=ROOT,
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("req_id=")]
    assert len(lines) == 2 and all(f"status=max_seq tokens={want[:4]}" in l for l in lines), proc.stdout
    bad = subprocess.run([sys.executable, "-m", "poor_mans_mamba_b200", d, "256", "CPU"], cwd=ROOT,
                         capture_output=True, text=True, timeout=120)
    assert bad.returncode == 1 and "no CPU path" in bad.stderr


def test_smoke_entry():
    sys.path.insert(0, ROOT)
    import __graft_entry__
    __graft_entry__.smoke()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_one_step_ahead_gives_the_same_tokens(case, dtype):
    """The decode path launches a step before the previous one's ids have reached the host: greedy
    and sampled outputs, stop tokens (seen a step late), requests of different lengths and a poll in
    the middle all equal the step-by-step engine."""
    from poor_mans_mamba_b200.engine.scheduler import SamplingParams
    from poor_mans_mamba_b200.entry import Engine
    which, d, cfg, weights = case
    prompts, _ = prompts_of(which)

    def run(run_ahead, params, poll_at=None):
        eng = Engine(d, dtype=dtype, max_tokens=2048, max_seqs=4, page_size=16, run_ahead=run_ahead)
        ids = [eng.submit(p, sp) for p, sp in zip(prompts, params)]
        n = 0
        while eng.has_work():
            eng.step()
            n += 1
            if poll_at is not None and n == poll_at:
                assert all(-1 not in eng.poll(i).tokens for i in ids)
        out = [eng.poll(i) for i in ids]
        assert eng.cache.free_slots == 4 and eng.cache.min_free_pages() == eng.cache.groups[next(iter(eng.cache.groups))].num_pages
        return [(r.tokens, r.status) for r in out], eng

    lens = [24, 9, 17, 30][:len(prompts)]
    greedy = [SamplingParams(max_new_tokens=n, eos_id=-1) for n in lens]
    base, _ = run(False, greedy)
    ahead, eng = run(True, greedy)
    assert ahead == base and eng.runner.graphs.replays > 0
    assert run(True, greedy, poll_at=7)[0] == base
    # stop tokens taken from the free-running outputs: in the middle of one request, at the end of another
    stops = [base[0][0][len(base[0][0]) // 2], -1, base[2][0][-1] if len(base) > 2 else -1, -1][:len(prompts)]
    with_stop = [SamplingParams(max_new_tokens=n, eos_id=e) for n, e in zip(lens, stops)]
    assert run(True, with_stop)[0] == run(False, with_stop)[0]
    sampled = [SamplingParams(max_new_tokens=n, eos_id=-1, temperature=0.8, seed=5 + i) for i, n in enumerate(lens)]
    assert run(True, sampled)[0] == run(False, sampled)[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_max_seq_len_ends_a_request_in_the_middle_of_decoding(case, dtype):
    """One of three requests reaches max_seq_len while the engine runs a step ahead of the host: it
    ends with what it has (status max_seq), the others go on, the tokens equal the step-by-step
    engine's, and nothing the graph decoder kept for a request outlives it."""
    from poor_mans_mamba_b200.engine.scheduler import SamplingParams
    from poor_mans_mamba_b200.entry import Engine
    which, d, cfg, weights = case
    prompts, _ = prompts_of(which)
    prompts = prompts[-3:]
    limit = len(prompts[-1]) + 9   # the longest prompt may be fed 9 of its own tokens

    def run(run_ahead):
        eng = Engine(d, dtype=dtype, max_tokens=2048, max_seqs=4, page_size=16, run_ahead=run_ahead, max_seq_len=limit)
        ids = [eng.submit(p, SamplingParams(max_new_tokens=20, eos_id=-1)) for p in prompts]
        while eng.has_work():
            eng.step()
        out = [eng.poll(i) for i in ids]
        assert eng.cache.free_slots == 4
        if eng.runner.graphs is not None:
            assert len(eng.runner.graphs._rows) == 0
        return [(r.tokens, r.status) for r in out], eng

    base, _ = run(False)
    ahead, eng = run(True)
    assert ahead == base and eng.runner.graphs.replays > 0
    assert base[-1][1] == "max_seq" and len(base[-1][0]) == 10   # 9 fed back, the 10th sampled at the last place
    assert all(s == "done" and len(t) == 20 for t, s in base[:-1])
    if dtype == "float32":
        want = greedy_generate(prompts[-1], 10, weights, cfg)
        assert base[-1][0] == want
    too_long = eng.submit(list(range(1, limit + 2)))
    while eng.has_work():
        eng.step()
    assert eng.poll(too_long).status == "max_seq" and eng.poll(too_long).tokens == []


def test_an_abandoned_wait_inside_a_kernel_is_reported(case):
    """Kernels with bounded waits record a code in a status word when a wait gives up.  The word is
    set from the host here (no kernel is made to wait): the next result the host fetches raises,
    the word is cleared, and the engine serves on."""
    from poor_mans_mamba_b200.entry import Engine
    from poor_mans_mamba_b200.kernels import ops as K
    which, d, cfg, weights = case
    prompts, _ = prompts_of(which)
    for run_ahead in (False, True):
        eng = Engine(d, dtype="bfloat16", max_tokens=1024, max_seqs=4, page_size=16, run_ahead=run_ahead)
        good = eng.generate(prompts[:2], max_new_tokens=6, eos_token_id=-1)
        K._watch(eng.device).words[0] = 13
        with pytest.raises(K.KernelError, match="code 13"):
            eng.generate(prompts[:2], max_new_tokens=6, eos_token_id=-1)
        assert K.tc_gemm_status(eng.device) == 0
        eng2 = Engine(d, dtype="bfloat16", max_tokens=1024, max_seqs=4, page_size=16, run_ahead=run_ahead)
        assert eng2.generate(prompts[:2], max_new_tokens=6, eos_token_id=-1) == good
