"""The engine against the plain implementation under every way of cutting the work, in
float32 and bfloat16, on both tiny configurations (GPU)."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import gpu_harness as H
from model_dirs import make_model_dir
from tiny_configs import token_sequences

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def long_sequences(which, cfg):
    """The configuration's own workload plus sequences that span many pages and SSD chunks."""
    rng = random.Random(100 + ord(which))
    v = cfg["vocab_size"]
    return token_sequences(which) + [[rng.randrange(v) for _ in range(n)] for n in (150, 97, 203)]


@pytest.fixture(scope="module", params=["A", "B"])
def case(request, tmp_path_factory):
    which = request.param
    d, cfg, weights = make_model_dir(which, str(tmp_path_factory.mktemp(f"tiny{which}")))
    seqs = long_sequences(which, cfg)
    refs = H.reference_logits(seqs, weights, cfg)
    return which, d, cfg, seqs, refs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_cuttings_agree_with_plain(case, dtype, cutting):
    which, d, cfg, seqs, refs = case
    page_size = 16
    if cutting == "mixed":
        # so few pages that they are used again: the pool holds the largest sequence plus a little
        budget = max((len(s) + page_size - 1) // page_size for s in seqs) + 6
        runner = H.make_runner(d, dtype, page_size=page_size, num_pages=budget, num_slots=4)
        script = H.script_mixed(seqs, max_live=4, seed=3, budget_pages=budget, page_size=page_size)
        assert max(len(p) for p, _ in script) >= 3  # really mixed
        assert any(len(p) > 1 and any(n == 1 for _, _, n in p) and any(n > 1 for _, _, n in p) for p, _ in script)
    else:
        runner = H.make_runner(d, dtype, page_size=page_size, num_pages=16, num_slots=2)
        script = {"whole": H.script_whole, "tail": H.script_tail_one_by_one, "portions": H.script_portions}[cutting](seqs)
    out = H.run_script(runner, seqs, script)
    for i, ref in enumerate(refs):
        H.check_rows(out[i], ref, dtype, f"tiny {which} {dtype} {cutting} seq {i} (len {len(seqs[i])})")
    assert runner.cache.min_free_pages() == runner.cache.groups[next(iter(runner.cache.groups))].num_pages
    if cutting == "mixed":
        pool = next(iter(runner.cache.groups.values())).pool
        assert pool.high_water <= pool.num_pages and sum(len(s) for s in seqs) > pool.num_pages * page_size


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_page_sizes_and_first_tokens(case, dtype):
    """Page size 64 (the serving default) and 32; the first tokens of a sequence one by one."""
    which, d, cfg, seqs, refs = case
    for page_size in (64, 32):
        runner = H.make_runner(d, dtype, page_size=page_size, num_pages=8, num_slots=2)
        i = len(seqs) - 1
        script = [([(i, p, 1)], []) for p in range(5)] + [([(i, 5, len(seqs[i]) - 5)], [i])]
        out = H.run_script(runner, seqs, script)
        H.check_rows(out[i], refs[i], dtype, f"tiny {which} {dtype} page {page_size} first tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(case, dtype):
    """A short prompt, then every token one by one across many pages and chunks."""
    which, d, cfg, seqs, refs = case
    runner = H.make_runner(d, dtype, page_size=16, num_pages=16, num_slots=1)
    i = len(seqs) - 1
    script = [([(i, 0, 3)], [])] + [([(i, p, 1)], [i] if p == len(seqs[i]) - 1 else []) for p in range(3, len(seqs[i]))]
    out = H.run_script(runner, seqs, script)
    H.check_rows(out[i], refs[i], dtype, f"tiny {which} {dtype} long decoding")


def test_wanted_rows_and_errors(case):
    which, d, cfg, seqs, refs = case
    runner = H.make_runner(d, "float32", page_size=16, num_pages=8, num_slots=2)
    from poor_mans_mamba_b200.cache import OutOfPages
    from poor_mans_mamba_b200.engine import StepEntry
    s = seqs[1]
    lg = runner.step([StepEntry("x", s[:10], [9, 0, 4])]).cpu()
    H.check_rows(lg, refs[1][[9, 0, 4]], "float32", "wanted rows in the asked order")
    assert runner.step([StepEntry("x", s[10:12], [])]).shape == (0, cfg["vocab_size"])
    lg = runner.step([StepEntry("x", s[12:13], [0])]).cpu()
    H.check_rows(lg, refs[1][12:13], "float32", "after a step without wanted rows")
    with pytest.raises(ValueError, match="out of range"):
        runner.step([StepEntry("x", [cfg["vocab_size"]], [0])])
    with pytest.raises(ValueError, match="twice"):
        runner.step([StepEntry("x", [1], [0]), StepEntry("x", [1], [0])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("y", [1] * (8 * 16), [0])])
    assert not runner.cache.has("y")  # refused before anything was taken
    runner.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(case, dtype, tmp_path):
    """bin/trace_run in a process of its own: mixed steps, ends, a pool that is used again."""
    which, d, cfg, seqs, refs = case
    page = 64
    budget_pages = max((len(s) + page - 1) // page for s in seqs) + 3
    script = H.script_mixed(seqs, max_live=4, seed=11, budget_pages=budget_pages, page_size=page)
    lines, wanted = [], []
    for step, (portions, ended) in enumerate(script):
        entries = [{"id": f"r{i}", "tokens": seqs[i][a:a + n], "want": list(range(n))[::2] if step % 3 else list(range(n))}
                   for i, a, n in portions]
        wanted.append([(i, a + w) for (i, a, n), e in zip(portions, entries) for w in e["want"]])
        lines.append(json.dumps({"step": step, "entries": entries, "end": [f"r{i}" for i in ended]}))
    out_dir = tmp_path / f"out_{dtype}"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(budget_pages * page)],
                          input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in range(len(script)) for w in ("done", str(s))]
    v = cfg["vocab_size"]
    for step, rows in enumerate(wanted):
        path = out_dir / f"{step}.f32"
        if not rows:
            assert not path.exists()
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(len(rows), v).copy())
        ref = torch.stack([refs[i][p] for i, p in rows])
        H.check_rows(got, ref, dtype, f"trace_run {dtype} step {step}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_through_cuda_graphs(case, dtype):
    """Decode-only steps served from captured graphs: batches of changing size (buckets with
    padded rows), requests that end and slots and pages that are used again."""
    from poor_mans_mamba_b200.engine import StepEntry
    which, d, cfg, seqs, refs = case
    runner = H.make_runner(d, dtype, page_size=16, num_pages=40, num_slots=4)
    runner.enable_graphs(max_seq_len=256)
    order = [3, 1, 5, 2, 4, 0]  # sequence indices, three live at a time
    live, nxt, pos = [], 0, {}
    while live or nxt < len(order):
        while len(live) < 3 and nxt < len(order):
            i = order[nxt]
            nxt += 1
            head = max(len(seqs[i]) // 3, 1)
            lg = runner.step([StepEntry(("g", i), seqs[i][:head], list(range(head)))]).cpu()
            H.check_rows(lg, refs[i][:head], dtype, f"graph case prompt of seq {i}")
            pos[i] = head
            live.append(i)
        reqs = [("g", i) for i in live]
        ids = runner.decode_tokens(reqs, [seqs[i][pos[i]] for i in live])
        assert ids.shape == (len(live),)
        logits = runner.graphs.last_logits(len(live)).cpu()
        for row, i in enumerate(list(live)):
            H.check_rows(logits[row:row + 1], refs[i][pos[i]:pos[i] + 1], dtype,
                         f"graph decode seq {i} pos {pos[i]} batch {len(live)}")
            assert int(ids[row]) == int(torch.argmax(logits[row]))
            pos[i] += 1
            if pos[i] == len(seqs[i]):
                runner.finish(("g", i))
                live.remove(i)
        runner.cache.check()
    assert runner.graphs.replays > 100 and {b for b, _ in runner.graphs.buckets} <= {1, 2, 4}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_step_shapes_replay_from_graphs(case, dtype, tmp_path):
    """A step shape that comes again is recorded into a CUDA graph and replayed from then on:
    same logits as the plain implementation for different requests, contents, slots and pages."""
    from poor_mans_mamba_b200.engine import StepEntry
    which, d, cfg, seqs, refs = case
    rng = random.Random(7)
    v = cfg["vocab_size"]
    from model_dirs import make_model_dir  # weights of the case again, for fresh references
    _, _, weights = make_model_dir(which, str(tmp_path))
    runner = H.make_runner(d, dtype, page_size=16, num_pages=64, num_slots=3)
    runner.enable_graphs(max_seq_len=512)
    for rep in range(4):
        a = [rng.randrange(v) for _ in range(300)]
        b = [rng.randrange(v) for _ in range(40)]
        ref_a, ref_b = H.reference_logits([a, b], weights, cfg)
        # a filler request of changing length takes other pages and another slot first
        runner.step([StepEntry(("f", rep), [1] * (1 + 17 * rep), [])])
        # step 1: 280 tokens of a + 20 of b (same shape every repetition); step 2: the rest
        lg1 = runner.step([StepEntry(("a", rep), a[:280], [0, 279]), StepEntry(("b", rep), b[:20], [19])]).cpu()
        H.check_rows(lg1, torch.stack([ref_a[0], ref_a[279], ref_b[19]]), dtype, f"repetition {rep} first step")
        lg2 = runner.step([StepEntry(("a", rep), a[280:], [19]), StepEntry(("b", rep), b[20:], [19])]).cpu()
        H.check_rows(lg2, torch.stack([ref_a[299], ref_b[39]]), dtype, f"repetition {rep} second step")
        for name in ("b", "f", "a"):
            runner.finish((name, rep))
        runner.cache.check()
    recorded = [k for k, e in runner._step_graphs.items() if e.get("graph") is not None]
    assert any(k[0] == (280, 20) for k in recorded)
    # the short second step (20 + 20 tokens) has a cache of its own: recorded there, and the many
    # fillers of ever new lengths did not push the large shape out
    small = [k for k, e in runner._small_step_graphs.items() if e.get("graph") is not None]
    assert any(k[0] == (20, 20) for k in small) and not any(k[0] == (20, 20) for k in runner._step_graphs)
