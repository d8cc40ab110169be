"""The plain implementation against the reference's own CUDA code, run on this GPU.

The reference's Falcon-H1 runner (src/runtime/runner/falconh1_runner.cpp:216-248) is built
unmodified with nvcc and cuBLAS by baseline/build_reference.py; its driver reads the same
model.safetensors bytes as the engine.  Tolerance: 1e-4 absolute, the default of the reference's
own GPU-vs-CPU comparisons (tests/ops/gpu/gpu_test_utils.h:83-89)."""
import tempfile

import numpy as np
import pytest
import torch

import reference_arm
from gpu_harness import check_rows, make_runner, run_script, script_whole
from plain.falcon_h1_plain import forward_logits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def binary():
    try:
        return reference_arm.driver_binary()
    except RuntimeError as exc:
        pytest.skip(f"the reference arm cannot be built here: {exc}")


@pytest.mark.parametrize("name", sorted(reference_arm.anchor_configs()))
def test_plain_equals_reference_cuda(binary, name):
    cfg, seed, seqs, lens = reference_arm.anchor_configs()[name]
    with tempfile.TemporaryDirectory() as d:
        weights = reference_arm.write_anchor_model(cfg, seed, d)
        for seq, n_prompt in zip(seqs, lens):
            ref = reference_arm.reference_logits(binary, d, seq, n_prompt, cfg["vocab_size"])
            plain = forward_logits(seq, weights, cfg, torch.float64)[reference_arm.rows_of(seq, n_prompt)].numpy()
            assert ref.shape == plain.shape
            assert np.isfinite(ref).all()
            err = np.abs(ref.astype(np.float64) - plain)
            assert err.max() <= 1e-4, (f"{name}, prompt of {n_prompt}: |plain - reference| = {err.max():.3e} at row "
                                       f"{int(err.max(axis=1).argmax())} (largest logit {np.abs(plain).max():.2f})")
            assert np.abs(plain).max() > 0.2, "logits too small for the comparison to mean anything"


@pytest.mark.parametrize("name", sorted(reference_arm.anchor_configs()))
def test_engine_float32_equals_reference_cuda(binary, name):
    """The engine's float32 path against the reference's binaries directly."""
    cfg, seed, seqs, lens = reference_arm.anchor_configs()[name]
    with tempfile.TemporaryDirectory() as d:
        reference_arm.write_anchor_model(cfg, seed, d)
        runner = make_runner(d, "float32")
        got = run_script(runner, seqs, script_whole(seqs))
        for i, (seq, n_prompt) in enumerate(zip(seqs, lens)):
            ref = reference_arm.reference_logits(binary, d, seq, n_prompt, cfg["vocab_size"])
            mine = got[i][reference_arm.rows_of(seq, n_prompt)].numpy()
            err = np.abs(ref.astype(np.float64) - mine)
            assert err.max() <= 1e-4, f"{name}, sequence {i}: |engine - reference| = {err.max():.3e}"
