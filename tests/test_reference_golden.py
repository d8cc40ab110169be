"""The plain implementation against logits that the reference's own binaries produced.

tests/golden/reference_cuda_tiny.json was written by tests/golden/make_reference_golden.py on a
B200 from the unmodified CUDA path of AlterHoodie/poor_mans_mamba (FalconH1Runner, FP32,
cublasSgemm).  Here, on the CPU, the same random models are written again from their seeds and
the plain implementation's rows are compared with the recorded ones at the reference's own
tolerance (1e-4 absolute, tests/ops/gpu/gpu_test_utils.h:83-89)."""
import json
import os
import tempfile

import numpy as np
import pytest
import torch

import reference_arm
from plain.falcon_h1_plain import forward_logits

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_cuda_tiny.json")


@pytest.mark.parametrize("name", sorted(reference_arm.anchor_configs()))
def test_plain_matches_recorded_reference_logits(name):
    with open(GOLDEN) as fh:
        golden = json.load(fh)[name]
    cfg, seed, seqs, lens = reference_arm.anchor_configs()[name]
    assert golden["config"] == cfg and golden["weight_seed"] == seed, "the golden file was made for other settings"
    with tempfile.TemporaryDirectory() as d:
        weights = reference_arm.write_anchor_model(cfg, seed, d)
    for seq, n_prompt, rec in zip(seqs, lens, golden["sequences"]):
        assert rec["tokens"] == list(seq) and rec["n_prompt"] == n_prompt
        plain = forward_logits(seq, weights, cfg, torch.float64)[reference_arm.rows_of(seq, n_prompt)].numpy()
        first = np.array(rec["first24"], dtype=np.float64)
        assert np.abs(plain[:, :24] - first).max() <= 1e-4
        assert np.abs(plain.sum(axis=1) - np.array(rec["row_sum"])).max() <= 1e-4 * plain.shape[1]
        assert np.abs(np.abs(plain).max(axis=1) - np.array(rec["abs_max"])).max() <= 1e-4
        for r, want in enumerate(rec["argmax"]):
            got = int(plain[r].argmax())
            assert got == want or abs(plain[r, got] - plain[r, want]) <= 2e-4
