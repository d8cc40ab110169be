"""Writes tests/golden/plain_tiny.json: a few logits of the plain implementation on the two
tiny random models, as a regression anchor for the oracle itself.

These numbers pin the oracle against itself (both tiny configurations as they stand, with the
gated mixer norm and the projection biases that the reference's Falcon-H1 runner does not have).
The anchor on the reference's own binaries is reference_cuda_tiny.json, written by
make_reference_golden.py.

    python tests/golden/make_golden.py
"""
import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from plain.falcon_h1_plain import forward_logits  # noqa: E402
from tiny_configs import TINY_WORKLOADS, tiny_config, token_sequences  # noqa: E402

from poor_mans_mamba_b200.weights import ModelFiles, write_random_model  # noqa: E402


def main() -> None:
    out = {}
    for which in ("A", "B"):
        cfg = tiny_config(which)
        seed = TINY_WORKLOADS[which][0]
        with tempfile.TemporaryDirectory() as d:
            write_random_model(cfg, seed, d)
            files = ModelFiles(d)
            weights = {k: files.tensor(k).float() for k in files.keys()}
            files.close()
        seq = token_sequences(which)[-1]
        logits = forward_logits(seq, weights, cfg, torch.float64)
        out[which] = {
            "tokens": seq,
            "positions": [0, len(seq) // 2, len(seq) - 1],
            "first8": [[round(float(v), 9) for v in logits[p, :8]] for p in (0, len(seq) // 2, len(seq) - 1)],
            "argmax": [int(logits[p].argmax()) for p in range(len(seq))],
            "row_sums": [round(float(logits[p].sum()), 8) for p in (0, len(seq) - 1)],
        }
    with open(os.path.join(HERE, "plain_tiny.json"), "w") as fh:
        json.dump(out, fh, indent=1)
    print("wrote", os.path.join(HERE, "plain_tiny.json"))


if __name__ == "__main__":
    main()
