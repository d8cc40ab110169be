"""Writes tests/golden/reference_cuda_tiny.json: logits computed by the reference's own binaries.

Run on a machine with a GPU (the reference's CPU path needs Eigen and cannot be built offline):

    python baseline/build_reference.py && python tests/golden/make_reference_golden.py

For each anchor configuration of tests/reference_arm.py (tiny B without projection biases; tiny A
with the gated norm off and multipliers away from one) and each sequence of its workload, the
unmodified FalconH1Runner of AlterHoodie/poor_mans_mamba (CUDA backend, FP32, cublasSgemm)
prefills the prompt in one call and decodes the remaining tokens one by one from the same
model.safetensors bytes the engine reads.  Kept per returned row: the first 24 logits, the row's
argmax, its sum and its largest absolute value.  tests/test_reference_golden.py recomputes the
rows with the plain implementation on the CPU and compares.
"""
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import reference_arm  # noqa: E402


def main() -> None:
    binary = reference_arm.driver_binary()
    out = {}
    for name, (cfg, seed, seqs, lens) in reference_arm.anchor_configs().items():
        entry = {"config": cfg, "weight_seed": seed, "sequences": []}
        with tempfile.TemporaryDirectory() as d:
            reference_arm.write_anchor_model(cfg, seed, d)
            for seq, n_prompt in zip(seqs, lens):
                ref = reference_arm.reference_logits(binary, d, seq, n_prompt, cfg["vocab_size"])
                entry["sequences"].append({
                    "tokens": list(seq), "n_prompt": n_prompt,
                    "first24": [[float(np.float32(v)) for v in row[:24]] for row in ref],
                    "argmax": [int(row.argmax()) for row in ref],
                    "row_sum": [float(row.astype(np.float64).sum()) for row in ref],
                    "abs_max": [float(np.abs(row).max()) for row in ref],
                })
        out[name] = entry
    path = os.path.join(HERE, "reference_cuda_tiny.json")
    with open(path, "w") as fh:
        json.dump(out, fh)
    print("wrote", path)


if __name__ == "__main__":
    main()
