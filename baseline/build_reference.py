#!/usr/bin/env python3
"""Builds the reference arm: the UNMODIFIED CUDA path of AlterHoodie/poor_mans_mamba plus the
host driver `ref_driver.cu` of this folder, with nvcc and cuBLAS only.

    python baseline/build_reference.py [--reference DIR] [--force]

The reference is a CMake project whose configure step fetches Eigen, nlohmann_json,
safetensors-cpp, tokenizers-cpp and googletest from the network, and `pip install` of its tree
fails (no setup.py / pyproject.toml).  Its GPU path needs none of those: the translation units
listed in SOURCES include only the project's own headers, <cuda_runtime.h> and <cublas_v2.h>.
They are copied byte for byte to `baseline/_ref/src/` (so the build also works on a machine where
the reference tree is not mounted) and compiled for sm_100a into `baseline/_ref/ref_driver`.
`baseline/_ref/` is not tracked by git.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SRC = os.path.join(OUT, "src")
BINARY = os.path.join(OUT, "ref_driver")

SOURCES = [
    "src/ops/gpu/attention.cu", "src/ops/gpu/conv.cu", "src/ops/gpu/element_wise.cu", "src/ops/gpu/embed.cu",
    "src/ops/gpu/linear.cu", "src/ops/gpu/mamba2_scan.cu", "src/ops/gpu/rms_norm.cu", "src/ops/gpu/reductions.cu",
    "src/ops/cuda_backend.cu", "src/core/device.cpp", "src/core/cuda_allocator.cu",
    "src/runtime/cache/cache_layout.cpp", "src/runtime/cache/cache_pool.cpp",
    "src/runtime/runner/falconh1_runner.cpp",
]


def _digest(paths):
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def copy_reference(reference: str) -> None:
    """include/ and the listed sources, unchanged."""
    if os.path.isdir(SRC):
        shutil.rmtree(SRC)
    os.makedirs(SRC)
    shutil.copytree(os.path.join(reference, "include"), os.path.join(SRC, "include"))
    for rel in SOURCES:
        dst = os.path.join(SRC, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(reference, rel), dst)


def build(reference: str | None = None, force: bool = False, verbose: bool = True) -> str:
    """Returns the path of the driver binary; raises RuntimeError with the compiler's words."""
    driver = os.path.join(HERE, "ref_driver.cu")
    reference = reference or os.environ.get("PMM_REFERENCE_DIR", "/root/reference")
    have_copy = all(os.path.isfile(os.path.join(SRC, rel)) for rel in SOURCES)
    if not have_copy:
        if not os.path.isdir(os.path.join(reference, "src", "ops", "gpu")):
            raise RuntimeError(f"the reference tree is not at {reference} and no copy is under {SRC}")
        copy_reference(reference)
    stamp_path = os.path.join(OUT, "ref_driver.sha256")
    stamp = _digest([driver] + [os.path.join(SRC, rel) for rel in SOURCES])
    if not force and os.path.isfile(BINARY) and os.path.isfile(stamp_path):
        with open(stamp_path) as fh:
            if fh.read().strip() == stamp:
                return BINARY
    nvcc = os.environ.get("PMM_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-std=c++20", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-DMAMBASERVE_WITH_CUDA",
           "-I", os.path.join(SRC, "include"), "-o", BINARY, driver]
    cmd += [os.path.join(SRC, rel) for rel in SOURCES]
    cmd += ["-lcublas"]
    if verbose:
        print("[reference] " + " ".join(cmd), file=sys.stderr, flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout[-2000:] + proc.stderr[-4000:])
    with open(stamp_path, "w") as fh:
        fh.write(stamp + "\n")
    return BINARY


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    try:
        print(build(args.reference, args.force))
    except RuntimeError as exc:
        print(f"build_reference: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
