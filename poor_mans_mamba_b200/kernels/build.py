"""Builds and loads the CUDA kernel library (sm_100a only).

The sources under ``csrc/`` are plain CUDA with a C ABI (no framework headers), so a
build is a handful of ``nvcc -c`` calls that run in parallel plus one link.  The
library is kept in-tree under ``csrc/_build/``; it is rebuilt when the hash of the
sources and flags changes, and built at first use when absent (a fresh checkout needs
nothing but nvcc).  There is no fallback: if the library cannot be built or loaded the
import of the kernels fails with the reason.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

CSRC_DIR = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
LIB_NAME = "libpmm_kernels.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--compiler-options", "-fPIC,-fvisibility=hidden",
]


class KernelBuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[poor_mans_mamba_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("PMM_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (looked at $PMM_NVCC, PATH, $CUDA_HOME/bin, "
                           "/usr/local/cuda/bin); the CUDA kernels cannot be built and there is no "
                           "fallback path")


def source_files() -> List[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _header_files() -> List[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR)
                  if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    for path in source_files() + _header_files():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    in_tree = os.path.join(CSRC_DIR, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return in_tree
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"pmm_b200_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC_DIR, "-c", src, "-o", obj]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"nvcc failed on {os.path.basename(src)}:\n{proc.stdout}")


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile every ``csrc/*.cu`` for sm_100a and link the shared library.  Returns its path."""
    bdir = _build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, LIB_NAME + ".hash")
    want = source_hash()
    lock_path = os.path.join(bdir, ".lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and os.path.isfile(lib) and os.path.isfile(stamp):
                with open(stamp) as fh:
                    if fh.read().strip() == want:
                        return lib
            nvcc = find_nvcc()
            srcs = source_files()
            if verbose:
                _say(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} ...")
            t0 = time.time()
            objs = [os.path.join(bdir, os.path.basename(s)[:-3] + ".o") for s in srcs]
            with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
                futs = [pool.submit(_compile_one, nvcc, s, o) for s, o in zip(srcs, objs)]
                for i, (fut, s) in enumerate(zip(futs, srcs)):
                    fut.result()
                    if verbose:
                        _say(f"  [{i + 1}/{len(srcs)}] {os.path.basename(s)} ({time.time() - t0:.0f}s)")
            tmp_lib = lib + f".tmp{os.getpid()}"
            proc = subprocess.run([nvcc, "-shared", "-o", tmp_lib, *objs, "-gencode",
                                   "arch=compute_100a,code=sm_100a"],
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if proc.returncode != 0:
                raise KernelBuildError(f"link failed:\n{proc.stdout}")
            os.replace(tmp_lib, lib)
            with open(stamp, "w") as fh:
                fh.write(want)
            if verbose:
                _say(f"built {lib} in {time.time() - t0:.0f}s")
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


_LIB: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """The loaded kernel library (built first if needed)."""
    global _LIB
    if _LIB is None:
        path = build()
        try:
            _LIB = ctypes.CDLL(path)
        except OSError as exc:
            raise KernelBuildError(f"cannot load {path}: {exc}") from exc
    return _LIB


def library_path() -> str:
    return os.path.join(_build_dir(), LIB_NAME)
