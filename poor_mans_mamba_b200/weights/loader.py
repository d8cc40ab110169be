"""Loading a model's tensors by name.

Every tensor the model's parts declare is looked up by its full name; the file's shapes
are checked against the configuration before anything is copied, and one error lists
everything that is wrong: missing tensors, wrong shapes and unusable dtypes, and beside them
the tensors nobody asked for (the reference reports only the first missing name,
src/io/model_loader.cpp:43-45, and checks shapes per call, src/ops/cpu_backend.cpp:98-105).
Tensors nobody asked for are not an error by themselves: the reference loads by name and never
looks at the rest (src/model/falconh1_loader.cpp:27-58), so an exporter's extra buffers, or a
tied checkpoint that still carries its output head, load with their names listed on stderr;
``strict=True`` refuses them.

Types on the device: matrices and embeddings keep bfloat16 in the bfloat16 mode (a
float32-stored matrix is rounded once, with a note on stderr) and are widened to float32
in the float32 mode (exact); per-channel vectors are float32 in both modes (a 32-bit
tensor stays 32-bit, a bfloat16 one is widened exactly); integer tables become int32.
"""
from __future__ import annotations

import sys
from typing import Dict, List, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors_io import ModelFiles, SafetensorsError

_FLOAT_NAMES = ("F32", "BF16", "F16", "F64")
_INT_NAMES = ("I64", "I32", "I16", "I8", "U8")


class WeightsError(ValueError):
    """The model folder's tensors do not match what the configuration needs."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[Tuple[str, tuple, tuple]],
                 wrong_dtype: List[Tuple[str, str]]):
        self.missing, self.unexpected = missing, unexpected
        self.wrong_shape, self.wrong_dtype = wrong_shape, wrong_dtype
        lines = ["model tensors do not match the configuration:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        if wrong_dtype:
            lines.append(f"  unusable dtype ({len(wrong_dtype)}): " + ", ".join(
                f"{n} is {d}" for n, d in wrong_dtype))
        super().__init__("\n".join(lines))


def check_tensors(specs: Dict[str, ParamSpec], ignored: List[str], files: ModelFiles,
                  strict: bool = False) -> List[str]:
    """Raises one WeightsError for everything that is wrong; returns the names of tensors that
    nobody asked for (an error only with ``strict``)."""
    present = set(files.keys())
    missing = sorted(n for n in specs if n not in present)
    unexpected = sorted(n for n in present if n not in specs and n not in set(ignored))
    wrong_shape, wrong_dtype = [], []
    for name, spec in specs.items():
        if name not in present:
            continue
        dt, shape = files.info(name)
        if shape != tuple(spec.shape) and shape not in spec.alt_shapes:
            wrong_shape.append((name, shape, tuple(spec.shape)))
        ok = dt in _INT_NAMES if spec.kind == "table" else dt in _FLOAT_NAMES
        if not ok:
            wrong_dtype.append((name, dt))
    if missing or wrong_shape or wrong_dtype or (strict and unexpected):
        raise WeightsError(missing, unexpected, wrong_shape, wrong_dtype)
    return unexpected


def load_tensors(model_dir: str, specs: Dict[str, ParamSpec], ignored: List[str],
                 dtype: torch.dtype, device: torch.device, strict: bool = False) -> Dict[str, torch.Tensor]:
    """name -> tensor on ``device`` in the policy type of its spec, shaped as the spec says."""
    try:
        files = ModelFiles(model_dir)
    except SafetensorsError as exc:
        raise WeightsError([f"(no readable weights: {exc})"], [], [], []) from exc
    try:
        unexpected = check_tensors(specs, ignored, files, strict)
        if unexpected:
            shown = ", ".join(unexpected[:20]) + (f", ... ({len(unexpected) - 20} more)" if len(unexpected) > 20 else "")
            print(f"[poor_mans_mamba_b200] note: {len(unexpected)} tensors of the model folder are not used by "
                  f"this configuration and were ignored: {shown}", file=sys.stderr)
        out: Dict[str, torch.Tensor] = {}
        rounded = 0
        for name, spec in specs.items():
            t = files.tensor(name).reshape(tuple(spec.shape))
            if spec.kind == "table":
                t = t.to(torch.int32)
            elif spec.kind == "vector":
                t = t.to(torch.float32)
            else:
                if dtype == torch.bfloat16 and t.dtype in (torch.float32, torch.float64):
                    if not torch.equal(t.to(torch.bfloat16).to(t.dtype), t):
                        rounded += 1
                t = t.to(dtype)
            out[name] = t.to(device).contiguous()
        if rounded:
            print(f"[poor_mans_mamba_b200] note: {rounded} matrices stored in 32-bit were rounded to "
                  "bfloat16 for the bfloat16 mode", file=sys.stderr)
        return out
    finally:
        files.close()
