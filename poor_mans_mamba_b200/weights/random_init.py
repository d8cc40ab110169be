"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

Every tensor the parts declare is filled by the rule of its ParamSpec: matrices and
embeddings N(0, 0.02); norm weights and D one; A_log = log(U[1, 16]); dt_bias the
inverse softplus of a log-uniform step in [1e-3, 0.1]; biases N(0, 0.02).  Each tensor
has its own generator keyed by (seed, tensor name), so a tensor's values do not depend on
which other tensors exist.  Values are rounded to bfloat16 before they are stored
(matrices as BF16, vectors as F32 holding bfloat16-representable values), so the
bfloat16 and the float32 mode of the engine, and any other reader, see identical
weights; ``store_dtype="float32"`` stores every tensor as F32 instead (same values).
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from typing import Any, Dict

import torch

from ..config.registry import resolve_architecture
from ..parts.base import ParamSpec
from .safetensors_io import save_file


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def make_tensor(spec: ParamSpec, seed: int, full_name: str) -> torch.Tensor:
    g = _generator(seed, full_name)
    shape = tuple(spec.stored_shape or spec.shape)
    kind = spec.init[0]
    if kind == "normal":
        t = torch.randn(shape, generator=g, dtype=torch.float32) * float(spec.init[1])
    elif kind == "ones":
        t = torch.ones(shape, dtype=torch.float32)
    elif kind == "zeros":
        t = torch.zeros(shape, dtype=torch.float32)
    elif kind == "log_uniform":  # log of a uniform draw from [lo, hi]
        lo, hi = float(spec.init[1]), float(spec.init[2])
        t = torch.log(lo + (hi - lo) * torch.rand(shape, generator=g, dtype=torch.float32))
    elif kind == "inv_softplus_log_uniform":  # softplus(t) is log-uniform in [lo, hi]
        lo, hi = float(spec.init[1]), float(spec.init[2])
        dt = torch.exp(math.log(lo) + (math.log(hi) - math.log(lo)) * torch.rand(shape, generator=g,
                                                                                  dtype=torch.float32))
        t = dt + torch.log(-torch.expm1(-dt))
    else:
        raise ValueError(f"unknown init rule {spec.init!r} for {full_name}")
    return t.to(torch.bfloat16).to(torch.float32)  # bfloat16-representable values


def write_random_model(config: Dict[str, Any], seed: int, out_dir: str, store_dtype: str = "bfloat16") -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns out_dir."""
    from ..engine.model import Model  # local import: the model skeleton needs no device
    import poor_mans_mamba_b200.architectures  # noqa: F401  (registration)

    if store_dtype not in ("bfloat16", "float32"):
        raise ValueError("store_dtype must be 'bfloat16' or 'float32'")
    arch = resolve_architecture(config)
    cfg = arch.parse_config(config)
    model = Model(arch.model_spec(cfg))
    tensors = {}
    for name, spec in model.param_specs().items():
        t = make_tensor(spec, seed, name)
        if spec.kind == "matrix" and store_dtype == "bfloat16":
            t = t.to(torch.bfloat16)
        tensors[name] = t
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(config, fh, indent=1)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed), "generator": "poor_mans_mamba_b200.random_init"})
    return out_dir
