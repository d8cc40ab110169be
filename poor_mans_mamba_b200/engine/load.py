"""From a model folder to a model on the device."""
from __future__ import annotations

from typing import Tuple

import torch

from .. import architectures  # noqa: F401  (registers the architectures)
from ..config.registry import open_model_dir
from ..weights.loader import load_tensors
from .model import Model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be bfloat16 or float32")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}") from None


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0") -> Tuple[Model, object]:
    """(model with its tensors on ``device``, typed config).  The model class is chosen by
    config.json through the architecture registry."""
    dt = parse_dtype(dtype)
    dev = torch.device(device)
    arch, cfg = open_model_dir(model_dir)
    model = Model(arch.model_spec(cfg))
    tensors = load_tensors(model_dir, model.param_specs(), model.ignored_names(), dt, dev)
    model.bind(tensors, dt, dev)
    return model, cfg
