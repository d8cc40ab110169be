"""Model folders for the tests: the tiny configurations with random weights, made *loud*.

With every matrix drawn from N(0, 0.02) the state-space path and the attention scores
are numerically silent: removing the SSM state term changes the logits by 1e-6 or less,
and the attention is almost uniform, so a wrong state, page or rotation would pass any
tolerance.  The loud variant multiplies the mixer input projection, the conv weights and
the query/key projections by powers of two (exact in bfloat16), after which the state
term moves the logits by ~0.5 and the rotation by ~0.05.
"""
from __future__ import annotations

import os
from typing import Dict, Tuple

import torch

from tiny_configs import TINY_WORKLOADS, tiny_config

from poor_mans_mamba_b200.weights import ModelFiles, save_file, write_random_model

LOUD = {"mamba.in_proj.weight": 8.0, "mamba.in_proj.bias": 8.0, "conv1d.weight": 16.0, "q_proj.weight": 8.0,
        "k_proj.weight": 8.0}
LOUD_OTHER_MATRICES = 2.0
_FROM_THE_STREAM = ("mamba.in_proj.weight", "mamba.in_proj.bias", "q_proj.weight", "k_proj.weight")


def loud_scales(hidden_size: int = 0) -> dict:
    """The factors by tensor-name suffix.  The factor 8 of the projections that read the normalised
    stream suits the tiny widths (a row of N(0, 0.02) weights times 64..96 unit inputs has a standard
    deviation of 0.16..0.2); at a width of ``hidden_size`` the same loudness (about 1.3) needs the
    power of two nearest to 1.3 / (0.02 sqrt(width)): 2 at 1,024 and 1,280, 1 at 3,072."""
    scales = dict(LOUD)
    if hidden_size > 0:
        import math
        s = 2.0 ** round(math.log2(1.3 / (0.02 * math.sqrt(hidden_size))))
        for k in _FROM_THE_STREAM:
            scales[k] = s
    return scales


def make_loud(model_dir: str, hidden_size: int = 0) -> None:
    """``hidden_size`` > 0: factors for that width (see `loud_scales`); 0: the tiny models' factors."""
    files = ModelFiles(model_dir)
    tensors = {k: files.tensor(k) for k in files.keys()}
    files.close()
    loud = loud_scales(hidden_size)
    for k in list(tensors):
        scale = None
        for suffix, s in loud.items():
            if k.endswith(suffix):
                scale = s
        if scale is None and tensors[k].dim() >= 2 and "embed" not in k and "lm_head" not in k:
            scale = LOUD_OTHER_MATRICES
        if scale is not None:
            tensors[k] = (tensors[k].float() * scale).to(tensors[k].dtype)
    save_file(tensors, os.path.join(model_dir, "model.safetensors"))


def make_model_dir(which: str, out_dir: str, loud: bool = True, config_patch: dict = None
                   ) -> Tuple[str, dict, Dict[str, torch.Tensor]]:
    """(folder, config dict, float32 weights by name) of tiny configuration ``which``."""
    cfg = tiny_config(which)
    if config_patch:
        cfg.update(config_patch)
    write_random_model(cfg, TINY_WORKLOADS[which][0], out_dir)
    if loud:
        make_loud(out_dir)
    files = ModelFiles(out_dir)
    weights = {k: files.tensor(k).float() for k in files.keys()}
    files.close()
    return out_dir, cfg, weights
