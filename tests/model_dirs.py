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


def make_loud(model_dir: str) -> None:
    files = ModelFiles(model_dir)
    tensors = {k: files.tensor(k) for k in files.keys()}
    files.close()
    for k in list(tensors):
        scale = None
        for suffix, s in LOUD.items():
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
