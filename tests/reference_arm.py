"""Access to the reference arm for tests: the unmodified CUDA path of AlterHoodie/poor_mans_mamba
built by baseline/build_reference.py, run through its driver's `logits` mode."""
from __future__ import annotations

import copy
import importlib.util
import os
import subprocess
import tempfile
from typing import List, Sequence

import numpy as np

from tiny_configs import TINY_WORKLOADS, tiny_config, token_sequences

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def anchor_configs():
    """The two configurations the reference's Falcon-H1 runner can compute (it has no projection
    biases and never loads the gated mixer norm, src/model/falconh1_loader.cpp:27-58 and
    src/runtime/runner/falconh1_runner.cpp:50-57): tiny B without projection biases, and tiny A
    with the gated norm off and multipliers away from one.  name -> (config, weight seed, sequences,
    prompt lengths)."""
    b = tiny_config("B")
    b["mamba_proj_bias"] = False
    a = tiny_config("A")
    a.update(mamba_rms_norm=False, mamba_conv_bias=True, embedding_multiplier=2.5, lm_head_multiplier=0.75,
             attention_in_multiplier=1.25, attention_out_multiplier=0.5, key_multiplier=1.5, ssm_in_multiplier=0.75,
             ssm_out_multiplier=1.5, ssm_multipliers=[1.25, 0.75, 1.5, 0.5, 1.125], mlp_multipliers=[0.75, 1.25])
    out = {}
    for name, which, cfg in (("B_no_proj_bias", "B", b), ("A_ungated_scaled", "A", a)):
        seed, lens, _ = TINY_WORKLOADS[which]
        out[name] = (copy.deepcopy(cfg), seed, token_sequences(which), list(lens))
    return out


def driver_binary() -> str:
    """Path of the built driver; raises RuntimeError when it cannot be built here."""
    spec = importlib.util.spec_from_file_location("build_reference", os.path.join(ROOT, "baseline", "build_reference.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(verbose=False)


def reference_logits(binary: str, model_dir: str, tokens: Sequence[int], n_prompt: int, vocab: int) -> np.ndarray:
    """[1 + len(tokens) - n_prompt, vocab]: the reference's logits after prefilling tokens[:n_prompt]
    in one call and after each further token fed through its decode call."""
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "logits.f32")
        cmd = [binary, "logits", "--model", model_dir, "--max-seq", str(len(tokens) + 8),
               "--tokens", ",".join(str(t) for t in tokens[:n_prompt]),
               "--decode", ",".join(str(t) for t in tokens[n_prompt:]), "--out", out]
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        if proc.returncode != 0:
            raise RuntimeError(f"reference driver failed ({proc.returncode}): {proc.stderr[-2000:]}")
        return np.fromfile(out, dtype="<f4").reshape(-1, vocab)


def write_anchor_model(cfg: dict, seed: int, out_dir: str):
    """Model folder with loud random weights; returns float32 weights by name."""
    from model_dirs import make_loud
    from poor_mans_mamba_b200.weights import ModelFiles, write_random_model
    write_random_model(cfg, seed, out_dir)
    make_loud(out_dir)
    files = ModelFiles(out_dir)
    weights = {k: files.tensor(k).float() for k in files.keys()}
    files.close()
    return weights


def rows_of(tokens: Sequence[int], n_prompt: int) -> List[int]:
    """Positions whose logits the driver returns: the prompt's last, then every later token."""
    return list(range(n_prompt - 1, len(tokens)))
