#!/usr/bin/env python3
"""Serving benchmark in the manner of the reference's generate harness
(benchmarks/generate_bench.cpp:205-386: prefill tok/s, decode tok/s, batch always 1 there).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  Default: Falcon-H1-0.5B layer sizes with
random weights (seed 2), bfloat16, batch 8, every request at a context that ends at 4,096
tokens.  Prints ONE JSON line:
  value    decoded tokens/s over K steps, timed on the device with CUDA events;
  e2e      the same through the Python entry point (Engine.step: scheduler, the step's indices
           in from pinned memory and the sampled ids back to the host every step; the engine
           launches a decode step before the previous step's ids have arrived, feeding it the
           ids that are still on the device, so the two copies overlap the next step);
  prefill  one 2,048-token prompt in one step: tokens/s, ms, fraction of the bf16 peak;
  roofline bytes the decode step must read (every weight once, the cache of the live
           requests) / its time, against the HBM copy peak;
  points   decode tokens/s at batch 1 and 64.
Peaks come from MEASURED_PEAKS.json beside this file when present, else from the stated
fallback.  Inputs of a decode step (1 GB of weights plus the caches) exceed the L2, so no
L2 flush is needed between timed iterations.
"""
from __future__ import annotations

import argparse
import atexit
import gc
import json
import os
import random
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

# BASELINE.json configs[2]: Falcon-H1-0.5B layer sizes
CONFIG_05B = {
    "model_type": "falcon_h1", "architectures": ["FalconH1ForCausalLM"],
    "num_hidden_layers": 36, "hidden_size": 1024, "vocab_size": 32784, "intermediate_size": 2048,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64, "rope_theta": 1e11,
    "attention_bias": False, "attention_dropout": 0.0, "mlp_bias": False,
    "mamba_d_ssm": 1536, "mamba_n_heads": 24, "mamba_d_head": 64, "mamba_d_state": 128,
    "mamba_n_groups": 1, "mamba_d_conv": 4, "mamba_chunk_size": 128, "mamba_conv_bias": True,
    "mamba_proj_bias": False, "mamba_rms_norm": False, "mamba_norm_before_gate": False,
    "rms_norm_eps": 1e-5, "hidden_act": "silu", "tie_word_embeddings": False,
    "embedding_multiplier": 1.0, "lm_head_multiplier": 1.0, "attention_in_multiplier": 1.0,
    "attention_out_multiplier": 1.0, "key_multiplier": 1.0, "ssm_in_multiplier": 1.0,
    "ssm_out_multiplier": 1.0, "ssm_multipliers": [1.0] * 5, "mlp_multipliers": [1.0, 1.0],
    "bos_token_id": 1, "eos_token_id": 11, "pad_token_id": 0,
}
FULL_LAYERS = 36

# Other Falcon-H1 layer sizes (BASELINE.json configs[3] and configs[4]) for measurements beside the
# benchmark's own configuration: `--sizes 7b --layers 4`.  name -> (changed keys, layers of the full model)
OTHER_SIZES = {
    "1.5b-deep": (dict(hidden_size=1280, num_attention_heads=6, num_key_value_heads=2, head_dim=128,
                       intermediate_size=3072, vocab_size=65537, mamba_d_ssm=2560, mamba_n_heads=40, mamba_d_head=64,
                       mamba_d_state=256, mamba_chunk_size=256), 66),
    "7b": (dict(hidden_size=3072, num_attention_heads=12, num_key_value_heads=2, head_dim=128,
                intermediate_size=12288, vocab_size=130049, mamba_d_ssm=6144, mamba_n_heads=48, mamba_d_head=128,
                mamba_d_state=256, mamba_chunk_size=256), 44),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as fh:
                data = json.load(fh)
            out = {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                   "source": "measured"}
            if "bf16_tflops_sustained" in data:
                out["bf16_tflops_sustained"] = float(data["bf16_tflops_sustained"])
            return out
        except (OSError, KeyError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True,
                                     timeout=5).stdout.strip().splitlines()
                if out:
                    f = [x.strip() for x in out[0].split(",")]
                    self.samples.append(float(f[0]))
                    self.max_mhz = float(f[1])
                    for n, v in zip(names, f[2:]):
                        if v.lower().startswith("active"):
                            self.reasons.add(n)
            except (OSError, ValueError, subprocess.SubprocessError, IndexError):
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def model_numbers(cfg):
    """Bytes and flops of the configuration, from its sizes alone."""
    D, L, V, F = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["vocab_size"], cfg["intermediate_size"]
    Hq, Hkv, Dh = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    I, H, P, N, G, Kc = (cfg["mamba_d_ssm"], cfg["mamba_n_heads"], cfg["mamba_d_head"], cfg["mamba_d_state"],
                         cfg["mamba_n_groups"], cfg["mamba_d_conv"])
    conv_dim = I + 2 * G * N
    proj = I + conv_dim + H
    layer_mat = D * (proj + (Hq + 2 * Hkv) * Dh) + I * D + Hq * Dh * D + 3 * D * F
    layer_vec = 2 * D + conv_dim * Kc + conv_dim + 3 * H
    return {
        "layer_matrix_params": layer_mat, "layer_vector_params": layer_vec,
        "weight_bytes_per_step": L * (2 * layer_mat + 4 * layer_vec) + 2 * V * D + 2 * D + 4 * D,
        "kv_bytes_per_token": L * 2 * Hkv * Dh * 2,
        "state_bytes_per_seq": L * (H * P * N * 4 + (Kc - 1) * conv_dim * 4),
        "flops_per_token_matmul": 2 * L * layer_mat,
        "attn_flops": lambda T: L * 4 * Hq * Dh * T * (T + 1) // 2,
        "ssd_flops_per_token": L * 6 * H * P * N,
        "head_flops_per_row": 2 * V * D,
        "params": L * (layer_mat + layer_vec) + 2 * V * D + D,
    }

def sized_config(args):
    """config.json dict of the run and the layer count of the full model."""
    cfg = dict(CONFIG_05B)
    full_layers = FULL_LAYERS
    if args.sizes != "0.5b":
        cfg.update(OTHER_SIZES[args.sizes][0])
        full_layers = OTHER_SIZES[args.sizes][1]
    if args.layers is None:
        args.layers = full_layers
    cfg["num_hidden_layers"] = args.layers
    return cfg, full_layers


def config_record(cfg, args, full_layers):
    """The flat `config` of the JSON line: every size of the run, the same keys for both arms."""
    return {"model": f"falcon-h1-{args.sizes}-sizes", "layers": args.layers, "layers_full": full_layers,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "d_ssm": cfg["mamba_d_ssm"],
            "ssm_heads": cfg["mamba_n_heads"], "d_state": cfg["mamba_d_state"], "d_conv": cfg["mamba_d_conv"],
            "chunk": cfg["mamba_chunk_size"], "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "single-gpu", "page_size": 64, "l2": "inputs exceed L2 (no flush)"}


def check_against_plain(cfg, args) -> dict:
    """The engine against the plain implementation of the test-suite on the first two layers of
    the run's model (same seed, so the same tensors as the timed model's layers 0 and 1, scaled
    loud as the tests' models are so that a wrong key range, page or state moves the logits) and
    on the benchmark's schedule.  Raises AssertionError at the first row beyond the tolerance."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import parity_at_sizes
    from model_dirs import make_loud

    from poor_mans_mamba_b200.weights import ModelFiles, write_random_model

    small = dict(cfg)
    small["num_hidden_layers"] = min(2, cfg["num_hidden_layers"])
    ctx = args.context
    contexts = sorted({max(16, int(ctx * f)) - 6 for f in (0.075, 0.13, 0.25, 0.32, 0.5, 0.56, 0.76, 1.0)})
    t0 = time.time()
    with tempfile.TemporaryDirectory(prefix="pmm_bench_check_") as d:
        write_random_model(small, seed=2, out_dir=d)
        make_loud(d, hidden_size=small["hidden_size"])
        files = ModelFiles(d)
        weights = {k: files.tensor(k).float() for k in files.keys()}
        files.close()
        with torch.cuda.device(0):
            summary = parity_at_sizes.run_parity(d, small, weights, args.dtype, prompt_len=min(2048, ctx // 2),
                                                 contexts=contexts, decode_steps=6, max_seq_len=ctx + 64)
        torch.cuda.empty_cache()
    return {"layers": small["num_hidden_layers"], "rows": summary["rows"],
            "worst_error_over_tolerance": summary["worst_error_over_tolerance"], "seconds": round(time.time() - t0, 1)}


def reference_arm(args) -> int:
    """`--impl reference`: the UNMODIFIED CUDA path of the reference (FalconH1Runner + CUDABackend +
    src/ops/gpu/*.cu: FP32, cublasSgemm, one request per cache slot), built with nvcc and cuBLAS by
    baseline/build_reference.py and driven by baseline/ref_driver.cu.  Same layer sizes, layer
    count, batch, context, step count and warm-up as this repository's arm; random weights made by
    the driver.  Batch B > 1 is B slots on B streams, the way the reference's worker runs them
    (src/runtime/worker.cpp:121-142); batch 1 follows benchmarks/generate_bench.cpp:329-367.
    `value` is timed with CUDA events on the slots' streams; `e2e` is the wall clock of the same
    steps, which include, every step, the token ids going to the device and the logits coming back
    for the host argmax (the reference samples on the host).  Nothing under
    poor_mans_mamba_b200/ is imported."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("build_reference",
                                                  os.path.join(ROOT, "baseline", "build_reference.py"))
    builder = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(builder)
    try:
        binary = builder.build()
    except RuntimeError as exc:
        first = str(exc).strip().splitlines()
        print(json.dumps({"impl": "reference", "unavailable": "the reference's CUDA path could not be built with "
                          "nvcc and cuBLAS here: " + " | ".join(first[:3])[:400]}))
        return 0
    cfg, full_layers = sized_config(args)
    tmp = tempfile.mkdtemp(prefix="pmm_ref_bench_")
    atexit.register(shutil.rmtree, tmp, ignore_errors=True)
    with open(os.path.join(tmp, "config.json"), "w") as fh:
        json.dump(cfg, fh)

    def run(batch, steps, run_prompts, prefill_len):
        cmd = [binary, "bench", "--config", tmp, "--batch", str(batch), "--context", str(args.context),
               "--steps", str(steps), "--warmup", str(args.warmup), "--run-prompts", "1" if run_prompts else "0",
               "--prefill-len", str(prefill_len), "--seed", "2"]
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
        if proc.returncode != 0:
            raise RuntimeError(f"ref_driver exited {proc.returncode}: {proc.stderr.strip()[-400:]}")
        return json.loads(proc.stdout.strip().splitlines()[-1])

    try:
        with ClockSampler() as clocks:
            main_run = run(args.batch, args.steps, True, 2048)
        points = {}
        if not args.no_points:
            for b in (1, 64):
                if b == args.batch:
                    continue
                # the caches of these points keep the zeros the pool starts with instead of running
                # b prompts of ~4,000 tokens (8 s each): the decode kernels' time does not depend on values
                points[f"decode_b{b}"] = round(run(b, min(args.steps, 32 if b == 1 else 8), False, 0)
                                               ["decode_tok_s_device"], 1)
    except (RuntimeError, subprocess.SubprocessError, ValueError) as exc:
        print(json.dumps({"impl": "reference", "unavailable": f"the built reference driver failed: {exc}"[:500]}))
        return 0
    result = {
        "metric": f"decode tokens/s (Falcon-H1-{args.sizes.upper()} layer sizes, random weights)",
        "value": round(main_run["decode_tok_s_device"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["device_ms"] / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic: uniform random token ids, random-init weights made by the driver (seed 2)",
        "config": config_record(cfg, args, full_layers), "clocks": clocks.summary(),
        "e2e": {"value": round(main_run["decode_tok_s_e2e"], 2), "unit": "tokens/s",
                "h2d_bytes_per_step": 4 * args.batch, "d2h_bytes_per_step": main_run["logit_bytes_d2h_per_step"]},
        "itl_ms": {"mean": main_run["itl_mean_ms"], "p50": main_run["itl_p50_ms"], "p95": main_run["itl_p95_ms"]},
        "prefill": {"value": round(2048 / (main_run["prefill_ms"] / 1e3), 1), "tokens": 2048,
                    "ms": round(main_run["prefill_ms"], 3)},
        "points": points, "impl": "reference",
        "how": "unmodified reference CUDA path (FalconH1Runner, CUDABackend, FP32, cublasSgemm), one slot and "
               "stream per request; host argmax over logits copied back every step",
    }
    print(json.dumps(result))
    return 0


def serve_workload(args, cfg, full_layers, model_dir, checked) -> int:
    """`--workload serve`: bursts of 32 requests through the Python entry point (`Engine.generate`:
    scheduler, chunked prefill under a budget of 2,048 tokens a step, decoding of all live
    requests, sampling).  Every burst has new prompts of 200 to 1,500 tokens (uniform, seed 5) and
    generates 128 tokens per request, so no two prefill steps are cut alike.  `value` is tokens
    (prompt and generated) per second of wall time, host token ids in and out, over --steps
    bursts after --warmup bursts (at least 28, about ten seconds: recordings of step shapes are made
    while warming up, as a server makes them in its first seconds)."""
    import torch

    from poor_mans_mamba_b200.entry import Engine

    n_req, new_tokens, bursts, warm = 32, 128, max(1, args.steps // 8), max(28, args.warmup)
    rng = random.Random(5)
    vocab = cfg["vocab_size"]

    def burst():
        return [[rng.randrange(vocab) for _ in range(rng.randrange(200, 1500))] for _ in range(n_req)]

    with torch.cuda.device(0):
        eng = Engine(model_dir, dtype=args.dtype, max_tokens=(n_req + 8) * 2048, max_seqs=64, page_size=64,
                     max_batched_tokens=2048, max_seq_len=2048)
        for _ in range(warm):
            eng.generate(burst(), max_new_tokens=new_tokens, eos_token_id=-1)
        torch.cuda.synchronize()
        launches0 = eng.runner.mark_launches()
        tokens, wall = 0, 0.0
        with ClockSampler() as clocks:
            for _ in range(bursts):
                prompts = burst()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                out = eng.generate(prompts, max_new_tokens=new_tokens, eos_token_id=-1)
                wall += time.perf_counter() - t0
                tokens += sum(map(len, prompts)) + sum(map(len, out))
        launches = eng.runner.kernels_launched_since(launches0)
        eng.runner.check_kernels(wait=True)
        recorded = sorted(k[1:] for k in eng.runner._step_graphs if k[0] == "rounded")
    record = config_record(cfg, args, full_layers)
    record.update({"global_batch": n_req, "seq_len": 2048, "prompt_tokens": "200..1500", "new_tokens": new_tokens,
                   "token_budget": 2048})
    result = {
        "metric": f"served tokens/s (bursts of 32 requests through Engine.generate, Falcon-H1-{args.sizes.upper()} layer sizes)",
        "value": round(tokens / wall, 1), "unit": "tokens/s", "n_gpus": 1, "steps": bursts, "warmup": warm,
        "ms_per_step": round(wall / bursts * 1e3, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: uniform random token ids and prompt lengths (seed 5), random-init weights (seed 2)",
        "config": record, "clocks": clocks.summary(), "gpu_launches": int(launches),
        "rounded_step_shapes_recorded": len(recorded), "impl": "ours", "checked": checked is not None,
    }
    if checked is not None:
        result["check"] = checked
    print(json.dumps(result))
    return 0


def mixed_workload(args, cfg, full_layers, nums, peaks, model_dir, checked) -> int:
    """`--workload mixed`: one step that mixes 32 decoding requests (contexts spread over
    1,024..4,096 tokens) with four prompt portions of 512 tokens (at depths 0, 512, 1,024 and 1,536
    of 2,048-token prompts; a prompt that ends is replaced by a new one, so every timed step has the
    same shape: 2,080 tokens, 33 rows of logits).  Token ids uniform from seed 3.  `value` is the
    step's tokens/s timed on the device; `e2e` the same with host token ids in from pinned memory and
    the sampled ids back on the host every step.  The roofline is the slower of the step's bytes
    (weights once, keys/values and states of the live requests) at the measured copy rate and its
    flops at the measured bf16 rate."""
    import torch

    from poor_mans_mamba_b200.engine.runner import StepEntry
    from poor_mans_mamba_b200.entry import Engine

    n_dec, n_pf, chunk, prompt_total = 32, 4, 512, 2048
    K_steps, W = args.steps, args.warmup
    rng = random.Random(3)
    vocab = cfg["vocab_size"]
    hi = args.context - K_steps - W - 2
    contexts = [1024 + (hi - 1024) * i // (n_dec - 1) for i in range(n_dec)]
    with torch.cuda.device(0):
        eng = Engine(model_dir, dtype=args.dtype, max_tokens=n_dec * (args.context + 64) + (n_pf + 1) * (prompt_total + 64),
                     max_seqs=n_dec + n_pf + 1, page_size=64, max_batched_tokens=8192, max_seq_len=args.context + 64)
        runner = eng.runner
        dec = [("dec", i) for i in range(n_dec)]
        for r, c in zip(dec, contexts):
            runner.step([StepEntry(r, [rng.randrange(vocab) for _ in range(c)], [])])
        serial = [0]

        # every prompt's token ids exist on the host before the timed regions, as a request's do
        prompt_ids = [[rng.randrange(vocab) for _ in range(prompt_total)] for _ in range(2 * K_steps + W + n_pf + 4)]

        def new_prompt():
            serial[0] += 1
            return [("pf", serial[0]), prompt_ids[serial[0] % len(prompt_ids)], 0]

        prompts = []
        for j in range(n_pf):  # prompt j starts j portions deep
            p = new_prompt()
            for _ in range(j):
                runner.step([StepEntry(p[0], p[1][p[2]:p[2] + chunk], [])])
                p[2] += chunk
            prompts.append(p)

        def one_step(fetch: bool):
            entries = [StepEntry(r, [rng.randrange(vocab)], [0]) for r in dec]
            for p in prompts:
                last = p[2] + chunk == prompt_total
                entries.append(StepEntry(p[0], p[1][p[2]:p[2] + chunk], [chunk - 1] if last else []))
            logits = runner.step(entries)
            ids = eng.sampler.sample(logits) if fetch else eng.sampler.sample_device(logits)
            for j, p in enumerate(prompts):
                p[2] += chunk
                if p[2] == prompt_total:
                    runner.finish(p[0])
                    prompts[j] = new_prompt()
            return ids

        for _ in range(W + 2):  # the second occurrence of the shape records its graph
            one_step(False)
        torch.cuda.synchronize()
        if args.profile_steps:  # one step between the profiler's marks, for `ncu --profile-from-start off`
            torch.cuda.profiler.start()
            one_step(False)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
            print(json.dumps({"profile_steps": "done", "workload": "mixed", "layers": cfg["num_hidden_layers"]}))
            return 0
        launches0 = runner.mark_launches()
        with ClockSampler() as clocks:
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(K_steps + 1)]
            marks[0].record()
            for s in range(K_steps):
                one_step(False)
                marks[s + 1].record()
            torch.cuda.synchronize()
        ms = marks[0].elapsed_time(marks[-1]) / K_steps
        launches = runner.kernels_launched_since(launches0)
        h2d0 = runner.h2d_bytes
        t0 = time.perf_counter()
        for _ in range(K_steps):
            one_step(True)
        e2e_s = (time.perf_counter() - t0) / K_steps
        h2d = (runner.h2d_bytes - h2d0) // K_steps
        runner.check_kernels(wait=True)

    T = n_dec + n_pf * chunk
    ctx_mid = [c + W + 2 + K_steps // 2 for c in contexts]
    depths = [k * chunk for k in range(n_pf)]
    L, Hq, Dh = cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["head_dim"]
    read_bytes = (nums["weight_bytes_per_step"] + sum(nums["kv_bytes_per_token"] * c for c in ctx_mid)
                  + sum(nums["kv_bytes_per_token"] * d for d in depths) + (n_dec + n_pf) * nums["state_bytes_per_seq"])
    attn_flops = L * 4 * Hq * Dh * (sum(ctx_mid) + sum(chunk * d + chunk * (chunk + 1) // 2 for d in depths))
    flops = T * (nums["flops_per_token_matmul"] + nums["ssd_flops_per_token"]) + attn_flops + 33 * nums["head_flops_per_row"]
    t_bytes = read_bytes / (peaks["hbm_gbs"] * 1e9)
    t_flops = flops / (peaks["bf16_tflops"] * 1e12)
    bound = "hbm" if t_bytes >= t_flops else "tensor"
    record = config_record(cfg, args, full_layers)
    record.update({"global_batch": n_dec + n_pf, "decode_requests": n_dec, "prompt_portions": n_pf, "portion_tokens": chunk})
    result = {
        "metric": f"mixed-step tokens/s (32 decoding requests + 4 x 512 prompt tokens, Falcon-H1-{args.sizes.upper()} layer sizes)",
        "value": round(T / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": K_steps, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: uniform random token ids (seed 3), random-init weights (seed 2)",
        "config": record, "clocks": clocks.summary(),
        "e2e": {"value": round(T / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4 * 33},
        "gpu_launches": int(launches),
        "roofline": {"bound": bound, "ms_at_peak": round(max(t_bytes, t_flops) * 1e3, 4),
                     "frac": round(max(t_bytes, t_flops) * 1e3 / ms, 4), "read_gb": round(read_bytes / 1e9, 3),
                     "tflop": round(flops / 1e12, 3), "frac_hbm": round(t_bytes * 1e3 / ms, 4),
                     "frac_tensor": round(t_flops * 1e3 / ms, 4), "peak_source": peaks["source"]},
        "impl": "ours", "checked": checked is not None,
    }
    if checked is not None:
        result["check"] = checked
    print(json.dumps(result))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096, help="context length at which decoding ends")
    ap.add_argument("--sizes", default=None, choices=["0.5b"] + sorted(OTHER_SIZES),
                    help="layer sizes; 0.5b is the benchmark's configuration, the others are for measurements "
                         "beside it (give --layers: a few layers of them already fill the memory system)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has "
                    "(same layer sizes) where memory or time needs it")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed", "serve"],
                    help="decode: the benchmark (decode steps of a batch, with prefill and other points beside it); "
                         "mixed: one step of 32 decoding requests at contexts of 1,024..4,096 tokens beside four "
                         "prompt portions of 512 tokens, by default at Falcon-H1-1.5B-Deep layer sizes; "
                         "serve: bursts of 32 requests with prompts of 200..1,500 tokens and 128 generated tokens "
                         "each through Engine.generate (--steps / 8 timed bursts), tokens/s of wall time")
    ap.add_argument("--no-check", dest="check", action="store_false",
                    help="skip the comparison with the plain implementation that runs before the timing: the first "
                         "two layers of the run's model, in the run's dtype, on the benchmark's schedule (a "
                         "2,048-token prompt step twice, then decode steps of a batch of 8 at contexts spread up to "
                         "--context through the CUDA graphs), every row against float64")
    ap.add_argument("--without", default="",
                    help="comma-separated names of kernel wrappers of poor_mans_mamba_b200.kernels.ops (for instance "
                         "flash_decode_attention,ssm_scan_seq) that are turned into no-ops: the results are wrong, "
                         "the shape of the step stays, and the difference in time shows what lies on the step's "
                         "critical chain (implies --no-check; the line says \"invalid\": \"without ...\")")
    ap.add_argument("--profile-steps", action="store_true",
                    help="small workload for a profiler instead of the benchmark: after an untimed set-up, one "
                         "2,048-token prefill step and two decode steps of the batch, issued kernel by kernel "
                         "(no CUDA graphs) between cudaProfilerStart and cudaProfilerStop; use with --layers 2")
    args = ap.parse_args()

    if args.sizes is None:
        args.sizes = "1.5b-deep" if args.workload == "mixed" else "0.5b"
    if args.gpus != 1:
        print(f"bench.py: this engine serves from one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)

    import torch

    from poor_mans_mamba_b200.engine.runner import StepEntry
    from poor_mans_mamba_b200.engine.scheduler import SamplingParams
    from poor_mans_mamba_b200.entry import Engine
    from poor_mans_mamba_b200.kernels import ops as K
    from poor_mans_mamba_b200.weights import write_random_model

    without = [n for n in args.without.split(",") if n]
    for name in without:
        if not callable(getattr(K, name, None)):
            print(f"bench.py: --without {name}: poor_mans_mamba_b200.kernels.ops has no such function")
            return 2
        setattr(K, name, lambda *a, **k: None)
    if without:
        args.check = False

    peaks = load_peaks()
    cfg, full_layers = sized_config(args)
    nums = model_numbers(cfg)
    K_steps, W = args.steps, args.warmup
    ctx_len = args.context
    rng = random.Random(2)
    vocab = cfg["vocab_size"]

    tmp = tempfile.mkdtemp(prefix="pmm_bench_")
    atexit.register(shutil.rmtree, tmp, ignore_errors=True)  # the model folder goes when the run ends
    t0 = time.time()
    write_random_model(cfg, seed=2, out_dir=tmp)
    print(f"[bench] wrote random model in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)

    if args.profile_steps and args.workload == "decode":
        with torch.cuda.device(0):
            eng = Engine(tmp, dtype=args.dtype, max_tokens=args.batch * (ctx_len + 64) + 4096, max_seqs=args.batch + 1,
                         page_size=64, max_batched_tokens=8192, max_seq_len=ctx_len + 64, cuda_graphs=False)
            run = eng.runner
            reqs = list(range(args.batch))
            for r in reqs:
                run.step([StepEntry(r, [rng.randrange(vocab) for _ in range(ctx_len - 8)], [])])
            run.decode_tokens(reqs, [1] * args.batch)
            run.step([StepEntry("warm", [rng.randrange(vocab) for _ in range(2048)], [2047])])
            run.finish("warm")
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            run.step([StepEntry("prefill", [rng.randrange(vocab) for _ in range(2048)], [2047])])
            run.decode_tokens(reqs, [2] * args.batch)
            run.decode_tokens(reqs, [3] * args.batch)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        print(json.dumps({"profile_steps": "done", "layers": args.layers, "batch": args.batch, "context": ctx_len}))
        return 0

    checked = None
    if args.check:
        checked = check_against_plain(cfg, args)
        print(f"[bench] checked against the plain implementation: {checked}", file=sys.stderr, flush=True)

    def make_engine(batch, end_context=None):
        end = ctx_len if end_context is None else end_context
        return Engine(tmp, dtype=args.dtype, max_tokens=batch * (end + 64), max_seqs=batch, page_size=64,
                      max_batched_tokens=8192, max_seq_len=end + 64)

    def percentile(sorted_ms, p):
        """Linear interpolation between the two nearest ranks (benchmarks/generate_bench.cpp:96-107)."""
        if not sorted_ms:
            return 0.0
        idx = (p / 100.0) * (len(sorted_ms) - 1)
        lo, hi = int(idx), min(int(idx) + 1, len(sorted_ms) - 1)
        return sorted_ms[lo] * (1.0 - (idx - lo)) + sorted_ms[hi] * (idx - lo)

    def decode_device_timed(eng, batch, steps, warmup, end_context=None):
        """tokens/s with CUDA events around `steps` decode steps of `batch` requests whose context
        ends at `end_context` (default: --context); host work (index packing, launches) runs
        concurrently and is not waited for.  An event after every step gives the time between
        tokens (mean, p50, p95 as the reference's harness reports them)."""
        end = ctx_len if end_context is None else end_context
        prompt_len = end - steps - warmup
        runner = eng.runner
        reqs = [("bench", i) for i in range(batch)]
        for r in reqs:  # prefill, untimed, in portions of <= 8192 tokens per step
            toks = [rng.randrange(vocab) for _ in range(prompt_len)]
            for a in range(0, prompt_len, 8192):
                runner.step([StepEntry(r, toks[a:a + 8192], [])])
        feed = [[rng.randrange(vocab) for _ in range(batch)] for _ in range(steps + warmup)]
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        launches0 = None
        for s in range(steps + warmup):
            if s == warmup:
                torch.cuda.synchronize()
                launches0 = runner.mark_launches()
                marks[0].record()
            # the first step feeds host ids, the others the ids the device just sampled
            runner.decode_tokens(reqs, feed[s] if s == 0 else None)
            if s >= warmup:
                marks[s - warmup + 1].record()
        torch.cuda.synchronize()
        ms = marks[0].elapsed_time(marks[-1])
        gaps = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
        itl = {"mean": round(ms / steps, 4), "p50": round(percentile(gaps, 50.0), 4),
               "p95": round(percentile(gaps, 95.0), 4)}
        launches = runner.kernels_launched_since(launches0)
        for r in reqs:
            runner.finish(r)
        return batch * steps / (ms / 1e3), ms / steps, launches, itl

    def prefill_timed(eng, n_tokens, portions=1, reps=3):
        """Median device time of one prompt of n_tokens fed as `portions` equal steps, the wanted
        row being the last one (the reference's prefill returns that row's logits)."""
        toks = [rng.randrange(vocab) for _ in range(n_tokens)]
        cut = n_tokens // portions
        times = []
        for it in range(W + reps):
            s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s_ev.record()
            for k in range(portions):
                last = k == portions - 1
                part = toks[k * cut:] if last else toks[k * cut:(k + 1) * cut]
                eng.runner.step([StepEntry(("pf", n_tokens, portions, it), part, [len(part) - 1] if last else [])])
            e_ev.record()
            torch.cuda.synchronize()
            eng.runner.finish(("pf", n_tokens, portions, it))
            if it >= W:
                times.append(s_ev.elapsed_time(e_ev))
        return statistics.median(times)

    def prefill_flops(T):
        return (T * (nums["flops_per_token_matmul"] + nums["ssd_flops_per_token"]) + nums["attn_flops"](T)
                + nums["head_flops_per_row"])

    if args.workload == "mixed":
        return mixed_workload(args, cfg, full_layers, nums, peaks, tmp, checked)
    if args.workload == "serve":
        return serve_workload(args, cfg, full_layers, tmp, checked)

    result = {}
    with torch.cuda.device(0):
        eng = make_engine(args.batch)
        with ClockSampler() as clocks:
            tok_s, ms_step, launches, itl = decode_device_timed(eng, args.batch, K_steps, W)
        clock_summary = clocks.summary()

        # end to end through the entry point: scheduler + pinned host ids in + sampled ids out
        # No request may end (and no batch shrink) inside the timed steps.  Requests whose prompts are
        # done early decode while the others' prompts still run in portions, one token per such step,
        # so every request is allowed that many more tokens, and its prompt is that much shorter.
        prefill_steps = -(-args.batch * ctx_len // 8192) + args.batch
        new_tokens = K_steps + W + 32 + prefill_steps
        prompt_len = ctx_len - new_tokens
        if prompt_len < 1:
            raise SystemExit("bench.py: --context is too short for this batch's prompts to be cut into portions")
        ids = [eng.submit([rng.randrange(vocab) for _ in range(prompt_len)],
                          SamplingParams(max_new_tokens=new_tokens, eos_id=-1)) for _ in range(args.batch)]
        while any(r.pending > 1 or r.status == "waiting" for r in eng.scheduler.requests.values() if not r.finished):
            eng.step()
        for _ in range(W):
            eng.step()
        torch.cuda.synchronize()
        gc.collect()
        gc.disable()  # a collection of the whole heap inside the timed loop costs tens of milliseconds
        h2d0 = eng.runner.h2d_bytes
        decoded0 = eng.scheduler.counters["decode_tokens"]
        replays0 = eng.runner.graphs.replays if eng.runner.graphs is not None else 0
        t1 = time.perf_counter()
        step_times = []
        for _ in range(K_steps - 1):
            ts = time.perf_counter()
            eng.step()
            step_times.append(time.perf_counter() - ts)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t1
        gc.enable()
        if os.environ.get("PMM_BENCH_DEBUG"):
            print("[bench] e2e step ms:", " ".join(f"{t * 1e3:.2f}" for t in step_times), file=sys.stderr)
            print("[bench] preemptions:", eng.scheduler.counters, file=sys.stderr)
            print("[bench] graph replays in the timed end-to-end steps:",
                  (eng.runner.graphs.replays - replays0) if eng.runner.graphs is not None else None,
                  "lengths", sorted(set(eng.cache.lengths.values()))[:4], file=sys.stderr)
        e2e_steps = K_steps - 1
        e2e_tokens = eng.scheduler.counters["decode_tokens"] - decoded0  # what the timed steps really decoded
        assert e2e_tokens == args.batch * e2e_steps, (e2e_tokens, args.batch, e2e_steps)
        h2d_per_step = (eng.runner.h2d_bytes - h2d0) // e2e_steps
        while eng.has_work():
            eng.step()
        assert all(len(eng.poll(i).tokens) == new_tokens for i in ids)
        e2e = {"value": e2e_tokens / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": int(h2d_per_step),
               "d2h_bytes_per_step": 4 * args.batch}

        read_bytes = nums["weight_bytes_per_step"] + args.batch * (
            nums["kv_bytes_per_token"] * (ctx_len - K_steps // 2) + nums["state_bytes_per_seq"])
        achieved = read_bytes / (ms_step / 1e3) / 1e9
        roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peaks["source"]}

        prefill, points, extra = None, {}, {}
        if not args.no_points:
            T = 2048
            pf_ms = prefill_timed(eng, T)
            flops = prefill_flops(T)
            prefill = {"value": round(T / (pf_ms / 1e3), 1), "tokens": T, "ms": round(pf_ms, 3),
                       "frac": round(flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4),
                       "flops": flops, "peak_tflops": peaks["bf16_tflops"], "peak_source": peaks["source"]}
            # the same prompt as four portions of 512 tokens, and the prompt lengths of the reference's
            # harness (benchmarks/generate_bench.cpp:45-47), each as one step
            ms4 = prefill_timed(eng, T, portions=4)
            extra["prefill_4x512"] = {"value": round(T / (ms4 / 1e3), 1), "ms": round(ms4, 3)}
            sweep = {}
            for n in (32, 128, 512, 1024):
                ms_n = prefill_timed(eng, n)
                sweep[str(n)] = {"value": round(n / (ms_n / 1e3), 1), "ms": round(ms_n, 3)}
            sweep[str(T)] = {"value": prefill["value"], "ms": prefill["ms"]}
            extra["prefill_by_length"] = sweep
            del eng
            torch.cuda.empty_cache()
            itl_points = {f"decode_b{args.batch}": itl}
            for b in (1, 64):
                if b == args.batch:
                    continue
                e = make_engine(b)
                steps_b = min(K_steps, 32)
                v, _, _, itl_b = decode_device_timed(e, b, steps_b, W)
                points[f"decode_b{b}"] = round(v, 1)
                itl_points[f"decode_b{b}"] = itl_b
                del e
                torch.cuda.empty_cache()
            # the batch again right after a 2,048-token prompt (context 2,048 -> 2,048 + steps)
            short_end = 2048 + K_steps + W
            e = make_engine(args.batch, short_end)
            v, _, _, itl_short = decode_device_timed(e, args.batch, K_steps, W, short_end)
            points[f"decode_b{args.batch}_ctx2048"] = round(v, 1)
            itl_points[f"decode_b{args.batch}_ctx2048"] = itl_short
            del e
            torch.cuda.empty_cache()
            extra["itl_ms"] = itl_points
        else:
            extra["itl_ms"] = {f"decode_b{args.batch}": itl}

    result = {
        "metric": f"decode tokens/s (Falcon-H1-{args.sizes.upper()} layer sizes, random weights)", "value": round(tok_s, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": K_steps, "warmup": W, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: uniform random token ids (seed 2), random-init weights (seed 2)",
        "config": config_record(cfg, args, full_layers),
        "clocks": clock_summary, "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(launches), "roofline": roofline, "impl": "ours",
    }
    result.update(extra)
    if without:
        result["invalid"] = "without " + ",".join(without)
    result["checked"] = checked is not None
    if checked is not None:
        result["check"] = checked
    if prefill is not None:
        result["prefill"] = prefill
    if points:
        result["points"] = points
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
