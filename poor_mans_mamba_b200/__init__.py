"""poor_mans_mamba_b200: a single-GPU inference engine for the Falcon-H1 hybrid
architecture on NVIDIA B200 (sm_100a): typed config and registry, safetensors loading and
a random-weights mode, layers built from parts, a paged cache with fixed-state slots, one
step function for mixed prefill/decode batches, a scheduler with greedy and temperature
sampling, trace replay, and hand-written CUDA kernels with a true float32 path."""
__version__ = "0.1.0"
