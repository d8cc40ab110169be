"""The hand-written CUDA kernels (sources under ``csrc/``) and their Python face."""
