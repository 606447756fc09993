"""S-X8 v4.3 hot path for NVIDIA B200 (sm_100a): decode GEMV, prefill GEMM, embedding
rows, full-tensor decode and the quantizer's per-block search, as hand-written CUDA
kernels behind a C ABI (libsx8b200.so, include/sx8_b200.h), with drop-in replacements
for the reference's Python wrapper modules."""
__version__ = "0.1.0"
