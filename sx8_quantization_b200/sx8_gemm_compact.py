"""Drop-in for the reference's scripts/sx8_gemm_compact.py (ref :42-74):

    gemm_sx8_compact(X, qt, bases_info, hdr_t, lvl_t, bas_t, sca_t, hdr_bytes=6,
                     in_f=None, n_cb=None) -> Y f32 (M, N)

X (M, K) f16 CUDA; K shorter than n_cb*32 is zero-extended inside the kernel (the
reference pads X on the host, ref :66-71).  The reference decodes tensors with fewer
than 64 rows to fp16 and calls a library matmul (ref :54-59); here every N runs on the
fused kernels (the T16 layout pads the last 16-column tile with zero blocks)."""
import torch

from . import ops


def gemm_sx8_compact(X, qt, bases_info, hdr_t=None, lvl_t=None, bas_t=None, sca_t=None,
                     hdr_bytes=6, in_f=None, n_cb=None):
    if in_f is None:
        in_f = qt["shape"][1]
    if n_cb is None:
        n_cb = qt["n_cb"]
    out_f = int(qt["shape"][0])
    if lvl_t is None:
        from .sx8_decode1_v3 import make_tensors_v44
        hdr_t, lvl_t, bas_t, sca_t = make_tensors_v44(qt, bases_info, hdr_aligned=(hdr_bytes == 8),
                                                      device=X.device)
    Xc = X.contiguous().half()
    K = min(int(Xc.shape[1]), int(n_cb) * 32)
    return ops.gemm(Xc, lvl_t, bas_t, sca_t, out_f, K, int(n_cb), out_dtype=torch.float32)
