"""Drop-in for the reference's scripts/sx8_fused_wmma.py (ref :60-104):

    make_tensors(qt_kbmajor, bases_info, device) -> dict
    gemm_sx8_wmma_cached(X, tensors, n_cb) -> Y f32 (M, N)
    gemm_sx8_wmma(X, qt_kbmajor, bases_info, n_cb) -> Y f32 (M, N)
    decode1_sx8_cached(X, tensors, n_cb) -> Y f32 (N,)

The reference keeps ten planar kb-major arrays per tensor (44 B/block more than the
packed data, ref :69-87).  Here the dict carries the same keys for the planes the
callers may look at, and the kernels run from the 30 B/block T16 blob that is
assembled once, on the device, from those planes."""
import numpy as np
import torch

from . import ops


def make_tensors(qt_kbmajor, bases_info, device):
    dev = torch.device(device)
    t = {
        "rlo": None, "step": None,  # legacy fp16 tables of the superseded M=1 kernel: not built
        "dmin": torch.as_tensor(np.asarray(qt_kbmajor["dmin"], dtype=np.float16), device=dev),
        "dmax": torch.as_tensor(np.asarray(qt_kbmajor["dmax"], dtype=np.float16), device=dev),
        "config": torch.as_tensor(np.asarray(qt_kbmajor["config"], dtype=np.uint8), device=dev),
        "coeff": torch.as_tensor(np.asarray(qt_kbmajor["coeff"], dtype=np.uint8).reshape(-1), device=dev),
        "hi": torch.as_tensor(np.asarray(qt_kbmajor["levels_hi"], dtype=np.uint8), device=dev),
        "lo": torch.as_tensor(np.asarray(qt_kbmajor["levels_lo"], dtype=np.uint8), device=dev),
        "basis": torch.as_tensor(np.asarray(bases_info["data"]).reshape(-1).astype(np.float32), device=dev),
        "scales": torch.as_tensor(np.asarray(bases_info["scales"]).reshape(-1).astype(np.float32), device=dev),
    }
    return t


def _t16(tensors, n_cb):
    """Planar kb-major arrays (bid = kb*N + n) -> T16 blob, once per tensor, on the device."""
    v = tensors.get("_t16")
    if v is None:
        n_blk = tensors["config"].numel()
        N = n_blk // n_cb
        nm = lambda a, per: a.reshape(n_cb, N, per).transpose(0, 1).contiguous().reshape(-1)
        wt = ops.repack_t16(nm(tensors["dmin"].view(torch.uint8), 2), nm(tensors["dmax"].view(torch.uint8), 2),
                            nm(tensors["config"], 1), nm(tensors["coeff"], 1), nm(tensors["hi"], 16),
                            nm(tensors["lo"], 8), N, n_cb)
        v = (wt, tensors["basis"].reshape(-1, 64), tensors["scales"].reshape(-1, 2), N)
        tensors["_t16"] = v
    return v


def gemm_sx8_wmma_cached(X, tensors, n_cb):
    n_cb = int(n_cb)
    wt, bas, sca, N = _t16(tensors, n_cb)
    Xc = X.contiguous().half()
    return ops.gemm(Xc, wt, bas, sca, N, min(int(Xc.shape[1]), n_cb * 32), n_cb, out_dtype=torch.float32)


def gemm_sx8_wmma(X, qt_kbmajor, bases_info, n_cb):
    return gemm_sx8_wmma_cached(X, make_tensors(qt_kbmajor, bases_info, X.device), n_cb)


def decode1_sx8_cached(X, tensors, n_cb):
    n_cb = int(n_cb)
    wt, bas, sca, N = _t16(tensors, n_cb)
    Xc = X.contiguous().half().reshape(1, -1)
    return ops.gemv(Xc, wt, bas, sca, N, min(int(Xc.shape[1]), n_cb * 32), n_cb)[0]
