"""Drop-in for the reference's scripts/sx8_fused_wmma.py (ref :60-104):

    make_tensors(qt_kbmajor, bases_info, device) -> dict
    gemm_sx8_wmma_cached(X, tensors, n_cb) -> Y f32 (M, N)
    gemm_sx8_wmma(X, qt_kbmajor, bases_info, n_cb) -> Y f32 (M, N)
    decode1_sx8_cached(X, tensors, n_cb) -> Y f32 (N,)

The reference keeps ten planar kb-major arrays per tensor (44 B/block more than the
packed data, ref :69-87).  Here the dict carries the same keys for the planes the
callers may look at, and the kernels run from the 30 B/block hdr/levels pair that is
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


def _v44(tensors):
    v = tensors.get("_v44")
    if v is None:
        n_blk = tensors["config"].numel()
        hdr = torch.cat([tensors["dmin"].view(torch.uint8).reshape(n_blk, 2),
                         tensors["dmax"].view(torch.uint8).reshape(n_blk, 2),
                         tensors["config"].reshape(n_blk, 1), tensors["coeff"].reshape(n_blk, 1)], dim=1).contiguous()
        lev = torch.cat([tensors["hi"].reshape(n_blk, 16), tensors["lo"].reshape(n_blk, 8)], dim=1).contiguous()
        v = (hdr, lev, tensors["basis"].reshape(-1, 64), tensors["scales"].reshape(-1, 2))
        tensors["_v44"] = v
    return v


def gemm_sx8_wmma_cached(X, tensors, n_cb):
    hdr, lev, bas, sca = _v44(tensors)
    n_cb = int(n_cb)
    N = hdr.shape[0] // n_cb
    Xc = X.contiguous().half()
    return ops.gemm(Xc, hdr, lev, bas, sca, N, min(int(Xc.shape[1]), n_cb * 32), n_cb, 6,
                    out_dtype=torch.float32)


def gemm_sx8_wmma(X, qt_kbmajor, bases_info, n_cb):
    return gemm_sx8_wmma_cached(X, make_tensors(qt_kbmajor, bases_info, X.device), n_cb)


def decode1_sx8_cached(X, tensors, n_cb):
    hdr, lev, bas, sca = _v44(tensors)
    n_cb = int(n_cb)
    N = hdr.shape[0] // n_cb
    Xc = X.contiguous().half().reshape(1, -1)
    return ops.gemv(Xc, hdr, lev, bas, sca, N, min(int(Xc.shape[1]), n_cb * 32), n_cb, 6)[0]
