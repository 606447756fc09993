"""Drop-in for the reference's scripts/sx8_decode1_v3.py: same public names, argument
meaning and return values (ref scripts/sx8_decode1_v3.py:57-110), backed by
libsx8b200.so instead of a JIT-compiled torch extension.

    make_tensors_v44(qt, bases_info, hdr_aligned=False) -> (hdr_t, lvl_t, bas_t, sca_t)
    best_split_k(N, n_cb) -> int
    decode1_v44(X, qt, bases_info, hdr_t, lvl_t, bas_t, sca_t, hdr_bytes=6, split_k=1)
        -> (Y f32 (N,), tensors)

Differences, all outside the numerical contract: the file planes are uploaded once and
transposed to the kb-major layout by a device kernel (the reference transposes with
numpy on the host, ref scripts/prepare_v44.py:35-79); X may also be (M, K) with
M <= 8, in which case Y is (M, N); split_k is accepted and ignored exactly as the
reference ignores it (ref cuda/sx8_decode1_v3.cu:206-218) -- the kernel picks its own
deterministic cluster split."""
import numpy as np
import torch

from . import ops

DEV = torch.device("cuda")


def _dev_u8(a, device):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1)).to(device, non_blocking=False)


def make_tensors_v44(qt, bases_info, hdr_aligned=False, device=None):
    """ref scripts/sx8_decode1_v3.py:57-66.  Returns CUDA tensors hdr (n_blk,6|8) u8,
    levels (n_blk,24) u8, bases (n_cb,64) f32, scales (n_cb,2) f32, kb-major."""
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    out_f, _ = qt["shape"]
    n_cb = int(qt["n_cb"])
    f16 = lambda a: _dev_u8(np.asarray(a).reshape(-1).astype(np.float16, copy=False), device)
    u8 = lambda a: _dev_u8(np.asarray(a).reshape(-1).astype(np.uint8, copy=False), device)
    hdr_t, lvl_t = ops.repack_v44(f16(qt["dmin"]), f16(qt["dmax"]), u8(qt["config"]), u8(qt["coeff"]),
                                  u8(qt["levels_hi"]), u8(qt["levels_lo"]), out_f, n_cb,
                                  8 if hdr_aligned else 6)
    bas_t = torch.from_numpy(np.ascontiguousarray(np.asarray(bases_info["data"]).reshape(-1, 64),
                                                  dtype=np.float32)).to(device)
    sca_t = torch.from_numpy(np.ascontiguousarray(np.asarray(bases_info["scales"]).reshape(-1, 2),
                                                  dtype=np.float32)).to(device)
    return hdr_t, lvl_t, bas_t, sca_t


def best_split_k(N, n_cb):
    """ref scripts/sx8_decode1_v3.py:69-77 (kept for callers; the value is advisory)."""
    n_blocks = (N + 63) // 64
    want = 540
    sk = max(1, (want + n_blocks - 1) // n_blocks)
    return min(sk, 16)


_BUF = {}


def _buf(key, shape, device):
    """Pooled fp32 output buffers, as ref scripts/sx8_decode1_v3.py:80-88: the returned
    Y aliases the pool and is overwritten by the next call with the same shape."""
    key = (key, device.index)
    b = _BUF.get(key)
    if b is None or tuple(b.shape) != tuple(shape):
        b = torch.empty(*shape, dtype=torch.float32, device=device)
        _BUF[key] = b
    return b


def decode1_v44(X, qt, bases_info, hdr_t=None, lvl_t=None, bas_t=None, sca_t=None,
                hdr_bytes=6, split_k=1):
    """ref scripts/sx8_decode1_v3.py:91-110."""
    if hdr_t is None:
        hdr_t, lvl_t, bas_t, sca_t = make_tensors_v44(qt, bases_info, hdr_aligned=(hdr_bytes == 8),
                                                      device=X.device if X.is_cuda else None)
    n_cb = int(qt["n_cb"])
    N = int(qt["shape"][0])
    Xc = X.contiguous().half()
    one_d = Xc.dim() == 1
    K = Xc.shape[-1]
    M = 1 if one_d else Xc.shape[0]
    Y = _buf(("Y", N, M), (M, N), Xc.device)
    ops.gemv(Xc, hdr_t, lvl_t, bas_t, sca_t, N, K, n_cb, hdr_bytes, out=Y)
    return (Y[0] if one_d else Y), (hdr_t, lvl_t, bas_t, sca_t)
