"""Drop-in for the reference's scripts/sx8_decode1_v3.py: same public names, argument
meaning and return values (ref scripts/sx8_decode1_v3.py:57-110), backed by
libsx8b200.so instead of a JIT-compiled torch extension.

    make_tensors_v44(qt, bases_info, hdr_aligned=False) -> (hdr_t, lvl_t, bas_t, sca_t)
    best_split_k(N, n_cb) -> int
    decode1_v44(X, qt, bases_info, hdr_t, lvl_t, bas_t, sca_t, hdr_bytes=6, split_k=1)
        -> (Y f32 (N,), tensors)

Differences, all outside the numerical contract: the file planes are uploaded once and
permuted on the device into this library's T16 layout (the reference transposes with
numpy on the host into its kb-major v4.4 pair, ref scripts/prepare_v44.py:35-79), so
in the returned tuple `lvl_t` is the T16 blob and `hdr_t` a small descriptor
[N, n_cb]; callers treat the tuple as opaque, as the reference's do; hdr_aligned /
hdr_bytes=8 (the reference's padded-header experiment) are accepted and map to the same
30-byte layout; X may also be (M, K) with
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
    """ref scripts/sx8_decode1_v3.py:57-66.  Returns (hdr_t, lvl_t, bas_t, sca_t):
    hdr_t = int64 descriptor [N, n_cb] (host), lvl_t = T16 blob (units, 480) u8 CUDA,
    bas_t (n_cb,64) f32, sca_t (n_cb,2) f32."""
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    out_f, _ = qt["shape"]
    n_cb = int(qt["n_cb"])
    f16 = lambda a: _dev_u8(np.asarray(a).reshape(-1).astype(np.float16, copy=False), device)
    u8 = lambda a: _dev_u8(np.asarray(a).reshape(-1).astype(np.uint8, copy=False), device)
    lvl_t = ops.repack_t16(f16(qt["dmin"]), f16(qt["dmax"]), u8(qt["config"]), u8(qt["coeff"]),
                           u8(qt["levels_hi"]), u8(qt["levels_lo"]), int(out_f), n_cb)
    hdr_t = torch.tensor([int(out_f), n_cb], dtype=torch.int64)
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


def _buf(N, M, device):
    """Pooled fp32 output buffers, as ref scripts/sx8_decode1_v3.py:80-88: the returned
    Y aliases the pool and is overwritten by the next call with the same N (and batch).
    Returns (Y (M,N), its row 0 as a 1-D view)."""
    key = (N, M, device.index)
    b = _BUF.get(key)
    if b is None:
        y = torch.empty(M, N, dtype=torch.float32, device=device)
        b = _BUF[key] = (y, y[0])
    return b


def decode1_v44(X, qt, bases_info, hdr_t=None, lvl_t=None, bas_t=None, sca_t=None,
                hdr_bytes=6, split_k=1):
    """ref scripts/sx8_decode1_v3.py:91-110.  Launched with programmatic dependent launch: when
    the previous kernel on the stream is another of this library's, the weight stream of this
    call starts under its tail."""
    if lvl_t is None:
        hdr_t, lvl_t, bas_t, sca_t = make_tensors_v44(qt, bases_info, hdr_aligned=(hdr_bytes == 8),
                                                      device=X.device if X.is_cuda else None)
    n_cb = qt["n_cb"]
    N = qt["shape"][0]
    if X.dtype is not torch.float16 or not X.is_contiguous():
        X = X.contiguous().half()
    one_d = X.dim() == 1
    K = X.shape[-1]
    Y, Y0 = _buf(N, 1 if one_d else X.shape[0], X.device)
    ops.gemv(X, lvl_t, bas_t, sca_t, N, K if K < n_cb * 32 else n_cb * 32, n_cb, out=Y, flags=ops.SX8_F_PDL)
    return (Y0 if one_d else Y), (hdr_t, lvl_t, bas_t, sca_t)
