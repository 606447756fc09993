"""Tensor-level entry points over the C ABI: PyTorch supplies device memory and the
current CUDA stream, the library does the work.  Every function validates devices and
dtypes, and raises SX8Error on any failure; none has a fallback path."""
import torch

from . import _lib
from ._lib import SX8Error, SX8_F_PDL  # noqa: F401


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _need(t, dtype, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise SX8Error("%s must be a CUDA tensor" % name)
    if t.dtype != dtype:
        raise SX8Error("%s must be %s (got %s)" % (name, dtype, t.dtype))
    if not t.is_contiguous():
        raise SX8Error("%s must be contiguous" % name)
    return t


class Workspace:
    """Grow-only device scratch buffers, one per (device, stream, tag); the analogue of the
    reference's pooled Z/Y buffers (ref scripts/sx8_decode1_v3.py:80-88).  Calls on different
    streams get different buffers (a workspace is private to a call until it completes on its
    stream).  A buffer that is outgrown is kept alive, never freed: a CUDA graph captured
    earlier may have its address baked in."""
    _bufs = {}
    _retired = []

    @classmethod
    def get(cls, device, nbytes, tag="gemv"):
        idx = device.index if device.index is not None else torch.cuda.current_device()
        key = (idx, torch.cuda.current_stream(idx).cuda_stream, tag)
        b = cls._bufs.get(key)
        if b is None or b.numel() < nbytes:
            if b is not None:
                cls._retired.append(b)
            b = torch.empty(max(int(nbytes), 1 << 16), dtype=torch.uint8, device=device)
            cls._bufs[key] = b
        return b


def _wt(wt16, N, n_cb):
    _need(wt16, torch.uint8, "wt16")
    need = _lib.lib().sx8_t16_bytes(N, n_cb)
    if wt16.numel() != need:
        raise SX8Error("wt16 has %d bytes, the T16 layout of (N=%d, n_cb=%d) has %d" % (wt16.numel(), N, n_cb, need))
    return wt16


_NO_WS = None


def _no_workspace(device):
    """Stand-in passed to the torch binding when a call needs no staging (never dereferenced)."""
    global _NO_WS
    if _NO_WS is None or _NO_WS.device != device:
        _NO_WS = torch.empty(0, dtype=torch.uint8, device=device)
    return _NO_WS


def gemv(x, wt16, bases, scales, N, K, n_cb, out=None, flags=0, workspace=None):
    """y (M,N) f32 = x (M,K) f16 times the packed matrix (T16 blob); M in 1..8."""
    if x.dim() == 1:
        x = x.unsqueeze(0)
    if not x.is_cuda or x.dtype != torch.float16:
        raise SX8Error("x must be a CUDA float16 tensor")
    if x.stride(1) != 1 or x.stride(0) < x.shape[1]:
        x = x.contiguous()
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    if workspace is None:
        # scratch is only used to stage activations that bulk copies cannot fetch as they are
        if (K & 31) or (x.stride(0) & 7) or (x.data_ptr() & 15):
            workspace = Workspace.get(x.device, _lib.lib().sx8_gemv_workspace_bytes(n_cb, M))
    E = _lib.ext()
    if E is not None:
        try:
            rc = E.gemv(x, wt16, bases, scales, N, K, n_cb, out, workspace if workspace is not None else _no_workspace(x.device),
                        flags)
        except RuntimeError as e:       # argument checks of the binding
            raise SX8Error(str(e).split("\n")[0]) from None
        if rc:
            _lib.check(rc, "sx8_gemv")
        return out
    _wt(wt16, N, n_cb)
    _need(bases, torch.float32, "bases"); _need(scales, torch.float32, "scales")
    _need(out, torch.float32, "out")
    if out.numel() != M * N:
        raise SX8Error("out has %d elements, need %d" % (out.numel(), M * N))
    L = _lib.lib()
    ws = workspace
    with torch.cuda.device(x.device):
        rc = L.sx8_gemv(x.data_ptr(), M, K, x.stride(0), wt16.data_ptr(), bases.data_ptr(), scales.data_ptr(),
                        N, n_cb, out.data_ptr(), ws.data_ptr() if ws is not None else None,
                        ws.numel() if ws is not None else 0, flags, _stream(x))
    _lib.check(rc, "sx8_gemv")
    return out


class MultiGemv:
    """Prepared argument block for sx8_gemv_multi: up to four matrices that share x (q|k|v,
    gate|up) run in one launch.  Build once per group of tensors, call per step."""

    def __init__(self, tensors, M, device):
        import ctypes
        if not 1 <= len(tensors) <= 4:
            raise SX8Error("1..4 matrices per launch")
        self.n_cb = tensors[0]["n_cb"]
        self.K = tensors[0]["K"]
        if any(t["n_cb"] != self.n_cb or t["K"] != self.K for t in tensors):
            raise SX8Error("all matrices of a launch must have the same K")
        n = len(tensors)
        self.tensors = tensors
        self.M = M
        self.outs = [torch.empty((M, t["N"]), dtype=torch.float32, device=device) for t in tensors]
        VP, I = ctypes.c_void_p * n, ctypes.c_int * n
        self._wt = VP(*[t["wt16"].data_ptr() for t in tensors])
        self._ba = VP(*[t["bases"].data_ptr() for t in tensors])
        self._sc = VP(*[t["scales"].data_ptr() for t in tensors])
        self._y = VP(*[o.data_ptr() for o in self.outs])
        self._N = I(*[t["N"] for t in tensors])
        self.count = n

    def __call__(self, x, flags=0, workspace=None):
        if x.dtype != torch.float16 or not x.is_cuda or x.shape[0] != self.M or x.stride(1) != 1:
            raise SX8Error("x must be CUDA float16 (M, K) with unit inner stride")
        L = _lib.lib()
        ws = workspace if workspace is not None else Workspace.get(x.device, L.sx8_gemv_workspace_bytes(self.n_cb, self.M))
        with torch.cuda.device(x.device):
            rc = L.sx8_gemv_multi(x.data_ptr(), self.M, self.K, x.stride(0), self.count, self._wt, self._ba, self._sc,
                                  self._N, self._y, self.n_cb, ws.data_ptr(), ws.numel(), flags, _stream(x))
        _lib.check(rc, "sx8_gemv_multi")
        return self.outs


class MultiGemm:
    """Prepared argument block for sx8_gemm_multi: up to three matrices that share x (q|k|v,
    gate|up) in one tensor-core launch.  Build once per group of tensors; every call returns new
    output tensors (M may differ between calls)."""

    def __init__(self, tensors):
        import ctypes
        if not 1 <= len(tensors) <= 3:
            raise SX8Error("1..3 matrices per launch")
        self.n_cb = tensors[0]["n_cb"]
        self.K = tensors[0]["K"]
        if any(t["n_cb"] != self.n_cb or t["K"] != self.K for t in tensors):
            raise SX8Error("all matrices of a launch must have the same K")
        n = len(tensors)
        self.tensors = tensors
        VP, I = ctypes.c_void_p * n, ctypes.c_int * n
        self._VP = VP
        self._wt = VP(*[t["wt16"].data_ptr() for t in tensors])
        self._ba = VP(*[t["bases"].data_ptr() for t in tensors])
        self._sc = VP(*[t["scales"].data_ptr() for t in tensors])
        self._N = I(*[t["N"] for t in tensors])
        self.count = n

    def __call__(self, x, out_dtype=torch.float32, outs=None, workspace=None):
        if x.dtype != torch.float16 or not x.is_cuda or x.dim() != 2 or x.stride(1) != 1:
            raise SX8Error("x must be CUDA float16 (M, K) with unit inner stride")
        if out_dtype not in (torch.float32, torch.float16):
            raise SX8Error("out_dtype must be float32 or float16")
        M = x.shape[0]
        if outs is None:
            outs = [torch.empty((M, t["N"]), dtype=out_dtype, device=x.device) for t in self.tensors]
        elif any(o.dtype != out_dtype or o.shape != (M, t["N"]) or not o.is_contiguous() for o, t in zip(outs, self.tensors)):
            raise SX8Error("outs must be contiguous (M, N_i) tensors of out_dtype")
        L = _lib.lib()
        need = L.sx8_gemm_multi_workspace_bytes(M, self.count, self._N, self.n_cb)
        ws = workspace if workspace is not None else Workspace.get(x.device, need, tag="gemm")
        y = self._VP(*[o.data_ptr() for o in outs])
        with torch.cuda.device(x.device):
            rc = L.sx8_gemm_multi(x.data_ptr(), M, self.K, x.stride(0), self.count, self._wt, self._ba, self._sc, self._N,
                                  y, int(out_dtype == torch.float16), self.n_cb, ws.data_ptr(), ws.numel(), _stream(x))
        _lib.check(rc, "sx8_gemm_multi")
        return outs


def gemv_allreduce(x, wt16, bases, scales, N, K, n_cb, peers, out=None, flags=0, workspace=None):
    """Row-parallel partial GEMV fused with its all-reduce over peer memory: y (M,N) f32 on
    every rank = sum over ranks of x_r @ W_r^T.  `peers` is a _lib.Peers descriptor."""
    if x.dim() == 1:
        x = x.unsqueeze(0)
    if not x.is_cuda or x.dtype != torch.float16:
        raise SX8Error("x must be a CUDA float16 tensor")
    if x.stride(1) != 1 or x.stride(0) < x.shape[1]:
        x = x.contiguous()
    M = x.shape[0]
    _wt(wt16, N, n_cb)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    L = _lib.lib()
    need = L.sx8_gemv_workspace_bytes(n_cb, M)
    ws = workspace if workspace is not None else Workspace.get(x.device, need)
    import ctypes
    with torch.cuda.device(x.device):
        rc = L.sx8_gemv_allreduce(x.data_ptr(), M, K, x.stride(0), wt16.data_ptr(), bases.data_ptr(),
                                  scales.data_ptr(), N, n_cb, out.data_ptr(), ws.data_ptr(), ws.numel(), flags,
                                  ctypes.addressof(peers), _stream(x))
    _lib.check(rc, "sx8_gemv_allreduce")
    return out


def gemm(x, wt16, bases, scales, N, K, n_cb, out_dtype=torch.float32, out=None):
    """Y (M,N) = X (M,K) f16 times the packed matrix, any M >= 1; fp32 accumulate."""
    x = _need(x.contiguous(), torch.float16, "x")
    M = x.shape[0]
    _wt(wt16, N, n_cb)
    _need(bases, torch.float32, "bases"); _need(scales, torch.float32, "scales")
    if out_dtype not in (torch.float32, torch.float16):
        raise SX8Error("out_dtype must be float32 or float16")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    else:
        _need(out, out_dtype, "out")
    if M == 0:
        return out
    L = _lib.lib()
    need = L.sx8_gemm_workspace_bytes(M, N, n_cb)
    ws = Workspace.get(x.device, need, "gemm")
    E = _lib.ext()
    if E is not None:
        try:
            rc = E.gemm(x, wt16, bases, scales, N, K, n_cb, out, ws)
        except RuntimeError as e:
            raise SX8Error(str(e).split("\n")[0]) from None
        if rc:
            _lib.check(rc, "sx8_gemm")
        return out
    with torch.cuda.device(x.device):
        rc = L.sx8_gemm(x.data_ptr(), M, K, x.stride(0), wt16.data_ptr(), bases.data_ptr(), scales.data_ptr(),
                        N, n_cb, out.data_ptr(), int(out_dtype == torch.float16), ws.data_ptr(), ws.numel(),
                        _stream(x))
    _lib.check(rc, "sx8_gemm")
    return out


def embed(ids, wt16, bases, scales, K, N, n_cb, out=None):
    """out (T,K) f16 = decoded rows ids[t] (float32 reference arithmetic)."""
    ids = _need(ids.reshape(-1).to(torch.long).contiguous(), torch.long, "ids")
    T = ids.numel()
    _wt(wt16, N, n_cb)
    if out is None:
        out = torch.empty((T, K), dtype=torch.float16, device=ids.device)
    else:
        _need(out, torch.float16, "out")
        if out.numel() < T * K:
            raise SX8Error("out too small")
    E = _lib.ext()
    if E is not None:
        try:
            rc = E.embed(ids, wt16, bases, scales, K, N, n_cb, out)
        except RuntimeError as e:
            raise SX8Error(str(e).split("\n")[0]) from None
        if rc:
            _lib.check(rc, "sx8_embed")
        return out
    with torch.cuda.device(ids.device):
        rc = _lib.lib().sx8_embed(ids.data_ptr(), T, wt16.data_ptr(), bases.data_ptr(), scales.data_ptr(),
                                  K, N, n_cb, out.data_ptr(), _stream(ids))
    _lib.check(rc, "sx8_embed")
    return out


def dequant_planes(dmin, dmax, config, coeff, hi, lo, bases, scales, out_f, in_f, n_cb, use_pca=True):
    """(out_f,in_f) f16 from n-major file planes (float64 reference arithmetic)."""
    out = torch.empty((out_f, in_f), dtype=torch.float16, device=hi.device)
    with torch.cuda.device(hi.device):
        rc = _lib.lib().sx8_dequant_planes(dmin.data_ptr(), dmax.data_ptr(), config.data_ptr(), coeff.data_ptr(),
                                           hi.data_ptr(), lo.data_ptr(), bases.data_ptr(), scales.data_ptr(),
                                           out_f, in_f, n_cb, int(use_pca), out.data_ptr(), _stream(hi))
    _lib.check(rc, "sx8_dequant_planes")
    return out


def dequant_t16(wt16, bases, scales, out_f, in_f, n_cb, use_pca=True):
    """(out_f,in_f) f16 from the T16 device blob (float64 reference arithmetic)."""
    _wt(wt16, out_f, n_cb)
    out = torch.empty((out_f, in_f), dtype=torch.float16, device=wt16.device)
    with torch.cuda.device(wt16.device):
        rc = _lib.lib().sx8_dequant_t16(wt16.data_ptr(), bases.data_ptr(), scales.data_ptr(), out_f, in_f, n_cb,
                                        int(use_pca), out.data_ptr(), _stream(wt16))
    _lib.check(rc, "sx8_dequant_t16")
    return out


ARITH = {"cuda": 0, "cpu": 1}   # SX8_ARITH_TORCH_CUDA / SX8_ARITH_TORCH_CPU


def quantize_blocks(w, want_levels=False, arith="cuda"):
    """Per-block search + packing of w (out_f,in_f) f16|f32 -> dict of n-major planes
    (dmin, dmax f16; config, levels_hi, levels_lo u8 [, levels (n_blk,32) u8]).
    arith: "cuda" = the reference's bits as it runs on torch-CUDA, "cpu" = on torch CPU."""
    if arith not in ARITH:
        raise SX8Error("arith must be 'cuda' or 'cpu'")
    if w.dtype not in (torch.float16, torch.float32):
        raise SX8Error("w must be float16 or float32")
    if not w.is_cuda or w.dim() != 2 or w.stride(1) != 1:
        raise SX8Error("w must be a 2-D CUDA tensor with unit inner stride")
    out_f, in_f = w.shape
    n_cb = (in_f + 31) // 32
    n_blk = out_f * n_cb
    dev = w.device
    dmin = torch.empty(n_blk, dtype=torch.float16, device=dev)
    dmax = torch.empty(n_blk, dtype=torch.float16, device=dev)
    config = torch.empty(n_blk, dtype=torch.uint8, device=dev)
    hi = torch.empty(n_blk * 16, dtype=torch.uint8, device=dev)
    lo = torch.empty(n_blk * 8, dtype=torch.uint8, device=dev)
    lv = torch.empty((n_blk, 32), dtype=torch.uint8, device=dev) if want_levels else None
    with torch.cuda.device(dev):
        rc = _lib.lib().sx8_quantize_blocks(w.data_ptr(), int(w.dtype == torch.float16), out_f, in_f, w.stride(0),
                                            dmin.data_ptr(), dmax.data_ptr(), config.data_ptr(), hi.data_ptr(),
                                            lo.data_ptr(), lv.data_ptr() if lv is not None else None, ARITH[arith],
                                            _stream(w))
    _lib.check(rc, "sx8_quantize_blocks")
    out = {"dmin": dmin, "dmax": dmax, "config": config, "levels_hi": hi, "levels_lo": lo,
           "n_cb": n_cb, "n_blocks": n_blk, "shape": (out_f, in_f)}
    if lv is not None:
        out["levels"] = lv
    return out


def _pca_in(w, q):
    if w.dtype not in (torch.float16, torch.float32) or not w.is_cuda or w.dim() != 2 or w.stride(1) != 1:
        raise SX8Error("w must be a 2-D CUDA float16 or float32 tensor with unit inner stride")
    return (w.data_ptr(), int(w.dtype == torch.float16), w.shape[0], w.shape[1], w.stride(0), q["dmin"].data_ptr(),
            q["dmax"].data_ptr(), q["config"].data_ptr(), q["levels_hi"].data_ptr(), q["levels_lo"].data_ptr())


def pca_gram(w, q):
    """(n_cb, 32, 32) f64 Gram matrices of the quantisation residual of w against the planes q
    (the result of quantize_blocks on the same w), one per block column."""
    out_f, in_f = w.shape
    n_cb = (in_f + 31) // 32
    L = _lib.lib()
    gram = torch.empty((n_cb, 32, 32), dtype=torch.float64, device=w.device)
    nbytes = L.sx8_pca_gram_scratch_bytes(out_f, in_f)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        rc = L.sx8_pca_gram(*_pca_in(w, q), gram.data_ptr(), scratch.data_ptr(), nbytes, _stream(w))
    _lib.check(rc, "sx8_pca_gram")
    return gram


def pca_project(w, q, bases):
    """coef (n_cb, 2, out_f) f32: every block's residual on the two bases (n_cb, 2, 32) f32 of its column."""
    out_f, in_f = w.shape
    n_cb = (in_f + 31) // 32
    if bases.dtype != torch.float32 or not bases.is_contiguous() or bases.numel() != n_cb * 64:
        raise SX8Error("bases must be contiguous float32 with n_cb * 64 elements")
    coef = torch.empty((n_cb, 2, out_f), dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        rc = _lib.lib().sx8_pca_project(*_pca_in(w, q), bases.data_ptr(), coef.data_ptr(), _stream(w))
    _lib.check(rc, "sx8_pca_project")
    return coef


def pca_pack(coef, scales):
    """coef (n_cb, 2, out_f) f32, scales (n_cb, 2) f32 -> coeff bytes (out_f * n_cb,) u8, n-major."""
    n_cb, _, out_f = coef.shape
    if coef.dtype != torch.float32 or scales.dtype != torch.float32 or not coef.is_contiguous() or not scales.is_contiguous():
        raise SX8Error("coef and scales must be contiguous float32")
    coeff = torch.empty(out_f * n_cb, dtype=torch.uint8, device=coef.device)
    with torch.cuda.device(coef.device):
        rc = _lib.lib().sx8_pca_pack(coef.data_ptr(), scales.data_ptr(), out_f, n_cb, coeff.data_ptr(), _stream(coef))
    _lib.check(rc, "sx8_pca_pack")
    return coeff


def repack_t16(dmin, dmax, config, coeff, hi, lo, out_f, n_cb):
    """n-major file planes -> T16 device blob, (ceil(out_f/16)*n_cb, 480) u8."""
    dev = hi.device
    nbytes = _lib.lib().sx8_t16_bytes(out_f, n_cb)
    blob = torch.empty((nbytes // 480, 480), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().sx8_repack_t16(dmin.data_ptr(), dmax.data_ptr(), config.data_ptr(), coeff.data_ptr(),
                                       hi.data_ptr(), lo.data_ptr(), out_f, n_cb, blob.data_ptr(), _stream(hi))
    _lib.check(rc, "sx8_repack_t16")
    return blob


def repack_v44(dmin, dmax, config, coeff, hi, lo, out_f, n_cb, hdr_bytes=6):
    """n-major file planes -> kb-major (hdr (n_blk,hdr_bytes), levels (n_blk,24)) on the device."""
    dev = hi.device
    n_blk = out_f * n_cb
    hdr = torch.empty((n_blk, hdr_bytes), dtype=torch.uint8, device=dev)
    lev = torch.empty((n_blk, 24), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().sx8_repack_v44(dmin.data_ptr(), dmax.data_ptr(), config.data_ptr(), coeff.data_ptr(),
                                       hi.data_ptr(), lo.data_ptr(), out_f, n_cb, hdr_bytes, hdr.data_ptr(),
                                       lev.data_ptr(), _stream(hi))
    _lib.check(rc, "sx8_repack_v44")
    return hdr, lev


def repack_t16_blocks(blocks, out_f, n_cb):
    """Interleaved 30-byte block_sx8 records (out_f*n_cb, 30) u8, n-major -- a GGUF tensor's
    data -- -> T16 device blob."""
    blocks = _need(blocks, torch.uint8, "blocks")
    if blocks.numel() != out_f * n_cb * 30:
        raise SX8Error("blocks has %d bytes, need %d" % (blocks.numel(), out_f * n_cb * 30))
    nbytes = _lib.lib().sx8_t16_bytes(out_f, n_cb)
    blob = torch.empty((nbytes // 480, 480), dtype=torch.uint8, device=blocks.device)
    with torch.cuda.device(blocks.device):
        rc = _lib.lib().sx8_repack_t16_blocks(blocks.data_ptr(), out_f, n_cb, blob.data_ptr(), _stream(blocks))
    _lib.check(rc, "sx8_repack_t16_blocks")
    return blob


def blocks_from_planes(dmin, dmax, config, coeff, hi, lo):
    """n-major planes -> (n_blk, 30) u8 interleaved records, byte-identical to the reference's
    blockify_vec (ref scripts/convert_pkl_to_gguf_sx8.py:20-38)."""
    n_blk = config.numel()
    out = torch.empty((n_blk, 30), dtype=torch.uint8, device=config.device)
    with torch.cuda.device(config.device):
        rc = _lib.lib().sx8_blocks_from_planes(dmin.data_ptr(), dmax.data_ptr(), config.data_ptr(), coeff.data_ptr(),
                                               hi.data_ptr(), lo.data_ptr(), n_blk, out.data_ptr(), _stream(config))
    _lib.check(rc, "sx8_blocks_from_planes")
    return out


def planes_from_blocks(blocks):
    """(n_blk, 30) u8 records -> dict of n-major planes (dmin, dmax f16; config, coeff, levels_hi,
    levels_lo u8)."""
    blocks = _need(blocks, torch.uint8, "blocks")
    n_blk = blocks.numel() // 30
    if n_blk * 30 != blocks.numel():
        raise SX8Error("blocks is not a whole number of 30-byte records")
    dev = blocks.device
    q = {"dmin": torch.empty(n_blk, dtype=torch.float16, device=dev), "dmax": torch.empty(n_blk, dtype=torch.float16, device=dev),
         "config": torch.empty(n_blk, dtype=torch.uint8, device=dev), "coeff": torch.empty(n_blk, dtype=torch.uint8, device=dev),
         "levels_hi": torch.empty(n_blk * 16, dtype=torch.uint8, device=dev),
         "levels_lo": torch.empty(n_blk * 8, dtype=torch.uint8, device=dev)}
    with torch.cuda.device(dev):
        rc = _lib.lib().sx8_planes_from_blocks(blocks.data_ptr(), n_blk, q["dmin"].data_ptr(), q["dmax"].data_ptr(),
                                               q["config"].data_ptr(), q["coeff"].data_ptr(), q["levels_hi"].data_ptr(),
                                               q["levels_lo"].data_ptr(), _stream(blocks))
    _lib.check(rc, "sx8_planes_from_blocks")
    return q


# ---- decoder glue (sx8_glue_*): thin wrappers, all tensors preallocated by the caller
def glue_add_rmsnorm(h, y, gamma, eps, x_out):
    """h (B,H) f32 += y (or None); x_out (B,H) f16 = rmsnorm(h) * gamma."""
    B, H = h.shape
    with torch.cuda.device(h.device):
        rc = _lib.lib().sx8_glue_add_rmsnorm(h.data_ptr(), 0 if y is None else y.data_ptr(), gamma.data_ptr(), B, H,
                                             float(eps), x_out.data_ptr(), _stream(h))
    _lib.check(rc, "sx8_glue_add_rmsnorm")
    return x_out


def glue_allreduce_add_rmsnorm(peers, h, gamma, eps, x_out):
    """Row-parallel consumer over peer memory: h (M,H) f32 += sum over ranks of the partials that
    every rank wrote into its own exchange slot; x_out (M,H) f16 = rmsnorm(h) * gamma.  `peers`
    is a _lib.Peers descriptor (tp.PeerExchange)."""
    import ctypes
    M, H = h.shape
    with torch.cuda.device(h.device):
        rc = _lib.lib().sx8_glue_allreduce_add_rmsnorm(ctypes.addressof(peers), M, H, h.data_ptr(), gamma.data_ptr(),
                                                       float(eps), x_out.data_ptr(), _stream(h))
    _lib.check(rc, "sx8_glue_allreduce_add_rmsnorm")
    return x_out


def glue_rope_cache(q, k, v, pos, cos_t, sin_t, hq, hkv, D, q_out, k_cache, v_cache):
    """q (B,hq*D), k, v (B,hkv*D) f32; caches (B,hkv,S,D) f16 written at position pos[0]."""
    B, S = q.shape[0], k_cache.shape[2]
    with torch.cuda.device(q.device):
        rc = _lib.lib().sx8_glue_rope_cache(q.data_ptr(), k.data_ptr(), v.data_ptr(), pos.data_ptr(), cos_t.data_ptr(),
                                            sin_t.data_ptr(), B, hq, hkv, D, S, q_out.data_ptr(), k_cache.data_ptr(),
                                            v_cache.data_ptr(), _stream(q))
    _lib.check(rc, "sx8_glue_rope_cache")
    return q_out


def glue_attn_scratch(B, hq, hkv, D, device):
    """Zeroed scratch for glue_attn_decode (arrival counters + partial results)."""
    return torch.zeros(_lib.lib().sx8_glue_attn_scratch_bytes(B, hq, hkv, D), dtype=torch.uint8, device=device)


def glue_attn_decode(q16, k_cache, v_cache, pos, hq, hkv, D, scale, out, scratch):
    B, S = q16.shape[0], k_cache.shape[2]
    with torch.cuda.device(q16.device):
        rc = _lib.lib().sx8_glue_attn_decode(q16.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(), B, hq,
                                             hkv, D, S, float(scale), out.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                             _stream(q16))
    _lib.check(rc, "sx8_glue_attn_decode")
    return out


def glue_silu_mul(g, u, act_out):
    with torch.cuda.device(g.device):
        rc = _lib.lib().sx8_glue_silu_mul(g.data_ptr(), u.data_ptr(), g.numel(), act_out.data_ptr(), _stream(g))
    _lib.check(rc, "sx8_glue_silu_mul")
    return act_out
