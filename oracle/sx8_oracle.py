"""CPU oracle for the S-X8 v4.3 hot path (numpy + the C restatement).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline / reference legs -- never by the product package.

Each function names the reference file:line it restates (paths are relative to the
reference project, MarlaLabsAI/sx8-quantization).  Dict formats are the reference's:
  qt  = {shape,(orig_shape),n_blocks,n_cb,dmin,dmax,config,levels_hi,levels_lo,coeff}
        (scripts/quantize_qwen35_4b_sx8_v43_gpu.py:266-272, n-major planes)
  bi  = {n_cb, data (n_cb,64) f32, scales (n_cb,2) f32}
        (scripts/sx8_container_v43.py:112-115)
  v44 = {levels (n_blk,24) u8, hdr (n_blk,6|8) u8, n_cb, shape, bases, scales}
        (scripts/prepare_v44.py:72-79, kb-major)
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "libsx8oracle.so")
        if not os.path.exists(path):
            import importlib.util
            spec = importlib.util.spec_from_file_location("_sx8_oracle_build",
                                                          os.path.join(_HERE, "build.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_oracle()
        _lib = ctypes.CDLL(path)
        _lib.sx8o_num_threads.restype = ctypes.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# --------------------------------------------------------------------------- synthetic data

def synth_weight(out_f, in_f, seed):
    """BASELINE config 0 distribution: N(0, 0.02) with 0.1 % of entries x10, cast to
    fp16.  numpy PCG64 streams, so the same seed gives the same matrix in the tests,
    the benchmark and the golden-fixture script on any machine."""
    rng = np.random.default_rng(int(seed))
    w = rng.standard_normal((out_f, in_f), dtype=np.float32) * np.float32(0.02)
    mask = rng.random((out_f, in_f), dtype=np.float32) < np.float32(0.001)
    w[mask] *= np.float32(10.0)
    return w.astype(np.float16)


def synth_x(m, k, seed, scale=1.0):
    """Activations fp16 ~ N(0, scale)."""
    rng = np.random.default_rng(int(seed))
    return (rng.standard_normal((m, k), dtype=np.float32) * np.float32(scale)).astype(np.float16)


# --------------------------------------------------------------------------- quantizer

def to_blocks(w):
    """scripts/quantize_qwen35_4b_sx8_v43_gpu.py:236-247: float32, zero-pad the
    input dimension to a multiple of 32, reshape to (n_blk, 32) n-major."""
    w = np.asarray(w, dtype=np.float32)
    out_f, in_f = w.shape
    n_cb = (in_f + 31) // 32
    pad = n_cb * 32 - in_f
    if pad:
        w = np.pad(w, ((0, 0), (0, pad)))
    return np.ascontiguousarray(w.reshape(out_f * n_cb, 32)), n_cb


def quant_search(blocks, arith="cpu"):
    """v6_encode_6bit_gpu (quantize...py:22-47) -> levels u8 (n_blk,32), dmin f32,
    dmax f32, config i32.  arith: "cpu" = the function as torch CPU evaluates it (the golden
    fixtures), "cuda" = as torch CUDA does (the back end the reference runs on); they differ in
    the division by 63 and in the summation order of the mean (see sx8_oracle.c)."""
    blocks = _c(blocks, np.float32)
    n = blocks.shape[0]
    levels = np.empty((n, 32), np.uint8)
    dmin = np.empty(n, np.float32)
    dmax = np.empty(n, np.float32)
    cfg = np.empty(n, np.int32)
    lib().sx8o_quant_search2(_p(blocks), ctypes.c_long(n), _p(levels), _p(dmin), _p(dmax), _p(cfg),
                             ctypes.c_int({"cpu": 0, "cuda": 1}[arith]))
    return levels, dmin, dmax, cfg


def pack_levels(levels):
    """pack_levels_6bit (quantize...py:148-167) -> (hi (n_blk*16,), lo (n_blk*8,))."""
    levels = _c(levels, np.uint8)
    n = levels.shape[0]
    hi = np.empty(n * 16, np.uint8)
    lo = np.empty(n * 8, np.uint8)
    lib().sx8o_pack_levels(_p(levels), ctypes.c_long(n), _p(hi), _p(lo))
    return hi, lo


def pca_correct(levels, dmin, dmax, config, blocks, n_cb):
    """pca_correct_gpu (quantize...py:75-142) restated in numpy float32.  The SVD is
    not bit-reproducible across LAPACK builds (singular-vector signs are arbitrary),
    so this is a FUNCTIONAL restatement: PARITY UNPINNED for coeff/bases/scales bytes.
    Returns coeff (n_blk,1) u8, data (n_cb,64) f32, scales (n_cb,2) f32."""
    f32 = np.float32
    n_blk = blocks.shape[0]
    d = np.maximum(dmax - dmin, f32(1e-10)).astype(f32)
    Q = (d / f32(4.0)).astype(f32)
    L = f32(63.0)
    lo_j = np.stack([dmin, dmin, dmax - Q, dmin + Q]).astype(f32)
    st_j = np.stack([d / L, Q / L, Q / L, np.maximum(d - f32(2) * Q, f32(1e-10)) / L]).astype(f32)
    lv_f = levels.astype(f32)
    coeff = np.zeros((n_blk, 1), np.uint8)
    data = np.zeros((n_cb, 64), f32)
    scales = np.zeros((n_cb, 2), f32)
    idx = np.arange(n_blk)
    for cb in range(n_cb):
        si = idx[idx % n_cb == cb]
        if si.size < 4:
            continue
        rec = np.zeros((si.size, 32), f32)
        cfg_s = config[si].astype(np.int64)
        for sb in range(4):
            st = (cfg_s >> (sb * 2)) & 3
            lo_sb = lo_j[st, si]
            st_sb = st_j[st, si]
            rec[:, sb * 8:sb * 8 + 8] = lo_sb[:, None] + st_sb[:, None] * lv_f[si][:, sb * 8:sb * 8 + 8]
        err = (blocks[si] - rec).astype(f32)
        _, _, vh = np.linalg.svd(err, full_matrices=False)
        basis = vh[:4]
        raw = basis @ err.T
        sc = np.maximum(np.median(np.abs(raw), axis=1) / f32(3.0), f32(1e-10)).astype(f32)
        cq = np.clip(np.rint(raw / sc[:, None]), -8, 7).astype(np.int8)
        coeff[si, 0] = (cq[0].astype(np.uint8) & 0xF) | ((cq[1].astype(np.uint8) & 0xF) << 4)
        data[cb] = basis[:2].reshape(-1)
        scales[cb] = sc[:2]
    return coeff, data, scales


def quantize(w, with_pca=True, arith="cpu"):
    """Whole-tensor quantisation in the reference's order (quantize...py:235-272):
    search -> PCA -> fp16 endpoints -> pack.  Returns (qt, bi)."""
    out_f, in_f = w.shape
    blocks, n_cb = to_blocks(w)
    levels, dmin, dmax, cfg = quant_search(blocks, arith)
    if with_pca:
        coeff, data, scales = pca_correct(levels, dmin, dmax, cfg, blocks, n_cb)
    else:
        coeff = np.zeros((blocks.shape[0], 1), np.uint8)
        data = np.zeros((n_cb, 64), np.float32)
        scales = np.zeros((n_cb, 2), np.float32)
    hi, lo = pack_levels(levels)
    qt = {"shape": (out_f, in_f), "orig_shape": (out_f, in_f), "n_blocks": blocks.shape[0],
          "n_cb": n_cb, "dmin": dmin.astype(np.float16), "dmax": dmax.astype(np.float16),
          "config": cfg.astype(np.uint8), "levels_hi": hi, "levels_lo": lo, "coeff": coeff}
    bi = {"n_cb": n_cb, "data": data, "scales": scales}
    return qt, bi


# --------------------------------------------------------------------------- layout

def to_v44(qt, bi, hdr_aligned=False):
    """to_v44 (scripts/prepare_v44.py:35-79)."""
    out_f, in_f = qt["shape"]
    n_cb, n_blk = qt["n_cb"], qt["n_blocks"]
    hb = 8 if hdr_aligned else 6
    hdr = np.empty((n_blk, hb), np.uint8)
    lev = np.empty((n_blk, 24), np.uint8)
    lib().sx8o_to_v44(ctypes.c_long(out_f), ctypes.c_long(n_cb),
                      _p(_c(qt["dmin"], np.float16).view(np.uint16)),
                      _p(_c(qt["dmax"], np.float16).view(np.uint16)),
                      _p(_c(qt["config"], np.uint8)), _p(_c(np.asarray(qt["coeff"]).reshape(-1), np.uint8)),
                      _p(_c(qt["levels_hi"], np.uint8)), _p(_c(qt["levels_lo"], np.uint8)),
                      ctypes.c_int(hb), _p(hdr), _p(lev))
    return {"levels": lev, "hdr": hdr, "n_cb": n_cb, "shape": (out_f, in_f),
            "bases": _c(np.asarray(bi["data"]).reshape(-1, 64), np.float32),
            "scales": _c(np.asarray(bi["scales"]).reshape(-1, 2), np.float32)}


def extract_levels(qt):
    """extract_levels_v43 (scripts/prepare_v44.py:82-93) -> (n_blk,32) u8."""
    n = qt["n_blocks"]
    hi = np.asarray(qt["levels_hi"]).reshape(n, 16)
    lo = np.asarray(qt["levels_lo"]).reshape(n, 8)
    t = np.arange(32)
    nib = (hi[:, t >> 1] >> ((t & 1) * 4)) & 0xF
    qua = (lo[:, t >> 2] >> ((3 - (t & 3)) * 2)) & 0x3
    return ((nib << 2) | qua).astype(np.uint8)


# --------------------------------------------------------------------------- decoders

def dequant_d64(qt, bi, use_pca=True):
    """decode_tensor_gpu_fast (scripts/kernel_sx8_v43.py:109-145): the float64
    numba decode, float32 store, reshape/slice to (out_f, in_f), fp16 cast."""
    out_f, in_f = qt["shape"]
    n_cb, n_blk = qt["n_cb"], qt["n_blocks"]
    out = np.empty(n_blk * 32, np.float32)
    lib().sx8o_dequant_d64(_p(_c(qt["dmin"], np.float16).view(np.uint16)),
                           _p(_c(qt["dmax"], np.float16).view(np.uint16)),
                           _p(_c(qt["config"], np.uint8)),
                           _p(_c(np.asarray(qt["coeff"]).reshape(-1), np.uint8)),
                           _p(_c(qt["levels_hi"], np.uint8)), _p(_c(qt["levels_lo"], np.uint8)),
                           _p(_c(np.asarray(bi["data"]).reshape(-1), np.float32)),
                           _p(_c(np.asarray(bi["scales"]).reshape(-1), np.float32)),
                           ctypes.c_long(n_blk), ctypes.c_long(n_cb), ctypes.c_int(int(use_pca)),
                           _p(out))
    w = out.reshape(out_f, n_cb * 32)[:, :in_f]
    return w.astype(np.float16)


def embed_d32(ids, v44, contract=True):
    """sx8_embed_v44_kernel (cuda/sx8_embed_v44.cu:21-77) -> (T, K) fp16."""
    out_f, in_f = v44["shape"]
    ids = _c(np.asarray(ids).reshape(-1), np.int64)
    hb = v44["hdr"].shape[1]
    out = np.zeros((ids.size, in_f), np.float16)
    lib().sx8o_embed_d32(_p(ids), ctypes.c_long(ids.size), _p(_c(v44["hdr"], np.uint8)),
                         _p(_c(v44["levels"], np.uint8)), _p(_c(v44["bases"], np.float32)),
                         _p(_c(v44["scales"], np.float32)), ctypes.c_long(in_f),
                         ctypes.c_long(out_f), ctypes.c_long(v44["n_cb"]), ctypes.c_int(hb),
                         ctypes.c_int(int(contract)), _p(out.view(np.uint16)))
    return out


def gemv_d32(x, v44):
    """Reformulated float32 GEMV in the reference kernel's own order
    (cuda/sx8_decode1_v3.cu:44-167), one row of x at a time -> (M,N) f32."""
    out_f, _ = v44["shape"]
    n_cb = v44["n_cb"]
    x = np.asarray(x, np.float16)
    if x.ndim == 1:
        x = x[None]
    xp = np.zeros((x.shape[0], n_cb * 32), np.float16)
    xp[:, :x.shape[1]] = x
    y = np.empty((x.shape[0], out_f), np.float32)
    lib().sx8o_gemv_d32(_p(xp.view(np.uint16)), ctypes.c_long(x.shape[0]),
                        _p(_c(v44["hdr"], np.uint8)), _p(_c(v44["levels"], np.uint8)),
                        _p(_c(v44["bases"], np.float32)), _p(_c(v44["scales"], np.float32)),
                        ctypes.c_long(out_f), ctypes.c_long(n_cb),
                        ctypes.c_int(v44["hdr"].shape[1]), _p(y))
    return y


def matmul_ref(x, w_f16):
    """The reference's own comparator (scripts/sx8_decode1_v3.py:130-131,
    scripts/sx8_fused_wmma.py:127-128): Y_ref = X.float() @ W.float().t() with
    W the D64 dequantised tensor."""
    return np.asarray(x, np.float32) @ np.asarray(w_f16, np.float32).T


def num_threads():
    return int(lib().sx8o_num_threads())


# --------------------------------------------------------------------------- T16 device layout

T16_UNIT = 480  # bytes per (16-column tile, kb) unit: 384 level bytes + 96 header bytes
_T16_ORDER = (0, 2, 1, 3)  # byte j of a level word holds weight _T16_ORDER[j] of its group of four


def t16_bytes(out_f, n_cb):
    return ((out_f + 15) // 16) * n_cb * T16_UNIT


def to_t16(qt):
    """The library's own device layout ("T16"), restated in numpy as the checker for
    sx8_repack_t16.  It is a byte/bit permutation of the reference's 30-byte block
    (docs/SX8_FLASH_V4_3_SPEC.md:13-25): nothing is added or dropped.

    blob[(T*n_cb + kb)*480 ...]: unit of tile T (columns 16T..16T+15) and block row kb.
      lane L = 4g + t (g = 0..7, t = 0..3) owns sub-block t of column A = 16T+g and of
      column B = 16T+g+8.  With a_i / b_i the 6-bit levels of weight 8t+i:
        word W0 at unit + 0*128 + 4L : bytes [a0,a2,a1,a3] << 2, low 2 bits = bits 1:0 of [b4,b6,b5,b7]
        word W1 at unit + 1*128 + 4L : bytes [a4,a6,a5,a7] << 2, low 2 bits = bits 3:2 of [b4,b6,b5,b7]
        word W2 at unit + 2*128 + 4L : bytes [b0,b2,b1,b3] << 2, low 2 bits = bits 5:4 of [b4,b6,b5,b7]
      header words at unit + 384: H0[g] = dmin(A) | dmax(A) << 16, H1[g] (+32) the same for B,
        H2[g] (+64) = c0(A) | c0(B) << 4 | config(A) << 8 | c1(A) << 16 | c1(B) << 20 | config(B) << 24,
        c0 / c1 being the low / high nibble of the coeff byte.
    Columns past out_f are zero blocks."""
    out_f, _ = qt["shape"]
    n_cb = qt["n_cb"]
    nt = (out_f + 15) // 16
    npad = nt * 16
    lv = np.zeros((npad, n_cb, 4, 8), np.uint32)
    lv[:out_f] = extract_levels(qt).reshape(out_f, n_cb, 4, 8)
    dmin = np.zeros((npad, n_cb), np.uint32); dmax = np.zeros((npad, n_cb), np.uint32)
    cfg = np.zeros((npad, n_cb), np.uint32); co = np.zeros((npad, n_cb), np.uint32)
    dmin[:out_f] = np.asarray(qt["dmin"], np.float16).view(np.uint16).reshape(out_f, n_cb)
    dmax[:out_f] = np.asarray(qt["dmax"], np.float16).view(np.uint16).reshape(out_f, n_cb)
    cfg[:out_f] = np.asarray(qt["config"], np.uint8).reshape(out_f, n_cb)
    co[:out_f] = np.asarray(qt["coeff"], np.uint8).reshape(out_f, n_cb)
    # (tile, half, g, kb, ...) views: column = 16T + 8*half + g
    lv = lv.reshape(nt, 2, 8, n_cb, 4, 8)
    a, b = lv[:, 0], lv[:, 1]                     # (nt, g, kb, t, 8)
    o = list(_T16_ORDER)
    e = b[..., [4 + j for j in o]]                # extras source bytes [b4,b6,b5,b7]

    def word(src4, shift):
        w = np.zeros(src4.shape[:-1], np.uint32)
        for j in range(4):
            byte = (src4[..., j] << 2) | ((e[..., j] >> shift) & 3)
            w |= byte << (8 * j)
        return w

    w0 = word(a[..., o], 0)
    w1 = word(a[..., [4 + j for j in o]], 2)
    w2 = word(b[..., o], 4)
    # -> (nt, kb, plane, g, t)
    lev = np.stack([w0, w1, w2], axis=0).transpose(1, 3, 0, 2, 4)     # (nt, kb, 3, g, t)
    hd = lambda x: x.reshape(nt, 2, 8, n_cb)
    dm, dx, cf, cc = hd(dmin), hd(dmax), hd(cfg), hd(co)
    h0 = dm[:, 0] | (dx[:, 0] << 16)
    h1 = dm[:, 1] | (dx[:, 1] << 16)
    h2 = ((cc[:, 0] & 15) | ((cc[:, 1] & 15) << 4) | (cf[:, 0] << 8) | ((cc[:, 0] >> 4) << 16)
          | ((cc[:, 1] >> 4) << 20) | (cf[:, 1] << 24))
    hdr = np.stack([h0, h1, h2], axis=0).transpose(1, 3, 0, 2)        # (nt, kb, 3, g)
    blob = np.empty((nt, n_cb, 120), np.uint32)
    blob[:, :, :96] = lev.reshape(nt, n_cb, 96)
    blob[:, :, 96:] = hdr.reshape(nt, n_cb, 24)
    return np.ascontiguousarray(blob).view(np.uint8).reshape(-1)


# ---------------------------------------------------------------- interleaved 30-byte blocks
def blocks_from_planes(qt):
    """(n_blk, 30) u8 block_sx8 records {dmin, dmax, config, qh[16], ql[8], coeff}: the layout
    ref scripts/convert_pkl_to_gguf_sx8.py:20-38 (blockify_vec) writes into GGUF tensors and
    docs/SX8_FLASH_V4_3_SPEC.md:13-25 specifies."""
    nb = int(qt["n_blocks"])
    out = np.empty((nb, 30), np.uint8)
    out[:, 0:2] = np.ascontiguousarray(qt["dmin"], dtype=np.float16).reshape(-1).view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = np.ascontiguousarray(qt["dmax"], dtype=np.float16).reshape(-1).view(np.uint8).reshape(nb, 2)
    out[:, 4] = np.asarray(qt["config"], dtype=np.uint8).reshape(-1)
    out[:, 5:21] = np.asarray(qt["levels_hi"], dtype=np.uint8).reshape(nb, 16)
    out[:, 21:29] = np.asarray(qt["levels_lo"], dtype=np.uint8).reshape(nb, 8)
    out[:, 29] = np.asarray(qt["coeff"], dtype=np.uint8).reshape(-1)
    return out


def planes_from_blocks(blocks, shape):
    """Inverse of blocks_from_planes: the container's plane dict for a tensor of `shape`."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 30)
    nb = b.shape[0]
    out_f, in_f = shape
    return {"shape": (out_f, in_f), "n_blocks": nb, "n_cb": nb // out_f,
            "dmin": np.ascontiguousarray(b[:, 0:2]).view(np.float16).reshape(-1),
            "dmax": np.ascontiguousarray(b[:, 2:4]).view(np.float16).reshape(-1),
            "config": b[:, 4].copy(), "levels_hi": np.ascontiguousarray(b[:, 5:21]).reshape(-1),
            "levels_lo": np.ascontiguousarray(b[:, 21:29]).reshape(-1), "coeff": b[:, 29].copy()}
