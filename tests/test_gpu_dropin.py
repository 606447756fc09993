"""The five drop-in modules, exercised the way the reference's callers use them (positional
arguments, dict tensors, pooled buffers), against the CPU oracle.

ref scripts/sx8_decode1_v3.py:57-110      make_tensors_v44, decode1_v44, best_split_k
ref scripts/sx8_gemm_compact.py:42-74     gemm_sx8_compact
ref scripts/sx8_fused_wmma.py:60-104      make_tensors, gemm_sx8_wmma_cached, gemm_sx8_wmma, decode1_sx8_cached
ref scripts/sx8_embed_v44.py:40-72        SX8EmbeddingV44
ref scripts/kernel_sx8_v43.py:109-145     decode_tensor_gpu_fast
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import sx8_oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu

TOL = 2e-3          # of max|Y_ref|; the reference's own tests accept 5e-3 (ref scripts/sx8_fused_wmma.py:130)

_CASES = {}


def case(out_f, in_f, seed):
    key = (out_f, in_f, seed)
    if key not in _CASES:
        qt, bi = orc.quantize(orc.synth_weight(out_f, in_f, seed), with_pca=True)
        _CASES[key] = (qt, bi, orc.dequant_d64(qt, bi))
    return _CASES[key]


def xdev(m, k, seed):
    x = orc.synth_x(m, k, seed)
    return x, torch.from_numpy(x).cuda()


def close(y, ref, tol=TOL):
    y = y.detach().float().cpu().numpy()
    assert y.shape == ref.shape
    assert np.isfinite(y).all()
    return np.abs(y - ref).max() <= tol * np.abs(ref).max()


def kb_major(qt):
    """The reorder SX8Linear.__init__ applies before make_tensors (ref scripts/integrate_fused.py:46-58):
    block id kb*N + n instead of n*n_cb + kb."""
    N, n_cb = qt["shape"][0], qt["n_cb"]
    r1 = lambda a: np.asarray(a).reshape(N, n_cb).T.reshape(-1).copy()
    r2 = lambda a, per: np.asarray(a).reshape(N, n_cb, per).transpose(1, 0, 2).reshape(-1).copy()
    return {"dmin": r1(qt["dmin"]).astype(np.float16), "dmax": r1(qt["dmax"]).astype(np.float16),
            "config": r1(qt["config"]).astype(np.uint8), "coeff": r1(np.asarray(qt["coeff"]).reshape(-1)).astype(np.uint8),
            "levels_hi": r2(qt["levels_hi"], 16).astype(np.uint8), "levels_lo": r2(qt["levels_lo"], 8).astype(np.uint8)}


# --------------------------------------------------------------------------- sx8_decode1_v3

@pytest.mark.parametrize("shape", [(1024, 2560), (136, 1000)])
def test_make_tensors_v44_then_decode1_v44(shape):
    from sx8_quantization_b200 import sx8_decode1_v3 as m
    qt, bi, w = case(shape[0], shape[1], 201)
    t = m.make_tensors_v44(qt, bi, hdr_aligned=False)
    assert len(t) == 4 and t[1].is_cuda and t[2].shape == (qt["n_cb"], 64) and t[3].shape == (qt["n_cb"], 2)
    assert np.array_equal(t[1].cpu().numpy().reshape(-1), orc.to_t16(qt))
    hdr_t, lvl_t, bas_t, sca_t = t
    # the caller's exact call (ref scripts/integrate_fused_v44.py:55-57): 1-D x, nine positional arguments
    x, xd = xdev(1, shape[1], 5)
    y, back = m.decode1_v44(xd[0], qt, bi, hdr_t, lvl_t, bas_t, sca_t, 6, m.best_split_k(shape[0], qt["n_cb"]))
    assert y.dtype == torch.float32 and y.shape == (shape[0],)
    assert back[1] is lvl_t
    assert close(y, orc.matmul_ref(x, w)[0])
    # batch rows (not in the reference, which has M = 1 only)
    for M in (2, 8):
        x, xd = xdev(M, shape[1], 6 + M)
        y, _ = m.decode1_v44(xd, qt, bi, hdr_t, lvl_t, bas_t, sca_t)
        assert y.shape == (M, shape[0]) and close(y, orc.matmul_ref(x, w))


def test_decode1_v44_builds_tensors_when_none_given_and_accepts_float_x():
    from sx8_quantization_b200 import sx8_decode1_v3 as m
    qt, bi, w = case(64, 256, 202)
    x, xd = xdev(1, 256, 9)
    y, t = m.decode1_v44(xd[0].float(), qt, bi)          # ref :95-101: tensors built on first use, X.half()
    assert close(y, orc.matmul_ref(x, w)[0])
    y8, _ = m.decode1_v44(xd[0], qt, bi, *t, hdr_bytes=8)  # the padded-header variant maps to the same data
    assert torch.equal(y8, y)


def test_decode1_v44_output_aliases_the_pool_like_the_reference():
    """ref scripts/sx8_decode1_v3.py:80-88,103-104: Y is a pooled buffer keyed by N, overwritten
    by the next call with the same N; callers copy it (y.half()) before the next linear."""
    from sx8_quantization_b200 import sx8_decode1_v3 as m
    qt, bi, w = case(1024, 2560, 201)
    t = m.make_tensors_v44(qt, bi)
    xa, xad = xdev(1, 2560, 21)
    xb, xbd = xdev(1, 2560, 22)
    ya, _ = m.decode1_v44(xad[0], qt, bi, *t)
    keep = ya.clone()
    yb, _ = m.decode1_v44(xbd[0], qt, bi, *t)
    assert ya.data_ptr() == yb.data_ptr()
    assert close(keep, orc.matmul_ref(xa, w)[0]) and close(yb, orc.matmul_ref(xb, w)[0])
    assert not torch.equal(keep, yb)
    assert m.best_split_k(1024, 80) == 16 and m.best_split_k(151936, 80) == 1   # ref :69-77


# --------------------------------------------------------------------------- sx8_gemm_compact

@pytest.mark.parametrize("shape,M", [((1024, 2560), 64), ((136, 1000), 40), ((48, 80), 2), ((4096, 2560), 300)])
def test_gemm_sx8_compact(shape, M):
    """K = 1000 and 80 are shorter than n_cb*32: the reference zero-pads X on the host
    (ref scripts/sx8_gemm_compact.py:66-71); out_f = 48 < 64 is the reference's decode + matmul
    fallback (ref :54-59)."""
    from sx8_quantization_b200 import sx8_decode1_v3 as d1, sx8_gemm_compact as m
    qt, bi, w = case(shape[0], shape[1], 203)
    hdr_t, lvl_t, bas_t, sca_t = d1.make_tensors_v44(qt, bi)
    x, xd = xdev(M, shape[1], 31)
    y = m.gemm_sx8_compact(xd, qt, bi, hdr_t, lvl_t, bas_t, sca_t, 6)     # ref scripts/integrate_fused_v44.py:69-70
    assert y.dtype == torch.float32 and y.shape == (M, shape[0])
    assert close(y, orc.matmul_ref(x, w))
    y2 = m.gemm_sx8_compact(xd, qt, bi)                                    # tensors built on demand
    assert close(y2, orc.matmul_ref(x, w))


# --------------------------------------------------------------------------- sx8_fused_wmma

@pytest.mark.parametrize("shape,M", [((1024, 2560), 128), ((136, 1000), 33), ((512, 64), 16)])
def test_make_tensors_kb_major_then_wmma_and_decode1(shape, M):
    from sx8_quantization_b200 import sx8_fused_wmma as m
    qt, bi, w = case(shape[0], shape[1], 204)
    kbm = kb_major(qt)
    t = m.make_tensors(kbm, bi, torch.device("cuda"))
    for k in ("dmin", "dmax", "config", "coeff", "hi", "lo", "basis", "scales"):
        assert t[k].is_cuda
    assert np.array_equal(t["hi"].cpu().numpy(), kbm["levels_hi"])
    x, xd = xdev(M, shape[1], 41)
    y = m.gemm_sx8_wmma_cached(xd, t, qt["n_cb"])
    assert y.dtype == torch.float32 and close(y, orc.matmul_ref(x, w))
    # the kb-major -> T16 transform ran once and is kept
    assert np.array_equal(t["_t16"][0].cpu().numpy().reshape(-1), orc.to_t16(qt))
    x1, x1d = xdev(1, shape[1], 42)
    y1 = m.decode1_sx8_cached(x1d[0], t, qt["n_cb"])                       # ref scripts/integrate_fused.py:69-70
    assert y1.shape == (shape[0],) and close(y1, orc.matmul_ref(x1, w)[0])
    y3 = m.gemm_sx8_wmma(xd, kbm, bi, qt["n_cb"])
    assert torch.equal(y3, y)


# --------------------------------------------------------------------------- sx8_embed_v44

def test_embedding_module_forward_2d_ids_and_buffer_growth():
    from sx8_quantization_b200.sx8_embed_v44 import SX8EmbeddingV44
    qt, bi, _ = case(1024, 2560, 205)
    v44 = orc.to_v44(qt, bi)
    emb = SX8EmbeddingV44(qt, bi)
    rng = np.random.default_rng(3)
    ids = rng.integers(0, 1024, (3, 7))
    out = emb(torch.from_numpy(ids).cuda())
    assert out.shape == (3, 7, 2560) and out.dtype == torch.float16
    ref = orc.embed_d32(ids.reshape(-1), v44).reshape(3, 7, 2560)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), ref.view(np.uint16))
    ids2 = rng.integers(0, 1024, (64,))                   # more tokens than the buffer held: it grows (ref :65-67)
    out2 = emb(torch.from_numpy(ids2).cuda())
    assert np.array_equal(out2.cpu().numpy().view(np.uint16), orc.embed_d32(ids2, v44).view(np.uint16))
    ids3 = rng.integers(0, 1024, (1, 1))                  # decode step: one token, buffer reused
    out3 = emb(torch.from_numpy(ids3).cuda())
    assert out3.shape == (1, 1, 2560) and out3.data_ptr() == out2.data_ptr()
    assert np.array_equal(out3.cpu().numpy().view(np.uint16).reshape(-1), orc.embed_d32(ids3.reshape(-1), v44).view(np.uint16).reshape(-1))
    cpu_ids = torch.from_numpy(ids3)                       # ids still on the host
    assert torch.equal(emb(cpu_ids), out3)


# --------------------------------------------------------------------------- kernel_sx8_v43

def test_decode_tensor_gpu_fast_orig_shape_and_out():
    from sx8_quantization_b200 import kernel_sx8_v43 as m
    qt, bi, w = case(136, 1000, 206)
    W = m.decode_tensor_gpu_fast(qt, bi)
    assert W.dtype == torch.float16 and W.shape == (136, 1000)
    assert np.array_equal(W.cpu().numpy().view(np.uint16), w.view(np.uint16))
    # a tensor stored as 2-D blocks of a 4-D original (ref scripts/kernel_sx8_v43.py:138-140)
    qt4 = dict(qt)
    qt4["orig_shape"] = (136, 10, 10, 10)
    W4 = m.decode_tensor_gpu_fast(qt4, bi)
    assert W4.shape == (136, 10, 10, 10)
    assert np.array_equal(W4.cpu().numpy().view(np.uint16).reshape(136, 1000), w.view(np.uint16))
    out = torch.zeros(136, 1000, dtype=torch.float16, device="cuda")
    back = m.decode_tensor_gpu_fast(qt, bi, out)
    assert back is out and torch.equal(out, W)
    with pytest.raises(ValueError):
        m.decode_tensor_gpu_fast(qt, bi, torch.zeros(136, 999, dtype=torch.float16, device="cuda"))
    assert torch.equal(m.decode_tensor_gpu(qt, bi), W)
