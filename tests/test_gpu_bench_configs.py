"""Every launch configuration that bench.py times, checked for values.

The full result is compared with a float32 matmul on the library's own full-tensor decode
(bit-exact against the oracle in test_gpu_parity.py), and a sample of >= 256 output columns
with the CPU oracle itself (float64 decode of those rows + the reference's comparator, and the
float32 restatement of the reference kernel's formula): the oracle would need minutes for all
151,936 rows of the largest case.

  * lm_head-sized GEMVs: N = 151936 (K = 2560) takes the no-split launch rule for thousands of
    tile groups -- four-tile groups on a plain grid at batch <= 4, eight-tile groups on a
    persistent grid at batch 8 -- and N = 128256 (K = 8192) the same rule with a long K;
  * the tensor-core GEMM instantiations of the BASELINE prefill sizes: the gate projection at
    M = 128 (76 one-CTA 128-column tiles, no split-K) and M = 512 (two-CTA tiles), the narrow
    projections at M = 512 / 2048 (one-CTA 256 x 128 tiles over several row tiles, with and
    without the split-K cluster), the four-CTA split-K cluster of narrow matrices at small M (one and
    two accumulators, ragged K), and a vocabulary-sized N at M = 32 and 256 (256-column tiles);
  * the PCA stage of the quantizer driver (functional parity with the reference algorithm).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import sx8_oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu


def _tensor(n, k, seed):
    from sx8_quantization_b200 import ops, quantizer
    t = quantizer.quantize_tensor(quantizer.synth_weight_gpu(n, k, seed), with_pca=True, keep_planes=True)
    w = ops.dequant_t16(t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"], True)
    return t, w


def _x(m, k, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(m, k, generator=g, device="cuda").half()


def _rows_for_oracle(t, rows):
    """qt / bases_info dicts (the reference's formats) of the given output rows only."""
    p, n_cb = t["planes"], t["n_cb"]
    r = torch.as_tensor(rows, device="cuda")
    take = lambda a, per: a.reshape(t["N"], n_cb * per)[r].cpu().numpy().reshape(-1)
    qt = {"shape": (len(rows), t["K"]), "n_blocks": len(rows) * n_cb, "n_cb": n_cb,
          "dmin": take(p["dmin"].view(torch.int16), 1).view(np.float16), "dmax": take(p["dmax"].view(torch.int16), 1).view(np.float16),
          "config": take(p["config"], 1), "levels_hi": take(p["levels_hi"], 16), "levels_lo": take(p["levels_lo"], 8),
          "coeff": take(p["coeff"], 1).reshape(-1, 1)}
    bi = {"n_cb": n_cb, "data": t["bases"].cpu().numpy(), "scales": t["scales"].cpu().numpy()}
    return qt, bi


def _check_against_oracle(y, x, t, n_sample=256, tol=2e-3, kernel_tol=None):
    rng = np.random.default_rng(t["N"] + t["K"])
    rows = np.sort(rng.choice(t["N"], size=min(n_sample, t["N"]), replace=False))
    rows[0], rows[-1] = 0, t["N"] - 1                       # the first and the last tile always
    qt, bi = _rows_for_oracle(t, rows)
    xh = x.cpu().numpy()
    ref = orc.matmul_ref(xh, orc.dequant_d64(qt, bi))       # the reference's comparator on those rows
    got = y[:, torch.as_tensor(rows, device="cuda")].float().cpu().numpy()
    scale = np.abs(ref).max()
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= tol * scale
    if kernel_tol is not None:                              # float32 restatement of the reference kernel's formula
        krn = orc.gemv_d32(xh, orc.to_v44(qt, bi))
        assert np.abs(got - krn).max() <= kernel_tol * scale


@pytest.mark.parametrize("shape,M", [((151936, 2560), 1), ((151936, 2560), 4), ((151936, 2560), 8),
                                     ((128256, 8192), 1)])
def test_gemv_lm_head_sizes(shape, M):
    from sx8_quantization_b200 import ops, _lib
    n, k = shape
    t, w = _tensor(n, k, 400 + M)
    x = _x(M, k, 17)
    y = ops.gemv(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"])
    ref = x.float() @ w.float().t()
    assert (y - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()
    _check_against_oracle(y, x, t, kernel_tol=1e-4)
    y2 = ops.gemv(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"])
    assert torch.equal(y, y2)
    assert _lib.device_error_flag() == 0


@pytest.mark.parametrize("shape,M", [((9728, 2560), 128), ((9728, 2560), 512), ((4096, 2560), 128), ((2560, 9728), 512),
                                     ((1024, 2560), 2048), ((4096, 2560), 512), ((2560, 4096), 2048),
                                     ((19456, 512), 32), ((19456, 512), 256), ((151936, 2560), 32),
                                     ((2560, 4096), 32), ((2560, 4096), 200), ((2560, 9728), 128), ((1000, 2100), 64),
                                     ((1024, 8192), 200), ((1000, 4100), 64)])
@pytest.mark.parametrize("f16out", [True, False])
def test_gemm_bench_instantiations(shape, M, f16out):
    from sx8_quantization_b200 import ops, _lib
    n, k = shape
    t, w = _tensor(n, k, 410)
    x = _x(M, k, 19)
    od = torch.float16 if f16out else torch.float32
    y = ops.gemm(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"], out_dtype=od)
    ref = x.float() @ w.float().t()
    tol = 3e-3 + (2.0 ** -10 if f16out else 0.0)            # weights are rounded to fp16 inside the GEMM
    assert (y.float() - ref).abs().max().item() <= tol * ref.abs().max().item()
    _check_against_oracle(y, x, t, tol=tol)
    assert torch.equal(y, ops.gemm(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"], out_dtype=od))
    assert _lib.device_error_flag() == 0


def test_gemm_small_m_f16_output_at_an_odd_pair_offset():
    """M < 32 with f16 output runs the GEMV passes and a conversion kernel; the output view here
    starts 4 bytes into an allocation, so it is 4-byte but not 8-byte aligned."""
    from sx8_quantization_b200 import ops
    n, k, M = 272, 1024, 9
    t, w = _tensor(n, k, 420)
    x = _x(M, k, 21)
    buf = torch.zeros(M * n + 2, dtype=torch.float16, device="cuda")
    out = buf[2:].view(M, n)
    assert out.data_ptr() % 8 == 4
    ops.gemm(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"], out_dtype=torch.float16, out=out)
    ref = x.float() @ w.float().t()
    assert (out.float() - ref).abs().max().item() <= (2e-3 + 2.0 ** -10) * ref.abs().max().item()
    assert buf[:2].abs().sum().item() == 0


@pytest.mark.parametrize("shape", [(1024, 2560), (256, 1000)])
def test_quantizer_pca_stage_functional_parity(shape):
    """ref scripts/quantize_qwen35_4b_sx8_v43_gpu.py:75-142 against quantizer._pca_correct: the
    singular vectors are only defined up to sign and LAPACK build, so the comparison is
    functional -- reconstruction error after the correction no worse than 1.02 x the reference
    algorithm's (the oracle's pca_correct on the same matrix), coefficients in the signed
    4-bit range, orthonormal bases, and a real gain over no correction."""
    from sx8_quantization_b200 import ops, quantizer
    out_f, in_f = shape
    w16 = orc.synth_weight(out_f, in_f, 77)
    wd = torch.from_numpy(w16).cuda()
    t = quantizer.quantize_tensor(wd, with_pca=True, keep_planes=True)
    n_cb = t["n_cb"]
    qt_o, bi_o = orc.quantize(w16, with_pca=True, arith="cuda")   # the driver searches in the torch-CUDA arithmetic
    # the search stage is bit-exact, so both PCA stages start from the same levels
    assert np.array_equal(t["planes"]["levels_hi"].cpu().numpy(), qt_o["levels_hi"])
    w32 = w16.astype(np.float32)
    mse = lambda W: float(((W.astype(np.float32)[:, :in_f] - w32) ** 2).mean())
    qt_g, bi_g = quantizer.to_host_dicts(t)
    e_ours = mse(orc.dequant_d64(qt_g, bi_g))
    e_ref = mse(orc.dequant_d64(qt_o, bi_o))
    e_none = mse(orc.dequant_d64(qt_o, bi_o, use_pca=False))
    assert e_ours <= 1.02 * e_ref
    assert e_ours < 0.99 * e_none
    # the library's own decode of its own tensor agrees with the oracle's decode of it, bit for bit
    W_lib = ops.dequant_t16(t["wt16"], t["bases"], t["scales"], out_f, in_f, n_cb, True).cpu().numpy()
    assert np.array_equal(W_lib.view(np.uint16), orc.dequant_d64(qt_g, bi_g).view(np.uint16))
    c = qt_g["coeff"].reshape(-1).astype(np.int16)
    c0, c1 = c & 15, c >> 4
    assert c0.max() <= 15 and c1.max() <= 15
    s4 = lambda v: np.where(v < 8, v, v - 16)
    assert s4(c0).min() >= -8 and s4(c0).max() <= 7 and s4(c1).min() >= -8
    assert len(np.unique(s4(c0))) > 4                         # the range is used, not collapsed
    B = bi_g["data"].reshape(n_cb, 2, 32).astype(np.float64)
    gram = np.einsum("kit,kjt->kij", B, B)
    assert np.abs(gram - np.eye(2)[None]).max() < 1e-4
    assert (bi_g["scales"] > 0).all()


@pytest.mark.parametrize("shape,dtype", [((1024, 2560), "f16"), ((256, 1000), "f16"), ((130, 96), "f32"), ((4100, 264), "f32")])
def test_quantizer_pca_kernels_against_torch_ops(shape, dtype):
    """sx8_pca_gram / sx8_pca_project / sx8_pca_pack against the same stage written with torch
    tensor operations on the materialised residual (ref scripts/quantize_qwen35_4b_sx8_v43_gpu.py
    :84-97 residual, :127-139 projection and packing).  The Gram matrix and the projections are
    float32 sums in another order, so they agree to float32 rounding of the sums, not bit for bit;
    the packed bytes are compared with the projection's own values as input, where they must be
    identical."""
    from sx8_quantization_b200 import ops, quantizer
    out_f, in_f = shape
    w = quantizer.synth_weight_gpu(out_f, in_f, 88)
    if dtype == "f32":
        w = w.float() * 1.0001
    q = ops.quantize_blocks(w, want_levels=True)
    n_cb = q["n_cb"]
    w32 = torch.nn.functional.pad(w.float(), (0, n_cb * 32 - in_f))
    ref = quantizer._pca_correct_torch(w32, q, n_cb)
    G = ops.pca_gram(w, q)
    Gr = torch.bmm(ref["E"].double().transpose(1, 2), ref["E"].double())
    assert (G - Gr).abs().max().item() <= 1e-5 * Gr.abs().max().item()
    assert torch.equal(G, ops.pca_gram(w, q))                  # chunks are added in a fixed order
    assert (G - G.transpose(1, 2)).abs().max().item() <= 1e-6 * Gr.abs().max().item()
    coef = ops.pca_project(w, q, ref["basis"])
    assert (coef - ref["coef"]).abs().max().item() <= 1e-5 * ref["coef"].abs().max().item()
    byte = ops.pca_pack(coef, ref["scales"])
    cq = (coef / ref["scales"].unsqueeze(-1)).round().clamp(-8, 7).to(torch.int16)
    want = ((cq[:, 0] & 0xF) | ((cq[:, 1] & 0xF) << 4)).to(torch.uint8).t().contiguous().reshape(-1)
    assert torch.equal(byte, want)
    # end to end: same bytes as the torch stage except where a coefficient sits on a rounding boundary
    assert (byte != ref["coeff"]).float().mean().item() < 1e-3


@pytest.mark.parametrize("Ns,K,M", [((4096, 1024, 1024), 2560, 32), ((4096, 1024, 1024), 2560, 512), ((9728, 9728), 2560, 2048),
                                     ((512, 256, 272), 1024, 40), ((1024, 1000), 1000, 64),
                                     ((272, 512), 1024, 100), ((4096, 1024, 1024), 2560, 12), ((4096, 1024, 1024), 2560, 16),
                                     ((528, 16, 1000), 1000, 9), ((4096, 1024, 1024), 2560, 5)])
@pytest.mark.parametrize("f16out", [True, False])
def test_gemm_multi_matches_separate_calls(Ns, K, M, f16out):
    """sx8_gemm_multi: q|k|v and gate|up in one tensor-core launch (every matrix but the last a
    multiple of 256 columns wide, M > 16), in one launch of the GEMV kernel (M <= 16 with float32
    output: two row blocks at 9..16 rows with one activation table per matrix, ragged K and N), and
    its per-matrix route for the rest (first matrix 272 columns wide; float16 output at M <= 16).
    Each output against a float32 matmul on the library's own decode and against the
    single-matrix call."""
    from sx8_quantization_b200 import ops, _lib
    ts = [_tensor(n, K, 500 + i)[0] for i, n in enumerate(Ns)]
    x = _x(M, K, 23)
    od = torch.float16 if f16out else torch.float32
    mg = ops.MultiGemm(ts)
    outs = mg(x, out_dtype=od)
    tol = 3e-3 + (2.0 ** -10 if f16out else 0.0)
    for t, y in zip(ts, outs):
        w = ops.dequant_t16(t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], True)
        ref = x.float() @ w.float().t()
        assert y.shape == (M, t["N"]) and y.dtype == od
        assert (y.float() - ref).abs().max().item() <= tol * ref.abs().max().item()
        one = ops.gemm(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], out_dtype=od)
        assert (y.float() - one.float()).abs().max().item() <= 2e-3 * ref.abs().max().item()
    again = mg(x, out_dtype=od)
    assert all(torch.equal(a, b) for a, b in zip(outs, again))
    assert _lib.device_error_flag() == 0


def test_gemm_multi_rejects_bad_arguments():
    from sx8_quantization_b200 import ops
    t1, _ = _tensor(256, 512, 1)
    t2, _ = _tensor(256, 1024, 2)
    with pytest.raises(ops.SX8Error):
        ops.MultiGemm([t1, t2])                                  # different K
    with pytest.raises(ops.SX8Error):
        ops.MultiGemm([t1, t1, t1, t1])                          # more than three
    mg = ops.MultiGemm([t1, t1])
    with pytest.raises(ops.SX8Error):
        mg(_x(32, 512, 1), outs=[torch.empty(32, 256, device="cuda"), torch.empty(31, 256, device="cuda")])


def test_gemm_chain_back_to_back_matches_synchronised_calls():
    """Tensor-core GEMMs launch as programmatic dependent launches: a GEMM prefetches its weights while the
    kernel ahead still runs, and the kernel that rewrites the shared PCA table waits for the GEMM
    that still reads it.  A chain in which every GEMM consumes the previous one's output through
    the same workspace, issued back to back and replayed from a CUDA graph, must give the bits of the
    same chain run with a device synchronisation after every call."""
    from sx8_quantization_b200 import ops, _lib
    dims = [1024, 2560, 1024, 512, 2560]                       # K of link i = N of link i - 1
    ts = [_tensor(dims[i + 1], dims[i], 600 + i)[0] for i in range(len(dims) - 1)]
    x = _x(200, dims[0], 31) * 0.05

    def chain(sync):
        a = x
        outs = []
        for t in ts:
            a = ops.gemm(a, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], out_dtype=torch.float16)
            if sync:
                torch.cuda.synchronize()
            outs.append(a)
        return outs

    want = chain(True)
    for _ in range(3):
        got = chain(False)
        torch.cuda.synchronize()
        assert all(torch.equal(g, w) for g, w in zip(got, want))
    assert torch.isfinite(want[-1].float()).all() and want[-1].float().abs().max().item() > 0
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        chain(False)
        st.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            cap = chain(False)
        for _ in range(3):
            gr.replay()
        st.synchronize()
    assert all(torch.equal(g, w) for g, w in zip(cap, want))
    assert _lib.device_error_flag() == 0
