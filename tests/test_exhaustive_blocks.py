"""Exhaustive micro-cases of the block format, built directly as planes (no quantizer): every
config byte (256 rows) x every coeff byte (256 block rows) = 65,536 blocks, levels running
through 0..63 at every position, and a grid of (dmin, dmax) pairs with degenerate, negative,
positive, mixed, subnormal and near-maximum ranges.

CPU: the C oracle's float64 decode against an independent numpy statement of the decode formula
(docs/SX8_FLASH_V4_3_SPEC.md:27-47 with the numba kernel's float64 typing,
scripts/kernel_sx8_v43.py:28-51).  GPU: every kernel against the oracle on the same planes."""
import numpy as np
import pytest

from oracle import sx8_oracle as orc

N, NCB = 256, 256
K = NCB * 32


def exhaustive_case():
    rng = np.random.default_rng(1234)
    n_blk = N * NCB
    row, kb = np.divmod(np.arange(n_blk), NCB)
    config = row.astype(np.uint8)                   # every range-strategy combination
    coeff = kb.astype(np.uint8)                     # every pair of signed 4-bit coefficients
    levels = ((np.arange(32)[None, :] * 5 + (row * 7 + kb * 3)[:, None]) % 64).astype(np.uint8)
    pairs = np.array([(0.0, 0.0), (0.0123, 0.0123), (-1.0, 1.0), (-0.5, -0.25), (0.25, 0.75), (-6.0e-8, 6.0e-8),
                      (0.0, 6.0e-8), (-60000.0, 60000.0), (-0.02, 0.03), (1.0e-4, 1.5e-4), (-3.0, -3.0),
                      (-65504.0, 0.0), (0.0, 65504.0), (-0.07, 0.0), (0.001, 0.002), (-1.5e-5, 2.5e-5)], np.float32)
    pick = (row * 5 + kb * 11) % len(pairs)
    dmin, dmax = pairs[pick, 0].astype(np.float16), pairs[pick, 1].astype(np.float16)
    hi, lo = orc.pack_levels(levels)
    qt = {"shape": (N, K), "n_blocks": n_blk, "n_cb": NCB, "dmin": dmin, "dmax": dmax, "config": config,
          "levels_hi": hi, "levels_lo": lo, "coeff": coeff.reshape(-1, 1)}
    bases = rng.standard_normal((NCB, 64)).astype(np.float32) * 0.2
    scales = (rng.random((NCB, 2)).astype(np.float32) * 0.01 + 1e-4)
    scales[::7] = 0.0                                # some blocks rows without a PCA term
    bi = {"n_cb": NCB, "data": bases, "scales": scales}
    return qt, bi, levels


def numpy_decode_f64(qt, bi, levels):
    """w = rlo + step * level + c0*s0*b0[t] + c1*s1*b1[t] in float64, stored as float32, cast
    to float16 -- written from the format specification, independently of the C oracle."""
    n_blk = qt["n_blocks"]
    lo = qt["dmin"].astype(np.float32).astype(np.float64)[:, None]
    hi = qt["dmax"].astype(np.float32).astype(np.float64)[:, None]
    q = (hi - lo) * 0.25
    sb = np.arange(32) >> 3
    s = (qt["config"].astype(np.int64)[:, None] >> (2 * sb)[None, :]) & 3
    rlo = lo + q * np.where(s == 2, 3.0, np.where(s == 3, 1.0, 0.0))
    rhi = hi - q * np.where(s == 1, 3.0, np.where(s == 3, 1.0, 0.0))
    step = (rhi - rlo) * 0.015873
    step = np.where(step < 1e-10, 1e-10, step)
    w = rlo + step * levels.astype(np.float64)
    c = np.asarray(qt["coeff"]).reshape(-1).astype(np.int64)
    c0, c1 = c & 15, c >> 4
    c0, c1 = np.where(c0 < 8, c0, c0 - 16), np.where(c1 < 8, c1, c1 - 16)
    kb = np.arange(n_blk) % qt["n_cb"]
    sc = bi["scales"].astype(np.float64)[kb]
    b = bi["data"].astype(np.float64)[kb]
    w = w + (c0[:, None] * sc[:, :1]) * b[:, :32] + (c1[:, None] * sc[:, 1:]) * b[:, 32:]
    with np.errstate(over="ignore"):
        return w.astype(np.float32).astype(np.float16).reshape(N, K)


def test_oracle_decode_matches_the_formula_on_every_block_kind():
    qt, bi, levels = exhaustive_case()
    assert np.array_equal(orc.extract_levels(qt), levels)
    got = orc.dequant_d64(qt, bi)
    want = numpy_decode_f64(qt, bi, levels)
    g, w = got.view(np.uint16).astype(np.int64), want.view(np.uint16).astype(np.int64)
    # the two float64 evaluations may associate the PCA terms differently: identical but for
    # isolated last-place differences of the float16 result
    same = g == w
    assert same.mean() >= 0.9999
    assert np.abs(g - w).max() <= 1
    assert np.array_equal(orc.dequant_d64(qt, bi, use_pca=False), numpy_decode_f64(
        qt, {"n_cb": NCB, "data": bi["data"] * 0, "scales": bi["scales"]}, levels))


@pytest.mark.gpu
def test_gpu_kernels_on_every_block_kind():
    import torch
    from sx8_quantization_b200 import ops, _lib
    qt, bi, levels = exhaustive_case()
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    planes = (d(qt["dmin"].view(np.uint8)).view(torch.float16), d(qt["dmax"].view(np.uint8)).view(torch.float16),
              d(qt["config"]), d(qt["coeff"].reshape(-1)), d(qt["levels_hi"]), d(qt["levels_lo"]))
    bas, sca = d(bi["data"]), d(bi["scales"])
    # layouts: bit-exact
    wt = ops.repack_t16(*planes, N, NCB)
    assert np.array_equal(wt.cpu().numpy().reshape(-1), orc.to_t16(qt).reshape(-1))
    blocks = ops.blocks_from_planes(*planes)
    assert np.array_equal(blocks.cpu().numpy(), orc.blocks_from_planes(qt))
    assert torch.equal(ops.repack_t16_blocks(blocks, N, NCB), wt)
    v44 = orc.to_v44(qt, bi)
    hdr, lev = ops.repack_v44(*planes, N, NCB)
    assert np.array_equal(hdr.cpu().numpy(), v44["hdr"]) and np.array_equal(lev.cpu().numpy(), v44["levels"])
    # float64 decode: bit-exact from both layouts, with and without the PCA term
    for pca in (True, False):
        ref = orc.dequant_d64(qt, bi, use_pca=pca).view(np.uint16)
        a = ops.dequant_planes(*planes, bas, sca, N, K, NCB, pca).cpu().numpy().view(np.uint16)
        b = ops.dequant_t16(wt, bas, sca, N, K, NCB, pca).cpu().numpy().view(np.uint16)
        assert np.array_equal(a, ref) and np.array_equal(b, ref)
    # float32 embedding rows: bit-exact, every row
    ids = np.arange(N, dtype=np.int64)
    rows = ops.embed(d(ids), wt, bas, sca, K, N, NCB).cpu().numpy().view(np.uint16)
    assert np.array_equal(rows, orc.embed_d32(ids, v44).view(np.uint16))
    # GEMV and GEMM against the float32 matmul on the decoded weights.  Rows whose blocks reach
    # +-60000 dominate the scale, so compare per output column, relative to that column's
    # absolute-value product (the bound of its rounding error).
    w = orc.dequant_d64(qt, bi).astype(np.float32)
    x = orc.synth_x(8, K, 77, scale=0.05)
    ref = x.astype(np.float32) @ w.T
    bound = np.abs(x.astype(np.float32)) @ np.abs(w).T + 1e-20
    y = ops.gemv(d(x), wt, bas, sca, N, K, NCB).cpu().numpy()
    assert np.isfinite(y).all() and (np.abs(y - ref) / bound).max() <= 2e-3
    # The GEMM rounds weights to fp16 (as the reference's tensor-core path does); blocks with an
    # endpoint of magnitude >= 32768 form them in float32 first, so the +-65504 blocks stay finite.
    xg = orc.synth_x(160, K, 78, scale=0.05)
    refg = xg.astype(np.float32) @ w.T
    boundg = np.abs(xg.astype(np.float32)) @ np.abs(w).T + 1e-20
    yg = ops.gemm(d(xg), wt, bas, sca, N, K, NCB).cpu().numpy()
    assert np.isfinite(yg).all() and (np.abs(yg - refg) / boundg).max() <= 4e-3
    assert _lib.device_error_flag() == 0
