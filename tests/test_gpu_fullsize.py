"""Full-size checks of the paths that only large shapes reach: the launch rule and the long
activation table of 70B-class GEMVs, and the two-CTA tensor-core GEMM at BASELINE sizes.
The CPU oracle would take minutes at these sizes, so the comparator is a float32 matmul on
the dequantised weights (sx8_dequant_t16, itself bit-exact against the oracle in
test_gpu_parity.py), plus properties that do not depend on size: agreement between launch
shapes, determinism, linearity, empty inputs."""

import pytest

pytestmark = pytest.mark.gpu


def _tensor(n, k, seed, with_pca=True):
    import torch
    from sx8_quantization_b200 import ops, quantizer
    t = quantizer.quantize_tensor(quantizer.synth_weight_gpu(n, k, seed), with_pca=with_pca)
    w = ops.dequant_t16(t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"], True).float()
    return t, w


def _x(m, k, seed):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(m, k, generator=g, device="cuda").half()


def _rel(a, b):
    return (a - b).abs().max().item() / max(1e-30, b.abs().max().item())


@pytest.mark.parametrize("shape", [(8192, 8192), (2048, 28672), (28672, 2048)])
@pytest.mark.parametrize("M", [1, 2, 5, 8])
def test_gemv_large_shapes_against_float32_matmul(shape, M):
    """(8192, 8192) is above the 48 MB threshold of the large-matrix launch rule; K = 28672
    gives 896 block rows, i.e. CTAs whose activation table spans hundreds of block rows."""
    from sx8_quantization_b200 import ops, _lib
    n, k = shape
    t, w = _tensor(n, k, 70 + M)
    x = _x(M, k, 3)
    y = ops.gemv(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"])
    ref = x.float() @ w.t()
    assert _rel(y, ref) <= 2e-3          # the reference's own acceptance is 5e-3 of max
    assert _lib.device_error_flag() == 0


def test_gemv_launch_shapes_agree_and_are_deterministic():
    """The same product through forced launch shapes (tile-group width, split-K) differs only
    by float32 summation order; each shape is bit-reproducible."""
    import torch
    from sx8_quantization_b200 import ops, _lib
    n, k = 4096, 8192
    t, w = _tensor(n, k, 81)
    x = _x(4, k, 5)
    L = _lib.lib()
    outs = []
    try:
        for nt, split in ((0, 0), (8, 1), (8, 4), (4, 2), (2, 8)):
            L.sx8_gemv_tune(nt if nt else -1, split if split else -1, -1)
            a = ops.gemv(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"]).clone()
            b = ops.gemv(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"]).clone()
            assert torch.equal(a, b)
            outs.append(a)
    finally:
        L.sx8_gemv_tune(-1, -1, -1)
    for o in outs[1:]:
        assert _rel(o, outs[0]) <= 1e-4
    assert _rel(outs[0], x.float() @ w.t()) <= 2e-3


@pytest.mark.parametrize("M", [300, 2048, 8192])
@pytest.mark.parametrize("f16out", [True, False])
def test_gemm_gate_projection_full_size(M, f16out):
    """BASELINE config 2 shape (9728 x 2560): M = 300 runs the two-CTA tiles with a ragged last
    row tile, 2048 and 8192 several waves of them."""
    import torch
    from sx8_quantization_b200 import ops, _lib
    n, k = 9728, 2560
    t, w = _tensor(n, k, 90)
    x = _x(M, k, 7)
    y = ops.gemm(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"],
                 out_dtype=torch.float16 if f16out else torch.float32)
    ref = x.float() @ w.t()
    # weights are rounded to fp16 inside the GEMM (as in the reference's tensor-core path)
    assert _rel(y.float(), ref) <= (4e-3 if f16out else 3e-3)
    assert _lib.device_error_flag() == 0


def test_gemm_linearity_and_row_independence():
    """Y(x1 + x2) = Y(x1) + Y(x2) up to rounding, and a row of Y depends on its row of X only
    (the same row gives the same bits whatever the other rows and whatever M is)."""
    import torch
    from sx8_quantization_b200 import ops
    n, k = 2560, 4096
    t, _ = _tensor(n, k, 91)
    a, b = _x(600, k, 11), _x(600, k, 12)
    f = lambda x: ops.gemm(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"], out_dtype=torch.float32)
    ya, yb, yab = f(a), f(b), f((a.float() + b.float()).half())
    assert _rel(yab, ya + yb) <= 3e-3
    mixed = torch.cat([a[:100], b[:500]])
    assert torch.equal(f(mixed)[:100], ya[:100])
    assert torch.equal(f(a[:300]), ya[:300])          # the same tile shape for M = 300 and 600


def test_empty_inputs():
    import torch
    from sx8_quantization_b200 import ops
    n, k = 64, 256
    t, _ = _tensor(n, k, 92)
    y = ops.gemm(torch.empty(0, k, dtype=torch.float16, device="cuda"), t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"])
    assert y.shape == (0, n)
    e = ops.embed(torch.empty(0, dtype=torch.long, device="cuda"), t["wt16"], t["bases"], t["scales"], k, n, t["n_cb"])
    assert e.shape == (0, k)


@pytest.mark.parametrize("shape,M", [((2560, 9728), 128), ((2560, 9728), 256), ((4096, 2592), 100), ((1024, 2560), 33)])
@pytest.mark.parametrize("f16out", [True, False])
def test_gemm_split_k_cluster(shape, M, f16out):
    """Few column tiles and M <= 256: two CTAs of a cluster share a tile, each taking half of K
    (K = 2592 gives an odd number of 64-wide K stages, 21 + 20); the result is deterministic."""
    import torch
    from sx8_quantization_b200 import ops, _lib
    n, k = shape
    t, w = _tensor(n, k, 95)
    x = _x(M, k, 13)
    od = torch.float16 if f16out else torch.float32
    y = ops.gemm(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"], out_dtype=od)
    y2 = ops.gemm(x, t["wt16"], t["bases"], t["scales"], n, k, t["n_cb"], out_dtype=od)
    assert torch.equal(y, y2)
    assert _rel(y.float(), x.float() @ w.t()) <= (4e-3 if f16out else 3e-3)
    assert _lib.device_error_flag() == 0
