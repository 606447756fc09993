"""The workspace-free GEMM entry point (sx8_gemm_static), called through the C ABI.

Some hosts may not allocate device memory once they are running (all memory already
handed to their own arena, or a plug-in contract that forbids cudaMalloc).  For them the
library keeps the GEMM's scratch in a fixed internal array.  This test checks, on two
calls in a row with different tensors (the array keeps the first call's contents), that
the result equals the regular entry point's, and that oversize problems are refused.
The file name sorts last so that a run stopping at the first failure has already run
every other test."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import sx8_oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _case(N, K, seed):
    qt, bi = orc.quantize(orc.synth_weight(N, K, seed))
    return qt, _dev(orc.to_t16(qt)), _dev(bi["data"]), _dev(bi["scales"])


def test_static_gemm_matches_workspace_gemm_twice():
    from sx8_quantization_b200 import _lib, ops
    L = _lib.lib()
    assert L.sx8_gemm_static_max_ncb() == 1024
    stream = torch.cuda.current_stream().cuda_stream
    # second case has fewer block rows than the first: stale table rows beyond it must not matter
    for (N, K, M, seed, f16) in [(512, 2560, 200, 71, False), (272, 1024, 96, 72, True)]:
        qt, wt, bas, sca = _case(N, K, seed)
        x = _dev(orc.synth_x(M, K, seed + 1))
        dt = torch.float16 if f16 else torch.float32
        want = ops.gemm(x, wt, bas, sca, N, K, qt["n_cb"], out_dtype=dt)
        got = torch.empty(M, N, dtype=dt, device="cuda")
        rc = L.sx8_gemm_static(x.data_ptr(), M, K, x.stride(0), wt.data_ptr(), bas.data_ptr(), sca.data_ptr(),
                               N, qt["n_cb"], got.data_ptr(), int(f16), stream)
        assert rc == 0, L.sx8_last_error()
        torch.cuda.synchronize()
        ref = orc.matmul_ref(x.cpu().numpy(), orc.dequant_d64(qt, {"data": bas.cpu().numpy(), "scales": sca.cpu().numpy()}))
        tol = 2e-3 + (2.0 ** -10 if f16 else 0.0)          # the suite's GEMM tolerance
        assert np.abs(got.float().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
        assert torch.equal(got, want)                        # same kernel, same table: same bits
    assert _lib.device_error_flag() == 0


@pytest.mark.parametrize("N,K,ldx,M", [(272, 2592, 2592, 96),     # odd number of block rows (81): last stage half filled
                                       (272, 1000, 1000, 40),     # K not a multiple of 32: x tail zero-filled by the copy
                                       (512, 1024, 1024, 1),      # fewer rows than this entry point's smallest tile
                                       (512, 1024, 1032, 8)])     # padded row stride
def test_static_gemm_small_and_ragged_cases(N, K, ldx, M):
    """Shapes that only this entry point sends to the tensor-core kernel (sx8_gemm runs M < 32
    on the GEMV kernel).  A large call comes first so that the shared array holds another
    tensor's table rows beyond the ones these cases rewrite."""
    from sx8_quantization_b200 import _lib, ops
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    qt0, wt0, bas0, sca0 = _case(64, 8192, 80)
    x0 = _dev(orc.synth_x(32, 8192, 81))
    y0 = torch.empty(32, 64, dtype=torch.float32, device="cuda")
    assert L.sx8_gemm_static(x0.data_ptr(), 32, 8192, 8192, wt0.data_ptr(), bas0.data_ptr(), sca0.data_ptr(),
                             64, qt0["n_cb"], y0.data_ptr(), 0, stream) == 0, L.sx8_last_error()
    qt, wt, bas, sca = _case(N, K, 73)
    xh = orc.synth_x(M, K, 74)
    xbuf = torch.zeros(M, ldx, dtype=torch.float16, device="cuda")
    xbuf[:, :K] = _dev(xh)
    ref = orc.matmul_ref(xh, orc.dequant_d64(qt, {"data": bas.cpu().numpy(), "scales": sca.cpu().numpy()}))
    for _ in range(2):
        got = torch.empty(M, N, dtype=torch.float32, device="cuda")
        rc = L.sx8_gemm_static(xbuf.data_ptr(), M, K, ldx, wt.data_ptr(), bas.data_ptr(), sca.data_ptr(),
                               N, qt["n_cb"], got.data_ptr(), 0, stream)
        assert rc == 0, L.sx8_last_error()
        torch.cuda.synchronize()
        assert np.abs(got.cpu().numpy() - ref).max() <= 2e-3 * np.abs(ref).max()
    if M >= 32:
        assert torch.equal(got, ops.gemm(xbuf[:, :K], wt, bas, sca, N, K, qt["n_cb"]))
    assert _lib.device_error_flag() == 0


def test_static_gemm_rejects_what_it_cannot_hold():
    from sx8_quantization_b200 import _lib
    L = _lib.lib()
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    n_cb = 1025
    rc = L.sx8_gemm_static(p, 8, n_cb * 32, n_cb * 32, p, p, p, 16, n_cb, p, 0, None)
    assert rc == -1 and b"exceeds the built-in scratch" in L.sx8_last_error()
    rc = L.sx8_gemm_static(p + 2, 8, 64, 64, p, p, p, 16, 2, p, 0, None)      # misaligned x
    assert rc == -1 and b"16-byte aligned" in L.sx8_last_error()
    rc = L.sx8_gemm_static(p, 8, 64, 68, p, p, p, 16, 2, p, 0, None)          # row stride not a multiple of 8
    assert rc == -1
    rc = L.sx8_gemm_static(p, 8, 64, 56, p, p, p, 16, 2, p, 0, None)          # row stride shorter than a row
    assert rc == -1 and b"< K" in L.sx8_last_error()
    rc = L.sx8_gemm_static(p, 8, 64, 64, p, p, p + 2, 16, 2, p, 0, None)      # misaligned scales
    assert rc == -1 and b"misaligned" in L.sx8_last_error()
