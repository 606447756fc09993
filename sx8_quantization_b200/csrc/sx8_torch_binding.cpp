// sx8_torch_binding.cpp -- thin PyTorch binding over the C ABI of libsx8b200.so.
//
// The reference binds its kernels with pybind through torch's load_inline
// (ref scripts/sx8_decode1_v3.py:36-53): one foreign call per kernel, tensors in, the current
// CUDA stream taken inside.  This module is the same shape of binding for the hot calls --
// one call per operation taking tensors, the device guard and the current stream resolved in
// C++ -- and nothing else: every function forwards to an `extern "C"` entry point of
// include/sx8_b200.h and returns its status code (0, or a negative SX8_E_* with the message in
// sx8_last_error()), so that the Python layer raises the same SX8Error on every binding.
// It exists because the per-call host cost is what an eager decode loop pays 250 times per
// token: resolving stream, device and seven data pointers from Python costs more than the
// kernel launch itself.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "sx8_b200.h"

namespace {

inline void need(const at::Tensor& t, at::ScalarType dt, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.scalar_type() == dt, name, " has the wrong dtype");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

inline void need_x(const at::Tensor& x) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kHalf, "x must be a CUDA float16 tensor");
    TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.stride(0) >= x.size(1), "x must be (M, K) with unit inner stride");
}

// y (M, N) f32 = x (M, K) f16 * W^T, M <= 8 (sx8_gemv).  Returns the C ABI's status.
int64_t gemv(const at::Tensor& x, const at::Tensor& wt16, const at::Tensor& bases, const at::Tensor& scales,
             int64_t N, int64_t K, int64_t n_cb, const at::Tensor& out, const at::Tensor& workspace, int64_t flags) {
    need_x(x);
    need(wt16, at::kByte, "wt16");
    need(bases, at::kFloat, "bases");
    need(scales, at::kFloat, "scales");
    need(out, at::kFloat, "out");
    need(workspace, at::kByte, "workspace");
    const int64_t M = x.size(0);
    TORCH_CHECK(out.numel() == M * N, "out has ", out.numel(), " elements, need ", M * N);
    TORCH_CHECK((size_t)wt16.numel() == sx8_t16_bytes((long)N, (int)n_cb), "wt16 does not have the T16 size of (N, n_cb)");
    c10::cuda::CUDAGuard guard(x.device());
    return sx8_gemv(x.data_ptr(), (int)M, (int)K, (long)x.stride(0), wt16.data_ptr(), bases.data_ptr<float>(),
                    scales.data_ptr<float>(), (int)N, (int)n_cb, out.data_ptr<float>(), workspace.data_ptr(),
                    (size_t)workspace.numel(), (unsigned)flags, c10::cuda::getCurrentCUDAStream(x.device().index()).stream());
}

// Y (M, N) = X (M, K) f16 * W^T, any M (sx8_gemm); out is f32 or f16.
int64_t gemm(const at::Tensor& x, const at::Tensor& wt16, const at::Tensor& bases, const at::Tensor& scales,
             int64_t N, int64_t K, int64_t n_cb, const at::Tensor& out, const at::Tensor& workspace) {
    need_x(x);
    need(wt16, at::kByte, "wt16");
    need(bases, at::kFloat, "bases");
    need(scales, at::kFloat, "scales");
    need(workspace, at::kByte, "workspace");
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && (out.scalar_type() == at::kFloat || out.scalar_type() == at::kHalf),
                "out must be a contiguous CUDA float32 or float16 tensor");
    const int64_t M = x.size(0);
    TORCH_CHECK(out.numel() == M * N, "out has ", out.numel(), " elements, need ", M * N);
    TORCH_CHECK((size_t)wt16.numel() == sx8_t16_bytes((long)N, (int)n_cb), "wt16 does not have the T16 size of (N, n_cb)");
    c10::cuda::CUDAGuard guard(x.device());
    return sx8_gemm(x.data_ptr(), (int)M, (int)K, (long)x.stride(0), wt16.data_ptr(), bases.data_ptr<float>(),
                    scales.data_ptr<float>(), (int)N, (int)n_cb, out.data_ptr(), out.scalar_type() == at::kHalf ? 1 : 0,
                    workspace.data_ptr(), (size_t)workspace.numel(),
                    c10::cuda::getCurrentCUDAStream(x.device().index()).stream());
}

// out (T, K) f16 = decoded rows ids[t] (sx8_embed).
int64_t embed(const at::Tensor& ids, const at::Tensor& wt16, const at::Tensor& bases, const at::Tensor& scales,
              int64_t K, int64_t N, int64_t n_cb, const at::Tensor& out) {
    need(ids, at::kLong, "ids");
    need(wt16, at::kByte, "wt16");
    need(bases, at::kFloat, "bases");
    need(scales, at::kFloat, "scales");
    need(out, at::kHalf, "out");
    TORCH_CHECK(out.numel() >= ids.numel() * K, "out too small");
    c10::cuda::CUDAGuard guard(ids.device());
    return sx8_embed(ids.data_ptr<int64_t>(), (long)ids.numel(), wt16.data_ptr(), bases.data_ptr<float>(),
                     scales.data_ptr<float>(), (int)K, (int)N, (int)n_cb, out.data_ptr(),
                     c10::cuda::getCurrentCUDAStream(ids.device().index()).stream());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "thin torch binding over the C ABI of libsx8b200.so";
    m.def("gemv", &gemv);
    m.def("gemm", &gemm);
    m.def("embed", &embed);
    m.def("last_error", []() { return std::string(sx8_last_error()); });
    m.def("gemv_workspace_bytes", [](int64_t n_cb, int64_t M) { return (int64_t)sx8_gemv_workspace_bytes((int)n_cb, (int)M); });
    m.def("gemm_workspace_bytes",
          [](int64_t M, int64_t N, int64_t n_cb) { return (int64_t)sx8_gemm_workspace_bytes((int)M, (int)N, (int)n_cb); });
}
