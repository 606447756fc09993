// sx8_gemm.cu -- S-X8 v4.3 prefill GEMM entry point (Y = X * W^T, W decoded on the fly).
//
// M <= 16 runs on the decode-GEMV kernel in one pass over the weights (two blocks of 8
// activation rows per decoded weight fragment); larger M runs on the tcgen05 kernel in
// sx8_gemm_tc.cu.
#include "sx8_common.cuh"

namespace sx8 {
int gemv_launch(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                const float* scales, int N, int n_cb, float* y, void* workspace, unsigned flags,
                cudaStream_t stream);
int gemv_rows_launch(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                     const float* scales, int N, int n_cb, float* y, void* xstage, void* table, unsigned flags,
                     cudaStream_t stream);
int gemv_rows_launch_multi(const void* x, int M, int K, long ldx, int count, const void* const* wt16,
                           const float* const* bases, const float* const* scales, const int* N, float* const* y,
                           int n_cb, void* xstage, void* table, unsigned flags, cudaStream_t stream);
int gemv_launch_multi(const void* x, int M, int K, long ldx, int count, const void* const* wt16,
                      const float* const* bases, const float* const* scales, const int* N, float* const* y,
                      int n_cb, void* workspace, unsigned flags, cudaStream_t stream);
int gemv_check(const char* who, const void* x, int M, int Mmax, int K, long ldx, const void* wt16,
               const float* bases, const float* scales, int N, int n_cb, const void* y);
size_t gemm_tc_workspace_bytes(int M, int N, int n_cb);
bool gemm_tc_supported(int M, int N, int K, int n_cb);
int gemm_tc_launch(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                   const float* scales, int N, int n_cb, void* y, int out_f16, void* workspace,
                   cudaStream_t stream);
size_t gemm_tc_multi_workspace_bytes(int M, int n_cb, int nmat);
int gemm_tc_launch_multi(const void* x, int M, int K, long ldx, int nmat, const void* const* wt16,
                         const float* const* bases, const float* const* scales, const int* N, int n_cb,
                         void* const* y, int out_f16, void* workspace, cudaStream_t stream);

__global__ void __launch_bounds__(256) f32_to_f16_kernel(const float* __restrict__ in, __half* __restrict__ out, long n) {
    long i = ((long)blockIdx.x * 256 + threadIdx.x) * 4;
    // 8-byte stores only when `out` allows them (an f16 view at an odd element-pair offset is
    // 4-byte aligned only); uniform over the grid
    const bool vec_ok = (reinterpret_cast<uintptr_t>(out) & 7) == 0;
    if (i + 3 < n && vec_ok) {
        float4 v = *reinterpret_cast<const float4*>(in + i);
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 o = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
        *reinterpret_cast<uint2*>(out + i) = o;
    } else {
        for (long e = i + 4 < n ? i + 4 : n; i < e; i++) out[i] = __float2half_rn(in[i]);
    }
}
}  // namespace sx8

using namespace sx8;

static size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }
static const int kGemvRowsMax = 16;   // batch rows the GEMV kernel takes in one pass

extern "C" size_t sx8_gemm_workspace_bytes(int M, int N, int n_cb) {
    if (M <= 0 || N <= 0 || n_cb <= 0) return 0;
    // small-M path: [staged x (M, 32 n_cb) f16][activation table n_cb * M * 16][f32 result when Y is f16]
    size_t a = 0;
    if (M <= kGemvRowsMax)
        a = round256((size_t)M * n_cb * 64) + round256((size_t)M * n_cb * 16) + round256((size_t)M * (size_t)N * 4);
    size_t tc = gemm_tc_workspace_bytes(M, N, n_cb);
    return a > tc ? a : tc;
}

extern "C" int sx8_gemm(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                        const float* scales, int N, int n_cb, void* y, int out_f16, void* workspace,
                        size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    int rc = gemv_check("sx8_gemm", x, M, 0x7FFFFFFF, K, ldx, wt16, bases, scales, N, n_cb, y);
    if (rc != SX8_OK) return rc;
    SX8_REQUIRE((long)M * (long)N < (1L << 40), "sx8_gemm: output too large");
    if (!workspace || workspace_bytes < sx8_gemm_workspace_bytes(M, N, n_cb) ||
        (reinterpret_cast<uintptr_t>(workspace) % 256) != 0) {
        set_error("sx8_gemm: workspace must be 256-byte aligned and hold %zu bytes (got %zu)",
                  sx8_gemm_workspace_bytes(M, N, n_cb), workspace_bytes);
        return SX8_E_WORKSPACE;
    }
    if (M > kGemvRowsMax && gemm_tc_supported(M, N, K, n_cb))
        return gemm_tc_launch(x, M, K, ldx, wt16, bases, scales, N, n_cb, y, out_f16, workspace, stream);
    if (M > kGemvRowsMax) {
        set_error("sx8_gemm: the tensor-core path is unavailable (driver without cuTensorMapEncodeTiled) and M=%d is "
                  "beyond the %d rows of the GEMV path", M, kGemvRowsMax);
        return SX8_E_UNSUPPORTED;
    }
    uint8_t* xstage = (uint8_t*)workspace;
    uint8_t* table = xstage + round256((size_t)M * n_cb * 64);
    float* y32 = out_f16 ? (float*)(table + round256((size_t)M * n_cb * 16)) : (float*)y;
    if (M <= 8)
        rc = gemv_launch(x, M, K, ldx, wt16, bases, scales, N, n_cb, y32, xstage, 0u, stream);
    else
        rc = gemv_rows_launch(x, M, K, ldx, wt16, bases, scales, N, n_cb, y32, xstage, table, 0u, stream);
    if (rc != SX8_OK) return rc;
    if (out_f16) {
        long n = (long)M * N;
        f32_to_f16_kernel<<<(unsigned)((n / 4 + 255) / 256 + 1), 256, 0, stream>>>(y32, (__half*)y, n);
        SX8_LAUNCH_CHECK("f32_to_f16_kernel");
    }
    return SX8_OK;
}

// ---- several prefill GEMMs on the same activations -------------------------------------------
static const int kGemmMultiMax = 3;

// One launch when the tensor-core path takes the call (M > 16) and every matrix but the last is a
// multiple of 256 columns wide, or when the GEMV kernel takes it (M <= 16) and Y is float32;
// otherwise one sx8_gemm per matrix, with the same results.
static bool gemm_multi_fusable(int M, int count, const int* N, int K, int n_cb) {
    if (M <= kGemvRowsMax || count < 2 || !gemm_tc_supported(M, N[0], K, n_cb)) return false;
    for (int i = 0; i + 1 < count; i++)
        if (N[i] % 256 != 0) return false;
    return true;
}

extern "C" size_t sx8_gemm_multi_workspace_bytes(int M, int count, const int* N, int n_cb) {
    if (M <= 0 || count <= 0 || count > kGemmMultiMax || !N || n_cb <= 0) return 0;
    size_t need = gemm_tc_multi_workspace_bytes(M, n_cb, count);
    if (M <= kGemvRowsMax) {   // [staged x][count activation tables]
        size_t g = round256((size_t)M * n_cb * 64) + round256((size_t)count * M * n_cb * 16);
        if (g > need) need = g;
    }
    for (int i = 0; i < count; i++) {
        size_t one = sx8_gemm_workspace_bytes(M, N[i], n_cb);
        if (one > need) need = one;
    }
    return need;
}

extern "C" int sx8_gemm_multi(const void* x, int M, int K, long ldx, int count, const void* const* wt16,
                              const float* const* bases, const float* const* scales, const int* N,
                              void* const* y, int out_f16, int n_cb, void* workspace, size_t workspace_bytes,
                              void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    SX8_REQUIRE(count >= 1 && count <= kGemmMultiMax, "sx8_gemm_multi: count must be 1..%d (got %d)", kGemmMultiMax, count);
    SX8_REQUIRE(wt16 && bases && scales && N && y, "sx8_gemm_multi: null array");
    long total = 0;
    for (int i = 0; i < count; i++) {
        int rc = gemv_check("sx8_gemm_multi", x, M, 0x7FFFFFFF, K, ldx, wt16[i], bases[i], scales[i], N[i], n_cb, y[i]);
        if (rc != SX8_OK) return rc;
        total += N[i];
    }
    SX8_REQUIRE((long)M * total < (1L << 40) && total < 0x7FFFFFFFL, "sx8_gemm_multi: output too large");
    if (!workspace || workspace_bytes < sx8_gemm_multi_workspace_bytes(M, count, N, n_cb) ||
        (reinterpret_cast<uintptr_t>(workspace) % 256) != 0) {
        set_error("sx8_gemm_multi: workspace must be 256-byte aligned and hold %zu bytes (got %zu)",
                  sx8_gemm_multi_workspace_bytes(M, count, N, n_cb), workspace_bytes);
        return SX8_E_WORKSPACE;
    }
    if (gemm_multi_fusable(M, count, N, K, n_cb))
        return gemm_tc_launch_multi(x, M, K, ldx, count, wt16, bases, scales, N, n_cb, y, out_f16, workspace, stream);
    if (M <= kGemvRowsMax && !out_f16 && count >= 2) {
        uint8_t* xstage = (uint8_t*)workspace;
        if (M <= 8)
            return gemv_launch_multi(x, M, K, ldx, count, wt16, bases, scales, N, (float* const*)y, n_cb, xstage, 0u, stream);
        return gemv_rows_launch_multi(x, M, K, ldx, count, wt16, bases, scales, N, (float* const*)y, n_cb, xstage,
                                      xstage + round256((size_t)M * n_cb * 64), 0u, stream);
    }
    for (int i = 0; i < count; i++) {
        int rc = sx8_gemm(x, M, K, ldx, wt16[i], bases[i], scales[i], N[i], n_cb, y[i], out_f16, workspace, workspace_bytes, stream_);
        if (rc != SX8_OK) return rc;
    }
    return SX8_OK;
}
