// sx8_common.cuh -- shared device/host helpers for the S-X8 v4.3 kernels (sm_100a).
#pragma once
#include <stdlib.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/sx8_b200.h"

namespace sx8 {

// ----------------------------------------------------------------------------- errors
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define SX8_REQUIRE(cond, ...)            \
    do {                                  \
        if (!(cond)) {                    \
            sx8::set_error(__VA_ARGS__);  \
            return SX8_E_INVALID;         \
        }                                 \
    } while (0)

#define SX8_LAUNCH_CHECK(what)                                   \
    do {                                                         \
        cudaError_t e__ = cudaGetLastError();                    \
        if (e__ != cudaSuccess) return sx8::cuda_fail(e__, what); \
    } while (0)

// Device-side error word: set by a bounded wait that ran out (see sx8_gemv.cu).
extern __device__ unsigned g_sx8_error_flag;

// ----------------------------------------------------------------------------- decode
// Signed 4-bit PCA coefficient: ref docs/SX8_FLASH_V4_3_SPEC.md:25.
__device__ __forceinline__ int s4(int x) { return x < 8 ? x : x - 16; }

// Level of weight i (0..7) of one sub-block from its v4.4 words:
// hi4 = 8 nibbles (weight i at bits 4i), lo2 = 2 bytes (weight i at bits
// (i>>2)*8 + (3-(i&3))*2).  ref cuda/sx8_decode1_v3.cu:147-149.
__device__ __forceinline__ int level_of(uint32_t hi4, uint32_t lo2, int i) {
    int nib = (int)((hi4 >> (i * 4)) & 0xF);
    int qua = (int)((lo2 >> ((i >> 2) * 8 + (3 - (i & 3)) * 2)) & 0x3);
    return (nib << 2) | qua;
}

// float32 range decode of one sub-block, the reference CUDA kernels' arithmetic
// (ref cuda/sx8_embed_v44.cu:50-56) with nvcc's default multiply-add contraction
// frozen as explicit fused operations.
__device__ __forceinline__ void range_d32(float lo_f, float hi_f, int s, float& rlo, float& step) {
    float q = __fmul_rn(__fsub_rn(hi_f, lo_f), 0.25f);
    float kl = (float)(3 * (s == 2) + (s == 3));
    float kh = (float)(3 * (s == 1) + (s == 3));
    rlo = __fmaf_rn(q, kl, lo_f);
    float rhi = __fmaf_rn(-q, kh, hi_f);
    step = __fmul_rn(__fsub_rn(rhi, rlo), 0.015873f);
    if (step < 1e-10f) step = 1e-10f;
}

// float64 decode of one weight, the numba reference decoder's arithmetic
// (ref scripts/kernel_sx8_v43.py:28-49): float32 subtraction for the range, float64
// for everything after it, fused multiply-adds where NVVM contracts them.
struct RangeD64 {
    double rlo, step;
};
__device__ __forceinline__ RangeD64 range_d64(float lo_f, float hi_f, int s) {
    float d32 = __fsub_rn(hi_f, lo_f);
    double q = __dmul_rn((double)d32, 0.25);
    double rlo, rhi;
    if (s == 0) { rlo = lo_f; rhi = hi_f; }
    else if (s == 1) { rlo = lo_f; rhi = __dadd_rn((double)lo_f, q); }
    else if (s == 2) { rlo = __dsub_rn((double)hi_f, q); rhi = hi_f; }
    else { rlo = __dadd_rn((double)lo_f, q); rhi = __dsub_rn((double)hi_f, q); }
    double step = __dmul_rn(__dsub_rn(rhi, rlo), 0.015873);
    if (step < 1e-10) step = 1e-10;
    return {rlo, step};
}

// Launch-shape and timing experiments are compiled in only with -DSX8_EXPERIMENT (some of them
// make the kernels produce wrong results on purpose); the default build reads no environment
// variable and carries none of those branches.
#ifdef SX8_EXPERIMENT
inline int exp_env(const char* name, int dflt) {
    const char* v = getenv(name);
    return v ? atoi(v) : dflt;
}
#define SX8_DBG(p) ((p).debug)
#else
#define exp_env(name, dflt) (dflt)
#define SX8_DBG(p) 0
#endif

__device__ __forceinline__ float h2f_bits(uint16_t b) { return __half2float(__ushort_as_half(b)); }

}  // namespace sx8
