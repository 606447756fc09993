// sx8_codec.cu -- S-X8 v4.3 codec kernels for sm_100a.  Bit-exact with the reference: full-tensor
// decode, embedding-row decode, quantizer search + packing, file-plane -> device-layout repack.
// Functional parity (the reference's result depends on its LAPACK build): the three passes of the
// quantizer's PCA stage.  All of it is byte/float work on CUDA cores in which one thread owns one
// 8-weight sub-block, so a warp touches 8 consecutive blocks with 4-, 8- and 16-byte accesses.
#include "sx8_common.cuh"
#include "sx8_layout.cuh"

namespace sx8 {

// Store up to 8 halfs at dst (row-major output), vectorised when the row allows it.
__device__ __forceinline__ void store8(__half* dst, const __half (&v)[8], int n_valid, bool vec_ok) {
    if (n_valid >= 8 && vec_ok) {
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(v);
    } else {
        for (int i = 0; i < 8; i++)
            if (i < n_valid) dst[i] = v[i];
    }
}

// ------------------------------------------------------------------ dequant (float64)
// LAYOUT 0: n-major file planes (bid = n*n_cb + kb); LAYOUT 1: the T16 device blob (in .levels).
struct DequantArgs {
    const uint16_t* dmin;
    const uint16_t* dmax;
    const uint8_t* config;
    const uint8_t* coeff;
    const uint8_t* hi;
    const uint8_t* lo;
    const uint8_t* hdr;
    const uint8_t* levels;
    const float* bases;
    const float* scales;
    long out_f, in_f;
    int n_cb, hdr_bytes, use_pca;
    __half* out;
};

// Exact integer -> double without the conversion unit: 2^52 + u has u in its low mantissa bits.
__device__ __forceinline__ double u2d(uint32_t u) {
    return __dsub_rn(__hiloint2double(0x43300000, (int)u), 4503599627370496.0);
}

// One CTA decodes 32 rows x 8 block columns (four passes of 8 rows; thread = (row, kb, sub-block), sub-block
// fastest): per row it reads 128 contiguous bytes of levels_hi and writes 512 contiguous bytes.  The two bases and
// the scales of the CTA's 8 block columns are converted to double once, into shared memory; levels and the signed
// coefficients become doubles by exponent arithmetic.  What is left for the (slow) conversion unit per weight is the
// float64 -> float32 rounding and half of a float32 -> float16 pair.  The arithmetic itself is unchanged: every
// double operation of the reference decoder, in its order (ref scripts/kernel_sx8_v43.py:22-51).
constexpr int kDqKb = 8, kDqRows = 32;

template <int LAYOUT>
__global__ void __launch_bounds__(256) dequant_d64_kernel(DequantArgs a) {
    // basis value (kl, j, t) at kl * 84 + j * 36 + (t >> 3) * 9 + (t & 7): the 16 lanes of a half-warp (4 block
    // columns x 4 sub-blocks) then read 16 different 8-byte banks
    __shared__ double B[kDqKb * 84];
    __shared__ double S[kDqKb][2];
    const int tid = threadIdx.x;
    const long kgroups = (a.n_cb + kDqKb - 1) / kDqKb;
    const long rt = (long)blockIdx.x / kgroups;
    const int kb0 = (int)((long)blockIdx.x - rt * kgroups) * kDqKb;
    const long r0 = rt * kDqRows;
    if (a.use_pca) {
        for (int i = tid; i < kDqKb * 64; i += 256) {
            const int kb = kb0 + (i >> 6);
            const int t = i & 31;
            B[(i >> 6) * 84 + ((i >> 5) & 1) * 36 + (t >> 3) * 9 + (t & 7)] = (kb < a.n_cb) ? (double)a.bases[(long)kb * 64 + (i & 63)] : 0.0;
        }
        if (tid < kDqKb * 2) {
            const int kb = kb0 + (tid >> 1);
            S[tid >> 1][tid & 1] = (kb < a.n_cb) ? (double)a.scales[kb * 2 + (tid & 1)] : 0.0;
        }
    }
    __syncthreads();
    const int sb = tid & 3, kl = (tid >> 2) & 7, kb = kb0 + kl;
    const bool vec_ok = (a.in_f % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.out) & 15) == 0);
    const long k0 = (long)kb * 32 + sb * 8;
    const long nv = a.in_f - k0;
    if (kb >= a.n_cb || nv <= 0) return;
#pragma unroll 1
    for (int p = 0; p < kDqRows / 8; p++) {
        const long n = r0 + p * 8 + (tid >> 5);
        if (n >= a.out_f) break;
        const long blk = n * a.n_cb + kb;
        uint32_t hi4, lo2, cfg, co;
        float lo_f, hi_f;
        if (LAYOUT == 0) {
            hi4 = *reinterpret_cast<const uint32_t*>(a.hi + blk * 16 + sb * 4);
            lo2 = *reinterpret_cast<const uint16_t*>(a.lo + blk * 8 + sb * 2);
            lo_f = h2f_bits(a.dmin[blk]);
            hi_f = h2f_bits(a.dmax[blk]);
            cfg = a.config[blk];
            co = a.coeff[blk];
        } else {
            T16Sub q = t16_read(a.levels, n, kb, sb, a.n_cb);
            hi4 = 0; lo2 = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {   // back to the file-format words so both layouts share one decode
                hi4 |= (q.lv[i] >> 2) << (4 * i);
                lo2 |= (q.lv[i] & 3) << ((i >> 2) * 8 + (3 - (i & 3)) * 2);
            }
            lo_f = h2f_bits((uint16_t)q.dmin);
            hi_f = h2f_bits((uint16_t)q.dmax);
            cfg = q.cfg;
            co = q.coeff;
        }
        RangeD64 r = range_d64(lo_f, hi_f, (cfg >> (sb * 2)) & 3);
        double p0 = 0.0, p1 = 0.0;
        if (a.use_pca) {   // signed nibble c: (c ^ 8) - 8
            p0 = __dmul_rn(__dsub_rn(u2d((co & 0xF) ^ 8u), 8.0), S[kl][0]);
            p1 = __dmul_rn(__dsub_rn(u2d(((co >> 4) & 0xF) ^ 8u), 8.0), S[kl][1]);
        }
        __align__(16) __half v[8];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            float f[2];
#pragma unroll
            for (int j = 0; j < 2; j++) {
                double w = __fma_rn(r.step, u2d((uint32_t)level_of(hi4, lo2, i + j)), r.rlo);
                if (a.use_pca) {
                    w = __fma_rn(p0, B[kl * 84 + sb * 9 + i + j], w);
                    w = __fma_rn(p1, B[kl * 84 + 36 + sb * 9 + i + j], w);
                }
                f[j] = __double2float_rn(w);
            }
            *reinterpret_cast<__half2*>(&v[i]) = __floats2half2_rn(f[0], f[1]);
        }
        store8(a.out + n * a.in_f + k0, v, (int)(nv > 8 ? 8 : nv), vec_ok);
    }
}

// ------------------------------------------------------------------ embedding (float32)
// grid (T, ceil(n_cb/64)), block 256: thread = (kb_local = tid>>2, sb = tid&3).  In the
// T16 blob the consecutive kb of one row are 480 bytes apart (same tile), so a block's
// reads stay within one 30 KB span per 64 kb.
__global__ void __launch_bounds__(256)
embed_d32_kernel(const int64_t* __restrict__ ids, const uint8_t* __restrict__ blob,
                 const float* __restrict__ bases, const float* __restrict__ scales,
                 __half* __restrict__ out, int K, int N, int n_cb) {
    long t = blockIdx.x;
    int kb = blockIdx.y * 64 + (threadIdx.x >> 2);
    int sb = threadIdx.x & 3;
    if (kb >= n_cb) return;
    long k0 = (long)kb * 32 + sb * 8;
    long nv = (long)K - k0;
    if (nv <= 0) return;
    bool vec_ok = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    __half* dst = out + t * (long)K + k0;
    __align__(16) __half v[8];
    long row = ids[t];
    if (row < 0 || row >= N) {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __float2half_rn(0.0f);
        store8(dst, v, (int)(nv > 8 ? 8 : nv), vec_ok);
        return;
    }
    T16Sub q = t16_read(blob, row, kb, sb, n_cb);
    float lo_f = h2f_bits((uint16_t)q.dmin), hi_f = h2f_bits((uint16_t)q.dmax);
    float rlo, step;
    range_d32(lo_f, hi_f, (q.cfg >> (sb * 2)) & 3, rlo, step);
    // ((float)c0 * scales) first, then one fused multiply-add per term, in the order
    // of the reference expression (ref cuda/sx8_embed_v44.cu:72-74).
    float p0 = __fmul_rn((float)s4(q.coeff & 0xF), scales[kb * 2]);
    float p1 = __fmul_rn((float)s4((q.coeff >> 4) & 0xF), scales[kb * 2 + 1]);
    const float4* b0 = reinterpret_cast<const float4*>(bases + kb * 64 + sb * 8);
    const float4* b1 = reinterpret_cast<const float4*>(bases + kb * 64 + 32 + sb * 8);
    float4 b0a = b0[0], b0b = b0[1], b1a = b1[0], b1b = b1[1];
    float bb0[8] = {b0a.x, b0a.y, b0a.z, b0a.w, b0b.x, b0b.y, b0b.z, b0b.w};
    float bb1[8] = {b1a.x, b1a.y, b1a.z, b1a.w, b1b.x, b1b.y, b1b.z, b1b.w};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float w = __fmaf_rn(step, (float)q.lv[i], rlo);
        w = __fmaf_rn(p0, bb0[i], w);
        w = __fmaf_rn(p1, bb1[i], w);
        v[i] = __float2half_rn(w);
    }
    store8(dst, v, (int)(nv > 8 ? 8 : nv), vec_ok);
}

// ------------------------------------------------------------------ quantizer search
// ref scripts/quantize_qwen35_4b_sx8_v43_gpu.py:22-47, torch eager float32 semantics:
// IEEE division of tensor by tensor, separately rounded multiply and add, round-half-even,
// strict '<' with the lowest strategy winning ties.  Two operations of that function give
// different bits on torch's CUDA and CPU back ends, and the reference runs on CUDA (ref :9):
//   (hi - lo) / 63     CUDA: multiplied by float(1/63) (a tensor divided by a host scalar is
//                      turned into a multiplication by the reciprocal); CPU: IEEE division
//   mean over 8        CUDA: butterfly sum ((e0+e4)+(e2+e6)) + ((e1+e5)+(e3+e7)), times 1/8;
//                      CPU: left-to-right sum, divided by 8
// Both orders were fixed by comparing against torch on a B200 (8M rows, 0 differences) and
// against torch CPU.  CUDA_ARITH selects the first set (SX8_ARITH_TORCH_CUDA).
template <bool F16IN, bool CUDA_ARITH>
__global__ void __launch_bounds__(256)
quantize_kernel(const void* __restrict__ w_, long out_f, long in_f, long ldw, int n_cb,
                __half* __restrict__ dmin_o, __half* __restrict__ dmax_o,
                uint8_t* __restrict__ config_o, uint8_t* __restrict__ hi_o,
                uint8_t* __restrict__ lo_o, uint8_t* __restrict__ lv_o) {
    long gid = (long)blockIdx.x * 256 + threadIdx.x;
    long blk = gid >> 2;
    int sb = (int)(gid & 3);
    long n_blk = out_f * n_cb;
    bool valid = blk < n_blk;
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = 0.0f;
    if (valid) {
        long n = blk / n_cb;
        long k0 = (blk - n * n_cb) * 32 + sb * 8;
        long nv = in_f - k0;
        if (F16IN) {
            const __half* src = reinterpret_cast<const __half*>(w_) + n * ldw + k0;
            if (nv >= 8 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
                uint4 raw = *reinterpret_cast<const uint4*>(src);
                const __half* hh = reinterpret_cast<const __half*>(&raw);
#pragma unroll
                for (int i = 0; i < 8; i++) x[i] = __half2float(hh[i]);
            } else {
                for (int i = 0; i < 8; i++)
                    if (i < nv) x[i] = __half2float(src[i]);
            }
        } else {
            const float* src = reinterpret_cast<const float*>(w_) + n * ldw + k0;
            if (nv >= 8 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
                float4 a = reinterpret_cast<const float4*>(src)[0];
                float4 b = reinterpret_cast<const float4*>(src)[1];
                x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
                x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
            } else {
                for (int i = 0; i < 8; i++)
                    if (i < nv) x[i] = src[i];
            }
        }
    }
    float mn = x[0], mx = x[0];
#pragma unroll
    for (int i = 1; i < 8; i++) {
        mn = fminf(mn, x[i]);
        mx = fmaxf(mx, x[i]);
    }
    mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
    mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, 2));
    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));

    float d = fmaxf(__fsub_rn(mx, mn), 1e-10f);
    float q = __fmul_rn(d, 0.25f);          // d / 4 exactly
    float best = __int_as_float(0x7F800000);
    int best_r = 0;
    float best_pa = 0.f, best_pb = 0.f;     // the winner's levels, four per float: c0 + 64 c1 + 4096 c2 + 262144 c3
#pragma unroll
    for (int r = 0; r < 4; r++) {
        float lo = (r == 2) ? __fsub_rn(mx, q) : ((r == 3) ? __fadd_rn(mn, q) : mn);
        float hi = (r == 1) ? __fadd_rn(mn, q) : ((r == 3) ? __fsub_rn(mx, q) : mx);
        const float kInv63 = 1.0f / 63.0f;   // rounded to float32 once, as torch does on the host
        float step = CUDA_ARITH ? fmaxf(__fmul_rn(__fsub_rn(hi, lo), kInv63), 1e-10f)
                                : fmaxf(__fdiv_rn(__fsub_rn(hi, lo), 63.0f), 1e-10f);
        // round((x - lo) / step) with the IEEE quotient, eight times per range: the quotient is taken
        // as (x - lo) * (1 / step) -- within 1.5 * 2^-23 relative of the exact one, so for quotients
        // that matter (the result is clamped to 0..63) within 1.2e-5 absolute of the IEEE-rounded
        // one -- and rounded; only when it lies within 2e-5 of a rounding boundary k + 0.5 can the
        // two roundings differ, and then the IEEE division is done (about one weight in 10,000).
        const float rstep = __frcp_rn(step);
        float e2[8], c[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float a = __fsub_rn(x[i], lo);
            float ci = rintf(__fmul_rn(a, rstep));
            if (fabsf(__fsub_rn(__fmul_rn(a, rstep), ci)) > 0.49998f) ci = rintf(__fdiv_rn(a, step));
            ci = fminf(fmaxf(ci, 0.0f), 63.0f);
            c[i] = ci;
            float rec = __fadd_rn(lo, __fmul_rn(step, ci));
            float e = __fsub_rn(x[i], rec);
            e2[i] = __fmul_rn(e, e);
        }
        float mse;
        if (CUDA_ARITH) {
            float a = __fadd_rn(__fadd_rn(e2[0], e2[4]), __fadd_rn(e2[2], e2[6]));
            float b = __fadd_rn(__fadd_rn(e2[1], e2[5]), __fadd_rn(e2[3], e2[7]));
            mse = __fmul_rn(__fadd_rn(a, b), 0.125f);
        } else {
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) sum = __fadd_rn(sum, e2[i]);
            mse = __fmul_rn(sum, 0.125f);   // sum / 8 exactly
        }
        if (mse < best) {
            best = mse;
            best_r = r;
            // integers below 2^24: exact in float32
            best_pa = fmaf(c[3], 262144.0f, fmaf(c[2], 4096.0f, fmaf(c[1], 64.0f, c[0])));
            best_pb = fmaf(c[7], 262144.0f, fmaf(c[6], 4096.0f, fmaf(c[5], 64.0f, c[4])));
        }
    }
    // the winner's levels -> the file's bit layout (ref quantize...py:148-167): levels_hi nibble i of
    // the 32-bit word, levels_lo pair i at bit (i >> 2) * 8 + (3 - (i & 3)) * 2 of the 16-bit word
    uint32_t best_hi = 0, best_lo = 0;
    {
        const uint32_t pa = (uint32_t)best_pa, pb = (uint32_t)best_pb;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t ci = ((i < 4 ? pa : pb) >> (6 * (i & 3))) & 63u;
            best_hi |= (ci >> 2) << (4 * i);
            best_lo |= (ci & 3u) << ((i >> 2) * 8 + (3 - (i & 3)) * 2);
        }
    }
    uint32_t cfg = (uint32_t)best_r << (2 * sb);
    cfg |= __shfl_xor_sync(0xFFFFFFFFu, cfg, 1);
    cfg |= __shfl_xor_sync(0xFFFFFFFFu, cfg, 2);
    if (!valid) return;
    *reinterpret_cast<uint32_t*>(hi_o + blk * 16 + sb * 4) = best_hi;
    *reinterpret_cast<uint16_t*>(lo_o + blk * 8 + sb * 2) = (uint16_t)best_lo;
    if (lv_o) {
        uint32_t a = 0, b = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            a |= (uint32_t)level_of(best_hi, best_lo, i) << (8 * i);
            b |= (uint32_t)level_of(best_hi, best_lo, i + 4) << (8 * i);
        }
        *reinterpret_cast<uint2*>(lv_o + blk * 32 + sb * 8) = make_uint2(a, b);
    }
    if (sb == 0) {
        dmin_o[blk] = __float2half_rn(mn);
        dmax_o[blk] = __float2half_rn(mx);
        config_o[blk] = (uint8_t)cfg;
    }
}

// ------------------------------------------------------------------ quantizer PCA stage
// ref scripts/quantize_qwen35_4b_sx8_v43_gpu.py:75-142 (pca_correct_gpu): per block column kb
// the residual E = w - (lo_sb + st_sb * level) of every row is formed, its top two right
// singular vectors become the two bases of that column, the residual's coordinates on them the
// per-block coefficients, their median magnitude / 3 the two scales.  The reference materialises
// E (4 bytes per weight) and hands it to a batched SVD.  Here E never reaches HBM: the kernels
// below recompute it from the weights and the packed planes wherever it is needed (34 bytes read
// per block for f16 weights), the 32x32 Gram matrix E^T E per column is accumulated in registers,
// and only the n_cb small symmetric eigenproblems are left to a library.
//
// One thread owns one 8-weight sub-block, as in the search kernel.  The residual uses the
// reference's encode-side endpoints (ref :84-87): Q = d / 4, lo in {dmin, dmin, dmax - Q,
// dmin + Q}, step in {d, Q, Q, max(d - 2 Q, 1e-10)} / 63, all float32 from the f16 endpoints.
template <bool F16IN>
__device__ __forceinline__ void pca_residual8(const void* __restrict__ w_, long n, int kb, int sb, long in_f, long ldw,
                                              int n_cb, const uint16_t* __restrict__ dmin, const uint16_t* __restrict__ dmax,
                                              const uint8_t* __restrict__ config, const uint8_t* __restrict__ hi,
                                              const uint8_t* __restrict__ lo, float (&e)[8]) {
    const long blk = n * n_cb + kb;
    const long k0 = (long)kb * 32 + sb * 8;
    const long nv = in_f - k0;
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = 0.0f;
    if (F16IN) {
        const __half* src = reinterpret_cast<const __half*>(w_) + n * ldw + k0;
        if (nv >= 8 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
            uint4 raw = __ldg(reinterpret_cast<const uint4*>(src));
            const __half* hh = reinterpret_cast<const __half*>(&raw);
#pragma unroll
            for (int i = 0; i < 8; i++) x[i] = __half2float(hh[i]);
        } else {
            for (int i = 0; i < 8; i++)
                if (i < nv) x[i] = __half2float(src[i]);
        }
    } else {
        const float* src = reinterpret_cast<const float*>(w_) + n * ldw + k0;
        if (nv >= 8 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
            float4 a = __ldg(reinterpret_cast<const float4*>(src));
            float4 b = __ldg(reinterpret_cast<const float4*>(src) + 1);
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
            x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        } else {
            for (int i = 0; i < 8; i++)
                if (i < nv) x[i] = src[i];
        }
    }
    const float mn = h2f_bits(dmin[blk]), mx = h2f_bits(dmax[blk]);
    const int s = (config[blk] >> (sb * 2)) & 3;
    const uint32_t hi4 = *reinterpret_cast<const uint32_t*>(hi + blk * 16 + sb * 4);
    const uint32_t lo2 = *reinterpret_cast<const uint16_t*>(lo + blk * 8 + sb * 2);
    const float kInv63 = 1.0f / 63.0f;
    const float d = fmaxf(__fsub_rn(mx, mn), 1e-10f);
    const float q = __fmul_rn(d, 0.25f);
    const float rlo = (s == 2) ? __fsub_rn(mx, q) : ((s == 3) ? __fadd_rn(mn, q) : mn);
    const float span = (s == 0) ? d : ((s == 3) ? fmaxf(__fsub_rn(d, __fmul_rn(2.0f, q)), 1e-10f) : q);
    const float step = __fmul_rn(span, kInv63);
#pragma unroll
    for (int i = 0; i < 8; i++)
        e[i] = __fsub_rn(x[i], __fadd_rn(rlo, __fmul_rn(step, (float)level_of(hi4, lo2, i))));
}

struct PcaArgs {
    const void* w;
    long out_f, in_f, ldw;
    int n_cb;
    const uint16_t *dmin, *dmax;
    const uint8_t *config, *hi, *lo;
};

constexpr int kPcaKb = 4;        // block columns per CTA: 64 bytes of levels_hi and 256 of f16 weights per row
constexpr int kPcaRows = 64;     // rows staged in shared memory between two accumulation phases
constexpr int kPcaLd = 36;       // floats per staged row: 32 + 4, keeps every 4-float group 16-byte aligned

// Partial Gram matrices.  grid (ceil(n_cb / 4), chunks), block 256.  Each CTA walks its chunk
// of rows 64 at a time: the 256 threads form the residuals of 16 rows x 4 block columns x 4
// sub-blocks per pass into shared memory, then every thread adds the 64 staged rows into its
// 4 x 4 patch of one column's 32 x 32 matrix (two 16-byte shared loads per 16 multiply-adds).
// Output: part[chunk][kb][32][32]; a second kernel adds the chunks in order, so the result does
// not depend on scheduling.
template <bool F16IN>
__global__ void __launch_bounds__(256) pca_gram_kernel(PcaArgs a, long rows_per_cta, float* __restrict__ part) {
    __shared__ __align__(16) float E[kPcaKb][kPcaRows][kPcaLd];
    const int tid = threadIdx.x;
    const int kb0 = blockIdx.x * kPcaKb;
    const long r_begin = (long)blockIdx.y * rows_per_cta;
    const long r_end = (r_begin + rows_per_cta < a.out_f) ? r_begin + rows_per_cta : a.out_f;
    // loader role: (row_l, kb_l, sb) with sb fastest, so a row's 4 columns are one contiguous run
    const int l_sb = tid & 3, l_kb = (tid >> 2) & 3, l_row = tid >> 4;
    // accumulator role: column c_kb, patch rows i0..i0+3, patch columns j0..j0+3
    const int c_kb = tid >> 6, i0 = ((tid & 63) >> 3) * 4, j0 = (tid & 7) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    for (long r0 = r_begin; r0 < r_end; r0 += kPcaRows) {
#pragma unroll
        for (int p = 0; p < kPcaRows / 16; p++) {
            const int rl = p * 16 + l_row;
            const long n = r0 + rl;
            const int kb = kb0 + l_kb;
            float e[8];
#pragma unroll
            for (int i = 0; i < 8; i++) e[i] = 0.0f;
            if (n < r_end && kb < a.n_cb)
                pca_residual8<F16IN>(a.w, n, kb, l_sb, a.in_f, a.ldw, a.n_cb, a.dmin, a.dmax, a.config, a.hi, a.lo, e);
            float4* dst = reinterpret_cast<float4*>(&E[l_kb][rl][l_sb * 8]);
            dst[0] = make_float4(e[0], e[1], e[2], e[3]);
            dst[1] = make_float4(e[4], e[5], e[6], e[7]);
        }
        __syncthreads();
#pragma unroll 8
        for (int r = 0; r < kPcaRows; r++) {
            const float4 u = *reinterpret_cast<const float4*>(&E[c_kb][r][i0]);
            const float4 v = *reinterpret_cast<const float4*>(&E[c_kb][r][j0]);
            const float uu[4] = {u.x, u.y, u.z, u.w}, vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(uu[i], vv[j], acc[i][j]);
        }
        __syncthreads();
    }
    const int kb = kb0 + c_kb;
    if (kb < a.n_cb) {
        float* dst = part + ((long)blockIdx.y * a.n_cb + kb) * 1024;
#pragma unroll
        for (int i = 0; i < 4; i++)
            *reinterpret_cast<float4*>(dst + (i0 + i) * 32 + j0) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    }
}

// gram[kb][i][j] = sum over chunks, in chunk order (float64 accumulation, stored as float64 for
// the eigen-solver).
__global__ void __launch_bounds__(256) pca_gram_reduce_kernel(const float* __restrict__ part, int chunks, long n_elem,
                                                              double* __restrict__ gram) {
    long i = (long)blockIdx.x * 256 + threadIdx.x;
    if (i >= n_elem) return;
    double s = 0.0;
    for (int c = 0; c < chunks; c++) s += (double)part[(long)c * n_elem + i];
    gram[i] = s;
}

// Coordinates of every block's residual on the two bases of its column:
// coef[kb][j][n] = sum_t E[n][kb][t] * bases[kb][j][t].  Same tiling as the Gram kernel (grid
// (ceil(n_cb / 4), ceil(out_f / 64)), block 256); the four sub-block partial sums meet through
// two shuffles, and the results of a tile leave through shared memory so that each (kb, j) run
// of 64 rows is one contiguous 256-byte store.
template <bool F16IN>
__global__ void __launch_bounds__(256) pca_project_kernel(PcaArgs a, const float* __restrict__ bases, float* __restrict__ coef) {
    __shared__ float B[kPcaKb][64];
    __shared__ float C[kPcaKb][2][kPcaRows];
    const int tid = threadIdx.x;
    const int kb0 = blockIdx.x * kPcaKb;
    const long r0 = (long)blockIdx.y * kPcaRows;
    {
        const int kb = kb0 + (tid >> 6);
        B[tid >> 6][tid & 63] = (kb < a.n_cb) ? bases[(long)kb * 64 + (tid & 63)] : 0.0f;
    }
    __syncthreads();
    const int l_sb = tid & 3, l_kb = (tid >> 2) & 3, l_row = tid >> 4;
#pragma unroll
    for (int p = 0; p < kPcaRows / 16; p++) {
        const int rl = p * 16 + l_row;
        const long n = r0 + rl;
        const int kb = kb0 + l_kb;
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; i++) e[i] = 0.0f;
        if (n < a.out_f && kb < a.n_cb)
            pca_residual8<F16IN>(a.w, n, kb, l_sb, a.in_f, a.ldw, a.n_cb, a.dmin, a.dmax, a.config, a.hi, a.lo, e);
        float c0 = 0.0f, c1 = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            c0 = fmaf(e[i], B[l_kb][l_sb * 8 + i], c0);
            c1 = fmaf(e[i], B[l_kb][32 + l_sb * 8 + i], c1);
        }
        c0 += __shfl_xor_sync(0xFFFFFFFFu, c0, 1);
        c1 += __shfl_xor_sync(0xFFFFFFFFu, c1, 1);
        c0 += __shfl_xor_sync(0xFFFFFFFFu, c0, 2);
        c1 += __shfl_xor_sync(0xFFFFFFFFu, c1, 2);
        if (l_sb == 0) {
            C[l_kb][0][rl] = c0;
            C[l_kb][1][rl] = c1;
        }
    }
    __syncthreads();
    for (int o = tid; o < kPcaKb * 2 * kPcaRows; o += 256) {
        const int rl = o & (kPcaRows - 1), j = (o >> 6) & 1, kl = o >> 7;
        const int kb = kb0 + kl;
        const long n = r0 + rl;
        if (kb < a.n_cb && n < a.out_f) coef[((long)kb * 2 + j) * a.out_f + n] = C[kl][j][rl];
    }
}

// coeff byte of block (n, kb) = (round(c0 / s0) clamped to -8..7) & 15 | the same of c1 << 4
// (ref :131-139), written n-major.  32 x 32 tiles transposed through shared memory: reads run
// along n, writes along kb.
__global__ void __launch_bounds__(256) pca_pack_kernel(const float* __restrict__ coef, const float* __restrict__ scales,
                                                       long out_f, int n_cb, uint8_t* __restrict__ coeff) {
    __shared__ uint8_t T[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    const long n0 = (long)blockIdx.x * 32;
    const int kb0 = blockIdx.y * 32;
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const int kl = p * 8 + ty;
        const int kb = kb0 + kl;
        const long n = n0 + tx;
        uint8_t b = 0;
        if (kb < n_cb && n < out_f) {
            const float q0 = rintf(__fdiv_rn(coef[((long)kb * 2 + 0) * out_f + n], scales[kb * 2 + 0]));
            const float q1 = rintf(__fdiv_rn(coef[((long)kb * 2 + 1) * out_f + n], scales[kb * 2 + 1]));
            const int i0 = (int)fminf(fmaxf(q0, -8.0f), 7.0f), i1 = (int)fminf(fmaxf(q1, -8.0f), 7.0f);
            b = (uint8_t)((i0 & 15) | ((i1 & 15) << 4));
        }
        T[kl][tx] = b;
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const int nl = p * 8 + ty;
        const long n = n0 + nl;
        const int kb = kb0 + tx;
        if (kb < n_cb && n < out_f) coeff[n * n_cb + kb] = T[tx][nl];
    }
}

// Row chunks of the Gram kernel: enough CTAs to fill the machine a few times over, chunks a
// multiple of the staging depth.
static long pca_rows_per_cta(long out_f, int n_cb) {
    const long groups = (n_cb + kPcaKb - 1) / kPcaKb;
    long chunks = (148L * 8 + groups - 1) / groups;
    const long max_chunks = (out_f + kPcaRows - 1) / kPcaRows;
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks < 1) chunks = 1;
    long rows = (out_f + chunks - 1) / chunks;
    return (rows + kPcaRows - 1) / kPcaRows * kPcaRows;
}
static long pca_chunks(long out_f, int n_cb) {
    const long rows = pca_rows_per_cta(out_f, n_cb);
    return (out_f + rows - 1) / rows;
}

// ------------------------------------------------------------------ repack to v4.4
// ref scripts/prepare_v44.py:35-79.  One thread per destination block (kb, n), n
// fastest, so the kb-major writes are contiguous across the warp.
template <int HDR>
__global__ void __launch_bounds__(256)
repack_v44_kernel(const uint16_t* __restrict__ dmin, const uint16_t* __restrict__ dmax,
                  const uint8_t* __restrict__ config, const uint8_t* __restrict__ coeff,
                  const uint8_t* __restrict__ hi, const uint8_t* __restrict__ lo, long out_f,
                  int n_cb, uint8_t* __restrict__ hdr_o, uint8_t* __restrict__ lev_o) {
    long dst = (long)blockIdx.x * 256 + threadIdx.x;
    if (dst >= out_f * n_cb) return;
    long kb = dst / out_f, n = dst - kb * out_f;
    long src = n * n_cb + kb;
    uint4 h = *reinterpret_cast<const uint4*>(hi + src * 16);
    uint2 l = *reinterpret_cast<const uint2*>(lo + src * 8);
    uint2* lv = reinterpret_cast<uint2*>(lev_o + dst * 24);
    lv[0] = make_uint2(h.x, h.y);
    lv[1] = make_uint2(h.z, h.w);
    lv[2] = l;
    uint16_t cc = (uint16_t)(config[src] | (coeff[src] << 8));
    uint16_t* ho = reinterpret_cast<uint16_t*>(hdr_o + dst * HDR);
    ho[0] = dmin[src];
    ho[1] = dmax[src];
    ho[2] = cc;
    if (HDR == 8) ho[3] = 0;
}

// ------------------------------------------------------------------ repack to T16
// One thread per (tile, kb, lane): gathers the two sub-blocks it owns from the n-major
// file planes and writes its three level words; lanes t = 0,1,2 also write H0,H1,H2.
// Where the repack reads a block from: the container's separate planes, or interleaved
// 30-byte block_sx8 records {dmin f16, dmax f16, config, qh[16], ql[8], coeff} (the GGUF
// tensor data, ref scripts/convert_pkl_to_gguf_sx8.py:20-38).
struct PlaneSrc {
    const uint16_t *dmin, *dmax;
    const uint8_t *config, *coeff, *hi, *lo;
    __device__ __forceinline__ uint32_t hi4(long bid, int t) const { return *reinterpret_cast<const uint32_t*>(hi + bid * 16 + t * 4); }
    __device__ __forceinline__ uint32_t lo2(long bid, int t) const { return *reinterpret_cast<const uint16_t*>(lo + bid * 8 + t * 2); }
    __device__ __forceinline__ uint32_t ends(long bid) const { return (uint32_t)dmin[bid] | ((uint32_t)dmax[bid] << 16); }
    __device__ __forceinline__ uint32_t cc(long bid) const { return (uint32_t)config[bid] | ((uint32_t)coeff[bid] << 8); }
};
struct BlockSrc {
    const uint8_t* blk;   // records are 2-byte aligned (30 is even); qh/ql sit at odd offsets
    __device__ __forceinline__ uint32_t hi4(long bid, int t) const {
        const uint8_t* q = blk + bid * SX8_BLOCK_BYTES + 5 + t * 4;
        return (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) | ((uint32_t)q[3] << 24);
    }
    __device__ __forceinline__ uint32_t lo2(long bid, int t) const {
        const uint8_t* q = blk + bid * SX8_BLOCK_BYTES + 21 + t * 2;
        return (uint32_t)q[0] | ((uint32_t)q[1] << 8);
    }
    __device__ __forceinline__ uint32_t ends(long bid) const {
        const uint16_t* h = reinterpret_cast<const uint16_t*>(blk + bid * SX8_BLOCK_BYTES);
        return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
    }
    __device__ __forceinline__ uint32_t cc(long bid) const {
        const uint8_t* q = blk + bid * SX8_BLOCK_BYTES;
        return (uint32_t)q[4] | ((uint32_t)q[29] << 8);
    }
};

template <class SRC>
__global__ void __launch_bounds__(256)
repack_t16_kernel(SRC src, long N, int n_cb, uint8_t* __restrict__ blob) {
    long gid = (long)blockIdx.x * 256 + threadIdx.x;
    long n_units = t16_tiles(N) * n_cb;
    long unit = gid >> 5;
    if (unit >= n_units) return;
    int L = (int)(gid & 31), g = L >> 2, t = L & 3;
    long T = unit / n_cb, kb = unit - T * n_cb;
    long colA = T * 16 + g, colB = colA + 8;
    uint32_t a[8], b[8];
    uint32_t hA = 0, hB = 0, ccA = 0, ccB = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) { a[i] = 0; b[i] = 0; }
    if (colA < N) {
        long bid = colA * n_cb + kb;
        uint32_t hi4 = src.hi4(bid, t), lo2 = src.lo2(bid, t);
#pragma unroll
        for (int i = 0; i < 8; i++) a[i] = (uint32_t)level_of(hi4, lo2, i);
        hA = src.ends(bid);
        ccA = src.cc(bid);
    }
    if (colB < N) {
        long bid = colB * n_cb + kb;
        uint32_t hi4 = src.hi4(bid, t), lo2 = src.lo2(bid, t);
#pragma unroll
        for (int i = 0; i < 8; i++) b[i] = (uint32_t)level_of(hi4, lo2, i);
        hB = src.ends(bid);
        ccB = src.cc(bid);
    }
    const int ord[4] = {0, 2, 1, 3};
    uint32_t W0 = 0, W1 = 0, W2 = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t e = b[4 + ord[j]];
        W0 |= ((a[ord[j]] << 2) | (e & 3)) << (8 * j);
        W1 |= ((a[4 + ord[j]] << 2) | ((e >> 2) & 3)) << (8 * j);
        W2 |= ((b[ord[j]] << 2) | ((e >> 4) & 3)) << (8 * j);
    }
    uint32_t* u = reinterpret_cast<uint32_t*>(blob + unit * T16_UNIT);
    u[L] = W0;
    u[32 + L] = W1;
    u[64 + L] = W2;
    if (t == 0) u[96 + g] = hA;
    if (t == 1) u[104 + g] = hB;
    if (t == 2) {
        uint32_t cfA = ccA & 0xFF, coA = ccA >> 8, cfB = ccB & 0xFF, coB = ccB >> 8;
        u[112 + g] = (coA & 15) | ((coB & 15) << 4) | (cfA << 8) | ((coA >> 4) << 16) | ((coB >> 4) << 20) | (cfB << 24);
    }
}

// planes <-> interleaved 30-byte records, one thread per block (15 two-byte moves)
template <bool TO_BLOCKS>
__global__ void __launch_bounds__(256)
blocks_kernel(uint16_t* dmin, uint16_t* dmax, uint8_t* config, uint8_t* coeff, uint8_t* hi, uint8_t* lo, long n_blk,
              uint8_t* blk) {
    long bid = (long)blockIdx.x * 256 + threadIdx.x;
    if (bid >= n_blk) return;
    uint8_t* r = blk + bid * SX8_BLOCK_BYTES;
    uint16_t* r16 = reinterpret_cast<uint16_t*>(r);
    if (TO_BLOCKS) {
        uint8_t h[16], l[8];
        *reinterpret_cast<uint4*>(h) = *reinterpret_cast<const uint4*>(hi + bid * 16);
        *reinterpret_cast<uint2*>(l) = *reinterpret_cast<const uint2*>(lo + bid * 8);
        r16[0] = dmin[bid];
        r16[1] = dmax[bid];
        r16[2] = (uint16_t)config[bid] | ((uint16_t)h[0] << 8);
#pragma unroll
        for (int i = 0; i < 7; i++) r16[3 + i] = (uint16_t)h[2 * i + 1] | ((uint16_t)h[2 * i + 2] << 8);
        r16[10] = (uint16_t)h[15] | ((uint16_t)l[0] << 8);
#pragma unroll
        for (int i = 0; i < 3; i++) r16[11 + i] = (uint16_t)l[2 * i + 1] | ((uint16_t)l[2 * i + 2] << 8);
        r16[14] = (uint16_t)l[7] | ((uint16_t)coeff[bid] << 8);
    } else {
        uint16_t w[15];
#pragma unroll
        for (int i = 0; i < 15; i++) w[i] = r16[i];
        dmin[bid] = w[0];
        dmax[bid] = w[1];
        config[bid] = (uint8_t)w[2];
        uint8_t h[16], l[8];
        h[0] = (uint8_t)(w[2] >> 8);
#pragma unroll
        for (int i = 0; i < 7; i++) { h[2 * i + 1] = (uint8_t)w[3 + i]; h[2 * i + 2] = (uint8_t)(w[3 + i] >> 8); }
        h[15] = (uint8_t)w[10];
        l[0] = (uint8_t)(w[10] >> 8);
#pragma unroll
        for (int i = 0; i < 3; i++) { l[2 * i + 1] = (uint8_t)w[11 + i]; l[2 * i + 2] = (uint8_t)(w[11 + i] >> 8); }
        l[7] = (uint8_t)w[14];
        coeff[bid] = (uint8_t)(w[14] >> 8);
        *reinterpret_cast<uint4*>(hi + bid * 16) = *reinterpret_cast<const uint4*>(h);
        *reinterpret_cast<uint2*>(lo + bid * 8) = *reinterpret_cast<const uint2*>(l);
    }
}

}  // namespace sx8

// =================================================================== C ABI
using namespace sx8;

static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

extern "C" int sx8_dequant_planes(const void* dmin, const void* dmax, const uint8_t* config,
                                  const uint8_t* coeff, const uint8_t* hi, const uint8_t* lo,
                                  const float* bases, const float* scales, long out_f, long in_f,
                                  int n_cb, int use_pca, void* out, void* stream) {
    SX8_REQUIRE(dmin && dmax && config && coeff && hi && lo && out, "sx8_dequant_planes: null pointer");
    SX8_REQUIRE(!use_pca || (bases && scales), "sx8_dequant_planes: use_pca needs bases and scales");
    SX8_REQUIRE(out_f > 0 && in_f > 0 && n_cb == (in_f + 31) / 32,
                "sx8_dequant_planes: need out_f>0, in_f>0, n_cb == ceil(in_f/32) (got %ld, %ld, %d)", out_f, in_f, n_cb);
    SX8_REQUIRE(aligned(hi, 4) && aligned(lo, 2) && aligned(dmin, 2) && aligned(dmax, 2) && aligned(out, 2),
                "sx8_dequant_planes: misaligned plane pointer");
    DequantArgs a{(const uint16_t*)dmin, (const uint16_t*)dmax, config, coeff, hi, lo, nullptr, nullptr,
                  bases, scales, out_f, in_f, n_cb, 6, use_pca, (__half*)out};
    const long ctas = ((out_f + kDqRows - 1) / kDqRows) * ((n_cb + kDqKb - 1) / kDqKb);
    SX8_REQUIRE(ctas <= 0x7FFFFFFFL, "sx8_dequant_planes: tensor too large for one launch");
    dequant_d64_kernel<0><<<(unsigned)ctas, 256, 0, (cudaStream_t)stream>>>(a);
    SX8_LAUNCH_CHECK("dequant_d64_kernel<planes>");
    return SX8_OK;
}

extern "C" int sx8_dequant_t16(const void* wt16, const float* bases, const float* scales, long out_f,
                               long in_f, int n_cb, int use_pca, void* out, void* stream) {
    SX8_REQUIRE(wt16 && out, "sx8_dequant_t16: null pointer");
    SX8_REQUIRE(!use_pca || (bases && scales), "sx8_dequant_t16: use_pca needs bases and scales");
    SX8_REQUIRE(out_f > 0 && in_f > 0 && n_cb == (in_f + 31) / 32,
                "sx8_dequant_t16: need out_f>0, in_f>0, n_cb == ceil(in_f/32) (got %ld, %ld, %d)", out_f, in_f, n_cb);
    SX8_REQUIRE(aligned(wt16, 16) && aligned(out, 2), "sx8_dequant_t16: misaligned pointer");
    DequantArgs a{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, (const uint8_t*)wt16,
                  bases, scales, out_f, in_f, n_cb, 6, use_pca, (__half*)out};
    const long ctas = ((out_f + kDqRows - 1) / kDqRows) * ((n_cb + kDqKb - 1) / kDqKb);
    SX8_REQUIRE(ctas <= 0x7FFFFFFFL, "sx8_dequant_t16: tensor too large for one launch");
    dequant_d64_kernel<1><<<(unsigned)ctas, 256, 0, (cudaStream_t)stream>>>(a);
    SX8_LAUNCH_CHECK("dequant_d64_kernel<t16>");
    return SX8_OK;
}

extern "C" int sx8_embed(const int64_t* ids, long T, const void* wt16, const float* bases,
                         const float* scales, int K, int N, int n_cb, void* out, void* stream) {
    if (T == 0) return SX8_OK;
    SX8_REQUIRE(ids && wt16 && bases && scales && out, "sx8_embed: null pointer");
    SX8_REQUIRE(T > 0 && T <= 0x7FFFFFFF, "sx8_embed: T out of range (%ld)", T);
    SX8_REQUIRE(K > 0 && N > 0 && n_cb == (K + 31) / 32, "sx8_embed: need K>0, N>0, n_cb == ceil(K/32) (got %d, %d, %d)", K, N, n_cb);
    SX8_REQUIRE(aligned(wt16, 16) && aligned(bases, 16) && aligned(out, 2) && aligned(ids, 8),
                "sx8_embed: misaligned pointer");
    dim3 grid((unsigned)T, (unsigned)((n_cb + 63) / 64));
    embed_d32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(ids, (const uint8_t*)wt16, bases, scales, (__half*)out, K, N, n_cb);
    SX8_LAUNCH_CHECK("embed_d32_kernel");
    return SX8_OK;
}

extern "C" size_t sx8_t16_bytes(long N, int n_cb) { return (N > 0 && n_cb > 0) ? t16_bytes(N, n_cb) : 0; }

extern "C" int sx8_repack_t16(const void* dmin, const void* dmax, const uint8_t* config,
                              const uint8_t* coeff, const uint8_t* hi, const uint8_t* lo, long out_f,
                              int n_cb, void* wt16_out, void* stream) {
    SX8_REQUIRE(dmin && dmax && config && coeff && hi && lo && wt16_out, "sx8_repack_t16: null pointer");
    SX8_REQUIRE(out_f > 0 && n_cb > 0, "sx8_repack_t16: need out_f>0, n_cb>0");
    SX8_REQUIRE(aligned(hi, 4) && aligned(lo, 2) && aligned(dmin, 2) && aligned(dmax, 2) && aligned(wt16_out, 16),
                "sx8_repack_t16: misaligned pointer");
    long threads = t16_tiles(out_f) * n_cb * 32;
    SX8_REQUIRE((threads + 255) / 256 <= 0x7FFFFFFFL, "sx8_repack_t16: tensor too large for one launch");
    PlaneSrc src{(const uint16_t*)dmin, (const uint16_t*)dmax, config, coeff, hi, lo};
    repack_t16_kernel<PlaneSrc><<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        src, out_f, n_cb, (uint8_t*)wt16_out);
    SX8_LAUNCH_CHECK("repack_t16_kernel");
    return SX8_OK;
}

extern "C" int sx8_repack_t16_blocks(const void* blocks, long out_f, int n_cb, void* wt16_out, void* stream) {
    SX8_REQUIRE(blocks && wt16_out, "sx8_repack_t16_blocks: null pointer");
    SX8_REQUIRE(out_f > 0 && n_cb > 0, "sx8_repack_t16_blocks: need out_f>0, n_cb>0");
    SX8_REQUIRE(aligned(blocks, 2) && aligned(wt16_out, 16), "sx8_repack_t16_blocks: misaligned pointer");
    long threads = t16_tiles(out_f) * n_cb * 32;
    SX8_REQUIRE((threads + 255) / 256 <= 0x7FFFFFFFL, "sx8_repack_t16_blocks: tensor too large for one launch");
    BlockSrc src{(const uint8_t*)blocks};
    repack_t16_kernel<BlockSrc><<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        src, out_f, n_cb, (uint8_t*)wt16_out);
    SX8_LAUNCH_CHECK("repack_t16_kernel<blocks>");
    return SX8_OK;
}

extern "C" int sx8_blocks_from_planes(const void* dmin, const void* dmax, const uint8_t* config, const uint8_t* coeff,
                                      const uint8_t* hi, const uint8_t* lo, long n_blk, void* blocks_out,
                                      void* stream) {
    SX8_REQUIRE(dmin && dmax && config && coeff && hi && lo && blocks_out, "sx8_blocks_from_planes: null pointer");
    SX8_REQUIRE(n_blk > 0 && (n_blk + 255) / 256 <= 0x7FFFFFFFL, "sx8_blocks_from_planes: bad block count %ld", n_blk);
    SX8_REQUIRE(aligned(dmin, 2) && aligned(dmax, 2) && aligned(hi, 16) && aligned(lo, 8) && aligned(blocks_out, 2),
                "sx8_blocks_from_planes: misaligned pointer");
    blocks_kernel<true><<<(unsigned)((n_blk + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (uint16_t*)dmin, (uint16_t*)dmax, (uint8_t*)config, (uint8_t*)coeff, (uint8_t*)hi, (uint8_t*)lo, n_blk,
        (uint8_t*)blocks_out);
    SX8_LAUNCH_CHECK("blocks_kernel<to>");
    return SX8_OK;
}

extern "C" int sx8_planes_from_blocks(const void* blocks, long n_blk, void* dmin, void* dmax, uint8_t* config,
                                      uint8_t* coeff, uint8_t* hi, uint8_t* lo, void* stream) {
    SX8_REQUIRE(dmin && dmax && config && coeff && hi && lo && blocks, "sx8_planes_from_blocks: null pointer");
    SX8_REQUIRE(n_blk > 0 && (n_blk + 255) / 256 <= 0x7FFFFFFFL, "sx8_planes_from_blocks: bad block count %ld", n_blk);
    SX8_REQUIRE(aligned(dmin, 2) && aligned(dmax, 2) && aligned(hi, 16) && aligned(lo, 8) && aligned(blocks, 2),
                "sx8_planes_from_blocks: misaligned pointer");
    blocks_kernel<false><<<(unsigned)((n_blk + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (uint16_t*)dmin, (uint16_t*)dmax, config, coeff, hi, lo, n_blk, (uint8_t*)blocks);
    SX8_LAUNCH_CHECK("blocks_kernel<from>");
    return SX8_OK;
}

extern "C" int sx8_quantize_blocks(const void* w, int w_is_f16, long out_f, long in_f, long ldw,
                                   void* dmin, void* dmax, uint8_t* config, uint8_t* hi, uint8_t* lo,
                                   uint8_t* levels_u8, int arith, void* stream) {
    SX8_REQUIRE(w && dmin && dmax && config && hi && lo, "sx8_quantize_blocks: null pointer");
    SX8_REQUIRE(arith == SX8_ARITH_TORCH_CUDA || arith == SX8_ARITH_TORCH_CPU,
                "sx8_quantize_blocks: arith must be SX8_ARITH_TORCH_CUDA (0) or SX8_ARITH_TORCH_CPU (1), got %d", arith);
    SX8_REQUIRE(out_f > 0 && in_f > 0 && ldw >= in_f, "sx8_quantize_blocks: need out_f>0, in_f>0, ldw>=in_f (got %ld, %ld, %ld)", out_f, in_f, ldw);
    SX8_REQUIRE(aligned(w, w_is_f16 ? 2 : 4) && aligned(hi, 4) && aligned(lo, 2) && aligned(dmin, 2) && aligned(dmax, 2) &&
                    (!levels_u8 || aligned(levels_u8, 8)),
                "sx8_quantize_blocks: misaligned pointer");
    int n_cb = (int)((in_f + 31) / 32);
    long threads = out_f * n_cb * 4;
    SX8_REQUIRE((threads + 255) / 256 <= 0x7FFFFFFFL, "sx8_quantize_blocks: tensor too large for one launch");
    unsigned grid = (unsigned)((threads + 255) / 256);
#define SX8_QLAUNCH(F16, CU) quantize_kernel<F16, CU><<<grid, 256, 0, (cudaStream_t)stream>>>( \
        w, out_f, in_f, ldw, n_cb, (__half*)dmin, (__half*)dmax, config, hi, lo, levels_u8)
    const bool cu = arith == SX8_ARITH_TORCH_CUDA;
    if (w_is_f16) { if (cu) SX8_QLAUNCH(true, true); else SX8_QLAUNCH(true, false); }
    else          { if (cu) SX8_QLAUNCH(false, true); else SX8_QLAUNCH(false, false); }
#undef SX8_QLAUNCH
    SX8_LAUNCH_CHECK("quantize_kernel");
    return SX8_OK;
}

static bool pca_args(PcaArgs& a, const char* who, const void* w, int w_is_f16, long out_f, long in_f, long ldw,
                     const void* dmin, const void* dmax, const uint8_t* config, const uint8_t* hi, const uint8_t* lo) {
    if (!(w && dmin && dmax && config && hi && lo)) { set_error("%s: null pointer", who); return false; }
    if (!(out_f > 0 && in_f > 0 && ldw >= in_f)) { set_error("%s: need out_f>0, in_f>0, ldw>=in_f (got %ld, %ld, %ld)", who, out_f, in_f, ldw); return false; }
    if (!(aligned(w, w_is_f16 ? 2 : 4) && aligned(hi, 4) && aligned(lo, 2) && aligned(dmin, 2) && aligned(dmax, 2))) {
        set_error("%s: misaligned pointer", who);
        return false;
    }
    a.w = w; a.out_f = out_f; a.in_f = in_f; a.ldw = ldw;
    a.n_cb = (int)((in_f + 31) / 32);
    a.dmin = (const uint16_t*)dmin; a.dmax = (const uint16_t*)dmax;
    a.config = config; a.hi = hi; a.lo = lo;
    return true;
}

extern "C" size_t sx8_pca_gram_scratch_bytes(long out_f, long in_f) {
    if (out_f <= 0 || in_f <= 0) return 0;
    const int n_cb = (int)((in_f + 31) / 32);
    return (size_t)pca_chunks(out_f, n_cb) * n_cb * 1024 * sizeof(float);
}

extern "C" int sx8_pca_gram(const void* w, int w_is_f16, long out_f, long in_f, long ldw, const void* dmin,
                            const void* dmax, const uint8_t* config, const uint8_t* hi, const uint8_t* lo,
                            double* gram, void* scratch, size_t scratch_bytes, void* stream) {
    PcaArgs a;
    if (!pca_args(a, "sx8_pca_gram", w, w_is_f16, out_f, in_f, ldw, dmin, dmax, config, hi, lo)) return SX8_E_INVALID;
    SX8_REQUIRE(gram && scratch && aligned(gram, 8) && aligned(scratch, 16), "sx8_pca_gram: gram / scratch null or misaligned");
    SX8_REQUIRE(scratch_bytes >= sx8_pca_gram_scratch_bytes(out_f, in_f), "sx8_pca_gram: scratch has %zu bytes, need %zu",
                scratch_bytes, sx8_pca_gram_scratch_bytes(out_f, in_f));
    const long rows = pca_rows_per_cta(out_f, a.n_cb), chunks = pca_chunks(out_f, a.n_cb);
    SX8_REQUIRE(chunks <= 65535, "sx8_pca_gram: tensor too large for one launch");
    dim3 grid((unsigned)((a.n_cb + kPcaKb - 1) / kPcaKb), (unsigned)chunks);
    if (w_is_f16) pca_gram_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(a, rows, (float*)scratch);
    else          pca_gram_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(a, rows, (float*)scratch);
    SX8_LAUNCH_CHECK("pca_gram_kernel");
    const long n_elem = (long)a.n_cb * 1024;
    pca_gram_reduce_kernel<<<(unsigned)((n_elem + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float*)scratch, (int)chunks, n_elem, gram);
    SX8_LAUNCH_CHECK("pca_gram_reduce_kernel");
    return SX8_OK;
}

extern "C" int sx8_pca_project(const void* w, int w_is_f16, long out_f, long in_f, long ldw, const void* dmin,
                               const void* dmax, const uint8_t* config, const uint8_t* hi, const uint8_t* lo,
                               const float* bases, float* coef, void* stream) {
    PcaArgs a;
    if (!pca_args(a, "sx8_pca_project", w, w_is_f16, out_f, in_f, ldw, dmin, dmax, config, hi, lo)) return SX8_E_INVALID;
    SX8_REQUIRE(bases && coef && aligned(bases, 4) && aligned(coef, 4), "sx8_pca_project: bases / coef null or misaligned");
    const long tiles = (out_f + kPcaRows - 1) / kPcaRows;
    SX8_REQUIRE(tiles <= 65535, "sx8_pca_project: more than 65535 x 64 rows; split the tensor by rows");
    dim3 grid((unsigned)((a.n_cb + kPcaKb - 1) / kPcaKb), (unsigned)tiles);
    if (w_is_f16) pca_project_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(a, bases, coef);
    else          pca_project_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(a, bases, coef);
    SX8_LAUNCH_CHECK("pca_project_kernel");
    return SX8_OK;
}

extern "C" int sx8_pca_pack(const float* coef, const float* scales, long out_f, int n_cb, uint8_t* coeff, void* stream) {
    SX8_REQUIRE(coef && scales && coeff, "sx8_pca_pack: null pointer");
    SX8_REQUIRE(out_f > 0 && n_cb > 0, "sx8_pca_pack: need out_f>0, n_cb>0 (got %ld, %d)", out_f, n_cb);
    const long tn = (out_f + 31) / 32, tk = (n_cb + 31) / 32;
    SX8_REQUIRE(tn <= 0x7FFFFFFFL && tk <= 65535, "sx8_pca_pack: tensor too large for one launch");
    pca_pack_kernel<<<dim3((unsigned)tn, (unsigned)tk), 256, 0, (cudaStream_t)stream>>>(coef, scales, out_f, n_cb, coeff);
    SX8_LAUNCH_CHECK("pca_pack_kernel");
    return SX8_OK;
}

extern "C" int sx8_repack_v44(const void* dmin, const void* dmax, const uint8_t* config,
                              const uint8_t* coeff, const uint8_t* hi, const uint8_t* lo, long out_f,
                              int n_cb, int hdr_bytes, void* hdr_out, void* levels_out, void* stream) {
    SX8_REQUIRE(dmin && dmax && config && coeff && hi && lo && hdr_out && levels_out, "sx8_repack_v44: null pointer");
    SX8_REQUIRE(hdr_bytes == 6 || hdr_bytes == 8, "sx8_repack_v44: hdr_bytes must be 6 or 8 (got %d)", hdr_bytes);
    SX8_REQUIRE(out_f > 0 && n_cb > 0, "sx8_repack_v44: need out_f>0, n_cb>0");
    SX8_REQUIRE(aligned(hi, 16) && aligned(lo, 8) && aligned(dmin, 2) && aligned(dmax, 2) && aligned(hdr_out, 2) && aligned(levels_out, 8),
                "sx8_repack_v44: misaligned pointer");
    long n_blk = out_f * n_cb;
    unsigned grid = (unsigned)((n_blk + 255) / 256);
    if (hdr_bytes == 6)
        repack_v44_kernel<6><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)dmin, (const uint16_t*)dmax, config, coeff, hi, lo, out_f, n_cb, (uint8_t*)hdr_out, (uint8_t*)levels_out);
    else
        repack_v44_kernel<8><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)dmin, (const uint16_t*)dmax, config, coeff, hi, lo, out_f, n_cb, (uint8_t*)hdr_out, (uint8_t*)levels_out);
    SX8_LAUNCH_CHECK("repack_v44_kernel");
    return SX8_OK;
}
