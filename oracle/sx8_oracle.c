/* sx8_oracle.c -- CPU restatement of the S-X8 v4.3 hot-path arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA kernels: the
 * test-suite, the smoke test and the CPU-baseline leg of the benchmark link it;
 * the product library never does.
 *
 * Every function restates, in plain scalar C, one piece of the reference
 * (MarlaLabsAI/sx8-quantization); the reference file:line it follows is cited
 * above each function.  Build with
 *     gcc -O2 -ffp-contract=off -fno-fast-math -shared -fPIC
 * so that the compiler neither fuses nor reorders floating-point operations:
 * fused multiply-adds appear only where fmaf()/fma() is written out.
 *
 * Pinning status (what the restatement has been checked against):
 *   - quantizer search + packing : bit-exact against the reference's own torch
 *     functions run on CPU (fixtures under tests/golden, full-size checksums).
 *   - v4.4 layout transform      : bit-exact against the reference's to_v44.
 *   - reformulated GEMV          : against the reference's decode_v44_numpy.
 *   - D64 full-tensor decode     : PARITY UNPINNED -- the reference decoder is a
 *     numba-CUDA kernel that needs a GPU; its typing rules are restated by
 *     reading (float32 loads, float64 arithmetic, float32 store, fp16 cast).
 *   - D32 embedding rows         : restated from the CUDA-C kernel with nvcc's
 *     default multiply-add contraction written out as fmaf(); pinned on a GPU
 *     box against the reference kernel when oracle/_ref holds its build.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- fp16 <-> fp32 */

static inline float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* round-to-nearest-even, like numpy astype(float16), torch .half(), __float2half */
static inline uint16_t f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0));
    if (ax >= 0x477FF000u) /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    if (ax < 0x33000001u) /* < 2^-25 (or == 2^-25 tie -> 0) */
        return (uint16_t)sign;
    int e = (int)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t hexp;
    if (e < -14) { /* subnormal result */
        shift = 13 + (-14 - e);
        hexp = 0;
    } else {
        shift = 13;
        hexp = (uint32_t)(e + 15);
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    uint32_t h;
    if (hexp == 0)
        h = q; /* may carry into exponent 1: correct */
    else
        h = ((hexp - 1) << 10) + q; /* q includes the hidden bit (0x400) */
    return (uint16_t)(sign | h);
}

void sx8o_f16_to_f32(const uint16_t* in, float* out, long n) {
    for (long i = 0; i < n; i++) out[i] = h2f(in[i]);
}

void sx8o_f32_to_f16(const float* in, uint16_t* out, long n) {
    for (long i = 0; i < n; i++) out[i] = f2h(in[i]);
}

/* ------------------------------------------------------------- level extraction
 * docs/SX8_FLASH_V4_3_SPEC.md:13-25, scripts/prepare_v44.py:82-93.
 * File layout (v4.3): qh[w>>1] bits (w&1)*4.., ql[w>>2] bits (3-(w&3))*2..   */
static inline int level_v43(const uint8_t* hi16, const uint8_t* lo8, int w) {
    int nib = (hi16[w >> 1] >> ((w & 1) * 4)) & 0xF;
    int qua = (lo8[w >> 2] >> ((3 - (w & 3)) * 2)) & 0x3;
    return (nib << 2) | qua;
}

static inline int s4(int x) { return x < 8 ? x : x - 16; }

/* ------------------------------------------------------------ quantizer search
 * scripts/quantize_qwen35_4b_sx8_v43_gpu.py:22-47 (v6_encode_6bit_gpu), torch
 * eager float32 semantics restated op by op: IEEE division, separate multiply
 * and add, round-half-even, strict '<' (lowest strategy wins ties).
 * cuda_arith = 0: torch CPU -- (hi - lo) / 63 is an IEEE division and the mean over 8 a
 *   left-to-right sum divided by 8 (pinned by the golden fixtures, which were made by
 *   running the reference's functions on torch CPU).
 * cuda_arith = 1: torch CUDA, the back end the reference script runs on (:9) -- a tensor
 *   divided by the host scalar 63 is multiplied by float(1/63), and the mean over 8 is
 *   the butterfly sum ((e0+e4)+(e2+e6)) + ((e1+e5)+(e3+e7)) times 1/8 (both observed on a
 *   B200 against torch 2.11: 0 differences in 8M rows; pinned by the GPU test that runs the
 *   reference's functions with DEV = cuda).
 * blocks: (n_blk, 32) f32.  Outputs: levels (n_blk,32) u8, dmin/dmax f32,
 * config i32.                                                                  */
void sx8o_quant_search2(const float* blocks, long n_blk, uint8_t* levels,
                        float* dmin_out, float* dmax_out, int32_t* config_out, int cuda_arith) {
    const float inv63 = 1.0f / 63.0f;
#pragma omp parallel for schedule(static)
    for (long b = 0; b < n_blk; b++) {
        const float* x = blocks + b * 32;
        float dmin = x[0], dmax = x[0];
        for (int t = 1; t < 32; t++) {
            if (x[t] < dmin) dmin = x[t];
            if (x[t] > dmax) dmax = x[t];
        }
        float d = dmax - dmin;
        if (d < 1e-10f) d = 1e-10f;
        float q = d / 4.0f;
        float slo[4] = {dmin, dmin, dmax - q, dmin + q};
        float shi[4] = {dmax, dmin + q, dmax, dmax - q};
        int cfg = 0;
        for (int sb = 0; sb < 4; sb++) {
            const float* s = x + sb * 8;
            float best = INFINITY;
            int best_r = 0;
            uint8_t best_lv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int r = 0; r < 4; r++) {
                float lo = slo[r], hi = shi[r];
                float step = cuda_arith ? (hi - lo) * inv63 : (hi - lo) / 63.0f;
                if (step < 1e-10f) step = 1e-10f;
                uint8_t lv[8];
                float sq[8];
                for (int i = 0; i < 8; i++) {
                    float c = rintf((s[i] - lo) / step);
                    if (c < 0.0f) c = 0.0f;
                    if (c > 63.0f) c = 63.0f;
                    int ci = (int)c;
                    lv[i] = (uint8_t)ci;
                    float prod = step * (float)ci;
                    float rec = lo + prod;
                    float e = s[i] - rec;
                    sq[i] = e * e;
                }
                float mse;
                if (cuda_arith) {
                    float a = (sq[0] + sq[4]) + (sq[2] + sq[6]);
                    float b2 = (sq[1] + sq[5]) + (sq[3] + sq[7]);
                    mse = (a + b2) * 0.125f;
                } else {
                    float sum = 0.0f;
                    for (int i = 0; i < 8; i++) sum = sum + sq[i];
                    mse = sum / 8.0f;
                }
                if (mse < best) {
                    best = mse;
                    best_r = r;
                    memcpy(best_lv, lv, 8);
                }
            }
            memcpy(levels + b * 32 + sb * 8, best_lv, 8);
            cfg |= best_r << (2 * sb);
        }
        dmin_out[b] = dmin;
        dmax_out[b] = dmax;
        config_out[b] = cfg;
    }
}

void sx8o_quant_search(const float* blocks, long n_blk, uint8_t* levels,
                       float* dmin_out, float* dmax_out, int32_t* config_out) {
    sx8o_quant_search2(blocks, n_blk, levels, dmin_out, dmax_out, config_out, 0);
}

/* scripts/quantize_qwen35_4b_sx8_v43_gpu.py:148-167 (pack_levels_6bit).
 * levels (n_blk,32) -> hi (n_blk,16): w even in the low nibble; lo (n_blk,8):
 * weight 4k in bits 7:6, 4k+1 in 5:4, 4k+2 in 3:2, 4k+3 in 1:0.                */
void sx8o_pack_levels(const uint8_t* levels, long n_blk, uint8_t* hi, uint8_t* lo) {
    for (long b = 0; b < n_blk; b++) {
        const uint8_t* lv = levels + b * 32;
        for (int k = 0; k < 16; k++) {
            int a = (lv[2 * k] & 0x3F) >> 2, c = (lv[2 * k + 1] & 0x3F) >> 2;
            hi[b * 16 + k] = (uint8_t)((a & 0xF) | ((c << 4) & 0xF0));
        }
        for (int k = 0; k < 8; k++) {
            lo[b * 8 + k] = (uint8_t)(((lv[4 * k] & 3) << 6) | ((lv[4 * k + 1] & 3) << 4) |
                                      ((lv[4 * k + 2] & 3) << 2) | (lv[4 * k + 3] & 3));
        }
    }
}

/* ------------------------------------------------------------- layout transform
 * scripts/prepare_v44.py:35-79 (to_v44).  n-major planes -> kb-major
 * hdr (n_blk, hdr_bytes) = dmin,dmax (fp16 bits), config, coeff [, 2 pad] and
 * levels (n_blk,24) = hi of sub-block 0..3 (4 B each) then lo of 0..3 (2 B each). */
void sx8o_to_v44(long out_f, long n_cb, const uint16_t* dmin, const uint16_t* dmax,
                 const uint8_t* config, const uint8_t* coeff, const uint8_t* hi,
                 const uint8_t* lo, int hdr_bytes, uint8_t* hdr_out, uint8_t* levels_out) {
    for (long n = 0; n < out_f; n++) {
        for (long kb = 0; kb < n_cb; kb++) {
            long src = n * n_cb + kb, dst = kb * out_f + n;
            uint8_t* h = hdr_out + dst * hdr_bytes;
            memset(h, 0, (size_t)hdr_bytes);
            h[0] = (uint8_t)(dmin[src] & 0xFF);
            h[1] = (uint8_t)(dmin[src] >> 8);
            h[2] = (uint8_t)(dmax[src] & 0xFF);
            h[3] = (uint8_t)(dmax[src] >> 8);
            h[4] = config[src];
            h[5] = coeff[src];
            uint8_t* l = levels_out + dst * 24;
            memcpy(l, hi + src * 16, 16);      /* hi of sb: bytes 4sb..4sb+3 */
            memcpy(l + 16, lo + src * 8, 8);   /* lo of sb: bytes 16+2sb..   */
        }
    }
}

/* ------------------------------------------------------- D64 full-tensor decode
 * scripts/kernel_sx8_v43.py:14-51 (sx8_v43_kernel) with the host side of
 * decode_tensor_gpu_fast (:123-141).  numba typing restated: dmin/dmax/scales/
 * basis are float32 loads; (hi_f - lo_f) is a float32 subtraction; every Python
 * float literal is float64, so q, rlo, rhi, step, w and the PCA terms are
 * float64; NVVM contracts a*b+c into one fma; the store rounds to float32.
 * planes are n-major (bid = n*n_cb + kb).  out32: (n_blk*32) f32 -- the caller
 * reshapes to (out_f, n_cb*32), slices [:, :in_f] and casts to fp16.           */
void sx8o_dequant_d64(const uint16_t* dmin, const uint16_t* dmax, const uint8_t* config,
                      const uint8_t* coeff, const uint8_t* hi, const uint8_t* lo,
                      const float* basis, const float* scales, long n_blk, long n_cb,
                      int use_pca, float* out32) {
#pragma omp parallel for schedule(static)
    for (long bid = 0; bid < n_blk; bid++) {
        float lo_f = h2f(dmin[bid]), hi_f = h2f(dmax[bid]);
        float d32 = hi_f - lo_f;               /* float32 - float32 */
        double q = (double)d32 * 0.25;
        int cfg = config[bid];
        int b0 = coeff[bid];
        int c0 = s4(b0 & 0xF), c1 = s4((b0 >> 4) & 0xF);
        long cb = bid % n_cb;
        for (int tid = 0; tid < 32; tid++) {
            int lv = level_v43(hi + bid * 16, lo + bid * 8, tid);
            int strat = (cfg >> ((tid >> 3) * 2)) & 3;
            double rlo, rhi;
            if (strat == 0) { rlo = lo_f; rhi = hi_f; }
            else if (strat == 1) { rlo = lo_f; rhi = (double)lo_f + q; }
            else if (strat == 2) { rlo = (double)hi_f - q; rhi = hi_f; }
            else { rlo = (double)lo_f + q; rhi = (double)hi_f - q; }
            double step = (rhi - rlo) * 0.015873;
            if (step < 1e-10) step = 1e-10;
            double w = fma(step, (double)lv, rlo);
            if (use_pca) {
                double p0 = 1.0 * (double)c0 * (double)scales[cb * 2 + 0];
                w = fma(p0, (double)basis[cb * 64 + tid], w);
                double p1 = 1.0 * (double)c1 * (double)scales[cb * 2 + 1];
                w = fma(p1, (double)basis[cb * 64 + 32 + tid], w);
            }
            out32[bid * 32 + tid] = (float)w;
        }
    }
}

/* --------------------------------------------------------------- D32 decode core
 * cuda/sx8_embed_v44.cu:36-75 and cuda/sx8_decode1_v3.cu:108-150: float32
 * throughout, constant 0.015873f.  contract != 0 writes nvcc's default
 * multiply-add contraction (-fmad=true) out as fmaf(); contract == 0 rounds
 * every product.                                                               */
static inline void d32_range(float lo_f, float hi_f, int s, int contract, float* rlo_o,
                             float* step_o) {
    float q = (hi_f - lo_f) * 0.25f;
    float kl = (float)(3 * (s == 2) + (s == 3));
    float kh = (float)(3 * (s == 1) + (s == 3));
    float rlo, rhi;
    if (contract) {
        rlo = fmaf(q, kl, lo_f);
        rhi = fmaf(-q, kh, hi_f);
    } else {
        float a = q * kl; rlo = lo_f + a;
        float c = q * kh; rhi = hi_f - c;
    }
    float step = (rhi - rlo) * 0.015873f;
    if (step < 1e-10f) step = 1e-10f;
    *rlo_o = rlo;
    *step_o = step;
}

/* v4.4 level of weight i (0..7) of sub-block sb: cuda/sx8_decode1_v3.cu:147-149 */
static inline int level_v44(const uint8_t* lv24, int sb, int i) {
    uint32_t hi4;
    uint16_t lo2;
    memcpy(&hi4, lv24 + sb * 4, 4);
    memcpy(&lo2, lv24 + 16 + sb * 2, 2);
    int nib = (int)((hi4 >> (i * 4)) & 0xF);
    int qua = (int)((lo2 >> ((i >> 2) * 8 + (3 - (i & 3)) * 2)) & 0x3);
    return (nib << 2) | qua;
}

/* Embedding rows, cuda/sx8_embed_v44.cu:21-77.  v4.4 layout (kb-major, 6-byte
 * hdr).  out: (T, K) fp16 bits.  Rows with id >= N are left untouched, as in
 * the reference (:34); negative ids are rejected by the product, not here.     */
void sx8o_embed_d32(const int64_t* ids, long T, const uint8_t* hdr, const uint8_t* levels,
                    const float* basis, const float* scales, long K, long N, long n_cb,
                    int hdr_bytes, int contract, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (long t = 0; t < T; t++) {
        int64_t row = ids[t];
        if (row >= N || row < 0) continue;
        for (long k = 0; k < K; k++) {
            long kb = k >> 5;
            int tid = (int)(k & 31);
            long bid = kb * N + row;
            const uint8_t* h = hdr + bid * hdr_bytes;
            uint16_t h0, h1;
            memcpy(&h0, h, 2);
            memcpy(&h1, h + 2, 2);
            int cfg = h[4], co = h[5];
            float lo_f = h2f(h0), hi_f = h2f(h1);
            int sb = tid >> 3;
            int s = (cfg >> (sb * 2)) & 3;
            float rlo, step;
            d32_range(lo_f, hi_f, s, contract, &rlo, &step);
            int c0 = s4(co & 0xF), c1 = s4((co >> 4) & 0xF);
            int lv = level_v44(levels + bid * 24, sb, tid & 7);
            float p0 = (float)c0 * scales[kb * 2];
            float p1 = (float)c1 * scales[kb * 2 + 1];
            float w;
            if (contract) {
                w = fmaf(step, (float)lv, rlo);
                w = fmaf(p0, basis[kb * 64 + tid], w);
                w = fmaf(p1, basis[kb * 64 + 32 + tid], w);
            } else {
                float a = step * (float)lv; w = rlo + a;
                float b = p0 * basis[kb * 64 + tid]; w = w + b;
                float c = p1 * basis[kb * 64 + 32 + tid]; w = w + c;
            }
            out[t * K + k] = f2h(w);
        }
    }
}

/* Reformulated GEMV in float32, one batch row at a time:
 * cuda/sx8_decode1_v3.cu:44-65 (Z) and :75-167 (Y), same expression order as the
 * kernel per lane; the cross-lane order (4 sub-blocks of a column) is the
 * butterfly of :161-162.  Tolerance-checked only (the CUDA kernels here sum in a
 * different order).  x: (M,K) fp16 bits, K = n_cb*32; y: (M,N) f32.             */
void sx8o_gemv_d32(const uint16_t* x, long M, const uint8_t* hdr, const uint8_t* levels,
                   const float* basis, const float* scales, long N, long n_cb, int hdr_bytes,
                   float* y) {
    long K = n_cb * 32;
    for (long m = 0; m < M; m++) {
        const uint16_t* xr = x + m * K;
#pragma omp parallel for schedule(static)
        for (long n = 0; n < N; n++) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (long kb = 0; kb < n_cb; kb++) {
                long bid = kb * N + n;
                const uint8_t* h = hdr + bid * hdr_bytes;
                uint16_t h0, h1;
                memcpy(&h0, h, 2);
                memcpy(&h1, h + 2, 2);
                int cfg = h[4], co = h[5];
                float lo_f = h2f(h0), hi_f = h2f(h1);
                for (int sb = 0; sb < 4; sb++) {
                    float rlo, step;
                    d32_range(lo_f, hi_f, (cfg >> (sb * 2)) & 3, 1, &rlo, &step);
                    for (int i = 0; i < 8; i++) {
                        int lv = level_v44(levels + bid * 24, sb, i);
                        float w = fmaf(step, (float)lv, rlo);
                        acc[sb] = fmaf(h2f(xr[kb * 32 + sb * 8 + i]), w, acc[sb]);
                    }
                }
                /* PCA once per block on the sub-block-0 lane */
                float z0 = 0.f, z1 = 0.f;
                for (int t = 0; t < 32; t++) {
                    float xv = h2f(xr[kb * 32 + t]);
                    z0 = fmaf(xv, basis[kb * 64 + t], z0);
                    z1 = fmaf(xv, basis[kb * 64 + 32 + t], z1);
                }
                z0 = scales[kb * 2] * z0;
                z1 = scales[kb * 2 + 1] * z1;
                int c0 = s4(co & 0xF), c1 = s4((co >> 4) & 0xF);
                float p = fmaf((float)c1, z1, (float)c0 * z0);
                acc[0] = acc[0] + p;
            }
            y[m * N + n] = (acc[0] + acc[2]) + (acc[1] + acc[3]);
        }
    }
}

int sx8o_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
