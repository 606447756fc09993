// sx8_glue.cu -- the small kernels between the S-X8 linears of one decode step: residual add +
// RMSNorm, rotary embedding + KV-cache write, single-position attention over the cache, SwiGLU.
// They exist so that a captured decode step is nine launches per layer instead of about
// thirty framework kernels; none of them has a counterpart among the reference's kernels (the
// reference leaves this work to the host framework's model code).
//
// Shapes: B <= 64 sequences, residual stream h (B, H) f32, GEMV outputs f32, activations handed
// to the next linear f16.  The position is read from device memory so that one captured graph
// serves every step.
#include "sx8_common.cuh"

namespace sx8 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// h[b] += y[b] (when y != null); x[b] = f16( h[b] * rsqrt(mean(h[b]^2) + eps) * gamma )
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ y, const float* __restrict__ gamma, int H, float eps,
                   __half* __restrict__ x) {
    __shared__ float red[8];
    const long row = blockIdx.x;
    float* hr = h + row * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) {
        float v = hr[i];
        if (y) {
            v += y[row * H + i];
            hr[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot += red[w];
    const float r = rsqrtf(tot / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += 256) x[row * H + i] = __float2half_rn(hr[i] * r * gamma[i]);
}

// Rotary embedding (half-split convention) of q and k at position *pos; q -> f16 (B, hq, D);
// k, v -> f16 cache rows (B, hkv, S, D) at position *pos.  One CTA per (sequence, head); heads
// 0..hq-1 are q, hq..hq+hkv-1 are k, the rest v.  cos/sin: (S, D/2) f32.
__global__ void __launch_bounds__(64)
rope_cache_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const long* __restrict__ pos_p, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                  int hq, int hkv, int D, int S, __half* __restrict__ q_out, __half* __restrict__ k_cache,
                  __half* __restrict__ v_cache) {
    const int b = blockIdx.y, head = blockIdx.x;
    const long pos = *pos_p;
    if (pos < 0 || pos >= S) return;
    const int half = D / 2;
    if (head < hq + hkv) {
        const bool is_q = head < hq;
        const float* src = is_q ? q + ((long)b * hq + head) * D : k + ((long)b * hkv + (head - hq)) * D;
        __half* dst = is_q ? q_out + ((long)b * hq + head) * D
                           : k_cache + (((long)b * hkv + (head - hq)) * S + pos) * D;
        for (int i = threadIdx.x; i < half; i += 64) {
            float c = cos_t[pos * half + i], s = sin_t[pos * half + i];
            float x1 = src[i], x2 = src[half + i];
            dst[i] = __float2half_rn(x1 * c - x2 * s);
            dst[half + i] = __float2half_rn(x2 * c + x1 * s);
        }
    } else {
        const int hv = head - hq - hkv;
        const float* src = v + ((long)b * hkv + hv) * D;
        __half* dst = v_cache + (((long)b * hkv + hv) * S + pos) * D;
        for (int i = threadIdx.x; i < D; i += 64) dst[i] = __float2half_rn(src[i]);
    }
}

// Attention of one new position over the cache: out (B, hq*D) f16.  One CTA per (sequence, kv
// head); the GRP = hq/hkv query heads of the group share every K and V row read.  Scores of
// positions 0..*pos are kept in shared memory (S floats per query head).
template <int D, int GRP>
__global__ void __launch_bounds__(256)
attn_decode_kernel(const __half* __restrict__ q, const __half* __restrict__ k_cache, const __half* __restrict__ v_cache,
                   const long* __restrict__ pos_p, int hkv, int S, float scale, __half* __restrict__ out) {
    extern __shared__ float sc[];                 // GRP * S scores, then GRP * D query values
    float* qs = sc + (size_t)GRP * S;
    __shared__ float red[GRP][8];
    const int b = blockIdx.y, hv = blockIdx.x;
    const int n = (int)min((long)S, *pos_p + 1);  // positions in the cache, the new one included
    const __half* qg = q + ((long)b * hkv + hv) * GRP * D;
    for (int i = threadIdx.x; i < GRP * D; i += 256) qs[i] = __half2float(qg[i]) * scale;
    __syncthreads();
    const __half* kb = k_cache + ((long)b * hkv + hv) * (long)S * D;
    const __half* vb = v_cache + ((long)b * hkv + hv) * (long)S * D;
    // scores: one thread per position, all GRP heads at once (the K row is read once)
    float mx[GRP];
#pragma unroll
    for (int g = 0; g < GRP; g++) mx[g] = -INFINITY;
    for (int t = threadIdx.x; t < n; t += 256) {
        const uint4* kr = reinterpret_cast<const uint4*>(kb + (long)t * D);
        float acc[GRP];
#pragma unroll
        for (int g = 0; g < GRP; g++) acc[g] = 0.f;
#pragma unroll 4
        for (int c = 0; c < D / 8; c++) {
            uint4 raw = kr[c];
            const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 kv = __half22float2(h2[j]);
#pragma unroll
                for (int g = 0; g < GRP; g++) {
                    acc[g] = fmaf(kv.x, qs[g * D + c * 8 + 2 * j], acc[g]);
                    acc[g] = fmaf(kv.y, qs[g * D + c * 8 + 2 * j + 1], acc[g]);
                }
            }
        }
#pragma unroll
        for (int g = 0; g < GRP; g++) {
            sc[g * S + t] = acc[g];
            mx[g] = fmaxf(mx[g], acc[g]);
        }
    }
    // block-wide max and sum per head
    float m[GRP], den[GRP];
#pragma unroll
    for (int g = 0; g < GRP; g++) {
        float w = warp_max(mx[g]);
        if ((threadIdx.x & 31) == 0) red[g][threadIdx.x >> 5] = w;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GRP; g++) {
        float w = red[g][0];
#pragma unroll
        for (int i = 1; i < 8; i++) w = fmaxf(w, red[g][i]);
        m[g] = w;
    }
    __syncthreads();
    float part[GRP];
#pragma unroll
    for (int g = 0; g < GRP; g++) part[g] = 0.f;
    for (int t = threadIdx.x; t < n; t += 256) {
#pragma unroll
        for (int g = 0; g < GRP; g++) {
            float e = __expf(sc[g * S + t] - m[g]);
            sc[g * S + t] = e;
            part[g] += e;
        }
    }
#pragma unroll
    for (int g = 0; g < GRP; g++) {
        float w = warp_sum(part[g]);
        if ((threadIdx.x & 31) == 0) red[g][threadIdx.x >> 5] = w;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GRP; g++) {
        float w = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) w += red[g][i];
        den[g] = w;
    }
    // out[g][d] = sum_t p[g][t] * V[t][d]: thread = (slice of positions, pair of dims); D/2 threads
    // cover a V row with 4-byte loads, 256 / (D/2) slices split the positions
    constexpr int TPR = D / 2, SL = 256 / TPR;
    const int dp = threadIdx.x % TPR, sl = threadIdx.x / TPR;
    float o0[GRP], o1[GRP];
#pragma unroll
    for (int g = 0; g < GRP; g++) { o0[g] = 0.f; o1[g] = 0.f; }
    for (int t = sl; t < n; t += SL) {
        float2 vv = __half22float2(*reinterpret_cast<const __half2*>(vb + (long)t * D + 2 * dp));
#pragma unroll
        for (int g = 0; g < GRP; g++) {
            float pw = sc[g * S + t];
            o0[g] = fmaf(pw, vv.x, o0[g]);
            o1[g] = fmaf(pw, vv.y, o1[g]);
        }
    }
    __syncthreads();                              // scores are dead: reuse the buffer for the slices
    float* acc = sc;                              // (SL, GRP, D)
#pragma unroll
    for (int g = 0; g < GRP; g++) {
        acc[(sl * GRP + g) * D + 2 * dp] = o0[g];
        acc[(sl * GRP + g) * D + 2 * dp + 1] = o1[g];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < GRP * D; i += 256) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < SL; j++) s += acc[j * GRP * D + i];
        out[((long)b * hkv + hv) * GRP * D + i] = __float2half_rn(s / den[i / D]);
    }
}

// act = f16( silu(g) * u )
__global__ void __launch_bounds__(256)
silu_mul_kernel(const float* __restrict__ g, const float* __restrict__ u, long n, __half* __restrict__ act) {
    long i = (long)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float a = g[i];
    act[i] = __float2half_rn(a / (1.0f + __expf(-a)) * u[i]);
}

}  // namespace sx8

using namespace sx8;

extern "C" int sx8_glue_add_rmsnorm(void* h, const void* y, const void* gamma, int B, int H, float eps, void* x_out,
                                    void* stream) {
    SX8_REQUIRE(h && gamma && x_out, "sx8_glue_add_rmsnorm: null pointer");
    SX8_REQUIRE(B > 0 && H > 0, "sx8_glue_add_rmsnorm: need B>0, H>0");
    add_rmsnorm_kernel<<<(unsigned)B, 256, 0, (cudaStream_t)stream>>>((float*)h, (const float*)y, (const float*)gamma, H, eps,
                                                                       (__half*)x_out);
    SX8_LAUNCH_CHECK("add_rmsnorm_kernel");
    return SX8_OK;
}

extern "C" int sx8_glue_rope_cache(const void* q, const void* k, const void* v, const void* pos, const void* cos_t,
                                   const void* sin_t, int B, int hq, int hkv, int D, int S, void* q_out, void* k_cache,
                                   void* v_cache, void* stream) {
    SX8_REQUIRE(q && k && v && pos && cos_t && sin_t && q_out && k_cache && v_cache, "sx8_glue_rope_cache: null pointer");
    SX8_REQUIRE(B > 0 && hq > 0 && hkv > 0 && D > 0 && (D % 2) == 0 && S > 0, "sx8_glue_rope_cache: bad sizes");
    dim3 grid((unsigned)(hq + 2 * hkv), (unsigned)B, 1);
    rope_cache_kernel<<<grid, 64, 0, (cudaStream_t)stream>>>((const float*)q, (const float*)k, (const float*)v, (const long*)pos,
                                                             (const float*)cos_t, (const float*)sin_t, hq, hkv, D, S,
                                                             (__half*)q_out, (__half*)k_cache, (__half*)v_cache);
    SX8_LAUNCH_CHECK("rope_cache_kernel");
    return SX8_OK;
}

extern "C" int sx8_glue_attn_decode(const void* q, const void* k_cache, const void* v_cache, const void* pos, int B, int hq,
                                    int hkv, int D, int S, float scale, void* out, void* stream) {
    SX8_REQUIRE(q && k_cache && v_cache && pos && out, "sx8_glue_attn_decode: null pointer");
    SX8_REQUIRE(B > 0 && hkv > 0 && S > 0 && hq % hkv == 0, "sx8_glue_attn_decode: bad sizes");
    const int grp = hq / hkv;
    SX8_REQUIRE((D == 128 || D == 64) && (grp == 4 || grp == 2 || grp == 1 || grp == 8),
                "sx8_glue_attn_decode: supports head_dim 64 or 128 and 1, 2, 4 or 8 query heads per kv head (got %d, %d)", D, grp);
    // scores (grp * S floats) + scaled queries (grp * D); the buffer is reused for the
    // (256 / (D/2)) x grp x D partial outputs
    size_t smem = sizeof(float) * ((size_t)grp * S + (size_t)grp * D);
    size_t need2 = sizeof(float) * (size_t)(256 / (D / 2)) * grp * D;
    if (need2 > smem) smem = need2;
    SX8_REQUIRE(smem <= 200 * 1024, "sx8_glue_attn_decode: cache length %d needs %zu bytes of shared memory", S, smem);
    dim3 grid((unsigned)hkv, (unsigned)B, 1);
    cudaStream_t st = (cudaStream_t)stream;
#define SX8_ATTN(DD, GG)                                                                                              \
    do {                                                                                                              \
        if (smem > 48 * 1024) {                                                                                       \
            cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<DD, GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                                          \
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(attn_decode)");                          \
        }                                                                                                             \
        attn_decode_kernel<DD, GG><<<grid, 256, smem, st>>>((const __half*)q, (const __half*)k_cache,                 \
                                                            (const __half*)v_cache, (const long*)pos, hkv, S, scale,  \
                                                            (__half*)out);                                            \
    } while (0)
    if (D == 128 && grp == 4) SX8_ATTN(128, 4);
    else if (D == 128 && grp == 8) SX8_ATTN(128, 8);
    else if (D == 128 && grp == 2) SX8_ATTN(128, 2);
    else if (D == 128 && grp == 1) SX8_ATTN(128, 1);
    else if (D == 64 && grp == 4) SX8_ATTN(64, 4);
    else if (D == 64 && grp == 8) SX8_ATTN(64, 8);
    else if (D == 64 && grp == 2) SX8_ATTN(64, 2);
    else SX8_ATTN(64, 1);
#undef SX8_ATTN
    SX8_LAUNCH_CHECK("attn_decode_kernel");
    return SX8_OK;
}

extern "C" int sx8_glue_silu_mul(const void* g, const void* u, long n, void* act_out, void* stream) {
    SX8_REQUIRE(g && u && act_out, "sx8_glue_silu_mul: null pointer");
    SX8_REQUIRE(n > 0 && (n + 255) / 256 <= 0x7FFFFFFFL, "sx8_glue_silu_mul: bad size %ld", n);
    silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float*)g, (const float*)u, n,
                                                                                    (__half*)act_out);
    SX8_LAUNCH_CHECK("silu_mul_kernel");
    return SX8_OK;
}
