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

// Programmatic dependent launch: let the next kernel of the stream (a GEMV, which then starts
// streaming its weights) be scheduled at once, and wait for the preceding kernel before
// touching any input.  Both are no-ops for a launch without the attribute.
__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Launch with the programmatic-stream-serialization attribute.
template <class... KArgs, class... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

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

// h[b] += y[b] (when y != null); x[b] = f16( h[b] * rsqrt(mean(h[b]^2) + eps) * gamma ).
// One CTA of 1024 threads per row; a thread keeps its (up to kRmsPer) float4 of the row in
// registers between the sum and the scaling, so the row is read once (H % 4 == 0,
// H <= 4096 * kRmsPer).
constexpr int kRmsThreads = 1024, kRmsPer = 4;
__global__ void __launch_bounds__(kRmsThreads)
add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ y, const float* __restrict__ gamma, int H, float eps,
                   __half* __restrict__ x) {
    pdl_prologue();
    __shared__ float red[32];
    const long row = blockIdx.x;
    float4* hr = reinterpret_cast<float4*>(h + row * H);
    const float4* yr = y ? reinterpret_cast<const float4*>(y + row * H) : nullptr;
    const int n4 = H >> 2;
    float4 v[kRmsPer];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kRmsPer; j++) {
        const int i = threadIdx.x + j * kRmsThreads;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            v[j] = hr[i];
            if (yr) {
                float4 w = yr[i];
                v[j].x += w.x; v[j].y += w.y; v[j].z += w.z; v[j].w += w.w;
                hr[i] = v[j];
            }
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 32; w++) tot += red[w];
    const float r = rsqrtf(tot / (float)H + eps);
    const float4* gr = reinterpret_cast<const float4*>(gamma);
    uint2* xr = reinterpret_cast<uint2*>(x + row * H);
#pragma unroll
    for (int j = 0; j < kRmsPer; j++) {
        const int i = threadIdx.x + j * kRmsThreads;
        if (i < n4) {
            float4 g = gr[i];
            __half2 lo = __floats2half2_rn(v[j].x * r * g.x, v[j].y * r * g.y);
            __half2 hi = __floats2half2_rn(v[j].z * r * g.z, v[j].w * r * g.w);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&lo);
            o.y = *reinterpret_cast<uint32_t*>(&hi);
            xr[i] = o;
        }
    }
}

// ------------------------------------------------------------------ all-reduce + residual + RMSNorm
// The consumer of a row-parallel linear in a tensor-parallel decode step, as ONE kernel over peer
// memory: every rank has written its partial y_r (M, H) f32 into its own exchange buffer (slot
// `epoch & 1`); this kernel tells every peer "my partial of this epoch is complete", waits --
// bounded -- for the same word from every peer, then reads all partials straight from the peers'
// memory (plain loads over NVLink; no multicast, no bulk copies), sums them in rank order (so all
// ranks compute the same bits), adds the sum to the residual stream and normalises.  One CTA per
// batch row; a thread keeps its part of the row in registers, so every partial is read once.
//
// The epoch is a call counter kept in device memory (so that a CUDA graph that replays these
// calls keeps counting): every CTA reads it at its start, the last CTA to finish advances it.
// Buffer re-use: the caller alternates between two slots, so a rank writes a slot again two
// calls later.  Before that it has passed this kernel's wait of the call in between, i.e. every
// peer has started that call's kernel, which in stream order comes after the peer finished
// reading the earlier call's partials.
struct ArParams {
    const float* part[8];       // rank q's partial (this call's slot) as mapped in this process
    unsigned* flag_out[8];      // word [rank] of rank q's epoch array
    const unsigned* flag_in;    // this rank's epoch array: word [q] is written by rank q
    unsigned* ctr;              // this rank's call counter and the count of CTAs done with this call
    int world, rank;
};
constexpr uint32_t kArSpinLimit = 1u << 22;

__global__ void __launch_bounds__(kRmsThreads)
allreduce_add_rmsnorm_kernel(ArParams a, float* __restrict__ h, const float* __restrict__ gamma, int H, float eps,
                             __half* __restrict__ x) {
    pdl_prologue();   // this rank's own GEMV has completed: its partial is in memory
    __shared__ float red[32];
    __shared__ unsigned s_epoch;
    if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile unsigned*>(a.ctr) + 1u;
    __syncthreads();
    const unsigned epoch = s_epoch;
    if (blockIdx.x == 0 && (int)threadIdx.x < a.world) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flag_out[threadIdx.x]), "r"(epoch) : "memory");
    }
    if ((int)threadIdx.x < a.world) {
        int ok = 0;
        for (uint32_t i = 0; i < kArSpinLimit; i++) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.flag_in + threadIdx.x) : "memory");
            if ((int)(v - epoch) >= 0) { ok = 1; break; }
        }
        if (!ok) atomicOr(&g_sx8_error_flag, 8u);   // a peer never arrived: record it, sum what is there
    }
    __syncthreads();
    const long row = blockIdx.x;
    float4* hr = reinterpret_cast<float4*>(h + row * H);
    const int n4 = H >> 2;
    float4 v[kRmsPer];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kRmsPer; j++) {
        const int i = threadIdx.x + j * kRmsThreads;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int q = 0; q < a.world; q++) {
                const float4 w = __ldcv(reinterpret_cast<const float4*>(a.part[q] + row * H) + i);
                acc.x += w.x; acc.y += w.y; acc.z += w.z; acc.w += w.w;
            }
            float4 t = hr[i];
            t.x += acc.x; t.y += acc.y; t.z += acc.z; t.w += acc.w;
            hr[i] = t;
            v[j] = t;
            ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 32; w++) tot += red[w];
    const float r = rsqrtf(tot / (float)H + eps);
    const float4* gr = reinterpret_cast<const float4*>(gamma);
    uint2* xr = reinterpret_cast<uint2*>(x + row * H);
#pragma unroll
    for (int j = 0; j < kRmsPer; j++) {
        const int i = threadIdx.x + j * kRmsThreads;
        if (i < n4) {
            float4 g = gr[i];
            __half2 lo = __floats2half2_rn(v[j].x * r * g.x, v[j].y * r * g.y);
            __half2 hi = __floats2half2_rn(v[j].z * r * g.z, v[j].w * r * g.w);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&lo);
            o.y = *reinterpret_cast<uint32_t*>(&hi);
            xr[i] = o;
        }
    }
    // the last CTA to finish advances the call counter (every CTA has read it by then)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(a.ctr + 1, 1u);
        if (prev == gridDim.x - 1) {
            a.ctr[1] = 0u;
            a.ctr[0] = epoch;
            __threadfence();
        }
    }
}


// Rotary embedding (half-split convention) of q and k at position *pos; q -> f16 (B, hq, D);
// k, v -> f16 cache rows (B, hkv, S, D) at position *pos.  One CTA per (sequence, head); heads
// 0..hq-1 are q, hq..hq+hkv-1 are k, the rest v.  cos/sin: (S, D/2) f32.
__global__ void __launch_bounds__(64)
rope_cache_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const long* __restrict__ pos_p, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                  int hq, int hkv, int D, int S, __half* __restrict__ q_out, __half* __restrict__ k_cache,
                  __half* __restrict__ v_cache) {
    pdl_prologue();
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

// Attention of one new position over the cache: out (B, hq*D) f16.  Grid (kv head, sequence,
// kAttnSplit): a CTA takes one slice of the cached positions 0..*pos of one kv head; the
// GRP = hq/hkv query heads of the group share every K and V row it reads.  It writes its
// running maximum, its sum of exponentials and its unnormalised output to scratch; the CTA
// that finishes last for a (sequence, kv head) -- decided by a counter in scratch, which it
// resets -- merges the kAttnSplit partial results.  Everything here is latency: a 768-position
// cache of one head is 190 KB, so the point of the split is to put 8 times as many loads in
// flight, not to share bandwidth.
constexpr int kAttnSplit = 8, kAttnThreads = 256;
template <int D, int GRP>
__global__ void __launch_bounds__(kAttnThreads)
attn_decode_kernel(const __half* __restrict__ q, const __half* __restrict__ k_cache, const __half* __restrict__ v_cache,
                   const long* __restrict__ pos_p, int hkv, int S, float scale, float* __restrict__ part,
                   unsigned* __restrict__ counters, __half* __restrict__ out) {
    pdl_prologue();
    constexpr int CH = 128;                       // at most 128 positions per CTA (S <= 1024)
    __shared__ float sc[GRP][CH];
    __shared__ float qs[GRP * D];
    __shared__ float red[GRP][8];
    __shared__ float acc_s[(kAttnThreads / (D / 2)) * GRP * D];
    __shared__ unsigned s_last;
    const int b = blockIdx.y, hv = blockIdx.x, sp = blockIdx.z;
    const int n = (int)min((long)S, *pos_p + 1);  // positions in the cache, the new one included
    const int chunk = (n + kAttnSplit - 1) / kAttnSplit;
    const int t0 = sp * chunk, cnt = max(0, min(chunk, n - t0));
    const __half* qg = q + ((long)b * hkv + hv) * GRP * D;
    for (int i = threadIdx.x; i < GRP * D; i += kAttnThreads) qs[i] = __half2float(qg[i]) * scale;
    __syncthreads();
    const __half* kb = k_cache + (((long)b * hkv + hv) * (long)S + t0) * D;
    const __half* vb = v_cache + (((long)b * hkv + hv) * (long)S + t0) * D;
    // scores: two threads per position (each half of the head dimension), all GRP heads at once
    float mx[GRP];
#pragma unroll
    for (int g = 0; g < GRP; g++) mx[g] = -INFINITY;
    {
        const int t = threadIdx.x >> 1, hf = threadIdx.x & 1;
        float acc[GRP];
#pragma unroll
        for (int g = 0; g < GRP; g++) acc[g] = 0.f;
        if (t < cnt) {
            const uint4* kr = reinterpret_cast<const uint4*>(kb + (long)t * D + hf * (D / 2));
            uint4 raw[D / 16];
#pragma unroll
            for (int c = 0; c < D / 16; c++) raw[c] = kr[c];
#pragma unroll
            for (int c = 0; c < D / 16; c++) {
                const __half2* h2 = reinterpret_cast<const __half2*>(&raw[c]);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    float2 kv = __half22float2(h2[j]);
                    const int d = hf * (D / 2) + c * 8 + 2 * j;
#pragma unroll
                    for (int g = 0; g < GRP; g++) {
                        acc[g] = fmaf(kv.x, qs[g * D + d], acc[g]);
                        acc[g] = fmaf(kv.y, qs[g * D + d + 1], acc[g]);
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < GRP; g++) {
            acc[g] += __shfl_xor_sync(0xFFFFFFFFu, acc[g], 1);
            if (t < cnt) {
                if (hf == 0) sc[g][t] = acc[g];
                mx[g] = acc[g];
            }
        }
    }
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
    float psum[GRP];
#pragma unroll
    for (int g = 0; g < GRP; g++) psum[g] = 0.f;
    if (threadIdx.x < cnt) {
#pragma unroll
        for (int g = 0; g < GRP; g++) {
            float e = __expf(sc[g][threadIdx.x] - m[g]);
            sc[g][threadIdx.x] = e;
            psum[g] = e;
        }
    }
#pragma unroll
    for (int g = 0; g < GRP; g++) {
        float w = warp_sum(psum[g]);
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
    // o[g][d] = sum_t p[g][t] * V[t][d]: D/2 threads cover a V row with 4-byte loads, the
    // 256 / (D/2) slices split the positions; four rows are in flight per thread
    constexpr int TPR = D / 2, SL = kAttnThreads / TPR;
    const int dp = threadIdx.x % TPR, sl = threadIdx.x / TPR;
    float o0[GRP], o1[GRP];
#pragma unroll
    for (int g = 0; g < GRP; g++) { o0[g] = 0.f; o1[g] = 0.f; }
    for (int tb = sl; tb < cnt; tb += 4 * SL) {
        __half2 vv[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int t = tb + u * SL;
            vv[u] = (t < cnt) ? *reinterpret_cast<const __half2*>(vb + (long)t * D + 2 * dp) : __half2();
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int t = tb + u * SL;
            if (t < cnt) {
                float2 f = __half22float2(vv[u]);
#pragma unroll
                for (int g = 0; g < GRP; g++) {
                    float pw = sc[g][t];
                    o0[g] = fmaf(pw, f.x, o0[g]);
                    o1[g] = fmaf(pw, f.y, o1[g]);
                }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < GRP; g++) {
        acc_s[(sl * GRP + g) * D + 2 * dp] = o0[g];
        acc_s[(sl * GRP + g) * D + 2 * dp + 1] = o1[g];
    }
    __syncthreads();
    // partial result of this slice: [GRP][D] outputs, then GRP maxima, then GRP sums
    constexpr int PSZ = GRP * (D + 2);
    float* mine = part + (((long)b * hkv + hv) * kAttnSplit + sp) * PSZ;
    for (int i = threadIdx.x; i < GRP * D; i += kAttnThreads) {
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < SL; j++) sum += acc_s[j * GRP * D + i];
        mine[i] = sum;
    }
    if (threadIdx.x < GRP) {
        mine[GRP * D + threadIdx.x] = m[threadIdx.x];
        mine[GRP * D + GRP + threadIdx.x] = den[threadIdx.x];
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&counters[b * hkv + hv], 1u);
    __syncthreads();
    if (s_last != kAttnSplit - 1) return;
    __threadfence();
    // merge the slices (this CTA arrived last, so all of them are in scratch)
    const float* all = part + ((long)b * hkv + hv) * kAttnSplit * PSZ;
    for (int i = threadIdx.x; i < GRP * D; i += kAttnThreads) {
        const int g = i / D;
        float M = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < kAttnSplit; s2++) M = fmaxf(M, __ldcg(all + s2 * PSZ + GRP * D + g));
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < kAttnSplit; s2++) {
            float ms = __ldcg(all + s2 * PSZ + GRP * D + g);
            float w = (ms == -INFINITY) ? 0.f : __expf(ms - M);
            L = fmaf(w, __ldcg(all + s2 * PSZ + GRP * D + GRP + g), L);
            O = fmaf(w, __ldcg(all + s2 * PSZ + i), O);
        }
        out[((long)b * hkv + hv) * GRP * D + i] = __float2half_rn(O / L);
    }
    if (threadIdx.x == 0) counters[b * hkv + hv] = 0u;   // ready for the next call
}

// act = f16( silu(g) * u )
__global__ void __launch_bounds__(256)
silu_mul_kernel(const float* __restrict__ g, const float* __restrict__ u, long n, __half* __restrict__ act) {
    pdl_prologue();
    long i = (long)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float a = g[i];
    act[i] = __float2half_rn(a / (1.0f + __expf(-a)) * u[i]);
}

}  // namespace sx8

using namespace sx8;

extern "C" int sx8_glue_allreduce_add_rmsnorm(const sx8_peers_t* peers, int M, int H, void* h, const void* gamma,
                                              float eps, void* x_out, void* stream) {
    SX8_REQUIRE(peers && h && gamma && x_out, "sx8_glue_allreduce_add_rmsnorm: null pointer");
    SX8_REQUIRE(peers->world >= 1 && peers->world <= 8 && peers->rank >= 0 && peers->rank < peers->world,
                "sx8_glue_allreduce_add_rmsnorm: bad rank/world (%d/%d, at most 8 ranks)", peers->rank, peers->world);
    SX8_REQUIRE(M > 0 && H > 0 && (H % 4) == 0 && H <= 4 * kRmsThreads * kRmsPer,
                "sx8_glue_allreduce_add_rmsnorm: need M>0 and H a multiple of 4 up to %d (got %d)", 4 * kRmsThreads * kRmsPer, H);
    SX8_REQUIRE(peers->slot_elems >= (long)M * H, "sx8_glue_allreduce_add_rmsnorm: slot_elems (%ld) < M*H (%ld)",
                peers->slot_elems, (long)M * H);
    ArParams a;
    memset(&a, 0, sizeof(a));
    const long slot = (long)(peers->parity & 1) * peers->world * peers->slot_elems;
    for (int q = 0; q < peers->world; q++) {
        SX8_REQUIRE(peers->data[q] && peers->flags[q] && (reinterpret_cast<uintptr_t>(peers->data[q]) % 16) == 0 &&
                        (reinterpret_cast<uintptr_t>(peers->flags[q]) % 4) == 0,
                    "sx8_glue_allreduce_add_rmsnorm: null or misaligned peer pointer for rank %d", q);
        a.part[q] = (const float*)peers->data[q] + slot;
        a.flag_out[q] = (unsigned*)peers->flags[q] + 8 + peers->rank;
    }
    a.flag_in = (const unsigned*)peers->flags[peers->rank] + 8;
    a.ctr = (unsigned*)peers->flags[peers->rank] + 4;
    a.world = peers->world; a.rank = peers->rank;
    cudaError_t e = launch_pdl(allreduce_add_rmsnorm_kernel, dim3((unsigned)M), dim3(kRmsThreads), 0, (cudaStream_t)stream, a,
                               (float*)h, (const float*)gamma, H, eps, (__half*)x_out);
    if (e != cudaSuccess) return cuda_fail(e, "launch(allreduce_add_rmsnorm_kernel)");
    return SX8_OK;
}

extern "C" int sx8_glue_add_rmsnorm(void* h, const void* y, const void* gamma, int B, int H, float eps, void* x_out,
                                    void* stream) {
    SX8_REQUIRE(h && gamma && x_out, "sx8_glue_add_rmsnorm: null pointer");
    SX8_REQUIRE(B > 0 && H > 0 && (H % 4) == 0 && H <= 4 * kRmsThreads * kRmsPer,
                "sx8_glue_add_rmsnorm: need B>0 and H a multiple of 4 up to %d (got %d)", 4 * kRmsThreads * kRmsPer, H);
    cudaError_t e = launch_pdl(add_rmsnorm_kernel, dim3((unsigned)B), dim3(kRmsThreads), 0, (cudaStream_t)stream, (float*)h,
                               (const float*)y, (const float*)gamma, H, eps, (__half*)x_out);
    if (e != cudaSuccess) return cuda_fail(e, "launch(add_rmsnorm_kernel)");
    return SX8_OK;
}

extern "C" int sx8_glue_rope_cache(const void* q, const void* k, const void* v, const void* pos, const void* cos_t,
                                   const void* sin_t, int B, int hq, int hkv, int D, int S, void* q_out, void* k_cache,
                                   void* v_cache, void* stream) {
    SX8_REQUIRE(q && k && v && pos && cos_t && sin_t && q_out && k_cache && v_cache, "sx8_glue_rope_cache: null pointer");
    SX8_REQUIRE(B > 0 && hq > 0 && hkv > 0 && D > 0 && (D % 2) == 0 && S > 0, "sx8_glue_rope_cache: bad sizes");
    dim3 grid((unsigned)(hq + 2 * hkv), (unsigned)B, 1);
    cudaError_t e = launch_pdl(rope_cache_kernel, grid, dim3(64), 0, (cudaStream_t)stream, (const float*)q, (const float*)k,
                               (const float*)v, (const long*)pos, (const float*)cos_t, (const float*)sin_t, hq, hkv, D, S,
                               (__half*)q_out, (__half*)k_cache, (__half*)v_cache);
    if (e != cudaSuccess) return cuda_fail(e, "launch(rope_cache_kernel)");
    return SX8_OK;
}

extern "C" size_t sx8_glue_attn_scratch_bytes(int B, int hq, int hkv, int D) {
    if (B <= 0 || hq <= 0 || hkv <= 0 || D <= 0) return 0;
    // counters (one per sequence and kv head, rounded up to 256 bytes), then the partial results
    size_t cnt = (((size_t)B * hkv * sizeof(unsigned)) + 255) & ~(size_t)255;
    return cnt + (size_t)B * hkv * kAttnSplit * (size_t)(hq / hkv) * (D + 2) * sizeof(float);
}

extern "C" int sx8_glue_attn_decode(const void* q, const void* k_cache, const void* v_cache, const void* pos, int B, int hq,
                                    int hkv, int D, int S, float scale, void* out, void* scratch, size_t scratch_bytes,
                                    void* stream) {
    SX8_REQUIRE(q && k_cache && v_cache && pos && out && scratch, "sx8_glue_attn_decode: null pointer");
    SX8_REQUIRE(B > 0 && hkv > 0 && S > 0 && hq % hkv == 0, "sx8_glue_attn_decode: bad sizes");
    const int grp = hq / hkv;
    SX8_REQUIRE((D == 128 || D == 64) && (grp == 4 || grp == 2 || grp == 1 || grp == 8),
                "sx8_glue_attn_decode: supports head_dim 64 or 128 and 1, 2, 4 or 8 query heads per kv head (got %d, %d)", D, grp);
    SX8_REQUIRE(S <= 128 * kAttnSplit, "sx8_glue_attn_decode: cache length %d exceeds %d", S, 128 * kAttnSplit);
    SX8_REQUIRE(scratch_bytes >= sx8_glue_attn_scratch_bytes(B, hq, hkv, D) && (reinterpret_cast<uintptr_t>(scratch) % 16) == 0,
                "sx8_glue_attn_decode: scratch too small or misaligned (need %zu bytes)", sx8_glue_attn_scratch_bytes(B, hq, hkv, D));
    unsigned* counters = (unsigned*)scratch;
    float* part = (float*)((uint8_t*)scratch + ((((size_t)B * hkv * sizeof(unsigned)) + 255) & ~(size_t)255));
    dim3 grid((unsigned)hkv, (unsigned)B, (unsigned)kAttnSplit);
    cudaStream_t st = (cudaStream_t)stream;
#define SX8_ATTN(DD, GG)                                                                                              \
    do {                                                                                                              \
        cudaError_t e2 = launch_pdl(attn_decode_kernel<DD, GG>, grid, dim3(kAttnThreads), 0, st, (const __half*)q,    \
                                    (const __half*)k_cache, (const __half*)v_cache, (const long*)pos, hkv, S, scale,  \
                                    part, counters, (__half*)out);                                                    \
        if (e2 != cudaSuccess) return cuda_fail(e2, "launch(attn_decode_kernel)");                                    \
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
    return SX8_OK;
}

extern "C" int sx8_glue_silu_mul(const void* g, const void* u, long n, void* act_out, void* stream) {
    SX8_REQUIRE(g && u && act_out, "sx8_glue_silu_mul: null pointer");
    SX8_REQUIRE(n > 0 && (n + 255) / 256 <= 0x7FFFFFFFL, "sx8_glue_silu_mul: bad size %ld", n);
    cudaError_t e = launch_pdl(silu_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                               (const float*)g, (const float*)u, n, (__half*)act_out);
    if (e != cudaSuccess) return cuda_fail(e, "launch(silu_mul_kernel)");
    return SX8_OK;
}
