// sx8_gemv.cu -- S-X8 v4.3 decode GEMV for batch 1..8 on sm_100a (T16 device layout).
//
//   y[m, n] = sum_kb { base(kb,n) * D(kb,n,m) + lo(kb,n) * SxB(kb,m)
//                      + c0(kb,n) * Z0(kb,m) + c1(kb,n) * Z1(kb,m) }
//   D      = sum_t x[m, 32kb+t] * (mult_sb * level_t + 63 * off_sb)      (exact integers in fp16)
//   base   = (dmax - dmin) * 0.25 * 0.015873,   lo = dmin
//   (mult, off) = (4,0) (1,0) (1,3) (2,1) for range strategy 0..3 of sub-block sb
//   SxB    = sum of the 32 activations of the block,  Zj = scale_j * <x_block, basis_j>
//
// This is the reference's reformulated decode (ref cuda/sx8_decode1_v3.cu:7-13,
// :108-157: w = rlo + step*level, PCA as 2 multiply-adds per block) regrouped so that
// the per-weight work is bit extraction only: rlo = lo + off*q and step =
// mult*q*0.015873 with q = (dmax-dmin)/4, and off/0.015873 is taken as 63*off
// (relative deviation 1e-6 on that term; the step clamp at 1e-10 only acts on blocks
// with dmax == dmin, where it moves a weight by < 7e-9).  Products of small fp16
// integers and fp16 activations are exact in the tensor-core fp32 accumulation, so the
// result carries fp32-accumulate error only.
//
// One launch per GEMV.  A producer warp streams, per pipeline stage, one contiguous
// [kb-range x 480 B] slab per 16-column tile of the T16 blob plus the matching slice of
// every activation row into shared memory with TMA bulk copies (one copy per lane)
// behind an mbarrier ring; weights are requested before, activations after the
// programmatic-dependent-launch wait.  Eight consumer warps first build the small table
// of activation-side operands (SxB and Z, split into fp16 hi/lo) for the CTA's kb range,
// then decode levels with byte-parallel masks and feed mma.sync m16n8k16 with the <= 8
// activation rows as the n = 8 operand, so batch 1..8 cost the same.  Split-K across a
// thread-block cluster is reduced through distributed shared memory in rank order
// (deterministic).
#include <stdlib.h>

#include "sx8_common.cuh"
#include "sx8_layout.cuh"
#include "../../include/sx8_b200_test.h"

#define SX8_MAX_PEERS 8

namespace sx8 {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr uint32_t kSpinLimit = 1u << 22;
// Per-CTA activation table: 16 bytes per (block row, batch row): [t = 0,1] x {lo-term word,
// coefficient-term word}; a block row takes 16*M bytes.  32 KB of table keep three CTAs per SM,
// so a CTA can cover 256 block rows at batch 8 and 1024 at batch 1 or 2 (a lane group of the
// main loop that belongs to a batch row >= M reads past its block row's entries; the table is
// padded by 128 bytes for the last one, and those lanes' results are never stored).
constexpr int kTableBytes = 32768;
__host__ __device__ inline int table_stride(int M) { return 16 * M; }
inline int max_kb_per_cta(int M) {
    int v = kTableBytes / table_stride(M);
    return v > 1024 ? 1024 : v;
}

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One wait attempt.  The thread is suspended by the hardware until the phase completes or the
// time hint (ns) runs out, so a waiting warp does not burn issue slots polling: the producer
// warp waits for an empty stage most of the time and shares its scheduler with two consumer
// warps (measured on 151936 x 2560: the polling loops were ~25 of 108 instructions per
// 512-weight unit).
constexpr uint32_t kWaitHintNs = 100000u;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    return ok != 0;
}
// Non-blocking probe of a phase.  A wait costs a shared-memory round trip even when the
// phase completed long ago, so the consumers probe the NEXT stage's barrier before they start
// on the current stage and read the answer afterwards.
__device__ __forceinline__ uint32_t mbar_probe(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait: gives up after kSpinLimit attempts or about two seconds, whichever comes first,
// records the failure in the device error word and returns false; the caller then stops
// waiting for the rest of the kernel.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned code) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint32_t i = 0; i < kSpinLimit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 15u) {
            unsigned long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > 2000000000ull) break;
        }
    }
    atomicOr(&g_sx8_error_flag, code);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// d = A * B (accumulator input zero: no registers to clear)
__device__ __forceinline__ void mma16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t local_addr, uint32_t rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(ra));
    return v;
}
__device__ __forceinline__ void consumer_bar() {  // the 8 consumer warps only
    asm volatile("bar.sync 1, 256;" ::: "memory");
}

// fp32 -> (hi, lo) fp16 pair: hi + lo == v to ~22 bits.
__device__ __forceinline__ void split_hilo(float v, uint32_t& hi, uint32_t& lo) {
    __half h = __float2half_rn(v);
    __half l = __float2half_rn(v - __half2float(h));
    hi = __half_as_ushort(h);
    lo = __half_as_ushort(l);
}

// ------------------------------------------------------------------ x staging
// Copies x (M, K) with row stride ldx into a dense, zero-padded (M, Kp) buffer
// (Kp = 32*n_cb) when the rows cannot be fetched by 16-byte bulk copies as they are.
__global__ void __launch_bounds__(256)
xpad_kernel(const __half* __restrict__ x, int M, int K, long ldx, int Kp, __half* __restrict__ out) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    long i = (long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long)M * Kp) return;
    int m = (int)(i / Kp), k = (int)(i - (long)m * Kp);
    out[i] = (k < K) ? x[(long)m * ldx + k] : __float2half_rn(0.0f);
}

// ------------------------------------------------------------------ main kernel
// One packed matrix of a launch.  A launch may carry up to four matrices that share the
// activations (q|k|v, gate|up): tile groups are numbered through all of them, matrix i owning
// groups [group0, group0 + ceil(n_tiles / NT)).
struct SegDesc {
    const uint8_t* blob;   // T16
    const float* bases;
    const float* scales;
    float* y;
    int N, n_tiles, group0;
};
constexpr int kMaxSeg = 4;

struct GemvParams {
    SegDesc seg[kMaxSeg];
    const __half* x;       // (M, >= 32*n_cb), rows 16-byte aligned
    long ldx;
    int nseg, n_cb, M, split, groups;
    const uint8_t* table;  // batches above 8 rows: the activation tables in global scratch, (n_cb, M, 16 B) per matrix
    // Row-parallel exchange (world > 1): instead of y, every finished tile is stored into slot
    // `rank` of each peer's receive buffer (peer memory, plain stores over NVLink), then a
    // per-peer arrival counter is bumped; reduce_peers_kernel sums the slots.
    float* peer_data[SX8_MAX_PEERS];       // base of each rank's receive buffer (this parity)
    unsigned* peer_flag[SX8_MAX_PEERS];    // each rank's arrival counter (this parity)
    long slot_elems;                       // elements per slot
    int rank, world;
};

// Stores one finished value, locally or into every peer's slot.
__device__ __forceinline__ void put_out(const GemvParams& p, float* y, long idx, float v) {
    if (p.world <= 1) {
        y[idx] = v;
    } else {
#pragma unroll 1
        for (int q = 0; q < p.world; q++) p.peer_data[q][(long)p.rank * p.slot_elems + idx] = v;
    }
}
// After a warp has stored a whole tile: make the stores visible system-wide, then count the
// tile on every peer (lane q signals peer q).
__device__ __forceinline__ void signal_tile(const GemvParams& p, int lane) {
    if (p.world <= 1) return;
    __threadfence_system();
    __syncwarp();
    if (lane < p.world) atomicAdd_system(p.peer_flag[lane], 1u);
}

// Activation-side operands of one (block row kb, batch row m): 16 bytes, two 8-byte entries
// read by lanes t = 0 and t = 1 of the main loop:
//   entry t=0: { {SxB_hi, 0}, {Z0_hi, Z1_hi} }    entry t=1: { {SxB_lo, 0}, {Z0_lo, Z1_lo} }
// The first word multiplies the {dmin, dmax} pair of a column (the zero half cancels dmax), the
// second the {c0, c1} * 2^-10 pair; Zj (ref cuda/sx8_decode1_v3.cu:44-65) is pre-multiplied by
// 1024.  The four lanes t = 0..3 of a lane group compute one item from 8 activations each.
__device__ __forceinline__ void act_item(const uint4 raw, const float4 (&bq)[4], float s0, float s1, int t,
                                         uint32_t& w0, uint32_t& w1) {
    const __half* hh = reinterpret_cast<const __half*>(&raw);
    const float bb0[8] = {bq[0].x, bq[0].y, bq[0].z, bq[0].w, bq[1].x, bq[1].y, bq[1].z, bq[1].w};
    const float bb1[8] = {bq[2].x, bq[2].y, bq[2].z, bq[2].w, bq[3].x, bq[3].y, bq[3].z, bq[3].w};
    float sx = 0.f, z0 = 0.f, z1 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float xv = __half2float(hh[i]);
        sx += xv;
        z0 = fmaf(xv, bb0[i], z0);
        z1 = fmaf(xv, bb1[i], z1);
    }
#pragma unroll
    for (int off = 1; off <= 2; off <<= 1) {
        sx += __shfl_xor_sync(0xFFFFFFFFu, sx, off);
        z0 += __shfl_xor_sync(0xFFFFFFFFu, z0, off);
        z1 += __shfl_xor_sync(0xFFFFFFFFu, z1, off);
    }
    z0 = s0 * z0 * 1024.0f;
    z1 = s1 * z1 * 1024.0f;
    uint32_t sh, sl, z0h, z0l, z1h, z1l;
    split_hilo(sx, sh, sl);
    split_hilo(z0, z0h, z0l);
    split_hilo(z1, z1h, z1l);
    w0 = (t == 0) ? sh : sl;
    w1 = (t == 0) ? (z0h | (z1h << 16)) : (z0l | (z1l << 16));
}

// The table for batches above 8 rows, built once per launch into global scratch (n_cb, M, 16 B)
// instead of once per CTA into shared memory: the main kernel's producer then brings each
// stage's slice in with one bulk copy, and a CTA's K range is not limited by table space.
struct ActTableArgs {
    const float* bases[kMaxSeg];
    const float* scales[kMaxSeg];
};
// grid (ceil(n_cb * M / 64), matrices): the table of matrix i starts at table + i * n_cb * M * 2.
__global__ void __launch_bounds__(256)
act_table_kernel(const __half* __restrict__ x, long ldx, int M, int n_cb, ActTableArgs a, uint2* __restrict__ table) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float* __restrict__ bases = a.bases[blockIdx.y];
    const float* __restrict__ scales = a.scales[blockIdx.y];
    table += (long)blockIdx.y * n_cb * M * 2;
    const int t = threadIdx.x & 3;
    const long n_items = (long)n_cb * M;
    long item = (long)blockIdx.x * 64 + (threadIdx.x >> 2);
    const bool valid = item < n_items;
    if (!valid) item = n_items - 1;
    const int kb = (int)(item / M), m = (int)(item - (long)kb * M);
    float4 bq[4];
    const float4* b0p = reinterpret_cast<const float4*>(bases + (long)kb * 64 + t * 8);
    const float4* b1p = reinterpret_cast<const float4*>(bases + (long)kb * 64 + 32 + t * 8);
    bq[0] = b0p[0]; bq[1] = b0p[1]; bq[2] = b1p[0]; bq[3] = b1p[1];
    uint4 raw = *reinterpret_cast<const uint4*>(x + (long)m * ldx + (long)kb * 32 + t * 8);
    uint32_t w0, w1;
    act_item(raw, bq, scales[kb * 2], scales[kb * 2 + 1], t, w0, w1);
    if (t < 2 && valid) table[item * 2 + t] = make_uint2(w0, w1);
}

// MB = batch rows in blocks of 8 (1 or 2): a decoded weight fragment feeds MB activation
// blocks, so the decode cost per weight is paid once for up to 16 rows.
template <int NT, int KB_S, int STAGES, int MB>
struct GemvCfg {
    static constexpr int KS = kConsumerWarps / NT;        // warps sharing a tile split the kb rows
    static constexpr int XROW = KB_S * 64 + 64;           // padded: conflict-free 128-bit x reads
    static constexpr int OFF_X = NT * KB_S * T16_UNIT;
    static constexpr int OFF_T = OFF_X + 8 * MB * XROW;   // MB > 1: this stage's slice of the global table
    static constexpr int STAGE = OFF_T + (MB > 1 ? KB_S * 8 * MB * 16 : 0);
    static constexpr int RED_BYTES = kConsumerWarps * 32 * 16 * MB;
    static constexpr int FIXED = STAGES * STAGE + RED_BYTES + 2 * STAGES * 8 + 16 + 16;
    // MB == 1: the CTA's own table (kb_per_cta rows) follows, padded for the lanes of rows >= M
    static int smem_bytes(int kb_per_cta, int M) { return FIXED + (MB > 1 ? 0 : kb_per_cta * table_stride(M) + 128); }
};

template <int NT, int KB_S, int STAGES, int MINB, int MB>
__global__ void __launch_bounds__(kThreads, MINB) gemv_kernel(GemvParams p) {
    using C = GemvCfg<NT, KB_S, STAGES, MB>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t red = sbase + STAGES * C::STAGE;
    const uint32_t bar_full = red + C::RED_BYTES;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t zslot = bar_empty + STAGES * 8 + 16;   // 16 zero bytes: table operand of lanes t >= 2
    const uint32_t dtab = zslot + 16;
    const int dt_kb = table_stride(p.M);

    asm volatile("griddepcontrol.launch_dependents;");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = blockIdx.y;
    const int kb_per = (p.n_cb + p.split - 1) / p.split;
    const int kb_begin = min(p.n_cb, rank * kb_per);
    const int kb_end = min(p.n_cb, kb_begin + kb_per);
    const int n_iter = (kb_end - kb_begin + KB_S - 1) / KB_S;
    const int my_groups = ((int)blockIdx.x < p.groups) ? (p.groups - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int total_iters = my_groups * n_iter;
    constexpr bool kDirectStore = (C::KS == 1);   // with split == 1 a warp owns its tile for all of K
    // the matrix this CTA works on (launches with several matrices give each CTA one tile group)
    int si = 0;
    for (int i = 1; i < p.nseg; i++)
        if ((int)blockIdx.x >= p.seg[i].group0) si = i;
    const SegDesc sg = p.seg[si];

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, kConsumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        sts32(zslot, 0u); sts32(zslot + 4, 0u); sts32(zslot + 8, 0u); sts32(zslot + 12, 0u);
    }
    __syncthreads();

    float accF[MB][4], accD[MB][4];
#pragma unroll
    for (int nb = 0; nb < MB; nb++)
#pragma unroll
        for (int i = 0; i < 4; i++) accF[nb][i] = accD[nb][i] = 0.f;
    const float kBase = 0.25f * 0.015873f * 16384.0f;   // q = (dmax-dmin)/4, step unit 0.015873, operands scaled by 2^-14

    if (warp == kConsumerWarps) {
        // ---------------------------------------------- producer warp: lane i < NT copies the
        // slab of tile i, lane m < M the slice of activation row m, lane 31 the table slice.
        // Stage coordinates advance incrementally (tile group, K step): no divisions in the loop.
        struct Pos { int grp, j, s; uint32_t ph; };
        auto advance = [&](Pos& q) {
            if (++q.j == n_iter) { q.j = 0; q.grp += (int)gridDim.x; }
            if (++q.s == STAGES) { q.s = 0; q.ph ^= 1u; }
        };
        auto issue = [&](const Pos& q, bool with_w, bool with_x) {
            const int kb0 = kb_begin + q.j * KB_S;
            const int rows = min(KB_S, kb_end - kb0);
            const uint32_t stage = sbase + q.s * C::STAGE, bar = bar_full + 8 * q.s;
            if (with_w) {
                if (lane == 0) {
                    int tiles = min(NT, sg.n_tiles - q.grp * NT);
                    mbar_expect_tx(bar, (uint32_t)rows * ((uint32_t)tiles * T16_UNIT + (uint32_t)p.M * (MB > 1 ? 80u : 64u)));
                }
                __syncwarp();
                long T = (long)q.grp * NT + lane;
                if (lane < NT && T < sg.n_tiles)
                    bulk_g2s(stage + lane * (KB_S * T16_UNIT), sg.blob + (T * p.n_cb + kb0) * T16_UNIT,
                             (uint32_t)rows * T16_UNIT, bar);
            }
            if (with_x) {
                if (lane < p.M)
                    bulk_g2s(stage + C::OFF_X + lane * C::XROW, p.x + (long)lane * p.ldx + (long)kb0 * 32,
                             (uint32_t)rows * 64u, bar);
                if (MB > 1 && lane == 31)
                    bulk_g2s(stage + C::OFF_T, p.table + ((long)si * p.n_cb + kb0) * dt_kb, (uint32_t)(rows * dt_kb), bar);
            }
        };
        bool ok = true;
        // Weights do not depend on the preceding kernel: request them before waiting
        // for it (programmatic dependent launch); activations (and their table) after.
        const int pre = min(total_iters, STAGES);
        Pos q{(int)blockIdx.x - sg.group0, 0, 0, 0u};
        Pos q0 = q;
        for (int it = 0; it < pre; it++) { issue(q, true, false); advance(q); }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int it = 0; it < pre; it++) { issue(q0, false, true); advance(q0); }
        // q.ph is the parity of the fill about to be issued; the consumers' release of the
        // previous fill of the same stage completed phase (q.ph ^ 1) of its empty barrier
        for (int it = pre; it < total_iters; it++) {
            if (ok) ok = mbar_wait(bar_empty + 8 * q.s, q.ph ^ 1u, 1u);
            issue(q, true, true);
            advance(q);
        }
    } else {
        // ---------------------------------------------- consumers
        const int ti = warp % NT, kpart = warp / NT;
        const int g = lane >> 2, t = lane & 3;
        if (MB == 1) {
            // ---- the CTA's own activation table for kb_begin..kb_end (act_item).  A work item is
            // (block row kb, batch row m); a warp takes 2 x 8 items per pass, the CTA 128: at batch
            // 1 that is 128 block rows per pass, so even a CTA with a long K range builds its table
            // in one round of loads.  PCA bases and scales are weights: those of the first pass are
            // fetched before waiting for the preceding kernel, like the producer's weight copies.
            const int n_items = (kb_end - kb_begin) * p.M;
            constexpr int kPass = 16 * kConsumerWarps;
            float4 bq[2][4];
            float sc[2][2];
            int ikb[2], im[2];
            auto locate = [&](int i0) {
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    int item = min(i0 + u * (kPass / 2) + warp * 8 + g, max(n_items - 1, 0));
                    int q = item / p.M;
                    ikb[u] = kb_begin + q;
                    im[u] = item - q * p.M;
                }
            };
            auto load_bases = [&]() {
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const int kb = ikb[u];
                    const float4* b0p = reinterpret_cast<const float4*>(sg.bases + (long)kb * 64 + t * 8);
                    const float4* b1p = reinterpret_cast<const float4*>(sg.bases + (long)kb * 64 + 32 + t * 8);
                    bq[u][0] = b0p[0]; bq[u][1] = b0p[1]; bq[u][2] = b1p[0]; bq[u][3] = b1p[1];
                    sc[u][0] = sg.scales[kb * 2 + 0];
                    sc[u][1] = sg.scales[kb * 2 + 1];
                }
            };
            if (n_items > 0) {
                locate(0);
                load_bases();
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i0 = 0; i0 < n_items; i0 += kPass) {
                uint4 raw[2];
                if (i0 > 0) {
                    locate(i0);
                    load_bases();
                }
#pragma unroll
                for (int u = 0; u < 2; u++)
                    raw[u] = *reinterpret_cast<const uint4*>(p.x + (long)im[u] * p.ldx + (long)ikb[u] * 32 + t * 8);
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const bool valid = i0 + u * (kPass / 2) + warp * 8 + g < n_items;
                    uint32_t w0, w1;
                    act_item(raw[u], bq[u], sc[u][0], sc[u][1], t, w0, w1);
                    if (t < 2 && valid) {
                        uint32_t a = dtab + (ikb[u] - kb_begin) * dt_kb + im[u] * 16 + t * 8;
                        sts32(a, w0);
                        sts32(a + 4, w1);
                    }
                }
            }
            consumer_bar();
        } else {
            asm volatile("griddepcontrol.wait;" ::: "memory");
        }

        const uint32_t sh2 = 8u + 2u * (uint32_t)t;
        // Shared-memory operand addresses of this lane.  Rows beyond M read the last row (their
        // results are never stored); lanes t >= 2 read the zero slot instead of the table (stride 0).
        uint32_t xoff[MB];
#pragma unroll
        for (int nb = 0; nb < MB; nb++) xoff[nb] = (uint32_t)(min(nb * 8 + g, p.M - 1) * C::XROW + t * 16);
        const uint32_t tstride = (t < 2) ? (uint32_t)dt_kb : 0u;        // per block row
        const uint32_t tnb = (t < 2) ? 128u : 0u;                       // per block of 8 batch rows
        const uint32_t tlane = (t < 2) ? (uint32_t)(g * 16 + t * 8) : 0u;

        // One (16-column tile, block row) unit: 512 weights of this warp.
        //   unit: the 480-byte T16 unit; xa: this block row in the activation rows; ta: its table row
        auto unit_body = [&](const uint32_t unit, const uint32_t xa, const uint32_t ta) {
            uint32_t W0 = lds32(unit + lane * 4), W1 = lds32(unit + 128 + lane * 4), W2 = lds32(unit + 256 + lane * 4);
            uint32_t H0 = lds32(unit + 384 + g * 4), H1 = lds32(unit + 416 + g * 4), H2 = lds32(unit + 448 + g * 4);
            // per sub-block constants looked up by range strategy:
            //   mult * 2^8  = 1024, 256, 256, 512     63*off * 2^-14 = 0, 0, 189*2^-14, 63*2^-14
            uint32_t u = (H2 >> sh2) & 0x00030003u;
            uint32_t sel = u * 0x2222u + 0x10101010u;
            uint32_t selB = sel >> 16;
            uint32_t mA = __byte_perm(0x5C006400u, 0x60005C00u, sel);
            uint32_t aA = __byte_perm(0x00000000u, 0x1BE021E8u, sel);
            uint32_t mB = __byte_perm(0x5C006400u, 0x60005C00u, selB);
            uint32_t aB = __byte_perm(0x00000000u, 0x1BE021E8u, selB);
            // bytes hold level << 2; read as fp16 bit patterns they are level * 2^-22, so
            // fma gives (mult*level + 63*off) * 2^-14, exact
            uint32_t V3 = ((W0 << 2) & 0x0C0C0C0Cu) | ((W1 << 4) & 0x30303030u) | ((W2 << 6) & 0xC0C0C0C0u);
            uint32_t fa0 = hfma2_u32(W0 & 0x00FC00FCu, mA, aA);
            uint32_t fa1 = hfma2_u32((W0 >> 8) & 0x00FC00FCu, mA, aA);
            uint32_t fa2 = hfma2_u32(W1 & 0x00FC00FCu, mA, aA);
            uint32_t fa3 = hfma2_u32((W1 >> 8) & 0x00FC00FCu, mA, aA);
            uint32_t fb0 = hfma2_u32(W2 & 0x00FC00FCu, mB, aB);
            uint32_t fb1 = hfma2_u32((W2 >> 8) & 0x00FC00FCu, mB, aB);
            uint32_t fb2 = hfma2_u32(V3 & 0x00FF00FFu, mB, aB);
            uint32_t fb3 = hfma2_u32((V3 >> 8) & 0x00FF00FFu, mB, aB);
            // Signed 4-bit coefficient n -> fp16 n * 2^-10: (n ^ 8) under the exponent of 1024
            // (column A, nibble at mantissa bits 0..3) or (column B, bits 4..7: 1024 + 16 (n ^ 8)).
            uint32_t ccA = hfma2_u32((H2 & 0x000F000Fu) ^ 0x64086408u, 0x14001400u, 0xBC08BC08u);
            uint32_t ccB = hfma2_u32((H2 & 0x00F000F0u) ^ 0x64806480u, 0x04000400u, 0xAC80AC80u);
            // (dmax - dmin) per column; the constant 0.25 * 0.015873 * 2^14 is applied once, at the end
            float2 eA = __half22float2(*reinterpret_cast<const __half2*>(&H0));
            float2 eB = __half22float2(*reinterpret_cast<const __half2*>(&H1));
            const float baseA = eA.y - eA.x, baseB = eB.y - eB.x;
#pragma unroll
            for (int nb = 0; nb < MB; nb++) {
                uint4 xq = lds128(xa + xoff[nb]);
                uint32_t dv0, dv1;
                asm("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(dv0), "=r"(dv1) : "r"(ta + nb * tnb) : "memory");
                float d[4];
                mma16816_z(d, fa0, fb0, fa1, fb1, xq.x, xq.y);
                mma16816(d, fa2, fb2, fa3, fb3, xq.z, xq.w);
                // direct terms: {dmin,dmax} x {SxB_hi|lo, 0} and {c0,c1} * 2^-10 x 1024*Z; lanes
                // t = 0,1 carry the hi and lo halves of the activation sums, lanes 2,3 zeros
                mma1688(accD[nb], H0, H1, dv0);
                mma1688(accD[nb], ccA, ccB, dv1);
                accF[nb][0] = fmaf(baseA, d[0], accF[nb][0]);
                accF[nb][1] = fmaf(baseA, d[1], accF[nb][1]);
                accF[nb][2] = fmaf(baseB, d[2], accF[nb][2]);
                accF[nb][3] = fmaf(baseB, d[3], accF[nb][3]);
            }
        };
        constexpr int kRowsPerWarp = KB_S / C::KS;
        const uint32_t unit0 = sbase + (ti * KB_S + kpart) * T16_UNIT;
        const uint32_t x0 = sbase + C::OFF_X + kpart * 64;
        // MB == 1: the CTA's table, indexed by block row within the K range; MB > 1: the stage's slice
        const uint32_t tab0 = (t < 2) ? ((MB > 1 ? sbase + C::OFF_T : dtab) + kpart * (uint32_t)dt_kb + tlane) : zslot;
        bool ok = true;
        int s = 0;            // stage of this iteration and the parity of its current fill
        uint32_t ph = 0u;
        uint32_t pre = 0;   // answer of the early probe of this iteration's barrier
        for (int gi = 0; gi < my_groups; gi++) {
            const int grp = (int)blockIdx.x + gi * (int)gridDim.x - sg.group0;
            for (int j = 0; j < n_iter; j++) {
                if (!pre && ok) ok = mbar_wait(bar_full + 8 * s, ph, 2u);
                int s1 = s + 1;
                uint32_t ph1 = ph;
                if (s1 == STAGES) { s1 = 0; ph1 ^= 1u; }
                pre = mbar_probe(bar_full + 8 * s1, ph1);
                const int rows = min(KB_S, kb_end - (kb_begin + j * KB_S));
                const uint32_t so = (uint32_t)(s * C::STAGE);
                const uint32_t tj = tab0 + (MB > 1 ? ((t < 2) ? so : 0u) : (uint32_t)(j * KB_S) * tstride);
                if (rows == KB_S) {   // full stage: no per-row checks
#pragma unroll
                    for (int ri = 0; ri < kRowsPerWarp; ri++)
                        unit_body(unit0 + so + ri * C::KS * T16_UNIT, x0 + so + ri * C::KS * 64,
                                  tj + (uint32_t)(ri * C::KS) * tstride);
                } else {
#pragma unroll 1
                    for (int ri = 0; ri < kRowsPerWarp; ri++) {
                        if (kpart + ri * C::KS >= rows) break;
                        unit_body(unit0 + so + ri * C::KS * T16_UNIT, x0 + so + ri * C::KS * 64,
                                  tj + (uint32_t)(ri * C::KS) * tstride);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty + 8 * s);
                s = s1;
                ph = ph1;
            }
            if (kDirectStore && p.split == 1) {
                const int nA = (grp * NT + ti) * 16 + g, nB = nA + 8;
#pragma unroll
                for (int nb = 0; nb < MB; nb++) {
                    const int m0 = nb * 8 + 2 * t, m1 = m0 + 1;
                    float v0 = fmaf(accF[nb][0], kBase, accD[nb][0]), v1 = fmaf(accF[nb][1], kBase, accD[nb][1]),
                          v2 = fmaf(accF[nb][2], kBase, accD[nb][2]), v3 = fmaf(accF[nb][3], kBase, accD[nb][3]);
                    if (nA < sg.N) {
                        if (m0 < p.M) put_out(p, sg.y, (long)m0 * sg.N + nA, v0);
                        if (m1 < p.M) put_out(p, sg.y, (long)m1 * sg.N + nA, v1);
                    }
                    if (nB < sg.N) {
                        if (m0 < p.M) put_out(p, sg.y, (long)m0 * sg.N + nB, v2);
                        if (m1 < p.M) put_out(p, sg.y, (long)m1 * sg.N + nB, v3);
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) accF[nb][i] = accD[nb][i] = 0.f;
                }
                if (grp * NT + ti < sg.n_tiles) signal_tile(p, lane);
            }
        }
        if (!(kDirectStore && p.split == 1)) {
#pragma unroll
            for (int nb = 0; nb < MB; nb++)
                asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(red + ((nb * kConsumerWarps + warp) * 32 + lane) * 16),
                             "f"(fmaf(accF[nb][0], kBase, accD[nb][0])), "f"(fmaf(accF[nb][1], kBase, accD[nb][1])),
                             "f"(fmaf(accF[nb][2], kBase, accD[nb][2])), "f"(fmaf(accF[nb][3], kBase, accD[nb][3]))
                             : "memory");
        }
    }
    if (kDirectStore && p.split == 1) return;   // uniform over the whole grid
    __syncthreads();

    // ---- reduce the KS kb-parts of each tile, in fixed order, into slot kpart 0
    if (warp < NT) {
#pragma unroll
        for (int nb = 0; nb < MB; nb++) {
            uint32_t a = red + ((nb * kConsumerWarps + warp) * 32 + lane) * 16;
            float4 v;
            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
            for (int k = 1; k < C::KS; k++) {
                float4 u;
                asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                             : "=f"(u.x), "=f"(u.y), "=f"(u.z), "=f"(u.w)
                             : "r"(a + k * NT * 32 * 16));
                v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
            }
            accF[nb][0] = v.x; accF[nb][1] = v.y; accF[nb][2] = v.z; accF[nb][3] = v.w;
            if (p.split > 1)
                asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
        }
    }
    if (p.split > 1) {
        cluster_sync_all();
        if (rank == 0 && warp < NT) {
#pragma unroll
            for (int nb = 0; nb < MB; nb++) {
                uint32_t a = red + ((nb * kConsumerWarps + warp) * 32 + lane) * 16;
                // all remote loads first (a load from a peer's shared memory takes several hundred
                // nanoseconds: one after the other they were the longest phase of a small GEMV), then the
                // sum in rank order
                float4 u[7];
#pragma unroll
                for (int rk = 1; rk < 8; rk++)
                    if (rk < p.split) u[rk - 1] = ld_cluster_f4(a, (uint32_t)rk);
#pragma unroll
                for (int rk = 1; rk < 8; rk++)
                    if (rk < p.split) {
                        accF[nb][0] += u[rk - 1].x; accF[nb][1] += u[rk - 1].y;
                        accF[nb][2] += u[rk - 1].z; accF[nb][3] += u[rk - 1].w;
                    }
            }
        }
        cluster_sync_all();  // peers keep their shared memory alive until rank 0 has read it
    }
    if (rank == 0 && warp < NT && (int)blockIdx.x < p.groups) {
        const int g = lane >> 2, t = lane & 3;
        const int tl = ((int)blockIdx.x - sg.group0) * NT + warp;   // tile within this CTA's matrix
        const int nA = tl * 16 + g, nB = nA + 8;
#pragma unroll
        for (int nb = 0; nb < MB; nb++) {
            const int m0 = nb * 8 + 2 * t, m1 = m0 + 1;
            if (nA < sg.N) {
                if (m0 < p.M) put_out(p, sg.y, (long)m0 * sg.N + nA, accF[nb][0]);
                if (m1 < p.M) put_out(p, sg.y, (long)m1 * sg.N + nA, accF[nb][1]);
            }
            if (nB < sg.N) {
                if (m0 < p.M) put_out(p, sg.y, (long)m0 * sg.N + nB, accF[nb][2]);
                if (m1 < p.M) put_out(p, sg.y, (long)m1 * sg.N + nB, accF[nb][3]);
            }
        }
        if (tl < sg.n_tiles) signal_tile(p, lane);
    }
}

// Second half of the row-parallel exchange: waits (bounded) until every rank has delivered all
// of its tiles into this rank's slots, then sums the slots in rank order -- deterministic --
// into y.  The last CTA to finish re-arms the arrival counter for the call after next (the
// buffers alternate between two parities, and no rank can run two calls ahead of a peer).
__global__ void __launch_bounds__(256)
reduce_peers_kernel(const float* __restrict__ slots, unsigned* flag, unsigned* done, float* __restrict__ y,
                    long n_elems, long slot_elems, int world, unsigned expected) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // this rank's own GEMV has finished
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        int ok = 0;
        for (uint32_t i = 0; i < (1u << 24); i++) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v >= expected) { ok = 1; break; }
        }
        if (!ok) atomicOr(&g_sx8_error_flag, 4u);
        s_ok = ok;
    }
    __syncthreads();
    for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < n_elems; i += (long)gridDim.x * 256) {
        float acc = 0.f;
        for (int r = 0; r < world; r++) acc += __ldcv(slots + (long)r * slot_elems + i);
        y[i] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        unsigned prev = atomicAdd(done, 1u);
        if (prev == gridDim.x - 1) {
            *done = 0u;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(0u) : "memory");
        }
    }
}

}  // namespace sx8

// =================================================================== host side
using namespace sx8;

namespace {

constexpr int kSMs = 148;

struct Choice {
    int nt, split, grid_x;
};

int g_tune_nt = -1, g_tune_split = -1, g_tune_grid = -1;   // -1: take the environment / automatic choice


// The three instantiations of the decode GEMV (NT tiles per group: KB_S block rows per stage,
// stages): wide groups take fewer, larger stages -- eight units per warp and stage instead of
// four halve the per-stage bookkeeping, and at batch 8 eight tiles share each activation slice.
using Cfg8 = GemvCfg<8, 8, 2, 1>;
using Cfg4 = GemvCfg<4, 8, 3, 1>;
using Cfg2 = GemvCfg<2, 8, 4, 1>;

// Tile-group width NT (x16 columns), cluster split-K and grid size: a score over the candidates
// whose constants were fitted to a sweep on B200 of every (NT, split) over the Qwen3-4B- and
// Llama-70B-shaped projections and their 2/4/8-way tensor-parallel shards (29 shapes, batch 1
// and 8; mean distance of the chosen shape from the best measured one 2.4 %).  It aims at 80 % of
// the CTAs that can be resident at once (shared memory decides: three per SM, two when the
// activation table of a batch-8 launch is large -- fewer than all leave room for the next
// launch's prefetching CTAs), prefers wide tile groups, few waves, little split-K and at least 16
// block rows per CTA.  Very large N runs without split-K on eight-tile groups and a persistent
// grid (151936 x 2560 at batch 1: 88 us against 93 us with four-tile groups on a plain grid),
// except with a long K at batch <= 4, where the four-tile groups are level or ahead.
Choice choose(int N, int n_cb, int M) {
    static const int e_nt = exp_env("SX8_GEMV_NT", 0), e_split = exp_env("SX8_GEMV_SPLIT", 0),
                     e_grid = exp_env("SX8_GEMV_GRID", 0);
    const int f_nt = g_tune_nt >= 0 ? g_tune_nt : e_nt, f_split = g_tune_split >= 0 ? g_tune_split : e_split,
              f_grid = g_tune_grid >= 0 ? g_tune_grid : e_grid;   // test hook (sx8_b200_test.h), else automatic
    const int n_tiles = (int)t16_tiles(N);
    const int min_split = (n_cb + max_kb_per_cta(M) - 1) / max_kb_per_cta(M);
    constexpr int kSmemPerSM = 228 * 1024, kSmemReserved = 1024;   // per SM, per resident CTA
    Choice best{8, min_split, 0};
    double best_score = -1e30;
    const int nts[3] = {8, 4, 2};
    const double nt_pen[3] = {0.0, 0.02, 0.1};
    for (int a = 0; a < 3; a++) {
        int nt = nts[a];
        if (f_nt && nt != f_nt) continue;
        int groups = (n_tiles + nt - 1) / nt;
        for (int split = min_split; split <= 8; split++) {
            if (f_split && split != f_split) continue;
            if (split > min_split && n_cb / split < 4) break;
            const int kb_per = (n_cb + split - 1) / split;
            long ctas = (long)groups * split;
            double score;
            if (split == 1 && (n_tiles + 7) / 8 >= 6 * kSMs) {
                const int want = (M <= 4 && n_cb > 128) ? 4 : 8;
                score = (nt == want) ? 1.0 : 0.9;
            } else {
                const int smem = nt == 8 ? Cfg8::smem_bytes(kb_per, M) : nt == 4 ? Cfg4::smem_bytes(kb_per, M) : Cfg2::smem_bytes(kb_per, M);
                int resident = kSmemPerSM / (smem + kSmemReserved);
                resident = resident > 3 ? 3 : (resident < 1 ? 1 : resident);   // 72 registers x 288 threads: three at most
                const double target = 0.8 * resident * kSMs;
                long waves = (ctas + resident * kSMs - 1) / (resident * kSMs);
                double per_wave = (double)ctas / (double)waves;
                double dev = per_wave > target ? (per_wave - target) / target : (target - per_wave) / target;
                if (ctas < kSMs) dev = 2.0 - (double)ctas / kSMs;   // fewer CTAs than SMs: parallelism first
                score = -(dev + 0.05 * (double)(waves - 1) + nt_pen[a] + 0.01 * split + 0.005 * (kb_per < 16 ? 16 - kb_per : 0));
            }
            if (score > best_score) {
                best_score = score;
                best = Choice{nt, split, 0};
            }
        }
    }
    int groups = (n_tiles + best.nt - 1) / best.nt;
    best.grid_x = groups;
    static const int verbose = exp_env("SX8_GEMV_VERBOSE", 0);
    if (verbose) fprintf(stderr, "sx8 gemv launch shape: N=%d n_cb=%d M=%d -> nt=%d split=%d groups=%d\n", N, n_cb, M, best.nt, best.split, groups);
    if (best.split == 1) {   // persistent grid: eight-tile groups by default, others on request
        int cap = f_grid > 0 ? f_grid : (best.nt == 8 ? 3 * kSMs : 0);
        if (cap > 0 && groups > cap) {   // equal number of tile groups per CTA
            int per = (groups + cap - 1) / cap;
            best.grid_x = (groups + per - 1) / per;
        }
    }
    return best;
}

template <int NT, int KB_S, int STAGES, int MINB = 3, int MB = 1>
int launch_gemv(const GemvParams& p, int grid_x, unsigned flags, cudaStream_t stream) {
    using C = GemvCfg<NT, KB_S, STAGES, MB>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        e = cudaFuncSetAttribute(gemv_kernel<NT, KB_S, STAGES, MINB, MB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 C::smem_bytes(kTableBytes / 16, 1));
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemv smem)");
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    int kb_per = (p.n_cb + p.split - 1) / p.split;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid_x, (unsigned)p.split, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = (size_t)C::smem_bytes(kb_per, p.M);
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    unsigned na = 0;
    if (p.split > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = 1;
        attrs[na].val.clusterDim.y = (unsigned)p.split;
        attrs[na].val.clusterDim.z = 1;
        na++;
    }
    if (flags & SX8_F_PDL) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    e = cudaLaunchKernelEx(&cfg, gemv_kernel<NT, KB_S, STAGES, MINB, MB>, p);
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(gemv_kernel)");
    return SX8_OK;
}

}  // namespace

extern "C" void sx8_gemv_tune(int nt, int split, int grid) {
    g_tune_nt = nt;
    g_tune_split = split;
    g_tune_grid = grid;
}

extern "C" size_t sx8_gemv_workspace_bytes(int n_cb, int M) {
    if (n_cb <= 0 || M <= 0) return 0;
    size_t b = (size_t)(M > 8 ? 8 : M) * (size_t)n_cb * 64;   // staged activations (M, 32*n_cb) f16
    return (b + 255) & ~(size_t)255;
}

namespace sx8 {
// x can be fetched by 16-byte bulk copies as it is: no staging copy, no workspace needed
static inline bool x_direct(const void* x, int K, long ldx, int n_cb) {
    return K == n_cb * 32 && (ldx % 8) == 0 && (reinterpret_cast<uintptr_t>(x) % 16) == 0;
}

// Shared by sx8_gemv and the 8-row passes of sx8_gemm.  Arguments already validated.
int gemv_launch_ex(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                   const float* scales, int N, int n_cb, float* y, void* workspace, unsigned flags,
                   const sx8_peers_t* peers, cudaStream_t stream);

int gemv_launch(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                const float* scales, int N, int n_cb, float* y, void* workspace, unsigned flags,
                cudaStream_t stream) {
    return gemv_launch_ex(x, M, K, ldx, wt16, bases, scales, N, n_cb, y, workspace, flags, nullptr, stream);
}

int gemv_launch_ex(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                   const float* scales, int N, int n_cb, float* y, void* workspace, unsigned flags,
                   const sx8_peers_t* peers, cudaStream_t stream) {
    const __half* xp = (const __half*)x;
    long ld = ldx;
    const int Kp = n_cb * 32;
    if (!x_direct(x, K, ldx, n_cb)) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(((long)M * Kp + 255) / 256), 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.stream = stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = (flags & SX8_F_PDL) ? 1 : 0;
        cudaError_t e = cudaLaunchKernelEx(&cfg, xpad_kernel, (const __half*)x, M, K, ldx, Kp, (__half*)workspace);
        if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(xpad_kernel)");
        xp = (const __half*)workspace;
        ld = Kp;
    }
    Choice c = choose(N, n_cb, M);
    const int n_tiles = (int)t16_tiles(N);
    GemvParams p{};
    p.nseg = 1;
    p.seg[0] = SegDesc{(const uint8_t*)wt16, bases, scales, y, N, n_tiles, 0};
    p.x = xp; p.ldx = ld;
    p.n_cb = n_cb; p.M = M; p.split = c.split;
    p.groups = (n_tiles + c.nt - 1) / c.nt;
    p.rank = 0; p.world = 1; p.slot_elems = 0;
    if (peers && peers->world > 1) {
        const int par = peers->parity & 1;
        for (int q = 0; q < peers->world; q++) {
            p.peer_data[q] = (float*)peers->data[q] + (long)par * peers->world * peers->slot_elems;
            p.peer_flag[q] = (unsigned*)peers->flags[q] + par;
        }
        p.slot_elems = peers->slot_elems; p.rank = peers->rank; p.world = peers->world;
    }
    int rc;
    if (c.nt == 8) rc = launch_gemv<8, 8, 2>(p, c.grid_x, flags, stream);
    else if (c.nt == 4) rc = launch_gemv<4, 8, 3>(p, c.grid_x, flags, stream);
    else rc = launch_gemv<2, 8, 4>(p, c.grid_x, flags, stream);
    if (rc != SX8_OK || p.world <= 1) return rc;
    // second half of the exchange: sum the world slots of this rank's receive buffer into y
    const int par = peers->parity & 1;
    const long n_elems = (long)M * N;
    cudaLaunchConfig_t cfg = {};
    unsigned blocks = (unsigned)((n_elems + 1023) / 1024);
    cfg.gridDim = dim3(blocks < 1 ? 1 : (blocks > 64 ? 64 : blocks), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = (flags & SX8_F_PDL) ? 1 : 0;
    unsigned* fl = (unsigned*)peers->flags[peers->rank];
    cudaError_t e = cudaLaunchKernelEx(&cfg, reduce_peers_kernel,
                                       (const float*)peers->data[peers->rank] + (long)par * peers->world * peers->slot_elems,
                                       fl + par, fl + 2 + par, y, n_elems, (long)peers->slot_elems, peers->world,
                                       (unsigned)(peers->world * n_tiles));
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(reduce_peers_kernel)");
    return SX8_OK;
}

// 9..16 batch rows in one pass over the weights: the activation table goes to global scratch
// (one small launch), then the GEMV kernel with two blocks of 8 rows per decoded fragment.
// xstage: (M, 32*n_cb) f16 scratch, used only when x cannot be fetched as it is; table:
// n_cb * M * 16 bytes, 16-byte aligned.  Arguments already validated.
// 9..16 rows: count <= 4 matrices on the same x in one launch (count == 1: the plain case).  table holds
// count activation tables of n_cb * M * 16 bytes.
int gemv_rows_launch_multi(const void* x, int M, int K, long ldx, int count, const void* const* wt16,
                           const float* const* bases, const float* const* scales, const int* N, float* const* y,
                           int n_cb, void* xstage, void* table, unsigned flags, cudaStream_t stream) {
    const __half* xp = (const __half*)x;
    long ld = ldx;
    const int Kp = n_cb * 32;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cfg.attrs = &attr;
    cfg.numAttrs = (flags & SX8_F_PDL) ? 1 : 0;
    if (!x_direct(x, K, ldx, n_cb)) {
        cfg.gridDim = dim3((unsigned)(((long)M * Kp + 255) / 256), 1, 1);
        cudaError_t e = cudaLaunchKernelEx(&cfg, xpad_kernel, (const __half*)x, M, K, ldx, Kp, (__half*)xstage);
        if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(xpad_kernel)");
        xp = (const __half*)xstage;
        ld = Kp;
    }
    ActTableArgs ta = {};
    for (int i = 0; i < count; i++) { ta.bases[i] = bases[i]; ta.scales[i] = scales[i]; }
    cfg.gridDim = dim3((unsigned)(((long)n_cb * M + 63) / 64), (unsigned)count, 1);
    cudaError_t e = cudaLaunchKernelEx(&cfg, act_table_kernel, xp, ld, M, n_cb, ta, (uint2*)table);
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(act_table_kernel)");
    // four-tile groups, one per CTA (two warps share a tile here, and their partial sums are only
    // combined once, at the end of the CTA), two CTAs per SM; groups never straddle matrices
    GemvParams p{};
    p.nseg = count;
    int groups = 0;
    for (int i = 0; i < count; i++) {
        const int nt_i = (int)t16_tiles(N[i]);
        p.seg[i] = SegDesc{(const uint8_t*)wt16[i], bases[i], scales[i], y[i], N[i], nt_i, groups};
        groups += (nt_i + 3) / 4;
    }
    int split = 1;
    while (split < 8 && (long)groups * split < 2 * kSMs && n_cb / (split + 1) >= 8) split++;
    p.x = xp; p.ldx = ld; p.table = (const uint8_t*)table;
    p.n_cb = n_cb; p.M = M; p.split = split; p.groups = groups;
    p.rank = 0; p.world = 1; p.slot_elems = 0;
    // Two row blocks only: every further block adds two m16n8k16 and two m16n8k8 mma.sync per
    // 512 weights, and on this GPU those run at about 32 and 16 cycles each per scheduler
    // (28672 x 8192: 72 us at 8 rows, 106 us at 16, 234 us at 32 with four blocks against 137 us
    // on the tcgen05 kernel), so from 17 rows on the tensor-core GEMM is the faster path.
    return launch_gemv<4, 8, 3, 2, 2>(p, groups, flags, stream);
}

int gemv_rows_launch(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                     const float* scales, int N, int n_cb, float* y, void* xstage, void* table, unsigned flags,
                     cudaStream_t stream) {
    return gemv_rows_launch_multi(x, M, K, ldx, 1, &wt16, &bases, &scales, &N, &y, n_cb, xstage, table, flags, stream);
}

// Several matrices that share the activations, one launch (q|k|v, gate|up).  Each CTA owns one
// tile group of one matrix; groups never straddle matrices.
int gemv_launch_multi(const void* x, int M, int K, long ldx, int count, const void* const* wt16,
                      const float* const* bases, const float* const* scales, const int* N, float* const* y,
                      int n_cb, void* workspace, unsigned flags, cudaStream_t stream) {
    const __half* xp = (const __half*)x;
    long ld = ldx;
    const int Kp = n_cb * 32;
    if (!x_direct(x, K, ldx, n_cb)) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(((long)M * Kp + 255) / 256), 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.stream = stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = (flags & SX8_F_PDL) ? 1 : 0;
        cudaError_t e = cudaLaunchKernelEx(&cfg, xpad_kernel, (const __half*)x, M, K, ldx, Kp, (__half*)workspace);
        if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(xpad_kernel)");
        xp = (const __half*)workspace;
        ld = Kp;
    }
    long n_total = 0;
    for (int i = 0; i < count; i++) n_total += (long)t16_tiles(N[i]) * 16;
    Choice c = choose((int)n_total, n_cb, M);
    GemvParams p{};
    p.nseg = count;
    int g0 = 0;
    for (int i = 0; i < count; i++) {
        int nt_i = (int)t16_tiles(N[i]);
        p.seg[i] = SegDesc{(const uint8_t*)wt16[i], bases[i], scales[i], y[i], N[i], nt_i, g0};
        g0 += (nt_i + c.nt - 1) / c.nt;
    }
    p.x = xp; p.ldx = ld; p.n_cb = n_cb; p.M = M; p.split = c.split; p.groups = g0;
    p.rank = 0; p.world = 1; p.slot_elems = 0;
    if (c.nt == 8) return launch_gemv<8, 8, 2>(p, g0, flags, stream);   // one group per CTA: grid = groups
    if (c.nt == 4) return launch_gemv<4, 8, 3>(p, g0, flags, stream);
    return launch_gemv<2, 8, 4>(p, g0, flags, stream);
}

int gemv_workspace_check(const char* who, const void* x, int M, int K, long ldx, int n_cb, const void* workspace,
                         size_t workspace_bytes) {
    if (x_direct(x, K, ldx, n_cb)) return SX8_OK;
    if (!workspace || workspace_bytes < sx8_gemv_workspace_bytes(n_cb, M) ||
        (reinterpret_cast<uintptr_t>(workspace) % 256) != 0) {
        set_error("%s: x needs a staging copy (K not a multiple of 32, or rows not 16-byte aligned): workspace must be "
                  "256-byte aligned and hold %zu bytes (got %zu)", who, sx8_gemv_workspace_bytes(n_cb, M), workspace_bytes);
        return SX8_E_WORKSPACE;
    }
    return SX8_OK;
}

int gemv_check(const char* who, const void* x, int M, int Mmax, int K, long ldx, const void* wt16,
               const float* bases, const float* scales, int N, int n_cb, const void* y) {
    SX8_REQUIRE(x && wt16 && bases && scales && y, "%s: null pointer", who);
    SX8_REQUIRE(M >= 1 && M <= Mmax, "%s: M must be in 1..%d (got %d)", who, Mmax, M);
    SX8_REQUIRE(N > 0, "%s: N must be positive (got %d)", who, N);
    SX8_REQUIRE(K > 0 && n_cb == (K + 31) / 32, "%s: need K>0 and n_cb == ceil(K/32) (got K=%d n_cb=%d)", who, K, n_cb);
    SX8_REQUIRE(n_cb <= 8 * max_kb_per_cta(M > 8 ? 8 : (M < 1 ? 1 : M)), "%s: K too large for this batch (n_cb=%d, limit %d)", who,
                n_cb, 8 * max_kb_per_cta(M > 8 ? 8 : (M < 1 ? 1 : M)));
    SX8_REQUIRE(ldx >= K, "%s: ldx (%ld) < K (%d)", who, ldx, K);
    SX8_REQUIRE((reinterpret_cast<uintptr_t>(wt16) % 16) == 0, "%s: wt16 must be 16-byte aligned (TMA bulk copies)", who);
    SX8_REQUIRE((reinterpret_cast<uintptr_t>(bases) % 16) == 0 && (reinterpret_cast<uintptr_t>(x) % 2) == 0 &&
                    (reinterpret_cast<uintptr_t>(y) % 4) == 0,
                "%s: misaligned x / bases / y", who);
    return SX8_OK;
}
}  // namespace sx8

extern "C" int sx8_gemv(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                        const float* scales, int N, int n_cb, float* y, void* workspace,
                        size_t workspace_bytes, unsigned flags, void* stream) {
    int rc = gemv_check("sx8_gemv", x, M, SX8_GEMV_MAX_BATCH, K, ldx, wt16, bases, scales, N, n_cb, y);
    if (rc != SX8_OK) return rc;
    rc = gemv_workspace_check("sx8_gemv", x, M, K, ldx, n_cb, workspace, workspace_bytes);
    if (rc != SX8_OK) return rc;
    return gemv_launch(x, M, K, ldx, wt16, bases, scales, N, n_cb, y, workspace, flags, (cudaStream_t)stream);
}

extern "C" int sx8_gemv_allreduce(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                                  const float* scales, int N, int n_cb, float* y, void* workspace,
                                  size_t workspace_bytes, unsigned flags, const sx8_peers_t* peers, void* stream) {
    int rc = gemv_check("sx8_gemv_allreduce", x, M, SX8_GEMV_MAX_BATCH, K, ldx, wt16, bases, scales, N, n_cb, y);
    if (rc != SX8_OK) return rc;
    SX8_REQUIRE(peers, "sx8_gemv_allreduce: null peer descriptor");
    SX8_REQUIRE(peers->world >= 1 && peers->world <= SX8_MAX_PEERS && peers->rank >= 0 && peers->rank < peers->world,
                "sx8_gemv_allreduce: bad rank/world (%d/%d, at most %d ranks)", peers->rank, peers->world, SX8_MAX_PEERS);
    SX8_REQUIRE(peers->slot_elems >= (long)M * N, "sx8_gemv_allreduce: slot_elems (%ld) < M*N (%ld)", peers->slot_elems,
                (long)M * N);
    for (int q = 0; q < peers->world; q++)
        SX8_REQUIRE(peers->data[q] && peers->flags[q] && (reinterpret_cast<uintptr_t>(peers->data[q]) % 16) == 0 &&
                        (reinterpret_cast<uintptr_t>(peers->flags[q]) % 4) == 0,
                    "sx8_gemv_allreduce: null or misaligned peer pointer for rank %d", q);
    rc = gemv_workspace_check("sx8_gemv_allreduce", x, M, K, ldx, n_cb, workspace, workspace_bytes);
    if (rc != SX8_OK) return rc;
    return gemv_launch_ex(x, M, K, ldx, wt16, bases, scales, N, n_cb, y, workspace, flags, peers,
                          (cudaStream_t)stream);
}

extern "C" int sx8_gemv_multi(const void* x, int M, int K, long ldx, int count, const void* const* wt16,
                              const float* const* bases, const float* const* scales, const int* N,
                              float* const* y, int n_cb, void* workspace, size_t workspace_bytes,
                              unsigned flags, void* stream) {
    SX8_REQUIRE(count >= 1 && count <= kMaxSeg, "sx8_gemv_multi: count must be in 1..%d (got %d)", kMaxSeg, count);
    SX8_REQUIRE(wt16 && bases && scales && N && y, "sx8_gemv_multi: null array");
    int rc = SX8_OK;
    for (int i = 0; i < count; i++) {
        rc = gemv_check("sx8_gemv_multi", x, M, SX8_GEMV_MAX_BATCH, K, ldx, wt16[i], bases[i], scales[i], N[i],
                            n_cb, y[i]);
        if (rc != SX8_OK) return rc;
    }
    rc = gemv_workspace_check("sx8_gemv_multi", x, M, K, ldx, n_cb, workspace, workspace_bytes);
    if (rc != SX8_OK) return rc;
    return gemv_launch_multi(x, M, K, ldx, count, wt16, bases, scales, N, y, n_cb, workspace, flags,
                             (cudaStream_t)stream);
}
