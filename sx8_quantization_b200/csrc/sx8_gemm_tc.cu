// sx8_gemm_tc.cu -- S-X8 v4.3 prefill GEMM on the 5th-generation tensor cores (sm_100a).
//
//   Y (M, N) = X (M, K) * W^T,  W decoded on the fly from the T16 blob, fp32 accumulate.
//
// Tiles.  M > 256: a cluster of two CTAs computes 512 rows x 256 columns with two-CTA MMAs
// (tcgen05.mma.cta_group::2, M=256, N=256, K=16, two accumulators): each CTA loads its own
// 256 rows of X and decodes 128 of the 256 columns.  M <= 256: one CTA computes 128*MT rows x
// BN columns (cta_group::1).  K step 64 (two block rows).  Warp roles:
//   warp 0      producer : X tiles by 2-D TMA (128-byte swizzle)
//   warp 18     producer : packed slabs of the blob (one 2-D tensor copy per stage) and the
//                          fp16 PCA table, running up to 8 stages ahead
//   warp 1      issuer   : in the leader CTA one thread issues the MMAs on shared-memory
//                          descriptors; accumulators live in TMEM (all 512 columns);
//                          tcgen05.commit releases the stages (in both CTAs of a pair).  In the
//                          peer CTA this warp tells the leader when the peer's X tiles landed.
//   warps 2..17 decoders : bit-extract 6-bit levels from the packed slab, form fp16 weights
//                          w = dmin + base*(mult*level + 63*off) + c0*s0*b0[t] + c1*s1*b1[t]
//                          (the arithmetic of ref cuda/sx8_fused_wmma.cu:83-96, in fp16 pairs)
//                          and store them as the K-major, 128-byte-swizzled B operand tile;
//                          afterwards the same warps read TMEM back (tcgen05.ld) and write Y
//                          through swizzled staging and TMA stores.
// Every role probes the barriers of its next stage early (mbarrier.test_wait) and reads the
// answer one iteration later: a blocking wait costs a shared-memory round trip even when the
// phase completed long ago.
// Every wait on an mbarrier is bounded; a wait that runs out sets the device error word and
// the kernel drains and frees its TMEM.
#include <atomic>
#include <cuda.h>

#include "sx8_common.cuh"
#include "sx8_layout.cuh"

namespace sx8 {

namespace tc {

constexpr int BK = 64, KB_STAGE = 2;
constexpr int kDecodeWarps = 16, kWarps = kDecodeWarps + 3, kThreads = kWarps * 32;
constexpr int kSmemMax = 232448;                 // opt-in shared memory per CTA on sm_100
constexpr int A_TILE = 128 * 128;                 // 128 rows x 64 fp16, bytes
constexpr int P_TAB = KB_STAGE * 128;             // PCA table: per kb 2 x 32 fp16
constexpr uint32_t kSpin = 1u << 22;

// MT = accumulators per CTA (1 or 2), BN = columns a CTA decodes per stage (64, 128 or 256),
// PAIR = CTAs that share one MMA (1, or 2 = a cluster of two CTAs issuing cta_group::2 MMAs of
// 256 rows: each CTA supplies its own 128 rows of X and half of the decoded columns, so every
// decoded weight feeds twice as many rows).  An accumulator is 128 rows x BN*PAIR columns.
template <int MT, int BN, int PAIR>
struct Cfg {
    static constexpr int TILES = BN / 16;
    static constexpr int BNU = BN * PAIR;                       // MMA N = accumulator columns
    static constexpr int B_TILE = BN * 128;                     // BN rows x 64 fp16
    static constexpr int P_SLAB = TILES * KB_STAGE * T16_UNIT;  // TILES tiles x 2 kb
    static constexpr int P_STAGE = P_SLAB + P_TAB;
    // Stage counts are launch parameters (Params::sa/sb/sp): X-tile stages, decoded-operand
    // stages, packed-slab stages.  Shared memory, in order: X tiles, operand tiles, slabs,
    // barriers, the tensor-memory address.
    static constexpr int smem_bytes(int sa, int sb, int sp) {
        return sa * MT * A_TILE + sb * B_TILE + sp * P_STAGE + (3 * sa + 2 * sb + 2 * sp + 2) * 8 + 16 +
               1024;   // + slack to align the base to 1024 B
    }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// CL = true: acquire at cluster scope (the barrier is arrived on by the peer CTA of a pair or
// by a two-CTA tcgen05.commit).
template <bool CL>
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    if constexpr (CL)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Non-blocking probe.  A wait costs a shared-memory round trip (a few hundred cycles) even
// when the phase has long completed, and a warp that waits on two barriers per stage pays it
// twice, serially, before its real work.  So every role probes the barriers of its NEXT
// stage before it starts on the current one and looks at the answer afterwards.
template <bool CL>
__device__ __forceinline__ uint32_t mbar_probe(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    if constexpr (CL)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
template <bool CL>
__device__ __forceinline__ bool mbar_wait_t(uint32_t bar, uint32_t parity, unsigned code) {
    for (uint32_t i = 0; i < kSpin; i++)
        if (mbar_try_wait<CL>(bar, parity)) return true;
    atomicOr(&g_sx8_error_flag, code);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned code) {
    return mbar_wait_t<false>(bar, parity, code);
}
__device__ __forceinline__ bool mbar_wait_cl(uint32_t bar, uint32_t parity, unsigned code) {
    return mbar_wait_t<true>(bar, parity, code);
}
// Position in a ring of n stages: slot s, round r (the phase parity of a "full" barrier is
// r & 1; an "empty" barrier is waited on from round 1 with parity (r - 1) & 1).
struct Ring {
    int s, n;
    uint32_t r;
    __device__ __forceinline__ Ring(int n_) : s(0), n(n_), r(0) {}
    __device__ __forceinline__ Ring next() const {
        Ring q = *this;
        if (++q.s == q.n) { q.s = 0; q.r++; }
        return q;
    }
};
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cl(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
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
__device__ __forceinline__ void sts128(uint32_t a, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t dup_lo(uint32_t v) { return __byte_perm(v, 0u, 0x1010u); }
__device__ __forceinline__ uint32_t dup_hi(uint32_t v) { return __byte_perm(v, 0u, 0x3232u); }

// K-major, 128-byte-swizzled shared-memory matrix descriptor (sm_100): start address >> 4 in
// bits 0-13, stride between 8-row groups (1024 B) >> 4 in bits 32-45, descriptor version 1 in
// bits 46-47, swizzle mode 2 (128 B) in bits 61-63.  The leading-dimension field is unused
// for swizzled K-major operands.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: D = f32, A = B = f16, both K-major, N = bn, M = m.
__host__ __device__ constexpr uint32_t idesc_for(int bn, int m) {
    return (1u << 4) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Two-CTA forms: one thread of the leader CTA issues the MMA for both CTAs; the commit arrives
// on the barrier at the same shared-memory offset in both CTAs of the pair.
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Split-K hand-over: a 32 x 32 block of accumulator values (one row per lane) as 8 swizzled
// 16-byte chunks per lane.  store_xfer writes it to this CTA's shared memory, add_xfer adds the
// block found at a shared::cluster address (the peer CTA's copy) to v.
__device__ __forceinline__ void store_xfer(uint32_t base, int lane, const uint32_t (&v)[32]) {
#pragma unroll
    for (int q = 0; q < 8; q++)
        sts128(base + lane * 128 + (((uint32_t)q ^ ((uint32_t)lane & 7u)) << 4),
               make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
}
__device__ __forceinline__ void add_xfer(uint32_t cluster_base, int lane, uint32_t (&v)[32]) {
#pragma unroll
    for (int q = 0; q < 8; q++) {
        float4 u;
        asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(u.x), "=f"(u.y), "=f"(u.z), "=f"(u.w)
                     : "r"(cluster_base + lane * 128 + (((uint32_t)q ^ ((uint32_t)lane & 7u)) << 4))
                     : "memory");
        v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + u.x);
        v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + u.y);
        v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + u.z);
        v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + u.w);
    }
}

// PCA table: pb[kb][j][t] = fp16(scales[kb][j] * bases[kb][32j + t] * 1024), 128 bytes per kb.
// (The coefficient operand carries the matching 2^-10; the pre-scale keeps the products of
// small scales and basis entries out of the fp16 subnormal range.)
// Launched with programmatic stream serialization: the GEMM that follows may start (and prefetch its
// weights) while this kernel runs, and this kernel may start while the GEMM before it -- which
// reads the same table when calls share a workspace -- is still running: bases and scales are
// weights and are read at once, the table is written only after that GEMM has completed.
struct TableArgs {
    const float* bases[3];
    const float* scales[3];
};
// grid (ceil(n_cb * 64 / 256), matrices); the table of matrix i starts at pb + i * n_cb * 64.
__global__ void __launch_bounds__(256) pca_table_kernel(TableArgs a, int n_cb, __half* __restrict__ pb) {
    asm volatile("griddepcontrol.launch_dependents;");
    const int i = blockIdx.x * 256 + threadIdx.x, mi = blockIdx.y;
    const float* __restrict__ bases = a.bases[mi];
    const float* __restrict__ scales = a.scales[mi];
    __half v = __float2half_rn(0.0f);
    if (i < n_cb * 64) {
        int kb = i >> 6, j = (i >> 5) & 1;
        v = __float2half_rn(scales[kb * 2 + j] * bases[i] * 1024.0f);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (i < n_cb * 64) pb[(long)mi * n_cb * 64 + i] = v;
}

// One launch can serve up to kMaxMats matrices that share X (q|k|v, gate|up): their columns are
// laid side by side in one virtual N (every matrix but the last a multiple of 256 columns wide,
// so no tile straddles two matrices); a CTA finds its matrix from its first column and uses that
// matrix's blob, PCA table and output.
constexpr int kMaxMats = 3;
struct Mat {
    const uint8_t* blob;   // host side only: the tensor map is built from it
    void* y;               // (M, N) row-major
    int col0, N, n_tiles;  // first virtual column, columns, 16-column tiles
};
struct Params {
    const __half* pb;      // PCA tables, one of n_cb * 64 halves per matrix
    int nmat;
    Mat mat[kMaxMats];
    int M, N, n_cb, out_f16;   // N: virtual columns of all matrices
    int tma_store;   // Y rows are 16-byte multiples: the epilogue stores through the Y tensor map
    int sa, sb, sp;  // pipeline depths: X-tile, decoded-operand and packed-slab stages
    int debug;       // timing experiments only (results are wrong): 1 = skip the decode math, 2 = skip the
                     // MMAs, 4 = skip the packed-slab copies, 8 = skip the X-tile copies
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(src) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}


// G = decode groups: the 16 decode warps form G groups of 16/G warps that take every G-th stage.
// KS = 2 or 4 (one-CTA tiles only): a cluster of KS CTAs shares one output tile, each taking 1/KS
// of the K range; CTAs 1 .. KS-1 hand their accumulators to CTA 0 through distributed shared
// memory.  For small M, where there are fewer tiles than SMs and decoding the weights bounds the time.
template <int MT, int BN, int PAIR, int G, int KS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap ymap0,
               const __grid_constant__ CUtensorMap ymap1, const __grid_constant__ CUtensorMap ymap2,
               const __grid_constant__ CUtensorMap wmap0, const __grid_constant__ CUtensorMap wmap1,
               const __grid_constant__ CUtensorMap wmap2, Params p) {
    using C = Cfg<MT, BN, PAIR>;
    constexpr int kGroupWarps = kDecodeWarps / G;
    constexpr int B_TILE = C::B_TILE, P_SLAB = C::P_SLAB, P_STAGE = C::P_STAGE, TILES = C::TILES, BNU = C::BNU;
    static_assert(MT * BNU <= 512, "accumulators exceed tensor memory");
    static_assert(KS == 1 || PAIR == 1, "split-K is for one-CTA tiles");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int SA = p.sa, SB = p.sb, SP = p.sp;
    const uint32_t sA = sbase, sB = sA + SA * MT * A_TILE, sP = sB + SB * B_TILE;
    const uint32_t bar0 = sP + SP * P_STAGE;
    const uint32_t a_full = bar0, a_empty = a_full + 8 * SA;
    const uint32_t b_full = a_empty + 8 * SA, b_empty = b_full + 8 * SB;
    const uint32_t p_full = b_empty + 8 * SB, p_empty = p_full + 8 * SP;
    const uint32_t acc_full = p_empty + 8 * SP;
    const uint32_t a_peer = acc_full + 8;        // leader only: the peer CTA's X tiles have landed
    const uint32_t xfer_full = a_peer + 8 * SA;   // KS == 2, CTA 0: the peer's accumulator is in its shared memory
    const uint32_t tmem_slot = xfer_full + 8;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // PAIR == 2: the cluster is two consecutive CTAs along x; rank 0 leads (issues the MMAs).
    const int rank = (PAIR == 2) ? (int)(blockIdx.x & 1) : 0;
    static_assert(KS == 1 || KS == 2 || KS == 4, "split-K over a cluster of 2 or 4");
    const int krank = (KS > 1) ? (int)(blockIdx.x & (KS - 1)) : 0;
    const int nv0 = (int)(blockIdx.x / (PAIR * KS)) * BNU;   // first accumulator column among all matrices' columns
    const int m0 = blockIdx.y * (128 * MT * PAIR);
    // the matrix of this CTA
    int mi = 0;
    if (p.nmat > 1 && nv0 >= p.mat[1].col0) mi = 1;
    if (p.nmat > 2 && nv0 >= p.mat[2].col0) mi = 2;
    const CUtensorMap* const wmap = (mi == 0) ? &wmap0 : ((mi == 1) ? &wmap1 : &wmap2);
    const CUtensorMap* const ymap = (mi == 0) ? &ymap0 : ((mi == 1) ? &ymap1 : &ymap2);
    const int n0 = nv0 - ((mi == 0) ? p.mat[0].col0 : ((mi == 1) ? p.mat[1].col0 : p.mat[2].col0));   // column within the matrix
    const int mat_N = (mi == 0) ? p.mat[0].N : ((mi == 1) ? p.mat[1].N : p.mat[2].N);
    const int mat_tiles = (mi == 0) ? p.mat[0].n_tiles : ((mi == 1) ? p.mat[1].n_tiles : p.mat[2].n_tiles);
    void* const mat_y = (mi == 0) ? p.mat[0].y : ((mi == 1) ? p.mat[1].y : p.mat[2].y);
    const __half* const mat_pb = p.pb + (long)mi * p.n_cb * 64;
    const int tile0 = (n0 + rank * BN) >> 4;                 // first 16-column tile this CTA decodes
    const int n_ks_all = (p.n_cb + KB_STAGE - 1) / KB_STAGE;
    const int ks_half = (n_ks_all + KS - 1) / KS;            // K stages per CTA of the cluster
    const int ks0 = krank * ks_half;                         // first K stage of this CTA
    const int n_ks = (KS > 1) ? max(0, min(ks_half, n_ks_all - ks0)) : n_ks_all;

    if (threadIdx.x == 0) {
        mbar_init(xfer_full, kDecodeWarps * (KS > 1 ? KS - 1 : 1));
        for (int s = 0; s < SA; s++) { mbar_init(a_full + 8 * s, 1); mbar_init(a_empty + 8 * s, 1); }
        for (int s = 0; s < SA; s++) mbar_init(a_peer + 8 * s, 1);
        for (int s = 0; s < SB; s++) { mbar_init(b_full + 8 * s, kGroupWarps * PAIR); mbar_init(b_empty + 8 * s, 1); }
        for (int s = 0; s < SP; s++) { mbar_init(p_full + 8 * s, 1); mbar_init(p_empty + 8 * s, kGroupWarps); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // TMEM: all 512 columns (two 128 x 256 fp32 accumulators)
        if constexpr (PAIR == 2) {   // one warp of each CTA of the pair takes part
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR == 2 || KS > 1) cluster_sync_all();   // the peer's barriers exist before anyone arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = lds32(tmem_slot);

    // Programmatic dependent launch: the kernel after this one may begin its own set-up now; this
    // kernel was itself allowed to start before the one ahead of it finished.  The packed weights
    // do not depend on that kernel and are requested at once; X, the PCA table and Y are touched
    // only after griddepcontrol.wait (which every role that reaches global memory executes).
    asm volatile("griddepcontrol.launch_dependents;");

    if (warp == kWarps - 1) {
        // ------------------------------------------------------------ producer of packed slabs
        bool ok = true;
        Ring rp(SP);
        // One tensor copy brings the slabs of all TILES tiles: the blob is a 2-D array of
        // 32-bit words, one row of n_cb * 120 words per 16-column tile; the box is
        // TILES rows x 240 words (two block rows).  Tiles or block rows past the end
        // arrive as zeros (and count as bytes).  The PCA table rows of the stage follow as a
        // second copy onto the same barrier.
        auto issue = [&](int ks, int s, bool weights, bool table) {
            const int kb0 = (ks0 + ks) * KB_STAGE;
            const int rows = min(KB_STAGE, p.n_cb - kb0);
            const uint32_t dst = sP + s * P_STAGE;
            if (lane == 0) {
                if (weights) {
                    mbar_expect_tx(p_full + 8 * s, (uint32_t)P_SLAB + (uint32_t)rows * 128u);
                    tma_load_2d(dst, wmap, kb0 * (T16_UNIT / 4), tile0, p_full + 8 * s);
                }
                if (table) bulk_g2s(dst + P_SLAB, mat_pb + (long)kb0 * 64, (uint32_t)rows * 128u, p_full + 8 * s);
            }
            __syncwarp();
        };
        const int pre = (SX8_DBG(p) & 4) ? 0 : min(n_ks, SP);   // stages filled before the wait: weights only
        for (int ks = 0; ks < pre; ks++) issue(ks, ks, true, false);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int ks = 0; ks < pre; ks++) { issue(ks, ks, false, true); rp = rp.next(); }
        for (int ks = pre; ks < n_ks; ks++) {
            const int s = rp.s;
            if (rp.r > 0 && ok) ok = mbar_wait(p_empty + 8 * s, (rp.r - 1) & 1, 0x10u);
            rp = rp.next();
            if (SX8_DBG(p) & 4) {
                if (lane == 0) mbar_arrive(p_full + 8 * s);
                continue;
            }
            issue(ks, s, true, true);
        }
    } else if (warp == 0) {
        // ------------------------------------------------------------ producer of X tiles
        bool ok = true;
        Ring ra(SA);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int ks = 0; ks < n_ks; ks++) {
            {   // MT boxes of 64 (K) x 128 (rows); columns/rows out of range read as zero
                const int s = ra.s;
                if (ra.r > 0 && ok) ok = mbar_wait(a_empty + 8 * s, (ra.r - 1) & 1, 0x20u);
                ra = ra.next();
                if (SX8_DBG(p) & 8) {
                    if (lane == 0) mbar_arrive(a_full + 8 * s);
                    continue;
                }
                if (lane == 0) {
                    mbar_expect_tx(a_full + 8 * s, (uint32_t)(MT * A_TILE));
                    for (int mt = 0; mt < MT; mt++)
                        tma_load_2d(sA + (s * MT + mt) * A_TILE, &xmap, (ks0 + ks) * BK, m0 + (mt * PAIR + rank) * 128,
                                    a_full + 8 * s);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1 && rank != 0) {
        // ------------------------------------------------------------ relay (peer CTA of a pair)
        // tells the leader that this CTA's X tiles of a stage have landed
        bool ok = true;
        const uint32_t remote = mapa_u32(a_peer, 0u);
        Ring ra(SA);
        for (int ks = 0; ks < n_ks; ks++) {
            if (ok) ok = mbar_wait(a_full + 8 * ra.s, ra.r & 1, 0x800u);
            __syncwarp();
            if (lane == 0) mbar_arrive_cl(remote + 8 * ra.s);
            ra = ra.next();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        bool ok = true;
        Ring ra(SA), rb(SB);
        uint32_t pre_a = 0, pre_b = 0, pre_c = (PAIR == 2) ? 0u : 1u;   // answers of the early probes
        for (int ks = 0; ks < n_ks; ks++) {
            const int sa = ra.s, sb = rb.s;
            if (!pre_a && ok) ok = mbar_wait(a_full + 8 * sa, ra.r & 1, 0x40u);
            if (!pre_c && ok) ok = mbar_wait_cl(a_peer + 8 * sa, ra.r & 1, 0x1000u);
            if (!pre_b && ok) ok = mbar_wait_t<PAIR == 2>(b_full + 8 * sb, rb.r & 1, 0x80u);
            ra = ra.next();
            rb = rb.next();
            if (ks + 1 < n_ks) {   // probe the next stage now, read the answers next iteration
                pre_a = mbar_probe<false>(a_full + 8 * ra.s, ra.r & 1);
                if constexpr (PAIR == 2) pre_c = mbar_probe<true>(a_peer + 8 * ra.s, ra.r & 1);
                pre_b = mbar_probe<PAIR == 2>(b_full + 8 * rb.s, rb.r & 1);
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint64_t bdesc = umma_desc(sB + sb * B_TILE);
#pragma unroll
                for (int mt = 0; mt < MT && !(SX8_DBG(p) & 2); mt++) {
                    const uint64_t adesc = umma_desc(sA + (sa * MT + mt) * A_TILE);
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) {   // +32 bytes along K inside the swizzle atom
                        if constexpr (PAIR == 2)
                            umma_f16_pair(tmem_base + mt * BNU, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2),
                                          idesc_for(BNU, 256), (ks > 0 || k > 0) ? 1u : 0u);
                        else
                            umma_f16(tmem_base + mt * BNU, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2),
                                     idesc_for(BNU, 128), (ks > 0 || k > 0) ? 1u : 0u);
                    }
                }
                if (SX8_DBG(p) & 32) {   // handshake experiment: plain arrivals instead of commits
                    mbar_arrive(a_empty + 8 * sa);
                    mbar_arrive(b_empty + 8 * sb);
                    if (ks == n_ks - 1) mbar_arrive(acc_full);
                } else if constexpr (PAIR == 2) {
                    umma_commit_pair(a_empty + 8 * sa);
                    umma_commit_pair(b_empty + 8 * sb);
                    if (ks == n_ks - 1) umma_commit_pair(acc_full);
                } else {
                    umma_commit(a_empty + 8 * sa);
                    umma_commit(b_empty + 8 * sb);
                    if (ks == n_ks - 1) umma_commit(acc_full);
                }
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ decoders
        const int dw = warp - 2;                 // 0..15: tile dw of the CTA's 16
        const int g = lane >> 2, t = lane & 3;
        const uint32_t sh2 = 8u + 2u * (uint32_t)t;
        const float kBase = 0.25f * 0.015873f * 512.0f;   // levels are formed scaled by 2^-9
        bool ok = true;
        const uint32_t b_full_leader = (PAIR == 2) ? mapa_u32(b_full, 0u) : b_full;
        // The warps form G groups that take every G-th stage: the fixed cost a warp pays per
        // stage (barrier round trips, the proxy fence -- the largest stall of this kernel) is
        // spread over G times the items, and one group's waits overlap the others' arithmetic.
        const int grp = dw / kGroupWarps, gw = dw % kGroupWarps;
        Ring rp(SP), rb(SB);
        for (int i = 0; i < grp; i++) { rp = rp.next(); rb = rb.next(); }
        uint32_t pre_p = 0, pre_b = (rb.r == 0) ? 1u : 0u;   // answers of the early probes
        for (int ks = grp; ks < n_ks; ks += G) {
            const int sp = rp.s, sb = rb.s;
            const int rows = min(KB_STAGE, p.n_cb - (ks0 + ks) * KB_STAGE);
            if (!pre_p && ok) ok = mbar_wait(p_full + 8 * sp, rp.r & 1, 0x100u);
            if (!pre_b && ok) ok = mbar_wait_t<PAIR == 2>(b_empty + 8 * sb, (rb.r - 1) & 1, 0x200u);
#pragma unroll
            for (int i = 0; i < G; i++) { rp = rp.next(); rb = rb.next(); }
            if (ks + G < n_ks) {   // probe this group's next stage now, read the answers next iteration
                pre_p = mbar_probe<false>(p_full + 8 * rp.s, rp.r & 1);
                pre_b = (rb.r == 0) ? 1u : mbar_probe<PAIR == 2>(b_empty + 8 * rb.s, (rb.r - 1) & 1);
            }
            const uint32_t pst = sP + sp * P_STAGE, bst = sB + sb * B_TILE;
            // work items (tile, block row) are dealt round-robin to the group's warps
#pragma unroll
            for (int item = gw; item < TILES * KB_STAGE && !(SX8_DBG(p) & 1); item += kGroupWarps) {
                const int tl = item % TILES, r = item / TILES;
                const bool tile_ok = tile0 + tl < mat_tiles;
                // Column 16*tl + g sits in operand row 16*tl + rho(g), rho(g) = 4*(g&1) + (g>>1): the
                // eight lanes of a quarter-warp then store to eight different 16-byte bank groups.
                // The epilogue undoes the permutation when it reads the accumulator columns.
                const uint32_t rowA = (uint32_t)(tl * 16 + (((g & 1) << 2) | (g >> 1))), rowB = rowA + 8;
                {
                    uint4 wa = make_uint4(0u, 0u, 0u, 0u), wb = wa;
                    if (r < rows && tile_ok) {
                        const uint32_t unit = pst + (tl * KB_STAGE + r) * T16_UNIT;
                        uint32_t W0 = lds32(unit + lane * 4), W1 = lds32(unit + 128 + lane * 4),
                                 W2 = lds32(unit + 256 + lane * 4);
                        uint32_t H0 = lds32(unit + 384 + g * 4), H1 = lds32(unit + 416 + g * 4),
                                 H2 = lds32(unit + 448 + g * 4);
                        uint4 s0 = lds128(pst + P_SLAB + r * 128 + t * 16);        // 1024*s0*b0[8t..8t+7]
                        uint4 s1 = lds128(pst + P_SLAB + r * 128 + 64 + t * 16);   // 1024*s1*b1[8t..8t+7]
                        uint32_t u = (H2 >> sh2) & 0x00030003u;
                        uint32_t sel = u * 0x2222u + 0x10101010u;
                        uint32_t selB = sel >> 16;
                        // mult * 2^13 = 32768, 8192, 8192, 16384 ; 63*off * 2^-9 = 0, 0, 189/512, 63/512
                        uint32_t mA = __byte_perm(0x70007800u, 0x74007000u, sel);
                        uint32_t aA = __byte_perm(0x00000000u, 0x2FE035E8u, sel);
                        uint32_t mB = __byte_perm(0x70007800u, 0x74007000u, selB);
                        uint32_t aB = __byte_perm(0x00000000u, 0x2FE035E8u, selB);
                        uint32_t V3 = ((W0 << 2) & 0x0C0C0C0Cu) | ((W1 << 4) & 0x30303030u) | ((W2 << 6) & 0xC0C0C0C0u);
                        // (mult*level + 63*off) * 2^-9, exact (level bytes read as fp16 are level * 2^-22)
                        wa.x = hfma2_u32(W0 & 0x00FC00FCu, mA, aA);
                        wa.y = hfma2_u32((W0 >> 8) & 0x00FC00FCu, mA, aA);
                        wa.z = hfma2_u32(W1 & 0x00FC00FCu, mA, aA);
                        wa.w = hfma2_u32((W1 >> 8) & 0x00FC00FCu, mA, aA);
                        wb.x = hfma2_u32(W2 & 0x00FC00FCu, mB, aB);
                        wb.y = hfma2_u32((W2 >> 8) & 0x00FC00FCu, mB, aB);
                        wb.z = hfma2_u32(V3 & 0x00FF00FFu, mB, aB);
                        wb.w = hfma2_u32((V3 >> 8) & 0x00FF00FFu, mB, aB);
                        // w = dmin + base * (...)   (fp16 pairs; base = (dmax-dmin)*0.25*0.015873*2^9)
                        const float loAf = h2f_bits((uint16_t)H0), hiAf = h2f_bits((uint16_t)(H0 >> 16));
                        const float loBf = h2f_bits((uint16_t)H1), hiBf = h2f_bits((uint16_t)(H1 >> 16));
                        float bAf = (hiAf - loAf) * kBase;
                        float bBf = (hiBf - loBf) * kBase;
                        // PCA: + (c0 * 2^-10) * (1024*s0*b0[t]) + (c1 * 2^-10) * (1024*s1*b1[t])
                        uint32_t ccA = hfma2_u32((H2 & 0x000F000Fu) ^ 0x64086408u, 0x14001400u, 0xBC08BC08u);
                        uint32_t ccB = hfma2_u32(((H2 >> 4) & 0x000F000Fu) ^ 0x64086408u, 0x14001400u, 0xBC08BC08u);
                        // A block with an endpoint of magnitude >= 32768 (possible in the format, absent from
                        // real weights) can hold weights next to the fp16 maximum; formed in fp16 arithmetic
                        // (step rounded to fp16 first) such a weight could round to infinity.  Those blocks
                        // form their weights in float32, as the reference's decode does
                        // (ref cuda/sx8_fused_wmma.cu:83-96), and round once.
                        auto wide = [&](uint4& w, float base, float lo, uint32_t cc) {
                            const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&cc));   // {c0, c1} * 2^-10
                            uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
                            const uint32_t* p0 = reinterpret_cast<const uint32_t*>(&s0);
                            const uint32_t* p1 = reinterpret_cast<const uint32_t*>(&s1);
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const float2 l = __half22float2(*reinterpret_cast<const __half2*>(&wp[i]));
                                const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&p0[i]));
                                const float2 a1 = __half22float2(*reinterpret_cast<const __half2*>(&p1[i]));
                                const float v0 = fmaf(c.y, a1.x, fmaf(c.x, a0.x, fmaf(base, l.x, lo)));
                                const float v1 = fmaf(c.y, a1.y, fmaf(c.x, a0.y, fmaf(base, l.y, lo)));
                                __half2 h = __floats2half2_rn(v0, v1);
                                wp[i] = *reinterpret_cast<uint32_t*>(&h);
                            }
                        };
                        const bool wideA = fmaxf(fabsf(loAf), fabsf(hiAf)) >= 32768.0f;
                        const bool wideB = fmaxf(fabsf(loBf), fabsf(hiBf)) >= 32768.0f;
                        if (wideA) {
                            wide(wa, bAf, loAf, ccA);
                        } else {
                            // a range above ~29,500 would overflow the fp16 step: move a factor 64 from it to the levels
                            if (bAf > 60000.0f) {
                                bAf *= 0.015625f;
                                wa.x = hfma2_u32(wa.x, 0x54005400u, 0u); wa.y = hfma2_u32(wa.y, 0x54005400u, 0u);
                                wa.z = hfma2_u32(wa.z, 0x54005400u, 0u); wa.w = hfma2_u32(wa.w, 0x54005400u, 0u);
                            }
                            __half2 bA2 = __float2half2_rn(bAf);
                            const uint32_t bA = *reinterpret_cast<uint32_t*>(&bA2), loA = dup_lo(H0);
                            wa.x = hfma2_u32(wa.x, bA, loA); wa.y = hfma2_u32(wa.y, bA, loA);
                            wa.z = hfma2_u32(wa.z, bA, loA); wa.w = hfma2_u32(wa.w, bA, loA);
                            const uint32_t c0A = dup_lo(ccA), c1A = dup_hi(ccA);
                            wa.x = hfma2_u32(c0A, s0.x, wa.x); wa.y = hfma2_u32(c0A, s0.y, wa.y);
                            wa.z = hfma2_u32(c0A, s0.z, wa.z); wa.w = hfma2_u32(c0A, s0.w, wa.w);
                            wa.x = hfma2_u32(c1A, s1.x, wa.x); wa.y = hfma2_u32(c1A, s1.y, wa.y);
                            wa.z = hfma2_u32(c1A, s1.z, wa.z); wa.w = hfma2_u32(c1A, s1.w, wa.w);
                        }
                        if (wideB) {
                            wide(wb, bBf, loBf, ccB);
                        } else {
                            if (bBf > 60000.0f) {
                                bBf *= 0.015625f;
                                wb.x = hfma2_u32(wb.x, 0x54005400u, 0u); wb.y = hfma2_u32(wb.y, 0x54005400u, 0u);
                                wb.z = hfma2_u32(wb.z, 0x54005400u, 0u); wb.w = hfma2_u32(wb.w, 0x54005400u, 0u);
                            }
                            __half2 bB2 = __float2half2_rn(bBf);
                            const uint32_t bB = *reinterpret_cast<uint32_t*>(&bB2), loB = dup_lo(H1);
                            wb.x = hfma2_u32(wb.x, bB, loB); wb.y = hfma2_u32(wb.y, bB, loB);
                            wb.z = hfma2_u32(wb.z, bB, loB); wb.w = hfma2_u32(wb.w, bB, loB);
                            const uint32_t c0B = dup_lo(ccB), c1B = dup_hi(ccB);
                            wb.x = hfma2_u32(c0B, s0.x, wb.x); wb.y = hfma2_u32(c0B, s0.y, wb.y);
                            wb.z = hfma2_u32(c0B, s0.z, wb.z); wb.w = hfma2_u32(c0B, s0.w, wb.w);
                            wb.x = hfma2_u32(c1B, s1.x, wb.x); wb.y = hfma2_u32(c1B, s1.y, wb.y);
                            wb.z = hfma2_u32(c1B, s1.z, wb.z); wb.w = hfma2_u32(c1B, s1.w, wb.w);
                        }
                    }
                    // 16-byte chunk c = 4r + t of the 128-byte row, XOR-swizzled with (row & 7)
                    const uint32_t c = (uint32_t)(r * 4 + t);
                    sts128(bst + rowA * 128 + ((c ^ (rowA & 7u)) << 4), wa);
                    sts128(bst + rowB * 128 + ((c ^ (rowB & 7u)) << 4), wb);
                }
            }
            if (!(SX8_DBG(p) & 64))
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic stores -> tensor-core reads
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR == 2) mbar_arrive_cl(b_full_leader + 8 * sb);
                else mbar_arrive(b_full + 8 * sb);
                mbar_arrive(p_empty + 8 * sp);
            }
        }
        // ------------------------------------------------------------ epilogue
        if constexpr (PAIR == 2) { if (ok) ok = mbar_wait_cl(acc_full, 0u, 0x400u); }
        else { if (ok) ok = mbar_wait(acc_full, 0u, 0x400u); }
        asm volatile("griddepcontrol.wait;" ::: "memory");   // Y may be read by the kernel before this one
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int quarter = warp & 3;            // TMEM lanes 32*quarter .. +31 are this warp's
        const int part = dw >> 2;                // the four warps of a quarter share the BN columns
        // Staging for the TMA store: 4 KB per warp in the (now idle) A and B stages; rows of 128
        // bytes, 16-byte chunks XOR-swizzled with the row index (the Y tensor map's swizzle).
        // (the host checks that the X and operand stages together hold the 64 KB of staging)
        const uint32_t stg = sA + (uint32_t)dw * 4096u;
        // Split-K: CTAs 1 .. KS-1 park their accumulators in their (idle) X, operand and slab stages, 4 KB
        // per (accumulator, 32-column chunk, lane quarter), and tell CTA 0; CTA 0 adds them in below, in
        // rank order.
        uint32_t peer_xfer[KS > 1 ? KS - 1 : 1] = {};
        auto xfer_off = [&](int mt, int c32) { return (uint32_t)(((mt * (BNU / 32) + c32) * 4 + quarter) * 4096); };
        auto add_peers = [&](int mt, int c32, uint32_t (&v)[32]) {
#pragma unroll
            for (int r = 0; r < KS - 1; r++) add_xfer(peer_xfer[r] + xfer_off(mt, c32), lane, v);
        };
        if constexpr (KS > 1) {
            if (krank != 0) {
#pragma unroll 1
                for (int mt = 0; mt < MT; mt++)
#pragma unroll 1
                    for (int c32 = part; c32 < BNU / 32; c32 += 4) {
                        uint32_t v[32];
                        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * BNU + c32 * 32), v);
                        store_xfer(sA + xfer_off(mt, c32), lane, v);
                    }
                asm volatile("fence.acq_rel.cluster;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_cl(mapa_u32(xfer_full, 0u));
            } else {
                if (ok) ok = mbar_wait_cl(xfer_full, 0u, 0x2000u);
#pragma unroll
                for (int r = 0; r < KS - 1; r++) peer_xfer[r] = mapa_u32(sA, (uint32_t)(r + 1));
            }
        }
#pragma unroll 1
        for (int mt = 0; mt < ((KS > 1 && krank != 0) ? 0 : MT); mt++) {
            const int mrow0 = m0 + (mt * PAIR + rank) * 128 + quarter * 32;
            const long m = (long)mrow0 + lane;
            if (p.tma_store && p.out_f16) {
              // 64-column x 32-row boxes of fp16
#pragma unroll 1
              for (int c64 = part; c64 < BNU / 64; c64 += 4) {
                uint32_t v[32], w[32];
                const int col = c64 * 64;
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * BNU + col), v);
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * BNU + col + 32), w);
                if constexpr (KS > 1) {
                    add_peers(mt, 2 * c64, v);
                    add_peers(mt, 2 * c64 + 1, w);
                }
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                __syncwarp();
                uint32_t h[32];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    // inverse of col_of on the 8-group: accumulator index of output column c
                    const int a0 = (c & ~7) | ((((c & 7) & 1) << 2) | ((c & 7) >> 1));
                    const int a1 = ((c + 1) & ~7) | (((((c + 1) & 7) & 1) << 2) | (((c + 1) & 7) >> 1));
                    __half2 lo = __floats2half2_rn(__uint_as_float(v[a0]), __uint_as_float(v[a1]));
                    __half2 hi = __floats2half2_rn(__uint_as_float(w[a0]), __uint_as_float(w[a1]));
                    h[c / 2] = *reinterpret_cast<uint32_t*>(&lo);
                    h[16 + c / 2] = *reinterpret_cast<uint32_t*>(&hi);
                }
#pragma unroll
                for (int q = 0; q < 8; q++)
                    sts128(stg + lane * 128 + (((uint32_t)q ^ ((uint32_t)lane & 7u)) << 4),
                           make_uint4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]));
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) tma_store_2d(ymap, stg, n0 + col, mrow0);
              }
            } else {
#pragma unroll 1
                for (int c32 = part; c32 < BNU / 32; c32 += 4) {
                    const int col = c32 * 32;
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * BNU + col), v);
                    if constexpr (KS > 1) add_peers(mt, c32, v);
                    if (p.tma_store) {
                        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // staging free again
                        __syncwarp();
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            // output columns 4q..4q+3 <- accumulator columns rho(g) of the same 8-group
                            const int c0 = 4 * q;
                            const int a0 = (c0 & ~7) | ((((c0 & 7) & 1) << 2) | ((c0 & 7) >> 1));
                            const int a1 = ((c0 + 1) & ~7) | (((((c0 + 1) & 7) & 1) << 2) | (((c0 + 1) & 7) >> 1));
                            const int a2 = ((c0 + 2) & ~7) | (((((c0 + 2) & 7) & 1) << 2) | (((c0 + 2) & 7) >> 1));
                            const int a3 = ((c0 + 3) & ~7) | (((((c0 + 3) & 7) & 1) << 2) | (((c0 + 3) & 7) >> 1));
                            sts128(stg + lane * 128 + (((uint32_t)q ^ ((uint32_t)lane & 7u)) << 4),
                                   make_uint4(v[a0], v[a1], v[a2], v[a3]));
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) tma_store_2d(ymap, stg, n0 + col, mrow0);
                    } else if (m < p.M) {
                        // rows of Y are not 16-byte multiples: plain guarded stores
                        const int n = n0 + col;
                        for (int c = 0; c < 32; c++) {
                            const int a = (c & ~7) | ((((c & 7) & 1) << 2) | ((c & 7) >> 1));
                            if (n + c < mat_N) {
                                if (p.out_f16)
                                    reinterpret_cast<__half*>(mat_y)[m * mat_N + n + c] = __float2half_rn(__uint_as_float(v[a]));
                                else
                                    reinterpret_cast<float*>(mat_y)[m * mat_N + n + c] = __uint_as_float(v[a]);
                            }
                        }
                    }
                }
            }
        }
        if (p.tma_store && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    // PAIR == 2: neither CTA may free its tensor memory or leave (its shared memory is read by
    // the pair's MMAs and its barriers are arrived on remotely) before both are done.
    if constexpr (PAIR == 2 || KS > 1) cluster_sync_all();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if constexpr (PAIR == 2)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace tc

// =================================================================== host side
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    }
    return fn;
}

size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

int launch_pca_table(int nmat, const float* const* bases, const float* const* scales, int n_cb, __half* pb,
                     cudaStream_t stream) {
    tc::TableArgs ta = {};
    for (int i = 0; i < nmat; i++) { ta.bases[i] = bases[i]; ta.scales[i] = scales[i]; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((n_cb * 64 + 255) / 256), (unsigned)nmat, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, tc::pca_table_kernel, ta, n_cb, pb);
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(pca_table_kernel)");
    return SX8_OK;
}

__global__ void __launch_bounds__(256)
xstage_kernel(const __half* __restrict__ x, int M, int K, long ldx, int Kp, __half* __restrict__ out) {
    long i = (long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long)M * Kp) return;
    int m = (int)(i / Kp), k = (int)(i - (long)m * Kp);
    out[i] = (k < K) ? x[(long)m * ldx + k] : __float2half_rn(0.0f);
}

// Tensor map of Y for the epilogue's TMA stores: boxes of 32 rows x 128 bytes (32 f32 or 64 f16
// columns), 128-byte swizzle.  Returns false when Y's rows are not 16-byte multiples.
bool make_ymap(CUtensorMap* map, void* y, int M, int N, int out_f16) {
    const size_t es = out_f16 ? 2 : 4;
    if (((size_t)N * es) % 16 != 0 || (reinterpret_cast<uintptr_t>(y) % 16) != 0) return false;
    cuuint64_t gdim[2] = {(cuuint64_t)N, (cuuint64_t)M};
    cuuint64_t gstr[1] = {(cuuint64_t)N * es};
    cuuint32_t box[2] = {out_f16 ? 64u : 32u, 32u};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = encode_fn()(map, out_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, y,
                             gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int MT, int BN, int PAIR, int G = 2, int KS = 1>
int launch_tc_bn(const CUtensorMap& map, tc::Params p, cudaStream_t stream) {
    using C = tc::Cfg<MT, BN, PAIR>;
    CUtensorMap ymap[tc::kMaxMats], wmap[tc::kMaxMats];
    memset(ymap, 0, sizeof(ymap));
    memset(wmap, 0, sizeof(wmap));
    p.tma_store = 1;   // only if every matrix's Y can be addressed by a tensor map
    for (int i = 0; i < p.nmat; i++)
        if (!make_ymap(&ymap[i], p.mat[i].y, p.M, p.mat[i].N, p.out_f16)) p.tma_store = 0;
    for (int i = 1; i < p.nmat; i++)
        if (p.mat[i].col0 % C::BNU != 0) {
            set_error("sx8_gemm: matrix %d starts at column %d, not a multiple of the %d-column tile", i, p.mat[i].col0, C::BNU);
            return SX8_E_INVALID;
        }
    // Pipeline depths.  The packed slabs come from HBM with the longest latency and get every
    // stage that is left (at most 8); X tiles come from L2.
    static const int env_sa = exp_env("SX8_GEMM_SA", 0);
    static const int env_sb = exp_env("SX8_GEMM_SB", 0);
    static const int env_sp = exp_env("SX8_GEMM_SP", 0);
    static const int env_debug = exp_env("SX8_GEMM_DEBUG", 0);
    p.debug = env_debug;
    p.sa = env_sa > 0 ? env_sa : 3;
    p.sb = env_sb > 0 ? env_sb : ((BN >= 256) ? 2 : (PAIR == 2 ? 4 : 3));
    if (env_sp > 0) {
        p.sp = env_sp;
    } else {
        p.sp = 8;
        while (p.sp > 2 && C::smem_bytes(p.sa, p.sb, p.sp) > tc::kSmemMax) p.sp--;
    }
    const int smem = C::smem_bytes(p.sa, p.sb, p.sp);
    if (p.sa < 2 || p.sb < 2 || p.sp < 2 || smem > tc::kSmemMax ||
        p.sa * MT * tc::A_TILE + p.sb * C::B_TILE < tc::kDecodeWarps * 4096) {
        set_error("sx8_gemm: pipeline depths (%d, %d, %d) do not fit shared memory", p.sa, p.sb, p.sp);
        return SX8_E_UNSUPPORTED;
    }
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        e = cudaFuncSetAttribute(tc::gemm_tc_kernel<MT, BN, PAIR, G, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 tc::kSmemMax);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemm_tc smem)");
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    for (int i = 0; i < p.nmat; i++) {
        cuuint64_t gdim[2] = {(cuuint64_t)p.n_cb * (T16_UNIT / 4), (cuuint64_t)p.mat[i].n_tiles};
        cuuint64_t gstr[1] = {(cuuint64_t)p.n_cb * T16_UNIT};
        cuuint32_t box[2] = {(cuuint32_t)(tc::KB_STAGE * T16_UNIT / 4), (cuuint32_t)C::TILES};
        cuuint32_t estr[2] = {1u, 1u};
        CUresult r = encode_fn()(&wmap[i], CU_TENSOR_MAP_DATA_TYPE_INT32, 2, (void*)p.mat[i].blob, gdim, gstr, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            set_error("sx8_gemm: cuTensorMapEncodeTiled(blob) failed (%d)", (int)r);
            return SX8_E_CUDA;
        }
    }
    // (the hand-over may run on from the X and operand stages into the slab stages: all idle by then)
    if (KS > 1 && p.sa * MT * tc::A_TILE + p.sb * C::B_TILE + p.sp * C::P_STAGE < MT * C::BNU * 512) {
        set_error("sx8_gemm: split-K hand-over does not fit the pipeline stages");
        return SX8_E_UNSUPPORTED;
    }
    dim3 grid((unsigned)(PAIR * KS * ((p.N + C::BNU - 1) / C::BNU)),
              (unsigned)((p.M + 128 * MT * PAIR - 1) / (128 * MT * PAIR)), 1);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(tc::kThreads, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see the kernel: weights are prefetched under the kernel ahead
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    na++;
    if (PAIR * KS > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = PAIR * KS;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    e = cudaLaunchKernelEx(&cfg, tc::gemm_tc_kernel<MT, BN, PAIR, G, KS>, map, ymap[0], ymap[1], ymap[2], wmap[0], wmap[1],
                           wmap[2], p);
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(gemm_tc_kernel)");
    return SX8_OK;
}

// Columns per CTA: the widest tile (most reuse of each decoded weight and each X tile), narrowed
// only while twice as many CTAs still fit in one wave -- a second wave costs more than it gains.
template <int MT>
int launch_tc(const CUtensorMap& map, const tc::Params& p, cudaStream_t stream) {
    static const int force_bn = exp_env("SX8_GEMM_BN", 0);
    const long mtiles = (p.M + 128 * MT - 1) / (128 * MT);
    int bn = 256;
    if (((p.N + 127) / 128) * mtiles <= 148) bn = 128;
    // Split-K over a cluster of two when the 128-column tiles leave at least half of the SMs
    // idle (74 two-SM clusters fit at once) and K is long enough to halve: 9472 x 2560 at
    // M = 128 runs in 28.8 us against 35.0, 2560 x 9728 in 61.7 against 86.4 with 64-column
    // tiles (SX8_GEMM_KSPLIT=0 switches it off).
    // Over a cluster of four when even that fills at most half of the SMs and K is long: the
    // hand-over of three accumulator sets has to be paid for by the stages saved (2560 x 9728 at
    // M = 32: 58 -> 43 us, 2560 x 4096: 29 -> 27 us; with K = 2560 it loses: 22 -> 24 us; with two
    // accumulators per CTA it pays from K = 8192 on).
    static const int ksplit = exp_env("SX8_GEMM_KSPLIT", 1);
    const long tiles128 = (long)((p.N + 127) / 128) * mtiles;
    const bool can_split = ksplit && tiles128 <= 74 && p.n_cb >= 32;
    const bool can_split4 = ksplit != 2 && can_split && tiles128 <= 37 && p.n_cb >= (MT == 1 ? 128 : 256);
    if (bn == 128 && !can_split && ((p.N + 63) / 64) * mtiles <= 148 && tiles128 <= 37) bn = 64;
    if (force_bn == 64 || force_bn == 128 || force_bn == 256) bn = force_bn;
    if (bn == 128 && can_split4) return launch_tc_bn<MT, 128, 1, 2, 4>(map, p, stream);
    if (bn == 128 && can_split) return launch_tc_bn<MT, 128, 1, 2, 2>(map, p, stream);
    if (bn == 256) return launch_tc_bn<MT, 256, 1>(map, p, stream);
    if (bn == 128) return launch_tc_bn<MT, 128, 1>(map, p, stream);
    return launch_tc_bn<MT, 64, 1>(map, p, stream);
}

// Shape rule.  Two-CTA tiles (512 rows x 256 columns per pair) halve the decode work and the
// operand reads per MMA and win as soon as M fills them; up to 256 rows the one-CTA tiles.
// SX8_GEMM_PAIR overrides for experiments: 0 = never pair, 2 = always 512-row pairs,
// 3 = always 256-row pairs.
int launch_auto(const CUtensorMap& map, const tc::Params& p, cudaStream_t stream) {
    static const int pair_mode = exp_env("SX8_GEMM_PAIR", 1);
    static const int force_mt = exp_env("SX8_GEMM_MT", 0);
    if (pair_mode == 3) return launch_tc_bn<1, 128, 2>(map, p, stream);
    static const int groups = exp_env("SX8_GEMM_GROUPS", 4);
    if (pair_mode == 1 && p.M > 256) {
        // Narrow matrices at a few hundred rows give the 512 x 256 pair tiles too few CTAs (1024 x 2560
        // at M = 2048: 32 of 148 SMs; 2560 x 9728 at M = 512: 20).  The one-CTA 256 x 128 tiles, with
        // their split-K over a cluster of two when at most 74 tiles exist, then fill the GPU in one
        // wave and halve the decode work per CTA.
        const long pair_ctas = 2L * ((p.N + 255) / 256) * ((p.M + 511) / 512);
        const long one_tiles = (long)((p.N + 127) / 128) * ((p.M + 255) / 256);
        const long one_ctas = (one_tiles <= 37 && p.n_cb >= 256) ? 4 * one_tiles
                              : ((one_tiles <= 74 && p.n_cb >= 32) ? 2 * one_tiles : one_tiles);   // launch_tc's split-K
        if (pair_ctas < 100 && one_ctas <= 148 && one_ctas > pair_ctas) return launch_tc<2>(map, p, stream);
    }
    if (pair_mode == 2 || (pair_mode == 1 && p.M > 256)) {
        if (groups == 2) return launch_tc_bn<2, 128, 2, 2>(map, p, stream);
        return launch_tc_bn<2, 128, 2, 4>(map, p, stream);
    }
    if (force_mt == 1) return launch_tc<1>(map, p, stream);
    if (p.M > 128) return launch_tc<2>(map, p, stream);
    return launch_tc<1>(map, p, stream);
}

}  // namespace

size_t gemm_tc_multi_workspace_bytes(int M, int n_cb, int nmat);
size_t gemm_tc_workspace_bytes(int M, int N, int n_cb) {
    (void)N;
    return gemm_tc_multi_workspace_bytes(M, n_cb, 1);
}

bool gemm_tc_supported(int M, int N, int K, int n_cb) {
    (void)N; (void)K; (void)n_cb;
    return M >= 1 && encode_fn() != nullptr;
}

// X tensor map; stages x through the workspace when a tensor map cannot address it as it is.
static int make_xmap(CUtensorMap* map, const void* x, int M, int K, long ldx, int n_cb, void* xstage, cudaStream_t stream) {
    const __half* xp = (const __half*)x;
    long ld = ldx;
    int Kx = K;
    if ((ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x) % 16) != 0) {
        if (!xstage) {
            set_error("sx8_gemm: x must be 16-byte aligned with a row stride that is a multiple of 8 elements");
            return SX8_E_INVALID;
        }
        int Kp = n_cb * 32;
        xstage_kernel<<<(unsigned)(((long)M * Kp + 255) / 256), 256, 0, stream>>>((const __half*)x, M, K, ldx, Kp, (__half*)xstage);
        SX8_LAUNCH_CHECK("xstage_kernel");
        xp = (const __half*)xstage; ld = Kp; Kx = Kp;
    }
    cuuint64_t gdim[2] = {(cuuint64_t)Kx, (cuuint64_t)M};
    cuuint64_t gstr[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)tc::BK, 128u};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)xp, gdim, gstr, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("sx8_gemm: cuTensorMapEncodeTiled failed (%d)", (int)r);
        return SX8_E_CUDA;
    }
    return SX8_OK;
}

// workspace: [PCA tables, n_cb*128 B per matrix][staged x (M, 32*n_cb) f16, only when x is not TMA-addressable]
size_t gemm_tc_multi_workspace_bytes(int M, int n_cb, int nmat) {
    return round256((size_t)nmat * n_cb * 128) + round256((size_t)M * (size_t)n_cb * 64);
}

// nmat <= 3 matrices with the same K on the same x; N[i] columns each, all but the last a multiple of 256.
int gemm_tc_launch_multi(const void* x, int M, int K, long ldx, int nmat, const void* const* wt16,
                         const float* const* bases, const float* const* scales, const int* N, int n_cb,
                         void* const* y, int out_f16, void* workspace, cudaStream_t stream) {
    __half* pb = (__half*)workspace;
    int rc = launch_pca_table(nmat, bases, scales, n_cb, pb, stream);
    if (rc != SX8_OK) return rc;
    CUtensorMap map;
    rc = make_xmap(&map, x, M, K, ldx, n_cb, (uint8_t*)workspace + round256((size_t)nmat * n_cb * 128), stream);
    if (rc != SX8_OK) return rc;
    tc::Params p = {};
    p.pb = pb;
    p.nmat = nmat;
    int col = 0;
    for (int i = 0; i < nmat; i++) {
        p.mat[i] = tc::Mat{(const uint8_t*)wt16[i], y[i], col, N[i], (int)t16_tiles(N[i])};
        col += N[i];
    }
    p.M = M; p.N = col; p.n_cb = n_cb; p.out_f16 = out_f16;
    return launch_auto(map, p, stream);
}

int gemm_tc_launch(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                   const float* scales, int N, int n_cb, void* y, int out_f16, void* workspace,
                   cudaStream_t stream) {
    return gemm_tc_launch_multi(x, M, K, ldx, 1, &wt16, &bases, &scales, &N, n_cb, &y, out_f16, workspace, stream);
}

}  // namespace sx8

// =================================================================== allocation-free variant
// sx8_gemm_static: the tensor-core GEMM with its scratch (the fp16 PCA table) held in a
// fixed array inside the library image instead of a caller-supplied workspace.  Meant for
// hosts that may not allocate device memory at all once they are running -- a serving
// process that handed its whole memory budget to its own arena at start-up, or a plug-in
// host that forbids cudaMalloc in plug-ins because an allocation synchronises the device
// and can fail late.  Such a caller passes inputs and outputs only.
//
// The array costs kStaticPcaBytes of device memory on every GPU that loads the library,
// until the process exits.  It is shared by every call and keeps the previous call's
// contents; each call rewrites the part it uses (n_cb * 128 bytes) before reading it, so
// nothing has to start at zero -- but two calls that overlap on the GPU (different
// streams, or different threads) would overwrite each other's table: callers must order
// them.  The device address of the array is looked up once per device by the first call
// made with that device current; make that first call before starting any stream capture.
namespace sx8 {
namespace {

constexpr int kStaticMaxNcb = 1024;                       // K <= 32768
constexpr size_t kStaticPcaBytes = (size_t)kStaticMaxNcb * 128;
static __device__ __align__(256) unsigned char g_static_pca[kStaticPcaBytes];

// In host code `g_static_pca` is only a handle for the runtime, not a device address:
// the address is obtained per device with cudaGetSymbolAddress and cached.
int static_pca_ptr(__half** out) {
    static std::atomic<void*> cache[64] = {};   // written once per device, possibly from several host threads
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) {
        set_error("sx8_gemm_static: device index %d out of range", dev);
        return SX8_E_UNSUPPORTED;
    }
    void* ptr = cache[dev].load(std::memory_order_acquire);
    if (!ptr) {
        e = cudaGetSymbolAddress(&ptr, g_static_pca);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static PCA table)");
        cache[dev].store(ptr, std::memory_order_release);   // every thread looks up the same address
    }
    *out = (__half*)ptr;
    return SX8_OK;
}

}  // namespace
}  // namespace sx8

extern "C" size_t sx8_gemm_static_max_ncb(void) { return (size_t)sx8::kStaticMaxNcb; }

extern "C" int sx8_gemm_static(const void* x, int M, int K, long ldx, const void* wt16, const float* bases,
                               const float* scales, int N, int n_cb, void* y, int out_f16, void* stream_) {
    using namespace sx8;
    cudaStream_t stream = (cudaStream_t)stream_;
    SX8_REQUIRE(x && wt16 && bases && scales && y, "sx8_gemm_static: null pointer");
    SX8_REQUIRE(M >= 1 && N > 0 && K > 0 && n_cb == (K + 31) / 32,
                "sx8_gemm_static: need M>=1, N>0, K>0, n_cb == ceil(K/32) (got M=%d N=%d K=%d n_cb=%d)", M, N, K, n_cb);
    SX8_REQUIRE(n_cb <= kStaticMaxNcb,
                "sx8_gemm_static: n_cb=%d exceeds the built-in scratch (max n_cb %d, i.e. K <= %d); use sx8_gemm "
                "with a caller workspace", n_cb, kStaticMaxNcb, kStaticMaxNcb * 32);
    SX8_REQUIRE(ldx >= K, "sx8_gemm_static: ldx (%ld) < K (%d)", ldx, K);
    SX8_REQUIRE((ldx % 8) == 0 && (reinterpret_cast<uintptr_t>(x) % 16) == 0,
                "sx8_gemm_static: x must be 16-byte aligned with a row stride that is a multiple of 8 elements "
                "(no scratch is available to stage it); got ldx=%ld", ldx);
    SX8_REQUIRE((reinterpret_cast<uintptr_t>(wt16) % 16) == 0 && (reinterpret_cast<uintptr_t>(bases) % 4) == 0 &&
                    (reinterpret_cast<uintptr_t>(scales) % 4) == 0 &&
                    (reinterpret_cast<uintptr_t>(y) % (out_f16 ? 2 : 4)) == 0,
                "sx8_gemm_static: misaligned wt16 / bases / scales / y");
    if (!encode_fn()) {
        set_error("sx8_gemm_static: the driver does not provide cuTensorMapEncodeTiled");
        return SX8_E_UNSUPPORTED;
    }
    __half* pb = nullptr;
    int rc = static_pca_ptr(&pb);
    if (rc != SX8_OK) return rc;
    rc = launch_pca_table(1, &bases, &scales, n_cb, pb, stream);
    if (rc != SX8_OK) return rc;
    CUtensorMap map;
    rc = make_xmap(&map, x, M, K, ldx, n_cb, nullptr, stream);   // (alignment was checked above: nothing to stage)
    if (rc != SX8_OK) return rc;
    tc::Params p = {};
    p.pb = pb;
    p.nmat = 1;
    p.mat[0] = tc::Mat{(const uint8_t*)wt16, y, 0, N, (int)t16_tiles(N)};
    p.M = M; p.N = N; p.n_cb = n_cb; p.out_f16 = out_f16;
    return launch_auto(map, p, stream);
}
