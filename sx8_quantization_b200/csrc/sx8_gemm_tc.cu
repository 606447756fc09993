// sx8_gemm_tc.cu -- S-X8 v4.3 prefill GEMM on the 5th-generation tensor cores (sm_100a).
//
//   Y (M, N) = X (M, K) * W^T,  W decoded on the fly from the T16 blob, fp32 accumulate.
//
// CTA tile: 128*MT rows x 256 columns (MT = 1 or 2), K step 64 (two block rows).  Warp roles:
//   warp 0      producer : X tiles by 2-D TMA (128-byte swizzle), packed 16-column slabs of
//                          the blob and the fp16 PCA table by TMA bulk copies
//   warp 1      issuer   : one thread issues tcgen05.mma (M=128, N=256, K=16, kind::f16) on
//                          shared-memory descriptors; accumulators live in TMEM (256 columns
//                          per 128-row tile); tcgen05.commit releases the stages
//   warps 2..9  decoders : bit-extract 6-bit levels from the packed slab, form fp16 weights
//                          w = dmin + base*(mult*level + 63*off) + c0*s0*b0[t] + c1*s1*b1[t]
//                          (the arithmetic of ref cuda/sx8_fused_wmma.cu:83-96, in fp16 pairs)
//                          and store them as the K-major, 128-byte-swizzled B operand tile;
//                          afterwards the same warps read TMEM back (tcgen05.ld) and write Y.
// Every wait on an mbarrier is bounded; a wait that runs out sets the device error word and
// the kernel drains and frees its TMEM.
#include <cuda.h>

#include "sx8_common.cuh"
#include "sx8_layout.cuh"

namespace sx8 {

namespace tc {

constexpr int BN = 256, BK = 64, KB_STAGE = 2;
constexpr int kWarps = 10, kThreads = kWarps * 32, kDecodeWarps = 8;
constexpr int A_TILE = 128 * 128;                 // 128 rows x 64 fp16, bytes
constexpr int B_TILE = BN * 128;                  // 256 rows x 64 fp16
constexpr int P_SLAB = 16 * KB_STAGE * T16_UNIT;  // 16 tiles x 2 kb
constexpr int P_TAB = KB_STAGE * 128;             // PCA table: per kb 2 x 32 fp16
constexpr int P_STAGE = P_SLAB + P_TAB;
constexpr uint32_t kSpin = 1u << 22;

template <int MT>
struct Cfg {
    static constexpr int SA = 3, SB = 2, SP = 3;
    static constexpr int OFF_A = 0;
    static constexpr int OFF_B = OFF_A + SA * MT * A_TILE;
    static constexpr int OFF_P = OFF_B + SB * B_TILE;
    static constexpr int OFF_BAR = OFF_P + SP * P_STAGE;
    static constexpr int N_BAR = 2 * SA + 2 * SB + 2 * SP + 1;
    static constexpr int OFF_TMEM = OFF_BAR + N_BAR * 8;
    static constexpr int SMEM = OFF_TMEM + 16 + 1024;   // + slack to align the base to 1024 B
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
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned code) {
    for (uint32_t i = 0; i < kSpin; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicOr(&g_sx8_error_flag, code);
    return false;
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
// kind::f16 instruction descriptor: D = f32, A = B = f16, both K-major, N = 256, M = 128.
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate) : "memory");
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

// PCA table: pb[kb][j][t] = fp16(scales[kb][j] * bases[kb][32j + t] * 1024), 128 bytes per kb.
// (The coefficient operand carries the matching 2^-10; the pre-scale keeps the products of
// small scales and basis entries out of the fp16 subnormal range.)
__global__ void __launch_bounds__(256)
pca_table_kernel(const float* __restrict__ bases, const float* __restrict__ scales, int n_cb, __half* __restrict__ pb) {
    int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n_cb * 64) return;
    int kb = i >> 6, j = (i >> 5) & 1;
    pb[i] = __float2half_rn(scales[kb * 2 + j] * bases[i] * 1024.0f);
}

struct Params {
    const uint8_t* blob;
    const __half* pb;
    void* y;
    int M, N, n_cb, n_tiles, out_f16;
};
