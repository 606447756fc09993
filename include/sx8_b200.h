/* sx8_b200.h -- C ABI of libsx8b200.so: the S-X8 v4.3 hot path on NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as
 * void*, a cudaStream_t), launches asynchronously on that stream, performs no
 * synchronisation and allocates no memory.  Return value: 0 on success, a negative
 * SX8_E_* code on a rejected call (nothing was launched); sx8_last_error() gives the
 * message of the calling thread's last failure.  Arguments are validated on the
 * host; the reference's extension performs no checks at all.
 *
 * Paths cited as "ref:" are files of the reference project
 * (MarlaLabsAI/sx8-quantization) whose interface the entry point replaces.
 *
 * Device layout "T16" (this library's own; a byte/bit permutation of the reference's
 * 30-byte block, docs/SX8_FLASH_V4_3_SPEC.md:13-25 -- still exactly 30 bytes per block):
 *   wt16 = blob of ceil(N/16) * n_cb units of 480 bytes, unit (T, kb) at (T*n_cb + kb)*480,
 *   holding block row kb of columns 16T..16T+15 (zero blocks past N).  Lane L = 4g+t
 *   (g = 0..7, t = 0..3) owns sub-block t of column A = 16T+g and B = 16T+g+8; with
 *   a_i / b_i the 6-bit level of weight 8t+i:
 *     W0 @ +0   +4L : bytes [a0,a2,a1,a3] << 2 | bits 1:0 of [b4,b6,b5,b7]
 *     W1 @ +128 +4L : bytes [a4,a6,a5,a7] << 2 | bits 3:2 of [b4,b6,b5,b7]
 *     W2 @ +256 +4L : bytes [b0,b2,b1,b3] << 2 | bits 5:4 of [b4,b6,b5,b7]
 *     H0[g] @ +384+4g : dmin(A) | dmax(A)<<16 ; H1[g] @ +416+4g : same for B ;
 *     H2[g] @ +448+4g : c0(A) | c0(B)<<4 | config(A)<<8 | c1(A)<<16 | c1(B)<<20 | config(B)<<24
 *                       (c0 / c1 = low / high nibble of the coeff byte)
 *   It replaces the reference's kb-major "v4.4" pair hdr (n_blk,6) + levels (n_blk,24)
 *   (ref: scripts/prepare_v44.py:35-79), which sx8_repack_v44 still produces for
 *   interchange.  bases (n_cb, 64) f32 and scales (n_cb, 2) f32 are as in the reference.
 * File planes (ref: scripts/sx8_container_v43.py:30-38, "v4.3", n-major, bid = n*n_cb + kb):
 *   dmin, dmax (n_blk) f16; config (n_blk) u8; levels_hi (n_blk*16) u8;
 *   levels_lo (n_blk*8) u8; coeff (n_blk) u8.
 */
#ifndef SX8_B200_H
#define SX8_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SX8_OK 0
#define SX8_E_INVALID (-1)   /* bad argument: null pointer, size, alignment, range */
#define SX8_E_WORKSPACE (-2) /* workspace missing or too small */
#define SX8_E_CUDA (-3)      /* a CUDA runtime call failed */
#define SX8_E_UNSUPPORTED (-4)

#define SX8_GEMV_MAX_BATCH 8

/* Library version (major*10000 + minor*100 + patch). */
int sx8_version(void);

/* Message of the calling thread's last failed call ("" if none). */
const char* sx8_last_error(void);

/* ---- decode GEMV, batch 1..8 ------------------------------------------------------
 * y[m, n] = sum_k x[m, k] * W[n, k] with W decoded on the fly (PCA correction
 * included), fp32 accumulate.   x: (M, K) f16 with row stride ldx (elements); columns
 * k >= K count as zero.   y: (M, N) f32 row-major.
 * Replaces ref: cuda/sx8_decode1_v3.cu:185-246 (compute_z44, decode1_v44,
 * decode1_v44_combined) and, for M in 2..8, the small-M use of
 * ref: cuda/sx8_gemm_compact.cu:157-194.
 * workspace: sx8_gemv_workspace_bytes(n_cb, M) bytes of device scratch, 256-byte
 * aligned, private to this call until it completes on the stream: used to stage x when
 * K is not a multiple of 32 or x is not 16-byte aligned row by row (ldx a multiple of
 * 8).  When x needs no staging the workspace is not touched and may be NULL.
 * flags: SX8_F_PDL launches with programmatic dependent launch so that the weight
 * prefetch overlaps the preceding kernel on the stream.
 * Requires n_cb <= 1024.                                                             */
#define SX8_F_PDL 1u
size_t sx8_gemv_workspace_bytes(int n_cb, int M);
int sx8_gemv(const void* x_f16, int M, int K, long ldx, const void* wt16, const float* bases,
             const float* scales, int N, int n_cb, float* y, void* workspace,
             size_t workspace_bytes, unsigned flags, void* stream);

/* ---- several decode GEMVs on the same activations, one launch ----------------------
 * No counterpart in the reference (it launches every projection separately; fused
 * multi-projection launches are its stated next step, ref: CHANGELOG.md:21-23).  y[i] =
 * x * W_i^T for count <= 4 matrices with the same K (q|k|v, gate|up): one kernel, one pass
 * over x, tile groups of all matrices scheduled together.  Arrays are host arrays of device
 * pointers / sizes.                                                                      */
int sx8_gemv_multi(const void* x_f16, int M, int K, long ldx, int count, const void* const* wt16,
                   const float* const* bases, const float* const* scales, const int* N,
                   float* const* y, int n_cb, void* workspace, size_t workspace_bytes,
                   unsigned flags, void* stream);

/* ---- row-parallel decode GEMV fused with its all-reduce ---------------------------
 * No counterpart in the reference (it has no multi-GPU code).  One rank of a tensor-parallel
 * group computes its partial y over its K range; the GEMV's epilogue stores every finished
 * tile straight into slot `rank` of each peer's receive buffer (plain stores to peer-mapped
 * memory over NVLink, overlapping the rest of the GEMV) and bumps the peer's arrival counter;
 * a small second kernel waits -- bounded -- for all ranks' tiles and sums the slots in rank
 * order (deterministic) into y, which then holds the full sum on every rank.
 * peers: data[q]  = rank q's receive buffer as mapped in THIS process, 2*world*slot_elems f32
 *                   (two parities x world slots), 16-byte aligned;
 *        flags[q] = rank q's four u32 counters {arrive[2], done[2]}, zero before first use;
 *        parity   = call counter & 1, advanced by the caller on every call that shares the
 *                   buffers (all ranks make the same calls in the same order);
 *        slot_elems >= M*N.
 * All ranks must call with the same shapes.  world == 1 degenerates to sx8_gemv.          */
typedef struct sx8_peers {
    void* data[8];
    void* flags[8];
    long slot_elems;
    int rank, world, parity;
} sx8_peers_t;
int sx8_gemv_allreduce(const void* x_f16, int M, int K, long ldx, const void* wt16, const float* bases,
                       const float* scales, int N, int n_cb, float* y, void* workspace,
                       size_t workspace_bytes, unsigned flags, const sx8_peers_t* peers, void* stream);

/* ---- prefill GEMM, any M ----------------------------------------------------------
 * Y (M, N) = X (M, K) * W^T, fp32 accumulate; out_f16 != 0 writes Y as f16, else f32.
 * M <= 16 runs on the GEMV kernel (one pass over the weights), larger M on the tensor cores.
 * Replaces ref: cuda/sx8_gemm_compact.cu:157-194 (compute_z44_batch, gemm_compact) and
 * ref: cuda/sx8_fused_wmma.cu:134-154 (fused_forward).                               */
size_t sx8_gemm_workspace_bytes(int M, int N, int n_cb);
int sx8_gemm(const void* x_f16, int M, int K, long ldx, const void* wt16, const float* bases,
             const float* scales, int N, int n_cb, void* y, int out_f16, void* workspace,
             size_t workspace_bytes, void* stream);

/* ---- several prefill GEMMs on the same activations ---------------------------------
 * No counterpart in the reference (see sx8_gemv_multi).  y[i] (M, N[i]) = X * W_i^T for count <= 3
 * matrices with the same K (q|k|v, gate|up).  When M > 16 and every N[i] but the last is a
 * multiple of 256, all of them run in ONE launch of the tensor-core kernel (their columns side by
 * side in one grid: the small k and v projections no longer leave most SMs idle, and one launch
 * replaces three); when M <= 16 and Y is float32, in one launch of the GEMV kernel; otherwise the
 * call is count calls of sx8_gemm.  Same results either way.
 * Arrays are host arrays of device pointers / sizes.                                   */
size_t sx8_gemm_multi_workspace_bytes(int M, int count, const int* N, int n_cb);
int sx8_gemm_multi(const void* x_f16, int M, int K, long ldx, int count, const void* const* wt16,
                   const float* const* bases, const float* const* scales, const int* N,
                   void* const* y, int out_f16, int n_cb, void* workspace, size_t workspace_bytes,
                   void* stream);

/* ---- prefill GEMM without any workspace -------------------------------------------
 * No counterpart in the reference.  For callers that are not allowed to allocate device
 * memory while running (a server that gave all of its memory to its own arena at
 * start-up, a plug-in host that bans cudaMalloc in plug-ins): same result as sx8_gemm's
 * tensor-core path, but the kernel's scratch lives in a fixed 128 KB array inside the
 * library (held on every GPU that loads the library until the process exits), so the
 * caller passes inputs and outputs only and the call allocates nothing.
 * Limits: n_cb <= sx8_gemm_static_max_ncb() (1024, i.e. K <= 32768), x 16-byte aligned
 * with ldx a multiple of 8; anything else is rejected with SX8_E_INVALID and a message.
 * The array is shared by all calls: calls that overlap on the GPU race on it, so order
 * them (one stream, or events).  The first call on each device looks up the array's
 * device address; make that call before any stream capture begins.                   */
size_t sx8_gemm_static_max_ncb(void);
int sx8_gemm_static(const void* x_f16, int M, int K, long ldx, const void* wt16, const float* bases,
                    const float* scales, int N, int n_cb, void* y, int out_f16, void* stream);

/* ---- embedding rows ---------------------------------------------------------------
 * out[t, 0..K) = f16(decode(row ids[t])) in the reference kernel's float32 arithmetic.
 * Replaces ref: cuda/sx8_embed_v44.cu:80-94 (sx8_embed_v44).  ids: (T) int64 on the
 * device.  Rows with id outside [0, N) are written as zeros (the reference leaves them
 * untouched and does not guard negative ids).                                        */
int sx8_embed(const int64_t* ids, long T, const void* wt16, const float* bases,
              const float* scales, int K, int N, int n_cb, void* out_f16, void* stream);

/* ---- full-tensor dequantisation ---------------------------------------------------
 * out (out_f, in_f) f16 = the reference decoder's result: float64 arithmetic, float32
 * rounding, then f16.  Replaces ref: scripts/kernel_sx8_v43.py:14-51,109-145
 * (sx8_v43_kernel / decode_tensor_gpu_fast).  Inputs are the n-major file planes.    */
int sx8_dequant_planes(const void* dmin_f16, const void* dmax_f16, const uint8_t* config,
                       const uint8_t* coeff, const uint8_t* levels_hi, const uint8_t* levels_lo,
                       const float* bases, const float* scales, long out_f, long in_f, int n_cb,
                       int use_pca, void* out_f16, void* stream);
/* Same result from the T16 device blob. */
int sx8_dequant_t16(const void* wt16, const float* bases, const float* scales, long out_f,
                    long in_f, int n_cb, int use_pca, void* out_f16, void* stream);

/* ---- quantizer: per-block strategy search + bit packing ---------------------------
 * w: (out_f, in_f) row-major, f16 (w_is_f16 != 0) or f32, zero-padded on the fly to
 * n_cb*32 columns.  Writes the n-major file planes dmin/dmax (f16), config, levels_hi,
 * levels_lo, and optionally the unpacked levels (n_blk, 32) u8 (may be NULL).
 * Bit-exact restatement of ref: scripts/quantize_qwen35_4b_sx8_v43_gpu.py:22-69
 * (v6_encode_6bit_gpu / chunked_v6_encode), :148-167 (pack_levels_6bit), :258-260.
 * arith: the reference is torch eager code whose bits depend on torch's back end in two
 * places (a tensor divided by the host scalar 63, and the summation order of the mean over
 * 8 squared errors).  SX8_ARITH_TORCH_CUDA reproduces the reference as it runs -- on a GPU
 * (ref :9 DEV = cuda) --, SX8_ARITH_TORCH_CPU the same functions run on torch CPU (the
 * arithmetic of golden vectors made without a GPU).  The two differ in about 0.015 % of
 * the levels.                                                                        */
#define SX8_ARITH_TORCH_CUDA 0
#define SX8_ARITH_TORCH_CPU 1
int sx8_quantize_blocks(const void* w, int w_is_f16, long out_f, long in_f, long ldw,
                        void* dmin_f16, void* dmax_f16, uint8_t* config, uint8_t* levels_hi,
                        uint8_t* levels_lo, uint8_t* levels_u8, int arith, void* stream);

/* ---- quantizer: PCA correction stage ----------------------------------------------
 * The three device passes of ref: scripts/quantize_qwen35_4b_sx8_v43_gpu.py:75-142
 * (pca_correct_gpu), over the same w and the planes sx8_quantize_blocks wrote.  The residual
 * E = w - (lo_sb + st_sb * level) (ref :84-97) is recomputed from w and the packed planes inside
 * each kernel and never stored.  Between the passes the caller solves the n_cb symmetric
 * 32 x 32 eigenproblems (the reference calls a batched SVD of E, whose right singular vectors
 * are the eigenvectors of E^T E) and takes the per-column medians of |coef|: small library work.
 *   sx8_pca_gram     gram (n_cb, 32, 32) f64 = sum over rows of E[n][kb]^T E[n][kb]; the sum
 *                    is formed in float32 per chunk of rows and the chunks added in order in
 *                    float64, so it does not depend on scheduling.  scratch: at least
 *                    sx8_pca_gram_scratch_bytes(out_f, in_f) bytes, 16-byte aligned.
 *   sx8_pca_project  coef (n_cb, 2, out_f) f32: coef[kb][j][n] = E[n][kb] . bases[kb][j]
 *                    (bases (n_cb, 2, 32) f32, the file's layout)            (ref :127-128)
 *   sx8_pca_pack     coeff (out_f * n_cb) u8, n-major: signed 4-bit round(coef / scale)
 *                    clamped to -8..7, c0 in the low nibble                 (ref :131-139) */
size_t sx8_pca_gram_scratch_bytes(long out_f, long in_f);
int sx8_pca_gram(const void* w, int w_is_f16, long out_f, long in_f, long ldw, const void* dmin_f16,
                 const void* dmax_f16, const uint8_t* config, const uint8_t* levels_hi,
                 const uint8_t* levels_lo, double* gram, void* scratch, size_t scratch_bytes, void* stream);
int sx8_pca_project(const void* w, int w_is_f16, long out_f, long in_f, long ldw, const void* dmin_f16,
                    const void* dmax_f16, const uint8_t* config, const uint8_t* levels_hi,
                    const uint8_t* levels_lo, const float* bases, float* coef, void* stream);
int sx8_pca_pack(const float* coef, const float* scales, long out_f, int n_cb, uint8_t* coeff, void* stream);

/* ---- file planes -> device layout -------------------------------------------------
 * sx8_repack_t16 replaces ref: scripts/sx8_decode1_v3.py:57-66 (make_tensors_v44) /
 * scripts/prepare_v44.py:35-79 (to_v44) as the load-time transform, done on the device.
 * wt16_out: sx8_t16_bytes(out_f, n_cb) bytes, 16-byte aligned.                        */
size_t sx8_t16_bytes(long N, int n_cb);
int sx8_repack_t16(const void* dmin_f16, const void* dmax_f16, const uint8_t* config,
                   const uint8_t* coeff, const uint8_t* levels_hi, const uint8_t* levels_lo,
                   long out_f, int n_cb, void* wt16_out, void* stream);
/* The reference's own kb-major "v4.4" pair, byte-identical to to_v44
 * (ref: scripts/prepare_v44.py:35-79), for interchange with code that expects it.    */
int sx8_repack_v44(const void* dmin_f16, const void* dmax_f16, const uint8_t* config,
                   const uint8_t* coeff, const uint8_t* levels_hi, const uint8_t* levels_lo,
                   long out_f, int n_cb, int hdr_bytes, void* hdr_out, void* levels_out,
                   void* stream);

/* ---- interleaved 30-byte blocks (GGUF tensor data) -----------------------------------
 * A block_sx8 record is {dmin f16 @0, dmax f16 @2, config @4, qh[16] @5, ql[8] @21,
 * coeff @29}, n-major (bid = n*n_cb + kb): the layout of the llama.cpp fork's GGUF files
 * (ref: scripts/convert_pkl_to_gguf_sx8.py:20-38 blockify_vec; llama-cpp-sx8.patch
 * :136-144 struct block_sx8) and of docs/SX8_FLASH_V4_3_SPEC.md:13-25.
 * sx8_repack_t16_blocks: records -> device layout in one pass (GGUF tensor -> GEMV-ready).
 * sx8_blocks_from_planes / sx8_planes_from_blocks: the container's planes <-> records,
 * byte-exact both ways.  `blocks` must be 2-byte aligned.                              */
int sx8_repack_t16_blocks(const void* blocks, long out_f, int n_cb, void* wt16_out, void* stream);
int sx8_blocks_from_planes(const void* dmin_f16, const void* dmax_f16, const uint8_t* config,
                           const uint8_t* coeff, const uint8_t* levels_hi, const uint8_t* levels_lo,
                           long n_blk, void* blocks_out, void* stream);
int sx8_planes_from_blocks(const void* blocks, long n_blk, void* dmin_f16, void* dmax_f16,
                           uint8_t* config, uint8_t* coeff, uint8_t* levels_hi, uint8_t* levels_lo,
                           void* stream);

/* ---- decoder glue -----------------------------------------------------------------------
 * The small kernels between the S-X8 linears of one decode step, so that a captured step is
 * nine launches per layer.  No counterpart among the reference's kernels: the reference
 * leaves this work to the host framework's model code (it swaps only the Linear / Embedding
 * modules, ref: scripts/integrate_fused_v44.py:85-116).  f32 residual stream and GEMV
 * outputs, f16 activations and KV cache (B, hkv, S, D); `pos` points to one int64 in device
 * memory (the position being written), so a captured graph serves every step.
 *   add_rmsnorm : h += y (y may be NULL); x_out = f16(rmsnorm(h) * gamma)
 *   rope_cache  : rotary embedding (half-split) of q, k at *pos; q_out f16 (B, hq, D); k, v
 *                 written to the caches at *pos; cos_t / sin_t are (S, D/2) f32 tables
 *   attn_decode : softmax(q K^T * scale) V over cache positions 0..*pos; out f16 (B, hq*D);
 *                 D in {64, 128}, hq/hkv in {1, 2, 4, 8}, S <= 1024.  The positions are split
 *                 over 8 CTAs per (sequence, kv head) that merge through `scratch`
 *                 (sx8_glue_attn_scratch_bytes, 16-byte aligned; its first
 *                 B*hkv*4 bytes are arrival counters: zero them once, the kernel leaves
 *                 them zero); calls that share a scratch buffer must be stream-ordered
 *   silu_mul    : act_out = f16(silu(g) * u), n elements                                   */
int sx8_glue_add_rmsnorm(void* h_f32, const void* y_f32, const void* gamma_f32, int B, int H, float eps,
                         void* x_out_f16, void* stream);
int sx8_glue_rope_cache(const void* q_f32, const void* k_f32, const void* v_f32, const void* pos,
                        const void* cos_t, const void* sin_t, int B, int hq, int hkv, int D, int S,
                        void* q_out_f16, void* k_cache_f16, void* v_cache_f16, void* stream);
size_t sx8_glue_attn_scratch_bytes(int B, int hq, int hkv, int D);
int sx8_glue_attn_decode(const void* q_f16, const void* k_cache_f16, const void* v_cache_f16,
                         const void* pos, int B, int hq, int hkv, int D, int S, float scale,
                         void* out_f16, void* scratch, size_t scratch_bytes, void* stream);
int sx8_glue_silu_mul(const void* g_f32, const void* u_f32, long n, void* act_out_f16, void* stream);

/* ---- row-parallel partial sums -> residual + RMSNorm, one kernel over peer memory -----------
 * No counterpart in the reference (it has no multi-GPU code).  The consumer of a row-parallel
 * linear of a tensor-parallel decode step: every rank has written its partial y_r (M, H) f32 --
 * with sx8_gemv / sx8_gemm, straight into slot 0 of half (parity & 1) of ITS OWN exchange buffer
 * (peers->data[rank] + (parity & 1) * world * slot_elems) -- and then calls this on the same
 * stream.  The kernel publishes "my partial of this call is complete" to every peer, waits --
 * bounded -- for the same from every peer, reads all partials from the peers' memory (plain loads
 * over NVLink), sums them in rank order (identical bits on every rank), and does
 *     h += sum;  x_out = f16(rmsnorm(h) * gamma)                       (as sx8_glue_add_rmsnorm).
 * peers->parity selects the half of the buffers, advanced by the caller on every call (all ranks
 * make the same calls in the same order); the calls are counted in device memory, so a CUDA
 * graph that captured an even number of them can be replayed.  peers->flags[q] must hold at
 * least 16 u32, zero before the first call (words 4, 5 and 8..15 are this protocol's, words 0..3
 * sx8_gemv_allreduce's).  A wait that runs out sets bit 3 of the
 * device error word; the exchange is then out of step and must be rebuilt (zero the flags on all
 * ranks, barrier) before it is used again -- the same holds for bit 2 and sx8_gemv_allreduce.    */
int sx8_glue_allreduce_add_rmsnorm(const sx8_peers_t* peers, int M, int H, void* h_f32, const void* gamma_f32,
                                   float eps, void* x_out_f16, void* stream);

/* Device-side error word of the bounded waits inside the pipelined kernels: 0 when no
 * wait ever ran out.  Reads back synchronously (cudaMemcpy) -- for tests and health
 * checks, not for the hot path.                                                      */
int sx8_device_error_flag(unsigned* flag_out);

#ifdef __cplusplus
}
#endif
#endif /* SX8_B200_H */
