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
 * Device layouts (ref: scripts/prepare_v44.py:35-79, "v4.4", kb-major, bid = kb*N + n):
 *   hdr     (n_cb*N, hdr_bytes) u8 : dmin f16 | dmax f16 | config u8 | coeff u8 [| 2 pad]
 *   levels  (n_cb*N, 24)        u8 : hi nibbles of sub-block 0..3 (4 B each), then
 *                                    lo pairs of sub-block 0..3 (2 B each)
 *   bases   (n_cb, 64) f32, scales (n_cb, 2) f32
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
 * included), fp32 accumulate.   x: (M, ldx) f16, row stride ldx >= n_cb*32 halfs is
 * not required: columns k >= K are treated as zero.   y: (M, N) f32 row-major.
 * Replaces ref: cuda/sx8_decode1_v3.cu:185-246 (compute_z44, decode1_v44,
 * decode1_v44_combined) and, for M in 2..8, the small-M use of
 * ref: cuda/sx8_gemm_compact.cu:157-194.
 * workspace: sx8_gemv_workspace_bytes(n_cb, M) bytes of device scratch, 256-byte
 * aligned, private to this call until it completes on the stream.
 * flags: SX8_F_PDL launches the main kernel with programmatic dependent launch so
 * that its weight prefetch overlaps the preceding kernel on the stream.
 * Requires N % 8 == 0 and hdr_bytes in {6, 8}.                                      */
#define SX8_F_PDL 1u
size_t sx8_gemv_workspace_bytes(int n_cb, int M);
int sx8_gemv(const void* x_f16, int M, int K, long ldx, const void* hdr, const void* levels,
             const float* bases, const float* scales, int N, int n_cb, int hdr_bytes,
             float* y, void* workspace, size_t workspace_bytes, unsigned flags, void* stream);

/* ---- prefill GEMM, any M ----------------------------------------------------------
 * Y (M, N) = X (M, K) * W^T, fp32 accumulate; out_f16 != 0 writes Y as f16, else f32.
 * Replaces ref: cuda/sx8_gemm_compact.cu:157-194 (compute_z44_batch, gemm_compact) and
 * ref: cuda/sx8_fused_wmma.cu:134-154 (fused_forward).                               */
size_t sx8_gemm_workspace_bytes(int M, int N, int n_cb);
int sx8_gemm(const void* x_f16, int M, int K, long ldx, const void* hdr, const void* levels,
             const float* bases, const float* scales, int N, int n_cb, int hdr_bytes,
             void* y, int out_f16, void* workspace, size_t workspace_bytes, void* stream);

/* ---- embedding rows ---------------------------------------------------------------
 * out[t, 0..K) = f16(decode(row ids[t])) in the reference kernel's float32 arithmetic.
 * Replaces ref: cuda/sx8_embed_v44.cu:80-94 (sx8_embed_v44).  ids: (T) int64 on the
 * device.  Rows with id outside [0, N) are written as zeros (the reference leaves them
 * untouched and does not guard negative ids).                                        */
int sx8_embed(const int64_t* ids, long T, const void* hdr, const void* levels,
              const float* bases, const float* scales, int K, int N, int n_cb, int hdr_bytes,
              void* out_f16, void* stream);

/* ---- full-tensor dequantisation ---------------------------------------------------
 * out (out_f, in_f) f16 = the reference decoder's result: float64 arithmetic, float32
 * rounding, then f16.  Replaces ref: scripts/kernel_sx8_v43.py:14-51,109-145
 * (sx8_v43_kernel / decode_tensor_gpu_fast).  Inputs are the n-major file planes.    */
int sx8_dequant_planes(const void* dmin_f16, const void* dmax_f16, const uint8_t* config,
                       const uint8_t* coeff, const uint8_t* levels_hi, const uint8_t* levels_lo,
                       const float* bases, const float* scales, long out_f, long in_f, int n_cb,
                       int use_pca, void* out_f16, void* stream);
/* Same result from the kb-major device layout. */
int sx8_dequant_v44(const void* hdr, const void* levels, const float* bases, const float* scales,
                    long out_f, long in_f, int n_cb, int hdr_bytes, int use_pca, void* out_f16,
                    void* stream);

/* ---- quantizer: per-block strategy search + bit packing ---------------------------
 * w: (out_f, in_f) row-major, f16 (w_is_f16 != 0) or f32, zero-padded on the fly to
 * n_cb*32 columns.  Writes the n-major file planes dmin/dmax (f16), config, levels_hi,
 * levels_lo, and optionally the unpacked levels (n_blk, 32) u8 (may be NULL).
 * Bit-exact restatement of ref: scripts/quantize_qwen35_4b_sx8_v43_gpu.py:22-69
 * (v6_encode_6bit_gpu / chunked_v6_encode), :148-167 (pack_levels_6bit), :258-260.   */
int sx8_quantize_blocks(const void* w, int w_is_f16, long out_f, long in_f, long ldw,
                        void* dmin_f16, void* dmax_f16, uint8_t* config, uint8_t* levels_hi,
                        uint8_t* levels_lo, uint8_t* levels_u8, void* stream);

/* ---- file planes -> device layout -------------------------------------------------
 * Replaces ref: scripts/prepare_v44.py:35-79 (to_v44), done on the device.           */
int sx8_repack_v44(const void* dmin_f16, const void* dmax_f16, const uint8_t* config,
                   const uint8_t* coeff, const uint8_t* levels_hi, const uint8_t* levels_lo,
                   long out_f, int n_cb, int hdr_bytes, void* hdr_out, void* levels_out,
                   void* stream);

/* Device-side error word of the bounded waits inside the pipelined kernels: 0 when no
 * wait ever ran out.  Reads back synchronously (cudaMemcpy) -- for tests and health
 * checks, not for the hot path.                                                      */
int sx8_device_error_flag(unsigned* flag_out);

#ifdef __cplusplus
}
#endif
#endif /* SX8_B200_H */
