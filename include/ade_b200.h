/*
 * ade_b200.h -- C ABI of the B200 (sm_100a) delta-application kernels.
 *
 * The library replaces the native half of the reference's src/kernels.py: the two CUDA
 * extensions that file builds at run time (ade_recon_int4, src/kernels.py:383-397, and
 * run_a / run_b / run_ab, src/kernels.py:935-954).  Every entry point takes plain device
 * pointers and sizes, launches on the stream it is given, allocates nothing and returns
 * an int status (0 = ok, negative = rejected before any launch).  Nothing throws across
 * this boundary.
 *
 * All 16-bit floating-point buffers are bfloat16.  "Packed delta" below is the device
 * stored form described at ade_delta_t; it is produced from the six tensors that the
 * reference's src/quantization.py:276-285 writes by ade_b200_pack_* (or by the Python
 * helper ade_b200.kernels.pack_int4, which replaces src/kernels.py:164-188).
 */
#ifndef ADE_B200_H
#define ADE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ADE_B200_GROUP 128          /* ranks per quantization group (G); the only supported value */
#define ADE_B200_MAX_RANK 2048
#define ADE_B200_MAX_BLOCKS 4          /* blocks of a block-diagonal U^ (ade_delta_t.n_blocks) */
#define ADE_B200_MAX_TOKENS 128     /* largest T of the factored path (src/serving.py:105) */

/* return codes */
#define ADE_OK 0
#define ADE_ERR_NULL (-1)           /* a required pointer is NULL */
#define ADE_ERR_SHAPE (-2)          /* a dimension is out of the supported set */
#define ADE_ERR_ALIGN (-3)          /* a pointer is not 16-byte aligned */
#define ADE_ERR_SCRATCH (-4)        /* scratch buffer too small */
#define ADE_ERR_CUDA (-5)           /* a CUDA runtime call failed (see ade_b200_last_cuda_error) */
#define ADE_ERR_DEVICE (-6)         /* current device is not compute capability 10.x */

/* device-side status word values written by the reconstruction kernel (0 = clean run) */
#define ADE_DEV_OK 0
#define ADE_DEV_TIMEOUT_FULL 1      /* MMA warp gave up waiting for an operand stage */
#define ADE_DEV_TIMEOUT_EMPTY 2     /* unpack warps gave up waiting for a free operand stage */
#define ADE_DEV_TIMEOUT_TMEM_FULL 3 /* epilogue gave up waiting for an accumulator */
#define ADE_DEV_TIMEOUT_TMEM_EMPTY 4/* MMA warp gave up waiting for a free accumulator */
#define ADE_DEV_TIMEOUT_SCALES 5     /* epilogue gave up waiting for the scale tables of a tile */
#define ADE_DEV_TIMEOUT_BASE 6       /* epilogue gave up waiting for its box of w_b */
#define ADE_DEV_TIMEOUT_STRIP_FREE 7 /* unpack warps gave up waiting for the resident U strip to retire */
#define ADE_DEV_TIMEOUT_RAW_FULL 8   /* unpack warps gave up waiting for packed codes */
#define ADE_DEV_TIMEOUT_STRIP_FULL 9 /* MMA warp gave up waiting for the resident U strip */
#define ADE_DEV_TIMEOUT_RAW_EMPTY 10 /* load thread gave up waiting for a free raw slot */
#define ADE_DEV_TIMEOUT_SCALES_FREE 11 /* scale warp gave up waiting for a free table buffer */

/*
 * Device stored form of one compressed module (all pointers are device memory, 16-byte
 * aligned).  M = d_o, N = d_i, r = rank (multiple of 128), ng = r / 128.
 *
 *   uq  uint8 [M][r/2]   codes of U^, two per byte, packed along the rank axis.  Inside
 *                        each group of 8 consecutive codes c0..c7 (one 32-bit word) nibble i
 *                        (bits 4i..4i+3) holds c0,c2,c4,c6,c1,c3,c5,c7 for i = 0..7, so that
 *                        (w >> 4j) & 0x000F000F yields the adjacent pair (c2j, c2j+1).
 *   vq  uint8 [N][r/2]   codes of V^ (V^T transposed), same packing along the rank axis;
 *                        read by the reconstruction kernel.
 *   vt  uint8 [r][N/2]   codes of V^T in their natural orientation, same packing along the
 *                        d_i axis; read by the factored kernel.
 *   us  bf16  [M][ng]    per-group scales of U^           (U_scale, src/quantization.py:164)
 *   uz  uint8 [M][ng]    per-group zero-points of U^, 0..15 (U_zero, src/quantization.py:165)
 *   vs  bf16  [ng][N]    per-group scales of V^T           (Vt_scale, src/quantization.py:198)
 *   vz  uint8 [ng][N]    per-group zero-points of V^T      (Vt_zero, src/quantization.py:199)
 *
 * This replaces the reference's stored form {uq, vq, R, C} (src/kernels.py:164-188): the
 * FP32 side tables R / C are not stored; the zero-points are subtracted from the codes
 * before the integer contraction, exactly as src/quantization.py:305-308 does.
 */
typedef struct ade_delta {
    const uint8_t* uq;
    const uint8_t* vq;
    const uint8_t* vt;
    const uint16_t* us;
    const uint8_t* uz;
    const uint16_t* vs;
    const uint8_t* vz;
    int M, N, r;
    /* Optional hint for a block-diagonal U^ (several modules that share their input served as one launch:
     * d_o and rank are the members' sums, V^T is stacked along the rank axis): rows [block_rows[i], block_rows[i+1]) hold non-zero codes only in the rank
     * groups [block_groups[i], block_groups[i+1]), i < n_blocks <= ADE_B200_MAX_BLOCKS, and (code - zero) is
     * exactly 0 elsewhere.  The factored kernel then skips the other groups of those rows.  n_blocks = 0: dense.
     * No counterpart in the reference. */
    int n_blocks;
    int block_rows[ADE_B200_MAX_BLOCKS + 1];
    int block_groups[ADE_B200_MAX_BLOCKS + 1];
} ade_delta_t;

/* Library / device checks.  Replaces decode_kernel_status / recon_kernel_status
 * (src/kernels.py:86-124): returns ADE_OK when the current CUDA device can run the
 * kernels (compute capability 10.x), ADE_ERR_DEVICE / ADE_ERR_CUDA otherwise. */
int ade_b200_device_status(void);
int ade_b200_version(void);
/* cudaError_t of the most recent failing runtime call on this thread, 0 if none */
int ade_b200_last_cuda_error(void);

/*
 * Stored-form packing on the device (replaces the CPU packing of src/kernels.py:145-188).
 * codes: uint8 [rows][K], one 4-bit code per byte (src/quantization.py:162-163,196-197).
 * out:   uint8 [rows][K/2] in the nibble order documented at ade_delta_t.  K % 8 == 0.
 * With transpose != 0 the input is read as [K][rows] (used to build vq from Vt_codes).
 */
int ade_b200_pack_codes(const uint8_t* codes, uint8_t* out, int rows, int K, int transpose, void* stream);
/* zero-points: bfloat16 holding an integer 0..15 -> uint8 (count elements) */
int ade_b200_pack_zeros(const uint16_t* zeros_bf16, uint8_t* out, size_t count, void* stream);

/*
 * Producer side of the format on the device: one factor of a truncated SVD to codes, scales and zero-points in one
 * pass (replaces, per factor, the chain of src/quantization.py:244-285: scaling by sqrt(S) :266-268, the shared
 * rotation H :270-272, and quantize_rowwise / quantize_colwise :134-199 with _pin_zero_in_range :109-131).
 *   x        float32 [rows][r]: U (d_o, r), or V (d_i, r) with its singular vectors as columns.
 *   sqrt_s   float32 [r] multiplied into every row first, or NULL.
 *   rotate   != 0: apply the normalised Sylvester Hadamard rotation of order r (a power of two) inside the kernel,
 *            as a fast Walsh-Hadamard transform; 0: x is quantised as it is (the caller applied another rotation,
 *            e.g. the seeded random orthogonal matrix the reference uses for other ranks).
 *   transposed == 0: codes uint8 [rows][r] (one 4-bit code per byte), scale / zero bf16 [rows][r/128]: the U side.
 *   transposed != 0: codes [r][rows], scale / zero [r/128][rows]: the V side, H^T (sqrt(S) V^T) = ((V sqrt(S)) H)^T.
 * The quantisation is the reference's float32 arithmetic operation for operation: with rotate == 0 the outputs are
 * bit-identical to quantize_rowwise / quantize_colwise on the same input.  r % 128 == 0, r <= 2048.
 */
int ade_b200_compress_rows(const float* x, const float* sqrt_s, uint8_t* codes, uint16_t* scale, uint16_t* zero,
                           int rows, int r, int rotate, int transposed, void* stream);

/*
 * Factored application, T <= 128 tokens (replaces run_ab, src/kernels.py:946-954, and the
 * F.linear that precedes it in src/serving.py:106):
 *
 *     out[t][m] = base_term[t][m] + sum_k U^[m][k] * ( sum_n V^T[k][n] * x[t][n] )
 *
 * base_term is y_dense[t][m] when y_dense != NULL (the reference's calling convention,
 * src/kernels.py:1182-1200), or sum_n w_b[m][n] x[t][n] computed inside the same kernel
 * when w_b != NULL (exactly one of the two must be given).
 *   x bf16 [T][N], y_dense bf16 [T][M], w_b bf16 [M][N], out bf16 [T][M].
 *   scratch: device buffer, ade_b200_factored_scratch_bytes(T, r) bytes recommended.  It holds
 *   h = V^T x (bf16 [T][r]; for T <= 16 two float32 partial sums [2][T][r], one per half of the
 *   d_i axis), at byte offset ade_b200_factored_sync_offset(T, r) 256 bytes of which the first four
 *   32-bit words order the phases of the kernel, and behind them, for T > 16, float32 partial sums
 *   [parts][T][r] that let about 128 CTAs share the computation of h instead of r / 16 (parts =
 *   2048 / r, at most 8).  A buffer that ends right behind the 256 bytes (sync offset + 256) is
 *   accepted too: h is then computed by r / 16 CTAs, which is slower for T > 32.
 *   The sync words must be ZERO before the first
 *   call that uses the buffer (one cudaMemset after allocation) and are left zero by every
 *   call that completes normally, so the buffer can be reused call after call.  Word 2 is a
 *   status word: it becomes 1 if the kernel's bounded wait for h expired (output undefined;
 *   zero the words before reusing the buffer).  Calls that share a scratch buffer must
 *   not overlap on the GPU (use one buffer per stream).
 * Requirements: 1 <= T <= 128, M >= 1 (at most 320 rows per SM), N % 128 == 0, r % 128 == 0.
 * One kernel is launched on `stream` (one CTA per SM; for T <= 16 four extra warps per CTA compute
 * h while the others already stream w_b); the call does not synchronise.
 *   The CTAs of that kernel wait for one another, so the launch is cooperative: the grid starts only when
 *   every SM can take its CTA (work of other streams that holds SMs delays the start instead of starving the
 *   wait), and a device that cannot hold the grid at all makes the call return ADE_ERR_CUDA.  Should the wait
 *   for h expire all the same, status word 2 says so: read it (cudaMemcpy of 4 bytes at sync offset + 8)
 *   wherever a wrong result must not go unnoticed.
 */
size_t ade_b200_factored_scratch_bytes(int T, int r);
size_t ade_b200_factored_sync_offset(int T, int r);
int ade_b200_factored(const ade_delta_t* d, const void* x, const void* y_dense, const void* w_b,
                      void* out, void* scratch, size_t scratch_bytes, int T, void* stream);

/*
 * Factored application without a caller-supplied scratch buffer.  No counterpart in the reference.
 *
 * Same arithmetic, arguments and requirements as ade_b200_factored, but h = V^T x and the kernel's sync
 * words live in a fixed array inside the library (ADE_B200_STATIC_SCRATCH_BYTES of device memory, held by
 * every GPU that loads the library until the process exits).  It is meant for callers that must not
 * allocate device memory at the point of the call and have no buffer of their own to lend: code that
 * runs inside another framework's memory plan, under a fixed memory budget, or in a context where
 * cudaMalloc's implicit device synchronisation is not acceptable.  The entry point calls no cudaMalloc,
 * cudaFree or allocating library routine.
 *   Limit: 256 + T * r * (T <= 16 ? 8 : 2) <= ADE_B200_STATIC_SCRATCH_BYTES, i.e. T * r <= 131072 above 16
 *   tokens (T = 128 at r = 1024) and every supported rank up to 16 tokens; beyond it ADE_ERR_SCRATCH.
 *   Above 16 tokens ade_b200_factored slices the computation of h over d_i when its scratch has room for
 *   the float32 partial sums; here the slices are as many as fit behind h in the array, possibly fewer,
 *   possibly one (T = 128 at r = 512 runs unsliced).  With fewer slices the call is slower (about 1.5x at
 *   T = 128) and h is summed in another order, so the output can differ from ade_b200_factored's in the last
 *   bit; with the same number of slices the two outputs are identical.
 *   The first call on each device looks the array's address up (cudaGetSymbolAddress, with that device
 *   current); make that first call outside any stream capture.
 *   All calls on a device share the one array, and it keeps the previous call's contents; every call
 *   clears the sync words on `stream` before its launch.  Two calls that overlap on the GPU (different
 *   streams without ordering) race on h and on the sync words: serialise them, or use ade_b200_factored
 *   with one buffer per stream.
 *   The status word (1 = a wait for h expired in some call, output of that call undefined) is kept in the
 *   array too and survives later calls; ade_b200_factored_static_status copies it out.
 */
#define ADE_B200_STATIC_SCRATCH_BYTES 262400
int ade_b200_factored_static(const ade_delta_t* d, const void* x, const void* y_dense, const void* w_b,
                             void* out, int T, void* stream);
/* Copies the status word of the current device's built-in scratch array to *dst (host or device memory; one
 * 4-byte cudaMemcpyAsync on `stream`, ordered after the calls issued on it) and, when clear != 0, zeroes the
 * word afterwards.  Allocates nothing.  No counterpart in the reference. */
int ade_b200_factored_static_status(int* dst, int clear, void* stream);

/*
 * Reconstructed application (replaces ade_recon_int4, src/kernels.py:383-397):
 *
 *     w_out[m][n] = bf16( float(w_b[m][n]) + sum_g (us[m][g] * vs[g][n]) * float(P_g[m][n]) )
 *     P_g[m][n]   = sum_{k in group g} (Ucode[m][k] - uz[m][g]) * (Vcode[k][n] - vz[g][n])   (INT32)
 *
 * the arithmetic of src/quantization.py:303-315 followed by the add of src/serving.py:92,
 * in the same order and with the same float32 roundings.  P_g is contracted with
 * tcgen05 kind::i8 MMAs into tensor memory.  Ranks up to 1024 run a kernel that keeps a 128-row strip
 * of U expanded in shared memory and moves all global data with TMA (tensor maps are encoded per call
 * on the host; no device memory is allocated); larger ranks run the general kernel.
 *   w_b, w_out bf16 [M][N] (may not alias).  Requirements: N % 128 == 0, r % 128 == 0, M >= 1.
 *   dbg_acc: optional int32 [ng][M][N]; when non-NULL every P_g is also written there.
 *   status_dev: optional device int; set to a non-zero ADE_DEV_* code if a bounded wait
 *   inside the kernel expired (the kernel then still terminates; w_out is undefined).
 *   It is not cleared by the call.
 */
int ade_b200_recon(const ade_delta_t* d, const void* w_b, void* w_out,
                   int32_t* dbg_acc, int* status_dev, void* stream);

/*
 * Reconstructed application from expanded operands.  The reference's kernel unpacks the 4-bit codes and subtracts
 * the zero-points inside its main loop (src/kernels.py:296-331); a module that serves many reconstructions can do
 * that once instead:
 *
 *     ade_b200_expand_codes    writes u8 [M][r] and v8 [N][r] int8 = code - zero-point, in the order of the
 *                              contraction the kernel uses (r bytes per row; (M + N) * r bytes in all);
 *     ade_b200_recon_expanded  is ade_b200_recon reading those arrays by TMA straight into the operand tiles
 *                              (no unpack role in the kernel); same arithmetic, bit-identical w_out and dbg_acc.
 *
 * d still supplies the scales (us, vs) and the shape; u8, v8 16-byte aligned.  Ranks above 1024 are served by
 * ade_b200_recon (the arrays are then ignored).
 */
int ade_b200_expand_codes(const ade_delta_t* d, void* u8, void* v8, void* stream);
int ade_b200_recon_expanded(const ade_delta_t* d, const void* u8, const void* v8, const void* w_b, void* w_out,
                            int32_t* dbg_acc, int* status_dev, void* stream);

/*
 * Elementwise pieces of a LLaMA decoder layer at decode sizes, one launch each.  No counterpart in the reference, which
 * leaves them to transformers (src/evaluate.py:241 calls model.generate): there an RMSNorm is eight elementwise
 * kernels, the rotary embedding fourteen, SiLU and product two, and inside a CUDA graph of the decode step they cost
 * more than the delta application they surround.  Same arithmetic and the same bfloat16 roundings as the torch
 * operations they stand in for; all tensors bfloat16, strides in elements.
 *   ade_b200_rmsnorm   out[t][:] = weight * bf16(x[t][:] * rsqrt(mean(x[t][:]^2) + eps)), float32 statistics.
 *   ade_b200_add_rmsnorm  the residual connection and the RMSNorm behind it: sum_out = bf16(x + residual), out = rmsnorm(sum_out).
 *   ade_b200_rope      q [B][T][q_heads][head_dim] and k [B][T][k_heads][head_dim], given with their row strides (the
 *                      projections may be column slices of one fused output), rotated with cos / sin [B or 1][T][head_dim]
 *                      (cs_batch_stride = T * head_dim, or 0 for one shared table) into q_out [B][q_heads][T][head_dim]
 *                      and k_out [B][k_heads][T][head_dim]: x cos + rotate_half(x) sin.
 *   ade_b200_silu_mul  out[r][c] = bf16(silu(gate[r][c])) * up[r][c]; out contiguous [rows][cols].
 *   ade_b200_attn_decode  one new token per sequence: rotary embedding of q [B][q_heads*head_dim] and k, write of k and v
 *                      ([B][k_heads*head_dim], row strides free) into the static KV cache ([B][k_heads][cache_len][head_dim],
 *                      contiguous) at position *pos (device int64), and softmax(q K^T scale) V over the positions that
 *                      mask (bool [B][cache_len], true = attend, includes *pos; NULL = positions 0..*pos) allows, written to
 *                      out [B][q_heads*head_dim].  Scores and sums in float32.  q_heads % k_heads == 0, head_dim a multiple
 *                      of 32 up to 256, (7 head_dim + cache_len) floats of shared memory <= 48 KB.  With ticket != NULL (a
 *                      device counter of this cache layer's own, zero before its first use) the launch advances *pos by
 *                      one after every CTA has read it; with NULL *pos is left to the caller.
 */
int ade_b200_rmsnorm(const void* x, const void* weight, void* out, int rows, int H, long long x_row_stride, float eps, void* stream);
int ade_b200_add_rmsnorm(const void* x, const void* residual, const void* weight, void* sum_out, void* out, int rows, int H,
                         long long x_row_stride, long long residual_row_stride, float eps, void* stream);
int ade_b200_rope(const void* q, const void* k, const void* cos_t, const void* sin_t, void* q_out, void* k_out, int B, int T,
                  int q_heads, int k_heads, int head_dim, long long q_row_stride, long long k_row_stride, long long cs_batch_stride,
                  void* stream);
int ade_b200_silu_mul(const void* gate, const void* up, void* out, int rows, int cols, long long gate_row_stride,
                      long long up_row_stride, void* stream);
int ade_b200_attn_decode(const void* q, const void* k, const void* v, const void* cos_t, const void* sin_t, const void* mask,
                         void* k_cache, void* v_cache, long long* pos, unsigned int* ticket, void* out, int B, int q_heads, int k_heads,
                         int head_dim, int cache_len, long long q_row_stride, long long k_row_stride, long long v_row_stride,
                         long long cs_batch_stride, long long mask_row_stride, float scale, void* stream);

/*
 * Process-wide options.  No counterpart in the reference.
 *   ADE_OPT_WAIT_LIMIT_CYCLES   clock cycles a wait inside a kernel (for h, for an operand stage, ...) may take
 *                               before the kernel gives up, records its status and runs to its end; 0 restores the
 *                               default of about one second.
 *   ADE_OPT_COOPERATIVE_LAUNCH  1 (default): the factored kernel is launched cooperatively; 0: plain launch, for
 *                               callers that guarantee an otherwise idle device themselves.
 *   ADE_OPT_DROP_SIGNALS        diagnostic, default 0.  With 1 the producers inside the kernels stay silent (the
 *                               phase-A units of the factored kernel do not report, the reconstruction kernels
 *                               issue no code loads), so every wait that depends on them runs into the limit
 *                               above: the way to exercise the time-out path without any fault.  Outputs of
 *                               such calls are undefined.
 *   ADE_OPT_ATTN_SINGLE_PASS    1 (default): ade_b200_attn_decode walks the cache once with a running softmax when the
 *                               head dimension is 32, 64, 128 or 256; 0: always the two-pass kernel.
 * Returns ADE_OK, or ADE_ERR_SHAPE for an unknown option or a negative limit.
 */
#define ADE_OPT_WAIT_LIMIT_CYCLES 1
#define ADE_OPT_COOPERATIVE_LAUNCH 2
#define ADE_OPT_DROP_SIGNALS 3
#define ADE_OPT_ATTN_SINGLE_PASS 4
int ade_b200_set_option(int option, long long value);

#ifdef __cplusplus
}
#endif
#endif /* ADE_B200_H */
