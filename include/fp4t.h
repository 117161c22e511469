/*
 * fp4t -- C ABI of the B200 (sm_100a) quantized-linear training path.
 *
 * One shared library, plain pointers and sizes.  Every entry point
 *   - takes DEVICE pointers owned by the caller (unless a parameter says "host"),
 *   - enqueues its kernels on the given CUDA stream and returns without
 *     synchronising,
 *   - allocates nothing, creates no stream and keeps no reference to caller memory
 *     (exceptions: fp4t_set_status_word and fp4t_set_seed_offset_word store the pointer they are
 *     given until it is replaced),
 *   - returns FP4T_OK (0) or a negative FP4T_ERR_* code; the text of the last
 *     error on the calling thread is available from fp4t_last_error().
 *
 * Layout conventions (identical to what the reference hands to cuBLASLt):
 *   - NVFP4 codes: E2M1, two per byte, element 2j in bits 0..3 and element 2j+1
 *     in bits 4..7 of byte j of a row; rows are contiguous, [outer, K/2] bytes.
 *   - MXFP8 codes: E4M3 bytes, [outer, K].
 *   - Scale factors: one byte per block of 16 (NVFP4, UE4M3) or 32 (MXFP8,
 *     UE8M0) elements along K, stored in the 128x4 tile layout: for the logical
 *     matrix [outer, kblocks] the byte of (o, i) sits at
 *        ((o/128) * ceil(kblocks/4) + i/4) * 512 + (o%32)*16 + ((o%128)/32)*4 + i%4
 *     and the buffer is zero padded to whole 512-byte tiles
 *     (fp4t_sf_bytes() gives its size).
 *
 * "Replaces" comments cite the reference project (vuiseng9/fp4-training) by
 * file:line within that project.
 */
#ifndef FP4T_H_
#define FP4T_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FP4T_API __attribute__((visibility("default")))
#else
#define FP4T_API
#endif

typedef struct CUstream_st* fp4t_stream_t; /* a cudaStream_t / CUstream */

enum {
  FP4T_OK = 0,
  FP4T_ERR_ARG = -1,      /* bad pointer, size, alignment or enum value            */
  FP4T_ERR_CUDA = -2,     /* a CUDA runtime / driver call failed                   */
  FP4T_ERR_UNSUPPORTED = -3, /* valid request that this build does not implement   */
  FP4T_ERR_DEVICE = -4    /* the device is not an sm_100 part                      */
};

enum { FP4T_DT_BF16 = 0, FP4T_DT_F32 = 1 };

/* Stochastic rounding of NVFP4 codes. */
enum {
  FP4T_SR_NONE = 0,   /* round to nearest even                                      */
  FP4T_SR_NOISE = 1,  /* u ~ U[0,1) read from caller tensors (bit-exact parity mode) */
  FP4T_SR_HASH = 2    /* u generated in the kernel from (seed, element index)        */
};

/* Operand layout selector of the reference op signature (custom/linear/cublaslt.py:14-17). */
enum { FP4T_TN = 0, FP4T_NN = 1, FP4T_NT = 2 };

FP4T_API const char* fp4t_last_error(void);
FP4T_API int fp4t_version(void);

/*
 * Device int32[4] that kernels launched afterwards from this host thread write a nonzero
 * code into if one of their bounded waits runs out (entry points with their own `status`
 * parameter prefer that one).  Null switches the reporting off.  The caller owns the
 * memory and zeroes it.
 */
FP4T_API int fp4t_set_status_word(int32_t* device_word);

/*
 * Stochastic rounding with FP4T_SR_HASH derives its noise from (seed, element index).  A launch
 * that is replayed from a CUDA graph carries the seed it was captured with, so every replay
 * would round with the same noise.  After this call, quantizer kernels launched on the CURRENT
 * device add  *device_word * 0x9E3779B97F4A7C15  to their seed when they RUN: a program that
 * increments the word between replays (on the stream, e.g. inside the graph) gets fresh noise
 * each time.  The library keeps the pointer until it is replaced (null switches it off); the
 * caller owns the memory.  Process-wide per device (the backward pass of an autograd engine
 * runs on other host threads than the one that set it).  No counterpart in the reference,
 * which draws torch.rand_like per call (custom/quantize.py:88).
 */
FP4T_API int fp4t_set_seed_offset_word(const uint64_t* device_word);

/*
 * Every spin in the kernels (on an mbarrier, on a peer GPU's flag) is bounded: when the limit
 * runs out the kernel writes a role code into the status word, lets its copies in flight land,
 * frees its tensor memory and returns, so the context stays usable.  This sets the limit, in
 * nanoseconds, for kernels launched afterwards on the CURRENT device (default 4 s; the peer
 * waits of the all-reduce use half of it).  A synchronising set-up call.  No counterpart in
 * the reference (cuBLASLt and NCCL have their own watchdogs).
 */
FP4T_API int fp4t_set_wait_timeout_ns(uint64_t ns);

/*
 * Process-wide cap on the number of SMs the persistent kernels fill (0 = all).  A data-parallel
 * job sets it a little below the SM count so that a collective running on another stream finds
 * free SMs instead of waiting behind a grid that occupies every one.
 */
FP4T_API int fp4t_set_sm_limit(int sms);

/*
 * The persistent kernels draw their tiles from per-stream device counters that every launch
 * leaves at zero.  A launch that gave up on a wait (nonzero status word) may leave them
 * nonzero; this puts all counters of the current device back to zero (stream-ordered on
 * `stream`).  No counterpart in the reference.
 */
FP4T_API int fp4t_reset_tile_counters(fp4t_stream_t stream);

/* Bytes of the swizzled scale buffer for a logical [outer, kblocks] scale matrix. */
FP4T_API int64_t fp4t_sf_bytes(int64_t outer, int64_t kblocks);

/*
 * Fused NVFP4 quantizer: reads x [rows, cols] (row-major, leading dimension ld
 * elements) ONCE and writes any of
 *   codes   [rows, cols/2], sf   = swizzled scales of logical [rows, cols/16]
 *   codes_t [cols, rows/2], sf_t = swizzled scales of logical [cols, rows/16]
 * (the second pair is the quantization of x transposed, 1x16 blocks along rows).
 * A null codes/codes_t pointer skips that output.  Per-tensor scale is 1.
 * sr_mode FP4T_SR_NOISE reads noise [rows, cols] and noise_t [cols, rows] (fp32).
 * Requirements: cols % 16 == 0 for the row-wise output, rows % 32 == 0 for the
 * transposed one; bf16 input additionally wants x and ld 16-byte aligned
 * (otherwise a slower generic kernel is used).
 *
 * Replaces custom/quantize.py:57-122 (quantize_nvfp4, q_nvfp4_rowwise), the
 * transposes at custom/linear/nvfp4.py:59,74-75, the scale swizzle at
 * custom/swizzle.py:6-23 and the FP4 pack kernel at
 * custom/backend/csrc/cublaslt_mm_nvfp4.cu:145-166,275-306.
 */
FP4T_API int fp4t_quantize_nvfp4(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                        void* codes, void* sf, void* codes_t, void* sf_t,
                        int sr_mode, const float* noise, const float* noise_t, uint64_t seed,
                        fp4t_stream_t stream);

/*
 * Fused MXFP8 quantizer, same shape contract with 1x32 blocks:
 *   codes   [rows, cols]   sf   ~ logical [rows, cols/32]
 *   codes_t [cols, rows]   sf_t ~ logical [cols, rows/32]
 * Requirements: cols % 32 == 0 (row-wise), rows % 32 == 0 (transposed).
 *
 * Replaces custom/quantize.py:8-49 (q_mxfp8_rowwise / q_mxfp8_colwise through
 * microxcaling's quantize_mx_op) and custom/swizzle.py:6-60.
 */
FP4T_API int fp4t_quantize_mxfp8(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                        void* codes, void* sf, void* codes_t, void* sf_t,
                        fp4t_stream_t stream);

/*
 * The quantizers with the activation in front of them fused in: the output is the quantization
 * of GELU(x) -- as torch computes it for a bf16 tensor: in fp32, x * 0.5 * (1 + erf(x / sqrt 2)),
 * rounded to bf16 -- without that bf16 tensor ever being written to or read from HBM.  x is the
 * bf16 pre-activation [rows, cols] (16-byte aligned rows); outputs as fp4t_quantize_*.
 *
 * Replaces `act` followed by the quantizer call inside `down_proj` in the reference's MLP
 * (models/transformer_block.py:45-52 -> custom/linear/nvfp4.py:28-33) where no dropout sits
 * between them (inference, or dropout 0).
 */
FP4T_API int fp4t_quantize_nvfp4_gelu(const void* x_bf16, int64_t rows, int64_t cols, int64_t ld,
                             void* codes, void* sf, void* codes_t, void* sf_t, fp4t_stream_t stream);
FP4T_API int fp4t_quantize_mxfp8_gelu(const void* x_bf16, int64_t rows, int64_t cols, int64_t ld,
                             void* codes, void* sf, void* codes_t, void* sf_t, fp4t_stream_t stream);

/*
 * NVFP4 with a second, per-tensor scale level (the two-level recipe the reference lists as a
 * TODO in its README's "Features to Add" and that its quantizer, custom/quantize.py:100-137,
 * leaves at one level): the block quantization is applied to x * tensor_scale, so a tensor whose
 * magnitudes sit below the reach of the UE4M3 block scale (smallest value 2^-9, i.e. blocks
 * with amax < 6 * 2^-9 lose resolution, gradients late in training) is lifted into range first.
 * Codes and block scales then describe x * tensor_scale; the product of two such operands is
 * brought back by fp4t_gemm_nvfp4_scaled's alpha = 1 / (tensor_scale_p * tensor_scale_q).
 * A power-of-two tensor_scale with bf16 input runs on the tiled kernel (the scale folds into the
 * block-scale arithmetic exactly); any other positive value takes the general kernel.
 * sr_mode: FP4T_SR_NONE or FP4T_SR_HASH.  tensor_scale = 1 gives fp4t_quantize_nvfp4 bit for bit.
 */
FP4T_API int fp4t_quantize_nvfp4_scaled(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                               void* codes, void* sf, void* codes_t, void* sf_t, int sr_mode, uint64_t seed,
                               float tensor_scale, fp4t_stream_t stream);

/*
 * NVFP4 with a random Hadamard transform of every 16-element block in front of the block
 * quantization (outlier spreading; the other recipe step the reference's README lists as to
 * be added): block b of the quantized axis becomes H16 . diag(signs) . b / 4, with the signs
 * from bits 0..15 of sign_mask (bit j set = element j negated) and H16 the Sylvester-ordered
 * Hadamard matrix.  The map is orthogonal, so a GEMM of two operands transformed with the same
 * sign_mask along K equals the GEMM of the untransformed operands up to quantization error.
 * The row-wise output transforms blocks along the columns, the transposed output blocks along
 * the rows (rows % 16 == 0).  Round-to-nearest-even; runs on the general kernel.
 */
FP4T_API int fp4t_quantize_nvfp4_rht(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                            void* codes, void* sf, void* codes_t, void* sf_t, uint32_t sign_mask,
                            float tensor_scale, fp4t_stream_t stream);

/*
 * The same quantizers with the bias gradient fused in: while the kernel walks dY for the
 * transposed operand it also accumulates the column sums of dY, so
 *   bias_grad[c] = sum_r x[r, c]      (bf16 or fp32, selected by bias_grad_dtype)
 * comes out of the pass that already reads every element.  colsum_scratch is caller-owned
 * scratch of cols fp32 values (contents on entry are ignored; it is cleared on the stream,
 * accumulated into with atomics and read by a small finishing kernel).  The sum is taken in
 * fp32; its last bits depend on the order of the atomics.
 *
 * Replaces `grad_b = grad_Y.sum(dim=0)` at custom/linear/nvfp4.py:88 and
 * custom/linear/mxfp8.py:83 (a separate full read of dY in the reference).
 */
FP4T_API int fp4t_quantize_nvfp4_bgrad(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                       void* codes, void* sf, void* codes_t, void* sf_t,
                                       int sr_mode, const float* noise, const float* noise_t, uint64_t seed,
                                       float* colsum_scratch, void* bias_grad, int bias_grad_dtype,
                                       fp4t_stream_t stream);
FP4T_API int fp4t_quantize_mxfp8_bgrad(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                       void* codes, void* sf, void* codes_t, void* sf_t,
                                       float* colsum_scratch, void* bias_grad, int bias_grad_dtype,
                                       fp4t_stream_t stream);

/*
 * fp4t_quantize_nvfp4_bgrad without any caller-provided scratch.  (No counterpart in the
 * reference: this entry point exists for hosts that may not allocate device memory around the
 * call.)
 *
 * Some callers cannot hand over a scratch buffer because they cannot obtain one: a plugin
 * whose host framework owns all device memory and gives plugins only their input and output
 * tensors, a service that reserved the whole GPU for its own pool at start-up so that a
 * cudaMalloc made later fails or stalls, or a latency-critical loop that must not hit the
 * device-wide synchronisation an allocation can cause.  For them the column-sum scratch is a
 * fixed array inside the library: FP4T_STATIC_BGRAD_MAX_COLS fp32 values (64 KiB) that every
 * GPU using the library keeps until the process ends.  Inputs and outputs are still the
 * caller's.  The call itself performs no cudaMalloc / cudaFree and uses no allocating library
 * routine.
 *
 *  - cols larger than FP4T_STATIC_BGRAD_MAX_COLS is rejected with FP4T_ERR_ARG.
 *  - The first call on each device looks up the array's device address (a one-time host-side
 *    set-up, done with that device current); make that first call before starting any stream
 *    capture on the device.
 *  - All calls on a device share the one array, and it still holds the previous call's sums
 *    when a call begins; each call clears the columns it uses on its stream before
 *    accumulating.  Two calls that may run on the GPU at the same time (different streams
 *    without an ordering between them) would race on it: serialise them.
 * Results are those of fp4t_quantize_nvfp4_bgrad (identical codes and scales; the bias
 * gradient differs only by fp32 summation order).
 */
#define FP4T_STATIC_BGRAD_MAX_COLS 16384
FP4T_API int fp4t_quantize_nvfp4_bgrad_static(const void* x, int x_dtype, int64_t rows, int64_t cols,
                                              int64_t ld, void* codes, void* sf, void* codes_t, void* sf_t,
                                              int sr_mode, const float* noise, const float* noise_t,
                                              uint64_t seed, void* bias_grad, int bias_grad_dtype,
                                              fp4t_stream_t stream);

/*
 * Block-scaled GEMMs on tcgen05:  D[rows, cols] = P[rows, K] . Q[cols, K]^T (+ bias[cols]),
 * fp32 accumulation in tensor memory, D written as bf16 or fp32 (row-major,
 * leading dimension ldd elements).  P/Q are code matrices, p_sf/q_sf their
 * swizzled scales; bias is bf16 or null.
 * Requirements: NVFP4 K % 32 == 0, MXFP8 K % 16 == 0; code pointers 16-byte aligned;
 * scale pointers 16-byte aligned; ldd*sizeof(elem) % 16 == 0.
 *
 * Replaces custom/backend/csrc/cublaslt_mm_nvfp4.cu:184-448 and
 * custom/backend/csrc/cublaslt_mm_mxfp8.cu:103-320 (mode TN; P is the binding's
 * B argument, Q its A argument, D its Dt[n, m]).
 * status, when not null, is a device int32[4] the kernel writes a nonzero code
 * into if one of its bounded waits ran out (0 otherwise left untouched).
 */
FP4T_API int fp4t_gemm_nvfp4(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                    const void* bias_bf16, void* d, int d_dtype, int64_t ldd,
                    int64_t rows, int64_t cols, int64_t k, int32_t* status,
                    fp4t_stream_t stream);
FP4T_API int fp4t_gemm_mxfp8(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                    const void* bias_bf16, void* d, int d_dtype, int64_t ldd,
                    int64_t rows, int64_t cols, int64_t k, int32_t* status,
                    fp4t_stream_t stream);

/*
 * The same GEMMs with a block-quantized OUTPUT: the epilogue turns each row's 32-column pieces
 * of the fp32 accumulator (+ bias) into the row-wise operand of a following GEMM whose K is
 * this GEMM's `cols`, so a chain GEMM -> GEMM needs no bf16 round trip and no quantizer launch:
 *   out_fmt FP4T_QOUT_MXFP8  d_codes [rows, cols] E4M3 bytes, d_sf ~ logical [rows, cols/32] UE8M0
 *   out_fmt FP4T_QOUT_NVFP4  d_codes [rows, cols/2] packed E2M1, d_sf ~ logical [rows, cols/16] UE4M3
 * (scales in the tile layout; the call zeroes the scale buffer's padding on the stream).  ldd is
 * the pitch of d_codes in BYTES (a multiple of 16); cols must be a multiple of 32.  The
 * conversion is the quantizers' (true divisions; E4M3 elements round half away from zero, E2M1
 * to nearest even), applied to the fp32 accumulator instead of a bf16 tensor.
 *
 * Finishes what custom/backend/csrc/cublaslt_mm_mxfp8.cu:155-161,247-253 (Dout = uint8: E4M3
 * output + scaleDout) and cublaslt_mm_nvfp4.cu:241-247,374-380 (Dout = uint8: E2M1 output,
 * marked TODO there) start through cuBLASLt's D_OUT scale mode.
 */
enum { FP4T_QOUT_MXFP8 = 1, FP4T_QOUT_NVFP4 = 2 };
FP4T_API int fp4t_gemm_nvfp4_qout(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                         const void* bias_bf16, void* d_codes, void* d_sf, int out_fmt, int64_t ldd,
                         int64_t rows, int64_t cols, int64_t k, int32_t* status, fp4t_stream_t stream);
FP4T_API int fp4t_gemm_mxfp8_qout(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                         const void* bias_bf16, void* d_codes, void* d_sf, int out_fmt, int64_t ldd,
                         int64_t rows, int64_t cols, int64_t k, int32_t* status, fp4t_stream_t stream);

/*
 * fp4t_gemm_nvfp4 with D = alpha * (P . Q^T) + bias: alpha undoes the per-tensor scales of
 * operands made by fp4t_quantize_nvfp4_scaled (alpha = 1 / (t_p * t_q)).  workspace may be null
 * (or point at fp4t_gemm_splitk_workspace_bytes(rows, cols) bytes to allow the split-K form).
 */
FP4T_API int fp4t_gemm_nvfp4_scaled(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                           const void* bias_bf16, void* d, int d_dtype, int64_t ldd, int64_t rows,
                           int64_t cols, int64_t k, float alpha, void* workspace, int64_t workspace_bytes,
                           int32_t* status, fp4t_stream_t stream);

/*
 * The GEMMs with an optional split-K workspace (caller-owned, 16-byte aligned, contents
 * ignored and overwritten).  When the output has so few tiles that most SMs would idle -- the
 * wgrad of a small layer over a long batch: dW 192 x 192 with K = 25600 is ONE tile -- the K loop
 * is split over the idle SMs: every split writes its fp32 partial to a slice of the workspace and
 * a small kernel adds the slices (+ bias) into d.  With a null or too small workspace, or a
 * shape that fills the machine anyway, the call is exactly fp4t_gemm_*.
 * fp4t_gemm_splitk_workspace_bytes(rows, cols) is the size that allows the full split (0 when
 * the output is large enough not to need one).  The sum over splits is taken in a fixed order,
 * so results are deterministic; they differ from the unsplit kernel's by fp32 summation order.
 * No counterpart in the reference (cuBLASLt picks split-K kernels by itself).
 */
FP4T_API int64_t fp4t_gemm_splitk_workspace_bytes(int64_t rows, int64_t cols);
FP4T_API int fp4t_gemm_nvfp4_splitk(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                           const void* bias_bf16, void* d, int d_dtype, int64_t ldd, int64_t rows, int64_t cols,
                           int64_t k, void* workspace, int64_t workspace_bytes, int32_t* status,
                           fp4t_stream_t stream);
FP4T_API int fp4t_gemm_mxfp8_splitk(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                           const void* bias_bf16, void* d, int d_dtype, int64_t ldd, int64_t rows, int64_t cols,
                           int64_t k, void* workspace, int64_t workspace_bytes, int32_t* status,
                           fp4t_stream_t stream);

/*
 * A whole linear layer per call.  fmt: 0 = NVFP4, 1 = MXFP8.
 *
 * fp4t_linear_forward quantizes W [oc, ic] and X [n, ic] (emitting the transposed operands of
 * the backward GEMMs as well when `keep` asks for them: bit 0 = W^T for dgrad, bit 1 = X^T for
 * wgrad) and computes Y [n, oc] = X W^T + bias.  All codes and scales go to `workspace`
 * (fp4t_linear_workspace_bytes(fmt, n, ic, oc) bytes, 256-byte aligned, caller-owned), which
 * the caller keeps until the backward call.
 * fp4t_linear_backward quantizes dY [n, oc] once (stochastic rounding per sr_mode for NVFP4),
 * and computes any of dX [n, ic] = dY W, dW [oc, ic] = dY^T X and db [oc] = column sums of dY
 * (null pointers skip an output) from the forward workspace and a second workspace of
 * fp4t_linear_backward_workspace_bytes(fmt, n, oc, ic) bytes (it includes the fp32 slices of a
 * split-K wgrad when dW is small).  Outputs are written in out_dtype.
 * fp4t_set_layer_concurrency(1) (or FP4T_CONCURRENT_LAYER=1 in the environment; default off)
 * lets large layers run part of a call (X's quantizer in forward, dX's GEMM in backward) on a
 * helper stream the library keeps per (device, caller stream), beside its independent sibling;
 * `stream` waits for it before the call's work ends in stream order, so to the caller
 * everything is ordered on `stream` as usual (also under graph capture).  It fills the partly
 * filled last wave of tiles of the sibling kernel (about 2 % of a step at 8192 x 4096 x 4096).
 * Keep it off while kernels that wait for another GPU (fp4t_rank_meet,
 * fp4t_allreduce_sum_bf16_multimem) can be in flight on the same device: work of the helper
 * stream can be queued behind such a kernel in a hardware queue the two streams share.
 * Shape requirements are those of the quantizer and GEMM entry points (ic, oc multiples of the
 * block size; n % 32 == 0 for the transposed operands).
 *
 * Replaces the bodies of Nvfp4Matmul.forward / .backward (custom/linear/nvfp4.py:25-90) and
 * Mxfp8MatMul.forward / .backward (custom/linear/mxfp8.py:27-85).
 */
FP4T_API int fp4t_set_layer_concurrency(int on);
FP4T_API int64_t fp4t_linear_workspace_bytes(int fmt, int64_t n, int64_t ic, int64_t oc);
FP4T_API int64_t fp4t_linear_backward_workspace_bytes(int fmt, int64_t n, int64_t oc, int64_t ic);
FP4T_API int fp4t_linear_forward(int fmt, const void* x, int x_dtype, int64_t n, int64_t ic, int64_t ldx,
                                 const void* w, int w_dtype, int64_t oc, int64_t ldw, const void* bias_bf16,
                                 void* y, int y_dtype, int64_t ldy, void* workspace, int keep,
                                 int32_t* status, fp4t_stream_t stream);
FP4T_API int fp4t_linear_backward(int fmt, const void* g, int g_dtype, int64_t n, int64_t oc, int64_t ldg,
                                  int64_t ic, const void* fwd_workspace, void* bwd_workspace,
                                  void* dx, int64_t lddx, void* dw, int64_t lddw, void* db, int out_dtype,
                                  int sr_mode, const float* noise, const float* noise_t, uint64_t seed,
                                  int32_t* status, fp4t_stream_t stream);

/*
 * fp32 values that already lie on the E2M1 grid -> packed codes (RNE, saturate
 * to +-6) and back.  Replaces pack_rowwise_to_2xfp4,
 * custom/backend/csrc/cublaslt_mm_nvfp4.cu:109-182.  in_dtype selects fp32/bf16 input.
 */
FP4T_API int fp4t_pack_e2m1(const void* values, int in_dtype, void* codes, int64_t rows, int64_t cols,
                   fp4t_stream_t stream);
FP4T_API int fp4t_unpack_e2m1(const void* codes, float* values, int64_t rows, int64_t cols,
                     fp4t_stream_t stream);

/*
 * Scale-matrix re-layouts on bytes.
 *  fp4t_swizzle_rowwise: logical [outer, inner] -> 128x4 tile layout (custom/swizzle.py:6-23).
 *  fp4t_swizzle_colwise: logical [inner, outer] -> the layout of custom/swizzle.py:43-60.
 *  fp4t_unswizzle_colwise_to_rowwise: bytes in the layout of custom/swizzle.py:43-60 for a
 *    logical [inner, outer] matrix -> canonical tile layout of its transpose [outer, inner].
 * dst must hold fp4t_sf_bytes(outer, inner) bytes.
 */
FP4T_API int fp4t_swizzle_rowwise(const void* logical, void* dst, int64_t outer, int64_t inner,
                         fp4t_stream_t stream);
FP4T_API int fp4t_swizzle_colwise(const void* logical, void* dst, int64_t inner, int64_t outer,
                         fp4t_stream_t stream);
FP4T_API int fp4t_unswizzle_colwise_to_rowwise(const void* src, void* dst, int64_t inner, int64_t outer,
                                      fp4t_stream_t stream);

/*
 * Data-parallel exchange of the weight gradients (in the reference: torch DDP's NCCL all-reduce
 * of weight.grad / bias.grad after custom/linear/nvfp4.py:88-90).  In-place SUM all-reduce of a
 * bf16 buffer over the `world` GPUs of one NVSwitch domain, reduced inside the switch:
 *   multicast_ptr  multicast address of the buffer; every rank allocated it symmetrically and
 *                  bound it to one NVLink multicast object (e.g. torch symmetric memory)
 *   flag_ptrs      host array of `world` device pointers: rank r's flag array as mapped into
 *                  this process, FP4T_ALLREDUCE_FLAG_WORDS 32-bit words each, zero before the
 *                  first call and owned by this function afterwards
 *   epoch          1, 2, 3, ... : the same value on every rank for the same call
 *   ctas           upper bound on CTAs (the same on every rank); the kernel is small enough
 *                  (256 threads, 40 registers) to be resident beside the persistent kernels
 * Every rank must make the call; stream-ordered after the producer of the buffer.  A wait on a
 * peer that runs out (2 s) writes 41 / 42 into `status` and ends the kernel.
 */
#define FP4T_ALLREDUCE_MAX_CTAS 256
#define FP4T_ALLREDUCE_FLAG_WORDS (FP4T_ALLREDUCE_MAX_CTAS * 8)
FP4T_API int fp4t_allreduce_sum_bf16_multimem(void* multicast_ptr, const void* const* flag_ptrs, int rank, int world,
                                     int64_t numel, uint32_t epoch, int ctas, int32_t* status,
                                     fp4t_stream_t stream);

/*
 * Building blocks of the same exchange with the bulk bytes on the copy engines instead of on
 * SMs (the persistent quantizer and GEMM kernels of the next step keep every SM): a
 * reduce-scatter + all-gather whose transfers are peer-to-peer cudaMemcpyAsync calls issued by
 * the host side (dp.CopyEngineAllReducer), held together by these two small launches.
 *
 * fp4t_rank_meet: a one-warp rendezvous of the `world` ranks.  Everything that precedes the
 *   call in stream order on each rank is complete and readable by the peers once the call has
 *   passed on every rank.  flag_ptrs: as above (FP4T_ALLREDUCE_FLAG_WORDS words per rank, zero
 *   before the first call; do not share the array with fp4t_allreduce_sum_bf16_multimem);
 *   slot 0..15: independent rendezvous points; calls of one slot are counted in a device word,
 *   so the launch may be captured in a CUDA graph and replayed.  A wait that runs out (half the
 *   library's wait limit) writes 43 into `status`.
 * fp4t_sum_bf16_shards: dst[i] = bf16(src[0][i] + ... + src[n_src-1][i]) accumulated in fp32 in
 *   the order given; numel % 8 == 0, 16-byte aligned pointers, at most `ctas` CTAs.
 */
FP4T_API int fp4t_rank_meet(const void* const* flag_ptrs, int rank, int world, int slot, int32_t* status,
                   fp4t_stream_t stream);
FP4T_API int fp4t_sum_bf16_shards(void* dst, const void* const* srcs, int n_src, int64_t numel, int ctas,
                         fp4t_stream_t stream);
/* fp4t_reduce_shard_bf16_multimem: dst[i] = sum over the ranks of element i of the symmetric
 *   buffer region at multicast_shard_ptr (a multicast address, 16-byte aligned; numel % 8 == 0),
 *   added inside the switch in fp32 and rounded once to bf16; dst is local memory.  With the
 *   rendezvous calls around it and peer copies of the reduced shards this replaces the pulls and
 *   the sum above on GPUs that offer NVLink multicast: only 1/world of the buffer passes
 *   through SMs. */
FP4T_API int fp4t_reduce_shard_bf16_multimem(const void* multicast_shard_ptr, void* dst, int64_t numel, int ctas,
                                    fp4t_stream_t stream);

/*
 * LayerNorm in front of the quantized projections (replaces nn.LayerNorm `preln` in the
 * reference's blocks, models/transformer_block.py:45-52,89-93, together with the cast of its
 * output to the projections' input dtype that autocast inserts).
 *
 * forward:  y[r, :] = (x[r, :] - mean_r) * rstd_r * gamma + beta, statistics in fp32 over the
 *   `cols` elements of a row (biased variance, rstd = 1 / sqrt(var + eps)), x and y each fp32 or
 *   bf16 (FP4T_DT_*), row pitches ldx / ldy in elements; mean and rstd ([rows] fp32) are kept
 *   for the backward pass.  cols % 4 == 0, cols <= 1024, 16-byte aligned rows.
 * backward: dx (dtype and pitch rule of x) and dgamma / dbeta ([cols] fp32) from dy (fp32 or
 *   bf16), x and the saved statistics.  workspace: fp4t_layernorm_backward_workspace_bytes(rows,
 *   cols) bytes, 16-byte aligned; the column sums are added in a fixed order (reproducible).
 */
FP4T_API int fp4t_layernorm_forward(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ldx,
                           const float* gamma, const float* beta, float eps, void* y, int y_dtype,
                           int64_t ldy, float* mean, float* rstd, fp4t_stream_t stream);
FP4T_API int64_t fp4t_layernorm_backward_workspace_bytes(int64_t rows, int64_t cols);
FP4T_API int fp4t_layernorm_backward(const void* dy, int dy_dtype, int64_t lddy, const void* x, int x_dtype,
                            int64_t ldx, const float* mean, const float* rstd, const float* gamma,
                            int64_t rows, int64_t cols, void* dx, int64_t lddx, float* dgamma,
                            float* dbeta, void* workspace, fp4t_stream_t stream);

/* Byte-matrix transpose [rows, cols] -> [cols, rows] (E4M3 codes for the NN / NT operand
 * forms of custom/backend/csrc/cublaslt_mm_mxfp8.cu:70-88). */
FP4T_API int fp4t_transpose_bytes(const void* src, void* dst, int64_t rows, int64_t cols,
                         fp4t_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FP4T_H_ */
