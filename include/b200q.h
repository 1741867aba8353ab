/*
 * b200q — C ABI of the B200 (sm_100a) weight-only quantized linear kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream,
 * launches asynchronously on that stream, performs no host synchronisation
 * and returns 0 on success or a negative B200Q_E* status.  After a non-zero
 * return b200q_last_error() gives a message for the calling thread.
 *
 * Each declaration names the interface of the reference project that it
 * replaces (paths relative to the reference's root).
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define B200Q_OK 0
#define B200Q_EINVAL (-1)      /* argument failed validation                  */
#define B200Q_EUNSUPPORTED (-2) /* valid request with no kernel (type, shape)  */
#define B200Q_ECUDA (-3)       /* a CUDA runtime call or launch failed         */
#define B200Q_ESCRATCH (-4)    /* scratch / workspace too small                */

/* activation / output element type */
#define B200Q_F16 0
#define B200Q_BF16 1

/* flags for b200q_marlin_gemm (mirror the op's trailing booleans) */
#define B200Q_FLAG_K_FULL 1u
#define B200Q_FLAG_ATOMIC_ADD 2u
#define B200Q_FLAG_FP32_REDUCE 4u
#define B200Q_FLAG_ZP_FLOAT 8u

/* opaque stream handle: a cudaStream_t (CUstream) */
typedef void* b200q_stream_t;

/* Message of the last failure on the calling thread ("" if none). */
const char* b200q_last_error(void);

/* Library version, encoded major*10000 + minor*100 + patch. */
int b200q_version(void);

/* Number of SMs of the current device (0 on error).  The reference sizes the
 * GEMM workspace from this (marlin_utils.py:237-245). */
int b200q_sm_count(void);

/* Error word of the kernels that wait on hand-offs (tensor-core GEMM, all-reduce)
 * on the current device: 0, or a code naming the first wait that ran into its
 * poll limit (the kernel then drains and returns instead of hanging; codes with
 * bit 16 set come from the all-reduce, low byte = peer rank).  Synchronises the device.  reset != 0 clears
 * it.  No counterpart in the reference, whose device-side waits are unbounded
 * (csrc/quantization/gptq_marlin/marlin_template.h:225-235). */
int b200q_device_error(int reset);

/* Number of kernels this library has launched in the process so far (all
 * entry points, all threads).  Lets a caller count the launches of a timed
 * region.  No counterpart in the reference. */
unsigned long long b200q_kernel_launches(void);

/*
 * GPTQ checkpoint layout -> Marlin tile layout.
 * Replaces: gptq_marlin_repack, csrc/quantization/gptq_marlin/gptq_marlin_repack.cu:251-322
 *           (op schema csrc/torch_bindings.cpp:319-321).
 *   b_q_weight  int32 [size_k/pf, size_n], value k%pf of a word at bit (k%pf)*bits
 *   perm        int32 [size_k] row gather (output row k reads input row perm[k]) or NULL
 *   out         int32 [size_k/16, size_n*16/pf]
 *   size_k % 16 == 0, size_n % 64 == 0, num_bits in {4, 8}; pf = 32/num_bits.
 */
int b200q_gptq_marlin_repack(const uint32_t* b_q_weight, const int32_t* perm,
                             uint32_t* out, int64_t size_k, int64_t size_n,
                             int num_bits, b200q_stream_t stream);

/*
 * AWQ checkpoint layout -> Marlin tile layout.
 * Replaces: awq_marlin_repack, csrc/quantization/gptq_marlin/awq_marlin_repack.cu:189-248
 *           (op schema csrc/torch_bindings.cpp:325-327).
 *   b_q_weight  int32 [size_k, size_n/pf], AWQ interleaved column packing
 *   out         int32 [size_k/16, size_n*16/pf]
 */
int b200q_awq_marlin_repack(const uint32_t* b_q_weight, uint32_t* out,
                            int64_t size_k, int64_t size_n, int num_bits,
                            b200q_stream_t stream);

/*
 * out[m, k] = a[m, perm[k]] for 16-bit elements.
 * Replaces: permute_cols, csrc/permute_cols.cu:14-88 (op schema
 *           csrc/torch_bindings.cpp:304-305).
 *   a    [size_m, size_k] 16-bit, row stride lda elements
 *   out  [size_m, size_k] contiguous
 */
int b200q_permute_cols(const void* a, int64_t lda, const int32_t* perm, void* out,
                       int64_t size_m, int64_t size_k, b200q_stream_t stream);

/*
 * Bytes of device scratch b200q_marlin_gemm needs for this problem (split-K
 * partial sums, and the gathered activations for act-order).  Never fails;
 * returns an upper bound valid for any workspace_len.
 * Replaces the in-op allocations of c_tmp / a_tmp,
 * csrc/quantization/gptq_marlin/gptq_marlin.cu:751-763,798-799.
 */
size_t b200q_marlin_gemm_scratch_bytes(int64_t size_m, int64_t size_n,
                                       int64_t size_k, int has_act_order);

/*
 * Scratch size with which b200q_marlin_gemm runs fastest: the size above plus room
 * for the fp32 partial sums of the tensor-core kernel's k-split (used when a
 * problem has fewer output tiles than the GPU has SMs; at most 64 MiB).  Any size
 * between the two is accepted: the split shrinks to what the scratch holds.
 */
size_t b200q_marlin_gemm_preferred_scratch_bytes(int64_t size_m, int64_t size_n,
                                                 int64_t size_k, int has_act_order);

/*
 * C[M,N] = A[M,K] * dequant(B) (+ bias): the mixed-precision GEMM.
 * Replaces: gptq_marlin_gemm, csrc/quantization/gptq_marlin/gptq_marlin.cu:674-959
 *           (op schema csrc/torch_bindings.cpp:308-315).
 *   a            [size_m, size_k] fp16/bf16, row stride lda (lda % 8 == 0, 16 B aligned)
 *   b_q_weight   Marlin layout int32 [size_k/16, size_n*16/pf]
 *   b_scales     [num_groups, size_n] of a's type, already marlin_permute_scales'd
 *   b_zeros      int32 [num_groups, size_n/pf] Marlin zero-points, or NULL
 *   g_idx, perm  int32 [size_k] (sorted group ids / sort permutation), both or neither
 *   b_bias       [size_n] of a's type, marlin_permute_bias'd, or NULL
 *   c            [size_m, size_n] contiguous, written
 *   scratch      >= b200q_marlin_gemm_scratch_bytes(...) bytes, 256 B aligned
 *   workspace    int32 [workspace_len], all zero on entry, zero again when the
 *                kernels finish; workspace_len >= 1 (the reference passes #SMs)
 *   b_q_type_id  ScalarType id (csrc/core/scalar_type.hpp:124-157): uint4b8,
 *                uint8b128 without zero-points; uint4, uint8 with zero-points
 *   a_dtype      B200Q_F16 or B200Q_BF16
 */
int b200q_marlin_gemm(const void* a, int64_t lda, const uint32_t* b_q_weight,
                      const void* b_scales, const uint32_t* b_zeros,
                      const int32_t* g_idx, const int32_t* perm,
                      const void* b_bias, void* c, void* scratch,
                      size_t scratch_bytes, int32_t* workspace,
                      int64_t workspace_len, int64_t b_q_type_id, int a_dtype,
                      int64_t size_m, int64_t size_n, int64_t size_k,
                      int64_t num_groups, unsigned flags, b200q_stream_t stream);

/*
 * One-shot SUM all-reduce of a 16-bit tensor across the ranks of a tensor-parallel
 * group, over NVLink peer memory (plain loads / stores; fp32 accumulation in rank
 * order, so every rank gets bitwise the same result).
 * Replaces: the custom all-reduce behind RowParallelLinear's output,
 *           csrc/custom_all_reduce.cu:62-105 / csrc/custom_all_reduce.cuh:298-314
 *           (vllm/distributed/device_communicators/custom_all_reduce.py:267-283).
 *   peer_bufs   device array [world] of every rank's receive buffer (peer-mapped), each
 *               of b200q_all_reduce_buffer_bytes(world, max_message_bytes) bytes, zero
 *               before the first call
 *   state       local device memory, b200q_all_reduce_state_bytes() bytes, zero
 *               before the first call; the kernels keep the call number there, so
 *               a captured CUDA graph can be replayed
 *   in          this rank's partial [n_elems], local memory, complete in stream order
 *   out         local output [n_elems] (may be `in`); n_elems % 8 == 0,
 *               n_elems * 2 <= max_message_bytes
 * All ranks must make the same sequence of calls (of this function and of
 * b200q_marlin_gemm_all_reduce) with the same sizes on one link.  Waits are bounded
 * (see b200q_device_error).
 */
size_t b200q_all_reduce_state_bytes(void);
size_t b200q_all_reduce_buffer_bytes(int world, int64_t max_message_bytes);
/*
 * How many times a thread polls its own receive buffer for a peer's packets before it
 * gives up, records 0x1ff in the device error word (b200q_device_error returns 0x101ff)
 * and skips its output; applies to the calls made after it, process-wide.  0 restores the
 * default (2^21 polls, about a second).  The reference's kernels wait without a bound
 * (csrc/custom_all_reduce.cuh:180-262); a bound keeps a lost peer from hanging the GPU.
 */
void b200q_all_reduce_set_poll_limit(uint32_t polls);
int b200q_all_reduce(void* const* peer_bufs, uint32_t* state, int rank, int world,
                     int64_t max_message_bytes, const void* in, void* out, int64_t n_elems,
                     int dtype, b200q_stream_t stream);

/*
 * The same GEMM for float4_e2m1f weights (b_q_type float4_e2m1f of
 * csrc/quantization/gptq_marlin/gptq_marlin.cu:818-829, 907-917, which the reference
 * selects by the dtype of b_scales):
 *   scale_kind B200Q_FP4_SCALES_E4M3  NVFP4: group size 16, b_scales = bytes [K/16, N] as
 *              nvfp4_marlin_process_scales returns them (float8_e4m3fn-typed tensor),
 *              global_scale = one 16-bit value as nvfp4_marlin_process_global_scale
 *              returns it (vllm/model_executor/layers/quantization/utils/marlin_utils_fp4.py:28-90)
 *   scale_kind B200Q_FP4_SCALES_E8M0  MXFP4: group size 32, b_scales = bytes [K/32, N] as
 *              mxfp4_marlin_process_scales returns them (float8_e8m0fnu), global_scale
 *              null, bfloat16 activations only
 * b_q_weight is the Marlin layout of the 4-bit codes (gptq_marlin_repack with num_bits 4);
 * no zero-points, no act-order; K / group size must be even.  The other arguments as in
 * b200q_marlin_gemm.
 */
#define B200Q_FP4_SCALES_E4M3 1
#define B200Q_FP4_SCALES_E8M0 2
int b200q_marlin_gemm_fp4(const void* a, int64_t lda, const uint32_t* b_q_weight,
                          const void* b_scales, const void* global_scale, int scale_kind,
                          const void* b_bias, void* c, void* scratch, size_t scratch_bytes,
                          int32_t* workspace, int64_t workspace_len, int a_dtype, int64_t size_m,
                          int64_t size_n, int64_t size_k, int64_t num_groups,
                          b200q_stream_t stream);

/*
 * The mixture-of-experts form of the GEMM: moe_wna16_marlin_gemm of
 * csrc/moe/marlin_moe_wna16/ops.cu:693-960 (torch schema csrc/moe/torch_bindings.cpp:62-73).
 *   a                  [size_m, size_k] 16-bit activations (one row per token), row stride lda
 *   b_q_weight         [num_experts][size_k/16, size_n*16/pack_factor] Marlin layout per expert
 *   b_scales           [num_experts][num_groups, size_n] permuted as for b200q_marlin_gemm
 *   b_zeros            [num_experts][num_groups, size_n/pack_factor] or null
 *   b_bias             [num_experts][size_n] permuted, or null
 *   c                  [size_m * top_k, size_n]: row id = token * top_k + slot
 *   sorted_token_ids   [sorted_len] ids grouped by expert in blocks of moe_block_size, padded
 *                      with values >= size_m * top_k (what moe_align_block_size returns)
 *   expert_ids         [sorted_len / moe_block_size] expert of each block; -1 = skip (expert
 *                      parallelism)
 *   num_tokens_past_padded  device scalar: how many sorted ids are in use
 *   topk_weights       [size_m * top_k] fp32; output rows are multiplied by it when
 *                      mul_topk_weights != 0
 * Rows of c whose id appears in no block are not written.  moe_block_size in {8, 16, 32, 48, 64};
 * integer weight types (uint4b8, uint8b128, uint4, uint8), channel-wise or grouped scales; no
 * act-order.  No scratch: a (block, column slice) is computed over the whole K by one CTA.
 */
int b200q_moe_wna16_marlin_gemm(
    const void* a, int64_t lda, const uint32_t* b_q_weight, const void* b_scales,
    const uint32_t* b_zeros, const void* b_bias, void* c, const int32_t* sorted_token_ids,
    const int32_t* expert_ids, const int32_t* num_tokens_past_padded, const float* topk_weights,
    int64_t sorted_len, int64_t moe_block_size, int64_t top_k, int mul_topk_weights,
    int64_t num_experts, int64_t b_q_type_id, int a_dtype, int64_t size_m, int64_t size_n,
    int64_t size_k, int64_t num_groups, b200q_stream_t stream);

/*
 * b200q_marlin_gemm followed by the SUM all-reduce of C over the same peer link, as
 * RowParallelLinear does (vllm/model_executor/layers/linear.py:1386-1411: the
 * quantized matmul of the K shard, then tensor_model_parallel_all_reduce).  Where one
 * decode launch covers the problem (size_m <= 32) the GEMM kernel itself pushes its
 * rounded output tile to the peers and reduces: one kernel, no second launch;
 * otherwise the all-reduce kernel runs on C in place.  The result equals
 * b200q_marlin_gemm + b200q_all_reduce bit for bit.
 * size_m * size_n * 2 <= max_message_bytes; the other arguments as in the two calls.
 */
int b200q_marlin_gemm_all_reduce(
    const void* a, int64_t lda, const uint32_t* b_q_weight, const void* b_scales,
    const uint32_t* b_zeros, const int32_t* g_idx, const int32_t* perm, const void* b_bias,
    void* c, void* scratch, size_t scratch_bytes, int32_t* workspace, int64_t workspace_len,
    int64_t b_q_type_id, int a_dtype, int64_t size_m, int64_t size_n, int64_t size_k,
    int64_t num_groups, unsigned flags, void* const* peer_bufs, uint32_t* state, int rank,
    int world, int64_t max_message_bytes, b200q_stream_t stream);

/*
 * residual += input; input = rms_norm(residual) * weight, in place, one row per token.
 * With residual == NULL: input = rms_norm(input) * weight.
 * Replaces: fused_add_rms_norm / rms_norm, csrc/layernorm_kernels.cu:17-58,60-149
 *           (vllm/_custom_ops.py:328-339); same rounding points: the sum is rounded to
 *           16 bits, the variance is taken from the rounded sum in fp32, (z * rstd) is
 *           rounded, then multiplied by the weight in 16 bits.
 *   input     [num_tokens, hidden_size] 16-bit, row stride ld_input elements
 *   residual  [num_tokens, hidden_size] contiguous, or NULL
 *   weight    [hidden_size]; hidden_size % 8 == 0; all pointers 16 B aligned
 */
int b200q_fused_add_rms_norm(void* input, int64_t ld_input, void* residual, const void* weight,
                             float epsilon, int64_t num_tokens, int64_t hidden_size, int dtype,
                             b200q_stream_t stream);

/*
 * The same with the SUM all-reduce of `input` over the peer link in front, in one
 * kernel: what follows RowParallelLinear in a decoder layer (all-reduce, residual
 * add, RMSNorm; the reference fuses these through a pattern-matching pass,
 * vllm/compilation/collective_fusion.py:656-775).  `input` holds this rank's partial
 * on entry (contiguous) and the normalised row on exit; link arguments as in
 * b200q_all_reduce; num_tokens * hidden_size * 2 <= max_message_bytes.
 */
int b200q_all_reduce_fused_add_rms_norm(void* const* peer_bufs, uint32_t* state, int rank, int world,
                                        int64_t max_message_bytes, void* input, void* residual,
                                        const void* weight, float epsilon, int64_t num_tokens,
                                        int64_t hidden_size, int dtype, b200q_stream_t stream);

/*
 * out[t, i] = silu(input[t, i]) * input[t, d + i]  (the MLP step between the gate_up and
 * down projections).  Replaces: silu_and_mul, csrc/activation_kernels.cu:22-38,85-89.
 *   input [num_tokens, 2 * d], out [num_tokens, d], contiguous, d % 8 == 0
 */
int b200q_silu_and_mul(void* out, const void* input, int64_t num_tokens, int64_t d, int dtype,
                       b200q_stream_t stream);

/*
 * b200q_marlin_gemm for callers that cannot allocate device memory (a plugin
 * running inside another framework's fixed memory plan, code that runs while a
 * stream is being captured, a process whose device memory belongs to another
 * component).  Same arguments as b200q_marlin_gemm without scratch /
 * scratch_bytes: the scratch is a fixed array inside the library, of
 * b200q_marlin_gemm_noalloc_max_scratch() bytes (16 MiB), which every GPU that
 * loads the library holds until the process exits.  The call allocates nothing
 * and calls no allocating routine.
 *   - Problems whose b200q_marlin_gemm_scratch_bytes(...) exceeds that size are
 *     rejected with B200Q_ESCRATCH (use b200q_marlin_gemm with your own scratch).
 *   - The first call on each device resolves the array's device address
 *     (cudaGetSymbolAddress); make that first call before any stream capture.
 *     The address stays valid for the life of the device's primary context
 *     (reload the library after cudaDeviceReset).
 *   - The array of the CURRENT device is used: the device that owns the tensors
 *     and the stream must be current (a mismatch is rejected with B200Q_EINVAL
 *     where the output pointer shows it).
 *   - All calls on a device share the one array: calls that can overlap on the
 *     GPU (different streams) race on it and must be ordered by the caller.
 * This entry point has no counterpart in the reference.
 */
size_t b200q_marlin_gemm_noalloc_max_scratch(void);
int b200q_marlin_gemm_noalloc(const void* a, int64_t lda, const uint32_t* b_q_weight,
                              const void* b_scales, const uint32_t* b_zeros,
                              const int32_t* g_idx, const int32_t* perm,
                              const void* b_bias, void* c, int32_t* workspace,
                              int64_t workspace_len, int64_t b_q_type_id, int a_dtype,
                              int64_t size_m, int64_t size_n, int64_t size_k,
                              int64_t num_groups, unsigned flags, b200q_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
