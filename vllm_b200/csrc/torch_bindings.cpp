// Torch operator registration for the quantized linear path: the ops of the
// reference's csrc/torch_bindings.cpp:304-327 (permute_cols, gptq_marlin_gemm,
// gptq_marlin_repack, awq_marlin_repack) with the same schemas, implemented for
// the CUDA dispatch key on top of the C ABI of libb200q.so, plus one op the
// reference does not have: the row-parallel GEMM with the all-reduce in the same
// call (gptq_marlin_gemm_all_reduce).
//
// The argument checks mirror gptq_marlin.cu:688-902, gptq_marlin_repack.cu:251-322,
// awq_marlin_repack.cu:189-248 and permute_cols.cu:74-88 (same conditions, same
// messages where the reference has one), so a caller sees the errors it would see
// from the reference; a status from the library becomes a c10::Error carrying
// b200q_last_error().
//
// The namespace is chosen at load time (b200q_torch_register): "_C" to stand in
// for the reference's extension, another name when a different extension already
// owns those operator names in the process.
//
// Compiled with the host compiler only (no device code here); links libb200q.so.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>

#include "../../include/b200q.h"

namespace {

#define B200Q_TORCH_OK(rc, what) TORCH_CHECK((rc) == B200Q_OK, what, ": ", b200q_last_error())

// ScalarType ids (csrc/core/scalar_type.hpp:17-157): exponent | mantissa << 8 | signed << 16 |
// bias << 17 | finite_values_only << 49 | nan_repr << 50.
struct TypeInfo {
  int bits;
  bool int_with_bias, is_float;
};
bool decode_type(int64_t id, TypeInfo* t) {
  const int exponent = (int)(id & 0xff), mantissa = (int)((id >> 8) & 0xff);
  const bool is_signed = (id >> 16) & 1;
  const int64_t bias = (id >> 17) & 0xffffffffll;
  t->bits = exponent + mantissa + (is_signed ? 1 : 0);
  t->is_float = exponent != 0;
  t->int_with_bias = exponent == 0 && bias != 0;
  return t->bits == 4 || t->bits == 8;
}

// Scratch of the GEMM: fp32 partial sums, and the gathered activations of act-order
// layers.  One grow-only buffer per (device, stream): calls on one stream are ordered,
// so they can share it; calls on different streams must not.
at::Tensor& scratch_for(const at::Device& dev, cudaStream_t stream, size_t bytes) {
  static std::mutex mu;
  static std::unordered_map<uint64_t, at::Tensor> cache;
  const uint64_t key = ((uint64_t)(uintptr_t)stream << 8) ^ (uint64_t)(dev.index() & 0xff);
  std::lock_guard<std::mutex> lock(mu);
  at::Tensor& t = cache[key];
  if (!t.defined() || (size_t)t.numel() < bytes)
    t = at::empty({(int64_t)bytes}, at::TensorOptions().dtype(at::kByte).device(dev));
  return t;
}

struct GemmArgs {
  const void *a, *scales, *bias;
  const void* global_scale;  // NVFP4
  int fp4_scales;            // 0, or B200Q_FP4_SCALES_* for float4_e2m1f weights
  const uint32_t *b, *zeros;
  const int32_t *g_idx, *perm;
  int64_t lda, num_groups;
  int dtype;
  unsigned flags;
  bool act_order;
};

// Checks of gptq_marlin.cu:688-902; fills `g` and returns the output tensor.
at::Tensor check_gemm(const at::Tensor& a, const std::optional<at::Tensor>& c_or_none,
                      const at::Tensor& b_q_weight, const std::optional<at::Tensor>& b_bias_or_none,
                      const at::Tensor& b_scales, const std::optional<at::Tensor>& global_scale,
                      const std::optional<at::Tensor>& b_zeros_or_none,
                      const std::optional<at::Tensor>& g_idx_or_none,
                      const std::optional<at::Tensor>& perm_or_none, const at::Tensor& workspace,
                      int64_t b_q_type, int64_t size_m, int64_t size_n, int64_t size_k,
                      bool is_k_full, bool use_atomic_add, bool use_fp32_reduce, bool is_zp_float,
                      GemmArgs* g) {
  TypeInfo qt;
  TORCH_CHECK(decode_type(b_q_type, &qt),
              "b_q_type must be uint4b8, uint8b128 (has_zp = False) or u4, u8 (has_zp = True); id ",
              b_q_type, " is not supported");
  const int pf = 32 / qt.bits;
  TORCH_CHECK(a.dim() == 2 && a.size(0) == size_m, "Shape mismatch: a.size(0) = ", a.size(0),
              ", size_m = ", size_m);
  TORCH_CHECK(a.size(1) == size_k, "Shape mismatch: a.size(1) = ", a.size(1), ", size_k = ", size_k);
  TORCH_CHECK(size_k % 16 == 0, "size_k = ", size_k, " is not divisible by tile_size = 16");
  TORCH_CHECK(b_q_weight.dim() == 2 && size_k / 16 == b_q_weight.size(0),
              "Shape mismatch: b_q_weight.size(0) = ", b_q_weight.size(0), ", size_k = ", size_k,
              ", tile_size = 16");
  TORCH_CHECK(b_q_weight.size(1) % 16 == 0, "b_q_weight.size(1) = ", b_q_weight.size(1),
              " is not divisible by tile_size = 16");
  const int64_t actual_n = b_q_weight.size(1) / 16 * pf;
  TORCH_CHECK(size_n == actual_n, "size_n = ", size_n, ", actual_size_n = ", actual_n);
  TORCH_CHECK(a.is_cuda(), "A is not on GPU");
  TORCH_CHECK(a.stride(1) == 1, "A.stride(1) is not 1");
  TORCH_CHECK(a.stride(0) % 8 == 0, "A.stride(0) must divisible by 8");
  TORCH_CHECK(((uintptr_t)a.data_ptr()) % 16 == 0, "A must aligned to 16 bytes");
  TORCH_CHECK(b_q_weight.is_cuda(), "b_q_weight is not on GPU");
  TORCH_CHECK(b_q_weight.is_contiguous(), "b_q_weight is not contiguous");
  TORCH_CHECK(b_scales.is_cuda(), "b_scales is not on GPU");
  TORCH_CHECK(b_scales.is_contiguous(), "b_scales is not contiguous");
  TORCH_CHECK(a.scalar_type() == at::kHalf || a.scalar_type() == at::kBFloat16,
              "gpt_marlin_gemm only supports bfloat16 and float16");
  // float4_e2m1f weights carry 8-bit scales: float8_e4m3fn per 16 values (NVFP4) or
  // float8_e8m0fnu per 32 (MXFP4) (gptq_marlin.cu:907-917)
  const bool is_fp4 = qt.is_float && qt.bits == 4;
  g->fp4_scales = 0;
  g->global_scale = nullptr;
  if (is_fp4) {
    if (b_scales.scalar_type() == at::kFloat8_e4m3fn) g->fp4_scales = B200Q_FP4_SCALES_E4M3;
    else if (b_scales.scalar_type() == at::kFloat8_e8m0fnu) g->fp4_scales = B200Q_FP4_SCALES_E8M0;
    else TORCH_CHECK(false, "float4_e2m1f only supports group_size == 16 (NVFP4) ",
                     "and group_size == 32 (MXFP4): b_scales must be float8_e4m3fn or float8_e8m0fnu");
  } else {
    TORCH_CHECK(b_scales.scalar_type() == a.scalar_type(), "b_scales must have the dtype of a");
  }

  at::Tensor c;
  if (c_or_none.has_value()) {
    c = c_or_none.value();
    TORCH_CHECK(c.is_cuda(), "c is not on GPU");
    TORCH_CHECK(c.is_contiguous(), "c is not contiguous");
    TORCH_CHECK(c.size(0) == size_m, "Shape mismatch: c.size(0) = ", c.size(0), ", size_m = ", size_m);
    TORCH_CHECK(c.size(1) == size_n, "Shape mismatch: c.size(1) = ", c.size(1), ", size_n = ", size_n);
    TORCH_CHECK(c.scalar_type() == a.scalar_type(), "c must have the dtype of a");
  } else {
    c = at::empty({size_m, size_n}, a.options());
  }
  g->act_order = false;
  if (size_m == 0) return c;

  TORCH_CHECK(b_scales.dim() == 2, "b_scales rank = ", b_scales.dim(), " is not 2");
  TORCH_CHECK(b_scales.size(1) == size_n, "b_scales dim 1 = ", b_scales.size(1),
              " is not size_n = ", size_n);
  g->num_groups = b_scales.size(0);

  g->g_idx = g->perm = nullptr;
  if (g_idx_or_none.has_value() && perm_or_none.has_value()) {
    const at::Tensor& g_idx = g_idx_or_none.value();
    const at::Tensor& perm = perm_or_none.value();
    TORCH_CHECK(g_idx.is_cuda(), "g_idx is not on GPU");
    TORCH_CHECK(g_idx.is_contiguous(), "g_idx is not contiguous");
    TORCH_CHECK(perm.is_cuda(), "perm is not on GPU");
    TORCH_CHECK(perm.is_contiguous(), "perm is not contiguous");
    TORCH_CHECK((g_idx.size(-1) == 0 && perm.size(-1) == 0) ||
                    (g_idx.size(-1) == size_k && perm.size(-1) == size_k),
                "Unexpected g_idx.size(-1) = ", g_idx.size(-1), " and perm.size(-1) = ",
                perm.size(-1), ", where size_k = ", size_k);
    if (g_idx.size(-1) != 0) {
      TORCH_CHECK(g_idx.scalar_type() == at::kInt && perm.scalar_type() == at::kInt,
                  "g_idx and perm must be int32");
      g->g_idx = g_idx.data_ptr<int32_t>();
      g->perm = perm.data_ptr<int32_t>();
      g->act_order = true;
    }
  }
  if (global_scale.has_value()) {
    TORCH_CHECK(g->fp4_scales == B200Q_FP4_SCALES_E4M3,
                "global_scale can only be used for nvfp4 format.");
    const at::Tensor& gs = global_scale.value();
    TORCH_CHECK(gs.is_cuda() && gs.numel() == 1 && gs.scalar_type() == a.scalar_type(),
                "global_scale must be one value of the dtype of a, on the GPU");
    g->global_scale = gs.data_ptr();
  } else {
    TORCH_CHECK(g->fp4_scales != B200Q_FP4_SCALES_E4M3,
                "the global_scale parameter must be passed for nvfp4 format.");
  }

  g->bias = nullptr;
  if (b_bias_or_none.has_value()) {
    const at::Tensor& bias = b_bias_or_none.value();
    TORCH_CHECK(bias.is_cuda(), "b_bias is not on GPU");
    TORCH_CHECK(bias.is_contiguous(), "b_bias is not contiguous");
    TORCH_CHECK(bias.size(0) == size_n, "b_bias.size(0) != size_n");
    TORCH_CHECK(bias.scalar_type() == a.scalar_type(), "b_bias must have the dtype of a");
    g->bias = bias.data_ptr();
  }

  g->zeros = nullptr;
  bool has_zp = false;
  if (b_zeros_or_none.has_value()) {
    const at::Tensor& z = b_zeros_or_none.value();
    TORCH_CHECK(z.is_cuda(), "b_zeros is not on GPU");
    TORCH_CHECK(z.is_contiguous(), "b_zeros is not contiguous");
    if (z.size(-1) > 0) {
      has_zp = true;
      TORCH_CHECK(!qt.int_with_bias && !qt.is_float,
                  "b_q_type must be u4 or u8 when has_zp = True. Got id = ", b_q_type);
      TORCH_CHECK(z.dim() == 2, "b_zeros rank = ", z.dim(), " is not 2");
      TORCH_CHECK(z.size(0) == g->num_groups, "b_zeros dim 0 = ", z.size(0),
                  " is not num_groups = ", g->num_groups);
      if (is_zp_float) {
        TORCH_CHECK(a.scalar_type() == at::kHalf,
                    "Computation type must be float16 (half) when using float zero points.");
        TORCH_CHECK(z.size(1) == size_n, "b_zeros dim 1 = ", z.size(1), " is not size_n = ", size_n);
        TORCH_CHECK(z.scalar_type() == a.scalar_type(), "float zero-points must have the dtype of a");
      } else {
        TORCH_CHECK(z.size(1) == size_n / pf, "b_zeros dim 1 = ", z.size(1),
                    " is not size_n / pack_factor = ", size_n / pf);
        TORCH_CHECK(z.scalar_type() == at::kInt, "b_zeros must be int32");
      }
      g->zeros = static_cast<const uint32_t*>(z.data_ptr());
    }
  }
  if (!has_zp)
    TORCH_CHECK(qt.int_with_bias || qt.is_float,
                "b_q_type must be uint4b8, uint8b128, float8_e4m3fn or float4_e2m1f when "
                "has_zp = False. Got id = ", b_q_type);

  TORCH_CHECK(size_n % 64 == 0, "size_n = ", size_n, ", is not divisible by min_thread_n = 64");
  TORCH_CHECK(workspace.is_cuda() && workspace.scalar_type() == at::kInt,
              "workspace must be int32 on GPU");
  const int sms = b200q_sm_count();
  TORCH_CHECK(workspace.numel() >= sms, "workspace.numel = ", workspace.numel(),
              " is below min_workspace_size = ", sms);
  g->a = a.data_ptr();
  g->lda = a.stride(0);
  g->b = static_cast<const uint32_t*>(b_q_weight.data_ptr());
  g->scales = b_scales.data_ptr();
  g->dtype = a.scalar_type() == at::kBFloat16 ? B200Q_BF16 : B200Q_F16;
  g->flags = (is_k_full ? B200Q_FLAG_K_FULL : 0) | (use_atomic_add ? B200Q_FLAG_ATOMIC_ADD : 0) |
             (use_fp32_reduce ? B200Q_FLAG_FP32_REDUCE : 0) |
             ((is_zp_float && has_zp) ? B200Q_FLAG_ZP_FLOAT : 0);
  return c;
}

// gptq_marlin_gemm, csrc/quantization/gptq_marlin/gptq_marlin.cu:674-959
at::Tensor gptq_marlin_gemm(at::Tensor& a, std::optional<at::Tensor> c_or_none,
                            at::Tensor& b_q_weight, std::optional<at::Tensor> const& b_bias_or_none,
                            at::Tensor& b_scales, std::optional<at::Tensor> const& global_scale,
                            std::optional<at::Tensor> const& b_zeros_or_none,
                            std::optional<at::Tensor> const& g_idx_or_none,
                            std::optional<at::Tensor> const& perm_or_none, at::Tensor& workspace,
                            int64_t b_q_type, int64_t size_m, int64_t size_n, int64_t size_k,
                            bool is_k_full, bool use_atomic_add, bool use_fp32_reduce,
                            bool is_zp_float) {
  GemmArgs g{};
  at::Tensor c = check_gemm(a, c_or_none, b_q_weight, b_bias_or_none, b_scales, global_scale,
                            b_zeros_or_none, g_idx_or_none, perm_or_none, workspace, b_q_type,
                            size_m, size_n, size_k, is_k_full, use_atomic_add, use_fp32_reduce,
                            is_zp_float, &g);
  if (size_m == 0) return c;
  const c10::cuda::OptionalCUDAGuard guard(device_of(a));
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream(a.get_device());
  const size_t nbytes =
      b200q_marlin_gemm_preferred_scratch_bytes(size_m, size_n, size_k, g.act_order ? 1 : 0);
  at::Tensor& scratch = scratch_for(a.device(), stream, nbytes);
  int rc;
  if (g.fp4_scales != 0) {
    TORCH_CHECK(g.zeros == nullptr && !g.act_order,
                "float4_e2m1f weights take neither zero-points nor act_order");
    rc = b200q_marlin_gemm_fp4(g.a, g.lda, g.b, g.scales, g.global_scale, g.fp4_scales, g.bias,
                               c.data_ptr(), scratch.data_ptr(), (size_t)scratch.numel(),
                               workspace.data_ptr<int32_t>(), workspace.numel(), g.dtype, size_m,
                               size_n, size_k, g.num_groups, stream);
  } else {
    rc = b200q_marlin_gemm(g.a, g.lda, g.b, g.scales, g.zeros, g.g_idx, g.perm, g.bias,
                           c.data_ptr(), scratch.data_ptr(), (size_t)scratch.numel(),
                           workspace.data_ptr<int32_t>(), workspace.numel(), b_q_type, g.dtype,
                           size_m, size_n, size_k, g.num_groups, g.flags, stream);
  }
  B200Q_TORCH_OK(rc, "gptq_marlin_gemm");
  return c;
}

// The row-parallel form: the same GEMM on this rank's K shard followed by the SUM all-reduce
// of the output over the peer-memory link (vllm/model_executor/layers/linear.py:1386-1411 does
// the two as separate steps).  peer_ptrs: int64 device tensor [world] of the ranks' receive
// buffers; state: int32 device tensor of b200q_all_reduce_state_bytes().
at::Tensor gptq_marlin_gemm_all_reduce(
    at::Tensor& a, std::optional<at::Tensor> c_or_none, at::Tensor& b_q_weight,
    std::optional<at::Tensor> const& b_bias_or_none, at::Tensor& b_scales,
    std::optional<at::Tensor> const& global_scale, std::optional<at::Tensor> const& b_zeros_or_none,
    std::optional<at::Tensor> const& g_idx_or_none, std::optional<at::Tensor> const& perm_or_none,
    at::Tensor& workspace, int64_t b_q_type, int64_t size_m, int64_t size_n, int64_t size_k,
    bool is_k_full, bool use_atomic_add, bool use_fp32_reduce, bool is_zp_float,
    at::Tensor& peer_ptrs, at::Tensor& state, int64_t rank, int64_t world,
    int64_t max_message_bytes) {
  GemmArgs g{};
  at::Tensor c = check_gemm(a, c_or_none, b_q_weight, b_bias_or_none, b_scales, global_scale,
                            b_zeros_or_none, g_idx_or_none, perm_or_none, workspace, b_q_type,
                            size_m, size_n, size_k, is_k_full, use_atomic_add, use_fp32_reduce,
                            is_zp_float, &g);
  TORCH_CHECK(g.fp4_scales == 0, "gptq_marlin_gemm_all_reduce does not take float4_e2m1f weights");
  if (size_m == 0) return c;
  TORCH_CHECK(peer_ptrs.is_cuda() && peer_ptrs.scalar_type() == at::kLong &&
                  peer_ptrs.numel() >= world,
              "peer_ptrs must be an int64 CUDA tensor with one entry per rank");
  TORCH_CHECK(state.is_cuda() && state.scalar_type() == at::kInt &&
                  (size_t)state.numel() * 4 >= b200q_all_reduce_state_bytes(),
              "state must be an int32 CUDA tensor of b200q_all_reduce_state_bytes()");
  const c10::cuda::OptionalCUDAGuard guard(device_of(a));
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream(a.get_device());
  const size_t nbytes =
      b200q_marlin_gemm_preferred_scratch_bytes(size_m, size_n, size_k, g.act_order ? 1 : 0);
  at::Tensor& scratch = scratch_for(a.device(), stream, nbytes);
  const int rc = b200q_marlin_gemm_all_reduce(
      g.a, g.lda, g.b, g.scales, g.zeros, g.g_idx, g.perm, g.bias, c.data_ptr(), scratch.data_ptr(),
      (size_t)scratch.numel(), workspace.data_ptr<int32_t>(), workspace.numel(), b_q_type, g.dtype,
      size_m, size_n, size_k, g.num_groups, g.flags,
      reinterpret_cast<void* const*>(peer_ptrs.data_ptr<int64_t>()),
      reinterpret_cast<uint32_t*>(state.data_ptr<int32_t>()), (int)rank, (int)world,
      max_message_bytes, stream);
  B200Q_TORCH_OK(rc, "gptq_marlin_gemm_all_reduce");
  return c;
}

// gptq_marlin_repack, csrc/quantization/gptq_marlin/gptq_marlin_repack.cu:251-322
at::Tensor gptq_marlin_repack(at::Tensor& b_q_weight, at::Tensor& perm, int64_t size_k,
                              int64_t size_n, int64_t num_bits) {
  TORCH_CHECK(size_k % 16 == 0, "size_k = ", size_k, " is not divisible by tile_k_size = 16");
  TORCH_CHECK(size_n % 64 == 0, "size_n = ", size_n, " is not divisible by tile_n_size = 64");
  TORCH_CHECK(num_bits == 4 || num_bits == 8, "num_bits must be 4 or 8. Got = ", num_bits);
  const int64_t pf = 32 / num_bits;
  TORCH_CHECK(b_q_weight.is_cuda(), "b_q_weight is not on GPU");
  TORCH_CHECK(b_q_weight.is_contiguous(), "b_q_weight is not contiguous");
  TORCH_CHECK(b_q_weight.scalar_type() == at::kInt, "b_q_weight type is not kInt");
  TORCH_CHECK(b_q_weight.dim() == 2 && b_q_weight.size(0) == size_k / pf,
              "Shape mismatch: b_q_weight.size(0) = ", b_q_weight.size(0), ", size_k = ", size_k,
              ", pack_factor = ", pf);
  TORCH_CHECK(b_q_weight.size(1) == size_n, "b_q_weight.size(1) = ", b_q_weight.size(1),
              " is not size_n = ", size_n);
  TORCH_CHECK(perm.is_cuda(), "perm is not on GPU");
  TORCH_CHECK(perm.is_contiguous(), "perm is not contiguous");
  TORCH_CHECK(perm.scalar_type() == at::kInt, "perm type is not at::kInt");
  const bool has_perm = perm.numel() > 0;
  TORCH_CHECK(!has_perm || perm.numel() == size_k, "perm.numel() = ", perm.numel(),
              " is not size_k");
  const c10::cuda::OptionalCUDAGuard guard(device_of(b_q_weight));
  at::Tensor out = at::empty({size_k / 16, size_n * 16 / pf}, b_q_weight.options());
  const int rc = b200q_gptq_marlin_repack(
      static_cast<const uint32_t*>(b_q_weight.data_ptr()),
      has_perm ? perm.data_ptr<int32_t>() : nullptr, static_cast<uint32_t*>(out.data_ptr()), size_k,
      size_n, (int)num_bits, at::cuda::getCurrentCUDAStream(b_q_weight.get_device()));
  B200Q_TORCH_OK(rc, "gptq_marlin_repack");
  return out;
}

// awq_marlin_repack, csrc/quantization/gptq_marlin/awq_marlin_repack.cu:189-248
at::Tensor awq_marlin_repack(at::Tensor& b_q_weight, int64_t size_k, int64_t size_n,
                             int64_t num_bits) {
  TORCH_CHECK(size_k % 16 == 0, "size_k = ", size_k, " is not divisible by tile_k_size = 16");
  TORCH_CHECK(size_n % 64 == 0, "size_n = ", size_n, " is not divisible by tile_n_size = 64");
  TORCH_CHECK(num_bits == 4 || num_bits == 8, "num_bits must be 4 or 8. Got = ", num_bits);
  const int64_t pf = 32 / num_bits;
  TORCH_CHECK(b_q_weight.is_cuda(), "b_q_weight is not on GPU");
  TORCH_CHECK(b_q_weight.is_contiguous(), "b_q_weight is not contiguous");
  TORCH_CHECK(b_q_weight.scalar_type() == at::kInt, "b_q_weight type is not kInt");
  TORCH_CHECK(b_q_weight.dim() == 2 && b_q_weight.size(0) == size_k, "b_q_weight.size(0) = ",
              b_q_weight.size(0), " is not size_k = ", size_k);
  TORCH_CHECK(b_q_weight.size(1) == size_n / pf, "Shape mismatch: b_q_weight.size(1) = ",
              b_q_weight.size(1), ", size_n = ", size_n, ", pack_factor = ", pf);
  const c10::cuda::OptionalCUDAGuard guard(device_of(b_q_weight));
  at::Tensor out = at::empty({size_k / 16, size_n * 16 / pf}, b_q_weight.options());
  const int rc = b200q_awq_marlin_repack(
      static_cast<const uint32_t*>(b_q_weight.data_ptr()), static_cast<uint32_t*>(out.data_ptr()),
      size_k, size_n, (int)num_bits, at::cuda::getCurrentCUDAStream(b_q_weight.get_device()));
  B200Q_TORCH_OK(rc, "awq_marlin_repack");
  return out;
}

// permute_cols, csrc/permute_cols.cu:74-88
at::Tensor permute_cols(at::Tensor const& A, at::Tensor const& perm) {
  TORCH_CHECK(A.is_cuda() && perm.is_cuda(), "permute_cols: tensors must be on GPU");
  TORCH_CHECK(A.dim() == 2 && A.stride(1) == 1, "A must be a row major tensor");
  TORCH_CHECK(A.scalar_type() == at::kHalf || A.scalar_type() == at::kBFloat16,
              "A must be a 16-bit float tensor");
  TORCH_CHECK(perm.scalar_type() == at::kInt && perm.is_contiguous() && perm.numel() == A.size(1),
              "perm must be a contiguous int32 tensor of A.size(1) entries");
  const c10::cuda::OptionalCUDAGuard guard(device_of(A));
  at::Tensor out = at::empty({A.size(0), A.size(1)}, A.options());
  const int rc = b200q_permute_cols(A.data_ptr(), A.stride(0), perm.data_ptr<int32_t>(),
                                    out.data_ptr(), A.size(0), A.size(1),
                                    at::cuda::getCurrentCUDAStream(A.get_device()));
  B200Q_TORCH_OK(rc, "permute_cols");
  return out;
}

std::unique_ptr<torch::Library> g_defs, g_impls;

}  // namespace

// Define the operators in namespace `ns` and register the CUDA implementations.  Returns 0,
// or -1 when the definitions clash with operators that already exist there (nothing is then
// registered by this call that was not registered before the clash).
// moe_wna16_marlin_gemm, csrc/moe/marlin_moe_wna16/ops.cu:693-960
at::Tensor moe_wna16_marlin_gemm(
    at::Tensor& a, std::optional<at::Tensor> const& c_or_none, at::Tensor& b_q_weight,
    std::optional<at::Tensor> const& b_bias_or_none, at::Tensor& b_scales,
    std::optional<at::Tensor> const& global_scale_or_none,
    std::optional<at::Tensor> const& b_zeros_or_none, std::optional<at::Tensor> const& g_idx_or_none,
    std::optional<at::Tensor> const& perm_or_none, at::Tensor& workspace,
    at::Tensor& sorted_token_ids, at::Tensor& expert_ids, at::Tensor& num_tokens_past_padded,
    at::Tensor& topk_weights, int64_t moe_block_size, int64_t top_k, bool mul_topk_weights,
    bool is_ep, int64_t b_q_type_id, int64_t size_m, int64_t size_n, int64_t size_k, bool is_k_full,
    bool use_atomic_add, bool use_fp32_reduce, bool is_zp_float) {
  (void)workspace; (void)is_ep; (void)is_k_full; (void)use_atomic_add; (void)use_fp32_reduce;
  TypeInfo qt;
  TORCH_CHECK(decode_type(b_q_type_id, &qt) && !qt.is_float,
              "moe_wna16_marlin_gemm: b_q_type must be uint4b8, uint8b128, uint4 or uint8; id ",
              b_q_type_id, " is not supported");
  const int pf = 32 / qt.bits;
  TORCH_CHECK(moe_block_size == 8 ||
                  (moe_block_size % 16 == 0 && moe_block_size >= 16 && moe_block_size <= 64),
              "unsupported moe_block_size=", moe_block_size);
  TORCH_CHECK(a.dim() == 2 && a.size(0) == size_m && a.size(1) == size_k,
              "Shape mismatch: a = [", a.size(0), ", ", a.size(1), "], size_m = ", size_m,
              ", size_k = ", size_k);
  TORCH_CHECK(a.is_cuda() && a.stride(1) == 1 && a.stride(0) % 8 == 0, "A must be a CUDA tensor ",
              "with unit inner stride and a row stride divisible by 8");
  TORCH_CHECK(a.scalar_type() == at::kHalf || a.scalar_type() == at::kBFloat16,
              "moe_wna16_marlin_gemm only supports bfloat16 and float16");
  TORCH_CHECK(b_q_weight.is_cuda() && b_q_weight.is_contiguous() && b_q_weight.dim() == 3,
              "b_q_weight must be a contiguous CUDA tensor [experts, size_k / 16, size_n * 16 / pack_factor]");
  const int64_t num_experts = b_q_weight.size(0);
  TORCH_CHECK(size_k % 16 == 0 && b_q_weight.size(1) == size_k / 16,
              "Shape mismatch: b_q_weight.size(1) = ", b_q_weight.size(1), ", size_k = ", size_k);
  TORCH_CHECK(b_q_weight.size(2) % 16 == 0 && b_q_weight.size(2) / 16 * pf == size_n,
              "size_n = ", size_n, ", actual_size_n = ", b_q_weight.size(2) / 16 * pf);
  TORCH_CHECK(b_scales.is_cuda() && b_scales.is_contiguous() && b_scales.dim() == 3 &&
                  b_scales.size(0) == num_experts && b_scales.size(2) == size_n &&
                  b_scales.scalar_type() == a.scalar_type(),
              "b_scales must be [experts, groups, size_n] of the dtype of a");
  const int64_t num_groups = b_scales.size(1);
  TORCH_CHECK(!global_scale_or_none.has_value(), "global_scale can only be used for nvfp4 format.");
  TORCH_CHECK(!is_zp_float, "moe_wna16_marlin_gemm: float zero-points are not supported");
  bool act_order = false;
  if (g_idx_or_none.has_value() && perm_or_none.has_value())
    act_order = g_idx_or_none.value().size(-1) > 0 || perm_or_none.value().size(-1) > 0;
  TORCH_CHECK(!act_order, "moe_wna16_marlin_gemm: act_order is not supported");
  const uint32_t* zeros = nullptr;
  if (b_zeros_or_none.has_value() && b_zeros_or_none.value().size(-1) > 0) {
    const at::Tensor& z = b_zeros_or_none.value();
    TORCH_CHECK(z.is_cuda() && z.is_contiguous() && z.dim() == 3, "b_zeros rank = ", z.dim(), " is not 3");
    TORCH_CHECK(z.size(0) == num_experts && z.size(1) == num_groups && z.size(2) == size_n / pf &&
                    z.scalar_type() == at::kInt,
                "b_zeros must be int32 [experts, groups, size_n / pack_factor]");
    zeros = static_cast<const uint32_t*>(z.data_ptr());
  }
  const void* bias = nullptr;
  if (b_bias_or_none.has_value()) {
    const at::Tensor& b = b_bias_or_none.value();
    TORCH_CHECK(b.is_cuda() && b.is_contiguous() && b.numel() == num_experts * size_n &&
                    b.scalar_type() == a.scalar_type(),
                "b_bias must be [experts, size_n] of the dtype of a");
    bias = b.data_ptr();
  }
  TORCH_CHECK(sorted_token_ids.is_cuda() && sorted_token_ids.is_contiguous() &&
                  sorted_token_ids.scalar_type() == at::kInt,
              "sorted_token_ids must be a contiguous int32 CUDA tensor");
  TORCH_CHECK(expert_ids.is_cuda() && expert_ids.is_contiguous() && expert_ids.scalar_type() == at::kInt,
              "expert_ids must be a contiguous int32 CUDA tensor");
  TORCH_CHECK(num_tokens_past_padded.is_cuda() && num_tokens_past_padded.scalar_type() == at::kInt &&
                  num_tokens_past_padded.numel() >= 1,
              "num_tokens_past_padded must be an int32 CUDA tensor");
  const int64_t sorted_len = sorted_token_ids.numel() / moe_block_size * moe_block_size;
  TORCH_CHECK(expert_ids.numel() >= sorted_len / moe_block_size, "expert_ids has ", expert_ids.numel(),
              " entries for ", sorted_len / moe_block_size, " blocks");
  TORCH_CHECK(topk_weights.is_cuda() && topk_weights.scalar_type() == at::kFloat &&
                  topk_weights.is_contiguous() && (!mul_topk_weights || topk_weights.numel() >= size_m * top_k),
              "topk_weights must be a contiguous float32 CUDA tensor of size_m * top_k values");
  at::Tensor c;
  if (c_or_none.has_value()) {
    c = c_or_none.value();
    TORCH_CHECK(c.is_cuda() && c.is_contiguous() && c.size(0) == size_m * top_k && c.size(1) == size_n &&
                    c.scalar_type() == a.scalar_type(),
                "c must be [size_m * top_k, size_n] of the dtype of a");
  } else {
    c = at::empty({size_m * top_k, size_n}, a.options());
  }
  if (size_m == 0) return c;
  const c10::cuda::OptionalCUDAGuard guard(device_of(a));
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream(a.get_device());
  const int rc = b200q_moe_wna16_marlin_gemm(
      a.data_ptr(), a.stride(0), static_cast<const uint32_t*>(b_q_weight.data_ptr()),
      b_scales.data_ptr(), zeros, bias, c.data_ptr(), sorted_token_ids.data_ptr<int32_t>(),
      expert_ids.data_ptr<int32_t>(), num_tokens_past_padded.data_ptr<int32_t>(),
      topk_weights.data_ptr<float>(), sorted_len, moe_block_size, top_k, mul_topk_weights ? 1 : 0,
      num_experts, b_q_type_id, a.scalar_type() == at::kBFloat16 ? B200Q_BF16 : B200Q_F16, size_m,
      size_n, size_k, num_groups, stream);
  B200Q_TORCH_OK(rc, "moe_wna16_marlin_gemm");
  return c;
}

std::unique_ptr<torch::Library> g_moe_defs, g_moe_impls;

extern "C" int b200q_torch_register(const char* ns) {
  if (g_defs) return 0;
  try {
    const std::string name(ns);
    g_defs = std::make_unique<torch::Library>(torch::Library::FRAGMENT, name, std::nullopt, __FILE__,
                                              __LINE__);
    // schemas of csrc/torch_bindings.cpp:304-327
    g_defs->def("permute_cols(Tensor A, Tensor perm) -> Tensor");
    g_defs->def(
        "gptq_marlin_gemm(Tensor a, Tensor? c_or_none, Tensor b_q_weight, "
        "Tensor? b_bias_or_none, Tensor b_scales, Tensor? global_scale, "
        "Tensor? b_zeros_or_none, Tensor? g_idx_or_none, Tensor? perm_or_none, "
        "Tensor workspace, int b_q_type, SymInt size_m, SymInt size_n, "
        "SymInt size_k, bool is_k_full, bool use_atomic_add, "
        "bool use_fp32_reduce, bool is_zp_float) -> Tensor");
    g_defs->def(
        "gptq_marlin_repack(Tensor b_q_weight, Tensor perm, SymInt size_k, "
        "SymInt size_n, int num_bits) -> Tensor");
    g_defs->def(
        "awq_marlin_repack(Tensor b_q_weight, SymInt size_k, SymInt size_n, "
        "int num_bits) -> Tensor");
    // no counterpart in the reference: the same arguments, then the peer-memory link
    g_defs->def(
        "gptq_marlin_gemm_all_reduce(Tensor a, Tensor? c_or_none, Tensor b_q_weight, "
        "Tensor? b_bias_or_none, Tensor b_scales, Tensor? global_scale, "
        "Tensor? b_zeros_or_none, Tensor? g_idx_or_none, Tensor? perm_or_none, "
        "Tensor workspace, int b_q_type, SymInt size_m, SymInt size_n, "
        "SymInt size_k, bool is_k_full, bool use_atomic_add, "
        "bool use_fp32_reduce, bool is_zp_float, Tensor peer_ptrs, Tensor(a!) state, "
        "int rank, int world, int max_message_bytes) -> Tensor");
    g_impls = std::make_unique<torch::Library>(torch::Library::IMPL, name, c10::DispatchKey::CUDA,
                                               __FILE__, __LINE__);
    g_impls->impl("permute_cols", &permute_cols);
    g_impls->impl("gptq_marlin_gemm", &gptq_marlin_gemm);
    g_impls->impl("gptq_marlin_repack", &gptq_marlin_repack);
    g_impls->impl("awq_marlin_repack", &awq_marlin_repack);
    g_impls->impl("gptq_marlin_gemm_all_reduce", &gptq_marlin_gemm_all_reduce);
  } catch (const std::exception&) {
    g_impls.reset();
    g_defs.reset();
    return -1;
  }
  return 0;
}

// The mixture-of-experts operator lives in its own namespace in the reference (`_moe_C`,
// csrc/moe/torch_bindings.cpp:62-73).
extern "C" int b200q_torch_register_moe(const char* ns) {
  if (g_moe_defs) return 0;
  try {
    const std::string name(ns);
    g_moe_defs = std::make_unique<torch::Library>(torch::Library::FRAGMENT, name, std::nullopt,
                                                  __FILE__, __LINE__);
    g_moe_defs->def(
        "moe_wna16_marlin_gemm(Tensor! a, Tensor? c_or_none,"
        "Tensor! b_q_weight, Tensor? b_bias_or_none,"
        "Tensor! b_scales, Tensor? global_scale, Tensor? "
        "b_zeros_or_none,"
        "Tensor? g_idx_or_none, Tensor? perm_or_none, Tensor! workspace,"
        "Tensor sorted_token_ids,"
        "Tensor! expert_ids, Tensor! num_tokens_past_padded,"
        "Tensor! topk_weights, int moe_block_size, int top_k, "
        "bool mul_topk_weights, bool is_ep, int b_q_type_id,"
        "int size_m, int size_n, int size_k,"
        "bool is_full_k, bool use_atomic_add,"
        "bool use_fp32_reduce, bool is_zp_float) -> Tensor");
    g_moe_impls = std::make_unique<torch::Library>(torch::Library::IMPL, name,
                                                   c10::DispatchKey::CUDA, __FILE__, __LINE__);
    g_moe_impls->impl("moe_wna16_marlin_gemm", &moe_wna16_marlin_gemm);
  } catch (const std::exception&) {
    g_moe_impls.reset();
    g_moe_defs.reset();
    return -1;
  }
  return 0;
}
