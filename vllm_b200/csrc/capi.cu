// extern "C" surface of libb200q: argument validation (mirroring the checks of
// the reference op, csrc/quantization/gptq_marlin/gptq_marlin.cu:688-902), kernel
// selection and scratch accounting.  No torch types cross this boundary.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "gemm_params.cuh"

namespace b200q {

namespace {
thread_local char g_error[512] = "";
int g_sm_count[64];
int g_smem_optin[64];
}  // namespace

static std::atomic<unsigned long long> g_launches{0};
void note_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

static void query_device(int dev) {
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess)
    g_sm_count[dev & 63] = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess)
    g_smem_optin[dev & 63] = v;
}

// The one debugging variable of the library: B200Q_DEBUG is a comma-separated list of
//   no_pdl       launch without programmatic dependent launch
//   no_tc        route every M through the decode kernels
//   no_fused_ar  always run the stand-alone all-reduce kernel after the GEMM
// read once per process.
bool debug_flag(const char* name) {
  static const char* env = [] {
    const char* e = getenv("B200Q_DEBUG");
    return e ? e : "";
  }();
  const size_t n = strlen(name);
  for (const char* p = env; (p = strstr(p, name)) != nullptr; p += n) {
    const bool starts = p == env || p[-1] == ',';
    const bool ends = p[n] == '\0' || p[n] == ',';
    if (starts && ends) return true;
  }
  return false;
}

bool pdl_enabled() {
  static const bool on = !debug_flag("no_pdl");
  return on;
}

int device_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (g_sm_count[dev & 63] == 0) query_device(dev);
  return g_sm_count[dev & 63];
}

int device_max_smem_optin() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (g_smem_optin[dev & 63] == 0) query_device(dev);
  return g_smem_optin[dev & 63];
}

template <typename T, int BITS>
int dispatch_stream(const StreamParams& p, bool has_zp, int gm, int mb, int ntw, int max_ctas,
                    cudaStream_t stream);

bool tc_gemm_supported(int64_t size_m, int64_t size_n, int64_t size_k, int gm);
int launch_tc_gemm(const void* a, int64_t lda, const uint32_t* b, const void* scales,
                   const uint32_t* zeros, const void* bias, void* c, int a_dtype, int bits,
                   int64_t size_m, int64_t size_n, int64_t size_k, int group_blocks,
                   int channelwise, void* scratch, int64_t scratch_bytes, cudaStream_t stream);
int64_t tc_gemm_scratch_bytes(int64_t size_m, int64_t size_n, int64_t size_k);
int tc_error_flag(bool reset);
int ar_error_flag(bool reset);


int launch_permute_cols(const void* a, int64_t lda, const int32_t* perm, void* out, int64_t size_m,
                        int64_t size_k, cudaStream_t stream);

namespace {

constexpr int kMaxRowsPerLaunch = 64;
// upper bound of CTAs any streaming variant launches (2 per SM, <= 256 SMs)
constexpr int64_t kMaxGrid = 512;

bool tc_path_enabled() {
  static const bool on = !debug_flag("no_tc");
  return on;
}

inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// partial-sum scratch: (grid + slices) slots of (rows x slice width) floats
int64_t partial_bytes(int64_t size_n) {
  // a slot holds at most 4096 floats (rows x slice width: 32 x 128 or 64 x 64);
  // slots are indexed cta + slice < grid + slices <= kMaxGrid + N/64
  const int64_t nt = size_n / 64;
  return (kMaxGrid + nt) * 64 * 64 * 4;
}

// first region of the scratch: decode partial sums or the tensor-core kernel's k-split partials
int64_t work_bytes(int64_t size_m, int64_t size_n, int64_t size_k) {
  const int64_t tc = tc_path_enabled() ? tc_gemm_scratch_bytes(size_m, size_n, size_k) : 0;
  const int64_t dec = partial_bytes(size_n);
  return align_up(tc > dec ? tc : dec, 256);
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" const char* b200q_last_error(void) { return g_error; }
extern "C" int b200q_version(void) { return 100; }
extern "C" unsigned long long b200q_kernel_launches(void) { return g_launches.load(); }
extern "C" int b200q_sm_count(void) { return device_sm_count(); }
extern "C" int b200q_device_error(int reset) {
  const int tc = tc_error_flag(reset != 0);
  const int ar = ar_error_flag(reset != 0);
  return tc != 0 ? tc : (ar != 0 ? (0x10000 | ar) : 0);
}

extern "C" size_t b200q_marlin_gemm_scratch_bytes(int64_t size_m, int64_t size_n, int64_t size_k,
                                                  int has_act_order) {
  if (size_m <= 0 || size_n <= 0 || size_k <= 0) return 256;
  int64_t bytes = align_up(partial_bytes(size_n), 256);
  if (has_act_order) bytes += align_up(size_m * size_k * 2, 256);
  return (size_t)bytes;
}

extern "C" size_t b200q_marlin_gemm_preferred_scratch_bytes(int64_t size_m, int64_t size_n,
                                                            int64_t size_k, int has_act_order) {
  if (size_m <= 0 || size_n <= 0 || size_k <= 0) return 256;
  int64_t bytes = work_bytes(size_m, size_n, size_k);
  if (has_act_order) bytes += align_up(size_m * size_k * 2, 256);
  return (size_t)bytes;
}

namespace b200q {
int launch_all_reduce(const ArLink& link, const void* in, void* out, int64_t n_elems, int dtype,
                      cudaStream_t stream);
int check_link(void* const* peer_bufs, uint32_t* state, int rank, int world,
               int64_t max_message_bytes, ArLink* link);
}  // namespace b200q

static bool fused_ar_enabled() {
  static const bool on = !debug_flag("no_fused_ar");
  return on;
}

// The GEMM behind both entry points.  With `link` the output is all-reduced over the
// peer link: inside the GEMM kernel where one decode launch covers the problem,
// otherwise by the stand-alone kernel on the finished output.
static int gemm_impl(const void* a, int64_t lda, const uint32_t* b_q_weight, const void* b_scales,
                     const uint32_t* b_zeros, const int32_t* g_idx, const int32_t* perm,
                     const void* b_bias, void* c, void* scratch, size_t scratch_bytes,
                     int32_t* workspace, int64_t workspace_len, int64_t b_q_type_id, int a_dtype,
                     int64_t size_m, int64_t size_n, int64_t size_k, int64_t num_groups,
                     unsigned flags, cudaStream_t stream, const ArLink* link,
                     const void* global_scale = nullptr, int fp4_scales = 0) {
  // ---- type contract ---------------------------------------------------------------
  int bits = 0;
  bool type_has_zp = false;
  bool w_fp8 = false;
  bool w_fp4 = false;
  if (b_q_type_id == kTypeU4B8) { bits = 4; }
  else if (b_q_type_id == kTypeU8B128) { bits = 8; }
  else if (b_q_type_id == kTypeU4) { bits = 4; type_has_zp = true; }
  else if (b_q_type_id == kTypeU8) { bits = 8; type_has_zp = true; }
  else if (b_q_type_id == kTypeFE4M3fn) { bits = 8; w_fp8 = true; }
  else if (b_q_type_id == kTypeFE2M1f) { bits = 4; w_fp4 = true; }
  else {
    set_error("b_q_type id %lld is not supported (uint4b8, uint8b128, uint4, uint8, float8_e4m3fn, "
              "float4_e2m1f)", (long long)b_q_type_id);
    return B200Q_EUNSUPPORTED;
  }
  const bool has_zp = b_zeros != nullptr;
  B200Q_REQUIRE(!has_zp || type_has_zp, B200Q_EINVAL,
                "b_q_type must be u4 or u8 when has_zp = True");
  B200Q_REQUIRE(has_zp || !type_has_zp, B200Q_EINVAL,
                "b_q_type must be uint4b8, uint8b128 or float8_e4m3fn when has_zp = False");
  const bool zp_float = has_zp && (flags & B200Q_FLAG_ZP_FLOAT);
  B200Q_REQUIRE(!zp_float || a_dtype == B200Q_F16, B200Q_EINVAL,
                "Computation type must be float16 (half) when using float zero points.");
  B200Q_REQUIRE(a_dtype == B200Q_F16 || a_dtype == B200Q_BF16, B200Q_EINVAL,
                "gpt_marlin_gemm only supports bfloat16 and float16");
  // ---- shapes ------------------------------------------------------------------------
  B200Q_REQUIRE(size_m >= 0 && size_n >= 0 && size_k >= 0, B200Q_EINVAL, "negative size");
  B200Q_REQUIRE(size_k % 16 == 0, B200Q_EINVAL, "size_k = %lld is not divisible by tile_size = 16",
                (long long)size_k);
  B200Q_REQUIRE(size_n % 64 == 0, B200Q_EINVAL,
                "size_n = %lld, is not divisible by min_thread_n = 64", (long long)size_n);
  if (size_m == 0) return B200Q_OK;
  B200Q_REQUIRE(size_n > 0 && size_k > 0, B200Q_EINVAL, "Invalid MNK = [%lld, %lld, %lld]",
                (long long)size_m, (long long)size_n, (long long)size_k);
  B200Q_REQUIRE(size_n < (1ll << 31) && size_k < (1ll << 31) && size_m < (1ll << 31), B200Q_EINVAL,
                "size too large");
  B200Q_REQUIRE(a && b_q_weight && b_scales && c && workspace, B200Q_EINVAL,
                "null tensor pointer");
  B200Q_REQUIRE(lda >= size_k && lda % 8 == 0, B200Q_EINVAL, "A.stride(0) must divisible by 8");
  B200Q_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0, B200Q_EINVAL,
                "A must aligned to 16 bytes");
  B200Q_REQUIRE((reinterpret_cast<uintptr_t>(c) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(b_q_weight) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(b_scales) & 15) == 0 &&
                    (!b_zeros || (reinterpret_cast<uintptr_t>(b_zeros) & 15) == 0),
                B200Q_EINVAL, "tensors must be aligned to 16 bytes");
  B200Q_REQUIRE(num_groups >= 1, B200Q_EINVAL, "b_scales dim 0 = %lld is not valid",
                (long long)num_groups);
  B200Q_REQUIRE((g_idx == nullptr) == (perm == nullptr), B200Q_EINVAL,
                "g_idx and perm must be given together");
  const bool has_act_order = g_idx != nullptr;
  const bool is_k_full = flags & B200Q_FLAG_K_FULL;
  B200Q_REQUIRE(workspace_len >= 1, B200Q_ESCRATCH, "workspace.numel = %lld is below 1",
                (long long)workspace_len);

  // ---- group handling (gptq_marlin.cu:765-819) -----------------------------------------
  int gm;
  int group_blocks;
  const int kt_total = (int)(size_k / 16);
  if (has_act_order) {
    B200Q_REQUIRE(!has_zp, B200Q_EUNSUPPORTED, "act_order with zero-points is not supported");
    if (is_k_full) {
      B200Q_REQUIRE(num_groups > 1, B200Q_EINVAL, "For act_order, num_groups must be > 1");
      B200Q_REQUIRE(size_k % num_groups == 0, B200Q_EINVAL,
                    "size_k = %lld, is not divisible by num_groups = %lld", (long long)size_k,
                    (long long)num_groups);
      gm = kGrouped;
    } else {
      gm = kLookup;
    }
  } else if (num_groups > 1) {
    B200Q_REQUIRE(size_k % num_groups == 0, B200Q_EINVAL,
                  "size_k = %lld, is not divisible by b_scales.size(0) = %lld", (long long)size_k,
                  (long long)num_groups);
    gm = kGrouped;
  } else {
    gm = kChannel;
  }
  if (gm == kGrouped) {
    const int64_t group_size = size_k / num_groups;
    B200Q_REQUIRE(group_size % 16 == 0, B200Q_EUNSUPPORTED,
                  "group_size = %lld is not a multiple of 16", (long long)group_size);
    group_blocks = (int)(group_size / 16);
  } else {
    group_blocks = kt_total;  // single group: zero-points (if any) load once
  }

  // ---- scratch -----------------------------------------------------------------------
  // the k-split of the tensor-core kernel is optional: it shrinks to what the scratch holds
  const int64_t a_tmp_bytes = has_act_order ? align_up(size_m * size_k * 2, 256) : 0;
  const size_t need = b200q_marlin_gemm_scratch_bytes(size_m, size_n, size_k, has_act_order);
  B200Q_REQUIRE(scratch && scratch_bytes >= need, B200Q_ESCRATCH,
                "scratch of %zu bytes is below the required %zu", scratch_bytes, need);
  B200Q_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255) == 0, B200Q_EINVAL,
                "scratch must be aligned to 256 bytes");
  float* partials = static_cast<float*>(scratch);
  const void* a_used = a;
  int64_t lda_used = lda;
  if (has_act_order) {
    // gather the activation columns into sorted-row order once
    // (gptq_marlin.cu:549-564); the GEMM then reads a contiguous matrix
    void* a_tmp = static_cast<char*>(scratch) + (scratch_bytes - a_tmp_bytes) / 256 * 256;
    int rc = launch_permute_cols(a, lda, perm, a_tmp, size_m, size_k, stream);
    if (rc != B200Q_OK) return rc;
    a_used = a_tmp;
    lda_used = size_k;
  }

  if (zp_float)
    B200Q_REQUIRE(gm == kGrouped && !has_act_order, B200Q_EUNSUPPORTED,
                  "float zero-points need grouped scales without act_order");
  if (w_fp8)
    B200Q_REQUIRE(!has_act_order, B200Q_EUNSUPPORTED, "float8_e4m3fn weights with act_order");
  if (w_fp4) {
    // gptq_marlin.cu:818-829, 907-917: fp8-e4m3 scales per 16 values + a global scale (NVFP4),
    // or e8m0 scales per 32 values (MXFP4)
    B200Q_REQUIRE(fp4_scales == 1 || fp4_scales == 2, B200Q_EINVAL,
                  "float4_e2m1f weights come through b200q_marlin_gemm_fp4 (8-bit scales)");
    B200Q_REQUIRE(!has_act_order && gm == kGrouped, B200Q_EUNSUPPORTED,
                  "float4_e2m1f weights need grouped scales without act_order");
    const int64_t group_size = size_k / num_groups;
    B200Q_REQUIRE(group_size == (fp4_scales == 1 ? 16 : 32), B200Q_EINVAL,
                  "float4_e2m1f only supports group_size == 16 (NVFP4) and group_size == 32 (MXFP4)");
    B200Q_REQUIRE(num_groups % 2 == 0, B200Q_EUNSUPPORTED,
                  "float4_e2m1f scales are laid out in pairs of groups: num_groups = %lld is odd",
                  (long long)num_groups);
    B200Q_REQUIRE((fp4_scales == 1) == (global_scale != nullptr), B200Q_EINVAL,
                  fp4_scales == 1 ? "the global_scale parameter must be passed for nvfp4 format."
                                  : "global_scale can only be used for nvfp4 format.");
    B200Q_REQUIRE(fp4_scales == 1 || a_dtype == B200Q_BF16, B200Q_EUNSUPPORTED,
                  "e8m0 scales (MXFP4) need bfloat16 activations");
  } else {
    B200Q_REQUIRE(global_scale == nullptr && fp4_scales == 0, B200Q_EINVAL,
                  "global_scale can only be used for nvfp4 format.");
  }
  // these run the reference-order kernel at every row count
  const bool general_only = zp_float || w_fp8 || w_fp4;
  // ---- prefill regime: tensor-core kernel ----------------------------------------------
  if (!general_only && tc_path_enabled() && group_blocks >= 2 && tc_gemm_supported(size_m, size_n, size_k, gm)) {
    int rc = launch_tc_gemm(a_used, lda_used, b_q_weight, b_scales, b_zeros, b_bias, c, a_dtype,
                            bits, size_m, size_n, size_k, group_blocks, gm == kChannel, scratch,
                            (int64_t)((scratch_bytes - a_tmp_bytes) / 256 * 256), stream);
    if (rc != B200Q_OK || !link) return rc;
    return launch_all_reduce(*link, c, c, size_m * size_n, a_dtype, stream);
  }
  // one decode launch of the streaming kernel covers the problem: it all-reduces itself
  const bool fuse_ar = link && size_m <= 32 && gm != kLookup && !general_only && fused_ar_enabled();

  // ---- decode regime: chunks of up to 64 rows --------------------------------------------
  const int nt = (int)(size_n / 64);
  int64_t max_ctas = workspace_len < kMaxGrid ? workspace_len : kMaxGrid;
  for (int64_t m0 = 0; m0 < size_m; m0 += kMaxRowsPerLaunch) {
    const int rows = (int)((size_m - m0) < kMaxRowsPerLaunch ? (size_m - m0) : kMaxRowsPerLaunch);
    // 8-row blocks of A handled per launch: 1, 2, 4 or 8
    int mb = rows <= 8 ? 1 : rows <= 16 ? 2 : rows <= 32 ? 4 : 8;
    // slice width in 64-column tiles: two where the accumulators fit in registers
    int ntw = 1;
    if (nt % 2 == 0 && !general_only) {
      if (gm == kChannel && mb <= 4) ntw = 2;
      if (gm == kGrouped && mb <= 2) ntw = 2;
    }
    StreamParams p = {};
    p.a = static_cast<const char*>(a_used) + (size_t)m0 * lda_used * 2;
    p.lda = lda_used;
    p.b = b_q_weight;
    p.scales = b_scales;
    p.zeros = b_zeros;
    p.g_idx = g_idx;
    p.bias = b_bias;
    p.c = static_cast<char*>(c) + (size_t)m0 * size_n * 2;
    p.partials = partials;
    p.counters = workspace;
    p.m = rows;
    p.n = (int)size_n;
    p.k = (int)size_k;
    p.kt_total = kt_total;
    p.slices = nt / ntw;
    p.group_blocks = group_blocks;
    p.num_groups = (int)num_groups;
    p.zp_float = zp_float ? 1 : 0;
    p.w_fp8 = w_fp8 ? 1 : 0;
    p.w_fp4 = w_fp4 ? fp4_scales : 0;
    p.global_scale = global_scale;
    p.ar = ArLink{};
    if (fuse_ar) p.ar = *link;
    int rc;
    if (a_dtype == B200Q_F16) {
      rc = bits == 4 ? dispatch_stream<half, 4>(p, has_zp, gm, mb, ntw, (int)max_ctas, stream)
                     : dispatch_stream<half, 8>(p, has_zp, gm, mb, ntw, (int)max_ctas, stream);
    } else {
      rc = bits == 4
               ? dispatch_stream<__nv_bfloat16, 4>(p, has_zp, gm, mb, ntw, (int)max_ctas, stream)
               : dispatch_stream<__nv_bfloat16, 8>(p, has_zp, gm, mb, ntw, (int)max_ctas, stream);
    }
    if (rc == B200Q_EUNSUPPORTED && g_error[0] == 0)
      set_error("Unsupported shapes: MNK = [%lld, %lld, %lld]", (long long)size_m,
                (long long)size_n, (long long)size_k);
    if (rc != B200Q_OK) return rc;
  }
  if (link && !fuse_ar) return launch_all_reduce(*link, c, c, size_m * size_n, a_dtype, stream);
  return B200Q_OK;
}

extern "C" int b200q_marlin_gemm(const void* a, int64_t lda, const uint32_t* b_q_weight,
                                 const void* b_scales, const uint32_t* b_zeros,
                                 const int32_t* g_idx, const int32_t* perm, const void* b_bias,
                                 void* c, void* scratch, size_t scratch_bytes, int32_t* workspace,
                                 int64_t workspace_len, int64_t b_q_type_id, int a_dtype,
                                 int64_t size_m, int64_t size_n, int64_t size_k,
                                 int64_t num_groups, unsigned flags, b200q_stream_t stream) {
  return gemm_impl(a, lda, b_q_weight, b_scales, b_zeros, g_idx, perm, b_bias, c, scratch,
                   scratch_bytes, workspace, workspace_len, b_q_type_id, a_dtype, size_m, size_n,
                   size_k, num_groups, flags, static_cast<cudaStream_t>(stream), nullptr);
}

// Mixture-of-experts GEMM: see include/b200q.h
extern "C" int b200q_moe_wna16_marlin_gemm(
    const void* a, int64_t lda, const uint32_t* b_q_weight, const void* b_scales,
    const uint32_t* b_zeros, const void* b_bias, void* c, const int32_t* sorted_token_ids,
    const int32_t* expert_ids, const int32_t* num_tokens_past_padded, const float* topk_weights,
    int64_t sorted_len, int64_t moe_block_size, int64_t top_k, int mul_topk_weights,
    int64_t num_experts, int64_t b_q_type_id, int a_dtype, int64_t size_m, int64_t size_n,
    int64_t size_k, int64_t num_groups, b200q_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int bits = 0;
  bool type_has_zp = false;
  if (b_q_type_id == kTypeU4B8) { bits = 4; }
  else if (b_q_type_id == kTypeU8B128) { bits = 8; }
  else if (b_q_type_id == kTypeU4) { bits = 4; type_has_zp = true; }
  else if (b_q_type_id == kTypeU8) { bits = 8; type_has_zp = true; }
  else {
    set_error("moe: b_q_type id %lld is not supported (uint4b8, uint8b128, uint4, uint8)",
              (long long)b_q_type_id);
    return B200Q_EUNSUPPORTED;
  }
  const bool has_zp = b_zeros != nullptr;
  B200Q_REQUIRE(has_zp == type_has_zp, B200Q_EINVAL,
                "b_q_type must be u4 or u8 with zero-points, uint4b8 or uint8b128 without");
  B200Q_REQUIRE(a_dtype == B200Q_F16 || a_dtype == B200Q_BF16, B200Q_EINVAL,
                "moe_wna16_marlin_gemm only supports bfloat16 and float16");
  // ops.cu:709-713
  B200Q_REQUIRE(moe_block_size == 8 || (moe_block_size % 16 == 0 && moe_block_size >= 16 &&
                                        moe_block_size <= 64),
                B200Q_EINVAL, "unsupported moe_block_size=%lld", (long long)moe_block_size);
  B200Q_REQUIRE(size_k % 16 == 0 && size_n % 64 == 0 && size_n > 0 && size_k > 0, B200Q_EINVAL,
                "Invalid MNK = [%lld, %lld, %lld]", (long long)size_m, (long long)size_n, (long long)size_k);
  B200Q_REQUIRE(top_k >= 1 && num_experts >= 1 && num_groups >= 1 && size_m >= 0, B200Q_EINVAL,
                "invalid top_k / num_experts / num_groups");
  if (size_m == 0 || sorted_len == 0) return B200Q_OK;
  B200Q_REQUIRE(a && b_q_weight && b_scales && c && sorted_token_ids && expert_ids &&
                    num_tokens_past_padded, B200Q_EINVAL, "null tensor pointer");
  B200Q_REQUIRE(!mul_topk_weights || topk_weights, B200Q_EINVAL, "mul_topk_weights without topk_weights");
  B200Q_REQUIRE(lda >= size_k && lda % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0,
                B200Q_EINVAL, "A must be aligned to 16 bytes with a row stride divisible by 8");
  B200Q_REQUIRE(size_k % num_groups == 0, B200Q_EINVAL, "size_k = %lld, is not divisible by num_groups = %lld",
                (long long)size_k, (long long)num_groups);
  const int kt_total = (int)(size_k / 16);
  int gm = kChannel, group_blocks = kt_total;
  if (num_groups > 1) {
    const int64_t group_size = size_k / num_groups;
    B200Q_REQUIRE(group_size % 16 == 0, B200Q_EUNSUPPORTED, "group_size = %lld is not a multiple of 16",
                  (long long)group_size);
    gm = kGrouped;
    group_blocks = (int)(group_size / 16);
  }
  StreamParams p = {};
  p.a = a; p.lda = lda; p.b = b_q_weight; p.scales = b_scales; p.zeros = b_zeros; p.bias = b_bias;
  p.c = c;
  p.m = (int)moe_block_size; p.n = (int)size_n; p.k = (int)size_k;
  p.kt_total = kt_total;
  p.slices = (int)(size_n / 64);
  p.group_blocks = group_blocks;
  p.num_groups = (int)num_groups;
  p.moe_sorted_ids = sorted_token_ids;
  p.moe_expert_ids = expert_ids;
  p.moe_num_padded = num_tokens_past_padded;
  p.moe_topk_weights = mul_topk_weights ? topk_weights : nullptr;
  p.moe_blocks = (int)(sorted_len / moe_block_size);
  p.moe_rows = (int)(size_m * top_k);
  p.moe_top_k = (int)top_k;
  p.moe_b_stride = (long long)kt_total * size_n * 16 * bits / 32;      // words per expert
  p.moe_s_stride = (long long)num_groups * size_n;
  p.moe_z_stride = (long long)num_groups * size_n * bits / 32;
  p.moe_bias_stride = size_n;
  if (p.moe_blocks == 0) return B200Q_OK;
  const int mb8 = (int)(moe_block_size / 8);  // 8-row blocks: 2, 4, 6, 8
  int rc;
  if (a_dtype == B200Q_F16)
    rc = bits == 4 ? dispatch_stream<half, 4>(p, has_zp, gm, mb8, 1, 1 << 20, stream)
                   : dispatch_stream<half, 8>(p, has_zp, gm, mb8, 1, 1 << 20, stream);
  else
    rc = bits == 4 ? dispatch_stream<__nv_bfloat16, 4>(p, has_zp, gm, mb8, 1, 1 << 20, stream)
                   : dispatch_stream<__nv_bfloat16, 8>(p, has_zp, gm, mb8, 1, 1 << 20, stream);
  if (rc == B200Q_EUNSUPPORTED && g_error[0] == 0) set_error("moe: unsupported configuration");
  return rc;
}

extern "C" int b200q_marlin_gemm_fp4(const void* a, int64_t lda, const uint32_t* b_q_weight,
                                     const void* b_scales, const void* global_scale, int scale_kind,
                                     const void* b_bias, void* c, void* scratch, size_t scratch_bytes,
                                     int32_t* workspace, int64_t workspace_len, int a_dtype,
                                     int64_t size_m, int64_t size_n, int64_t size_k,
                                     int64_t num_groups, b200q_stream_t stream) {
  B200Q_REQUIRE(scale_kind == B200Q_FP4_SCALES_E4M3 || scale_kind == B200Q_FP4_SCALES_E8M0,
                B200Q_EINVAL, "scale_kind must be B200Q_FP4_SCALES_E4M3 or B200Q_FP4_SCALES_E8M0");
  return gemm_impl(a, lda, b_q_weight, b_scales, nullptr, nullptr, nullptr, b_bias, c, scratch,
                   scratch_bytes, workspace, workspace_len, kTypeFE2M1f, a_dtype, size_m, size_n,
                   size_k, num_groups, B200Q_FLAG_K_FULL, static_cast<cudaStream_t>(stream), nullptr,
                   global_scale, scale_kind);
}

extern "C" int b200q_marlin_gemm_all_reduce(
    const void* a, int64_t lda, const uint32_t* b_q_weight, const void* b_scales,
    const uint32_t* b_zeros, const int32_t* g_idx, const int32_t* perm, const void* b_bias, void* c,
    void* scratch, size_t scratch_bytes, int32_t* workspace, int64_t workspace_len,
    int64_t b_q_type_id, int a_dtype, int64_t size_m, int64_t size_n, int64_t size_k,
    int64_t num_groups, unsigned flags, void* const* peer_bufs, uint32_t* state, int rank, int world, int64_t max_message_bytes, b200q_stream_t stream) {
  ArLink link;
  int rc = check_link(peer_bufs, state, rank, world, max_message_bytes, &link);
  if (rc != B200Q_OK) return rc;
  B200Q_REQUIRE(size_m >= 0 && size_n >= 0 && size_m * size_n * 2 <= max_message_bytes,
                B200Q_EINVAL, "output of %lld x %lld exceeds the slot size %lld",
                (long long)size_m, (long long)size_n, (long long)max_message_bytes);
  return gemm_impl(a, lda, b_q_weight, b_scales, b_zeros, g_idx, perm, b_bias, c, scratch,
                   scratch_bytes, workspace, workspace_len, b_q_type_id, a_dtype, size_m, size_n,
                   size_k, num_groups, flags, static_cast<cudaStream_t>(stream), &link);
}
