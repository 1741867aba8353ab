// Instantiations of the decode-regime GEMM kernels for one (element type,
// weight bits) pair, selected at compile time with -DINST_BF16={0,1}
// -DINST_BITS={4,8} so that the four translation units build in parallel.
#include "gemm_lookup.cuh"
#include "gemm_stream.cuh"

#ifndef INST_BF16
#error "compile with -DINST_BF16=0|1 -DINST_BITS=4|8"
#endif

namespace b200q {

#if INST_BF16
using InstT = __nv_bfloat16;
#else
using InstT = half;
#endif

template <typename T, int BITS>
int dispatch_stream(const StreamParams& p, bool has_zp, int gm, int mb, int ntw, int max_ctas,
                    cudaStream_t stream);

namespace {

using T = InstT;
constexpr int B = INST_BITS;

// `rows8` = 8-row blocks of A (1, 2, 4, 8); 8 blocks (64 rows) hold too many
// accumulators for the streaming kernel and run the reference-order kernel.
template <bool HAS_ZP>
int channel(const StreamParams& p, int rows8, int ntw, int max_ctas, cudaStream_t stream) {
  switch (rows8 * 10 + ntw) {
    case 11: return launch_stream<T, B, HAS_ZP, kChannel, 1, 1>(p, max_ctas, stream);
    case 12: return launch_stream<T, B, HAS_ZP, kChannel, 1, 2>(p, max_ctas, stream);
    case 21: return launch_stream<T, B, HAS_ZP, kChannel, 2, 1>(p, max_ctas, stream);
    case 22: return launch_stream<T, B, HAS_ZP, kChannel, 2, 2>(p, max_ctas, stream);
    case 41: return launch_stream<T, B, HAS_ZP, kChannel, 4, 1>(p, max_ctas, stream);
    case 42: return launch_stream<T, B, HAS_ZP, kChannel, 4, 2>(p, max_ctas, stream);
    case 81: return launch_lookup<T, B, HAS_ZP, kChannel, 4, 1>(p, max_ctas, stream);
  }
  return B200Q_EUNSUPPORTED;
}

template <bool HAS_ZP>
int grouped(const StreamParams& p, int rows8, int ntw, int max_ctas, cudaStream_t stream) {
  switch (rows8 * 10 + ntw) {
    case 11: return launch_stream<T, B, HAS_ZP, kGrouped, 1, 1>(p, max_ctas, stream);
    case 12: return launch_stream<T, B, HAS_ZP, kGrouped, 1, 2>(p, max_ctas, stream);
    case 21: return launch_stream<T, B, HAS_ZP, kGrouped, 2, 1>(p, max_ctas, stream);
    case 22: return launch_stream<T, B, HAS_ZP, kGrouped, 2, 2>(p, max_ctas, stream);
    case 41: return launch_stream<T, B, HAS_ZP, kGrouped, 4, 1>(p, max_ctas, stream);
    case 81: return launch_lookup<T, B, HAS_ZP, kGrouped, 4, 1>(p, max_ctas, stream);
  }
  return B200Q_EUNSUPPORTED;
}

// float zero-points (HQQ): the reference-order kernel for every row count
int grouped_zp_float(const StreamParams& p, int rows8, int ntw, int max_ctas, cudaStream_t stream) {
  if (ntw != 1) return B200Q_EUNSUPPORTED;
  const int mb = (rows8 + 1) / 2;  // 16-row blocks
  switch (mb) {
    case 1: return launch_lookup<T, B, true, kGrouped, 1, 1, true>(p, max_ctas, stream);
    case 2: return launch_lookup<T, B, true, kGrouped, 2, 1, true>(p, max_ctas, stream);
    case 4: return launch_lookup<T, B, true, kGrouped, 4, 1, true>(p, max_ctas, stream);
  }
  return B200Q_EUNSUPPORTED;
}

// float8_e4m3fn weights: the reference-order kernel for every row count
int fp8_weights(const StreamParams& p, int gm, int rows8, int ntw, int max_ctas, cudaStream_t stream) {
  if constexpr (B == 8) {
    if (ntw != 1) return B200Q_EUNSUPPORTED;
    const int mb = (rows8 + 1) / 2;  // 16-row blocks
    if (gm == kGrouped) {
      switch (mb) {
        case 1: return launch_lookup<T, B, false, kGrouped, 1, 1, false, true>(p, max_ctas, stream);
        case 2: return launch_lookup<T, B, false, kGrouped, 2, 1, false, true>(p, max_ctas, stream);
        case 4: return launch_lookup<T, B, false, kGrouped, 4, 1, false, true>(p, max_ctas, stream);
      }
    } else if (gm == kChannel) {
      switch (mb) {
        case 1: return launch_lookup<T, B, false, kChannel, 1, 1, false, true>(p, max_ctas, stream);
        case 2: return launch_lookup<T, B, false, kChannel, 2, 1, false, true>(p, max_ctas, stream);
        case 4: return launch_lookup<T, B, false, kChannel, 4, 1, false, true>(p, max_ctas, stream);
      }
    }
  }
  return B200Q_EUNSUPPORTED;
}

// float4_e2m1f weights (NVFP4 / MXFP4): the reference-order kernel for every row count
int fp4_weights(const StreamParams& p, int gm, int rows8, int ntw, int max_ctas, cudaStream_t stream) {
  if constexpr (B == 4) {
    if (ntw != 1 || gm != kGrouped) return B200Q_EUNSUPPORTED;
    const int mb = (rows8 + 1) / 2;  // 16-row blocks
    switch (mb) {
      case 1: return launch_lookup<T, B, false, kGrouped, 1, 1, false, false, true>(p, max_ctas, stream);
      case 2: return launch_lookup<T, B, false, kGrouped, 2, 1, false, false, true>(p, max_ctas, stream);
      case 4: return launch_lookup<T, B, false, kGrouped, 4, 1, false, false, true>(p, max_ctas, stream);
    }
  }
  return B200Q_EUNSUPPORTED;
}

// mixture-of-experts form: the reference-order kernel over (block of sorted ids, column slice)
template <bool HAS_ZP, int GM>
int moe_blocks(const StreamParams& p, int rows8, int max_ctas, cudaStream_t stream) {
  // blocks of up to 32 ids: the decode kernel; above: the reference-order kernel
  switch (rows8) {
    case 1: return launch_stream<T, B, HAS_ZP, GM, 1, 1, true>(p, max_ctas, stream);
    case 2: return launch_stream<T, B, HAS_ZP, GM, 2, 1, true>(p, max_ctas, stream);
    case 4: return launch_stream<T, B, HAS_ZP, GM, 4, 1, true>(p, max_ctas, stream);
  }
  const int mb = (rows8 + 1) / 2;  // 16-row blocks
  switch (mb) {
    case 1: return launch_lookup<T, B, HAS_ZP, GM, 1, 1, false, false, false, true>(p, max_ctas, stream);
    case 2: return launch_lookup<T, B, HAS_ZP, GM, 2, 1, false, false, false, true>(p, max_ctas, stream);
    case 3:
    case 4: return launch_lookup<T, B, HAS_ZP, GM, 4, 1, false, false, false, true>(p, max_ctas, stream);
  }
  return B200Q_EUNSUPPORTED;
}

int moe(const StreamParams& p, bool has_zp, int gm, int rows8, int ntw, int max_ctas, cudaStream_t stream) {
  if (ntw != 1 || p.zp_float) return B200Q_EUNSUPPORTED;
  if (gm == kChannel)
    return has_zp ? moe_blocks<true, kChannel>(p, rows8, max_ctas, stream)
                  : moe_blocks<false, kChannel>(p, rows8, max_ctas, stream);
  if (gm == kGrouped)
    return has_zp ? moe_blocks<true, kGrouped>(p, rows8, max_ctas, stream)
                  : moe_blocks<false, kGrouped>(p, rows8, max_ctas, stream);
  return B200Q_EUNSUPPORTED;
}

int lookup(const StreamParams& p, int rows8, int ntw, int max_ctas, cudaStream_t stream) {
  if (ntw != 1) return B200Q_EUNSUPPORTED;
  const int mb = (rows8 + 1) / 2;  // 16-row blocks
  switch (mb) {
    case 1: return launch_lookup<T, B, false, kLookup, 1, 1>(p, max_ctas, stream);
    case 2: return launch_lookup<T, B, false, kLookup, 2, 1>(p, max_ctas, stream);
    case 4: return launch_lookup<T, B, false, kLookup, 4, 1>(p, max_ctas, stream);
  }
  return B200Q_EUNSUPPORTED;
}

}  // namespace

template <>
int dispatch_stream<InstT, INST_BITS>(const StreamParams& p, bool has_zp, int gm, int mb, int ntw,
                                      int max_ctas, cudaStream_t stream) {
  if (p.moe_sorted_ids) return (p.w_fp8 || p.w_fp4) ? B200Q_EUNSUPPORTED : moe(p, has_zp, gm, mb, ntw, max_ctas, stream);
  if (p.w_fp8) return has_zp ? B200Q_EUNSUPPORTED : fp8_weights(p, gm, mb, ntw, max_ctas, stream);
  if (p.w_fp4) return has_zp ? B200Q_EUNSUPPORTED : fp4_weights(p, gm, mb, ntw, max_ctas, stream);
  if (p.zp_float)
    return (has_zp && gm == kGrouped) ? grouped_zp_float(p, mb, ntw, max_ctas, stream)
                                      : B200Q_EUNSUPPORTED;
  if (gm == kChannel)
    return has_zp ? channel<true>(p, mb, ntw, max_ctas, stream)
                  : channel<false>(p, mb, ntw, max_ctas, stream);
  if (gm == kGrouped)
    return has_zp ? grouped<true>(p, mb, ntw, max_ctas, stream)
                  : grouped<false>(p, mb, ntw, max_ctas, stream);
  if (has_zp) return B200Q_EUNSUPPORTED;
  return lookup(p, mb, ntw, max_ctas, stream);
}

}  // namespace b200q
