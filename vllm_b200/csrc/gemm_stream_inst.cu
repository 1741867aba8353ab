// Instantiations of the streaming GEMM for one (element type, weight bits)
// pair, selected at compile time with -DINST_BF16={0,1} -DINST_BITS={4,8} so
// that the four translation units build in parallel.
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

namespace {

template <bool HAS_ZP, int GM>
int by_shape(const StreamParams& p, int mb, int ntw, int max_ctas, cudaStream_t stream) {
  using T = InstT;
  constexpr int B = INST_BITS;
  if constexpr (GM == kLookup) {  // slow path: one tile width only
    if (ntw != 1) return B200Q_EUNSUPPORTED;
    switch (mb) {
      case 1: return launch_stream<T, B, HAS_ZP, GM, 1, 1>(p, max_ctas, stream);
      case 2: return launch_stream<T, B, HAS_ZP, GM, 2, 1>(p, max_ctas, stream);
      case 4: return launch_stream<T, B, HAS_ZP, GM, 4, 1>(p, max_ctas, stream);
    }
    return B200Q_EUNSUPPORTED;
  } else {
    switch (mb * 10 + ntw) {
      case 11: return launch_stream<T, B, HAS_ZP, GM, 1, 1>(p, max_ctas, stream);
      case 12: return launch_stream<T, B, HAS_ZP, GM, 1, 2>(p, max_ctas, stream);
      case 21: return launch_stream<T, B, HAS_ZP, GM, 2, 1>(p, max_ctas, stream);
      case 22: return launch_stream<T, B, HAS_ZP, GM, 2, 2>(p, max_ctas, stream);
      case 41: return launch_stream<T, B, HAS_ZP, GM, 4, 1>(p, max_ctas, stream);
    }
    return B200Q_EUNSUPPORTED;
  }
}

}  // namespace

template <>
int dispatch_stream<InstT, INST_BITS>(const StreamParams& p, bool has_zp, int gm, int mb, int ntw,
                                      int max_ctas, cudaStream_t stream) {
  if (has_zp) {
    if (gm == kChannel) return by_shape<true, kChannel>(p, mb, ntw, max_ctas, stream);
    if (gm == kGrouped) return by_shape<true, kGrouped>(p, mb, ntw, max_ctas, stream);
    return B200Q_EUNSUPPORTED;
  }
  if (gm == kChannel) return by_shape<false, kChannel>(p, mb, ntw, max_ctas, stream);
  if (gm == kGrouped) return by_shape<false, kGrouped>(p, mb, ntw, max_ctas, stream);
  return by_shape<false, kLookup>(p, mb, ntw, max_ctas, stream);
}

}  // namespace b200q
