// Shared device/host helpers for the b200q kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/b200q.h"

namespace b200q {

// ---- host-side error reporting ---------------------------------------------
void set_error(const char* fmt, ...);

#define B200Q_REQUIRE(cond, code, ...)  \
  do {                                  \
    if (!(cond)) {                      \
      ::b200q::set_error(__VA_ARGS__);  \
      return (code);                    \
    }                                   \
  } while (0)

#define B200Q_CUDA_OK(expr)                                                      \
  do {                                                                           \
    cudaError_t e__ = (expr);                                                    \
    if (e__ != cudaSuccess) {                                                    \
      ::b200q::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));       \
      return B200Q_ECUDA;                                                        \
    }                                                                            \
  } while (0)

// ScalarType ids (exponent | mantissa<<8 | signed<<16 | bias<<17 | ...).
constexpr int64_t kTypeU4B8 = 4ll << 8 | 8ll << 17 | 1ll << 50;
constexpr int64_t kTypeU4 = 4ll << 8 | 1ll << 50;
constexpr int64_t kTypeU8B128 = 8ll << 8 | 128ll << 17 | 1ll << 50;
constexpr int64_t kTypeFE4M3fn = 2814749767172868ll;  // float8_e4m3fn (csrc/core/scalar_type.hpp)
constexpr int64_t kTypeFE2M1f = 562949953487106ll;    // float4_e2m1f
constexpr int64_t kTypeU8 = 8ll << 8 | 1ll << 50;

// bump the process-wide launch counter (b200q_kernel_launches)
void note_launch(int n = 1);

// true when the comma-separated debugging variable B200Q_DEBUG names `name`
bool debug_flag(const char* name);
// false with B200Q_DEBUG=no_pdl (programmatic dependent launch off)
bool pdl_enabled();

int device_sm_count();
int device_max_smem_optin();

// ---- device helpers ----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte async copy global -> shared, L2 only; src_bytes in {0, 16}: 0 zero-fills.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes = 16) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src),
               "r"(src_bytes));
}
// The same for a full 16-byte copy, with compile-time byte offsets folded into both addresses.
template <int DOFF, int SOFF>
__device__ __forceinline__ void cp_async16_off(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0+%2], [%1+%3], 16;\n" ::"r"(dst), "l"(src), "n"(DOFF),
               "n"(SOFF));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
  return v;
}

// D(16x8,f32) += A(16x16) * B(16x8), 16-bit operands.
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4],
                                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- packed 16-bit pair arithmetic on raw uint32 ------------------------------
template <typename T>
struct Pair;
template <>
struct Pair<half> {
  static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
    half2 r = __hsub2(*reinterpret_cast<half2*>(&a), *reinterpret_cast<half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
    half2 r = __hmul2(*reinterpret_cast<half2*>(&a), *reinterpret_cast<half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
    half2 r = __hfma2(*reinterpret_cast<half2*>(&a), *reinterpret_cast<half2*>(&b),
                      *reinterpret_cast<half2*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ float to_float(uint16_t v) {
    return __half2float(__ushort_as_half(v));
  }
  static __device__ __forceinline__ uint16_t from_float(float f) {
    return __half_as_ushort(__float2half_rn(f));
  }
};
template <>
struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
    __nv_bfloat162 r =
        __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
    __nv_bfloat162 r =
        __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
    __nv_bfloat162 r =
        __hfma2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b),
                *reinterpret_cast<__nv_bfloat162*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ float to_float(uint16_t v) {
    return __uint_as_float(static_cast<uint32_t>(v) << 16);
  }
  static __device__ __forceinline__ uint16_t from_float(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
  }
};

// Duplicate the low / high 16 bits of x into both halves.
__device__ __forceinline__ uint32_t dup_lo(uint32_t x) { return __byte_perm(x, x, 0x1010); }
__device__ __forceinline__ uint32_t dup_hi(uint32_t x) { return __byte_perm(x, x, 0x3232); }

// ---- integer code -> 16-bit float pairs (exact) --------------------------------
// One 32-bit word of the Marlin layout expands to pairs (k, k+1) for the two
// 8-column blocks of a 16-column sub-tile:
//   4-bit: out[0] = rows {2q,2q+1} block 0, out[1] = rows {2q+8,2q+9} block 0,
//          out[2], out[3] the same for block 1.
//   8-bit: out[0] = rows {2q,2q+1}, out[1] = rows {2q+8,2q+9} of ONE block.
// BIASED selects the built-in offset (8 / 128); otherwise the raw code value is
// produced (zero-point types, and the zero-points themselves).
// Integers up to 2^11 (fp16) / 2^8 (bf16) are exact in the target type, so the
// "or into the mantissa of 1024.0 / 128.0, then subtract" conversion is exact.
// (a & mask) | ex as ONE logic instruction.  Written with two immediates the compiler emits
// two; constants that come out of an opaque move stay in registers and the three-input form
// takes all of them.
template <uint32_t V>
__device__ __forceinline__ uint32_t reg_const() {
  uint32_t r;
  asm("mov.u32 %0, %1;\n" : "=r"(r) : "n"(V));
  return r;
}
__device__ __forceinline__ uint32_t mask_or(uint32_t a, uint32_t mask, uint32_t ex) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(d) : "r"(a), "r"(mask), "r"(ex));
  return d;
}

template <typename T, bool BIASED>
__device__ __forceinline__ void dequant4(uint32_t q, uint32_t (&out)[4]);

template <>
__device__ __forceinline__ void dequant4<half, true>(uint32_t q, uint32_t (&out)[4]) {
  const uint32_t EX = 0x64006400u;   // 1024.0
  const uint32_t SUB = 0x64086408u;  // 1032.0
  const uint32_t MUL = 0x2c002c00u;  // 1/16
  const uint32_t ADD = 0xd480d480u;  // -72.0
  const uint32_t ex = reg_const<EX>(), lo = reg_const<0x000f000fu>(), hi = reg_const<0x00f000f0u>();
  out[0] = Pair<half>::sub(mask_or(q, lo, ex), SUB);
  out[1] = Pair<half>::fma(mask_or(q, hi, ex), MUL, ADD);
  q >>= 8;
  out[2] = Pair<half>::sub(mask_or(q, lo, ex), SUB);
  out[3] = Pair<half>::fma(mask_or(q, hi, ex), MUL, ADD);
}
template <>
__device__ __forceinline__ void dequant4<half, false>(uint32_t q, uint32_t (&out)[4]) {
  const uint32_t EX = 0x64006400u;
  const uint32_t MUL = 0x2c002c00u;
  const uint32_t ADD = 0xd400d400u;  // -64.0
  const uint32_t ex = reg_const<EX>(), lo = reg_const<0x000f000fu>(), hi = reg_const<0x00f000f0u>();
  out[0] = Pair<half>::sub(mask_or(q, lo, ex), EX);
  out[1] = Pair<half>::fma(mask_or(q, hi, ex), MUL, ADD);
  q >>= 8;
  out[2] = Pair<half>::sub(mask_or(q, lo, ex), EX);
  out[3] = Pair<half>::fma(mask_or(q, hi, ex), MUL, ADD);
}
template <>
__device__ __forceinline__ void dequant4<__nv_bfloat16, true>(uint32_t q, uint32_t (&out)[4]) {
  const uint32_t EX = 0x43004300u;   // 128.0
  const uint32_t SUB = 0x43084308u;  // 136.0
  const uint32_t ex = reg_const<EX>(), lo = reg_const<0x000f000fu>();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[i] = Pair<__nv_bfloat16>::sub(mask_or(q, lo, ex), SUB);
    q >>= 4;
  }
}
template <>
__device__ __forceinline__ void dequant4<__nv_bfloat16, false>(uint32_t q, uint32_t (&out)[4]) {
  const uint32_t EX = 0x43004300u;
  const uint32_t ex = reg_const<EX>(), lo = reg_const<0x000f000fu>();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[i] = Pair<__nv_bfloat16>::sub(mask_or(q, lo, ex), EX);
    q >>= 4;
  }
}

template <typename T, bool BIASED>
__device__ __forceinline__ void dequant8(uint32_t q, uint32_t (&out)[2]);

template <>
__device__ __forceinline__ void dequant8<half, true>(uint32_t q, uint32_t (&out)[2]) {
  const uint32_t SUB = 0x64806480u;  // 1152.0
  out[0] = Pair<half>::sub(__byte_perm(q, 0x64646464u, 0x4240), SUB);
  out[1] = Pair<half>::sub(__byte_perm(q, 0x64646464u, 0x4341), SUB);
}
template <>
__device__ __forceinline__ void dequant8<half, false>(uint32_t q, uint32_t (&out)[2]) {
  const uint32_t SUB = 0x64006400u;
  out[0] = Pair<half>::sub(__byte_perm(q, 0x64646464u, 0x4240), SUB);
  out[1] = Pair<half>::sub(__byte_perm(q, 0x64646464u, 0x4341), SUB);
}
template <bool BIASED>
__device__ __forceinline__ void dequant8_bf16(uint32_t q, uint32_t (&out)[2]) {
  // 8-bit codes do not fit bf16's 7 mantissa bits: go through fp32
  // (2^23 + code) and convert the exact small integer back.
  const float off = BIASED ? 8388736.0f : 8388608.0f;
  float f0 = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7440)) - off;
  float f1 = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7441)) - off;
  float f2 = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7442)) - off;
  float f3 = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7443)) - off;
  __nv_bfloat162 p0 = __floats2bfloat162_rn(f0, f2);
  __nv_bfloat162 p1 = __floats2bfloat162_rn(f1, f3);
  out[0] = *reinterpret_cast<uint32_t*>(&p0);
  out[1] = *reinterpret_cast<uint32_t*>(&p1);
}
template <>
__device__ __forceinline__ void dequant8<__nv_bfloat16, true>(uint32_t q, uint32_t (&out)[2]) {
  dequant8_bf16<true>(q, out);
}
template <>
__device__ __forceinline__ void dequant8<__nv_bfloat16, false>(uint32_t q, uint32_t (&out)[2]) {
  dequant8_bf16<false>(q, out);
}

// float8_e4m3fn codes (four per word, Marlin 8-bit layout) to 16-bit pairs: sign and the seven
// exponent / mantissa bits move into the 16-bit format's fields, which leaves the exponent
// biased by 2^(bias16 - 7); kFp8Rebias<T> (exact power of two) undoes that.  out[0] = bytes
// (0, 2), out[1] = bytes (1, 3), as dequant8.  Follows the reference's bit manipulation
// (csrc/quantization/gptq_marlin/dequant.h:320-395); all 254 finite codes convert exactly,
// subnormals included.
template <typename T>
struct Fp8Cvt;
template <>
struct Fp8Cvt<half> {
  static constexpr int kShift = 1;               // 5 - 4 exponent bits
  static constexpr uint32_t kRebias = 0x5c005c00u;  // 2^8 as a half pair
  static constexpr float kRebiasInv = 1.0f / 256.0f;
};
template <>
struct Fp8Cvt<__nv_bfloat16> {
  static constexpr int kShift = 4;               // 8 - 4 exponent bits
  static constexpr uint32_t kRebias = 0x7b807b80u;  // 2^120 as a bfloat16 pair
  static constexpr float kRebiasInv = 7.52316384526264e-37f;  // 2^-120
};
template <typename T>
__device__ __forceinline__ void dequant_fp8(uint32_t q, uint32_t (&out)[2]) {
  const uint32_t q8 = q << 8;
  out[0] = (q8 & 0x80008000u) | ((q8 & 0x7f007f00u) >> Fp8Cvt<T>::kShift);
  out[1] = (q & 0x80008000u) | ((q & 0x7f007f00u) >> Fp8Cvt<T>::kShift);
}

// Position of output column n inside the 32-column "single" permutation used
// for channel-wise scales and bias: stored position 8*i + jj of a chunk holds
// column 2*i + [0,1,8,9,16,17,24,25][jj].
__host__ __device__ __forceinline__ int single_perm_pos(int n) {
  int r = n & 31;
  return (n & ~31) + 8 * ((r & 7) >> 1) + 2 * (r >> 3) + (r & 1);
}
// Position of column n inside the 64-column grouped-scale permutation: stored
// position 8*i + j holds column i + 8*j.
__host__ __device__ __forceinline__ int grouped_perm_pos(int n) {
  int r = n & 63;
  return (n & ~63) + 8 * (r & 7) + (r >> 3);
}

}  // namespace b200q
