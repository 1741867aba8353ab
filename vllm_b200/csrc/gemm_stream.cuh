// Streaming mixed-precision GEMM for the decode regime (up to 32 rows of A per
// launch): C[M,N] = A[M,K] * dequant(B), grouped or channel-wise scales.
//
// The kernel is meant to be HBM-bound: the packed weights are read exactly once.
//
// Data movement.  One persistent CTA per SM: a producer warp and 16 consumer warps
// around a ring of shared-memory stages.  The producer's lanes issue, per stage,
//   * 1-D bulk copies (cp.async.bulk, no multicast) of runs of Marlin tiles: the
//     WN 64-column tiles of a slice are contiguous inside a k-tile row, so one
//     copy of WN * 512 B (4-bit) brings a whole k-tile of the slice;
//   * one 2-D tensor copy (cp.async.bulk.tensor, 32-byte swizzle, rows beyond M
//     zero-filled) per k-tile for the 16 activation columns that meet it;
// all completing on the stage's mbarrier.  Consumers never compute an address for
// global memory in the main loop and issue no copy instructions: they wait on the
// stage barrier, read their tile with one 128-bit shared load, expand, and feed
// mma.sync.m16n8k16 with fp32 accumulation.  A stage is handed back through a
// second mbarrier.  Group scales / zero-points are prefetched straight into
// registers one group ahead (a group is 8 k-tiles of work away).
//
// Arithmetic (unchanged from the first version of this kernel):
//  * Weights are the 16-row operand of the MMA (C^T = W^T A^T): one MMA covers
//    a 16(N) x 16(K) sub-tile of weights and 8 rows of A, and the four 16-bit
//    pairs that one 32-bit word of the Marlin layout expands to are exactly the
//    four operand registers of that MMA.
//  * No subtract, no scale multiply before the MMA.  A 4-bit code w is OR-ed
//    into the mantissa of a 16-bit constant, giving x = OFF + U*w exactly
//    (fp16: 1024 + w and 1024 + 16 w; bf16: 128 + w and 128 + 8 w, the second
//    form for codes that sit 4 bits higher in the word): one LOP3 per pair of
//    weights.  The k-rows of A that meet the U-scaled codes are pre-multiplied
//    by 1/U (exact power of two).  The MMA then yields
//    T = sum_k a_k (w_k + OFF_k/U_k).
//  * The offset term is itself a product with A, so one extra MMA per k-tile
//    against a constant weight fragment gives corr = sum_k a_k (OFF_k/U_k + bias)
//    and T - corr = sum_k a_k (w_k - bias) up to fp32 rounding.  A second
//    constant MMA gives the plain row sums needed for zero-points.
//  * Group scales are applied to the fp32 group sum (T - corr) when the group
//    ends, not to every weight: acc += s[n] * (T - corr - z[n] * rowsum).
//
// Work decomposition.  The weight matrix is cut into column slices of WN tiles;
// the (slice, k-tile) space is cut into equal contiguous stripes, one per CTA, so
// every SM streams the same number of bytes whatever the shape.  Inside a CTA
// the part of a stripe that lies in one slice (a "piece") is shared out among the
// warps: by tile (and half tile when SUBS = 2) and by k sub-range.  Warp sums meet
// in shared memory.  A piece that does not cover the whole K of its slice leaves
// fp32 partial sums in the scratch; the last CTA to arrive at the slice (counter
// in the workspace, reset on the way out) adds the partials in k order and writes
// C: no atomics on data, bitwise reproducible.
#pragma once

#include <cuda.h>

#include <cstdlib>

#include "gemm_params.cuh"

namespace b200q {

// How weight codes become MMA operands for (element type, weight bits).
// kEx / kMaskLo / kMaskHi reach the kernel through StreamParams so that they
// live in registers and every and-or is a single three-register LOP3.
template <typename T, int BITS>
struct Emb;

template <>
struct Emb<half, 4> {
  static constexpr bool kEmbed = true, kPrescale = true;
  static constexpr uint32_t kEx = 0x64006400u, kMaskLo = 0x000f000fu, kMaskHi = 0x00f000f0u;
  static constexpr int kShiftHi = 0;
  static constexpr uint32_t kAScaleHi = 0x2c002c00u;  // 1/16
  // offsets as seen by the (prescaled) A rows: lo rows 1024 + bias, hi rows 16 * (64 + bias)
  static constexpr uint32_t kOffLoBiased = 0x64086408u, kOffHiBiased = 0x64806480u;  // 1032, 1152
  static constexpr uint32_t kOffLoRaw = 0x64006400u, kOffHiRaw = 0x64006400u;        // 1024, 1024
  static constexpr uint32_t kOneLo = 0x3c003c00u, kOneHi = 0x4c004c00u;              // 1, 16
};
template <>
struct Emb<__nv_bfloat16, 4> {
  static constexpr bool kEmbed = true, kPrescale = true;
  static constexpr uint32_t kEx = 0x43004300u, kMaskLo = 0x000f000fu, kMaskHi = 0x00780078u;
  static constexpr int kShiftHi = 1;
  static constexpr uint32_t kAScaleHi = 0x3e003e00u;  // 1/8
  // lo rows 128 + bias, hi rows 8 * (16 + bias)
  static constexpr uint32_t kOffLoBiased = 0x43084308u, kOffHiBiased = 0x43404340u;  // 136, 192
  static constexpr uint32_t kOffLoRaw = 0x43004300u, kOffHiRaw = 0x43004300u;        // 128, 128
  static constexpr uint32_t kOneLo = 0x3f803f80u, kOneHi = 0x41004100u;              // 1, 8
};
template <>
struct Emb<half, 8> {
  static constexpr bool kEmbed = true, kPrescale = false;
  static constexpr uint32_t kEx = 0x64646464u, kMaskLo = 0, kMaskHi = 0;
  static constexpr int kShiftHi = 0;
  static constexpr uint32_t kAScaleHi = 0;
  static constexpr uint32_t kOffLoBiased = 0x64806480u, kOffHiBiased = 0x64806480u;  // 1152
  static constexpr uint32_t kOffLoRaw = 0x64006400u, kOffHiRaw = 0x64006400u;        // 1024
  static constexpr uint32_t kOneLo = 0x3c003c00u, kOneHi = 0x3c003c00u;
};
template <>
struct Emb<__nv_bfloat16, 8> {
  // 8-bit codes do not fit bf16's mantissa: convert exactly through fp32 instead
  static constexpr bool kEmbed = false, kPrescale = false;
  static constexpr uint32_t kEx = 0, kMaskLo = 0, kMaskHi = 0;
  static constexpr int kShiftHi = 0;
  static constexpr uint32_t kAScaleHi = 0;
  static constexpr uint32_t kOffLoBiased = 0, kOffHiBiased = 0, kOffLoRaw = 0, kOffHiRaw = 0;
  static constexpr uint32_t kOneLo = 0x3f803f80u, kOneHi = 0x3f803f80u;
};

// (a & b) | c in one instruction, all operands in registers
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// The four operand registers of the weight side of one MMA (16 columns x 16
// k-rows): {cols 0-7 k 0-7, cols 8-15 k 0-7, cols 0-7 k 8-15, cols 8-15 k 8-15}.
// `w` holds the words of the warp's sub-tiles in order, `s` is the index among them.
template <typename T, int BITS, bool BIASED>
__device__ __forceinline__ void expand(const uint32_t* w, int s, uint32_t ex, uint32_t mlo,
                                       uint32_t mhi, uint32_t (&f)[4]) {
  using E = Emb<T, BITS>;
  if constexpr (BITS == 4) {
    const uint32_t q = w[s];
    f[0] = and_or(q, mlo, ex);
    f[1] = and_or(q >> 8, mlo, ex);
    f[2] = and_or(q >> E::kShiftHi, mhi, ex);
    f[3] = and_or(q >> (8 + E::kShiftHi), mhi, ex);
  } else if constexpr (E::kEmbed) {
    f[0] = __byte_perm(w[2 * s], ex, 0x4240);
    f[1] = __byte_perm(w[2 * s + 1], ex, 0x4240);
    f[2] = __byte_perm(w[2 * s], ex, 0x4341);
    f[3] = __byte_perm(w[2 * s + 1], ex, 0x4341);
  } else {
    uint32_t t0[2], t1[2];
    dequant8<T, BIASED>(w[2 * s], t0);
    dequant8<T, BIASED>(w[2 * s + 1], t1);
    f[0] = t0[0]; f[1] = t1[0]; f[2] = t0[1]; f[3] = t1[1];
  }
}

template <typename T>
__device__ __forceinline__ float lo16_to_float(uint32_t x);
template <typename T>
__device__ __forceinline__ float hi16_to_float(uint32_t x);
template <>
__device__ __forceinline__ float lo16_to_float<half>(uint32_t x) {
  return __half2float(__ushort_as_half((uint16_t)(x & 0xffffu)));
}
template <>
__device__ __forceinline__ float hi16_to_float<half>(uint32_t x) {
  return __half2float(__ushort_as_half((uint16_t)(x >> 16)));
}
template <>
__device__ __forceinline__ float lo16_to_float<__nv_bfloat16>(uint32_t x) {
  return __uint_as_float(x << 16);
}
template <>
__device__ __forceinline__ float hi16_to_float<__nv_bfloat16>(uint32_t x) {
  return __uint_as_float(x & 0xffff0000u);
}

__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r0), "=r"(r1)
               : "r"(addr));
}

namespace sk {

constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 216 * 1024;
constexpr uint32_t kSpinLimit = 1u << 20;      // polls, each may suspend up to kSuspendNs: ~1 s
constexpr uint32_t kSuspendNs = 1000;

// Error word (StreamParams::error, owned by capi.cu): 0 = ok; else the id of the first wait
// that ever timed out (sticky, read by the host): 1 producer waiting for a free stage,
// 2 consumer waiting for a full stage, 3 producer waiting for its last copies at exit.

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Bounded wait on a phase parity; on time-out records `what`, tells the rest of the CTA
// through `abort` (shared memory) and carries on; once a CTA has given up none of its
// waits waits again, so the kernel always terminates promptly (its output is then invalid
// and the host sees the error word).
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int what, int* error,
                                          volatile int* abort) {
  if (*abort != 0) return;
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kSuspendNs)
        : "memory");
    if (done) return;
    if ((spin & 1023u) == 1023u && *abort != 0) return;
  }
  *abort = 1;
  atomicCAS(error, 0, what);
}
// packed weights are read once: keep them from displacing A, scales and partials in L2
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;\n" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
template <int N>
__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;\n" ::"n"(N) : "memory");
}

// MT = 8-row blocks of A (1, 2, 4); SUBS = 16-column sub-tiles of a 64-column tile per warp
// (4: a warp owns a whole tile; 2: two warps share a tile, which halves the accumulators);
// NCW = consumer warps (16, or 12 where a warp needs up to 128 registers: register files are
// handed out to four warps at a time, so 12 + the producer warp get 128 each, 16 + 1 get 96).
template <int BITS, int MT, int SUBS, int NCW>
struct Cfg {
  static constexpr int kConsumers = NCW * 32;
  static constexpr int kThreads = kConsumers + 32;               // + the producer warp
  static constexpr int kTileBytes = 16 * 64 * BITS / 8;          // one weight tile
  static constexpr int kKps = 32 / (SUBS * BITS);                // k-steps per stage
  static constexpr int kTileWarps = 4 / SUBS;                    // warps per tile
  static constexpr int kABoxBytes = MT * 8 * 32;                 // one k-tile of A rows
  static constexpr int kWordsPerSub = BITS / 4;
  static constexpr int kWords = SUBS * kWordsPerSub;             // words per lane per step
  // reduction buffer: one 8-row block of every k sub-range, [sub-range][row][64 WN + 4 floats];
  // sub-ranges x WN = NCW / kTileWarps, so one-tile slices (WN = 1) need the most
  static constexpr int kRedBytes = (NCW / kTileWarps) * 8 * (64 + 4) * 4;
  // packed weights per ring stage: every (tile, k sub-range) pair of the CTA, kKps k-steps
  static constexpr int kWStageBytes = kKps * (NCW / kTileWarps) * kTileBytes;
  static constexpr int kBarOff = 0;                              // barriers first, then ring
  static constexpr int kRingOff = 1024;
  static_assert(kKps >= 1, "stage holds at least one k-step");
};

template <typename T, int BITS, bool HAS_ZP, int GM, int MT, int SUBS, int NCW>
__global__ void __launch_bounds__((NCW + 1) * 32, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap a_map, const StreamParams p) {
  using C = Cfg<BITS, MT, SUBS, NCW>;
  constexpr int kConsumerWarps = NCW;
  constexpr int kWStageBytes = C::kWStageBytes;
  using E = Emb<T, BITS>;
  static_assert(GM == kChannel || GM == kGrouped, "lookup mode runs gemm_lookup_kernel");
  constexpr bool kBiased = !HAS_ZP;
  constexpr int KPS = C::kKps;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ int s_is_last;
  __shared__ int s_abort;  // a wait of this CTA timed out: stop waiting

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int KT = p.kt_total;
  const int NT = p.n / 64;
  const int wn = p.wn;                                   // tiles per slice: 1, 2 or 4
  const int ksub = kConsumerWarps / (wn * C::kTileWarps);  // k sub-ranges of a piece
  const int runs = KPS * ksub;                           // (k-step, sub-range) pairs per stage: <= 32
  const int D = p.ring_stages;
  const uint32_t run_bytes = wn * C::kTileBytes;
  const uint32_t stage_bytes = kWStageBytes + runs * C::kABoxBytes;
  const uint32_t bars = smem_u32(smem) + C::kBarOff;     // full[D], then empty[D]
  const uint32_t ring = smem_u32(smem) + C::kRingOff;
  float* red = reinterpret_cast<float*>(smem + C::kRingOff + (size_t)D * stage_bytes);

  const long long total = (long long)p.slices * KT;
  const long long u_begin = total * blockIdx.x / gridDim.x;
  const long long u_end = total * (blockIdx.x + 1) / gridDim.x;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < D; ++s) {
      mbar_init(bars + 8 * s, 1);                        // full: the producer's expect_tx arrival
      mbar_init(bars + 8 * (D + s), kConsumerWarps);     // empty: one arrival per consumer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  // let the next kernel in the stream start its own weight prefetch early
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

  if (warp == kConsumerWarps) {
    // ================= producer warp =====================================================
    // lane x serves run x of every stage: k-step x / ksub of the stage, sub-range x % ksub
    const uint64_t policy = policy_evict_first();
    const int sp = lane / ksub, r = lane % ksub;
    // mode 0: before the wait on the previous kernel: arm the first D stages and start their
    // weight copies (weights do not depend on that kernel).  mode 1: the activation copies
    // of those stages, then whole stages.
#pragma unroll 1
    for (int mode = 0; mode < 2; ++mode) {
      int it = 0;
      bool stop = false;
#pragma unroll 1
      for (long long u = u_begin; u < u_end && !stop;) {
        const int slice = (int)(u / KT);
        const int kt0 = (int)(u % KT);
        const int kt1 = (int)min((long long)KT, kt0 + (u_end - u));
        u += kt1 - kt0;
        const int len = kt1 - kt0;
        const int nst = ((len + ksub - 1) / ksub + KPS - 1) / KPS;
        const int kb = kt0 + (int)((long long)len * r / ksub);
        const int mylen = kt0 + (int)((long long)len * (r + 1) / ksub) - kb;
        const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(p.b) +
                                    ((size_t)kb * NT + (size_t)slice * wn) * C::kTileBytes;
        const size_t w_kt_stride = (size_t)NT * C::kTileBytes;
#pragma unroll 1
        for (int st = 0; st < nst; ++st, ++it) {
          if (mode == 0 && it == D) { stop = true; break; }
          const int slot = it % D;
          const int step = st * KPS + sp;
          const bool valid = lane < runs && step < mylen;
          const uint32_t full = bars + 8 * slot;
          const uint32_t base = ring + slot * stage_bytes;
          const bool early = it < D;                      // stage armed in mode 0
          if (mode == 1 && !early) mbar_wait(bars + 8 * (D + slot), ((it / D) - 1) & 1, 1, p.error, &s_abort);
          if (mode == 0 || !early) {
            const unsigned nvalid = __popc(__ballot_sync(0xffffffffu, valid));
            if (lane == 0) mbar_expect_tx(full, nvalid * (run_bytes + C::kABoxBytes));
            __syncwarp();
            if (valid)
              bulk_load_1d(base + lane * run_bytes, wsrc + (size_t)step * w_kt_stride, run_bytes,
                           full, policy);
          }
          if (mode == 1 && valid)
            tma_load_2d(base + kWStageBytes + lane * C::kABoxBytes, &a_map, (kb + step) * 16, 0,
                        full);
        }
      }
      if (mode == 0) {
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
      } else {
        // no copy of this CTA may still be in flight when it ends: wait (bounded) for the
        // last stages; in a healthy run the consumers are waiting on the same barriers
        for (int t = it > D ? it - D : 0; t < it; ++t)
          mbar_wait(bars + 8 * (t % D), (t / D) & 1, 3, p.error, &s_abort);
      }
    }
    return;
  }

  // ================= consumer warps ========================================================
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const int q = lane & 3;
  const int c8 = lane >> 2;
  const uint16_t* __restrict__ S = static_cast<const uint16_t*>(p.scales);
  const uint32_t ex = p.c_ex, mlo = p.c_mask_lo, mhi = p.c_mask_hi;
  // role of this warp: tile j of the slice, part `hsel` of the tile, k sub-range r
  const int tw = warp / C::kTileWarps;            // (tile, sub-range) index
  const int hsel = warp % C::kTileWarps;          // which SUBS sub-tiles of the tile
  const int j = tw % wn;
  const int r = tw / wn;
  const int sub0 = hsel * SUBS;                   // first 16-column sub-tile of this warp
  // byte offset of the lane's words inside a tile
  const uint32_t w_lane_off = j * C::kTileBytes + lane * (4 * BITS) + hsel * (SUBS * BITS);
  // ldmatrix source of this lane inside an A box (rows of 32 B, 32-byte swizzle):
  // matrix mi = lane / 8 -> (8-row block mi / 2, k half mi % 2), row lane % 8
  const int lmi = (MT == 1) ? ((lane >> 3) & 1) : (lane >> 3);
  const int lr = (lane & 7) + 8 * (lmi >> 1), lh = lmi & 1;
  const uint32_t a_ld_off = (2 * lr + (lh ^ ((lr >> 2) & 1))) * 16;
  const int gb = p.group_blocks;
  const int red_stride = 64 * wn + 4;             // floats; +4 keeps the scalar stores conflict-free
  const int zrow_words = p.n * BITS / 32;         // zero-point words per group row

  int it = 0;
#pragma unroll 1
  for (long long u = u_begin; u < u_end;) {
    const int slice = (int)(u / KT);
    const int kt0 = (int)(u % KT);
    const int kt1 = (int)min((long long)KT, kt0 + (u_end - u));
    u += kt1 - kt0;
    const int len = kt1 - kt0;
    const int nst = ((len + ksub - 1) / ksub + KPS - 1) / KPS;
    const int kb = kt0 + (int)((long long)len * r / ksub);
    const int mylen = kt0 + (int)((long long)len * (r + 1) / ksub) - kb;
    const int nt0 = slice * wn;

    // acc[mt][s][el]: column 16 (sub0 + s) + c8 + 8 (el >> 1) of tile j, row 8 mt + 2 q + (el & 1)
    float acc[MT][SUBS][4];                                // scaled sums (kGrouped) / running sums
    float grp[GM == kGrouped ? MT : 1][SUBS][4];           // sums of the open group
    float corr[MT][4], rsum[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) corr[i][e] = rsum[i][e] = 0.f;
#pragma unroll
      for (int s = 0; s < SUBS; ++s)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[i][s][e] = 0.f;
          if constexpr (GM == kGrouped) grp[i][s][e] = 0.f;
        }
    }

    // scales / zero-points of the open group, fetched when the group opens
    uint32_t sw[SUBS];
    uint32_t zw[2] = {0u, 0u};
    (void)sw; (void)zw;
    auto fetch_group = [&](int g) {
      if constexpr (GM == kGrouped) {
        // chunk c8 of the permuted scale row of tile j: columns c8 + 8 jj, jj = 2 sub + (el >> 1)
        const uint16_t* src = S + (size_t)g * p.n + (size_t)(nt0 + j) * 64 + c8 * 8 + sub0 * 2;
        if constexpr (SUBS == 4) {
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
          sw[0] = v.x; sw[1] = v.y; sw[2] = v.z; sw[3] = v.w;
        } else {
          const uint2 v = __ldg(reinterpret_cast<const uint2*>(src));
          sw[0] = v.x; sw[1] = v.y;
        }
        if constexpr (HAS_ZP) {
          const uint32_t* zsrc = p.zeros + (size_t)g * zrow_words + (size_t)(nt0 + j) * (2 * BITS);
          if constexpr (BITS == 4) {
            zw[0] = __ldg(zsrc + c8);
          } else {
            zw[0] = __ldg(zsrc + 2 * c8);
            zw[1] = __ldg(zsrc + 2 * c8 + 1);
          }
        }
      }
    };
    // zero-point of column jj = 2 sub + h of this lane's chunk
    auto zp_of = [&](int sub, int h) -> float {
      const int jj = 2 * sub + h;
      if constexpr (BITS == 4) {
        const int t = (jj >> 1) + 4 * (jj & 1);  // column c8 + 8 jj sits at nibble [0,4,1,5,2,6,3,7][jj]
        return (float)((zw[0] >> (4 * t)) & 15u);
      } else {
        const int t = ((jj & 1) << 1) | ((jj >> 1) & 1);  // word jj / 4, byte [0,2,1,3][jj % 4]
        return (float)((zw[jj >> 2] >> (8 * t)) & 255u);
      }
    };
    // group end: fold the open group's sums into acc
    auto close_group = [&]() {
      if constexpr (GM == kGrouped) {
#pragma unroll
        for (int s = 0; s < SUBS; ++s) {
          const float sc[2] = {lo16_to_float<T>(sw[s]), hi16_to_float<T>(sw[s])};
          float zf[2] = {0.f, 0.f};
          if constexpr (HAS_ZP) {
            zf[0] = zp_of(sub0 + s, 0);
            zf[1] = zp_of(sub0 + s, 1);
          }
#pragma unroll
          for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int el = 0; el < 4; ++el) {
              float v = grp[i][s][el];
              if (E::kEmbed) v -= corr[i][el & 1];
              if (HAS_ZP) v = fmaf(-zf[el >> 1], rsum[i][el & 1], v);
              acc[i][s][el] = fmaf(sc[el >> 1], v, acc[i][s][el]);
              grp[i][s][el] = 0.f;
            }
        }
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) corr[i][e] = rsum[i][e] = 0.f;
      }
    };

    int c_g = (GM == kGrouped) ? kb / gb : 0;
    int c_left = (GM == kGrouped) ? gb - kb % gb : 0;
    if (mylen > 0) fetch_group(c_g);

#pragma unroll 1
    for (int st = 0; st < nst; ++st, ++it) {
      const int slot = it % D;
      const uint32_t base = ring + slot * stage_bytes;
      mbar_wait(bars + 8 * slot, (it / D) & 1, 2, p.error, &s_abort);
#pragma unroll
      for (int sp = 0; sp < KPS; ++sp) {
        const int step = st * KPS + sp;
        if (step < mylen) {
          const int x = sp * ksub + r;
          const uint32_t a_box = base + kWStageBytes + x * C::kABoxBytes;
          // activations: act[mt][0] = k 0..7, act[mt][1] = k 8..15 of 8 rows
          uint32_t act[MT][2];
          if constexpr (MT == 1) {
            ldmatrix_x2(act[0][0], act[0][1], a_box + a_ld_off);
          } else {
#pragma unroll
            for (int i = 0; i < MT / 2; ++i) {
              uint32_t rr[4];
              ldmatrix_x4(rr, a_box + i * 512 + a_ld_off);
              act[2 * i][0] = rr[0]; act[2 * i][1] = rr[1];
              act[2 * i + 1][0] = rr[2]; act[2 * i + 1][1] = rr[3];
            }
          }
          uint32_t w[C::kWords];
          {
            const uint32_t wa = base + x * run_bytes + w_lane_off;
            if constexpr (C::kWords == 8) {
              const uint4 v0 = lds128(wa), v1 = lds128(wa + 16);
              w[0] = v0.x; w[1] = v0.y; w[2] = v0.z; w[3] = v0.w;
              w[4] = v1.x; w[5] = v1.y; w[6] = v1.z; w[7] = v1.w;
            } else if constexpr (C::kWords == 4) {
              const uint4 v0 = lds128(wa);
              w[0] = v0.x; w[1] = v0.y; w[2] = v0.z; w[3] = v0.w;
            } else {
              uint32_t v0, v1;
              asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v0), "=r"(v1) : "r"(wa));
              w[0] = v0; w[1] = v1;
            }
          }
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            if (E::kPrescale) act[i][1] = Pair<T>::mul(act[i][1], E::kAScaleHi);
            if (E::kEmbed) {
              const uint32_t off[4] = {kBiased ? E::kOffLoBiased : E::kOffLoRaw,
                                       kBiased ? E::kOffLoBiased : E::kOffLoRaw,
                                       kBiased ? E::kOffHiBiased : E::kOffHiRaw,
                                       kBiased ? E::kOffHiBiased : E::kOffHiRaw};
              mma16816<T>(corr[i], off, act[i][0], act[i][1]);
            }
            if (HAS_ZP) {
              const uint32_t one[4] = {E::kOneLo, E::kOneLo, E::kOneHi, E::kOneHi};
              mma16816<T>(rsum[i], one, act[i][0], act[i][1]);
            }
          }
#pragma unroll
          for (int s = 0; s < SUBS; ++s) {
            uint32_t f[4];
            expand<T, BITS, kBiased>(w, s, ex, mlo, mhi, f);
#pragma unroll
            for (int i = 0; i < MT; ++i) {
              if constexpr (GM == kGrouped)
                mma16816<T>(grp[i][s], f, act[i][0], act[i][1]);
              else
                mma16816<T>(acc[i][s], f, act[i][0], act[i][1]);
            }
          }
          if (GM == kGrouped) {
            if (--c_left == 0 || step == mylen - 1) {
              close_group();
              ++c_g;
              c_left = gb;
              if (step < mylen - 1) fetch_group(c_g);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (D + slot));
    }

    if constexpr (GM == kChannel) {
      // remove the offset (and zero-point) terms once, at the end of the warp's range
      if (E::kEmbed || HAS_ZP) {
        if constexpr (HAS_ZP) {
          const uint32_t* zsrc = p.zeros + (size_t)(nt0 + j) * (2 * BITS);
          if constexpr (BITS == 4) {
            zw[0] = __ldg(zsrc + c8);
          } else {
            zw[0] = __ldg(zsrc + 2 * c8);
            zw[1] = __ldg(zsrc + 2 * c8 + 1);
          }
        }
#pragma unroll
        for (int s = 0; s < SUBS; ++s) {
          float zf[2] = {0.f, 0.f};
          if constexpr (HAS_ZP) {
            zf[0] = zp_of(sub0 + s, 0);
            zf[1] = zp_of(sub0 + s, 1);
          }
#pragma unroll
          for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int el = 0; el < 4; ++el) {
              float v = acc[i][s][el];
              if (E::kEmbed) v -= corr[i][el & 1];
              if (HAS_ZP) v = fmaf(-zf[el >> 1], rsum[i][el & 1], v);
              acc[i][s][el] = v;
            }
        }
      }
    }

    // ---- intra-CTA reduction over the k sub-ranges, one 8-row block at a time -------------
    // consumer thread t owns, per pass o, 4 consecutive columns of one row of the block:
    // float4 number t + o * kConsumers of the [8 rows][width] block
    constexpr int NOUT = (512 + C::kConsumers - 1) / C::kConsumers;  // 512 float4 at WN = 4
    const int width = 64 * wn;
    int o_row[NOUT], o_col[NOUT];
    bool o_active[NOUT];
#pragma unroll
    for (int o = 0; o < NOUT; ++o) {
      const int idx = (threadIdx.x + o * C::kConsumers) * 4;
      o_active[o] = idx < 8 * width;
      o_row[o] = idx / width;                          // 0..7
      o_col[o] = idx % width;                          // inside the slice
    }
    float outv[MT][NOUT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i > 0) consumer_barrier<C::kConsumers>();    // previous block's sums have been read
      {
        float* mine = red + r * (8 * red_stride) + j * 64 + (sub0 * 16 + c8);
#pragma unroll
        for (int s = 0; s < SUBS; ++s)
#pragma unroll
          for (int el = 0; el < 4; ++el)
            mine[(2 * q + (el & 1)) * red_stride + s * 16 + 8 * (el >> 1)] = acc[i][s][el];
      }
      consumer_barrier<C::kConsumers>();
#pragma unroll
      for (int o = 0; o < NOUT; ++o) {
        outv[i][o][0] = outv[i][o][1] = outv[i][o][2] = outv[i][o][3] = 0.f;
        if (o_active[o]) {
          for (int rr = 0; rr < ksub; ++rr) {
            const float4 v = *reinterpret_cast<const float4*>(red + rr * (8 * red_stride) +
                                                              o_row[o] * red_stride + o_col[o]);
            outv[i][o][0] += v.x; outv[i][o][1] += v.y; outv[i][o][2] += v.z; outv[i][o][3] += v.w;
          }
        }
      }
    }

    // ---- cross-CTA reduction for slices shared by several CTAs ---------------------------
    const long long s_first_u = (long long)slice * KT;
    const int first_cta = (int)(((s_first_u + 1) * gridDim.x - 1) / total);
    const int last_cta = (int)(((s_first_u + KT) * gridDim.x - 1) / total);
    const bool split = first_cta != last_cta;
    bool do_store = true;
    const int slot_floats = MT * 8 * width;
    if (split) {
      float* slot = p.partials + (size_t)(blockIdx.x + slice) * slot_floats;
#pragma unroll
      for (int o = 0; o < NOUT; ++o)
        if (o_active[o]) {
#pragma unroll
          for (int i = 0; i < MT; ++i)
            if (i * 8 < p.m)
              __stcg(reinterpret_cast<float4*>(slot + (i * 8 + o_row[o]) * width + o_col[o]),
                     make_float4(outv[i][o][0], outv[i][o][1], outv[i][o][2], outv[i][o][3]));
        }
      __threadfence();
      consumer_barrier<C::kConsumers>();
      if (threadIdx.x == 0) {
        const int prev = atomicAdd(p.counters + first_cta, 1);
        s_is_last = (prev == last_cta - first_cta);
      }
      consumer_barrier<C::kConsumers>();
      do_store = s_is_last != 0;
      if (do_store) {
        __threadfence();
#pragma unroll
        for (int o = 0; o < NOUT; ++o)
          if (o_active[o]) {
#pragma unroll
            for (int i = 0; i < MT; ++i)
              outv[i][o][0] = outv[i][o][1] = outv[i][o][2] = outv[i][o][3] = 0.f;
            for (int cta = first_cta; cta <= last_cta; ++cta) {
              const float* src = p.partials + (size_t)(cta + slice) * slot_floats;
#pragma unroll
              for (int i = 0; i < MT; ++i)
                if (i * 8 < p.m) {
                  const float4 v = __ldcg(reinterpret_cast<const float4*>(
                      src + (i * 8 + o_row[o]) * width + o_col[o]));
                  outv[i][o][0] += v.x; outv[i][o][1] += v.y;
                  outv[i][o][2] += v.z; outv[i][o][3] += v.w;
                }
            }
          }
        if (threadIdx.x == 0) p.counters[first_cta] = 0;
      }
    } else {
      consumer_barrier<C::kConsumers>();  // the reduction buffer is free for the next piece
    }

    // ---- epilogue: channel scale, bias, convert, store (or all-reduce) -------------------
    uint32_t call = 0, flag = 0;
    long long parity_off = 0;
    if (p.ar.world != 0) {
      call = ar_ld_volatile(p.ar.state);
      flag = ar_flag(call);
      parity_off = (long long)(call & 1) * p.ar.world * p.ar.slot_bytes;
    }
#pragma unroll
    for (int o = 0; o < NOUT; ++o) {
      if (!(do_store && o_active[o])) continue;
      const int n_base = nt0 * 64 + o_col[o];
      uint32_t packed[MT][2];
      {
        float cs[4], bs[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          cs[e] = (GM == kChannel) ? Pair<T>::to_float(S[single_perm_pos(n_base + e)]) : 1.f;
          bs[e] = p.bias ? Pair<T>::to_float(
                               static_cast<const uint16_t*>(p.bias)[single_perm_pos(n_base + e)])
                         : 0.f;
        }
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int e = 0; e < 4; e += 2) {
            const float v0 = outv[i][o][e] * cs[e] + bs[e];
            const float v1 = outv[i][o][e + 1] * cs[e + 1] + bs[e + 1];
            packed[i][e / 2] =
                (uint32_t)Pair<T>::from_float(v0) | ((uint32_t)Pair<T>::from_float(v1) << 16);
          }
      }
      if (p.ar.world == 0) {
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          if (i * 8 + o_row[o] >= p.m) continue;
          uint16_t* dst = static_cast<uint16_t*>(p.c) + (size_t)(i * 8 + o_row[o]) * p.n + n_base;
          *reinterpret_cast<uint2*>(dst) = make_uint2(packed[i][0], packed[i][1]);
        }
      } else {
        // All-reduce over the peer link (protocol in ar_link.cuh): the rounded partial of
        // this rank goes to every peer as flagged packets, each thread then collects the
        // peers' packets for its own elements and sums in rank order.
        const ArLink& l = p.ar;
        for (int rk = 0; rk < l.world; ++rk) {
          if (rk == l.rank) continue;
          char* pslot = static_cast<char*>(l.bufs[rk]) + parity_off + l.rank * l.slot_bytes;
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            if (i * 8 + o_row[o] >= p.m) continue;
            // 2 values per 8-byte packet
            char* dst = pslot + ((size_t)(i * 8 + o_row[o]) * p.n + n_base) * 4;
            ar_put2(dst, packed[i][0], packed[i][1], flag);
          }
        }
        const char* mybuf = static_cast<const char*>(l.bufs[l.rank]) + parity_off;
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          if (i * 8 + o_row[o] >= p.m) continue;
          const size_t el = (size_t)(i * 8 + o_row[o]) * p.n + n_base;
          uint32_t d[kArMaxWorld][2];
          if (!ar_collect<2>(l, mybuf, el * 4, flag, d)) break;
          float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int rk = 0; rk < kArMaxWorld; ++rk) {
            if (rk < l.world) {
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const uint32_t v = (rk == l.rank) ? packed[i][e] : d[rk][e];
                sum[2 * e] += Pair<T>::to_float((uint16_t)(v & 0xffffu));
                sum[2 * e + 1] += Pair<T>::to_float((uint16_t)(v >> 16));
              }
            }
          }
          const uint32_t o0 = (uint32_t)Pair<T>::from_float(sum[0]) |
                              ((uint32_t)Pair<T>::from_float(sum[1]) << 16);
          const uint32_t o1 = (uint32_t)Pair<T>::from_float(sum[2]) |
                              ((uint32_t)Pair<T>::from_float(sum[3]) << 16);
          *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.c) + el) = make_uint2(o0, o1);
        }
      }
    }
  }
  if (p.ar.world != 0) {
    // every CTA reports once, after all its threads are done with the link
    const uint32_t call = ar_ld_volatile(p.ar.state);
    consumer_barrier<C::kConsumers>();
    if (threadIdx.x == 0) ar_arrive(p.ar, call, gridDim.x);
  }
}

}  // namespace sk

typedef CUresult (*StreamEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                        const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                        const cuuint32_t*, CUtensorMapInterleave,
                                        CUtensorMapSwizzle, CUtensorMapL2promotion,
                                        CUtensorMapFloatOOBfill);
StreamEncodeTiledFn stream_encode_fn();  // capi.cu: cuTensorMapEncodeTiled through the runtime
int* stream_error_ptr();                 // capi.cu: device address of the kernel's error word

// Slice width (64-column tiles) for a problem: the widest of 4, 2, 1 that divides the tile
// count and keeps a partial-sum slot (rows x width floats) within 4096 floats.
inline int stream_slice_tiles(int nt, int mt) {
  const int cap = mt >= 4 ? 2 : 4;
  for (int w = cap; w > 1; w /= 2)
    if (nt % w == 0) return w;
  return 1;
}

// Host launcher for one (type, bits, zp, group mode, MT) variant.
template <typename T, int BITS, bool HAS_ZP, int GM, int MT>
int launch_stream(StreamParams p, int max_ctas, cudaStream_t stream) {
  // a warp owns a whole tile up to 16 rows (12 consumer warps of up to 128 registers from 9
  // rows up), half a tile above
  constexpr int SUBS = MT >= 4 ? 2 : 4;
  constexpr int NCW = MT >= 2 ? 12 : 16;
  using C = sk::Cfg<BITS, MT, SUBS, NCW>;
  using E = Emb<T, BITS>;
  auto kernel = sk::gemm_stream_kernel<T, BITS, HAS_ZP, GM, MT, SUBS, NCW>;
  static bool attr_done[64] = {};  // per device; benign race: the call is idempotent
  int dev = 0;
  B200Q_CUDA_OK(cudaGetDevice(&dev));
  if (!attr_done[dev & 63]) {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       sk::kSmemBudget));
    attr_done[dev & 63] = true;
  }
  p.error = stream_error_ptr();
  B200Q_REQUIRE(p.error != nullptr, B200Q_ECUDA, "cudaGetSymbolAddress(error word) failed");
  p.c_ex = E::kEx;
  p.c_mask_lo = E::kMaskLo;
  p.c_mask_hi = E::kMaskHi;
  const int nt = p.n / 64;
  p.wn = stream_slice_tiles(nt, MT);
  p.slices = nt / p.wn;
  const int ksub = NCW / (p.wn * C::kTileWarps);
  const int runs = C::kKps * ksub;
  const int stage_bytes = C::kWStageBytes + runs * C::kABoxBytes;
  int stages = (sk::kSmemBudget - C::kRingOff - C::kRedBytes) / stage_bytes;
  if (stages > sk::kMaxStages) stages = sk::kMaxStages;
  B200Q_REQUIRE(stages >= 2, B200Q_EUNSUPPORTED, "streaming kernel: ring does not fit");
  p.ring_stages = stages;
  const int smem_bytes = C::kRingOff + stages * stage_bytes + C::kRedBytes;

  // activations as a [M, K] tensor of 16-bit elements; box = one k-tile of MT * 8 rows
  StreamEncodeTiledFn encode = stream_encode_fn();
  B200Q_REQUIRE(encode != nullptr, B200Q_ECUDA, "cuTensorMapEncodeTiled is not available");
  CUtensorMap a_map;
  const cuuint64_t gdim[2] = {(cuuint64_t)p.k, (cuuint64_t)p.m};
  const cuuint64_t gstride[1] = {(cuuint64_t)p.lda * 2};
  const cuuint32_t box[2] = {16, (cuuint32_t)(MT * 8)};
  const cuuint32_t estride[2] = {1, 1};
  const CUresult r = encode(&a_map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(p.a), gdim,
                            gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200Q_REQUIRE(r == CUDA_SUCCESS, B200Q_ECUDA, "cuTensorMapEncodeTiled (activations) failed with %d",
                (int)r);

  // one CTA per SM, every CTA an equal stripe of (slice, k-tile) units; small problems
  // take fewer CTAs so that a stripe holds at least 8 k-tiles of a slice
  const long long total = (long long)p.slices * p.kt_total;
  long long grid = device_sm_count();
  if (grid > max_ctas) grid = max_ctas;
  const long long by_work = (total + 7) / 8;
  if (grid > by_work) grid = by_work;
  if (grid < 1) grid = 1;

  // programmatic dependent launch: the kernel may start while its predecessor in
  // the stream drains; it orders itself with griddepcontrol.wait
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, a_map, p));
  note_launch();
  B200Q_CUDA_OK(cudaGetLastError());
  return B200Q_OK;
}

}  // namespace b200q
