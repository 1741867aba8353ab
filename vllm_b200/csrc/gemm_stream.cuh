// Streaming mixed-precision GEMM for the decode regime (up to 32 rows of A per
// launch): C[M,N] = A[M,K] * dequant(B), grouped or channel-wise scales.
//
// The kernel is meant to be HBM-bound: the packed weights are read exactly
// once, in 512 B (4-bit) / 1 KB (8-bit) tiles that are contiguous in the Marlin
// layout, through a deep per-warp cp.async ring, and fed to mma.sync.m16n8k16
// with fp32 accumulation.  What limits a streaming kernel of this kind is the
// instruction count per byte, so the arithmetic is arranged to need almost no
// ALU work per weight:
//
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
//    This is also more accurate than rounding w*s to 16 bits first.
//
// Work decomposition.  The weight matrix is cut into column "slices" of NTW
// 64-column tiles.  A slice is owned by a thread-block cluster of 1, 2, 4 or 8
// CTAs that split K evenly (enough CTAs to fill the GPU); inside a CTA the 8
// warps split the CTA's k-range again.  Warp sums meet in shared memory; CTA
// sums meet through distributed shared memory: every CTA publishes its tile,
// and after a cluster barrier each CTA adds the ranks' copies of its share of
// the rows in rank order and stores C.  No global scratch, no atomics, no
// spinning, and the result is bitwise reproducible.
#pragma once

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
template <typename T, int BITS, bool BIASED>
__device__ __forceinline__ void expand(const uint32_t* w, int sub, uint32_t ex, uint32_t mlo,
                                       uint32_t mhi, uint32_t (&f)[4]) {
  using E = Emb<T, BITS>;
  if constexpr (BITS == 4) {
    const uint32_t q = w[sub];
    f[0] = and_or(q, mlo, ex);
    f[1] = and_or(q >> 8, mlo, ex);
    f[2] = and_or(q >> E::kShiftHi, mhi, ex);
    f[3] = and_or(q >> (8 + E::kShiftHi), mhi, ex);
  } else if constexpr (E::kEmbed) {
    f[0] = __byte_perm(w[2 * sub], ex, 0x4240);
    f[1] = __byte_perm(w[2 * sub + 1], ex, 0x4240);
    f[2] = __byte_perm(w[2 * sub], ex, 0x4341);
    f[3] = __byte_perm(w[2 * sub + 1], ex, 0x4341);
  } else {
    uint32_t t0[2], t1[2];
    dequant8<T, BIASED>(w[2 * sub], t0);
    dequant8<T, BIASED>(w[2 * sub + 1], t1);
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

// MT = number of 8-row blocks of A (1, 2, 4); NTW = 64-column tiles per slice.
template <int BITS, bool HAS_ZP, int GM, int MT, int NTW>
struct StreamCfg {
  static constexpr int kTileBytes = 16 * 64 * BITS / 8;  // one weight tile
  static constexpr int kAOff = NTW * kTileBytes;         // A rows (32 B each) after the weights
  static constexpr int kABytes = MT * 256;
  static constexpr int kStageBytes = kAOff + kABytes;
  // per-warp group slots (scales, zero-points), used in rotation; more slots than
  // ring stages, so a slot is never refilled while its group is still open
  static constexpr int kSlots = 8;
  static constexpr int kSlotZOff = NTW * 128;
  static constexpr int kSlotBytes =
      (GM == kGrouped) ? (kSlotZOff + (HAS_ZP ? NTW * 8 * BITS : 0)) : 0;
  static constexpr int kGroupBytes = kSlots * kSlotBytes;
  // ring depth: as deep as ~88 KB of shared memory per CTA allows, 3..8 stages
  static constexpr int kDepthFit = (88 * 1024 / kStreamWarps - kGroupBytes) / kStageBytes;
  static constexpr int kDepth = kDepthFit > 8 ? 8 : (kDepthFit < 3 ? 3 : kDepthFit);
  static constexpr int kWarpBytes = kStageBytes * kDepth + kGroupBytes;
  static constexpr int kRingBytes = kWarpBytes * kStreamWarps;
  // reduction buffer: one 8-row block of every warp's accumulators, [row][column]
  static constexpr int kRedStride = 64 * NTW + 4;  // floats; +4 keeps the scalar stores conflict-free
  static constexpr int kRedBytes = kStreamWarps * 8 * kRedStride * 4;
  // the CTA's finished tile, published to the cluster after the reduction
  static constexpr int kXBytes = MT * 8 * 64 * NTW * 4;
  static constexpr int kSmemBytes =
      kRingBytes > kRedBytes + kXBytes ? kRingBytes : kRedBytes + kXBytes;
  static constexpr int kEpt = 2 * NTW;  // output elements per thread per 8-row block
};

// MOE: the mixture-of-experts form (see gemm_lookup.cuh): blockIdx.y is a block of p.m sorted
// ids, the rows of A come through the ids (row = id / top_k), the block's expert selects the
// weights, output rows are the ids themselves.
template <typename T, int BITS, bool HAS_ZP, int GM, int MT, int NTW, int MINB, bool MOE = false>
__global__ void __launch_bounds__(kStreamThreads, MINB) gemm_stream_kernel(const StreamParams p) {
  using Cfg = StreamCfg<BITS, HAS_ZP, GM, MT, NTW>;
  using E = Emb<T, BITS>;
  static_assert(GM == kChannel || GM == kGrouped, "lookup mode runs gemm_lookup_kernel");
  constexpr int D = Cfg::kDepth;
  constexpr bool kBiased = !HAS_ZP;
  constexpr int kWordsPerTile = BITS == 4 ? 4 : 8;  // words per lane per tile
  extern __shared__ __align__(128) unsigned char smem[];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q = lane & 3;
  const int c8 = lane >> 2;
  const int KT = p.kt_total;
  const int NT = p.n / 64;
  const uint16_t* __restrict__ S = static_cast<const uint16_t*>(p.scales);
  const uint32_t ex = p.c_ex, mlo = p.c_mask_lo, mhi = p.c_mask_hi;
  const unsigned char* __restrict__ Bw = reinterpret_cast<const unsigned char*>(p.b);
  const uint32_t* __restrict__ Zp = p.zeros;
  const uint16_t* __restrict__ Bias = static_cast<const uint16_t*>(p.bias);
  const int32_t* moe_ids = nullptr;   // this block's sorted ids
  if constexpr (MOE) {
    // (uniform over the cluster: its CTAs share blockIdx.y)
    if ((int)blockIdx.y * p.m >= *p.moe_num_padded) return;
    const int expert = p.moe_expert_ids[blockIdx.y];
    if (expert < 0) return;
    moe_ids = p.moe_sorted_ids + (size_t)blockIdx.y * p.m;
    Bw += (size_t)expert * p.moe_b_stride * 4;
    S += (size_t)expert * p.moe_s_stride;
    if (HAS_ZP) Zp += (size_t)expert * p.moe_z_stride;
    if (p.bias) Bias += (size_t)expert * p.moe_bias_stride;
  }

  // cluster = the CTAs that share one column slice; rank = which part of K
  uint32_t ksplit, krank;
  asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(ksplit));
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(krank));

  const uint32_t ring = smem_u32(smem) + warp * Cfg::kWarpBytes;
  const uint32_t slots = ring + D * Cfg::kStageBytes;
  float* red = reinterpret_cast<float*>(smem);
  // this CTA's finished tile, read by the other CTAs of the cluster
  float* xbuf = reinterpret_cast<float*>(smem + Cfg::kRedBytes);

  // ---- lane-constant addressing of the A rows inside a stage -------------------------
  // A is staged as rows of 32 B (16 k-values); 16 B chunk (row r, half h) lives at
  // chunk position 2r + (h ^ ((r >> 2) & 1)) so that ldmatrix reads are conflict-free.
  // fill: lane copies (row lane/2, half lane%2) of every 16-row block (8 rows when MT == 1:
  // the upper lanes repeat the lower ones instead of diverging)
  const int fr = (MT == 1) ? ((lane >> 1) & 7) : (lane >> 1), fh = lane & 1;
  const uint32_t a_fill_off = (2 * fr + (fh ^ ((fr >> 2) & 1))) * 16;
  // load: matrix mi = lane/8 -> (8-row block mi/2, half mi%2), row lane%8
  const int lmi = (MT == 1) ? ((lane >> 3) & 1) : (lane >> 3);
  const int lr = (lane & 7) + 8 * (lmi >> 1), lh = lmi & 1;
  const uint32_t a_ld_off = (2 * lr + (lh ^ ((lr >> 2) & 1))) * 16;
  const size_t w_kt_stride = (size_t)NT * Cfg::kTileBytes;  // bytes between k-tiles
  constexpr int kABlocks = (MT + 1) / 2;                    // 16-row blocks of A
  const size_t a_blk_stride = (size_t)16 * p.lda * 2;
  int a_bytes[kABlocks];
  long long a_row[kABlocks];  // source row of A this lane stages for each 16-row block
#pragma unroll
  for (int i = 0; i < kABlocks; ++i) {
    a_bytes[i] = (i * 16 + fr < p.m) ? 16 : 0;
    a_row[i] = i * 16 + fr;
    if constexpr (MOE) {
      const int id = a_bytes[i] ? moe_ids[i * 16 + fr] : p.moe_rows;
      a_bytes[i] = id < p.moe_rows ? 16 : 0;
      a_row[i] = id / p.moe_top_k;
    }
  }

  // let the next kernel in the stream start its own weight prefetch early
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  bool first_piece = true;

  {
    const int slice = blockIdx.x / ksplit;
    const int kt0 = (int)((long long)KT * krank / ksplit);
    const int kt1 = (int)((long long)KT * (krank + 1) / ksplit);
    const int nt0 = slice * NTW;  // first 64-column tile of the slice

    // this warp's contiguous share of [kt0, kt1)
    const int len = kt1 - kt0;
    const int wb = kt0 + (int)((long long)len * warp / kStreamWarps);
    const int we = kt0 + (int)((long long)len * (warp + 1) / kStreamWarps);
    const int n_steps = we - wb;

    // acc[mt][j][sub][el]: column 64 j + 16 sub + c8 + 8 (el >> 1), row 8 mt + 2 q + (el & 1)
    float acc[MT][NTW][4][4];  // scaled sums (kGrouped) / running sums (kChannel)
    float grp[GM == kGrouped ? MT : 1][GM == kGrouped ? NTW : 1][4][4];  // sums of the open group
    float corr[MT][4], rsum[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) corr[i][e] = rsum[i][e] = 0.f;
#pragma unroll
      for (int j = 0; j < NTW; ++j)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[i][j][b][e] = 0.f;
            if constexpr (GM == kGrouped) grp[i][j][b][e] = 0.f;
          }
    }

    // ---- producer state -------------------------------------------------------------
    const unsigned char* i_w = Bw + ((size_t)wb * NT + nt0) * Cfg::kTileBytes + lane * 16;
    // running address of block 0's row; the other blocks at a constant distance from it
    const unsigned char* i_a = static_cast<const unsigned char*>(p.a) +
                               ((size_t)(a_bytes[0] ? a_row[0] : 0) * p.lda + (size_t)wb * 16 + fh * 8) * 2;
    long long a_delta[MOE ? kABlocks : 1];  // moe: the rows of a block are wherever the ids say
    (void)a_delta;
    if constexpr (MOE) {
#pragma unroll
      for (int i = 0; i < kABlocks; ++i)
        a_delta[i] = a_bytes[i] ? (a_row[i] - (a_bytes[0] ? a_row[0] : 0)) * (long long)p.lda * 2 : 0;
    }
    uint32_t i_st = ring;  // next stage to fill
    const uint32_t ring_end = ring + D * Cfg::kStageBytes;
    const int gb = p.group_blocks;
    int i_g = (GM == kGrouped) ? wb / gb : 0;  // group of the next k-tile to issue
    int i_left = 0;                            // k-tiles until the next group load
    int i_first_left = (GM == kGrouped) ? gb - wb % gb : 0;
    int issued = 0;

    // next stage to fill with weights (runs ahead only in the prologue); the lane's own byte
    // offset is part of the running address, tile offsets are immediates of the copies
    const uint32_t w_lane_off = (BITS == 4) ? lane * 16 : (lane & 1) * 512 + (lane >> 1) * 16;
    uint32_t i_stw = ring + w_lane_off;
    const uint32_t ring_end_w = ring_end + w_lane_off;
    auto issue_w = [&]() {
      if constexpr (BITS == 4) {
        cp_async16_off<0, 0>(i_stw, i_w);
        if constexpr (NTW == 2) cp_async16_off<512, 512>(i_stw, i_w);
      } else {
        // 16 B chunk ch of a tile belongs to lane ch/2, half ch%2
        cp_async16_off<0, 0>(i_stw, i_w);
        cp_async16_off<256, 512>(i_stw, i_w);
        if constexpr (NTW == 2) {
          cp_async16_off<1024, 1024>(i_stw, i_w);
          cp_async16_off<1024 + 256, 1024 + 512>(i_stw, i_w);
        }
      }
      i_w += w_kt_stride;
      i_stw += Cfg::kStageBytes;
      if (i_stw == ring_end_w) i_stw = ring + w_lane_off;
    };
    auto issue_a = [&]() {
#pragma unroll
      for (int i = 0; i < kABlocks; ++i)
        if constexpr (MOE)
          cp_async16(i_st + Cfg::kAOff + i * 512 + a_fill_off, a_bytes[i] ? i_a + a_delta[i] : i_a,
                     a_bytes[i]);
        else
          cp_async16(i_st + Cfg::kAOff + i * 512 + a_fill_off,
                     a_bytes[i] ? i_a + i * a_blk_stride : i_a, a_bytes[i]);
      if (GM == kGrouped) {
        if (i_left == 0) {
          const uint32_t slot = slots + (i_g & (Cfg::kSlots - 1)) * Cfg::kSlotBytes;
          // NTW * 8 chunks of scales; surplus lanes repeat a chunk instead of diverging
          const int sl = lane & (NTW * 8 - 1);
          cp_async16(slot + sl * 16, S + (size_t)i_g * p.n + nt0 * 64 + sl * 8);
          if (HAS_ZP) {
            constexpr int kChunks = NTW * 8 * BITS / 16;  // 16 B chunks of zero-point words
            const int zl = lane & (kChunks - 1);
            cp_async16(slot + Cfg::kSlotZOff + zl * 16,
                       Zp + (size_t)i_g * (p.n * BITS / 32) + nt0 * (2 * BITS) + zl * 4);
          }
          ++i_g;
          i_left = i_first_left;
          i_first_left = gb;
        }
        --i_left;
      }
      i_a += 32;
      i_st += Cfg::kStageBytes;
      if (i_st == ring_end) i_st = ring;
    };
    auto issue = [&]() {
      issue_w();
      issue_a();
    };

    // ---- group end: fold the open group's sums into acc ---------------------------------
    auto close_group = [&](int g) {
      if constexpr (GM == kGrouped) {
        const uint32_t slot = slots + (g & (Cfg::kSlots - 1)) * Cfg::kSlotBytes;
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          // chunk c8 of the permuted scale row: columns c8 + 8 jj, jj = 2 sub + (el >> 1)
          const uint4 c0 = lds128(slot + j * 128 + c8 * 16);
          const uint32_t cw[4] = {c0.x, c0.y, c0.z, c0.w};
          uint32_t zw[2];
          (void)zw;
          if (HAS_ZP) {
            if (BITS == 4) {
              zw[0] = lds32(slot + Cfg::kSlotZOff + j * 32 + c8 * 4);
            } else {
              zw[0] = lds32(slot + Cfg::kSlotZOff + j * 64 + c8 * 8);
              zw[1] = lds32(slot + Cfg::kSlotZOff + j * 64 + c8 * 8 + 4);
            }
          }
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            float sc[2], zf[2];
            sc[0] = lo16_to_float<T>(cw[sub]);
            sc[1] = hi16_to_float<T>(cw[sub]);
            if (HAS_ZP) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int jj = 2 * sub + h;
                if (BITS == 4) {
                  // column c8 + 8 jj sits at nibble [0,4,1,5,2,6,3,7][jj]
                  const int t = (jj >> 1) + 4 * (jj & 1);
                  zf[h] = (float)((zw[0] >> (4 * t)) & 15u);
                } else {
                  // word jj/4, byte [0,2,1,3][jj%4]
                  const int t = ((jj & 1) << 1) | ((jj >> 1) & 1);
                  zf[h] = (float)((zw[jj >> 2] >> (8 * t)) & 255u);
                }
              }
            }
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
              for (int el = 0; el < 4; ++el) {
                float v = grp[i][j][sub][el];
                if (E::kEmbed) v -= corr[i][el & 1];
                if (HAS_ZP) v = fmaf(-zf[el >> 1], rsum[i][el & 1], v);
                acc[i][j][sub][el] = fmaf(sc[el >> 1], v, acc[i][j][sub][el]);
                grp[i][j][sub][el] = 0.f;
              }
          }
        }
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) corr[i][e] = rsum[i][e] = 0.f;
      }
    };

    if (first_piece) {
      // The weights do not depend on the kernel before this one in the stream:
      // start streaming them, and only then wait for that kernel to finish
      // (programmatic dependent launch) before touching A, scales' consumers,
      // scratch or C.  The whole prologue forms one cp.async group.
      first_piece = false;
      const int pw = n_steps < D - 1 ? n_steps : D - 1;
#pragma unroll
      for (int s = 0; s < D - 1; ++s)
        if (s < pw) issue_w();
      asm volatile("griddepcontrol.wait;\n" ::: "memory");
#pragma unroll
      for (int s = 0; s < D - 1; ++s)
        if (s < pw) issue_a();
      issued = pw;
#pragma unroll
      for (int s = 0; s < D - 1; ++s) cp_async_commit();
    } else {
#pragma unroll
      for (int s = 0; s < D - 1; ++s) {
        if (issued < n_steps) {
          issue();
          ++issued;
        }
        cp_async_commit();
      }
    }

    uint32_t c_st = ring;
    int c_g = (GM == kGrouped) ? wb / gb : 0;
    int c_left = (GM == kGrouped) ? gb - wb % gb : 0;

    for (int s = 0; s < n_steps; ++s) {
      cp_async_wait<D - 2>();
      __syncwarp();
      if (issued < n_steps) {
        issue();
        ++issued;
      }
      cp_async_commit();
      const uint32_t st = c_st;
      c_st += Cfg::kStageBytes;
      if (c_st == ring_end) c_st = ring;

      // activations: act[mt][0] = k 0..7, act[mt][1] = k 8..15 of 8 rows
      uint32_t act[MT][2];
      if constexpr (MT == 1) {
        ldmatrix_x2(act[0][0], act[0][1], st + Cfg::kAOff + a_ld_off);
      } else {
#pragma unroll
        for (int i = 0; i < MT / 2; ++i) {
          uint32_t r[4];
          ldmatrix_x4(r, st + Cfg::kAOff + i * 512 + a_ld_off);
          act[2 * i][0] = r[0]; act[2 * i][1] = r[1];
          act[2 * i + 1][0] = r[2]; act[2 * i + 1][1] = r[3];
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
      for (int j = 0; j < NTW; ++j) {
        uint32_t w[kWordsPerTile];
        {
          const uint4 w4 = lds128(st + j * Cfg::kTileBytes + lane * 16);
          w[0] = w4.x; w[1] = w4.y; w[2] = w4.z; w[3] = w4.w;
          if (BITS == 8) {
            const uint4 w5 = lds128(st + j * Cfg::kTileBytes + 512 + lane * 16);
            w[4] = w5.x; w[5] = w5.y; w[6] = w5.z; w[7] = w5.w;
          }
        }
#pragma unroll
        for (int sub = 0; sub < 4; ++sub) {
          uint32_t f[4];
          expand<T, BITS, kBiased>(w, sub, ex, mlo, mhi, f);
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            if constexpr (GM == kGrouped)
              mma16816<T>(grp[i][j][sub], f, act[i][0], act[i][1]);
            else
              mma16816<T>(acc[i][j][sub], f, act[i][0], act[i][1]);
          }
        }
      }

      if (GM == kGrouped) {
        if (--c_left == 0 || s == n_steps - 1) {
          close_group(c_g);
          ++c_g;
          c_left = gb;
        }
      }
    }
    cp_async_wait<0>();

    if constexpr (GM == kChannel) {
      // remove the offset (and zero-point) terms once, at the end of the warp's range
      if (E::kEmbed || HAS_ZP) {
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          uint32_t zw[2];
          (void)zw;
          if (HAS_ZP) {
            const uint32_t* zrow = Zp + (size_t)(nt0 + j) * (2 * BITS);
            if (BITS == 4) {
              zw[0] = __ldg(zrow + c8);
            } else {
              zw[0] = __ldg(zrow + 2 * c8);
              zw[1] = __ldg(zrow + 2 * c8 + 1);
            }
          }
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            float zf[2] = {0.f, 0.f};
            if (HAS_ZP) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int jj = 2 * sub + h;
                if (BITS == 4) {
                  const int t = (jj >> 1) + 4 * (jj & 1);
                  zf[h] = (float)((zw[0] >> (4 * t)) & 15u);
                } else {
                  const int t = ((jj & 1) << 1) | ((jj >> 1) & 1);
                  zf[h] = (float)((zw[jj >> 2] >> (8 * t)) & 255u);
                }
              }
            }
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
              for (int el = 0; el < 4; ++el) {
                float v = acc[i][j][sub][el];
                if (E::kEmbed) v -= corr[i][el & 1];
                if (HAS_ZP) v = fmaf(-zf[el >> 1], rsum[i][el & 1], v);
                acc[i][j][sub][el] = v;
              }
          }
        }
      }
    }

    // ---- intra-CTA reduction, one 8-row block at a time ----------------------------

    float outv[MT][Cfg::kEpt];
    const int o_row = threadIdx.x >> 5;                // 0..7
    const int o_col = (threadIdx.x & 31) * Cfg::kEpt;  // inside the slice
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      __syncthreads();  // ring (or previous block's sums) no longer in use
      {
        float* mine = red + warp * (8 * Cfg::kRedStride);
#pragma unroll
        for (int j = 0; j < NTW; ++j)
#pragma unroll
          for (int sub = 0; sub < 4; ++sub)
#pragma unroll
            for (int el = 0; el < 4; ++el)
              mine[(2 * q + (el & 1)) * Cfg::kRedStride + j * 64 + sub * 16 + c8 + 8 * (el >> 1)] =
                  acc[i][j][sub][el];
      }
      __syncthreads();
#pragma unroll
      for (int e = 0; e < Cfg::kEpt; ++e) outv[i][e] = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < kStreamWarps; ++w8) {
        const float* src = red + w8 * (8 * Cfg::kRedStride) + o_row * Cfg::kRedStride + o_col;
        if constexpr (Cfg::kEpt == 4) {
          const float4 v = *reinterpret_cast<const float4*>(src);
          outv[i][0] += v.x; outv[i][1] += v.y; outv[i][2] += v.z; outv[i][3] += v.w;
        } else {
          const float2 v = *reinterpret_cast<const float2*>(src);
          outv[i][0] += v.x; outv[i][1] += v.y;
        }
      }
    }

    // ---- cross-CTA reduction inside the cluster, through distributed shared memory ----
    // Every CTA publishes its tile in its own shared memory; after a cluster
    // barrier the 8-row blocks of the tile are shared out among the CTAs (block % ksplit),
    // and each sums the ranks' copies in rank order (bitwise reproducible).
    bool do_store = true;
    if (ksplit > 1) {
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        float* dst = xbuf + (i * 8 + o_row) * (64 * NTW) + o_col;
        if constexpr (Cfg::kEpt == 4)
          *reinterpret_cast<float4*>(dst) = make_float4(outv[i][0], outv[i][1], outv[i][2], outv[i][3]);
        else
          *reinterpret_cast<float2*>(dst) = make_float2(outv[i][0], outv[i][1]);
      }
      asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
      do_store = false;
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const int row = i * 8 + o_row;
        if ((uint32_t)i % ksplit == krank) {
          do_store = true;
#pragma unroll
          for (int e = 0; e < Cfg::kEpt; ++e) outv[i][e] = 0.f;
          const uint32_t local = smem_u32(xbuf + row * (64 * NTW) + o_col);
          for (uint32_t r = 0; r < ksplit; ++r) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(r));
            if constexpr (Cfg::kEpt == 4) {
              float4 v;
              asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                           : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                           : "r"(remote)
                           : "memory");
              outv[i][0] += v.x; outv[i][1] += v.y; outv[i][2] += v.z; outv[i][3] += v.w;
            } else {
              float2 v;
              asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];\n"
                           : "=f"(v.x), "=f"(v.y)
                           : "r"(remote)
                           : "memory");
              outv[i][0] += v.x; outv[i][1] += v.y;
            }
          }
        }
      }
    }

    // no CTA may exit while others still read its shared memory; after this barrier
    // CTAs without output rows leave at once and make room for the next kernel
    if (ksplit > 1) {
      asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    }

    // ---- epilogue: channel scale, bias, convert, store (or all-reduce) ---------------
    const int n_base = nt0 * 64 + o_col;
    uint32_t packed[MT][Cfg::kEpt / 2];
    if (do_store) {
      float cs[Cfg::kEpt], bs[Cfg::kEpt];
#pragma unroll
      for (int e = 0; e < Cfg::kEpt; ++e) {
        cs[e] = (GM == kChannel) ? Pair<T>::to_float(S[single_perm_pos(n_base + e)]) : 1.f;
        bs[e] = p.bias ? Pair<T>::to_float(Bias[single_perm_pos(n_base + e)]) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        float tw = 1.f;
        if constexpr (MOE) {
          if (p.moe_topk_weights && i * 8 + o_row < p.m) {
            const int id = moe_ids[i * 8 + o_row];
            if (id < p.moe_rows) tw = p.moe_topk_weights[id];
          }
        }
#pragma unroll
        for (int e = 0; e < Cfg::kEpt; e += 2) {
          const float v0 = (outv[i][e] * cs[e] + bs[e]) * tw;
          const float v1 = (outv[i][e + 1] * cs[e + 1] + bs[e + 1]) * tw;
          packed[i][e / 2] =
              (uint32_t)Pair<T>::from_float(v0) | ((uint32_t)Pair<T>::from_float(v1) << 16);
        }
      }
    }
    auto blk_mine = [&](int i) {
      return do_store && i * 8 + o_row < p.m && (ksplit == 1 || (uint32_t)i % ksplit == krank);
    };
    if (p.ar.world == 0) {
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        if (!blk_mine(i)) continue;
        long long out_row = i * 8 + o_row;
        if constexpr (MOE) {
          out_row = moe_ids[i * 8 + o_row];      // output row = the sorted id; padding writes nothing
          if (out_row >= p.moe_rows) continue;
        }
        uint16_t* dst = static_cast<uint16_t*>(p.c) + (size_t)out_row * p.n + n_base;
        if constexpr (Cfg::kEpt == 4)
          *reinterpret_cast<uint2*>(dst) = make_uint2(packed[i][0], packed[i][1]);
        else
          *reinterpret_cast<uint32_t*>(dst) = packed[i][0];
      }
    } else {
      // All-reduce over the peer link (protocol in ar_link.cuh): the rounded partial of
      // this rank goes to every peer as flagged packets, each thread then collects the
      // peers' packets for its own elements and sums in rank order.
      const ArLink& l = p.ar;
      const uint32_t call = ar_ld_volatile(l.state);
      const uint32_t flag = ar_flag(call);
      const long long parity_off = (long long)(call & 1) * l.world * l.slot_bytes;
      for (int r = 0; r < l.world; ++r) {
        if (r == l.rank) continue;
        char* slot = static_cast<char*>(l.bufs[r]) + parity_off + l.rank * l.slot_bytes;
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          if (!blk_mine(i)) continue;
          char* dst = slot + ((size_t)(i * 8 + o_row) * p.n + n_base) * 4;  // 2 values per 8 B
          if constexpr (Cfg::kEpt == 4)
            ar_put2(dst, packed[i][0], packed[i][1], flag);
          else
            ar_put1(dst, packed[i][0], flag);
        }
      }
      const char* mybuf = static_cast<const char*>(l.bufs[l.rank]) + parity_off;
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        if (!blk_mine(i)) continue;
        const size_t el = (size_t)(i * 8 + o_row) * p.n + n_base;
        uint32_t d[kArMaxWorld][Cfg::kEpt / 2];
        if (!ar_collect<Cfg::kEpt / 2>(l, mybuf, el * 4, flag, d)) break;
        float sum[Cfg::kEpt];
#pragma unroll
        for (int e = 0; e < Cfg::kEpt; ++e) sum[e] = 0.f;
#pragma unroll
        for (int r = 0; r < kArMaxWorld; ++r) {
          if (r < l.world) {
#pragma unroll
            for (int e = 0; e < Cfg::kEpt / 2; ++e) {
              const uint32_t v = (r == l.rank) ? packed[i][e] : d[r][e];
              sum[2 * e] += Pair<T>::to_float((uint16_t)(v & 0xffffu));
              sum[2 * e + 1] += Pair<T>::to_float((uint16_t)(v >> 16));
            }
          }
        }
        uint32_t o[2];
#pragma unroll
        for (int e = 0; e < Cfg::kEpt / 2; ++e)
          o[e] = (uint32_t)Pair<T>::from_float(sum[2 * e]) |
                 ((uint32_t)Pair<T>::from_float(sum[2 * e + 1]) << 16);
        uint16_t* dst = static_cast<uint16_t*>(p.c) + el;
        if constexpr (Cfg::kEpt == 4)
          *reinterpret_cast<uint2*>(dst) = make_uint2(o[0], o[1]);
        else
          *reinterpret_cast<uint32_t*>(dst) = o[0];
      }
      __syncthreads();
      if (threadIdx.x == 0) ar_arrive(l, call, gridDim.x);
    }
  }
}

// Host launcher for one (type, bits, zp, group mode, MT, NTW) variant.
template <typename T, int BITS, bool HAS_ZP, int GM, int MT, int NTW, bool MOE = false>
int launch_stream(StreamParams p, int max_ctas, cudaStream_t stream) {
  using Cfg = StreamCfg<BITS, HAS_ZP, GM, MT, NTW>;
  using E = Emb<T, BITS>;
  // accumulator registers: acc (+ grp when grouped)
  constexpr int kAccRegs = MT * NTW * 16 * (GM == kGrouped ? 2 : 1);
  constexpr int kMinBlocks = (kAccRegs <= 64 && MT <= 2 && Cfg::kSmemBytes <= 112 * 1024) ? 2 : 1;
  auto kernel = gemm_stream_kernel<T, BITS, HAS_ZP, GM, MT, NTW, kMinBlocks, MOE>;
  static bool attr_done[64] = {};  // per device; benign race: the call is idempotent
  int dev = 0;
  B200Q_CUDA_OK(cudaGetDevice(&dev));
  if (!attr_done[dev & 63]) {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::kSmemBytes));
    attr_done[dev & 63] = true;
  }
  p.c_ex = E::kEx;
  p.c_mask_lo = E::kMaskLo;
  p.c_mask_hi = E::kMaskHi;
  // K is split over a cluster of 1, 2, 4 or 8 CTAs: enough to fill the GPU, at
  // least 8 k-tiles (one per warp) each
  const int target = device_sm_count() * kMinBlocks;
  int ksplit = 1;
  const int blocks = MOE ? p.moe_blocks : 1;
  while (ksplit < 8 && p.slices * blocks * ksplit * 2 <= target && p.kt_total / (ksplit * 2) >= 8) ksplit *= 2;
  (void)max_ctas;
  const int grid = p.slices * ksplit;
  // programmatic dependent launch: the kernel may start while its predecessor in
  // the stream drains; it orders itself with griddepcontrol.wait
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, blocks);
  cfg.blockDim = dim3(kStreamThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, p));
  note_launch();
  B200Q_CUDA_OK(cudaGetLastError());
  return B200Q_OK;
}

}  // namespace b200q
