// Decode-regime GEMM, reference-order arithmetic: weights are dequantised to
// 16-bit and multiplied by their scale before the MMA.  This is the general
// path; it is used for act-order layers that hold a partial K range, where the
// scale group of every row comes from g_idx (group lookup) and so cannot be
// factored out of the MMA, for float zero-points (HQQ), and for 33..64-row
// launches the tensor-core kernel cannot take.  The grouped / channel-wise
// decode cases run the faster kernel of gemm_stream.cuh.
//
// Work decomposition: the (column slice, k-tile) space is cut into equal stripes,
// one per CTA; a CTA whose stripe covers part of a slice leaves fp32 partial sums
// in the scratch and the last CTA to arrive at a slice (counter in the workspace,
// reset on the way out) adds them up and writes C.
#pragma once

#include <type_traits>

#include "gemm_params.cuh"

namespace b200q {

// ZPF: the zero-points are 16-bit floats [G, N] in the scales' layout (HQQ) instead of packed codes.
template <int BITS, bool HAS_ZP, int GM, int MB, int NTW, bool ZPF = false>
struct LookupCfg {
  static constexpr int kTileBytes = 16 * 64 * BITS / 8;                  // one weight tile
  static constexpr int kWOff = 0;
  static constexpr int kAOff = kWOff + NTW * kTileBytes;                 // MB x 512 B
  static constexpr int kSOff = kAOff + MB * 512;                         // NTW x 128 B scales
  static constexpr int kZOff = kSOff + (GM == kGrouped ? NTW * 128 : 0); // NTW x (32|64) B zeros
  static constexpr int kZBytes = ZPF ? NTW * 128 : (HAS_ZP ? NTW * 8 * BITS : 0);
  static constexpr int kStageBytes = (kZOff + kZBytes + 127) / 128 * 128;
  // ring depth: as deep as ~96 KB of shared memory per CTA allows, 3..8 stages
  static constexpr int kDepthFit = 96 * 1024 / (kStageBytes * kStreamWarps);
  static constexpr int kDepth = kDepthFit > 8 ? 8 : (kDepthFit < 3 ? 3 : kDepthFit);
  static constexpr int kRingBytes = kStageBytes * kDepth * kStreamWarps;
  // reduction buffer: one 16-row block of every warp's accumulators
  static constexpr int kRedStride = 64 * NTW + 8;  // floats; +8 keeps float2 stores conflict-free
  static constexpr int kRedBytes = kStreamWarps * 16 * kRedStride * 4;
  static constexpr int kSmemBytes = kRingBytes > kRedBytes ? kRingBytes : kRedBytes;
  static constexpr int kEpt = 4 * NTW;  // output elements per thread per 16-row block
  static constexpr int kSlotFloats = MB * 16 * 64 * NTW;
};

// FP8: the 8-bit codes are float8_e4m3fn values; the scales carry the exponent re-bias factor
// (2^8 for fp16, 2^120 for bf16), as the reference's host code prepares them.
// FP4: the 4-bit codes are float4_e2m1f values (sign, two exponent bits, one mantissa bit); the
// scales are bytes in the regrouped layout of the reference's host code (a lane's eight scales of
// both groups of a pair are 16 adjacent bytes).  NVFP4 (p.w_fp4 = 1): the exponent field is moved
// into the 16-bit format without re-biasing and the scale bytes expand to s * 2^7; the global
// scale, applied to the fp32 sums, carries the two corrections (dequant.h:398-414, 470-499,
// marlin_template.h:1180-1188, 1500-1502).  MXFP4 (2): the weights are re-biased exactly and the
// scale bytes are bf16 exponent fields (dequant.h:452-468, 501-513).
// MOE: the mixture-of-experts form (csrc/moe/marlin_moe_wna16/marlin_template.h:374-530, 585-590,
// 920-930, 1500-1550): the rows of A are gathered through blocks of p.m sorted ids
// (row = id / top_k, ids >= moe_rows are padding), block b multiplies with the weights of expert
// expert_ids[b] (-1: skipped), output row = id, optionally scaled by topk_weights[id].  A work
// unit is (block, column slice) over the whole K: no partial sums cross CTAs.
template <typename T, int BITS, bool HAS_ZP, int GM, int MB, int NTW, int MINB, bool ZPF = false,
          bool FP8 = false, bool FP4 = false, bool MOE = false>
__global__ void __launch_bounds__(kStreamThreads, MINB) gemm_lookup_kernel(const StreamParams p) {
  static_assert(!MOE || (!ZPF && !FP8 && !FP4 && GM != kLookup), "moe: integer weight types");
  static_assert(!FP4 || (BITS == 4 && !HAS_ZP && GM == kGrouped && !FP8), "fp4 weights: grouped scales");
  static_assert(!ZPF || (HAS_ZP && GM == kGrouped), "float zero-points come with grouped scales");
  static_assert(!FP8 || (BITS == 8 && !HAS_ZP && GM != kLookup), "fp8 weights: 8 bits, no zero-points");
  using Cfg = LookupCfg<BITS, HAS_ZP, GM, MB, NTW, ZPF>;
  constexpr int D = Cfg::kDepth;
  static_assert(D >= 2, "ring too shallow");
  extern __shared__ __align__(128) unsigned char smem[];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int c8 = lane >> 2;  // column inside an 8-wide block
  const int KT = p.kt_total;
  const int NT = p.n / 64;
  const uint16_t* __restrict__ A = static_cast<const uint16_t*>(p.a);
  const uint16_t* __restrict__ S = static_cast<const uint16_t*>(p.scales);
  const uint4* __restrict__ Bw = reinterpret_cast<const uint4*>(p.b);
  const uint32_t* __restrict__ Zp = p.zeros;
  const uint16_t* __restrict__ Bias = static_cast<const uint16_t*>(p.bias);

  const long long n_slices = MOE ? (long long)p.moe_blocks * p.slices : p.slices;
  const long long total = n_slices * KT;
  // moe: whole (block, slice) units per CTA
  const long long u_begin = MOE ? n_slices * blockIdx.x / gridDim.x * KT : total * blockIdx.x / gridDim.x;
  const long long u_end = MOE ? n_slices * (blockIdx.x + 1) / gridDim.x * KT
                              : total * (blockIdx.x + 1) / gridDim.x;

  const uint32_t ring = smem_u32(smem) + warp * (D * Cfg::kStageBytes);
  float* red = reinterpret_cast<float*>(smem);
  __shared__ int s_is_last;

  for (long long u = u_begin; u < u_end;) {
    const int slice = (int)(u / KT);
    const int kt0 = (int)(u % KT);
    const int kt1 = (int)min((long long)KT, kt0 + (u_end - u));
    u += kt1 - kt0;
    int moe_block = 0;
    int a_row[MB];   // moe: source row of A for each 16-row block's row this lane stages, -1 = none
    (void)a_row;
    if (MOE) {
      moe_block = slice / p.slices;
      if (moe_block * p.m >= *p.moe_num_padded) continue;
      const int expert = p.moe_expert_ids[moe_block];
      if (expert < 0) continue;
      Bw = reinterpret_cast<const uint4*>(p.b + (size_t)expert * p.moe_b_stride);
      S = static_cast<const uint16_t*>(p.scales) + (size_t)expert * p.moe_s_stride;
      if (HAS_ZP) Zp = p.zeros + (size_t)expert * p.moe_z_stride;
      if (p.bias) Bias = static_cast<const uint16_t*>(p.bias) + (size_t)expert * p.moe_bias_stride;
#pragma unroll
      for (int i = 0; i < MB; ++i) {
        const int row = i * 16 + (lane >> 1);
        const int id = row < p.m ? p.moe_sorted_ids[moe_block * p.m + row] : p.moe_rows;
        a_row[i] = id < p.moe_rows ? id / p.moe_top_k : -1;
      }
    }
    const int nt0 = (MOE ? slice % p.slices : slice) * NTW;  // first 64-column tile of the slice

    // this warp's contiguous share of [kt0, kt1)
    const int len = kt1 - kt0;
    const int wb = kt0 + (int)((long long)len * warp / kStreamWarps);
    const int we = kt0 + (int)((long long)len * (warp + 1) / kStreamWarps);

    float acc[MB][NTW][8][4];
#pragma unroll
    for (int i = 0; i < MB; ++i)
#pragma unroll
      for (int j = 0; j < NTW; ++j)
#pragma unroll
        for (int b = 0; b < 8; ++b)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[i][j][b][e] = 0.f;

    // ---- producer: one ring stage = weights + A tile (+ scales, zeros) of one k-tile
    // scales (kGrouped) and zero-points ride in the stage of the first k-tile
    // of a group, and of the warp's first k-tile
    auto has_scales = [&](int kt) {
      return (GM == kGrouped || HAS_ZP) && (kt == wb || kt % p.group_blocks == 0);
    };
    auto issue = [&](int kt, int stage) {
      const uint32_t st = ring + stage * Cfg::kStageBytes;
      if (kt < we) {
        const uint4* wsrc = Bw + ((size_t)kt * NT + nt0) * (Cfg::kTileBytes / 16);
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          if (BITS == 4) {
            cp_async16(st + Cfg::kWOff + j * 512 + lane * 16, wsrc + j * 32 + lane);
          } else {
            // chunk ch of the tile belongs to lane ch/2, half ch%2
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int ch = lane + 32 * h;
              cp_async16(st + Cfg::kWOff + j * 1024 + (ch & 1) * 512 + (ch >> 1) * 16,
                         wsrc + j * 64 + ch);
            }
          }
        }
        {
          const int r = lane >> 1, h = lane & 1;
          const int pos = 2 * r + (h ^ ((r >> 2) & 1));
#pragma unroll
          for (int i = 0; i < MB; ++i) {
            const int row = MOE ? a_row[i] : i * 16 + r;
            const bool ok = MOE ? row >= 0 : row < p.m;
            const uint16_t* src = A + (size_t)(ok ? row : 0) * p.lda + kt * 16 + h * 8;
            cp_async16(st + Cfg::kAOff + i * 512 + pos * 16, src, ok ? 16 : 0);
          }
        }
        if (has_scales(kt)) {
          const int g = kt / p.group_blocks;
          if (GM == kGrouped && !FP4 && lane < NTW * 8)
            cp_async16(st + Cfg::kSOff + lane * 16, S + (size_t)g * p.n + nt0 * 64 + lane * 8);
          if (ZPF) {
            if (lane < NTW * 8)
              cp_async16(st + Cfg::kZOff + lane * 16,
                         reinterpret_cast<const uint16_t*>(p.zeros) + (size_t)g * p.n + nt0 * 64 +
                             lane * 8);
          } else if (HAS_ZP) {
            constexpr int kChunks = NTW * 8 * BITS / 16;  // 16 B chunks of zero-point words
            if (lane < kChunks)
              cp_async16(st + Cfg::kZOff + lane * 16,
                         Zp + (size_t)g * (p.n * BITS / 32) + nt0 * (2 * BITS) + lane * 4);
          }
        }
      }
      cp_async_commit();
    };

    // scale / zero-point state carried across k-tiles of a group
    uint32_t sdup[NTW][8];
    uint32_t zdup[NTW][8];
    (void)sdup;
    (void)zdup;

    auto load_group_from_stage = [&](uint32_t st, int kt) {
#pragma unroll
      for (int j = 0; j < NTW; ++j) {
        if (FP4) {
          // this lane's eight scale bytes of the group: byte 4 (sub / 2) + 2 h + sub % 2 belongs
          // to column 16 sub + c8 + 8 h of the tile
          const int g = kt / p.group_blocks;
          const unsigned char* src = reinterpret_cast<const unsigned char*>(p.scales) +
                                     (size_t)(g & ~1) * p.n + 16 * (8 * (nt0 + j) + c8) + 8 * (g & 1);
          const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src));
          const uint32_t word[2] = {raw.x, raw.y};
#pragma unroll
          for (int sub = 0; sub < 4; ++sub)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t b = (word[sub >> 1] >> (8 * (2 * h + (sub & 1)))) & 0xffu;
              uint32_t v;
              if (p.w_fp4 == 2) v = b << 7;                                         // e8m0 -> bf16 exponent
              else if (std::is_same<T, half>::value) v = b << 7;                    // S0E5M3 -> fp16 bits 14..7
              else v = ((b & 0x80u) << 7) | ((b & 0x7fu) << 4);                     // -> bf16: top bit, then 7 bits
              sdup[j][2 * sub + h] = v | (v << 16);
            }
        } else if (GM == kGrouped) {
          const uint4 s4 = lds128(st + Cfg::kSOff + j * 128 + c8 * 16);
          const uint32_t sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            sdup[j][2 * sub] = dup_lo(sv[sub]);
            sdup[j][2 * sub + 1] = dup_hi(sv[sub]);
          }
        }
        if (ZPF) {
          // -(zero-point * scale), rounded once like the reference's __hmul2
          // (marlin_template.h:1235-1240); the weights then take one fma each
          const uint4 z4 = lds128(st + Cfg::kZOff + j * 128 + c8 * 16);
          const uint32_t zv[4] = {z4.x, z4.y, z4.z, z4.w};
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            zdup[j][2 * sub] = Pair<T>::mul(dup_lo(zv[sub]), sdup[j][2 * sub]) ^ 0x80008000u;
            zdup[j][2 * sub + 1] = Pair<T>::mul(dup_hi(zv[sub]), sdup[j][2 * sub + 1]) ^ 0x80008000u;
          }
        } else if (HAS_ZP) {
          uint32_t zp[4];
          if (BITS == 4) {
            dequant4<T, false>(lds32(st + Cfg::kZOff + j * 32 + c8 * 4), zp);
          } else {
            uint32_t t0[2], t1[2];
            dequant8<T, false>(lds32(st + Cfg::kZOff + j * 64 + c8 * 8), t0);
            dequant8<T, false>(lds32(st + Cfg::kZOff + j * 64 + c8 * 8 + 4), t1);
            zp[0] = t0[0]; zp[1] = t0[1]; zp[2] = t1[0]; zp[3] = t1[1];
          }
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            zdup[j][2 * sub] = dup_lo(zp[sub]);
            zdup[j][2 * sub + 1] = dup_hi(zp[sub]);
          }
        }
      }
    };

    // kLookup: group of every row this lane touches, straight from global memory
    auto load_group_lookup = [&](int kt, int j, uint32_t (&s_rows)[4][4]) {
      const int q = lane & 3;
      const int rows[4] = {2 * q, 2 * q + 1, 2 * q + 8, 2 * q + 9};
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int g = p.g_idx[kt * 16 + rows[r]];
        const uint4 s4 = *reinterpret_cast<const uint4*>(S + (size_t)g * p.n + (nt0 + j) * 64 + c8 * 8);
        s_rows[r][0] = s4.x; s_rows[r][1] = s4.y; s_rows[r][2] = s4.z; s_rows[r][3] = s4.w;
      }
    };

#pragma unroll
    for (int s = 0; s < D - 1; ++s) issue(wb + s, s);

    for (int kt = wb; kt < we; ++kt) {
      const int stage = (kt - wb) % D;
      cp_async_wait<D - 2>();
      __syncwarp();
      issue(kt + D - 1, (kt - wb + D - 1) % D);
      const uint32_t st = ring + stage * Cfg::kStageBytes;

      if (has_scales(kt)) load_group_from_stage(st, kt);

      uint32_t afrag[MB][4];
      {
        const int r = (lane & 7) + 8 * ((lane >> 3) & 1), h = lane >> 4;
        const int pos = 2 * r + (h ^ ((r >> 2) & 1));
#pragma unroll
        for (int i = 0; i < MB; ++i) ldmatrix_x4(afrag[i], st + Cfg::kAOff + i * 512 + pos * 16);
      }

#pragma unroll
      for (int j = 0; j < NTW; ++j) {
        uint32_t s_rows[4][4];
        (void)s_rows;
        if (GM == kLookup) load_group_lookup(kt, j, s_rows);

        uint32_t w[BITS == 4 ? 4 : 8];
        {
          const uint4 w4 = lds128(st + Cfg::kWOff + j * Cfg::kTileBytes + lane * 16);
          w[0] = w4.x; w[1] = w4.y; w[2] = w4.z; w[3] = w4.w;
          if (BITS == 8) {
            const uint4 w5 = lds128(st + Cfg::kWOff + j * Cfg::kTileBytes + 512 + lane * 16);
            w[4] = w5.x; w[5] = w5.y; w[6] = w5.z; w[7] = w5.w;
          }
        }
#pragma unroll
        for (int sub = 0; sub < 4; ++sub) {
          uint32_t f[4];  // block 0: f[0] rows lo, f[1] rows hi; block 1: f[2], f[3]
          if (FP4) {
            // nibble i of the word sits where the uint4 codes do: f[i] takes nibbles i and i + 4
            constexpr int kShift = std::is_same<T, half>::value ? 3 : 6;
            const uint32_t q = w[sub];
            auto conv = [](uint32_t x) { return (x & 0x80008000u) | ((x & 0x70007000u) >> kShift); };
            f[3] = conv(q);
            f[2] = conv(q << 4);
            f[1] = conv(q << 8);
            f[0] = conv(q << 12);
            if (p.w_fp4 == 2) {
              // exact re-bias: 2^126 as a bfloat16 pair
#pragma unroll
              for (int e = 0; e < 4; ++e) f[e] = Pair<T>::mul(f[e], 0x7e807e80u);
            }
          } else if (BITS == 4) {
            dequant4<T, !HAS_ZP>(w[sub], f);
          } else {
            uint32_t t0[2], t1[2];
            if (FP8) {
              dequant_fp8<T>(w[2 * sub], t0);
              dequant_fp8<T>(w[2 * sub + 1], t1);
              if (GM == kChannel) {
                // bring the values to their true magnitude before the MMA (exact); the
                // channel scale gives the factor back in the epilogue
                t0[0] = Pair<T>::mul(t0[0], Fp8Cvt<T>::kRebias);
                t0[1] = Pair<T>::mul(t0[1], Fp8Cvt<T>::kRebias);
                t1[0] = Pair<T>::mul(t1[0], Fp8Cvt<T>::kRebias);
                t1[1] = Pair<T>::mul(t1[1], Fp8Cvt<T>::kRebias);
              }
            } else {
              dequant8<T, !HAS_ZP>(w[2 * sub], t0);
              dequant8<T, !HAS_ZP>(w[2 * sub + 1], t1);
            }
            f[0] = t0[0]; f[1] = t0[1]; f[2] = t1[0]; f[3] = t1[1];
          }
          if (ZPF) {
            // q * s - zp * s (scale_and_sub, marlin_template.h:174-181)
            f[0] = Pair<T>::fma(f[0], sdup[j][2 * sub], zdup[j][2 * sub]);
            f[1] = Pair<T>::fma(f[1], sdup[j][2 * sub], zdup[j][2 * sub]);
            f[2] = Pair<T>::fma(f[2], sdup[j][2 * sub + 1], zdup[j][2 * sub + 1]);
            f[3] = Pair<T>::fma(f[3], sdup[j][2 * sub + 1], zdup[j][2 * sub + 1]);
          } else if (HAS_ZP) {
            f[0] = Pair<T>::sub(f[0], zdup[j][2 * sub]);
            f[1] = Pair<T>::sub(f[1], zdup[j][2 * sub]);
            f[2] = Pair<T>::sub(f[2], zdup[j][2 * sub + 1]);
            f[3] = Pair<T>::sub(f[3], zdup[j][2 * sub + 1]);
          }
          if (ZPF) {
            // scaled by the fma above
          } else if (GM == kGrouped) {
            f[0] = Pair<T>::mul(f[0], sdup[j][2 * sub]);
            f[1] = Pair<T>::mul(f[1], sdup[j][2 * sub]);
            f[2] = Pair<T>::mul(f[2], sdup[j][2 * sub + 1]);
            f[3] = Pair<T>::mul(f[3], sdup[j][2 * sub + 1]);
          } else if (GM == kLookup) {
            // pair (row lo, row lo+1) of block 0 uses scale word `sub` low halves
            // of those two rows; block 1 the high halves
            const uint32_t s00 = __byte_perm(s_rows[0][sub], s_rows[1][sub], 0x5410);
            const uint32_t s01 = __byte_perm(s_rows[2][sub], s_rows[3][sub], 0x5410);
            const uint32_t s10 = __byte_perm(s_rows[0][sub], s_rows[1][sub], 0x7632);
            const uint32_t s11 = __byte_perm(s_rows[2][sub], s_rows[3][sub], 0x7632);
            f[0] = Pair<T>::mul(f[0], s00);
            f[1] = Pair<T>::mul(f[1], s01);
            f[2] = Pair<T>::mul(f[2], s10);
            f[3] = Pair<T>::mul(f[3], s11);
          }
#pragma unroll
          for (int i = 0; i < MB; ++i) {
            mma16816<T>(acc[i][j][2 * sub], afrag[i], f[0], f[1]);
            mma16816<T>(acc[i][j][2 * sub + 1], afrag[i], f[2], f[3]);
          }
        }
      }
    }
    cp_async_wait<0>();

    // ---- intra-CTA reduction, one 16-row block at a time -------------------------
    const long long s_first_u = (long long)slice * KT;
    const int first_cta = (int)(((s_first_u + 1) * gridDim.x - 1) / total);
    const int last_cta = (int)(((s_first_u + KT) * gridDim.x - 1) / total);
    const bool split = !MOE && first_cta != last_cta;

    float outv[MB][Cfg::kEpt];
    const int o_row = threadIdx.x >> 4;                // 0..15
    const int o_col = (threadIdx.x & 15) * Cfg::kEpt;  // inside the slice
#pragma unroll
    for (int i = 0; i < MB; ++i) {
      __syncthreads();  // ring (or previous block's sums) no longer in use
      {
        float* mine = red + warp * (16 * Cfg::kRedStride);
        const int q = lane & 3;
#pragma unroll
        for (int j = 0; j < NTW; ++j)
#pragma unroll
          for (int b = 0; b < 8; ++b) {
            const int col = j * 64 + b * 8 + 2 * q;
            *reinterpret_cast<float2*>(mine + c8 * Cfg::kRedStride + col) =
                make_float2(acc[i][j][b][0], acc[i][j][b][1]);
            *reinterpret_cast<float2*>(mine + (c8 + 8) * Cfg::kRedStride + col) =
                make_float2(acc[i][j][b][2], acc[i][j][b][3]);
          }
      }
      __syncthreads();
#pragma unroll
      for (int e = 0; e < Cfg::kEpt; ++e) outv[i][e] = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < kStreamWarps; ++w8) {
        const float* src = red + w8 * (16 * Cfg::kRedStride) + o_row * Cfg::kRedStride + o_col;
#pragma unroll
        for (int e = 0; e < Cfg::kEpt; e += 4) {
          const float4 v = *reinterpret_cast<const float4*>(src + e);
          outv[i][e] += v.x; outv[i][e + 1] += v.y; outv[i][e + 2] += v.z; outv[i][e + 3] += v.w;
        }
      }
    }

    // ---- cross-CTA reduction for split slices --------------------------------------
    bool do_store = true;
    if (split) {
      float* slot = p.partials + (size_t)(blockIdx.x + slice) * Cfg::kSlotFloats;
#pragma unroll
      for (int i = 0; i < MB; ++i)
#pragma unroll
        for (int e = 0; e < Cfg::kEpt; e += 4)
          __stcg(reinterpret_cast<float4*>(slot + (i * 16 + o_row) * (64 * NTW) + o_col + e),
                 make_float4(outv[i][e], outv[i][e + 1], outv[i][e + 2], outv[i][e + 3]));
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const int prev = atomicAdd(p.counters + first_cta, 1);
        s_is_last = (prev == last_cta - first_cta);
      }
      __syncthreads();
      do_store = s_is_last != 0;
      if (do_store) {
        __threadfence();
#pragma unroll
        for (int i = 0; i < MB; ++i)
#pragma unroll
          for (int e = 0; e < Cfg::kEpt; ++e) outv[i][e] = 0.f;
        for (int cta = first_cta; cta <= last_cta; ++cta) {
          const float* src = p.partials + (size_t)(cta + slice) * Cfg::kSlotFloats;
#pragma unroll
          for (int i = 0; i < MB; ++i)
#pragma unroll
            for (int e = 0; e < Cfg::kEpt; e += 4) {
              const float4 v = __ldcg(
                  reinterpret_cast<const float4*>(src + (i * 16 + o_row) * (64 * NTW) + o_col + e));
              outv[i][e] += v.x; outv[i][e + 1] += v.y; outv[i][e + 2] += v.z; outv[i][e + 3] += v.w;
            }
        }
        if (threadIdx.x == 0) p.counters[first_cta] = 0;
      }
    }

    // ---- epilogue: channel scale, bias, convert, store -----------------------------
    if (do_store) {
      const int n_base = nt0 * 64 + o_col;
      float cs[Cfg::kEpt], bs[Cfg::kEpt];
#pragma unroll
      for (int e = 0; e < Cfg::kEpt; ++e) {
        cs[e] = (GM == kChannel) ? Pair<T>::to_float(S[single_perm_pos(n_base + e)]) : 1.f;
        if (FP8 && GM == kChannel) cs[e] *= Fp8Cvt<T>::kRebiasInv;
        if (FP4 && p.w_fp4 == 1) cs[e] = Pair<T>::to_float(*static_cast<const uint16_t*>(p.global_scale));
        bs[e] = p.bias ? Pair<T>::to_float(Bias[single_perm_pos(n_base + e)]) : 0.f;
      }
      uint16_t* C = static_cast<uint16_t*>(p.c);
#pragma unroll
      for (int i = 0; i < MB; ++i) {
        int row = i * 16 + o_row;
        bool live = row < p.m;
        float tw = 1.f;
        if (MOE) {
          // output row = the sorted id itself; padding ids write nothing
          const int id = live ? p.moe_sorted_ids[moe_block * p.m + row] : p.moe_rows;
          live = id < p.moe_rows;
          row = id;
          if (live && p.moe_topk_weights) tw = p.moe_topk_weights[id];
        }
        if (live) {
          uint32_t packed[Cfg::kEpt / 2];
#pragma unroll
          for (int e = 0; e < Cfg::kEpt; e += 2) {
            const float v0 = (outv[i][e] * cs[e] + bs[e]) * tw;
            const float v1 = (outv[i][e + 1] * cs[e + 1] + bs[e + 1]) * tw;
            packed[e / 2] = (uint32_t)Pair<T>::from_float(v0) | ((uint32_t)Pair<T>::from_float(v1) << 16);
          }
          uint16_t* dst = C + (size_t)row * p.n + n_base;
          if (Cfg::kEpt == 8)
            *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          else
            *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
        }
      }
    }
    __syncthreads();  // reduction buffer is reused as the ring of the next piece
  }
}

// Host launcher for one (type, bits, zp, group mode, MB, NTW) variant.
template <typename T, int BITS, bool HAS_ZP, int GM, int MB, int NTW, bool ZPF = false, bool FP8 = false,
          bool FP4 = false, bool MOE = false>
int launch_lookup(const StreamParams& p, int max_ctas, cudaStream_t stream) {
  using Cfg = LookupCfg<BITS, HAS_ZP, GM, MB, NTW, ZPF>;
  constexpr int kMinBlocks = (MB * NTW <= 2 && Cfg::kSmemBytes <= 112 * 1024) ? 2 : 1;
  auto kernel = gemm_lookup_kernel<T, BITS, HAS_ZP, GM, MB, NTW, kMinBlocks, ZPF, FP8, FP4, MOE>;
  static bool attr_done[64] = {};  // per device; benign race: the call is idempotent
  int dev = 0;
  B200Q_CUDA_OK(cudaGetDevice(&dev));
  if (!attr_done[dev & 63]) {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::kSmemBytes));
    attr_done[dev & 63] = true;
  }
  const long long total = (long long)p.slices * p.kt_total * (MOE ? p.moe_blocks : 1);
  long long want = (long long)device_sm_count() * kMinBlocks * (MOE ? 4 : 1);  // moe: many blocks are empty
  if (want > max_ctas) want = max_ctas;
  const long long by_work = (total + 15) / 16;  // at least 16 k-tiles per CTA
  int grid = (int)(want < by_work ? want : by_work);
  if (grid < 1) grid = 1;
  kernel<<<grid, kStreamThreads, Cfg::kSmemBytes, stream>>>(p);
  note_launch();
  B200Q_CUDA_OK(cudaGetLastError());
  return B200Q_OK;
}

}  // namespace b200q
