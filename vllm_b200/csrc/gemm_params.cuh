// Parameter block and constants shared by the decode-regime GEMM kernels.
#pragma once

#include "ar_link.cuh"
#include "common.cuh"

namespace b200q {

enum GroupMode : int {
  kChannel = 0,  // one scale per column, applied in fp32 in the epilogue
  kGrouped = 1,  // scale group = k / group_size
  kLookup = 2,   // scale group = g_idx[k] (act-order with a partial K range)
};

struct StreamParams {
  const void* a;           // [M, K] 16-bit, row stride lda
  int64_t lda;
  const uint32_t* b;       // Marlin layout
  const void* scales;      // [G, N] 16-bit, permuted
  const uint32_t* zeros;   // [G, N/pf] or null
  const int32_t* g_idx;    // [K] or null
  const void* bias;        // [N] permuted or null
  void* c;                 // [M, N]
  float* partials;         // scratch for split slices
  int32_t* counters;       // zero on entry / exit
  int m, n, k;
  int kt_total;            // K / 16
  int slices;              // N / (64 * NTW)
  int group_blocks;        // k-tiles per scale group (kGrouped)
  int num_groups;
  int zp_float;            // zeros holds 16-bit floats [G, N] in the scales' layout
  int w_fp8;               // the 8-bit codes are float8_e4m3fn values
  int w_fp4;               // the 4-bit codes are float4_e2m1f values; scales are bytes [G, N] in
                           // the regrouped layout: 1 = fp8 S0E5M3 (NVFP4), 2 = e8m0 (MXFP4)
  const void* global_scale;  // NVFP4: one 16-bit value (with the exponent corrections folded in)
  // mixture-of-experts form (moe_wna16_marlin_gemm): rows come in blocks of `m` sorted ids, a
  // block uses the weights of one expert; null / 0 otherwise
  const int32_t* moe_sorted_ids;   // [moe_blocks * m]: token * top_k + slot, >= moe_rows = padding
  const int32_t* moe_expert_ids;   // [moe_blocks]: expert of a block, -1 = not on this rank
  const int32_t* moe_num_padded;   // device scalar: sorted ids in use (a multiple of m)
  const float* moe_topk_weights;   // [moe_rows] or null: output row scale
  int moe_blocks, moe_rows, moe_top_k;
  long long moe_b_stride, moe_s_stride, moe_z_stride, moe_bias_stride;  // per expert: words / elements
  // weight-embedding constants of the streaming kernel (filled by its launcher)
  uint32_t c_ex, c_mask_lo, c_mask_hi;
  // when ar.world > 0 the streaming kernel all-reduces its output over the link
  ArLink ar;
};

constexpr int kStreamWarps = 8;
constexpr int kStreamThreads = kStreamWarps * 32;

}  // namespace b200q
