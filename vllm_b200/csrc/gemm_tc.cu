// Prefill-regime mixed-precision GEMM on the 5th-generation tensor cores:
// C[M,N] = A[M,K] * dequant(B) from 33 rows up, tcgen05.mma with TMEM accumulators.
//
// One persistent CTA per SM walks over BM x BN output tiles (BM, BN in {128,
// 256}; m fastest so that CTAs running together share weight tiles).  The k
// loop advances 64 at a time through a ring of shared-memory stages:
//
//   producer warp   TMA (cp.async.bulk.tensor.2d, 128B swizzle, no multicast)
//                   brings the A tile [BM x 64]; 1-D bulk copies bring the packed
//                   weights of the stage (Marlin tiles are contiguous) and the
//                   scale / zero-point rows of the groups the stage touches;
//   16 dequant warps (each a quarter of the columns of one k-tile) read the packed words, convert them exactly to 16-bit
//                   (mantissa embedding), subtract the bias or zero-point,
//                   multiply by the group scale (one 16-bit rounding, the same
//                   point at which the reference rounds) and store the
//                   [BN x 64] K-major, 128B-swizzled B operand;
//   MMA warp        one thread issues tcgen05.mma.kind::f16 (128 x BN x 16,
//                   four per stage and 128-row accumulator) into TMEM and
//                   commits the stage back to the producer;
//   4 epilogue warps tcgen05.ld the finished accumulator, add bias, convert and
//                   store C; when two accumulator sets fit in TMEM (all but
//                   256 x 256) the MMA warp meanwhile fills the other one.
//
// Problems with fewer tiles than SMs split K: a work item is (tile, share of the k
// range), items leave fp32 partials in the caller's scratch and splitk_reduce_kernel
// adds them in split order (plan_tiles picks tile shape and split from measured
// per-step times).
//
// All hand-offs are mbarriers.  Every wait is bounded: after kSpinLimit polls
// a role records an error code in g_tc_error, stops waiting and lets the
// kernel drain (TMEM is still freed), so a broken hand-off can not hang the GPU.
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "gemm_params.cuh"

namespace b200q {

int launch_permute_cols(const void* a, int64_t lda, const int32_t* perm, void* out, int64_t size_m,
                        int64_t size_k, cudaStream_t stream);

namespace tc {

constexpr int kBK = 64;           // k per stage: one 128-byte swizzle row of 16-bit values
constexpr int kDequantWarps = 16;  // k-tile of the stage = warp % 4, column quarter = warp / 4
constexpr int kEpiWarp0 = kDequantWarps;           // 4 warps: TMEM lane quadrant = warp % 4
constexpr int kProducerWarp = kEpiWarp0 + 4;
constexpr int kMmaWarp = kProducerWarp + 1;
constexpr int kThreads = 32 * (kMmaWarp + 1);
constexpr int64_t kMaxSplitBytes = 64ll << 20;  // cap on the fp32 partials of a k-split
constexpr uint32_t kSpinLimit = 1u << 24;   // polls (try_wait without a suspend-time hint: a waiter
                                            // given a 1 us hint was seen to sleep the hint out)

// 0 = ok; else (role << 8) | barrier id of the first wait that ever timed out (sticky, for the
// host to read).  Roles of the same CTA tell each other to stop through a shared-memory flag.
__device__ int g_tc_error;

struct TcParams {
  const uint32_t* b;      // Marlin layout
  const void* scales;     // [G, N] permuted
  const uint32_t* zeros;  // [G, N/pf] or null
  const void* bias;       // [N] permuted or null
  void* c;                // [M, N]
  int m, n, k;
  int group_blocks;       // k-tiles (16 rows) per scale group; K/16 when there is one group
  int channelwise;        // scales use the 32-column "single" permutation
  // split-K: a tile's k-range is shared by `ksplit` work items; each leaves fp32 partial
  // sums in `partials`, which splitk_reduce_kernel adds up in split order afterwards
  int ksplit;
  float* partials;        // [tiles * ksplit][BM][BN] fp32
};

// ---- PTX wrappers ------------------------------------------------------------------
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
// Bounded wait on a phase parity.  Returns false (and records `what`) on time-out.
// SLEEP_NS > 0: back off between polls, so that roles with long waits (epilogue, producer) do
// not take issue slots from the dequant warps.
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int what,
                                          volatile int* cta_abort) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
    // now and then: stop early if another role of this CTA has already given up
    if ((spin & 1023u) == 1023u && *cta_abort != 0) return false;
  }
  *cta_abort = 1;
  atomicCAS(&g_tc_error, 0, what);
  return false;
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem], 128 x 128 x 16, 16-bit inputs, fp32 accumulate
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on an mbarrier when all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::
                   "r"(bar)
               : "memory");
}
// 32 lanes x 32 consecutive fp32 columns of TMEM -> 32 registers per thread
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
      "%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// st.shared / ld.shared with a compile-time byte offset folded into the instruction
template <int OFF>
__device__ __forceinline__ void sts32_off(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0+%2], %1;\n" ::"r"(addr), "r"(v), "n"(OFF) : "memory");
}
template <int OFF>
__device__ __forceinline__ uint32_t lds32_off(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 B
// apart, 8-row atoms 1024 B apart (version 1 = sm_100 format).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
         (2ull << 61);
}

template <int BM, int BN, int BITS>
struct TcCfg {
  static constexpr int kNT = BN / 64;                      // 64-column Marlin tiles per tile
  static constexpr int kABytes = BM * 128;
  static constexpr int kBBytes = BN * 128;
  static constexpr int kTileBytes = 16 * 64 * BITS / 8;    // one packed 16 x 64 weight tile
  static constexpr int kWBytes = 4 * kNT * kTileBytes;     // 4 k-tiles x kNT column tiles
  // the weights of a stage arrive as 2-D copies of at most 256 8-byte elements per row
  static constexpr int kCopyTiles = (kNT * kTileBytes / 8 <= 256) ? kNT : 256 * 8 / kTileBytes;
  static constexpr int kCopies = kNT / kCopyTiles;
  static constexpr int kCopyRowBytes = kCopyTiles * kTileBytes;
  static constexpr int kSRow = BN * 2;                     // one group's scales for the tile
  static constexpr int kZRow = kNT * 8 * BITS;             // one group's packed zero-points
  static constexpr int kSOff = kABytes + kBBytes + kWBytes;
  static constexpr int kZOff = kSOff + 2 * kSRow;          // up to two groups per stage
  static constexpr int kStageBytes = (kZOff + 2 * kZRow + 1023) / 1024 * 1024;
  static constexpr int kStagesFit = (222 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesFit > 6 ? 6 : kStagesFit;
  static constexpr int kAccs = BM / 128;                   // 128-row accumulators per tile
  static constexpr int kBufs = (2 * kAccs * BN <= 512) ? 2 : 1;
  static constexpr int kTmemCols = (kBufs * kAccs * BN <= 256) ? 256 : 512;
  static constexpr int kBarBytes = 1024;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;  // + alignment slack
};

// instruction descriptor: fp32 accumulate, A and B K-major, M = 128, N = bn
template <typename T>
__device__ __forceinline__ uint32_t make_idesc(int bn);
template <>
__device__ __forceinline__ uint32_t make_idesc<half>(int bn) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(bn >> 3) << 17) | ((128u >> 4) << 24);
}
template <>
__device__ __forceinline__ uint32_t make_idesc<__nv_bfloat16>(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((128u >> 4) << 24);
}

template <typename T, int BITS, bool HAS_ZP, int BM, int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
               const TcParams p) {
  using Cfg = TcCfg<BM, BN, BITS>;
  constexpr int S = Cfg::kStages;
  constexpr int NTT = Cfg::kNT;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = smem_base + S * Cfg::kStageBytes;
  // barrier ids (8 bytes each)
  auto full_a = [&](int s) { return bars + 8 * s; };
  auto full_w = [&](int s) { return bars + 8 * (S + s); };
  auto full_b = [&](int s) { return bars + 8 * (2 * S + s); };
  auto empty = [&](int s) { return bars + 8 * (3 * S + s); };
  auto tmem_full = [&](int b) { return bars + 8 * (4 * S + b); };
  auto tmem_empty = [&](int b) { return bars + 8 * (4 * S + 2 + b); };
  const uint32_t tmem_slot = bars + 8 * (4 * S + 4);
  auto stage_a = [&](int s) { return smem_base + s * Cfg::kStageBytes; };
  auto stage_b = [&](int s) { return smem_base + s * Cfg::kStageBytes + Cfg::kABytes; };
  auto stage_w = [&](int s) { return smem_base + s * Cfg::kStageBytes + Cfg::kABytes + Cfg::kBBytes; };
  auto stage_s = [&](int s) { return smem_base + s * Cfg::kStageBytes + Cfg::kSOff; };
  auto stage_z = [&](int s) { return smem_base + s * Cfg::kStageBytes + Cfg::kZOff; };

  // a k-split's reduce kernel may be scheduled while this kernel runs (it waits for
  // this kernel's completion itself)
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  __shared__ int s_abort;
  volatile int* cta_abort = &s_abort;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (p.m + BM - 1) / BM;
  const int n_tiles = (p.n + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int kb_total = p.k / kBK;
  const int KS = p.ksplit;
  const int total_items = total_tiles * KS;  // work item = (tile, share of the k-range)
  const int NT = p.n / 64;  // 64-column Marlin tiles
  const int gb = p.group_blocks;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(full_a(s), 1);
      mbar_init(full_w(s), 1);
      mbar_init(full_b(s), kDequantWarps);
      mbar_init(empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full(b), 1);
      mbar_init(tmem_empty(b), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == kMmaWarp) tmem_alloc(tmem_slot, Cfg::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == kProducerWarp) {
    // ================= producer: TMA for A, bulk copies for weights / scales / zeros =====
    if (lane == 0) {
      uint32_t it = 0;
      int st_i = 0;
      uint32_t st_ph = 0;
      bool ok = true;
      // A comes from the kernel before this one in the stream (programmatic dependent launch:
      // this kernel's launch and set-up overlap that kernel's tail)
      asm volatile("griddepcontrol.wait;\n" ::: "memory");
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int t = item / KS, ks = item - t * KS;
        const int kb0 = (int)((long long)kb_total * ks / KS);
        const int kb1 = (int)((long long)kb_total * (ks + 1) / KS);
        const int tn = t / m_tiles, tm = t % m_tiles;
        const int nt0 = tn * NTT;
        const int nt_valid = min(NTT, NT - nt0);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = st_i;
          const uint32_t ph = st_ph;
          if (++st_i == S) { st_i = 0; st_ph ^= 1; }
          if (!(ok = mbar_wait(empty(s), ph ^ 1, (1 << 8) | 3, cta_abort))) break;
          mbar_expect_tx(full_a(s), Cfg::kABytes);
#pragma unroll
          for (int h = 0; h < Cfg::kAccs; ++h)
            tma_load_2d(stage_a(s) + h * 128 * 128, &a_map, kb * kBK, tm * BM + h * 128, full_a(s));
          // at most two groups per stage (gb >= 2); one when a group spans whole stages
          const int g0 = (kb * 4) / gb, g1 = (gb & 3) == 0 ? g0 : (kb * 4 + 3) / gb;
          const int ng = g1 - g0 + 1;
          const uint32_t s_bytes = nt_valid * 128, z_bytes = nt_valid * 8 * BITS;
          // packed weights: one 2-D copy of 4 k-tile rows x (NTT tiles of 8-byte elements);
          // columns past N are zero-filled and still counted in the transaction bytes
          mbar_expect_tx(full_w(s), Cfg::kWBytes + ng * s_bytes + (HAS_ZP ? ng * z_bytes : 0));
#pragma unroll
          for (int c = 0; c < Cfg::kCopies; ++c)
            tma_load_2d(stage_w(s) + c * 4 * Cfg::kCopyRowBytes, &b_map,
                        (nt0 + c * Cfg::kCopyTiles) * (Cfg::kTileBytes / 8), kb * 4, full_w(s));
          for (int gi = 0; gi < ng; ++gi) {
            bulk_load_1d(stage_s(s) + gi * Cfg::kSRow,
                         static_cast<const uint16_t*>(p.scales) + (size_t)(g0 + gi) * p.n + nt0 * 64,
                         s_bytes, full_w(s));
            if (HAS_ZP)
              bulk_load_1d(stage_z(s) + gi * Cfg::kZRow,
                           p.zeros + (size_t)(g0 + gi) * (p.n * BITS / 32) + nt0 * (2 * BITS),
                           z_bytes, full_w(s));
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issuer ========================================================
    if (lane == 0) {
      const uint32_t idesc = make_idesc<T>(BN);
      uint32_t it = 0, tile_i = 0;
      int st_i = 0;
      uint32_t st_ph = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++tile_i) {
        const int ks = item % KS;
        const int kb0 = (int)((long long)kb_total * ks / KS);
        const int kb1 = (int)((long long)kb_total * (ks + 1) / KS);
        const int buf = Cfg::kBufs == 2 ? (tile_i & 1) : 0;
        const uint32_t bph = Cfg::kBufs == 2 ? ((tile_i >> 1) & 1) : (tile_i & 1);
        if (!(ok = mbar_wait(tmem_empty(buf), bph ^ 1, (2 << 8) | 5, cta_abort))) break;
        tc_fence_after();
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = st_i;
          const uint32_t ph = st_ph;
          if (++st_i == S) { st_i = 0; st_ph ^= 1; }
          if (!(ok = mbar_wait(full_a(s), ph, (2 << 8) | 0, cta_abort))) break;
          if (!(ok = mbar_wait(full_b(s), ph, (2 << 8) | 2, cta_abort))) break;
          tc_fence_after();
#pragma unroll
          for (int h = 0; h < Cfg::kAccs; ++h) {
            const uint32_t d = tmem_base + (buf * Cfg::kAccs + h) * BN;
            const uint64_t da = smem_desc_sw128(stage_a(s) + h * 128 * 128);
            const uint64_t db = smem_desc_sw128(stage_b(s));
#pragma unroll
            for (int k16 = 0; k16 < kBK / 16; ++k16)
              umma_f16(d, da + 2 * k16, db + 2 * k16, idesc, (kb > kb0) || (k16 != 0));
          }
          umma_commit(empty(s));  // stage reusable once these MMAs have read it
        }
        if (ok) umma_commit(tmem_full(buf));
      }
    }
  } else if (warp < kDequantWarps) {
    // ================= dequant warps: packed codes -> scaled 16-bit B operand ============
    const int c8 = lane >> 2, q = lane & 3;
    const bool gb_mult4 = (gb & 3) == 0;
    const int kt = warp & 3;             // k-tile of the stage handled by this warp
    const int quarter = warp >> 2;       // which quarter of the tile's columns
    // BN = 256: one 64-column tile, all four 16-column sub-tiles; BN = 128: half a tile
    constexpr int kSubs = (BN == 256) ? 4 : 2;
    const int nt = (BN == 256) ? quarter : (quarter >> 1);
    const int sub0 = (BN == 256) ? 0 : 2 * (quarter & 1);
    // byte offsets of this lane's two k-positions (k = 16 kt + 2q, +8) inside a 128 B row
    const uint32_t off_lo = (((2 * kt) ^ c8) << 4) + 4 * q;
    const uint32_t off_hi = (((2 * kt + 1) ^ c8) << 4) + 4 * q;
    // stage-relative addresses of everything this lane touches
    // weights of the stage: [copy][k-tile][tile within the copy]
    const uint32_t w_rel = Cfg::kABytes + Cfg::kBBytes + (nt / Cfg::kCopyTiles) * 4 * Cfg::kCopyRowBytes +
                           kt * Cfg::kCopyRowBytes + (nt % Cfg::kCopyTiles) * Cfg::kTileBytes;
    // converted operand: row of sub-tile sub0 for this lane; the other sub-tiles are 16 rows
    // (2048 B) further, the second column block 8 rows (1024 B): immediates of the stores
    const uint32_t b_lo_rel = Cfg::kABytes + (nt * 64 + sub0 * 16 + c8) * 128 + off_lo;
    const uint32_t b_hi_rel = Cfg::kABytes + (nt * 64 + sub0 * 16 + c8) * 128 + off_hi;
    // scales of the lane's columns (grouped layout: 16 B per c8 of a tile, 4 B per sub-tile)
    const uint32_t s_rel = Cfg::kSOff + nt * 128 + c8 * 16 + sub0 * 4;
    uint32_t sbase = smem_base;  // base of the current stage
    // The proxy fence that publishes the converted operand is slow compared with the
    // conversion of one stage; with a ring of four or more stages two stages share one fence.
    constexpr bool kPairStages = S >= 4;
    int pending = -1;  // stage converted but not yet published
    uint32_t it = 0;
    int st_i = 0;
    uint32_t st_ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const int t = item / KS, ks = item - t * KS;
      const int kb0 = (int)((long long)kb_total * ks / KS);
      const int kb1 = (int)((long long)kb_total * (ks + 1) / KS);
      const int tn = t / m_tiles;
      const int nt0 = tn * NTT;
      const int nt_valid = min(NTT, NT - nt0);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = st_i;
        const uint32_t ph = st_ph;
        if (++st_i == S) { st_i = 0; st_ph ^= 1; }
        if (!(ok = mbar_wait(full_w(s), ph, (3 << 8) | 1, cta_abort))) break;
        // which of the stage's (at most two) groups: always the first when a group spans whole stages
        const int slot = gb_mult4 ? 0 : (kb * 4 + kt) / gb - (kb * 4) / gb;
        const uint32_t wsrc = sbase + w_rel;
        const uint32_t ssrc = sbase + Cfg::kSOff + slot * Cfg::kSRow;
        const uint32_t zsrc = sbase + Cfg::kZOff + slot * Cfg::kZRow;
        const uint32_t b_lo = sbase + b_lo_rel, b_hi = sbase + b_hi_rel;
        const uint32_t s_lane = sbase + s_rel + slot * Cfg::kSRow;
        sbase = (s + 1 == S) ? smem_base : sbase + Cfg::kStageBytes;
        if (nt < nt_valid) {
          // packed words of this lane for sub-tiles sub0 .. sub0 + kSubs - 1
          uint32_t wv[kSubs * (BITS == 4 ? 1 : 2)];
          if (BITS == 4) {
            if (kSubs == 4) {
              const uint4 w4 = lds128(wsrc + lane * 16);
              wv[0] = w4.x; wv[1] = w4.y; wv[2] = w4.z; wv[3] = w4.w;
            } else {
              wv[0] = lds32(wsrc + lane * 16 + sub0 * 4);
              wv[1] = lds32(wsrc + lane * 16 + sub0 * 4 + 4);
            }
          } else {
#pragma unroll
            for (int v = 0; v < kSubs / 2; ++v) {
              const uint4 w4 = lds128(wsrc + lane * 32 + sub0 * 8 + v * 16);
              wv[4 * v] = w4.x; wv[4 * v + 1] = w4.y; wv[4 * v + 2] = w4.z; wv[4 * v + 3] = w4.w;
            }
          }
          uint32_t zw[2] = {0, 0};  // zero-point words of (group, tile, c8)
          if (HAS_ZP) {
            if (BITS == 4) {
              zw[0] = lds32(zsrc + nt * 32 + c8 * 4);
            } else {
              zw[0] = lds32(zsrc + nt * 64 + c8 * 8);
              zw[1] = lds32(zsrc + nt * 64 + c8 * 8 + 4);
            }
          }
          // one sub-tile; `si` is a compile-time constant so that the offsets of the scale
          // load and of the four stores fold into the instructions
          auto convert_sub = [&](auto si_c, auto cw_c) {
            constexpr int si = decltype(si_c)::value;
            constexpr bool kChannelwise = decltype(cw_c)::value;
            const int sub = sub0 + si;
            // scales of columns c8 + 16 sub (low half) and + 8 (high half)
            uint32_t sv;
            if constexpr (kChannelwise) {
              // 32-column permutation: column r of a chunk sits at 8 ((r&7)>>1) + 2 (r>>3) + (r&1)
              const int jj = 2 * sub;
              const uint32_t pos = (jj >> 2) * 32 + 8 * (c8 >> 1) + 2 * (jj & 3) + (c8 & 1);
              uint32_t lo, hi;
              asm volatile("ld.shared.u16 %0, [%1];\n" : "=r"(lo) : "r"(ssrc + nt * 128 + pos * 2));
              asm volatile("ld.shared.u16 %0, [%1];\n" : "=r"(hi) : "r"(ssrc + nt * 128 + pos * 2 + 4));
              sv = lo | (hi << 16);
            } else {
              sv = lds32_off<si * 4>(s_lane);
            }
            const uint32_t s_lo = dup_lo(sv), s_hi = dup_hi(sv);
            uint32_t f[4];  // (cols c8, k lo), (c8, k hi), (c8 + 8, k lo), (c8 + 8, k hi)
            if (BITS == 4) {
              dequant4<T, !HAS_ZP>(wv[si], f);
            } else {
              uint32_t t0[2], t1[2];
              dequant8<T, !HAS_ZP>(wv[2 * si], t0);
              dequant8<T, !HAS_ZP>(wv[2 * si + 1], t1);
              f[0] = t0[0]; f[1] = t0[1]; f[2] = t1[0]; f[3] = t1[1];
            }
            if (HAS_ZP) {
              // zero-points of the same two columns as exact integers in T
              uint32_t zpair;
              if (BITS == 4) {
                // nibbles `sub` and `sub + 4` of the word
                uint32_t z4[4];
                dequant4<T, false>(zw[0] >> (4 * sub), z4);
                zpair = z4[0];
              } else {
                // word sub / 2, bytes (0, 2) for even sub, (1, 3) for odd
                uint32_t z8[2];
                dequant8<T, false>((sub & 2) ? zw[1] : zw[0], z8);
                zpair = (sub & 1) ? z8[1] : z8[0];
              }
              const uint32_t z_lo = dup_lo(zpair), z_hi = dup_hi(zpair);
              f[0] = Pair<T>::sub(f[0], z_lo);
              f[1] = Pair<T>::sub(f[1], z_lo);
              f[2] = Pair<T>::sub(f[2], z_hi);
              f[3] = Pair<T>::sub(f[3], z_hi);
            }
            f[0] = Pair<T>::mul(f[0], s_lo);
            f[1] = Pair<T>::mul(f[1], s_lo);
            f[2] = Pair<T>::mul(f[2], s_hi);
            f[3] = Pair<T>::mul(f[3], s_hi);
            sts32_off<si * 2048>(b_lo, f[0]);
            sts32_off<si * 2048>(b_hi, f[1]);
            sts32_off<si * 2048 + 1024>(b_lo, f[2]);
            sts32_off<si * 2048 + 1024>(b_hi, f[3]);
          };
          // the layout of the scales is a property of the launch: branch once per step, not
          // per sub-tile (predicated copies of the other layout's loads would still issue)
          auto convert_all = [&](auto cw_c) {
            convert_sub(std::integral_constant<int, 0>{}, cw_c);
            convert_sub(std::integral_constant<int, 1>{}, cw_c);
            if constexpr (kSubs == 4) {
              convert_sub(std::integral_constant<int, 2>{}, cw_c);
              convert_sub(std::integral_constant<int, 3>{}, cw_c);
            }
          };
          if (p.channelwise)
            convert_all(std::true_type{});
          else
            convert_all(std::false_type{});
        }
        if (kPairStages && pending < 0) {
          pending = s;
        } else {
          fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core
          __syncwarp();
          if (lane == 0) {
            if (pending >= 0) mbar_arrive(full_b(pending));
            mbar_arrive(full_b(s));
          }
          pending = -1;
        }
      }
    }
    if (pending >= 0) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_b(pending));
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + 4) {
    // ================= epilogue: TMEM -> registers -> C ==================================
    const int quad = warp & 3;  // TMEM lanes 32 quad .. 32 quad + 31
    const uint16_t* bias = static_cast<const uint16_t*>(p.bias);
    uint16_t* C = static_cast<uint16_t*>(p.c);
    uint32_t tile_i = 0;
    bool ok = true;
    // bias, rounding and the store of 16 consecutive columns of one row
    auto store16 = [&](int row, int n0, const float (&v)[16]) {
      uint32_t packed[8];
#pragma unroll
      for (int e = 0; e < 16; e += 2) {
        float v0 = v[e], v1 = v[e + 1];
        if (bias) {
          v0 += Pair<T>::to_float(bias[single_perm_pos(n0 + e)]);
          v1 += Pair<T>::to_float(bias[single_perm_pos(n0 + e + 1)]);
        }
        packed[e / 2] =
            (uint32_t)Pair<T>::from_float(v0) | ((uint32_t)Pair<T>::from_float(v1) << 16);
      }
      uint4* dst = reinterpret_cast<uint4*>(C + (size_t)row * p.n + n0);
      dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    };
    // C and the partial sums may still be read by the kernel before this one
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++tile_i) {
      const int t = item / KS;
      const int tn = t / m_tiles, tm = t % m_tiles;
      const int buf = Cfg::kBufs == 2 ? (tile_i & 1) : 0;
      const uint32_t bph = Cfg::kBufs == 2 ? ((tile_i >> 1) & 1) : (tile_i & 1);
      if (!(ok = mbar_wait(tmem_full(buf), bph, (4 << 8) | 4, cta_abort))) break;
      tc_fence_after();
#pragma unroll
      for (int h = 0; h < Cfg::kAccs; ++h) {
        const int trow = h * 128 + quad * 32 + lane;  // row inside the tile
        const int row = tm * BM + trow;
        float* part = p.partials + ((size_t)item * BM + trow) * BN;
#pragma unroll 1
        for (int cb = 0; cb < BN / 32; ++cb) {
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (buf * Cfg::kAccs + h) * BN + cb * 32,
                    r);
          tmem_ld_wait();
          const int n0 = tn * BN + cb * 32;
          if (row < p.m && n0 < p.n) {
            if (KS == 1) {
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                float v[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(r[16 * hh + e]);
                store16(row, n0 + 16 * hh, v);
              }
            } else {
              float4* dst = reinterpret_cast<float4*>(part + cb * 32);
#pragma unroll
              for (int v4 = 0; v4 < 8; ++v4)
                __stcg(dst + v4, make_float4(__uint_as_float(r[4 * v4]), __uint_as_float(r[4 * v4 + 1]),
                                             __uint_as_float(r[4 * v4 + 2]),
                                             __uint_as_float(r[4 * v4 + 3])));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty(buf));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// Sum of a k-split's partials in split order, bias, rounding: one thread per row and
// eight consecutive columns.
template <typename T>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partials, const void* __restrict__ bias_, void* c,
                     int m, int n, int bm, int bn, int ks) {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const int n8 = n / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)m * n8) return;
  const int row = (int)(idx / n8), n0 = (int)(idx % n8) * 8;
  const int m_tiles = (m + bm - 1) / bm;
  const int t = (n0 / bn) * m_tiles + row / bm;
  const float* src = partials + ((size_t)t * ks * bm + row % bm) * bn + n0 % bn;
  const size_t split_stride = (size_t)bm * bn;
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = 0.f;
  for (int s2 = 0; s2 < ks; ++s2) {
    const float4 x0 = __ldcg(reinterpret_cast<const float4*>(src + s2 * split_stride));
    const float4 x1 = __ldcg(reinterpret_cast<const float4*>(src + s2 * split_stride) + 1);
    v[0] += x0.x; v[1] += x0.y; v[2] += x0.z; v[3] += x0.w;
    v[4] += x1.x; v[5] += x1.y; v[6] += x1.z; v[7] += x1.w;
  }
  const uint16_t* bias = static_cast<const uint16_t*>(bias_);
  uint32_t packed[4];
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    float v0 = v[e], v1 = v[e + 1];
    if (bias) {
      v0 += Pair<T>::to_float(bias[single_perm_pos(n0 + e)]);
      v1 += Pair<T>::to_float(bias[single_perm_pos(n0 + e + 1)]);
    }
    packed[e / 2] = (uint32_t)Pair<T>::from_float(v0) | ((uint32_t)Pair<T>::from_float(v1) << 16);
  }
  *reinterpret_cast<uint4*>(static_cast<uint16_t*>(c) + (size_t)row * n + n0) =
      make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

// ---- host side ----------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// Tensor map over the packed weights seen as [K/16 rows][N * bits * 2 bytes] of 8-byte
// elements; box = 4 rows x (BN/64 tiles).
static int make_b_map(CUtensorMap* map, const TcParams& p, int bits, int bn) {
  const cuuint64_t row_elems = (cuuint64_t)p.n * bits * 2 / 8;  // 8-byte elements per k-tile row
  const cuuint64_t gdim[2] = {row_elems, (cuuint64_t)(p.k / 16)};
  const cuuint64_t gstride[1] = {row_elems * 8};
  const int tile_elems = 16 * 64 * bits / 8 / 8;  // 8-byte elements per 16 x 64 tile
  const int copy_tiles = (bn / 64) * tile_elems <= 256 ? (bn / 64) : 256 / tile_elems;
  const cuuint32_t box[2] = {(cuuint32_t)(copy_tiles * tile_elems), 4};
  const cuuint32_t estride[2] = {1, 1};
  CUresult r = get_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint32_t*>(p.b),
                               gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200Q_REQUIRE(r == CUDA_SUCCESS, B200Q_ECUDA, "cuTensorMapEncodeTiled (weights) failed with %d",
                (int)r);
  return B200Q_OK;
}

template <typename T, int BITS, bool HAS_ZP, int BM, int BN>
static int launch_one(const CUtensorMap& map, const TcParams& p, cudaStream_t stream) {
  CUtensorMap b_map;
  {
    const int rc = make_b_map(&b_map, p, BITS, BN);
    if (rc != B200Q_OK) return rc;
  }
  using Cfg = TcCfg<BM, BN, BITS>;
  auto kernel = gemm_tc_kernel<T, BITS, HAS_ZP, BM, BN>;
  static bool attr_done[64] = {};
  int dev = 0;
  B200Q_CUDA_OK(cudaGetDevice(&dev));
  if (!attr_done[dev & 63]) {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::kSmemBytes));
    attr_done[dev & 63] = true;
  }
  const int items = ((p.m + BM - 1) / BM) * ((p.n + BN - 1) / BN) * p.ksplit;
  const int sms = device_sm_count();
  const int grid = items < sms ? items : sms;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // early launch only where this kernel's fixed costs matter: with many rows the waiting CTAs
    // would take the SMs from an act-order gather still running in front (measured: down-proj
    // M = 1024 129 -> 142 us)
    cfg.numAttrs = (pdl_enabled() && p.m <= 128) ? 1 : 0;
    B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, map, b_map, p));
  }
  note_launch();
  B200Q_CUDA_OK(cudaGetLastError());
  if (p.ksplit > 1) {
    const long long threads = (long long)p.m * (p.n / 8);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((threads + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<T>, (const float*)p.partials, p.bias,
                                     p.c, p.m, p.n, BM, BN, p.ksplit));
    note_launch();
  }
  return B200Q_OK;
}

template <typename T, int BITS, bool HAS_ZP>
static int launch_tile(const CUtensorMap& map, const TcParams& p, int bm, int bn,
                       cudaStream_t stream) {
  if (bm == 128)
    return bn == 128 ? launch_one<T, BITS, HAS_ZP, 128, 128>(map, p, stream)
                     : launch_one<T, BITS, HAS_ZP, 128, 256>(map, p, stream);
  return bn == 128 ? launch_one<T, BITS, HAS_ZP, 256, 128>(map, p, stream)
                   : launch_one<T, BITS, HAS_ZP, 256, 256>(map, p, stream);
}

template <typename T, int BITS>
static int launch_bits(const CUtensorMap& map, const TcParams& p, bool has_zp, int bm, int bn,
                       cudaStream_t stream) {
  return has_zp ? launch_tile<T, BITS, true>(map, p, bm, bn, stream)
                : launch_tile<T, BITS, false>(map, p, bm, bn, stream);
}

// Tile shape and k-split for a problem: least estimated time.  A work item takes
// (its k-steps + a fixed fill / drain cost) x the time of one k-step of the tile
// shape; the relative step times were measured on B200 (the dequant warps' time per
// k-step is nearly constant, so tiles with more MMA work per converted column run
// closer to the tensor-pipe rate; small tiles are bound by the latency of the stage
// ring).  Splitting K pays when there are fewer tiles than SMs; it costs one more
// launch and the fp32 partial traffic.  `scratch_bytes` bounds the partials.
struct TcPlan {
  int bm, bn, ksplit;
  int64_t partial_bytes;
};
static TcPlan plan_tiles(int64_t m, int64_t n, int64_t k, int sms, int64_t scratch_bytes) {
  // microseconds per 64-deep k-step of one tile on one SM
  static const struct { int bm, bn; double step_us; } kCand[4] = {
      {256, 256, 0.74}, {256, 128, 0.52}, {128, 256, 0.58}, {128, 128, 0.42}};
  const int kb_total = (int)(k / kBK);
  TcPlan best = {128, 128, 1, 0};
  double best_cost = 1e300;
  for (const auto& c : kCand) {
    if (c.bm == 256 && m <= 128) continue;
    if (c.bn == 256 && n <= 128) continue;
    const int64_t tiles = ((m + c.bm - 1) / c.bm) * ((n + c.bn - 1) / c.bn);
    for (int ks = 1; ks <= 8; ++ks) {
      const int64_t bytes = ks > 1 ? tiles * ks * c.bm * c.bn * 4 : 0;
      if (ks > 1 && (kb_total / ks < 2 || bytes > scratch_bytes)) break;
      const double waves = (double)((tiles * ks + sms - 1) / sms);
      double cost = waves * ((double)kb_total / ks + 6.0 + (ks > 1 ? 2.0 : 0.0)) * c.step_us;
      if (ks > 1) cost += 2.5 + (double)ks * m * n * 4 / 3.0e6;  // reduce kernel: launch + 3 TB/s
      if (cost < best_cost) {
        best_cost = cost;
        best = {c.bm, c.bn, ks, bytes};
      }
    }
  }
  return best;
}

}  // namespace tc

// True when the tensor-core kernel can take this problem.
bool tc_gemm_supported(int64_t size_m, int64_t size_n, int64_t size_k, int gm) {
  const bool rows_ok = size_m >= 33;
  return rows_ok && size_k % tc::kBK == 0 && size_n % 64 == 0 && gm != kLookup &&
         tc::get_encode_fn() != nullptr;  // group_blocks >= 2 is checked by the caller
}

// a: [M, K] 16-bit row-major with row stride lda (already gathered for act-order).
int launch_tc_gemm(const void* a, int64_t lda, const uint32_t* b, const void* scales,
                   const uint32_t* zeros, const void* bias, void* c, int a_dtype, int bits,
                   int64_t size_m, int64_t size_n, int64_t size_k, int group_blocks,
                   int channelwise, void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
  CUtensorMap map;
  const cuuint64_t gdim[2] = {(cuuint64_t)size_k, (cuuint64_t)size_m};
  const cuuint64_t gstride[1] = {(cuuint64_t)lda * 2};
  const cuuint32_t box[2] = {(cuuint32_t)tc::kBK, 128};
  const cuuint32_t estride[2] = {1, 1};
  CUresult r = tc::get_encode_fn()(
      &map, a_dtype == B200Q_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
      2, const_cast<void*>(a), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200Q_REQUIRE(r == CUDA_SUCCESS, B200Q_ECUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  tc::TcParams p;
  p.b = b; p.scales = scales; p.zeros = zeros; p.bias = bias; p.c = c;
  p.m = (int)size_m; p.n = (int)size_n; p.k = (int)size_k;
  p.group_blocks = group_blocks; p.channelwise = channelwise;
  const tc::TcPlan plan = tc::plan_tiles(size_m, size_n, size_k, device_sm_count(), scratch_bytes);
  const int bm = plan.bm, bn = plan.bn;
  p.ksplit = plan.ksplit;
  p.partials = static_cast<float*>(scratch);
  const bool has_zp = zeros != nullptr;
  if (a_dtype == B200Q_F16)
    return bits == 4 ? tc::launch_bits<half, 4>(map, p, has_zp, bm, bn, stream)
                     : tc::launch_bits<half, 8>(map, p, has_zp, bm, bn, stream);
  return bits == 4 ? tc::launch_bits<__nv_bfloat16, 4>(map, p, has_zp, bm, bn, stream)
                   : tc::launch_bits<__nv_bfloat16, 8>(map, p, has_zp, bm, bn, stream);
}

// Scratch the tensor-core kernel would like for this problem (fp32 partials of a k-split).
int64_t tc_gemm_scratch_bytes(int64_t size_m, int64_t size_n, int64_t size_k) {
  if (size_m <= 32 || size_k % tc::kBK != 0 || size_n % 64 != 0) return 0;
  return tc::plan_tiles(size_m, size_n, size_k, device_sm_count(), tc::kMaxSplitBytes).partial_bytes;
}

int tc_error_flag(bool reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, tc::g_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(tc::g_tc_error, &zero, sizeof(int));
  }
  return v;
}

}  // namespace b200q
