// Peer-memory link shared by the all-reduce kernel and the GEMM kernel whose
// epilogue all-reduces its own output tile.
//
// Every rank owns a receive buffer that all ranks can address (plain stores over
// NVLink / NVSwitch, no multicast), laid out as [2 parities][world slots][slot_bytes].
// Data travels as 8-byte packets {two 16-bit values, 32-bit flag}: an aligned 8-byte
// store is one transaction, so a reader that sees the expected flag also sees the
// data: no fence, no separate flag round trip, no barrier between threads.
// A call (one kernel per rank, the same sequence on every rank):
//   push    every thread stores the packets of its share of this rank's rounded
//           partial into slot `rank` of every peer's buffer, parity = call number & 1,
//           flag = a function of the call number that is never 0;
//   reduce  the same thread polls the same packet positions of the other slots of
//           its own buffer (local memory) until the flag shows, and sums the values
//           with its own in rank order in fp32: every rank gets the same bits.
// Two parities are enough: a rank can start call j+2 (which reuses the parity of
// call j) only after finishing call j+1, for which it needed packets that a peer
// sends in its call j+1, i.e. after that peer's call j kernel has completed.  The
// call number lives in device memory (state[0]) and is advanced by the last CTA
// of each call (arrival count in state[1]), so a captured CUDA graph can be
// replayed.  The buffer must be zero before the first call.  Polls are bounded:
// on time-out the thread records an error word and gives up on its output.
#pragma once

#include <cstdint>

namespace b200q {

constexpr int kArMaxWorld = 8;
constexpr uint32_t kArSpinLimit = 1u << 21;  // default poll limit: a second or so of local polls

struct ArLink {
  void* const* bufs;         // device array [world]: every rank's receive buffer
  uint32_t* state;           // local: {call number, arrivals}
  int* error;                // local: 0 = ok, 0x1ff after a poll of the peers' packets timed out
  long long slot_bytes;      // packet bytes of one (parity, rank) slot = 2 x the largest message
  int rank, world;           // world == 0: link not in use
  uint32_t spin_limit;       // polls of local memory before a wait gives up
};

__device__ __forceinline__ uint32_t ar_ld_volatile(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Flag of a call: differs between consecutive uses of a parity, never 0.
__device__ __forceinline__ uint32_t ar_flag(uint32_t call) { return (call >> 1) % 0xffffffffu + 1u; }

__device__ __forceinline__ void ar_put1(void* dst, uint32_t d, uint32_t flag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};\n" ::"l"(dst), "r"(d), "r"(flag)
               : "memory");
}
// two adjacent packets in one 16-byte store (each half is a complete packet)
__device__ __forceinline__ void ar_put2(void* dst, uint32_t d0, uint32_t d1, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};\n" ::"l"(dst), "r"(d0), "r"(flag),
               "r"(d1)
               : "memory");
}
// Collect P adjacent packets (P = 1, 2 or 4) at byte offset `off` of every peer's slot
// in this rank's buffer.  The loads of all peers are issued together and polled as a
// batch, so the wait costs about one memory latency, not one per peer.  d[r] is left
// untouched for r == rank and r >= world.  Returns false on time-out.
template <int P>
__device__ __forceinline__ bool ar_collect(const ArLink& l, const char* mybuf, size_t off,
                                           uint32_t flag, uint32_t (&d)[kArMaxWorld][P]) {
  static_assert(P == 1 || P == 2 || P == 4, "packets per element");
  for (uint32_t spin = 0; spin < l.spin_limit; ++spin) {
    bool all = true;
#pragma unroll
    for (int r = 0; r < kArMaxWorld; ++r) {
      if (r < l.world && r != l.rank) {
        const char* src = mybuf + r * l.slot_bytes + off;
        if constexpr (P == 1) {
          uint32_t f;
          asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];\n"
                       : "=r"(d[r][0]), "=r"(f)
                       : "l"(src)
                       : "memory");
          all = all && f == flag;
        } else {
#pragma unroll
          for (int h = 0; h < P / 2; ++h) {
            uint32_t f0, f1;
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                         : "=r"(d[r][2 * h]), "=r"(f0), "=r"(d[r][2 * h + 1]), "=r"(f1)
                         : "l"(src + 16 * h)
                         : "memory");
            all = all && f0 == flag && f1 == flag;
          }
        }
      }
    }
    if (all) return true;
  }
  atomicCAS(l.error, 0, 0x1ff);
  return false;
}

// Four adjacent packets (32 bytes) of one peer.
__device__ __forceinline__ bool ar_get4(const ArLink& l, const char* src, uint32_t flag, uint32_t& w0,
                                        uint32_t& w1, uint32_t& w2, uint32_t& w3) {
  for (uint32_t spin = 0; spin < l.spin_limit; ++spin) {
    uint32_t f0, f1, f2, f3;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(w0), "=r"(f0), "=r"(w1), "=r"(f1)
                 : "l"(src)
                 : "memory");
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(w2), "=r"(f2), "=r"(w3), "=r"(f3)
                 : "l"(src + 16)
                 : "memory");
    if (f0 == flag && f1 == flag && f2 == flag && f3 == flag) return true;
  }
  atomicCAS(l.error, 0, 0x1ff);
  return false;
}

// One thread per CTA, once, after all threads of the CTA have read the call number
// and finished polling.
__device__ __forceinline__ void ar_arrive(const ArLink& l, uint32_t call, uint32_t n_ctas) {
  __threadfence();
  const uint32_t old = atomicAdd(&l.state[1], 1u);
  if (old == n_ctas - 1) {
    l.state[1] = 0;
    l.state[0] = call + 1;
  }
}

}  // namespace b200q
