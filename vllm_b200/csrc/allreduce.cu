// One-shot all-reduce of the row-parallel GEMM output over NVLink peer memory:
// the stand-alone kernel (the protocol is described in ar_link.cuh; the decode
// GEMM runs the same three steps in its own epilogue).
//
// The counterpart in the reference is the custom all-reduce of
// csrc/custom_all_reduce.cuh:298-314 (one-stage variant, pull-based, two barriers,
// unbounded waits).
#include <cstdlib>

#include <atomic>

#include "ar_link.cuh"
#include "common.cuh"

namespace b200q {
__device__ int g_ar_error;  // error word of this device (ArLink::error points here)

namespace ar {

constexpr int kMaxBlocks = 32;
constexpr int kThreads = 512;

struct ArParams {
  ArLink link;
  const void* in;    // local partial
  void* out;         // local output (may alias in)
  long long n_vec;   // 16-byte vectors in the message
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 1) allreduce_oneshot_kernel(const ArParams p) {
  // the partial was written by the kernel before this one in the stream
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  // the GEMM that follows may start prefetching its weights
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const ArLink& l = p.link;
  const uint32_t call = ar_ld_volatile(l.state);
  const uint32_t flag = ar_flag(call);
  const long long parity_off = (long long)(call & 1) * l.world * l.slot_bytes;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const uint4* in = static_cast<const uint4*>(p.in);
  const char* mybuf = static_cast<const char*>(l.bufs[l.rank]) + parity_off;

  // a 16-byte vector of the message is four packets = 32 bytes of a slot
  for (long long v = v0; v < p.n_vec; v += stride) {
    const uint4 x = in[v];
    for (int r = 0; r < l.world; ++r) {
      if (r == l.rank) continue;
      char* dst = static_cast<char*>(l.bufs[r]) + parity_off + l.rank * l.slot_bytes + v * 32;
      ar_put2(dst, x.x, x.y, flag);
      ar_put2(dst + 16, x.z, x.w, flag);
    }
  }
  for (long long v = v0; v < p.n_vec; v += stride) {
    uint32_t d[kArMaxWorld][4];
    if (!ar_collect<4>(l, mybuf, (size_t)v * 32, flag, d)) break;
    const uint4 x = in[v];
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
    for (int r = 0; r < kArMaxWorld; ++r) {
      if (r < l.world) {
        const bool me = r == l.rank;
        const uint32_t w0 = me ? x.x : d[r][0], w1 = me ? x.y : d[r][1];
        const uint32_t w2 = me ? x.z : d[r][2], w3 = me ? x.w : d[r][3];
        acc[0] += Pair<T>::to_float((uint16_t)(w0 & 0xffffu));
        acc[1] += Pair<T>::to_float((uint16_t)(w0 >> 16));
        acc[2] += Pair<T>::to_float((uint16_t)(w1 & 0xffffu));
        acc[3] += Pair<T>::to_float((uint16_t)(w1 >> 16));
        acc[4] += Pair<T>::to_float((uint16_t)(w2 & 0xffffu));
        acc[5] += Pair<T>::to_float((uint16_t)(w2 >> 16));
        acc[6] += Pair<T>::to_float((uint16_t)(w3 & 0xffffu));
        acc[7] += Pair<T>::to_float((uint16_t)(w3 >> 16));
      }
    }
    uint4 o;
    o.x = (uint32_t)Pair<T>::from_float(acc[0]) | ((uint32_t)Pair<T>::from_float(acc[1]) << 16);
    o.y = (uint32_t)Pair<T>::from_float(acc[2]) | ((uint32_t)Pair<T>::from_float(acc[3]) << 16);
    o.z = (uint32_t)Pair<T>::from_float(acc[4]) | ((uint32_t)Pair<T>::from_float(acc[5]) << 16);
    o.w = (uint32_t)Pair<T>::from_float(acc[6]) | ((uint32_t)Pair<T>::from_float(acc[7]) << 16);
    reinterpret_cast<uint4*>(p.out)[v] = o;
  }
  __syncthreads();
  if (threadIdx.x == 0) ar_arrive(l, call, gridDim.x);
}

// Two-shot variant for larger messages on four or more ranks: every rank owns a chunk of
// the message.  Phase 1 sends each vector only to the owner of its chunk, the owner sums
// in rank order and sends the reduced vector to everybody (phase 2), and everybody picks
// up the other owners' chunks (phase 3).  Per rank about twice the message crosses NVLink
// instead of (world - 1) times.  Partial and reduced packets of one sender never share
// an offset of its slot: the former sit in the receiver's chunk, the latter in the sender's.
template <typename T>
__global__ void __launch_bounds__(kThreads, 1) allreduce_twoshot_kernel(const ArParams p) {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const ArLink& l = p.link;
  const uint32_t call = ar_ld_volatile(l.state);
  const uint32_t flag = ar_flag(call);
  const long long parity_off = (long long)(call & 1) * l.world * l.slot_bytes;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const uint4* in = static_cast<const uint4*>(p.in);
  uint4* out = static_cast<uint4*>(p.out);
  const char* mybuf = static_cast<const char*>(l.bufs[l.rank]) + parity_off;
  const long long chunk = (p.n_vec + l.world - 1) / l.world;
  const long long mine_off = parity_off + (long long)l.rank * l.slot_bytes;

  for (long long v = v0; v < p.n_vec; v += stride) {
    const int owner = (int)(v / chunk);
    if (owner == l.rank) continue;
    const uint4 x = in[v];
    char* dst = static_cast<char*>(l.bufs[owner]) + mine_off + v * 32;
    ar_put2(dst, x.x, x.y, flag);
    ar_put2(dst + 16, x.z, x.w, flag);
  }
  const long long lo = (long long)l.rank * chunk;
  const long long hi = lo + chunk < p.n_vec ? lo + chunk : p.n_vec;
  bool ok = true;
  for (long long v = lo + v0; v < hi && ok; v += stride) {
    uint32_t d[kArMaxWorld][4];
    if (!ar_collect<4>(l, mybuf, (size_t)v * 32, flag, d)) {
      ok = false;
      break;
    }
    const uint4 x = in[v];
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
    for (int r = 0; r < kArMaxWorld; ++r) {
      if (r < l.world) {
        const bool me = r == l.rank;
        const uint32_t w0 = me ? x.x : d[r][0], w1 = me ? x.y : d[r][1];
        const uint32_t w2 = me ? x.z : d[r][2], w3 = me ? x.w : d[r][3];
        acc[0] += Pair<T>::to_float((uint16_t)(w0 & 0xffffu));
        acc[1] += Pair<T>::to_float((uint16_t)(w0 >> 16));
        acc[2] += Pair<T>::to_float((uint16_t)(w1 & 0xffffu));
        acc[3] += Pair<T>::to_float((uint16_t)(w1 >> 16));
        acc[4] += Pair<T>::to_float((uint16_t)(w2 & 0xffffu));
        acc[5] += Pair<T>::to_float((uint16_t)(w2 >> 16));
        acc[6] += Pair<T>::to_float((uint16_t)(w3 & 0xffffu));
        acc[7] += Pair<T>::to_float((uint16_t)(w3 >> 16));
      }
    }
    uint4 o;
    o.x = (uint32_t)Pair<T>::from_float(acc[0]) | ((uint32_t)Pair<T>::from_float(acc[1]) << 16);
    o.y = (uint32_t)Pair<T>::from_float(acc[2]) | ((uint32_t)Pair<T>::from_float(acc[3]) << 16);
    o.z = (uint32_t)Pair<T>::from_float(acc[4]) | ((uint32_t)Pair<T>::from_float(acc[5]) << 16);
    o.w = (uint32_t)Pair<T>::from_float(acc[6]) | ((uint32_t)Pair<T>::from_float(acc[7]) << 16);
    out[v] = o;
    for (int r = 0; r < l.world; ++r) {
      if (r == l.rank) continue;
      char* dst = static_cast<char*>(l.bufs[r]) + mine_off + v * 32;
      ar_put2(dst, o.x, o.y, flag);
      ar_put2(dst + 16, o.z, o.w, flag);
    }
  }
  for (long long v = v0; v < p.n_vec && ok; v += stride) {
    const int owner = (int)(v / chunk);
    if (owner == l.rank) continue;
    uint4 o;
    if (!ar_get4(l, mybuf + (long long)owner * l.slot_bytes + v * 32, flag, o.x, o.y, o.z, o.w)) break;
    out[v] = o;
  }
  __syncthreads();
  if (threadIdx.x == 0) ar_arrive(l, call, gridDim.x);
}

}  // namespace ar

int ar_error_flag(bool reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ar_error, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_ar_error, &zero, sizeof(int));
  }
  return v;
}

}  // namespace b200q

using namespace b200q;

extern "C" size_t b200q_all_reduce_state_bytes(void) { return 2 * sizeof(uint32_t); }
extern "C" size_t b200q_all_reduce_buffer_bytes(int world, int64_t max_message_bytes) {
  return (size_t)2 * (size_t)world * (size_t)(2 * max_message_bytes);  // parities x slots x packets
}

namespace b200q {
int launch_all_reduce(const ArLink& link, const void* in, void* out, int64_t n_elems, int dtype,
                      cudaStream_t stream) {
  B200Q_REQUIRE(n_elems >= 0 && n_elems % 8 == 0, B200Q_EINVAL,
                "message must be a whole number of 16-byte vectors (n_elems = %lld)",
                (long long)n_elems);
  B200Q_REQUIRE(n_elems * 4 <= link.slot_bytes, B200Q_EINVAL,
                "message of %lld bytes exceeds the largest message %lld", (long long)n_elems * 2,
                link.slot_bytes / 2);
  B200Q_REQUIRE(((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(in)) & 15) == 0,
                B200Q_EINVAL, "in / out must be aligned to 16 bytes");
  if (n_elems == 0) return B200Q_OK;
  ar::ArParams p;
  p.link = link;
  p.in = in;
  p.out = out;
  p.n_vec = n_elems / 8;
  long long blocks = (p.n_vec + ar::kThreads - 1) / ar::kThreads;
  if (blocks > ar::kMaxBlocks) blocks = ar::kMaxBlocks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(ar::kThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  // two-shot from 256 KiB on four or more ranks; B200Q_DEBUG=twoshot_any selects it for every
  // message and group size (how the two-rank tests reach it)
  static const bool twoshot_any = debug_flag("twoshot_any");
  const bool twoshot = twoshot_any || (link.world >= 4 && n_elems * 2 >= 256ll * 1024);
  if (dtype == B200Q_F16)
    B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, twoshot ? ar::allreduce_twoshot_kernel<half>
                                                   : ar::allreduce_oneshot_kernel<half>, p));
  else
    B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, twoshot ? ar::allreduce_twoshot_kernel<__nv_bfloat16>
                                                   : ar::allreduce_oneshot_kernel<__nv_bfloat16>, p));
  note_launch();
  return B200Q_OK;
}

// polls before a wait on peer packets gives up (b200q_all_reduce_set_poll_limit)
static std::atomic<uint32_t> g_poll_limit{kArSpinLimit};

int check_link(void* const* peer_bufs, uint32_t* state, int rank,
               int world, int64_t max_message_bytes, ArLink* link) {
  B200Q_REQUIRE(world >= 2 && world <= kArMaxWorld, B200Q_EINVAL,
                "all-reduce world size %d is not in [2, %d]", world, kArMaxWorld);
  B200Q_REQUIRE(rank >= 0 && rank < world, B200Q_EINVAL, "rank %d out of range", rank);
  B200Q_REQUIRE(peer_bufs && state, B200Q_EINVAL, "null pointer");
  B200Q_REQUIRE(max_message_bytes > 0 && max_message_bytes % 16 == 0, B200Q_EINVAL,
                "slot size must be a positive multiple of 16 bytes");
  static int* err_ptr[64] = {};  // per device; benign race: the lookup is idempotent
  int dev = 0;
  B200Q_CUDA_OK(cudaGetDevice(&dev));
  if (!err_ptr[dev & 63]) {
    void* sym = nullptr;
    B200Q_CUDA_OK(cudaGetSymbolAddress(&sym, g_ar_error));
    err_ptr[dev & 63] = static_cast<int*>(sym);
  }
  link->error = err_ptr[dev & 63];
  link->bufs = peer_bufs;
  link->state = state;
  link->slot_bytes = 2 * max_message_bytes;
  link->rank = rank;
  link->world = world;
  link->spin_limit = g_poll_limit.load(std::memory_order_relaxed);
  return B200Q_OK;
}
}  // namespace b200q

extern "C" void b200q_all_reduce_set_poll_limit(uint32_t polls) {
  g_poll_limit.store(polls == 0 ? kArSpinLimit : polls, std::memory_order_relaxed);
}

extern "C" int b200q_all_reduce(void* const* peer_bufs, uint32_t* state, int rank, int world,
                                int64_t max_message_bytes,
                                const void* in, void* out, int64_t n_elems, int dtype,
                                b200q_stream_t stream_) {
  ArLink link;
  int rc = check_link(peer_bufs, state, rank, world, max_message_bytes, &link);
  if (rc != B200Q_OK) return rc;
  B200Q_REQUIRE(dtype == B200Q_F16 || dtype == B200Q_BF16, B200Q_EINVAL, "dtype must be fp16/bf16");
  B200Q_REQUIRE(in && out, B200Q_EINVAL, "null pointer");
  return launch_all_reduce(link, in, out, n_elems, dtype, static_cast<cudaStream_t>(stream_));
}
