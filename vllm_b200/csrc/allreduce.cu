// One-shot all-reduce of the row-parallel GEMM output over NVLink peer memory.
//
// Every rank owns a receive buffer that all ranks of the tensor-parallel group
// can address (peer pointers; plain stores over NVLink / NVSwitch, no multicast),
// laid out as [2 parities][world slots][slot_bytes].  One kernel per rank:
//   1. push     - block b stores its share of this rank's partial (read from local
//                 memory) into slot `rank` of every peer's buffer, parity = call
//                 number mod 2;
//   2. signal   - after the block's stores, one thread per peer publishes
//                 flag[b][rank] = epoch + 1 in that peer's flag array
//                 (st.release.sys) and waits for the peer's flag in its own array;
//   3. reduce   - the block sums the slots of its own buffer (local reads) and its
//                 own partial in rank order with fp32 accumulation, so all ranks
//                 produce bitwise identical results, rounds once and stores.
// One flag round per call: a rank can only be two calls ahead of a peer after the
// peer has signalled the call in between, i.e. finished reading the parity that is
// about to be overwritten.  The call number lives in device memory, one counter
// per block, advanced by the kernel, so a captured CUDA graph can replay it.
// Flags only ever grow: no reset traffic.  Every wait is bounded; on time-out the
// kernel records an error word and returns without reducing.
//
// The counterpart in the reference is the custom all-reduce of
// csrc/custom_all_reduce.cuh:298-314 (one-stage variant, pull-based, two barriers,
// unbounded waits).
#include "common.cuh"

namespace b200q {
namespace ar {

constexpr int kMaxWorld = 8;
constexpr int kMaxBlocks = 32;
constexpr int kThreads = 512;
constexpr uint32_t kSpinLimit = 1u << 22;  // polls of a local flag: seconds at most

__device__ int g_ar_error;  // 0 = ok, else 0x100 | peer rank of the first wait that timed out

struct ArParams {
  void* const* bufs;            // device array [world]: every rank's receive buffer
  uint32_t* const* flags;       // device array [world]: every rank's flag array [kMaxBlocks * world]
  uint32_t* epochs;             // local: one call counter per block
  const void* in;               // local partial
  void* out;                    // local output
  long long slot_bytes;         // size of one (parity, rank) slot of a receive buffer
  long long n_vec;              // 16-byte vectors in the message
  int rank, world;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) allreduce_oneshot_kernel(const ArParams p) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_fail;
  // the partial was written by the kernel before this one in the stream
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  // the GEMM that follows may start prefetching its weights
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  if (threadIdx.x == 0) {
    s_epoch = p.epochs[blockIdx.x];
    p.epochs[blockIdx.x] = s_epoch + 1;
    s_fail = 0;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const long long parity_off = (long long)(epoch & 1) * p.world * p.slot_bytes;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const uint4* in = static_cast<const uint4*>(p.in);

  // 1. push this block's vectors into slot `rank` of every peer
  for (long long v = v0; v < p.n_vec; v += stride) {
    const uint4 x = in[v];
    for (int r = 0; r < p.world; ++r) {
      if (r == p.rank) continue;
      char* dst = static_cast<char*>(p.bufs[r]) + parity_off + p.rank * p.slot_bytes;
      reinterpret_cast<uint4*>(dst)[v] = x;
    }
  }
  __syncthreads();
  // 2. signal every peer, wait for every peer (threads 0 .. world-1, one peer each)
  if (threadIdx.x < p.world && threadIdx.x != p.rank) {
    const int t = threadIdx.x;
    st_release_sys(p.flags[t] + (blockIdx.x * p.world + p.rank), epoch + 1);
    const uint32_t* mine = p.flags[p.rank] + (blockIdx.x * p.world + t);
    bool ok = false;
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
      if ((int32_t)(ld_acquire_sys(mine) - (epoch + 1)) >= 0) {
        ok = true;
        break;
      }
    }
    if (!ok) {
      s_fail = 1;
      atomicCAS(&g_ar_error, 0, 0x100 | t);
    }
  }
  __syncthreads();
  if (s_fail) return;

  // 3. reduce in rank order from local memory
  const char* mybuf = static_cast<const char*>(p.bufs[p.rank]) + parity_off;
  for (long long v = v0; v < p.n_vec; v += stride) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int r = 0; r < p.world; ++r) {
      const uint4 x = (r == p.rank)
                          ? in[v]
                          : __ldcv(reinterpret_cast<const uint4*>(mybuf + r * p.slot_bytes) + v);
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += Pair<T>::to_float((uint16_t)(w[e] & 0xffffu));
        acc[2 * e + 1] += Pair<T>::to_float((uint16_t)(w[e] >> 16));
      }
    }
    uint4 o;
    o.x = (uint32_t)Pair<T>::from_float(acc[0]) | ((uint32_t)Pair<T>::from_float(acc[1]) << 16);
    o.y = (uint32_t)Pair<T>::from_float(acc[2]) | ((uint32_t)Pair<T>::from_float(acc[3]) << 16);
    o.z = (uint32_t)Pair<T>::from_float(acc[4]) | ((uint32_t)Pair<T>::from_float(acc[5]) << 16);
    o.w = (uint32_t)Pair<T>::from_float(acc[6]) | ((uint32_t)Pair<T>::from_float(acc[7]) << 16);
    reinterpret_cast<uint4*>(p.out)[v] = o;
  }
}

}  // namespace ar

int ar_error_flag(bool reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, ar::g_ar_error, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(ar::g_ar_error, &zero, sizeof(int));
  }
  return v;
}

}  // namespace b200q

using namespace b200q;

extern "C" size_t b200q_all_reduce_flag_bytes(void) {
  return (size_t)ar::kMaxBlocks * ar::kMaxWorld * sizeof(uint32_t);
}
extern "C" size_t b200q_all_reduce_epoch_bytes(void) { return ar::kMaxBlocks * sizeof(uint32_t); }
extern "C" size_t b200q_all_reduce_buffer_bytes(int world, int64_t max_message_bytes) {
  return (size_t)2 * (size_t)world * (size_t)max_message_bytes;
}

extern "C" int b200q_all_reduce(void* const* peer_bufs, uint32_t* const* peer_flags,
                                uint32_t* epochs, int rank, int world, int64_t max_message_bytes,
                                const void* in, void* out, int64_t n_elems, int dtype,
                                b200q_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200Q_REQUIRE(world >= 2 && world <= ar::kMaxWorld, B200Q_EINVAL,
                "all-reduce world size %d is not in [2, %d]", world, ar::kMaxWorld);
  B200Q_REQUIRE(rank >= 0 && rank < world, B200Q_EINVAL, "rank %d out of range", rank);
  B200Q_REQUIRE(dtype == B200Q_F16 || dtype == B200Q_BF16, B200Q_EINVAL, "dtype must be fp16/bf16");
  B200Q_REQUIRE(peer_bufs && peer_flags && epochs && in && out, B200Q_EINVAL, "null pointer");
  B200Q_REQUIRE(n_elems >= 0 && n_elems % 8 == 0, B200Q_EINVAL,
                "message must be a whole number of 16-byte vectors (n_elems = %lld)",
                (long long)n_elems);
  B200Q_REQUIRE(max_message_bytes % 16 == 0 && n_elems * 2 <= max_message_bytes, B200Q_EINVAL,
                "message of %lld bytes exceeds the slot size %lld", (long long)n_elems * 2,
                (long long)max_message_bytes);
  B200Q_REQUIRE(((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(in)) & 15) == 0,
                B200Q_EINVAL, "in / out must be aligned to 16 bytes");
  if (n_elems == 0) return B200Q_OK;
  ar::ArParams p;
  p.bufs = peer_bufs;
  p.flags = peer_flags;
  p.epochs = epochs;
  p.in = in;
  p.out = out;
  p.slot_bytes = max_message_bytes;
  p.n_vec = n_elems / 8;
  p.rank = rank;
  p.world = world;
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
  if (dtype == B200Q_F16)
    B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, ar::allreduce_oneshot_kernel<half>, p));
  else
    B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, ar::allreduce_oneshot_kernel<__nv_bfloat16>, p));
  note_launch();
  return B200Q_OK;
}
