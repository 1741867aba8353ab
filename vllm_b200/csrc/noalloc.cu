// b200q_marlin_gemm_noalloc: the mixed-precision GEMM for callers that cannot
// allocate device memory.
//
// Some callers of this library run where no allocator is available to them: a
// plugin invoked from inside a host framework's pre-planned memory arena, a
// callback running while a stream is being captured, or a process whose device
// memory is owned entirely by another component.  b200q_marlin_gemm needs
// scratch (fp32 partial sums of split column slices, and the gathered
// activations of act-order layers) and normally makes the caller supply it.
// This variant supplies it from a fixed array that is part of the library
// image, so the call itself allocates nothing.
#include "common.cuh"

namespace b200q {
namespace {

// 16 MiB of device memory per GPU that loads the library, held until the
// process exits.  Enough for every decode-regime problem with
// b200q_marlin_gemm_scratch_bytes(...) <= this size, e.g. N up to 32768 without
// act-order, or N = 28672, K = 4096, M <= 64 with it (see the check below).
constexpr size_t kNoAllocBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// Device address of the array, per device.  In host code the array's name is
// only a handle for the runtime, never an address a kernel may use; the
// address comes from cudaGetSymbolAddress with the right device current.
// Two host threads making the first call on a device race on this plain store;
// the race is benign, both store the same address.  An address is valid for the
// life of the device's primary context: after cudaDeviceReset the library must be
// reloaded (the cached address would be stale).
void* g_scratch_addr[64] = {};

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" size_t b200q_marlin_gemm_noalloc_max_scratch(void) { return kNoAllocBytes; }

extern "C" int b200q_marlin_gemm_noalloc(const void* a, int64_t lda, const uint32_t* b_q_weight,
                                         const void* b_scales, const uint32_t* b_zeros,
                                         const int32_t* g_idx, const int32_t* perm,
                                         const void* b_bias, void* c, int32_t* workspace,
                                         int64_t workspace_len, int64_t b_q_type_id, int a_dtype,
                                         int64_t size_m, int64_t size_n, int64_t size_k,
                                         int64_t num_groups, unsigned flags,
                                         b200q_stream_t stream) {
  int dev = 0;
  B200Q_CUDA_OK(cudaGetDevice(&dev));
  B200Q_REQUIRE(dev >= 0 && dev < 64, B200Q_EUNSUPPORTED, "device index %d out of range", dev);
  if (g_scratch_addr[dev] == nullptr) {
    // first call on this device: resolve the array's device address (do this
    // once, outside any stream capture)
    void* ptr = nullptr;
    B200Q_CUDA_OK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    B200Q_REQUIRE(ptr != nullptr, B200Q_ECUDA, "cudaGetSymbolAddress returned a null address");
    g_scratch_addr[dev] = ptr;
  }
  // The array used is the current device's: the output must live there too (a stream
  // or tensors of another GPU would run against the wrong device's scratch).
  cudaPointerAttributes attr;
  if (c != nullptr && cudaPointerGetAttributes(&attr, c) == cudaSuccess &&
      attr.type == cudaMemoryTypeDevice)
    B200Q_REQUIRE(attr.device == dev, B200Q_EINVAL,
                  "c lives on device %d but device %d is current", attr.device, dev);
  const size_t need =
      b200q_marlin_gemm_scratch_bytes(size_m, size_n, size_k, g_idx != nullptr ? 1 : 0);
  B200Q_REQUIRE(need <= kNoAllocBytes, B200Q_ESCRATCH,
                "problem [M=%lld, N=%lld, K=%lld] needs %zu bytes of scratch; the built-in scratch "
                "of b200q_marlin_gemm_noalloc holds %zu - use b200q_marlin_gemm with caller scratch",
                (long long)size_m, (long long)size_n, (long long)size_k, need, kNoAllocBytes);
  // Nothing in the scratch has to start at zero: partial sums are fully written
  // before they are read, and the counters live in the caller's workspace.
  return b200q_marlin_gemm(a, lda, b_q_weight, b_scales, b_zeros, g_idx, perm, b_bias, c,
                           g_scratch_addr[dev], kNoAllocBytes, workspace, workspace_len,
                           b_q_type_id, a_dtype, size_m, size_n, size_k, num_groups, flags, stream);
}
