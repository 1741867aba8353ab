// The element-wise steps on either side of the row-parallel quantized GEMM:
//   * fused_add_rms_norm: residual += x; x = rmsnorm(residual) * weight, optionally with
//     the tensor-parallel all-reduce of x in front (one kernel: partial sums go to the
//     peers as flagged packets, see ar_link.cuh, and each block normalises the row it
//     has just reduced);
//   * silu_and_mul: out = silu(x[:, :d]) * x[:, d:].
// Rounding points follow the reference kernels so that results can be compared
// bit for bit up to the order of the fp32 sum of squares:
//   csrc/layernorm_kernels.cu:60-149 (z = x + r rounded to 16 bits, variance from the
//   rounded z in fp32, (T)(z * rstd) rounded, then * weight rounded) and
//   csrc/activation_kernels.cu:22-38 ((T)(x / (1 + exp(-x))) rounded, then * y rounded).
// The all-reduce in front rounds the sum to 16 bits first, as the separate
// all-reduce kernel does.
#include "ar_link.cuh"
#include "common.cuh"

namespace b200q {

int check_link(void* const* peer_bufs, uint32_t* state, int rank, int world,
               int64_t max_message_bytes, ArLink* link);

namespace ew {

constexpr int kNormThreads = 512;

struct NormParams {
  void* x;            // [M, N] in: (partial) input, out: normalised; row stride ldx elements
  int64_t ldx;
  void* residual;     // [M, N] contiguous, in/out; may be null (plain rms_norm of x)
  const void* weight; // [N]
  float eps;
  int m, n;
  ArLink link;        // world == 0: no all-reduce
};

template <typename T>
__device__ __forceinline__ float lo_f(uint32_t v) { return Pair<T>::to_float((uint16_t)(v & 0xffffu)); }
template <typename T>
__device__ __forceinline__ float hi_f(uint32_t v) { return Pair<T>::to_float((uint16_t)(v >> 16)); }
template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  return (uint32_t)Pair<T>::from_float(a) | ((uint32_t)Pair<T>::from_float(b) << 16);
}

// One block per row; a thread handles 16-byte vectors v = tid, tid + blockDim, ...
template <typename T>
__global__ void __launch_bounds__(kNormThreads, 1) fused_add_rms_norm_kernel(const NormParams p) {
  __shared__ float s_part[kNormThreads / 32];
  __shared__ float s_rstd;
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int row = blockIdx.x;
  const int vecs = p.n / 8;
  uint4* xrow = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.x) + (size_t)row * p.ldx);
  uint4* rrow = p.residual
                    ? reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.residual) + (size_t)row * p.n)
                    : nullptr;
  const ArLink& l = p.link;
  uint32_t call = 0, flag = 0;
  long long parity_off = 0;
  if (l.world) {
    call = ar_ld_volatile(l.state);
    flag = ar_flag(call);
    parity_off = (long long)(call & 1) * l.world * l.slot_bytes;
    // push this rank's partial row to every peer (a vector = four packets = 32 bytes)
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      const uint4 x = xrow[v];
      const size_t pkt = ((size_t)row * vecs + v) * 32;
      for (int r = 0; r < l.world; ++r) {
        if (r == l.rank) continue;
        char* dst = static_cast<char*>(l.bufs[r]) + parity_off + l.rank * l.slot_bytes + pkt;
        ar_put2(dst, x.x, x.y, flag);
        ar_put2(dst + 16, x.z, x.w, flag);
      }
    }
  }
  const char* mybuf = l.world ? static_cast<const char*>(l.bufs[l.rank]) + parity_off : nullptr;
  float ss = 0.f;
  bool ok = true;
  for (int v = threadIdx.x; v < vecs && ok; v += blockDim.x) {
    uint4 x = xrow[v];
    if (l.world) {
      // all-reduce: fp32 sum in rank order, one rounding (what the separate kernel stores)
      uint32_t d[kArMaxWorld][4];
      if (!ar_collect<4>(l, mybuf, ((size_t)row * vecs + v) * 32, flag, d)) {
        ok = false;
        break;
      }
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
      for (int r = 0; r < kArMaxWorld; ++r) {
        if (r < l.world) {
          const bool me = r == l.rank;
          const uint32_t w0 = me ? x.x : d[r][0], w1 = me ? x.y : d[r][1];
          const uint32_t w2 = me ? x.z : d[r][2], w3 = me ? x.w : d[r][3];
          acc[0] += lo_f<T>(w0); acc[1] += hi_f<T>(w0); acc[2] += lo_f<T>(w1); acc[3] += hi_f<T>(w1);
          acc[4] += lo_f<T>(w2); acc[5] += hi_f<T>(w2); acc[6] += lo_f<T>(w3); acc[7] += hi_f<T>(w3);
        }
      }
      x.x = pack2<T>(acc[0], acc[1]); x.y = pack2<T>(acc[2], acc[3]);
      x.z = pack2<T>(acc[4], acc[5]); x.w = pack2<T>(acc[6], acc[7]);
    }
    if (rrow) {
      const uint4 r = rrow[v];
      x.x = pack2<T>(lo_f<T>(x.x) + lo_f<T>(r.x), hi_f<T>(x.x) + hi_f<T>(r.x));
      x.y = pack2<T>(lo_f<T>(x.y) + lo_f<T>(r.y), hi_f<T>(x.y) + hi_f<T>(r.y));
      x.z = pack2<T>(lo_f<T>(x.z) + lo_f<T>(r.z), hi_f<T>(x.z) + hi_f<T>(r.z));
      x.w = pack2<T>(lo_f<T>(x.w) + lo_f<T>(r.w), hi_f<T>(x.w) + hi_f<T>(r.w));
      rrow[v] = x;
    } else {
      xrow[v] = x;  // the reduced row, normalised in place below
    }
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = lo_f<T>(w[e]), b = hi_f<T>(w[e]);
      ss += a * a + b * b;
    }
  }
  // block sum of squares
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_part[w];
    s_rstd = rsqrtf(tot / (float)p.n + p.eps);
  }
  __syncthreads();
  const float rstd = s_rstd;
  const uint4* wrow = static_cast<const uint4*>(p.weight);
  const uint4* zrow = rrow ? rrow : xrow;
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    const uint4 z = zrow[v];
    const uint4 g = wrow[v];
    const uint32_t zw[4] = {z.x, z.y, z.z, z.w}, gw[4] = {g.x, g.y, g.z, g.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // (T)(z * rstd), then the 16-bit product with the weight
      const float a = Pair<T>::to_float(Pair<T>::from_float(lo_f<T>(zw[e]) * rstd));
      const float b = Pair<T>::to_float(Pair<T>::from_float(hi_f<T>(zw[e]) * rstd));
      o[e] = pack2<T>(a * lo_f<T>(gw[e]), b * hi_f<T>(gw[e]));
    }
    xrow[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (l.world) {
    __syncthreads();
    if (threadIdx.x == 0) ar_arrive(l, call, gridDim.x);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) silu_and_mul_kernel(const uint16_t* __restrict__ in,
                                                           uint16_t* __restrict__ out, int64_t m,
                                                           int d) {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int vecs = d / 8;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= m * vecs) return;
  const int64_t row = idx / vecs;
  const int v = (int)(idx % vecs);
  const uint4 x = reinterpret_cast<const uint4*>(in + row * 2 * d)[v];
  const uint4 y = reinterpret_cast<const uint4*>(in + row * 2 * d + d)[v];
  const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
  uint32_t o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float a = lo_f<T>(xw[e]), b = hi_f<T>(xw[e]);
    const float sa = Pair<T>::to_float(Pair<T>::from_float(a / (1.0f + expf(-a))));
    const float sb = Pair<T>::to_float(Pair<T>::from_float(b / (1.0f + expf(-b))));
    o[e] = pack2<T>(sa * lo_f<T>(yw[e]), sb * hi_f<T>(yw[e]));
  }
  reinterpret_cast<uint4*>(out + row * d)[v] = make_uint4(o[0], o[1], o[2], o[3]);
}

template <typename K, typename... Args>
int launch_pdl(K kernel, dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, args...));
  note_launch();
  return B200Q_OK;
}

int launch_norm(NormParams p, int dtype, cudaStream_t stream) {
  B200Q_REQUIRE(dtype == B200Q_F16 || dtype == B200Q_BF16, B200Q_EINVAL, "dtype must be fp16/bf16");
  B200Q_REQUIRE(p.m >= 0 && p.n > 0 && p.n % 8 == 0, B200Q_EINVAL,
                "hidden size %d must be a positive multiple of 8", p.n);
  B200Q_REQUIRE(p.x && p.weight, B200Q_EINVAL, "null pointer");
  B200Q_REQUIRE(p.ldx >= p.n && p.ldx % 8 == 0, B200Q_EINVAL, "row stride must be a multiple of 8");
  B200Q_REQUIRE(((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.weight) |
                  reinterpret_cast<uintptr_t>(p.residual)) & 15) == 0,
                B200Q_EINVAL, "tensors must be aligned to 16 bytes");
  if (p.m == 0) return B200Q_OK;
  int threads = (p.n / 8 + 31) / 32 * 32;
  if (threads > kNormThreads) threads = kNormThreads;
  if (dtype == B200Q_F16)
    return launch_pdl(fused_add_rms_norm_kernel<half>, dim3(p.m), dim3(threads), stream, p);
  return launch_pdl(fused_add_rms_norm_kernel<__nv_bfloat16>, dim3(p.m), dim3(threads), stream, p);
}

}  // namespace ew
}  // namespace b200q

using namespace b200q;

extern "C" int b200q_fused_add_rms_norm(void* input, int64_t ld_input, void* residual,
                                        const void* weight, float epsilon, int64_t num_tokens,
                                        int64_t hidden_size, int dtype, b200q_stream_t stream) {
  B200Q_REQUIRE(num_tokens >= 0 && num_tokens < (1ll << 31) && hidden_size < (1ll << 31),
                B200Q_EINVAL, "size out of range");
  ew::NormParams p = {};
  p.x = input;
  p.ldx = ld_input;
  p.residual = residual;
  p.weight = weight;
  p.eps = epsilon;
  p.m = (int)num_tokens;
  p.n = (int)hidden_size;
  return ew::launch_norm(p, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int b200q_all_reduce_fused_add_rms_norm(void* const* peer_bufs, uint32_t* state, int rank,
                                                   int world, int64_t max_message_bytes, void* input,
                                                   void* residual, const void* weight, float epsilon,
                                                   int64_t num_tokens, int64_t hidden_size, int dtype,
                                                   b200q_stream_t stream) {
  B200Q_REQUIRE(num_tokens >= 0 && num_tokens < (1ll << 31) && hidden_size < (1ll << 31),
                B200Q_EINVAL, "size out of range");
  ew::NormParams p = {};
  int rc = check_link(peer_bufs, state, rank, world, max_message_bytes, &p.link);
  if (rc != B200Q_OK) return rc;
  B200Q_REQUIRE(num_tokens * hidden_size * 2 <= max_message_bytes, B200Q_EINVAL,
                "message of %lld bytes exceeds the largest message %lld",
                (long long)(num_tokens * hidden_size * 2), (long long)max_message_bytes);
  p.x = input;
  p.ldx = hidden_size;
  p.residual = residual;
  p.weight = weight;
  p.eps = epsilon;
  p.m = (int)num_tokens;
  p.n = (int)hidden_size;
  return ew::launch_norm(p, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int b200q_silu_and_mul(void* out, const void* input, int64_t num_tokens, int64_t d,
                                  int dtype, b200q_stream_t stream) {
  B200Q_REQUIRE(dtype == B200Q_F16 || dtype == B200Q_BF16, B200Q_EINVAL, "dtype must be fp16/bf16");
  B200Q_REQUIRE(num_tokens >= 0 && d > 0 && d % 8 == 0 && d < (1ll << 31), B200Q_EINVAL,
                "d = %lld must be a positive multiple of 8", (long long)d);
  B200Q_REQUIRE(out && input, B200Q_EINVAL, "null pointer");
  B200Q_REQUIRE(((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(input)) & 15) == 0,
                B200Q_EINVAL, "tensors must be aligned to 16 bytes");
  if (num_tokens == 0) return B200Q_OK;
  const int64_t threads = num_tokens * (d / 8);
  const dim3 grid((unsigned)((threads + 255) / 256));
  if (dtype == B200Q_F16)
    return ew::launch_pdl(ew::silu_and_mul_kernel<half>, grid, dim3(256), static_cast<cudaStream_t>(stream),
                          static_cast<const uint16_t*>(input), static_cast<uint16_t*>(out), num_tokens,
                          (int)d);
  return ew::launch_pdl(ew::silu_and_mul_kernel<__nv_bfloat16>, grid, dim3(256),
                        static_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(input),
                        static_cast<uint16_t*>(out), num_tokens, (int)d);
}
