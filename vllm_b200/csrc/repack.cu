// Checkpoint-format -> Marlin tile layout re-tiling, and the activation column
// gather used by act-order.  Pure integer / byte movement: HBM-bound.
//
// Output layout (int32 [K/16, N*16/pf]): for k-tile kt and 64-column tile nt the
// tile's words are contiguous at ((kt * N/64) + nt) * W, W = 128 (4-bit) or 256
// (8-bit).  Inside a tile, lane = 4*c + q (c = 0..7, q = 0..3) owns column c
// (+8 for block 1) of each 16-column sub-tile `sub` and rows 2q + {0,1,8,9}:
//   4-bit: word lane*4 + sub, nibble t holds (row, block) =
//          t:0 (2q,0) 1 (2q+8,0) 2 (2q,1) 3 (2q+8,1) 4 (2q+1,0) 5 (2q+9,0) 6 (2q+1,1) 7 (2q+9,1)
//   8-bit: word lane*8 + sub*2 + block, byte t holds row 2q + {0, 8, 1, 9}[t]
#include "common.cuh"

namespace b200q {

namespace {

constexpr int kRepackThreads = 256;
constexpr int kRepackTiles = 4;  // 64-column tiles per block -> 256 columns

// Source element accessors: code of (k, n) from the staged rows in shared memory.
// Staging holds, for each of the 16 rows of the k-tile, the packed source words
// that contain the block's 256 columns.

template <int BITS, bool HAS_PERM>
__global__ void __launch_bounds__(kRepackThreads)
gptq_repack_kernel(const uint32_t* __restrict__ in, const int32_t* __restrict__ perm,
                   uint32_t* __restrict__ out, int size_k, int size_n) {
  constexpr int PF = 32 / BITS;
  constexpr int W = 16 * 64 / PF;              // words per output tile
  constexpr int COLS = 64 * kRepackTiles;      // columns per block
  // staged[r][n]: the packed word holding row r of the k-tile for column n, and
  // shift[r]: bit offset of that row inside the word
  __shared__ uint32_t staged[16][COLS];
  __shared__ int shift[16];

  const int n_tiles = size_n / 64;
  const int kt = blockIdx.y;
  const int nt0 = blockIdx.x * kRepackTiles;
  const int tiles_here = min(kRepackTiles, n_tiles - nt0);
  const int cols_here = tiles_here * 64;
  const int n0 = nt0 * 64;

  if (HAS_PERM) {
    // every one of the 16 rows may come from a different packed row
    for (int i = threadIdx.x; i < 16 * COLS; i += kRepackThreads) {
      int r = i / COLS, n = i % COLS;
      if (n < cols_here) {
        int src_k = perm[kt * 16 + r];
        staged[r][n] = in[(size_t)(src_k / PF) * size_n + n0 + n];
        if (n == 0) shift[r] = (src_k % PF) * BITS;
      }
    }
  } else {
    // 16 rows live in 16/PF packed rows
    constexpr int SRC_ROWS = 16 / PF;
    for (int i = threadIdx.x; i < SRC_ROWS * COLS; i += kRepackThreads) {
      int sr = i / COLS, n = i % COLS;
      if (n < cols_here) staged[sr][n] = in[(size_t)(kt * SRC_ROWS + sr) * size_n + n0 + n];
    }
  }
  __syncthreads();

  auto code = [&](int row, int col) -> uint32_t {
    if (HAS_PERM) return (staged[row][col] >> shift[row]) & ((1u << BITS) - 1);
    return (staged[row / PF][col] >> ((row % PF) * BITS)) & ((1u << BITS) - 1);
  };

  uint32_t* out_tile = out + ((size_t)kt * n_tiles + nt0) * W;
  for (int w = threadIdx.x; w < tiles_here * W; w += kRepackThreads) {
    const int tile = w / W, wi = w % W;
    uint32_t word = 0;
    if (BITS == 4) {
      const int lane = wi >> 2, sub = wi & 3;
      const int c = lane >> 2, q = lane & 3;
      const int col = tile * 64 + sub * 16 + c;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const int row = 2 * q + (t >> 2) + 8 * (t & 1);
        const int blk = (t >> 1) & 1;
        word |= code(row, col + 8 * blk) << (4 * t);
      }
    } else {
      const int lane = wi >> 3, sub = (wi >> 1) & 3, blk = wi & 1;
      const int c = lane >> 2, q = lane & 3;
      const int col = tile * 64 + sub * 16 + c + 8 * blk;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int row = 2 * q + (t >> 1) + 8 * (t & 1);
        word |= code(row, col) << (8 * t);
      }
    }
    out_tile[w] = word;
  }
}

template <int BITS>
__global__ void __launch_bounds__(kRepackThreads)
awq_repack_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, int size_k,
                  int size_n) {
  constexpr int PF = 32 / BITS;
  constexpr int W = 16 * 64 / PF;
  constexpr int COLS = 64 * kRepackTiles;
  constexpr int WORDS = COLS / PF;  // packed source words per row of the block
  __shared__ uint32_t staged[16][WORDS];

  const int n_tiles = size_n / 64;
  const int kt = blockIdx.y;
  const int nt0 = blockIdx.x * kRepackTiles;
  const int tiles_here = min(kRepackTiles, n_tiles - nt0);
  const int words_here = tiles_here * 64 / PF;
  const int in_stride = size_n / PF;
  const int w0 = nt0 * 64 / PF;

  for (int i = threadIdx.x; i < 16 * WORDS; i += kRepackThreads) {
    int r = i / WORDS, w = i % WORDS;
    if (w < words_here) staged[r][w] = in[(size_t)(kt * 16 + r) * in_stride + w0 + w];
  }
  __syncthreads();

  // AWQ stores column 8w+i of a 4-bit word at nibble [0,4,1,5,2,6,3,7][i]
  // (the inverse of its [0,2,4,6,1,3,5,7] interleave); 8-bit: [0,2,1,3][i].
  auto code = [&](int row, int col) -> uint32_t {
    const int i = col % PF;
    const int pos = (BITS == 4) ? ((i >> 1) + 4 * (i & 1)) : (((i & 1) << 1) | (i >> 1));
    return (staged[row][col / PF] >> (pos * BITS)) & ((1u << BITS) - 1);
  };

  uint32_t* out_tile = out + ((size_t)kt * n_tiles + nt0) * W;
  for (int w = threadIdx.x; w < tiles_here * W; w += kRepackThreads) {
    const int tile = w / W, wi = w % W;
    uint32_t word = 0;
    if (BITS == 4) {
      const int lane = wi >> 2, sub = wi & 3;
      const int c = lane >> 2, q = lane & 3;
      const int col = tile * 64 + sub * 16 + c;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const int row = 2 * q + (t >> 2) + 8 * (t & 1);
        const int blk = (t >> 1) & 1;
        word |= code(row, col + 8 * blk) << (4 * t);
      }
    } else {
      const int lane = wi >> 3, sub = (wi >> 1) & 3, blk = wi & 1;
      const int c = lane >> 2, q = lane & 3;
      const int col = tile * 64 + sub * 16 + c + 8 * blk;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int row = 2 * q + (t >> 1) + 8 * (t & 1);
        word |= code(row, col) << (8 * t);
      }
    }
    out_tile[w] = word;
  }
}

// out[m, k] = a[m, perm[k]].  One block per row (grid-stride); the row is staged
// in shared memory with coalesced 16-byte loads when it fits, so both the read
// and the write of every row are coalesced.
__global__ void __launch_bounds__(256)
permute_cols_kernel(const uint16_t* __restrict__ a, int64_t lda, const int32_t* __restrict__ perm,
                    uint16_t* __restrict__ out, int size_m, int size_k, int stage_in_smem) {
  extern __shared__ __align__(16) uint16_t row_buf[];
  // 16-byte stores and permutation loads need K % 8 == 0 and aligned bases
  const bool vec_out = (size_k % 8 == 0) && ((reinterpret_cast<uintptr_t>(perm) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  // the GEMM that follows may start prefetching its weights right away
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  for (int m = blockIdx.x; m < size_m; m += gridDim.x) {
    const uint16_t* src = a + (size_t)m * lda;
    uint16_t* dst = out + (size_t)m * size_k;
    if (stage_in_smem) {
      // lda % 8 == 0 and a 16 B aligned base make every row 16 B aligned
      const int vecs = size_k / 8;
      for (int i = threadIdx.x; i < vecs; i += blockDim.x)
        reinterpret_cast<uint4*>(row_buf)[i] = reinterpret_cast<const uint4*>(src)[i];
      for (int i = vecs * 8 + threadIdx.x; i < size_k; i += blockDim.x) row_buf[i] = src[i];
      __syncthreads();
      if (vec_out) {
        // eight outputs per thread: two 16-byte loads of the permutation, one 16-byte store
        for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
          const int4 p0 = __ldg(reinterpret_cast<const int4*>(perm) + 2 * i);
          const int4 p1 = __ldg(reinterpret_cast<const int4*>(perm) + 2 * i + 1);
          uint4 v;
          v.x = (uint32_t)row_buf[p0.x] | ((uint32_t)row_buf[p0.y] << 16);
          v.y = (uint32_t)row_buf[p0.z] | ((uint32_t)row_buf[p0.w] << 16);
          v.z = (uint32_t)row_buf[p1.x] | ((uint32_t)row_buf[p1.y] << 16);
          v.w = (uint32_t)row_buf[p1.z] | ((uint32_t)row_buf[p1.w] << 16);
          reinterpret_cast<uint4*>(dst)[i] = v;
        }
      } else {
        for (int k = threadIdx.x; k < size_k; k += blockDim.x) dst[k] = row_buf[perm[k]];
      }
      __syncthreads();
    } else {
      for (int k = threadIdx.x; k < size_k; k += blockDim.x) dst[k] = src[perm[k]];
    }
  }
}

// Few rows (decode): one thread per 8 output elements, many blocks per row, so
// that the gather is spread over the whole GPU; the reads hit L2.
__global__ void __launch_bounds__(256)
permute_cols_small_kernel(const uint16_t* __restrict__ a, int64_t lda,
                          const int32_t* __restrict__ perm, uint16_t* __restrict__ out, int size_k) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int m = blockIdx.y;
  const int k0 = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (k0 >= size_k) return;
  const uint16_t* src = a + (size_t)m * lda;
  // the permutation is a constant of the layer: fetch it while the kernel before this one
  // in the stream drains, then wait for that kernel (it produced `a` and may still read `out`)
  const int4 p0 = *reinterpret_cast<const int4*>(perm + k0);
  const int4 p1 = *reinterpret_cast<const int4*>(perm + k0 + 4);
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  uint4 v;
  v.x = (uint32_t)src[p0.x] | ((uint32_t)src[p0.y] << 16);
  v.y = (uint32_t)src[p0.z] | ((uint32_t)src[p0.w] << 16);
  v.z = (uint32_t)src[p1.x] | ((uint32_t)src[p1.y] << 16);
  v.w = (uint32_t)src[p1.z] | ((uint32_t)src[p1.w] << 16);
  *reinterpret_cast<uint4*>(out + (size_t)m * size_k + k0) = v;
}

}  // namespace

int launch_permute_cols(const void* a, int64_t lda, const int32_t* perm, void* out, int64_t size_m,
                        int64_t size_k, cudaStream_t stream) {
  if (size_m == 0 || size_k == 0) return B200Q_OK;
  if (size_m <= 64 && size_k % 8 == 0 && (reinterpret_cast<uintptr_t>(perm) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    dim3 grid((unsigned)((size_k / 8 + 255) / 256), (unsigned)size_m);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    B200Q_CUDA_OK(cudaLaunchKernelEx(&cfg, permute_cols_small_kernel, static_cast<const uint16_t*>(a),
                                     lda, perm, static_cast<uint16_t*>(out), (int)size_k));
    note_launch();
    return B200Q_OK;
  }
  const size_t row_bytes = (size_t)size_k * 2;
  const bool aligned = (lda % 8 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
  int stage = aligned && row_bytes <= (size_t)device_max_smem_optin() - 1024;
  size_t smem = stage ? row_bytes : 0;
  if (smem > 48 * 1024)
    B200Q_CUDA_OK(cudaFuncSetAttribute(permute_cols_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int blocks = (int)(size_m < 4 * (int64_t)device_sm_count() ? size_m : 4 * device_sm_count());
  permute_cols_kernel<<<blocks, 256, smem, stream>>>(
      static_cast<const uint16_t*>(a), lda, perm, static_cast<uint16_t*>(out), (int)size_m,
      (int)size_k, stage);
  note_launch();
  B200Q_CUDA_OK(cudaGetLastError());
  return B200Q_OK;
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_gptq_marlin_repack(const uint32_t* b_q_weight, const int32_t* perm,
                                        uint32_t* out, int64_t size_k, int64_t size_n, int num_bits,
                                        b200q_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200Q_REQUIRE(num_bits == 4 || num_bits == 8, B200Q_EINVAL, "num_bits must be 4 or 8. Got = %d",
                num_bits);
  B200Q_REQUIRE(size_k >= 0 && size_k % 16 == 0, B200Q_EINVAL,
                "size_k = %lld is not divisible by tile_k_size = 16", (long long)size_k);
  B200Q_REQUIRE(size_n >= 0 && size_n % 64 == 0, B200Q_EINVAL,
                "size_n = %lld is not divisible by tile_n_size = 64", (long long)size_n);
  B200Q_REQUIRE(size_k / 16 <= 65535, B200Q_EUNSUPPORTED, "size_k = %lld too large",
                (long long)size_k);
  if (size_k == 0 || size_n == 0) return B200Q_OK;
  B200Q_REQUIRE(b_q_weight && out, B200Q_EINVAL, "null tensor pointer");
  dim3 grid((unsigned)((size_n / 64 + kRepackTiles - 1) / kRepackTiles), (unsigned)(size_k / 16));
  if (num_bits == 4) {
    if (perm)
      gptq_repack_kernel<4, true><<<grid, kRepackThreads, 0, stream>>>(b_q_weight, perm, out,
                                                                         (int)size_k, (int)size_n);
    else
      gptq_repack_kernel<4, false><<<grid, kRepackThreads, 0, stream>>>(b_q_weight, perm, out,
                                                                          (int)size_k, (int)size_n);
  } else {
    if (perm)
      gptq_repack_kernel<8, true><<<grid, kRepackThreads, 0, stream>>>(b_q_weight, perm, out,
                                                                         (int)size_k, (int)size_n);
    else
      gptq_repack_kernel<8, false><<<grid, kRepackThreads, 0, stream>>>(b_q_weight, perm, out,
                                                                          (int)size_k, (int)size_n);
  }
  note_launch();
  B200Q_CUDA_OK(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_awq_marlin_repack(const uint32_t* b_q_weight, uint32_t* out, int64_t size_k,
                                       int64_t size_n, int num_bits, b200q_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200Q_REQUIRE(num_bits == 4 || num_bits == 8, B200Q_EINVAL, "num_bits must be 4 or 8. Got = %d",
                num_bits);
  B200Q_REQUIRE(size_k >= 0 && size_k % 16 == 0, B200Q_EINVAL,
                "size_k = %lld is not divisible by tile_k_size = 16", (long long)size_k);
  B200Q_REQUIRE(size_n >= 0 && size_n % 64 == 0, B200Q_EINVAL,
                "size_n = %lld is not divisible by tile_n_size = 64", (long long)size_n);
  B200Q_REQUIRE(size_k / 16 <= 65535, B200Q_EUNSUPPORTED, "size_k = %lld too large",
                (long long)size_k);
  if (size_k == 0 || size_n == 0) return B200Q_OK;
  B200Q_REQUIRE(b_q_weight && out, B200Q_EINVAL, "null tensor pointer");
  dim3 grid((unsigned)((size_n / 64 + kRepackTiles - 1) / kRepackTiles), (unsigned)(size_k / 16));
  if (num_bits == 4)
    awq_repack_kernel<4><<<grid, kRepackThreads, 0, stream>>>(b_q_weight, out, (int)size_k,
                                                               (int)size_n);
  else
    awq_repack_kernel<8><<<grid, kRepackThreads, 0, stream>>>(b_q_weight, out, (int)size_k,
                                                               (int)size_n);
  note_launch();
  B200Q_CUDA_OK(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_permute_cols(const void* a, int64_t lda, const int32_t* perm, void* out,
                                  int64_t size_m, int64_t size_k, b200q_stream_t stream) {
  B200Q_REQUIRE(size_m >= 0 && size_k >= 0, B200Q_EINVAL, "negative size");
  if (size_m == 0 || size_k == 0) return B200Q_OK;
  B200Q_REQUIRE(a && perm && out, B200Q_EINVAL, "null tensor pointer");
  B200Q_REQUIRE(lda >= size_k, B200Q_EINVAL, "lda = %lld < size_k = %lld", (long long)lda,
                (long long)size_k);
  return launch_permute_cols(a, lda, perm, out, size_m, size_k, static_cast<cudaStream_t>(stream));
}
