// Projection GEMM of the fused multi-head-attention forward for the shapes and types the tcgen05 kernel does not take
// (fp32 operands, head sizes other than 64 / 128, model widths that are not a multiple of 128):
//   C[b, s, n] = sum_k A[b, s, k] * W[k, n]
// fp32 FFMA arithmetic, any sizes, the same head-major scatter in the epilogue (column n lands in head n / head_dim).
// A 64 x 64 tile per CTA of 256 threads, 16-wide K slices through shared memory, a 4 x 4 micro-tile per thread; every
// output element is summed by one thread in ascending k, so results do not depend on the launch geometry.
//
// This is the exact route of the engine's MultiHeadAttentionForward: with fp32 tensors it meets the 1e-4 bound of the
// reference's own tests of the fused call (tests/AiDotNet.Tensors.Tests/Engines/MultiHeadAttentionForwardTests.cs:123),
// including their head sizes of 2 to 8 (src/AiDotNet.Tensors/Engines/CpuEngine.MultiHeadAttention.cs:155-338).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace aidn {
namespace {

constexpr int kTile = 64;
constexpr int kSlice = 16;

template <typename T>
__device__ __forceinline__ float to_f32(T v) {
  return static_cast<float>(v);
}

template <typename T>
__device__ __forceinline__ void store_as(void* base, int64_t off, float v, bool f32) {
  if (f32) static_cast<float*>(base)[off] = v;
  else static_cast<T*>(base)[off] = static_cast<T>(v);
}
template <>
__device__ __forceinline__ void store_as<float>(void* base, int64_t off, float v, bool) {
  static_cast<float*>(base)[off] = v;
}

struct GenericGemmParams {
  const void* a;
  const void* w[3];
  void* c[3];
  int64_t cs[3];
  int64_t rows;   // batch * seq
  int32_t seq, k, n, head_dim;
  int32_t out_f32;
};

template <typename T>
__global__ void __launch_bounds__(256) proj_gemm_generic_kernel(const GenericGemmParams g) {
  __shared__ float a_s[kSlice][kTile + 4];   // a_s[kk][row]: transposed on the way in
  __shared__ float w_s[kSlice][kTile + 4];
  const int mat = blockIdx.z;
  const T* a = static_cast<const T*>(g.a);
  const T* w = static_cast<const T*>(mat == 0 ? g.w[0] : (mat == 1 ? g.w[1] : g.w[2]));   // no indexed copy of the parameters
  const int64_t row0 = (int64_t)blockIdx.y * kTile;
  const int col0 = blockIdx.x * kTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < g.k; k0 += kSlice) {
    // A slice: 64 rows x 16 k; thread t reads row t / 4, k offsets 4 * (t % 4) ..
    {
      const int r = threadIdx.x >> 2, kq = (threadIdx.x & 3) * 4;
      const int64_t row = row0 + r;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kk = k0 + kq + i;
        a_s[kq + i][r] = (row < g.rows && kk < g.k) ? to_f32(a[row * g.k + kk]) : 0.f;
      }
    }
    // W slice: 16 k x 64 columns; thread t reads k row t / 16, columns 4 * (t % 16) ..
    {
      const int kr = threadIdx.x >> 4, cq = (threadIdx.x & 15) * 4;
      const int kk = k0 + kr;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = col0 + cq + i;
        w_s[kr][cq + i] = (kk < g.k && col < g.n) ? to_f32(w[(int64_t)kk * g.n + col]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSlice; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[i] = a_s[kk][ty * 4 + i];
        wv[i] = w_s[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
  void* c = mat == 0 ? g.c[0] : (mat == 1 ? g.c[1] : g.c[2]);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t row = row0 + ty * 4 + i;
    if (row >= g.rows) continue;
    const int64_t b = row / g.seq, s = row - b * g.seq;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = col0 + tx * 4 + j;
      if (col >= g.n) continue;
      const int h = col / g.head_dim;
      const int64_t off = b * g.cs[0] + (int64_t)h * g.cs[1] + s * g.cs[2] + (col - h * g.head_dim);
      store_as<T>(c, off, acc[i][j], g.out_f32 != 0);
    }
  }
}

template <typename T>
cudaError_t launch_t(const ProjGemm& p, cudaStream_t stream) {
  GenericGemmParams g;
  g.a = p.a;
  for (int i = 0; i < 3; ++i) {
    g.w[i] = p.w[i < p.num_mats ? i : 0];
    g.c[i] = p.c[i < p.num_mats ? i : 0];
    g.cs[i] = p.c_stride[i];
  }
  g.rows = p.batch * p.seq;
  g.seq = (int)p.seq;
  g.k = (int)p.k;
  g.n = (int)p.n;
  g.head_dim = p.head_dim;
  g.out_f32 = p.out_f32 ? 1 : 0;
  const int64_t row_tiles = (g.rows + kTile - 1) / kTile;
  if (row_tiles > 65535) return cudaErrorInvalidValue;
  dim3 grid((unsigned)((p.n + kTile - 1) / kTile), (unsigned)row_tiles, (unsigned)p.num_mats);
  proj_gemm_generic_kernel<T><<<grid, 256, 0, stream>>>(g);
  return cudaGetLastError();
}

}  // namespace

bool proj_gemm_generic_supported(const ProjGemm& g, const char** why) {
  if (g.num_mats < 1 || g.num_mats > 3) { *why = "projection GEMM takes 1 to 3 weight matrices"; return false; }
  if (g.batch <= 0 || g.seq <= 0 || g.k <= 0 || g.n <= 0 || g.head_dim <= 0 || g.n % g.head_dim != 0) {
    *why = "projection GEMM: dimensions must be positive and heads * head_dim == n";
    return false;
  }
  if (g.seq > 0x7fffffffll || g.k > 0x7fffffffll || g.n > 0x7fffffffll || (g.batch * g.seq + kTile - 1) / kTile > 65535) {
    *why = "projection GEMM: more than 65535 * 64 rows or a dimension above 2^31";
    return false;
  }
  return true;
}

cudaError_t launch_proj_gemm_generic(const ProjGemm& g, int dtype, cudaStream_t stream) {
  if (dtype == AIDN_F32) return launch_t<float>(g, stream);
  if (dtype == AIDN_BF16) return launch_t<__nv_bfloat16>(g, stream);
  return launch_t<__half>(g, stream);
}

}  // namespace aidn
