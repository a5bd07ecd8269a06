// dtype staging kernels: the GPU engine of the reference keeps fp32 buffers and converts to a 16-bit
// type right before a half-precision kernel (src/AiDotNet.Tensors/Engines/DirectGpuTensorEngine.cs:3040-3049
// ResolveToFp16 -> IDirectGpuBackend.ConvertToFp16, IDirectGpuBackend.cs:1890, 1911).
//
// float -> bfloat16 follows BFloat16.FromFloat bit for bit
// (src/AiDotNet.Tensors/NumericOperations/BFloat16.cs:65-84): round to nearest even by adding
// 0x7FFF + lsb, and a NaN keeps its sign and top payload bits and gets the quiet bit (CUDA's own
// conversion would canonicalise NaN to 0x7FFF instead).
#include "common.cuh"

namespace aidn {
namespace {

__device__ __forceinline__ uint16_t f32_to_bf16_bits(float x) {
  const uint32_t bits = __float_as_uint(x);
  if ((bits & 0x7F800000u) == 0x7F800000u && (bits & 0x007FFFFFu) != 0u) return (uint16_t)((bits >> 16) | 0x0040u);
  const uint32_t lsb = (bits >> 16) & 1u;
  return (uint16_t)((bits + 0x7FFFu + lsb) >> 16);
}

// kind: 0 f32->bf16, 1 f32->f16, 2 bf16->f32, 3 f16->f32
template <int KIND>
__global__ void __launch_bounds__(256) cast_kernel(const void* __restrict__ src, void* __restrict__ dst, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    if constexpr (KIND == 0) {
      static_cast<uint16_t*>(dst)[i] = f32_to_bf16_bits(static_cast<const float*>(src)[i]);
    } else if constexpr (KIND == 1) {
      static_cast<__half*>(dst)[i] = __float2half_rn(static_cast<const float*>(src)[i]);
    } else if constexpr (KIND == 2) {
      static_cast<float*>(dst)[i] = __uint_as_float(((uint32_t) static_cast<const uint16_t*>(src)[i]) << 16);
    } else {
      static_cast<float*>(dst)[i] = __half2float(static_cast<const __half*>(src)[i]);
    }
  }
}

// Vectorised body for 16-byte aligned buffers: 8 elements per thread-iteration.
template <int KIND>
__global__ void __launch_bounds__(256) cast_kernel_v8(const void* __restrict__ src, void* __restrict__ dst, int64_t n8) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    if constexpr (KIND == 0 || KIND == 1) {
      const float4 a = static_cast<const float4*>(src)[2 * i];
      const float4 b = static_cast<const float4*>(src)[2 * i + 1];
      const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint16_t lo, hi;
        if constexpr (KIND == 0) {
          lo = f32_to_bf16_bits(f[2 * j]);
          hi = f32_to_bf16_bits(f[2 * j + 1]);
        } else {
          lo = __half_as_ushort(__float2half_rn(f[2 * j]));
          hi = __half_as_ushort(__float2half_rn(f[2 * j + 1]));
        }
        w[j] = (uint32_t)lo | ((uint32_t)hi << 16);
      }
      static_cast<uint4*>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      const uint4 u = static_cast<const uint4*>(src)[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if constexpr (KIND == 2) {
          f[2 * j] = __uint_as_float(w[j] << 16);
          f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        } else {
          f[2 * j] = __half2float(__ushort_as_half((uint16_t)(w[j] & 0xffffu)));
          f[2 * j + 1] = __half2float(__ushort_as_half((uint16_t)(w[j] >> 16)));
        }
      }
      static_cast<float4*>(dst)[2 * i] = make_float4(f[0], f[1], f[2], f[3]);
      static_cast<float4*>(dst)[2 * i + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
  }
}

template <int KIND>
cudaError_t launch_kind(const void* src, void* dst, int64_t n, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  const size_t in_sz = (KIND <= 1) ? 4 : 2, out_sz = (KIND <= 1) ? 2 : 4;
  const bool aligned = ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0);
  const int64_t n8 = aligned ? n / 8 : 0;
  if (n8 > 0) {
    const int64_t blocks = (n8 + 255) / 256;
    const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
    cast_kernel_v8<KIND><<<grid, 256, 0, stream>>>(src, dst, n8);
  }
  const int64_t rest = n - n8 * 8;
  if (rest > 0) {
    const int64_t blocks = (rest + 255) / 256;
    const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
    cast_kernel<KIND><<<grid, 256, 0, stream>>>(static_cast<const char*>(src) + n8 * 8 * in_sz,
                                                static_cast<char*>(dst) + n8 * 8 * out_sz, rest);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_cast(int kind, const void* src, void* dst, int64_t n, cudaStream_t stream) {
  switch (kind) {
    case 0: return launch_kind<0>(src, dst, n, stream);
    case 1: return launch_kind<1>(src, dst, n, stream);
    case 2: return launch_kind<2>(src, dst, n, stream);
    default: return launch_kind<3>(src, dst, n, stream);
  }
}

// ---- paged KV append ----------------------------------------------------------------------------------------------
// The device half of DevicePagedKVCache.Append (src/AiDotNet.Tensors/Engines/DirectGpu/DevicePagedKVCache.cs:113-202):
// new K / V rows [tokens, row_bytes] go to pool rows block_table[(start + t) / block_size] * block_size +
// (start + t) % block_size.  The reference issues one device-to-device copy per run that stays inside a block (two
// per block crossed); here one kernel scatters all rows of K and V with 16-byte copies.  Block bookkeeping (free list,
// reference counts, copy-on-write) stays with the caller.
namespace {
__global__ void __launch_bounds__(256) paged_append_kernel(const uint4* __restrict__ src_k, const uint4* __restrict__ src_v,
                                                           uint4* __restrict__ pool_k, uint4* __restrict__ pool_v,
                                                           const int32_t* __restrict__ block_table, int64_t start,
                                                           int64_t tokens, int block_size, int num_blocks, int row_vecs) {
  const int64_t total = tokens * row_vecs;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / row_vecs;
    const int vec = (int)(idx - t * row_vecs);
    const int64_t pos = start + t;
    const int32_t blk = block_table[pos / block_size];
    if (blk < 0 || blk >= num_blocks) continue;   // an entry outside the pool is skipped, not written through
    const int64_t row = (int64_t)blk * block_size + pos % block_size;
    pool_k[row * row_vecs + vec] = src_k[idx];
    pool_v[row * row_vecs + vec] = src_v[idx];
  }
}
}  // namespace

cudaError_t launch_paged_append(const void* src_k, const void* src_v, void* pool_k, void* pool_v,
                                const int32_t* block_table, int64_t start, int64_t tokens, int block_size, int num_blocks,
                                int64_t row_bytes, cudaStream_t stream) {
  if (tokens <= 0) return cudaSuccess;
  const int row_vecs = (int)(row_bytes / 16);
  const int64_t total = tokens * row_vecs;
  const int64_t blocks = (total + 255) / 256;
  const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
  paged_append_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint4*>(src_k), static_cast<const uint4*>(src_v),
                                                static_cast<uint4*>(pool_k), static_cast<uint4*>(pool_v), block_table,
                                                start, tokens, block_size, num_blocks, row_vecs);
  return cudaGetLastError();
}

}  // namespace aidn
