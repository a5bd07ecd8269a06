// Split-KV decode (seq_q == 1): the HBM-bound half of the attention path.
//
// One CTA streams one chunk of one (batch, kv head)'s keys and values exactly once with 16-byte
// coalesced loads (a key row of D elements is covered by D*sizeof(T)/16 adjacent lanes), serves all
// query heads of that kv head from registers, and writes an un-normalised partial (max, sum, acc[D]);
// a second kernel merges the partials of a (batch, head) by log-sum-exp.  Only keys below kv_len[b]
// (and the causal limit) are touched, so padding costs no bandwidth.
//
// Supersedes flash_decode_partial / flash_decode_reduce of the reference
// (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/Kernels/CudaFlashDecodeKernels.cs:19-81), which run one
// thread per (head, split) with a serial, uncoalesced walk over the cache and take a single sequence.
// The PAGED instantiation reads K/V through a block table and supersedes paged_attention_decode{,_gqa}
// (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/Kernels/CudaPagedAttentionKernels.cs:23-55, :97-124), which run
// one thread per head over the whole sequence.
//
// Scratch layout (fp32): acc[B][Hc][nchunks][D] followed by ml[B][Hc][nchunks][2], Hc = heads of the shard.
#include <mutex>

#include "common.cuh"

namespace aidn {
namespace {

constexpr int kDecWarps = 4;
constexpr int kUnroll = 4;

template <typename T>
struct Vec16 {
  static constexpr int EPL = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& u, float* f);
template <>
__device__ __forceinline__ void unpack16<float>(const uint4& u, float* f) {
  f[0] = __uint_as_float(u.x);
  f[1] = __uint_as_float(u.y);
  f[2] = __uint_as_float(u.z);
  f[3] = __uint_as_float(u.w);
}
template <>
__device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void unpack16<__half>(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 ld_stream16(const void* ptr) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(ptr));
  return r;
}

// Visible key count of a decode query of batch entry b: padding limit, then the causal limit of query 0.
__device__ __forceinline__ int64_t decode_len(const SdpaParams& p, int b) {
  int64_t L = kv_limit_of(p, b);
  if (p.causal) {
    int64_t c = p.causal_offset + 1;
    if (c < 0) c = 0;
    if (c < L) L = c;
  }
  return L;
}

template <typename T, int D, int GT, bool PAGED>
__global__ void __launch_bounds__(kDecWarps * 32)
    sdpa_decode_partial_kernel(const SdpaParams p, const int chunk, const int nchunks, float* __restrict__ ws,
                               const int direct) {
  constexpr int EPL = Vec16<T>::EPL;
  constexpr int LPK = D / EPL;    // lanes per key row
  constexpr int KPI = 32 / LPK;   // keys per warp-wide load
  constexpr int NG = kDecWarps * KPI;
  static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "head_dim not coverable by one warp load");

  __shared__ float sm_m[NG][GT];
  __shared__ float sm_l[NG][GT];
  __shared__ __align__(16) float sm_acc[NG][GT][D];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = lane / LPK, gl = lane % LPK, d0 = gl * EPL;
  const int gchunks = (p.group + GT - 1) / GT;
  const int b = blockIdx.z;
  const int kvh = p.head_begin / p.group + (int)blockIdx.y / gchunks;
  const int gc = (int)blockIdx.y % gchunks;
  const int h0 = kvh * p.group + gc * GT;
  const int nheads = min(GT, p.group - gc * GT);
  const int c = blockIdx.x;

  const int64_t L = decode_len(p, b);
  const int64_t start = (int64_t)c * chunk;
  const int Hc = p.head_count;

  if (start >= L) {
    if (direct && c == 0) {  // nothing visible: zero output, -inf LSE
      for (int idx = tid; idx < nheads * D; idx += kDecWarps * 32) {
        const int g = idx / D, d = idx - g * D;
        store_out<T>(p.out, b * p.os[0] + (int64_t)(h0 + g) * p.os[1] + d, 0.f, p.out_f32);
        if (p.lse && d == 0) p.lse[((int64_t)b * p.num_q_heads + h0 + g) * p.seq_q] = -INFINITY;
      }
    }
    return;
  }
  const int64_t end = (start + chunk < L) ? start + chunk : L;

  float qf[GT][EPL];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    const int h = h0 + (g < nheads ? g : 0);
    const T* qp = static_cast<const T*>(p.q) + b * p.qs[0] + (int64_t)h * p.qs[1] + d0;
    const uint4 u = *reinterpret_cast<const uint4*>(qp);
    unpack16<T>(u, qf[g]);
  }
  const T* kbase = static_cast<const T*>(p.k) + (PAGED ? 0 : b * p.ks[0]) + (int64_t)kvh * p.ks[1] + d0;
  const T* vbase = static_cast<const T*>(p.v) + (PAGED ? 0 : b * p.vs[0]) + (int64_t)kvh * p.vs[1] + d0;

  float m[GT], l[GT], acc[GT][EPL];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }

  constexpr int KPW = KPI * kUnroll;
  for (int64_t kb = start + warp * KPW; kb < end; kb += kDecWarps * KPW) {
    uint4 kv[kUnroll], vv[kUnroll];
    bool ok[kUnroll];
    int64_t row[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t key = kb + u * KPI + grp;
      ok[u] = key < end;
      row[u] = key;
      if constexpr (PAGED) {  // one block-table read per key, then the same 16-byte row loads
        row[u] = ok[u] ? kv_row_of(p, b, key) : -1;
        ok[u] = row[u] >= 0;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) kv[u] = ok[u] ? ld_stream16(kbase + row[u] * p.ks[2]) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) vv[u] = ok[u] ? ld_stream16(vbase + row[u] * p.vs[2]) : make_uint4(0, 0, 0, 0);

    float s[GT][kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float kf[EPL];
      unpack16<T>(kv[u], kf);
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) dot = fmaf(qf[g][e], kf[e], dot);
        s[g][u] = dot;
      }
    }
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) s[g][u] += __shfl_xor_sync(0xffffffffu, s[g][u], o);
      }

#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float mt = -INFINITY;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t key = kb + u * KPI + grp;
        float val = -INFINITY;
        if (ok[u] && g < nheads) val = finish_logit(p, s[g][u] * p.scale, b, h0 + g, 0, key, L);
        s[g][u] = val;
        mt = fmaxf(mt, val);
      }
      const float m_new = fmaxf(m[g], mt);
      if (m_new != -INFINITY) {
        const float corr = (m[g] == -INFINITY) ? 0.f : softmax_exp<T>(m[g] - m_new);
        float psum = 0.f;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          s[g][u] = (s[g][u] == -INFINITY) ? 0.f : softmax_exp<T>(s[g][u] - m_new);
          psum += s[g][u];
        }
        l[g] = l[g] * corr + psum;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] *= corr;
        m[g] = m_new;
      } else {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) s[g][u] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float vf[EPL];
      unpack16<T>(vv[u], vf);
#pragma unroll
      for (int g = 0; g < GT; ++g)
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = fmaf(s[g][u], vf[e], acc[g][e]);
    }
  }

  // merge the NG lane groups of the CTA
  const int ng = warp * KPI + grp;
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (gl == 0) {
      sm_m[ng][g] = m[g];
      sm_l[ng][g] = l[g];
    }
    if constexpr (EPL == 8) {
      *reinterpret_cast<float4*>(&sm_acc[ng][g][d0]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
      *reinterpret_cast<float4*>(&sm_acc[ng][g][d0 + 4]) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
    } else {
      *reinterpret_cast<float4*>(&sm_acc[ng][g][d0]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    }
  }
  __syncthreads();

  for (int idx = tid; idx < nheads * D; idx += kDecWarps * 32) {
    const int g = idx / D, d = idx - g * D;
    float M = -INFINITY;
#pragma unroll
    for (int n = 0; n < NG; ++n) M = fmaxf(M, sm_m[n][g]);
    float a = 0.f, lsum = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int n = 0; n < NG; ++n) {
        const float mn = sm_m[n][g];
        const float w = (mn == -INFINITY) ? 0.f : softmax_exp<T>(mn - M);
        a = fmaf(w, sm_acc[n][g][d], a);
        lsum = fmaf(w, sm_l[n][g], lsum);
      }
    }
    const int h = h0 + g;
    if (direct) {
      store_out<T>(p.out, b * p.os[0] + (int64_t)h * p.os[1] + d, lsum > 0.f ? a / lsum : 0.f, p.out_f32);
      if (p.lse && d == 0)
        p.lse[((int64_t)b * p.num_q_heads + h) * p.seq_q] = lsum > 0.f ? M + logf(lsum) : -INFINITY;
    } else {
      const int64_t slot = ((int64_t)b * Hc + (h - p.head_begin)) * nchunks + c;
      ws[slot * D + d] = a;
      if (d == 0) {
        float* ml = ws + (int64_t)p.batch * Hc * nchunks * D;
        ml[slot * 2] = M;
        ml[slot * 2 + 1] = lsum;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
    sdpa_decode_combine_kernel(const SdpaParams p, const int chunk, const int nchunks, const float* __restrict__ ws) {
  const int b = blockIdx.y;
  const int hl = blockIdx.x;
  const int h = p.head_begin + hl;
  const int D = p.head_dim;
  const int Hc = p.head_count;
  const int64_t L = decode_len(p, b);
  int nvalid = (int)((L + chunk - 1) / chunk);
  if (nvalid > nchunks) nvalid = nchunks;
  const int64_t slot0 = ((int64_t)b * Hc + hl) * nchunks;
  const float* ml = ws + (int64_t)p.batch * Hc * nchunks * D;

  float M = -INFINITY;
  for (int c = 0; c < nvalid; ++c) M = fmaxf(M, ml[(slot0 + c) * 2]);
  float lsum = 0.f;
  if (M != -INFINITY)
    for (int c = 0; c < nvalid; ++c) {
      const float mc = ml[(slot0 + c) * 2];
      if (mc != -INFINITY) lsum = fmaf(softmax_exp<T>(mc - M), ml[(slot0 + c) * 2 + 1], lsum);
    }
  const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    if (M != -INFINITY)
      for (int c = 0; c < nvalid; ++c) {
        const float mc = ml[(slot0 + c) * 2];
        if (mc != -INFINITY) a = fmaf(softmax_exp<T>(mc - M), ws[(slot0 + c) * D + d], a);
      }
    store_out<T>(p.out, b * p.os[0] + (int64_t)h * p.os[1] + d, a * inv, p.out_f32);
  }
  if (p.lse && threadIdx.x == 0)
    p.lse[((int64_t)b * p.num_q_heads + h) * p.seq_q] = lsum > 0.f ? M + logf(lsum) : -INFINITY;
}

template <typename T, int D, int GT>
cudaError_t launch_partial(const SdpaParams& p, int chunk, int nchunks, float* ws, int direct, cudaStream_t stream) {
  const int gchunks = (p.group + GT - 1) / GT;
  dim3 grid((unsigned)nchunks, (unsigned)((p.head_count / p.group) * gchunks), (unsigned)p.batch);
  if (p.block_table) sdpa_decode_partial_kernel<T, D, GT, true><<<grid, kDecWarps * 32, 0, stream>>>(p, chunk, nchunks, ws, direct);
  else sdpa_decode_partial_kernel<T, D, GT, false><<<grid, kDecWarps * 32, 0, stream>>>(p, chunk, nchunks, ws, direct);
  return cudaGetLastError();
}

template <typename T, int D>
cudaError_t launch_partial_g(const SdpaParams& p, int chunk, int nchunks, float* ws, int direct, cudaStream_t stream) {
  if (p.group == 1) return launch_partial<T, D, 1>(p, chunk, nchunks, ws, direct, stream);
  if (p.group == 2) return launch_partial<T, D, 2>(p, chunk, nchunks, ws, direct, stream);
  if (p.group <= 4) return launch_partial<T, D, 4>(p, chunk, nchunks, ws, direct, stream);
  return launch_partial<T, D, 8>(p, chunk, nchunks, ws, direct, stream);
}

template <typename T>
cudaError_t launch_decode_t(const SdpaParams& p, int chunk, int nchunks, float* ws, cudaStream_t stream,
                            int* launches) {
  const int direct = nchunks == 1 ? 1 : 0;
  cudaError_t e;
  switch (p.head_dim) {
    case 64: e = launch_partial_g<T, 64>(p, chunk, nchunks, ws, direct, stream); break;
    case 128: e = launch_partial_g<T, 128>(p, chunk, nchunks, ws, direct, stream); break;
    case 256:
      if constexpr (sizeof(T) == 2) {
        e = launch_partial_g<T, 256>(p, chunk, nchunks, ws, direct, stream);
        break;
      }
      return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
  }
  *launches = 1;
  if (e != cudaSuccess || direct) return e;
  dim3 grid((unsigned)p.head_count, (unsigned)p.batch);
  sdpa_decode_combine_kernel<T><<<grid, 128, 0, stream>>>(p, chunk, nchunks, ws);
  *launches = 2;
  return cudaGetLastError();
}


// ---- decode with library-owned static scratch ---------------------------------------------------------------
// Some callers may not allocate device memory at the point where they decode: code running inside a CUDA-graph
// capture or a real-time serving loop where cudaMalloc (which can synchronise the device) is forbidden, or a
// host whose memory budget was handed out up front.  For them the split-KV partials live in this fixed array
// instead of a caller or handle allocation.  Every GPU that loads the library holds the array until exit.
constexpr int64_t kStaticScratchFloats = 4ll * 1024 * 1024;  // 16 MiB
static __device__ __align__(256) float g_decode_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
float* g_static_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_static_scratch_mutex;

// In host code the array's name is only a stand-in; the device address has to be asked for, per device, with
// that device current.
cudaError_t static_scratch_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_ptr[dev]) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_decode_static_scratch);
    if (e != cudaSuccess) return e;
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return cudaSuccess;
}

}  // namespace

bool decode_supported(int dtype, int head_dim) {
  if (head_dim == 64 || head_dim == 128) return true;
  return head_dim == 256 && dtype != AIDN_F32;
}

cudaError_t launch_decode(const SdpaParams& p, int dtype, int chunk, int nchunks, float* workspace, cudaStream_t stream,
                          int* launches) {
  switch (dtype) {
    case AIDN_F32: return launch_decode_t<float>(p, chunk, nchunks, workspace, stream, launches);
    case AIDN_F16: return launch_decode_t<__half>(p, chunk, nchunks, workspace, stream, launches);
    default: return launch_decode_t<__nv_bfloat16>(p, chunk, nchunks, workspace, stream, launches);
  }
}

}  // namespace aidn

namespace aidn {

int64_t decode_static_scratch_bytes() { return kStaticScratchFloats * (int64_t)sizeof(float); }

// Same two kernels as launch_decode, with the partials in the library's static array.  `need_bytes` is what the
// shape requires; the caller has already checked it against decode_static_scratch_bytes().
cudaError_t launch_decode_static(const SdpaParams& p, int dtype, int chunk, int nchunks, cudaStream_t stream,
                                 int* launches) {
  float* scratch = nullptr;
  cudaError_t e = static_scratch_address(&scratch);
  if (e != cudaSuccess) return e;
  return launch_decode(p, dtype, chunk, nchunks, scratch, stream, launches);
}

}  // namespace aidn
