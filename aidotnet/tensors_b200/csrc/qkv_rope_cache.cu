// Decode-step front end: y = W x + b for the packed Q/K/V projection of up to 8 resident tokens, interleaved RoPE on
// the Q and K heads, Q written out and the K / V rows written straight into the KV cache the decode kernel reads.
//
// Replaces CudaBackend.QkvProjectionRoPECacheD64 of the reference
// (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/CudaBackend.cs:8389-8439: one fp32 token, head_dim 64, cache
// [capacity, heads, 64]; its general path is cuBLAS GEMV + BiasAdd + rope_interleaved + three device copies through
// three scratch allocations) and rope_interleaved (CUDA/Kernels/CudaAttentionKernels.cs:1023-1050).
//
// The step is a GEMV: every weight is used once per token, so it is bound by streaming W from HBM
// ((heads + 2 kv_heads) * head_dim * model * sizeof(weight) bytes; nothing here is shaped for tensor cores).  A warp owns
// one rotation pair of output rows (2r, 2r+1) - the two rows RoPE mixes - streams both with 16-byte no-allocate loads,
// reads the tokens' activations from shared memory or through L1, and finishes the pair in registers: bias, rotation by the token's
// (cos, sin), store in the destination dtype.  Up to 8 tokens share one pass over W.
#include "common.cuh"

namespace aidn {

namespace {


__device__ __forceinline__ uint4 ld_stream16(const void* ptr) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(ptr));
  return r;
}

template <typename WT>
struct WVec;
template <>
struct WVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
};
template <>
struct WVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

__device__ __forceinline__ void store_as(void* base, int64_t idx, float x, int dtype) {
  if (dtype == AIDN_F32) static_cast<float*>(base)[idx] = x;
  else if (dtype == AIDN_F16) static_cast<__half*>(base)[idx] = __float2half_rn(x);
  else static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(x);
}

// T tokens starting at token t_base share this pass over W.  The activations of all T tokens sit in shared memory once
// per CTA, so the CTA is made wide (WARPS) when they are large: occupancy is then bounded by warps, not by CTAs.
// XS: the activations are staged in shared memory (measured faster with fp32 weights); otherwise they are read
// through L1 (measured faster with bf16 weights, and free of any size limit).
template <typename WT, int T, int WARPS, bool XS>
__global__ void __launch_bounds__(WARPS * 32) qkv_rope_cache_kernel(const QkvRopeParams p, const int t_base) {
  constexpr int kQkvWarps = WARPS;
  constexpr int N = WVec<WT>::N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int model = p.model;
  const int D = p.head_dim;
  const int ntok = min(T, p.tokens - t_base);

  extern __shared__ __align__(16) float xs[];   // [T][model] when XS
  if constexpr (XS) {
    constexpr int kStageUnroll = 4;   // independent loads in flight per thread
    const int tid = threadIdx.x;
    for (int base = tid * 4; base < T * model; base += kQkvWarps * 32 * 4 * kStageUnroll) {
      float4 v[kStageUnroll];
#pragma unroll
      for (int u = 0; u < kStageUnroll; ++u) {
        const int idx = base + u * kQkvWarps * 32 * 4;
        const int t = idx / model;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (idx < T * model && t < ntok)
          v[u] = *reinterpret_cast<const float4*>(p.input + (int64_t)(t_base + t) * model + (idx - t * model));
      }
#pragma unroll
      for (int u = 0; u < kStageUnroll; ++u) {
        const int idx = base + u * kQkvWarps * 32 * 4;
        if (idx < T * model) *reinterpret_cast<float4*>(xs + idx) = v[u];
      }
    }
    __syncthreads();
  }
  const int q_rows = p.heads * D, kv_rows = p.kv_heads * D;
  const int pairs = (q_rows + 2 * kv_rows) / 2;
  const WT* W = static_cast<const WT*>(p.weights);

  for (int pair = blockIdx.x * kQkvWarps + warp; pair < pairs; pair += gridDim.x * kQkvWarps) {
    const int r0 = 2 * pair;
    const WT* w0 = W + (int64_t)r0 * model;
    const WT* w1 = w0 + model;
    float a0[T], a1[T];
#pragma unroll
    for (int t = 0; t < T; ++t) a0[t] = a1[t] = 0.f;

    constexpr int kUnroll = 4;
    for (int k0 = lane * N; k0 < model; k0 += 32 * N * kUnroll) {
      uint4 u0[kUnroll], u1[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int k = k0 + u * 32 * N;
        const bool ok = k < model;
        u0[u] = ok ? ld_stream16(w0 + k) : make_uint4(0, 0, 0, 0);
        u1[u] = ok ? ld_stream16(w1 + k) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int k = k0 + u * 32 * N;
        if (k >= model) continue;
        float f0[N], f1[N];
        WVec<WT>::unpack(u0[u], f0);
        WVec<WT>::unpack(u1[u], f1);
#pragma unroll
        for (int t = 0; t < T; ++t) {
          if (!XS && t >= ntok) continue;
          const float* x = XS ? xs + t * model + k : p.input + (int64_t)(t_base + t) * model + k;
#pragma unroll
          for (int e = 0; e < N; e += 4) {
            const float4 xv = XS ? *reinterpret_cast<const float4*>(x + e) : __ldg(reinterpret_cast<const float4*>(x + e));
            a0[t] = fmaf(f0[e], xv.x, a0[t]); a0[t] = fmaf(f0[e + 1], xv.y, a0[t]);
            a0[t] = fmaf(f0[e + 2], xv.z, a0[t]); a0[t] = fmaf(f0[e + 3], xv.w, a0[t]);
            a1[t] = fmaf(f1[e], xv.x, a1[t]); a1[t] = fmaf(f1[e + 1], xv.y, a1[t]);
            a1[t] = fmaf(f1[e + 2], xv.z, a1[t]); a1[t] = fmaf(f1[e + 3], xv.w, a1[t]);
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < T; ++t)
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        a0[t] += __shfl_xor_sync(0xffffffffu, a0[t], o);
        a1[t] += __shfl_xor_sync(0xffffffffu, a1[t], o);
      }

    // lane t finishes token t: bias, rotation, store
    if (lane < ntok) {
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int t = 0; t < T; ++t)
        if (lane == t) { y0 = a0[t]; y1 = a1[t]; }
      if (p.bias) { y0 += p.bias[r0]; y1 += p.bias[r0 + 1]; }
      const int tok = t_base + lane;
      const int64_t pos = p.positions ? p.positions[tok] : (int64_t)p.position + tok;
      const int64_t crow = p.cache_rows ? p.cache_rows[tok] : pos;
      const bool is_q = r0 < q_rows;
      const bool is_k = !is_q && r0 < q_rows + kv_rows;
      if (is_q || is_k) {   // interleaved RoPE: (x_even, x_odd) -> (x_even c - x_odd s, x_even s + x_odd c)
        const int within = is_q ? r0 : r0 - q_rows;
        const int i = (within % D) >> 1;
        float c = 1.f, s = 0.f;
        if (pos >= 0 && pos < p.max_position) {
          c = p.cosine[pos * (D / 2) + i];
          s = p.sine[pos * (D / 2) + i];
        }
        const float e = y0 * c - y1 * s, o = y0 * s + y1 * c;
        y0 = e;
        y1 = o;
      }
      if (is_q) {
        const int64_t at = (int64_t)tok * q_rows + r0;
        store_as(p.query, at, y0, p.query_dtype);
        store_as(p.query, at + 1, y1, p.query_dtype);
      } else if (crow >= 0 && crow < p.cache_capacity) {   // a row outside the cache is not written
        const int within = is_k ? r0 - q_rows : r0 - q_rows - kv_rows;
        const int64_t at = crow * kv_rows + within;
        void* dst = is_k ? p.key_cache : p.value_cache;
        store_as(dst, at, y0, p.cache_dtype);
        store_as(dst, at + 1, y1, p.cache_dtype);
      }
    }
  }
}

// ---- several tokens, bf16 weights: the same pass over W on the warp-level tensor cores ------------------------------
// With T tokens the FFMA form reads T activations from shared memory per weight and becomes bound by that.  Here a CTA
// of 16 warps takes 16 output rows (8 rotation pairs) at a time as the M dimension of mma.sync.m16n8k16, the tokens
// (padded to 8) as N, and splits K across its warps; the partial sums meet in shared memory and 64 threads finish the
// tile (bias, rotation, stores).  As in the decode kernel, the k order is free: a thread's 16-byte weight chunk feeds
// the k slots in the order it arrives and the activations are read in the matching order, so W goes from global
// memory straight into the A fragments.  The fp32 activations are split once per CTA into bf16 hi + lo (x = hi + lo
// to 2^-17) and multiplied in two MMAs, which keeps the result at fp32-GEMV accuracy.
constexpr int kMmaWarps = 16;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kMmaThreads = (kMmaWarps + 2) * 32;   // 16 streaming warps + 2 finishing warps

__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_bar_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__global__ void __launch_bounds__(kMmaThreads) qkv_rope_cache_mma_kernel(const QkvRopeParams p, const int t_base) {
  extern __shared__ __align__(16) uint8_t qsm[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int model = p.model, D = p.head_dim;
  const int ntok = min(8, p.tokens - t_base);
  const int pitch = model * 2 + 64;                       // bytes per token row of hi (and of lo): bank-conflict free
  uint8_t* x_hi = qsm;                                    // [8][pitch]
  uint8_t* x_lo = qsm + 8 * pitch;                        // [8][pitch]
  float* part = reinterpret_cast<float*>(qsm + 16 * pitch);   // [2 buffers][kMmaWarps][16 rows][8 tokens]
  float* rope = part + 2 * kMmaWarps * 128;                       // [8 tokens][D/2] cos, then [8][D/2] sin
  long long* tokrow = reinterpret_cast<long long*>(rope + 8 * D);   // [8] cache row of each token, -1 = none

  // stage the activations: four independent 16-byte loads per thread in flight, then split and store
  {
    const int n4 = 8 * model / 4;
    constexpr int kStageUnroll = 4;
    for (int base = tid; base < n4; base += kMmaThreads * kStageUnroll) {
      float4 v[kStageUnroll];
#pragma unroll
      for (int u = 0; u < kStageUnroll; ++u) {
        const int idx = base + u * kMmaThreads;
        const int t = idx / (model / 4), k = (idx - t * (model / 4)) * 4;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (idx < n4 && t < ntok) v[u] = *reinterpret_cast<const float4*>(p.input + (int64_t)(t_base + t) * model + k);
      }
#pragma unroll
      for (int u = 0; u < kStageUnroll; ++u) {
        const int idx = base + u * kMmaThreads;
        if (idx >= n4) continue;
        const int t = idx / (model / 4), k = (idx - t * (model / 4)) * 4;
        const float f[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
        __nv_bfloat16 h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          h[e] = __float2bfloat16_rn(f[e]);
          l[e] = __float2bfloat16_rn(f[e] - __bfloat162float(h[e]));
        }
        *reinterpret_cast<__nv_bfloat162*>(x_hi + t * pitch + k * 2) = __halves2bfloat162(h[0], h[1]);
        *reinterpret_cast<__nv_bfloat162*>(x_hi + t * pitch + k * 2 + 4) = __halves2bfloat162(h[2], h[3]);
        *reinterpret_cast<__nv_bfloat162*>(x_lo + t * pitch + k * 2) = __halves2bfloat162(l[0], l[1]);
        *reinterpret_cast<__nv_bfloat162*>(x_lo + t * pitch + k * 2 + 4) = __halves2bfloat162(l[2], l[3]);
      }
    }
  }
  // per-token rotation rows and cache rows, fetched once so that finishing a tile touches no dependent global loads
  for (int idx = tid; idx < 8 * (D / 2); idx += kMmaThreads) {
    const int t = idx / (D / 2), i = idx - t * (D / 2);
    float cs = 1.f, sn = 0.f;
    if (t < ntok) {
      const int tok = t_base + t;
      const int64_t pos = p.positions ? p.positions[tok] : (int64_t)p.position + tok;
      if (pos >= 0 && pos < p.max_position) {
        cs = p.cosine[pos * (D / 2) + i];
        sn = p.sine[pos * (D / 2) + i];
      }
      if (i == 0) {
        const int64_t crow = p.cache_rows ? p.cache_rows[tok] : pos;
        tokrow[t] = (crow >= 0 && crow < p.cache_capacity) ? crow : -1;
      }
    }
    rope[t * (D / 2) + i] = cs;
    rope[8 * (D / 2) + t * (D / 2) + i] = sn;
  }
  __syncthreads();

  const int q_rows = p.heads * D, kv_rows = p.kv_heads * D;
  const int tiles = (q_rows + 2 * kv_rows) / 16;
  const __nv_bfloat16* W = static_cast<const __nv_bfloat16*>(p.weights);
  const int chunks = model / 8;                     // 16-byte chunks per weight row
  const uint32_t hi_s = (uint32_t)__cvta_generic_to_shared(x_hi), lo_s = (uint32_t)__cvta_generic_to_shared(x_lo);

  // This warp's K slice is chunks warp*4 + c, + 64, + 128, ...; a batch is kBatch of them (all loads in flight at once).
  // The first batch of the next tile is requested before the current tile is handed to the finishing threads, so the
  // weight stream does not stop at the tile boundary.
  constexpr int kBatch = 8;
  constexpr int kChunkStep = 4 * kMmaWarps;
  uint4 we[kBatch], wo[kBatch];
  auto load_batch = [&](int tile, int ch0) {
    // MMA row m < 8 is weight row 16*tile + 2m (the even row of pair m), row m + 8 the odd row of the same pair
    const __nv_bfloat16* w_even = W + (int64_t)(16 * tile + 2 * g) * model;
    const __nv_bfloat16* w_odd = w_even + model;
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int ch = ch0 + u * kChunkStep;
      const bool ok = ch < chunks;
      we[u] = ok ? ld_stream16(w_even + ch * 8) : make_uint4(0, 0, 0, 0);
      wo[u] = ok ? ld_stream16(w_odd + ch * 8) : make_uint4(0, 0, 0, 0);
    }
  };
  // Warps 0..15 stream the weights; warps 16..17 finish the tiles.  The partial sums change hands through two buffers
  // and two pairs of named barriers (full: the tile's partials are written; free: they have been read), so the weight
  // stream never waits for a tile to be finished.
  if (warp < kMmaWarps) {
  const int ch_first = warp * 4 + c;
  if ((int)blockIdx.x < tiles) load_batch(blockIdx.x, ch_first);

  int it = 0;
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int ch0 = ch_first; ch0 < chunks; ch0 += kChunkStep * kBatch) {
      if (ch0 != ch_first) load_batch(tile, ch0);
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int ch = ch0 + u * kChunkStep;
        if (ch >= chunks) continue;
        // activations of token g for the same chunk: registers 2h / 2h+1 feed k-step h like the weight registers do
        uint32_t bh[4], bl[4];
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(bh[0]), "=r"(bh[1]), "=r"(bh[2]), "=r"(bh[3])
                     : "r"(hi_s + g * pitch + ch * 16));
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(bl[0]), "=r"(bl[1]), "=r"(bl[2]), "=r"(bl[3])
                     : "r"(lo_s + g * pitch + ch * 16));
        const uint32_t ae[4] = {we[u].x, we[u].y, we[u].z, we[u].w};
        const uint32_t ao[4] = {wo[u].x, wo[u].y, wo[u].z, wo[u].w};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mma_bf16_16816(acc, ae[2 * h], ao[2 * h], ae[2 * h + 1], ao[2 * h + 1], bh[2 * h], bh[2 * h + 1]);
          mma_bf16_16816(acc, ae[2 * h], ao[2 * h], ae[2 * h + 1], ao[2 * h + 1], bl[2 * h], bl[2 * h + 1]);
        }
      }
    }
    if (tile + (int)gridDim.x < tiles) load_batch(tile + gridDim.x, ch_first);
    // acc: [0,1] = even row of pair g for tokens 2c, 2c+1; [2,3] = odd row
    const int buf = it & 1;
    if (it >= 2) named_bar_sync(3 + buf, kMmaThreads);   // the finishing warps have read this buffer's previous tile
    float* mine = part + (buf * kMmaWarps + warp) * 128;
    mine[g * 8 + 2 * c] = acc[0];
    mine[g * 8 + 2 * c + 1] = acc[1];
    mine[(g + 8) * 8 + 2 * c] = acc[2];
    mine[(g + 8) * 8 + 2 * c + 1] = acc[3];
    __threadfence_block();
    named_bar_arrive(1 + buf, kMmaThreads);
  }
  } else {
  const int ftid = tid - kMmaWarps * 32;   // 0..63: (pair, token)
  int it = 0;
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
    const int buf = it & 1;
    named_bar_sync(1 + buf, kMmaThreads);
    const float* pb = part + buf * kMmaWarps * 128;
    {
      const int pr = ftid >> 3, t = ftid & 7;
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int w = 0; w < kMmaWarps; ++w) {
        y0 += pb[w * 128 + pr * 8 + t];
        y1 += pb[w * 128 + (pr + 8) * 8 + t];
      }
      if (t < ntok) {
        const int r0 = 16 * tile + 2 * pr;
        if (p.bias) { y0 += p.bias[r0]; y1 += p.bias[r0 + 1]; }
        const int tok = t_base + t;
        const int64_t crow = tokrow[t];
        const bool is_q = r0 < q_rows;
        const bool is_k = !is_q && r0 < q_rows + kv_rows;
        if (is_q || is_k) {
          const int within = is_q ? r0 : r0 - q_rows;
          const int i = (within % D) >> 1;
          const float cs = rope[t * (D / 2) + i], sn = rope[8 * (D / 2) + t * (D / 2) + i];
          const float e = y0 * cs - y1 * sn, o = y0 * sn + y1 * cs;
          y0 = e;
          y1 = o;
        }
        if (is_q) {
          const int64_t at = (int64_t)tok * q_rows + r0;
          store_as(p.query, at, y0, p.query_dtype);
          store_as(p.query, at + 1, y1, p.query_dtype);
        } else if (crow >= 0) {
          const int within = is_k ? r0 - q_rows : r0 - q_rows - kv_rows;
          const int64_t at = crow * kv_rows + within;
          void* dst = is_k ? p.key_cache : p.value_cache;
          store_as(dst, at, y0, p.cache_dtype);
          store_as(dst, at + 1, y1, p.cache_dtype);
        }
      }
    }
    named_bar_arrive(3 + buf, kMmaThreads);   // the buffer may be overwritten (tile it + 2)
  }
  }
}

cudaError_t launch_qkv_mma(const QkvRopeParams& p, int t_base, int num_sms, cudaStream_t stream) {
  const size_t smem = 16 * ((size_t)p.model * 2 + 64) + 2 * kMmaWarps * 128 * sizeof(float) + 8 * p.head_dim * sizeof(float) + 64;
  cudaError_t e = cudaFuncSetAttribute(qkv_rope_cache_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int tiles = (p.heads + 2 * p.kv_heads) * p.head_dim / 16;
  const int per_sm = smem <= 100 * 1024 ? 2 : 1;
  int grid = tiles < num_sms * per_sm ? tiles : num_sms * per_sm;
  qkv_rope_cache_mma_kernel<<<grid, kMmaThreads, smem, stream>>>(p, t_base);
  return cudaGetLastError();
}

__global__ void rope_interleaved_kernel(const float* __restrict__ in, const float* __restrict__ cosc,
                                        const float* __restrict__ sinc, float* __restrict__ out, int64_t rows,
                                        int head_dim, int seq_len, int start_position) {
  const int half = head_dim / 2;
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= rows * half) return;
  const int i = (int)(g % half);
  const int64_t row = g / half;
  const int64_t pos = start_position + row % seq_len;
  const float c = cosc[pos * half + i], s = sinc[pos * half + i];
  const float2 x = *reinterpret_cast<const float2*>(in + row * head_dim + 2 * i);
  *reinterpret_cast<float2*>(out + row * head_dim + 2 * i) = make_float2(x.x * c - x.y * s, x.x * s + x.y * c);
}

// CTAs for `pairs` row pairs, one pair per warp and round: at most eight CTAs per SM are resident, and when the pairs
// need more than one round every warp gets the same number of rounds (a grid-stride split that leaves a few warps with
// one pair more than the rest ends the launch with those warps alone).
inline int balanced_grid(int pairs, int warps_per_cta, int num_sms) {
  const int warp_cap = num_sms * 8 * warps_per_cta;
  const int rounds = (pairs + warp_cap - 1) / warp_cap;
  const int warps = (pairs + rounds - 1) / rounds;
  return (warps + warps_per_cta - 1) / warps_per_cta;
}

template <typename WT, int T>
cudaError_t launch_qkv_t(const QkvRopeParams& p, int t_base, int num_sms, cudaStream_t stream) {
  const int pairs = (p.heads + 2 * p.kv_heads) * p.head_dim / 2;
  const size_t xbytes = (size_t)T * p.model * sizeof(float);
  if (sizeof(WT) == 4 && xbytes <= 200 * 1024) {
    constexpr int kQkvWarps = T >= 4 ? 16 : (T == 2 ? 8 : 4);   // wide CTAs when the staged activations are large
    auto kern = qkv_rope_cache_kernel<WT, T, kQkvWarps, true>;
    if (xbytes > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)xbytes);
      if (e != cudaSuccess) return e;
    }
    const int grid = balanced_grid(pairs, kQkvWarps, num_sms);
    kern<<<grid, kQkvWarps * 32, xbytes, stream>>>(p, t_base);
  } else {
    constexpr int kQkvWarps = 4;
    const int grid = balanced_grid(pairs, kQkvWarps, num_sms);
    qkv_rope_cache_kernel<WT, T, kQkvWarps, false><<<grid, kQkvWarps * 32, 0, stream>>>(p, t_base);
  }
  return cudaGetLastError();
}

template <typename WT>
cudaError_t launch_qkv_w(const QkvRopeParams& p, int num_sms, cudaStream_t stream, int* launches) {
  *launches = 0;
  const size_t mma_smem = 16 * ((size_t)p.model * 2 + 64) + 2 * kMmaWarps * 128 * sizeof(float) + 8 * p.head_dim * sizeof(float) + 64;
  const bool mma_ok = sizeof(WT) == 2 && ((p.heads + 2 * p.kv_heads) * p.head_dim) % 16 == 0 && mma_smem <= 220 * 1024;
  const int fit = 8;   // tokens per pass over W on the FFMA path (its activations come through L1, any model size)
  for (int t_base = 0; t_base < p.tokens;) {
    const int left = p.tokens - t_base;
    cudaError_t e;
    int took;
    if (left >= 2 && mma_ok) {
      e = launch_qkv_mma(p, t_base, num_sms, stream);
      took = left < 8 ? left : 8;
    } else {
      // the kernel instantiated for T tokens stages T rows of activations whatever it is given: T must fit
      int tmpl = 1;
      if (fit >= 8 && left >= 5) tmpl = 8;
      else if (fit >= 4 && left >= 3) tmpl = 4;
      else if (fit >= 2 && left >= 2) tmpl = 2;
      took = left < tmpl ? left : tmpl;
      if (tmpl == 8) e = launch_qkv_t<WT, 8>(p, t_base, num_sms, stream);
      else if (tmpl == 4) e = launch_qkv_t<WT, 4>(p, t_base, num_sms, stream);
      else if (tmpl == 2) e = launch_qkv_t<WT, 2>(p, t_base, num_sms, stream);
      else e = launch_qkv_t<WT, 1>(p, t_base, num_sms, stream);
    }
    if (e != cudaSuccess) return e;
    ++*launches;
    t_base += took;
  }
  return cudaSuccess;
}

}  // namespace

// Largest model dimension served (index arithmetic is 32-bit within a weight row).
int64_t qkv_rope_max_model() { return 1 << 20; }

cudaError_t launch_qkv_rope_cache(const QkvRopeParams& p, int weight_dtype, int num_sms, cudaStream_t stream,
                                  int* launches) {
  if (weight_dtype == AIDN_F32) return launch_qkv_w<float>(p, num_sms, stream, launches);
  return launch_qkv_w<__nv_bfloat16>(p, num_sms, stream, launches);
}

cudaError_t launch_rope_interleaved(const float* in, const float* cosc, const float* sinc, float* out, int64_t rows,
                                    int head_dim, int seq_len, int start_position, cudaStream_t stream) {
  const int64_t n = rows * (head_dim / 2);
  if (n == 0) return cudaSuccess;
  rope_interleaved_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(in, cosc, sinc, out, rows, head_dim, seq_len,
                                                                          start_position);
  return cudaGetLastError();
}

}  // namespace aidn
