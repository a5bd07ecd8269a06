// Generic attention forward: fp32 FFMA arithmetic, online softmax, any head_dim <= 256, every mask kind.
//
// Serves (1) the fp32-input contract (<= 1e-5 relative against the fp32 CPU path), where tensor-core
// rounding of the inputs is not admissible, and (2) shapes and mask kinds the tcgen05 prefill kernel does
// not take.  Replaces the one-thread-per-row kernel of the reference
// (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/Kernels/CudaAttentionKernels.cs:28-112), which recomputes
// q.k up to D+2 times per key; here K/V tiles are staged once in shared memory per 16 query rows.
//
// A group of 4 warps takes 16 query rows (4 per warp) over key tiles of 32.  In the score phase lane j owns key j of
// the tile; in the P.V phase lane l owns output dims l, l+32, ...  A CTA is KS such groups on the same 16 rows: group
// g takes the key tiles g, g + KS, ..., keeps its own running max / sum / accumulator, and the groups' results are
// merged through shared memory at the end (the rescaling rule of the online softmax, applied once more).  KS = 4 is
// used when the launch has few CTAs: a small problem is one wave of CTAs whose length is the number of key tiles a
// group walks through, each with a lone warp per scheduler and nothing to hide its latencies behind
// (B1 H8 S512 D64: 72 us with KS = 1).
#include "common.cuh"

namespace aidn {
namespace {

constexpr int kRowsPerWarp = 4;
constexpr int kWarps = 4;
constexpr int kBM = kRowsPerWarp * kWarps;  // 16
constexpr int kBN = 32;

__device__ __forceinline__ void group_sync(int grp) {
  asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(kWarps * 32) : "memory");
}

// shared-memory floats of one group: its K and V tiles and its probabilities
template <int DMAX>
struct GroupFloats { static constexpr int value = 2 * kBN * (DMAX + 4) + kWarps * kRowsPerWarp * kBN; };

template <typename T, int DMAX, int KS>
__global__ void __launch_bounds__(KS * kWarps * 32) sdpa_generic_kernel(const SdpaParams p) {
  constexpr int PITCH = DMAX + 4;  // floats; keeps float4 rows 16-byte aligned and bank-conflict free
  constexpr int ND = DMAX / 32;
  constexpr int kGroupThreads = kWarps * 32;
  extern __shared__ __align__(16) float smem[];
  const int tid_cta = threadIdx.x;
  const int grp = tid_cta / kGroupThreads;          // key-split group
  const int tid = tid_cta - grp * kGroupThreads;    // thread within the group
  float* Qs = smem;                                             // [kBM][PITCH], shared by the groups
  float* Ks = Qs + kBM * PITCH + grp * GroupFloats<DMAX>::value;    // [kBN][PITCH]
  float* Vs = Ks + kBN * PITCH;                                 // [kBN][PITCH]
  float* Ps = Vs + kBN * PITCH;                                 // [kWarps][kRowsPerWarp][kBN]
  __shared__ int64_t kv_rows_all[KS][kBN];                      // pool rows of the tile's keys (paged K/V only)
  int64_t* kv_rows = kv_rows_all[grp];

  const int warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z;
  const int h = p.head_begin + blockIdx.y;
  const int kvh = h / p.group;
  const int64_t row0 = (int64_t)blockIdx.x * kBM;
  const int D = p.head_dim;

  const T* qb = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
  const bool paged = p.block_table != nullptr;
  const T* kb = static_cast<const T*>(p.k) + (paged ? 0 : b * p.ks[0]) + kvh * p.ks[1];
  const T* vb = static_cast<const T*>(p.v) + (paged ? 0 : b * p.vs[0]) + kvh * p.vs[1];

  for (int idx = tid_cta; idx < kBM * DMAX; idx += KS * kGroupThreads) {
    const int r = idx / DMAX, d = idx - r * DMAX;
    const int64_t row = row0 + r;
    Qs[r * PITCH + d] = (row < p.seq_q && d < D) ? to_float<T>(qb[row * p.qs[2] + d]) : 0.f;
  }
  if (KS > 1) __syncthreads();   // (a single group orders the Q stores with its first tile barrier)

  const int64_t kv_limit = kv_limit_of(p, b);
  int64_t kend = kv_limit;
  if (p.causal) {
    int64_t last_row = row0 + kBM - 1;
    if (last_row > p.seq_q - 1) last_row = p.seq_q - 1;
    const int64_t c = last_row + p.causal_offset + 1;
    if (c < kend) kend = c;
  }

  bool bad_block = false;
  float m[kRowsPerWarp], l[kRowsPerWarp], acc[kRowsPerWarp][ND];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[r][i] = 0.f;
  }

  // Contiguous K / V with head_dim <= 128: the next tile's elements are fetched into registers before the current
  // tile is multiplied, so the loads run under the arithmetic.  (Without it every tile paid a full memory latency,
  // which is what small problems - few CTAs, a handful of warps per SM - consist of: B1 H8 S512 D64 took 79 us.)
  constexpr int kPre = DMAX <= 128 ? (kBN * DMAX) / (kWarps * 32) : 1;
  const bool prefetch = DMAX <= 128 && !paged;
  T kreg[kPre], vreg[kPre];
  auto fetch_tile = [&](int64_t j0) {
#pragma unroll
    for (int e = 0; e < kPre; ++e) {
      const int idx = tid + e * kWarps * 32;
      const int j = idx / DMAX, d = idx - j * DMAX;
      const int64_t key = j0 + j;
      // keys past this CTA's last visible key (padding beyond kv_len, the causal future) are never read: their
      // probability is 0, and 0 * (NaN or Inf left in unused memory) would be NaN
      const bool ok = key < kend && d < D;
      kreg[e] = ok ? kb[key * p.ks[2] + d] : T(0.f);
      vreg[e] = ok ? vb[key * p.vs[2] + d] : T(0.f);
    }
  };
  const int64_t j_first = (int64_t)grp * kBN, j_step = (int64_t)KS * kBN;
  if (prefetch && j_first < kend) fetch_tile(j_first);

  for (int64_t j0 = j_first; j0 < kend; j0 += j_step) {
    group_sync(grp);  // previous tile fully consumed (also orders the Q stores before first use)
    if (prefetch) {
#pragma unroll
      for (int e = 0; e < kPre; ++e) {
        const int idx = tid + e * kWarps * 32;
        const int j = idx / DMAX, d = idx - j * DMAX;
        Ks[j * PITCH + d] = to_float<T>(kreg[e]);
        Vs[j * PITCH + d] = to_float<T>(vreg[e]);
      }
      group_sync(grp);
      if (j0 + j_step < kend) fetch_tile(j0 + j_step);
    } else {
      if (paged) {
        if (tid < kBN) kv_rows[tid] = (j0 + tid < kend) ? kv_row_of(p, b, j0 + tid, bad_block) : -1;
        group_sync(grp);
      }
      for (int idx = tid; idx < kBN * DMAX; idx += kWarps * 32) {
        const int j = idx / DMAX, d = idx - j * DMAX;
        const int64_t key = j0 + j;
        const int64_t row = paged ? kv_rows[j] : key;
        // keys past this CTA's last visible key (padding beyond kv_len, a partly filled pool block, the causal
        // future) are never read: their probability is 0, and 0 * (NaN or Inf left in unused memory) would be NaN
        const bool ok = key < kend && d < D && row >= 0;
        Ks[j * PITCH + d] = ok ? to_float<T>(kb[row * p.ks[2] + d]) : 0.f;
        Vs[j * PITCH + d] = ok ? to_float<T>(vb[row * p.vs[2] + d]) : 0.f;
      }
      group_sync(grp);
    }

    float s[kRowsPerWarp] = {0.f, 0.f, 0.f, 0.f};
    const float4* krow = reinterpret_cast<const float4*>(Ks + lane * PITCH);
#pragma unroll 4
    for (int d4 = 0; d4 < DMAX / 4; ++d4) {
      const float4 kv = krow[d4];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        const float4 qv = reinterpret_cast<const float4*>(Qs + (warp * kRowsPerWarp + r) * PITCH)[d4];
        s[r] = fmaf(qv.x, kv.x, s[r]);
        s[r] = fmaf(qv.y, kv.y, s[r]);
        s[r] = fmaf(qv.z, kv.z, s[r]);
        s[r] = fmaf(qv.w, kv.w, s[r]);
      }
    }

    const int64_t key = j0 + lane;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const int64_t row = row0 + warp * kRowsPerWarp + r;
      float val = -INFINITY;
      if (row < p.seq_q && key < p.seq_kv && !(paged && kv_rows[lane] < 0))
        val = finish_logit(p, s[r] * p.scale, b, h, row, key, kv_limit);
      float mt = val;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
      const float m_new = fmaxf(m[r], mt);
      float pj = 0.f, corr = 1.f;
      if (m_new != -INFINITY) {
        corr = (m[r] == -INFINITY) ? 0.f : softmax_exp<T>(m[r] - m_new);
        pj = (val == -INFINITY) ? 0.f : softmax_exp<T>(val - m_new);
      }
      float ps = pj;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      l[r] = l[r] * corr + ps;
      m[r] = m_new;
#pragma unroll
      for (int i = 0; i < ND; ++i) acc[r][i] *= corr;
      Ps[(warp * kRowsPerWarp + r) * kBN + lane] = pj;
    }
    __syncwarp();

#pragma unroll 2
    for (int j4 = 0; j4 < kBN / 4; ++j4) {
      float4 pv[kRowsPerWarp];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r)
        pv[r] = reinterpret_cast<const float4*>(Ps + (warp * kRowsPerWarp + r) * kBN)[j4];
#pragma unroll
      for (int i = 0; i < ND; ++i) {
        const float v0 = Vs[(j4 * 4 + 0) * PITCH + lane + 32 * i];
        const float v1 = Vs[(j4 * 4 + 1) * PITCH + lane + 32 * i];
        const float v2 = Vs[(j4 * 4 + 2) * PITCH + lane + 32 * i];
        const float v3 = Vs[(j4 * 4 + 3) * PITCH + lane + 32 * i];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
          acc[r][i] = fmaf(pv[r].x, v0, acc[r][i]);
          acc[r][i] = fmaf(pv[r].y, v1, acc[r][i]);
          acc[r][i] = fmaf(pv[r].z, v2, acc[r][i]);
          acc[r][i] = fmaf(pv[r].w, v3, acc[r][i]);
        }
      }
    }
    __syncwarp();
  }

  if constexpr (KS > 1) {
    // Merge the groups: each writes (acc, m, l) of its 16 rows over its own K tile, then every group forms the same
    // final max / sum / accumulator (the weights pass below needs the final statistics in every group).
    constexpr int MP = DMAX + 2;
    group_sync(grp);   // this group's last tile has been multiplied
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      float* mine = Ks + (warp * kRowsPerWarp + r) * MP;
#pragma unroll
      for (int i = 0; i < ND; ++i) mine[lane + 32 * i] = acc[r][i];
      if (lane == 0) { mine[DMAX] = m[r]; mine[DMAX + 1] = l[r]; }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      float mg[KS], m_all = -INFINITY;
#pragma unroll
      for (int g = 0; g < KS; ++g) {
        mg[g] = (Qs + kBM * PITCH + g * GroupFloats<DMAX>::value)[(warp * kRowsPerWarp + r) * MP + DMAX];
        m_all = fmaxf(m_all, mg[g]);
      }
      float l_all = 0.f, a_all[ND];
#pragma unroll
      for (int i = 0; i < ND; ++i) a_all[i] = 0.f;
#pragma unroll
      for (int g = 0; g < KS; ++g) {
        const float* theirs = Qs + kBM * PITCH + g * GroupFloats<DMAX>::value + (warp * kRowsPerWarp + r) * MP;
        const float f = (mg[g] == -INFINITY) ? 0.f : softmax_exp<T>(mg[g] - m_all);
        l_all = fmaf(theirs[DMAX + 1], f, l_all);
#pragma unroll
        for (int i = 0; i < ND; ++i) a_all[i] = fmaf(theirs[lane + 32 * i], f, a_all[i]);
      }
      m[r] = m_all;
      l[r] = l_all;
#pragma unroll
      for (int i = 0; i < ND; ++i) acc[r][i] = a_all[i];
    }
    __syncthreads();   // the partial results have been read: the K tiles may be reused by the weights pass
  }

  // Probabilities on request (the reference's `out attentionWeights`; its GQA kernel writes them the same way, from
  // the final row statistics: CUDA/Kernels/CudaAttentionKernels.cs:628-642): a second pass over the keys recomputes
  // every logit and stores exp(logit - max) / sum.  Masked positions and fully masked rows give exact zeros.
  if (p.weights) {
    for (int64_t j0 = j_first; j0 < p.seq_kv; j0 += j_step) {
      group_sync(grp);
      const bool live = j0 < kend;   // tiles past the last visible key only need their zeros written
      if (live) {   // (the host refuses weights together with a block table, so keys are rows of K here)
        for (int idx = tid; idx < kBN * DMAX; idx += kWarps * 32) {
          const int j = idx / DMAX, d = idx - j * DMAX;
          const int64_t key = j0 + j;
          Ks[j * PITCH + d] = (key < kend && d < D) ? to_float<T>(kb[key * p.ks[2] + d]) : 0.f;
        }
        group_sync(grp);
      }
      float s[kRowsPerWarp] = {0.f, 0.f, 0.f, 0.f};
      if (live) {
        const float4* krow = reinterpret_cast<const float4*>(Ks + lane * PITCH);
#pragma unroll 4
        for (int d4 = 0; d4 < DMAX / 4; ++d4) {
          const float4 kv = krow[d4];
#pragma unroll
          for (int r = 0; r < kRowsPerWarp; ++r) {
            const float4 qv = reinterpret_cast<const float4*>(Qs + (warp * kRowsPerWarp + r) * PITCH)[d4];
            s[r] = fmaf(qv.x, kv.x, s[r]);
            s[r] = fmaf(qv.y, kv.y, s[r]);
            s[r] = fmaf(qv.z, kv.z, s[r]);
            s[r] = fmaf(qv.w, kv.w, s[r]);
          }
        }
      }
      const int64_t key = j0 + lane;
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        const int64_t row = row0 + warp * kRowsPerWarp + r;
        if (row >= p.seq_q || key >= p.seq_kv) continue;
        float w = 0.f;
        if (live && l[r] > 0.f) {
          const float val = finish_logit(p, s[r] * p.scale, b, h, row, key, kv_limit);
          if (val != -INFINITY) w = softmax_exp<T>(val - m[r]) / l[r];
        }
        p.weights[(((int64_t)b * p.num_q_heads + h) * p.seq_q + row) * p.seq_kv + key] = w;
      }
    }
  }

  report_bad_block(p, bad_block);
  if (grp != 0) return;   // every group holds the merged result; the first one stores it
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int64_t row = row0 + warp * kRowsPerWarp + r;
    if (row >= p.seq_q) continue;
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
    const int64_t obase = b * p.os[0] + h * p.os[1] + row * p.os[2];
#pragma unroll
    for (int i = 0; i < ND; ++i) {
      const int d = lane + 32 * i;
      if (d < D) store_out<T>(p.out, obase + d, acc[r][i] * inv, p.out_f32);
    }
    if (p.lse && lane == 0)
      p.lse[((int64_t)b * p.num_q_heads + h) * p.seq_q + row] = (l[r] > 0.f) ? m[r] + logf(l[r]) : -INFINITY;
  }
}

template <typename T, int DMAX, int KS>
cudaError_t launch_k(const SdpaParams& p, cudaStream_t stream) {
  constexpr int PITCH = DMAX + 4;
  const size_t smem = sizeof(float) * (kBM * PITCH + KS * GroupFloats<DMAX>::value);
  auto kern = sdpa_generic_kernel<T, DMAX, KS>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  dim3 grid((unsigned)((p.seq_q + kBM - 1) / kBM), (unsigned)p.head_count, (unsigned)p.batch);
  kern<<<grid, KS * kWarps * 32, smem, stream>>>(p);
  return cudaGetLastError();
}

template <typename T, int DMAX>
cudaError_t launch_t(const SdpaParams& p, cudaStream_t stream) {
  // Few CTAs and several key tiles each: split the keys over four groups per CTA (head_dim <= 128: the four K / V
  // tile pairs fit in shared memory).  A B200 has 148 SMs; up to two CTAs per SM still leave most schedulers with a
  // single warp.
  const int64_t ctas = ((p.seq_q + kBM - 1) / kBM) * (int64_t)p.head_count * p.batch;
  if constexpr (DMAX <= 128) {
    if (ctas <= 2 * 148 && p.seq_kv >= 4 * kBN) return launch_k<T, DMAX, 4>(p, stream);
  }
  return launch_k<T, DMAX, 1>(p, stream);
}

template <typename T>
cudaError_t launch_d(const SdpaParams& p, cudaStream_t stream) {
  if (p.head_dim <= 64) return launch_t<T, 64>(p, stream);
  if (p.head_dim <= 128) return launch_t<T, 128>(p, stream);
  return launch_t<T, 256>(p, stream);
}

}  // namespace

cudaError_t launch_generic(const SdpaParams& p, int dtype, cudaStream_t stream) {
  switch (dtype) {
    case AIDN_F32: return launch_d<float>(p, stream);
    case AIDN_F16: return launch_d<__half>(p, stream);
    default: return launch_d<__nv_bfloat16>(p, stream);
  }
}

}  // namespace aidn
