// Attention backward with LSE recompute: dQ, dK, dV from dO, Q, K, V, O and the forward's log-sum-exp.
//
// Replaces flash_attention_backward_gradq_deterministic / _gradkv_deterministic of the reference
// (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/Kernels/CudaAttentionKernels.cs:251-390; host
// CUDA/CudaBackend.cs:8580-8704; CPU Engines/CpuEngine.cs:29474): one thread per query row, and one thread per
// (key, d) that recomputes the whole score row per query.  As there, every output cell is owned by one thread and
// summed in a fixed order, so the result is deterministic (no atomics).
//
//   P  = exp(S - lse),  S = scale * Q K^T (+ bias, masks)          delta_i = sum_d dO_id O_id
//   dV = P^T dO         dP = dO V^T        dS = P * (dP - delta)   dQ = scale * dS K     dK = scale * dS^T Q
//
// fp32 FFMA arithmetic with K/V (or Q/dO) tiles staged in shared memory, any head_dim <= 256, every mask kind of the
// forward, grouped-query attention (dK / dV sum over the query heads of the group).  A correctness-first kernel: it
// shares the generic forward kernel's tiling, not the tcgen05 kernel's.
#include <type_traits>

#include "common.cuh"
#include "mma_sync.cuh"
#include "sm100_ptx.cuh"

namespace aidn {
namespace {

constexpr int kRows = 16;      // query rows per tile
constexpr int kKeys = 32;      // keys per tile
constexpr int kBwdWarps = 4;

template <typename T>
__device__ __forceinline__ float load_o(const void* base, int64_t idx, int f32) {
  return f32 ? static_cast<const float*>(base)[idx] : to_float<T>(static_cast<const T*>(base)[idx]);
}

// delta[b, h, i] = sum_d dO * O; one warp per row.
template <typename T>
__global__ void __launch_bounds__(128) bwd_delta_kernel(const BwdParams bp) {
  const SdpaParams& p = bp.p;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int hl = blockIdx.y, b = blockIdx.z;
  if (row >= p.seq_q) return;
  const int h = p.head_begin + hl;
  const int64_t ob = b * p.os[0] + (int64_t)h * p.os[1] + row * p.os[2];
  const int64_t gb = b * bp.dos[0] + (int64_t)h * bp.dos[1] + row * bp.dos[2];
  float acc = 0.f;
  T* gt = bp.dout_t ? static_cast<T*>(bp.dout_t) + (((int64_t)b * p.head_count + hl) * p.seq_q + row) * p.head_dim : nullptr;
  // fp32 O and dO with 16-byte aligned rows: four elements per lane and load
  const bool vec = p.out_f32 && p.head_dim % 4 == 0 && ((ob | gb) & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(bp.dout)) & 15) == 0 &&
                   (!gt || sizeof(T) == 2) && ((reinterpret_cast<uintptr_t>(bp.dout_t) & 7) == 0);
  if (vec) {
    const float4* o4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.out) + ob);
    const float4* g4 = reinterpret_cast<const float4*>(static_cast<const float*>(bp.dout) + gb);
    for (int d4 = lane; d4 < p.head_dim / 4; d4 += 32) {
      const float4 o = o4[d4];
      float4 g = g4[d4];
      if (gt) {
        T t4[4] = {from_float<T>(g.x), from_float<T>(g.y), from_float<T>(g.z), from_float<T>(g.w)};
        *reinterpret_cast<uint2*>(gt + 4 * d4) = *reinterpret_cast<const uint2*>(t4);
        if (bp.round_dout) g = make_float4(to_float<T>(t4[0]), to_float<T>(t4[1]), to_float<T>(t4[2]), to_float<T>(t4[3]));
      }
      acc += g.x * o.x + g.y * o.y + g.z * o.z + g.w * o.w;
    }
  } else {
    for (int d = lane; d < p.head_dim; d += 32) {
      float go = load_o<T>(bp.dout, gb + d, p.out_f32);
      if (gt) {
        gt[d] = from_float<T>(go);   // the tensor-core dK / dV kernels stream dO in the input dtype
        if (bp.round_dout) go = to_float<T>(gt[d]);
      }
      acc += go * load_o<T>(p.out, ob + d, p.out_f32);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) bp.delta[((int64_t)b * p.head_count + hl) * p.seq_q + row] = acc;
}

// Probability and score gradient of (row, key): p = exp(logit - lse), ds = p * (dp - delta).
__device__ __forceinline__ void prob_and_ds(const SdpaParams& p, float s, float dp, float lse, float delta, int b, int h,
                                            int64_t row, int64_t key, int64_t kv_limit, float& pj, float& ds) {
  pj = 0.f;
  if (row < p.seq_q && key < p.seq_kv && lse != -INFINITY) {
    const float val = finish_logit(p, s * p.scale, b, h, row, key, kv_limit);
    if (val != -INFINITY) pj = expf(val - lse);
  }
  ds = pj * (dp - delta);
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(kBwdWarps * 32) bwd_dq_kernel(const BwdParams bp) {
  const SdpaParams& p = bp.p;
  constexpr int PITCH = DMAX + 4;
  constexpr int ND = DMAX / 32;
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;                       // [kRows][PITCH]
  float* Gs = Qs + kRows * PITCH;         // dO, [kRows][PITCH]
  float* Ks = Gs + kRows * PITCH;         // [kKeys][PITCH]
  float* Vs = Ks + kKeys * PITCH;         // [kKeys][PITCH]
  float* Ds = Vs + kKeys * PITCH;         // dS, [kRows][kKeys]
  __shared__ int64_t kv_rows[kKeys];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, hl = blockIdx.y, h = p.head_begin + hl, kvh = h / p.group;
  const int64_t row0 = (int64_t)blockIdx.x * kRows;
  const int D = p.head_dim;
  const bool paged = p.block_table != nullptr;
  const T* qb = static_cast<const T*>(p.q) + b * p.qs[0] + (int64_t)h * p.qs[1];
  const T* kb = static_cast<const T*>(p.k) + (paged ? 0 : b * p.ks[0]) + (int64_t)kvh * p.ks[1];
  const T* vb = static_cast<const T*>(p.v) + (paged ? 0 : b * p.vs[0]) + (int64_t)kvh * p.vs[1];

  for (int idx = tid; idx < kRows * DMAX; idx += kBwdWarps * 32) {
    const int r = idx / DMAX, d = idx - r * DMAX;
    const int64_t row = row0 + r;
    const bool ok = row < p.seq_q && d < D;
    Qs[r * PITCH + d] = ok ? to_float<T>(qb[row * p.qs[2] + d]) : 0.f;
    Gs[r * PITCH + d] = ok ? load_o<T>(bp.dout, b * bp.dos[0] + (int64_t)h * bp.dos[1] + row * bp.dos[2] + d, p.out_f32) : 0.f;
  }
  float lse[4], delta[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int64_t row = row0 + warp * 4 + r;
    lse[r] = row < p.seq_q ? p.lse[((int64_t)b * p.num_q_heads + h) * p.seq_q + row] : -INFINITY;
    delta[r] = row < p.seq_q ? bp.delta[((int64_t)b * p.head_count + hl) * p.seq_q + row] : 0.f;
  }
  const int64_t kv_limit = kv_limit_of(p, b);
  int64_t kend = kv_limit;
  if (p.causal) {
    int64_t last_row = row0 + kRows - 1;
    if (last_row > p.seq_q - 1) last_row = p.seq_q - 1;
    const int64_t c = last_row + p.causal_offset + 1;
    if (c < kend) kend = c;
  }
  bool bad_block = false;
  float acc[4][ND];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[r][i] = 0.f;

  for (int64_t j0 = 0; j0 < kend; j0 += kKeys) {
    __syncthreads();
    if (paged) {
      if (tid < kKeys) kv_rows[tid] = (j0 + tid < kend) ? kv_row_of(p, b, j0 + tid, bad_block) : -1;
      __syncthreads();
    }
    for (int idx = tid; idx < kKeys * DMAX; idx += kBwdWarps * 32) {
      const int j = idx / DMAX, d = idx - j * DMAX;
      const int64_t key = j0 + j;
      const int64_t row = paged ? kv_rows[j] : key;
      const bool ok = key < p.seq_kv && d < D && row >= 0;
      Ks[j * PITCH + d] = ok ? to_float<T>(kb[row * p.ks[2] + d]) : 0.f;
      Vs[j * PITCH + d] = ok ? to_float<T>(vb[row * p.vs[2] + d]) : 0.f;
    }
    __syncthreads();

    float s[4] = {0.f, 0.f, 0.f, 0.f}, dp[4] = {0.f, 0.f, 0.f, 0.f};
    const float4* krow = reinterpret_cast<const float4*>(Ks + lane * PITCH);
    const float4* vrow = reinterpret_cast<const float4*>(Vs + lane * PITCH);
#pragma unroll 2
    for (int d4 = 0; d4 < DMAX / 4; ++d4) {
      const float4 kv = krow[d4], vv = vrow[d4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float4 qv = reinterpret_cast<const float4*>(Qs + (warp * 4 + r) * PITCH)[d4];
        const float4 gv = reinterpret_cast<const float4*>(Gs + (warp * 4 + r) * PITCH)[d4];
        s[r] = fmaf(qv.x, kv.x, s[r]); s[r] = fmaf(qv.y, kv.y, s[r]); s[r] = fmaf(qv.z, kv.z, s[r]); s[r] = fmaf(qv.w, kv.w, s[r]);
        dp[r] = fmaf(gv.x, vv.x, dp[r]); dp[r] = fmaf(gv.y, vv.y, dp[r]); dp[r] = fmaf(gv.z, vv.z, dp[r]); dp[r] = fmaf(gv.w, vv.w, dp[r]);
      }
    }
    const int64_t key = j0 + lane;
    const bool key_ok = !(paged && kv_rows[lane] < 0);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      float pj, ds;
      prob_and_ds(p, s[r], dp[r], key_ok ? lse[r] : -INFINITY, delta[r], b, h, row0 + warp * 4 + r, key, kv_limit, pj, ds);
      Ds[(warp * 4 + r) * kKeys + lane] = ds;
    }
    __syncwarp();
#pragma unroll 2
    for (int j4 = 0; j4 < kKeys / 4; ++j4) {
      float4 dv4[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) dv4[r] = reinterpret_cast<const float4*>(Ds + (warp * 4 + r) * kKeys)[j4];
#pragma unroll
      for (int i = 0; i < ND; ++i) {
        const float k0 = Ks[(j4 * 4 + 0) * PITCH + lane + 32 * i], k1 = Ks[(j4 * 4 + 1) * PITCH + lane + 32 * i];
        const float k2 = Ks[(j4 * 4 + 2) * PITCH + lane + 32 * i], k3 = Ks[(j4 * 4 + 3) * PITCH + lane + 32 * i];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          acc[r][i] = fmaf(dv4[r].x, k0, acc[r][i]); acc[r][i] = fmaf(dv4[r].y, k1, acc[r][i]);
          acc[r][i] = fmaf(dv4[r].z, k2, acc[r][i]); acc[r][i] = fmaf(dv4[r].w, k3, acc[r][i]);
        }
      }
    }
    __syncwarp();
  }
  report_bad_block(p, bad_block);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int64_t row = row0 + warp * 4 + r;
    if (row >= p.seq_q) continue;
    float* out = bp.dq + (((int64_t)b * p.head_count + hl) * p.seq_q + row) * D;
#pragma unroll
    for (int i = 0; i < ND; ++i) {
      const int d = lane + 32 * i;
      if (d < D) out[d] = acc[r][i] * p.scale;
    }
  }
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(kBwdWarps * 32) bwd_dkv_kernel(const BwdParams bp) {
  const SdpaParams& p = bp.p;
  constexpr int PITCH = DMAX + 4;
  constexpr int ND = DMAX / 32;
  constexpr int KPW = kKeys / kBwdWarps;   // keys owned by a warp in the accumulation phase
  extern __shared__ __align__(16) float smem[];
  float* Ks = smem;                       // [kKeys][PITCH]
  float* Vs = Ks + kKeys * PITCH;
  float* Qs = Vs + kKeys * PITCH;         // [kRows][PITCH]
  float* Gs = Qs + kRows * PITCH;
  float* Ps = Gs + kRows * PITCH;         // [kRows][kKeys]
  float* Ds = Ps + kRows * kKeys;         // [kRows][kKeys]
  __shared__ int64_t kv_rows[kKeys];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z;
  const int kvl = blockIdx.y;                              // kv head within the shard
  const int kvh = p.head_begin / p.group + kvl;
  const int64_t j0 = (int64_t)blockIdx.x * kKeys;
  const int D = p.head_dim;
  const bool paged = p.block_table != nullptr;
  const T* kb = static_cast<const T*>(p.k) + (paged ? 0 : b * p.ks[0]) + (int64_t)kvh * p.ks[1];
  const T* vb = static_cast<const T*>(p.v) + (paged ? 0 : b * p.vs[0]) + (int64_t)kvh * p.vs[1];
  const int64_t kv_limit = kv_limit_of(p, b);
  bool bad_block = false;

  if (paged) {
    if (tid < kKeys) kv_rows[tid] = (j0 + tid < kv_limit) ? kv_row_of(p, b, j0 + tid, bad_block) : -1;
    __syncthreads();
  }
  for (int idx = tid; idx < kKeys * DMAX; idx += kBwdWarps * 32) {
    const int j = idx / DMAX, d = idx - j * DMAX;
    const int64_t key = j0 + j;
    const int64_t row = paged ? kv_rows[j] : key;
    const bool ok = key < p.seq_kv && d < D && row >= 0;
    Ks[j * PITCH + d] = ok ? to_float<T>(kb[row * p.ks[2] + d]) : 0.f;
    Vs[j * PITCH + d] = ok ? to_float<T>(vb[row * p.vs[2] + d]) : 0.f;
  }

  float accK[KPW][ND], accV[KPW][ND];
#pragma unroll
  for (int jj = 0; jj < KPW; ++jj)
#pragma unroll
    for (int i = 0; i < ND; ++i) accK[jj][i] = accV[jj][i] = 0.f;

  // first query row that can see key j0 (causal: key <= row + offset)
  int64_t r_first = 0;
  if (p.causal) {
    r_first = j0 - p.causal_offset;
    if (r_first < 0) r_first = 0;
    r_first = r_first / kRows * kRows;
  }
  const bool tile_visible = j0 < kv_limit;

  for (int g = 0; g < p.group && tile_visible; ++g) {
    const int h = kvh * p.group + g, hl = h - p.head_begin;
    const T* qb = static_cast<const T*>(p.q) + b * p.qs[0] + (int64_t)h * p.qs[1];
    for (int64_t row0 = r_first; row0 < p.seq_q; row0 += kRows) {
      __syncthreads();   // previous tile consumed (and K/V staged before the first use)
      for (int idx = tid; idx < kRows * DMAX; idx += kBwdWarps * 32) {
        const int r = idx / DMAX, d = idx - r * DMAX;
        const int64_t row = row0 + r;
        const bool ok = row < p.seq_q && d < D;
        Qs[r * PITCH + d] = ok ? to_float<T>(qb[row * p.qs[2] + d]) : 0.f;
        Gs[r * PITCH + d] = ok ? load_o<T>(bp.dout, b * bp.dos[0] + (int64_t)h * bp.dos[1] + row * bp.dos[2] + d, p.out_f32) : 0.f;
      }
      __syncthreads();
      // phase A: warp w takes rows 4w..4w+3, lane j takes key j0 + j
      {
        float s[4] = {0.f, 0.f, 0.f, 0.f}, dp[4] = {0.f, 0.f, 0.f, 0.f};
        const float4* krow = reinterpret_cast<const float4*>(Ks + lane * PITCH);
        const float4* vrow = reinterpret_cast<const float4*>(Vs + lane * PITCH);
#pragma unroll 2
        for (int d4 = 0; d4 < DMAX / 4; ++d4) {
          const float4 kv = krow[d4], vv = vrow[d4];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const float4 qv = reinterpret_cast<const float4*>(Qs + (warp * 4 + r) * PITCH)[d4];
            const float4 gv = reinterpret_cast<const float4*>(Gs + (warp * 4 + r) * PITCH)[d4];
            s[r] = fmaf(qv.x, kv.x, s[r]); s[r] = fmaf(qv.y, kv.y, s[r]); s[r] = fmaf(qv.z, kv.z, s[r]); s[r] = fmaf(qv.w, kv.w, s[r]);
            dp[r] = fmaf(gv.x, vv.x, dp[r]); dp[r] = fmaf(gv.y, vv.y, dp[r]); dp[r] = fmaf(gv.z, vv.z, dp[r]); dp[r] = fmaf(gv.w, vv.w, dp[r]);
          }
        }
        const int64_t key = j0 + lane;
        const bool key_ok = !(paged && kv_rows[lane] < 0);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int64_t row = row0 + warp * 4 + r;
          float lse = -INFINITY, delta = 0.f;
          if (row < p.seq_q && key_ok) {
            lse = p.lse[((int64_t)b * p.num_q_heads + h) * p.seq_q + row];
            delta = bp.delta[((int64_t)b * p.head_count + hl) * p.seq_q + row];
          }
          float pj, ds;
          prob_and_ds(p, s[r], dp[r], lse, delta, b, h, row, key, kv_limit, pj, ds);
          Ps[(warp * 4 + r) * kKeys + lane] = pj;
          Ds[(warp * 4 + r) * kKeys + lane] = ds;
        }
      }
      __syncthreads();
      // phase B: warp w owns keys KPW*w .. KPW*w + KPW - 1, lane owns dims lane + 32 i; rows in ascending order
#pragma unroll 2
      for (int r = 0; r < kRows; ++r) {
        float pw[KPW], dw[KPW];
#pragma unroll
        for (int jj = 0; jj < KPW; ++jj) {
          pw[jj] = Ps[r * kKeys + warp * KPW + jj];
          dw[jj] = Ds[r * kKeys + warp * KPW + jj];
        }
#pragma unroll
        for (int i = 0; i < ND; ++i) {
          const float gq = Gs[r * PITCH + lane + 32 * i], qq = Qs[r * PITCH + lane + 32 * i];
#pragma unroll
          for (int jj = 0; jj < KPW; ++jj) {
            accV[jj][i] = fmaf(pw[jj], gq, accV[jj][i]);
            accK[jj][i] = fmaf(dw[jj], qq, accK[jj][i]);
          }
        }
      }
    }
  }
  report_bad_block(p, bad_block);
#pragma unroll
  for (int jj = 0; jj < KPW; ++jj) {
    const int64_t key = j0 + warp * KPW + jj;
    if (key >= p.seq_kv) continue;
    const int64_t base = (((int64_t)b * (p.head_count / p.group) + kvl) * p.seq_kv + key) * D;
#pragma unroll
    for (int i = 0; i < ND; ++i) {
      const int d = lane + 32 * i;
      if (d < D) {
        bp.dk[base + d] = accK[jj][i] * p.scale;
        bp.dv[base + d] = accV[jj][i];
      }
    }
  }
}

// ---- dQ on the warp-level tensor cores (fp16 / bf16 inputs, head_dim 64 or 128, contiguous K / V) ------------------
// A CTA of 4 warps takes 64 query rows (16 per warp, held as resident A fragments of Q and dO) and streams K and V in
// 32-key tiles through a 3-stage cp.async ring shared by the warps.  Per 16 keys a warp computes S = Q K^T and
// dP = dO V^T (mma.sync, the 16-byte chunks of a K / V row feeding the k slots in arrival order as in the decode
// kernel), turns them into dS = P (dP - delta) in registers, and accumulates dQ^T += K^T dS^T with the rows as the N
// dimension: the dS accumulators are, as they stand, the B fragments, and the A fragments pair two keys of one d by a
// byte permute of two K rows.  K is read in both patterns from one shared-memory copy; the chunk swizzle
// 2*((row/2)&3) ^ 4*(row&1) keeps both reads bank-conflict free.  Deterministic: one thread owns each dQ cell.
constexpr int kMmaRows = 64;
constexpr int kMmaKeys = 32;
constexpr int kMmaStages = 3;

__device__ __forceinline__ int tile_swz(int row) { return (((row >> 1) & 3) << 1) ^ ((row & 1) << 2); }

__device__ __forceinline__ void lds128(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// 8 consecutive elements of a row as four registers of T pairs; `f32` rows are converted.
template <typename T>
__device__ __forceinline__ void load_frag8(const void* base, int64_t idx, int f32, bool ok, uint32_t (&r)[4]) {
  r[0] = r[1] = r[2] = r[3] = 0u;
  if (!ok) return;
  if (f32) {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx + 4);
    r[0] = pack_pair<T>(a.x, a.y); r[1] = pack_pair<T>(a.z, a.w); r[2] = pack_pair<T>(b.x, b.y); r[3] = pack_pair<T>(b.z, b.w);
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const T*>(base) + idx);
    r[0] = u.x; r[1] = u.y; r[2] = u.z; r[3] = u.w;
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(128, 2) bwd_dq_mma_kernel(const BwdParams bp) {
  const SdpaParams& p = bp.p;
  constexpr int KI = D / 32, VX = D / 64, MT = D / 16, CH = D / 8, ROWB = D * 2;
  constexpr int TILEB = kMmaKeys * ROWB, STAGEB = 2 * TILEB;
  extern __shared__ __align__(128) uint8_t bsm[];
  const uint32_t s0 = ptx::smem_u32(bsm);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int b = blockIdx.z, hl = blockIdx.y, h = p.head_begin + hl, kvh = h / p.group;
  const int64_t cta_row0 = (int64_t)blockIdx.x * kMmaRows;
  const int64_t row0 = cta_row0 + warp * 16;
  const int64_t rA = row0 + g, rB = row0 + g + 8;

  uint32_t qa[KI][4], qb[KI][4], ga[KI][4], gb[KI][4];
  {
    const int64_t qbase = b * p.qs[0] + (int64_t)h * p.qs[1], gbase = b * bp.dos[0] + (int64_t)h * bp.dos[1];
#pragma unroll
    for (int i = 0; i < KI; ++i) {
      const int col = (i * 4 + c) * 8;
      load_frag8<T>(p.q, qbase + rA * p.qs[2] + col, 0, rA < p.seq_q, qa[i]);
      load_frag8<T>(p.q, qbase + rB * p.qs[2] + col, 0, rB < p.seq_q, qb[i]);
      load_frag8<T>(bp.dout, gbase + rA * bp.dos[2] + col, p.out_f32, rA < p.seq_q, ga[i]);
      load_frag8<T>(bp.dout, gbase + rB * bp.dos[2] + col, p.out_f32, rB < p.seq_q, gb[i]);
    }
  }
  float lseA = -INFINITY, lseB = -INFINITY, dlA = 0.f, dlB = 0.f;
  if (rA < p.seq_q) {
    lseA = p.lse[((int64_t)b * p.num_q_heads + h) * p.seq_q + rA];
    dlA = bp.delta[((int64_t)b * p.head_count + hl) * p.seq_q + rA];
  }
  if (rB < p.seq_q) {
    lseB = p.lse[((int64_t)b * p.num_q_heads + h) * p.seq_q + rB];
    dlB = bp.delta[((int64_t)b * p.head_count + hl) * p.seq_q + rB];
  }
  const int64_t kv_limit = kv_limit_of(p, b);
  int64_t kend = kv_limit;
  if (p.causal) {
    int64_t last_row = cta_row0 + kMmaRows - 1;
    if (last_row > p.seq_q - 1) last_row = p.seq_q - 1;
    const int64_t cl = last_row + p.causal_offset + 1;
    if (cl < kend) kend = cl;
  }
  if (kend < 0) kend = 0;
  const int nsteps = (int)((kend + kMmaKeys - 1) / kMmaKeys);

  const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + (int64_t)kvh * p.ks[1];
  const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + (int64_t)kvh * p.vs[1];
  // the CTA's 128 threads copy a 32-key tile of K and of V: CH chunks per row
  auto issue = [&](int step) {
    const uint32_t base = s0 + (step % kMmaStages) * STAGEB;
    const int64_t j0 = (int64_t)step * kMmaKeys;
#pragma unroll
    for (int r = 0; r < kMmaKeys * CH / 128; ++r) {
      const int idx = tid + r * 128;
      const int row = idx / CH, ch = idx - row * CH;
      const int64_t key = j0 + row;
      const bool valid = key < kend;
      const int64_t ko = valid ? key : 0;
      const uint32_t off = (uint32_t)(row * ROWB + ((ch ^ tile_swz(row)) << 4));
      cp_async16(base + off, kbase + ko * p.ks[2] + ch * 8, valid);
      cp_async16(base + TILEB + off, vbase + ko * p.vs[2] + ch * 8, valid);
    }
    cp_async_commit();
  };

  float acc[MT][2][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int hn = 0; hn < 2; ++hn) acc[m][hn][0] = acc[m][hn][1] = acc[m][hn][2] = acc[m][hn][3] = 0.f;

#pragma unroll
  for (int s = 0; s < kMmaStages; ++s) {
    if (s < nsteps) issue(s);
    else cp_async_commit();
  }
  for (int step = 0; step < nsteps; ++step) {
    cp_async_wait<kMmaStages - 1>();
    __syncthreads();
    const uint32_t kb_s = s0 + (step % kMmaStages) * STAGEB, vb_s = kb_s + TILEB;
    const int64_t j0 = (int64_t)step * kMmaKeys;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float sacc[2][4], pacc[2][4];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        sacc[t][0] = sacc[t][1] = sacc[t][2] = sacc[t][3] = 0.f;
        pacc[t][0] = pacc[t][1] = pacc[t][2] = pacc[t][3] = 0.f;
        const int kr = hh * 16 + t * 8 + g;
        const int sw = tile_swz(kr);
#pragma unroll
        for (int i = 0; i < KI; ++i) {
          uint32_t kw[4], vw[4];
          const uint32_t off = (uint32_t)(kr * ROWB + (((i * 4 + c) ^ sw) << 4));
          lds128(kb_s + off, kw);
          lds128(vb_s + off, vw);
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            mma16816<T>(sacc[t], qa[i][2 * h2], qb[i][2 * h2], qa[i][2 * h2 + 1], qb[i][2 * h2 + 1], kw[2 * h2], kw[2 * h2 + 1]);
            mma16816<T>(pacc[t], ga[i][2 * h2], gb[i][2 * h2], ga[i][2 * h2 + 1], gb[i][2 * h2 + 1], vw[2 * h2], vw[2 * h2 + 1]);
          }
        }
      }
      float ds[2][4];
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int64_t key = j0 + hh * 16 + t * 8 + 2 * c + e;
          float pj;
          prob_and_ds(p, sacc[t][e], pacc[t][e], lseA, dlA, b, h, rA, key, kv_limit, pj, ds[t][e]);
          prob_and_ds(p, sacc[t][2 + e], pacc[t][2 + e], lseB, dlB, b, h, rB, key, kv_limit, pj, ds[t][2 + e]);
        }
      const uint32_t bA0 = pack_pair<T>(ds[0][0], ds[0][1]), bA1 = pack_pair<T>(ds[1][0], ds[1][1]);
      const uint32_t bB0 = pack_pair<T>(ds[0][2], ds[0][3]), bB1 = pack_pair<T>(ds[1][2], ds[1][3]);
      uint32_t kt[4][VX][4];
#pragma unroll
      for (int e4 = 0; e4 < 4; ++e4) {
        const int kr = hh * 16 + 2 * c + (e4 & 1) + (e4 >> 1) * 8;
        const int sw = tile_swz(kr);
#pragma unroll
        for (int x = 0; x < VX; ++x) lds128(kb_s + (uint32_t)(kr * ROWB + (((g + 8 * x) ^ sw) << 4)), kt[e4][x]);
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const uint32_t sel = (m & 1) ? 0x7632u : 0x5410u;
        constexpr int xh = VX - 1;
        const int wl = m >> 1, wh = (D == 128) ? (m >> 1) : 2 + (m >> 1);
        const uint32_t a0 = __byte_perm(kt[0][0][wl], kt[1][0][wl], sel);
        const uint32_t a1 = __byte_perm(kt[0][xh][wh], kt[1][xh][wh], sel);
        const uint32_t a2 = __byte_perm(kt[2][0][wl], kt[3][0][wl], sel);
        const uint32_t a3 = __byte_perm(kt[2][xh][wh], kt[3][xh][wh], sel);
        mma16816<T>(acc[m][0], a0, a1, a2, a3, bA0, bA1);
        mma16816<T>(acc[m][1], a0, a1, a2, a3, bB0, bB1);
      }
    }
    __syncthreads();   // every warp is done with the stage before it is refilled
    if (step + kMmaStages < nsteps) issue(step + kMmaStages);
    else cp_async_commit();
  }

  // acc[m][hn][e]: row row0 + 8 hn + 2c + (e & 1), d = d_lo(m) for e < 2, d_hi(m) for e >= 2
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const int d_lo = g * 8 + m, d_hi = (D == 128) ? (g + 8) * 8 + m : g * 8 + 4 + m;
#pragma unroll
    for (int hn = 0; hn < 2; ++hn)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int64_t row = row0 + 8 * hn + 2 * c + e;
        if (row >= p.seq_q) continue;
        float* out = bp.dq + (((int64_t)b * p.head_count + hl) * p.seq_q + row) * D;
        out[d_lo] = acc[m][hn][e] * p.scale;
        out[d_hi] = acc[m][hn][2 + e] * p.scale;
      }
  }
}

// ---- dK, dV on the warp-level tensor cores ---------------------------------------------------------------------------
// A CTA of 4 warps owns 64 keys of one KV head (16 per warp; their K and V rows sit in shared memory for the whole
// kernel) and streams Q and dO in 32-row tiles through a 3-stage cp.async ring, over the query heads of the group and
// the row tiles that can see the keys.  Per 16 rows a warp computes S^T = K Q^T and dP^T = V dO^T (keys as M), turns
// them into P^T and dS^T in registers, and accumulates dV^T += dO^T P and dK^T += Q^T dS with its keys as the N
// dimension: P^T / dS^T accumulators are the B fragments as they stand, the A fragments pair two rows of one d by a
// byte permute.  Rows are visited in ascending order by one warp per key: deterministic.
template <typename T, int D>
__global__ void __launch_bounds__(128, 2) bwd_dkv_mma_kernel(const BwdParams bp) {
  const SdpaParams& p = bp.p;
  constexpr int KI = D / 32, VX = D / 64, MT = D / 16, CH = D / 8, ROWB = D * 2;
  constexpr int kOwn = 64;                                  // keys per CTA
  constexpr int OWNB = kOwn * ROWB;                         // K (and V) of the CTA's keys
  constexpr int TILEB = kMmaKeys * ROWB;                    // 32 rows of Q (and of dO)
  constexpr int STAGEB = 2 * TILEB + 2 * kMmaKeys * 4;      // + lse[32] + delta[32]
  extern __shared__ __align__(128) uint8_t bsm[];
  const uint32_t s0 = ptx::smem_u32(bsm);
  const uint32_t k_s = s0, v_s = s0 + OWNB, ring = s0 + 2 * OWNB;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int b = blockIdx.z, kvl = blockIdx.y, kvh = p.head_begin / p.group + kvl;
  const int64_t key0 = (int64_t)blockIdx.x * kOwn;
  const int64_t kv_limit = kv_limit_of(p, b);
  const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + (int64_t)kvh * p.ks[1];
  const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + (int64_t)kvh * p.vs[1];

  // own keys (zero rows past the end)
#pragma unroll
  for (int r = 0; r < kOwn * CH / 128; ++r) {
    const int idx = tid + r * 128;
    const int row = idx / CH, ch = idx - row * CH;
    const int64_t key = key0 + row;
    const bool valid = key < p.seq_kv;
    const int64_t ko = valid ? key : 0;
    const uint32_t off = (uint32_t)(row * ROWB + ((ch ^ tile_swz(row)) << 4));
    cp_async16(k_s + off, kbase + ko * p.ks[2] + ch * 8, valid);
    cp_async16(v_s + off, vbase + ko * p.vs[2] + ch * 8, valid);
  }
  cp_async_commit();

  // row tiles that can see key0 or later keys of the CTA (causal: key <= row + offset)
  int64_t r_first = 0;
  if (p.causal) {
    r_first = key0 - p.causal_offset;
    if (r_first < 0) r_first = 0;
    r_first = r_first / kMmaKeys * kMmaKeys;
  }
  const int tiles_per_head = key0 < kv_limit && r_first < p.seq_q ? (int)((p.seq_q - r_first + kMmaKeys - 1) / kMmaKeys) : 0;
  const int nsteps = tiles_per_head * p.group;
  const int dstr = p.head_dim;   // dO scratch rows are dense
  const T* gsrc = bp.dout_t ? static_cast<const T*>(bp.dout_t) : static_cast<const T*>(bp.dout);

  auto issue = [&](int step) {
    const int gi = step / tiles_per_head, ti = step - gi * tiles_per_head;
    const int h = kvh * p.group + gi, hl = h - p.head_begin;
    const int64_t rbase = r_first + (int64_t)ti * kMmaKeys;
    const uint32_t base = ring + (step % kMmaStages) * STAGEB;
    const T* qsrc = static_cast<const T*>(p.q) + b * p.qs[0] + (int64_t)h * p.qs[1];
    const int64_t g_off = bp.dout_t ? (((int64_t)b * p.head_count + hl) * p.seq_q) * dstr : b * bp.dos[0] + (int64_t)h * bp.dos[1];
    const int64_t g_rs = bp.dout_t ? dstr : bp.dos[2];
#pragma unroll
    for (int r = 0; r < kMmaKeys * CH / 128; ++r) {
      const int idx = tid + r * 128;
      const int row = idx / CH, ch = idx - row * CH;
      const int64_t qr = rbase + row;
      const bool valid = qr < p.seq_q;
      const int64_t ro = valid ? qr : 0;
      const uint32_t off = (uint32_t)(row * ROWB + ((ch ^ tile_swz(row)) << 4));
      cp_async16(base + off, qsrc + ro * p.qs[2] + ch * 8, valid);
      cp_async16(base + TILEB + off, gsrc + g_off + ro * g_rs + ch * 8, valid);
    }
    if (tid < 2 * kMmaKeys) {   // lse and delta of the tile's rows: 4-byte copies, rows past the end zero-filled
      const int row = tid & (kMmaKeys - 1);
      const int64_t qr = rbase + row;
      const bool valid = qr < p.seq_q;
      const int64_t ro = valid ? qr : 0;
      const float* src = tid < kMmaKeys ? p.lse + ((int64_t)b * p.num_q_heads + h) * p.seq_q + ro
                                        : bp.delta + ((int64_t)b * p.head_count + hl) * p.seq_q + ro;
      const uint32_t n = valid ? 4u : 0u;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(base + 2 * TILEB + tid * 4), "l"(src), "r"(n) : "memory");
    }
    cp_async_commit();
  };

  float accV[MT][2][4], accK[MT][2][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int hn = 0; hn < 2; ++hn)
#pragma unroll
      for (int e = 0; e < 4; ++e) accV[m][hn][e] = accK[m][hn][e] = 0.f;

#pragma unroll
  for (int s = 0; s < kMmaStages; ++s) {
    if (s < nsteps) issue(s);
    else cp_async_commit();
  }
  const int okA = warp * 16 + g, okB = okA + 8;               // this thread's key rows in the CTA's K / V tiles
  const int64_t keyA = key0 + okA, keyB = key0 + okB;
  for (int step = 0; step < nsteps; ++step) {
    cp_async_wait<kMmaStages - 1>();   // also covers the own-keys group, committed first
    __syncthreads();
    const int gi = step / tiles_per_head, ti = step - gi * tiles_per_head;
    const int h = kvh * p.group + gi;
    const int64_t rbase = r_first + (int64_t)ti * kMmaKeys;
    const uint32_t q_s = ring + (step % kMmaStages) * STAGEB, g_s = q_s + TILEB;
    const float* stat = reinterpret_cast<const float*>(bsm + (2 * OWNB + (step % kMmaStages) * STAGEB + 2 * TILEB));
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float sacc[2][4], pacc[2][4];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        sacc[t][0] = sacc[t][1] = sacc[t][2] = sacc[t][3] = 0.f;
        pacc[t][0] = pacc[t][1] = pacc[t][2] = pacc[t][3] = 0.f;
        const int rr = hh * 16 + t * 8 + g;     // B-fragment column g = row rr of the tile
        const int swr = tile_swz(rr), swa = tile_swz(okA), swb = tile_swz(okB);
#pragma unroll
        for (int i = 0; i < KI; ++i) {
          uint32_t ka[4], kb[4], va[4], vb[4], qw[4], gw[4];
          const int ch = i * 4 + c;
          lds128(k_s + (uint32_t)(okA * ROWB + ((ch ^ swa) << 4)), ka);
          lds128(k_s + (uint32_t)(okB * ROWB + ((ch ^ swb) << 4)), kb);
          lds128(v_s + (uint32_t)(okA * ROWB + ((ch ^ swa) << 4)), va);
          lds128(v_s + (uint32_t)(okB * ROWB + ((ch ^ swb) << 4)), vb);
          lds128(q_s + (uint32_t)(rr * ROWB + ((ch ^ swr) << 4)), qw);
          lds128(g_s + (uint32_t)(rr * ROWB + ((ch ^ swr) << 4)), gw);
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            mma16816<T>(sacc[t], ka[2 * h2], kb[2 * h2], ka[2 * h2 + 1], kb[2 * h2 + 1], qw[2 * h2], qw[2 * h2 + 1]);
            mma16816<T>(pacc[t], va[2 * h2], vb[2 * h2], va[2 * h2 + 1], vb[2 * h2 + 1], gw[2 * h2], gw[2 * h2 + 1]);
          }
        }
      }
      // accumulators: [t][e] = (key A, row hh*16 + t*8 + 2c + e), [t][2 + e] = (key B, same row)
      float pr[2][4], ds[2][4];
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int rt = hh * 16 + t * 8 + 2 * c + e;
          const int64_t row = rbase + rt;
          const float lse = row < p.seq_q ? stat[rt] : -INFINITY, dl = stat[kMmaKeys + rt];
          prob_and_ds(p, sacc[t][e], pacc[t][e], lse, dl, b, h, row, keyA, kv_limit, pr[t][e], ds[t][e]);
          prob_and_ds(p, sacc[t][2 + e], pacc[t][2 + e], lse, dl, b, h, row, keyB, kv_limit, pr[t][2 + e], ds[t][2 + e]);
        }
      // B fragments: n-tile 0 = keys A (g), n-tile 1 = keys B (g + 8); k = rows 2c, 2c+1 | 2c+8, 2c+9 of the half
      const uint32_t pA0 = pack_pair<T>(pr[0][0], pr[0][1]), pA1 = pack_pair<T>(pr[1][0], pr[1][1]);
      const uint32_t pB0 = pack_pair<T>(pr[0][2], pr[0][3]), pB1 = pack_pair<T>(pr[1][2], pr[1][3]);
      const uint32_t sA0 = pack_pair<T>(ds[0][0], ds[0][1]), sA1 = pack_pair<T>(ds[1][0], ds[1][1]);
      const uint32_t sB0 = pack_pair<T>(ds[0][2], ds[0][3]), sB1 = pack_pair<T>(ds[1][2], ds[1][3]);
#pragma unroll
      for (int which = 0; which < 2; ++which) {   // 0: dV^T += dO^T P, 1: dK^T += Q^T dS
        const uint32_t src_s = which == 0 ? g_s : q_s;
        uint32_t rt4[4][VX][4];
#pragma unroll
        for (int e4 = 0; e4 < 4; ++e4) {
          const int rr = hh * 16 + 2 * c + (e4 & 1) + (e4 >> 1) * 8;
          const int sw = tile_swz(rr);
#pragma unroll
          for (int x = 0; x < VX; ++x) lds128(src_s + (uint32_t)(rr * ROWB + (((g + 8 * x) ^ sw) << 4)), rt4[e4][x]);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const uint32_t sel = (m & 1) ? 0x7632u : 0x5410u;
          constexpr int xh = VX - 1;
          const int wl = m >> 1, wh = (D == 128) ? (m >> 1) : 2 + (m >> 1);
          const uint32_t a0 = __byte_perm(rt4[0][0][wl], rt4[1][0][wl], sel);
          const uint32_t a1 = __byte_perm(rt4[0][xh][wh], rt4[1][xh][wh], sel);
          const uint32_t a2 = __byte_perm(rt4[2][0][wl], rt4[3][0][wl], sel);
          const uint32_t a3 = __byte_perm(rt4[2][xh][wh], rt4[3][xh][wh], sel);
          if (which == 0) {
            mma16816<T>(accV[m][0], a0, a1, a2, a3, pA0, pA1);
            mma16816<T>(accV[m][1], a0, a1, a2, a3, pB0, pB1);
          } else {
            mma16816<T>(accK[m][0], a0, a1, a2, a3, sA0, sA1);
            mma16816<T>(accK[m][1], a0, a1, a2, a3, sB0, sB1);
          }
        }
      }
    }
    __syncthreads();
    if (step + kMmaStages < nsteps) issue(step + kMmaStages);
    else cp_async_commit();
  }
  cp_async_wait<0>();

  // acc[m][hn][e]: key key0 + warp*16 + 8 hn + 2c + (e & 1), d = d_lo(m) for e < 2, d_hi(m) for e >= 2
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const int d_lo = g * 8 + m, d_hi = (D == 128) ? (g + 8) * 8 + m : g * 8 + 4 + m;
#pragma unroll
    for (int hn = 0; hn < 2; ++hn)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int64_t key = key0 + warp * 16 + 8 * hn + 2 * c + e;
        if (key >= p.seq_kv) continue;
        const int64_t base = (((int64_t)b * (p.head_count / p.group) + kvl) * p.seq_kv + key) * D;
        bp.dv[base + d_lo] = accV[m][hn][e];
        bp.dv[base + d_hi] = accV[m][hn][2 + e];
        bp.dk[base + d_lo] = accK[m][hn][e] * p.scale;
        bp.dk[base + d_hi] = accK[m][hn][2 + e] * p.scale;
      }
  }
}

// 16-byte vector loads of Q, K, V, dO rows: bases and strides must allow them.
inline bool mma_aligned(const BwdParams& bp) {
  const SdpaParams& p = bp.p;
  auto ok = [](const void* ptr, const int64_t* st, size_t esz) {
    if ((uintptr_t)ptr % 16) return false;
    for (int i = 0; i < 3; ++i)
      if ((st[i] * (int64_t)esz) % 16) return false;
    return true;
  };
  return ok(p.q, p.qs, 2) && ok(p.k, p.ks, 2) && ok(p.v, p.vs, 2) && ok(bp.dout, bp.dos, p.out_f32 ? 4 : 2);
}

template <typename T, int DMAX>
cudaError_t launch_bwd_t(const BwdParams& bp, cudaStream_t stream, int* launches, int* used_tcgen05) {
  const SdpaParams& p = bp.p;
  constexpr int PITCH = DMAX + 4;
  dim3 g0((unsigned)((p.seq_q + 3) / 4), (unsigned)p.head_count, (unsigned)p.batch);
  {
    // the tensor-core families multiply with dO in the input dtype: sum delta from the same rounded values
    bool tensor_cores = false;
    if constexpr (sizeof(T) == 2 && (DMAX == 64 || DMAX == 128))
      tensor_cores = p.head_dim == DMAX && !p.block_table && mma_aligned(bp) && (bp.dout_t || !p.out_f32);
    BwdParams b0 = bp;
    b0.round_dout = tensor_cores ? 1 : 0;
    bwd_delta_kernel<T><<<g0, 128, 0, stream>>>(b0);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  *used_tcgen05 = 0;
  if constexpr (sizeof(T) == 2 && (DMAX == 64 || DMAX == 128)) {
    const int dtype = std::is_same_v<T, __half> ? AIDN_F16 : AIDN_BF16;
    if (!bp.no_tcgen05 && p.head_dim == DMAX && backward_sm100_supported(bp, dtype)) {
      const char* why = "";
      *launches = 1;
      *used_tcgen05 = 1;
      return launch_backward_sm100(bp, dtype, stream, launches, &why);
    }
  }
  const size_t smem_q = sizeof(float) * ((2 * kRows + 2 * kKeys) * PITCH + kRows * kKeys);
  const size_t smem_kv = sizeof(float) * ((2 * kRows + 2 * kKeys) * PITCH + 2 * kRows * kKeys);
  auto kq = bwd_dq_kernel<T, DMAX>;
  auto kkv = bwd_dkv_kernel<T, DMAX>;
  if (smem_kv > 48 * 1024) {
    e = cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv);
    if (e != cudaSuccess) return e;
  }
  bool dq_done = false;
  if constexpr (sizeof(T) == 2 && (DMAX == 64 || DMAX == 128)) {
    if (p.head_dim == DMAX && !p.block_table && mma_aligned(bp)) {
      auto kq_mma = bwd_dq_mma_kernel<T, DMAX>;
      const size_t smem_mma = (size_t)kMmaStages * 2 * kMmaKeys * DMAX * 2;
      e = cudaFuncSetAttribute(kq_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mma);
      if (e != cudaSuccess) return e;
      dim3 gm((unsigned)((p.seq_q + kMmaRows - 1) / kMmaRows), (unsigned)p.head_count, (unsigned)p.batch);
      kq_mma<<<gm, 128, smem_mma, stream>>>(bp);
      dq_done = true;
    }
  }
  if (!dq_done) {
    dim3 g1((unsigned)((p.seq_q + kRows - 1) / kRows), (unsigned)p.head_count, (unsigned)p.batch);
    kq<<<g1, kBwdWarps * 32, smem_q, stream>>>(bp);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  bool dkv_done = false;
  if constexpr (sizeof(T) == 2 && (DMAX == 64 || DMAX == 128)) {
    if (dq_done && (bp.dout_t || !p.out_f32)) {
      auto kkv_mma = bwd_dkv_mma_kernel<T, DMAX>;
      const size_t smem_mma = 2 * 64 * (size_t)DMAX * 2 + (size_t)kMmaStages * (2 * kMmaKeys * DMAX * 2 + 2 * kMmaKeys * 4);
      e = cudaFuncSetAttribute(kkv_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mma);
      if (e != cudaSuccess) return e;
      dim3 gm((unsigned)((p.seq_kv + 63) / 64), (unsigned)(p.head_count / p.group), (unsigned)p.batch);
      kkv_mma<<<gm, 128, smem_mma, stream>>>(bp);
      dkv_done = true;
    }
  }
  if (!dkv_done) {
    dim3 g2((unsigned)((p.seq_kv + kKeys - 1) / kKeys), (unsigned)(p.head_count / p.group), (unsigned)p.batch);
    kkv<<<g2, kBwdWarps * 32, smem_kv, stream>>>(bp);
  }
  *launches = 3;
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_bwd_d(const BwdParams& bp, cudaStream_t stream, int* launches, int* used_tcgen05) {
  if (bp.p.head_dim <= 64) return launch_bwd_t<T, 64>(bp, stream, launches, used_tcgen05);
  if (bp.p.head_dim <= 128) return launch_bwd_t<T, 128>(bp, stream, launches, used_tcgen05);
  return launch_bwd_t<T, 256>(bp, stream, launches, used_tcgen05);
}

}  // namespace

cudaError_t launch_backward(const BwdParams& bp, int dtype, cudaStream_t stream, int* launches, int* used_tcgen05) {
  switch (dtype) {
    case AIDN_F32: return launch_bwd_d<float>(bp, stream, launches, used_tcgen05);
    case AIDN_F16: return launch_bwd_d<__half>(bp, stream, launches, used_tcgen05);
    default: return launch_bwd_d<__nv_bfloat16>(bp, stream, launches, used_tcgen05);
  }
}

}  // namespace aidn
