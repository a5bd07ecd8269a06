// Split-KV decode (seq_q == 1): the HBM-bound half of the attention path.
//
// One CTA streams one chunk of one (batch, kv head)'s keys and values exactly once, serves all query heads of that
// kv head, and writes an un-normalised partial (max, sum, acc[D]); a second kernel merges the partials of a
// (batch, head) by log-sum-exp.  Only keys below kv_len[b] (and the causal limit) are touched, so padding costs no
// bandwidth.  Two partial kernels:
//   * sdpa_decode_gqa_ring_kernel - fp16 / bf16, head_dim 64 or 128, up to 16 query heads per kv head (plain
//     multi-head attention included): K/V go through a per-warp cp.async shared-memory ring and both products run
//     on mma.sync with the heads as the M / N dimension.  This is the kernel the benchmark's decode step uses.
//   * sdpa_decode_partial_kernel  - everything else (fp32 inputs, head_dim 256, more than 16 heads per kv head):
//     16-byte streaming loads straight into registers and FFMA arithmetic.
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
#include "sm100_ptx.cuh"
#include "mma_sync.cuh"

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

template <typename T, int D, int GT, bool PAGED, bool HEAD_FAST>
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
  // Token-major caches ([S, Hkv, D] and the paged pool) interleave the heads of one token: there the grid's fast
  // axis is the head, so that CTAs running together read neighbouring 256-byte pieces of the same DRAM pages.
  const int by = HEAD_FAST ? blockIdx.x : blockIdx.y;
  const int kvh = p.head_begin / p.group + by / gchunks;
  const int gc = by % gchunks;
  const int h0 = kvh * p.group + gc * GT;
  const int nheads = min(GT, p.group - gc * GT);
  const int c = HEAD_FAST ? blockIdx.y : blockIdx.x;

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

  bool bad_block = false;
  constexpr int KPW = KPI * kUnroll;
  // Paged: one block-table read per key, issued an iteration ahead of the row loads that need it; the entry stays
  // raw in its register until then.
  int32_t blk_next[kUnroll];
  if constexpr (PAGED) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t key = start + warp * KPW + u * KPI + grp;
      blk_next[u] = key < end ? kv_block_read(p, b, key) : 0;
    }
  }
  for (int64_t kb = start + warp * KPW; kb < end; kb += kDecWarps * KPW) {
    uint4 kv[kUnroll], vv[kUnroll];
    bool ok[kUnroll];
    int64_t row[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t key = kb + u * KPI + grp;
      ok[u] = key < end;
      row[u] = key;
      if constexpr (PAGED) {
        row[u] = ok[u] ? kv_row_from(p, key, blk_next[u], bad_block) : -1;
        ok[u] = row[u] >= 0;
        const int64_t key_next = key + kDecWarps * KPW;
        blk_next[u] = key_next < end ? kv_block_read(p, b, key_next) : 0;
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

  report_bad_block(p, bad_block);
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

// ---- grouped-query decode on the warp-level tensor-core path ---------------------------------------------------
// With several query heads per KV head the FFMA kernel above is bound by its shuffle reductions (one per head and
// key), not by HBM.  Here the heads of one KV head are the M dimension of mma.sync.m16n8k16 (up to 16, zero padded):
// a warp takes 16 keys per step, S[16 heads x 16 keys] = Q K^T and O[16 heads x D] += P V run on the tensor
// cores, and K and V still stream from global memory exactly once with 16-byte loads straight into the fragment
// registers.  That works without shared memory or ldmatrix because a dot product does not care about the order of
// its terms: the d index is assigned to the MMA's k slots (for Q K^T) and to its n columns (for P V) in whatever
// order the coalesced 16-byte loads deliver it, Q is loaded once in the matching order, and the output columns are
// un-permuted when the accumulators are written out.  The one re-arrangement needed, pairing two keys of the same
// d in one 32-bit B register for P V, is a byte permute of two loaded registers.
//
// Fragment geometry (g = lane / 4, c = lane % 4), per 16-key step starting at key kb:
//   K: thread loads rows kb + g and kb + 8 + g, 16-byte chunks i*4 + c (i < D/32); chunk register pair h supplies
//      k-step 2i + h: slots (2c, 2c+1) <- d = (i*4+c)*8 + 4h + {0,1}, slots (2c+8, 2c+9) <- d = ... + 2 + {0,1}.
//   V: P V runs transposed, O^T[d x heads] += V^T[d x keys] P^T[keys x heads], so that the 8 (or 16) live heads
//      are the N dimension and no accumulator register is spent on padding.  The thread loads rows
//      kb + {2c, 2c+1, 2c+8, 2c+9}; for D = 128 chunks g and g + 8, for D = 64 chunk g.  M-tile m has its row r at
//      d = r*8 + m (D = 128) or d = (r % 8)*8 + 4*(r / 8) + m (D = 64); the S accumulators of Q K^T are, as they
//      stand, the B fragments of P^T.

// Feeding: each warp owns a ring of kRingStages shared-memory stages (16 keys of K and 16 of V each) filled with
// 16-byte cp.async copies - a warp-wide copy moves two whole rows, so requests are fully coalesced - and retired in
// order with cp.async.wait_group: up to kRingStages steps per warp are in flight whatever the register budget (a
// variant that prefetched into registers held one step in flight and reached 0.71 of the HBM peak where this one
// reaches 0.85), there is no flag to spin on, and rows past the chunk's end or outside the pool are zero-filled by
// the copy itself (source size 0).  Rows are stored un-padded with their 16-byte chunks XOR-swizzled
// (K: chunk ^ 4*(row & 1); V: chunk ^ 2*((row / 2) & 3)) so that the fragment reads of both products are
// bank-conflict free.  After the loop a warp reuses its own ring for the partials it hands to the merge.
// NH16: more than 8 query heads per KV head (rows 8..15 of the tile are live).
constexpr int kRingStages = 3;

template <int D>
struct RingCfg {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kKBytes = 16 * kRowBytes;
  static constexpr int kStageBytes = 2 * kKBytes;
  static constexpr int kWarpBytes = kRingStages * kStageBytes;
  static constexpr int kSmemBytes = kDecWarps * kWarpBytes;
  static_assert(kWarpBytes >= 16 * (D + 2) * 4, "a warp's partials must fit in its ring");
};


template <typename T, int D, bool NH16, bool PAGED, bool HEAD_FAST>
__global__ void __launch_bounds__(kDecWarps * 32, 2)
    sdpa_decode_gqa_ring_kernel(const SdpaParams p, const int chunk, const int nchunks, float* __restrict__ ws,
                                const int direct) {
  static_assert(sizeof(T) == 2 && (D == 64 || D == 128), "16-bit inputs, head_dim 64 or 128");
  using R = RingCfg<D>;
  constexpr int KI = D / 32, VX = D / 64, MT = D / 16;
  constexpr int HN = NH16 ? 2 : 1;
  constexpr int ROWS = NH16 ? 16 : 8;
  constexpr int NG = kDecWarps;
  constexpr int kStep = 16;

  extern __shared__ __align__(128) uint8_t ring_smem[];
  const uint32_t smem0 = ptx::smem_u32(ring_smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int b = blockIdx.z;
  const int kvh = p.head_begin / p.group + (HEAD_FAST ? (int)blockIdx.x : (int)blockIdx.y);
  const int h0 = kvh * p.group;
  const int nheads = p.group;
  const int cidx = HEAD_FAST ? blockIdx.y : blockIdx.x;

  const int64_t L = decode_len(p, b);
  const int64_t start = (int64_t)cidx * chunk;
  const int Hc = p.head_count;

  if (start >= L) {
    if (direct && cidx == 0) {
      for (int idx = tid; idx < nheads * D; idx += kDecWarps * 32) {
        const int hh = idx / D, d = idx - hh * D;
        store_out<T>(p.out, b * p.os[0] + (int64_t)(h0 + hh) * p.os[1] + d, 0.f, p.out_f32);
        if (p.lse && d == 0) p.lse[((int64_t)b * p.num_q_heads + h0 + hh) * p.seq_q] = -INFINITY;
      }
    }
    return;
  }
  const int64_t end = (start + chunk < L) ? start + chunk : L;

  const uint32_t my_ring = smem0 + warp * R::kWarpBytes;
  const T* kbase = static_cast<const T*>(p.k) + (PAGED ? 0 : b * p.ks[0]) + (int64_t)kvh * p.ks[1];
  const T* vbase = static_cast<const T*>(p.v) + (PAGED ? 0 : b * p.vs[0]) + (int64_t)kvh * p.vs[1];
  bool bad_block = false;

  constexpr int CH = D / 8;          // 16-byte chunks per row
  constexpr int RPL = 16 * CH / 32;  // rows each lane copies per step (of K, and of V)
  const int my_ch = lane % CH, my_r0 = lane / CH;
  // Raw block-table entry of key kb + lane % 16 (paged), read a step before the copies that need it are issued.
  auto entry_of = [&](int64_t kb) -> int32_t {
    if constexpr (PAGED) {
      const int64_t key = kb + (lane & 15);
      return key < end ? kv_block_read(p, b, key) : 0;
    } else {
      return 0;
    }
  };
  // Issues the copies of the step at kb into `stage` and commits them as one group.  Returns the step's row mask
  // (bit i: key kb + i is inside the chunk and its row inside the pool); the other rows are zero-filled.
  auto issue = [&](int stage, int64_t kb, int32_t entry) -> uint32_t {
    const int64_t key = kb + (lane & 15);
    int64_t row = -1;
    if (key < end) {
      if constexpr (PAGED) row = kv_row_from(p, key, entry, bad_block);
      else row = key;
    }
    const uint32_t base = my_ring + stage * R::kStageBytes;
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
      const int ri = my_r0 + (32 / CH) * r;
      const int64_t rr = __shfl_sync(0xffffffffu, row, ri);
      const bool valid = rr >= 0;
      const int64_t ro = valid ? rr : 0;
      cp_async16(base + ri * R::kRowBytes + ((my_ch ^ ((ri & 1) << 2)) << 4), kbase + ro * p.ks[2] + my_ch * 8, valid);
      cp_async16(base + R::kKBytes + ri * R::kRowBytes + ((my_ch ^ (((ri >> 1) & 3) << 1)) << 4),
                 vbase + ro * p.vs[2] + my_ch * 8, valid);
    }
    cp_async_commit();
    return __ballot_sync(0xffffffffu, row >= 0) & 0xffffu;
  };

  // Q in fragment order
  uint32_t qa[KI][4], qb[KI][4];
#pragma unroll
  for (int i = 0; i < KI; ++i) {
    uint4 u = make_uint4(0, 0, 0, 0), w = make_uint4(0, 0, 0, 0);
    if (g < nheads)
      u = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.q) + b * p.qs[0] + (int64_t)(h0 + g) * p.qs[1] + (i * 4 + c) * 8);
    if (NH16 && g + 8 < nheads)
      w = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.q) + b * p.qs[0] + (int64_t)(h0 + g + 8) * p.qs[1] + (i * 4 + c) * 8);
    qa[i][0] = u.x; qa[i][1] = u.y; qa[i][2] = u.z; qa[i][3] = u.w;
    qb[i][0] = w.x; qb[i][1] = w.y; qb[i][2] = w.z; qb[i][3] = w.w;
  }

  float acc[MT][HN][4];
#pragma unroll
  for (int j = 0; j < MT; ++j)
#pragma unroll
    for (int hn = 0; hn < HN; ++hn) acc[j][hn][0] = acc[j][hn][1] = acc[j][hn][2] = acc[j][hn][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // prologue: fill the ring (a group is committed per stage even when it is empty, so that wait_group counts steps)
  const int64_t kb0 = start + warp * kStep;
  constexpr int64_t kStride = NG * kStep;
  uint32_t row_mask[kRingStages];
#pragma unroll
  for (int s = 0; s < kRingStages; ++s) {
    const int64_t kbs = kb0 + s * kStride;
    row_mask[s] = 0;
    if (kbs < end) row_mask[s] = issue(s, kbs, entry_of(kbs));
    else cp_async_commit();
  }
  int32_t ent_next = entry_of(kb0 + kRingStages * kStride);

  int step = 0;
  for (int64_t kb = kb0; kb < end; kb += kStride, ++step) {
    const int stage = step % kRingStages;
    cp_async_wait<kRingStages - 1>();   // this step's group has landed (later steps may still be in flight)
    __syncwarp();                       // ... for every lane's copies
    const uint32_t base = my_ring + stage * R::kStageBytes;
    uint32_t rows_ok = 0;
#pragma unroll
    for (int s = 0; s < kRingStages; ++s)
      if (s == stage) rows_ok = row_mask[s];

    // ---- S = Q K^T ------------------------------------------------------------------------------------
    float sacc[2][4];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      sacc[t][0] = sacc[t][1] = sacc[t][2] = sacc[t][3] = 0.f;
#pragma unroll
      for (int i = 0; i < KI; ++i) {
        uint32_t kw[4];
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(kw[0]), "=r"(kw[1]), "=r"(kw[2]), "=r"(kw[3])
                     : "r"(base + (t * 8 + g) * R::kRowBytes + (((i * 4 + c) ^ ((g & 1) << 2)) << 4)));
#pragma unroll
        for (int h = 0; h < 2; ++h)
          mma16816<T>(sacc[t], qa[i][2 * h], qb[i][2 * h], qa[i][2 * h + 1], qb[i][2 * h + 1], kw[2 * h], kw[2 * h + 1]);
      }
    }
    // ---- V fragments to registers, then the stage is free for the copies two steps ahead ---------------
    uint32_t vw[4][VX][4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
#pragma unroll
      for (int x = 0; x < VX; ++x) {
        const int vr = 2 * c + (e & 1) + (e >> 1) * 8;   // (vr / 2) & 3 == c
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(vw[e][x][0]), "=r"(vw[e][x][1]), "=r"(vw[e][x][2]), "=r"(vw[e][x][3])
                     : "r"(base + R::kKBytes + vr * R::kRowBytes + (((g + 8 * x) ^ (c << 1)) << 4)));
      }
    __syncwarp();   // every lane has read the stage: refill it with the step kRingStages ahead
    {
      const int64_t kb_new = kb + kRingStages * kStride;
      const int32_t ent_new = ent_next;
      ent_next = entry_of(kb_new + kStride);
      uint32_t mask_new = 0;
      if (kb_new < end) mask_new = issue(stage, kb_new, ent_new);
      else cp_async_commit();
#pragma unroll
      for (int s = 0; s < kRingStages; ++s)
        if (s == stage) row_mask[s] = mask_new;
    }

    // ---- online softmax over the step's 16 keys ---------------------------------------------------------
    float pr[2][4];
    {
      float mt0 = -INFINITY, mt1 = -INFINITY;
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int idx = t * 8 + 2 * c + e;
          const int64_t key = kb + idx;
          const bool ok = (rows_ok >> idx) & 1u;
          float v0 = -INFINITY, v1 = -INFINITY;
          if (ok && g < nheads) v0 = finish_logit(p, sacc[t][e] * p.scale, b, h0 + g, 0, key, L);
          if (NH16 && ok && g + 8 < nheads) v1 = finish_logit(p, sacc[t][2 + e] * p.scale, b, h0 + g + 8, 0, key, L);
          sacc[t][e] = v0;
          sacc[t][2 + e] = v1;
          mt0 = fmaxf(mt0, v0);
          mt1 = fmaxf(mt1, v1);
        }
      mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, 1));
      mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, 2));
      if (NH16) {
        mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, 1));
        mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, 2));
      }
      const float n0 = fmaxf(m0, mt0), n1 = fmaxf(m1, mt1);
      const float c0 = (m0 == -INFINITY) ? 0.f : softmax_exp<T>(m0 - n0);
      const float c1 = (m1 == -INFINITY) ? 0.f : softmax_exp<T>(m1 - n1);
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          pr[t][e] = (sacc[t][e] == -INFINITY) ? 0.f : softmax_exp<T>(sacc[t][e] - n0);
          pr[t][2 + e] = (!NH16 || sacc[t][2 + e] == -INFINITY) ? 0.f : softmax_exp<T>(sacc[t][2 + e] - n1);
          s0 += pr[t][e];
          s1 += pr[t][2 + e];
        }
      l0 = l0 * c0 + s0;
      l1 = l1 * c1 + s1;
      m0 = n0;
      m1 = n1;
      const float ca = __shfl_sync(0xffffffffu, c0, 8 * c), cb = __shfl_sync(0xffffffffu, c0, 8 * c + 4);
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        acc[j][0][0] *= ca;
        acc[j][0][1] *= cb;
        acc[j][0][2] *= ca;
        acc[j][0][3] *= cb;
      }
      if (NH16) {
        const float cc = __shfl_sync(0xffffffffu, c1, 8 * c), cd = __shfl_sync(0xffffffffu, c1, 8 * c + 4);
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          acc[j][HN - 1][0] *= cc;
          acc[j][HN - 1][1] *= cd;
          acc[j][HN - 1][2] *= cc;
          acc[j][HN - 1][3] *= cd;
        }
      }
    }
    const uint32_t pb0 = pack_pair<T>(pr[0][0], pr[0][1]), pb1 = pack_pair<T>(pr[1][0], pr[1][1]);
    const uint32_t pc0 = pack_pair<T>(pr[0][2], pr[0][3]), pc1 = pack_pair<T>(pr[1][2], pr[1][3]);

    // ---- O^T += V^T P^T ------------------------------------------------------------------------------------
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const uint32_t sel = (m & 1) ? 0x7632u : 0x5410u;
      constexpr int xh = VX - 1;
      const int wl = m >> 1, wh = (D == 128) ? (m >> 1) : 2 + (m >> 1);
      const uint32_t a0 = __byte_perm(vw[0][0][wl], vw[1][0][wl], sel);
      const uint32_t a1 = __byte_perm(vw[0][xh][wh], vw[1][xh][wh], sel);
      const uint32_t a2 = __byte_perm(vw[2][0][wl], vw[3][0][wl], sel);
      const uint32_t a3 = __byte_perm(vw[2][xh][wh], vw[3][xh][wh], sel);
      mma16816<T>(acc[m][0], a0, a1, a2, a3, pb0, pb1);
      if (NH16) mma16816<T>(acc[m][HN - 1], a0, a1, a2, a3, pc0, pc1);
    }
  }

  report_bad_block(p, bad_block);
  cp_async_wait<0>();
  __syncwarp();
  // The warp's ring is free now: its partials go there.
  float* sm_acc = reinterpret_cast<float*>(ring_smem + warp * R::kWarpBytes);   // [ROWS][D], then m[ROWS], l[ROWS]
  float* sm_m = sm_acc + ROWS * D;
  float* sm_l = sm_m + ROWS;
  constexpr int kWarpFloats = R::kWarpBytes / 4;
  // ---- merge the warps of the CTA ---------------------------------------------------------------------------
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (c == 0) {
    sm_m[g] = m0;
    sm_l[g] = l0;
    if (NH16) {
      sm_m[g + 8] = m1;
      sm_l[g + 8] = l1;
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const int d_lo = g * 8 + m, d_hi = (D == 128) ? (g + 8) * 8 + m : g * 8 + 4 + m;
#pragma unroll
    for (int hn = 0; hn < HN; ++hn)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        sm_acc[(8 * hn + 2 * c + e) * D + d_lo] = acc[m][hn][e];
        sm_acc[(8 * hn + 2 * c + e) * D + d_hi] = acc[m][hn][2 + e];
      }
  }
  __syncthreads();

  const float* all = reinterpret_cast<const float*>(ring_smem);   // warp n's partials start at n * kWarpFloats
  for (int idx = tid; idx < nheads * D; idx += kDecWarps * 32) {
    const int hh = idx / D, d = idx - hh * D;
    float M = -INFINITY;
#pragma unroll
    for (int n = 0; n < NG; ++n) M = fmaxf(M, all[n * kWarpFloats + ROWS * D + hh]);
    float a = 0.f, lsum = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int n = 0; n < NG; ++n) {
        const float mn = all[n * kWarpFloats + ROWS * D + hh];
        const float wgt = (mn == -INFINITY) ? 0.f : softmax_exp<T>(mn - M);
        a = fmaf(wgt, all[n * kWarpFloats + hh * D + d], a);
        lsum = fmaf(wgt, all[n * kWarpFloats + ROWS * D + ROWS + hh], lsum);
      }
    }
    const int h = h0 + hh;
    if (direct) {
      store_out<T>(p.out, b * p.os[0] + (int64_t)h * p.os[1] + d, lsum > 0.f ? a / lsum : 0.f, p.out_f32);
      if (p.lse && d == 0)
        p.lse[((int64_t)b * p.num_q_heads + h) * p.seq_q] = lsum > 0.f ? M + logf(lsum) : -INFINITY;
    } else {
      const int64_t slot = ((int64_t)b * Hc + (h - p.head_begin)) * nchunks + cidx;
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
  const unsigned heads_y = (unsigned)((p.head_count / p.group) * gchunks);
  const bool head_fast = p.ks[1] < p.ks[2] && nchunks <= 65535;
  if (head_fast) {
    dim3 grid(heads_y, (unsigned)nchunks, (unsigned)p.batch);
    if (p.block_table) sdpa_decode_partial_kernel<T, D, GT, true, true><<<grid, kDecWarps * 32, 0, stream>>>(p, chunk, nchunks, ws, direct);
    else sdpa_decode_partial_kernel<T, D, GT, false, true><<<grid, kDecWarps * 32, 0, stream>>>(p, chunk, nchunks, ws, direct);
  } else {
    dim3 grid((unsigned)nchunks, heads_y, (unsigned)p.batch);
    if (p.block_table) sdpa_decode_partial_kernel<T, D, GT, true, false><<<grid, kDecWarps * 32, 0, stream>>>(p, chunk, nchunks, ws, direct);
    else sdpa_decode_partial_kernel<T, D, GT, false, false><<<grid, kDecWarps * 32, 0, stream>>>(p, chunk, nchunks, ws, direct);
  }
  return cudaGetLastError();
}

template <typename T, int D, bool NH16>
cudaError_t launch_gqa(const SdpaParams& p, int chunk, int nchunks, float* ws, int direct, cudaStream_t stream) {
  const unsigned kvheads = (unsigned)(p.head_count / p.group);
  const bool head_fast = p.ks[1] < p.ks[2] && nchunks <= 65535;
  const dim3 grid = head_fast ? dim3(kvheads, (unsigned)nchunks, (unsigned)p.batch)
                              : dim3((unsigned)nchunks, kvheads, (unsigned)p.batch);
  const bool paged = p.block_table != nullptr;
  constexpr int smem = RingCfg<D>::kSmemBytes;
#define AIDN_GQA_LAUNCH(PG, HF)                                                                                 \
  do {                                                                                                          \
    auto kern = sdpa_decode_gqa_ring_kernel<T, D, NH16, PG, HF>;                                                \
    cudaError_t ea = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);             \
    if (ea != cudaSuccess) return ea;                                                                           \
    kern<<<grid, kDecWarps * 32, smem, stream>>>(p, chunk, nchunks, ws, direct);                                \
  } while (0)
  if (paged && head_fast) AIDN_GQA_LAUNCH(true, true);
  else if (paged) AIDN_GQA_LAUNCH(true, false);
  else if (head_fast) AIDN_GQA_LAUNCH(false, true);
  else AIDN_GQA_LAUNCH(false, false);
#undef AIDN_GQA_LAUNCH
  return cudaGetLastError();
}

template <typename T, int D>
cudaError_t launch_partial_g(const SdpaParams& p, int chunk, int nchunks, float* ws, int direct, cudaStream_t stream) {
  if constexpr (sizeof(T) == 2 && (D == 64 || D == 128)) {
    // 16-bit inputs with up to 16 query heads per KV head (plain multi-head attention included: the padding rows
    // of the MMA tile cost nothing on an HBM-bound kernel): the tensor-core kernel with the cp.async ring
    if (p.group <= 8) return launch_gqa<T, D, false>(p, chunk, nchunks, ws, direct, stream);
    if (p.group > 8 && p.group <= 16) return launch_gqa<T, D, true>(p, chunk, nchunks, ws, direct, stream);
  }
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

// The array has one address per CUDA context, not per device ordinal: a process may hold the primary context and a
// context of its own making (the reference's backend creates one with cuCtxCreate) on the same GPU, and each has its
// own copy of the library's device image.  The address is therefore looked up once per context and remembered under
// the context's id (cuCtxGetId: unique for the life of the process, unlike the handle, which a later context may reuse).
constexpr int kMaxContexts = 64;
struct ScratchSlot {
  unsigned long long ctx_id;
  float* ptr;
};
ScratchSlot g_static_scratch[kMaxContexts] = {};
int g_static_scratch_used = 0;
std::mutex g_static_scratch_mutex;

typedef int (*CtxGetIdFn)(void*, unsigned long long*);   // CUresult cuCtxGetId(CUcontext, unsigned long long*)
CtxGetIdFn ctx_get_id_fn() {
  static CtxGetIdFn fn = nullptr;   // written under g_static_scratch_mutex
  if (!fn) {
    void* raw = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuCtxGetId", &raw, cudaEnableDefault, &qres) == cudaSuccess && raw &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<CtxGetIdFn>(raw);
  }
  return fn;
}

// In host code the array's name is only a stand-in; the device address has to be asked for with the context that
// will run the kernel current.
cudaError_t static_scratch_address(float** out) {
  // binds the runtime to the caller's current context (or to the primary one when the thread has none)
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  unsigned long long id = 0;
  CtxGetIdFn get = ctx_get_id_fn();
  const bool have_id = get && get(nullptr, &id) == 0;   // a null context means the current one
  if (have_id)
    for (int i = 0; i < g_static_scratch_used; ++i)
      if (g_static_scratch[i].ctx_id == id) {
        *out = g_static_scratch[i].ptr;
        return cudaSuccess;
      }
  float* ptr = nullptr;
  e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_decode_static_scratch);
  if (e != cudaSuccess) return e;
  // without a context id (or with the table full) the address is simply looked up again on every call
  if (have_id && g_static_scratch_used < kMaxContexts) g_static_scratch[g_static_scratch_used++] = {id, ptr};
  *out = ptr;
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
