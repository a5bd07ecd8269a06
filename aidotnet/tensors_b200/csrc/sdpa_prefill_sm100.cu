// FlashAttention-style prefill forward for sm_100a: TMA + mbarrier pipeline, tcgen05 UMMA with TMEM
// accumulators, warp-specialised roles, online softmax in registers.
//
// One CTA owns TWO 128-row query tiles that share one KV head, so every K/V tile fetched into shared
// memory feeds two score MMAs and two P.V MMAs.  The two tiles are two query heads of the same GQA group at
// the same rows (group size even) or two consecutive row tiles of one head.
//
//   warps 0-3   softmax of tile 0: thread t owns row t of the tile (TMEM lane == row), reads S from TMEM,
//   warps 4-7   softmax of tile 1  keeps the running max / sum, rescales O lazily, writes P (16-bit) back
//                                  into the S columns, and at the end normalises and stores O
//   warp  8     TMA producer: Q tiles once, then K0, V0, K1, V1, ... through a ring of shared-memory slots
//   warp  9     UMMA issuer (one lane): S_i = Q_i K^T (smem x smem), O_i += P_i V (TMEM x smem); owns TMEM
//
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D); P_i aliases the first 64 columns
// of S_i.  The issue order per KV tile j is  PV_0(j), QK_0(j+1), PV_1(j), QK_1(j+1): UMMAs execute in issue
// order, so QK_i(j+1) overwriting S_i cannot pass PV_i(j) reading P_i, and while one tile waits for its
// softmax the tensor core works on the other.
//
// Supersedes flash_attention_v2 / grouped_query_attention / scaled_dot_product_attention of the reference
// (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/Kernels/CudaAttentionKernels.cs:28-234, 527-646) and its
// sm_86-only mma.sync kernel (CUDA/Ptx/PtxOnlineFusedAttention128x64Kernel.cs), whose numerics it keeps:
// fp32 scores, exp as ex2.approx((s - max) * scale * log2e), row sum over un-rounded fp32 probabilities,
// P rounded to 16 bit for the second MMA, O rescale skipped while the max moves little (:711-802).
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace aidn {
namespace {

using namespace ptx;

constexpr int kBM = 128;           // rows per query tile
constexpr int kBN = 128;           // keys per KV tile
constexpr int kSoftmaxWarps = 8;   // 2 tiles x 4 warps
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kThreads = 384;          // 3 warpgroups: softmax 0, softmax 1, {producer, UMMA issuer, 2 idle}
constexpr int kSoftmaxRegs = 224;      // per-thread registers after setmaxnreg (8*32*224 + 4*32*56 == 384*168)
constexpr int kOtherRegs = 56;
constexpr int kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units: P stays below 2^8 between rescales

template <int HD>
struct Cfg {
  static constexpr int kTileBytes = kBN * HD * 2;         // one K or V tile == one Q tile
  static constexpr int kStages = HD == 128 ? 4 : 6;       // K/V ring slots
  static constexpr int kHalves = HD / 64;                 // 64-element (128-byte) column blocks per tile
  static constexpr int kHalfBytes = kBN * 128;            // 16 KiB
  static constexpr int kSmemTiles = (2 + kStages) * kTileBytes;
  static constexpr int kNumBars = 2 + 2 * kStages + 2 + 2 + 2;
  static constexpr int kSmemBytes = kSmemTiles + kNumBars * 8 + 16 /*tmem ptr + abort*/ + 1024 /*align slack*/;
  static constexpr int kOCol = 256;
};

struct PrefillParams {
  SdpaParams p;
  int32_t row_tiles;       // ceil(seq_q / 128)
  int32_t pair_heads;      // 1: the two tiles are heads (h, h+1) at one row tile; 0: row tiles (2u, 2u+1) of one head
  int32_t ranks;           // scheduling ranks along the row-tile axis (heavy first)
  int32_t items_per_rank;  // batch * work items per rank
  int32_t per_batch;       // work items per rank per batch entry
  float* debug;            // optional tap: scores of CTA 0 at j == 0, un-normalised O, l, m
  int32_t debug_mode;      // 1: value tap of CTA 0; 2: per-CTA timeline (16 x u64 per CTA)
};

struct TileInfo {
  int h;          // q head
  int t;          // row tile index
  int n;          // KV tiles to process (0 = none visible)
  bool valid;     // tile exists
};

template <typename T, int HD>
__global__ void __launch_bounds__(kThreads, 1)
    sdpa_prefill_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                              const __grid_constant__ CUtensorMap tm_v, const PrefillParams pp) {
  using C = Cfg<HD>;
  constexpr bool kBf16 = !std::is_same_v<T, __half>;
  const SdpaParams& p = pp.p;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base;                           // 2 tiles
  const uint32_t kv_smem = smem_base + 2 * C::kTileBytes;      // kStages tiles
  const uint32_t bars = smem_base + C::kSmemTiles;
  const uint32_t bar_q_full = bars;                            // [2]
  const uint32_t bar_kv_full = bars + 16;                      // [kStages]
  const uint32_t bar_kv_empty = bar_kv_full + 8 * C::kStages;  // [kStages]
  const uint32_t bar_s_full = bar_kv_empty + 8 * C::kStages;   // [2]
  const uint32_t bar_p_full = bar_s_full + 16;                 // [2]
  const uint32_t bar_o_full = bar_p_full + 16;                 // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_gen + C::kSmemTiles + C::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Timeline tap (debug_mode 2): slot k of this CTA's 16-entry record receives a globaltimer stamp.
  unsigned long long* trace = pp.debug_mode == 2 ? reinterpret_cast<unsigned long long*>(pp.debug) + (size_t)blockIdx.x * 16 : nullptr;
  auto stamp = [&](int slot) { if (trace) trace[slot] = globaltimer_ns(); };
  if (threadIdx.x == 0) stamp(0);

  // ---- work item ---------------------------------------------------------------------------------
  const int item = blockIdx.x;
  const int rank = item / pp.items_per_rank;
  const int rem = item - rank * pp.items_per_rank;
  const int b = rem / pp.per_batch;
  const int w = rem - b * pp.per_batch;
  TileInfo tile[2];
  if (pp.pair_heads) {
    const int t = pp.row_tiles - 1 - rank;
    tile[0].h = p.head_begin + 2 * w;
    tile[1].h = tile[0].h + 1;
    tile[0].t = tile[1].t = t;
    tile[0].valid = tile[1].valid = true;
  } else {
    const int u = pp.ranks - 1 - rank;
    tile[0].h = tile[1].h = p.head_begin + w;
    tile[0].t = 2 * u;
    tile[1].t = 2 * u + 1;
    tile[0].valid = true;
    tile[1].valid = tile[1].t < pp.row_tiles;
  }
  const int kvh = tile[0].h / p.group;
  const int64_t kv_limit = kv_limit_of(p, b);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int64_t kend = 0;
    if (tile[i].valid) {
      kend = kv_limit;
      if (p.causal) {
        int64_t last_row = (int64_t)tile[i].t * kBM + kBM - 1;
        if (last_row > p.seq_q - 1) last_row = p.seq_q - 1;
        const int64_t c = last_row + p.causal_offset + 1;
        if (c < kend) kend = c;
      }
      if (kend < 0) kend = 0;
    }
    tile[i].n = (int)((kend + kBN - 1) / kBN);
  }
  const int n_max = tile[0].n > tile[1].n ? tile[0].n : tile[1].n;

  // ---- setup ---------------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_full + 8, 1);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_kv_full + 8 * s, 1);
      mbar_init(bar_kv_empty + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_p_full + 8 * i, 128);
      mbar_init(bar_o_full + 8 * i, 1);
    }
    fence_mbar_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_ptr_smem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  if (threadIdx.x == 0) {
    stamp(1);
    if (trace) {
      unsigned smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      trace[15] = ((unsigned long long)smid << 32) | (unsigned)n_max;
    }
  }

  const float sl2 = p.scale * kLog2e;

  if (warp < kSoftmaxWarps) {
    // =================================== softmax / epilogue ===================================
    setmaxnreg_inc<kSoftmaxRegs>();
    const int i = warp >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const TileInfo ti = tile[i];
    const int64_t qrow = (int64_t)ti.t * kBM + row_in_tile;
    const bool row_valid = ti.valid && qrow < p.seq_q;
    const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + lane_bits + (uint32_t)(i * kBN);
    const uint32_t t_o = tmem_base + lane_bits + (uint32_t)(C::kOCol + i * HD);
    // last visible key of this row
    int64_t kmax_row = kv_limit - 1;
    if (p.causal && qrow + p.causal_offset < kmax_row) kmax_row = qrow + p.causal_offset;

    float m = -INFINITY, l = 0.f;
    bool alive = true;

    for (int j = 0; j < ti.n && alive; ++j) {
      bool ok = mbar_wait(bar_s_full + 8 * i, (uint32_t)(j & 1), abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { alive = false; break; }
      tc_fence_after();
      if (j == 0 && row_in_tile == 0) stamp(2 + 4 * i);

      uint32_t sr[128];
      tmem_ld32(t_s + 0, sr + 0);
      tmem_ld32(t_s + 32, sr + 32);
      tmem_ld32(t_s + 64, sr + 64);
      tmem_ld32(t_s + 96, sr + 96);
      tc_wait_ld();
      float* s = reinterpret_cast<float*>(sr);

      if (pp.debug_mode == 1 && blockIdx.x == 0 && j == 0) {
        float* dbg = pp.debug + (size_t)(i * kBM + row_in_tile) * kBN;
#pragma unroll
        for (int c = 0; c < kBN; ++c) dbg[c] = s[c];
      }

      const int64_t col0 = (int64_t)j * kBN;
      if (col0 + kBN - 1 > kmax_row) {
        const int64_t lim = kmax_row - col0;  // columns > lim are masked (lim may be negative)
#pragma unroll
        for (int c = 0; c < kBN; ++c)
          if (c > lim) s[c] = -INFINITY;
      }

      float mx0 = s[0], mx1 = s[1], mx2 = s[2], mx3 = s[3];
#pragma unroll
      for (int c = 4; c < kBN; c += 4) {
        mx0 = fmaxf(mx0, s[c]);
        mx1 = fmaxf(mx1, s[c + 1]);
        mx2 = fmaxf(mx2, s[c + 2]);
        mx3 = fmaxf(mx3, s[c + 3]);
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_new = fmaxf(m, mx);

      if (j == 0) {
        m = m_new;
      } else {
        const bool need = (m_new - m) * sl2 > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          float f;
          if (m_new == -INFINITY) f = 1.f;
          else if (m == -INFINITY) f = 0.f;
          else f = ex2_approx((m - m_new) * sl2);
          l *= f;
          m = m_new;
#pragma unroll
          for (int c0 = 0; c0 < HD; c0 += 32) {
            uint32_t orr[32];
            tmem_ld32(t_o + c0, orr);
            tc_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; ++c) orr[c] = __float_as_uint(__uint_as_float(orr[c]) * f);
            tmem_st32(t_o + c0, orr);
          }
          tc_wait_st();
        }
      }

      const float neg_ms = (m == -INFINITY) ? 0.f : -m * sl2;
      float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
#pragma unroll
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const float p0 = ex2_approx(fmaf(s[c0 + c], sl2, neg_ms));
          const float p1 = ex2_approx(fmaf(s[c0 + c + 1], sl2, neg_ms));
          const float p2 = ex2_approx(fmaf(s[c0 + c + 2], sl2, neg_ms));
          const float p3 = ex2_approx(fmaf(s[c0 + c + 3], sl2, neg_ms));
          ls0 += p0;
          ls1 += p1;
          ls2 += p2;
          ls3 += p3;
          pk[c >> 1] = pack2<kBf16>(p0, p1);
          pk[(c >> 1) + 1] = pack2<kBf16>(p2, p3);
        }
        tmem_st16(t_s + (c0 >> 1), pk);
      }
      l += (ls0 + ls1) + (ls2 + ls3);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p_full + 8 * i);
    }

    if (row_in_tile == 0) stamp(3 + 4 * i);
    // ---- epilogue: O / l -> global -----------------------------------------------------------------
    if (alive && ti.valid) {
      bool have_o = ti.n > 0;
      if (have_o) {
        bool ok = mbar_wait(bar_o_full + 8 * i, 0u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; have_o = false; }
      }
      if (alive) {
        tc_fence_after();
        if (row_in_tile == 0) stamp(4 + 4 * i);
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int64_t obase = b * p.os[0] + (int64_t)ti.h * p.os[1] + qrow * p.os[2];
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t orr[32];
          if (have_o) {
            tmem_ld32(t_o + c0, orr);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) orr[c] = 0u;
          }
          if (pp.debug_mode == 1 && blockIdx.x == 0) {
            float* dbg = pp.debug + 2 * kBM * kBN + (size_t)(i * kBM + row_in_tile) * HD + c0;
#pragma unroll
            for (int c = 0; c < 32; ++c) dbg[c] = __uint_as_float(orr[c]);
          }
          if (row_valid) {
            if (p.out_f32) {
              float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + obase + c0);
#pragma unroll
              for (int c = 0; c < 32; c += 4)
                dst[c >> 2] = make_float4(__uint_as_float(orr[c]) * inv, __uint_as_float(orr[c + 1]) * inv,
                                          __uint_as_float(orr[c + 2]) * inv, __uint_as_float(orr[c + 3]) * inv);
            } else {
              uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(p.out) + obase + c0);
#pragma unroll
              for (int c = 0; c < 32; c += 8) {
                uint4 u;
                u.x = pack2<kBf16>(__uint_as_float(orr[c]) * inv, __uint_as_float(orr[c + 1]) * inv);
                u.y = pack2<kBf16>(__uint_as_float(orr[c + 2]) * inv, __uint_as_float(orr[c + 3]) * inv);
                u.z = pack2<kBf16>(__uint_as_float(orr[c + 4]) * inv, __uint_as_float(orr[c + 5]) * inv);
                u.w = pack2<kBf16>(__uint_as_float(orr[c + 6]) * inv, __uint_as_float(orr[c + 7]) * inv);
                dst[c >> 3] = u;
              }
            }
          }
        }
        if (row_valid && p.lse)
          p.lse[((int64_t)b * p.num_q_heads + ti.h) * p.seq_q + qrow] =
              (l > 0.f) ? m * p.scale + logf(l) : -INFINITY;
        if (pp.debug_mode == 1 && blockIdx.x == 0) {
          float* dbg = pp.debug + 2 * kBM * kBN + 2 * kBM * HD + (size_t)(i * kBM + row_in_tile) * 2;
          dbg[0] = l;
          dbg[1] = m;
        }
        if (row_in_tile == 0) stamp(5 + 4 * i);
      }
    }
  } else {
    setmaxnreg_dec<kOtherRegs>();
  }
  if (warp == kProducerWarp) {
    // ========================================= TMA producer =========================================
    if (lane == 0 && n_max > 0) {
      bool alive = true;
      auto load_tile = [&](const CUtensorMap* tm, uint32_t dst, uint32_t bar, int row, int head) {
        mbar_expect_tx(bar, (uint32_t)C::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < C::kHalves; ++hf) tma_load_4d(dst + hf * C::kHalfBytes, tm, bar, hf * 64, row, head, b);
      };
      auto load_kv = [&](const CUtensorMap* tm, int t_idx, int key_tile) {
        const int slot = t_idx % C::kStages;
        const uint32_t phase = (uint32_t)((t_idx / C::kStages) & 1);
        if (!mbar_wait(bar_kv_empty + 8 * slot, phase ^ 1u, abort_flag)) { alive = false; return; }
        load_tile(tm, kv_smem + slot * C::kTileBytes, bar_kv_full + 8 * slot, key_tile * kBN, kvh);
      };
      if (tile[0].n > 0) load_tile(&tm_q, q_smem, bar_q_full, tile[0].t * kBM, tile[0].h);
      load_kv(&tm_k, 0, 0);
      if (tile[1].n > 0) load_tile(&tm_q, q_smem + C::kTileBytes, bar_q_full + 8, tile[1].t * kBM, tile[1].h);
      for (int j = 0; j < n_max && alive; ++j) {
        load_kv(&tm_v, 2 * j + 1, j);
        if (alive && j + 1 < n_max) load_kv(&tm_k, 2 * j + 2, j + 1);
      }
    }
  } else if (warp == kMmaWarp) {
    // ========================================== UMMA issuer ==========================================
    if (lane == 0 && n_max > 0) {
      constexpr uint32_t idesc_qk = make_idesc(kBM, kBN, kBf16, false);
      constexpr uint32_t idesc_pv = make_idesc(kBM, HD, kBf16, true);
      bool alive = true;
      auto kv_wait = [&](int t_idx) {
        const int slot = t_idx % C::kStages;
        if (!mbar_wait(bar_kv_full + 8 * slot, (uint32_t)((t_idx / C::kStages) & 1), abort_flag)) alive = false;
        return kv_smem + slot * C::kTileBytes;
      };
      auto kv_release = [&](int t_idx) { tc_commit(bar_kv_empty + 8 * (t_idx % C::kStages)); };
      auto issue_qk = [&](int i, uint32_t kaddr) {
        const uint32_t qaddr = q_smem + i * C::kTileBytes;
        const uint32_t d = tmem_base + (uint32_t)(i * kBN);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (uint32_t)((kk >> 2) * C::kHalfBytes + (kk & 3) * 32);
          mma_ss(d, make_smem_desc(qaddr + off, 16, 1024), make_smem_desc(kaddr + off, 16, 1024), idesc_qk,
                 kk > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int i, uint32_t vaddr, bool accumulate) {
        const uint32_t d = tmem_base + (uint32_t)(C::kOCol + i * HD);
        const uint32_t a = tmem_base + (uint32_t)(i * kBN);
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk)
          mma_ts(d, a + (uint32_t)(kk * 8), make_smem_desc(vaddr + (uint32_t)(kk * 2048), C::kHalfBytes, 1024),
                 idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
      };

      // S_i(0) = Q_i K_0^T
      uint32_t kaddr = kv_wait(0);
      for (int i = 0; i < 2 && alive; ++i) {
        if (tile[i].n == 0) continue;
        if (!mbar_wait(bar_q_full + 8 * i, 0u, abort_flag)) { alive = false; break; }
        tc_fence_after();
        issue_qk(i, kaddr);
        tc_commit(bar_s_full + 8 * i);
      }
      if (alive) kv_release(0);

      for (int j = 0; j < n_max && alive; ++j) {
        const uint32_t vaddr = kv_wait(2 * j + 1);
        uint32_t knext = 0;
        const bool has_next = j + 1 < n_max;
        if (alive && has_next) knext = kv_wait(2 * j + 2);
        for (int i = 0; i < 2 && alive; ++i) {
          if (j >= tile[i].n) continue;
          if (!mbar_wait(bar_p_full + 8 * i, (uint32_t)(j & 1), abort_flag)) { alive = false; break; }
          tc_fence_after();
          issue_pv(i, vaddr, j > 0);
          if (j + 1 < tile[i].n) {
            issue_qk(i, knext);
            tc_commit(bar_s_full + 8 * i);
          } else {
            tc_commit(bar_o_full + 8 * i);
          }
        }
        if (alive) {
          kv_release(2 * j + 1);
          if (has_next) kv_release(2 * j + 2);
        }
      }
    }
  }

  // ---- teardown -------------------------------------------------------------------------------------
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // Give loads that were already issued a bounded chance to land before shared memory is released.
    if (warp == kProducerWarp && lane == 0) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) {
      }
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusTimeout);
    __syncthreads();
  }
  if (threadIdx.x == 0) stamp(10);
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
    if (lane == 0) stamp(11);
  }
}

// ---- host side -----------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode = nullptr;

cudaError_t resolve_encode() {
  if (g_encode) return cudaSuccess;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return e;
  if (!fn || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return cudaSuccess;
}

// [B, H, S, D] 16-bit tensor viewed as a 4-D TMA tensor (D, S, H, B); box = 64 x 128 x 1 x 1, 128-byte swizzle.
bool encode_bhsd(CUtensorMap* tm, bool bf16, const void* base, int64_t D, int64_t S, int64_t H, int64_t B,
                 const int64_t* stride /*B,H,S in elements*/) {
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  // A dimension of extent 1 never advances; give it a harmless valid stride.
  const int64_t s_s = stride[2];
  const int64_t s_h = H > 1 ? stride[1] : s_s * S;
  const int64_t s_b = B > 1 ? stride[0] : (s_h * H > s_s * S ? s_h * H : s_s * S);
  cuuint64_t strides[3] = {(cuuint64_t)(s_s * 2), (cuuint64_t)(s_h * 2), (cuuint64_t)(s_b * 2)};
  cuuint32_t box[4] = {64u, (cuuint32_t)kBN, 1u, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  const CUresult r = g_encode(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool tma_ok(const void* base, const int64_t* stride, int64_t S, int64_t H, int64_t B) {
  if ((uintptr_t)base % 16 != 0) return false;
  if (stride[2] % 8 != 0 || stride[2] <= 0) return false;
  if (H > 1 && (stride[1] % 8 != 0 || stride[1] <= 0)) return false;
  if (B > 1 && (stride[0] % 8 != 0 || stride[0] <= 0)) return false;
  (void)S;
  return true;
}

template <typename T, int HD>
cudaError_t launch_t(const SdpaParams& p, cudaStream_t stream, float* debug, int debug_mode, const char** why) {
  using C = Cfg<HD>;
  cudaError_t e = resolve_encode();
  if (e != cudaSuccess) { *why = "cuTensorMapEncodeTiled is not available from the driver"; return e; }
  constexpr bool bf16 = !std::is_same_v<T, __half>;
  CUtensorMap tq, tk, tv;
  if (!encode_bhsd(&tq, bf16, p.q, HD, p.seq_q, p.num_q_heads, p.batch, p.qs) ||
      !encode_bhsd(&tk, bf16, p.k, HD, p.seq_kv, p.num_kv_heads, p.batch, p.ks) ||
      !encode_bhsd(&tv, bf16, p.v, HD, p.seq_kv, p.num_kv_heads, p.batch, p.vs)) {
    *why = "cuTensorMapEncodeTiled rejected a tensor (address or stride alignment)";
    return cudaErrorInvalidValue;
  }
  PrefillParams pp;
  pp.p = p;
  pp.debug = debug;
  pp.debug_mode = debug ? debug_mode : 0;
  pp.row_tiles = (int)((p.seq_q + kBM - 1) / kBM);
  pp.pair_heads = (p.group % 2 == 0) ? 1 : 0;
  if (pp.pair_heads) {
    pp.ranks = pp.row_tiles;
    pp.per_batch = p.head_count / 2;
  } else {
    pp.ranks = (pp.row_tiles + 1) / 2;
    pp.per_batch = p.head_count;
  }
  pp.items_per_rank = p.batch * pp.per_batch;
  const int64_t total = (int64_t)pp.ranks * pp.items_per_rank;
  if (total <= 0 || total > 0x7fffffff) { *why = "grid size out of range"; return cudaErrorInvalidValue; }
  auto kern = sdpa_prefill_sm100_kernel<T, HD>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) { *why = "cannot raise the dynamic shared memory limit"; return e; }
  kern<<<(unsigned)total, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, pp);
  return cudaGetLastError();
}

}  // namespace

bool prefill_sm100_supported(const SdpaParams& p, int dtype, const char** why) {
  if (dtype != AIDN_BF16 && dtype != AIDN_F16) { *why = "tcgen05 prefill takes fp16 or bf16 inputs"; return false; }
  if (p.head_dim != 64 && p.head_dim != 128) { *why = "tcgen05 prefill takes head_dim 64 or 128"; return false; }
  if (p.mask_kind != AIDN_MASK_NONE) { *why = "tcgen05 prefill takes no explicit mask (causal and kv_len only)"; return false; }
  if (p.softcap > 0.f) { *why = "tcgen05 prefill has no softcap"; return false; }
  if (!tma_ok(p.q, p.qs, p.seq_q, p.num_q_heads, p.batch) || !tma_ok(p.k, p.ks, p.seq_kv, p.num_kv_heads, p.batch) ||
      !tma_ok(p.v, p.vs, p.seq_kv, p.num_kv_heads, p.batch)) {
    *why = "Q/K/V base must be 16-byte aligned and strides multiples of 8 elements for TMA";
    return false;
  }
  const int out_elem = p.out_f32 ? 4 : 2;
  if ((uintptr_t)p.out % 16 != 0 || (p.os[2] * out_elem) % 16 != 0 || (p.os[1] * out_elem) % 16 != 0 ||
      (p.os[0] * out_elem) % 16 != 0) {
    *why = "output base and strides must be 16-byte aligned";
    return false;
  }
  if (p.seq_q > 0x7fffff00ll || p.seq_kv > 0x7fffff00ll) { *why = "sequence too long"; return false; }
  return true;
}

cudaError_t launch_prefill_sm100(const SdpaParams& p, int dtype, cudaStream_t stream, float* debug, int debug_mode,
                                 const char** why) {
  if (dtype == AIDN_BF16) {
    if (p.head_dim == 128) return launch_t<__nv_bfloat16, 128>(p, stream, debug, debug_mode, why);
    return launch_t<__nv_bfloat16, 64>(p, stream, debug, debug_mode, why);
  }
  if (p.head_dim == 128) return launch_t<__half, 128>(p, stream, debug, debug_mode, why);
  return launch_t<__half, 64>(p, stream, debug, debug_mode, why);
}

}  // namespace aidn
