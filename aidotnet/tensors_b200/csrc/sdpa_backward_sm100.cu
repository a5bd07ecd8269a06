// Attention backward on the sm_100a tensor cores: dQ and dK / dV as two launches of one warp-specialised kernel
// (TMA + mbarrier ring, tcgen05 UMMA with TMEM accumulators), recomputing the probabilities from the forward's
// log-sum-exp.  Deterministic: every gradient tile is accumulated by one CTA in a fixed order, no atomics.
//
// A work item is one 128-row tile that stays in shared memory ("stationary") while the 128-row tiles of the other
// sequence stream past it; persistent CTAs walk the items, heaviest first, and the loads and first score products of
// the next item run under the epilogue of the current one:
//   KEYS = true  (dK, dV): rows are keys.  X = K tile, Y = V tile; per step U = Q tile, W = dO tile of one query head
//                of the KV group.   S^T = X U^T,  dP^T = Y W^T,  dV += P^T W,  dK += dS^T U
//   KEYS = false (dQ):     rows are queries.  X = Q tile, Y = dO tile; per step U = K tile, W = V tile.
//                S = X U^T,  dP = Y W^T,  dQ += dS U
// with P = exp(scale * S - lse) under the causal / length masks and dS = P * (dP - delta).  The two score products
// take both operands from shared memory (K-major); the gradient products take P^T / dS (rounded to 16 bits, written
// back over the fp32 scores they came from) from TMEM as the A operand and read the streamed tile a second time as
// the MN-major B operand - one shared-memory image, two descriptors.
//
//   warp 0      TMA producer          warp 1      UMMA issuer (one elected lane); owns TMEM
//   warps 2-5   half 0, warps 6-9 half 1: one row per thread: TMEM -> registers, P and dS, -> TMEM; at the end the
//               two groups scale and store one accumulator (or one half of dQ) each
//
// A streamed tile is processed as two halves of 64 rows, each with its own S / dP columns in TMEM and its own group of
// four row warps, so that the tensor core computes the scores of one half (and the gradient products of the previous
// one) while the other half is turned into P and dS, and every scheduler has two row warps to switch between.  TMEM columns: half h: S [128h, 128h+64)  dP [128h+64, 128h+128);  dK or dQ [256,256+D);
// dV [256+D,256+2D).  Issue order  S(0) S(1) G(0) S(2) G(1) S(3) ...: UMMAs execute in issue order, so the scores of
// half i+2, which overwrite P / dS of half i, cannot pass the gradient products G(i) that read them.
//
// Serves 16-bit inputs, head_dim 64 / 128, contiguous K / V, causal and length masks, and (MASKED instantiation) an
// additive bias or a keep-mask read by the row threads; everything else stays on the kernels of sdpa_backward.cu.  Supersedes flash_attention_backward_deterministic_{dq,dkv} of the reference
// (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/Kernels/CudaAttentionKernels.cs:251-390), whose formulas it keeps.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tensor_map.hpp"

namespace aidn {
namespace {

using namespace ptx;

constexpr int kT = 128;          // rows of every tile
constexpr int kThreads = 320;     // producer, issuer, 2 x 4 row warps
constexpr int kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;

template <int HD>
struct BCfg {
  static constexpr int kTileBytes = kT * HD * 2;
  static constexpr int kHalfBytes = kT * 128;          // one 64-column block of a tile
  static constexpr int kHalves = HD / 64;
  static constexpr int kRing = HD == 128 ? 2 : 4;      // streamed (U, W) pairs in flight
  static constexpr int kRingOff = 2 * kTileBytes;
  static constexpr int kVecOff = kRingOff + kRing * 2 * kTileBytes;   // per-warp lse / delta rows: 8 warps x 2 x 2 x 64 floats
  static constexpr int kVecBytes = 8 * 2 * 2 * 64 * 4;
  static constexpr int kBarOff = kVecOff + kVecBytes;
  static constexpr int kNumBars = 8 + 2 * kRing;       // xy_full acc_full s_full[2] p_full[2] xy_empty acc_empty ring_full[R] ring_empty[R]
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kSmemBytes = kMiscOff + 16 + 1024;
  static constexpr int kAcc0 = 256;
  static constexpr int kAcc1 = 256 + HD;
};

struct BwdSm100Params {
  SdpaParams p;
  const float* delta;   // [B, Hc, Sq]
  float* dq;
  float* dk;
  float* dv;
  int32_t q_tiles, k_tiles;
  int32_t do_head_off;  // head coordinate of the dO tensor map = h - do_head_off
  int32_t total_items;
  int32_t withhold_loads;   // test hook: the producer issues no loads, so that the bounded waits run out
  uint64_t wait_budget_ns;
};

struct Work {
  int b, h, kvh;        // KEYS: h unused (steps walk the group's heads)
  int tile;             // stationary tile index
  int first, count;     // streamed tiles [first, first + count) per query head
  int steps;            // total steps (KEYS: group * count)
};

template <bool KEYS>
__device__ __forceinline__ Work decode_work(const BwdSm100Params& bp, int idx) {
  const SdpaParams& p = bp.p;
  Work w;
  if constexpr (KEYS) {
    const int hkv = p.head_count / p.group;
    const int per = hkv * p.batch;
    w.tile = idx / per;                      // key tile 0 (seen by every query under a causal mask) first
    const int rest = idx - w.tile * per;
    w.b = rest / hkv;
    w.kvh = p.head_begin / p.group + (rest - w.b * hkv);
    w.h = w.kvh * p.group;
    const int64_t k0 = (int64_t)w.tile * kT;
    int64_t first = 0;
    if (p.causal) {
      const int64_t qmin = k0 - p.causal_offset;   // first query that sees key k0
      first = qmin > 0 ? qmin / kT : 0;
    }
    int64_t count = (int64_t)bp.q_tiles - first;
    if (count < 0 || k0 >= kv_limit_of(p, w.b)) count = 0;
    w.first = (int)first;
    w.count = (int)count;
    w.steps = w.count * p.group;
  } else {
    const int per = p.head_count * p.batch;
    w.tile = bp.q_tiles - 1 - idx / per;     // the last query tile (most keys under a causal mask) first
    const int rest = idx % per;
    w.b = rest / p.head_count;
    w.h = p.head_begin + (rest - w.b * p.head_count);
    w.kvh = w.h / p.group;
    int64_t kmax = kv_limit_of(p, w.b);      // keys [0, kmax) can be visible
    if (p.causal) {
      const int64_t last_q = (int64_t)w.tile * kT + kT - 1;
      const int64_t lim = (last_q < p.seq_q ? last_q : p.seq_q - 1) + p.causal_offset + 1;
      if (lim < kmax) kmax = lim;
    }
    if (kmax < 0) kmax = 0;
    w.first = 0;
    w.count = (int)((kmax + kT - 1) / kT);
    w.steps = w.count;
  }
  return w;
}

// step j streams tile (first + j % count) of query head h + j / count (KEYS) or key tile j of the KV head
template <bool KEYS>
__device__ __forceinline__ int step_head(const Work& w, int j) { return KEYS ? w.h + j / w.count : w.kvh; }
template <bool KEYS>
__device__ __forceinline__ int step_tile(const Work& w, int j) { return KEYS ? w.first + j % w.count : j; }

template <typename T, int HD, bool KEYS, bool MASKED>
__global__ void __launch_bounds__(kThreads, 1)
    sdpa_backward_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                               const BwdSm100Params bp) {
  using C = BCfg<HD>;
  constexpr bool kBf16 = !std::is_same_v<T, __half>;
  const SdpaParams& p = bp.p;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t x_smem = smem_base, y_smem = smem_base + C::kTileBytes;
  const uint32_t ring_smem = smem_base + C::kRingOff;
  float* vec_smem = reinterpret_cast<float*>(smem_gen + C::kVecOff);
  const uint32_t bars = smem_base + C::kBarOff;
  const uint32_t bar_xy_full = bars, bar_acc_full = bars + 8, bar_s_full = bars + 16, bar_p_full = bars + 32;   // [2] each
  const uint32_t bar_xy_empty = bars + 48, bar_acc_empty = bars + 56;
  const uint32_t bar_ring_full = bars + 64, bar_ring_empty = bar_ring_full + 8 * C::kRing;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_gen + C::kMiscOff + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + C::kMiscOff + 12);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t wait_ns = bp.wait_budget_ns;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_xy_full, 1);
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_xy_empty, 1);
    mbar_init(bar_acc_empty, 8);   // one arrival per row warp
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_p_full + 8 * i, 128);
    }
    for (int s = 0; s < C::kRing; ++s) {
      mbar_init(bar_ring_full + 8 * s, 1);
      mbar_init(bar_ring_empty + 8 * s, 1);
    }
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_do);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // Persistent CTAs: CTA k takes items k, 2G-1-k, 2G+k, ... (G = grid size; the item list is ordered heaviest first, and
  // the snake keeps the sum per CTA even).  Counters that persist across items give every barrier its phase:
  // `live` = items with at least one step so far, `g` = steps so far.
  const int G = (int)gridDim.x;
  auto item_of = [&](int wave) {
    const int k = (wave & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x;
    return wave * G + k;
  };
  const int waves = (bp.total_items + G - 1) / G;

  if (warp == 0) {
    // ============================================ TMA producer ============================================
    const bool leader = elect_one();
    uint32_t g = 0, live = 0;
    bool alive = true;
    for (int wave = 0; wave < waves && alive; ++wave) {
      const int item = item_of(wave);
      if (item >= bp.total_items) continue;
      const Work w = decode_work<KEYS>(bp, item);
      if (w.steps == 0) continue;
      auto load_tile = [&](const CUtensorMap* tm, uint32_t dst, uint32_t bar, int row, int head) {
#pragma unroll
        for (int hf = 0; hf < C::kHalves; ++hf) tma_load_4d(dst + hf * C::kHalfBytes, tm, bar, hf * 64, row, head, w.b);
      };
      auto load_step = [&](int j) {
        const uint32_t gs = g + (uint32_t)j;
        const int s = (int)(gs % C::kRing);
        if (!mbar_wait(bar_ring_empty + 8 * s, ((gs / C::kRing) & 1u) ^ 1u, abort_flag, wait_ns)) { alive = false; return; }
        if (leader && !bp.withhold_loads) {
          const uint32_t bar = bar_ring_full + 8 * s;
          const uint32_t u_dst = ring_smem + s * 2 * C::kTileBytes, w_dst = u_dst + C::kTileBytes;
          const int head = step_head<KEYS>(w, j), row = step_tile<KEYS>(w, j) * kT;
          mbar_expect_tx(bar, 2u * C::kTileBytes);
          if (KEYS) {
            load_tile(&tm_q, u_dst, bar, row, head);
            load_tile(&tm_do, w_dst, bar, row, head - bp.do_head_off);
          } else {
            load_tile(&tm_k, u_dst, bar, row, head);
            load_tile(&tm_v, w_dst, bar, row, head);
          }
        }
      };
      // the first streamed tiles can land while the previous item still holds the stationary pair
      int j = 0;
      for (; j < C::kRing && j < w.steps && alive; ++j) load_step(j);
      if (alive && !mbar_wait(bar_xy_empty, (live & 1u) ^ 1u, abort_flag, wait_ns)) alive = false;
      if (alive && leader) {
        mbar_expect_tx(bar_xy_full, 2u * C::kTileBytes);
        if (KEYS) {
          load_tile(&tm_k, x_smem, bar_xy_full, w.tile * kT, w.kvh);
          load_tile(&tm_v, y_smem, bar_xy_full, w.tile * kT, w.kvh);
        } else {
          load_tile(&tm_q, x_smem, bar_xy_full, w.tile * kT, w.h);
          load_tile(&tm_do, y_smem, bar_xy_full, w.tile * kT, w.h - bp.do_head_off);
        }
      }
      for (; j < w.steps && alive; ++j) load_step(j);
      g += (uint32_t)w.steps;
      ++live;
    }
  } else if (warp == 1) {
    // ============================================ UMMA issuer =============================================
    const bool leader = elect_one();
    constexpr uint32_t idesc_s = make_idesc(kT, 64, kBf16, false);
    constexpr uint32_t idesc_g = make_idesc(kT, HD, kBf16, true);
    uint32_t g = 0, live = 0;
    bool alive = true;
    for (int wave = 0; wave < waves && alive; ++wave) {
      const int item = item_of(wave);
      if (item >= bp.total_items) continue;
      const Work w = decode_work<KEYS>(bp, item);
      if (w.steps == 0) continue;
      if (!mbar_wait(bar_xy_full, live & 1u, abort_flag, wait_ns)) break;
      const int halves = 2 * w.steps;
      // gradient products of half `hs`: acc0 += dS U (dK or dQ); KEYS: acc1 += P^T W (dV).  A from TMEM (16-bit, 8
      // columns per 16 of K), B = the 64 streamed rows of the half, MN-major
      auto issue_g = [&](int hs) {
        const int h = hs & 1, s = (int)((g + (uint32_t)(hs >> 1)) % C::kRing);
        if (hs == 0) {   // the row warps must have read the previous item's accumulators
          if (!mbar_wait(bar_acc_empty, (live & 1u) ^ 1u, abort_flag, wait_ns)) { alive = false; return; }
          tc_fence_after();
        }
        const uint32_t u_addr = ring_smem + s * 2 * C::kTileBytes, w_addr = u_addr + C::kTileBytes;
        const uint32_t t_half = tmem_base + (uint32_t)(h * 128);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t bd = make_smem_desc(u_addr + (uint32_t)((h * 4 + kk) * 2048), C::kHalfBytes, 1024);
          if (leader) mma_ts(tmem_base + (uint32_t)C::kAcc0, t_half + 64u + (uint32_t)(kk * 8), bd, idesc_g, (hs > 0 || kk > 0) ? 1u : 0u);
        }
        if constexpr (KEYS) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t bd = make_smem_desc(w_addr + (uint32_t)((h * 4 + kk) * 2048), C::kHalfBytes, 1024);
            if (leader) mma_ts(tmem_base + (uint32_t)C::kAcc1, t_half + (uint32_t)(kk * 8), bd, idesc_g, (hs > 0 || kk > 0) ? 1u : 0u);
          }
        }
        if (leader) {
          if (h == 1) tc_commit(bar_ring_empty + 8 * s);   // both halves of the streamed pair are consumed
          if (hs == halves - 1) {
            tc_commit(bar_acc_full);
            tc_commit(bar_xy_empty);                       // the stationary pair may be replaced
          }
        }
      };
      for (int hs = 0; hs < halves && alive; ++hs) {
        const int h = hs & 1;
        const uint32_t gs = g + (uint32_t)(hs >> 1);
        const int s = (int)(gs % C::kRing);
        if (h == 0) {
          if (!mbar_wait(bar_ring_full + 8 * s, (gs / C::kRing) & 1u, abort_flag, wait_ns)) { alive = false; break; }
        }
        tc_fence_after();
        const uint32_t u_addr = ring_smem + s * 2 * C::kTileBytes + (uint32_t)(h * 8192);   // rows 64h.. of each 64-column block
        const uint32_t w_addr = u_addr + C::kTileBytes;
        const uint32_t t_half = tmem_base + (uint32_t)(h * 128);
        // S (or S^T) = X U^T and dP = Y W^T over the half's 64 streamed rows: both operands K-major
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (uint32_t)((kk >> 2) * C::kHalfBytes + (kk & 3) * 32);
          const uint64_t ad = make_smem_desc(x_smem + off, 16, 1024), bd = make_smem_desc(u_addr + off, 16, 1024);
          if (leader) mma_ss(t_half, ad, bd, idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (uint32_t)((kk >> 2) * C::kHalfBytes + (kk & 3) * 32);
          const uint64_t ad = make_smem_desc(y_smem + off, 16, 1024), bd = make_smem_desc(w_addr + off, 16, 1024);
          if (leader) mma_ss(t_half + 64u, ad, bd, idesc_s, kk > 0 ? 1u : 0u);
        }
        if (leader) tc_commit(bar_s_full + 8 * h);
        if (hs >= 1) {
          const int prev = hs - 1;
          if (!mbar_wait(bar_p_full + 8 * (prev & 1), (g + (uint32_t)(prev >> 1)) & 1u, abort_flag, wait_ns)) { alive = false; break; }
          tc_fence_after();
          issue_g(prev);
        }
      }
      if (alive) {
        const int prev = halves - 1;
        if (mbar_wait(bar_p_full + 8 * (prev & 1), (g + (uint32_t)(prev >> 1)) & 1u, abort_flag, wait_ns)) {
          tc_fence_after();
          issue_g(prev);
        } else {
          alive = false;
        }
      }
      g += (uint32_t)w.steps;
      ++live;
    }
  } else {
    // ===================================== probabilities, dS, epilogue =====================================
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;   // which 64 streamed rows (= score columns) this warp's group handles
    const int row = quarter * 32 + lane;
    const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + lane_bits + (uint32_t)(half * 128), t_dp = t_s + 64u;
    const float sl2 = p.scale * kLog2e;
    float* my_vec = vec_smem + (warp - 2) * (2 * 2 * 64);   // [buffer][-lse*log2e, delta][64]
    uint32_t g = 0, live = 0;
    bool alive = true;
    for (int wave = 0; wave < waves && alive; ++wave) {
      const int item = item_of(wave);
      if (item >= bp.total_items) continue;
      const Work w = decode_work<KEYS>(bp, item);
      const int64_t kv_limit = kv_limit_of(p, w.b);
      const int64_t my_row = (int64_t)w.tile * kT + row;   // key (KEYS) or query index of this thread
      // rows are queries: the thread's own -lse*log2(e) and delta
      float my_nl = -INFINITY, my_dl = 0.f;
      if (!KEYS && my_row < p.seq_q) {
        const float lse = p.lse[((int64_t)w.b * p.num_q_heads + w.h) * p.seq_q + my_row];
        my_nl = (lse == -INFINITY || lse == INFINITY) ? -INFINITY : -lse * kLog2e;
        my_dl = bp.delta[((int64_t)w.b * p.head_count + (w.h - p.head_begin)) * p.seq_q + my_row];
      }
      for (int j = 0; j < w.steps; ++j) {
        const int64_t col0 = (int64_t)step_tile<KEYS>(w, j) * kT + half * 64;   // first query (KEYS) or key of this half
        const float* nls = my_vec + (j & 1) * (2 * 64);
        const float* dls = nls + 64;
        int64_t mask_base = 0;
        if constexpr (MASKED)
          mask_base = (int64_t)w.b * p.mask_stride[0] + (int64_t)(KEYS ? step_head<KEYS>(w, j) : w.h) * p.mask_stride[1];
        if constexpr (KEYS) {
          // the streamed queries' -lse*log2(e) and delta, one private copy per warp (no cross-warp barrier)
          const int h = step_head<KEYS>(w, j);
          float* wl = my_vec + (j & 1) * (2 * 64);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const int c = t * 32 + lane;
            const int64_t q = col0 + c;
            float nl = -INFINITY, dl = 0.f;
            if (q < p.seq_q) {
              const float lse = p.lse[((int64_t)w.b * p.num_q_heads + h) * p.seq_q + q];
              nl = (lse == -INFINITY || lse == INFINITY) ? -INFINITY : -lse * kLog2e;
              dl = bp.delta[((int64_t)w.b * p.head_count + (h - p.head_begin)) * p.seq_q + q];
            }
            wl[c] = nl;
            wl[64 + c] = dl;
          }
          __syncwarp();
        }
        // visible columns of this thread's row within the half: [lo, hi]
        int64_t lo = 0, hi = 63;
        if constexpr (KEYS) {
          if (my_row >= kv_limit) hi = -1;
          if (p.causal) lo = my_row - p.causal_offset - col0;   // query >= key - offset
        } else {
          hi = kv_limit - 1 - col0;
          if (p.causal) {
            const int64_t c = my_row + p.causal_offset - col0;
            if (c < hi) hi = c;
          }
        }
        const bool edge = __any_sync(0xffffffffu, lo > 0 || hi < 63);

        bool ok = mbar_wait(bar_s_full + 8 * half, (g + (uint32_t)j) & 1u, abort_flag, wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t sr[32], dr[32];
          tmem_ld32(t_s + (uint32_t)c0, sr);
          tmem_ld32(t_dp + (uint32_t)c0, dr);
          tc_wait_ld();
          uint32_t pk[16], dk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float pv[2], dv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int cc = c0 + c + e;
              float nl = KEYS ? nls[cc] : my_nl;
              const float dl = KEYS ? dls[cc] : my_dl;
              bool keep = true;
              if constexpr (MASKED) {
                // additive bias (after the scale) or keep-mask of this (query, key), as finish_logit() applies them
                const int64_t qi = KEYS ? col0 + cc : my_row, kj = KEYS ? my_row : col0 + cc;
                if (qi < p.seq_q && kj < p.seq_kv) {
                  const int64_t idx = mask_base + qi * p.mask_stride[2] + kj * p.mask_stride[3];
                  if (p.mask_kind == AIDN_MASK_KEEP_U8) keep = static_cast<const uint8_t*>(p.mask)[idx] != 0;
                  else if (p.mask_kind == AIDN_MASK_KEEP_F32) keep = static_cast<const float*>(p.mask)[idx] != 0.0f;
                  else nl = fmaf(static_cast<const float*>(p.mask)[idx], kLog2e, nl);
                }
              }
              float pe = ex2_approx(fmaf(__uint_as_float(sr[c + e]), sl2, nl));
              if (edge && (cc < lo || cc > hi)) keep = false;
              // selected, not multiplied: a masked position stays 0 whatever its score or dP is (0 * NaN is NaN)
              pe = keep ? pe : 0.f;
              pv[e] = pe;
              dv[e] = keep ? pe * (__uint_as_float(dr[c + e]) - dl) : 0.f;
            }
            pk[c >> 1] = pack2<kBf16>(pv[0], pv[1]);
            dk[c >> 1] = pack2<kBf16>(dv[0], dv[1]);
          }
          // 16-bit P and dS go back over the fp32 columns they came from (columns [c0/2, c0/2+16) were read already)
          if constexpr (KEYS) tmem_st16(t_s + (uint32_t)(c0 >> 1), pk);
          tmem_st16(t_dp + (uint32_t)(c0 >> 1), dk);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p_full + 8 * half);
      }
      if (!alive) break;

      // ---- epilogue: accumulators -> global, one row per thread ----------------------------------------------
      const bool have = w.steps > 0;
      if (have) {
        bool ok = mbar_wait(bar_acc_full, live & 1u, abort_flag, wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        tc_fence_after();
      }
      const int64_t rows_total = KEYS ? p.seq_kv : p.seq_q;
      const bool row_valid = my_row < rows_total;
      float* out0;
      float* out1 = nullptr;
      if constexpr (KEYS) {
        const int64_t base = (((int64_t)w.b * (p.head_count / p.group) + (w.kvh - p.head_begin / p.group)) * p.seq_kv + my_row) * HD;
        out0 = bp.dk + base;
        out1 = bp.dv + base;
      } else {
        out0 = bp.dq + (((int64_t)w.b * p.head_count + (w.h - p.head_begin)) * p.seq_q + my_row) * HD;
      }
      {
        // the two groups of row warps split the stores: dK | dV, or the two halves of dQ's columns
        const int a = KEYS ? half : 0;
        float* out = a == 0 ? out0 : out1;
        const float f = a == 0 ? p.scale : 1.f;
        const uint32_t t_acc = tmem_base + lane_bits + (uint32_t)(a == 0 ? C::kAcc0 : C::kAcc1);
        const int c_begin = KEYS ? 0 : half * (HD / 2), c_end = KEYS ? HD : c_begin + HD / 2;
#pragma unroll
        for (int c0 = c_begin; c0 < c_end; c0 += 32) {
          uint32_t r[32];
          if (have) {
            tmem_ld32(t_acc + (uint32_t)c0, r);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) r[c] = 0u;
          }
          if (row_valid) {
#pragma unroll
            for (int c = 0; c < 32; c += 8)
              st_global_v8(out + c0 + c, __float_as_uint(__uint_as_float(r[c]) * f), __float_as_uint(__uint_as_float(r[c + 1]) * f),
                           __float_as_uint(__uint_as_float(r[c + 2]) * f), __float_as_uint(__uint_as_float(r[c + 3]) * f),
                           __float_as_uint(__uint_as_float(r[c + 4]) * f), __float_as_uint(__uint_as_float(r[c + 5]) * f),
                           __float_as_uint(__uint_as_float(r[c + 6]) * f), __float_as_uint(__uint_as_float(r[c + 7]) * f));
          }
        }
      }
      if (have) {
        // every lane's reads of the accumulators are complete: the next item's gradient products may overwrite them
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty);
        g += (uint32_t)w.steps;
        ++live;
      }
    }
  }

  // ---- teardown -------------------------------------------------------------------------------------
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // Give loads that were already issued a bounded chance to land before shared memory is released.
    if (warp == 0 && lane == 0) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) {
      }
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusTimeout);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

bool aligned_bhs(const void* base, const int64_t* stride, int64_t H, int64_t B, int align) {
  if ((uintptr_t)base % align != 0) return false;
  if ((stride[2] * 2) % align != 0 || stride[2] <= 0) return false;
  if (H > 1 && ((stride[1] * 2) % align != 0 || stride[1] <= 0)) return false;
  if (B > 1 && ((stride[0] * 2) % align != 0 || stride[0] <= 0)) return false;
  return true;
}

template <typename T, int HD>
cudaError_t launch_t(const BwdParams& bp, cudaStream_t stream, int* launches, const char** why) {
  using C = BCfg<HD>;
  const SdpaParams& p = bp.p;
  cudaError_t e = tmap::resolve_encode();
  if (e != cudaSuccess) { *why = "cuTensorMapEncodeTiled is not available from the driver"; return e; }
  constexpr bool bf16 = !std::is_same_v<T, __half>;
  const CUtensorMapDataType dt16 = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUtensorMapSwizzle s128 = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tq, tk, tv, tdo;
  const void* dout16 = bp.dout_t ? bp.dout_t : bp.dout;
  const int64_t dense_do[3] = {(int64_t)p.head_count * p.seq_q * HD, p.seq_q * HD, HD};
  const int64_t* dos = bp.dout_t ? dense_do : bp.dos;
  const int64_t do_heads = bp.dout_t ? p.head_count : p.num_q_heads;
  if (!tmap::encode_bhsd(&tq, dt16, 2, s128, p.q, HD, p.seq_q, p.num_q_heads, p.batch, p.qs, 64, kT) ||
      !tmap::encode_bhsd(&tk, dt16, 2, s128, p.k, HD, p.seq_kv, p.num_kv_heads, p.batch, p.ks, 64, kT) ||
      !tmap::encode_bhsd(&tv, dt16, 2, s128, p.v, HD, p.seq_kv, p.num_kv_heads, p.batch, p.vs, 64, kT) ||
      !tmap::encode_bhsd(&tdo, dt16, 2, s128, dout16, HD, p.seq_q, do_heads, p.batch, dos, 64, kT)) {
    *why = "cuTensorMapEncodeTiled rejected a tensor (address or stride alignment)";
    return cudaErrorInvalidValue;
  }
  BwdSm100Params sp;
  sp.p = p;
  sp.delta = bp.delta;
  sp.dq = bp.dq;
  sp.dk = bp.dk;
  sp.dv = bp.dv;
  sp.q_tiles = (int)((p.seq_q + kT - 1) / kT);
  sp.k_tiles = (int)((p.seq_kv + kT - 1) / kT);
  sp.do_head_off = bp.dout_t ? p.head_begin : 0;
  sp.withhold_loads = bp.expire ? 1 : 0;
  sp.wait_budget_ns = bp.expire ? 20000000ull : kWaitBudgetNs;   // 20 ms in the time-out test
  const bool masked = p.mask_kind != AIDN_MASK_NONE;
  auto kq = masked ? sdpa_backward_sm100_kernel<T, HD, false, true> : sdpa_backward_sm100_kernel<T, HD, false, false>;
  auto kkv = masked ? sdpa_backward_sm100_kernel<T, HD, true, true> : sdpa_backward_sm100_kernel<T, HD, true, false>;
  e = cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) { *why = "cannot raise the dynamic shared memory limit"; return e; }
  const int64_t items_q = (int64_t)sp.q_tiles * p.head_count * p.batch;
  const int64_t items_kv = (int64_t)sp.k_tiles * (p.head_count / p.group) * p.batch;
  if (items_q > 0x7fffffffll || items_kv > 0x7fffffffll) { *why = "work item count out of range"; return cudaErrorInvalidValue; }
  int dev = 0, sms = 0;
  e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess || sms <= 0) { *why = "cannot read the SM count"; return e != cudaSuccess ? e : cudaErrorInvalidValue; }
  sp.total_items = (int)items_q;
  kq<<<(unsigned)(items_q < sms ? items_q : sms), kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, sp);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  sp.total_items = (int)items_kv;
  kkv<<<(unsigned)(items_kv < sms ? items_kv : sms), kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, sp);
  *launches += 2;
  return cudaGetLastError();
}

}  // namespace

bool backward_sm100_supported(const BwdParams& bp, int dtype) {
  const SdpaParams& p = bp.p;
  if (dtype != AIDN_BF16 && dtype != AIDN_F16) return false;
  if (p.head_dim != 64 && p.head_dim != 128) return false;
  if (p.block_table || p.softcap > 0.f || !p.lse) return false;
  if (p.mask_kind != AIDN_MASK_NONE && !p.mask) return false;
  if (!bp.dout_t && p.out_f32) return false;   // dO must be available in the input dtype
  if (!aligned_bhs(p.q, p.qs, p.num_q_heads, p.batch, 16) || !aligned_bhs(p.k, p.ks, p.num_kv_heads, p.batch, 16) ||
      !aligned_bhs(p.v, p.vs, p.num_kv_heads, p.batch, 16))
    return false;
  if (bp.dout_t) {
    if ((uintptr_t)bp.dout_t % 16 != 0) return false;
  } else if (!aligned_bhs(bp.dout, bp.dos, p.num_q_heads, p.batch, 16)) {
    return false;
  }
  if ((uintptr_t)bp.dq % 32 != 0 || (uintptr_t)bp.dk % 32 != 0 || (uintptr_t)bp.dv % 32 != 0) return false;
  if (p.seq_q > 0x3fffff00ll || p.seq_kv > 0x3fffff00ll) return false;
  return true;
}

cudaError_t launch_backward_sm100(const BwdParams& bp, int dtype, cudaStream_t stream, int* launches, const char** why) {
  if (dtype == AIDN_BF16) {
    if (bp.p.head_dim == 128) return launch_t<__nv_bfloat16, 128>(bp, stream, launches, why);
    return launch_t<__nv_bfloat16, 64>(bp, stream, launches, why);
  }
  if (bp.p.head_dim == 128) return launch_t<__half, 128>(bp, stream, launches, why);
  return launch_t<__half, 64>(bp, stream, launches, why);
}

}  // namespace aidn
