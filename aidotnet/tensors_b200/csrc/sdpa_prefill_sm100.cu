// FlashAttention-style prefill forward for sm_100a: TMA + mbarrier pipeline, tcgen05 UMMA with TMEM
// accumulators, warp-specialised roles, online softmax in registers, persistent CTAs.  Causal / padding masks are
// arithmetic; a second instantiation adds softcap, additive bias and keep-masks read by the softmax warps.
//
// A work item is TWO 128-row query tiles that share one KV head, so every K/V tile fetched into shared
// memory feeds the score and P.V products of both.  The two tiles are two query heads of the same GQA group at
// the same rows (group size even) or two consecutive row tiles of one head.  One CTA per SM walks a list of
// work items ordered heaviest first (causal), drawing the next item from a global counter when it finishes one.
//
//   warps 0-3   softmax of tile 0: thread t owns row t of the tile (TMEM lane == row), reads S from TMEM,
//   warps 4-7   softmax of tile 1  keeps the running max / sum, rescales O lazily, writes P (16-bit) back
//                                  into the S columns; at the end either runs the epilogue of its tile itself or
//                                  hands 1 / sum to the epilogue warps and goes on to the next item (struct Roles)
//   warps 12-15 epilogue (four-warpgroup layout only): read O_i out of TMEM (releasing it to the next item's first
//               P.V product), normalise, stage 128 bytes per row in swizzled shared memory (4 KiB boxes) and issue
//               TMA stores
//   warp  8     TMA producer + scheduler: Q tiles, then K and V sub-tiles of 64 keys through a ring of 8 slots, in the
//               order the issuers need them (K(0), K(1), V(0), K(2), V(1), ...): three sub-tiles of look-ahead, which
//               a TMA load under full load needs (2700 cycles from a slot's release to its data, measured)
//   warps 9,10  UMMA issuers (one lane each): S = Q K^T (smem x smem), O += P V (TMEM x smem); issuer b handles the
//               sub-tiles of parity b of both query tiles, the two take turns; warp 9 owns TMEM
//
// Scores are produced and consumed in SUB-TILES of 64 keys, and every query tile has TWO score buffers in TMEM:
//   S_i[b] at columns i*128 + b*64 (b = sub-tile index & 1), P_i[b] (16-bit) over the first 32 columns of S_i[b],
//   O_0 at [256, 256+D), O_1 at [256+D, 256+2D).
// The issuer runs the score product one sub-tile ahead of the softmax: right after P_i(u).V it issues Q_i.K(u+2)^T
// into the buffer that P_i(u) is being read from (UMMAs execute in issue order), so when the softmax warps finish
// sub-tile u the scores of u+1 are already waiting in the other buffer.  With a single 128-column score buffer per
// tile the chain  softmax -> P.V -> next scores -> softmax  was the period of the loop (3500 cycles per 128 keys,
// measured with clock stamps: 2000 softmax + 1030 UMMA issue-to-completion + 490 hand-offs) and left the tensor and
// MUFU pipes 55-60 % busy; here the softmax warps go from one sub-tile straight to the next and the loop runs at
// the rate of the slower of the two pipes.  N = 64 score UMMAs read more shared memory per flop than N = 128 ones
// (the Q operand is re-read for every 64 keys); the trade is measured in profiles/.
// With the softmax warps running the epilogue, an item of two equally long tiles costs its loop plus 4.5 us of
// hand-over (o_full wait 0.6, epilogue 2.6, restart 1.2 us; per-item timeline), during which the tensor pipe idles;
// a fourth warpgroup takes the epilogue over for such items.
//
// Supersedes flash_attention_v2 / grouped_query_attention / scaled_dot_product_attention of the reference
// (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/Kernels/CudaAttentionKernels.cs:28-234, 527-646) and its
// sm_86-only mma.sync kernel (CUDA/Ptx/PtxOnlineFusedAttention128x64Kernel.cs), whose numerics it keeps:
// fp32 scores, exp as ex2.approx((s - max) * scale * log2e), row sum over un-rounded fp32 probabilities,
// P rounded to 16 bit for the second MMA, O rescale skipped while the max moves little (:711-802).
#include <cuda.h>

#include <cstring>
#include <type_traits>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tensor_map.hpp"

// Development builds (-DAIDN_PREFILL_TRACE=1) carry a per-item timeline and a value tap in the hot loops; the
// library that ships is built without them, so they cost no registers or predicates there.
#ifndef AIDN_PREFILL_TRACE
#define AIDN_PREFILL_TRACE 0
#endif

namespace aidn {
namespace {

using namespace ptx;

constexpr int kBM = 128;           // rows per query tile
constexpr int kBS = 64;            // keys per score sub-tile: one softmax step, one K / V ring slot, one TMA box
constexpr int kSoftmaxWarps = 8;   // 2 tiles x 4 warps
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kEpilogueWarp = 12;      // warps 12-15: warp 12 + j reads TMEM lanes 32 j .. 32 j + 31, like softmax warp j
constexpr int kEpilogueWarps = 4;
constexpr int kStageBytes = 32768;     // epilogue staging: 32-row x 128-byte boxes (128-byte swizzle) of 4 KiB
constexpr int kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units: P stays below 2^8 between rescales

// Two role layouts, chosen by the host per launch.
//   EPI = false: 3 warpgroups (384 threads); the softmax warps run the epilogue of their own tile (one 4 KiB staging
//                buffer per warp).  Best when the two tiles of an item differ in length (row pairs under a causal mask:
//                the second tile runs two sub-tiles longer): the warpgroup that finishes first stores its tile under
//                the other's last sub-tiles and then starts the next item - where it gets the longer tile - ahead of it.
//   EPI = true:  4 warpgroups (512 threads); warps 12-15 run the epilogue (two 4 KiB staging buffers per warp) and the
//                softmax warps go straight on to the next item.  Best when both tiles end together (head pairs of a GQA
//                group, no causal mask): measured +4 % on B2 Hq32/Hkv8 S8192 and on B1 Hq8/Hkv1 S32768, -1 % on the
//                row pairs of B4 H32 S2048, which therefore keep the first layout.
// Per-thread registers after setmaxnreg: 8*32*184 + 4*32*136 == 384*168 and 8*32*176 + 8*32*80 == 512*128 - the figures
// must add up to what the CTA was launched with: setmaxnreg.inc waits, without any bound, for registers that another
// warpgroup of the same CTA has given up, and a sum above the launch allocation never becomes available.
template <bool EPI>
struct Roles {
  static constexpr int kThreads = EPI ? 512 : 384;
  static constexpr int kSoftmaxRegs = EPI ? 176 : 184;
  static constexpr int kOtherRegs = EPI ? 80 : 136;
  static constexpr int kOtherWarps = EPI ? 8 : 4;
  static constexpr int kStoreWarps = EPI ? kEpilogueWarps : kSoftmaxWarps;   // warps that stage and store O
  static constexpr int kStageBufs = EPI ? 2 : 1;                             // 4 KiB staging buffers per storing warp
  // consumers of the item mailbox: softmax warps, the two UMMA issuers, epilogue warps
  static constexpr int kSchedConsumers = kSoftmaxWarps + 2 + (EPI ? kEpilogueWarps : 0);
  static_assert(kSoftmaxWarps * 32 * kSoftmaxRegs + kOtherWarps * 32 * kOtherRegs <= kThreads * (EPI ? 128 : 168),
                "setmaxnreg budget exceeds the registers the CTA is launched with");
  static_assert(kStoreWarps * kStageBufs * 4096 == kStageBytes, "staging memory");
};
constexpr int kItemWords = 14;   // mailbox entry: item, b, kvh, n_max, (h, t, n, valid) of both tiles, v_tail

template <int HD>
struct Cfg {
  static constexpr int kTileBytes = kBM * HD * 2;         // one Q tile
  static constexpr int kSubBytes = kBS * HD * 2;          // one K or V sub-tile (64 keys): a ring slot
  static constexpr int kStages = HD == 128 ? 8 : 12;      // K/V ring slots
  static constexpr int kHalves = HD / 64;                 // 64-element (128-byte) column blocks per tile
  static constexpr int kHalfBytes = kBM * 128;            // 16 KiB: one column block of a Q tile
  static constexpr int kKvHalfBytes = kBS * 128;          // 8 KiB: one column block of a K / V sub-tile
  static constexpr int kStageOff = 2 * kTileBytes + kStages * kSubBytes;
  static constexpr int kBarOff = kStageOff + kStageBytes;
  // q_full[2] q_empty[2] kv_full[S] kv_empty[S] s_full[2][2] p_full[2][2] o_full[2] pv_done[2] sched_full[2] sched_empty[2]
  // stats_full[2] stats_empty[2] o_empty[2]
  static constexpr int kNumBars = 26 + 2 * kStages;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;  // issue lock, tmem ptr, abort flag, then the 2-slot item mailbox
  static constexpr int kMailOff = kMiscOff + 16;
  static constexpr int kStatsOff = kMailOff + 2 * kItemWords * 4;   // 1 / row sum of both tiles: [2][128] floats
  static constexpr int kSmemBytes = kStatsOff + 2 * kBM * 4 + 1024 /*align slack*/;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");
  static constexpr int kOCol = 256;
};

struct PrefillParams {
  SdpaParams p;
  int32_t row_tiles;       // ceil(seq_q / 128)
  int32_t pair_heads;      // 1: the two tiles are heads (h, h+1) at one row tile; 0: row tiles (2u, 2u+1) of one head
  int32_t ranks;           // scheduling ranks along the row-tile axis (heavy first)
  int32_t items_per_rank;  // batch * work items per rank
  int32_t per_batch;       // work items per rank per batch entry
  int32_t total_items;
  int32_t* sched;          // [0] next-item counter, [1] finished-CTA counter; both zero between launches
  float* debug;            // trace builds only: tap / timeline buffer
  int32_t debug_mode;      // 3: the producer withholds the Q tiles, so that the bounded waits run out (test hook);
                           // trace builds: 2 = per-item timeline (16 x u64 per item), 4 / 6 = per-step clock stamps of CTA 0,
                           // 7 = SM clock and wall-clock time at the start and end of every CTA
  uint64_t wait_budget_ns; // longest single wait before the CTA gives up
};

// Tensor maps of the other devices' output tensors (fused gather): every output box is stored to each of them too.
struct alignas(64) PeerMaps {
  CUtensorMap maps[AIDN_MAX_PEERS];
  int32_t count;
};

struct TileInfo {
  int h;          // q head
  int t;          // row tile index
  int n;          // 64-key score sub-tiles to process (0 = none visible)
  bool valid;     // tile exists
};

struct Item {
  TileInfo tile[2];
  int b, kvh;
  int n_max;      // sub-tiles of the longer tile = K and V sub-tiles the item streams
  int v_tail;     // > 0: rows of the item's last V sub-tile that hold keys of the sequence; the rows after them are
                  // cleared in shared memory before the P.V product (0 = nothing to clear)
};

// The producer decodes a work item once (two integer divisions and the tile counts) and hands the result to the
// nine consumer warps through shared memory, so that none of them repeats that work on its critical path.
__device__ __forceinline__ void publish_item(volatile int* box, int item, const Item& it) {
  box[1] = it.b; box[2] = it.kvh; box[3] = it.n_max;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    box[4 + 4 * i] = it.tile[i].h; box[5 + 4 * i] = it.tile[i].t;
    box[6 + 4 * i] = it.tile[i].n; box[7 + 4 * i] = it.tile[i].valid ? 1 : 0;
  }
  box[12] = it.v_tail;
  box[0] = item;
}

__device__ __forceinline__ Item read_item(const volatile int* box) {
  Item it;
  it.b = box[1]; it.kvh = box[2]; it.n_max = box[3];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    it.tile[i].h = box[4 + 4 * i]; it.tile[i].t = box[5 + 4 * i];
    it.tile[i].n = box[6 + 4 * i]; it.tile[i].valid = box[7 + 4 * i] != 0;
  }
  it.v_tail = box[12];
  return it;
}

__device__ __forceinline__ Item decode_item(const PrefillParams& pp, int item) {
  const SdpaParams& p = pp.p;
  Item it;
  const int rank = item / pp.items_per_rank;
  const int rem = item - rank * pp.items_per_rank;
  it.b = rem / pp.per_batch;
  const int w = rem - it.b * pp.per_batch;
  if (pp.pair_heads) {
    const int t = pp.row_tiles - 1 - rank;
    it.tile[0].h = p.head_begin + 2 * w;
    it.tile[1].h = it.tile[0].h + 1;
    it.tile[0].t = it.tile[1].t = t;
    it.tile[0].valid = it.tile[1].valid = true;
  } else {
    const int u = pp.ranks - 1 - rank;
    it.tile[0].h = it.tile[1].h = p.head_begin + w;
    it.tile[0].t = 2 * u;
    it.tile[1].t = 2 * u + 1;
    it.tile[0].valid = true;
    it.tile[1].valid = it.tile[1].t < pp.row_tiles;
  }
  it.kvh = it.tile[0].h / p.group;
  const int64_t kv_limit = kv_limit_of(p, it.b);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int64_t kend = 0;
    if (it.tile[i].valid) {
      kend = kv_limit;
      if (p.causal) {
        int64_t last_row = (int64_t)it.tile[i].t * kBM + kBM - 1;
        if (last_row > p.seq_q - 1) last_row = p.seq_q - 1;
        const int64_t c = last_row + p.causal_offset + 1;
        if (c < kend) kend = c;
      }
      if (kend < 0) kend = 0;
    }
    it.tile[i].n = (int)((kend + kBS - 1) / kBS);
  }
  it.n_max = it.tile[0].n > it.tile[1].n ? it.tile[0].n : it.tile[1].n;
  // Rows of the last V tile past the sequence's last key hold whatever the caller's buffer holds there (padding after
  // kv_len, the unused tail of a pool block).  Their probabilities are 0, but 0 * NaN is NaN in the P.V product, so
  // the UMMA warp clears them.  Rows past seq_kv of a contiguous tensor are zero-filled by TMA itself.
  it.v_tail = 0;
  if ((p.kv_len || p.block_table) && (int64_t)it.n_max * kBS > kv_limit)
    it.v_tail = (int)(kv_limit - (int64_t)(it.n_max - 1) * kBS);
  return it;
}

// Epilogue warps: O_i / l of one tile, 32 rows per warp: TMEM -> registers -> swizzled staging (128 bytes per row) -> TMA
// stores.  `n_stores` counts this warp's stores; store k stages through buffer k & 1.  `bar_o_empty` gets one arrival
// per warp as soon as the tile's last tcgen05.ld has completed.
template <int HD, bool kBf16>
__device__ __forceinline__ void store_o_tile(const SdpaParams& p, const CUtensorMap* tm_o, const PeerMaps& pm, uint32_t t_o,
                                             bool have_o, float inv, uint32_t my_stage, uint32_t& n_stores, int lane,
                                             int row0, int h, int b, uint32_t bar_o_empty) {
  // 128-byte staging rows under the 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7)
  const uint32_t my_swz = (uint32_t)(lane & 7);
  const bool box_valid = row0 < p.seq_q;
#pragma unroll
  for (int c0 = 0; c0 < HD; c0 += 32) {
    uint32_t orr[32];
    if (have_o) {
      tmem_ld32(t_o + c0, orr);
      tc_wait_ld();
      if (c0 + 32 == HD) {
        // O_i is in registers: the next item's first P.V product may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_o_empty);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 32; ++c) orr[c] = 0u;
    }
    // fp32 output: 32 columns fill the 128-byte row (one store per 32 columns); 16-bit output: 64 columns
    const int half = p.out_f32 ? 0 : ((c0 >> 5) & 1);
    const uint32_t buf = my_stage + (n_stores & 1u) * 4096u;
    const uint32_t my_row = buf + (uint32_t)(lane * 128);
    if (half == 0 && n_stores >= 2u) {
      // the store before the previous one used this buffer and must have finished reading it
      if (lane == 0) bulk_wait_read1();
      __syncwarp();
    }
    if (p.out_f32) {
#pragma unroll
      for (int c = 0; c < 8; ++c)
        st_shared_v4(my_row + (((uint32_t)c ^ my_swz) << 4),
                     __float_as_uint(__uint_as_float(orr[4 * c]) * inv),
                     __float_as_uint(__uint_as_float(orr[4 * c + 1]) * inv),
                     __float_as_uint(__uint_as_float(orr[4 * c + 2]) * inv),
                     __float_as_uint(__uint_as_float(orr[4 * c + 3]) * inv));
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        st_shared_v4(my_row + (((uint32_t)(half * 4 + c) ^ my_swz) << 4),
                     pack2<kBf16>(__uint_as_float(orr[8 * c]) * inv, __uint_as_float(orr[8 * c + 1]) * inv),
                     pack2<kBf16>(__uint_as_float(orr[8 * c + 2]) * inv, __uint_as_float(orr[8 * c + 3]) * inv),
                     pack2<kBf16>(__uint_as_float(orr[8 * c + 4]) * inv, __uint_as_float(orr[8 * c + 5]) * inv),
                     pack2<kBf16>(__uint_as_float(orr[8 * c + 6]) * inv, __uint_as_float(orr[8 * c + 7]) * inv));
    }
    if (p.out_f32 || half == 1) {
      fence_proxy_async_smem();
      __syncwarp();
      // the store is counted (and its group committed) whether or not the box lies inside the tensor
      if (lane == 0) {
        if (box_valid) {
          tma_store_4d(tm_o, buf, p.out_f32 ? c0 : c0 - 32, row0, h, b);
          for (int r = 0; r < pm.count; ++r) tma_store_4d(&pm.maps[r], buf, p.out_f32 ? c0 : c0 - 32, row0, h, b);
        }
        bulk_commit();
      }
      ++n_stores;
    }
  }
}

// MASKED: the softmax warps also apply softcap, an additive bias or a keep-mask read from global memory (one row
// per thread); the plain variant carries none of that code.
template <typename T, int HD, bool MASKED, bool EPI>
__global__ void __launch_bounds__(Roles<EPI>::kThreads, 1)
    sdpa_prefill_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                              const __grid_constant__ PeerMaps pm, const PrefillParams pp) {
  using C = Cfg<HD>;
  using R = Roles<EPI>;
  constexpr bool kBf16 = !std::is_same_v<T, __half>;
  const SdpaParams& p = pp.p;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base;                           // 2 tiles
  const uint32_t kv_smem = smem_base + 2 * C::kTileBytes;      // kStages sub-tiles
  const uint32_t stage_smem = smem_base + C::kStageOff;        // 4 KiB boxes: 2 per epilogue warp, or 1 per softmax warp
  const uint32_t bars = smem_base + C::kBarOff;
  const uint32_t bar_q_full = bars;                            // [2]
  const uint32_t bar_q_empty = bars + 16;                      // [2]
  const uint32_t bar_kv_full = bars + 32;                      // [kStages]
  const uint32_t bar_kv_empty = bar_kv_full + 8 * C::kStages;  // [kStages]
  const uint32_t bar_s_full = bar_kv_empty + 8 * C::kStages;   // [tile][buffer]
  const uint32_t bar_p_full = bar_s_full + 32;                 // [tile][buffer]
  const uint32_t bar_o_full = bar_p_full + 32;                 // [2]
  const uint32_t bar_pv_done = bar_o_full + 16;                // [2] one phase per P.V product of the tile
  const uint32_t bar_sched_full = bar_pv_done + 16;            // [2]
  const uint32_t bar_sched_empty = bar_sched_full + 16;        // [2]
  const uint32_t bar_stats_full = bar_sched_empty + 16;        // [2] the softmax warps of a tile have written its 1 / row sums
  const uint32_t bar_stats_empty = bar_stats_full + 16;        // [2] the epilogue warps have read them
  const uint32_t bar_o_empty = bar_stats_empty + 16;           // [2] the epilogue warps have read O_i out of TMEM
  volatile float* stats = reinterpret_cast<volatile float*>(smem_gen + C::kStatsOff);   // [2][kBM]
  volatile int* mailbox = reinterpret_cast<volatile int*>(smem_gen + C::kMailOff);  // [2][kItemWords]
  int* issue_turn = reinterpret_cast<int*>(smem_gen + C::kMiscOff);   // turns of the two UMMA issuers completed so far
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_gen + C::kMiscOff + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + C::kMiscOff + 12);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t wait_ns = pp.wait_budget_ns;

  // ---- setup ---------------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *issue_turn = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_q_full + 8 * i, 1);
      mbar_init(bar_q_empty + 8 * i, 2);   // both issuers read a Q tile
      mbar_init(bar_o_full + 8 * i, 1);
      mbar_init(bar_pv_done + 8 * i, 1);
      mbar_init(bar_sched_full + 8 * i, 1);
      mbar_init(bar_sched_empty + 8 * i, R::kSchedConsumers);
      mbar_init(bar_stats_full + 8 * i, 4);    // one arrival per softmax warp of the tile
      mbar_init(bar_stats_empty + 8 * i, kEpilogueWarps);
      mbar_init(bar_o_empty + 8 * i, kEpilogueWarps);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_p_full + 8 * i, 4);   // one arrival per softmax warp of the tile
    }
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_kv_full + 8 * s, 1);
      mbar_init(bar_kv_empty + 8 * s, 1);   // a sub-tile is read by one issuer
    }
    fence_mbar_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_o);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_ptr_smem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
#if AIDN_PREFILL_TRACE
  // mode 7: SM clock and wall-clock time at the start and end of every CTA (4 x u64 per CTA): the effective SM clock
  if (pp.debug_mode == 7 && threadIdx.x == 0) {
    unsigned long long* cl = reinterpret_cast<unsigned long long*>(pp.debug) + 4 * blockIdx.x;
    cl[0] = (unsigned long long)clock64();
    cl[1] = globaltimer_ns();
  }
#endif

  // Plain: scores stay raw and the scale is folded into the exponent (one FMA).  Masked: scores are scaled first
  // (softcap and bias act on scaled logits), so the exponent only needs log2(e).
  const float sl2 = MASKED ? kLog2e : p.scale * kLog2e;
  const float lse_scale = MASKED ? 1.f : p.scale;

  if (warp < kSoftmaxWarps) {
    // =================================== softmax / epilogue ===================================
    setmaxnreg_inc<R::kSoftmaxRegs>();
    const int i = warp >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + lane_bits + (uint32_t)(i * 2 * kBS);
    const uint32_t t_o = tmem_base + lane_bits + (uint32_t)(C::kOCol + i * HD);
    uint32_t s_par = 0;                // bit b: parity of the next phase of s_full[tile][b]
    uint32_t pv_par = 0;               // parity of the next phase of pv_done (one per item with two or more sub-tiles)
    uint32_t handed = 0;               // EPI: row statistics handed to the epilogue warps so far
    uint32_t o_cnt = 0;                // !EPI: completed phases of o_full
    bool stores_in_flight = false;     // !EPI: a TMA store of this warp may still be reading the staging buffer
    // !EPI: one 4 KiB staging buffer per softmax warp; 16-byte chunk c of row r sits at chunk c ^ (r & 7)
    const uint32_t my_stage = stage_smem + (uint32_t)(warp * 4096);
    const uint32_t my_row = my_stage + (uint32_t)(lane * 128);
    const uint32_t my_swz = (uint32_t)(lane & 7);
    bool alive = true;

    for (int seq = 0; alive; ++seq) {
      // next work item from the producer's 2-slot mailbox
      int item;
      {
        const int slot = seq & 1;
        bool ok = mbar_wait(bar_sched_full + 8 * slot, (uint32_t)((seq >> 1) & 1), abort_flag, wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        item = mailbox[slot * kItemWords];
      }
      if (item >= pp.total_items) break;   // no further mailbox traffic after the end marker
      const Item it = read_item(mailbox + (seq & 1) * kItemWords);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sched_empty + 8 * (seq & 1));
      const TileInfo ti = it.tile[i];
      if (!ti.valid) continue;
      const int b = it.b;
#if AIDN_PREFILL_TRACE
      unsigned long long* trace = pp.debug_mode == 2
          ? reinterpret_cast<unsigned long long*>(pp.debug) + (size_t)item * 16 : nullptr;
      const bool tracer = trace && row_in_tile == 0;
      if (tracer) {
        trace[1 + 8 * i] = globaltimer_ns();
        if (i == 0) {
          unsigned smid;
          asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
          trace[15] = ((unsigned long long)smid << 32) | (unsigned)it.n_max;
        }
      }
      // per-step clock stamps (mode 4): CTA 0, the first 8 items, up to 32 steps, 16 slots per step
      long long* steps = (((pp.debug_mode == 4) || (pp.debug_mode == 6 && i == 0)) && blockIdx.x == 0 && seq < 8 && row_in_tile == 0)
          ? reinterpret_cast<long long*>(pp.debug) + (size_t)seq * 32 * 16 + 5 * i : nullptr;
#define STEP_STAMP(j, slot) do { if (steps && (j) < 32) steps[(j) * 16 + (slot)] = clock64(); } while (0)
#else
      constexpr bool tracer = false;
      unsigned long long* const trace = nullptr;
#define STEP_STAMP(j, slot) do { } while (0)
#endif

      const int64_t qrow = (int64_t)ti.t * kBM + row_in_tile;
      const int64_t kv_limit = kv_limit_of(p, b);
      int64_t kmax_row = kv_limit - 1;   // last visible key of this row
      if (p.causal && qrow + p.causal_offset < kmax_row) kmax_row = qrow + p.causal_offset;

      float m = -INFINITY, l = 0.f;

      for (int u = 0; u < ti.n; ++u) {
        const uint32_t buf = (uint32_t)(u & 1);
        const uint32_t t_sb = t_s + buf * kBS;
        const uint32_t bar_off = 8u * (uint32_t)(2 * i) + 8u * buf;
        bool ok = mbar_wait(bar_s_full + bar_off, (s_par >> buf) & 1u, abort_flag, wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        tc_fence_after();
        if (tracer && u == 0) trace[2 + 8 * i] = globaltimer_ns();
        STEP_STAMP(u, 0);

        uint32_t sr[kBS];
        tmem_ld32(t_sb + 0, sr + 0);
        tmem_ld32(t_sb + 32, sr + 32);
        tc_wait_ld();
        STEP_STAMP(u, 1);
        float* s = reinterpret_cast<float*>(sr);

        const int64_t col0 = (int64_t)u * kBS;
        if constexpr (MASKED) {
          // scale -> softcap -> bias -> keep-mask, the order of the reference (CpuEngine.cs:27807-27816, 29218-29239)
          const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
          const int64_t mrow = qrow < p.seq_q ? qrow : p.seq_q - 1;   // rows past the end read a valid row
          const int64_t mbase = (int64_t)b * p.mask_stride[0] + (int64_t)ti.h * p.mask_stride[1] + mrow * p.mask_stride[2];
          const int64_t ms3 = p.mask_stride[3];
          const bool full_tile = col0 + kBS <= p.seq_kv;
          const int kind = p.mask_kind;
          if (kind == AIDN_MASK_NONE) {
#pragma unroll
            for (int c = 0; c < kBS; ++c) {
              float val = s[c] * p.scale;
              if (p.softcap > 0.f) val = p.softcap * tanh_approx(val * inv_cap);
              s[c] = val;
            }
          } else if (kind == AIDN_MASK_KEEP_U8) {
            const uint8_t* mp = static_cast<const uint8_t*>(p.mask) + mbase + col0 * ms3;
            const bool vec = ms3 == 1 && full_tile && ((reinterpret_cast<uintptr_t>(mp) & 15) == 0);
#pragma unroll
            for (int c0 = 0; c0 < kBS; c0 += 16) {
              uint32_t w[4];
              if (vec) {
                const uint4 u4 = *reinterpret_cast<const uint4*>(mp + c0);
                w[0] = u4.x; w[1] = u4.y; w[2] = u4.z; w[3] = u4.w;
              } else {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                  w[q4] = 0;
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const int c = c0 + q4 * 4 + e;
                    const uint32_t byte = (col0 + c < p.seq_kv) ? mp[(int64_t)c * ms3] : 0u;
                    w[q4] |= (byte != 0 ? 1u : 0u) << (8 * e);
                  }
                }
              }
#pragma unroll
              for (int c = 0; c < 16; ++c) {
                float val = s[c0 + c] * p.scale;
                if (p.softcap > 0.f) val = p.softcap * tanh_approx(val * inv_cap);
                if (((w[c >> 2] >> (8 * (c & 3))) & 0xffu) == 0u) val = -INFINITY;
                s[c0 + c] = val;
              }
            }
          } else {
            const float* mp = static_cast<const float*>(p.mask) + mbase + col0 * ms3;
            const bool vec = ms3 == 1 && full_tile && ((reinterpret_cast<uintptr_t>(mp) & 15) == 0);
#pragma unroll
            for (int c0 = 0; c0 < kBS; c0 += 4) {
              float mv[4];
              if (vec) {
                const float4 u4 = *reinterpret_cast<const float4*>(mp + c0);
                mv[0] = u4.x; mv[1] = u4.y; mv[2] = u4.z; mv[3] = u4.w;
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) mv[e] = (col0 + c0 + e < p.seq_kv) ? mp[(int64_t)(c0 + e) * ms3] : 0.f;
              }
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float val = s[c0 + e] * p.scale;
                if (p.softcap > 0.f) val = p.softcap * tanh_approx(val * inv_cap);
                if (kind == AIDN_MASK_ADD_F32) val += mv[e];
                else if (mv[e] == 0.0f) val = -INFINITY;
                s[c0 + e] = val;
              }
            }
          }
        }
        if (col0 + kBS - 1 > kmax_row) {
          const int64_t lim = kmax_row - col0;  // columns > lim are masked (lim may be negative)
#pragma unroll
          for (int c = 0; c < kBS; ++c)
            if (c > lim) s[c] = -INFINITY;
        }

        float mx0 = s[0], mx1 = s[1], mx2 = s[2], mx3 = s[3];
#pragma unroll
        for (int c = 4; c < kBS; c += 4) {
          mx0 = fmaxf(mx0, s[c]);
          mx1 = fmaxf(mx1, s[c + 1]);
          mx2 = fmaxf(mx2, s[c + 2]);
          mx3 = fmaxf(mx3, s[c + 3]);
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        const float m_new = fmaxf(m, mx);
        STEP_STAMP(u, 2);

        if (u == 0) {
          m = m_new;
        } else {
          const bool need = (m_new - m) * sl2 > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            // O is rescaled in TMEM by the row's owner.  The P.V product of the previous sub-tile accumulates into
            // the same columns and may still be running (the scores of this sub-tile were ready before it was even
            // issued), so its completion is awaited first.  It is covered by the commit behind the score product
            // that the issuer put right after it - the one for sub-tile u + 1, i.e. the other buffer's s_full, whose
            // phase is only tested here, not consumed - or, when there is no sub-tile u + 1, by pv_done.
            if (u + 1 < ti.n) {
              ok = mbar_wait(bar_s_full + 8u * (uint32_t)(2 * i) + 8u * (buf ^ 1u), (s_par >> (buf ^ 1u)) & 1u, abort_flag, wait_ns);
            } else {
              ok = mbar_wait(bar_pv_done + 8 * i, pv_par, abort_flag, wait_ns);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { alive = false; break; }
            tc_fence_after();
            float f;
            if (m_new == -INFINITY) f = 1.f;
            else if (m == -INFINITY) f = 0.f;
            else f = ex2_approx((m - m_new) * sl2);
            l *= f;
            m = m_new;
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 16) {
              uint32_t orr[16];
              tmem_ld16(t_o + c0, orr);
              tc_wait_ld();
#pragma unroll
              for (int c = 0; c < 16; ++c) orr[c] = __float_as_uint(__uint_as_float(orr[c]) * f);
              tmem_st16(t_o + c0, orr);
            }
            tc_wait_st();
          }
        }

        const float neg_ms = (m == -INFINITY) ? 0.f : -m * sl2;
        float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
        // (Computing one exponential in 2, 4 or 8 on the FMA pipe instead - a cubic after the 1.5 * 2^23 rounding trick -
        // was measured and is slower here, 6-10 %: with two softmax warps per scheduler the loop is bound by their
        // instruction stream, not by the MUFU unit.)
#pragma unroll
        for (int c0 = 0; c0 < kBS; c0 += 32) {
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
          tmem_st16(t_sb + (c0 >> 1), pk);
        }
        l += (ls0 + ls1) + (ls2 + ls3);
        STEP_STAMP(u, 3);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full + bar_off);   // one arrival per warp: 128 arrivals on one word serialise
        STEP_STAMP(u, 4);
        s_par ^= 1u << buf;
      }
      if (!alive) break;
      if (ti.n >= 2) pv_par ^= 1u;   // the issuer signalled pv_done once for this item
      if (tracer) trace[3 + 8 * i] = globaltimer_ns();

      if constexpr (EPI) {
        // ---- hand the row to the epilogue warps: 1 / l through shared memory, the log-sum-exp straight to memory ----
        bool ok = mbar_wait(bar_stats_empty + 8 * i, (handed & 1u) ^ 1u, abort_flag, wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        ++handed;
        const float inv = (l > 0.f && m != -INFINITY) ? 1.f / l : 0.f;
        stats[i * kBM + row_in_tile] = inv;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_stats_full + 8 * i);
        if (qrow < p.seq_q && p.lse)
          p.lse[((int64_t)b * p.num_q_heads + ti.h) * p.seq_q + qrow] =
              (inv > 0.f) ? m * lse_scale + logf(l) : -INFINITY;
      } else {
        // ---- epilogue: O / l -> swizzled staging (128 B per row) -> TMA stores ------------------------------
        {
          const bool have_o = ti.n > 0;
          if (have_o) {
            // the last two P.V products were issued by different warps: pv_done covers the second-to-last one
            bool ok = ti.n < 2 || mbar_wait(bar_pv_done + 8 * i, pv_par ^ 1u, abort_flag, wait_ns);
            ok = ok && mbar_wait(bar_o_full + 8 * i, o_cnt & 1u, abort_flag, wait_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { alive = false; break; }
            ++o_cnt;
            tc_fence_after();
          }
          if (tracer) trace[4 + 8 * i] = globaltimer_ns();
          const bool row_valid = qrow < p.seq_q;
          const float inv = (l > 0.f && m != -INFINITY) ? 1.f / l : 0.f;
          const int row0 = ti.t * kBM + quarter * 32;   // first row of this warp's 32-row box
          const bool box_valid = row0 < p.seq_q;
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
            // fp32 output: 32 columns fill the 128-byte row (one store per 32 columns); 16-bit output: 64 columns
            const int half = p.out_f32 ? 0 : ((c0 >> 5) & 1);
            if (half == 0 && stores_in_flight) {
              if (lane == 0) bulk_wait_read0();
              __syncwarp();
            }
            if (p.out_f32) {
#pragma unroll
              for (int c = 0; c < 8; ++c)
                st_shared_v4(my_row + (((uint32_t)c ^ my_swz) << 4),
                             __float_as_uint(__uint_as_float(orr[4 * c]) * inv),
                             __float_as_uint(__uint_as_float(orr[4 * c + 1]) * inv),
                             __float_as_uint(__uint_as_float(orr[4 * c + 2]) * inv),
                             __float_as_uint(__uint_as_float(orr[4 * c + 3]) * inv));
            } else {
#pragma unroll
              for (int c = 0; c < 4; ++c)
                st_shared_v4(my_row + (((uint32_t)(half * 4 + c) ^ my_swz) << 4),
                             pack2<kBf16>(__uint_as_float(orr[8 * c]) * inv, __uint_as_float(orr[8 * c + 1]) * inv),
                             pack2<kBf16>(__uint_as_float(orr[8 * c + 2]) * inv, __uint_as_float(orr[8 * c + 3]) * inv),
                             pack2<kBf16>(__uint_as_float(orr[8 * c + 4]) * inv, __uint_as_float(orr[8 * c + 5]) * inv),
                             pack2<kBf16>(__uint_as_float(orr[8 * c + 6]) * inv, __uint_as_float(orr[8 * c + 7]) * inv));
            }
            if (p.out_f32 || half == 1) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0 && box_valid) {
                tma_store_4d(&tm_o, my_stage, p.out_f32 ? c0 : c0 - 32, row0, ti.h, b);
                for (int r = 0; r < pm.count; ++r) tma_store_4d(&pm.maps[r], my_stage, p.out_f32 ? c0 : c0 - 32, row0, ti.h, b);
                bulk_commit();
              }
              stores_in_flight = true;
            }
          }
          if (row_valid && p.lse)
            p.lse[((int64_t)b * p.num_q_heads + ti.h) * p.seq_q + qrow] =
                (inv > 0.f) ? m * lse_scale + logf(l) : -INFINITY;
          if (tracer) trace[5 + 8 * i] = globaltimer_ns();
        }
      }
    }
    if constexpr (!EPI) {
      // staging memory must outlive the bulk stores that read it
      if (lane == 0) bulk_wait_all();
      __syncwarp();
    }
  } else {
    setmaxnreg_dec<R::kOtherRegs>();
  }

  if (warp == kProducerWarp) {
    // ==================================== TMA producer + scheduler ====================================
    // warp-uniform like the UMMA issuer: one elected lane issues the TMA loads and barrier operations
    {
      const bool leader = elect_one();
      bool alive = true;
      uint32_t t_load = 0;          // K/V tiles loaded so far (ring position)
      uint32_t q_uses[2] = {0, 0};  // loads of each Q tile so far
      int item = blockIdx.x;
      for (int seq = 0; alive; ++seq) {
        const int slot = seq & 1;
        if (!mbar_wait(bar_sched_empty + 8 * slot, (uint32_t)(((seq >> 1) & 1) ^ 1), abort_flag, wait_ns)) break;
        Item it;
        if (item < pp.total_items) {
          it = decode_item(pp, item);
          // Row pairs: the second tile runs two sub-tiles longer.  Alternating which softmax warpgroup gets it keeps
          // that lag from building up on one side from item to item.
          if (!pp.pair_heads && (seq & 1)) {
            const TileInfo t0 = it.tile[0];
            it.tile[0] = it.tile[1];
            it.tile[1] = t0;
          }
        }
        if (leader) {
          if (item < pp.total_items) publish_item(mailbox + slot * kItemWords, item, it);
          else mailbox[slot * kItemWords] = item;   // end marker
          mbar_arrive(bar_sched_full + 8 * slot);
        }
        if (item >= pp.total_items) break;
#if AIDN_PREFILL_TRACE
        unsigned long long* ptrace = pp.debug_mode == 2
            ? reinterpret_cast<unsigned long long*>(pp.debug) + (size_t)item * 16 : nullptr;
        if (ptrace && leader) ptrace[6] = globaltimer_ns();
#else
        unsigned long long* const ptrace = nullptr;
#endif
        auto load_tile = [&](const CUtensorMap* tm, uint32_t dst, uint32_t bar, int row, int head) {
          if (leader) {
            mbar_expect_tx(bar, (uint32_t)C::kTileBytes);
#pragma unroll
            for (int hf = 0; hf < C::kHalves; ++hf)
              tma_load_4d(dst + hf * C::kHalfBytes, tm, bar, hf * 64, row, head, it.b);
          }
        };
        auto load_q = [&](int i) {
          if (it.tile[i].n == 0 || pp.debug_mode == 3) return;
          if (!mbar_wait(bar_q_empty + 8 * i, (q_uses[i] & 1u) ^ 1u, abort_flag, wait_ns)) { alive = false; return; }
          load_tile(&tm_q, q_smem + i * C::kTileBytes, bar_q_full + 8 * i, it.tile[i].t * kBM, it.tile[i].h);
          ++q_uses[i];
        };
        // Paged K/V: a sub-tile of 64 keys is 64 / block_size pool blocks, each fetched by its own TMA box (block_size
        // rows) into its slice of the ring slot - the 128-byte swizzle is a function of the shared-memory address, so
        // the slices compose into the same image as one 64-row box - or, with 128-token blocks, half of one block.
        // Lane i holds the pool block of slice i.
        const bool paged = p.block_table != nullptr;
        int64_t last_blk = 0;
        if (paged) last_blk = (kv_limit_of(p, it.b) - 1) >> p.block_shift;
        auto load_kv = [&](const CUtensorMap* tm, int key_sub) {
          const int s = (int)(t_load % C::kStages);
          const uint32_t phase = (t_load / C::kStages) & 1u;
          if (!mbar_wait(bar_kv_empty + 8 * s, phase ^ 1u, abort_flag, wait_ns)) { alive = false; return; }
          const uint32_t dst = kv_smem + s * C::kSubBytes, bar = bar_kv_full + 8 * s;
          if (leader) mbar_expect_tx(bar, (uint32_t)C::kSubBytes);
          if (!paged) {
            if (leader) {
#pragma unroll
              for (int hf = 0; hf < C::kHalves; ++hf)
                tma_load_4d(dst + hf * C::kKvHalfBytes, tm, bar, hf * 64, key_sub * kBS, it.kvh, it.b);
            }
          } else {
            const int rows = p.block_size < kBS ? p.block_size : kBS;   // rows per box
            const int parts = kBS / rows;
            // Logical blocks past the sequence's last one repeat it: their keys are masked and the table has no
            // entry for them (the V rows among them are cleared before use, the K rows only feed masked scores).
            const int64_t key = (int64_t)key_sub * kBS + (int64_t)lane * rows;
            int64_t lb = key >> p.block_shift;
            if (lb > last_blk) lb = last_blk;
            int32_t blk = 0;
            if (lane < parts) {
              blk = __ldg(p.block_table + (int64_t)it.b * p.bt_stride + lb);
              if ((blk < 0 || blk >= p.num_blocks) && p.status) atomicOr(p.status, kStatusBadBlock);
            }
            const int in_block = (int)(((int64_t)key_sub * kBS) & (int64_t)(p.block_size - 1));   // non-zero only for 128-token blocks
            for (int part = 0; part < parts; ++part) {
              // an entry outside the pool gives an out-of-range coordinate, which TMA fills with zeros
              const int32_t phys = __shfl_sync(0xffffffffu, blk, part);
              if (leader) {
#pragma unroll
                for (int hf = 0; hf < C::kHalves; ++hf)
                  tma_load_4d(dst + hf * C::kKvHalfBytes + part * (rows * 128), tm, bar, hf * 64,
                              phys * p.block_size + (parts == 1 ? in_block : 0), it.kvh, 0);
              }
            }
          }
          ++t_load;
        };
        // Ring order of an item with n sub-tiles: K(0), then K(u+1), V(u) for u = 0 .. n-2, then V(n-1) - the order in
        // which the issuers need them (the score product runs two sub-tiles ahead of the P.V product).
        const int n_sub = it.n_max;
        if (n_sub > 0) {
          load_q(0);
          if (alive) load_kv(&tm_k, 0);
          if (ptrace && leader) ptrace[0] = globaltimer_ns();
          if (alive) load_q(1);
          for (int u = 0; u < n_sub && alive; ++u) {
            if (u + 1 < n_sub) load_kv(&tm_k, u + 1);
            if (alive) load_kv(&tm_v, u);
          }
        }
        {
          int next = 0;
          if (leader) next = atomicAdd(pp.sched, 1) + (int)gridDim.x;
          item = __shfl_sync(0xffffffffu, next, 0);   // elect.sync picks the lowest lane of the full warp
        }
      }
    }
  } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
    // ========================================== UMMA issuers ==========================================
    // Two issuer warps.  Issuer b owns score buffer b of BOTH query tiles, i.e. the sub-tiles u with (u & 1) == b:
    // in its turn it issues P_0(u).V, Q_0.K(u+2)^T, P_1(u).V, Q_1.K(u+2)^T - 24 UMMAs, about 1300 cycles of tensor
    // pipe - and then spends several hundred cycles on hand-offs (barrier tests, commits, the next turn's waits;
    // tcgen05.mma issue blocks once a few instructions are queued, and an issuer shares its scheduler with two busy
    // softmax warps).  The turns of the two issuers alternate, so one issuer's hand-offs run under the other's
    // burst.  Measured alternatives: one issuer for everything (its hand-offs, 530 cycles per tile and sub-tile, sat
    // between the bursts and idled the pipe half of the time) and one issuer per query tile (bursts of 12 UMMAs are
    // shorter than the hand-offs between them).
    // A counter in shared memory orders the turns (prologue of issuer 0, prologue of issuer 1, then sub-tile 0, 1,
    // 2, ... of the item); it is what guarantees that the first P.V of a tile, which overwrites O, is queued before
    // the second one, which accumulates.
    // Each warp runs its role in lockstep and only the tcgen05 instructions themselves are issued by one elected
    // lane: descriptors and addresses then stay warp-uniform (uniform registers), which a branch on lane == 0
    // around the role would prevent - every UMMA would first move its operands lane -> uniform.
    {
      const int b = warp - kMmaWarp;            // buffer / sub-tile parity owned by this issuer
      const bool leader = elect_one();
      constexpr uint32_t idesc_qk = make_idesc(kBM, kBS, kBf16, false);
      constexpr uint32_t idesc_pv = make_idesc(kBM, HD, kBf16, true);
      const uint32_t t_sc = tmem_base + (uint32_t)(b * kBS);            // S_0[b]; S_1[b] is 128 columns on
      const uint32_t t_acc = tmem_base + (uint32_t)C::kOCol;            // O_0; O_1 is HD columns on
      const uint64_t qdesc = make_smem_desc(q_smem, 16, 1024);          // Q_0; Q_1 is one tile on
      constexpr uint64_t kQTile = (uint64_t)(C::kTileBytes >> 4);
      volatile int* turn = issue_turn;
      bool alive = true;
      uint32_t t_cons = 0;            // K/V sub-tiles of earlier items (ring position)
      uint32_t q_par = 0;             // bit i: parity of the next phase of q_full[i]
      uint32_t p_par = 0;             // bit i: parity of the next phase of p_full[i][b]
      uint32_t oe_par = 3;            // bit i: parity to test on o_empty[i] before the tile's next first P.V product
      int g = 0;                      // turns of earlier items
      for (int seq = 0; alive; ++seq) {
        int item;
        {
          const int slot = seq & 1;
          if (!mbar_wait(bar_sched_full + 8 * slot, (uint32_t)((seq >> 1) & 1), abort_flag, wait_ns)) break;
          item = mailbox[slot * kItemWords];
        }
        if (item >= pp.total_items) break;
        const Item it = read_item(mailbox + (seq & 1) * kItemWords);
        __syncwarp();
        if (leader) mbar_arrive(bar_sched_empty + 8 * (seq & 1));
#if AIDN_PREFILL_TRACE
        unsigned long long* mtrace = (pp.debug_mode == 2 && b == 0)
            ? reinterpret_cast<unsigned long long*>(pp.debug) + (size_t)item * 16 : nullptr;
        if (mtrace && leader) mtrace[7] = globaltimer_ns();
        long long* msteps = ((pp.debug_mode == 4 || pp.debug_mode == 6) && blockIdx.x == 0 && seq < 8 && leader)
            ? reinterpret_cast<long long*>(pp.debug) + (size_t)seq * 32 * 16 + 10 : nullptr;
#define MMA_STAMP(j, slot) do { if (msteps && (j) < 32) msteps[(j) * 16 + (slot)] = clock64(); } while (0)
        // mode 6: the issuers' own phases in slots 5..9 of their sub-tiles (the tile-1 softmax columns are not written then)
        long long* dsteps = (pp.debug_mode == 6 && blockIdx.x == 0 && seq < 8 && leader)
            ? reinterpret_cast<long long*>(pp.debug) + (size_t)seq * 32 * 16 + 5 : nullptr;
#define DET_STAMP(j, slot) do { if (dsteps && (j) < 32) dsteps[(j) * 16 + (slot)] = clock64(); } while (0)
#else
        unsigned long long* const mtrace = nullptr;
#define MMA_STAMP(j, slot) do { } while (0)
#define DET_STAMP(j, slot) do { } while (0)
#endif
        const int n_max = it.n_max;
        if (n_max == 0) continue;
        const int n0 = it.tile[0].n, n1 = it.tile[1].n;
        // ring positions of the item's sub-tiles (the producer's order): K(0) at t0, K(s) at t0 + 2s - 1,
        // V(u) at t0 + 2u + 2 except the last one, which follows K(n_max - 1) directly
        const uint32_t t0 = t_cons;
        t_cons = t0 + 2 * (uint32_t)n_max;
        auto pos_k = [&](int sub) { return t0 + (uint32_t)(sub == 0 ? 0 : 2 * sub - 1); };
        auto pos_v = [&](int sub) { return t0 + (uint32_t)(sub + 1 < n_max ? 2 * sub + 2 : 2 * n_max - 1); };
        const int g0 = g;             // turn g0: prologue of issuer 0, g0 + 1: of issuer 1, g0 + 2 + u: sub-tile u
        g = g0 + 2 + n_max;
        auto kv_slot = [&](uint32_t t) { return (int)(t % C::kStages); };
        auto kv_wait = [&](uint32_t t) {
          const int s = kv_slot(t);
          if (!mbar_wait(bar_kv_full + 8 * s, (t / C::kStages) & 1u, abort_flag, wait_ns)) alive = false;
          return kv_smem + s * C::kSubBytes;
        };
        // the slot may be refilled when the products this warp has issued so far have read it
        auto kv_release = [&](uint32_t t) { if (leader) tc_commit(bar_kv_empty + 8 * kv_slot(t)); };
        auto wait_turn = [&](int my) {
          uint32_t spins = 0;
          while (*turn < my) {
            if ((++spins & 63u) == 0u && (*abort_flag || spins > (1u << 22))) { alive = false; break; }
          }
        };
        auto pass_turn = [&](int my) { if (leader) *turn = my + 1; };
        // S_i[b] = Q_i . K(sub-tile s)^T, s & 1 == b; kaddr is the ring slot that holds the sub-tile
        auto issue_qk = [&](int i, int s, uint32_t kaddr, int n_i, int pass_my) {
          const uint64_t kdesc = make_smem_desc(kaddr, 16, 1024);
          const uint64_t qd = qdesc + (uint64_t)i * kQTile;
          const uint32_t d = t_sc + (uint32_t)(i * 2 * kBS);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            // 16 head-dim elements = 32 bytes inside the 128-byte swizzle row; 64 elements on, the next column block
            const uint64_t qoff = (uint64_t)((kk >> 2) * (C::kHalfBytes >> 4) + (kk & 3) * 2);
            const uint64_t koff = (uint64_t)((kk >> 2) * (C::kKvHalfBytes >> 4) + (kk & 3) * 2);
            if (leader) mma_ss(d, qd + qoff, kdesc + koff, idesc_qk, kk > 0 ? 1u : 0u);
            // The turn goes on while the last few UMMAs of the burst are still to be queued: the other issuer needs
            // about that long to notice, and the tensor pipe has this burst's tail to run in the meantime.
            if (pass_my >= 0 && kk == HD / 16 - 4) pass_turn(pass_my);
          }
          if (leader) {
            tc_commit(bar_s_full + 8 * (2 * i + b));
            // this issuer's last score product of the tile: its half of "the Q tile may be overwritten"
            if (s + 2 >= n_i) tc_commit(bar_q_empty + 8 * i);
          }
        };
        // O_i (+)= P_i[b] . V(sub-tile u)
        auto issue_pv = [&](int i, int u, uint32_t vaddr) {
          const uint64_t vdesc = make_smem_desc(vaddr, C::kKvHalfBytes, 1024);
          const uint32_t a = t_sc + (uint32_t)(i * 2 * kBS);
          const uint32_t d = t_acc + (uint32_t)(i * HD);
#pragma unroll
          for (int kk = 0; kk < kBS / 16; ++kk)
            if (leader) mma_ts(d, a + (uint32_t)(kk * 8), vdesc + (uint64_t)(kk * (2048 >> 4)), idesc_pv, (u > 0 || kk > 0) ? 1u : 0u);
        };

        // ---- prologue turn: score sub-tile b of both query tiles ----
        {
          uint32_t kaddr0 = 0;
          if (b < n_max) kaddr0 = kv_wait(pos_k(b));
          if (mtrace && leader) mtrace[14] = globaltimer_ns();
          for (int i = 0; i < 2 && alive; ++i) {
            const int n_i = i ? n1 : n0;
            if (n_i == 0) continue;
            if (!mbar_wait(bar_q_full + 8 * i, (q_par >> i) & 1u, abort_flag, wait_ns)) { alive = false; break; }
            q_par ^= 1u << i;
          }
          if (!alive) break;
          if (mtrace && leader) mtrace[8] = globaltimer_ns();
          tc_fence_after();
          wait_turn(g0 + b);
          if (!alive) break;
          for (int i = 0; i < 2; ++i) {
            const int n_i = i ? n1 : n0;
            if (n_i > b) issue_qk(i, b, kaddr0, n_i, -1);
            else if (n_i > 0 && leader) tc_commit(bar_q_empty + 8 * i);   // a single sub-tile: issuer 1 never reads this Q tile
          }
          pass_turn(g0 + b);
          if (b < n_max) kv_release(pos_k(b));
        }

        // ---- this issuer's sub-tiles ----
        for (int u = b; u < n_max && alive; u += 2) {
          const uint32_t tv = pos_v(u), tk = pos_k(u + 2);
          const bool have_k = u + 2 < n_max;   // K(u + 2) exists (one of the query tiles needs its scores)
          DET_STAMP(u, 0);
          const uint32_t vaddr = kv_wait(tv);
          uint32_t knext = 0;
          if (have_k && alive) knext = kv_wait(tk);
          if (!alive) break;
          if (it.v_tail > 0 && u + 1 == n_max) {
            // clear the rows of the item's last V sub-tile that lie past the sequence's last key (see decode_item)
            const int chunks = (kBS - it.v_tail) * 8;   // 16-byte chunks per 64-column block
#pragma unroll
            for (int hf = 0; hf < C::kHalves; ++hf)
              for (int c = lane; c < chunks; c += 32)
                st_shared_v4(vaddr + (uint32_t)(hf * C::kKvHalfBytes + it.v_tail * 128 + c * 16), 0u, 0u, 0u, 0u);
            fence_proxy_async_smem();
            __syncwarp();
          }
          bool turn_mine = false;
          DET_STAMP(u, 1);
          for (int i = 0; i < 2 && alive; ++i) {
            const int n_i = i ? n1 : n0;
            if (u >= n_i) continue;
            if (!mbar_wait(bar_p_full + 8 * (2 * i + b), (p_par >> i) & 1u, abort_flag, wait_ns)) { alive = false; break; }
            p_par ^= 1u << i;
            if (EPI && u == 0) {
              // this product overwrites O_i: the epilogue warps must have read the previous item's out of TMEM
              if (!mbar_wait(bar_o_empty + 8 * i, (oe_par >> i) & 1u, abort_flag, wait_ns)) { alive = false; break; }
              oe_par ^= 1u << i;
            }
            tc_fence_after();
            if (!turn_mine) {
              DET_STAMP(u, 2);
              wait_turn(g0 + 2 + u);
              if (!alive) break;
              turn_mine = true;
              DET_STAMP(u, 3);
            }
            MMA_STAMP(u, 2 * i);
            issue_pv(i, u, vaddr);
            // the last tile of the burst hands the turn on from inside its score product, or right here without one
            const bool last_of_burst = i == 1 || u >= n1;
            if (u + 2 < n_i) {
              issue_qk(i, u + 2, knext, n_i, last_of_burst ? g0 + 2 + u : -1);
            } else {
              if (last_of_burst) pass_turn(g0 + 2 + u);
              if (leader) {
                // No further score product of this issuer will signal this P.V.  The second-to-last one of the tile
                // is signalled for a late O rescale and for the epilogue, the last one hands O to the epilogue.
                if (u + 2 == n_i) tc_commit(bar_pv_done + 8 * i);
                else tc_commit(bar_o_full + 8 * i);
              }
            }
            MMA_STAMP(u, 2 * i + 1);
          }
          if (!alive) break;
          kv_release(tv);
          if (have_k) kv_release(tk);
          DET_STAMP(u, 4);
        }
      }
    }
  }

  if constexpr (EPI) {
    if (warp >= kEpilogueWarp) {
      // ============================================ epilogue ============================================
      // O_i / l -> staging -> TMA stores, off the softmax warps' path: the first P.V product of the next item (which
      // overwrites O_i) waits for o_empty[i], i.e. only for the tcgen05.ld's of the tile, not for the stores.
      const int quarter = warp - kEpilogueWarp;
      const int row_in_tile = quarter * 32 + lane;
      const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
      const uint32_t my_stage = stage_smem + (uint32_t)(quarter * 2 * 4096);
      uint32_t st_par = 0;               // bit i: parity of the next phase of stats_full[i]
      uint32_t of_par = 0;               // bit i: parity of the next phase of o_full[i]
      uint32_t pv_par = 0;               // bit i: parity of the next phase of pv_done[i]
      uint32_t n_stores = 0;             // TMA stores issued by this warp
      bool alive = true;
      for (int seq = 0; alive; ++seq) {
        int item;
        {
          const int slot = seq & 1;
          bool ok = mbar_wait(bar_sched_full + 8 * slot, (uint32_t)((seq >> 1) & 1), abort_flag, wait_ns);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          item = mailbox[slot * kItemWords];
        }
        if (item >= pp.total_items) break;
        const Item it = read_item(mailbox + (seq & 1) * kItemWords);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sched_empty + 8 * (seq & 1));
#if AIDN_PREFILL_TRACE
        unsigned long long* trace = pp.debug_mode == 2
            ? reinterpret_cast<unsigned long long*>(pp.debug) + (size_t)item * 16 : nullptr;
        const bool tracer = trace && row_in_tile == 0;
#else
        constexpr bool tracer = false;
        unsigned long long* const trace = nullptr;
#endif
        for (int i = 0; i < 2 && alive; ++i) {
          const TileInfo ti = it.tile[i];
          if (!ti.valid) continue;
          bool ok = mbar_wait(bar_stats_full + 8 * i, (st_par >> i) & 1u, abort_flag, wait_ns);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) { alive = false; break; }
          st_par ^= 1u << i;
          const float inv = stats[i * kBM + row_in_tile];
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_stats_empty + 8 * i);
          const bool have_o = ti.n > 0;
          if (have_o) {
            // the last two P.V products were issued by different warps: pv_done covers the second-to-last one
            if (ti.n >= 2) {
              ok = mbar_wait(bar_pv_done + 8 * i, (pv_par >> i) & 1u, abort_flag, wait_ns);
              pv_par ^= 1u << i;
            }
            ok = ok && mbar_wait(bar_o_full + 8 * i, (of_par >> i) & 1u, abort_flag, wait_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { alive = false; break; }
            of_par ^= 1u << i;
            tc_fence_after();
          }
          if (tracer) trace[4 + 8 * i] = globaltimer_ns();
          store_o_tile<HD, kBf16>(p, &tm_o, pm, tmem_base + lane_bits + (uint32_t)(C::kOCol + i * HD), have_o, inv, my_stage,
                                     n_stores, lane, ti.t * kBM + quarter * 32, ti.h, it.b, bar_o_empty + 8 * i);
          if (tracer) trace[5 + 8 * i] = globaltimer_ns();
        }
      }
      // staging memory must outlive the bulk stores that read it
      if (lane == 0) bulk_wait_all();
      __syncwarp();
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
  if (threadIdx.x == 0) {
    // The last CTA to get here puts both scheduler counters back to zero for the next launch.
    __threadfence();
    const int done = atomicAdd(pp.sched + 1, 1);
    if (done == (int)gridDim.x - 1) {
      pp.sched[0] = 0;
      pp.sched[1] = 0;
      __threadfence();
    }
  }
#if AIDN_PREFILL_TRACE
  if (pp.debug_mode == 7 && threadIdx.x == 0) {
    unsigned long long* cl = reinterpret_cast<unsigned long long*>(pp.debug) + 4 * blockIdx.x;
    cl[2] = (unsigned long long)clock64();
    cl[3] = globaltimer_ns();
  }
#endif
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side -----------------------------------------------------------------------------------------

using tmap::encode_bhsd;
using tmap::resolve_encode;

// Base address and (B, H, S) strides must be multiples of `align` bytes.
bool aligned_bhs(const void* base, const int64_t* stride, int64_t H, int64_t B, int esz, int align) {
  if ((uintptr_t)base % align != 0) return false;
  if ((stride[2] * esz) % align != 0 || stride[2] <= 0) return false;
  if (H > 1 && ((stride[1] * esz) % align != 0 || stride[1] <= 0)) return false;
  if (B > 1 && ((stride[0] * esz) % align != 0 || stride[0] <= 0)) return false;
  return true;
}

template <typename T, int HD, bool MASKED, bool EPI>
cudaError_t launch_e(const SdpaParams& p, cudaStream_t stream, int32_t* sched, int num_sms, float* debug,
                     int debug_mode, PrefillMapCache* cache, const char** why) {
  using C = Cfg<HD>;
  constexpr bool bf16 = !std::is_same_v<T, __half>;
  // Paged pools are one "sequence" of num_blocks * block_size rows, fetched one block (box of block_size rows) at a time.
  const int64_t kv_rows = p.block_table ? (int64_t)p.num_blocks * p.block_size : p.seq_kv;
  const int kv_batch = p.block_table ? 1 : p.batch;
  const int kv_box = p.block_table ? (p.block_size < kBS ? p.block_size : kBS) : kBS;
  PrefillMapCache local;
  PrefillMapCache* mc = cache ? cache : &local;
  if (!cache) {
    local.valid = false;
    std::memset(local.attr_set, 0, sizeof(local.attr_set));
  }
  PrefillMapCache::Key key;
  std::memset(&key, 0, sizeof(key));
  key.q = p.q; key.k = p.k; key.v = p.v; key.out = p.out;
  for (int i = 0; i < 3; ++i) { key.qs[i] = p.qs[i]; key.ks[i] = p.ks[i]; key.vs[i] = p.vs[i]; key.os[i] = p.os[i]; }
  key.seq_q = p.seq_q; key.kv_rows = kv_rows;
  key.batch = p.batch; key.kv_batch = kv_batch; key.num_q_heads = p.num_q_heads; key.num_kv_heads = p.num_kv_heads;
  key.head_dim = HD; key.kv_box = kv_box; key.out_f32 = p.out_f32; key.dtype = bf16 ? AIDN_BF16 : AIDN_F16;
  CUtensorMap* tq = reinterpret_cast<CUtensorMap*>(mc->maps[0]);
  CUtensorMap* tk = reinterpret_cast<CUtensorMap*>(mc->maps[1]);
  CUtensorMap* tv = reinterpret_cast<CUtensorMap*>(mc->maps[2]);
  CUtensorMap* to = reinterpret_cast<CUtensorMap*>(mc->maps[3]);
  cudaError_t e = cudaSuccess;
  if (!mc->valid || std::memcmp(&mc->key, &key, sizeof(key)) != 0) {
    mc->valid = false;
    e = resolve_encode();
    if (e != cudaSuccess) { *why = "cuTensorMapEncodeTiled is not available from the driver"; return e; }
    const CUtensorMapDataType dt16 = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUtensorMapSwizzle s128 = CU_TENSOR_MAP_SWIZZLE_128B;
    // output boxes are 128 bytes x 32 rows: 32 fp32 or 64 16-bit columns
    const bool ok_o = p.out_f32
        ? encode_bhsd(to, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, s128, p.out, HD, p.seq_q, p.num_q_heads, p.batch, p.os, 32, 32)
        : encode_bhsd(to, dt16, 2, s128, p.out, HD, p.seq_q, p.num_q_heads, p.batch, p.os, 64, 32);
    if (!encode_bhsd(tq, dt16, 2, s128, p.q, HD, p.seq_q, p.num_q_heads, p.batch, p.qs, 64, kBM) ||
        !encode_bhsd(tk, dt16, 2, s128, p.k, HD, kv_rows, p.num_kv_heads, kv_batch, p.ks, 64, kv_box) ||
        !encode_bhsd(tv, dt16, 2, s128, p.v, HD, kv_rows, p.num_kv_heads, kv_batch, p.vs, 64, kv_box) || !ok_o) {
      *why = "cuTensorMapEncodeTiled rejected a tensor (address or stride alignment)";
      return cudaErrorInvalidValue;
    }
    mc->key = key;
    mc->valid = true;
  }
  // Fused gather: the same box geometry over the other devices' output tensors.  (Encoded per launch: a handful of
  // microseconds against a launch that is long enough to be sharded.)
  PeerMaps pm;
  std::memset(&pm, 0, sizeof(pm));
  pm.count = p.peer_count;
  for (int r = 0; r < p.peer_count; ++r) {
    const CUtensorMapDataType dt16 = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!aligned_bhs(p.peer_out[r], p.os, p.num_q_heads, p.batch, p.out_f32 ? 4 : 2, 16)) {
      *why = "peer_out must be 16-byte aligned like out";
      return cudaErrorInvalidValue;
    }
    e = resolve_encode();
    if (e != cudaSuccess) { *why = "cuTensorMapEncodeTiled is not available from the driver"; return e; }
    const bool ok = p.out_f32
        ? encode_bhsd(&pm.maps[r], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, CU_TENSOR_MAP_SWIZZLE_128B, p.peer_out[r], HD, p.seq_q,
                      p.num_q_heads, p.batch, p.os, 32, 32)
        : encode_bhsd(&pm.maps[r], dt16, 2, CU_TENSOR_MAP_SWIZZLE_128B, p.peer_out[r], HD, p.seq_q, p.num_q_heads, p.batch,
                      p.os, 64, 32);
    if (!ok) { *why = "cuTensorMapEncodeTiled rejected a peer output tensor"; return cudaErrorInvalidValue; }
  }
  PrefillParams pp;
  pp.p = p;
#if AIDN_PREFILL_TRACE
  pp.debug = debug;
  pp.debug_mode = (debug || debug_mode == 3) ? debug_mode : 0;
#else
  pp.debug = nullptr;
  pp.debug_mode = debug_mode == 3 ? 3 : 0;
#endif
  pp.wait_budget_ns = debug_mode == 3 ? 20000000ull : kWaitBudgetNs;   // 20 ms in the time-out test
  pp.sched = sched;
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
  if (total <= 0 || total > 0x3fffffff) { *why = "work item count out of range"; return cudaErrorInvalidValue; }
  pp.total_items = (int)total;
  auto kern = sdpa_prefill_sm100_kernel<T, HD, MASKED, EPI>;
  constexpr int inst = (EPI ? 8 : 0) + (bf16 ? 0 : 4) + (HD == 128 ? 2 : 0) + (MASKED ? 1 : 0);
  if (!mc->attr_set[inst]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) { *why = "cannot raise the dynamic shared memory limit"; return e; }
    mc->attr_set[inst] = true;
  }
  const unsigned grid = (unsigned)(total < num_sms ? total : num_sms);
  kern<<<grid, Roles<EPI>::kThreads, C::kSmemBytes, stream>>>(*tq, *tk, *tv, *to, pm, pp);
  return cudaGetLastError();
}

}  // namespace

bool prefill_sm100_supported(const SdpaParams& p, int dtype, const char** why) {
  if (dtype != AIDN_BF16 && dtype != AIDN_F16) { *why = "tcgen05 prefill takes fp16 or bf16 inputs"; return false; }
  if (p.head_dim != 64 && p.head_dim != 128) { *why = "tcgen05 prefill takes head_dim 64 or 128"; return false; }
  const int kv_batch = p.block_table ? 1 : p.batch;
  if (p.block_table) {
    if (p.block_shift < 3 || p.block_size > 128) {
      *why = "tcgen05 prefill reads paged K/V in blocks of 8, 16, 32, 64 or 128 tokens";
      return false;
    }
    if (p.num_blocks <= 0 || (int64_t)p.num_blocks * p.block_size > 0x7fffff00ll) {
      *why = "tcgen05 prefill needs aidn_paged_kv.num_blocks (pool rows below 2^31)";
      return false;
    }
  }
  if (!aligned_bhs(p.q, p.qs, p.num_q_heads, p.batch, 2, 16) || !aligned_bhs(p.k, p.ks, p.num_kv_heads, kv_batch, 2, 16) ||
      !aligned_bhs(p.v, p.vs, p.num_kv_heads, kv_batch, 2, 16)) {
    *why = "Q/K/V base must be 16-byte aligned and strides multiples of 8 elements for TMA";
    return false;
  }
  if (!aligned_bhs(p.out, p.os, p.num_q_heads, p.batch, p.out_f32 ? 4 : 2, 16)) {
    *why = "output base and strides must be 16-byte aligned for TMA";
    return false;
  }
  if (p.seq_q > 0x7fffff00ll || p.seq_kv > 0x7fffff00ll) { *why = "sequence too long"; return false; }
  return true;
}

// The epilogue warpgroup pays when both tiles of an item end together: head pairs, or row pairs without a causal mask.
template <typename T, int HD, bool MASKED>
cudaError_t launch_t(const SdpaParams& p, cudaStream_t stream, int32_t* sched, int num_sms, float* debug,
                     int debug_mode, PrefillMapCache* cache, const char** why) {
  const bool epi = (p.group % 2 == 0) || !p.causal;
  if (epi) return launch_e<T, HD, MASKED, true>(p, stream, sched, num_sms, debug, debug_mode, cache, why);
  return launch_e<T, HD, MASKED, false>(p, stream, sched, num_sms, debug, debug_mode, cache, why);
}

template <typename T, int HD>
cudaError_t launch_m(const SdpaParams& p, cudaStream_t stream, int32_t* sched, int num_sms, float* debug, int debug_mode,
                     PrefillMapCache* cache, const char** why) {
  if (p.mask_kind != AIDN_MASK_NONE || p.softcap > 0.f)
    return launch_t<T, HD, true>(p, stream, sched, num_sms, debug, debug_mode, cache, why);
  return launch_t<T, HD, false>(p, stream, sched, num_sms, debug, debug_mode, cache, why);
}

cudaError_t launch_prefill_sm100(const SdpaParams& p, int dtype, cudaStream_t stream, int32_t* sched, int num_sms,
                                 float* debug, int debug_mode, PrefillMapCache* cache, const char** why) {
  if (dtype == AIDN_BF16) {
    if (p.head_dim == 128) return launch_m<__nv_bfloat16, 128>(p, stream, sched, num_sms, debug, debug_mode, cache, why);
    return launch_m<__nv_bfloat16, 64>(p, stream, sched, num_sms, debug, debug_mode, cache, why);
  }
  if (p.head_dim == 128) return launch_m<__half, 128>(p, stream, sched, num_sms, debug, debug_mode, cache, why);
  return launch_m<__half, 64>(p, stream, sched, num_sms, debug, debug_mode, cache, why);
}

}  // namespace aidn
