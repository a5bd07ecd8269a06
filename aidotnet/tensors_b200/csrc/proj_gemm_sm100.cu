// Projection GEMM of the fused multi-head-attention forward for sm_100a:  C[b, s, n] = sum_k A[b, s, k] * W[k, n]
// with 16-bit A and W, fp32 accumulation in TMEM, and an epilogue that writes each head's columns straight into the
// layout the next stage reads - Q / K / V as [B, H, S, d] in 16 bits (no permute or cast pass after the GEMM), the
// output projection as [B, S, H*d] in fp32 or 16 bits.  One launch serves up to three weight matrices that share A
// (the Q, K and V projections), selected by the column-tile index.
//
//   warp 0      TMA producer: per 64-wide K block one A box (128 rows x 64) and BN/64 W boxes (64 x 64), 128-byte
//               swizzle, through a ring of 4 shared-memory stages
//   warp 1      UMMA issuer (one elected lane): tcgen05.mma 128 x BN x 16, A K-major from shared memory, W as the
//               MN-major B operand (rows of W are K, so the row-major weight needs no transpose); owns TMEM
//   warps 2-5   epilogue: TMEM -> registers -> swizzled 128-byte staging rows -> TMA stores clipped at the sequence end
//
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of one tile runs under the main loop of
// the next.  CTAs are persistent and walk the tiles in a fixed order, grouped so that the tiles in flight share a
// block of A rows and a block of weight columns that fit in L2 together.  Every wait is bounded; a CTA that gives up sets the
// time-out bit of the status word and leaves through the common teardown.
//
// Replaces, for the engine's MultiHeadAttentionForward (src/AiDotNet.Tensors/Engines/CpuEngine.MultiHeadAttention.cs:155-338:
// Sgemm + scatter into [B, heads, seq, dHead]; DirectGpuTensorEngine.MissingKernels.cs:5793-5870: three MatMuls +
// ReshapePermuteHeads, and the PermuteResidentGpu + MatMul of the output projection), the GEMM, permute and cast passes.
#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tensor_map.hpp"

namespace aidn {
namespace {

using namespace ptx;

constexpr int kBM = 128;       // rows (sequence positions) per tile
constexpr int kBK = 64;        // K elements per stage: one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kThreads = 192;  // producer, issuer, 4 epilogue warps
constexpr int kEpiBytesPerWarp = 4096;   // 32 rows x 128 B

template <int BN>
struct GCfg {
  static constexpr int kABytes = kBM * kBK * 2;   // 16 KiB
  static constexpr int kBBlock = kBK * 128;       // one 64-column block of W: 64 rows x 128 B
  static constexpr int kBBytes = (BN / 64) * kBBlock;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOff = kStages * kStageBytes;
  static constexpr int kBarOff = kEpiOff + 4 * kEpiBytesPerWarp;
  static constexpr int kNumBars = 2 * kStages + 4;   // full[S] empty[S] acc_full[2] acc_empty[2]
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kSmemBytes = kMiscOff + 16 + 1024 /*align slack*/;
  static constexpr int kTmemCols = 2 * BN;
};

struct GemmMaps {
  CUtensorMap a;      // A as (K, S, 1, B), box 64 x 128
  CUtensorMap w[3];   // W as (N, K, 1, 1), box 64 x 64
  CUtensorMap c[3];   // C as (d, S, H, B), box 64 (16-bit) or 32 (fp32) x 32
};

struct GemmParams {
  int32_t row_tiles_per_batch;   // ceil(seq / 128)
  int32_t row_tiles;             // batch * row_tiles_per_batch
  int32_t col_tiles_per_mat;     // n / BN
  int32_t col_tiles;             // col_tiles_per_mat * number of weight matrices
  int32_t total_tiles;
  int32_t k_blocks;              // ceil(k / 64)
  int32_t seq;
  int32_t head_dim;
  int32_t out_f32;
  int32_t* status;
  int32_t withhold_loads;        // test hook: the producer issues no loads, so that the bounded waits run out
  uint64_t wait_budget_ns;
};

struct Tile {
  int b, s0, mat, n0;
};

// Tile order: groups of kGroupRows row tiles; inside a group the row tile runs fastest, then the column tile.  The
// 148 tiles in flight then cover 16 row tiles x 9 column tiles (16 MB of A + 18 MB of W) instead of every row tile
// against two weight panels, and the A rows of a group stay in L2 while the group walks across the weights.
constexpr int kGroupRows = 16;

__device__ __forceinline__ Tile decode_tile(const GemmParams& gp, int tile, int bn) {
  Tile t;
  const int per_group = kGroupRows * gp.col_tiles;
  const int grp = tile / per_group, within = tile - grp * per_group;
  const int rows_left = gp.row_tiles - grp * kGroupRows;
  const int rows_here = rows_left < kGroupRows ? rows_left : kGroupRows;
  const int ct = within / rows_here;
  const int rt = grp * kGroupRows + (within - ct * rows_here);
  t.b = rt / gp.row_tiles_per_batch;
  t.s0 = (rt - t.b * gp.row_tiles_per_batch) * kBM;
  t.mat = ct / gp.col_tiles_per_mat;
  t.n0 = (ct - t.mat * gp.col_tiles_per_mat) * bn;
  return t;
}

template <int BN, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
    proj_gemm_sm100_kernel(const __grid_constant__ GemmMaps maps, const GemmParams gp) {
  using C = GCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t epi_smem = smem_base + C::kEpiOff;
  const uint32_t bars = smem_base + C::kBarOff;
  const uint32_t bar_full = bars;                          // [kStages]
  const uint32_t bar_empty = bars + 8 * kStages;           // [kStages]
  const uint32_t bar_acc_full = bars + 16 * kStages;       // [2]
  const uint32_t bar_acc_empty = bar_acc_full + 16;        // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_gen + C::kMiscOff + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + C::kMiscOff + 12);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t wait_ns = gp.wait_budget_ns;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_acc_full + 8 * i, 1);
      mbar_init(bar_acc_empty + 8 * i, 4);   // one arrival per epilogue warp
    }
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&maps.a);
    prefetch_tensormap(&maps.w[0]);
    prefetch_tensormap(&maps.c[0]);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ============================================ TMA producer ============================================
    const bool leader = elect_one();
    uint32_t kb_total = 0;   // K blocks loaded so far (ring position)
    bool alive = true;
    for (int tile = blockIdx.x; tile < gp.total_tiles && alive; tile += gridDim.x) {
      const Tile t = decode_tile(gp, tile, BN);
      const CUtensorMap* tw = &maps.w[t.mat];
      for (int kb = 0; kb < gp.k_blocks; ++kb, ++kb_total) {
        const int s = (int)(kb_total % kStages);
        const uint32_t phase = (kb_total / kStages) & 1u;
        if (!mbar_wait(bar_empty + 8 * s, phase ^ 1u, abort_flag, wait_ns)) { alive = false; break; }
        if (leader && !gp.withhold_loads) {
          const uint32_t bar = bar_full + 8 * s;
          const uint32_t a_dst = smem_base + s * C::kStageBytes;
          const uint32_t b_dst = a_dst + C::kABytes;
          mbar_expect_tx(bar, (uint32_t)C::kStageBytes);
          tma_load_4d(a_dst, &maps.a, bar, kb * kBK, t.s0, 0, t.b);
#pragma unroll
          for (int nb = 0; nb < BN / 64; ++nb)
            tma_load_4d(b_dst + nb * C::kBBlock, tw, bar, t.n0 + nb * 64, kb * kBK, 0, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ============================================ UMMA issuer =============================================
    const bool leader = elect_one();
    constexpr uint32_t idesc = make_idesc(kBM, BN, BF16, true);
    uint32_t kb_total = 0;
    bool alive = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < gp.total_tiles && alive; tile += gridDim.x, ++it) {
      const int slot = it & 1;
      if (!mbar_wait(bar_acc_empty + 8 * slot, (uint32_t)(((it >> 1) & 1) ^ 1), abort_flag, wait_ns)) break;
      tc_fence_after();
      const uint32_t d = tmem_base + (uint32_t)(slot * BN);
      for (int kb = 0; kb < gp.k_blocks; ++kb, ++kb_total) {
        const int s = (int)(kb_total % kStages);
        if (!mbar_wait(bar_full + 8 * s, (kb_total / kStages) & 1u, abort_flag, wait_ns)) { alive = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_base + s * C::kStageBytes;
        const uint32_t b_addr = a_addr + C::kABytes;
#pragma unroll
        for (int kk = 0; kk < kBK / 16; ++kk) {
          const uint64_t ad = make_smem_desc(a_addr + (uint32_t)(kk * 32), 16, 1024);
          const uint64_t bd = make_smem_desc(b_addr + (uint32_t)(kk * 2048), C::kBBlock, 1024);
          if (leader) mma_ss(d, ad, bd, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
        }
        if (leader) tc_commit(bar_empty + 8 * s);
      }
      if (alive && leader) tc_commit(bar_acc_full + 8 * slot);
    }
  } else {
    // ============================================== epilogue ==============================================
    const int quarter = warp & 3;   // the TMEM lanes a warp may read: 32 * (warp % 4) ...
    const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
    const uint32_t my_stage = epi_smem + (uint32_t)((warp - 2) * kEpiBytesPerWarp);
    const uint32_t my_row = my_stage + (uint32_t)(lane * 128);
    const uint32_t my_swz = (uint32_t)(lane & 7);
    const bool out_f32 = gp.out_f32 != 0;
    bool stores_in_flight = false;
    int it = 0;
    for (int tile = blockIdx.x; tile < gp.total_tiles; tile += gridDim.x, ++it) {
      const int slot = it & 1;
      const Tile t = decode_tile(gp, tile, BN);
      bool ok = mbar_wait(bar_acc_full + 8 * slot, (uint32_t)((it >> 1) & 1), abort_flag, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_bits + (uint32_t)(slot * BN);
      const CUtensorMap* tc = &maps.c[t.mat];
      const int row0 = t.s0 + quarter * 32;
      const bool box_valid = row0 < gp.seq;
#pragma unroll 2
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(t_acc + (uint32_t)c0, r);
        tc_wait_ld();
        const int half = out_f32 ? 0 : ((c0 >> 5) & 1);
        if (half == 0 && stores_in_flight) {
          if (lane == 0) bulk_wait_read0();
          __syncwarp();
        }
        if (out_f32) {
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared_v4(my_row + (((uint32_t)c ^ my_swz) << 4), r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            st_shared_v4(my_row + (((uint32_t)(half * 4 + c) ^ my_swz) << 4),
                         pack2<BF16>(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1])),
                         pack2<BF16>(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3])),
                         pack2<BF16>(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5])),
                         pack2<BF16>(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7])));
        }
        if (out_f32 || half == 1) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && box_valid) {
            const int n = t.n0 + (out_f32 ? c0 : c0 - 32);   // first column of the box within its matrix
            const int h = n / gp.head_dim;
            tma_store_4d(tc, my_stage, n - h * gp.head_dim, row0, h, t.b);
            bulk_commit();
          }
          stores_in_flight = true;
        }
      }
      // every lane's TMEM reads are complete (tcgen05.wait::ld above): hand the accumulator back
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * slot);
    }
    if (lane == 0) bulk_wait_all();   // staging memory must outlive the bulk stores that read it
    __syncwarp();
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
    if (threadIdx.x == 0 && gp.status) atomicOr(gp.status, kStatusTimeout);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int BN, bool BF16>
cudaError_t launch_t(const ProjGemm& g, cudaStream_t stream, int num_sms, int32_t* status, const char** why, bool expire) {
  using C = GCfg<BN>;
  cudaError_t e = tmap::resolve_encode();
  if (e != cudaSuccess) { *why = "cuTensorMapEncodeTiled is not available from the driver"; return e; }
  const CUtensorMapDataType dt16 = BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUtensorMapSwizzle s128 = CU_TENSOR_MAP_SWIZZLE_128B;
  GemmMaps maps;
  const int64_t a_stride[3] = {g.seq * g.k, g.seq * g.k, g.k};
  const int64_t w_stride[3] = {g.k * g.n, g.k * g.n, g.n};
  bool ok = tmap::encode_bhsd(&maps.a, dt16, 2, s128, g.a, g.k, g.seq, 1, g.batch, a_stride, kBK, kBM);
  const int64_t heads = g.n / g.head_dim;
  for (int i = 0; i < 3; ++i) {
    const int j = i < g.num_mats ? i : 0;   // unused slots repeat matrix 0 so that every map is valid
    ok = ok && tmap::encode_bhsd(&maps.w[i], dt16, 2, s128, g.w[j], g.n, g.k, 1, 1, w_stride, 64, kBK);
    ok = ok && (g.out_f32
        ? tmap::encode_bhsd(&maps.c[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, s128, g.c[j], g.head_dim, g.seq, heads,
                            g.batch, g.c_stride, 32, 32)
        : tmap::encode_bhsd(&maps.c[i], dt16, 2, s128, g.c[j], g.head_dim, g.seq, heads, g.batch, g.c_stride, 64, 32));
  }
  if (!ok) { *why = "cuTensorMapEncodeTiled rejected a tensor (address or stride alignment)"; return cudaErrorInvalidValue; }
  GemmParams gp;
  const int64_t row_tiles_per_batch = (g.seq + kBM - 1) / kBM, col_tiles = (g.n / BN) * g.num_mats;
  const int64_t total = g.batch * row_tiles_per_batch * col_tiles;
  if (total <= 0 || total > 0x3fffffff || kGroupRows * col_tiles > 0x3fffffff) { *why = "tile count out of range"; return cudaErrorInvalidValue; }
  gp.row_tiles_per_batch = (int)row_tiles_per_batch;
  gp.row_tiles = (int)(g.batch * row_tiles_per_batch);
  gp.col_tiles_per_mat = (int)(g.n / BN);
  gp.col_tiles = (int)col_tiles;
  gp.total_tiles = (int)total;
  gp.k_blocks = (int)((g.k + kBK - 1) / kBK);
  gp.seq = (int)g.seq;
  gp.head_dim = g.head_dim;
  gp.out_f32 = g.out_f32 ? 1 : 0;
  gp.status = status;
  gp.withhold_loads = expire ? 1 : 0;
  gp.wait_budget_ns = expire ? 20000000ull : kWaitBudgetNs;   // 20 ms in the time-out test
  auto kern = proj_gemm_sm100_kernel<BN, BF16>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) { *why = "cannot raise the dynamic shared memory limit"; return e; }
  const unsigned grid = (unsigned)(total < num_sms ? total : num_sms);
  kern<<<grid, kThreads, C::kSmemBytes, stream>>>(maps, gp);
  return cudaGetLastError();
}

}  // namespace

bool proj_gemm_sm100_supported(const ProjGemm& g, const char** why) {
  if (g.head_dim != 64 && g.head_dim != 128) { *why = "projection GEMM takes head_dim 64 or 128"; return false; }
  if (g.n <= 0 || g.n % 128 != 0 || g.n % g.head_dim != 0) { *why = "projection GEMM needs heads * head_dim to be a multiple of 128"; return false; }
  if (g.k <= 0 || g.k % 8 != 0) { *why = "projection GEMM needs an inner dimension that is a multiple of 8"; return false; }
  if (g.num_mats < 1 || g.num_mats > 3) { *why = "projection GEMM takes 1 to 3 weight matrices"; return false; }
  if (g.batch <= 0 || g.seq <= 0 || g.seq > 0x7fffff00ll || g.batch > 65535) { *why = "projection GEMM: batch or sequence out of range"; return false; }
  if ((uintptr_t)g.a % 16 != 0) { *why = "projection GEMM: input must be 16-byte aligned"; return false; }
  const int osz = g.out_f32 ? 4 : 2;
  for (int i = 0; i < g.num_mats; ++i) {
    if ((uintptr_t)g.w[i] % 16 != 0 || (uintptr_t)g.c[i] % 16 != 0) { *why = "projection GEMM: weights and outputs must be 16-byte aligned"; return false; }
  }
  for (int i = 0; i < 3; ++i)
    if (g.c_stride[i] <= 0 || (g.c_stride[i] * osz) % 16 != 0) { *why = "projection GEMM: output strides must be positive multiples of 16 bytes"; return false; }
  return true;
}

cudaError_t launch_proj_gemm_sm100(const ProjGemm& g, cudaStream_t stream, int num_sms, int32_t* status,
                                   const char** why, bool expire) {
  const bool wide = g.n % 256 == 0;
  if (g.bf16) return wide ? launch_t<256, true>(g, stream, num_sms, status, why, expire) : launch_t<128, true>(g, stream, num_sms, status, why, expire);
  return wide ? launch_t<256, false>(g, stream, num_sms, status, why, expire) : launch_t<128, false>(g, stream, num_sms, status, why, expire);
}

}  // namespace aidn
