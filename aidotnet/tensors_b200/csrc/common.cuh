// Shared definitions of the attention kernels: the flattened launch parameters, dtype helpers and the
// mask evaluation that every kernel uses so that mask semantics are defined once.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/aidn_sdpa.h"

namespace aidn {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Device status word values (bit flags) written by kernels that give up a bounded wait.
constexpr int kStatusTimeout = 1;
constexpr int kStatusBadBlock = 2;  // a block-table entry outside [0, num_blocks) was met (the key is skipped)

struct SdpaParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  float* weights;   // [B, Hq, Sq, Sk] fp32 probabilities, or null (generic kernel only)
  void* peer_out[8];   // other devices' `out` tensors, mapped here (tcgen05 prefill only)
  int32_t peer_count;
  const void* mask;
  const int32_t* kv_len;
  int64_t mask_stride[4];
  int64_t qs[3], ks[3], vs[3], os[3];  // element strides for (B, H, S)
  int64_t seq_q, seq_kv;
  int64_t causal_offset;
  int32_t batch;
  int32_t num_q_heads, num_kv_heads, group;  // group = Hq / Hkv
  int32_t head_begin, head_count;            // q-head shard computed by this launch
  int32_t head_dim;
  int32_t mask_kind;
  int32_t causal;
  int32_t out_f32;  // 1: output is fp32, 0: output has the input dtype
  float scale;
  float softcap;
  int32_t* status;  // device word, or null
  // Paged K/V (null block_table = contiguous): key t of batch entry b lives in row
  // block_table[b * bt_stride + t / block_size] * block_size + t % block_size of the pool, and that row index
  // takes the place of the key index in the K/V address (ks[2] / vs[2] = token stride, ks[0] / vs[0] unused).
  const int32_t* block_table;
  int64_t bt_stride;
  int32_t block_size;
  int32_t block_shift;  // log2(block_size) when it is a power of two, else -1
  int32_t num_blocks;   // > 0: entries are range-checked against it
};

template <typename T>
__device__ __forceinline__ float to_float(T x);
template <>
__device__ __forceinline__ float to_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ float from_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Stores one output element either as fp32 or in the input dtype.
template <typename T>
__device__ __forceinline__ void store_out(void* base, int64_t idx, float x, int out_f32) {
  if (out_f32) static_cast<float*>(base)[idx] = x;
  else static_cast<T*>(base)[idx] = from_float<T>(x);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// exp used by the softmax: exact expf for fp32 inputs (1e-5 relative contract), ex2.approx otherwise.
template <typename T>
__device__ __forceinline__ float softmax_exp(float x) {
  if constexpr (sizeof(T) == 4) return expf(x);
  else return ex2_approx(x * kLog2e);
}

// Applies softcap, additive bias and every mask to a scaled logit.
// Order: scale (done by the caller) -> softcap -> bias -> keep masks / causal / padding,
// as CpuEngine.cs:27807-27816 (SDPA) and :29218-29239 (FlashAttention) of the reference.
// Returns -inf for a masked position.
__device__ __forceinline__ float finish_logit(const SdpaParams& p, float s, int b, int h, int64_t qi, int64_t kj,
                                              int64_t kv_limit) {
  if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
  if (kj >= kv_limit) return -INFINITY;
  if (p.causal && kj > qi + p.causal_offset) return -INFINITY;
  if (p.mask_kind != AIDN_MASK_NONE) {
    const int64_t idx = b * p.mask_stride[0] + h * p.mask_stride[1] + qi * p.mask_stride[2] + kj * p.mask_stride[3];
    if (p.mask_kind == AIDN_MASK_KEEP_U8) {
      if (static_cast<const uint8_t*>(p.mask)[idx] == 0) return -INFINITY;
    } else if (p.mask_kind == AIDN_MASK_KEEP_F32) {
      if (static_cast<const float*>(p.mask)[idx] == 0.0f) return -INFINITY;
    } else {
      s += static_cast<const float*>(p.mask)[idx];
    }
  }
  return s;
}

// Number of keys a batch entry can see before causal masking: min(seq_kv, kv_len[b]).
// (With a block table the host has already capped seq_kv at the keys the table's rows can address.)
__device__ __forceinline__ int64_t kv_limit_of(const SdpaParams& p, int b) {
  int64_t lim = p.seq_kv;
  if (p.kv_len) {
    int64_t l = p.kv_len[b];
    if (l < 0) l = 0;
    if (l < lim) lim = l;
  }
  return lim;
}

// Paged K/V addressing in two halves, so that a kernel can issue the block-table read a step ahead and touch its
// result only when the row is needed (anything computed from the entry right after the read would make the warp
// wait for it there).
//   kv_block_read: the raw entry of key's block (volatile: issued where the caller placed it).
//   kv_row_from:   pool row of the key from that entry; -1, and `bad` set, for an entry outside the pool.  No
//                  branch on the entry; the caller reports `bad` once, at its end, with report_bad_block().
__device__ __forceinline__ int32_t kv_block_read(const SdpaParams& p, int b, int64_t key) {
  const uint32_t k32 = (uint32_t)key;
  const uint32_t blk = p.block_shift >= 0 ? (k32 >> p.block_shift) : (k32 / (uint32_t)p.block_size);
  int32_t phys;
  asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(phys) : "l"(p.block_table + (int64_t)b * p.bt_stride + blk));
  return phys;
}

__device__ __forceinline__ int64_t kv_row_from(const SdpaParams& p, int64_t key, int32_t phys, bool& bad) {
  const uint32_t k32 = (uint32_t)key;
  const uint32_t blk = p.block_shift >= 0 ? (k32 >> p.block_shift) : (k32 / (uint32_t)p.block_size);
  const bool out = phys < 0 || (p.num_blocks > 0 && phys >= p.num_blocks);
  bad = bad || out;
  const int64_t row = (int64_t)phys * p.block_size + (k32 - blk * (uint32_t)p.block_size);
  return out ? -1 : row;
}

// Pool row of key `key` of batch entry b (the key itself without a block table): read and use in one place.
__device__ __forceinline__ int64_t kv_row_of(const SdpaParams& p, int b, int64_t key, bool& bad) {
  if (!p.block_table) return key;
  return kv_row_from(p, key, kv_block_read(p, b, key), bad);
}

__device__ __forceinline__ void report_bad_block(const SdpaParams& p, bool bad) {
  if (bad && p.status) atomicOr(p.status, kStatusBadBlock);
}

// Host-side launchers (one per kernel family); each returns the CUDA error of its launch.
cudaError_t launch_generic(const SdpaParams& p, int dtype, cudaStream_t stream);
cudaError_t launch_decode(const SdpaParams& p, int dtype, int chunk, int nchunks, float* workspace, cudaStream_t stream,
                          int* launches);
bool decode_supported(int dtype, int head_dim);
int64_t decode_static_scratch_bytes();
cudaError_t launch_decode_static(const SdpaParams& p, int dtype, int chunk, int nchunks, cudaStream_t stream,
                                 int* launches);
cudaError_t launch_cast(int kind, const void* src, void* dst, int64_t n, cudaStream_t stream);
cudaError_t launch_paged_append(const void* src_k, const void* src_v, void* pool_k, void* pool_v,
                                const int32_t* block_table, int64_t start, int64_t tokens, int block_size, int num_blocks,
                                int64_t row_bytes, cudaStream_t stream);

// Attention backward (csrc/sdpa_backward.cu): the forward's parameter block (p.out = O, p.lse = log-sum-exp, both
// inputs here) plus dO, the gradient outputs and the delta scratch.
struct BwdParams {
  SdpaParams p;
  const void* dout;   // dtype of p.out
  int64_t dos[3];
  float* dq;          // [B, Hc, Sq, D] fp32, Hc = heads of the shard
  float* dk;          // [B, Hc / group, Sk, D] fp32
  float* dv;
  float* delta;       // [B, Hc, Sq] scratch
  void* dout_t;       // scratch: dO in the input dtype, dense [B, Hc, Sq, D] (16-bit inputs with an fp32 dO), or null
  int32_t no_tcgen05; // 1: stay on the mma.sync / FFMA kernels (desc.path == AIDN_PATH_GENERIC)
  int32_t expire;     // test hook of the tcgen05 kernels: loads are withheld and every bounded wait gives up after 20 ms
  int32_t round_dout; // set by the launcher: delta is summed from dO as rounded into dout_t (what the tensor-core
                      // kernels multiply with), so that every row of dS sums to zero as it does in exact arithmetic
};
// *used_tcgen05 tells which family ran the dQ and dK / dV launches.
cudaError_t launch_backward(const BwdParams& bp, int dtype, cudaStream_t stream, int* launches, int* used_tcgen05);
// tcgen05 dQ and dK / dV launches (csrc/sdpa_backward_sm100.cu); delta (and dout_t) must already be on the stream.
bool backward_sm100_supported(const BwdParams& bp, int dtype);
cudaError_t launch_backward_sm100(const BwdParams& bp, int dtype, cudaStream_t stream, int* launches, const char** why);

// Packed Q/K/V projection + RoPE + KV-cache write (csrc/qkv_rope_cache.cu).
struct QkvRopeParams {
  const float* input;
  const void* weights;
  const float* bias;
  const float* cosine;
  const float* sine;
  void* query;
  void* key_cache;
  void* value_cache;
  const int32_t* positions;
  const int32_t* cache_rows;
  int32_t tokens, heads, kv_heads, head_dim;
  int32_t position;
  int32_t query_dtype, cache_dtype;
  int64_t cache_capacity, max_position;
  int32_t model;
};

int64_t qkv_rope_max_model();
cudaError_t launch_qkv_rope_cache(const QkvRopeParams& p, int weight_dtype, int num_sms, cudaStream_t stream,
                                  int* launches);
cudaError_t launch_rope_interleaved(const float* in, const float* cosc, const float* sinc, float* out, int64_t rows,
                                    int head_dim, int seq_len, int start_position, cudaStream_t stream);

// Per-handle memory of the tcgen05 prefill launcher: the four TMA tensor maps of the last launch, with the tensors
// they were encoded for, and which kernel instantiations already had their shared-memory limit raised in the
// handle's context.  A launch whose pointers, extents and strides match re-uses the maps; encoding happens on the host
// only and is capture-safe either way.
struct alignas(64) PrefillMapCache {
  unsigned char maps[4][128];   // CUtensorMap images: q, k, v, out
  struct Key {
    const void* q; const void* k; const void* v; const void* out;
    int64_t qs[3], ks[3], vs[3], os[3];
    int64_t seq_q, kv_rows;
    int32_t batch, kv_batch, num_q_heads, num_kv_heads, head_dim, kv_box, out_f32, dtype;
  } key;
  bool valid;
  bool attr_set[16];            // by instantiation: (epilogue warpgroup ? 8 : 0) + (fp16 ? 4 : 0) + (head_dim 128 ? 2 : 0) + (masked ? 1 : 0)
};
bool prefill_sm100_supported(const SdpaParams& p, int dtype, const char** why);
// cache may be null (maps are then encoded on every call).
cudaError_t launch_prefill_sm100(const SdpaParams& p, int dtype, cudaStream_t stream, int32_t* sched, int num_sms,
                                 float* debug, int debug_mode, PrefillMapCache* cache, const char** why);

// Projection GEMM of the fused multi-head-attention forward (csrc/proj_gemm_sm100.cu):
// c[i][b, s, n] = sum_k a[b, s, k] * w[i][k, n] for up to three weight matrices that share a; column n lands at
// c[i] + b*c_stride[0] + (n / head_dim)*c_stride[1] + s*c_stride[2] + n % head_dim.
struct ProjGemm {
  const void* a;        // [batch, seq, k] dense; 16-bit for the tcgen05 kernel
  const void* w[3];     // [k, n] row-major, same type as a
  void* c[3];
  int64_t c_stride[3];  // elements for (batch, head, sequence position)
  int64_t batch, seq, k, n;
  int32_t num_mats;
  int32_t head_dim;
  bool out_f32;         // fp32 output, else the input dtype
  bool bf16;            // bf16 inputs, else fp16
};
bool proj_gemm_sm100_supported(const ProjGemm& g, const char** why);
// expire: test hook - the producer withholds its loads and every bounded wait gives up after 20 ms.
cudaError_t launch_proj_gemm_sm100(const ProjGemm& g, cudaStream_t stream, int num_sms, int32_t* status,
                                   const char** why, bool expire = false);
// The same contract in fp32 FFMA arithmetic for any sizes and for a / w of `dtype` (csrc/proj_gemm_generic.cu).
bool proj_gemm_generic_supported(const ProjGemm& g, const char** why);
cudaError_t launch_proj_gemm_generic(const ProjGemm& g, int dtype, cudaStream_t stream);

}  // namespace aidn
