// CPU oracle for the fused scaled-dot-product-attention forward path.
//
// TEST INFRASTRUCTURE ONLY. This file restates, in plain C++, the arithmetic of the reference
// library's CPU attention path so that the CUDA kernels can be checked against it. It is never
// linked into, called from, or shipped with the product library; only the test-suite, the smoke
// check and the benchmark's CPU-baseline leg load it.
//
// Parity status: PINNED. The reference ships no stored golden vectors for attention; its tests pin the
// path by recomputing scalar in-test references and closed forms
// (tests/AiDotNet.Tensors.Tests/Engines/BatchMatMulAndAttentionTests.cs:287-317 softcap closed form,
//  Engines/SdpaMaskBroadcastTests.cs:61-143, Engines/DirectGpu/GpuCpuConsistencyTests.cs:895-1061,
//  Engines/DirectGpu/RopeGqaOpenClTests.cs:200-279 GqaReference,
//  Engines/DirectGpu/FlashDecodeCudaTests.cs:43-126 DecodeOracle,
//  Engines/FlashAttentionBiasTests.cs). The same cases, with the same deterministic inputs where the
// reference gives them in-line, are replayed against this file by tests/test_oracle_pins.py and the
// committed fixtures under tests/golden/.
//
// What is restated (paths are relative to the reference project root):
//   src/AiDotNet.Tensors/Engines/CpuEngine.cs:27695-27881  ScaledDotProductAttentionFloat
//        per (batch, head): SGEMM S = Q.K^T -> pass 1: v = s*scale; softcap; mask -> -inf; row max
//        -> all-masked row => zero weights -> pass 2: e = exp(v - max), sum -> pass 3: e *= 1/sum
//        -> SGEMM O = W.V; parallel over batch*heads.
//   src/AiDotNet.Tensors/Engines/CpuEngine.cs:27297-27374  ScaledDotProductAttentionGqa
//        KV heads broadcast to query heads (kv = h / (Hq/Hkv)); causal plane j <= i + (Sk - Sq).
//   src/AiDotNet.Tensors/Engines/CpuEngine.cs:29146-29288  FlashAttentionFloat
//        additive bias after scale, causal j > i masked, stats = max + log(sum), -inf when fully masked.
//   src/AiDotNet.Tensors/Engines/CpuEngine.MultiHeadAttention.cs:344 BroadcastMaskIndex
//        a size-1 mask axis maps every index to 0 (expressed here as a zero stride).
//   src/AiDotNet.Tensors/NumericOperations/BFloat16.cs:65-92 FromFloat / ToFloat
//        round-to-nearest-even, NaN keeps sign and payload top bits and gets the quiet bit.
//
// The reference materialises the full [B,H,Sq,Sk] score and weight planes with 32-bit indices and so
// cannot run the largest configurations; this restatement computes the same per-row quantities in
// blocks of query rows with 64-bit indices, which changes memory use but not the per-row arithmetic.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

enum {
  ORACLE_MASK_NONE = 0,
  ORACLE_MASK_KEEP_U8 = 1,   // Tensor<bool>: non-zero byte = attend
  ORACLE_MASK_KEEP_F32 = 2,  // float mask as uploaded by the GPU engine: 0.0f = masked
  ORACLE_MASK_ADD_F32 = 3    // additive bias
};

struct aidn_oracle_args {
  const float* q;  // [B,Hq,Sq,D]   (strides below, innermost stride 1)
  const float* k;  // [B,Hkv,Sk,D]
  const float* v;  // [B,Hkv,Sk,Dv]
  float* out;      // [B,Hq,Sq,Dv]
  float* lse;      // [B,Hq,Sq] or null
  float* weights;  // [B,Hq,Sq,Sk] dense or null
  int64_t batch, q_heads, kv_heads, seq_q, seq_kv, head_dim, head_dim_v;
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3];  // elements, for (B,H,S)
  float scale;
  float softcap;          // <= 0 disables
  int32_t causal;         // keep k <= q + causal_offset
  int64_t causal_offset;
  int32_t mask_kind;
  const void* mask;
  int64_t mask_stride[4];  // elements for (B,H,Sq,Sk); 0 = broadcast axis
  const int32_t* kv_len;   // [B] or null: keys >= kv_len[b] are masked (padding)
  int32_t accumulate_f64;  // 1: GEMM and softmax sums in double (error attribution)
  int32_t faithful;        // 1: full-width GEMMs and a materialised KV broadcast copy, as the reference does
  int32_t threads;         // <= 0: OpenMP default
};

}  // extern "C"

namespace {

constexpr int ROW_BLOCK = 64;

#if defined(__x86_64__)
#define ORACLE_CLONES __attribute__((target_clones("arch=skylake-avx512", "arch=haswell", "default")))
#else
#define ORACLE_CLONES
#endif

// S[rows x n] = A[rows x kdim] . Bt[kdim x n]   (Bt is the per-head transposed key plane, as the
// reference builds it before SimdGemm.SgemmSequential, CpuEngine.cs:27778-27790).
ORACLE_CLONES void gemm_nn_f32(const float* a, int64_t lda, const float* bt, int64_t ldb, float* c, int64_t ldc,
                               int rows, int64_t n, int64_t kdim) {
  constexpr int JB = 64;
  for (int64_t j0 = 0; j0 < n; j0 += JB) {
    const int jn = (int)std::min<int64_t>(JB, n - j0);
    int i = 0;
    for (; i + 4 <= rows; i += 4) {
      float acc0[JB] = {0}, acc1[JB] = {0}, acc2[JB] = {0}, acc3[JB] = {0};
      const float* a0 = a + (int64_t)(i + 0) * lda;
      const float* a1 = a + (int64_t)(i + 1) * lda;
      const float* a2 = a + (int64_t)(i + 2) * lda;
      const float* a3 = a + (int64_t)(i + 3) * lda;
      for (int64_t d = 0; d < kdim; ++d) {
        const float* brow = bt + d * ldb + j0;
        const float x0 = a0[d], x1 = a1[d], x2 = a2[d], x3 = a3[d];
        if (jn == JB) {
#pragma omp simd
          for (int j = 0; j < JB; ++j) {
            const float b = brow[j];
            acc0[j] += x0 * b;
            acc1[j] += x1 * b;
            acc2[j] += x2 * b;
            acc3[j] += x3 * b;
          }
        } else {
          for (int j = 0; j < jn; ++j) {
            const float b = brow[j];
            acc0[j] += x0 * b;
            acc1[j] += x1 * b;
            acc2[j] += x2 * b;
            acc3[j] += x3 * b;
          }
        }
      }
      std::memcpy(c + (int64_t)(i + 0) * ldc + j0, acc0, sizeof(float) * jn);
      std::memcpy(c + (int64_t)(i + 1) * ldc + j0, acc1, sizeof(float) * jn);
      std::memcpy(c + (int64_t)(i + 2) * ldc + j0, acc2, sizeof(float) * jn);
      std::memcpy(c + (int64_t)(i + 3) * ldc + j0, acc3, sizeof(float) * jn);
    }
    for (; i < rows; ++i) {
      float acc[JB] = {0};
      const float* a0 = a + (int64_t)i * lda;
      for (int64_t d = 0; d < kdim; ++d) {
        const float* brow = bt + d * ldb + j0;
        const float x0 = a0[d];
        for (int j = 0; j < jn; ++j) acc[j] += x0 * brow[j];
      }
      std::memcpy(c + (int64_t)i * ldc + j0, acc, sizeof(float) * jn);
    }
  }
}

void gemm_nn_f64acc(const float* a, int64_t lda, const float* bt, int64_t ldb, float* c, int64_t ldc, int rows,
                    int64_t n, int64_t kdim) {
  std::vector<double> acc((size_t)n);
  for (int i = 0; i < rows; ++i) {
    std::fill(acc.begin(), acc.end(), 0.0);
    for (int64_t d = 0; d < kdim; ++d) {
      const double x = a[(int64_t)i * lda + d];
      const float* brow = bt + d * ldb;
      for (int64_t j = 0; j < n; ++j) acc[(size_t)j] += x * (double)brow[j];
    }
    for (int64_t j = 0; j < n; ++j) c[(int64_t)i * ldc + j] = (float)acc[(size_t)j];
  }
}

inline bool mask_keeps(const aidn_oracle_args& p, int64_t b, int64_t h, int64_t i, int64_t j, float* bias) {
  *bias = 0.f;
  if (p.kv_len && j >= (int64_t)p.kv_len[b]) return false;
  if (p.causal && j > i + p.causal_offset) return false;
  if (p.mask_kind == ORACLE_MASK_NONE || p.mask == nullptr) return true;
  const int64_t idx = b * p.mask_stride[0] + h * p.mask_stride[1] + i * p.mask_stride[2] + j * p.mask_stride[3];
  switch (p.mask_kind) {
    case ORACLE_MASK_KEEP_U8:
      return static_cast<const uint8_t*>(p.mask)[idx] != 0;
    case ORACLE_MASK_KEEP_F32:
      return static_cast<const float*>(p.mask)[idx] != 0.0f;
    case ORACLE_MASK_ADD_F32:
      *bias = static_cast<const float*>(p.mask)[idx];
      return true;
    default:
      return true;
  }
}

void one_head(const aidn_oracle_args& p, int64_t b, int64_t h, std::vector<float>& kt, std::vector<float>& vbuf,
              std::vector<float>& scores) {
  const int64_t Sq = p.seq_q, Sk = p.seq_kv, D = p.head_dim, Dv = p.head_dim_v;
  const int64_t group = p.q_heads / p.kv_heads;
  const int64_t kvh = h / group;  // CpuEngine.cs:27367 BroadcastKvHeads head map
  const float* qh = p.q + b * p.q_stride[0] + h * p.q_stride[1];
  const float* kh = p.k + b * p.k_stride[0] + kvh * p.k_stride[1];
  const float* vh = p.v + b * p.v_stride[0] + kvh * p.v_stride[1];
  float* oh = p.out + b * p.o_stride[0] + h * p.o_stride[1];

  // Width of the key range this head can ever see. The reference always runs the full width; the
  // trimmed width gives identical results because masked weights are exactly zero.
  int64_t width = Sk;
  if (!p.faithful) {
    if (p.kv_len) width = std::min<int64_t>(width, std::max<int32_t>(0, p.kv_len[b]));
    if (p.causal) width = std::min<int64_t>(width, std::max<int64_t>(0, (Sq - 1) + p.causal_offset + 1));
  }

  // K^T for this head (kt[d][j]); V gathered dense [j][dv].
  kt.assign((size_t)(D * std::max<int64_t>(width, 1)), 0.f);
  for (int64_t j = 0; j < width; ++j)
    for (int64_t d = 0; d < D; ++d) kt[(size_t)(d * width + j)] = kh[j * p.k_stride[2] + d];
  vbuf.resize((size_t)(std::max<int64_t>(width, 1) * Dv));
  for (int64_t j = 0; j < width; ++j)
    std::memcpy(&vbuf[(size_t)(j * Dv)], vh + j * p.v_stride[2], sizeof(float) * (size_t)Dv);

  const float neg_inf = -std::numeric_limits<float>::infinity();
  const bool use_cap = p.softcap > 0.f;
  const float cap = p.softcap, inv_cap = use_cap ? 1.f / p.softcap : 0.f;
  scores.resize((size_t)(ROW_BLOCK * std::max<int64_t>(width, 1)));
  std::vector<float> qblk((size_t)(ROW_BLOCK * D));

  for (int64_t i0 = 0; i0 < Sq; i0 += ROW_BLOCK) {
    const int rows = (int)std::min<int64_t>(ROW_BLOCK, Sq - i0);
    int64_t w = width;
    if (!p.faithful && p.causal) w = std::min<int64_t>(w, std::max<int64_t>(0, (i0 + rows - 1) + p.causal_offset + 1));
    for (int r = 0; r < rows; ++r)
      std::memcpy(&qblk[(size_t)(r * D)], qh + (i0 + r) * p.q_stride[2], sizeof(float) * (size_t)D);

    if (w > 0) {
      if (p.accumulate_f64)
        gemm_nn_f64acc(qblk.data(), D, kt.data(), width, scores.data(), w, rows, w, D);
      else
        gemm_nn_f32(qblk.data(), D, kt.data(), width, scores.data(), w, rows, w, D);
    }

    for (int r = 0; r < rows; ++r) {
      const int64_t i = i0 + r;
      float* srow = &scores[(size_t)((int64_t)r * w)];
      float max_val = neg_inf;
      // pass 1: scale, softcap, bias, mask, max  (CpuEngine.cs:27807-27816, 29218-29239)
      for (int64_t j = 0; j < w; ++j) {
        float val = srow[j] * p.scale;
        if (use_cap) val = cap * std::tanh(val * inv_cap);
        float bias;
        const bool keep = mask_keeps(p, b, h, i, j, &bias);
        val += bias;
        if (!keep) val = neg_inf;
        if (val > max_val) max_val = val;
        srow[j] = val;
      }
      float* wrow = p.weights ? p.weights + (((b * p.q_heads + h) * Sq + i) * Sk) : nullptr;
      if (max_val == neg_inf) {  // fully masked row: zero weights, LSE = -inf (27822-27827, 29244-29250)
        for (int64_t j = 0; j < w; ++j) srow[j] = 0.f;
        if (wrow) std::fill(wrow, wrow + Sk, 0.f);
        if (p.lse) p.lse[(b * p.q_heads + h) * Sq + i] = neg_inf;
        continue;
      }
      // pass 2: exp and sum; pass 3: normalise  (27829-27839)
      float inv;
      float sum_f = 0.f;
      double sum_d = 0.0;
      for (int64_t j = 0; j < w; ++j) {
        const float e = std::exp(srow[j] - max_val);
        srow[j] = e;
        sum_f += e;
        sum_d += (double)e;
      }
      const float sum = p.accumulate_f64 ? (float)sum_d : sum_f;
      inv = sum != 0.f ? 1.f / sum : 0.f;
      if (p.accumulate_f64) {
        const double invd = sum_d != 0.0 ? 1.0 / sum_d : 0.0;
        for (int64_t j = 0; j < w; ++j) srow[j] = (float)((double)srow[j] * invd);
      } else {
        for (int64_t j = 0; j < w; ++j) srow[j] *= inv;
      }
      if (wrow) {
        std::memcpy(wrow, srow, sizeof(float) * (size_t)w);
        std::fill(wrow + w, wrow + Sk, 0.f);
      }
      if (p.lse)
        p.lse[(b * p.q_heads + h) * Sq + i] =
            p.accumulate_f64 ? (float)((double)max_val + std::log(sum_d)) : max_val + std::log(sum);
    }

    // O = W . V  (CpuEngine.cs:27847-27859)
    std::vector<float> oblk((size_t)(rows * Dv), 0.f);
    if (w > 0) {
      if (p.accumulate_f64)
        gemm_nn_f64acc(scores.data(), w, vbuf.data(), Dv, oblk.data(), Dv, rows, Dv, w);
      else
        gemm_nn_f32(scores.data(), w, vbuf.data(), Dv, oblk.data(), Dv, rows, Dv, w);
    }
    for (int r = 0; r < rows; ++r)
      std::memcpy(oh + (i0 + r) * p.o_stride[2], &oblk[(size_t)(r * Dv)], sizeof(float) * (size_t)Dv);
  }
}

}  // namespace

extern "C" {

// Returns 0 on success, 1 on invalid arguments.
int aidn_oracle_sdpa(const aidn_oracle_args* pp) {
  if (!pp) return 1;
  const aidn_oracle_args& p = *pp;
  if (!p.q || !p.k || !p.v || !p.out) return 1;
  if (p.batch <= 0 || p.q_heads <= 0 || p.kv_heads <= 0 || p.seq_q <= 0 || p.seq_kv <= 0 || p.head_dim <= 0 ||
      p.head_dim_v <= 0)
    return 1;
  if (p.q_heads % p.kv_heads != 0) return 1;
  const int64_t bh = p.batch * p.q_heads;
#ifdef _OPENMP
  const int nthreads = p.threads > 0 ? p.threads : omp_get_max_threads();
#else
  const int nthreads = 1;
#endif
  (void)nthreads;
  // The reference copies each KV head to all of its query heads before attending (BroadcastKvHeads);
  // the copy only affects timing, so it is performed (and discarded) only in faithful mode.
  std::vector<float> kcopy, vcopy;
  if (p.faithful && p.q_heads != p.kv_heads) {
    const int64_t per_k = p.seq_kv * p.head_dim, per_v = p.seq_kv * p.head_dim_v;
    kcopy.resize((size_t)(bh * per_k));
    vcopy.resize((size_t)(bh * per_v));
    const int64_t group = p.q_heads / p.kv_heads;
    for (int64_t b = 0; b < p.batch; ++b)
      for (int64_t h = 0; h < p.q_heads; ++h) {
        const float* ks = p.k + b * p.k_stride[0] + (h / group) * p.k_stride[1];
        const float* vs = p.v + b * p.v_stride[0] + (h / group) * p.v_stride[1];
        for (int64_t j = 0; j < p.seq_kv; ++j) {
          std::memcpy(&kcopy[(size_t)((b * p.q_heads + h) * per_k + j * p.head_dim)], ks + j * p.k_stride[2],
                      sizeof(float) * (size_t)p.head_dim);
          std::memcpy(&vcopy[(size_t)((b * p.q_heads + h) * per_v + j * p.head_dim_v)], vs + j * p.v_stride[2],
                      sizeof(float) * (size_t)p.head_dim_v);
        }
      }
    asm volatile("" : : "r"(kcopy.data()), "r"(vcopy.data()) : "memory");
  }
#pragma omp parallel num_threads(nthreads)
  {
    std::vector<float> kt, vbuf, scores;
#pragma omp for schedule(dynamic, 1)
    for (int64_t idx = 0; idx < bh; ++idx) one_head(p, idx / p.q_heads, idx % p.q_heads, kt, vbuf, scores);
  }
  return 0;
}

// Number of hardware threads the OpenMP runtime will use by default.
int aidn_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// float -> bfloat16 bits, BFloat16.FromFloat (NumericOperations/BFloat16.cs:65-84).
uint16_t aidn_oracle_f32_to_bf16(float value) {
  uint32_t bits;
  std::memcpy(&bits, &value, 4);
  if ((bits & 0x7F800000u) == 0x7F800000u && (bits & 0x007FFFFFu) != 0) return (uint16_t)((bits >> 16) | 0x0040u);
  const uint32_t lsb = (bits >> 16) & 1u;
  return (uint16_t)((bits + 0x7FFFu + lsb) >> 16);
}

void aidn_oracle_f32_to_bf16_array(const float* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = aidn_oracle_f32_to_bf16(src[i]);
}

// bfloat16 bits -> float, BFloat16.ToFloat (BFloat16.cs:88-92).
void aidn_oracle_bf16_to_f32_array(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t bits = ((uint32_t)src[i]) << 16;
    std::memcpy(&dst[i], &bits, 4);
  }
}

}  // extern "C"
