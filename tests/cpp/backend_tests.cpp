// Port of the reference's CUDA-backend attention tests to the C++ host mirror (csrc/host/direct_gpu_backend.hpp).
// Each case names the reference test it replays (paths relative to tests/AiDotNet.Tensors.Tests/Engines/) and, as
// those tests do, recomputes its expectation with an in-test scalar reference.  Exit code 0 = all cases passed.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <limits>
#include <string>
#include <vector>

#include "../../aidotnet/tensors_b200/csrc/host/direct_gpu_backend.hpp"

using aidn::host::CudaBackend;
using aidn::host::GpuBuffer;

static int g_failed = 0;
#define EXPECT(cond, ...)                                  \
  do {                                                     \
    if (!(cond)) {                                         \
      std::printf("  FAILED %s:%d: ", __FILE__, __LINE__); \
      std::printf(__VA_ARGS__);                            \
      std::printf("\n");                                   \
      ++g_failed;                                          \
    }                                                      \
  } while (0)

struct DeviceArray {
  GpuBuffer buf;
  DeviceArray(const std::vector<float>& host, aidn_dtype dt = AIDN_F32) {
    buf.Size = (int64_t)host.size();
    buf.Dtype = dt;
    cudaMalloc(&buf.Handle, (size_t)buf.SizeInBytes());
    if (dt == AIDN_F32) {
      cudaMemcpy(buf.Handle, host.data(), host.size() * 4, cudaMemcpyHostToDevice);
    } else {
      std::vector<__nv_bfloat16> h(host.size());
      for (size_t i = 0; i < host.size(); ++i) h[i] = __float2bfloat16_rn(host[i]);
      cudaMemcpy(buf.Handle, h.data(), h.size() * 2, cudaMemcpyHostToDevice);
    }
  }
  explicit DeviceArray(int64_t n) {
    buf.Size = n;
    cudaMalloc(&buf.Handle, (size_t)n * 4);
    cudaMemset(buf.Handle, 0xff, (size_t)n * 4);
  }
  ~DeviceArray() { cudaFree(buf.Handle); }
  std::vector<float> download() const {
    std::vector<float> h((size_t)buf.Size);
    cudaMemcpy(h.data(), buf.Handle, h.size() * 4, cudaMemcpyDeviceToHost);
    return h;
  }
};

// Scalar reference in double: softmax(q k^T * scale [softcap] [+bias] [mask]) v, with the reference's conventions.
struct RefOpts {
  double scale = 1, softcap = 0;
  bool causal = false;
  long causal_offset = 0;
  const std::vector<float>* keep = nullptr;   // [B,H,Sq,Sk] float mask, 0 = masked
  const std::vector<float>* bias = nullptr;   // [B or 1,H,Sq,Sk]
  bool bias_has_batch = true;
  std::vector<double>* weights = nullptr;     // receives the [B,H,Sq,Sk] probabilities when set
};
static void reference(const std::vector<float>& q, const std::vector<float>& k, const std::vector<float>& v, int B,
                      int Hq, int Hkv, int Sq, int Sk, int D, const RefOpts& o, std::vector<double>& out,
                      std::vector<double>& lse, std::function<size_t(int, int, int, int)> kv_index = nullptr) {
  out.assign((size_t)B * Hq * Sq * D, 0.0);
  lse.assign((size_t)B * Hq * Sq, 0.0);
  if (o.weights) o.weights->assign((size_t)B * Hq * Sq * Sk, 0.0);
  const int g = Hq / Hkv;
  if (!kv_index) kv_index = [=](int b, int kh, int j, int d) { return (((size_t)b * Hkv + kh) * Sk + j) * D + d; };
  std::vector<double> s(Sk);
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hq; ++h)
      for (int i = 0; i < Sq; ++i) {
        double mx = -std::numeric_limits<double>::infinity();
        for (int j = 0; j < Sk; ++j) {
          double dot = 0;
          for (int d = 0; d < D; ++d) dot += (double)q[(((size_t)b * Hq + h) * Sq + i) * D + d] * k[kv_index(b, h / g, j, d)];
          double val = dot * o.scale;
          if (o.softcap > 0) val = o.softcap * std::tanh(val / o.softcap);
          const size_t mi = (((size_t)b * Hq + h) * Sq + i) * Sk + j;
          if (o.bias) val += (*o.bias)[o.bias_has_batch ? mi : (((size_t)h) * Sq + i) * Sk + j];
          if (o.keep && (*o.keep)[mi] == 0.0f) val = -std::numeric_limits<double>::infinity();
          if (o.causal && j > i + o.causal_offset) val = -std::numeric_limits<double>::infinity();
          s[j] = val;
          mx = std::max(mx, val);
        }
        double sum = 0;
        if (std::isinf(mx)) {
          lse[((size_t)b * Hq + h) * Sq + i] = mx;
          continue;
        }
        for (int j = 0; j < Sk; ++j) { s[j] = std::exp(s[j] - mx); sum += s[j]; }
        lse[((size_t)b * Hq + h) * Sq + i] = mx + std::log(sum);
        if (o.weights)
          for (int j = 0; j < Sk; ++j) (*o.weights)[(((size_t)b * Hq + h) * Sq + i) * Sk + j] = s[j] / sum;
        for (int d = 0; d < D; ++d) {
          double acc = 0;
          for (int j = 0; j < Sk; ++j) acc += s[j] / sum * v[kv_index(b, h / g, j, d)];
          out[(((size_t)b * Hq + h) * Sq + i) * D + d] = acc;
        }
      }
}

static std::vector<float> sequence(int n, float a, float b) {
  std::vector<float> r(n);
  for (int i = 0; i < n; ++i) r[i] = a + b * i;
  return r;
}
static std::vector<float> uniform(int n, unsigned seed) {   // LCG, U(-1, 1)
  std::vector<float> r(n);
  unsigned s = seed * 2654435761u + 12345u;
  for (int i = 0; i < n; ++i) { s = s * 1664525u + 1013904223u; r[i] = (float)((s >> 8) * (2.0 / 16777216.0) - 1.0); }
  return r;
}
static double max_abs_diff(const std::vector<float>& a, const std::vector<double>& b) {
  double m = 0;
  for (size_t i = 0; i < a.size(); ++i) m = std::max(m, std::fabs((double)a[i] - b[i]));
  return m;
}

int main() {
  cudaStream_t stream;
  cudaSetDevice(0);
  cudaStreamCreate(&stream);
  CudaBackend backend(0, stream);
  std::vector<double> ref, lse;

  {  // DirectGpu/GpuCpuConsistencyTests.cs:895-960  ScaledDotProductAttention_CrossAttention..., tolerance 2e-5
    std::printf("cross attention (Sq=2, Sk=3, D=3)\n");
    const int B = 2, H = 2, Sq = 2, Sk = 3, D = 3;
    auto q = sequence(B * H * Sq * D, -0.2f, 0.03f), k = sequence(B * H * Sk * D, 0.5f, -0.025f), v = sequence(B * H * Sk * D, -0.1f, 0.04f);
    DeviceArray dq(q), dk(k), dv(v), dout((int64_t)B * H * Sq * D);
    backend.ScaledDotProductAttention(dq.buf, dk.buf, dv.buf, dout.buf, nullptr, nullptr, B, H, Sq, Sk, D, 0.75f, false);
    backend.Synchronize();
    RefOpts o; o.scale = 0.75;
    reference(q, k, v, B, H, H, Sq, Sk, D, o, ref, lse);
    EXPECT(max_abs_diff(dout.download(), ref) <= 2e-5, "output mismatch %g", max_abs_diff(dout.download(), ref));

    // :1005-1061 full boolean mask, uploaded as floats (false -> 0.0f)
    std::printf("full boolean mask\n");
    std::vector<float> mask = {1,0,1,0,1,1, 1,1,0,1,0,0, 0,1,1,1,1,0, 1,0,0,0,1,0};
    DeviceArray dm(mask);
    backend.ScaledDotProductAttention(dq.buf, dk.buf, dv.buf, dout.buf, nullptr, &dm.buf, B, H, Sq, Sk, D, 0.75f, false);
    backend.Synchronize();
    o.keep = &mask;
    reference(q, k, v, B, H, H, Sq, Sk, D, o, ref, lse);
    EXPECT(max_abs_diff(dout.download(), ref) <= 2e-5, "masked output mismatch %g", max_abs_diff(dout.download(), ref));

    // :946-955, :1046-1060 the probabilities on request, with and without the mask, 2e-5
    std::printf("attention weights on request\n");
    std::vector<double> wref;
    o.weights = &wref;
    DeviceArray dw((int64_t)B * H * Sq * Sk);
    backend.ScaledDotProductAttention(dq.buf, dk.buf, dv.buf, dout.buf, &dw.buf, &dm.buf, B, H, Sq, Sk, D, 0.75f, false);
    backend.Synchronize();
    reference(q, k, v, B, H, H, Sq, Sk, D, o, ref, lse);
    EXPECT(max_abs_diff(dw.download(), wref) <= 2e-5, "masked weights mismatch %g", max_abs_diff(dw.download(), wref));
    EXPECT(max_abs_diff(dout.download(), ref) <= 2e-5, "output beside weights mismatch %g", max_abs_diff(dout.download(), ref));
    o.keep = nullptr;
    backend.ScaledDotProductAttention(dq.buf, dk.buf, dv.buf, dout.buf, &dw.buf, nullptr, B, H, Sq, Sk, D, 0.75f, false);
    backend.Synchronize();
    reference(q, k, v, B, H, H, Sq, Sk, D, o, ref, lse);
    EXPECT(max_abs_diff(dw.download(), wref) <= 2e-5, "weights mismatch %g", max_abs_diff(dw.download(), wref));
    DeviceArray tiny((int64_t)4);
    bool threw = false;
    try { backend.ScaledDotProductAttention(dq.buf, dk.buf, dv.buf, dout.buf, &tiny.buf, nullptr, B, H, Sq, Sk, D, 0.75f, false); }
    catch (const std::invalid_argument&) { threw = true; }
    EXPECT(threw, "a short weights buffer was accepted%s", "");
  }
  {  // :962-1003 ScaledDotProductAttention_LogitSoftcap_MatchesCpu
    std::printf("logit softcap\n");
    const int B = 2, H = 2, Sq = 2, Sk = 3, D = 3;
    auto q = sequence(B * H * Sq * D, -0.9f, 0.17f), k = sequence(B * H * Sk * D, 1.3f, -0.11f), v = sequence(B * H * Sk * D, -0.4f, 0.09f);
    DeviceArray dq(q), dk(k), dv(v), dout((int64_t)B * H * Sq * D);
    backend.ScaledDotProductAttention(dq.buf, dk.buf, dv.buf, dout.buf, nullptr, nullptr, B, H, Sq, Sk, D, 1.5f, false, 2.0f);
    backend.Synchronize();
    RefOpts o; o.scale = 1.5; o.softcap = 2.0;
    reference(q, k, v, B, H, H, Sq, Sk, D, o, ref, lse);
    EXPECT(max_abs_diff(dout.download(), ref) <= 2e-5, "softcap output mismatch %g", max_abs_diff(dout.download(), ref));
  }
  {  // DirectGpu/FlashDecodeCudaTests.cs:43-126  MhaDecode / GqaDecode, tolerance 2e-3 + 2e-3|e|
    std::printf("flash decode shape list\n");
    const int shapes[][5] = {{4, 4, 64, 40, 8}, {8, 8, 32, 100, 8}, {4, 4, 64, 7, 8}, {4, 4, 64, 64, 1}, {6, 6, 48, 77, 0},
                             {8, 2, 64, 50, 8}, {8, 1, 64, 40, 8}};
    for (auto& sh : shapes) {
      const int heads = sh[0], kvh = sh[1], D = sh[2], L = sh[3], splits = sh[4];
      auto k = uniform(L * kvh * D, 0xFDE + heads + kvh + L), v = uniform(L * kvh * D, 77 + L), q = uniform(heads * D, 5 + heads);
      DeviceArray dq(q), dk(k), dv(v), dout((int64_t)heads * D);
      const float scale = 1.0f / std::sqrt((float)D);
      backend.FlashDecode(dq.buf, dk.buf, dv.buf, dout.buf, heads, kvh, D, L, scale, splits);
      backend.Synchronize();
      RefOpts o; o.scale = scale;
      reference(q, k, v, 1, heads, kvh, 1, L, D, o, ref, lse,
                [=](int, int kh, int j, int d) { return ((size_t)j * kvh + kh) * D + d; });
      auto got = dout.download();
      bool ok = true;
      for (size_t i = 0; i < got.size(); ++i) ok = ok && std::fabs(got[i] - ref[i]) <= 2e-3 + 2e-3 * std::fabs(ref[i]);
      EXPECT(ok, "decode heads=%d kv=%d D=%d L=%d splits=%d", heads, kvh, D, L, splits);
    }
  }
  {  // DirectGpu/RopeGqaOpenClTests.cs:200-279  GroupedQueryAttention vs GqaReference (top-left causal), 1e-4
    std::printf("grouped query attention\n");
    const int B = 1, Hq = 6, Hkv = 2, S = 5, D = 8;
    auto q = uniform(B * Hq * S * D, 23), k = uniform(B * Hkv * S * D, 24), v = uniform(B * Hkv * S * D, 25);
    DeviceArray dq(q), dk(k), dv(v), dout((int64_t)B * Hq * S * D);
    for (int causal = 0; causal < 2; ++causal) {
      backend.GroupedQueryAttention(dq.buf, dk.buf, dv.buf, dout.buf, nullptr, B, Hq, Hkv, S, S, D, 1.0f / std::sqrt(8.0f), causal != 0);
      backend.Synchronize();
      RefOpts o; o.scale = 1.0 / std::sqrt(8.0); o.causal = causal != 0;
      reference(q, k, v, B, Hq, Hkv, S, S, D, o, ref, lse);
      EXPECT(max_abs_diff(dout.download(), ref) <= 1e-4, "gqa causal=%d mismatch", causal);
    }
  }
  {  // FlashAttentionBiasTests.cs: 3-D (batch-broadcast) and 4-D additive bias, stats = max + log(sum)
    std::printf("flash attention v2 with bias and statistics\n");
    const int B = 2, H = 3, S = 9, D = 16;
    auto q = uniform(B * H * S * D, 31), k = uniform(B * H * S * D, 32), v = uniform(B * H * S * D, 33);
    auto bias3 = uniform(H * S * S, 34), bias4 = uniform(B * H * S * S, 35);
    DeviceArray dq(q), dk(k), dv(v), db3(bias3), db4(bias4), dout((int64_t)B * H * S * D), dstats((int64_t)B * H * S);
    backend.FlashAttentionV2(dq.buf, dk.buf, dv.buf, dout.buf, dstats.buf, B, H, S, S, D, 0.25f, false, &db3.buf, 0);
    backend.Synchronize();
    RefOpts o; o.scale = 0.25; o.bias = &bias3; o.bias_has_batch = false;
    reference(q, k, v, B, H, H, S, S, D, o, ref, lse);
    EXPECT(max_abs_diff(dout.download(), ref) <= 2e-5 && max_abs_diff(dstats.download(), lse) <= 2e-5, "3-D bias mismatch");
    backend.FlashAttentionV2(dq.buf, dk.buf, dv.buf, dout.buf, dstats.buf, B, H, S, S, D, 0.25f, true, &db4.buf, H * S * S);
    backend.Synchronize();
    o.bias = &bias4; o.bias_has_batch = true; o.causal = true;
    reference(q, k, v, B, H, H, S, S, D, o, ref, lse);
    EXPECT(max_abs_diff(dout.download(), ref) <= 2e-5 && max_abs_diff(dstats.download(), lse) <= 2e-5, "4-D bias mismatch");
  }
  {  // bf16 prefill on the tcgen05 kernel (half-precision bar of DirectPtxWmmaTests.cs:474-477: 0.012 / LSE 0.02)
    std::printf("bf16 causal GQA prefill on the tensor-core kernel\n");
    const int B = 1, Hq = 4, Hkv = 2, S = 320, D = 128;
    auto round_bf16 = [](std::vector<float> x) { for (auto& f : x) f = __bfloat162float(__float2bfloat16_rn(f * 0.5f)); return x; };
    auto q = round_bf16(uniform(B * Hq * S * D, 41)), k = round_bf16(uniform(B * Hkv * S * D, 42)), v = round_bf16(uniform(B * Hkv * S * D, 43));
    DeviceArray dq(q, AIDN_BF16), dk(k, AIDN_BF16), dv(v, AIDN_BF16), dout((int64_t)B * Hq * S * D);
    backend.ScaledDotProductAttention(dq.buf, dk.buf, dv.buf, dout.buf, nullptr, nullptr, B, Hq, S, S, D, 1.0f / std::sqrt(128.0f), true, 0.0f, Hkv);
    backend.Synchronize();
    EXPECT(backend.LastPath() == AIDN_PATH_PREFILL_SM100, "expected the tcgen05 path, got %d", backend.LastPath());
    RefOpts o; o.scale = 1.0 / std::sqrt(128.0); o.causal = true;
    reference(q, k, v, B, Hq, Hkv, S, S, D, o, ref, lse);
    EXPECT(max_abs_diff(dout.download(), ref) <= 0.012, "bf16 prefill mismatch %g", max_abs_diff(dout.download(), ref));
  }
  {  // DirectGpu/PagedAttentionCudaTests.cs:43-205: scattered block table over a pool with spare blocks; decode,
     // prefill (query qi sees keys 0..startPos+qi) and their Gqa variants against a scalar reference in double
    std::printf("paged attention decode / prefill (+Gqa)\n");
    struct Case { int heads, kvHeads, D, bs, nq, start; };
    const Case cases[] = {{4, 4, 64, 16, 1, 39}, {2, 2, 128, 8, 1, 19}, {8, 8, 32, 32, 1, 99}, {4, 4, 64, 16, 8, 0},
                          {2, 2, 128, 8, 12, 5}, {8, 8, 32, 32, 20, 40}, {8, 2, 64, 16, 1, 51}, {8, 2, 64, 16, 9, 30}};
    for (const Case& c : cases) {
      const int keyLen = c.start + c.nq, nLogical = (keyLen + c.bs - 1) / c.bs, maxBlocks = nLogical + 5;
      const int pool = maxBlocks * c.bs * c.kvHeads * c.D;
      auto kc = uniform(pool, 51 + c.heads), vc = uniform(pool, 52 + c.heads), q = uniform(c.nq * c.heads * c.D, 53 + c.nq);
      std::vector<int> table(nLogical);
      for (int i = 0; i < nLogical; ++i) table[i] = (i * 5 + 3) % maxBlocks;   // 5 is coprime to every maxBlocks used (6..9)
      for (int i = 0; i < nLogical; ++i) for (int j = 0; j < i; ++j) if (table[i] == table[j]) table[i] = -1;
      bool distinct = true; for (int t : table) distinct = distinct && t >= 0;
      EXPECT(distinct, "test bug: block table has a repeated entry");
      const double scale = 1.0 / std::sqrt((double)c.D);
      std::vector<double> want((size_t)c.nq * c.heads * c.D, 0.0);
      for (int qi = 0; qi < c.nq; ++qi)
        for (int h = 0; h < c.heads; ++h) {
          const int kvh = h / (c.heads / c.kvHeads), len = c.start + qi + 1;
          std::vector<double> w(len);
          double mx = -1e300, sum = 0;
          for (int t = 0; t < len; ++t) {
            const size_t base = (((size_t)table[t / c.bs] * c.bs + t % c.bs) * c.kvHeads + kvh) * c.D;
            double dot = 0;
            for (int d = 0; d < c.D; ++d) dot += (double)q[((size_t)qi * c.heads + h) * c.D + d] * kc[base + d];
            w[t] = dot * scale; mx = std::max(mx, w[t]);
          }
          for (int t = 0; t < len; ++t) { w[t] = std::exp(w[t] - mx); sum += w[t]; }
          for (int t = 0; t < len; ++t) {
            const size_t base = (((size_t)table[t / c.bs] * c.bs + t % c.bs) * c.kvHeads + kvh) * c.D;
            for (int d = 0; d < c.D; ++d) want[((size_t)qi * c.heads + h) * c.D + d] += w[t] / sum * vc[base + d];
          }
        }
      DeviceArray dq(q), dk(kc), dv(vc), dout((int64_t)c.nq * c.heads * c.D);
      GpuBuffer bt; bt.Size = nLogical; bt.Dtype = AIDN_F32;   // 4-byte elements; holds int32 (AllocateIntBuffer)
      cudaMalloc(&bt.Handle, (size_t)nLogical * 4);
      cudaMemcpy(bt.Handle, table.data(), (size_t)nLogical * 4, cudaMemcpyHostToDevice);
      const bool gqa = c.kvHeads != c.heads;
      if (c.nq == 1 && !gqa) backend.PagedAttentionDecode(dq.buf, dk.buf, dv.buf, bt, dout.buf, c.heads, c.D, c.bs, keyLen, (float)scale);
      else if (c.nq == 1) backend.PagedAttentionDecodeGqa(dq.buf, dk.buf, dv.buf, bt, dout.buf, c.heads, c.kvHeads, c.D, c.bs, keyLen, (float)scale);
      else if (!gqa) backend.PagedAttentionPrefill(dq.buf, dk.buf, dv.buf, bt, dout.buf, c.heads, c.D, c.bs, c.nq, c.start, (float)scale);
      else backend.PagedAttentionPrefillGqa(dq.buf, dk.buf, dv.buf, bt, dout.buf, c.heads, c.kvHeads, c.D, c.bs, c.nq, c.start, (float)scale);
      backend.Synchronize();
      EXPECT(max_abs_diff(dout.download(), want) <= 2e-5, "paged heads=%d kv=%d D=%d bs=%d nq=%d start=%d: %g", c.heads,
             c.kvHeads, c.D, c.bs, c.nq, c.start, max_abs_diff(dout.download(), want));
      bool threw = false;
      try { backend.PagedAttentionDecode(dq.buf, dk.buf, dv.buf, bt, dout.buf, c.heads, c.D, c.bs, nLogical * c.bs + 1, (float)scale); }
      catch (const std::invalid_argument&) { threw = true; }
      EXPECT(threw, "a block table shorter than the sequence must throw");
      cudaFree(bt.Handle);
    }
  }
  {  // DirectGpu/DirectPtxWmmaTests.cs:2110-2113, 2307-2309: one fp32 token, head_dim 64, cache [capacity, heads, 64];
     // DirectGpu/RopeGqaOpenClTests.cs:92-117: interleaved RoPE against the scalar loop
    std::printf("qkv projection + RoPE + cache write, rope_interleaved\n");
    struct Case { int heads, capacity, position; };
    const Case cases[] = {{4, 16, 0}, {8, 64, 17}, {16, 128, 127}};
    for (const Case& c : cases) {
      const int D = 64, model = c.heads * D, half = D / 2;
      auto x = uniform(model, 61 + c.heads), w = uniform(3 * model * model, 62 + c.heads), b = uniform(3 * model, 63);
      for (auto& f : w) f /= std::sqrt((float)model);
      std::vector<float> cosv((size_t)c.capacity * half), sinv((size_t)c.capacity * half);
      for (int pos = 0; pos < c.capacity; ++pos)
        for (int i = 0; i < half; ++i) {
          const double angle = pos / std::pow(10000.0, (2.0 * i) / D);
          cosv[(size_t)pos * half + i] = (float)std::cos(angle);
          sinv[(size_t)pos * half + i] = (float)std::sin(angle);
        }
      std::vector<double> y(3 * model);
      for (int r = 0; r < 3 * model; ++r) {
        double acc = b[r];
        for (int k = 0; k < model; ++k) acc += (double)w[(size_t)r * model + k] * x[k];
        y[r] = acc;
      }
      std::vector<double> wantq(model), wantk((size_t)c.capacity * model, 0.0), wantv((size_t)c.capacity * model, 0.0);
      for (int r = 0; r < 2 * model; r += 2) {
        const int i = (r % D) / 2;
        const double cs = cosv[(size_t)c.position * half + i], sn = sinv[(size_t)c.position * half + i];
        const double e = y[r] * cs - y[r + 1] * sn, o = y[r] * sn + y[r + 1] * cs;
        if (r < model) { wantq[r] = e; wantq[r + 1] = o; }
        else { wantk[(size_t)c.position * model + r - model] = e; wantk[(size_t)c.position * model + r - model + 1] = o; }
      }
      for (int r = 0; r < model; ++r) wantv[(size_t)c.position * model + r] = y[2 * model + r];
      DeviceArray dx(x), dw(w), db(b), dc(cosv), ds(sinv), dq((int64_t)model);
      std::vector<float> zeros((size_t)c.capacity * model, 0.f);
      DeviceArray dk(zeros), dvv(zeros);
      backend.QkvProjectionRoPECacheD64(dx.buf, dw.buf, db.buf, dc.buf, ds.buf, dq.buf, dk.buf, dvv.buf, c.heads, c.capacity, c.position);
      backend.Synchronize();
      EXPECT(max_abs_diff(dq.download(), wantq) <= 2e-5 && max_abs_diff(dk.download(), wantk) <= 2e-5 &&
             max_abs_diff(dvv.download(), wantv) <= 2e-5, "qkv/rope/cache heads=%d capacity=%d position=%d", c.heads, c.capacity, c.position);
      bool threw = false;
      try { backend.QkvProjectionRoPECacheD64(dx.buf, dw.buf, db.buf, dc.buf, ds.buf, dq.buf, dk.buf, dvv.buf, c.heads, c.capacity, c.capacity); }
      catch (const std::invalid_argument&) { threw = true; }
      EXPECT(threw, "position == cacheCapacity must throw");
    }
    {
      const int heads = 3, seqLen = 6, headDim = 8, maxSeq = 32, rows = heads * seqLen, half = headDim / 2;
      auto x = uniform(rows * headDim, 71);
      std::vector<float> cosv(maxSeq * half), sinv(maxSeq * half);
      for (int pos = 0; pos < maxSeq; ++pos)
        for (int i = 0; i < half; ++i) {
          const double angle = pos / std::pow(10000.0, (2.0 * i) / headDim);
          cosv[pos * half + i] = (float)std::cos(angle);
          sinv[pos * half + i] = (float)std::sin(angle);
        }
      for (int start : {0, 5}) {
        std::vector<double> want(x.size());
        for (int row = 0; row < rows; ++row)
          for (int i = 0; i < half; ++i) {
            const int pos = start + row % seqLen;
            const double cs = cosv[pos * half + i], sn = sinv[pos * half + i];
            const double xe = x[row * headDim + 2 * i], xo = x[row * headDim + 2 * i + 1];
            want[row * headDim + 2 * i] = xe * cs - xo * sn;
            want[row * headDim + 2 * i + 1] = xe * sn + xo * cs;
          }
        DeviceArray dx(x), dc(cosv), ds(sinv), dout((int64_t)x.size());
        backend.RopeInterleaved(dx.buf, dc.buf, ds.buf, dout.buf, rows, headDim, seqLen, start);
        backend.Synchronize();
        EXPECT(max_abs_diff(dout.download(), want) <= 1e-6, "rope_interleaved start=%d", start);
      }
    }
  }
  {  // FlashAttentionBackward after FlashAttentionV2: dQ, dK, dV against a scalar reference in double (the formulas of
     // CUDA/Kernels/CudaAttentionKernels.cs:251-390), top-left causal
    std::printf("flash attention backward\n");
    const int B = 2, H = 2, S = 11, D = 16;
    const double scale = 0.25;
    auto q = uniform(B * H * S * D, 81), k = uniform(B * H * S * D, 82), v = uniform(B * H * S * D, 83), go = uniform(B * H * S * D, 84);
    DeviceArray dq_(q), dk_(k), dv_(v), dgo(go), dout((int64_t)B * H * S * D), dstats((int64_t)B * H * S);
    DeviceArray gq((int64_t)B * H * S * D), gk((int64_t)B * H * S * D), gv((int64_t)B * H * S * D);
    backend.FlashAttentionV2(dq_.buf, dk_.buf, dv_.buf, dout.buf, dstats.buf, B, H, S, S, D, (float)scale, true);
    backend.FlashAttentionBackward(dgo.buf, dq_.buf, dk_.buf, dv_.buf, dout.buf, dstats.buf, gq.buf, gk.buf, gv.buf, B, H, S, S, D, (float)scale, true);
    backend.Synchronize();
    std::vector<double> wq((size_t)B * H * S * D, 0.0), wk(wq.size(), 0.0), wv(wq.size(), 0.0);
    for (int bh = 0; bh < B * H; ++bh) {
      const size_t base = (size_t)bh * S * D;
      for (int i = 0; i < S; ++i) {
        std::vector<double> p(S, 0.0), dp(S, 0.0);
        double mx = -1e300, sum = 0, delta = 0;
        for (int j = 0; j <= i; ++j) {
          double dot = 0;
          for (int d = 0; d < D; ++d) dot += (double)q[base + i * D + d] * k[base + j * D + d];
          p[j] = dot * scale; mx = std::max(mx, p[j]);
        }
        for (int j = 0; j <= i; ++j) { p[j] = std::exp(p[j] - mx); sum += p[j]; }
        std::vector<double> o(D, 0.0);
        for (int j = 0; j <= i; ++j) { p[j] /= sum; for (int d = 0; d < D; ++d) o[d] += p[j] * v[base + j * D + d]; }
        for (int d = 0; d < D; ++d) delta += (double)go[base + i * D + d] * o[d];
        for (int j = 0; j <= i; ++j) {
          for (int d = 0; d < D; ++d) dp[j] += (double)go[base + i * D + d] * v[base + j * D + d];
          const double ds = p[j] * (dp[j] - delta);
          for (int d = 0; d < D; ++d) {
            wq[base + i * D + d] += ds * scale * k[base + j * D + d];
            wk[base + j * D + d] += ds * scale * q[base + i * D + d];
            wv[base + j * D + d] += p[j] * go[base + i * D + d];
          }
        }
      }
    }
    EXPECT(max_abs_diff(gq.download(), wq) <= 2e-5 && max_abs_diff(gk.download(), wk) <= 2e-5 && max_abs_diff(gv.download(), wv) <= 2e-5,
           "backward mismatch dq %g dk %g dv %g", max_abs_diff(gq.download(), wq), max_abs_diff(gk.download(), wk), max_abs_diff(gv.download(), wv));
  }
  {  // MultiHeadAttentionForward: fp32 tensors in and out (the engine's contract), a causal [1,1,S,S] keep-mask; the
     // scalar reference in double runs on the bf16-rounded operands (the call rounds fp32 operands to bf16)
    std::printf("multi-head attention forward\n");
    const int B = 2, S = 40, H = 2, Dh = 64, Dm = H * Dh;
    auto rounded = [](std::vector<float> v) { for (auto& f : v) f = __bfloat162float(__float2bfloat16_rn(f)); return v; };
    auto x = rounded(uniform(B * S * Dm, 91));
    std::vector<float> w[4];
    for (int i = 0; i < 4; ++i) { w[i] = uniform(Dm * Dm, 92 + i); for (auto& f : w[i]) f *= 0.1f; w[i] = rounded(w[i]); }
    std::vector<unsigned char> keep((size_t)S * S);
    for (int i = 0; i < S; ++i) for (int j = 0; j < S; ++j) keep[(size_t)i * S + j] = j <= i ? 1 : 0;
    GpuBuffer mask;
    mask.Size = (int64_t)keep.size();
    cudaMalloc(&mask.Handle, keep.size());
    cudaMemcpy(mask.Handle, keep.data(), keep.size(), cudaMemcpyHostToDevice);
    DeviceArray dx(x), dwq(w[0]), dwk(w[1]), dwv(w[2]), dwo(w[3]), dout((int64_t)B * S * Dm);
    const int mshape[4] = {1, 1, S, S};
    const int64_t before = backend.LaunchCount();
    backend.MultiHeadAttentionForward(dx.buf, dwq.buf, dwk.buf, dwv.buf, dwo.buf, dout.buf, B, S, Dm, H, &mask, mshape);
    backend.Synchronize();
    EXPECT(backend.LaunchCount() - before == 8, "expected 5 casts + 3 kernels, got %lld launches", (long long)(backend.LaunchCount() - before));
    auto proj = [&](const std::vector<double>& a, const std::vector<float>& wm) {
      std::vector<double> y((size_t)B * S * Dm, 0.0);
      for (int r = 0; r < B * S; ++r)
        for (int kk = 0; kk < Dm; ++kk) {
          const double av = a[(size_t)r * Dm + kk];
          for (int n = 0; n < Dm; ++n) y[(size_t)r * Dm + n] += av * wm[(size_t)kk * Dm + n];
        }
      return y;
    };
    std::vector<double> xd(x.begin(), x.end());
    auto qd = proj(xd, w[0]), kd = proj(xd, w[1]), vd = proj(xd, w[2]);
    std::vector<double> att((size_t)B * S * Dm, 0.0);
    for (int b = 0; b < B; ++b)
      for (int h = 0; h < H; ++h)
        for (int i = 0; i < S; ++i) {
          std::vector<double> p(S, 0.0);
          double mx = -1e300, sum = 0;
          for (int j = 0; j <= i; ++j) {
            double dot = 0;
            for (int d = 0; d < Dh; ++d) dot += qd[((size_t)b * S + i) * Dm + h * Dh + d] * kd[((size_t)b * S + j) * Dm + h * Dh + d];
            p[j] = dot / std::sqrt((double)Dh); mx = std::max(mx, p[j]);
          }
          for (int j = 0; j <= i; ++j) { p[j] = std::exp(p[j] - mx); sum += p[j]; }
          for (int j = 0; j <= i; ++j)
            for (int d = 0; d < Dh; ++d) att[((size_t)b * S + i) * Dm + h * Dh + d] += p[j] / sum * vd[((size_t)b * S + j) * Dm + h * Dh + d];
        }
    auto want = proj(att, w[3]);
    double mag = 0;
    for (double t : want) mag = std::max(mag, std::fabs(t));
    const double err = max_abs_diff(dout.download(), want);
    EXPECT(err <= 2e-2 * mag, "mha forward: max error %g against magnitude %g", err, mag);
    bool threw = false;
    try { backend.MultiHeadAttentionForward(dx.buf, dwq.buf, dwk.buf, dwv.buf, dwo.buf, dout.buf, B, S, Dm, 3); } catch (const std::invalid_argument&) { threw = true; }
    EXPECT(threw, "dModel %% numHeads != 0 must throw");
    threw = false;
    try { backend.MultiHeadAttentionForward(dx.buf, dwq.buf, dwk.buf, dwv.buf, dwo.buf, dout.buf, B, S, Dm, 0); } catch (const std::invalid_argument&) { threw = true; }
    EXPECT(threw, "numHeads = 0 must throw");
    // exact route: the same call in fp32 arithmetic meets the reference's own 1e-4 (MultiHeadAttentionForwardTests.cs:123);
    // so does a head size the tensor cores do not take (8 heads of 16)
    DeviceArray dexact((int64_t)B * S * Dm);
    backend.MultiHeadAttentionForward(dx.buf, dwq.buf, dwk.buf, dwv.buf, dwo.buf, dexact.buf, B, S, Dm, H, &mask, mshape, true);
    backend.Synchronize();
    EXPECT(max_abs_diff(dexact.download(), want) <= 1e-4, "mha forward, exact route: max error %g", max_abs_diff(dexact.download(), want));
    cudaFree(mask.Handle);
  }
  {  // argument errors throw, as ArgumentOutOfRangeException / ArgumentException do in the reference
    std::printf("argument errors\n");
    std::vector<float> z(64, 0.f);
    DeviceArray a(z), out(64);
    bool threw = false;
    try { backend.ScaledDotProductAttention(a.buf, a.buf, a.buf, out.buf, nullptr, nullptr, 0, 1, 1, 1, 8, 1.f, false); } catch (const std::invalid_argument&) { threw = true; }
    EXPECT(threw, "batch = 0 must throw");
    threw = false;
    try { backend.ScaledDotProductAttention(a.buf, a.buf, a.buf, out.buf, nullptr, nullptr, 1, 6, 1, 1, 8, 1.f, false, 0.f, 4); } catch (const std::invalid_argument&) { threw = true; }
    EXPECT(threw, "numHeads %% numKVHeads != 0 must throw");
    threw = false;
    try { backend.ScaledDotProductAttention(a.buf, a.buf, a.buf, out.buf, nullptr, nullptr, 4, 4, 4, 4, 8, 1.f, false); } catch (const std::invalid_argument&) { threw = true; }
    EXPECT(threw, "undersized buffers must throw");
  }
  std::printf(g_failed ? "%d case(s) FAILED\n" : "all cases passed (%d failures)\n", g_failed);
  cudaStreamDestroy(stream);
  return g_failed ? 1 : 0;
}
