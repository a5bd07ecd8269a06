// C++ host-side mirror of the attention slice of the reference's CUDA backend, on top of the C ABI
// (include/aidn_sdpa.h).  The reference host is C# (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/CudaBackend.cs);
// this class keeps its method names, argument order, argument meaning and error behaviour so that a port of the
// reference's backend tests reads the same:
//
//   ScaledDotProductAttention  CudaBackend.cs:8322-8379     FlashAttention        CudaBackend.cs:8522-8538
//   FlashAttentionV2           CudaBackend.cs:8540-8578     GroupedQueryAttention CudaBackend.cs:8721-8759
//   FlashDecode                CudaBackend.cs:2968-3021     PagedAttention{Decode,Prefill}{,Gqa} CudaBackend.cs:2845-2966
//   QkvProjectionRoPECacheD64  CudaBackend.cs:8389-8439     RopeInterleaved       CudaBackend.cs:8441-8470
//   FlashAttentionBackward     CudaBackend.cs:8580-8604     MultiHeadAttentionForward  Engines/IEngine.cs:4201-4208
//
// ArgumentException / ArgumentOutOfRangeException map to std::invalid_argument, InvalidOperationException to
// std::runtime_error.  There is no CPU fallback: a failing call throws.
#pragma once

#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <tuple>

#include "../../../../include/aidn_sdpa.h"

namespace aidn {
namespace host {

// Mirror of IGpuBuffer (Engines/DirectGpu/IDirectGpuBackend.cs:3776-3803): Size is an element count.
struct GpuBuffer {
  void* Handle = nullptr;
  int64_t Size = 0;
  aidn_dtype Dtype = AIDN_F32;
  int64_t SizeInBytes() const { return Size * (Dtype == AIDN_F32 ? 4 : 2); }
};

class CudaBackend {
 public:
  // `stream` is the backend's single CUstream / cudaStream_t (CudaBackend.cs:371-375).
  CudaBackend(int device, void* stream);
  ~CudaBackend();
  CudaBackend(const CudaBackend&) = delete;
  CudaBackend& operator=(const CudaBackend&) = delete;

  void ScaledDotProductAttention(const GpuBuffer& query, const GpuBuffer& key, const GpuBuffer& value,
                                 const GpuBuffer& output, const GpuBuffer* attentionWeights, const GpuBuffer* mask,
                                 int batch, int numHeads, int seqQ, int seqK, int headDim, float scale, bool isCausal,
                                 float softcap = 0.0f, int numKVHeads = 0);
  void FlashAttention(const GpuBuffer& query, const GpuBuffer& key, const GpuBuffer& value, const GpuBuffer& output,
                      const GpuBuffer* mask, int batch, int numHeads, int seqLen, int headDim, float scale,
                      bool isCausal);
  void FlashAttentionV2(const GpuBuffer& query, const GpuBuffer& key, const GpuBuffer& value, const GpuBuffer& output,
                        const GpuBuffer& softmaxStats, int batch, int numHeads, int seqQ, int seqK, int headDim,
                        float scale, bool isCausal, const GpuBuffer* attentionBias = nullptr, int biasBatchStride = 0);
  void GroupedQueryAttention(const GpuBuffer& query, const GpuBuffer& key, const GpuBuffer& value,
                             const GpuBuffer& output, const GpuBuffer* attentionWeights, int batch, int numQHeads,
                             int numKVHeads, int seqQ, int seqK, int headDim, float scale, bool isCausal);
  // The reference allocates and returns the output buffer; here the caller passes it (heads * headDim elements).
  void FlashDecode(const GpuBuffer& q, const GpuBuffer& k, const GpuBuffer& v, const GpuBuffer& output, int heads,
                   int kvHeads, int headDim, int seqLen, float scale, int splits = 0);

  // Paged K/V (IDirectGpuBackend.cs:3619-3632): pools [MaxBlocks, blockSize, kvHeads, headDim], int32 block table,
  // q / output [numQueries, heads, headDim].  The reference returns a new buffer; here the caller passes `output`.
  void PagedAttentionDecode(const GpuBuffer& q, const GpuBuffer& kcache, const GpuBuffer& vcache,
                            const GpuBuffer& blockTable, const GpuBuffer& output, int heads, int headDim, int blockSize,
                            int seqLen, float scale);
  void PagedAttentionPrefill(const GpuBuffer& q, const GpuBuffer& kcache, const GpuBuffer& vcache,
                             const GpuBuffer& blockTable, const GpuBuffer& output, int heads, int headDim,
                             int blockSize, int numQueries, int startPos, float scale);
  void PagedAttentionDecodeGqa(const GpuBuffer& q, const GpuBuffer& kcache, const GpuBuffer& vcache,
                               const GpuBuffer& blockTable, const GpuBuffer& output, int heads, int kvHeads,
                               int headDim, int blockSize, int seqLen, float scale);
  void PagedAttentionPrefillGqa(const GpuBuffer& q, const GpuBuffer& kcache, const GpuBuffer& vcache,
                                const GpuBuffer& blockTable, const GpuBuffer& output, int heads, int kvHeads,
                                int headDim, int blockSize, int numQueries, int startPos, float scale);

  // Backward of FlashAttentionV2 (CudaBackend.cs:8580-8604): fp32 gradient buffers, statistics from the forward.
  void FlashAttentionBackward(const GpuBuffer& gradOutput, const GpuBuffer& query, const GpuBuffer& key,
                              const GpuBuffer& value, const GpuBuffer& output, const GpuBuffer& softmaxStats,
                              const GpuBuffer& gradQuery, const GpuBuffer& gradKey, const GpuBuffer& gradValue, int batch,
                              int numHeads, int seqQ, int seqK, int headDim, float scale, bool isCausal,
                              const GpuBuffer* attentionBias = nullptr, int biasBatchStride = 0);

  // The decode step in front of attention (CudaBackend.cs:8389-8439 and :8441-8470).
  void QkvProjectionRoPECacheD64(const GpuBuffer& input, const GpuBuffer& packedWeights, const GpuBuffer& bias,
                                 const GpuBuffer& cosine, const GpuBuffer& sine, const GpuBuffer& query,
                                 const GpuBuffer& keyCache, const GpuBuffer& valueCache, int heads, int cacheCapacity,
                                 int position);
  void RopeInterleaved(const GpuBuffer& input, const GpuBuffer& cos, const GpuBuffer& sin, const GpuBuffer& output,
                       int rows, int headDim, int seqLen, int startPosition);

  // The in-library caller of attention (IEngine.cs:4201-4208; checks of CpuEngine.MultiHeadAttention.cs:76-103):
  // input / output [batch, seq, dModel], four [dModel, dModel] weights applied as x * W, optional boolean keep-mask
  // whose four dimensions `maskShape` broadcast to [batch, numHeads, seq, seq].  With head sizes 64 / 128 (dModel a
  // multiple of 128) fp32 buffers are rounded to bf16 on the way in and the tensor cores do the arithmetic; any other
  // shape, or exact == true with all-fp32 buffers, runs the fp32 route (the 1e-4 bound of the reference's tests).
  void MultiHeadAttentionForward(const GpuBuffer& input, const GpuBuffer& qWeight, const GpuBuffer& kWeight,
                                 const GpuBuffer& vWeight, const GpuBuffer& outWeight, const GpuBuffer& output, int batch,
                                 int seq, int dModel, int numHeads, const GpuBuffer* mask = nullptr,
                                 const int* maskShape = nullptr, bool exact = false);

  void Synchronize();
  int64_t LaunchCount() const { return launch_count_; }   // kernels enqueued (GpuLaunchProbe, CudaBackend.cs:5407)
  int LastPath() const { return last_path_; }             // aidn_path of the last call

 private:
  using Key = std::tuple<int, int, int, int, int, int, int, int, int, float, int, int64_t>;
  aidn_sdpa_t Handle(const aidn_sdpa_desc& d);
  void Run(aidn_sdpa_t h, aidn_sdpa_args& a, const aidn_paged_kv* paged = nullptr);
  void Paged(const char* op, const GpuBuffer& q, const GpuBuffer& kcache, const GpuBuffer& vcache,
             const GpuBuffer& blockTable, const GpuBuffer& output, int heads, int kvHeads, int headDim, int blockSize,
             int numQueries, int64_t keyLen, int startPos, float scale);
  static void Check(int status, const char* where);

  int device_;
  void* stream_;
  std::map<Key, aidn_sdpa_t> handles_;
  void* workspace_ = nullptr;
  int64_t workspace_bytes_ = 0;
  int64_t launch_count_ = 0;
  int last_path_ = 0;
};

}  // namespace host
}  // namespace aidn
