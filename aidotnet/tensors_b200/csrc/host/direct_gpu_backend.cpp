#include "direct_gpu_backend.hpp"

#include <cuda_runtime.h>

#include <cmath>
#include <cstring>

namespace aidn {
namespace host {

void CudaBackend::Check(int status, const char* where) {
  if (status == AIDN_OK) return;
  const std::string msg = std::string(where) + ": " + aidn_sdpa_last_error();
  if (status == AIDN_EINVAL) throw std::invalid_argument(msg);
  throw std::runtime_error(msg);
}

CudaBackend::CudaBackend(int device, void* stream) : device_(device), stream_(stream) {
  if (cudaSetDevice(device) != cudaSuccess) throw std::runtime_error("CudaBackend: cannot select the device");
  if (!aidn_sdpa_device_supported(device))
    throw std::runtime_error("CudaBackend: the device is not compute capability 10.x; there is no other path");
}

CudaBackend::~CudaBackend() {
  for (auto& kv : handles_) aidn_sdpa_destroy(kv.second);
  if (workspace_) cudaFree(workspace_);
}

aidn_sdpa_t CudaBackend::Handle(const aidn_sdpa_desc& d) {
  const Key key{d.qkv_dtype, d.out_dtype, d.head_dim, d.num_q_heads, d.num_kv_heads, d.causal, d.causal_bottom_right,
                d.mask_kind, d.emit_lse, d.softcap, d.decode_chunk, d.causal_offset};
  auto it = handles_.find(key);
  if (it != handles_.end()) return it->second;
  aidn_sdpa_t h = nullptr;
  Check(aidn_sdpa_create(&d, &h), "aidn_sdpa_create");
  handles_[key] = h;
  return h;
}

void CudaBackend::Run(aidn_sdpa_t h, aidn_sdpa_args& a, const aidn_paged_kv* paged) {
  const int64_t need = aidn_sdpa_workspace_bytes(h, a.batch, a.seq_q, a.seq_kv);
  if (need < 0) Check(AIDN_EINVAL, "aidn_sdpa_workspace_bytes");
  if (need > workspace_bytes_) {   // grown outside of launch, like the reference's pooled scratch buffers
    if (workspace_) cudaFree(workspace_);
    workspace_ = nullptr;
    workspace_bytes_ = 0;
    if (cudaMalloc(&workspace_, (size_t)need) != cudaSuccess) throw std::runtime_error("CudaBackend: out of device memory");
    workspace_bytes_ = need;
  }
  a.workspace = need > 0 ? workspace_ : nullptr;
  a.workspace_bytes = need > 0 ? workspace_bytes_ : 0;
  if (paged) Check(aidn_sdpa_launch_paged(h, &a, paged, stream_), "aidn_sdpa_launch_paged");
  else Check(aidn_sdpa_launch(h, &a, stream_), "aidn_sdpa_launch");
  launch_count_ += aidn_sdpa_last_launch_count(h);
  last_path_ = aidn_sdpa_last_path(h);
}

void CudaBackend::Synchronize() {
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)) != cudaSuccess)
    throw std::runtime_error("CudaBackend: stream synchronisation failed");
}

static aidn_sdpa_desc base_desc(int device, const GpuBuffer& q, const GpuBuffer& out, int headDim, int heads, int kvHeads) {
  aidn_sdpa_desc d;
  std::memset(&d, 0, sizeof(d));
  d.device = device;
  d.qkv_dtype = q.Dtype;
  d.out_dtype = out.Dtype;
  d.head_dim = headDim;
  d.num_q_heads = heads;
  d.num_kv_heads = kvHeads;
  return d;
}

void CudaBackend::ScaledDotProductAttention(const GpuBuffer& query, const GpuBuffer& key, const GpuBuffer& value,
                                            const GpuBuffer& output, const GpuBuffer* attentionWeights,
                                            const GpuBuffer* mask, int batch, int numHeads, int seqQ, int seqK,
                                            int headDim, float scale, bool isCausal, float softcap, int numKVHeads) {
  if (batch <= 0 || numHeads <= 0 || seqQ <= 0 || seqK <= 0 || headDim <= 0)
    throw std::invalid_argument("Attention dimensions must be positive.");
  const int kvHeads = numKVHeads > 0 ? numKVHeads : numHeads;
  if (numHeads % kvHeads != 0) throw std::invalid_argument("numHeads must be an integer multiple of numKVHeads.");
  const int64_t querySize = (int64_t)batch * numHeads * seqQ * headDim;
  const int64_t keyValueSize = (int64_t)batch * kvHeads * seqK * headDim;
  const int64_t weightsSize = (int64_t)batch * numHeads * seqQ * seqK;
  if (query.Size < querySize || key.Size < keyValueSize || value.Size < keyValueSize || output.Size < querySize)
    throw std::invalid_argument("Attention tensor buffers are smaller than the requested dimensions.");
  if (attentionWeights && (attentionWeights->Size < weightsSize || attentionWeights->Dtype != AIDN_F32))
    throw std::invalid_argument("The attention-weights buffer is too small.");   // CudaBackend.cs:8343-8344
  if (mask && mask->Size < (int64_t)seqQ * seqK)
    throw std::invalid_argument("The attention mask must contain at least seqQ * seqK elements.");
  aidn_sdpa_desc d = base_desc(device_, query, output, headDim, numHeads, kvHeads);
  d.causal = isCausal ? 1 : 0;
  d.causal_bottom_right = 1;                 // CudaAttentionKernels.cs:66: qPos = qi + (seqK - seqQ)
  d.softcap = softcap;
  d.mask_kind = mask ? AIDN_MASK_KEEP_F32 : AIDN_MASK_NONE;   // the engine uploads bool masks as floats, 0.0f = masked
  aidn_sdpa_args a;
  std::memset(&a, 0, sizeof(a));
  a.q = query.Handle; a.k = key.Handle; a.v = value.Handle; a.out = output.Handle;
  a.batch = batch; a.seq_q = seqQ; a.seq_kv = seqK; a.scale = scale;
  a.weights = attentionWeights ? static_cast<float*>(attentionWeights->Handle) : nullptr;
  if (mask) {
    a.mask = mask->Handle;
    const bool full = mask->Size >= weightsSize;   // maskMode rule, CudaBackend.cs:8355
    a.mask_stride[0] = full ? (int64_t)numHeads * seqQ * seqK : 0;
    a.mask_stride[1] = full ? (int64_t)seqQ * seqK : 0;
    a.mask_stride[2] = seqK;
    a.mask_stride[3] = 1;
  }
  Run(Handle(d), a);
}

void CudaBackend::FlashAttentionV2(const GpuBuffer& query, const GpuBuffer& key, const GpuBuffer& value,
                                   const GpuBuffer& output, const GpuBuffer& softmaxStats, int batch, int numHeads,
                                   int seqQ, int seqK, int headDim, float scale, bool isCausal,
                                   const GpuBuffer* attentionBias, int biasBatchStride) {
  if (batch <= 0 || numHeads <= 0 || seqQ <= 0 || seqK <= 0 || headDim <= 0)
    throw std::invalid_argument("Attention dimensions must be positive.");
  if (softmaxStats.Size < (int64_t)batch * numHeads * seqQ || softmaxStats.Dtype != AIDN_F32)
    throw std::invalid_argument("softmaxStats must hold batch*heads*seqQ fp32 values");
  aidn_sdpa_desc d = base_desc(device_, query, output, headDim, numHeads, numHeads);
  d.causal = isCausal ? 1 : 0;
  d.causal_bottom_right = 0;                 // CudaAttentionKernels.cs:197: ki > qi masked (top-left)
  d.causal_offset = 0;
  d.emit_lse = 1;
  d.mask_kind = attentionBias ? AIDN_MASK_ADD_F32 : AIDN_MASK_NONE;
  aidn_sdpa_args a;
  std::memset(&a, 0, sizeof(a));
  a.q = query.Handle; a.k = key.Handle; a.v = value.Handle; a.out = output.Handle;
  a.lse = static_cast<float*>(softmaxStats.Handle);
  a.batch = batch; a.seq_q = seqQ; a.seq_kv = seqK; a.scale = scale;
  if (attentionBias) {
    a.mask = attentionBias->Handle;
    a.mask_stride[0] = biasBatchStride;      // 0 broadcasts a [H,Sq,Sk] bias over the batch
    a.mask_stride[1] = (int64_t)seqQ * seqK;
    a.mask_stride[2] = seqK;
    a.mask_stride[3] = 1;
  }
  Run(Handle(d), a);
}

void CudaBackend::FlashAttention(const GpuBuffer& query, const GpuBuffer& key, const GpuBuffer& value,
                                 const GpuBuffer& output, const GpuBuffer* mask, int batch, int numHeads, int seqLen,
                                 int headDim, float scale, bool isCausal) {
  if (mask) {
    ScaledDotProductAttention(query, key, value, output, nullptr, mask, batch, numHeads, seqLen, seqLen, headDim, scale,
                              isCausal);
    return;
  }
  GpuBuffer stats;
  stats.Size = (int64_t)batch * numHeads * seqLen;
  stats.Dtype = AIDN_F32;
  if (cudaMalloc(&stats.Handle, (size_t)stats.SizeInBytes()) != cudaSuccess)
    throw std::runtime_error("CudaBackend: out of device memory");
  try {
    FlashAttentionV2(query, key, value, output, stats, batch, numHeads, seqLen, seqLen, headDim, scale, isCausal);
  } catch (...) {
    cudaFree(stats.Handle);
    throw;
  }
  Synchronize();
  cudaFree(stats.Handle);
}

void CudaBackend::GroupedQueryAttention(const GpuBuffer& query, const GpuBuffer& key, const GpuBuffer& value,
                                        const GpuBuffer& output, const GpuBuffer* attentionWeights, int batch,
                                        int numQHeads, int numKVHeads, int seqQ, int seqK, int headDim, float scale,
                                        bool isCausal) {
  if (batch <= 0 || numQHeads <= 0 || seqQ <= 0 || seqK <= 0 || headDim <= 0)
    throw std::invalid_argument("Attention dimensions must be positive.");
  if (numKVHeads <= 0 || numQHeads % numKVHeads != 0)
    throw std::invalid_argument("numQHeads must be divisible by numKVHeads");
  if (attentionWeights && (attentionWeights->Size < (int64_t)batch * numQHeads * seqQ * seqK || attentionWeights->Dtype != AIDN_F32))
    throw std::invalid_argument("The attention-weights buffer is too small.");
  aidn_sdpa_desc d = base_desc(device_, query, output, headDim, numQHeads, numKVHeads);
  d.causal = isCausal ? 1 : 0;
  d.causal_bottom_right = 0;                 // CudaAttentionKernels.cs:598 (top-left)
  aidn_sdpa_args a;
  std::memset(&a, 0, sizeof(a));
  a.q = query.Handle; a.k = key.Handle; a.v = value.Handle; a.out = output.Handle;
  a.batch = batch; a.seq_q = seqQ; a.seq_kv = seqK; a.scale = scale;
  a.weights = attentionWeights ? static_cast<float*>(attentionWeights->Handle) : nullptr;   // CudaBackend.cs:8731-8732
  Run(Handle(d), a);
}

void CudaBackend::FlashDecode(const GpuBuffer& q, const GpuBuffer& k, const GpuBuffer& v, const GpuBuffer& output,
                              int heads, int kvHeads, int headDim, int seqLen, float scale, int splits) {
  if (heads <= 0 || kvHeads <= 0 || headDim <= 0 || heads % kvHeads != 0)
    throw std::invalid_argument("heads must be a positive multiple of kvHeads");
  if (seqLen <= 0) throw std::invalid_argument("seqLen must be positive");
  const int64_t kvSize = (int64_t)seqLen * kvHeads * headDim;
  if (q.Size < (int64_t)heads * headDim || k.Size < kvSize || v.Size < kvSize || output.Size < (int64_t)heads * headDim)
    throw std::invalid_argument("FlashDecode buffers are smaller than the requested dimensions.");
  aidn_sdpa_desc d = base_desc(device_, q, output, headDim, heads, kvHeads);
  if (splits > 0) {
    const int s = splits < seqLen ? splits : seqLen;
    int chunk = (seqLen + s - 1) / s;
    chunk = (chunk + 7) / 8 * 8;
    d.decode_chunk = chunk < 8 ? 8 : chunk;
  }
  aidn_sdpa_args a;
  std::memset(&a, 0, sizeof(a));
  a.q = q.Handle; a.k = k.Handle; a.v = v.Handle; a.out = output.Handle;
  a.batch = 1; a.seq_q = 1; a.seq_kv = seqLen; a.scale = scale;
  // the cache is stored [seqLen, kvHeads, headDim] (CudaFlashDecodeKernels.cs): (B, H, S) strides in elements
  a.k_stride[0] = 0; a.k_stride[1] = headDim; a.k_stride[2] = (int64_t)kvHeads * headDim;
  a.v_stride[0] = 0; a.v_stride[1] = headDim; a.v_stride[2] = (int64_t)kvHeads * headDim;
  Run(Handle(d), a);
}

// ---- paged K/V ------------------------------------------------------------------------------------------------
// Guards as GpuKernelGuards.Attention / Gqa / PagedAttentionBuffers (Engines/DirectGpu/GpuKernelGuards.cs:15-35, 83-99).
void CudaBackend::Paged(const char* op, const GpuBuffer& q, const GpuBuffer& kcache, const GpuBuffer& vcache,
                        const GpuBuffer& blockTable, const GpuBuffer& output, int heads, int kvHeads, int headDim,
                        int blockSize, int numQueries, int64_t keyLen, int startPos, float scale) {
  const std::string o(op);
  if (heads <= 0) throw std::invalid_argument(o + ": heads must be > 0.");
  if (headDim <= 0 || headDim > 256) throw std::invalid_argument(o + ": headDim must be in [1, 256].");
  if (blockSize <= 0) throw std::invalid_argument(o + ": blockSize must be > 0.");
  if (numQueries <= 0 || keyLen <= 0) throw std::invalid_argument(o + ": sequence/query count must be > 0.");
  if (kvHeads <= 0 || kvHeads > heads || heads % kvHeads != 0)
    throw std::invalid_argument(o + ": kvHeads must satisfy 1 <= kvHeads <= heads and heads % kvHeads == 0.");
  const int64_t qSize = (int64_t)numQueries * heads * headDim;
  if (q.Size < qSize || output.Size < qSize) throw std::invalid_argument(o + ": q / output are smaller than numQueries*heads*headDim.");
  if (blockTable.Size < (keyLen + blockSize - 1) / blockSize) throw std::invalid_argument(o + ": blockTable is too short.");
  if (!kcache.Handle || !vcache.Handle) throw std::invalid_argument(o + ": K/V pools must not be null.");
  if (kcache.Size <= 0 || kcache.Size != vcache.Size)
    throw std::invalid_argument(o + ": kcache/vcache must be equal-sized, non-empty K/V pools.");
  const int64_t perBlock = (int64_t)blockSize * kvHeads * headDim;
  if (kcache.Size % perBlock != 0) throw std::invalid_argument(o + ": K/V pool size is not a whole number of blocks.");
  aidn_sdpa_desc d = base_desc(device_, q, output, headDim, heads, kvHeads);
  d.causal = numQueries > 1 ? 1 : 0;
  d.causal_bottom_right = 0;
  d.causal_offset = startPos;    // query qi sees keys 0..startPos+qi (CudaPagedAttentionKernels.cs:67)
  aidn_sdpa_args a;
  std::memset(&a, 0, sizeof(a));
  a.q = q.Handle; a.k = kcache.Handle; a.v = vcache.Handle; a.out = output.Handle;
  a.batch = 1; a.seq_q = numQueries; a.seq_kv = keyLen; a.scale = scale;
  // q / output are [numQueries, heads, headDim]: (B, H, S) strides in elements
  a.q_stride[0] = a.o_stride[0] = qSize;
  a.q_stride[1] = a.o_stride[1] = headDim;
  a.q_stride[2] = a.o_stride[2] = (int64_t)heads * headDim;
  aidn_paged_kv pg;
  std::memset(&pg, 0, sizeof(pg));
  pg.block_table = static_cast<const int32_t*>(blockTable.Handle);
  pg.block_size = blockSize;
  pg.num_blocks = (int32_t)(kcache.Size / perBlock);
  Run(Handle(d), a, &pg);
}

void CudaBackend::PagedAttentionDecode(const GpuBuffer& q, const GpuBuffer& kcache, const GpuBuffer& vcache,
                                       const GpuBuffer& blockTable, const GpuBuffer& output, int heads, int headDim,
                                       int blockSize, int seqLen, float scale) {
  Paged("PagedAttentionDecode", q, kcache, vcache, blockTable, output, heads, heads, headDim, blockSize, 1, seqLen, 0, scale);
}

void CudaBackend::PagedAttentionDecodeGqa(const GpuBuffer& q, const GpuBuffer& kcache, const GpuBuffer& vcache,
                                          const GpuBuffer& blockTable, const GpuBuffer& output, int heads, int kvHeads,
                                          int headDim, int blockSize, int seqLen, float scale) {
  Paged("PagedAttentionDecodeGqa", q, kcache, vcache, blockTable, output, heads, kvHeads, headDim, blockSize, 1, seqLen, 0,
        scale);
}

void CudaBackend::PagedAttentionPrefill(const GpuBuffer& q, const GpuBuffer& kcache, const GpuBuffer& vcache,
                                        const GpuBuffer& blockTable, const GpuBuffer& output, int heads, int headDim,
                                        int blockSize, int numQueries, int startPos, float scale) {
  if (startPos < 0) throw std::invalid_argument("PagedAttentionPrefill: startPos must be >= 0.");
  Paged("PagedAttentionPrefill", q, kcache, vcache, blockTable, output, heads, heads, headDim, blockSize, numQueries,
        (int64_t)startPos + numQueries, startPos, scale);
}

void CudaBackend::PagedAttentionPrefillGqa(const GpuBuffer& q, const GpuBuffer& kcache, const GpuBuffer& vcache,
                                           const GpuBuffer& blockTable, const GpuBuffer& output, int heads, int kvHeads,
                                           int headDim, int blockSize, int numQueries, int startPos, float scale) {
  if (startPos < 0) throw std::invalid_argument("PagedAttentionPrefillGqa: startPos must be >= 0.");
  Paged("PagedAttentionPrefillGqa", q, kcache, vcache, blockTable, output, heads, kvHeads, headDim, blockSize, numQueries,
        (int64_t)startPos + numQueries, startPos, scale);
}

void CudaBackend::FlashAttentionBackward(const GpuBuffer& gradOutput, const GpuBuffer& query, const GpuBuffer& key,
                                         const GpuBuffer& value, const GpuBuffer& output, const GpuBuffer& softmaxStats,
                                         const GpuBuffer& gradQuery, const GpuBuffer& gradKey, const GpuBuffer& gradValue,
                                         int batch, int numHeads, int seqQ, int seqK, int headDim, float scale,
                                         bool isCausal, const GpuBuffer* attentionBias, int biasBatchStride) {
  if (batch <= 0 || numHeads <= 0 || seqQ <= 0 || seqK <= 0 || headDim <= 0)
    throw std::invalid_argument("Attention dimensions must be positive.");
  const int64_t qsz = (int64_t)batch * numHeads * seqQ * headDim, ksz = (int64_t)batch * numHeads * seqK * headDim;
  if (gradOutput.Size < qsz || query.Size < qsz || output.Size < qsz || gradQuery.Size < qsz || key.Size < ksz ||
      value.Size < ksz || gradKey.Size < ksz || gradValue.Size < ksz || softmaxStats.Size < (int64_t)batch * numHeads * seqQ)
    throw std::invalid_argument("Attention tensor buffers are smaller than the requested dimensions.");
  if (gradQuery.Dtype != AIDN_F32 || gradKey.Dtype != AIDN_F32 || gradValue.Dtype != AIDN_F32 || softmaxStats.Dtype != AIDN_F32)
    throw std::invalid_argument("gradients and softmaxStats are fp32 buffers");
  aidn_sdpa_desc d = base_desc(device_, query, output, headDim, numHeads, numHeads);
  d.causal = isCausal ? 1 : 0;
  d.causal_bottom_right = 0;
  d.emit_lse = 1;
  d.mask_kind = attentionBias ? AIDN_MASK_ADD_F32 : AIDN_MASK_NONE;
  aidn_sdpa_t h = Handle(d);
  const int64_t need = aidn_sdpa_backward_workspace_bytes(h, batch, seqQ);
  if (need < 0) Check(AIDN_EINVAL, "aidn_sdpa_backward_workspace_bytes");
  if (need > workspace_bytes_) {
    if (workspace_) cudaFree(workspace_);
    workspace_ = nullptr;
    workspace_bytes_ = 0;
    if (cudaMalloc(&workspace_, (size_t)need) != cudaSuccess) throw std::runtime_error("CudaBackend: out of device memory");
    workspace_bytes_ = need;
  }
  aidn_sdpa_bwd_args a;
  std::memset(&a, 0, sizeof(a));
  a.fwd.q = query.Handle; a.fwd.k = key.Handle; a.fwd.v = value.Handle; a.fwd.out = output.Handle;
  a.fwd.lse = static_cast<float*>(softmaxStats.Handle);
  a.fwd.batch = batch; a.fwd.seq_q = seqQ; a.fwd.seq_kv = seqK; a.fwd.scale = scale;
  a.fwd.workspace = workspace_; a.fwd.workspace_bytes = workspace_bytes_;
  if (attentionBias) {
    a.fwd.mask = attentionBias->Handle;
    a.fwd.mask_stride[0] = biasBatchStride; a.fwd.mask_stride[1] = (int64_t)seqQ * seqK;
    a.fwd.mask_stride[2] = seqK; a.fwd.mask_stride[3] = 1;
  }
  a.dout = gradOutput.Handle;
  a.dq = static_cast<float*>(gradQuery.Handle); a.dk = static_cast<float*>(gradKey.Handle);
  a.dv = static_cast<float*>(gradValue.Handle);
  Check(aidn_sdpa_backward(h, &a, stream_), "aidn_sdpa_backward");
  launch_count_ += aidn_sdpa_last_launch_count(h);
}

// ---- the in-library caller of attention ----------------------------------------------------------------------------
void CudaBackend::MultiHeadAttentionForward(const GpuBuffer& input, const GpuBuffer& qWeight, const GpuBuffer& kWeight,
                                            const GpuBuffer& vWeight, const GpuBuffer& outWeight, const GpuBuffer& output,
                                            int batch, int seq, int dModel, int numHeads, const GpuBuffer* mask,
                                            const int* maskShape, bool exact) {
  if (!input.Handle || !qWeight.Handle || !kWeight.Handle || !vWeight.Handle || !outWeight.Handle || !output.Handle)
    throw std::invalid_argument("MultiHeadAttentionForward: null buffer");
  if (numHeads <= 0) throw std::invalid_argument("numHeads must be positive.");
  if (batch <= 0 || seq <= 0 || dModel <= 0)
    throw std::invalid_argument("MultiHeadAttentionForward expects a non-empty [B, seq, dModel] input.");
  if (dModel % numHeads != 0) throw std::invalid_argument("dModel must be divisible by numHeads.");
  const int64_t wsz = (int64_t)dModel * dModel, asz = (int64_t)batch * seq * dModel;
  if (qWeight.Size != wsz || kWeight.Size != wsz || vWeight.Size != wsz || outWeight.Size != wsz)
    throw std::invalid_argument("the projection weights must be [dModel, dModel].");
  if (input.Size < asz || output.Size < asz)
    throw std::invalid_argument("input / output buffers are smaller than [batch, seq, dModel].");
  if (kWeight.Dtype != qWeight.Dtype || vWeight.Dtype != qWeight.Dtype || outWeight.Dtype != qWeight.Dtype)
    throw std::invalid_argument("the four weights must share one dtype");
  const int head = dModel / numHeads;
  const bool tensor_shape = (head == 64 || head == 128) && dModel % 128 == 0;
  aidn_dtype compute = (tensor_shape && !exact) ? AIDN_BF16 : AIDN_F32;
  for (const GpuBuffer* b : {&input, &qWeight, &output})
    if (b->Dtype != AIDN_F32) compute = b->Dtype;
  for (const GpuBuffer* b : {&input, &qWeight, &output})
    if (b->Dtype != AIDN_F32 && b->Dtype != compute) throw std::invalid_argument("16-bit buffers must share one dtype");
  aidn_sdpa_desc d;
  std::memset(&d, 0, sizeof(d));
  d.device = device_;
  d.qkv_dtype = compute;
  d.out_dtype = compute;
  d.head_dim = dModel / numHeads;
  d.num_q_heads = numHeads;
  d.num_kv_heads = numHeads;
  d.mask_kind = mask ? AIDN_MASK_KEEP_U8 : AIDN_MASK_NONE;
  aidn_mha_args a;
  std::memset(&a, 0, sizeof(a));
  if (mask) {
    if (!maskShape) throw std::invalid_argument("maskShape must give the 4 mask dimensions");
    const int full[4] = {batch, numHeads, seq, seq};
    const int64_t dense[4] = {(int64_t)maskShape[1] * maskShape[2] * maskShape[3], (int64_t)maskShape[2] * maskShape[3],
                              maskShape[3], 1};
    for (int ax = 0; ax < 4; ++ax) {
      if (maskShape[ax] != 1 && maskShape[ax] != full[ax])
        throw std::invalid_argument("mask is not broadcastable to [batch, numHeads, seq, seq]");
      a.mask_stride[ax] = (maskShape[ax] == 1 && full[ax] != 1) ? 0 : dense[ax];
    }
    a.mask = mask->Handle;
  }
  aidn_sdpa_t h = Handle(d);
  const int64_t need = aidn_mha_workspace_bytes(h, batch, seq, input.Dtype, qWeight.Dtype);
  if (need < 0) Check(AIDN_EUNSUPPORTED, "aidn_mha_workspace_bytes");
  if (need > workspace_bytes_) {
    if (workspace_) cudaFree(workspace_);
    workspace_ = nullptr;
    workspace_bytes_ = 0;
    if (cudaMalloc(&workspace_, (size_t)need) != cudaSuccess) throw std::runtime_error("CudaBackend: out of device memory");
    workspace_bytes_ = need;
  }
  a.input = input.Handle;
  a.q_weight = qWeight.Handle; a.k_weight = kWeight.Handle; a.v_weight = vWeight.Handle; a.out_weight = outWeight.Handle;
  a.out = output.Handle;
  a.batch = batch; a.seq = seq;
  a.input_dtype = input.Dtype; a.weight_dtype = qWeight.Dtype; a.out_dtype = output.Dtype;
  a.workspace = workspace_;            // cudaMalloc memory is at least 256-byte aligned, which is what the call asks for
  a.workspace_bytes = workspace_bytes_;
  Check(aidn_mha_forward(h, &a, stream_), "aidn_mha_forward");
  launch_count_ += aidn_sdpa_last_launch_count(h);
}

// ---- the decode step in front of attention -----------------------------------------------------------------------
void CudaBackend::QkvProjectionRoPECacheD64(const GpuBuffer& input, const GpuBuffer& packedWeights, const GpuBuffer& bias,
                                            const GpuBuffer& cosine, const GpuBuffer& sine, const GpuBuffer& query,
                                            const GpuBuffer& keyCache, const GpuBuffer& valueCache, int heads,
                                            int cacheCapacity, int position) {
  if (!input.Handle || !packedWeights.Handle || !bias.Handle || !cosine.Handle || !sine.Handle || !query.Handle ||
      !keyCache.Handle || !valueCache.Handle)
    throw std::invalid_argument("QkvProjectionRoPECacheD64: buffers must not be null");   // ArgumentNullException
  if (heads <= 0) throw std::invalid_argument("heads must be > 0");
  if (cacheCapacity <= 0) throw std::invalid_argument("cacheCapacity must be > 0");
  if (position < 0 || position >= cacheCapacity) throw std::invalid_argument("position must be in [0, cacheCapacity)");
  const int64_t dimension = 64, model = heads * dimension, projection = 3 * model;
  const int64_t cacheElements = cacheCapacity * model, ropeElements = cacheCapacity * (dimension / 2);
  if (input.Size < model || packedWeights.Size < projection * model || bias.Size < projection ||
      cosine.Size < ropeElements || sine.Size < ropeElements || query.Size < model || keyCache.Size < cacheElements ||
      valueCache.Size < cacheElements)
    throw std::invalid_argument("QKV/RoPE/cache buffers are smaller than the requested canonical extents.");
  aidn_qkv_rope_args a;
  std::memset(&a, 0, sizeof(a));
  a.input = static_cast<const float*>(input.Handle);
  a.weights = packedWeights.Handle;
  a.bias = static_cast<const float*>(bias.Handle);
  a.cosine = static_cast<const float*>(cosine.Handle);
  a.sine = static_cast<const float*>(sine.Handle);
  a.query = query.Handle; a.key_cache = keyCache.Handle; a.value_cache = valueCache.Handle;
  a.tokens = 1; a.heads = heads; a.kv_heads = heads; a.head_dim = (int32_t)dimension; a.position = position;
  a.weight_dtype = packedWeights.Dtype; a.query_dtype = query.Dtype; a.cache_dtype = keyCache.Dtype;
  a.cache_capacity = cacheCapacity; a.max_position = cacheCapacity;
  Check(aidn_qkv_rope_cache(&a, stream_), "aidn_qkv_rope_cache");
  ++launch_count_;
}

void CudaBackend::RopeInterleaved(const GpuBuffer& input, const GpuBuffer& cos, const GpuBuffer& sin,
                                  const GpuBuffer& output, int rows, int headDim, int seqLen, int startPosition) {
  if (rows <= 0 || headDim <= 0 || seqLen <= 0) throw std::invalid_argument("rows, headDim and seqLen must be positive");
  if (input.Size < (int64_t)rows * headDim || output.Size < (int64_t)rows * headDim)
    throw std::invalid_argument("RoPE buffers are smaller than rows * headDim");
  const int64_t need = (int64_t)(startPosition + seqLen) * (headDim / 2);
  if (cos.Size < need || sin.Size < need) throw std::invalid_argument("cos/sin caches do not reach startPosition + seqLen");
  Check(aidn_rope_interleaved(static_cast<const float*>(input.Handle), static_cast<const float*>(cos.Handle),
                              static_cast<const float*>(sin.Handle), static_cast<float*>(output.Handle), rows, headDim,
                              seqLen, startPosition, stream_),
        "aidn_rope_interleaved");
  ++launch_count_;
}

}  // namespace host
}  // namespace aidn
