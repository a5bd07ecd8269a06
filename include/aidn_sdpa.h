/*
 * aidn_sdpa.h — C ABI of libaidotnet_sdpa_sm100: fused scaled-dot-product-attention forward for
 * NVIDIA B200 (sm_100a).
 *
 * The library is a drop-in for the attention methods of the reference's CUDA backend.  File:line
 * citations are relative to src/AiDotNet.Tensors/ of the reference project:
 *
 *   Engines/DirectGpu/IDirectGpuBackend.cs:1421-1424  ScaledDotProductAttention(query,key,value,output,
 *        attentionWeights?,mask?,batch,numHeads,seqQ,seqK,headDim,scale,isCausal,softcap,numKVHeads)
 *   Engines/DirectGpu/IDirectGpuBackend.cs:1448-1449  FlashAttention(...)
 *   Engines/DirectGpu/IDirectGpuBackend.cs:1468-1471  FlashAttentionV2(...,softmaxStats,...,attentionBias?,biasBatchStride)
 *   Engines/DirectGpu/IDirectGpuBackend.cs:1501-1503  GroupedQueryAttention(...)
 *   Engines/DirectGpu/CUDA/CudaBackend.cs:2968-3021   FlashDecode(q,k,v,heads,kvHeads,headDim,seqLen,scale,splits)
 *   Engines/DirectGpu/IDirectGpuBackend.cs:1890,1911  ConvertToFp16 / ConvertToFp32 (dtype staging)
 *   Engines/DirectGpu/IDirectGpuBackend.cs:3619-3632  PagedAttentionDecode / PagedAttentionPrefill and their Gqa
 *        variants (q,kcache,vcache,blockTable,heads[,kvHeads],headDim,blockSize,seqLen | numQueries,startPos,scale)
 *
 * Conventions inherited from that caller (CudaBackend.cs:371-375, 546, 5253-5272, 5389-5403):
 *   - every buffer is caller-owned device memory (IGpuBuffer.Handle, IDirectGpuBackend.cs:3776-3803);
 *   - the caller's CUDA context is current on the calling thread and all work is enqueued on the
 *     explicit stream argument; nothing here synchronises, creates a context or touches the default stream;
 *   - a launch allocates nothing: scratch is either passed in (workspace) or owned by the handle;
 *   - errors are status codes plus a thread-local message, never aborts.
 *
 * Tensor layout is [B, H, S, D] with a unit stride on D; the B, H and S strides are explicit so that
 * permuted views ([B,S,H,D] storage, the single-sequence [S,Hkv,D] decode cache) need no copy.
 *
 * Threading (CudaBackend.cs:66, 5392: the reference serialises its launches under GpuDispatchLock): handles are
 * independent of one another and create / destroy are thread-safe, but ONE handle is not re-entrant.  The persistent
 * tcgen05 kernels keep their work-item counters and their status word in memory owned by the handle, so two launches
 * of the same handle must not overlap on the GPU: issue them on one stream (or order them with events), do not replay
 * a captured graph that contains a launch of the handle beside a live launch of it, and call aidn_sdpa_poll only when
 * no launch of the handle is in flight on another stream.  Use one handle per stream.
 *
 * Debugging: with AIDOTNET_KERNEL_LAUNCH_CHECK=1 in the environment (the reference's own switch, CudaBackend.cs:5381-5421)
 * every entry point synchronises its stream after launching and returns a device error or an expired bounded wait as
 * its own status ("[LAUNCH-FAULT] ..." in aidn_sdpa_last_error()).  Off by default; ignored during stream capture.
 *
 * Padding: key / value rows that no query can see — rows at or past kv_len[b], the unused tail of the last pool block
 * of a paged sequence, rows past seq_kv — may hold anything, NaN and Inf included: the forward kernels never let
 * them reach the output.  aidn_sdpa_backward is the exception: K and V rows up to the end of the last 128-key tile
 * that a sequence touches must be finite there (the reference zero-fills its buffers, CudaBackend.AllocateBuffer).
 */
#ifndef AIDN_SDPA_H_
#define AIDN_SDPA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define AIDN_API __declspec(dllexport)
#else
#define AIDN_API __attribute__((visibility("default")))
#endif

typedef struct aidn_sdpa* aidn_sdpa_t;

typedef enum {
  AIDN_OK = 0,
  AIDN_EINVAL = 1,       /* bad argument (shape, stride, null pointer, alignment)            */
  AIDN_EUNSUPPORTED = 2, /* valid request that no kernel of this build serves               */
  AIDN_ECUDA = 3,        /* a CUDA call failed; aidn_sdpa_last_error() carries its message   */
  AIDN_EWORKSPACE = 4,   /* workspace missing or too small                                   */
  AIDN_ETIMEOUT = 5,     /* a bounded device-side wait expired (reported by aidn_sdpa_poll)  */
  AIDN_ENCCL = 6         /* NCCL missing or an NCCL call failed                              */
} aidn_status;

typedef enum { AIDN_F32 = 0, AIDN_F16 = 1, AIDN_BF16 = 2 } aidn_dtype;

/* How args.mask is read.  Every kind broadcasts over axes whose mask_stride is 0
 * (CpuEngine.MultiHeadAttention.cs:344 BroadcastMaskIndex). */
typedef enum {
  AIDN_MASK_NONE = 0,
  AIDN_MASK_KEEP_U8 = 1,  /* Tensor<bool>: non-zero = attend (IEngine.cs:4133-4140)                       */
  AIDN_MASK_KEEP_F32 = 2, /* the engine's float upload of a bool mask: 0.0f = masked
                             (CUDA/Kernels/CudaAttentionKernels.cs:74)                                   */
  AIDN_MASK_ADD_F32 = 3   /* additive bias, added after scale (CpuEngine.cs:29226-29233)                 */
} aidn_mask_kind;

/* Kernel selection.  AUTO picks: split-KV decode when seq_q == 1, the tcgen05 prefill kernel for 16-bit
 * inputs with head_dim 64 or 128, the generic FFMA kernel otherwise.  The others force one kernel (tests). */
typedef enum {
  AIDN_PATH_AUTO = 0,
  AIDN_PATH_GENERIC = 1,
  AIDN_PATH_DECODE = 2,
  AIDN_PATH_PREFILL_SM100 = 3
} aidn_path;

typedef struct {
  int32_t device;       /* CUDA ordinal; must be the device of the current context                     */
  int32_t qkv_dtype;    /* aidn_dtype of Q, K and V                                                    */
  int32_t out_dtype;    /* AIDN_F32 (the reference's contract) or the same as qkv_dtype                */
  int32_t head_dim;     /* D = Dv; 64 or 128 on the tcgen05 path, any multiple of 8 up to 256 elsewhere */
  int32_t num_q_heads;  /* Hq of the full tensor                                                       */
  int32_t num_kv_heads; /* Hkv; Hq % Hkv == 0; kv head of q head h is h / (Hq / Hkv)                   */
  int32_t causal;       /* keep key k for query q iff k <= q + causal_offset                           */
  int32_t causal_bottom_right; /* 1: causal_offset = seq_kv - seq_q per launch (SDPA / Gqa entry points,
                                  CpuEngine.cs:27333-27340); 0: use causal_offset as given
                                  (0 = top-left, the FlashAttention entry points, CpuEngine.cs:29235) */
  int64_t causal_offset;
  int32_t mask_kind;    /* aidn_mask_kind                                                              */
  int32_t emit_lse;     /* 1: args.lse receives max + ln(sum) per row, -inf for a fully masked row      */
  float softcap;        /* > 0: score = softcap * tanh(score * scale / softcap); 0 disables            */
  int32_t path;         /* aidn_path                                                                   */
  int32_t head_begin;   /* first q head this handle computes (head shard of a multi-GPU run)           */
  int32_t head_count;   /* number of q heads it computes; 0 = all.  Must cover whole KV groups.        */
  int32_t decode_chunk; /* keys per split of the decode kernel; 0 = choose from the shape              */
  int32_t max_batch;    /* > 0 together with max_seq_kv: the handle allocates its own decode scratch   */
  int64_t max_seq_q;    /*   for shapes up to these, so launch can be called with workspace == NULL    */
  int64_t max_seq_kv;
  void* nccl_comm;      /* ncclComm_t whose ranks hold consecutive head shards, or NULL                */
} aidn_sdpa_desc;

typedef struct {
  const void* q;        /* device pointers; element (b,h,s,d) at base + b*stride[0] + h*stride[1] + s*stride[2] + d */
  const void* k;
  const void* v;
  void* out;
  float* lse;           /* [B, Hq, Sq] dense, fp32; required iff desc.emit_lse                          */
  const void* mask;     /* per desc.mask_kind, or NULL                                                 */
  int64_t mask_stride[4]; /* elements for (B, H, Sq, Sk); 0 = broadcast                                 */
  const int32_t* kv_len;  /* [B] valid key count per batch entry (padding mask), or NULL                */
  int64_t batch, seq_q, seq_kv;
  int64_t q_stride[3];  /* elements for (B, H, S); all zero = dense [B,H,S,D]                           */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  float scale;          /* 0 = 1/sqrt(head_dim)                                                        */
  void* workspace;      /* device scratch of at least aidn_sdpa_workspace_bytes(), or NULL to use the handle's */
  int64_t workspace_bytes;
  int32_t gather_output;  /* 1: after the kernel, ncclAllGather the head shards of `out` in place on the same
                             stream (batch == 1 or per-batch-entry group call); needs desc.nccl_comm      */
  float* weights;         /* NULL, or [B, Hq, Sq, Sk] dense fp32: receives the attention probabilities, the
                             `out attentionWeights` of IEngine.ScaledDotProductAttention (IEngine.cs:4133-4140):
                             0 at masked positions, an all-zero row where every key is masked.  The call then runs
                             on the fp32 FFMA kernel whatever the input dtype, with a second pass over the keys -
                             sized for the training-time shapes that ask for weights, not for long prefill; the
                             buffer is B*Hq*Sq*Sk*4 bytes, counted in 64 bits.                              */
  int32_t peer_count;     /* 0, or the number of entries of peer_out (at most AIDN_MAX_PEERS)                     */
  void* peer_out[8];      /* Fused gather of a head-sharded prefill (tcgen05 kernel only): peer_out[i] is the `out`
                             tensor of another device - same shape, strides and dtype - mapped into this device's
                             address space (aidn_peer_open).  Every output tile is stored to `out` and to each
                             peer_out[i] by the kernel's own TMA stores, while the other tiles are still being
                             computed: the all-gather of NcclComm.AllGather (CUDA/NcclComm.cs:106-110) costs no
                             second pass.  A device's tensor is complete when EVERY rank's launch has completed:
                             synchronise the ranks (a barrier or a tiny collective on the stream) before reading.
                             Not together with gather_output.                                                 */
} aidn_sdpa_args;
#define AIDN_MAX_PEERS 8

/* Paged K/V (the vLLM-style pool of Engines/DirectGpu/DevicePagedKVCache.cs:10-18): args.k / args.v are the key and
 * value pools [num_blocks, block_size, Hkv, D]; key t of batch entry b is row
 * block_table[b * block_table_stride + t / block_size] * block_size + t % block_size of the pool.  In this mode
 * k_stride / v_stride mean: [0] unused, [1] head stride, [2] stride between pool rows; all zero = the dense pool
 * layout above (head stride D, row stride Hkv * D).  The table must hold ceil(n / block_size) entries per sequence,
 * n = the keys that sequence can see (kv_len[b] when given, else seq_kv). */
typedef struct {
  const int32_t* block_table; /* device, int32 (AllocateIntBuffer, CudaBackend.cs:5216-5234 convention)        */
  int64_t block_table_stride; /* entries between consecutive sequences; unused for batch == 1                  */
  int32_t block_size;         /* tokens per block, > 0; a multiple of 8 dividing 128 for the tcgen05 kernel    */
  int32_t num_blocks;         /* blocks in the pool; > 0 makes the kernels skip entries outside [0,num_blocks)
                                 and report them through aidn_sdpa_poll (AIDN_EINVAL); 0 = trust the table      */
} aidn_paged_kv;

/* Pointers passed with q/k/v/out index the FULL tensors: the handle offsets them by head_begin itself. */

/* Validates the descriptor, resolves driver entry points, sizes and allocates handle-owned scratch. */
AIDN_API int aidn_sdpa_create(const aidn_sdpa_desc* desc, aidn_sdpa_t* out);
/* Bytes of caller workspace a launch of this shape needs (0 for the prefill kernels); < 0 on error. */
AIDN_API int64_t aidn_sdpa_workspace_bytes(aidn_sdpa_t h, int64_t batch, int64_t seq_q, int64_t seq_kv);
/* Enqueues the attention forward on `cu_stream` (a CUstream / cudaStream_t).  No allocation, no synchronisation; safe
 * under stream capture once the handle has launched that kernel once outside capture (the first launch raises the
 * kernel's shared-memory limit).  Launches of one handle must be stream-ordered (see "Threading" above). */
AIDN_API int aidn_sdpa_launch(aidn_sdpa_t h, const aidn_sdpa_args* args, void* cu_stream);
/* The same forward with K and V read through a block table (see aidn_paged_kv).  Decode (seq_q == 1, any batch,
 * per-sequence kv_len) is PagedAttentionDecode{,Gqa}; seq_q > 1 with desc.causal and causal_bottom_right = 0,
 * causal_offset = startPos is PagedAttentionPrefill{,Gqa} — the reference's [numQueries, heads, D] query and output
 * are q_stride = o_stride = {0, D, heads * D}. */
AIDN_API int aidn_sdpa_launch_paged(aidn_sdpa_t h, const aidn_sdpa_args* args, const aidn_paged_kv* paged,
                                    void* cu_stream);
/* Synchronises `cu_stream` and returns AIDN_ETIMEOUT if a kernel of this handle gave up a bounded wait,
 * AIDN_EINVAL if a paged launch met a block-table entry outside the pool, AIDN_ECUDA on a CUDA error, else AIDN_OK.  For tests and diagnostics; not needed on the hot path. */
AIDN_API int aidn_sdpa_poll(aidn_sdpa_t h, void* cu_stream);
/* Which kernel the last launch used (aidn_path value), and how many kernels it enqueued. */
AIDN_API int aidn_sdpa_last_path(aidn_sdpa_t h);
AIDN_API int aidn_sdpa_last_launch_count(aidn_sdpa_t h);
AIDN_API int aidn_sdpa_destroy(aidn_sdpa_t h);
/* Thread-local message of the last failing call on this thread ("" if none). */
AIDN_API const char* aidn_sdpa_last_error(void);
/* 1 when `device` is compute capability 10.x and this build carries sm_100a code, else 0. */
AIDN_API int aidn_sdpa_device_supported(int32_t device);

/* Batched decode (seq_q == 1) that allocates nothing, for callers that are not allowed to: a serving loop or a
 * CUDA-graph-replaying runtime that fixed its device memory up front, or a host (such as a managed runtime whose GPU
 * buffers all come from one pre-sized pool) that cannot call cudaMalloc at the point where it decodes.  It needs no
 * handle and no workspace: the split-KV partials go to a fixed 16 MiB array that is part of the library image, so
 * every GPU that loads the library keeps those 16 MiB until the process exits.  The caller still passes Q, K, V,
 * out (and lse / mask / kv_len) exactly as for aidn_sdpa_launch; `desc` is read on every call (path, max_*, nccl_comm
 * are ignored) and `args.workspace` is ignored.
 *   - Limit: batch * heads_in_shard * ceil(seq_kv / chunk) * (head_dim + 2) * 4 bytes must fit in 16 MiB, where
 *     chunk is desc.decode_chunk or the library's choice: at most 1024 keys for 16-bit inputs with head_dim 64 / 128
 *     and up to 16 query heads per KV head, at most 512 keys otherwise (fp32 inputs, head_dim 256, larger groups).  A
 *     larger request returns AIDN_EWORKSPACE with the two sizes in aidn_sdpa_last_error().
 *   - desc.device must be the current device.  The first call in each CUDA context looks up the array's device
 *     address (the array has one copy per context: a process that uses the primary context and one created with
 *     cuCtxCreate on the same GPU gets two); make that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Nothing has to be
 *     cleared between calls, because the combine kernel reads only the slots the partial kernel of the same call
 *     wrote, but two calls whose kernels overlap on the GPU (different streams, or two host threads) race on it:
 *     run them on one stream or order them yourself.
 * No counterpart in the reference: its FlashDecode allocates three scratch buffers per call
 * (CudaBackend.cs:2994-2996). */
AIDN_API int aidn_sdpa_decode_noalloc(const aidn_sdpa_desc* desc, const aidn_sdpa_args* args, void* cu_stream);

/* The device half of DevicePagedKVCache.Append (Engines/DirectGpu/DevicePagedKVCache.cs:113-202): `tokens` new K / V
 * rows of `row_bytes` bytes each (kv_heads * head_dim * element size, a multiple of 16) are written to the pool rows of
 * sequence positions start_position .. start_position + tokens - 1, looked up in the sequence's block table.  One
 * kernel instead of one device copy per run inside a block; the free list, reference counts and copy-on-write stay in
 * the caller's cache object.  Entries outside [0, num_blocks) are skipped. */
AIDN_API int aidn_paged_kv_append(const void* new_keys, const void* new_values, void* key_pool, void* value_pool,
                                  const int32_t* block_table, int64_t start_position, int64_t tokens,
                                  int32_t block_size, int32_t num_blocks, int64_t row_bytes, void* cu_stream);

/* Backward of the same attention (FlashAttentionBackward, IDirectGpuBackend.cs:1479-1483, CudaBackend.cs:8580-8704;
 * CPU CpuEngine.cs:29474): dQ, dK, dV from dO, Q, K, V, O and the forward's log-sum-exp, deterministic (every gradient
 * cell is summed by one thread in a fixed order, as the reference's *_deterministic kernels do).  `fwd` is the forward
 * launch's argument block with fwd.out = O and fwd.lse = the statistics, both read here; masks, bias, causal offset,
 * kv_len, grouped-query heads and paged K/V mean what they mean forward (no gradient is produced for a bias).  dO has
 * O's dtype; the gradients are dense fp32: dq [B, Hc, Sq, D], dk / dv [B, Hc / group, Sk, D], Hc = the heads of the
 * handle's shard.  fwd.workspace must hold aidn_sdpa_backward_workspace_bytes().  Logit softcap is not supported. */
typedef struct {
  aidn_sdpa_args fwd;
  const aidn_paged_kv* paged; /* NULL for contiguous K / V                                                     */
  const void* dout;           /* dO, element (b,h,s,d) at do_stride (all zero = o_stride of fwd)               */
  int64_t do_stride[3];
  float* dq;
  float* dk;
  float* dv;
} aidn_sdpa_bwd_args;
AIDN_API int64_t aidn_sdpa_backward_workspace_bytes(aidn_sdpa_t h, int64_t batch, int64_t seq_q);
AIDN_API int aidn_sdpa_backward(aidn_sdpa_t h, const aidn_sdpa_bwd_args* args, void* cu_stream);

/* The decode step in front of the attention call: packed Q/K/V projection of resident tokens, bias, interleaved RoPE
 * on Q and K, Q written out and the K / V rows written into the KV cache, in one pass over the weights.  Replaces
 * CudaBackend.QkvProjectionRoPECacheD64 (CudaBackend.cs:8389-8439: one fp32 token, head_dim 64, cache
 * [capacity, heads, 64], `position` both the RoPE position and the cache row) and generalises it: any even head_dim,
 * grouped-query projections (heads + 2*kv_heads output heads), several tokens per call (each with its own position
 * and cache row - e.g. one token of every sequence of a decode batch, with cache rows taken from a paged pool), bf16
 * weights, and a 16-bit cache that the decode kernel reads directly.  All pointers are device memory. */
typedef struct {
  const float* input;        /* [tokens, model] fp32, model = heads * head_dim                                  */
  const void* weights;       /* [(heads + 2*kv_heads) * head_dim, model], output-major: Q rows, K rows, V rows  */
  const float* bias;         /* [(heads + 2*kv_heads) * head_dim], or NULL                                      */
  const float* cosine;       /* [max_position, head_dim / 2], indexed by absolute position                      */
  const float* sine;
  void* query;               /* [tokens, heads * head_dim], query_dtype                                         */
  void* key_cache;           /* [cache_capacity, kv_heads, head_dim], cache_dtype                               */
  void* value_cache;
  const int32_t* positions;  /* [tokens] RoPE position of each token, or NULL: position + token index           */
  const int32_t* cache_rows; /* [tokens] cache row each token's K / V goes to, or NULL: the token's position    */
  int32_t tokens, heads, kv_heads, head_dim;
  int32_t position;          /* first token's position when positions == NULL                                   */
  int32_t weight_dtype;      /* AIDN_F32 or AIDN_BF16                                                           */
  int32_t query_dtype;       /* aidn_dtype                                                                      */
  int32_t cache_dtype;       /* aidn_dtype                                                                      */
  int64_t cache_capacity;    /* rows of the caches; a token whose row lies outside writes no K / V              */
  int64_t max_position;      /* rows of cosine / sine; a position outside them is left unrotated                */
} aidn_qkv_rope_args;
AIDN_API int aidn_qkv_rope_cache(const aidn_qkv_rope_args* args, void* cu_stream);
/* rope_interleaved (CUDA/Kernels/CudaAttentionKernels.cs:1023-1050; CudaBackend.RopeInterleaved): rows of head_dim
 * fp32 values, row r at position start_position + r % seq_len, pairs (2i, 2i+1) rotated by (cos, sin)[position][i]. */
AIDN_API int aidn_rope_interleaved(const float* input, const float* cosine, const float* sine, float* output,
                                   int64_t rows, int32_t head_dim, int32_t seq_len, int32_t start_position,
                                   void* cu_stream);

/* ---- fused multi-head attention forward ---------------------------------------------------------------------
 * IEngine.MultiHeadAttentionForward (src/AiDotNet.Tensors/Engines/IEngine.cs:4201-4208; CPU
 * CpuEngine.MultiHeadAttention.cs:68-338, GPU composition DirectGpuTensorEngine.MissingKernels.cs:5793-5870):
 *   out = softmax((X Wq)(X Wk)^T / sqrt(d) [keep-mask]) (X Wv) Wout,   X [batch, seq, heads*d], each W [heads*d, heads*d]
 * row-major and applied as x * W.  Three launches on the stream: one GEMM for the Q, K and V projections that writes
 * [B, H, S, d] directly, the attention kernel of the handle, one GEMM for the output projection reading the attention
 * output as [B, S, H*d].  Two routes, chosen from the handle:
 *   - 16-bit qkv_dtype, head_dim 64 or 128, heads*head_dim a multiple of 128: tcgen05 GEMMs and the tcgen05 attention
 *     kernel, fp32 accumulation.  fp32 inputs or weights are first rounded to the 16-bit type inside the workspace
 *     (pass 16-bit weights, converted once with aidn_cast_*, to skip that per call).
 *   - anything else (fp32 qkv_dtype, other head sizes or widths, desc.path == AIDN_PATH_GENERIC): FFMA GEMMs and the
 *     generic attention kernel in fp32 arithmetic; with an fp32 handle this meets the 1e-4 bound of the reference's own
 *     tests of the fused call (tests/AiDotNet.Tensors.Tests/Engines/MultiHeadAttentionForwardTests.cs:123).
 * The handle gives heads, head_dim and the mask kind (none or a keep-mask broadcastable to [B, H, S, S]; a fully masked
 * row gives zeros, CpuEngine.MultiHeadAttention.cs:481-485; a handle created with desc.causal = 1 additionally applies
 * the causal rule without a materialised mask - an extension, the reference expresses causality through the mask); it
 * must have out_dtype == qkv_dtype,
 * num_kv_heads == num_q_heads, all heads, no log-sum-exp, softcap or additive bias (else AIDN_EUNSUPPORTED). */
typedef struct {
  const void* input;        /* [batch, seq, heads*head_dim], input_dtype                                         */
  const void* q_weight;     /* [heads*head_dim, heads*head_dim], weight_dtype                                    */
  const void* k_weight;
  const void* v_weight;
  const void* out_weight;
  void* out;                /* [batch, seq, heads*head_dim], out_dtype                                           */
  const void* mask;         /* per desc.mask_kind, or NULL                                                       */
  int64_t mask_stride[4];   /* elements for (B, H, Sq, Sk); 0 = broadcast                                        */
  int64_t batch, seq;
  int32_t input_dtype;      /* AIDN_F32 or desc.qkv_dtype                                                        */
  int32_t weight_dtype;     /* AIDN_F32 or desc.qkv_dtype                                                        */
  int32_t out_dtype;        /* AIDN_F32 or desc.qkv_dtype                                                        */
  int32_t reserved;
  void* workspace;          /* device scratch of at least aidn_mha_workspace_bytes(), 256-byte aligned           */
  int64_t workspace_bytes;
} aidn_mha_args;
AIDN_API int64_t aidn_mha_workspace_bytes(aidn_sdpa_t h, int64_t batch, int64_t seq, int32_t input_dtype,
                                          int32_t weight_dtype);
AIDN_API int aidn_mha_forward(aidn_sdpa_t h, const aidn_mha_args* args, void* cu_stream);

/* dtype staging (IDirectGpuBackend.cs:1890 ConvertToFp16, :1911 ConvertToFp32; bf16 rounding per
 * NumericOperations/BFloat16.cs:65-84: round-to-nearest-even, NaN keeps its top payload bits plus the quiet bit). */
/* Peer mappings for aidn_sdpa_args.peer_out, between processes of one node (one process per GPU).
 * aidn_peer_export: the 64-byte CUDA IPC handle of the allocation that holds `dev_ptr`, and the offset of dev_ptr in
 * it (the allocation must come from cudaMalloc, as torch's default allocator's blocks do).  aidn_peer_open: maps an
 * exported allocation of ANOTHER process into the current device's address space (peer access is enabled on
 * demand) and returns its base; the tensor is at base + offset.  aidn_peer_close unmaps it. */
AIDN_API int aidn_peer_export(const void* dev_ptr, void* handle64, int64_t* offset);
AIDN_API int aidn_peer_open(const void* handle64, void** base);
AIDN_API int aidn_peer_close(void* base);

AIDN_API int aidn_cast_f32_to_bf16(const float* src, void* dst, int64_t n, void* cu_stream);
AIDN_API int aidn_cast_f32_to_f16(const float* src, void* dst, int64_t n, void* cu_stream);
AIDN_API int aidn_cast_bf16_to_f32(const void* src, float* dst, int64_t n, void* cu_stream);
AIDN_API int aidn_cast_f16_to_f32(const void* src, float* dst, int64_t n, void* cu_stream);

#ifdef __cplusplus
}
#endif
#endif /* AIDN_SDPA_H_ */
