// C ABI of libaidotnet_sdpa_sm100 (declared in include/aidn_sdpa.h): argument validation, kernel selection
// and launch.  No torch types, no allocation on the launch path, no CPU fallback: a request no CUDA kernel
// of this build can serve is an error.
#include <dlfcn.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

#include "common.cuh"
#include "../../../include/aidn_sdpa_debug.h"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int fail_cuda(cudaError_t e, const char* what) {
  return fail(AIDN_ECUDA, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

// AIDOTNET_KERNEL_LAUNCH_CHECK=1, the reference's own debugging switch (CudaBackend.cs:5381-5421): every entry point
// then synchronises the stream right after its launches and reports a device error, or a bounded wait that gave up, as
// the failure of THAT call instead of some later one.  Skipped while the stream is being captured.  Read once.
bool launch_check_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("AIDOTNET_KERNEL_LAUNCH_CHECK");
    return v && v[0] == '1' && v[1] == 0;
  }();
  return on;
}

int post_launch_check(cudaStream_t stream, const char* what, int32_t* status_dev) {
  if (!launch_check_enabled()) return AIDN_OK;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return AIDN_OK;
  }
  cudaError_t e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(AIDN_ECUDA, "[LAUNCH-FAULT] %s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  if (status_dev) {
    int32_t st = 0;
    e = cudaMemcpy(&st, status_dev, sizeof(st), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_cuda(e, "launch check: status read");
    if (st & aidn::kStatusTimeout) return fail(AIDN_ETIMEOUT, "[LAUNCH-FAULT] %s: a kernel gave up a bounded wait (status word 0x%x)", what, st);
  }
  return AIDN_OK;
}

size_t elem_size(int dtype) { return dtype == AIDN_F32 ? 4 : 2; }

// ---- NCCL, resolved lazily so that the library loads on machines without it --------------------------
struct Nccl {
  void* lib = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*CommUserRank)(void*, int*) = nullptr;
  int (*CommCount)(void*, int*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
};
Nccl g_nccl;
std::once_flag g_nccl_once;

void load_nccl() {
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    g_nccl.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.lib) break;
  }
  if (!g_nccl.lib) return;
  g_nccl.AllGather = (decltype(g_nccl.AllGather))dlsym(g_nccl.lib, "ncclAllGather");
  g_nccl.GroupStart = (decltype(g_nccl.GroupStart))dlsym(g_nccl.lib, "ncclGroupStart");
  g_nccl.GroupEnd = (decltype(g_nccl.GroupEnd))dlsym(g_nccl.lib, "ncclGroupEnd");
  g_nccl.CommUserRank = (decltype(g_nccl.CommUserRank))dlsym(g_nccl.lib, "ncclCommUserRank");
  g_nccl.CommCount = (decltype(g_nccl.CommCount))dlsym(g_nccl.lib, "ncclCommCount");
  g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(g_nccl.lib, "ncclGetErrorString");
  g_nccl.ok = g_nccl.AllGather && g_nccl.GroupStart && g_nccl.GroupEnd && g_nccl.CommUserRank && g_nccl.CommCount;
}

constexpr int kNcclFloat32 = 7, kNcclFloat16 = 6, kNcclBfloat16 = 9;  // ncclDataType_t values (nccl.h)

}  // namespace

struct aidn_sdpa {
  aidn_sdpa_desc d;
  int group;
  int head_count;
  int32_t* status_dev;   // [0] status word, [1..2] scheduler counters of the persistent prefill kernel
  int num_sms;
  void* scratch;
  int64_t scratch_bytes;
  int last_path;
  int last_launches;
  float* debug;
  int debug_mode;
  aidn::PrefillMapCache prefill_maps;   // tensor maps of the last tcgen05 prefill launch (see common.cuh)
};

namespace {

// Keys per split of the decode kernel.  Enough CTAs to fill 148 SMs several times over, but never more than
// 512 keys per CTA so that ragged kv_len values balance, and never fewer than 64.
int pick_chunk(const aidn_sdpa* h, int64_t batch, int64_t seq_kv) {
  if (h->d.decode_chunk > 0) return h->d.decode_chunk;
  const int gt = h->group <= 2 ? h->group : (h->group <= 4 ? 4 : 8);  // as the FFMA decode launcher picks
  int gchunks = (h->group + gt - 1) / gt;
  int64_t cap = 512;
  // 16-bit inputs with up to 16 query heads per KV head run the tensor-core decode kernel: one CTA per KV head and
  // split, and chunks up to 1024 keys (its per-CTA prologue and merge are heavier, its steady state faster)
  if (h->d.qkv_dtype != AIDN_F32 && (h->d.head_dim == 64 || h->d.head_dim == 128) && h->group <= 16) {
    gchunks = 1;
    cap = 1024;
  }
  const int64_t items = batch * (h->head_count / h->group) * gchunks;
  const int64_t target = 148 * 8;
  int64_t splits = (target + items - 1) / items;
  if (splits < 1) splits = 1;
  int64_t chunk = align_up((seq_kv + splits - 1) / splits, 64);
  if (chunk > cap) chunk = cap;
  if (chunk < 64) chunk = 64;
  return (int)chunk;
}

int64_t decode_ws_bytes(const aidn_sdpa* h, int64_t batch, int64_t seq_kv, int* chunk_out, int* nchunks_out) {
  const int chunk = pick_chunk(h, batch, seq_kv);
  const int64_t nchunks = (seq_kv + chunk - 1) / chunk;
  if (chunk_out) *chunk_out = chunk;
  if (nchunks_out) *nchunks_out = (int)nchunks;
  if (nchunks <= 1) return 0;
  return align_up(batch * h->head_count * nchunks * (h->d.head_dim + 2) * (int64_t)sizeof(float), 256);
}

bool aligned16(const void* ptr, const int64_t* stride, size_t esz) {
  if ((uintptr_t)ptr % 16 != 0) return false;
  for (int i = 0; i < 3; ++i)
    if ((stride[i] * (int64_t)esz) % 16 != 0) return false;
  return true;
}

void dense_strides(int64_t* s, int64_t heads, int64_t seq, int64_t d) {
  s[2] = d;
  s[1] = seq * d;
  s[0] = heads * seq * d;
}

bool all_zero(const int64_t* s) { return s[0] == 0 && s[1] == 0 && s[2] == 0; }

}  // namespace

extern "C" {

const char* aidn_sdpa_last_error(void) { return g_err; }

int aidn_sdpa_device_supported(int32_t device) {
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return major == 10 ? 1 : 0;
}

int aidn_sdpa_create(const aidn_sdpa_desc* desc, aidn_sdpa_t* out) {
  g_err[0] = 0;
  if (!desc || !out) return fail(AIDN_EINVAL, "create: null argument");
  *out = nullptr;
  const aidn_sdpa_desc& d = *desc;
  if (d.qkv_dtype < AIDN_F32 || d.qkv_dtype > AIDN_BF16) return fail(AIDN_EINVAL, "create: unknown qkv_dtype %d", d.qkv_dtype);
  if (d.out_dtype != AIDN_F32 && d.out_dtype != d.qkv_dtype)
    return fail(AIDN_EINVAL, "create: out_dtype must be fp32 or equal to qkv_dtype");
  if (d.head_dim <= 0 || d.head_dim > 256) return fail(AIDN_EINVAL, "create: head_dim %d outside [1,256]", d.head_dim);
  if (d.num_q_heads <= 0 || d.num_kv_heads <= 0 || d.num_q_heads % d.num_kv_heads != 0)
    return fail(AIDN_EINVAL, "create: numHeads (%d) must be a positive multiple of numKVHeads (%d)", d.num_q_heads,
                d.num_kv_heads);
  if (d.mask_kind < AIDN_MASK_NONE || d.mask_kind > AIDN_MASK_ADD_F32) return fail(AIDN_EINVAL, "create: unknown mask_kind");
  if (d.path < AIDN_PATH_AUTO || d.path > AIDN_PATH_PREFILL_SM100) return fail(AIDN_EINVAL, "create: unknown path");
  if (!(d.softcap >= 0.f)) return fail(AIDN_EINVAL, "create: softcap must be >= 0");
  const int group = d.num_q_heads / d.num_kv_heads;
  const int head_count = d.head_count > 0 ? d.head_count : d.num_q_heads - d.head_begin;
  if (d.head_begin < 0 || head_count <= 0 || d.head_begin + head_count > d.num_q_heads)
    return fail(AIDN_EINVAL, "create: head shard [%d,%d) outside [0,%d)", d.head_begin, d.head_begin + head_count,
                d.num_q_heads);
  if (d.head_begin % group != 0 || head_count % group != 0)
    return fail(AIDN_EINVAL, "create: a head shard must cover whole KV groups (group size %d)", group);
  if (d.decode_chunk < 0 || (d.decode_chunk > 0 && d.decode_chunk % 8 != 0))
    return fail(AIDN_EINVAL, "create: decode_chunk must be 0 or a positive multiple of 8");

  int cur = -1;
  cudaError_t e = cudaGetDevice(&cur);
  if (e != cudaSuccess) return fail_cuda(e, "create: cudaGetDevice");
  if (cur != d.device) return fail(AIDN_EINVAL, "create: desc.device (%d) is not the current device (%d)", d.device, cur);
  if (!aidn_sdpa_device_supported(d.device))
    return fail(AIDN_EUNSUPPORTED, "create: device %d is not compute capability 10.x (this library carries sm_100a code only)",
                d.device);

  aidn_sdpa* h = new (std::nothrow) aidn_sdpa();
  if (!h) return fail(AIDN_ECUDA, "create: out of host memory");
  h->d = d;
  h->group = group;
  h->head_count = head_count;
  h->status_dev = nullptr;
  h->scratch = nullptr;
  h->scratch_bytes = 0;
  h->last_path = AIDN_PATH_AUTO;
  h->last_launches = 0;
  h->debug = nullptr;
  h->debug_mode = 0;
  h->num_sms = 0;
  std::memset(&h->prefill_maps, 0, sizeof(h->prefill_maps));
  e = cudaDeviceGetAttribute(&h->num_sms, cudaDevAttrMultiProcessorCount, d.device);
  if (e == cudaSuccess) e = cudaMalloc(&h->status_dev, 4 * sizeof(int32_t));
  if (e == cudaSuccess) e = cudaMemset(h->status_dev, 0, 4 * sizeof(int32_t));
  if (e != cudaSuccess) {
    if (h->status_dev) cudaFree(h->status_dev);
    delete h;
    return fail_cuda(e, "create: status word");
  }
  if (d.max_batch > 0 && d.max_seq_kv > 0) {
    const int64_t bytes = decode_ws_bytes(h, d.max_batch, d.max_seq_kv, nullptr, nullptr);
    if (bytes > 0) {
      e = cudaMalloc(&h->scratch, (size_t)bytes);
      if (e != cudaSuccess) {
        cudaFree(h->status_dev);
        delete h;
        return fail_cuda(e, "create: decode scratch");
      }
      h->scratch_bytes = bytes;
    }
  }
  *out = h;
  return AIDN_OK;
}

int aidn_sdpa_destroy(aidn_sdpa_t h) {
  if (!h) return AIDN_OK;
  if (h->scratch) cudaFree(h->scratch);
  if (h->status_dev) cudaFree(h->status_dev);
  delete h;
  return AIDN_OK;
}

int64_t aidn_sdpa_workspace_bytes(aidn_sdpa_t h, int64_t batch, int64_t seq_q, int64_t seq_kv) {
  if (!h || batch <= 0 || seq_q <= 0 || seq_kv <= 0) {
    fail(AIDN_EINVAL, "workspace_bytes: bad argument");
    return -1;
  }
  if (seq_q != 1 || h->d.path == AIDN_PATH_GENERIC || h->d.path == AIDN_PATH_PREFILL_SM100) return 0;
  if (!aidn::decode_supported(h->d.qkv_dtype, h->d.head_dim)) return 0;
  return decode_ws_bytes(h, batch, seq_kv, nullptr, nullptr);
}

int aidn_sdpa_last_path(aidn_sdpa_t h) { return h ? h->last_path : -1; }
int aidn_sdpa_last_launch_count(aidn_sdpa_t h) { return h ? h->last_launches : -1; }

// Test and development hook, declared in include/aidn_sdpa_debug.h.
int aidn_sdpa_debug_set(aidn_sdpa_t h, float* buf, int mode) {
  if (!h) return AIDN_EINVAL;
  h->debug = buf;
  h->debug_mode = (buf || mode == 3) ? mode : 0;
  return AIDN_OK;
}

int aidn_sdpa_poll(aidn_sdpa_t h, void* cu_stream) {
  g_err[0] = 0;
  if (!h) return fail(AIDN_EINVAL, "poll: null handle");
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)cu_stream);
  if (e != cudaSuccess) return fail_cuda(e, "poll: stream");
  int32_t st = 0;
  e = cudaMemcpy(&st, h->status_dev, sizeof(st), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail_cuda(e, "poll: status read");
  if (st != 0) {
    cudaMemset(h->status_dev, 0, 4 * sizeof(int32_t));
    if (st & aidn::kStatusTimeout)
      return fail(AIDN_ETIMEOUT, "poll: a kernel gave up a bounded wait (status word 0x%x)", st);
    return fail(AIDN_EINVAL, "poll: a block-table entry outside [0, num_blocks) was skipped (status word 0x%x)", st);
  }
  return AIDN_OK;
}

}  // extern "C"

namespace {

// Validates a launch request and flattens it into the kernels' parameter block (shared by the forward launches and
// the backward).
int build_params(aidn_sdpa_t h, const aidn_sdpa_args* a, const aidn_paged_kv* pg, aidn::SdpaParams& p) {
  g_err[0] = 0;
  if (!h || !a) return fail(AIDN_EINVAL, "launch: null argument");
  const aidn_sdpa_desc& d = h->d;
  if (!a->q || !a->k || !a->v || !a->out) return fail(AIDN_EINVAL, "launch: null tensor pointer");
  if (a->batch <= 0 || a->seq_q <= 0 || a->seq_kv <= 0)
    return fail(AIDN_EINVAL, "launch: attention dimensions must be positive");
  if (a->batch > 65535) return fail(AIDN_EINVAL, "launch: batch above 65535");
  if (d.emit_lse && !a->lse) return fail(AIDN_EINVAL, "launch: emit_lse set but lse pointer is null");
  if (d.mask_kind != AIDN_MASK_NONE && !a->mask) return fail(AIDN_EINVAL, "launch: mask_kind set but mask pointer is null");
  if (a->scale < 0.f || std::isnan(a->scale)) return fail(AIDN_EINVAL, "launch: scale must be >= 0");

  std::memset(&p, 0, sizeof(p));
  p.q = a->q;
  p.k = a->k;
  p.v = a->v;
  p.out = a->out;
  p.lse = d.emit_lse ? a->lse : nullptr;
  p.weights = a->weights;
  if (a->peer_count < 0 || a->peer_count > AIDN_MAX_PEERS) return fail(AIDN_EINVAL, "launch: peer_count out of range");
  p.peer_count = a->peer_count;
  for (int i = 0; i < a->peer_count; ++i) {
    if (!a->peer_out[i]) return fail(AIDN_EINVAL, "launch: peer_out[%d] is null", i);
    p.peer_out[i] = a->peer_out[i];
  }
  p.mask = d.mask_kind != AIDN_MASK_NONE ? a->mask : nullptr;
  p.mask_kind = d.mask_kind;
  p.kv_len = a->kv_len;
  for (int i = 0; i < 4; ++i) p.mask_stride[i] = a->mask_stride[i];
  p.seq_q = a->seq_q;
  p.seq_kv = a->seq_kv;
  p.batch = (int)a->batch;
  p.num_q_heads = d.num_q_heads;
  p.num_kv_heads = d.num_kv_heads;
  p.group = h->group;
  p.head_begin = d.head_begin;
  p.head_count = h->head_count;
  p.head_dim = d.head_dim;
  p.causal = d.causal ? 1 : 0;
  p.causal_offset = d.causal_bottom_right ? (a->seq_kv - a->seq_q) : d.causal_offset;
  p.out_f32 = d.out_dtype == AIDN_F32 ? 1 : 0;
  p.scale = a->scale > 0.f ? a->scale : 1.0f / std::sqrt((float)d.head_dim);
  p.softcap = d.softcap;
  p.status = h->status_dev;
  const int64_t D = d.head_dim;
  if (all_zero(a->q_stride)) dense_strides(p.qs, d.num_q_heads, a->seq_q, D);
  else std::memcpy(p.qs, a->q_stride, sizeof(p.qs));
  if (pg) {
    if (!pg->block_table) return fail(AIDN_EINVAL, "launch_paged: null block table");
    if (pg->block_size <= 0) return fail(AIDN_EINVAL, "launch_paged: block_size must be positive");
    if (pg->num_blocks < 0 || pg->block_table_stride < 0) return fail(AIDN_EINVAL, "launch_paged: negative num_blocks or stride");
    if (a->seq_kv > 0x7fffffffll) return fail(AIDN_EINVAL, "launch_paged: seq_kv above 2^31-1");
    if (a->batch > 1 && pg->block_table_stride * pg->block_size < a->seq_kv && !a->kv_len)
      return fail(AIDN_EINVAL, "launch_paged: block_table_stride (%lld) holds fewer than seq_kv keys",
                  (long long)pg->block_table_stride);
    // kv_len lives on the device and cannot be checked here: no key beyond what a table row can address is ever
    // looked up, whatever kv_len[b] says (it would read the next sequence's row, or past the table)
    if (a->batch > 1 && pg->block_table_stride * pg->block_size < p.seq_kv) p.seq_kv = pg->block_table_stride * pg->block_size;
    p.block_table = pg->block_table;
    p.bt_stride = pg->block_table_stride;
    p.block_size = pg->block_size;
    p.block_shift = -1;
    for (int sft = 0; sft < 31; ++sft)
      if ((1 << sft) == pg->block_size) p.block_shift = sft;
    p.num_blocks = pg->num_blocks;
    const int64_t pool_dense[3] = {0, D, (int64_t)d.num_kv_heads * D};
    std::memcpy(p.ks, all_zero(a->k_stride) ? pool_dense : a->k_stride, sizeof(p.ks));
    std::memcpy(p.vs, all_zero(a->v_stride) ? pool_dense : a->v_stride, sizeof(p.vs));
    p.ks[0] = p.vs[0] = 0;
  } else {
    if (all_zero(a->k_stride)) dense_strides(p.ks, d.num_kv_heads, a->seq_kv, D);
    else std::memcpy(p.ks, a->k_stride, sizeof(p.ks));
    if (all_zero(a->v_stride)) dense_strides(p.vs, d.num_kv_heads, a->seq_kv, D);
    else std::memcpy(p.vs, a->v_stride, sizeof(p.vs));
  }
  if (all_zero(a->o_stride)) dense_strides(p.os, d.num_q_heads, a->seq_q, D);
  else std::memcpy(p.os, a->o_stride, sizeof(p.os));
  for (int i = 0; i < 3; ++i)
    if (p.qs[i] < 0 || p.ks[i] < 0 || p.vs[i] < 0 || p.os[i] < 0) return fail(AIDN_EINVAL, "launch: negative stride");
  if (p.head_count > 65535) return fail(AIDN_EINVAL, "launch: more than 65535 heads in one shard");
  return AIDN_OK;
}

// The launch shared by aidn_sdpa_launch (pg == nullptr) and aidn_sdpa_launch_paged.
int launch_common(aidn_sdpa_t h, const aidn_sdpa_args* a, const aidn_paged_kv* pg, void* cu_stream) {
  aidn::SdpaParams p;
  const int rc = build_params(h, a, pg, p);
  if (rc != AIDN_OK) return rc;
  const aidn_sdpa_desc& d = h->d;
  cudaStream_t stream = (cudaStream_t)cu_stream;
  const int64_t D = d.head_dim;

  const size_t esz = elem_size(d.qkv_dtype);
  const bool vec_ok = aligned16(p.q, p.qs, esz) && aligned16(p.k, p.ks, esz) && aligned16(p.v, p.vs, esz);
  const bool decode_ok = a->seq_q == 1 && aidn::decode_supported(d.qkv_dtype, d.head_dim) && vec_ok;
  const char* why = "";
  const bool prefill_ok = aidn::prefill_sm100_supported(p, d.qkv_dtype, &why);

  int path = d.path;
  if (path == AIDN_PATH_AUTO) path = decode_ok ? AIDN_PATH_DECODE : (prefill_ok ? AIDN_PATH_PREFILL_SM100 : AIDN_PATH_GENERIC);
  if (p.weights) {
    // the probabilities are written by the fp32 kernel only
    if (d.path != AIDN_PATH_AUTO && d.path != AIDN_PATH_GENERIC)
      return fail(AIDN_EUNSUPPORTED, "launch: attention weights are produced by the generic kernel (desc.path AUTO or GENERIC)");
    if ((uintptr_t)p.weights % 4 != 0) return fail(AIDN_EINVAL, "launch: weights must be 4-byte aligned");
    if (pg) return fail(AIDN_EUNSUPPORTED, "launch: attention weights over paged K/V are not defined");
    path = AIDN_PATH_GENERIC;
  }
  if (p.peer_count > 0) {
    // the stores to the other devices are issued by the tcgen05 kernel's epilogue
    if (path != AIDN_PATH_PREFILL_SM100 || !prefill_ok)
      return fail(AIDN_EUNSUPPORTED, "launch: peer_out needs the tcgen05 prefill kernel (16-bit inputs, head_dim 64 or 128)");
    if (a->gather_output) return fail(AIDN_EINVAL, "launch: peer_out and gather_output are two ways to the same result");
  }
  if (path == AIDN_PATH_DECODE && !decode_ok)
    return fail(AIDN_EUNSUPPORTED,
                "launch: decode kernel needs seq_q == 1, head_dim 64/128 (256 for 16-bit) and 16-byte aligned Q/K/V rows");
  if (path == AIDN_PATH_PREFILL_SM100 && !prefill_ok) return fail(AIDN_EUNSUPPORTED, "launch: %s", why);

  cudaError_t e = cudaSuccess;
  int launches = 0;
  if (path == AIDN_PATH_DECODE) {
    int chunk = 0, nchunks = 0;
    const int64_t need = decode_ws_bytes(h, a->batch, a->seq_kv, &chunk, &nchunks);
    float* ws = nullptr;
    if (need > 0) {
      if (a->workspace) {
        if (a->workspace_bytes < need)
          return fail(AIDN_EWORKSPACE, "launch: workspace of %lld bytes, need %lld", (long long)a->workspace_bytes,
                      (long long)need);
        if ((uintptr_t)a->workspace % 16 != 0) return fail(AIDN_EINVAL, "launch: workspace must be 16-byte aligned");
        ws = static_cast<float*>(a->workspace);
      } else if (h->scratch && h->scratch_bytes >= need) {
        ws = static_cast<float*>(h->scratch);
      } else {
        return fail(AIDN_EWORKSPACE, "launch: decode needs %lld bytes of workspace and the handle owns %lld",
                    (long long)need, (long long)h->scratch_bytes);
      }
    }
    e = aidn::launch_decode(p, d.qkv_dtype, chunk, nchunks, ws, stream, &launches);
  } else if (path == AIDN_PATH_PREFILL_SM100) {
    e = aidn::launch_prefill_sm100(p, d.qkv_dtype, stream, h->status_dev + 1, h->num_sms, h->debug, h->debug_mode,
                                   &h->prefill_maps, &why);
    launches = 1;
    if (e != cudaSuccess && why[0]) return fail(AIDN_ECUDA, "launch: %s (%s)", why, cudaGetErrorName(e));
  } else {
    e = aidn::launch_generic(p, d.qkv_dtype, stream);
    launches = 1;
  }
  if (e != cudaSuccess) return fail_cuda(e, "launch");
  h->last_path = path;
  h->last_launches = launches;

  if (a->gather_output) {
    if (!d.nccl_comm) return fail(AIDN_ENCCL, "launch: gather_output needs desc.nccl_comm");
    std::call_once(g_nccl_once, load_nccl);
    if (!g_nccl.ok) return fail(AIDN_ENCCL, "launch: libnccl.so.2 could not be loaded");
    int nranks = 0, rank = -1;
    if (g_nccl.CommCount(d.nccl_comm, &nranks) != 0 || g_nccl.CommUserRank(d.nccl_comm, &rank) != 0)
      return fail(AIDN_ENCCL, "launch: cannot query the communicator");
    if (h->head_count * nranks != d.num_q_heads || d.head_begin != rank * h->head_count)
      return fail(AIDN_EINVAL, "launch: gather needs %d equal consecutive head shards, rank r owning heads [r*n,(r+1)*n)", nranks);
    if (p.os[2] != D || p.os[1] != a->seq_q * D)
      return fail(AIDN_EINVAL, "launch: gather needs a dense [B,H,S,D] output");
    const size_t osz = p.out_f32 ? 4 : 2;
    const int dt = p.out_f32 ? kNcclFloat32 : (d.qkv_dtype == AIDN_F16 ? kNcclFloat16 : kNcclBfloat16);
    const size_t count = (size_t)h->head_count * (size_t)a->seq_q * (size_t)D;
    int rc = g_nccl.GroupStart();
    for (int64_t b = 0; b < a->batch && rc == 0; ++b) {
      char* recv = static_cast<char*>(a->out) + (size_t)b * p.os[0] * osz;
      rc = g_nccl.AllGather(recv + (size_t)rank * count * osz, recv, count, dt, d.nccl_comm, stream);
    }
    const int rc2 = g_nccl.GroupEnd();
    if (rc == 0) rc = rc2;
    if (rc != 0)
      return fail(AIDN_ENCCL, "launch: ncclAllGather failed: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?");
    h->last_launches += 1;
  }
  return post_launch_check(stream, "aidn_sdpa_launch", h->status_dev);
}

}  // namespace

extern "C" {

int aidn_sdpa_launch(aidn_sdpa_t h, const aidn_sdpa_args* a, void* cu_stream) {
  return launch_common(h, a, nullptr, cu_stream);
}

int aidn_sdpa_launch_paged(aidn_sdpa_t h, const aidn_sdpa_args* a, const aidn_paged_kv* paged, void* cu_stream) {
  if (!paged) {
    g_err[0] = 0;
    return fail(AIDN_EINVAL, "launch_paged: null aidn_paged_kv");
  }
  return launch_common(h, a, paged, cu_stream);
}

int64_t aidn_sdpa_backward_workspace_bytes(aidn_sdpa_t h, int64_t batch, int64_t seq_q) {
  if (!h || batch <= 0 || seq_q <= 0) {
    fail(AIDN_EINVAL, "backward_workspace_bytes: bad argument");
    return -1;
  }
  int64_t bytes = align_up(batch * h->head_count * seq_q * (int64_t)sizeof(float), 256);   // delta
  if (h->d.qkv_dtype != AIDN_F32 && h->d.out_dtype == AIDN_F32)                              // dO in the input dtype
    bytes += align_up(batch * h->head_count * seq_q * (int64_t)h->d.head_dim * 2, 256);
  return bytes;
}

int aidn_sdpa_backward(aidn_sdpa_t h, const aidn_sdpa_bwd_args* a, void* cu_stream) {
  g_err[0] = 0;
  if (!h || !a) return fail(AIDN_EINVAL, "backward: null argument");
  if (!a->dout || !a->dq || !a->dk || !a->dv) return fail(AIDN_EINVAL, "backward: null gradient pointer");
  if (!a->fwd.lse) return fail(AIDN_EINVAL, "backward: the forward's log-sum-exp (fwd.lse) is required");
  if (h->d.softcap > 0.f) return fail(AIDN_EUNSUPPORTED, "backward: logit softcap is not differentiated here");
  aidn::BwdParams bp;
  const int rc = build_params(h, &a->fwd, a->paged, bp.p);
  if (rc != AIDN_OK) return rc;
  bp.p.lse = a->fwd.lse;   // read here, whatever desc.emit_lse says
  bp.p.weights = nullptr;
  const int64_t need = aidn_sdpa_backward_workspace_bytes(h, a->fwd.batch, a->fwd.seq_q);
  if (!a->fwd.workspace || a->fwd.workspace_bytes < need)
    return fail(AIDN_EWORKSPACE, "backward: workspace of %lld bytes, need %lld", (long long)a->fwd.workspace_bytes, (long long)need);
  if ((uintptr_t)a->fwd.workspace % 16 != 0) return fail(AIDN_EINVAL, "backward: workspace must be 16-byte aligned");
  bp.dout = a->dout;
  if (all_zero(a->do_stride)) std::memcpy(bp.dos, bp.p.os, sizeof(bp.dos));
  else std::memcpy(bp.dos, a->do_stride, sizeof(bp.dos));
  for (int i = 0; i < 3; ++i)
    if (bp.dos[i] < 0) return fail(AIDN_EINVAL, "backward: negative stride");
  bp.dq = a->dq; bp.dk = a->dk; bp.dv = a->dv;
  bp.delta = static_cast<float*>(a->fwd.workspace);
  bp.dout_t = nullptr;
  if (h->d.qkv_dtype != AIDN_F32 && h->d.out_dtype == AIDN_F32)
    bp.dout_t = static_cast<char*>(a->fwd.workspace) +
                align_up(a->fwd.batch * h->head_count * a->fwd.seq_q * (int64_t)sizeof(float), 256);
  bp.no_tcgen05 = h->d.path == AIDN_PATH_GENERIC ? 1 : 0;
  bp.round_dout = 0;
  bp.expire = h->debug_mode == 3 ? 1 : 0;
  int launches = 0, used_tcgen05 = 0;
  cudaError_t e = aidn::launch_backward(bp, h->d.qkv_dtype, (cudaStream_t)cu_stream, &launches, &used_tcgen05);
  if (e != cudaSuccess) return fail_cuda(e, "backward");
  h->last_path = used_tcgen05 ? AIDN_PATH_PREFILL_SM100 : AIDN_PATH_GENERIC;
  h->last_launches = launches;
  return post_launch_check((cudaStream_t)cu_stream, "aidn_sdpa_backward", h->status_dev);
}

// Decode for callers that cannot allocate device memory (no handle, no workspace): see include/aidn_sdpa.h.
int aidn_sdpa_decode_noalloc(const aidn_sdpa_desc* desc, const aidn_sdpa_args* a, void* cu_stream) {
  g_err[0] = 0;
  if (!desc || !a) return fail(AIDN_EINVAL, "decode_noalloc: null argument");
  const aidn_sdpa_desc& d = *desc;
  if (d.qkv_dtype < AIDN_F32 || d.qkv_dtype > AIDN_BF16) return fail(AIDN_EINVAL, "decode_noalloc: unknown qkv_dtype");
  if (d.out_dtype != AIDN_F32 && d.out_dtype != d.qkv_dtype)
    return fail(AIDN_EINVAL, "decode_noalloc: out_dtype must be fp32 or equal to qkv_dtype");
  if (d.num_q_heads <= 0 || d.num_kv_heads <= 0 || d.num_q_heads % d.num_kv_heads != 0)
    return fail(AIDN_EINVAL, "decode_noalloc: numHeads must be a positive multiple of numKVHeads");
  if (d.mask_kind < AIDN_MASK_NONE || d.mask_kind > AIDN_MASK_ADD_F32) return fail(AIDN_EINVAL, "decode_noalloc: unknown mask_kind");
  if (!(d.softcap >= 0.f)) return fail(AIDN_EINVAL, "decode_noalloc: softcap must be >= 0");
  if (d.decode_chunk < 0 || (d.decode_chunk > 0 && d.decode_chunk % 8 != 0))
    return fail(AIDN_EINVAL, "decode_noalloc: decode_chunk must be 0 or a positive multiple of 8");
  int cur = -1;
  cudaError_t ce = cudaGetDevice(&cur);
  if (ce != cudaSuccess) return fail_cuda(ce, "decode_noalloc: cudaGetDevice");
  if (cur != d.device)
    return fail(AIDN_EINVAL, "decode_noalloc: desc.device (%d) is not the current device (%d)", d.device, cur);
  if (!aidn_sdpa_device_supported(d.device))
    return fail(AIDN_EUNSUPPORTED, "decode_noalloc: device %d is not compute capability 10.x", d.device);
  aidn_sdpa tmp;  // on the stack: only the fields the chunk heuristic reads
  std::memset(&tmp, 0, sizeof(tmp));
  tmp.d = d;
  tmp.group = d.num_q_heads / d.num_kv_heads;
  tmp.head_count = d.head_count > 0 ? d.head_count : d.num_q_heads - d.head_begin;
  if (d.head_begin < 0 || tmp.head_count <= 0 || d.head_begin + tmp.head_count > d.num_q_heads ||
      d.head_begin % tmp.group != 0 || tmp.head_count % tmp.group != 0)
    return fail(AIDN_EINVAL, "decode_noalloc: the head shard must lie inside the tensor and cover whole KV groups");
  if (tmp.head_count > 65535) return fail(AIDN_EINVAL, "decode_noalloc: more than 65535 heads in one shard");
  if (!a->q || !a->k || !a->v || !a->out) return fail(AIDN_EINVAL, "decode_noalloc: null tensor pointer");
  if (a->batch <= 0 || a->batch > 65535 || a->seq_kv <= 0) return fail(AIDN_EINVAL, "decode_noalloc: bad batch or seq_kv");
  if (a->seq_q != 1) return fail(AIDN_EUNSUPPORTED, "decode_noalloc: seq_q must be 1");
  if (d.emit_lse && !a->lse) return fail(AIDN_EINVAL, "decode_noalloc: emit_lse set but lse pointer is null");
  if (d.mask_kind != AIDN_MASK_NONE && !a->mask) return fail(AIDN_EINVAL, "decode_noalloc: mask_kind set but mask pointer is null");
  if (a->scale < 0.f || std::isnan(a->scale)) return fail(AIDN_EINVAL, "decode_noalloc: scale must be >= 0");
  if (!aidn::decode_supported(d.qkv_dtype, d.head_dim))
    return fail(AIDN_EUNSUPPORTED, "decode_noalloc: head_dim must be 64 or 128 (256 for 16-bit inputs)");

  aidn::SdpaParams p;
  std::memset(&p, 0, sizeof(p));
  p.q = a->q; p.k = a->k; p.v = a->v; p.out = a->out;
  p.lse = d.emit_lse ? a->lse : nullptr;
  p.mask = d.mask_kind != AIDN_MASK_NONE ? a->mask : nullptr;
  p.mask_kind = d.mask_kind;
  p.kv_len = a->kv_len;
  for (int i = 0; i < 4; ++i) p.mask_stride[i] = a->mask_stride[i];
  p.seq_q = 1;
  p.seq_kv = a->seq_kv;
  p.batch = (int)a->batch;
  p.num_q_heads = d.num_q_heads;
  p.num_kv_heads = d.num_kv_heads;
  p.group = tmp.group;
  p.head_begin = d.head_begin;
  p.head_count = tmp.head_count;
  p.head_dim = d.head_dim;
  p.causal = d.causal ? 1 : 0;
  p.causal_offset = d.causal_bottom_right ? (a->seq_kv - 1) : d.causal_offset;
  p.out_f32 = d.out_dtype == AIDN_F32 ? 1 : 0;
  p.scale = a->scale > 0.f ? a->scale : 1.0f / std::sqrt((float)d.head_dim);
  p.softcap = d.softcap;
  p.status = nullptr;
  const int64_t D = d.head_dim;
  if (all_zero(a->q_stride)) dense_strides(p.qs, d.num_q_heads, 1, D); else std::memcpy(p.qs, a->q_stride, sizeof(p.qs));
  if (all_zero(a->k_stride)) dense_strides(p.ks, d.num_kv_heads, a->seq_kv, D); else std::memcpy(p.ks, a->k_stride, sizeof(p.ks));
  if (all_zero(a->v_stride)) dense_strides(p.vs, d.num_kv_heads, a->seq_kv, D); else std::memcpy(p.vs, a->v_stride, sizeof(p.vs));
  if (all_zero(a->o_stride)) dense_strides(p.os, d.num_q_heads, 1, D); else std::memcpy(p.os, a->o_stride, sizeof(p.os));
  for (int i = 0; i < 3; ++i)
    if (p.qs[i] < 0 || p.ks[i] < 0 || p.vs[i] < 0 || p.os[i] < 0) return fail(AIDN_EINVAL, "decode_noalloc: negative stride");
  const size_t esz = elem_size(d.qkv_dtype);
  if (!(aligned16(p.q, p.qs, esz) && aligned16(p.k, p.ks, esz) && aligned16(p.v, p.vs, esz)))
    return fail(AIDN_EUNSUPPORTED, "decode_noalloc: Q/K/V rows must be 16-byte aligned");

  int chunk = 0, nchunks = 0;
  const int64_t need = decode_ws_bytes(&tmp, a->batch, a->seq_kv, &chunk, &nchunks);
  const int64_t have = aidn::decode_static_scratch_bytes();
  if (need > have)
    return fail(AIDN_EWORKSPACE,
                "decode_noalloc: this shape needs %lld bytes of split-KV scratch but the library's static array holds %lld; "
                "lower batch*heads*ceil(seq_kv/chunk) (a larger decode_chunk helps) or use aidn_sdpa_launch with a workspace",
                (long long)need, (long long)have);
  int launches = 0;
  cudaError_t e = aidn::launch_decode_static(p, d.qkv_dtype, chunk, nchunks, (cudaStream_t)cu_stream, &launches);
  if (e != cudaSuccess) return fail_cuda(e, "decode_noalloc");
  return post_launch_check((cudaStream_t)cu_stream, "aidn_sdpa_decode_noalloc", nullptr);
}

int aidn_qkv_rope_cache(const aidn_qkv_rope_args* a, void* cu_stream) {
  g_err[0] = 0;
  if (!a) return fail(AIDN_EINVAL, "qkv_rope_cache: null argument");
  if (!a->input || !a->weights || !a->cosine || !a->sine || !a->query || !a->key_cache || !a->value_cache)
    return fail(AIDN_EINVAL, "qkv_rope_cache: null buffer");
  if (a->heads <= 0) return fail(AIDN_EINVAL, "qkv_rope_cache: heads must be > 0");
  if (a->kv_heads <= 0 || a->kv_heads > a->heads || a->heads % a->kv_heads != 0)
    return fail(AIDN_EINVAL, "qkv_rope_cache: kv_heads must divide heads");
  if (a->head_dim <= 0 || a->head_dim > 256 || a->head_dim % 2 != 0)
    return fail(AIDN_EINVAL, "qkv_rope_cache: head_dim must be even and in [2, 256]");
  if (a->tokens <= 0) return fail(AIDN_EINVAL, "qkv_rope_cache: tokens must be > 0");
  if (a->cache_capacity <= 0 || a->max_position <= 0) return fail(AIDN_EINVAL, "qkv_rope_cache: cache_capacity and max_position must be > 0");
  if (!a->positions && (a->position < 0 || (int64_t)a->position + a->tokens > a->max_position))
    return fail(AIDN_EINVAL, "qkv_rope_cache: position outside the cos/sin tables");
  if (!a->positions && !a->cache_rows && (int64_t)a->position + a->tokens > a->cache_capacity)
    return fail(AIDN_EINVAL, "qkv_rope_cache: position outside the cache");   /* ArgumentOutOfRangeException(position) */
  if (a->weight_dtype != AIDN_F32 && a->weight_dtype != AIDN_BF16) return fail(AIDN_EINVAL, "qkv_rope_cache: weights are fp32 or bf16");
  if (a->query_dtype < AIDN_F32 || a->query_dtype > AIDN_BF16 || a->cache_dtype < AIDN_F32 || a->cache_dtype > AIDN_BF16)
    return fail(AIDN_EINVAL, "qkv_rope_cache: unknown output dtype");
  const int64_t model = (int64_t)a->heads * a->head_dim;
  if (model % 8 != 0) return fail(AIDN_EUNSUPPORTED, "qkv_rope_cache: heads * head_dim must be a multiple of 8");
  if (model > aidn::qkv_rope_max_model())
    return fail(AIDN_EUNSUPPORTED, "qkv_rope_cache: heads * head_dim above %lld", (long long)aidn::qkv_rope_max_model());
  if ((uintptr_t)a->weights % 16 != 0 || (uintptr_t)a->input % 16 != 0)
    return fail(AIDN_EINVAL, "qkv_rope_cache: input and weights must be 16-byte aligned");
  // per-device facts, looked up once: this entry point has no handle to keep them in.  Unsynchronised on purpose:
  // two threads racing here write the same values (the lookups are idempotent), and g_sms is written last.
  static int g_sms[64] = {0};
  static int g_ok[64] = {0};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "qkv_rope_cache: device query");
  if (dev < 0 || dev >= 64) return fail(AIDN_EUNSUPPORTED, "qkv_rope_cache: device ordinal %d", dev);
  if (g_sms[dev] == 0) {
    int sms_q = 0;
    e = cudaDeviceGetAttribute(&sms_q, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return fail_cuda(e, "qkv_rope_cache: device query");
    g_ok[dev] = aidn_sdpa_device_supported(dev);
    g_sms[dev] = sms_q;
  }
  const int sms = g_sms[dev];
  if (!g_ok[dev]) return fail(AIDN_EUNSUPPORTED, "qkv_rope_cache: device %d is not compute capability 10.x", dev);
  aidn::QkvRopeParams p;
  std::memset(&p, 0, sizeof(p));
  p.input = a->input; p.weights = a->weights; p.bias = a->bias; p.cosine = a->cosine; p.sine = a->sine;
  p.query = a->query; p.key_cache = a->key_cache; p.value_cache = a->value_cache;
  p.positions = a->positions; p.cache_rows = a->cache_rows;
  p.tokens = a->tokens; p.heads = a->heads; p.kv_heads = a->kv_heads; p.head_dim = a->head_dim;
  p.position = a->position; p.query_dtype = a->query_dtype; p.cache_dtype = a->cache_dtype;
  p.cache_capacity = a->cache_capacity; p.max_position = a->max_position; p.model = (int32_t)model;
  int launches = 0;
  e = aidn::launch_qkv_rope_cache(p, a->weight_dtype, sms, (cudaStream_t)cu_stream, &launches);
  if (e != cudaSuccess) return fail_cuda(e, "qkv_rope_cache");
  return post_launch_check((cudaStream_t)cu_stream, "aidn_qkv_rope_cache", nullptr);
}

int aidn_rope_interleaved(const float* input, const float* cosine, const float* sine, float* output, int64_t rows,
                          int32_t head_dim, int32_t seq_len, int32_t start_position, void* cu_stream) {
  g_err[0] = 0;
  if (rows <= 0 || head_dim <= 0 || seq_len <= 0) return fail(AIDN_EINVAL, "rope_interleaved: rows, headDim and seqLen must be > 0");
  if (head_dim % 2 != 0) return fail(AIDN_EINVAL, "rope_interleaved: headDim must be even");
  if (start_position < 0) return fail(AIDN_EINVAL, "rope_interleaved: startPosition must be >= 0");
  if (!input || !cosine || !sine || !output) return fail(AIDN_EINVAL, "rope_interleaved: null buffer");
  if ((uintptr_t)input % 8 != 0 || (uintptr_t)output % 8 != 0) return fail(AIDN_EINVAL, "rope_interleaved: buffers must be 8-byte aligned");
  cudaError_t e = aidn::launch_rope_interleaved(input, cosine, sine, output, rows, head_dim, seq_len, start_position,
                                                (cudaStream_t)cu_stream);
  if (e != cudaSuccess) return fail_cuda(e, "rope_interleaved");
  return AIDN_OK;
}

int aidn_paged_kv_append(const void* new_keys, const void* new_values, void* key_pool, void* value_pool,
                         const int32_t* block_table, int64_t start_position, int64_t tokens, int32_t block_size,
                         int32_t num_blocks, int64_t row_bytes, void* cu_stream) {
  g_err[0] = 0;
  if (tokens < 0 || start_position < 0) return fail(AIDN_EINVAL, "paged_kv_append: newLen and the start position must be >= 0");
  if (tokens == 0) return AIDN_OK;
  if (!new_keys || !new_values || !key_pool || !value_pool || !block_table) return fail(AIDN_EINVAL, "paged_kv_append: null buffer");
  if (block_size <= 0 || num_blocks <= 0) return fail(AIDN_EINVAL, "paged_kv_append: block_size and num_blocks must be > 0");
  if (row_bytes <= 0 || row_bytes % 16 != 0) return fail(AIDN_EINVAL, "paged_kv_append: row_bytes must be a positive multiple of 16");
  if (start_position + tokens > (int64_t)num_blocks * block_size)
    return fail(AIDN_EINVAL, "paged_kv_append: the sequence would reach %lld tokens, above the pool capacity %lld",
                (long long)(start_position + tokens), (long long)num_blocks * block_size);   /* InvalidOperationException there */
  if ((uintptr_t)new_keys % 16 || (uintptr_t)new_values % 16 || (uintptr_t)key_pool % 16 || (uintptr_t)value_pool % 16)
    return fail(AIDN_EINVAL, "paged_kv_append: buffers must be 16-byte aligned");
  cudaError_t e = aidn::launch_paged_append(new_keys, new_values, key_pool, value_pool, block_table, start_position, tokens,
                                            block_size, num_blocks, row_bytes, (cudaStream_t)cu_stream);
  if (e != cudaSuccess) return fail_cuda(e, "paged_kv_append");
  return AIDN_OK;
}

// ---- fused multi-head attention forward ---------------------------------------------------------------------------
namespace {
struct MhaPlan {
  int64_t off_x, off_w, off_q, off_k, off_v, off_o, total;
};
MhaPlan mha_plan(const aidn_sdpa* h, int64_t batch, int64_t seq, int input_dtype, int weight_dtype) {
  const int64_t dm = (int64_t)h->d.num_q_heads * h->d.head_dim;
  const int64_t esz = (int64_t)elem_size(h->d.qkv_dtype);
  const int64_t act = align_up(batch * seq * dm * esz, 1024), wgt = align_up(dm * dm * esz, 1024);
  MhaPlan pl;
  int64_t off = 0;
  pl.off_x = off; off += input_dtype != h->d.qkv_dtype ? act : 0;
  pl.off_w = off; off += weight_dtype != h->d.qkv_dtype ? 4 * wgt : 0;
  pl.off_q = off; off += act;
  pl.off_k = off; off += act;
  pl.off_v = off; off += act;
  pl.off_o = off; off += act;
  pl.total = off;
  return pl;
}
int mha_check_handle(const aidn_sdpa* h) {
  const aidn_sdpa_desc& d = h->d;
  if (d.out_dtype != d.qkv_dtype)
    return fail(AIDN_EUNSUPPORTED, "mha: the handle must have out_dtype == qkv_dtype (the attention output feeds a projection)");
  if (d.num_kv_heads != d.num_q_heads || h->head_count != d.num_q_heads)
    return fail(AIDN_EUNSUPPORTED, "mha: the handle must cover all heads with num_kv_heads == num_q_heads");
  if (d.emit_lse || d.softcap > 0.f || d.nccl_comm)
    return fail(AIDN_EUNSUPPORTED, "mha: the handle must not ask for log-sum-exp, softcap or a gather");
  if (d.mask_kind == AIDN_MASK_ADD_F32) return fail(AIDN_EUNSUPPORTED, "mha: the mask is a keep-mask (Tensor<bool>) or absent");
  // desc.causal is honoured (causal self-attention without materialising the mask): an extension, the reference's
  // MultiHeadAttentionForward expresses causality through its boolean mask only.
  return AIDN_OK;
}
}  // namespace

int64_t aidn_mha_workspace_bytes(aidn_sdpa_t h, int64_t batch, int64_t seq, int32_t input_dtype, int32_t weight_dtype) {
  g_err[0] = 0;
  if (!h || batch <= 0 || seq <= 0) {
    fail(AIDN_EINVAL, "mha_workspace_bytes: bad argument");
    return -1;
  }
  if (mha_check_handle(h) != AIDN_OK) return -1;
  return mha_plan(h, batch, seq, input_dtype, weight_dtype).total;
}

int aidn_mha_forward(aidn_sdpa_t h, const aidn_mha_args* a, void* cu_stream) {
  g_err[0] = 0;
  if (!h || !a) return fail(AIDN_EINVAL, "mha: null argument");
  if (!a->input || !a->q_weight || !a->k_weight || !a->v_weight || !a->out_weight || !a->out)
    return fail(AIDN_EINVAL, "mha: null tensor pointer");
  if (a->batch <= 0 || a->seq <= 0) return fail(AIDN_EINVAL, "mha: batch and seq must be positive");
  int rc = mha_check_handle(h);
  if (rc != AIDN_OK) return rc;
  const aidn_sdpa_desc& d = h->d;
  auto dtype_ok = [&](int t) { return t == AIDN_F32 || t == d.qkv_dtype; };
  if (!dtype_ok(a->input_dtype) || !dtype_ok(a->weight_dtype) || !dtype_ok(a->out_dtype))
    return fail(AIDN_EINVAL, "mha: input, weight and output dtypes must be fp32 or the handle's qkv_dtype");
  if (d.mask_kind != AIDN_MASK_NONE && !a->mask) return fail(AIDN_EINVAL, "mha: mask_kind set but mask pointer is null");
  const MhaPlan pl = mha_plan(h, a->batch, a->seq, a->input_dtype, a->weight_dtype);
  if (!a->workspace || a->workspace_bytes < pl.total)
    return fail(AIDN_EWORKSPACE, "mha: workspace of %lld bytes, need %lld", (long long)(a->workspace ? a->workspace_bytes : 0),
                (long long)pl.total);
  if ((uintptr_t)a->workspace % 256 != 0) return fail(AIDN_EINVAL, "mha: workspace must be 256-byte aligned");
  cudaStream_t stream = (cudaStream_t)cu_stream;
  char* ws = static_cast<char*>(a->workspace);
  const int64_t H = d.num_q_heads, D = d.head_dim, dm = H * D, S = a->seq, B = a->batch;
  const int cast_kind = d.qkv_dtype == AIDN_BF16 ? 0 : 1;
  const int64_t esz = (int64_t)elem_size(d.qkv_dtype);
  // tcgen05 GEMMs for 16-bit arithmetic on head sizes 64 / 128; the fp32 FFMA GEMM for everything else
  const bool tensor_route = d.qkv_dtype != AIDN_F32 && (D == 64 || D == 128) && dm % 128 == 0 && d.path != AIDN_PATH_GENERIC;
  int launches = 0;
  cudaError_t e = cudaSuccess;

  const void* x = a->input;
  if (a->input_dtype != d.qkv_dtype) {
    e = aidn::launch_cast(cast_kind, a->input, ws + pl.off_x, B * S * dm, stream);
    if (e != cudaSuccess) return fail_cuda(e, "mha: input cast");
    x = ws + pl.off_x;
    ++launches;
  }
  const void* w[4] = {a->q_weight, a->k_weight, a->v_weight, a->out_weight};
  if (a->weight_dtype != d.qkv_dtype) {
    const int64_t wgt = align_up(dm * dm * esz, 1024);
    for (int i = 0; i < 4; ++i) {
      void* dst = ws + pl.off_w + i * wgt;
      e = aidn::launch_cast(cast_kind, w[i], dst, dm * dm, stream);
      if (e != cudaSuccess) return fail_cuda(e, "mha: weight cast");
      w[i] = dst;
      ++launches;
    }
  }

  const char* why = "";
  aidn::ProjGemm g;
  std::memset(&g, 0, sizeof(g));
  g.a = x;
  g.batch = B; g.seq = S; g.k = dm; g.n = dm;
  g.head_dim = (int)D;
  g.bf16 = d.qkv_dtype == AIDN_BF16;
  g.num_mats = 3;
  g.out_f32 = false;
  for (int i = 0; i < 3; ++i) g.w[i] = w[i];
  g.c[0] = ws + pl.off_q; g.c[1] = ws + pl.off_k; g.c[2] = ws + pl.off_v;
  g.c_stride[0] = H * S * D; g.c_stride[1] = S * D; g.c_stride[2] = D;    // [B, H, S, d]
  auto gemm = [&](const char* what) -> int {
    if (tensor_route) {
      if (!aidn::proj_gemm_sm100_supported(g, &why)) return fail(AIDN_EUNSUPPORTED, "mha: %s", why);
      e = aidn::launch_proj_gemm_sm100(g, stream, h->num_sms, h->status_dev, &why, h->debug_mode == 3);
    } else {
      if (!aidn::proj_gemm_generic_supported(g, &why)) return fail(AIDN_EUNSUPPORTED, "mha: %s", why);
      e = aidn::launch_proj_gemm_generic(g, d.qkv_dtype, stream);
    }
    if (e != cudaSuccess) return why[0] ? fail(AIDN_ECUDA, "mha: %s (%s)", why, cudaGetErrorName(e)) : fail_cuda(e, what);
    ++launches;
    return AIDN_OK;
  };
  rc = gemm("mha: QKV projection");
  if (rc != AIDN_OK) return rc;

  aidn_sdpa_args sa;
  std::memset(&sa, 0, sizeof(sa));
  sa.q = g.c[0]; sa.k = g.c[1]; sa.v = g.c[2];
  sa.out = ws + pl.off_o;
  sa.mask = a->mask;
  for (int i = 0; i < 4; ++i) sa.mask_stride[i] = a->mask_stride[i];
  sa.batch = B; sa.seq_q = S; sa.seq_kv = S;
  sa.o_stride[0] = S * dm; sa.o_stride[1] = D; sa.o_stride[2] = dm;      // heads side by side: [B, S, H*d]
  rc = launch_common(h, &sa, nullptr, cu_stream);
  if (rc != AIDN_OK) return rc;
  launches += h->last_launches;

  g.a = ws + pl.off_o;
  g.num_mats = 1;
  g.w[0] = w[3];
  g.c[0] = a->out;
  g.out_f32 = a->out_dtype == AIDN_F32;
  g.c_stride[0] = S * dm; g.c_stride[1] = D; g.c_stride[2] = dm;
  rc = gemm("mha: output projection");
  if (rc != AIDN_OK) return rc;
  h->last_launches = launches;
  return post_launch_check(stream, "aidn_mha_forward", h->status_dev);
}

static int cast_common(int kind, const void* src, void* dst, int64_t n, void* cu_stream) {
  g_err[0] = 0;
  if (n < 0 || (n > 0 && (!src || !dst))) return fail(AIDN_EINVAL, "cast: bad argument");
  cudaError_t e = aidn::launch_cast(kind, src, dst, n, (cudaStream_t)cu_stream);
  if (e != cudaSuccess) return fail_cuda(e, "cast");
  return AIDN_OK;
}

int aidn_peer_export(const void* dev_ptr, void* handle64, int64_t* offset) {
  g_err[0] = 0;
  if (!dev_ptr || !handle64 || !offset) return fail(AIDN_EINVAL, "peer_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handle size");
  // the handle names a whole allocation: find its base
  typedef int (*GetRangeFn)(unsigned long long*, size_t*, unsigned long long);   // CUresult cuMemGetAddressRange_v2
  static GetRangeFn get_range = nullptr;
  if (!get_range) {
    void* raw = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &raw, cudaEnableDefault, &qres) != cudaSuccess || !raw ||
        qres != cudaDriverEntryPointSuccess)
      return fail(AIDN_ECUDA, "peer_export: cuMemGetAddressRange is not available from the driver");
    get_range = reinterpret_cast<GetRangeFn>(raw);
  }
  unsigned long long base = 0;
  size_t size = 0;
  if (get_range(&base, &size, (unsigned long long)(uintptr_t)dev_ptr) != 0)
    return fail(AIDN_EINVAL, "peer_export: not a device allocation");
  cudaIpcMemHandle_t hdl;
  cudaError_t e = cudaIpcGetMemHandle(&hdl, reinterpret_cast<void*>((uintptr_t)base));
  if (e != cudaSuccess) return fail_cuda(e, "peer_export");
  std::memcpy(handle64, &hdl, 64);
  *offset = (int64_t)((uintptr_t)dev_ptr - (uintptr_t)base);
  return AIDN_OK;
}

int aidn_peer_open(const void* handle64, void** base) {
  g_err[0] = 0;
  if (!handle64 || !base) return fail(AIDN_EINVAL, "peer_open: null argument");
  cudaIpcMemHandle_t hdl;
  std::memcpy(&hdl, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(base, hdl, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail_cuda(e, "peer_open");
  return AIDN_OK;
}

int aidn_peer_close(void* base) {
  g_err[0] = 0;
  if (!base) return fail(AIDN_EINVAL, "peer_close: null argument");
  cudaError_t e = cudaIpcCloseMemHandle(base);
  if (e != cudaSuccess) return fail_cuda(e, "peer_close");
  return AIDN_OK;
}

int aidn_cast_f32_to_bf16(const float* src, void* dst, int64_t n, void* s) { return cast_common(0, src, dst, n, s); }
int aidn_cast_f32_to_f16(const float* src, void* dst, int64_t n, void* s) { return cast_common(1, src, dst, n, s); }
int aidn_cast_bf16_to_f32(const void* src, float* dst, int64_t n, void* s) { return cast_common(2, src, dst, n, s); }
int aidn_cast_f16_to_f32(const void* src, float* dst, int64_t n, void* s) { return cast_common(3, src, dst, n, s); }

}  // extern "C"
