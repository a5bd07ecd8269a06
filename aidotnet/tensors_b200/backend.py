"""Host-side mirror of the attention methods of the reference's CUDA backend, routed to the sm_100a library.

Method names, argument order, argument meaning and error behaviour follow
``src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/CudaBackend.cs`` of the reference:

    ScaledDotProductAttention  :8322-8379      FlashAttention      :8522-8538
    FlashAttentionV2           :8540-8578      GroupedQueryAttention :8721-8759
    FlashDecode                :2968-3021      PagedAttentionDecode/Prefill{,Gqa} :2845-2966
    QkvProjectionRoPECacheD64  :8389-8439      RopeInterleaved     :8441-8470
    FlashAttentionBackward     :8580-8604

and the interface they implement (``Engines/DirectGpu/IDirectGpuBackend.cs:1421-1503``).  Buffers are
``GpuBuffer`` objects (the mirror of ``IGpuBuffer``, ``IDirectGpuBackend.cs:3776-3803``): a device
allocation with ``Size`` (element count), ``SizeInBytes`` and ``Handle`` (device address).  torch is used
only to own device memory and streams.

Differences from the reference methods, all deliberate:
  * buffers may hold bf16 / fp16 as well as fp32 (``GpuBuffer.dtype``); the output buffer is fp32 or the input dtype;
  * element counts are 64-bit (the reference's ``checked(int)`` products overflow from S = 8192 on);
  * ``attentionWeights`` must be None: the weight-returning call stays on the reference's own kernel;
  * a failure raises; nothing falls back to a CPU path.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from . import native as N

_DTYPE = {torch.float32: N.F32, torch.float16: N.F16, torch.bfloat16: N.BF16}


class GpuBuffer:
    """Mirror of ``IGpuBuffer``: ``Size`` elements of ``dtype`` at device address ``Handle``."""

    def __init__(self, tensor: torch.Tensor):
        if not tensor.is_cuda:
            raise ValueError("GpuBuffer needs a CUDA tensor")
        if not tensor.is_contiguous():
            raise ValueError("GpuBuffer needs a contiguous allocation")
        self.tensor = tensor

    @property
    def Size(self) -> int:
        return self.tensor.numel()

    @property
    def SizeInBytes(self) -> int:
        return self.tensor.numel() * self.tensor.element_size()

    @property
    def Handle(self) -> int:
        return self.tensor.data_ptr()

    @property
    def dtype(self) -> torch.dtype:
        return self.tensor.dtype


class CudaBackend:
    """The attention slice of ``CudaBackend``: one device, one stream (``CudaBackend.cs:371-375``)."""

    def __init__(self, device: int = 0, stream: Optional[torch.cuda.Stream] = None, path: int = N.PATH_AUTO,
                 decode_chunk: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this backend has no CPU path")
        N.load()
        self.device = device
        torch.cuda.set_device(device)
        self._stream = stream
        self._path = path
        self._decode_chunk = decode_chunk
        self._handles: Dict[Tuple, N.Handle] = {}
        self._scratch: Optional[torch.Tensor] = None
        self.launch_count = 0  # kernels enqueued by this backend (the reference counts launches in GpuLaunchProbe)

    # -- plumbing ---------------------------------------------------------------------------------------
    @property
    def stream(self) -> torch.cuda.Stream:
        return self._stream if self._stream is not None else torch.cuda.current_stream(self.device)

    def AllocateBuffer(self, size: int, dtype: torch.dtype = torch.float32) -> GpuBuffer:
        return GpuBuffer(torch.empty(int(size), dtype=dtype, device=f"cuda:{self.device}"))

    def AllocateByteBuffer(self, size: int) -> GpuBuffer:
        return GpuBuffer(torch.empty(int(size), dtype=torch.uint8, device=f"cuda:{self.device}"))

    def ConvertToFp16(self, src: GpuBuffer, dst: GpuBuffer, size: int) -> None:
        N.cast("f32_to_f16", src.Handle, dst.Handle, size, self.stream.cuda_stream)

    def ConvertToFp32(self, src: GpuBuffer, dst: GpuBuffer, size: int) -> None:
        N.cast("f16_to_f32", src.Handle, dst.Handle, size, self.stream.cuda_stream)

    def ConvertToBf16(self, src: GpuBuffer, dst: GpuBuffer, size: int) -> None:
        N.cast("f32_to_bf16", src.Handle, dst.Handle, size, self.stream.cuda_stream)

    def Synchronize(self) -> None:
        self.stream.synchronize()

    def _handle(self, **kw) -> N.Handle:
        key = tuple(sorted(kw.items()))
        h = self._handles.get(key)
        if h is None:
            if len(self._handles) >= 128:  # e.g. one handle per startPos of a long chunked prefill: drop the oldest
                self._handles.pop(next(iter(self._handles))).close()
            h = N.Handle(device=self.device, path=self._path, decode_chunk=self._decode_chunk, **kw)
            self._handles[key] = h
        return h

    def _workspace(self, nbytes: int) -> Tuple[Optional[int], int]:
        if nbytes <= 0:
            return None, 0
        if self._scratch is None or self._scratch.numel() < nbytes:
            self._scratch = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{self.device}")
        return self._scratch.data_ptr(), self._scratch.numel()

    @staticmethod
    def _check_dims(batch, numHeads, seqQ, seqK, headDim):
        if batch <= 0 or numHeads <= 0 or seqQ <= 0 or seqK <= 0 or headDim <= 0:
            raise ValueError("Attention dimensions must be positive.")  # ArgumentOutOfRangeException in the reference

    def _run(self, h: N.Handle, *, query, key, value, output, batch, seqQ, seqK, scale, lse=None, mask=None,
             mask_stride=(0, 0, 0, 0), kv_len=None, q_stride=None, k_stride=None, v_stride=None, o_stride=None,
             block_table=None, block_table_stride=0, block_size=0, num_blocks=0, weights=None):
        ws, ws_bytes = self._workspace(h.workspace_bytes(batch, seqQ, seqK))
        h.launch(q=query.Handle, k=key.Handle, v=value.Handle, out=output.Handle, batch=batch, seq_q=seqQ, seq_kv=seqK,
                 stream=self.stream.cuda_stream, lse=lse.Handle if lse is not None else None,
                 mask=mask.Handle if mask is not None else None, mask_stride=mask_stride,
                 kv_len=kv_len.Handle if kv_len is not None else None, q_stride=q_stride, k_stride=k_stride,
                 v_stride=v_stride, o_stride=o_stride, scale=scale, workspace=ws, workspace_bytes=ws_bytes,
                 block_table=block_table.Handle if block_table is not None else None,
                 block_table_stride=block_table_stride, block_size=block_size, num_blocks=num_blocks,
                 weights=weights.Handle if weights is not None else None)
        self.launch_count += h.last_launch_count
        self.last_path = h.last_path

    @staticmethod
    def _check_weights(attentionWeights: Optional[GpuBuffer], weightsSize: int) -> None:
        """The optional ``attentionWeights`` buffer receives the fp32 probabilities [batch, heads, seqQ, seqK]
        (``CudaBackend.cs:8340-8349`` checks its size the same way)."""
        if attentionWeights is None:
            return
        if attentionWeights.dtype != torch.float32:
            raise ValueError("attentionWeights must be an fp32 buffer")
        if attentionWeights.Size < weightsSize:
            raise ValueError("Attention tensor buffers are smaller than the requested dimensions.")

    # -- IDirectGpuBackend attention methods ----------------------------------------------------------------
    def ScaledDotProductAttention(self, query: GpuBuffer, key: GpuBuffer, value: GpuBuffer, output: GpuBuffer,
                                  attentionWeights: Optional[GpuBuffer], mask: Optional[GpuBuffer], batch: int,
                                  numHeads: int, seqQ: int, seqK: int, headDim: int, scale: float, isCausal: bool,
                                  softcap: float = 0.0, numKVHeads: int = 0, kvLengths: Optional[GpuBuffer] = None) -> None:
        """softmax(Q K^T * scale [softcap] [mask]) V.  ``mask`` is the engine's float upload of a bool mask
        (0.0 = masked) or a uint8 bool mask: shared [seqQ*seqK] when it holds fewer than batch*heads*seqQ*seqK
        elements, full otherwise (``CudaBackend.cs:8355``).  Causal is bottom-right: key k is visible to query q
        iff k <= q + (seqK - seqQ) (``CudaAttentionKernels.cs:66``).  ``kvLengths`` (extension) is an int32 [batch]
        buffer of valid key counts: the padding mask of a batched decode step without materialising it."""
        self._check_dims(batch, numHeads, seqQ, seqK, headDim)
        kvHeads = numKVHeads if numKVHeads > 0 else numHeads
        if numHeads % kvHeads != 0:
            raise ValueError("numHeads must be an integer multiple of numKVHeads.")
        querySize = batch * numHeads * seqQ * headDim
        keyValueSize = batch * kvHeads * seqK * headDim
        weightsSize = batch * numHeads * seqQ * seqK
        if query.Size < querySize or key.Size < keyValueSize or value.Size < keyValueSize or output.Size < querySize:
            raise ValueError("Attention tensor buffers are smaller than the requested dimensions.")
        self._check_weights(attentionWeights, weightsSize)
        mask_kind, mask_stride = N.MASK_NONE, (0, 0, 0, 0)
        if mask is not None:
            if mask.Size < seqQ * seqK:
                raise ValueError("The attention mask must contain at least seqQ * seqK elements.")
            mask_kind = N.MASK_KEEP_U8 if mask.dtype in (torch.uint8, torch.bool) else N.MASK_KEEP_F32
            full = mask.Size >= weightsSize
            mask_stride = (numHeads * seqQ * seqK, seqQ * seqK, seqK, 1) if full else (0, 0, seqK, 1)
        if query.dtype != key.dtype or query.dtype != value.dtype:
            raise ValueError("query, key and value must share a dtype")
        h = self._handle(qkv_dtype=_DTYPE[query.dtype], out_dtype=_DTYPE[output.dtype], head_dim=headDim,
                         num_q_heads=numHeads, num_kv_heads=kvHeads, causal=bool(isCausal), causal_bottom_right=True,
                         mask_kind=mask_kind, softcap=float(softcap))
        self._run(h, query=query, key=key, value=value, output=output, batch=batch, seqQ=seqQ, seqK=seqK,
                  scale=float(scale), mask=mask, mask_stride=mask_stride, kv_len=kvLengths, weights=attentionWeights)

    def FlashAttention(self, query: GpuBuffer, key: GpuBuffer, value: GpuBuffer, output: GpuBuffer,
                       mask: Optional[GpuBuffer], batch: int, numHeads: int, seqLen: int, headDim: int, scale: float,
                       isCausal: bool) -> None:
        if mask is not None:
            self.ScaledDotProductAttention(query, key, value, output, None, mask, batch, numHeads, seqLen, seqLen,
                                           headDim, scale, isCausal)
            return
        stats = self.AllocateBuffer(batch * numHeads * seqLen)
        self.FlashAttentionV2(query, key, value, output, stats, batch, numHeads, seqLen, seqLen, headDim, scale, isCausal)

    def FlashAttentionV2(self, query: GpuBuffer, key: GpuBuffer, value: GpuBuffer, output: GpuBuffer,
                         softmaxStats: GpuBuffer, batch: int, numHeads: int, seqQ: int, seqK: int, headDim: int,
                         scale: float, isCausal: bool, attentionBias: Optional[GpuBuffer] = None,
                         biasBatchStride: int = 0) -> None:
        """Attention with log-sum-exp statistics and an optional additive bias [B,H,Sq,Sk] (``biasBatchStride`` =
        H*Sq*Sk) or [H,Sq,Sk] (``biasBatchStride`` = 0).  Causal is top-left: key k visible iff k <= q
        (``CudaAttentionKernels.cs:197``)."""
        self._check_dims(batch, numHeads, seqQ, seqK, headDim)
        if softmaxStats.Size < batch * numHeads * seqQ or softmaxStats.dtype != torch.float32:
            raise ValueError("softmaxStats must hold batch*heads*seqQ fp32 values")
        mask_kind, mask_stride = N.MASK_NONE, (0, 0, 0, 0)
        if attentionBias is not None:
            mask_kind = N.MASK_ADD_F32
            mask_stride = (int(biasBatchStride), seqQ * seqK, seqK, 1)
        h = self._handle(qkv_dtype=_DTYPE[query.dtype], out_dtype=_DTYPE[output.dtype], head_dim=headDim,
                         num_q_heads=numHeads, num_kv_heads=numHeads, causal=bool(isCausal), causal_bottom_right=False,
                         causal_offset=0, mask_kind=mask_kind, emit_lse=True)
        self._run(h, query=query, key=key, value=value, output=output, batch=batch, seqQ=seqQ, seqK=seqK,
                  scale=float(scale), lse=softmaxStats, mask=attentionBias, mask_stride=mask_stride)

    def GroupedQueryAttention(self, query: GpuBuffer, key: GpuBuffer, value: GpuBuffer, output: GpuBuffer,
                              attentionWeights: Optional[GpuBuffer], batch: int, numQHeads: int, numKVHeads: int,
                              seqQ: int, seqK: int, headDim: int, scale: float, isCausal: bool) -> None:
        """GQA with top-left causal masking (``CudaAttentionKernels.cs:598``)."""
        self._check_dims(batch, numQHeads, seqQ, seqK, headDim)
        if numKVHeads <= 0 or numQHeads % numKVHeads != 0:
            raise ValueError("numQHeads must be divisible by numKVHeads")
        self._check_weights(attentionWeights, batch * numQHeads * seqQ * seqK)
        h = self._handle(qkv_dtype=_DTYPE[query.dtype], out_dtype=_DTYPE[output.dtype], head_dim=headDim,
                         num_q_heads=numQHeads, num_kv_heads=numKVHeads, causal=bool(isCausal),
                         causal_bottom_right=False, causal_offset=0)
        self._run(h, query=query, key=key, value=value, output=output, batch=batch, seqQ=seqQ, seqK=seqK,
                  scale=float(scale), weights=attentionWeights)

    def FlashDecode(self, q: GpuBuffer, k: GpuBuffer, v: GpuBuffer, heads: int, kvHeads: int, headDim: int,
                    seqLen: int, scale: float, splits: int = 0) -> GpuBuffer:
        """Single-sequence decode over a cache stored [seqLen, kvHeads, headDim] (``CudaBackend.cs:2968-3021``).
        ``splits`` > 0 fixes the number of KV splits; 0 lets the library choose."""
        if heads <= 0 or kvHeads <= 0 or headDim <= 0 or heads % kvHeads != 0:
            raise ValueError("heads must be a positive multiple of kvHeads")
        if seqLen <= 0:
            raise ValueError("seqLen must be positive")
        if q.Size < heads * headDim or k.Size < seqLen * kvHeads * headDim or v.Size < seqLen * kvHeads * headDim:
            raise ValueError("FlashDecode buffers are smaller than the requested dimensions.")
        out = self.AllocateBuffer(heads * headDim)
        chunk = 0
        if splits > 0:
            chunk = max(8, (math.ceil(seqLen / min(splits, seqLen)) + 7) // 8 * 8)
        key = dict(qkv_dtype=_DTYPE[q.dtype], out_dtype=N.F32, head_dim=headDim, num_q_heads=heads,
                   num_kv_heads=kvHeads, causal=False)
        hkey = tuple(sorted(key.items())) + (("chunk", chunk),)
        h = self._handles.get(hkey)
        if h is None:
            h = N.Handle(device=self.device, path=self._path, decode_chunk=chunk or self._decode_chunk, **key)
            self._handles[hkey] = h
        stride = (0, headDim, kvHeads * headDim)  # (B, H, S) element strides of the [S, Hkv, D] cache
        self._run(h, query=q, key=k, value=v, output=out, batch=1, seqQ=1, seqK=seqLen, scale=float(scale),
                  k_stride=stride, v_stride=stride)
        return out

    # -- paged K/V (IDirectGpuBackend.cs:3619-3632) ---------------------------------------------------------
    MaxHeadDim = 256  # GpuKernelGuards.MaxHeadDim

    def _paged_guards(self, op, q, kcache, vcache, blockTable, heads, kvHeads, headDim, blockSize, keyLen, qRows):
        """``GpuKernelGuards.Attention`` / ``Gqa`` / ``PagedAttentionBuffers`` (``GpuKernelGuards.cs:15-35, 83-99``)."""
        if heads <= 0:
            raise ValueError(f"{op}: heads must be > 0 (got {heads}).")
        if headDim <= 0 or headDim > self.MaxHeadDim:
            raise ValueError(f"{op}: headDim must be in [1, {self.MaxHeadDim}] (got {headDim}).")
        if blockSize <= 0:
            raise ValueError(f"{op}: blockSize must be > 0 (got {blockSize}).")
        if qRows <= 0 or keyLen <= 0:
            raise ValueError(f"{op}: sequence/query count must be > 0.")
        if kvHeads <= 0 or kvHeads > heads or heads % kvHeads != 0:
            raise ValueError(f"{op}: kvHeads must satisfy 1 <= kvHeads <= heads and heads % kvHeads == 0 "
                             f"(heads={heads}, kvHeads={kvHeads}).")
        if q.Size < qRows * heads * headDim:
            raise ValueError(f"{op}: q holds fewer than {qRows * heads * headDim} elements.")
        if blockTable.Size < (keyLen + blockSize - 1) // blockSize:
            raise ValueError(f"{op}: blockTable holds fewer than {(keyLen + blockSize - 1) // blockSize} entries.")
        if blockTable.dtype != torch.int32:
            raise ValueError(f"{op}: blockTable must be an int32 buffer.")
        if kcache is None or vcache is None:
            raise ValueError(f"{op}: K/V pools must not be null.")
        if kcache.Size <= 0 or kcache.Size != vcache.Size:
            raise ValueError(f"{op}: kcache/vcache must be equal-sized, non-empty K/V pools.")
        perBlock = blockSize * kvHeads * headDim
        if kcache.Size % perBlock != 0:
            raise ValueError(f"{op}: K/V pool size {kcache.Size} is not a whole number of blocks.")
        return kcache.Size // perBlock

    def _paged(self, op, q, kcache, vcache, blockTable, heads, kvHeads, headDim, blockSize, numQueries, keyLen,
               startPos, scale, batch=1, seqLens=None, tableStride=0):
        numBlocks = self._paged_guards(op, q, kcache, vcache, blockTable, heads, kvHeads, headDim, blockSize, keyLen,
                                       numQueries * batch)
        out = self.AllocateBuffer(batch * numQueries * heads * headDim,
                                  torch.float32 if q.dtype == torch.float32 else q.dtype)
        causal = numQueries > 1
        h = self._handle(qkv_dtype=_DTYPE[q.dtype], out_dtype=_DTYPE[out.dtype], head_dim=headDim, num_q_heads=heads,
                         num_kv_heads=kvHeads, causal=causal, causal_bottom_right=False, causal_offset=int(startPos))
        # q / out are [batch, numQueries, heads, headDim]: (B, H, S) strides of that storage
        qo = (numQueries * heads * headDim, headDim, heads * headDim)
        self._run(h, query=q, key=kcache, value=vcache, output=out, batch=batch, seqQ=numQueries, seqK=keyLen,
                  scale=float(scale), kv_len=seqLens, q_stride=qo, o_stride=qo, block_table=blockTable,
                  block_table_stride=tableStride, block_size=blockSize, num_blocks=numBlocks)
        return out

    def PagedAttentionDecode(self, q: GpuBuffer, kcache: GpuBuffer, vcache: GpuBuffer, blockTable: GpuBuffer,
                             heads: int, headDim: int, blockSize: int, seqLen: int, scale: float) -> GpuBuffer:
        """out[h] = softmax(scale * q[h] . K[., h]) V[., h] over a pool [MaxBlocks, blockSize, heads, headDim] read
        through ``blockTable`` (``CudaBackend.cs:2845-2870``).  Returns a new [heads * headDim] buffer."""
        return self._paged("PagedAttentionDecode", q, kcache, vcache, blockTable, heads, heads, headDim, blockSize, 1,
                           seqLen, 0, scale)

    def PagedAttentionDecodeGqa(self, q: GpuBuffer, kcache: GpuBuffer, vcache: GpuBuffer, blockTable: GpuBuffer,
                                heads: int, kvHeads: int, headDim: int, blockSize: int, seqLen: int,
                                scale: float) -> GpuBuffer:
        """Grouped-query variant: the pool is [MaxBlocks, blockSize, kvHeads, headDim] (``CudaBackend.cs:2905-2933``)."""
        return self._paged("PagedAttentionDecodeGqa", q, kcache, vcache, blockTable, heads, kvHeads, headDim, blockSize,
                           1, seqLen, 0, scale)

    def PagedAttentionPrefill(self, q: GpuBuffer, kcache: GpuBuffer, vcache: GpuBuffer, blockTable: GpuBuffer,
                              heads: int, headDim: int, blockSize: int, numQueries: int, startPos: int,
                              scale: float) -> GpuBuffer:
        """Causal multi-query paged attention: query qi (q is [numQueries, heads, headDim]) attends to keys
        0..startPos+qi (``CudaBackend.cs:2875-2903``)."""
        if startPos < 0:
            raise ValueError("startPos must be >= 0")
        return self._paged("PagedAttentionPrefill", q, kcache, vcache, blockTable, heads, heads, headDim, blockSize,
                           numQueries, startPos + numQueries, startPos, scale)

    def PagedAttentionPrefillGqa(self, q: GpuBuffer, kcache: GpuBuffer, vcache: GpuBuffer, blockTable: GpuBuffer,
                                 heads: int, kvHeads: int, headDim: int, blockSize: int, numQueries: int, startPos: int,
                                 scale: float) -> GpuBuffer:
        """Grouped-query variant of ``PagedAttentionPrefill`` (``CudaBackend.cs:2935-2966``)."""
        if startPos < 0:
            raise ValueError("startPos must be >= 0")
        return self._paged("PagedAttentionPrefillGqa", q, kcache, vcache, blockTable, heads, kvHeads, headDim,
                           blockSize, numQueries, startPos + numQueries, startPos, scale)

    def PagedAttentionDecodeBatched(self, q: GpuBuffer, kcache: GpuBuffer, vcache: GpuBuffer, blockTables: GpuBuffer,
                                    seqLens: GpuBuffer, batch: int, heads: int, kvHeads: int, headDim: int,
                                    blockSize: int, maxSeqLen: int, blocksPerSeq: int, scale: float) -> GpuBuffer:
        """Extension with no reference counterpart (its paged calls take one sequence): one launch decodes ``batch``
        sequences that share a pool.  ``q`` is [batch, heads, headDim], ``blockTables`` int32 [batch, blocksPerSeq],
        ``seqLens`` int32 [batch] (each <= maxSeqLen <= blocksPerSeq * blockSize)."""
        if batch <= 0 or blocksPerSeq * blockSize < maxSeqLen:
            raise ValueError("PagedAttentionDecodeBatched: batch must be > 0 and blocksPerSeq * blockSize >= maxSeqLen")
        if blockTables.Size < batch * blocksPerSeq or seqLens.Size < batch or seqLens.dtype != torch.int32:
            raise ValueError("PagedAttentionDecodeBatched: blockTables / seqLens are too small or not int32")
        return self._paged("PagedAttentionDecodeBatched", q, kcache, vcache, blockTables, heads, kvHeads, headDim,
                           blockSize, 1, maxSeqLen, 0, scale, batch=batch, seqLens=seqLens, tableStride=blocksPerSeq)

    def FlashAttentionBackward(self, gradOutput: GpuBuffer, query: GpuBuffer, key: GpuBuffer, value: GpuBuffer,
                               output: GpuBuffer, softmaxStats: GpuBuffer, gradQuery: GpuBuffer, gradKey: GpuBuffer,
                               gradValue: GpuBuffer, batch: int, numHeads: int, seqQ: int, seqK: int, headDim: int,
                               scale: float, isCausal: bool, attentionBias: Optional[GpuBuffer] = None,
                               biasBatchStride: int = 0) -> None:
        """dQ, dK, dV from dO, Q, K, V, O and the statistics FlashAttentionV2 wrote (``CudaBackend.cs:8580-8604``);
        top-left causal, optional additive bias with the forward's batch stride; deterministic.  The gradient buffers
        are fp32."""
        self._check_dims(batch, numHeads, seqQ, seqK, headDim)
        qsz, ksz = batch * numHeads * seqQ * headDim, batch * numHeads * seqK * headDim
        if (gradOutput.Size < qsz or query.Size < qsz or output.Size < qsz or gradQuery.Size < qsz or key.Size < ksz or
                value.Size < ksz or gradKey.Size < ksz or gradValue.Size < ksz or softmaxStats.Size < batch * numHeads * seqQ):
            raise ValueError("Attention tensor buffers are smaller than the requested dimensions.")
        if any(g.dtype != torch.float32 for g in (gradQuery, gradKey, gradValue, softmaxStats)):
            raise ValueError("gradients and softmaxStats are fp32 buffers")
        if gradOutput.dtype != output.dtype:
            raise ValueError("gradOutput must have the dtype of output")
        h = self._handle(qkv_dtype=_DTYPE[query.dtype], out_dtype=_DTYPE[output.dtype], head_dim=headDim,
                         num_q_heads=numHeads, num_kv_heads=numHeads, causal=bool(isCausal), causal_bottom_right=False,
                         causal_offset=0, emit_lse=True,
                         mask_kind=N.MASK_ADD_F32 if attentionBias is not None else N.MASK_NONE)
        nbytes = h.backward_workspace_bytes(batch, seqQ)
        ws, ws_bytes = self._workspace(nbytes)
        h.backward(q=query.Handle, k=key.Handle, v=value.Handle, out=output.Handle, lse=softmaxStats.Handle,
                   dout=gradOutput.Handle, dq=gradQuery.Handle, dk=gradKey.Handle, dv=gradValue.Handle, batch=batch,
                   seq_q=seqQ, seq_kv=seqK, stream=self.stream.cuda_stream, workspace=ws, workspace_bytes=ws_bytes,
                   mask=attentionBias.Handle if attentionBias is not None else None,
                   mask_stride=(biasBatchStride, seqQ * seqK, seqK, 1) if attentionBias is not None else (0, 0, 0, 0),
                   scale=float(scale))
        self.launch_count += h.last_launch_count

    # -- the in-library caller of the attention path -------------------------------------------------------------
    def MultiHeadAttentionForward(self, input: GpuBuffer, qWeight: GpuBuffer, kWeight: GpuBuffer, vWeight: GpuBuffer,
                                  outWeight: GpuBuffer, output: GpuBuffer, batch: int, seq: int, dModel: int,
                                  numHeads: int, mask: Optional[GpuBuffer] = None,
                                  maskShape: Optional[Tuple[int, int, int, int]] = None, exact: bool = False) -> None:
        """``IEngine.MultiHeadAttentionForward`` (``Engines/IEngine.cs:4201-4208``; checks as in
        ``CpuEngine.MultiHeadAttention.cs:76-103``) on resident buffers: ``input`` [batch, seq, dModel], four
        [dModel, dModel] weights applied as ``x @ W``, optional boolean keep-mask of shape ``maskShape`` broadcastable
        to [batch, numHeads, seq, seq]; ``output`` [batch, seq, dModel].  With head sizes 64 / 128 (dModel a multiple
        of 128) fp32 buffers are rounded to bf16 on the way in and the arithmetic runs on the tensor cores with fp32
        accumulation; any other shape, or ``exact=True`` with all-fp32 buffers, runs the fp32 route, which meets the
        1e-4 bound of the reference's own tests of the fused call."""
        for name, buf in (("input", input), ("qWeight", qWeight), ("kWeight", kWeight), ("vWeight", vWeight),
                          ("outWeight", outWeight), ("output", output)):
            if buf is None:
                raise ValueError(f"{name} must not be null")          # ArgumentNullException
        if numHeads <= 0:
            raise ValueError("numHeads must be positive.")            # ArgumentOutOfRangeException
        if batch <= 0 or seq <= 0 or dModel <= 0:
            raise ValueError("MultiHeadAttentionForward expects a non-empty [B, seq, dModel] input.")
        if dModel % numHeads != 0:
            raise ValueError(f"dModel ({dModel}) must be divisible by numHeads ({numHeads}).")
        for name, w in (("qWeight", qWeight), ("kWeight", kWeight), ("vWeight", vWeight), ("outWeight", outWeight)):
            if w.Size != dModel * dModel:
                raise ValueError(f"{name} must be [{dModel}, {dModel}].")
        if input.Size < batch * seq * dModel or output.Size < batch * seq * dModel:
            raise ValueError("input / output buffers are smaller than [batch, seq, dModel].")
        wdt = {w.dtype for w in (qWeight, kWeight, vWeight, outWeight)}
        if len(wdt) != 1:
            raise ValueError("the four weights must share one dtype")
        sixteen = [b.dtype for b in (input, qWeight, output) if b.dtype != torch.float32]
        if len(set(sixteen)) > 1:
            raise ValueError("16-bit buffers must share one dtype")
        head = dModel // numHeads
        tensor_shape = head in (64, 128) and dModel % 128 == 0
        compute = sixteen[0] if sixteen else (torch.bfloat16 if tensor_shape and not exact else torch.float32)
        ms = (0, 0, 0, 0)
        if mask is not None:
            if maskShape is None or len(maskShape) != 4:
                raise ValueError("maskShape must give the 4 mask dimensions")
            full = (batch, numHeads, seq, seq)
            dense = (maskShape[1] * maskShape[2] * maskShape[3], maskShape[2] * maskShape[3], maskShape[3], 1)
            for ax in range(4):
                if maskShape[ax] not in (1, full[ax]):
                    raise ValueError("mask is not broadcastable to [batch, numHeads, seq, seq]")
            ms = tuple(0 if (maskShape[ax] == 1 and full[ax] != 1) else dense[ax] for ax in range(4))
        h = self._handle(qkv_dtype=_DTYPE[compute], out_dtype=_DTYPE[compute], head_dim=head,
                         num_q_heads=numHeads, num_kv_heads=numHeads,
                         mask_kind=N.MASK_KEEP_U8 if mask is not None else N.MASK_NONE)
        nbytes = h.mha_workspace_bytes(batch, seq, _DTYPE[input.dtype], _DTYPE[qWeight.dtype])
        ws, ws_bytes = self._workspace(nbytes + 1024)
        base = (ws + 1023) // 1024 * 1024
        h.mha_forward(input=input.Handle, q_weight=qWeight.Handle, k_weight=kWeight.Handle, v_weight=vWeight.Handle,
                      out_weight=outWeight.Handle, out=output.Handle, batch=batch, seq=seq,
                      input_dtype=_DTYPE[input.dtype], weight_dtype=_DTYPE[qWeight.dtype],
                      out_dtype=_DTYPE[output.dtype], workspace=base, workspace_bytes=ws_bytes - (base - ws),
                      stream=self.stream.cuda_stream, mask=mask.Handle if mask is not None else None, mask_stride=ms)
        self.launch_count += h.last_launch_count

    # -- the decode step in front of attention ----------------------------------------------------------------
    def QkvProjectionRoPECacheD64(self, input: GpuBuffer, packedWeights: GpuBuffer, bias: GpuBuffer, cosine: GpuBuffer,
                                  sine: GpuBuffer, query: GpuBuffer, keyCache: GpuBuffer, valueCache: GpuBuffer,
                                  heads: int, cacheCapacity: int, position: int) -> None:
        """One resident fp32 token through the packed Q/K/V weights (output-major, Q rows then K then V), + packed
        bias, interleaved RoPE on Q and K, Q written to ``query`` and the K / V rows to row ``position`` of the dense
        caches [cacheCapacity, heads, 64] (``CudaBackend.cs:8389-8439``).  One kernel, no scratch buffers; the weights
        may be bf16 and the caches 16-bit (``GpuBuffer.dtype``), which is what the decode kernel then reads."""
        for name, buf in (("input", input), ("packedWeights", packedWeights), ("bias", bias), ("cosine", cosine),
                          ("sine", sine), ("query", query), ("keyCache", keyCache), ("valueCache", valueCache)):
            if buf is None:
                raise ValueError(f"{name} must not be null")          # ArgumentNullException
        if heads <= 0:
            raise ValueError("heads must be > 0")
        if cacheCapacity <= 0:
            raise ValueError("cacheCapacity must be > 0")
        if position < 0 or position >= cacheCapacity:
            raise ValueError("position must be in [0, cacheCapacity)")
        dimension = 64
        model = heads * dimension
        projection = 3 * model
        if (input.Size < model or packedWeights.Size < projection * model or bias.Size < projection or
                cosine.Size < cacheCapacity * (dimension // 2) or sine.Size < cacheCapacity * (dimension // 2) or
                query.Size < model or keyCache.Size < cacheCapacity * model or valueCache.Size < cacheCapacity * model):
            raise ValueError("QKV/RoPE/cache buffers are smaller than the requested canonical extents.")
        N.qkv_rope_cache(input=input.Handle, weights=packedWeights.Handle, bias=bias.Handle, cosine=cosine.Handle,
                         sine=sine.Handle, query=query.Handle, key_cache=keyCache.Handle, value_cache=valueCache.Handle,
                         tokens=1, heads=heads, kv_heads=heads, head_dim=dimension, position=position,
                         weight_dtype=_DTYPE[packedWeights.dtype], query_dtype=_DTYPE[query.dtype],
                         cache_dtype=_DTYPE[keyCache.dtype], cache_capacity=cacheCapacity, max_position=cacheCapacity,
                         stream=self.stream.cuda_stream)
        self.launch_count += 1

    def RopeInterleaved(self, input: GpuBuffer, cos: GpuBuffer, sin: GpuBuffer, output: GpuBuffer, rows: int,
                        headDim: int, seqLen: int, startPosition: int) -> None:
        """Interleaved RoPE over ``rows`` rows of ``headDim`` fp32 values; row r sits at position
        startPosition + r % seqLen (``CudaBackend.cs:8441-8470``, kernel ``CudaAttentionKernels.cs:1023-1050``)."""
        if rows <= 0 or headDim <= 0 or seqLen <= 0:
            raise ValueError("rows, headDim and seqLen must be positive")
        if input.Size < rows * headDim or output.Size < rows * headDim:
            raise ValueError("RoPE buffers are smaller than rows * headDim")
        if cos.Size < (startPosition + seqLen) * (headDim // 2) or sin.Size < (startPosition + seqLen) * (headDim // 2):
            raise ValueError("cos/sin caches do not reach startPosition + seqLen")
        N.rope_interleaved(input.Handle, cos.Handle, sin.Handle, output.Handle, rows, headDim, seqLen, startPosition,
                           self.stream.cuda_stream)
        self.launch_count += 1

    def Dispose(self) -> None:
        for h in self._handles.values():
            h.close()
        self._handles.clear()
