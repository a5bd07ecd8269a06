// The sm_100a route of the reference's CUDA backend: bodies for the attention methods of IDirectGpuBackend that call
// libaidotnet_sdpa_sm100 through AidnSdpaNative instead of launching the NVRTC kernels.  Drop next to CudaBackend.cs
// (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/); CudaBackend is already a partial class.  Each public method of
// CudaBackend named below gains ONE line at its top, after `using var _ = PushContext();`:
//
//     if (TrySm100<Method>(...same arguments...)) return;          // or `return output;` for the buffer-returning ones
//
// ScaledDotProductAttention  CudaBackend.cs:8322     FlashAttentionV2        :8540     GroupedQueryAttention :8721
// FlashAttentionBackward     :8580                   FlashDecode             :2968     PagedAttentionDecode{,Gqa} :2845, :2905
// PagedAttentionPrefill{,Gqa} :2875, :2935           QkvProjectionRoPECacheD64 :8389   RopeInterleaved       :8441
//
// Source only: no .NET toolchain exists where this repository is built, so this file has not been compiled.  The same
// calls, with the same argument mapping, are made by the Python mirror (aidotnet/tensors_b200/backend.py) and the C++
// mirror (csrc/host/direct_gpu_backend.cpp), which are compiled and tested against the library on a B200.
using System;
using System.Collections.Generic;

namespace AiDotNet.Tensors.Engines.DirectGpu.CUDA
{
    public sealed partial class CudaBackend
    {
        // One native handle per distinct descriptor; created on first use (outside stream capture: create allocates a
        // 16-byte status word), destroyed with the backend.  Launches of a handle are serialised by GpuDispatchLock and
        // go to the backend's single stream, which is what the library requires of one handle.
        private readonly Dictionary<Sm100Key, IntPtr> _sm100Handles = new();
        private IGpuBuffer? _sm100Workspace;
        private bool? _sm100Usable;
        private int _sm100Device;      // the constructor's deviceIndex (CudaBackend.cs:315): one added line there, `_sm100Device = deviceIndex;`

        private readonly record struct Sm100Key(int Dtype, int OutDtype, int HeadDim, int Heads, int KvHeads, bool Causal,
            bool BottomRight, long CausalOffset, int MaskKind, bool EmitLse, float Softcap, int DecodeChunk);

        /// <summary>cc 10.x, library present, not switched off (AIDOTNET_SDPA_SM100=0).</summary>
        private bool Sm100Usable()
        {
            if (_sm100Usable is bool known) return known;
            bool ok = false;
            try { ok = AidnSdpaNative.Enabled && AidnSdpaNative.aidn_sdpa_device_supported(_sm100Device) == 1; }
            catch (DllNotFoundException) { }
            catch (EntryPointNotFoundException) { }
            _sm100Usable = ok;
            return ok;
        }

        private IntPtr Sm100Handle(in Sm100Key key)
        {
            if (_sm100Handles.TryGetValue(key, out IntPtr h)) return h;
            if (IsStreamCapturing())
                throw new InvalidOperationException("sm_100a attention handle must be created before stream capture (pre-warm the shape once).");
            var desc = new AidnSdpaDesc
            {
                device = _sm100Device, qkv_dtype = key.Dtype, out_dtype = key.OutDtype, head_dim = key.HeadDim,
                num_q_heads = key.Heads, num_kv_heads = key.KvHeads, causal = key.Causal ? 1 : 0,
                causal_bottom_right = key.BottomRight ? 1 : 0, causal_offset = key.CausalOffset, mask_kind = key.MaskKind,
                emit_lse = key.EmitLse ? 1 : 0, softcap = key.Softcap, path = (int)AidnPath.Auto,
                decode_chunk = key.DecodeChunk,
            };
            AidnSdpaNative.Check(AidnSdpaNative.aidn_sdpa_create(ref desc, out h));
            _sm100Handles[key] = h;
            return h;
        }

        /// <summary>Pooled scratch for split-KV decode and the backward; grown outside capture only.</summary>
        private IGpuBuffer Sm100Workspace(long bytes)
        {
            long have = _sm100Workspace is null ? 0 : (long)_sm100Workspace.Size * sizeof(float);
            if (have >= bytes) return _sm100Workspace!;
            if (IsStreamCapturing())
                throw new InvalidOperationException("sm_100a attention workspace must be sized before stream capture.");
            _sm100Workspace?.Dispose();
            _sm100Workspace = AllocateBuffer(checked((int)((bytes + 3) / 4)));
            return _sm100Workspace;
        }

        private void Sm100Dispose()      // call from Dispose()
        {
            foreach (IntPtr h in _sm100Handles.Values) AidnSdpaNative.aidn_sdpa_destroy(h);
            _sm100Handles.Clear();
            _sm100Workspace?.Dispose();
        }

        private static unsafe void SetMaskStrides(ref AidnSdpaArgs a, long batchStride, long headStride, long rowStride)
        {
            a.mask_stride[0] = batchStride; a.mask_stride[1] = headStride; a.mask_stride[2] = rowStride; a.mask_stride[3] = 1;
        }

        private void Sm100Launch(IntPtr handle, ref AidnSdpaArgs args)
        {
            lock (GpuDispatchLock)                                   // CudaBackend.cs:66, 5392
                AidnSdpaNative.Check(AidnSdpaNative.aidn_sdpa_launch(handle, ref args, _stream));
            GpuLaunchProbe.OnLaunch();                               // CudaBackend.cs:5407
        }

        // ---- IDirectGpuBackend.cs:1421-1424 ---------------------------------------------------------------------------
        private unsafe bool TrySm100ScaledDotProductAttention(IGpuBuffer query, IGpuBuffer key, IGpuBuffer value,
            IGpuBuffer output, IGpuBuffer? attentionWeights, IGpuBuffer? mask,
            int batch, int numHeads, int seqQ, int seqK, int headDim, float scale, bool isCausal, float softcap, int kvHeads)
        {
            if (!Sm100Usable() || headDim > 256 || headDim % 8 != 0) return false;
            long weightsSize = (long)batch * numHeads * seqQ * seqK;       // long: the int product overflows from S = 8192 on
            // the [B,H,Sq,Sk] probabilities on request (CudaBackend.cs:8343-8356): args.weights selects the fp32 kernel
            if (attentionWeights is not null && attentionWeights.Size < weightsSize)
                throw new ArgumentException("The attention-weights buffer is too small.", nameof(attentionWeights));
            if (mask is not null && mask.Size < (long)seqQ * seqK)
                throw new ArgumentException("The attention mask must contain at least seqQ * seqK elements.", nameof(mask));
            var k = new Sm100Key((int)AidnDtype.F32, (int)AidnDtype.F32, headDim, numHeads, kvHeads, isCausal, true, 0,
                mask is null ? (int)AidnMaskKind.None : (int)AidnMaskKind.KeepF32, false, softcap, 0);
            var args = new AidnSdpaArgs
            {
                q = query.Handle, k = key.Handle, v = value.Handle, @out = output.Handle,
                mask = mask?.Handle ?? IntPtr.Zero, batch = batch, seq_q = seqQ, seq_kv = seqK, scale = scale,
                weights = attentionWeights?.Handle ?? IntPtr.Zero,
            };
            // the maskMode rule of CudaBackend.cs:8355: a full [B,H,Sq,Sk] mask, else one [Sq,Sk] plane for all
            if (mask is not null)
            {
                if (mask.Size >= weightsSize) SetMaskStrides(ref args, (long)numHeads * seqQ * seqK, (long)seqQ * seqK, seqK);
                else SetMaskStrides(ref args, 0, 0, seqK);
            }
            if (seqQ == 1) Sm100AttachWorkspace(Sm100Handle(k), ref args);
            Sm100Launch(Sm100Handle(k), ref args);
            return true;
        }

        private void Sm100AttachWorkspace(IntPtr handle, ref AidnSdpaArgs args)
        {
            long need = AidnSdpaNative.aidn_sdpa_workspace_bytes(handle, args.batch, args.seq_q, args.seq_kv);
            if (need <= 0) return;
            IGpuBuffer ws = Sm100Workspace(need);
            args.workspace = ws.Handle;
            args.workspace_bytes = (long)ws.Size * sizeof(float);
        }

        // ---- IDirectGpuBackend.cs:1468-1471 ---------------------------------------------------------------------------
        private unsafe bool TrySm100FlashAttentionV2(IGpuBuffer query, IGpuBuffer key, IGpuBuffer value,
            IGpuBuffer output, IGpuBuffer softmaxStats, int batch, int numHeads, int seqQ, int seqK, int headDim, float scale,
            bool isCausal, IGpuBuffer? attentionBias, int biasBatchStride)
        {
            if (!Sm100Usable() || headDim > 256 || headDim % 8 != 0) return false;
            var k = new Sm100Key((int)AidnDtype.F32, (int)AidnDtype.F32, headDim, numHeads, numHeads, isCausal, false, 0,
                attentionBias is null ? (int)AidnMaskKind.None : (int)AidnMaskKind.AddF32, true, 0f, 0);
            var args = new AidnSdpaArgs
            {
                q = query.Handle, k = key.Handle, v = value.Handle, @out = output.Handle, lse = softmaxStats.Handle,
                mask = attentionBias?.Handle ?? IntPtr.Zero, batch = batch, seq_q = seqQ, seq_kv = seqK, scale = scale,
            };
            if (attentionBias is not null) SetMaskStrides(ref args, biasBatchStride, (long)seqQ * seqK, seqK);   // top-left causal: FlashAttention semantics
            Sm100Launch(Sm100Handle(k), ref args);
            return true;
        }

        // ---- IDirectGpuBackend.cs:1501-1503 ---------------------------------------------------------------------------
        private bool TrySm100GroupedQueryAttention(IGpuBuffer query, IGpuBuffer key, IGpuBuffer value, IGpuBuffer output,
            IGpuBuffer? attentionWeights, int batch, int numQHeads, int numKVHeads, int seqQ, int seqK, int headDim, float scale,
            bool isCausal)
        {
            if (!Sm100Usable() || headDim > 256 || headDim % 8 != 0) return false;
            if (attentionWeights is not null && attentionWeights.Size < (long)batch * numQHeads * seqQ * seqK)
                throw new ArgumentException("The attention-weights buffer is too small.", nameof(attentionWeights));
            var k = new Sm100Key((int)AidnDtype.F32, (int)AidnDtype.F32, headDim, numQHeads, numKVHeads, isCausal, false, 0,
                (int)AidnMaskKind.None, false, 0f, 0);
            var args = new AidnSdpaArgs
            {
                q = query.Handle, k = key.Handle, v = value.Handle, @out = output.Handle,
                batch = batch, seq_q = seqQ, seq_kv = seqK, scale = scale,
                weights = attentionWeights?.Handle ?? IntPtr.Zero,               // CudaBackend.cs:8731-8732
            };
            if (seqQ == 1) Sm100AttachWorkspace(Sm100Handle(k), ref args);
            Sm100Launch(Sm100Handle(k), ref args);
            return true;
        }

        // ---- IDirectGpuBackend.cs:1479-1483 ---------------------------------------------------------------------------
        private unsafe bool TrySm100FlashAttentionBackward(IGpuBuffer gradOutput, IGpuBuffer query, IGpuBuffer key, IGpuBuffer value,
            IGpuBuffer output, IGpuBuffer softmaxStats, IGpuBuffer gradQuery, IGpuBuffer gradKey, IGpuBuffer gradValue,
            int batch, int numHeads, int seqQ, int seqK, int headDim, float scale, bool isCausal,
            IGpuBuffer? attentionBias, int biasBatchStride)
        {
            if (!Sm100Usable() || headDim > 256 || headDim % 8 != 0) return false;
            var k = new Sm100Key((int)AidnDtype.F32, (int)AidnDtype.F32, headDim, numHeads, numHeads, isCausal, false, 0,
                attentionBias is null ? (int)AidnMaskKind.None : (int)AidnMaskKind.AddF32, true, 0f, 0);
            IntPtr handle = Sm100Handle(k);
            long need = AidnSdpaNative.aidn_sdpa_backward_workspace_bytes(handle, batch, seqQ);
            IGpuBuffer ws = Sm100Workspace(need);
            var bwd = new AidnSdpaBwdArgs
            {
                dout = gradOutput.Handle, dq = gradQuery.Handle, dk = gradKey.Handle, dv = gradValue.Handle,
            };
            bwd.fwd.q = query.Handle; bwd.fwd.k = key.Handle; bwd.fwd.v = value.Handle;
            bwd.fwd.@out = output.Handle; bwd.fwd.lse = softmaxStats.Handle;
            bwd.fwd.mask = attentionBias?.Handle ?? IntPtr.Zero;
            bwd.fwd.batch = batch; bwd.fwd.seq_q = seqQ; bwd.fwd.seq_kv = seqK; bwd.fwd.scale = scale;
            bwd.fwd.workspace = ws.Handle; bwd.fwd.workspace_bytes = (long)ws.Size * sizeof(float);
            if (attentionBias is not null) SetMaskStrides(ref bwd.fwd, biasBatchStride, (long)seqQ * seqK, seqK);
            lock (GpuDispatchLock)
                AidnSdpaNative.Check(AidnSdpaNative.aidn_sdpa_backward(handle, ref bwd, _stream));
            GpuLaunchProbe.OnLaunch();
            return true;       // deterministic by construction: the UseDeterministic switch of :8622-8640 needs no second kernel
        }

        // ---- CudaBackend.cs:2968-3021: single sequence, cache laid out [seqLen, kvHeads, headDim] -----------------------
        private unsafe bool TrySm100FlashDecode(IGpuBuffer q, IGpuBuffer k, IGpuBuffer v, IGpuBuffer output,
            int heads, int kvHeads, int headDim, int seqLen, float scale, int splits)
        {
            if (!Sm100Usable() || (headDim != 64 && headDim != 128)) return false;
            int chunk = splits > 0 ? ((seqLen + splits - 1) / splits + 7) / 8 * 8 : 0;
            var key = new Sm100Key((int)AidnDtype.F32, (int)AidnDtype.F32, headDim, heads, kvHeads, false, true, 0,
                (int)AidnMaskKind.None, false, 0f, chunk);
            var args = new AidnSdpaArgs { q = q.Handle, k = k.Handle, v = v.Handle, @out = output.Handle, batch = 1, seq_q = 1, seq_kv = seqLen, scale = scale };
            args.k_stride[0] = 0; args.k_stride[1] = headDim; args.k_stride[2] = (long)kvHeads * headDim;
            args.v_stride[0] = 0; args.v_stride[1] = headDim; args.v_stride[2] = (long)kvHeads * headDim;
            Sm100AttachWorkspace(Sm100Handle(key), ref args);       // replaces the three per-call scratch buffers of :2994-2996
            Sm100Launch(Sm100Handle(key), ref args);
            return true;
        }

        // ---- IDirectGpuBackend.cs:3619-3632: paged decode / prefill (kvHeads == heads for the non-Gqa overloads) -------
        private unsafe bool TrySm100PagedAttention(IGpuBuffer q, IGpuBuffer kcache, IGpuBuffer vcache, IGpuBuffer blockTable,
            IGpuBuffer output, int heads, int kvHeads, int headDim, int blockSize, int numQueries, int startPos, float scale)
        {
            if (!Sm100Usable() || headDim > 256 || headDim % 8 != 0) return false;
            bool prefill = numQueries > 1;
            var key = new Sm100Key((int)AidnDtype.F32, (int)AidnDtype.F32, headDim, heads, kvHeads, prefill, false, startPos,
                (int)AidnMaskKind.None, false, 0f, 0);
            long rowStride = (long)heads * headDim;                   // the reference's [numQueries, heads, D] query / output
            var args = new AidnSdpaArgs
            {
                q = q.Handle, k = kcache.Handle, v = vcache.Handle, @out = output.Handle,
                batch = 1, seq_q = numQueries, seq_kv = startPos + numQueries, scale = scale,
            };
            args.q_stride[0] = numQueries * rowStride; args.q_stride[1] = headDim; args.q_stride[2] = rowStride;
            args.o_stride[0] = numQueries * rowStride; args.o_stride[1] = headDim; args.o_stride[2] = rowStride;
            var paged = new AidnPagedKv
            {
                block_table = blockTable.Handle, block_table_stride = 0, block_size = blockSize,
                num_blocks = (int)(kcache.Size / ((long)blockSize * kvHeads * headDim)),
            };
            IntPtr handle = Sm100Handle(key);
            if (!prefill) Sm100AttachWorkspace(handle, ref args);
            lock (GpuDispatchLock)
                AidnSdpaNative.Check(AidnSdpaNative.aidn_sdpa_launch_paged(handle, ref args, ref paged, _stream));
            GpuLaunchProbe.OnLaunch();
            return true;
        }

        // ---- CudaBackend.cs:8389-8439 ---------------------------------------------------------------------------------
        private bool TrySm100QkvProjectionRoPECache(IGpuBuffer input, IGpuBuffer packedWeights, IGpuBuffer? bias,
            IGpuBuffer cosine, IGpuBuffer sine, IGpuBuffer query, IGpuBuffer keyCache, IGpuBuffer valueCache,
            int heads, int headDim, int position, int cacheCapacity)
        {
            if (!Sm100Usable()) return false;
            var a = new AidnQkvRopeArgs
            {
                input = input.Handle, weights = packedWeights.Handle, bias = bias?.Handle ?? IntPtr.Zero,
                cosine = cosine.Handle, sine = sine.Handle, query = query.Handle, key_cache = keyCache.Handle, value_cache = valueCache.Handle,
                tokens = 1, heads = heads, kv_heads = heads, head_dim = headDim, position = position,
                weight_dtype = (int)AidnDtype.F32, query_dtype = (int)AidnDtype.F32, cache_dtype = (int)AidnDtype.F32,
                cache_capacity = cacheCapacity, max_position = cacheCapacity,
            };
            lock (GpuDispatchLock)
                AidnSdpaNative.Check(AidnSdpaNative.aidn_qkv_rope_cache(ref a, _stream));
            GpuLaunchProbe.OnLaunch();
            return true;
        }

        // ---- CudaBackend.cs:8441-8470 ---------------------------------------------------------------------------------
        private bool TrySm100RopeInterleaved(IGpuBuffer input, IGpuBuffer cosine, IGpuBuffer sine, IGpuBuffer output,
            long rows, int headDim, int seqLen, int startPosition)
        {
            if (!Sm100Usable()) return false;
            lock (GpuDispatchLock)
                AidnSdpaNative.Check(AidnSdpaNative.aidn_rope_interleaved(input.Handle, cosine.Handle, sine.Handle, output.Handle,
                    rows, headDim, seqLen, startPosition, _stream));
            GpuLaunchProbe.OnLaunch();
            return true;
        }

        // ---- a resident 16-bit tensor (the engine guard edit admits Tensor<BFloat16> / Tensor<Half>) --------------------
        /// <summary>The same attention on bf16 / fp16 buffers (IGpuBuffer.Size counts 16-bit elements then): the tcgen05
        /// kernel.  fp32 tensors can be staged with aidn_cast_f32_to_bf16, bit-exact with BFloat16.FromFloat.</summary>
        internal unsafe void ScaledDotProductAttention16(IGpuBuffer query, IGpuBuffer key, IGpuBuffer value, IGpuBuffer output,
            AidnDtype dtype, bool outputIsFp32, int batch, int numHeads, int numKVHeads, int seqQ, int seqK, int headDim, float scale,
            bool isCausal, float softcap)
        {
            using var _ = PushContext();
            if (!Sm100Usable()) throw new InvalidOperationException("16-bit attention needs the sm_100a library; there is no CPU fallback on this path.");
            var k = new Sm100Key((int)dtype, outputIsFp32 ? (int)AidnDtype.F32 : (int)dtype, headDim, numHeads, numKVHeads, isCausal, true, 0,
                (int)AidnMaskKind.None, false, softcap, 0);
            var args = new AidnSdpaArgs { q = query.Handle, k = key.Handle, v = value.Handle, @out = output.Handle, batch = batch, seq_q = seqQ, seq_kv = seqK, scale = scale };
            if (seqQ == 1) Sm100AttachWorkspace(Sm100Handle(k), ref args);
            Sm100Launch(Sm100Handle(k), ref args);
        }
    }
}
