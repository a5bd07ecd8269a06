// P/Invoke binding of libaidotnet_sdpa_sm100 (C ABI: include/aidn_sdpa.h) for the reference's CUDA backend.
// Drop into src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/ next to CuBlasNative.cs.  Source only: it has not been
// compiled in the environment this repository was built in (no .NET toolchain there); field order, sizes and
// entry points mirror the header one to one, and the same layout is checked from Python (ctypes) in the tests.
using System;
using System.Runtime.InteropServices;

namespace AiDotNet.Tensors.Engines.DirectGpu.CUDA
{
    internal enum AidnStatus { Ok = 0, Inval = 1, Unsupported = 2, Cuda = 3, Workspace = 4, Timeout = 5, Nccl = 6 }
    internal enum AidnDtype { F32 = 0, F16 = 1, BF16 = 2 }
    internal enum AidnMaskKind { None = 0, KeepU8 = 1, KeepF32 = 2, AddF32 = 3 }
    internal enum AidnPath { Auto = 0, Generic = 1, Decode = 2, PrefillSm100 = 3 }

    [StructLayout(LayoutKind.Sequential)]
    internal struct AidnSdpaDesc
    {
        public int device, qkv_dtype, out_dtype, head_dim, num_q_heads, num_kv_heads, causal, causal_bottom_right;
        public long causal_offset;
        public int mask_kind, emit_lse;
        public float softcap;
        public int path, head_begin, head_count, decode_chunk, max_batch;
        public long max_seq_q, max_seq_kv;
        public IntPtr nccl_comm;
    }

    [StructLayout(LayoutKind.Sequential)]
    internal unsafe struct AidnSdpaArgs
    {
        public IntPtr q, k, v, @out, lse, mask;
        public fixed long mask_stride[4];
        public IntPtr kv_len;
        public long batch, seq_q, seq_kv;
        public fixed long q_stride[3];
        public fixed long k_stride[3];
        public fixed long v_stride[3];
        public fixed long o_stride[3];
        public float scale;
        public IntPtr workspace;
        public long workspace_bytes;
        public int gather_output;
        public IntPtr weights;     // [B, Hq, Sq, Sk] fp32 probabilities on request, or zero
        public int peer_count;     // fused gather: other devices' output tensors, mapped with aidn_peer_open
        public IntPtr peer_out0, peer_out1, peer_out2, peer_out3, peer_out4, peer_out5, peer_out6, peer_out7;
    }

    /// <summary>Paged K/V: the block pool of DevicePagedKVCache ([MaxBlocks, BlockSize, KvHeads, HeadDim]) and the
    /// int32 block table uploaded with AllocateIntBuffer.</summary>
    [StructLayout(LayoutKind.Sequential)]
    internal struct AidnPagedKv
    {
        public IntPtr block_table;
        public long block_table_stride;
        public int block_size;
        public int num_blocks;
    }

    /// <summary>Arguments of aidn_sdpa_backward: the forward block (out = O, lse = statistics) plus dO and the gradients.</summary>
    [StructLayout(LayoutKind.Sequential)]
    internal unsafe struct AidnSdpaBwdArgs
    {
        public AidnSdpaArgs fwd;
        public IntPtr paged;      // AidnPagedKv*, or zero
        public IntPtr dout;
        public fixed long do_stride[3];
        public IntPtr dq, dk, dv;
    }

    /// <summary>Arguments of aidn_mha_forward (IEngine.MultiHeadAttentionForward on resident buffers).</summary>
    [StructLayout(LayoutKind.Sequential)]
    internal unsafe struct AidnMhaArgs
    {
        public IntPtr input;                 // [batch, seq, heads*head_dim]
        public IntPtr q_weight, k_weight, v_weight, out_weight;   // [dModel, dModel], y = x * W
        public IntPtr @out;
        public IntPtr mask;                  // Tensor<bool> bytes, or zero
        public fixed long mask_stride[4];
        public long batch, seq;
        public int input_dtype, weight_dtype, out_dtype, reserved;
        public IntPtr workspace;
        public long workspace_bytes;
    }

    /// <summary>Arguments of aidn_qkv_rope_cache (QkvProjectionRoPECacheD64 generalised, see include/aidn_sdpa.h).</summary>
    [StructLayout(LayoutKind.Sequential)]
    internal struct AidnQkvRopeArgs
    {
        public IntPtr input, weights, bias, cosine, sine, query, key_cache, value_cache, positions, cache_rows;
        public int tokens, heads, kv_heads, head_dim, position, weight_dtype, query_dtype, cache_dtype;
        public long cache_capacity, max_position;
    }

    internal static class AidnSdpaNative
    {
        private const string Lib = "aidotnet_sdpa_sm100";

        static AidnSdpaNative()
        {
            // Same resolver mechanism as the cuBLAS / NVRTC bindings (Engines/NativeLibraryResolverRegistry.cs:35).
            NativeLibraryResolverRegistry.Register(Lib, new[] { "libaidotnet_sdpa_sm100.so", "aidotnet_sdpa_sm100.dll" });
        }

        /// <summary>Master switch, read once: AIDOTNET_SDPA_SM100=0 keeps the NVRTC kernels.</summary>
        public static readonly bool Enabled =
            Environment.GetEnvironmentVariable("AIDOTNET_SDPA_SM100") != "0";

        [DllImport(Lib)] public static extern int aidn_sdpa_create(ref AidnSdpaDesc desc, out IntPtr handle);
        [DllImport(Lib)] public static extern long aidn_sdpa_workspace_bytes(IntPtr handle, long batch, long seqQ, long seqKv);
        [DllImport(Lib)] public static extern int aidn_sdpa_launch(IntPtr handle, ref AidnSdpaArgs args, IntPtr cuStream);
        [DllImport(Lib)] public static extern int aidn_sdpa_launch_paged(IntPtr handle, ref AidnSdpaArgs args, ref AidnPagedKv paged, IntPtr cuStream);
        /// <summary>Batched decode without a handle or a workspace (split-KV partials in a 16 MiB array inside the
        /// library): for a backend that may not allocate device memory where it decodes.  First call per context
        /// outside stream capture; concurrent calls on one device share the array and must be stream-ordered.</summary>
        [DllImport(Lib)] public static extern int aidn_sdpa_decode_noalloc(ref AidnSdpaDesc desc, ref AidnSdpaArgs args, IntPtr cuStream);
        /// <summary>Peer mappings for AidnSdpaArgs.peer_out (fused gather of a head-sharded prefill): the 64-byte IPC
        /// handle and offset of a device allocation, and its mapping into another process of the same node.</summary>
        [DllImport(Lib)] public static extern int aidn_peer_export(IntPtr devPtr, byte[] handle64, out long offset);
        [DllImport(Lib)] public static extern int aidn_peer_open(byte[] handle64, out IntPtr basePtr);
        [DllImport(Lib)] public static extern int aidn_peer_close(IntPtr basePtr);
        [DllImport(Lib)] public static extern int aidn_paged_kv_append(IntPtr newKeys, IntPtr newValues, IntPtr keyPool, IntPtr valuePool, IntPtr blockTable, long startPosition, long tokens, int blockSize, int numBlocks, long rowBytes, IntPtr cuStream);
        [DllImport(Lib)] public static extern long aidn_sdpa_backward_workspace_bytes(IntPtr handle, long batch, long seqQ);
        [DllImport(Lib)] public static extern int aidn_sdpa_backward(IntPtr handle, ref AidnSdpaBwdArgs args, IntPtr cuStream);
        [DllImport(Lib)] public static extern long aidn_mha_workspace_bytes(IntPtr handle, long batch, long seq, int inputDtype, int weightDtype);
        [DllImport(Lib)] public static extern int aidn_mha_forward(IntPtr handle, ref AidnMhaArgs args, IntPtr cuStream);
        [DllImport(Lib)] public static extern int aidn_qkv_rope_cache(ref AidnQkvRopeArgs args, IntPtr cuStream);
        [DllImport(Lib)] public static extern int aidn_rope_interleaved(IntPtr input, IntPtr cosine, IntPtr sine, IntPtr output, long rows, int headDim, int seqLen, int startPosition, IntPtr cuStream);
        [DllImport(Lib)] public static extern int aidn_sdpa_poll(IntPtr handle, IntPtr cuStream);
        [DllImport(Lib)] public static extern int aidn_sdpa_last_path(IntPtr handle);
        [DllImport(Lib)] public static extern int aidn_sdpa_last_launch_count(IntPtr handle);
        [DllImport(Lib)] public static extern int aidn_sdpa_destroy(IntPtr handle);
        [DllImport(Lib)] private static extern IntPtr aidn_sdpa_last_error();
        [DllImport(Lib)] public static extern int aidn_sdpa_device_supported(int device);
        [DllImport(Lib)] public static extern int aidn_cast_f32_to_bf16(IntPtr src, IntPtr dst, long n, IntPtr cuStream);
        [DllImport(Lib)] public static extern int aidn_cast_f32_to_f16(IntPtr src, IntPtr dst, long n, IntPtr cuStream);
        [DllImport(Lib)] public static extern int aidn_cast_bf16_to_f32(IntPtr src, IntPtr dst, long n, IntPtr cuStream);
        [DllImport(Lib)] public static extern int aidn_cast_f16_to_f32(IntPtr src, IntPtr dst, long n, IntPtr cuStream);

        public static string LastError() => Marshal.PtrToStringAnsi(aidn_sdpa_last_error()) ?? string.Empty;

        /// <summary>Non-zero status becomes an exception; the sm_100a route has no CPU fallback.</summary>
        public static void Check(int status)
        {
            if (status == (int)AidnStatus.Ok) return;
            string message = $"aidn_sdpa status {(AidnStatus)status}: {LastError()}";
            if (status == (int)AidnStatus.Inval) throw new ArgumentException(message);
            throw new InvalidOperationException(message);
        }
    }
}
