"""CPU-side checks of the drop-in boundary: the CUDA library builds, loads and exports every symbol that
include/aidn_sdpa.h declares, and argument validation answers with status codes (no compute without a GPU)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from aidotnet.tensors_b200 import build
    return ctypes.CDLL(build.build())


def test_every_declared_symbol_is_exported(lib):
    header = "".join(open(os.path.join(ROOT, "include", name)).read() for name in ("aidn_sdpa.h", "aidn_sdpa_debug.h"))
    declared = set(re.findall(r"AIDN_API\s+[\w\s\*]+?\b(aidn_\w+)\s*\(", header))
    assert len(declared) >= 13
    from aidotnet.tensors_b200 import native
    assert declared == set(native.EXPORTS), declared ^ set(native.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_struct_layout_matches_header():
    """The ctypes mirrors must have the size the C compiler gives the header's structs."""
    import subprocess
    import tempfile
    from aidotnet.tensors_b200 import native
    src = '#include "aidn_sdpa.h"\n#include <stdio.h>\nint main(){printf("%zu %zu %zu %zu %zu %zu\\n", sizeof(aidn_sdpa_desc), sizeof(aidn_sdpa_args), sizeof(aidn_paged_kv), sizeof(aidn_qkv_rope_args), sizeof(aidn_sdpa_bwd_args), sizeof(aidn_mha_args));return 0;}\n'
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "t.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "t")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        a, b, c, d4, e5, f6 = map(int, subprocess.check_output([exe]).split())
    assert ctypes.sizeof(native.SdpaDesc) == a
    assert ctypes.sizeof(native.SdpaArgs) == b
    assert ctypes.sizeof(native.PagedKv) == c
    assert ctypes.sizeof(native.QkvRopeArgs) == d4
    assert ctypes.sizeof(native.SdpaBwdArgs) == e5
    assert ctypes.sizeof(native.MhaArgs) == f6


def test_validation_without_gpu():
    from aidotnet.tensors_b200 import native as N
    N.load()
    with pytest.raises(N.AidnError) as e:
        N.Handle(device=0, qkv_dtype=7, head_dim=128, num_q_heads=8)
    assert e.value.status == N.EINVAL and "qkv_dtype" in e.value.message
    with pytest.raises(N.AidnError) as e:
        N.Handle(device=0, qkv_dtype=N.BF16, head_dim=128, num_q_heads=6, num_kv_heads=4)
    assert e.value.status == N.EINVAL
    with pytest.raises(N.AidnError) as e:
        N.Handle(device=0, qkv_dtype=N.BF16, head_dim=128, num_q_heads=8, num_kv_heads=2, head_begin=2, head_count=4)
    assert e.value.status == N.EINVAL and "KV groups" in e.value.message
    import torch
    if not torch.cuda.is_available():
        # a well-formed request on a machine without a GPU is a CUDA error, never a silent CPU path
        with pytest.raises(N.AidnError) as e:
            N.Handle(device=0, qkv_dtype=N.BF16, head_dim=128, num_q_heads=8)
        assert e.value.status in (N.ECUDA, N.EUNSUPPORTED)
        assert N.load().aidn_sdpa_device_supported(0) == 0


def test_backend_refuses_to_run_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from aidotnet.tensors_b200.backend import CudaBackend
    with pytest.raises(RuntimeError):
        CudaBackend(0)
