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


def test_field_offsets_match_header():
    """Field by field: every member of the ctypes mirrors sits at the offset the C compiler gives the member of the same
    name in the header (a swapped or missing field with an unchanged total size would pass the size check above)."""
    import subprocess
    import tempfile
    from aidotnet.tensors_b200 import native
    pairs = [("aidn_sdpa_desc", native.SdpaDesc), ("aidn_sdpa_args", native.SdpaArgs), ("aidn_paged_kv", native.PagedKv),
             ("aidn_qkv_rope_args", native.QkvRopeArgs), ("aidn_sdpa_bwd_args", native.SdpaBwdArgs),
             ("aidn_mha_args", native.MhaArgs)]
    lines = ['#include "aidn_sdpa.h"', "#include <stddef.h>", "#include <stdio.h>", "int main(){"]
    expected = []
    for cname, mirror in pairs:
        for fname, _ in mirror._fields_:
            lines.append(f'printf("%zu\\n", offsetof({cname}, {fname}));')
            expected.append((cname, fname, getattr(mirror, fname).offset))
    lines.append("return 0;}")
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "t.c")
        open(c, "w").write("\n".join(lines) + "\n")
        exe = os.path.join(d, "t")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        got = list(map(int, subprocess.check_output([exe]).split()))
    assert len(got) == len(expected)
    for (cname, fname, off), g in zip(expected, got):
        assert off == g, f"{cname}.{fname}: ctypes offset {off}, header offset {g}"


def test_csharp_binding_lists_the_same_fields_in_the_same_order():
    """The P/Invoke structs cannot be compiled here (no .NET toolchain), so they are checked as text: every struct of
    bindings/AidnSdpaNative.cs names the fields of its ctypes mirror in the same order (`@out` = out; a C array member
    may be spelled as numbered fields)."""
    import re
    from aidotnet.tensors_b200 import native
    text = open(os.path.join(ROOT, "aidotnet", "tensors_b200", "bindings", "AidnSdpaNative.cs")).read()
    pairs = [("AidnSdpaDesc", native.SdpaDesc), ("AidnSdpaArgs", native.SdpaArgs), ("AidnPagedKv", native.PagedKv),
             ("AidnQkvRopeArgs", native.QkvRopeArgs), ("AidnSdpaBwdArgs", native.SdpaBwdArgs), ("AidnMhaArgs", native.MhaArgs)]
    for cs_name, mirror in pairs:
        m = re.search(r"struct\s+" + cs_name + r"\s*\{(.*?)\n    \}", text, re.S)
        assert m, f"{cs_name} not found in the C# binding"
        names = []
        for line in m.group(1).split("\n"):
            line = line.split("//")[0].strip()
            if not line.startswith("public"):
                continue
            decl = line.rstrip(";").split()
            body = " ".join(decl[2:]) if decl[1] != "fixed" else " ".join(decl[3:])
            for item in body.split(","):
                name = item.strip().lstrip("@")
                name = re.sub(r"\[.*\]$", "", name)
                name = re.sub(r"\d+$", "", name) if re.fullmatch(r"[a-z_]+\d", name) and name[:-1] + "0" in body else name
                if name and (not names or names[-1] != name):
                    names.append(name)
        expected = [f for f, _ in mirror._fields_]
        assert names == expected, f"{cs_name}: C# lists {names}, the C ABI has {expected}"


def test_csharp_binding_declares_every_entry_point():
    """Every exported entry point has a DllImport in the C# binding (the debug hook of aidn_sdpa_debug.h excepted:
    it is for this repository's tests)."""
    from aidotnet.tensors_b200 import native
    text = open(os.path.join(ROOT, "aidotnet", "tensors_b200", "bindings", "AidnSdpaNative.cs")).read()
    missing = [n for n in native.EXPORTS if n != "aidn_sdpa_debug_set" and f"extern" in text and f" {n}(" not in text]
    assert not missing, f"no DllImport for {missing}"


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
