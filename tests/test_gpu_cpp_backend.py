"""Runs the C++ port of the reference's backend attention tests (tests/cpp/backend_tests.cpp) against the C++ host
mirror of CudaBackend (aidotnet/tensors_b200/csrc/host), which calls the library through the C ABI."""
import subprocess

import pytest

pytestmark = pytest.mark.gpu


def test_cpp_backend_mirror_passes_the_ported_reference_tests():
    from aidotnet.tensors_b200 import build
    exe = build.build_host_tests()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(r.stdout[-3000:])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "all cases passed" in r.stdout
