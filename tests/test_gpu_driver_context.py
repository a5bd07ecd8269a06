"""The library inside the reference's context convention: a non-primary driver context (cuCtxCreate), the caller's own
stream, cuMemAlloc'd buffers - alone, and with torch's primary context alive on the same GPU.  The work is done by
tests/_driver_ctx_worker.py in a child process (a fresh process has no CUDA context until the script makes one)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("extra", [[], ["--with-torch"]])
def test_library_runs_in_a_caller_created_driver_context(extra):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_driver_ctx_worker.py"), *extra], capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0 and "driver-context run ok" in r.stdout, f"stdout:\n{r.stdout}\nstderr:\n{r.stderr[-3000:]}"
