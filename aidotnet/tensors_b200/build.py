"""Builds libaidotnet_sdpa_sm100.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m aidotnet.tensors_b200.build [--force] [--verbose]

Objects go to ``aidotnet/tensors_b200/build/`` and the library to ``aidotnet/tensors_b200/lib/``; both are
git-ignored.  The ptxas resource report of every kernel is kept in ``build/ptxas.log``.

Development variants: ``build_variant("trace", ["-DAIDN_PREFILL_TRACE=1"])`` compiles the same sources with extra
nvcc flags into ``lib/libaidotnet_sdpa_sm100.<name>.so`` (objects under ``build/<name>/``); ``native.load`` picks a
variant when the environment variable ``AIDN_SDPA_LIB`` names its path.  The shipped library is the flag-less one.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libaidotnet_sdpa_sm100.so")
SOURCES = ["aidn_api.cu", "sdpa_generic.cu", "sdpa_decode.cu", "sdpa_prefill_sm100.cu", "cast.cu", "qkv_rope_cache.cu", "sdpa_backward.cu", "proj_gemm_sm100.cu", "proj_gemm_generic.cu", "sdpa_backward_sm100.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _host_cxx() -> str:
    for cand in ("/usr/bin/g++", shutil.which("g++")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("g++ not found")


def _deps_mtime() -> float:
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(os.path.dirname(os.path.dirname(HERE)), "include", "aidn_sdpa.h"))
    files.append(os.path.abspath(__file__))
    return max(os.path.getmtime(f) for f in files)


def _compile(src: str, verbose: bool, outdir: str = BUILD, extra=()) -> str:
    obj = os.path.join(outdir, os.path.splitext(src)[0] + ".o")
    cmd = [_nvcc(), "-O3", "-std=c++17", *ARCH, "-lineinfo", "-ccbin", _host_cxx(), "-Xcompiler", "-fPIC,-fvisibility=hidden",
           "-Xptxas", "-v", "--expt-relaxed-constexpr", *extra, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr)
    return f"==== {src}\n{r.stderr}\n"


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    os.makedirs(BUILD, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        logs = list(ex.map(lambda s: _compile(s, verbose), SOURCES))
    with open(os.path.join(BUILD, "ptxas.log"), "w") as f:
        f.writelines(logs)
    objs = [os.path.join(BUILD, os.path.splitext(s)[0] + ".o") for s in SOURCES]
    cmd = [_nvcc(), "-shared", *ARCH, "-ccbin", _host_cxx(), "-cudart", "static", "-o", LIB, *objs, "-ldl", "-lpthread", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def build_variant(name: str, flags, verbose: bool = False, only=None) -> str:
    """Compiles the sources (or just those named in ``only``, linking the shipped build's objects for the rest) with
    the extra nvcc ``flags`` into ``lib/libaidotnet_sdpa_sm100.<name>.so``."""
    outdir = os.path.join(BUILD, name)
    os.makedirs(outdir, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    lib = os.path.join(LIBDIR, f"libaidotnet_sdpa_sm100.{name}.so")
    mine = [s for s in SOURCES if only is None or s in only]
    if only is not None:
        build()
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(mine)) as ex:
        logs = list(ex.map(lambda s: _compile(s, verbose, outdir, tuple(flags)), mine))
    with open(os.path.join(outdir, "ptxas.log"), "w") as f:
        f.writelines(logs)
    objs = [os.path.join(outdir if s in mine else BUILD, os.path.splitext(s)[0] + ".o") for s in SOURCES]
    cmd = [_nvcc(), "-shared", *ARCH, "-ccbin", _host_cxx(), "-cudart", "static", "-o", lib, *objs, "-ldl", "-lpthread", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


HOST_TEST_BIN = os.path.join(BUILD, "backend_tests")


def build_host_tests(force: bool = False) -> str:
    """Compiles the C++ host mirror (csrc/host) together with its test program (tests/cpp) against the library."""
    root = os.path.dirname(os.path.dirname(HERE))
    srcs = [os.path.join(root, "tests", "cpp", "backend_tests.cpp"), os.path.join(CSRC, "host", "direct_gpu_backend.cpp")]
    deps = srcs + [os.path.join(CSRC, "host", "direct_gpu_backend.hpp"), build(force)]
    if not force and os.path.exists(HOST_TEST_BIN) and os.path.getmtime(HOST_TEST_BIN) >= max(os.path.getmtime(f) for f in deps):
        return HOST_TEST_BIN
    cmd = [_nvcc(), "-O2", "-std=c++17", *ARCH, "-ccbin", _host_cxx(), "-o", HOST_TEST_BIN, *srcs, "-L", LIBDIR,
           "-laidotnet_sdpa_sm100", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"host test build failed:\n{r.stdout}\n{r.stderr}")
    return HOST_TEST_BIN


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_host_tests(force="--force" in sys.argv))
