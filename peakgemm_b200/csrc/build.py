"""In-tree build of the two shared libraries (sm_100a only).

  libPeakGemm_device.so   torch-free CUDA kernels behind the C ABI of include/peakgemm.h  (nvcc)
  libPeakGemm.so          the torch operator registration over that ABI                    (g++)

The reference project builds the same pair with CMake (CMakeLists.txt:11-40:
`${PROJECT}_device` SHARED from src/ops/*.cpp compiled as CUDA with -arch=native,
`${PROJECT}` MODULE from src/register.cpp).  Here the architecture is fixed to
sm_100a (`-arch native` needs a visible GPU) and torch headers never reach nvcc.

    python peakgemm_b200/csrc/build.py [--force] [--verbose] [--tuning]

--tuning compiles the benchmark-only PEAKGEMM_TUNE_* environment overrides in (-DPG_ENABLE_TUNING); the
library is shipped without them and then never reads the environment.

Run as a script (or loaded by path): it must work before the package can be
imported, because importing the package requires the built libraries.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.dirname(CSRC)
REPO_DIR = os.path.dirname(PKG_DIR)
INCLUDE = os.path.join(REPO_DIR, "include")

DEVICE_LIB = os.path.join(PKG_DIR, "libPeakGemm_device.so")
TORCH_LIB = os.path.join(PKG_DIR, "libPeakGemm.so")
# The same device library compiled with -DPG_TEST_SHORT_WAIT: bounded waits of 2 ms and a switch that makes one
# signal go missing.  Loaded only by tests/test_wait_timeout_gpu.py; nothing in the package opens it.
WAITTEST_LIB = os.path.join(PKG_DIR, "libPeakGemm_device_waittest.so")

DEVICE_SOURCES = ["gemm_sm100.cu", "rmsnorm.cu", "rmsnorm_staged.cu", "rmsnorm_static.cu", "rmsnorm_rstd.cu", "peer.cu", "sgemm.cu", "probes.cu", "api.cu"]
DEVICE_HEADERS = ["ptx.cuh", "gemm_sm100.h", "host_util.h", "rmsnorm.h", "sgemm.h", os.path.join(INCLUDE, "peakgemm.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found: cannot build libPeakGemm_device.so")
    return found


def _newer(target: str, deps: list[str]) -> bool:
    """True if target exists and is newer than every dependency."""
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print("+", " ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed ({r.returncode}): {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)


def build_device_lib(force: bool = False, verbose: bool = False, tuning: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in DEVICE_SOURCES]
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in DEVICE_HEADERS]
    if not force and _newer(DEVICE_LIB, srcs + hdrs):
        return DEVICE_LIB
    objs = []
    obj_dir = os.path.join(PKG_DIR, "build")
    os.makedirs(obj_dir, exist_ok=True)
    procs = []
    for s in srcs:
        o = os.path.join(obj_dir, os.path.basename(s) + ".o")
        objs.append(o)
        cmd = [_nvcc(), *NVCC_FLAGS, *(["-DPG_ENABLE_TUNING"] if tuning else []), "-I", INCLUDE, "-c", s, "-o", o]
        if verbose:
            print("+", " ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{out}")
    _run([_nvcc(), "-shared", "-o", DEVICE_LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    return DEVICE_LIB


def build_waittest_lib(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in DEVICE_SOURCES]
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in DEVICE_HEADERS]
    if not force and _newer(WAITTEST_LIB, srcs + hdrs):
        return WAITTEST_LIB
    obj_dir = os.path.join(PKG_DIR, "build", "waittest")
    os.makedirs(obj_dir, exist_ok=True)
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(obj_dir, os.path.basename(s) + ".o")
        objs.append(o)
        cmd = [_nvcc(), *NVCC_FLAGS, "-DPG_TEST_SHORT_WAIT", "-I", INCLUDE, "-c", s, "-o", o]
        if verbose:
            print("+", " ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{out}")
    _run([_nvcc(), "-shared", "-o", WAITTEST_LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    return WAITTEST_LIB


def build_torch_lib(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "torch_shim.cpp")
    if not force and _newer(TORCH_LIB, [src, os.path.join(INCLUDE, "peakgemm.h"), DEVICE_LIB]):
        return TORCH_LIB
    import torch
    from torch.utils import cpp_extension as ce

    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{cuda_home}/include", f"-I{INCLUDE}"]
    torch_lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [
        "g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        *inc, src, "-o", TORCH_LIB,
        f"-L{PKG_DIR}", "-lPeakGemm_device", "-Wl,-rpath,$ORIGIN",
        f"-L{torch_lib_dir}", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda", "-ltorch_cuda",
        f"-Wl,-rpath,{torch_lib_dir}",
    ]
    _run(cmd, verbose)
    return TORCH_LIB


def build_all(force: bool = False, verbose: bool = False, tuning: bool = False) -> tuple[str, str]:
    libs = build_device_lib(force or tuning, verbose, tuning), build_torch_lib(force, verbose)
    build_waittest_lib(force, verbose)
    return libs


if __name__ == "__main__":
    libs = build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv, tuning="--tuning" in sys.argv)
    print("\n".join(libs))
