"""TEST INFRASTRUCTURE — builds the checker libraries; nothing here is the product.

  oracle/_build/liboracle.so          gcc    gemm_oracle.c            (CPU restatement)
  oracle/_build/liboracle_device.so   nvcc   gemm_naive_device.cu     (device restatement)
  oracle/_ref/libref_peakgemm.so      nvcc   ref_wrapper.cu + the reference's own headers,
                                             compiled where they lie (only when a reference
                                             checkout is present; flags of its build_cuda.sh:1-2
                                             with the architecture made explicit)

    python oracle/build_oracle.py [--force] [--reference /path/to/PeakGemm]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "_build")
REF_OUT = os.path.join(HERE, "_ref")
CPU_LIB = os.path.join(BUILD, "liboracle.so")
DEV_LIB = os.path.join(BUILD, "liboracle_device.so")
REF_LIB = os.path.join(REF_OUT, "libref_peakgemm.so")
# A checkout of the reference project: PEAKGEMM_REFERENCE_DIR, else a directory named "reference" beside this
# repository.  Absent: the reference library is simply not built.
DEFAULT_REFERENCE = os.environ.get("PEAKGEMM_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def _stale(target: str, deps: list[str]) -> bool:
    return not os.path.exists(target) or any(os.path.getmtime(d) > os.path.getmtime(target) for d in deps)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")


def build_cpu(force: bool = False) -> str:
    src = os.path.join(HERE, "gemm_oracle.c")
    if force or _stale(CPU_LIB, [src]):
        os.makedirs(BUILD, exist_ok=True)
        # -mavx2 -mfma: vectorise the n-loop; rounding is unaffected (products are exact in fp32)
        _run(["gcc", "-O3", "-mavx2", "-mfma", "-fopenmp", "-fPIC", "-shared", src, "-o", CPU_LIB])
    return CPU_LIB


def build_device(force: bool = False) -> str:
    src = os.path.join(HERE, "gemm_naive_device.cu")
    if force or _stale(DEV_LIB, [src]):
        os.makedirs(BUILD, exist_ok=True)
        _run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-shared", src, "-o", DEV_LIB])
    return DEV_LIB


def build_reference(reference_dir: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    """Compiles the reference's own kernels; returns None when no reference checkout is present."""
    common = os.path.join(reference_dir, "src", "common")
    impl = os.path.join(reference_dir, "src", "impl")
    if not (os.path.isdir(common) and os.path.isdir(impl)):
        return REF_LIB if os.path.exists(REF_LIB) else None
    src = os.path.join(HERE, "ref_wrapper.cu")
    deps = [src, os.path.join(impl, "hgemm_wmma_impl.h"), os.path.join(impl, "sgemm_impl.h")]
    if force or _stale(REF_LIB, deps):
        os.makedirs(REF_OUT, exist_ok=True)
        _run([_nvcc(), "-x", "cu", "-O3", "--std=c++20", "--expt-relaxed-constexpr",
              "-gencode", "arch=compute_100a,code=sm_100a", f"-I{common}", f"-I{impl}",
              "-diag-suppress", "20012", "-Xcompiler", "-fPIC", "-shared", src, "-o", REF_LIB])
    return REF_LIB


def build_all(force: bool = False, reference_dir: str = DEFAULT_REFERENCE) -> dict:
    return {"cpu": build_cpu(force), "device": build_device(force),
            "reference": build_reference(reference_dir, force)}


if __name__ == "__main__":
    ref = DEFAULT_REFERENCE
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    for k, v in build_all("--force" in sys.argv, ref).items():
        print(f"{k}: {v}")
