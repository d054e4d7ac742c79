"""CPU: include/peakgemm.h compiles as C and as C++ and a caller written against it links the device library and
runs the calls that need no GPU (status strings, empty problems, argument errors, the configuration choice).
The reference's own C++ tests call its kernels the same way, without torch (test/cpp/test_gemm_half.cpp:1-2)."""
import os
import shutil
import subprocess

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(REPO, "tests", "abi", "caller.c")
LIB_DIR = os.path.join(REPO, "peakgemm_b200")


@pytest.mark.parametrize("compiler,lang", [("gcc", "c"), ("g++", "c++")])
def test_header_compiles_links_and_runs(tmp_path, compiler, lang):
    if shutil.which(compiler) is None:
        pytest.skip(f"{compiler} not installed")
    from peakgemm_b200 import capi  # noqa: F401  (builds the library if it is missing)

    exe = str(tmp_path / f"caller_{lang.replace('+', 'p')}")
    cmd = [compiler, "-x", lang, "-Wall", "-Werror", "-pedantic", "-I", os.path.join(REPO, "include"), SRC, "-o", exe,
           "-L", LIB_DIR, "-lPeakGemm_device", f"-Wl,-rpath,{LIB_DIR}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failure(s)" in r.stdout
