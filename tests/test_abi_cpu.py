"""CPU: the C-ABI library loads and exports every symbol include/peakgemm.h declares; calls that must
return before touching CUDA do so with the right status; the torch operators are registered with the
reference's schema.  No compute call is made here."""
import ctypes
import os
import re

import pytest
import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(REPO, "include", "peakgemm.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(pg_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("pg_hgemm", "pg_hgemm_ex", "pg_hgemm_ws", "pg_hgemm_workspace_bytes", "pg_hgemm_fused", "pg_rmsnorm_rstd", "pg_hgemm_multi", "pg_hgemm_mcast", "pg_sgemm", "pg_hgemm_config", "pg_rmsnorm_fwd", "pg_rmsnorm_bwd",
                 "pg_rmsnorm_bwd_workspace_bytes", "pg_rmsnorm_bwd_static", "pg_device_status",
                 "pg_status_string", "pg_last_cuda_error", "pg_version", "pg_peer_alloc", "pg_peer_open",
                 "pg_peer_close", "pg_peer_free", "pg_probe_tensor_peak", "pg_probe_copy"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from peakgemm_b200 import capi

    lib = ctypes.CDLL(capi.DEVICE_LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/peakgemm.h but not exported"
    assert sorted(capi.SIGNATURES) == declared_functions()     # the ctypes binding covers the same set


def test_status_strings():
    from peakgemm_b200 import capi

    L = capi.lib()
    assert L.pg_status_string(0) == b"PG_OK"
    seen = {L.pg_status_string(i) for i in range(0, 9)}
    assert len(seen) == 9 and all(s.startswith(b"PG_") for s in seen)
    assert L.pg_status_string(99) == b"unknown pg_status"
    assert L.pg_version() == b"0.1"


def test_argument_checks_return_before_any_cuda_call():
    from peakgemm_b200 import capi

    L = capi.lib()
    p = 4096                                     # a fake, aligned, never dereferenced address
    ex = lambda *a: L.pg_hgemm_ex(*a)            # noqa: E731
    assert L.pg_hgemm(p, p, p, 0, 64, 64, 64, 64, 64, 1, None) == 0           # m == 0: no-op
    assert L.pg_hgemm(p, p, p, 64, 0, 64, 64, 64, 0, 1, None) == 0            # n == 0: no-op
    assert L.pg_hgemm(p, p, p, -1, 64, 64, 64, 64, 64, 1, None) == 1
    assert L.pg_hgemm(p, p, p, 64, 64, 64, 64, 64, 64, 5, None) == 1          # dtype
    assert L.pg_hgemm(None, p, p, 64, 64, 64, 64, 64, 64, 1, None) == 1       # null C
    assert L.pg_hgemm(p, p, p, 64, 64, 64, 32, 64, 64, 1, None) == 1          # lda < k
    assert L.pg_hgemm(p, p, p, 64, 12, 64, 64, 64, 12, 1, None) == 3          # n % 8
    assert L.pg_hgemm(p, p, p, 64, 64, 20, 20, 20, 64, 1, None) == 3          # k % 8
    assert L.pg_hgemm(p, p, p, 64, 64, 64, 64, 64, 68, 1, None) == 3          # ldc % 8
    assert L.pg_hgemm(p, p, p, 2 ** 31, 64, 64, 64, 64, 64, 1, None) == 3     # size limit
    assert L.pg_hgemm(p + 2, p, p, 64, 64, 64, 64, 64, 64, 1, None) == 2      # misaligned
    assert ex(p, p, p, 64, 64, 64, 64, 64, 64, 1, 9, 0, 0, None) == 1         # variant
    assert ex(p, p, p, 64, 64, 64, 64, 64, 64, 1, 1, 100, 0, None) == 1       # block_n
    assert ex(p, p, p, 64, 64, 64, 64, 64, 64, 1, 1, 64, -1, None) == 1       # max_sms
    assert L.pg_sgemm(p, p, p, 0, 8, 8, 8, 8, 8, None) == 0
    assert L.pg_sgemm(p, p, p, 8, 8, 6, 8, 8, 8, None) == 3                   # k % 4
    assert L.pg_sgemm(None, p, p, 8, 8, 8, 8, 8, 8, None) == 1
    assert L.pg_rmsnorm_fwd(p, p, p, 0, 64, 1e-6, 1, None) == 0               # rows == 0
    assert L.pg_rmsnorm_fwd(p, p, p, 4, 60, 1e-6, 1, None) == 3               # h % 8
    assert L.pg_rmsnorm_fwd(p, p, p, 4, 0, 1e-6, 1, None) == 1
    assert L.pg_rmsnorm_fwd(p, None, p, 4, 64, 1e-6, 1, None) == 1
    assert L.pg_rmsnorm_bwd(p, None, p, p, p, 4, 64, 1e-6, 1, p, 1 << 20, None) == 1
    assert L.pg_rmsnorm_bwd(p, p, p, p, p, 4, 1 << 20, 1e-6, 1, p, 1 << 20, None) == 3    # h over the limit
    assert L.pg_rmsnorm_bwd_static(p, p, p, p, p, 4, 60, 1e-6, 1, None) == 3
    assert L.pg_rmsnorm_bwd_static(p, p, p, p, p, 4, 64, 1e-6, 9, None) == 1
    assert L.pg_device_status(None, None) == 1
    assert L.pg_hgemm_ws(p, p, p, 0, 64, 64, 64, 64, 64, 1, None, 0, None) == 0              # m == 0: no-op
    assert L.pg_hgemm_ws(p, p, p, 64, 64, 64, 64, 64, 64, 1, p + 16, 1 << 20, None) == 2     # workspace alignment
    assert L.pg_hgemm_ws(p, p, p, 64, 12, 64, 64, 64, 12, 1, None, 0, None) == 3             # n % 8
    assert L.pg_hgemm_workspace_bytes(0, 64, 64) == 0
    fu = lambda *a: L.pg_hgemm_fused(*a)         # noqa: E731
    assert fu(p, p, p, 0, 64, 64, 64, 64, 64, p, p, p, 64, 1, 0, None) == 0        # m == 0: no-op
    assert fu(p, p, p, 64, 64, 0, 0, 0, 64, None, None, None, 0, 1, 0, None) == 3  # k == 0 not accepted here
    assert fu(p, p, p, 64, 64, 64, 64, 64, 64, None, None, None, 0, 1, 2, None) == 1   # unknown flag
    assert fu(p, p, p, 64, 64, 64, 64, 64, 64, None, None, p, 32, 1, 0, None) == 1     # ldr < n
    assert fu(p, p, p, 64, 64, 64, 64, 64, 64, None, None, p, 68, 1, 0, None) == 3     # ldr % 8
    assert fu(p, p, p, 64, 64, 64, 64, 64, 64, None, p + 2, None, 0, 1, 0, None) == 2  # bias misaligned
    assert fu(p, p, p, 64, 64, 64, 64, 64, 64, p + 2, None, None, 0, 1, 0, None) == 2  # row_scale misaligned
    assert fu(None, p, p, 64, 64, 64, 64, 64, 64, None, None, None, 0, 1, 0, None) == 1
    assert L.pg_rmsnorm_rstd(p, p, 0, 64, 1e-6, 1, None) == 0
    assert L.pg_rmsnorm_rstd(p, p, 4, 60, 1e-6, 1, None) == 3
    assert L.pg_rmsnorm_rstd(None, p, 4, 64, 1e-6, 1, None) == 1
    assert capi.lib().pg_rmsnorm_bwd_workspace_bytes(0, 64) == 0


def test_config_choice_is_host_arithmetic():
    from peakgemm_b200 import capi

    assert capi.hgemm_config(8192, 8192, 8192) == (5, 256)        # headline shape: CTA pairs, 512 x 256 tiles
    assert capi.hgemm_config(16384, 16384, 16384) == (5, 256)
    assert capi.hgemm_config(32768, 4096, 16384) == (5, 256)      # one rank's block of the sharded benchmark shape
    assert capi.hgemm_config(2048, 2048, 2048) == (2, 256)        # 32 large tiles would idle most SM pairs
    assert capi.hgemm_config(4096, 14336, 4096) == (2, 256)       # 448 large tiles: 7 waves for 6.05 waves of work
    assert capi.hgemm_config(4096, 4096, 4096) == (2, 256)        # two waves of large tiles: no gain, the tie goes to 256 x 256
    assert capi.hgemm_config(8192, 3328, 256) == (5, 256)         # the shapes tests/test_fused_gpu.py and
    assert capi.hgemm_config(8000, 3304, 136) == (5, 256)         # tests/test_dist_gpu.py rely on: 208 large tiles, 3 waves
    v, bn = capi.hgemm_config(16, 4096, 4096)
    assert v == 1 and bn == 64                                    # one tile row: no pair, most CTAs
    v, bn = capi.hgemm_config(128, 128256, 4096)
    assert v == 1                                                 # m <= 128: a pair would idle half its rows
    for m in (1, 100, 129, 1000, 5000):
        for n in (8, 512, 4096, 14336):
            v, bn = capi.hgemm_config(m, n, 4096)
            assert v in (1, 2, 5) and bn in (64, 128, 256)
            assert not (v in (2, 5) and m <= 128)
    assert capi.lib().pg_hgemm_config(0, 8, 8, 148, None, None) == 1


def test_torch_operator_schemas_match_the_reference():
    import peakgemm_b200  # noqa: F401

    s = str(torch.ops.PeakGemm.gemm_peak.default._schema)
    # src/register.cpp:5 of the reference, verbatim
    assert s == "PeakGemm::gemm_peak(Tensor c, Tensor a, Tensor b, SymInt m, SymInt n, SymInt k) -> ()"
    assert str(torch.ops.PeakGemm.rms_norm_fwd.default._schema) == \
        "PeakGemm::rms_norm_fwd(Tensor y, Tensor x, Tensor gamma, float eps) -> ()"
    assert str(torch.ops.PeakGemm.rms_norm_bwd.default._schema) == \
        "PeakGemm::rms_norm_bwd(Tensor dx, Tensor dgamma, Tensor dy, Tensor x, Tensor gamma, float eps) -> ()"


def test_annotated_operators_trace_under_fake_tensors():
    """The `_out` / fused operators mark what they write and have fake implementations, so a tracer can
    run them without a GPU and without reaching the kernels (the reference's schema is un-annotated)."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    import peakgemm_b200 as pg

    ops = torch.ops.PeakGemm
    assert str(ops.gemm_peak_out.default._schema) == "PeakGemm::gemm_peak_out(Tensor(a!) c, Tensor a, Tensor b) -> ()"
    assert "Tensor(a!) d" in str(ops.gemm_peak_fused.default._schema)
    assert "Tensor(a!) dx, Tensor(b!) dgamma" in str(ops.rms_norm_bwd_out.default._schema)
    for name in ("gemm_peak_out", "rms_norm_fwd_out", "rms_norm_bwd_out", "rms_norm_rstd", "gemm_peak_fused"):
        assert getattr(ops, name).default._schema.is_mutable
    with FakeTensorMode():
        x = torch.empty(64, 128, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(32, 128, dtype=torch.bfloat16, device="cuda")
        out = torch.empty(64, 32, dtype=torch.bfloat16, device="cuda")
        gamma = torch.empty(128, device="cuda")
        rstd = pg.rms_norm_linear(out, x, w, bias=torch.empty(32, dtype=torch.bfloat16, device="cuda"), residual=out)
        assert rstd.shape == (64,) and rstd.dtype == torch.float32
        ops.gemm_peak_out(out, x, w)
        ops.rms_norm_fwd_out(x.clone(), x, gamma, 1e-6)
        ops.rms_norm_bwd_out(torch.empty_like(x), torch.empty_like(gamma), x, x, gamma, 1e-6)
    # no CPU fallback behind the CUDA-only registrations either
    with pytest.raises((RuntimeError, NotImplementedError)):
        ops.gemm_peak_out(torch.zeros(8, 8, dtype=torch.bfloat16), torch.zeros(8, 8, dtype=torch.bfloat16),
                          torch.zeros(8, 8, dtype=torch.bfloat16))


def test_fold_gamma_is_the_rounded_product():
    import peakgemm_b200 as pg

    g = torch.Generator().manual_seed(3)
    w = torch.randn(24, 64, generator=g).to(torch.bfloat16)
    gamma = 1 + 0.1 * torch.randn(64, generator=g)
    wf = pg.fold_gamma(w, gamma)
    assert wf.dtype == w.dtype and torch.equal(wf, (w.float() * gamma[None, :]).to(torch.bfloat16))


def test_python_surface_mirrors_the_reference_wrapper():
    """Same shape plumbing and asserts as PeakGemm/__init__.py:21-34; no CPU fallback."""
    import PeakGemm
    import peakgemm_b200

    assert PeakGemm.gemm_peak is peakgemm_b200.gemm_peak
    a = torch.zeros(2, 3, 16, dtype=torch.bfloat16)
    b = torch.zeros(8, 16, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        PeakGemm.gemm_peak(torch.zeros(2, 3, 8, dtype=torch.bfloat16), a, torch.zeros(8, 24, dtype=torch.bfloat16))
    with pytest.raises(AssertionError):
        PeakGemm.gemm_peak(torch.zeros(5, 8, dtype=torch.bfloat16), a, b)          # rows of c != rows of a
    with pytest.raises(AssertionError):
        PeakGemm.gemm_peak(torch.zeros(6, 8, dtype=torch.int32), a.int(), b.int())   # dtype assert
    with pytest.raises(RuntimeError, match="CUDA"):
        PeakGemm.gemm_peak(torch.zeros(2, 3, 8, dtype=torch.bfloat16), a, b)       # CPU tensors: refused
    with pytest.raises(RuntimeError, match="CUDA"):
        PeakGemm.rms_norm_fwd(torch.zeros(4, 16, dtype=torch.bfloat16), torch.zeros(4, 16, dtype=torch.bfloat16),
                              torch.ones(16))


def test_product_code_never_imports_the_oracle():
    """The oracle is test infrastructure: nothing under peakgemm_b200/ or PeakGemm/ may reference it."""
    for root in ("peakgemm_b200", "PeakGemm"):
        for dirpath, _, files in os.walk(os.path.join(REPO, root)):
            for f in files:
                if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                    text = open(os.path.join(dirpath, f)).read()
                    assert "import oracle" not in text and "from oracle" not in text and "oracle/" not in text, f
