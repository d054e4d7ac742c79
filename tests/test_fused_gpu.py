"""GPU: the callers either side of the GEMM — fused epilogue (row scale, bias, residual), RMSNorm folded
into the projection, CUDA-graph replay of norm -> GEMM chains, and tracing of the annotated operators.

The reference has none of this (plain cast epilogue, src/impl/wmma_utils.h:101-112; un-annotated schema,
src/register.cpp:5), so the oracle is the definition evaluated on the CPU (oracle.gemm_fused,
oracle.rmsnorm_linear) — parity unpinned.  Bounds, written once:
  * fused epilogue, per element: within one 16-bit ulp of the rounded oracle value, or within the fp32
    accumulation slack 2^-17 * |row_scale| * (|A| @ |B|^T) of the unrounded one; and the global GEMM bound
    max|D - D_ref| <= (2e-2 * sqrt(k/4096) + eps_out) * max|D_ref|;
  * rstd: relative error <= 1e-5 against float64;
  * RMSNorm -> projection chain: the global GEMM bound against the unfolded, unrounded definition.
"""
import pytest
import torch

import oracle
from tests import helpers

pytestmark = pytest.mark.gpu

BF16, F16 = torch.bfloat16, torch.float16

# one shape per kernel the automatic choice can take, tails included
SHAPES = [
    pytest.param(16, 4096, 4096, id="skinny-cluster"),
    pytest.param(40, 264, 520, id="skinny-tails"),
    pytest.param(128, 4096, 4096, id="split-k"),
    pytest.param(100, 520, 1000, id="split-k-tails"),
    pytest.param(128, 14336, 1024, id="one-cta"),
    pytest.param(1024, 4096, 1024, id="pair"),
    pytest.param(300, 456, 264, id="pair-tails"),
    pytest.param(8192, 3328, 256, id="pair-two-row-blocks"),
    pytest.param(8000, 3304, 136, id="pair-two-row-blocks-tails"),
]


def fused_inputs(m, n, k, dtype, seed):
    a, b = oracle.gemm_inputs_llm(m, n, k, dtype, seed)
    g = torch.Generator().manual_seed(seed + 1000)
    row_scale = 0.5 + torch.rand(m, generator=g)
    bias = torch.randn(n, generator=g).to(dtype)
    residual = torch.randn(m, n, generator=g).to(dtype)
    return a, b, row_scale, bias, residual


def check_fused(d_gpu, a, b, row_scale, bias, residual):
    k = a.shape[1]
    d = d_gpu.cpu()
    assert not torch.isnan(d.float()).any()
    ref = oracle.gemm_fused(a, b, row_scale, bias, residual)
    tol = oracle.gemm_tolerance(k, ref, d.dtype)
    err = (d.float() - ref).abs().max().item()
    assert err <= tol, f"max|D-D_ref| = {err} > {tol}"
    ok = oracle.within_ulp_or_slack(d, ref, oracle.gemm_fused_slack(a, b, row_scale), ulps=1)
    assert bool(ok.all()), f"{int((~ok).sum())} elements off by more than 1 ulp + accumulation slack"


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_identity_epilogue_is_bit_identical_to_plain_gemm(cuda, m, n, k):
    """row_scale = 1, bias = 0, residual = 0 must reproduce pg_hgemm bit for bit on every kernel."""
    from peakgemm_b200 import capi

    a, b = oracle.gemm_inputs_uniform(m, n, k, BF16, 31)
    ad, bd = a.cuda(), b.cuda()
    plain = helpers.garbage_like((m, n), BF16, "cuda")
    fused = helpers.garbage_like((m, n), BF16, "cuda")
    capi.hgemm(plain, ad, bd)
    capi.hgemm_fused(fused, ad, bd, row_scale=torch.ones(m, device="cuda"),
                     bias=torch.zeros(n, dtype=BF16, device="cuda"),
                     residual=torch.zeros(m, n, dtype=BF16, device="cuda"))
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    assert torch.equal(plain.view(torch.int16), fused.view(torch.int16))


@pytest.mark.parametrize("terms", ["scale", "bias", "residual", "scale+bias+residual"])
@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_fused_epilogue_terms(cuda, m, n, k, dtype, terms):
    from peakgemm_b200 import capi

    a, b, rs, bias, res = fused_inputs(m, n, k, dtype, 32)
    rs = rs if "scale" in terms else None
    bias = bias if "bias" in terms else None
    res = res if "residual" in terms else None
    d = helpers.garbage_like((m, n), dtype, "cuda")
    dev = lambda t: t.cuda() if t is not None else None     # noqa: E731
    capi.hgemm_fused(d, a.cuda(), b.cuda(), row_scale=dev(rs), bias=dev(bias), residual=dev(res))
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    check_fused(d, a, b, rs, bias, res)


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_residual_may_be_the_output_itself(cuda, m, n, k):
    """d += a @ b^T: the residual pointer is the output pointer."""
    from peakgemm_b200 import capi

    a, b, _, _, res = fused_inputs(m, n, k, BF16, 33)
    d = res.cuda()
    capi.hgemm_fused(d, a.cuda(), b.cuda(), residual=d)
    torch.cuda.synchronize()
    check_fused(d, a, b, None, None, res)


def test_residual_with_its_own_pitch_and_full_size_shape(cuda):
    """A residual that is a column block of a wider matrix (ldr > n), at a compute-bound size."""
    from peakgemm_b200 import capi

    m, n, k = 2048, 2048, 2048
    a, b, rs, bias, _ = fused_inputs(m, n, k, BF16, 34)
    g = torch.Generator().manual_seed(35)
    wide = torch.randn(m, n + 64, generator=g).to(BF16)
    wide_d = wide.cuda()
    d = helpers.garbage_like((m, n), BF16, "cuda")
    capi.hgemm_fused(d, a.cuda(), b.cuda(), row_scale=rs.cuda(), bias=bias.cuda(), residual=wide_d[:, 64:])
    torch.cuda.synchronize()
    check_fused(d, a, b, rs, bias, wide[:, 64:])


@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("rows,h", [(1, 8), (7, 136), (333, 4096), (2048, 8192), (64, 14336)])
def test_rstd(cuda, rows, h, dtype):
    from peakgemm_b200 import capi

    x, _, _ = oracle.rmsnorm_inputs(rows, h, dtype, 36)
    rstd = torch.full((rows,), float("nan"), device="cuda")
    capi.rmsnorm_rstd(rstd, x.cuda(), 1e-6)
    torch.cuda.synchronize()
    ref = oracle.rmsnorm_rstd(x, 1e-6)
    rel = ((rstd.cpu().double() - ref).abs() / ref).max().item()
    assert rel <= 1e-5, rel


@pytest.mark.parametrize("m,n,k", [(16, 4096, 4096), (128, 4096, 4096), (1024, 4096, 4096), (300, 520, 1000)])
def test_rms_norm_linear_matches_the_definition(cuda, m, n, k):
    """RMSNorm + projection as one GEMM over the raw activations (gamma folded into the weights), against the
    unfolded definition; and the two-operator chain (rms_norm_fwd, gemm_peak) measured against the same oracle."""
    import PeakGemm

    g = torch.Generator().manual_seed(37)
    x = torch.randn(m, k, generator=g).to(BF16)
    gamma = 1 + 0.1 * torch.randn(k, generator=g)
    w = (0.02 * torch.randn(n, k, generator=g)).to(BF16)
    ref = oracle.rmsnorm_linear(x, gamma, w, 1e-6)
    tol = oracle.gemm_tolerance(k, ref, BF16)

    xd, wd, gd = x.cuda(), w.cuda(), gamma.cuda()
    wf = PeakGemm.fold_gamma(wd, gd)
    out_pdl = helpers.garbage_like((m, n), BF16, "cuda")
    out_plain = helpers.garbage_like((m, n), BF16, "cuda")
    rstd = PeakGemm.rms_norm_linear(out_pdl, xd, wf, 1e-6, pdl=True)
    PeakGemm.rms_norm_linear(out_plain, xd, wf, 1e-6, pdl=False)
    y = torch.empty_like(xd)
    two_step = helpers.garbage_like((m, n), BF16, "cuda")
    PeakGemm.rms_norm_fwd(y, xd, gd, 1e-6)
    PeakGemm.gemm_peak(two_step, y, wd)
    torch.cuda.synchronize()

    assert torch.equal(out_pdl.view(torch.int16), out_plain.view(torch.int16))
    rel = ((rstd.cpu().double() - oracle.rmsnorm_rstd(x)).abs() / oracle.rmsnorm_rstd(x)).max().item()
    assert rel <= 1e-5
    err_fused = (out_pdl.float().cpu() - ref).abs().max().item()
    err_two = (two_step.float().cpu() - ref).abs().max().item()
    assert err_fused <= tol and err_two <= tol, (err_fused, err_two, tol)
    # one rounding less than the two-operator chain: never much worse than it
    assert err_fused <= 2.0 * err_two + 2.0 ** -8 * ref.abs().max().item()


def test_overlapped_launch_never_reads_stale_row_scales(cuda):
    """The GEMM launched with programmatic serialisation behind the rstd kernel may start early; its epilogue
    must still see the NEW rstd.  The same rstd buffer is reused for inputs of very different scale, so a
    stale read would be off by the ratio of the scales."""
    import PeakGemm

    m, n, k = 64, 2048, 2048
    g = torch.Generator().manual_seed(38)
    w = (0.02 * torch.randn(n, k, generator=g)).to(BF16).cuda()
    xs = [(torch.randn(m, k, generator=g) * (4.0 ** (i % 5))).to(BF16).cuda() for i in range(20)]
    rstd = torch.zeros(m, device="cuda")
    outs = [torch.empty(m, n, dtype=BF16, device="cuda") for _ in xs]
    for x, o in zip(xs, outs):                       # back to back, no synchronisation in between
        PeakGemm.rms_norm_linear(o, x, w, 1e-6, rstd=rstd, pdl=True)
    torch.cuda.synchronize()
    for x, o in zip(xs, outs):
        ref = torch.empty_like(o)
        PeakGemm.rms_norm_linear(ref, x, w, 1e-6, pdl=False)
        torch.cuda.synchronize()
        assert torch.equal(o.view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("m,n,k", [(16, 4096, 1024), (128, 4096, 4096), (512, 1024, 512)])
def test_overlapped_launch_flag_without_a_producer_kernel(cuda, m, n, k):
    """PG_FUSED_PDL on an idle stream, or behind a kernel that never releases its dependents early, degrades to
    an ordinary launch: same bits as without the flag, on the skinny, split-K and persistent kernels."""
    from peakgemm_b200 import capi

    a, b, rs, _, _ = fused_inputs(m, n, k, BF16, 41)
    ad, bd, rsd = a.cuda(), b.cuda(), rs.cuda()
    plain = helpers.garbage_like((m, n), BF16, "cuda")
    idle = helpers.garbage_like((m, n), BF16, "cuda")
    behind = helpers.garbage_like((m, n), BF16, "cuda")
    capi.hgemm_fused(plain, ad, bd, row_scale=rsd)
    torch.cuda.synchronize()
    capi.hgemm_fused(idle, ad, bd, row_scale=rsd, pdl=True)
    torch.cuda.synchronize()
    rsd2 = torch.zeros_like(rsd)
    rsd2.copy_(rsd)                                   # an ordinary kernel writes the scales just before
    capi.hgemm_fused(behind, ad, bd, row_scale=rsd2, pdl=True)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    assert torch.equal(plain.view(torch.int16), idle.view(torch.int16))
    assert torch.equal(plain.view(torch.int16), behind.view(torch.int16))


@pytest.mark.parametrize("pdl", [False, True])
def test_cuda_graph_replay_of_norm_gemm_chains(cuda, pdl):
    """Both chains are capturable (no allocation, no synchronisation, nothing host-side per call that
    depends on the data) and a replay on new inputs equals the eager result bit for bit."""
    import PeakGemm

    m, n, k = 256, 1024, 2048
    g = torch.Generator().manual_seed(39)
    gamma = (1 + 0.1 * torch.randn(k, generator=g)).cuda()
    w = (0.02 * torch.randn(n, k, generator=g)).to(BF16).cuda()
    wf = PeakGemm.fold_gamma(w, gamma)
    x = torch.randn(m, k, generator=g).to(BF16).cuda()
    y = torch.empty_like(x)
    rstd = torch.empty(m, device="cuda")
    out_two = torch.empty(m, n, dtype=BF16, device="cuda")
    out_fused = torch.empty(m, n, dtype=BF16, device="cuda")

    def chain():
        PeakGemm.rms_norm_fwd(y, x, gamma, 1e-6)
        PeakGemm.gemm_peak(out_two, y, w)
        PeakGemm.rms_norm_linear(out_fused, x, wf, 1e-6, rstd=rstd, pdl=pdl)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain()                                       # per-device set-up happens outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        chain()
    x.copy_(torch.randn(m, k, generator=g).to(BF16))  # new contents, same addresses
    graph.replay()
    torch.cuda.synchronize()
    replay_two, replay_fused = out_two.clone(), out_fused.clone()
    out_two.zero_()
    out_fused.zero_()
    chain()
    torch.cuda.synchronize()
    assert torch.equal(replay_two.view(torch.int16), out_two.view(torch.int16))
    assert torch.equal(replay_fused.view(torch.int16), out_fused.view(torch.int16))


def test_annotated_operators_survive_tracing(cuda):
    """torch.compile (aot_eager: trace + functionalise, no code generation) keeps the annotated operators
    and their writes; the result equals eager execution.  This tests the schemas and fake implementations,
    not a compiled hot path."""
    import PeakGemm  # noqa: F401

    m, n, k = 128, 512, 1024
    g = torch.Generator().manual_seed(40)
    x = torch.randn(m, k, generator=g).to(BF16).cuda()
    w = (0.02 * torch.randn(n, k, generator=g)).to(BF16).cuda()
    bias = torch.randn(n, generator=g).to(BF16).cuda()

    def f(x, w, bias):
        rstd = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
        out = torch.empty(x.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
        plain = torch.empty_like(out)
        torch.ops.PeakGemm.rms_norm_rstd(rstd, x, 1e-6)
        torch.ops.PeakGemm.gemm_peak_fused(out, x, w, rstd, bias, None, False)
        torch.ops.PeakGemm.gemm_peak_out(plain, x, w)
        return out, plain

    eager = f(x, w, bias)
    traced = torch.compile(f, backend="aot_eager", fullgraph=True)(x, w, bias)
    torch.cuda.synchronize()
    for e, t in zip(eager, traced):
        assert torch.equal(e.view(torch.int16), t.view(torch.int16))


def test_fused_operator_argument_errors(cuda):
    import PeakGemm

    a = torch.zeros(64, 128, dtype=BF16, device="cuda")
    b = torch.zeros(32, 128, dtype=BF16, device="cuda")
    d = torch.zeros(64, 32, dtype=BF16, device="cuda")
    with pytest.raises(RuntimeError, match="row_scale"):
        PeakGemm.gemm_peak_fused(d, a, b, row_scale=torch.zeros(63, device="cuda"))
    with pytest.raises(RuntimeError, match="bias"):
        PeakGemm.gemm_peak_fused(d, a, b, bias=torch.zeros(32, device="cuda"))          # float32 bias
    with pytest.raises(RuntimeError, match="residual"):
        PeakGemm.gemm_peak_fused(d, a, b, residual=torch.zeros(64, 32, dtype=F16, device="cuda"))
    with pytest.raises(RuntimeError, match="bias"):
        PeakGemm.gemm_peak_fused(d, a, b, bias=torch.zeros(32, dtype=BF16))               # a CPU tensor
