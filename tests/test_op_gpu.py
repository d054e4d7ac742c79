"""The torch operator surface on the GPU: same calls as the reference's test/test_gemm.py:24-42."""
import pytest
import torch

import oracle
from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_peak_like_reference_test(cuda, dtype):
    import PeakGemm

    m = n = k = 1024
    a, b = oracle.gemm_inputs_uniform(m, n, k, dtype, 21)
    c = torch.randn((m, n), dtype=dtype, device="cuda")      # pre-filled, as create_outputs() does
    assert PeakGemm.gemm_peak(c, a.cuda(), b.cuda()) is None
    torch.cuda.synchronize()
    helpers.check_gemm(c, a, b)


def test_gemm_peak_flattens_leading_dims(cuda):
    import PeakGemm

    a, b = oracle.gemm_inputs_uniform(4 * 96, 256, 512, torch.bfloat16, 22)
    c = torch.empty(4, 96, 256, dtype=torch.bfloat16, device="cuda")
    PeakGemm.gemm_peak(c, a.cuda().view(4, 96, 512), b.cuda())
    torch.cuda.synchronize()
    helpers.check_gemm(c.view(-1, 256), a, b)


def test_op_runs_on_current_stream_and_raw_op(cuda):
    a, b = oracle.gemm_inputs_uniform(256, 256, 256, torch.float16, 23)
    c = torch.empty(256, 256, dtype=torch.float16, device="cuda")
    s = torch.cuda.Stream()
    ad, bd = a.cuda(), b.cuda()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        torch.ops.PeakGemm.gemm_peak(c, ad, bd, 256, 256, 256)
    s.synchronize()
    helpers.check_gemm(c, a, b)


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (300, 200, 1000), (1, 8, 4), (1024, 1024, 2048), (130, 132, 36)])
def test_gemm_peak_float32_branch(cuda, m, n, k):
    """The operator's float branch (the reference's sgemm_peak): fp32 FMA accumulation, absolute bound 1e-4 * k/4096
    floor 1e-4 as in test/cpp/test_gemm_float.cpp:151, against a float64 product of the same inputs."""
    import PeakGemm

    g = torch.Generator().manual_seed(50)
    a = torch.rand(m, k, generator=g) * 2 - 1
    b = torch.rand(n, k, generator=g) * 2 - 1
    c = torch.randn(m, n, device="cuda")
    PeakGemm.gemm_peak(c, a.cuda(), b.cuda())
    torch.cuda.synchronize()
    ref = (a.double() @ b.double().t())
    err = (c.cpu().double() - ref).abs().max().item()
    assert err <= 1e-4 * max(1.0, k / 1024), err


def test_op_errors(cuda):
    import PeakGemm

    a = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        PeakGemm.gemm_peak(torch.zeros(64, 64, dtype=torch.float16, device="cuda"), a, a)   # dtype mismatch
    with pytest.raises(AssertionError):
        PeakGemm.gemm_peak(a.double(), a.double(), a.double())        # the wrapper's dtype assert (__init__.py:26)
    with pytest.raises(RuntimeError):
        torch.ops.PeakGemm.gemm_peak(a.double(), a.double(), a.double(), 64, 64, 64)         # fp64 not built
    with pytest.raises(RuntimeError):
        PeakGemm.gemm_peak(a, a.t(), a)                                                      # not contiguous
    with pytest.raises(RuntimeError):
        torch.ops.PeakGemm.gemm_peak(a, a, a, 64, 64, 128)                                   # sizes vs m,n,k
    with pytest.raises(RuntimeError):
        PeakGemm.gemm_peak(a.cpu(), a.cpu(), a.cpu())                                        # no CPU path
    b12 = torch.zeros(12, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        PeakGemm.gemm_peak(torch.zeros(64, 12, dtype=torch.bfloat16, device="cuda"), a, b12)  # n % 8


def test_rms_norm_ops(cuda):
    import PeakGemm

    x, dy, gamma = oracle.rmsnorm_inputs(6 * 50, 2048, torch.bfloat16, 24)
    xd = x.cuda().view(6, 50, 2048)
    y = torch.empty_like(xd)
    PeakGemm.rms_norm_fwd(y, xd, gamma.cuda())
    dx = torch.empty_like(xd)
    dg = torch.empty(2048, device="cuda")
    PeakGemm.rms_norm_bwd(dx, dg, dy.cuda().view(6, 50, 2048), xd, gamma.cuda())
    torch.cuda.synchronize()
    assert oracle.ulp_distance_16(y.cpu().view(-1, 2048), oracle.rmsnorm_fwd(x, gamma)).max() <= 1
    dx_ref, dg_ref = oracle.rmsnorm_bwd(dy, x, gamma)
    assert oracle.within_ulp_or_slack(dx.cpu().view(-1, 2048), dx_ref, oracle.rmsnorm_bwd_dx_slack(dy, x, gamma)).all()
    assert (dg.cpu() - dg_ref).abs().max() <= 1e-3 * dg_ref.abs().max()


def test_rms_norm_matches_torch_autograd(cuda):
    """Second opinion on the GPU: torch's own fp32 rms_norm and autograd on the same inputs."""
    import PeakGemm

    x, dy, gamma = oracle.rmsnorm_inputs(128, 1024, torch.bfloat16, 25)
    xd, dyd, gd = x.cuda(), dy.cuda(), gamma.cuda()
    xf = xd.float().requires_grad_(True)
    gf = gd.clone().requires_grad_(True)
    yt = torch.nn.functional.rms_norm(xf, (1024,), gf, 1e-6)
    yt.backward(dyd.float())
    y = torch.empty_like(xd)
    dx = torch.empty_like(xd)
    dg = torch.empty_like(gd)
    PeakGemm.rms_norm_fwd(y, xd, gd)
    PeakGemm.rms_norm_bwd(dx, dg, dyd, xd, gd)
    torch.cuda.synchronize()
    assert oracle.ulp_distance_16(y.cpu(), yt.detach().cpu()).max() <= 1
    assert oracle.within_ulp_or_slack(dx.cpu(), xf.grad.cpu(), oracle.rmsnorm_bwd_dx_slack(dy, x, gamma)).all()
    assert (dg - gf.grad).abs().max() <= 1e-3 * gf.grad.abs().max()
