"""GPU parity of the RMSNorm kernels with the fp32 oracle, through the C ABI.

Bounds: y and dx within 1 ulp (of the 16-bit output type) of the fp32 oracle result rounded to that
type — for dx plus the fp32 error bound of its own formula (oracle.rmsnorm_bwd_dx_slack: roundings of the
cancelling subtraction g - xhat*c and the summation error of c), which only matters where dx cancelled to
almost nothing; dgamma within 1e-3 * max|dgamma_ref|.  The reference project has no RMSNorm, so this oracle is
the textbook definition (parity unpinned by the reference).
"""
import pytest
import torch

import oracle
from tests import helpers

pytestmark = pytest.mark.gpu

BF16, F16 = torch.bfloat16, torch.float16


def run_fwd(rows, h, dtype, seed=3, eps=1e-6):
    from peakgemm_b200 import capi

    assert capi.device_status() == 0
    x, _, gamma = oracle.rmsnorm_inputs(rows, h, dtype, seed)
    y = helpers.garbage_like((rows, h), dtype, "cuda")
    capi.rmsnorm_fwd(y, x.cuda(), gamma.cuda(), eps)
    torch.cuda.synchronize()
    ref = oracle.rmsnorm_fwd(x, gamma, eps)
    d = oracle.ulp_distance_16(y.cpu(), ref)
    assert d.max().item() <= 1, f"y off by {d.max().item()} ulp"
    return (d > 0).float().mean().item()


def run_bwd(rows, h, dtype, seed=3, eps=1e-6):
    from peakgemm_b200 import capi

    x, dy, gamma = oracle.rmsnorm_inputs(rows, h, dtype, seed)
    dx = helpers.garbage_like((rows, h), dtype, "cuda")
    dgamma = torch.full((h,), float("nan"), device="cuda")
    ws_bytes = capi.rmsnorm_bwd_workspace_bytes(rows, h)
    assert ws_bytes > 0
    ws = torch.full((ws_bytes // 4,), float("nan"), device="cuda")   # the workspace needs no initialisation
    capi.rmsnorm_bwd(dx, dgamma, dy.cuda(), x.cuda(), gamma.cuda(), ws, eps)
    torch.cuda.synchronize()
    assert capi.device_status() == 0, "a kernel abandoned a bounded wait"
    dx_ref, dg_ref = oracle.rmsnorm_bwd(dy, x, gamma, eps)
    # dx within 1 ulp of the rounded oracle value, or, where g - xhat*c cancels, within the fp32 error bound of
    # the formula (oracle.rmsnorm_bwd_dx_slack).
    ok = oracle.within_ulp_or_slack(dx.cpu(), dx_ref, oracle.rmsnorm_bwd_dx_slack(dy, x, gamma, eps))
    assert ok.all(), f"dx: {(~ok).sum().item()} elements outside 1 ulp + cancellation slack"
    err = (dgamma.cpu() - dg_ref).abs().max().item()
    assert err <= 1e-3 * dg_ref.abs().max().item(), f"dgamma err {err}"


@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("rows,h", [(1, 8), (7, 64), (33, 256), (100, 1000), (257, 4096), (64, 8192),
                                    (19, 5120), (5, 16384), (3, 24576), (1, 2048), (301, 2048), (1000, 3072),
                                    (2000, 5120), (700, 6144), (900, 7168), (600, 7176)])
def test_fwd_shapes(cuda, rows, h, dtype):
    run_fwd(rows, h, dtype)


@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("rows,h", [(1, 8), (7, 64), (33, 256), (100, 1000), (257, 4096), (64, 8192),
                                    (19, 5120), (5, 16384), (3, 24576), (1000, 512), (1, 2048), (301, 2048),
                                    (1000, 3072)])
def test_bwd_shapes(cuda, rows, h, dtype):
    run_bwd(rows, h, dtype)


@pytest.mark.parametrize("h", [4096, 8192])
def test_config4_full_size(cuda, h):
    """benchmark config 4: x [32768, h] bf16, seed 3, eps 1e-6."""
    run_fwd(32768, h, BF16)
    run_bwd(32768, h, BF16)


def test_bwd_deterministic(cuda):
    from peakgemm_b200 import capi

    x, dy, gamma = oracle.rmsnorm_inputs(4096, 4096, BF16, 4)
    xd, dyd, gd = x.cuda(), dy.cuda(), gamma.cuda()
    ws = torch.empty(capi.rmsnorm_bwd_workspace_bytes(4096, 4096) // 4, device="cuda")
    outs = []
    for _ in range(3):
        dx = torch.empty_like(xd)
        dg = torch.empty(4096, device="cuda")
        capi.rmsnorm_bwd(dx, dg, dyd, xd, gd, ws)
        outs.append((dx, dg))
    torch.cuda.synchronize()
    for dx, dg in outs[1:]:
        assert torch.equal(dx, outs[0][0]) and torch.equal(dg, outs[0][1])


def test_rows_zero_and_errors(cuda):
    from peakgemm_b200 import capi

    L = capi.lib()
    dg = torch.full((64,), 5.0, device="cuda")
    assert L.pg_rmsnorm_bwd(None, dg.data_ptr(), None, None, None, 0, 64, 1e-6, 1, None, 0, None) == 0
    torch.cuda.synchronize()
    assert (dg == 0).all()
    x = torch.zeros(4, 64, dtype=BF16, device="cuda")
    g = torch.ones(64, device="cuda")
    assert L.pg_rmsnorm_fwd(x.data_ptr(), x.data_ptr(), g.data_ptr(), 4, 12, 1e-6, 1, None) == 3   # h % 8
    assert L.pg_rmsnorm_fwd(None, x.data_ptr(), g.data_ptr(), 4, 64, 1e-6, 1, None) == 1
    assert L.pg_rmsnorm_bwd(x.data_ptr(), dg.data_ptr(), x.data_ptr(), x.data_ptr(), g.data_ptr(), 4, 64, 1e-6, 1,
                            x.data_ptr(), 16, None) == 4                                           # workspace


def test_scale_invariance(cuda):
    """rms_norm(2x) == rms_norm(x) up to eps: a size-independent property checked at full width."""
    from peakgemm_b200 import capi

    x, _, gamma = oracle.rmsnorm_inputs(512, 8192, BF16, 6)
    xd, gd = x.cuda(), gamma.cuda()
    y1, y2 = torch.empty_like(xd), torch.empty_like(xd)
    capi.rmsnorm_fwd(y1, xd, gd, 0.0)
    capi.rmsnorm_fwd(y2, xd * 2, gd, 0.0)
    torch.cuda.synchronize()
    assert oracle.ulp_distance_16(y1.cpu(), y2.float().cpu()).max().item() <= 1
