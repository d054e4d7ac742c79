"""CPU: the oracle against the reference's golden outputs, against first principles, and against torch."""
import os

import numpy as np
import pytest
import torch

import oracle
from tests import helpers

GOLD = os.path.join(helpers.GOLDEN, "gemm_reference_outputs.npz")
DT = {"bf16": torch.bfloat16, "f16": torch.float16}


def _golden():
    assert os.path.exists(GOLD), "tests/golden/gemm_reference_outputs.npz missing (tests/golden/make_golden.py)"
    return np.load(GOLD)


def _cases(kind):
    g = _golden()
    for key in g.files:
        if key.startswith(kind + "_"):
            dt, shape = key[len(kind) + 1:].split("_")
            m, n, k = (int(v) for v in shape.split("x"))
            yield key, DT[dt], m, n, k


def test_golden_inputs_regenerate():
    g = _golden()
    seed = int(g["seed"])
    n_checked = 0
    for key, dt, m, n, k in _cases("a_head"):
        a, _ = oracle.gemm_inputs_uniform(m, n, k, dt, seed)
        head = a.view(torch.int16).numpy().view(np.uint16).ravel()[:64]
        assert np.array_equal(head, g[key]), key
        n_checked += 1
    assert n_checked == 6


def test_oracle_bit_exact_with_reference_naive_kernel():
    """gemm_exact reproduces sgemm::sgemm_naive<T> as run on a B200, bit for bit, for every golden case."""
    g = _golden()
    seed = int(g["seed"])
    n_checked = 0
    for key, dt, m, n, k in _cases("naive"):
        a, b = oracle.gemm_inputs_uniform(m, n, k, dt, seed)
        mine = oracle.gemm_exact(a, b).view(torch.int16).numpy().view(np.uint16)
        assert np.array_equal(mine, g[key]), key
        n_checked += 1
    assert n_checked == 6


def test_reference_hgemm_kernel_within_its_own_bound_of_the_oracle():
    """hgemm::hgemm_peak's golden outputs sit within 0.5*k/4096 (test_gemm_half.cpp:158,167) of the oracle,
    and within the acceptance bound our kernel is held to."""
    g = _golden()
    seed = int(g["seed"])
    for key, dt, m, n, k in _cases("hgemm"):
        a, b = oracle.gemm_inputs_uniform(m, n, k, dt, seed)
        ref_out = torch.from_numpy(g[key].view(np.int16).copy()).view(dt).float()
        exact = oracle.gemm_exact(a, b).float()
        fp32 = oracle.gemm_fp32(a, b)
        assert (ref_out - exact).abs().max().item() <= max(oracle.reference_abs_tolerance(k),
                                                           oracle.gemm_tolerance(k, fp32, dt)), key
        assert (ref_out - fp32).abs().max().item() <= oracle.gemm_tolerance(k, fp32, dt), key


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_gemm_exact_is_the_k_ordered_fp32_loop(dt):
    """Against a literal transcription of the reference formula in numpy float32 scalars."""
    a, b = oracle.gemm_inputs_uniform(5, 7, 40, dt, 3)
    af, bf = a.float().numpy(), b.float().numpy()
    acc = oracle.gemm_exact_acc(a, b).numpy()
    for i in range(5):
        for j in range(7):
            s = np.float32(0)
            for kk in range(40):
                s = np.float32(s + np.float32(af[i, kk] * bf[j, kk]))
            assert s == acc[i, j]
    assert torch.equal(oracle.gemm_exact(a, b), torch.from_numpy(acc).to(dt))


def test_gemm_exact_edge_shapes():
    for (m, n, k) in [(1, 8, 8), (3, 16, 0), (0, 8, 8), (2, 8, 24)]:
        a, b = oracle.gemm_inputs_uniform(m, n, k, torch.bfloat16, 1)
        c = oracle.gemm_exact(a, b)
        assert c.shape == (m, n)
        if k == 0:
            assert (c == 0).all()


def test_config1_exact_vs_fp32_matmul():
    """benchmark config 1 on the CPU: the two forms of the oracle agree far inside the acceptance bound."""
    a, b = oracle.gemm_inputs_uniform(2048, 2048, 2048, torch.bfloat16, 0)
    exact = oracle.gemm_exact_acc(a, b)
    fast = oracle.gemm_fp32(a, b)
    assert abs(float(fast.abs().max()) - 81.44) < 0.5          # max|C| of this seed: pins the input generator
    assert (exact - fast).abs().max().item() < 1e-3 * oracle.gemm_tolerance(2048, fast)


def test_tolerance_has_an_output_rounding_floor():
    ref = torch.tensor([[100.0]])
    assert oracle.gemm_tolerance(8, ref, torch.bfloat16) >= 100.0 * 2 ** -8
    assert oracle.gemm_tolerance(4096, ref, torch.float16) == pytest.approx(2.0 + 100.0 * 2 ** -11)


# ------------------------------------------------------------------ RMSNorm ----

def test_rmsnorm_oracle_matches_torch_autograd():
    x, dy, gamma = oracle.rmsnorm_inputs(37, 1000, torch.bfloat16, 3)
    xf = x.float().requires_grad_(True)
    gf = gamma.clone().requires_grad_(True)
    y = torch.nn.functional.rms_norm(xf, (1000,), gf, 1e-6)
    y.backward(dy.float())
    assert torch.allclose(oracle.rmsnorm_fwd(x, gamma), y.detach(), rtol=2e-6, atol=1e-6)
    dx, dg = oracle.rmsnorm_bwd(dy, x, gamma)
    assert torch.allclose(dx, xf.grad, rtol=1e-4, atol=2e-6)
    assert torch.allclose(dg, gf.grad, rtol=1e-5, atol=1e-5)


def test_rmsnorm_oracle_matches_float64():
    x, dy, gamma = oracle.rmsnorm_inputs(16, 512, torch.float16, 4)
    xd, dyd, gd = x.double().numpy(), dy.double().numpy(), gamma.double().numpy()
    rstd = 1.0 / np.sqrt((xd ** 2).mean(-1, keepdims=True) + 1e-6)
    xhat = xd * rstd
    g = dyd * gd
    dx64 = rstd * (g - xhat * (g * xhat).mean(-1, keepdims=True))
    dx, dg = oracle.rmsnorm_bwd(dy, x, gamma)
    slack = oracle.rmsnorm_bwd_dx_slack(dy, x, gamma).numpy()
    assert (np.abs(dx.numpy() - dx64) <= slack + 1e-7 * np.abs(dx64)).all()
    assert np.allclose(dg.numpy(), (dyd * xhat).sum(0), rtol=1e-5, atol=1e-5)
    assert np.allclose(oracle.rmsnorm_fwd(x, gamma).numpy(), xhat * gd, rtol=1e-5, atol=1e-6)


def test_ulp_distance():
    a = torch.tensor([1.0, -1.0, 0.0, 3.0]).to(torch.bfloat16)
    up = torch.tensor([1.0078125, -1.0078125, 0.0, 3.0])
    assert oracle.ulp_distance_16(a, up).tolist() == [1, 1, 0, 0]
    z = torch.tensor([0.0]).to(torch.bfloat16)
    tiny = torch.tensor([-9.1835e-41])      # smallest negative bf16 subnormal
    assert oracle.ulp_distance_16(z, tiny).item() == 1
    assert oracle.within_ulp_or_slack(a, up + 1e-3, torch.full((4,), 2e-3)).all()


def test_input_generators_are_seeded():
    a1, b1 = oracle.gemm_inputs_llm(16, 64, 64, torch.bfloat16, 2)
    a2, b2 = oracle.gemm_inputs_llm(16, 64, 64, torch.bfloat16, 2)
    assert torch.equal(a1, a2) and torch.equal(b1, b2)
    assert b1.float().std() < 0.03 and 0.8 < a1.float().std() < 1.2
    x, dy, g = oracle.rmsnorm_inputs(8, 64, torch.bfloat16, 3)
    assert g.dtype == torch.float32 and abs(float(g.mean()) - 1.0) < 0.1 and not torch.equal(x, dy)


def test_checker_rejects_a_truncating_epilogue_and_a_lost_product():
    """The per-element check of tests/helpers.py:check_gemm is not vacuous: a correctly rounded product passes, the
    same sums truncated toward zero fail, and so does a product with ONE term of every sum dropped, although both stay
    inside the global acceptance bound."""
    from tests import helpers

    a, b = oracle.gemm_inputs_uniform(96, 80, 2048, torch.bfloat16, 0)
    acc = oracle.gemm_exact_acc(a, b)
    helpers.check_gemm(oracle.gemm_fp32(a, b).to(torch.bfloat16), a, b, exact_rows=True)
    truncated = (acc.view(torch.int32) & ~0xFFFF).view(torch.float32).to(torch.bfloat16)
    tol = oracle.gemm_tolerance(2048, acc)
    assert (truncated.float() - acc).abs().max().item() <= tol          # the loose bound alone would accept it
    with pytest.raises(AssertionError):
        helpers.check_gemm(truncated, a, b, exact_rows=True)
    a_lost = a.clone()
    a_lost[:, 17] = 0                                                       # one product of 2048 missing per element
    lost = oracle.gemm_fp32(a_lost, b).to(torch.bfloat16)
    assert (lost.float() - acc).abs().max().item() <= tol
    with pytest.raises(AssertionError):
        helpers.check_gemm(lost, a, b, exact_rows=True)
