"""PeakGemm for B200: the reference project's PyTorch operator surface over sm_100a kernels.

Host-side mirror of the reference's ``PeakGemm/__init__.py`` (lines 10-34): the
torch extension ``libPeakGemm.so`` is loaded with ``torch.ops.load_library`` and
``gemm_peak(c, a, b)`` does the same shape plumbing before calling
``torch.ops.PeakGemm.gemm_peak(c, a, b, m, n, k)``.  ``rms_norm_fwd`` and
``rms_norm_bwd`` are additions that follow the same conventions (the reference
has no RMSNorm).

Callers either side of the GEMM (none of this exists in the reference, whose
epilogue is a plain cast and whose schema is not annotated):

* ``gemm_peak_fused``: row scale, bias and residual folded into the GEMM epilogue;
* ``fold_gamma`` + ``rms_norm_linear``: RMSNorm followed by a projection as ONE
  GEMM over the raw activations (rstd applied per row in the epilogue);
* ``torch.ops.PeakGemm.*_out`` / ``gemm_peak_fused`` / ``rms_norm_rstd``: schemas
  that mark the written tensors, with fake implementations registered here, so
  the operators survive ``torch.compile`` tracing and functionalisation.

There is no CPU or library fallback: importing this package without the built
extension raises ImportError, and the operators raise on non-CUDA tensors.
"""
from __future__ import annotations

import os

import torch

_this_dir = os.path.dirname(os.path.abspath(__file__))
TORCH_LIB_PATH = os.path.join(_this_dir, "libPeakGemm.so")
DEVICE_LIB_PATH = os.path.join(_this_dir, "libPeakGemm_device.so")

if not (os.path.exists(TORCH_LIB_PATH) and os.path.exists(DEVICE_LIB_PATH)):
    raise ImportError(
        "peakgemm_b200: libPeakGemm.so / libPeakGemm_device.so are not built; "
        "run `python peakgemm_b200/csrc/build.py` (needs nvcc and g++)"
    )
if os.environ.get("PEAKGEMM_VERBOSE"):
    print("Loading extension from:", TORCH_LIB_PATH)   # the reference prints this unconditionally
torch.ops.load_library(TORCH_LIB_PATH)

_gemm_peak = torch.ops.PeakGemm.gemm_peak
_rms_norm_fwd = torch.ops.PeakGemm.rms_norm_fwd
_rms_norm_bwd = torch.ops.PeakGemm.rms_norm_bwd


def gemm_peak(c: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> None:
    """c[..., n] = a[..., k] @ b[n, k]^T, fp32 accumulation, written into ``c`` in place.

    Same contract as the reference wrapper (PeakGemm/__init__.py:21-34): leading
    dimensions of ``a`` and ``c`` are flattened, ``b`` is stored ``[n, k]``,
    nothing is returned.  float16 / bfloat16 run on the tcgen05 kernels; float32 runs on
    a plain fp32 FFMA kernel, as in the reference (its unoptimised sgemm path).
    """
    assert a.dtype in [torch.float, torch.half, torch.bfloat16]
    k = a.shape[-1]
    a = a.view(-1, k)
    m = a.shape[0]
    n = b.shape[0]
    assert b.shape[1] == k
    c = c.view(-1, n)
    assert c.shape[0] == m
    _gemm_peak(c, a, b, m, n, k)


def rms_norm_fwd(y: torch.Tensor, x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> None:
    """y = x * rsqrt(mean(x^2, -1) + eps) * gamma, fp32 arithmetic, written into ``y`` in place.

    x, y: [..., h] float16/bfloat16; gamma: [h] float32.
    """
    assert x.dtype in [torch.half, torch.bfloat16]
    h = x.shape[-1]
    assert gamma.shape == (h,)
    _rms_norm_fwd(y.view(-1, h), x.view(-1, h), gamma, eps)


def rms_norm_bwd(dx: torch.Tensor, dgamma: torch.Tensor, dy: torch.Tensor, x: torch.Tensor,
                 gamma: torch.Tensor, eps: float = 1e-6) -> None:
    """Gradients of rms_norm_fwd, written into ``dx`` ([..., h], x's dtype) and ``dgamma`` ([h] float32).

    rstd is recomputed from ``x``; dgamma is summed over all rows in fp32 in a fixed order.
    """
    assert x.dtype in [torch.half, torch.bfloat16]
    h = x.shape[-1]
    assert gamma.shape == (h,) and dgamma.shape == (h,)
    _rms_norm_bwd(dx.view(-1, h), dgamma, dy.view(-1, h), x.view(-1, h), gamma, eps)


def gemm_peak_fused(d: torch.Tensor, a: torch.Tensor, b: torch.Tensor, *, row_scale: torch.Tensor | None = None,
                    bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                    pdl: bool = False) -> None:
    """d[..., n] = row_scale[..., None] * (a[..., k] @ b[n, k]^T) + bias[n] + residual[..., n], in place.

    Every term is optional.  The sum is formed in fp32 from the fp32 accumulator and rounded once.
    ``row_scale`` is float32 with one entry per row of ``a``; ``bias`` and ``residual`` have a's dtype;
    ``residual`` may be ``d`` itself.  ``pdl``: see ``rms_norm_linear``.
    """
    assert a.dtype in [torch.half, torch.bfloat16]
    k = a.shape[-1]
    n = b.shape[0]
    assert b.shape[1] == k
    a2 = a.view(-1, k)
    d2 = d.view(-1, n)
    assert d2.shape[0] == a2.shape[0]
    rs = row_scale.view(-1) if row_scale is not None else None
    res = residual.view(-1, n) if residual is not None else None
    torch.ops.PeakGemm.gemm_peak_fused(d2, a2, b, rs, bias, res, pdl)


def fold_gamma(w: torch.Tensor, gamma: torch.Tensor) -> torch.Tensor:
    """Weights with RMSNorm's gain folded in: w'[n, k] = round(w[n, k] * gamma[k]).  Done once per weight."""
    assert w.shape[1] == gamma.shape[0]
    return (w.float() * gamma.float()[None, :]).to(w.dtype)


def rms_norm_linear(out: torch.Tensor, x: torch.Tensor, w_folded: torch.Tensor, eps: float = 1e-6, *,
                    bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                    rstd: torch.Tensor | None = None, pdl: bool = True) -> torch.Tensor:
    """out = rms_norm(x; gamma) @ w^T (+ bias + residual) with ``w_folded = fold_gamma(w, gamma)``.

    Two launches: ``rms_norm_rstd`` (reads x once, writes one float per row) and one GEMM over the RAW x
    whose epilogue multiplies each row by its rstd.  The normalised activations are never materialised,
    so against ``rms_norm_fwd`` + ``gemm_peak`` this saves one write and one read of x's size and rounds
    once less (gamma is rounded into the weights instead of x*rstd*gamma into y).  With ``pdl`` the GEMM
    is launched with programmatic stream serialisation: its main loop overlaps the rstd kernel and only
    its epilogue waits for rstd.  Returns the rstd tensor (float32, one entry per row).
    """
    k = x.shape[-1]
    x2 = x.view(-1, k)
    if rstd is None:
        rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    torch.ops.PeakGemm.rms_norm_rstd(rstd, x2, eps)
    gemm_peak_fused(out, x, w_folded, row_scale=rstd, bias=bias, residual=residual, pdl=pdl)
    return rstd


def _register_fakes() -> None:
    """Fake (meta) implementations: every annotated operator only writes into tensors it is given."""
    def _nothing(*args, **kwargs):
        return None

    for name in ("gemm_peak_out", "rms_norm_fwd_out", "rms_norm_bwd_out", "rms_norm_rstd", "gemm_peak_fused"):
        torch.library.register_fake(f"PeakGemm::{name}")(_nothing)


_register_fakes()

__all__ = ["gemm_peak", "rms_norm_fwd", "rms_norm_bwd", "gemm_peak_fused", "fold_gamma", "rms_norm_linear",
           "TORCH_LIB_PATH", "DEVICE_LIB_PATH"]
