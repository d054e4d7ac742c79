"""PeakGemm for B200: the reference project's PyTorch operator surface over sm_100a kernels.

Host-side mirror of the reference's ``PeakGemm/__init__.py`` (lines 10-34): the
torch extension ``libPeakGemm.so`` is loaded with ``torch.ops.load_library`` and
``gemm_peak(c, a, b)`` does the same shape plumbing before calling
``torch.ops.PeakGemm.gemm_peak(c, a, b, m, n, k)``.  ``rms_norm_fwd`` and
``rms_norm_bwd`` are additions that follow the same conventions (the reference
has no RMSNorm).

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


__all__ = ["gemm_peak", "rms_norm_fwd", "rms_norm_bwd", "TORCH_LIB_PATH", "DEVICE_LIB_PATH"]
