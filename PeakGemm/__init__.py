"""Drop-in import name of the reference project: ``import PeakGemm; PeakGemm.gemm_peak(c, a, b)``.

Everything lives in :mod:`peakgemm_b200`; this module only re-exports it under
the package name the reference's callers use (test/test_gemm.py:13,41-42).
"""
from peakgemm_b200 import (  # noqa: F401
    fold_gamma, gemm_peak, gemm_peak_fused, rms_norm_bwd, rms_norm_fwd, rms_norm_linear,
)

__all__ = ["gemm_peak", "rms_norm_fwd", "rms_norm_bwd", "gemm_peak_fused", "fold_gamma", "rms_norm_linear"]
