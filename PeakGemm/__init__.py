"""Drop-in import name of the reference project: ``import PeakGemm; PeakGemm.gemm_peak(c, a, b)``.

Everything lives in :mod:`peakgemm_b200`; this module only re-exports it under
the package name the reference's callers use (test/test_gemm.py:13,41-42).
"""
from peakgemm_b200 import gemm_peak, rms_norm_fwd, rms_norm_bwd  # noqa: F401

__all__ = ["gemm_peak", "rms_norm_fwd", "rms_norm_bwd"]
