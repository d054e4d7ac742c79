"""ctypes binding of the C ABI in include/peakgemm.h (libPeakGemm_device.so).

This is the binding a non-torch host would write; the tests and the benchmark use
it to call the device library exactly as the torch shim does, with raw device
pointers.  Loading fails loudly if the library has not been built.
"""
from __future__ import annotations

import ctypes
import os

_this_dir = os.path.dirname(os.path.abspath(__file__))
DEVICE_LIB_PATH = os.path.join(_this_dir, "libPeakGemm_device.so")

PG_F16, PG_BF16 = 0, 1
PG_OK = 0
PG_ERR_DEVICE_TIMEOUT = 6

# name -> (restype, argtypes); every symbol include/peakgemm.h declares
_p, _i64, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
SIGNATURES = {
    "pg_status_string": (ctypes.c_char_p, [_i]),
    "pg_last_cuda_error": (_i, []),
    "pg_version": (ctypes.c_char_p, []),
    "pg_hgemm": (_i, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i, _p]),
    "pg_hgemm_ex": (_i, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _p]),
    "pg_hgemm_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "pg_hgemm_ws": (_i, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i, _p, _sz, _p]),
    "pg_hgemm_fused": (_i, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _p, _p, _p, _i64, _i, _i, _p]),
    "pg_rmsnorm_rstd": (_i, [_p, _p, _i64, _i64, ctypes.c_float, _i, _p]),
    "pg_hgemm_multi": (_i, [ctypes.POINTER(_p), _i, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _p]),
    "pg_hgemm_mcast": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _p]),
    "pg_peer_alloc": (_i, [_sz, ctypes.POINTER(_p), _p]),
    "pg_peer_open": (_i, [_p, ctypes.POINTER(_p)]),
    "pg_peer_close": (_i, [_p]),
    "pg_peer_free": (_i, [_p]),
    "pg_peer_last_cuda_error": (_i, []),
    "pg_sgemm": (_i, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _p]),
    "pg_probe_tensor_peak": (_i, [_i, _i, ctypes.POINTER(_f), ctypes.POINTER(_f)]),
    "pg_probe_copy": (_i, [_p, _p, _sz, _p]),
    "pg_hgemm_config": (_i, [_i64, _i64, _i64, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "pg_device_status": (_i, [ctypes.POINTER(_i), _p]),
    "pg_rmsnorm_fwd": (_i, [_p, _p, _p, _i64, _i64, _f, _i, _p]),
    "pg_rmsnorm_bwd_workspace_bytes": (_sz, [_i64, _i64]),
    "pg_rmsnorm_bwd": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _f, _i, _p, _sz, _p]),
    "pg_rmsnorm_bwd_static": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _f, _i, _p]),
}
PG_STATIC_SCRATCH_BYTES = 160 * 8192 * 4

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(DEVICE_LIB_PATH):
            raise ImportError(
                f"{DEVICE_LIB_PATH} is not built; run `python peakgemm_b200/csrc/build.py`"
            )
        l = ctypes.CDLL(DEVICE_LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


class PeakGemmError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().pg_status_string(status).decode()
        super().__init__(f"{where}: {msg} (cuda error {lib().pg_last_cuda_error()})")


def check(status: int, where: str) -> None:
    if status != PG_OK:
        raise PeakGemmError(status, where)


def dtype_code(torch_dtype) -> int:
    import torch

    if torch_dtype == torch.float16:
        return PG_F16
    if torch_dtype == torch.bfloat16:
        return PG_BF16
    raise TypeError(f"unsupported dtype {torch_dtype}")


def _stream_ptr(stream=None):
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def hgemm(c, a, b, *, variant: int = 0, block_n: int = 0, max_sms: int = 0, ldc: int | None = None,
          stream=None) -> None:
    """C[m,n] = A[m,k] @ B[n,k]^T through pg_hgemm_ex on torch CUDA tensors (2-D, row-major)."""
    m, k = a.shape
    n = b.shape[0]
    st = lib().pg_hgemm_ex(c.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, a.stride(0) if m > 1 else k,
                           b.stride(0) if n > 1 else k, ldc if ldc is not None else (c.stride(0) if m > 1 else n),
                           dtype_code(a.dtype), variant, block_n, max_sms, _stream_ptr(stream))
    check(st, "pg_hgemm_ex")


def hgemm_workspace_bytes(m: int, n: int, k: int) -> int:
    """Bytes of scratch with which pg_hgemm_ws splits the last partial wave of this shape (0: it would not)."""
    return int(lib().pg_hgemm_workspace_bytes(m, n, k))


def hgemm_ws(c, a, b, workspace=None, stream=None) -> None:
    """pg_hgemm_ws: C = A @ B^T, with `workspace` (a uint8 CUDA tensor or None) enabling the tail split."""
    m, k = a.shape
    n = b.shape[0]
    st = lib().pg_hgemm_ws(c.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, a.stride(0) if m > 1 else k,
                           b.stride(0) if n > 1 else k, c.stride(0) if m > 1 else n, dtype_code(a.dtype),
                           workspace.data_ptr() if workspace is not None else None,
                           workspace.numel() * workspace.element_size() if workspace is not None else 0,
                           _stream_ptr(stream))
    check(st, "pg_hgemm_ws")


PG_FUSED_PDL = 1


def hgemm_fused(d, a, b, *, row_scale=None, bias=None, residual=None, pdl: bool = False, stream=None) -> None:
    """pg_hgemm_fused: d = round(row_scale[:, None] * (a @ b^T) + bias[None, :] + residual), terms optional."""
    m, k = a.shape
    n = b.shape[0]
    ptr = lambda t: t.data_ptr() if t is not None else None
    ldr = (residual.stride(0) if m > 1 else n) if residual is not None else 0
    st = lib().pg_hgemm_fused(d.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, a.stride(0) if m > 1 else k,
                              b.stride(0) if n > 1 else k, d.stride(0) if m > 1 else n, ptr(row_scale), ptr(bias),
                              ptr(residual), ldr, dtype_code(a.dtype), PG_FUSED_PDL if pdl else 0,
                              _stream_ptr(stream))
    check(st, "pg_hgemm_fused")


def rmsnorm_rstd(rstd, x, eps: float = 1e-6, stream=None) -> None:
    """pg_rmsnorm_rstd: rstd[r] = rsqrt(mean(x[r, :]^2) + eps), float32."""
    rows, h = x.shape
    check(lib().pg_rmsnorm_rstd(rstd.data_ptr(), x.data_ptr(), rows, h, eps, dtype_code(x.dtype),
                                _stream_ptr(stream)), "pg_rmsnorm_rstd")


def hgemm_multi(c_ptrs, a, b, ldc: int, n: int | None = None, *, max_sms: int = 0, stream=None) -> None:
    """pg_hgemm_multi: C block = A @ B^T stored to every device address in c_ptrs (row pitch ldc elements)."""
    m, k = a.shape
    n = b.shape[0] if n is None else n
    arr = (ctypes.c_void_p * len(c_ptrs))(*[ctypes.c_void_p(int(p)) for p in c_ptrs])
    st = lib().pg_hgemm_multi(arr, len(c_ptrs), a.data_ptr(), b.data_ptr(), m, n, k, a.stride(0) if m > 1 else k,
                              b.stride(0) if n > 1 else k, ldc, dtype_code(a.dtype), max_sms, _stream_ptr(stream))
    check(st, "pg_hgemm_multi")


def hgemm_mcast(c_local_ptr: int, c_multicast_ptr: int, a, b, ldc: int, *, max_sms: int = 0, stream=None) -> None:
    """pg_hgemm_mcast: C block = A @ B^T written through a multicast address (replicated by the NVLink switch)."""
    m, k = a.shape
    n = b.shape[0]
    st = lib().pg_hgemm_mcast(ctypes.c_void_p(int(c_local_ptr)), ctypes.c_void_p(int(c_multicast_ptr)), a.data_ptr(),
                              b.data_ptr(), m, n, k, a.stride(0) if m > 1 else k, b.stride(0) if n > 1 else k, ldc,
                              dtype_code(a.dtype), max_sms, _stream_ptr(stream))
    check(st, "pg_hgemm_mcast")


PG_PEER_HANDLE_BYTES = 64


def peer_alloc(nbytes: int) -> tuple[int, bytes]:
    """(device pointer, IPC handle bytes) of a new peer-visible buffer on the current device."""
    ptr = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(PG_PEER_HANDLE_BYTES)
    st = lib().pg_peer_alloc(nbytes, ctypes.byref(ptr), handle)
    if st != PG_OK:
        raise PeakGemmError(st, f"pg_peer_alloc (cuda error {lib().pg_peer_last_cuda_error()})")
    return int(ptr.value), bytes(handle.raw)


def peer_open(handle: bytes) -> int:
    """Maps a peer's buffer for kernels of the CURRENT device; returns the device pointer."""
    ptr = ctypes.c_void_p()
    st = lib().pg_peer_open(ctypes.c_char_p(handle), ctypes.byref(ptr))
    if st != PG_OK:
        raise PeakGemmError(st, f"pg_peer_open (cuda error {lib().pg_peer_last_cuda_error()})")
    return int(ptr.value)


def peer_close(ptr: int) -> None:
    check(lib().pg_peer_close(ctypes.c_void_p(ptr)), "pg_peer_close")


def peer_free(ptr: int) -> None:
    check(lib().pg_peer_free(ctypes.c_void_p(ptr)), "pg_peer_free")


def sgemm(c, a, b, stream=None) -> None:
    """pg_sgemm on float32 torch CUDA tensors (2-D, row-major): C = A @ B^T."""
    m, k = a.shape
    n = b.shape[0]
    check(lib().pg_sgemm(c.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, a.stride(0) if m > 1 else k,
                         b.stride(0) if n > 1 else k, c.stride(0) if m > 1 else n, _stream_ptr(stream)), "pg_sgemm")


def probe_tensor_peak(dtype_is_bf16: bool = True, iters: int = 20000) -> tuple[float, float]:
    """(TFLOP/s, ms) of the back-to-back tcgen05.mma probe on all SM pairs."""
    tf, ms = ctypes.c_float(0), ctypes.c_float(0)
    check(lib().pg_probe_tensor_peak(PG_BF16 if dtype_is_bf16 else PG_F16, iters, ctypes.byref(tf), ctypes.byref(ms)),
          "pg_probe_tensor_peak")
    return tf.value, ms.value


def probe_copy(dst, src, stream=None) -> None:
    check(lib().pg_probe_copy(dst.data_ptr(), src.data_ptr(), src.numel() * src.element_size(), _stream_ptr(stream)),
          "pg_probe_copy")


def hgemm_config(m: int, n: int, k: int, sm_count: int = 148) -> tuple[int, int]:
    """(variant, block_n) pg_hgemm picks for this shape; host arithmetic only."""
    v, bn = ctypes.c_int(0), ctypes.c_int(0)
    check(lib().pg_hgemm_config(m, n, k, sm_count, ctypes.byref(v), ctypes.byref(bn)), "pg_hgemm_config")
    return v.value, bn.value


def device_status(stream=None) -> int:
    out = ctypes.c_int(0)
    st = lib().pg_device_status(ctypes.byref(out), _stream_ptr(stream))
    if st != PG_ERR_DEVICE_TIMEOUT:          # a give-up is reported through the returned code, not as an exception
        check(st, "pg_device_status")
    return out.value


def rmsnorm_fwd(y, x, gamma, eps: float = 1e-6, stream=None) -> None:
    rows, h = x.shape
    check(lib().pg_rmsnorm_fwd(y.data_ptr(), x.data_ptr(), gamma.data_ptr(), rows, h, eps,
                               dtype_code(x.dtype), _stream_ptr(stream)), "pg_rmsnorm_fwd")


def rmsnorm_bwd_workspace_bytes(rows: int, h: int) -> int:
    return int(lib().pg_rmsnorm_bwd_workspace_bytes(rows, h))


def rmsnorm_bwd(dx, dgamma, dy, x, gamma, workspace, eps: float = 1e-6, stream=None) -> None:
    rows, h = x.shape
    check(lib().pg_rmsnorm_bwd(dx.data_ptr(), dgamma.data_ptr(), dy.data_ptr(), x.data_ptr(), gamma.data_ptr(),
                               rows, h, eps, dtype_code(x.dtype), workspace.data_ptr(),
                               workspace.numel() * workspace.element_size(), _stream_ptr(stream)),
          "pg_rmsnorm_bwd")


def rmsnorm_bwd_static(dx, dgamma, dy, x, gamma, eps: float = 1e-6, stream=None) -> None:
    """pg_rmsnorm_bwd_static: the backward pass with the library's built-in scratch (no workspace argument)."""
    rows, h = x.shape
    check(lib().pg_rmsnorm_bwd_static(dx.data_ptr(), dgamma.data_ptr(), dy.data_ptr(), x.data_ptr(),
                                      gamma.data_ptr(), rows, h, eps, dtype_code(x.dtype), _stream_ptr(stream)),
          "pg_rmsnorm_bwd_static")
