"""Generates tests/golden/gemm_reference_outputs.npz — run on a machine with a B200.

    python tests/golden/make_golden.py [out_dir]

The reference project keeps no golden vectors (its tests draw unseeded random inputs), so these are made
by running the reference's OWN kernels, compiled unmodified for sm_100a into oracle/_ref/libref_peakgemm.so
(recipe: oracle/build_oracle.py), on seeded inputs that oracle.gemm_inputs_uniform regenerates bit for bit:

  naive_<dtype>_<m>x<n>x<k>   output bits of sgemm::sgemm_naive<T>   (src/impl/sgemm_impl.h:9-40)
  hgemm_<dtype>_<m>x<n>x<k>   output bits of hgemm::hgemm_peak       (src/impl/hgemm_wmma_impl.h:412-423)

The CPU tests then hold the oracle to them: bit-exact against `naive`, within the reference test's own
bound (0.5 * k / 4096) against `hgemm`.
"""
import ctypes
import os
import sys

import numpy as np
import torch

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, REPO)
import oracle  # noqa: E402

SEED = 77
CASES = [(128, 128, 64), (128, 256, 512), (256, 128, 1024)]
DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16}


def main(out_dir: str) -> None:
    lib = ctypes.CDLL(os.path.join(REPO, "oracle", "_ref", "libref_peakgemm.so"))
    p, u, i = ctypes.c_void_p, ctypes.c_uint, ctypes.c_int
    lib.ref_hgemm_peak.argtypes = [p, p, p, u, u, u, i, p]
    lib.ref_sgemm_naive.argtypes = [p, p, p, i, i, i, i, p]
    out = {}
    for name, dt in DTYPES.items():
        for (m, n, k) in CASES:
            a, b = oracle.gemm_inputs_uniform(m, n, k, dt, SEED)
            ad, bd = a.cuda(), b.cuda()
            for kind in ("naive", "hgemm"):
                c = torch.zeros(m, n, dtype=dt, device="cuda")
                if kind == "naive":
                    r = lib.ref_sgemm_naive(c.data_ptr(), ad.data_ptr(), bd.data_ptr(), m, n, k, int(name == "bf16"), None)
                else:
                    r = lib.ref_hgemm_peak(c.data_ptr(), ad.data_ptr(), bd.data_ptr(), m, n, k, int(name == "bf16"), None)
                assert r == 0, r
                torch.cuda.synchronize()
                out[f"{kind}_{name}_{m}x{n}x{k}"] = c.cpu().view(torch.int16).numpy().view(np.uint16)
            # first words of the inputs, so a change in the generator is noticed
            out[f"a_head_{name}_{m}x{n}x{k}"] = a.view(torch.int16).numpy().view(np.uint16).ravel()[:64].copy()
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "gemm_reference_outputs.npz")
    np.savez_compressed(path, seed=np.int64(SEED), **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
