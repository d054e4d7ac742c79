// TEST INFRASTRUCTURE — not part of the product.
//
// C entry points around the UNMODIFIED reference headers, which are included from
// where they lie in the reference checkout (-I<reference>/src/common
// -I<reference>/src/impl on the command line; nothing of the reference is copied
// into this repository).  The result, oracle/_ref/libref_peakgemm.so, is the
// reference's own GPU implementation of the path:
//   hgemm::hgemm_peak           src/impl/hgemm_wmma_impl.h:412-423   (mma.sync kernel)
//   sgemm::sgemm_naive<T>       src/impl/sgemm_impl.h:28-40          (its test oracle)
// It is used to pin the CPU oracle and as a same-GPU timing comparator.
//
// The reference kernel loads whole 128x128x16 tiles without bounds checks
// (hgemm_wmma_impl.h:61-84), so callers here only pass m, n multiples of 128 and
// k a multiple of 16 with k >= 48.
#include "sgemm_impl.h"
#include "hgemm_wmma_impl.h"

extern "C" int ref_hgemm_peak(void *c, const void *a, const void *b, unsigned m, unsigned n, unsigned k,
                              int is_bf16, void *stream) {
    if (m % 128 != 0 || n % 128 != 0 || k % 16 != 0 || k < 48) return -1;
    hgemm::hgemm_peak(static_cast<short *>(c), static_cast<const short *>(a), static_cast<const short *>(b), m, n,
                      k, is_bf16 != 0, static_cast<cudaStream_t>(stream));
    return static_cast<int>(cudaGetLastError());
}

extern "C" int ref_sgemm_naive(void *c, const void *a, const void *b, int m, int n, int k, int is_bf16,
                               void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (is_bf16)
        sgemm::sgemm_naive<__nv_bfloat16>(static_cast<__nv_bfloat16 *>(c), static_cast<const __nv_bfloat16 *>(a),
                                          static_cast<const __nv_bfloat16 *>(b), m, n, k, s);
    else
        sgemm::sgemm_naive<__half>(static_cast<__half *>(c), static_cast<const __half *>(a),
                                   static_cast<const __half *>(b), m, n, k, s);
    return static_cast<int>(cudaGetLastError());
}
