/* A plain C (and, compiled as C++, a plain C++) caller of include/peakgemm.h: includes the header,
 * links libPeakGemm_device.so and makes the calls that need no GPU.  The reference's C++ tests call
 * its kernels without torch in the same way (test/cpp/test_gemm_half.cpp:1-2,115-117).
 * Exit code 0 = every check passed. */
#include <stdio.h>
#include <string.h>

#include "peakgemm.h"

int main(void) {
    int failures = 0;
    int variant = 0, block_n = 0;
    char one[16] = {0};
    if (strcmp(pg_status_string(PG_OK), "PG_OK") != 0) ++failures;
    if (strncmp(pg_status_string(PG_ERR_DEVICE_TIMEOUT), "PG_ERR_DEVICE_TIMEOUT", 21) != 0) ++failures;
    if (pg_version() == NULL) ++failures;
    /* empty problems return before anything touches a device */
    if (pg_hgemm(one, one, one, 0, 64, 64, 64, 64, 64, PG_BF16, NULL) != PG_OK) ++failures;
    if (pg_hgemm(one, one, one, 64, 0, 64, 64, 64, 64, PG_F16, NULL) != PG_OK) ++failures;
    /* argument errors are found on the host */
    if (pg_hgemm(NULL, one, one, 8, 8, 8, 8, 8, 8, PG_BF16, NULL) != PG_ERR_BAD_ARG) ++failures;
    if (pg_hgemm(one, one, one, 8, 12, 8, 8, 8, 12, PG_BF16, NULL) != PG_ERR_UNSUPPORTED) ++failures;
    if (pg_hgemm(one, one, one, 8, 8, 8, 8, 8, 8, 7, NULL) != PG_ERR_BAD_ARG) ++failures;
    if (pg_rmsnorm_fwd(one, one, (const float *)one, 0, 64, 1e-6f, PG_BF16, NULL) != PG_OK) ++failures;
    /* the configuration choice is host arithmetic */
    if (pg_hgemm_config(8192, 8192, 8192, 148, &variant, &block_n) != PG_OK || block_n != 256) ++failures;
    if (PG_STATIC_SCRATCH_BYTES != 160u * 8192u * 4u) ++failures;
    printf("peakgemm.h caller: %d failure(s), variant %d block_n %d\n", failures, variant, block_n);
    return failures;
}
