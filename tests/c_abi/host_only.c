/* Plain C99 client of the C ABI: host-only entry points (no GPU needed) and the
 * behaviour of sddmm_create on a machine without a usable device.  Prints one
 * line per check; exit code 0 when all hold. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "sddmm_b200.h"

static int failures = 0;
#define CHECK(cond, what)                                 \
    do {                                                  \
        const int holds_ = (cond) ? 1 : 0; /* once */      \
        printf("%s: %s\n", holds_ ? "ok" : "FAILED", what); \
        if (!holds_) ++failures;                          \
    } while (0)

int main(int argc, char **argv)
{
    int expect_device = argc > 1 && strcmp(argv[1], "--expect-device") == 0;
    sddmm_mtx_t f = NULL;
    int64_t M = 0, N = 0, nnz = 0;
    char err[256] = "";
    int st = sddmm_gen_open("uniform:64:48:0.1:seed=2", &f, &M, &N, &nnz, err, (int)sizeof(err));
    CHECK(st == SDDMM_OK && M == 64 && N == 48 && nnz == 307, "sddmm_gen_open sizes");
    int32_t *rows = (int32_t *)malloc(sizeof(int32_t) * (size_t)nnz), *cols = (int32_t *)malloc(sizeof(int32_t) * (size_t)nnz);
    float *vals = (float *)malloc(sizeof(float) * (size_t)nnz);
    st = sddmm_mtx_read(f, rows, cols, vals);
    CHECK(st == SDDMM_OK && sddmm_coo_is_row_sorted(nnz, rows) == 1, "sddmm_mtx_read gives a row-sorted matrix");

    int64_t cuts[4], nnz_cuts[4];
    st = sddmm_partition_rows(M, nnz, rows, 3, 8, cuts, nnz_cuts);
    CHECK(st == SDDMM_OK && cuts[0] == 0 && cuts[3] == M && nnz_cuts[0] == 0 && nnz_cuts[3] == nnz &&
              cuts[1] % 8 == 0 && cuts[2] % 8 == 0 && cuts[1] <= cuts[2],
          "sddmm_partition_rows cuts");

    st = sddmm_gen_open("no-such-generator", &f, &M, &N, &nnz, err, (int)sizeof(err));
    CHECK(st == SDDMM_INVALID_ARG && err[0] != 0, "bad generator spec is an error with a message");

    sddmm_handle_t h = NULL;
    st = sddmm_create(&h, 0);
    if (expect_device) {
        CHECK(st == SDDMM_OK && h != NULL, "sddmm_create on a GPU box");
    } else {
        CHECK((st == SDDMM_NO_DEVICE && h == NULL) || st == SDDMM_OK, "sddmm_create without a device reports SDDMM_NO_DEVICE");
    }
    if (h) sddmm_destroy(h);
    CHECK(strcmp(sddmm_status_string(SDDMM_NO_DEVICE), "unknown status") != 0, "sddmm_status_string knows its codes");
    free(rows); free(cols); free(vals);
    return failures ? 1 : 0;
}
