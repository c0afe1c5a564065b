/* Host-only code of the library (Matrix Market / docword / binary readers, writers, the col-to-row
 * converter, the row partitioner, the synthetic generators) driven through the C ABI in a build with
 * AddressSanitizer and UndefinedBehaviorSanitizer: tests/test_host_logic.py compiles this file together
 * with csrc/mtx_io.cpp and csrc/gen.cpp under -fsanitize=address,undefined -fno-sanitize-recover=all and
 * runs it.  Includes the inputs the reference's loader mis-parses or runs off the end of
 * (HiPC18/src/sddmm.cu:257-281): truncated files, missing value column, indices out of range. */
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

static void write_text(const char *path, const char *text)
{
    FILE *f = fopen(path, "w");
    if (f) {
        fputs(text, f);
        fclose(f);
    }
}

static int open_status(const char *path, unsigned flags, int64_t *nnz_out)
{
    sddmm_mtx_t f = NULL;
    int64_t M = 0, N = 0, nnz = 0;
    char err[256] = "";
    int st = sddmm_mtx_open_ex(path, flags, &f, &M, &N, &nnz, err, (int)sizeof(err));
    if (st == SDDMM_OK) {
        int32_t *r = (int32_t *)malloc(sizeof(int32_t) * (size_t)(nnz + 1)), *c = (int32_t *)malloc(sizeof(int32_t) * (size_t)(nnz + 1));
        float *v = (float *)malloc(sizeof(float) * (size_t)(nnz + 1));
        st = sddmm_mtx_read(f, r, c, v);
        free(r); free(c); free(v);
    }
    if (nnz_out) *nnz_out = nnz;
    return st;
}

int main(int argc, char **argv)
{
    const char *dir = argc > 1 ? argv[1] : "/tmp";
    char path[512], path2[512];
    int64_t nnz = 0;

    /* well-formed inputs in every accepted form */
    snprintf(path, sizeof(path), "%s/a.mtx", dir);
    write_text(path, "%%MatrixMarket matrix coordinate real general\n% comment\n3 4 5\n1 1 1.5\n1 4 2\n2 2 -3\n3 1 4\n3 3 5e-1\n");
    CHECK(open_status(path, 0, &nnz) == SDDMM_OK && nnz == 5, "general real file");
    write_text(path, "%%MatrixMarket matrix coordinate pattern symmetric\n3 3 3\n1 1\n2 1\n3 2\n");
    CHECK(open_status(path, SDDMM_MTX_EXPAND_SYMMETRIC | SDDMM_MTX_SORT_ROWS, &nnz) == SDDMM_OK && nnz == 5, "pattern symmetric file, expanded and sorted");
    write_text(path, "4\n5\n3\n1 2 7\n3 5 1\n4 1 2\n");
    CHECK(open_status(path, 0, &nnz) == SDDMM_OK && nnz == 3, "headerless docword triples");

    /* malformed inputs: an error code, never a read past the end */
    write_text(path, "%%MatrixMarket matrix coordinate real general\n3 4 5\n1 1 1.5\n1 4 2\n");
    CHECK(open_status(path, 0, NULL) == SDDMM_PARSE_ERROR, "truncated file");
    write_text(path, "%%MatrixMarket matrix coordinate real general\n3 4 2\n1 1\n2 2\n");
    CHECK(open_status(path, 0, NULL) == SDDMM_PARSE_ERROR, "value column missing in a real file");
    write_text(path, "%%MatrixMarket matrix coordinate real general\n3 4 1\n4 1 1.0\n");
    CHECK(open_status(path, 0, NULL) != SDDMM_OK, "row index out of range");
    write_text(path, "%%MatrixMarket matrix coordinate real general\n3 4 1\n0 1 1.0\n");
    CHECK(open_status(path, 0, NULL) != SDDMM_OK, "index 0 in a 1-based file");
    write_text(path, "%%MatrixMarket matrix coordinate real general\n-3 4 1\n1 1 1.0\n");
    CHECK(open_status(path, 0, NULL) != SDDMM_OK, "negative size");
    write_text(path, "");
    CHECK(open_status(path, 0, NULL) != SDDMM_OK, "empty file");
    snprintf(path2, sizeof(path2), "%s/missing.mtx", dir);
    CHECK(open_status(path2, 0, NULL) == SDDMM_IO_ERROR, "missing file");

    /* generators, converter, partitioner, writer and the binary form, end to end */
    sddmm_mtx_t g = NULL;
    int64_t M = 0, N = 0;
    char err[256] = "";
    const char *specs[4] = {"uniform:200:150:0.05:seed=3", "zipf:120:80:2000:seed=4", "rmat:9:8:seed=5", "band:256:8:3:seed=6"};
    for (int s = 0; s < 4; ++s) {
        int st = sddmm_gen_open(specs[s], &g, &M, &N, &nnz, err, (int)sizeof(err));
        CHECK(st == SDDMM_OK && nnz > 0, specs[s]);
        if (st != SDDMM_OK) continue;
        int32_t *r = (int32_t *)malloc(sizeof(int32_t) * (size_t)nnz), *c = (int32_t *)malloc(sizeof(int32_t) * (size_t)nnz);
        float *v = (float *)malloc(sizeof(float) * (size_t)nnz);
        CHECK(sddmm_mtx_read(g, r, c, v) == SDDMM_OK && sddmm_coo_is_row_sorted(nnz, r) == 1, "generated matrix is row-sorted");
        int64_t cuts[9], nz[9];
        CHECK(sddmm_partition_rows(M, nnz, r, 8, 32, cuts, nz) == SDDMM_OK && cuts[8] == M && nz[8] == nnz, "partition into 8");
        CHECK(sddmm_partition_rows_weighted(M, nnz, r, 3, 1, 2.5, cuts, nz) == SDDMM_OK && cuts[3] == M, "weighted partition into 3");
        /* transpose-sort twice gives the matrix back */
        int64_t M2 = M, N2 = N;
        CHECK(sddmm_coo_sort_rows(&M2, &N2, nnz, r, c, v, 1) == SDDMM_OK && M2 == N && N2 == M, "col-to-row conversion (transposing)");
        CHECK(sddmm_coo_sort_rows(&M2, &N2, nnz, r, c, v, 1) == SDDMM_OK && M2 == M && sddmm_coo_is_row_sorted(nnz, r) == 1, "and back");
        snprintf(path, sizeof(path), "%s/g%d.mtx", dir, s);
        snprintf(path2, sizeof(path2), "%s/g%d.bin", dir, s);
        CHECK(sddmm_mtx_write(path, M, N, nnz, r, c, v) == SDDMM_OK, "Matrix Market writer");
        CHECK(sddmm_coo_save_binary(path2, M, N, nnz, r, c, v) == SDDMM_OK, "binary writer");
        int64_t n1 = 0, n2 = 0;
        CHECK(open_status(path, 0, &n1) == SDDMM_OK && n1 == nnz, "text form reads back");
        CHECK(open_status(path2, 0, &n2) == SDDMM_OK && n2 == nnz, "binary form reads back");
        /* a binary file cut short is refused (checksum / size), not read past its end */
        FILE *bf = fopen(path2, "rb");
        if (bf) {
            static char buf[4096];
            size_t got = fread(buf, 1, sizeof(buf), bf);
            fclose(bf);
            snprintf(path, sizeof(path), "%s/cut%d.bin", dir, s);
            FILE *cf = fopen(path, "wb");
            if (cf) {
                fwrite(buf, 1, got > 100 ? got - 37 : got / 2, cf);
                fclose(cf);
                CHECK(open_status(path, 0, NULL) != SDDMM_OK, "truncated binary file is refused");
            }
        }
        free(r); free(c); free(v);
    }
    CHECK(sddmm_gen_open("rmat:99:8", &g, &M, &N, &nnz, err, (int)sizeof(err)) != SDDMM_OK, "absurd generator size is refused");
    CHECK(sddmm_partition_rows(10, 0, NULL, 4, 1, (int64_t[5]){0}, (int64_t[5]){0}) == SDDMM_OK, "partition of an empty matrix");
    return failures ? 1 : 0;
}
