/*
 * Test-only bridge to the UNMODIFIED reference (isratnisa/SDDMM_GPU).
 *
 * The reference's hot path lives in one translation unit with a main()
 * (HiPC18/src/sddmm.cu, which pulls in util.h and kernel.h).  This file includes
 * that translation unit from where it lies in the read-only reference tree (the
 * build recipe passes its directory with -I; nothing is copied) and exports its
 * functions with C linkage so that the tests can pin oracle/sddmm_oracle.c against the
 * reference itself and the benchmark can time the reference's own CPU SDDMM.
 *
 * Two adaptations, both outside the reference's code:
 *   - main is renamed so that the object can live in a shared library;
 *   - the pre-Volta __shfl_xor its kernel uses (kernel.h:45-46) no longer exists
 *     for sm_70+; it is mapped to __shfl_xor_sync with a full mask.
 * Output goes to oracle/_ref/ only.  This is checker code, never the product.
 */
#include <cuda_runtime.h>
#define __shfl_xor(a, b) __shfl_xor_sync(0xffffffffu, (a), (b))
#define main sddmm_reference_main
#include "sddmm.cu"
#undef main

#include <unistd.h>

static Matrix make_matrix(const int *rows, const int *cols, const float *vals, long nnz,
                          long n_rows, long n_cols)
{
    Matrix S;
    S.n_rows = n_rows;
    S.n_cols = n_cols;
    S.nnz = nnz;
    if (rows) S.rows.assign(rows, rows + nnz);
    if (cols) S.cols.assign(cols, cols + nnz);
    if (vals) S.vals.assign(vals, vals + nnz);
    else S.vals.assign(nnz, 0.0f);
    return S;
}

extern "C" {

/* sddmm_CPU_COO (sddmm.cu:180-200).  Returns the wall seconds of the call,
 * which include the reference's by-value copies of all five vectors. */
double ref_sddmm_cpu_coo(const int *rows, const int *cols, const float *vals, long nnz,
                         long n_rows, long n_cols, const float *W, const float *H, int K,
                         float *P)
{
    k = K;
    Matrix S = make_matrix(rows, cols, vals, nnz, n_rows, n_cols);
    vector<float> Wv(W, W + n_rows * (long)K), Hv(H, H + n_cols * (long)K);
    double t0 = omp_get_wtime();
    sddmm_CPU_COO(S.rows, S.cols, S.vals, Wv, Hv, P, S);
    return omp_get_wtime() - t0;
}

/* Timing form for large inputs: the caller-visible work is nnz_run nonzeros
 * (a prefix), with the same vectors.  nnz_run = 0 measures the by-value copies
 * alone, which the reference's own timer (sddmm.cu:182,:196) leaves out. */
struct RefCooState {
    Matrix S;
    vector<float> W, H;
    vector<float> P;
};
void *ref_coo_state_create(const int *rows, const int *cols, const float *vals, long nnz,
                           long n_rows, long n_cols, const float *W, const float *H, int K)
{
    RefCooState *st = new RefCooState;
    st->S = make_matrix(rows, cols, vals, nnz, n_rows, n_cols);
    st->W.assign(W, W + n_rows * (long)K);
    st->H.assign(H, H + n_cols * (long)K);
    st->P.assign(nnz > 0 ? nnz : 1, 0.0f);
    k = K;
    return st;
}
double ref_coo_state_run(void *state, long nnz_run)
{
    RefCooState *st = (RefCooState *)state;
    Matrix hdr; /* only n_rows, n_cols, nnz are read by sddmm_CPU_COO */
    hdr.n_rows = st->S.n_rows;
    hdr.n_cols = st->S.n_cols;
    hdr.nnz = nnz_run;
    double t0 = omp_get_wtime();
    sddmm_CPU_COO(st->S.rows, st->S.cols, st->S.vals, st->W, st->H, st->P.data(), hdr);
    return omp_get_wtime() - t0;
}
void ref_coo_state_result(void *state, float *P, long n)
{
    RefCooState *st = (RefCooState *)state;
    memcpy(P, st->P.data(), sizeof(float) * n);
}
void ref_coo_state_destroy(void *state) { delete (RefCooState *)state; }

/* sddmm_CPU_CSR (sddmm.cu:153-177); row_ptr over all n_rows + 1 rows. */
void ref_sddmm_cpu_csr(int *row_ptr, int *cols, float *vals, long nnz, long n_rows,
                       long n_cols, const float *W, const float *H, int K, float *P)
{
    k = K;
    Matrix S = make_matrix(NULL, cols, vals, nnz, n_rows, n_cols);
    vector<float> Wv(W, W + n_rows * (long)K), Hv(H, H + n_cols * (long)K);
    sddmm_CPU_CSR(row_ptr, cols, vals, Wv, Hv, P, S);
}

/* make_HTasH (util.h:68-73). */
void ref_make_htash(const float *H, float *H_t, long n, int K)
{
    vector<float> h(H, H + n * (long)K), ht(n * (long)K);
    make_HTasH(h, ht, (int)n, K);
    memcpy(H_t, ht.data(), sizeof(float) * ht.size());
}

/* initial (util.h:75-81). */
void ref_initial(float *X, long n, int K)
{
    vector<float> v(n * (long)K);
    initial(v, n, K);
    memcpy(X, v.data(), sizeof(float) * v.size());
}

/* make_CSR (util.h:131-153).  row_ptr (n_rows + 2) and row_holder (n_rows + 1)
 * must come zero-filled: the reference leaves the tail unwritten.  The row
 * vector gets one padding element because the reference reads rows[nnz]. */
void ref_make_csr(const int *rows, long nnz, long n_rows, int *row_ptr, int *row_holder)
{
    vector<int> r(rows, rows + nnz), c(nnz, 0);
    vector<float> v(nnz, 0.0f);
    r.reserve(nnz + 1);
    r.push_back(-1);
    if (nnz == 0) { row_ptr[0] = 0; row_ptr[1] = 0; return; }
    make_CSR(r, c, v, nnz, n_rows, row_ptr, row_holder);
}

/* TiledMatrix ctor (util.h:52-65) + make_CSR + rewrite_matrix_1D (util.h:267-343),
 * as preprocessing() chains them (sddmm.cu:208,231,233).  panel_rows is the
 * CLI's argv[3] (tile_sizeY = actv_row_size), col_tile its argv[4] (tile_sizeX).
 * Output arrays are sized by the caller as the constructor sizes them. */
int ref_rewrite_matrix_1d(const int *rows, const int *cols, const float *vals, long nnz,
                          long n_rows, long n_cols, int panel_rows, int col_tile,
                          int *t_rows, int *t_cols, float *t_vals, int *tiled_ind,
                          int *lastIdx_tile, int *lastIdx_block_tile, int *active_row,
                          int *n_actv_row, int *sizes /* ntile_c, max_active_block */)
{
    tile_sizeY = panel_rows;
    tile_sizeX = col_tile;
    actv_row_size = panel_rows;
    Matrix S = make_matrix(rows, cols, vals, nnz, n_rows, n_cols);
    /* padding read by the reference one past the end (util.h:143,150,300) */
    S.rows.reserve(nnz + 1); S.cols.reserve(nnz + 1);
    TiledMatrix tS(S, tile_sizeX, tile_sizeY);
    tS.max_active_row = 0;
    tS.nnz = 0;
    vector<int> row_ptr(n_rows + 2, 0), row_holder(n_rows + 1, 0);
    {
        Matrix Sp = S;
        Sp.rows.push_back(-1);
        if (nnz > 0) make_CSR(Sp.rows, Sp.cols, Sp.vals, nnz, n_rows, row_ptr.data(), row_holder.data());
    }
    Matrix Sq = S;
    Sq.cols.push_back(0x7fffffff);
    int mar = rewrite_matrix_1D(Sq, tS, row_ptr.data(), tile_sizeX, row_holder.data());
    memcpy(t_rows, tS.rows.data(), sizeof(int) * nnz);
    memcpy(t_cols, tS.cols.data(), sizeof(int) * nnz);
    memcpy(t_vals, tS.vals.data(), sizeof(float) * nnz);
    memcpy(tiled_ind, tS.tiled_ind.data(), sizeof(int) * nnz);
    memcpy(lastIdx_tile, tS.lastIdx_tile.data(), sizeof(int) * tS.lastIdx_tile.size());
    memcpy(lastIdx_block_tile, tS.lastIdx_block_tile.data(), sizeof(int) * tS.lastIdx_block_tile.size());
    memcpy(active_row, tS.active_row.data(), sizeof(int) * tS.active_row.size());
    memcpy(n_actv_row, tS.n_actv_row.data(), sizeof(int) * tS.n_actv_row.size());
    sizes[0] = tS.ntile_c;
    sizes[1] = tS.max_active_block;
    return mar;
}

/* unsorted_make_CSR (util.h:82-128).  The reference dumps its result to a
 * hard-coded file name in the working directory; workdir is entered first so
 * that the file lands somewhere disposable.  Arrays are rewritten in place. */
int ref_unsorted_make_csr(int *rows, int *cols, float *vals, long nnz, long n_rows,
                          long n_cols, int *row_ptr, const char *workdir)
{
    char old[4096];
    if (!getcwd(old, sizeof(old))) return -1;
    if (chdir(workdir) != 0) return -2;
    unsorted_make_CSR(rows, cols, vals, nnz, n_rows, n_cols, row_ptr);
    if (chdir(old) != 0) return -3;
    return 0;
}

} /* extern "C" */
