/*
 * CPU oracle for the SDDMM hot path.  TEST INFRASTRUCTURE ONLY: this file is
 * the checker the CUDA path is compared with, and the timed CPU baseline of the
 * benchmark.  The product library never links, loads or calls it.
 *
 * Every function restates, in plain C, one function of the reference
 * (isratnisa/SDDMM_GPU); the reference location is cited above each one.
 * Parity is pinned: tests/test_oracle_golden.py compares each function
 * with the reference's own code compiled from its sources (oracle/ref_bridge.cu)
 * and with the fixtures under tests/golden/ that were produced by that code.
 *
 * Deliberate deviations from the reference, all of them outside the arithmetic:
 *   - 64-bit offsets (the reference's `int` row*k overflows for M*K >= 2^31);
 *   - arrays are passed by pointer, not std::vector by value;
 *   - the OpenMP thread count is the caller's choice (the reference forces 28,
 *     HiPC18/src/sddmm.cu:184);
 *   - make_csr / rewrite_matrix_1d never read uninitialised memory: slots past
 *     the number of non-empty rows are defined to be "no row" (the reference
 *     leaves them uninitialised, HiPC18/src/sddmm.cu:205,223).
 * Build with -O3 -fopenmp -ffp-contract=off and without -ffast-math or
 * -march=native so that every product and sum rounds as the reference's does.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

static double now_seconds(void)
{
#ifdef _OPENMP
    return omp_get_wtime();
#else
    return 0.0;
#endif
}

ORACLE_API int oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * HiPC18/src/sddmm.cu:180-200 (sddmm_CPU_COO): one sequential fp32 dot product
 * per nonzero, W and H row-major, result stored UNSCALED in input order
 * (the multiplication by the S value is commented out at :192).
 * Returns the seconds spent in the loop (the region the reference brackets
 * with omp_get_wtime at :182,:196).
 */
ORACLE_API double oracle_sddmm_coo(const int32_t *row_ind, const int32_t *col_ind,
                                   int64_t nnz, const float *W, const float *H,
                                   int k, float *p_ind, int threads)
{
    double t0 = now_seconds();
    if (threads < 1) threads = oracle_max_threads();
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int64_t ind = 0; ind < nnz; ind++) {
        float sm = 0;
        const float *w = W + (int64_t)row_ind[ind] * k;
        const float *h = H + (int64_t)col_ind[ind] * k;
        for (int t = 0; t < k; ++t)
            sm += w[t] * h[t];
        p_ind[ind] = sm;
    }
    return now_seconds() - t0;
}

/*
 * HiPC18/src/sddmm.cu:153-177 (sddmm_CPU_CSR): the same dot product per CSR
 * row, stored SCALED by the S value (:171) -- P = S o (W * H^T).
 * row_ptr has n_rows + 1 entries over ALL rows (empty rows repeat the offset).
 */
ORACLE_API double oracle_sddmm_csr(const int64_t *row_ptr, const int32_t *col_ind,
                                   const float *val_ind, int64_t n_rows,
                                   const float *W, const float *H, int k,
                                   float *p_ind, int threads)
{
    double t0 = now_seconds();
    if (threads < 1) threads = oracle_max_threads();
#pragma omp parallel for num_threads(threads) schedule(dynamic, 64)
    for (int64_t r = 0; r < n_rows; ++r) {
        const float *w = W + r * k;
        for (int64_t ind = row_ptr[r]; ind < row_ptr[r + 1]; ++ind) {
            const float *h = H + (int64_t)col_ind[ind] * k;
            float sm = 0;
            for (int t = 0; t < k; ++t)
                sm += w[t] * h[t];
            p_ind[ind] = sm * val_ind[ind];
        }
    }
    return now_seconds() - t0;
}

/*
 * Scaled COO form: sddmm_CPU_COO's loop (sddmm.cu:186-195) with the store of
 * sddmm_CPU_CSR (:171).  val_ind == NULL gives the unscaled COO result.
 */
ORACLE_API double oracle_sddmm_coo_scaled(const int32_t *row_ind, const int32_t *col_ind,
                                          const float *val_ind, int64_t nnz,
                                          const float *W, const float *H, int k,
                                          float *p_ind, int threads)
{
    double t0 = now_seconds();
    if (threads < 1) threads = oracle_max_threads();
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int64_t ind = 0; ind < nnz; ind++) {
        float sm = 0;
        const float *w = W + (int64_t)row_ind[ind] * k;
        const float *h = H + (int64_t)col_ind[ind] * k;
        for (int t = 0; t < k; ++t)
            sm += w[t] * h[t];
        p_ind[ind] = val_ind ? sm * val_ind[ind] : sm;
    }
    return now_seconds() - t0;
}

/*
 * Arbiter for the tolerance: the same loop in float64, plus the magnitude
 * scale A = sum_t |W[r,t] * H[c,t]| of each dot product.  A parity check
 * accepts |gpu - ref| <= tol * max(|ref|, A).
 */
ORACLE_API void oracle_sddmm_coo_f64(const int32_t *row_ind, const int32_t *col_ind,
                                     const float *val_ind, int64_t nnz,
                                     const float *W, const float *H, int k,
                                     double *p_out, double *abs_scale, int threads)
{
    if (threads < 1) threads = oracle_max_threads();
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int64_t ind = 0; ind < nnz; ind++) {
        double sm = 0, a = 0;
        const float *w = W + (int64_t)row_ind[ind] * k;
        const float *h = H + (int64_t)col_ind[ind] * k;
        for (int t = 0; t < k; ++t) {
            double p = (double)w[t] * (double)h[t];
            sm += p;
            a += fabs(p);
        }
        double s = val_ind ? (double)val_ind[ind] : 1.0;
        if (p_out) p_out[ind] = sm * s;
        if (abs_scale) abs_scale[ind] = a * fabs(s);
    }
}

/*
 * SpMM on the pattern of S, the step that follows SDDMM in its callers:
 *     Y[r, :] = sum over the nonzeros i of row r of  p_i * H[col_i, :]     (p_i = 1 when p is NULL)
 * NO COUNTERPART IN THE REFERENCE (it stops at SDDMM), so this loop is pinned to nothing but its own
 * definition: parity of the CUDA SpMM / fused kernels is "unpinned by the reference".  fp32, the
 * nonzeros of a row added in input order, one rounding per multiply and per add (no FMA contraction),
 * rows in parallel.  rows[] must be sorted.  The float64 companion also returns the magnitude
 * scale A[r, t] = sum_i |p_i * H[col_i, t]| for the tolerance |gpu - ref| <= tol * max(|ref|, A).
 */
ORACLE_API void oracle_spmm(const int32_t *row_ind, const int32_t *col_ind, const float *p, int64_t nnz,
                            int64_t n_rows, const float *H, int k, float *Y, int threads)
{
    if (threads < 1) threads = oracle_max_threads();
    int64_t *row_ptr = (int64_t *)calloc((size_t)n_rows + 1, sizeof(int64_t));
    for (int64_t i = 0; i < nnz; ++i) row_ptr[row_ind[i] + 1]++;
    for (int64_t r = 0; r < n_rows; ++r) row_ptr[r + 1] += row_ptr[r];
#pragma omp parallel for num_threads(threads) schedule(dynamic, 64)
    for (int64_t r = 0; r < n_rows; ++r) {
        float *y = Y + r * k;
        for (int t = 0; t < k; ++t) y[t] = 0.f;
        for (int64_t i = row_ptr[r]; i < row_ptr[r + 1]; ++i) {
            const float *h = H + (int64_t)col_ind[i] * k;
            const float pi = p ? p[i] : 1.f;
            for (int t = 0; t < k; ++t) y[t] += pi * h[t];
        }
    }
    free(row_ptr);
}

ORACLE_API void oracle_spmm_f64(const int32_t *row_ind, const int32_t *col_ind, const double *p, int64_t nnz,
                                int64_t n_rows, const float *H, int k, double *Y, double *A, int threads)
{
    if (threads < 1) threads = oracle_max_threads();
    int64_t *row_ptr = (int64_t *)calloc((size_t)n_rows + 1, sizeof(int64_t));
    for (int64_t i = 0; i < nnz; ++i) row_ptr[row_ind[i] + 1]++;
    for (int64_t r = 0; r < n_rows; ++r) row_ptr[r + 1] += row_ptr[r];
#pragma omp parallel for num_threads(threads) schedule(dynamic, 64)
    for (int64_t r = 0; r < n_rows; ++r) {
        double *y = Y + r * k, *a = A + r * k;
        for (int t = 0; t < k; ++t) y[t] = a[t] = 0.0;
        for (int64_t i = row_ptr[r]; i < row_ptr[r + 1]; ++i) {
            const float *h = H + (int64_t)col_ind[i] * k;
            const double pi = p ? p[i] : 1.0;
            for (int t = 0; t < k; ++t) {
                const double v = pi * (double)h[t];
                y[t] += v;
                a[t] += fabs(v);
            }
        }
    }
    free(row_ptr);
}

/* HiPC18/src/util.h:68-73 (make_HTasH): H_t[t*n + r] = H[r*k + t], the K-major copy of an n x k operand. */
ORACLE_API void oracle_make_htash(const float *H, float *H_t, int64_t n, int k)
{
    for (int64_t r = 0; r < n; ++r)
        for (int64_t t = 0; t < k; ++t)
            H_t[t * n + r] = H[r * k + t];
}

/* HiPC18/src/util.h:75-81 (initial): srand48(0) then X[r*k+t] = 0.1*drand48(). */
ORACLE_API void oracle_initial(float *X, int64_t n, int k)
{
    srand48(0L);
    for (int64_t r = 0; r < n; ++r)
        for (int64_t t = 0; t < k; ++t)
            X[r * k + t] = 0.1 * drand48();
}

/*
 * HiPC18/src/util.h:131-153 (make_CSR): run-length compression of the sorted
 * row array over NON-EMPTY rows only.  row_holder[h] = id of the h-th non-empty
 * row, row_ptr[h]..row_ptr[h+1] its nonzero range.  Returns the number of
 * non-empty rows.  Slots past it: row_ptr = nnz, row_holder = -1 (the reference
 * leaves them uninitialised and reads rows[nnz] one past the end).
 * row_ptr has n_rows + 2 entries, row_holder n_rows + 1.
 */
ORACLE_API int64_t oracle_make_csr(const int32_t *rows, int64_t nnz, int64_t n_rows,
                                   int32_t *row_ptr, int32_t *row_holder)
{
    int64_t idx = 0, holder = 0;
    for (int64_t i = 0; i < n_rows + 2; ++i) row_ptr[i] = (int32_t)nnz;
    for (int64_t i = 0; i < n_rows + 1; ++i) row_holder[i] = -1;
    row_ptr[0] = 0;
    while (idx < nnz) {
        int32_t r = rows[idx];
        row_holder[holder] = r;
        while (idx < nnz && rows[idx] == r) idx++;
        holder++;
        row_ptr[holder] = (int32_t)idx;
    }
    return holder;
}

/*
 * HiPC18/src/util.h:267-343 (rewrite_matrix_1D) with the sizes of the
 * TiledMatrix constructor (util.h:52-65).
 *
 * Column tiles of width TS; inside a tile the non-empty rows are walked in
 * order, the row's nonzeros with col < tile limit are appended, the row is
 * renamed to its tile-local active-row index, and every actv_row_size active
 * rows close a block.  Outputs (caller-allocated):
 *   t_rows, t_cols, t_vals, tiled_ind : nnz entries each
 *   lastIdx_tile       : ntile_c + 1             (ntile_c = n_cols/TS + 1)
 *   lastIdx_block_tile : (ntile_c + 1) * max_blk (max_blk = n_rows/actv_row_size + 1),
 *                        zero-filled first as std::vector::resize does
 *   active_row         : n_rows * ntile_c, zero-filled first
 *   n_actv_row         : ntile_c, zero-filled first
 * The reference pre-writes slot 0 of the NEXT tile's block table at the start
 * of every tile (:289-292); that quirk is reproduced.  Returns max_active_row.
 * n_holder = number of non-empty rows (the reference iterates holder < n_rows
 * over uninitialised tails; here the tail is skipped, which is what the
 * reference computes whenever its heap tail happens to be harmless).
 */
ORACLE_API int32_t oracle_rewrite_matrix_1d(
    const int32_t *s_cols, const float *s_vals, int64_t nnz, int64_t n_rows,
    int64_t n_cols, const int32_t *row_ptr, const int32_t *row_holder,
    int64_t n_holder, int TS, int actv_row_size, int32_t *t_rows, int32_t *t_cols,
    float *t_vals, int32_t *tiled_ind, int32_t *lastIdx_tile,
    int32_t *lastIdx_block_tile, int32_t *active_row, int32_t *n_actv_row)
{
    int64_t new_idx = 0;
    int64_t max_blk = n_rows / actv_row_size + 1;
    int64_t ntile_c = n_cols / TS + 1;
    int32_t max_active_row = 0;
    int64_t *row_lim = (int64_t *)malloc(sizeof(int64_t) * (size_t)(n_rows > 0 ? n_rows : 1));

    memset(lastIdx_tile, 0, sizeof(int32_t) * (size_t)(ntile_c + 1));
    memset(lastIdx_block_tile, 0, sizeof(int32_t) * (size_t)((ntile_c + 1) * max_blk));
    memset(active_row, 0, sizeof(int32_t) * (size_t)(n_rows * ntile_c));
    memset(n_actv_row, 0, sizeof(int32_t) * (size_t)ntile_c);

    for (int64_t tile_lim = TS; tile_lim <= n_cols + TS - 1; tile_lim += TS) {
        int64_t tile_no = tile_lim / TS; /* 1-based */
        int block_count = 0, cur_block = 0;
        n_actv_row[tile_no - 1] = 0;
        lastIdx_block_tile[tile_no * max_blk + 0] = (tile_no == 1) ? 0 : (int32_t)new_idx;

        for (int64_t holder = 0; holder < n_holder; ++holder) {
            int32_t r = row_holder[holder];
            int64_t idx;
            if (tile_lim == TS) { idx = row_ptr[holder]; row_lim[holder] = idx; }
            else idx = row_lim[holder];

            while (idx < row_ptr[holder + 1] && s_cols[idx] < tile_lim) {
                tiled_ind[new_idx] = (int32_t)idx;
                t_rows[new_idx] = n_actv_row[tile_no - 1];
                t_cols[new_idx] = s_cols[idx];
                t_vals[new_idx] = s_vals ? s_vals[idx] : 0.0f;
                new_idx++;
                idx++;
            }
            if (idx != row_lim[holder]) {
                active_row[(tile_no - 1) * n_rows + n_actv_row[tile_no - 1]++] = r;
                cur_block++;
            }
            row_lim[holder] = idx;
            if (cur_block >= actv_row_size) {
                cur_block = 0;
                lastIdx_block_tile[(tile_no - 1) * max_blk + block_count] = (int32_t)new_idx;
                block_count++;
            }
            /* the reference tests holder == n_rows-1; with the tail skipped the
             * last walked holder plays that role (identical when no row is empty) */
            if (holder == n_holder - 1 && cur_block > 0 && cur_block < actv_row_size)
                lastIdx_block_tile[(tile_no - 1) * max_blk + block_count] = (int32_t)new_idx;
        }
        if (n_actv_row[tile_no - 1] > max_active_row)
            max_active_row = n_actv_row[tile_no - 1];
        lastIdx_tile[tile_no] = (int32_t)new_idx;
    }
    free(row_lim);
    return max_active_row;
}

/*
 * HiPC18/src/util.h:82-128 (unsorted_make_CSR), the "conversion code from col
 * sorted to row sorted".  transpose != 0 follows the live code: tuples are
 * (col,row,val), sorted, and written back as rows = col+1, cols = row+1
 * (1-based, i.e. the TRANSPOSE of the input, 0-based in, 1-based out), with a
 * row pointer whose outer loop runs over the OLD row count (:102) -- entries
 * whose new row id >= n_rows are therefore never written back.  transpose == 0
 * is the commented variant (:93): a plain (row,col,val) sort.
 * Returns the number of entries written back.
 */
typedef struct { int32_t a, b; float v; } oracle_triple;

static int triple_cmp(const void *x, const void *y)
{
    const oracle_triple *p = (const oracle_triple *)x, *q = (const oracle_triple *)y;
    if (p->a != q->a) return p->a < q->a ? -1 : 1;
    if (p->b != q->b) return p->b < q->b ? -1 : 1;
    /* std::tuple compares the float last with operator< */
    if (p->v < q->v) return -1;
    if (q->v < p->v) return 1;
    return 0;
}

ORACLE_API int64_t oracle_unsorted_make_csr(int32_t *rows, int32_t *cols, float *vals,
                                            int64_t nnz, int64_t n_rows, int64_t n_cols,
                                            int32_t *row_ptr, int transpose)
{
    (void)n_cols;
    oracle_triple *items = (oracle_triple *)malloc(sizeof(oracle_triple) * (size_t)(nnz > 0 ? nnz : 1));
    for (int64_t i = 0; i < nnz; ++i) {
        items[i].a = transpose ? cols[i] : rows[i];
        items[i].b = transpose ? rows[i] : cols[i];
        items[i].v = vals[i];
    }
    qsort(items, (size_t)nnz, sizeof(oracle_triple), triple_cmp);
    int64_t idx = 0;
    row_ptr[0] = 0;
    for (int64_t r = 0; r < n_rows; ++r) {
        while (idx < nnz && items[idx].a == r) {
            rows[idx] = items[idx].a + 1;
            cols[idx] = items[idx].b + 1;
            vals[idx] = items[idx].v;
            idx++;
        }
        row_ptr[r + 1] = (int32_t)idx;
    }
    free(items);
    return idx;
}

/*
 * HiPC18_mpi/util.h:100-135 (make_CSC): greedy nnz-balanced COLUMN cuts for
 * n_p ranks: a cut closes when the running count reaches ceil(nnz/n_p) or at
 * the last column.  cols_in_rank[t] and nnz_in_rank[t] as the reference writes
 * them (note its off-by-one: the first panel's width is i - 0, later ones
 * i - previous i).  Returns the number of panels produced.
 */
ORACLE_API int oracle_make_csc_cuts(const int32_t *cols, int64_t nnz, int64_t n_cols,
                                    int n_p, int32_t *cols_in_rank, int32_t *nnz_in_rank)
{
    int32_t *nnz_col = (int32_t *)calloc((size_t)(n_cols + 1), sizeof(int32_t));
    int avg = (int)((nnz + n_p - 1) / n_p);
    for (int64_t i = 0; i < nnz; ++i) nnz_col[cols[i]]++;
    int tile = 0, tile_ct = 0, tile_col = 0;
    for (int64_t i = 0; i < n_cols; ++i) {
        tile_ct += nnz_col[i];
        if (tile_ct >= avg || i == n_cols - 1) {
            cols_in_rank[tile] = (int32_t)(i - tile_col);
            if (i == n_cols - 1) cols_in_rank[tile] = (int32_t)(n_cols - tile_col);
            tile_col = (int)i;
            nnz_in_rank[tile] = tile_ct;
            tile_ct = 0;
            tile++;
        }
    }
    free(nnz_col);
    return tile;
}
