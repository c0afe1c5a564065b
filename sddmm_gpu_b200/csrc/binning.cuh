// GPU binning pass: everything the reference prepares on the host before its
// launch loop (make_CSR, TiledMatrix, rewrite_matrix_1D -- HiPC18/src/util.h:52-65,
// 131-153, 267-343), done on the device from the row-sorted COO.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "common.cuh"

namespace sddmm {

// Device scratch whose lifetime is one binning call.
struct Scratch {
    void *ptr = nullptr;
    size_t bytes = 0;
    cudaError_t reserve(size_t n);
    void release();
    ~Scratch() { release(); }
};

// First offending nonzero index per class, or INT64_MAX when clean.
struct ValidationResult {
    long long first_unsorted;
    long long first_out_of_range;
};
cudaError_t validate_coo(const int32_t *d_rows, const int32_t *d_cols, int64_t nnz, int64_t M,
                         int64_t N, ValidationResult *host_out, cudaStream_t stream);

// row_ptr[r] = first nonzero of row r (M + 1 entries, empty rows repeat);
// *d_nonempty receives the number of rows with at least one nonzero.
cudaError_t build_row_ptr(const int32_t *d_rows, int64_t nnz, int64_t M, int64_t *d_row_ptr,
                          unsigned long long *d_nonempty, cudaStream_t stream);

// Number of distinct columns (marks a byte per column, then counts).
cudaError_t count_distinct_cols(const int32_t *d_cols, int64_t nnz, int64_t N, int64_t *host_out,
                                cudaStream_t stream);

// Stable partition of the nonzeros by column tile (tile = col / col_tile):
// d_perm[j] = input index of the j-th nonzero in tiled order (the reference's
// tiled_ind, util.h:301), d_rows_t/d_cols_t the permuted indices.
cudaError_t build_tiled_order(const int32_t *d_rows, const int32_t *d_cols, int64_t nnz, int64_t N,
                              int col_tile, int32_t *d_perm, int32_t *d_rows_t, int32_t *d_cols_t,
                              cudaStream_t stream);

// Work items over the processing-order arrays: maximal runs of nonzeros that
// share a column tile and a row panel (row / panel_rows), each cut into pieces of
// at most item_nnz nonzeros, plus the list of the distinct rows of every item
// (what the producer warp stages).  Allocates *d_items and *d_item_rows
// (cudaMalloc) and sets *n_items / *n_item_rows.
cudaError_t build_work_items(const int32_t *d_rows_p, const int32_t *d_cols_p, int64_t nnz,
                             int panel_rows, int col_tile, int item_nnz, WorkItem **d_items,
                             int64_t *n_items, int32_t **d_item_rows, int64_t *n_item_rows,
                             cudaStream_t stream);

// Ascending list of the rows of S that hold at least one nonzero (from the row
// pointer) or of the columns that do (from the column indices): the rows of W / H
// that an SDDMM actually reads.  Allocates *d_list (cudaMalloc) and sets *n_list.
cudaError_t build_used_row_list(const int64_t *d_row_ptr, int64_t M, int32_t **d_list, int64_t *n_list,
                                cudaStream_t stream);
cudaError_t build_used_col_list(const int32_t *d_cols, int64_t nnz, int64_t N, int32_t **d_list, int64_t *n_list,
                                cudaStream_t stream);

// Sort COO triples on the device, in place: by (a, b) keeping the input order of
// equal pairs (stable), or -- tie_by_value -- by (a, b, value), the order
// std::sort gives whole (a, b, value) tuples.  d_a / d_b are the major / minor
// index arrays (rows / cols, or cols / rows for a transposing sort).
cudaError_t sort_coo(int32_t *d_a, int32_t *d_b, float *d_v, int64_t nnz, bool tie_by_value, cudaStream_t stream);

// Hub-column hints for the ring kernel: d_cols_hinted[j] = d_cols_p[j] with bit 31
// set when the column is among the most popular ones whose rows of H together fit
// budget_bytes (chosen by exact column degree, most popular first).
cudaError_t build_hub_column_hints(const int32_t *d_cols_p, int64_t nnz, int64_t N, int64_t row_bytes,
                                   int64_t budget_bytes, int32_t *d_cols_hinted, int64_t *n_hub_cols,
                                   int *degree_threshold, cudaStream_t stream);

// Row groups for the SpMM ring kernel: every row's nonzeros cut into groups of B slots (B = rows of H per
// 4 KB ring slot), the last group of a row padded with slots that repeat the group's first column and carry
// index -1, so that all B lane sets of a warp always work on the same row of S.
struct RowGroups {
    int32_t *pcols = nullptr;  // [n_groups * B] column of every slot
    int32_t *pidx = nullptr;   // [n_groups * B] input index of the slot's nonzero, -1 for padding
    int32_t *grow = nullptr;   // [n_groups] row of the group; bit 31 = last group of its row
    int64_t n_groups = 0;
    int B = 0;
    void release();
};
// gstart_host receives the first group of every row (M + 1 entries), from which the tasks are built on the host.
cudaError_t build_row_groups(const int32_t *d_rows, const int32_t *d_cols, const int64_t *d_row_ptr, int64_t nnz, int64_t M,
                             int B, RowGroups *out, std::vector<int64_t> *gstart_host, cudaStream_t stream);

// Dense-cell classification.  S is cut into cells of DENSE_CELL_ROWS x
// DENSE_CELL_COLS -- over compacted (nearly) full rows, then compacted (nearly)
// full columns, then the regular grid; a cell holding at least min_density of its
// positions is "dense" and is computed as a small dense product by the dense-cell
// kernel, the nonzeros of all other cells form a row-sorted remainder that goes
// through the gather kernels with a permutation.  Nothing is built (n_cells == 0)
// when the dense cells would hold less than min_share of the nonzeros.
struct DensePlan {
    DenseCell *cells = nullptr;   // one descriptor per dense cell
    int64_t n_cells = 0;
    int32_t *idx = nullptr;       // input index of every dense-cell nonzero, grouped by cell, row-major inside
    uint16_t *rc = nullptr;       // (row - row0) << 8 | (col - col0)
    // Row-mask form of a cell (DenseCell::cls bit 8 set): per cell row a 64-bit column mask and the
    // input index of the row's first nonzero inside the cell.  Valid for cells in which the nonzeros of
    // every row are consecutive in the input with ascending columns (any (row, col)-sorted input, for
    // cells over a contiguous column range); such a cell's nonzeros need no per-nonzero list.
    unsigned long long *row_mask = nullptr;  // [n_cells][DENSE_CELL_ROWS]
    int32_t *row_base = nullptr;             // [n_cells][DENSE_CELL_ROWS]
    int64_t n_mask_cells = 0;
    int64_t n_dense_nnz = 0;
    int32_t *rows_s = nullptr, *cols_s = nullptr, *perm_s = nullptr;  // remainder: indices and input positions
    int64_t n_sparse = 0;
    int32_t *dense_rows = nullptr, *dense_cols = nullptr;  // ids of the compacted full rows / columns
    int64_t n_dense_rows = 0, n_dense_cols = 0;
    void release();
};
cudaError_t build_dense_cells(const int32_t *d_rows, const int32_t *d_cols, const int64_t *d_row_ptr, int64_t nnz,
                              int64_t M, int64_t N, float min_density, float min_share, DensePlan *out,
                              cudaStream_t stream);

// Reference-layout tiling tables (test hook); see sddmm_plan_export_tiling.
struct TilingTables {
    int32_t *t_rows, *t_cols, *tiled_ind, *lastIdx_tile, *lastIdx_block_tile, *active_row, *n_actv_row;
    int32_t *max_active_row;
};
cudaError_t export_reference_tiling(const int32_t *d_rows, const int32_t *d_cols, int64_t nnz, int64_t M,
                                    int64_t N, int panel_rows, int col_tile, const TilingTables &host_out,
                                    cudaStream_t stream);

}  // namespace sddmm
