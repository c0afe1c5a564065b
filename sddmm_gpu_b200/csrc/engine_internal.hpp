// Internal layout of the engine's handle and plan (shared by engine.cu and the
// multi-GPU layer); the public surface is include/sddmm_b200.h.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "binning.cuh"
#include "common.cuh"
#include "sddmm_b200.h"

using namespace sddmm;

// Host-operand pipeline: S is cut into at most this many chunks of consecutive nonzeros.
#define SDDMM_PIPE_MAX_CHUNKS 16

struct sddmm_handle_s {
    int device = 0;
    int sm_count = 0;
    size_t smem_optin = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int *d_status = nullptr;  // device status word of bounded waits
    unsigned long long *d_work_counter = nullptr;  // dynamic work distribution of the ring kernel
    int *h_status = nullptr;  // pinned mirror
    std::string last_error;
    // dense cells: 0 = fp32 FMA, 1 = 3xTF32 on mma.sync, 2 = 3xTF32 on tcgen05 / tensor memory (SDDMM_DENSE_TENSOR)
    int dense_mode = 2;
    // pipelined execution with host operands: compute and download streams, one
    // "uploaded" and one "computed" event per chunk (created on first use)
    cudaStream_t pipe_compute = nullptr, pipe_download = nullptr;
    cudaEvent_t pipe_uploaded[SDDMM_PIPE_MAX_CHUNKS] = {};
    cudaEvent_t pipe_started[SDDMM_PIPE_MAX_CHUNKS] = {}, pipe_computed[SDDMM_PIPE_MAX_CHUNKS] = {};  // timing events
    cudaEvent_t pipe_joined = nullptr;
    bool pipeline = true;  // SDDMM_PIPELINE=0 keeps upload, kernel and download strictly one after the other
    // pipelined calls whose host operands are page-locked and mapped upload only the rows of
    // W and H that a nonzero touches, read by the GPU (SDDMM_SPARSE_UPLOAD=0: whole arrays by cudaMemcpy)
    bool sparse_upload = true;
    int upload_ctas = 0;  // CTAs of the upload kernel (SDDMM_UPLOAD_CTAS; default half the SMs)
    int64_t n_launches = 0;  // kernels launched through this handle by sddmm_execute / sddmm_upload_rows
};

struct sddmm_plan_s {
    sddmm_handle_s *h = nullptr;
    int64_t M = 0, N = 0, nnz = 0;
    int K = 0;
    int col_tile = 0;     // == N (clamped) when there is a single column tile
    int n_col_tiles = 1;
    PanelConfig cfg{};
    // pattern, input order
    int32_t *d_rows = nullptr, *d_cols = nullptr;
    bool owns_rows = true, owns_cols = true;
    // pattern, tiled order (only when n_col_tiles > 1)
    int32_t *d_rows_t = nullptr, *d_cols_t = nullptr, *d_perm = nullptr;
    int64_t *d_row_ptr = nullptr;
    WorkItem *d_items = nullptr;
    int64_t n_items = 0;
    int32_t *d_item_rows = nullptr;  // distinct rows of every item, concatenated
    int32_t *d_cols_hint = nullptr;  // processing-order columns with hub marks (ring kernel), or null
    // column-tile kernel (few columns, many nonzeros per column): its own tiled order and tile offsets
    int32_t *d_ht_rows = nullptr, *d_ht_cols = nullptr, *d_ht_perm = nullptr;
    int64_t *d_ht_off = nullptr;
    int ht_col_tile = 0, ht_n_tiles = 0;
    // dense cells + row-sorted remainder (single-tile plans of locally dense matrices)
    DensePlan dense;
    WorkItem *d_items_s = nullptr;
    int64_t n_items_s = 0;
    int32_t *d_item_rows_s = nullptr;
    int64_t n_item_rows_s = 0;
    int64_t n_hub_cols = 0;
    int64_t n_item_rows = 0;
    int64_t n_nonempty_rows = 0, n_nonempty_cols = -1;
    // staging for host operands (allocated on first use)
    float *d_W = nullptr, *d_H = nullptr, *d_S = nullptr, *d_P = nullptr;
    float *d_Wt = nullptr, *d_Ht = nullptr;  // device copies of K-major host operands, before their transposition
    int64_t device_bytes = 0;
    float plan_ms = 0.f, last_ms = -1.f;
    // chunks of the host-operand pipeline (0 = not pipelined): nonzeros
    // [pipe_nnz[i], pipe_nnz[i+1]) touch the rows pipe_row_first[i] .. pipe_row_last[i] of W
    int n_pipe = 0;
    int64_t pipe_nnz[SDDMM_PIPE_MAX_CHUNKS + 1] = {};
    int32_t pipe_row_first[SDDMM_PIPE_MAX_CHUNKS] = {}, pipe_row_last[SDDMM_PIPE_MAX_CHUNKS] = {};
    // rows of W chunk i uploads: [pipe_w_begin[i], pipe_w_end[i]) (empty when an earlier chunk brought them),
    // = entries [pipe_list_begin[i], pipe_list_begin[i+1]) of the used-row list
    int64_t pipe_w_begin[SDDMM_PIPE_MAX_CHUNKS] = {}, pipe_w_end[SDDMM_PIPE_MAX_CHUNKS] = {};
    int64_t pipe_list_begin[SDDMM_PIPE_MAX_CHUNKS + 1] = {};
    int32_t *d_used_rows = nullptr, *d_used_cols = nullptr;  // ascending ids of the rows / columns holding a nonzero
    int64_t n_used_rows = 0, n_used_cols = 0;
    int64_t last_h2d_bytes = 0, last_d2h_bytes = 0;  // moved by the last sddmm_execute
    const char *last_kernel = "none";                // kernels the last sddmm_execute launched
    // SpMM / fused SDDMM->SpMM over the plan's rows (built on first use): tasks, long-row table, scratch
    SpmmTask *d_spmm_tasks = nullptr;
    SpmmLongRow *d_spmm_long = nullptr;
    float *d_spmm_scratch = nullptr;
    int64_t n_spmm_tasks = -1, n_spmm_long = 0, n_spmm_slots = 0;
    // the same for the ring form (K = 256, 512, 1024): padded row groups and tasks counted in groups
    RowGroups row_groups;
    SpmmTask *d_spmr_tasks = nullptr;
    SpmmLongRow *d_spmr_long = nullptr;
    float *d_spmr_scratch = nullptr;
    int64_t n_spmr_tasks = -1, n_spmr_long = 0;
};

