// C ABI of the engine: handle, plan (GPU binning pass), execute.
// Replaces the host driver sddmm_GPU of the reference (HiPC18/src/sddmm.cu:32-151):
// device memory for the pattern is owned by a reusable plan instead of being
// allocated and freed per call, errors come back as status codes instead of
// assert(), and there is exactly one kernel launch per execute.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <algorithm>
#include <string>
#include <vector>

#include "binning.cuh"
#include "common.cuh"
#include "sddmm_b200.h"

using namespace sddmm;

#include "engine_internal.hpp"

namespace {

int fail_cuda(sddmm_handle_s *h, cudaError_t e, const char *what)
{
    if (h) {
        h->last_error = std::string(what) + ": " + cudaGetErrorString(e);
    }
    (void)cudaGetLastError();  // clear the sticky-free error state
    return e == cudaErrorMemoryAllocation ? SDDMM_OUT_OF_MEMORY : SDDMM_CUDA_ERROR;
}

#define CUDA_TRY(h, expr)                                   \
    do {                                                    \
        cudaError_t _e = (expr);                            \
        if (_e != cudaSuccess) return fail_cuda((h), _e, #expr); \
    } while (0)

// A kernel launch: counted per handle (sddmm_kernel_launches).
#define LAUNCH_TRY(h, expr)   \
    do {                      \
        CUDA_TRY(h, expr);    \
        ++(h)->n_launches;    \
    } while (0)

bool is_device_ptr(const void *p)
{
    if (!p) return false;
    cudaPointerAttributes a;
    cudaError_t e = cudaPointerGetAttributes(&a, p);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// Device-side address of a page-locked host allocation that is mapped into the
// device's address space, or null (pageable memory, device memory, unknown).
const float *mapped_host_ptr(const float *p)
{
    if (!p) return nullptr;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    if (a.type != cudaMemoryTypeHost || !a.devicePointer) return nullptr;
    if (((uintptr_t)a.devicePointer & 15u) != 0) return nullptr;  // the row upload moves 16-byte vectors
    return static_cast<const float *>(a.devicePointer);
}

int check_k(int K)
{
    if (K <= 0 || (K % 4) != 0 || K > SDDMM_MAX_K) return SDDMM_K_UNSUPPORTED;
    return SDDMM_OK;
}

template <class T>
cudaError_t dev_alloc(sddmm_plan_s *p, T **ptr, size_t count)
{
    size_t bytes = sizeof(T) * (count ? count : 1);
    cudaError_t e = cudaMalloc((void **)ptr, bytes);
    if (e == cudaSuccess) p->device_bytes += (int64_t)bytes;
    return e;
}

void free_plan_memory(sddmm_plan_s *p)
{
    if (p->owns_rows) cudaFree(p->d_rows);
    if (p->owns_cols) cudaFree(p->d_cols);
    cudaFree(p->d_rows_t);
    cudaFree(p->d_cols_t);
    cudaFree(p->d_perm);
    cudaFree(p->d_ht_rows);
    cudaFree(p->d_ht_cols);
    cudaFree(p->d_ht_perm);
    cudaFree(p->d_ht_off);
    cudaFree(p->d_row_ptr);
    cudaFree(p->d_items);
    cudaFree(p->d_item_rows);
    cudaFree(p->d_cols_hint);
    p->dense.release();
    cudaFree(p->d_items_s);
    cudaFree(p->d_item_rows_s);
    cudaFree(p->d_used_rows);
    cudaFree(p->d_used_cols);
    p->row_groups.release();
    cudaFree(p->d_spmr_tasks);
    cudaFree(p->d_spmr_long);
    cudaFree(p->d_spmr_scratch);
    cudaFree(p->d_spmm_tasks);
    cudaFree(p->d_spmm_long);
    cudaFree(p->d_spmm_scratch);
    cudaFree(p->d_Wt);
    cudaFree(p->d_Ht);
    cudaFree(p->d_W);
    cudaFree(p->d_H);
    cudaFree(p->d_S);
    cudaFree(p->d_P);
}

// Streams and events of the host-operand pipeline, created on first use.
cudaError_t ensure_pipeline(sddmm_handle_s *h)
{
    if (h->pipe_joined) return cudaSuccess;
    cudaError_t e = cudaStreamCreateWithFlags(&h->pipe_compute, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->pipe_download, cudaStreamNonBlocking);
    for (int i = 0; i < SDDMM_PIPE_MAX_CHUNKS && e == cudaSuccess; ++i) {
        e = cudaEventCreateWithFlags(&h->pipe_uploaded[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreate(&h->pipe_started[i]);
        if (e == cudaSuccess) e = cudaEventCreate(&h->pipe_computed[i]);
    }
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->pipe_joined, cudaEventDisableTiming);
    return e;
}

// The gather kernel for ring-supported K.
cudaError_t launch_rows_gather(sddmm_handle_s *h, const int32_t *rows, const int32_t *cols, const int32_t *perm,
                               const float *sval, const float *W, const float *H, float *P, int64_t nnz, int K,
                               bool cols_hinted, cudaStream_t stream)
{
    return launch_ring(rows, cols, perm, sval, W, H, P, nnz, K, cols_hinted, h->sm_count, h->d_work_counter, h->d_status,
                       stream);
}

// After a synchronising point: turn the device status word into a status code.
int check_device_status(sddmm_handle_s *h)
{
    if (*h->h_status != DEV_OK) {
        h->last_error = "a bounded device-side wait (mbarrier) gave up";
        *h->h_status = DEV_OK;
        cudaMemsetAsync(h->d_status, 0, sizeof(int), h->stream);
        return SDDMM_DEVICE_TIMEOUT;
    }
    return SDDMM_OK;
}

}  // namespace

extern "C" {

const char *sddmm_status_string(int s)
{
    switch (s) {
    case SDDMM_OK: return "ok";
    case SDDMM_INVALID_ARG: return "invalid argument";
    case SDDMM_UNSORTED_INPUT: return "input is not sorted by row";
    case SDDMM_INDEX_OUT_OF_RANGE: return "row or column index out of range";
    case SDDMM_K_UNSUPPORTED: return "K must be a positive multiple of 4 not larger than SDDMM_MAX_K";
    case SDDMM_CUDA_ERROR: return "CUDA error";
    case SDDMM_NCCL_ERROR: return "NCCL error";
    case SDDMM_OUT_OF_MEMORY: return "out of device memory";
    case SDDMM_DEVICE_TIMEOUT: return "device-side wait timed out";
    case SDDMM_IO_ERROR: return "I/O error";
    case SDDMM_PARSE_ERROR: return "Matrix Market parse error";
    case SDDMM_NO_DEVICE: return "no usable CUDA device (this engine has no CPU fallback)";
    default: return "unknown status";
    }
}

int sddmm_create(sddmm_handle_t *out, int device)
{
    if (!out) return SDDMM_INVALID_ARG;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return SDDMM_NO_DEVICE;
    }
    if (device < 0 || device >= n) return SDDMM_INVALID_ARG;
    sddmm_handle_s *h = new (std::nothrow) sddmm_handle_s;
    if (!h) return SDDMM_OUT_OF_MEMORY;
    h->device = device;
    cudaError_t e = cudaSetDevice(device);
    cudaDeviceProp prop;
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device);
    if (e == cudaSuccess && prop.major < 10) {
        delete h;
        return SDDMM_NO_DEVICE;  // kernels are built for sm_100a only
    }
    if (e == cudaSuccess) {
        h->sm_count = prop.multiProcessorCount;
        h->smem_optin = prop.sharedMemPerBlockOptin;
        e = cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking);
    }
    if (e == cudaSuccess) e = cudaEventCreate(&h->ev0);
    if (e == cudaSuccess) e = cudaEventCreate(&h->ev1);
    if (e == cudaSuccess) e = cudaMalloc((void **)&h->d_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(h->d_status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc((void **)&h->d_work_counter, sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaHostAlloc((void **)&h->h_status, sizeof(int), cudaHostAllocDefault);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        sddmm_destroy(h);
        return SDDMM_CUDA_ERROR;
    }
    *h->h_status = DEV_OK;
    h->stream = h->own_stream;
    if (const char *env = std::getenv("SDDMM_DENSE_TENSOR")) {
        const int v = std::atoi(env);
        if (v >= 0 && v <= 2) h->dense_mode = v;
    }
    if (const char *env = std::getenv("SDDMM_PIPELINE")) h->pipeline = std::atoi(env) != 0;
    if (const char *env = std::getenv("SDDMM_SPARSE_UPLOAD")) h->sparse_upload = std::atoi(env) != 0;
    h->upload_ctas = h->sm_count / 2 > 0 ? h->sm_count / 2 : 1;
    if (const char *env = std::getenv("SDDMM_UPLOAD_CTAS")) {
        const int v = std::atoi(env);
        if (v > 0 && v <= 4096) h->upload_ctas = v;
    }
    *out = h;
    return SDDMM_OK;
}

int sddmm_destroy(sddmm_handle_t h)
{
    if (!h) return SDDMM_OK;
    cudaSetDevice(h->device);
    if (h->own_stream) cudaStreamDestroy(h->own_stream);
    if (h->ev0) cudaEventDestroy(h->ev0);
    if (h->ev1) cudaEventDestroy(h->ev1);
    if (h->d_status) cudaFree(h->d_status);
    if (h->d_work_counter) cudaFree(h->d_work_counter);
    if (h->h_status) cudaFreeHost(h->h_status);
    if (h->pipe_compute) cudaStreamDestroy(h->pipe_compute);
    if (h->pipe_download) cudaStreamDestroy(h->pipe_download);
    for (cudaEvent_t e : h->pipe_uploaded) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : h->pipe_started) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : h->pipe_computed) if (e) cudaEventDestroy(e);
    if (h->pipe_joined) cudaEventDestroy(h->pipe_joined);
    (void)cudaGetLastError();
    delete h;
    return SDDMM_OK;
}

const char *sddmm_last_error(sddmm_handle_t h) { return h ? h->last_error.c_str() : ""; }

int sddmm_set_stream(sddmm_handle_t h, void *cuda_stream)
{
    if (!h) return SDDMM_INVALID_ARG;
    h->stream = cuda_stream ? (cudaStream_t)cuda_stream : h->own_stream;
    return SDDMM_OK;
}

int sddmm_plan_coo(sddmm_handle_t h, int64_t M, int64_t N, int64_t nnz, const int32_t *rows,
                   const int32_t *cols, int K, int panel_rows_hint, int col_tile_hint, uint32_t flags,
                   sddmm_plan_t *out)
{
    if (!h || !out) return SDDMM_INVALID_ARG;
    *out = nullptr;
    if (M < 0 || N < 0 || nnz < 0 || (nnz > 0 && (!rows || !cols))) return SDDMM_INVALID_ARG;
    if (M > INT32_MAX || N > INT32_MAX || nnz >= INT32_MAX) return SDDMM_INVALID_ARG;  // int32 indices, as the reference
    if (nnz > 0 && (M == 0 || N == 0)) return SDDMM_INDEX_OUT_OF_RANGE;
    int st = check_k(K);
    if (st != SDDMM_OK) return st;
    CUDA_TRY(h, cudaSetDevice(h->device));

    sddmm_plan_s *p = new (std::nothrow) sddmm_plan_s;
    if (!p) return SDDMM_OUT_OF_MEMORY;
    p->h = h;
    p->M = M; p->N = N; p->nnz = nnz; p->K = K;
    cudaStream_t s = h->stream;
    cudaEvent_t t0 = nullptr, t1 = nullptr;

#define PLAN_TRY(expr)                                 \
    do {                                               \
        cudaError_t _e = (expr);                       \
        if (_e != cudaSuccess) {                       \
            int _st = fail_cuda(h, _e, #expr);         \
            free_plan_memory(p);                       \
            delete p;                                  \
            if (t0) cudaEventDestroy(t0);              \
            if (t1) cudaEventDestroy(t1);              \
            return _st;                                \
        }                                              \
    } while (0)

    const bool dev_idx = (flags & SDDMM_PLAN_DEVICE_INDICES) != 0;
    if (dev_idx) {
        p->d_rows = const_cast<int32_t *>(rows);
        p->owns_rows = false;
        if (((uintptr_t)cols & 15u) == 0) {
            p->d_cols = const_cast<int32_t *>(cols);
            p->owns_cols = false;
        } else {
            // the kernels read column indices with 16-byte vector loads: realign a borrowed array
            PLAN_TRY(dev_alloc(p, &p->d_cols, (size_t)nnz));
            if (nnz > 0) PLAN_TRY(cudaMemcpyAsync(p->d_cols, cols, sizeof(int32_t) * nnz, cudaMemcpyDeviceToDevice, s));
        }
    } else {
        PLAN_TRY(dev_alloc(p, &p->d_rows, (size_t)nnz));
        PLAN_TRY(dev_alloc(p, &p->d_cols, (size_t)nnz));
        if (nnz > 0) {
            PLAN_TRY(cudaMemcpyAsync(p->d_rows, rows, sizeof(int32_t) * nnz, cudaMemcpyHostToDevice, s));
            PLAN_TRY(cudaMemcpyAsync(p->d_cols, cols, sizeof(int32_t) * nnz, cudaMemcpyHostToDevice, s));
        }
    }
    PLAN_TRY(cudaEventCreate(&t0));
    PLAN_TRY(cudaEventCreate(&t1));
    PLAN_TRY(cudaEventRecord(t0, s));

    if (!(flags & SDDMM_PLAN_SKIP_VALIDATION)) {
        ValidationResult vr;
        PLAN_TRY(validate_coo(p->d_rows, p->d_cols, nnz, M, N, &vr, s));
        if (vr.first_out_of_range != LLONG_MAX || vr.first_unsorted != LLONG_MAX) {
            char buf[160];
            const bool oob = vr.first_out_of_range != LLONG_MAX;
            snprintf(buf, sizeof(buf), "%s at nonzero %lld", oob ? "index out of range" : "rows not sorted",
                     oob ? vr.first_out_of_range : vr.first_unsorted);
            h->last_error = buf;
            free_plan_memory(p);
            delete p;
            cudaEventDestroy(t0);
            cudaEventDestroy(t1);
            return oob ? SDDMM_INDEX_OUT_OF_RANGE : SDDMM_UNSORTED_INPUT;
        }
    }

    // row pointer over all rows (empty rows included)
    PLAN_TRY(dev_alloc(p, &p->d_row_ptr, (size_t)M + 1));
    {
        Scratch cnt;
        PLAN_TRY(cnt.reserve(sizeof(unsigned long long)));
        PLAN_TRY(build_row_ptr(p->d_rows, nnz, M, p->d_row_ptr, (unsigned long long *)cnt.ptr, s));
        unsigned long long ne = 0;
        PLAN_TRY(cudaMemcpyAsync(&ne, cnt.ptr, sizeof(ne), cudaMemcpyDeviceToHost, s));
        PLAN_TRY(cudaStreamSynchronize(s));
        p->n_nonempty_rows = (int64_t)ne;
    }

    // column tiles: a hint >= N (or <= 0) means one tile, the identity order
    p->cfg = choose_panel_config(K, panel_rows_hint, h->sm_count, h->smem_optin);
    int64_t ct = (col_tile_hint <= 0 || col_tile_hint >= N) ? (N > 0 ? N : 1) : col_tile_hint;
    p->col_tile = (int)ct;
    p->n_col_tiles = (int)((N + ct - 1) / ct);
    if (p->n_col_tiles < 1) p->n_col_tiles = 1;
    const int32_t *rows_p = p->d_rows, *cols_p = p->d_cols;
    if (p->n_col_tiles > 1 && nnz > 0) {
        PLAN_TRY(dev_alloc(p, &p->d_perm, (size_t)nnz));
        PLAN_TRY(dev_alloc(p, &p->d_rows_t, (size_t)nnz));
        PLAN_TRY(dev_alloc(p, &p->d_cols_t, (size_t)nnz));
        PLAN_TRY(build_tiled_order(p->d_rows, p->d_cols, nnz, N, p->col_tile, p->d_perm, p->d_rows_t, p->d_cols_t, s));
        rows_p = p->d_rows_t;
        cols_p = p->d_cols_t;
    }
    PLAN_TRY(build_work_items(rows_p, cols_p, nnz, p->cfg.panel_rows, p->col_tile, p->cfg.item_nnz, &p->d_items,
                              &p->n_items, &p->d_item_rows, &p->n_item_rows, s));
    p->device_bytes += (int64_t)(sizeof(WorkItem) * (size_t)p->n_items + sizeof(int32_t) * (size_t)p->n_item_rows);
    // Locally dense matrices (many nonzeros per row): cells that are at least a
    // quarter full go to the dense-cell kernel, if they hold half of S or more
    // (below that the second launch and the permuted remainder cost more than they save).
    // SDDMM_DENSE_CELLS=0 switches the classification off.
    {
        const char *env = std::getenv("SDDMM_DENSE_CELLS");
        const bool enabled = !(env && std::atoi(env) == 0);
        if (enabled && p->n_col_tiles == 1 && p->n_nonempty_rows > 0 && nnz / p->n_nonempty_rows >= 32) {
            PLAN_TRY(build_dense_cells(p->d_rows, p->d_cols, p->d_row_ptr, nnz, M, N, 0.25f, 0.5f, &p->dense, s));
            if (p->dense.n_cells > 0 && p->dense.n_sparse > 0 && !ring_supports(K)) {
                PLAN_TRY(build_work_items(p->dense.rows_s, p->dense.cols_s, p->dense.n_sparse, p->cfg.panel_rows,
                                          p->col_tile, p->cfg.item_nnz, &p->d_items_s, &p->n_items_s, &p->d_item_rows_s,
                                          &p->n_item_rows_s, s));
            }
            if (p->dense.n_cells > 0)
                p->device_bytes += (int64_t)(sizeof(DenseCell) * p->dense.n_cells + 6 * p->dense.n_dense_nnz +
                                             12 * p->dense.n_sparse);
        }
    }
    // Hub-column marks for the ring kernel, when H is too large to live in L2 as a
    // whole.  SDDMM_L2_HUB_MB overrides the share of L2 set aside for hub rows (0 = off).
    if (ring_supports(K) && nnz > 0) {
        int64_t budget_mb = 64;  // best of a 16..128 MB sweep on the scale-22 R-MAT matrix at K = 256
        if (const char *env = std::getenv("SDDMM_L2_HUB_MB")) budget_mb = std::atoll(env);
        const int64_t row_bytes = (int64_t)K * 4;
        if (budget_mb > 0 && N * row_bytes > budget_mb * (1ll << 20)) {
            PLAN_TRY(dev_alloc(p, &p->d_cols_hint, (size_t)nnz));
            int thr = 0;
            PLAN_TRY(build_hub_column_hints(cols_p, nnz, N, row_bytes, budget_mb * (1ll << 20), p->d_cols_hint,
                                            &p->n_hub_cols, &thr, s));
        }
    }
    // Few columns and many nonzeros per column (a bag-of-words matrix): H is a handful of shared-memory tiles, and
    // the column-tile kernel reads every H row of a nonzero from shared memory.  Worth it when a CTA's share of
    // the nonzeros is several times the rows of the tiles it has to load.  SDDMM_HTILE=0 switches it off.
    {
        const char *env = std::getenv("SDDMM_HTILE");
        const int tc = htile_cols(K);
        const int64_t n_tiles = tc > 0 ? (N + tc - 1) / tc : 0;
        if (!(env && std::atoi(env) == 0) && tc > 0 && p->n_col_tiles == 1 && p->dense.n_cells == 0 && n_tiles >= 1 &&
            n_tiles <= 64 && nnz >= 65536 && nnz / h->sm_count >= 8 * (int64_t)tc) {
            PLAN_TRY(dev_alloc(p, &p->d_ht_perm, (size_t)nnz));
            PLAN_TRY(dev_alloc(p, &p->d_ht_rows, (size_t)nnz));
            PLAN_TRY(dev_alloc(p, &p->d_ht_cols, (size_t)nnz));
            PLAN_TRY(dev_alloc(p, &p->d_ht_off, (size_t)n_tiles + 1));
            PLAN_TRY(build_tiled_order(p->d_rows, p->d_cols, nnz, N, tc, p->d_ht_perm, p->d_ht_rows, p->d_ht_cols, s));
            PLAN_TRY(build_htile_offsets(p->d_ht_cols, nnz, tc, (int)n_tiles, p->d_ht_off, s));
            p->ht_col_tile = tc;
            p->ht_n_tiles = (int)n_tiles;
        }
    }
    // Host-operand pipeline (sddmm_execute with W in host memory): cut S into chunks
    // of consecutive nonzeros, about 128 MB of W rows each, and note the first and
    // last row of every chunk -- rows are sorted, so a chunk needs one contiguous
    // block of W rows, and W rows between two chunks that no nonzero touches are
    // never uploaded.
    if (ring_supports(K) && p->n_col_tiles == 1 && p->dense.n_cells == 0 && nnz >= (1 << 20)) {
        int64_t chunks = (int64_t)sizeof(float) * M * K / (128ll << 20);
        if (chunks > SDDMM_PIPE_MAX_CHUNKS) chunks = SDDMM_PIPE_MAX_CHUNKS;
        if (chunks >= 2) {
            for (int i = 0; i < chunks; ++i) p->pipe_nnz[i] = (nnz * i / chunks) & ~(int64_t)31;
            p->pipe_nnz[chunks] = nnz;
            for (int i = 0; i < chunks; ++i) {
                PLAN_TRY(cudaMemcpyAsync(&p->pipe_row_first[i], p->d_rows + p->pipe_nnz[i], sizeof(int32_t),
                                         cudaMemcpyDeviceToHost, s));
                PLAN_TRY(cudaMemcpyAsync(&p->pipe_row_last[i], p->d_rows + p->pipe_nnz[i + 1] - 1, sizeof(int32_t),
                                         cudaMemcpyDeviceToHost, s));
            }
            p->n_pipe = (int)chunks;
            // the rows of W and H that are read at all, for the row upload from mapped host memory
            PLAN_TRY(build_used_row_list(p->d_row_ptr, M, &p->d_used_rows, &p->n_used_rows, s));
            PLAN_TRY(build_used_col_list(p->d_cols, nnz, N, &p->d_used_cols, &p->n_used_cols, s));
            p->device_bytes += (int64_t)sizeof(int32_t) * (p->n_used_rows + p->n_used_cols);
            std::vector<int32_t> used;
            try {
                used.resize((size_t)p->n_used_rows);
            } catch (const std::bad_alloc &) {
                PLAN_TRY(cudaErrorMemoryAllocation);
            }
            PLAN_TRY(cudaMemcpyAsync(used.data(), p->d_used_rows, sizeof(int32_t) * used.size(), cudaMemcpyDeviceToHost, s));
            PLAN_TRY(cudaStreamSynchronize(s));  // also completes the copies of the chunks' first and last rows
            int64_t next_row = 0;  // first row of W no earlier chunk uploads
            for (int i = 0; i < chunks; ++i) {
                const int64_t r0 = p->pipe_row_first[i] > next_row ? p->pipe_row_first[i] : next_row;
                const int64_t r1 = (int64_t)p->pipe_row_last[i] + 1;
                p->pipe_w_begin[i] = r0;
                p->pipe_w_end[i] = r1 > r0 ? r1 : r0;
                p->pipe_list_begin[i] = std::lower_bound(used.begin(), used.end(), (int32_t)r0) - used.begin();
                if (r1 > next_row) next_row = r1;
            }
            p->pipe_list_begin[chunks] = (int64_t)used.size();
        }
    }
    PLAN_TRY(cudaEventRecord(t1, s));
    PLAN_TRY(cudaEventSynchronize(t1));
    PLAN_TRY(cudaEventElapsedTime(&p->plan_ms, t0, t1));
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
#undef PLAN_TRY
    *out = p;
    return SDDMM_OK;
}

int sddmm_destroy_plan(sddmm_plan_t p)
{
    if (!p) return SDDMM_OK;
    cudaSetDevice(p->h->device);
    cudaStreamSynchronize(p->h->stream);
    free_plan_memory(p);
    (void)cudaGetLastError();
    delete p;
    return SDDMM_OK;
}

int sddmm_execute(sddmm_plan_t p, const float *W, const float *H, const float *Sval, float *P, uint32_t flags)
{
    if (!p) return SDDMM_INVALID_ARG;
    sddmm_handle_s *h = p->h;
    if (p->nnz == 0) { p->last_ms = 0.f; return SDDMM_OK; }
    if (!W || !H || !P) return SDDMM_INVALID_ARG;
    const bool use_gather = (flags & SDDMM_FLAG_KERNEL_GATHER) != 0;
    const bool tiled_out = (flags & SDDMM_FLAG_TILED_ORDER) != 0;
    const uint32_t forced = flags & (SDDMM_FLAG_KERNEL_GATHER | SDDMM_FLAG_KERNEL_PANEL | SDDMM_FLAG_KERNEL_RING);
    if (forced & (forced - 1)) return SDDMM_INVALID_ARG;  // at most one kernel may be forced
    if ((flags & SDDMM_FLAG_KERNEL_RING) && !ring_supports(p->K)) return SDDMM_K_UNSUPPORTED;
    // tiny inputs are launch-bound: the panel kernel needs no counter reset and starts faster
    const bool use_ring = (flags & SDDMM_FLAG_KERNEL_RING) || (!forced && ring_supports(p->K) && p->nnz >= 65536);
    if (use_gather && tiled_out && p->d_perm) return SDDMM_INVALID_ARG;
    CUDA_TRY(h, cudaSetDevice(h->device));
    cudaStream_t s = h->stream;

    const bool w_dev = is_device_ptr(W), h_dev = is_device_ptr(H), p_dev = is_device_ptr(P);
    const bool s_dev = Sval ? is_device_ptr(Sval) : true;
    const bool all_dev = w_dev && h_dev && p_dev && s_dev;
    if ((flags & SDDMM_FLAG_ASYNC) && !all_dev) return SDDMM_INVALID_ARG;

    if (flags & SDDMM_FLAG_OPERANDS_BF16) {
        // W and H hold bfloat16: the TMA rings over rows of 2K bytes, products and sums in fp32.  Opt-in and
        // outside the fp32 tolerance contract; device arrays only, no other layout or kernel flag.
        if (!ring_bf16_supports(p->K)) return SDDMM_K_UNSUPPORTED;
        if (!all_dev || (flags & ~(uint32_t)(SDDMM_FLAG_OPERANDS_BF16 | SDDMM_FLAG_ASYNC | SDDMM_FLAG_KERNEL_RING))) {
            h->last_error = "SDDMM_FLAG_OPERANDS_BF16 takes device arrays and no flag but ASYNC / KERNEL_RING";
            return SDDMM_INVALID_ARG;
        }
        if ((((uintptr_t)W | (uintptr_t)H) & 15u) != 0) {
            h->last_error = "W and H must be 16-byte aligned on the device";
            return SDDMM_INVALID_ARG;
        }
        const bool tiled = p->d_perm != nullptr;
        const int32_t *rows_p = tiled ? p->d_rows_t : p->d_rows;
        const int32_t *cols_p = p->d_cols_hint ? p->d_cols_hint : (tiled ? p->d_cols_t : p->d_cols);
        p->last_kernel = "ring (bf16 operands)";
        p->last_h2d_bytes = p->last_d2h_bytes = 0;
        CUDA_TRY(h, cudaEventRecord(h->ev0, s));
        LAUNCH_TRY(h, launch_ring_bf16(rows_p, cols_p, tiled ? p->d_perm : nullptr, Sval, W, H, P, p->nnz, p->K,
                                       p->d_cols_hint != nullptr, h->sm_count, h->d_work_counter, h->d_status, s));
        CUDA_TRY(h, cudaEventRecord(h->ev1, s));
        if (flags & SDDMM_FLAG_ASYNC) {
            p->last_ms = -1.f;
            return SDDMM_OK;
        }
        CUDA_TRY(h, cudaMemcpyAsync(h->h_status, h->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
        CUDA_TRY(h, cudaStreamSynchronize(s));
        CUDA_TRY(h, cudaEventElapsedTime(&p->last_ms, h->ev0, h->ev1));
        return check_device_status(h);
    }
    const float *dW = W, *dH = H, *dS = Sval;
    float *dP = P;
    const size_t wbytes = sizeof(float) * (size_t)p->M * p->K, hbytes = sizeof(float) * (size_t)p->N * p->K;
    const size_t nbytes = sizeof(float) * (size_t)p->nnz;
    // W in host memory and a plain ring-kernel plan: upload W (and S) chunk by chunk
    // and let every chunk's kernel and download run behind the later uploads
    const bool w_t = (flags & SDDMM_FLAG_W_TRANSPOSED) != 0, h_t = (flags & SDDMM_FLAG_H_TRANSPOSED) != 0;
    const bool pipelined = h->pipeline && p->n_pipe > 0 && !w_dev && use_ring && !tiled_out && !p->d_perm &&
                           p->dense.n_cells == 0 && !w_t && !h_t;
    // page-locked, mapped host arrays are read row by row by the GPU: only the rows a nonzero touches travel
    const float *W_mapped = (pipelined && h->sparse_upload) ? mapped_host_ptr(W) : nullptr;
    const float *H_mapped = (pipelined && h->sparse_upload && !h_dev) ? mapped_host_ptr(H) : nullptr;
    p->last_h2d_bytes = p->last_d2h_bytes = 0;
    // K-major operands (the layout make_HTasH builds, util.h:68-73): brought to the device if need be and
    // transposed there into the plan's row-major staging copy
    if (h_t) {
        const float *src = H;
        if (!h_dev) {
            if (!p->d_Ht) CUDA_TRY(h, dev_alloc(p, &p->d_Ht, (size_t)p->N * p->K));
            CUDA_TRY(h, cudaMemcpyAsync(p->d_Ht, H, hbytes, cudaMemcpyHostToDevice, s));
            p->last_h2d_bytes += (int64_t)hbytes;
            src = p->d_Ht;
        }
        if (!p->d_H) CUDA_TRY(h, dev_alloc(p, &p->d_H, (size_t)p->N * p->K));
        LAUNCH_TRY(h, launch_transpose_operand(src, p->d_H, p->N, p->K, s));
        dH = p->d_H;
    } else if (!h_dev) {
        if (!p->d_H) CUDA_TRY(h, dev_alloc(p, &p->d_H, (size_t)p->N * p->K));
        if (H_mapped) {
            LAUNCH_TRY(h, launch_upload_rows(H_mapped, p->d_H, p->d_used_cols, p->n_used_cols, p->K, h->upload_ctas, s));
            p->last_h2d_bytes += (int64_t)sizeof(float) * p->n_used_cols * p->K;
        } else {
            CUDA_TRY(h, cudaMemcpyAsync(p->d_H, H, hbytes, cudaMemcpyHostToDevice, s));
            p->last_h2d_bytes += (int64_t)hbytes;
        }
        dH = p->d_H;
    }
    if (w_t) {
        const float *src = W;
        if (!w_dev) {
            if (!p->d_Wt) CUDA_TRY(h, dev_alloc(p, &p->d_Wt, (size_t)p->M * p->K));
            CUDA_TRY(h, cudaMemcpyAsync(p->d_Wt, W, wbytes, cudaMemcpyHostToDevice, s));
            p->last_h2d_bytes += (int64_t)wbytes;
            src = p->d_Wt;
        }
        if (!p->d_W) CUDA_TRY(h, dev_alloc(p, &p->d_W, (size_t)p->M * p->K));
        LAUNCH_TRY(h, launch_transpose_operand(src, p->d_W, p->M, p->K, s));
        dW = p->d_W;
    } else if (!w_dev) {
        if (!p->d_W) CUDA_TRY(h, dev_alloc(p, &p->d_W, (size_t)p->M * p->K));
        if (!pipelined) {
            CUDA_TRY(h, cudaMemcpyAsync(p->d_W, W, wbytes, cudaMemcpyHostToDevice, s));
            p->last_h2d_bytes += (int64_t)wbytes;
        }
        dW = p->d_W;
    }
    if (Sval && !s_dev) {
        if (!p->d_S) CUDA_TRY(h, dev_alloc(p, &p->d_S, (size_t)p->nnz));
        if (!pipelined) CUDA_TRY(h, cudaMemcpyAsync(p->d_S, Sval, nbytes, cudaMemcpyHostToDevice, s));
        p->last_h2d_bytes += (int64_t)nbytes;
        dS = p->d_S;
    }
    if (!p_dev) {
        if (!p->d_P) CUDA_TRY(h, dev_alloc(p, &p->d_P, (size_t)p->nnz));
        dP = p->d_P;
        p->last_d2h_bytes = (int64_t)nbytes;
    }

    // every kernel moves 16-byte vectors
    if ((((uintptr_t)dW | (uintptr_t)dH) & 15u) != 0) {
        h->last_error = "W and H must be 16-byte aligned on the device";
        return SDDMM_INVALID_ARG;
    }
    const char *ring_name = p->K <= 128 ? "ring_small" : "ring";
    if (pipelined) {
        p->last_kernel = p->K <= 128 ? "ring_small (pipelined chunks)" : "ring (pipelined chunks)";
        CUDA_TRY(h, ensure_pipeline(h));
        const int32_t *cols_p = p->d_cols_hint ? p->d_cols_hint : p->d_cols;
        for (int i = 0; i < p->n_pipe; ++i) {
            const int64_t n0 = p->pipe_nnz[i], cnt = p->pipe_nnz[i + 1] - n0;
            const int64_t r0 = p->pipe_w_begin[i], r1 = p->pipe_w_end[i];
            if (W_mapped) {
                const int64_t l0 = p->pipe_list_begin[i], ln = p->pipe_list_begin[i + 1] - l0;
                LAUNCH_TRY(h, launch_upload_rows(W_mapped, p->d_W, p->d_used_rows + l0, ln, p->K, h->upload_ctas, s));
                p->last_h2d_bytes += (int64_t)sizeof(float) * ln * p->K;
            } else if (r1 > r0) {
                CUDA_TRY(h, cudaMemcpyAsync(p->d_W + r0 * p->K, W + r0 * p->K, sizeof(float) * (size_t)(r1 - r0) * p->K,
                                            cudaMemcpyHostToDevice, s));
                p->last_h2d_bytes += (int64_t)sizeof(float) * (r1 - r0) * p->K;
            }
            if (Sval && !s_dev)
                CUDA_TRY(h, cudaMemcpyAsync(p->d_S + n0, Sval + n0, sizeof(float) * (size_t)cnt, cudaMemcpyHostToDevice, s));
            CUDA_TRY(h, cudaEventRecord(h->pipe_uploaded[i], s));
            CUDA_TRY(h, cudaStreamWaitEvent(h->pipe_compute, h->pipe_uploaded[i], 0));
            CUDA_TRY(h, cudaEventRecord(h->pipe_started[i], h->pipe_compute));
            LAUNCH_TRY(h, launch_rows_gather(h, p->d_rows + n0, cols_p + n0, nullptr, dS ? dS + n0 : nullptr, dW, dH, dP + n0,
                                             cnt, p->K, p->d_cols_hint != nullptr, h->pipe_compute));
            CUDA_TRY(h, cudaEventRecord(h->pipe_computed[i], h->pipe_compute));
            if (!p_dev) {
                CUDA_TRY(h, cudaStreamWaitEvent(h->pipe_download, h->pipe_computed[i], 0));
                CUDA_TRY(h, cudaMemcpyAsync(P + n0, dP + n0, sizeof(float) * (size_t)cnt, cudaMemcpyDeviceToHost,
                                            h->pipe_download));
            }
        }
        // the caller's stream continues only after the last kernel and the last download
        cudaStream_t last = p_dev ? h->pipe_compute : h->pipe_download;
        CUDA_TRY(h, cudaEventRecord(h->pipe_joined, last));
        CUDA_TRY(h, cudaStreamWaitEvent(s, h->pipe_joined, 0));
        CUDA_TRY(h, cudaMemcpyAsync(h->h_status, h->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
        CUDA_TRY(h, cudaStreamSynchronize(s));
        p->last_ms = 0.f;  // kernel time only: the chunks' kernels, not the waits for uploads between them
        for (int i = 0; i < p->n_pipe; ++i) {
            float ms = 0.f;
            CUDA_TRY(h, cudaEventElapsedTime(&ms, h->pipe_started[i], h->pipe_computed[i]));
            p->last_ms += ms;
        }
        return check_device_status(h);
    }
    CUDA_TRY(h, cudaEventRecord(h->ev0, s));
    if (!forced && !tiled_out && p->dense.n_cells > 0) {
        // locally dense plan: dense cells as small dense products, the rest gathered
        {
            static const char *const names[3][3] = {
                {"dense_fma", "dense_fma+ring", "dense_fma+panel"},
                {"dense_mma_sync", "dense_mma_sync+ring", "dense_mma_sync+panel"},
                {"dense_tc", "dense_tc+ring", "dense_tc+panel"}};
            const int rest = p->dense.n_sparse == 0 ? 0 : (ring_supports(p->K) ? 1 : 2);
            p->last_kernel = names[h->dense_mode][rest];
            if (rest == 1 && p->K <= 128)
                p->last_kernel = h->dense_mode == 2 ? "dense_tc+ring_small"
                                                    : (h->dense_mode == 1 ? "dense_mma_sync+ring_small" : "dense_fma+ring_small");
        }
        if (h->dense_mode == 2)
            LAUNCH_TRY(h, launch_dense_cells_tc(p->dense.cells, p->dense.n_cells, p->dense.idx, p->dense.rc, p->dense.row_mask,
                                              p->dense.row_base, p->dense.dense_rows, p->dense.n_dense_rows,
                                              p->dense.dense_cols, p->dense.n_dense_cols, dS, dW, dH, dP, p->M, p->N, p->K,
                                              h->sm_count, h->d_status, s));
        else
            LAUNCH_TRY(h, launch_dense_cells(p->dense.cells, p->dense.n_cells, p->dense.idx, p->dense.rc, p->dense.row_mask,
                                           p->dense.row_base, p->dense.dense_rows, p->dense.n_dense_rows,
                                           p->dense.dense_cols, p->dense.n_dense_cols, dS, dW, dH, dP, p->M, p->N, p->K,
                                           h->dense_mode == 1, h->sm_count, s));
        if (p->dense.n_sparse > 0) {
            if (ring_supports(p->K))
                LAUNCH_TRY(h, launch_rows_gather(h, p->dense.rows_s, p->dense.cols_s, p->dense.perm_s, dS, dW, dH, dP,
                                                 p->dense.n_sparse, p->K, false, s));
            else
                LAUNCH_TRY(h, launch_panel(p->d_items_s, p->n_items_s, p->d_item_rows_s, p->dense.rows_s, p->dense.cols_s,
                                         p->dense.perm_s, dS, dW, dH, dP, p->K, p->cfg, h->sm_count, h->d_status, s));
        }
    } else if (use_gather) {
        p->last_kernel = "gather";
        LAUNCH_TRY(h, launch_gather(p->d_rows, p->d_cols, dS, dW, dH, dP, p->nnz, p->K, h->sm_count, s));
    } else {
        const bool tiled = p->d_perm != nullptr;
        const int32_t *rows_p = tiled ? p->d_rows_t : p->d_rows;
        const int32_t *cols_p = tiled ? p->d_cols_t : p->d_cols;
        // tiled processing order: results go back to input order through the
        // permutation unless the caller asked for the tiled order itself
        const int32_t *perm = (tiled && !tiled_out) ? p->d_perm : nullptr;
        if (tiled && tiled_out && dS) {
            // S values are in input order; the tiled-order result is produced
            // unscaled only (what the reference's kernel leaves in d_val)
            h->last_error = "SDDMM_FLAG_TILED_ORDER with S values is not supported on a multi-tile plan";
            return SDDMM_INVALID_ARG;
        }
        const bool use_htile = p->d_ht_off && !forced && !tiled && ((reinterpret_cast<uintptr_t>(dW) | reinterpret_cast<uintptr_t>(dH)) & 15u) == 0;
        p->last_kernel = use_htile ? "htile" : use_ring ? ring_name : "panel";
        if (use_htile)
            LAUNCH_TRY(h, launch_htile(p->d_ht_rows, p->d_ht_cols, p->d_ht_perm, dS, dW, dH, dP, p->nnz, p->N, p->K, p->ht_col_tile,
                                       p->d_ht_off, p->ht_n_tiles, h->sm_count, h->d_status, s));
        else if (use_ring)
            LAUNCH_TRY(h, launch_rows_gather(h, rows_p, p->d_cols_hint ? p->d_cols_hint : cols_p, perm, dS, dW, dH, dP, p->nnz,
                                             p->K, p->d_cols_hint != nullptr, s));
        else
            LAUNCH_TRY(h, launch_panel(p->d_items, p->n_items, p->d_item_rows, rows_p, cols_p, perm, dS, dW, dH, dP, p->K,
                                     p->cfg, h->sm_count, h->d_status, s));
    }
    CUDA_TRY(h, cudaEventRecord(h->ev1, s));
    if (!p_dev) CUDA_TRY(h, cudaMemcpyAsync(P, dP, nbytes, cudaMemcpyDeviceToHost, s));
    if (flags & SDDMM_FLAG_ASYNC) {
        p->last_ms = -1.f;
        return SDDMM_OK;
    }
    CUDA_TRY(h, cudaMemcpyAsync(h->h_status, h->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
    CUDA_TRY(h, cudaStreamSynchronize(s));
    CUDA_TRY(h, cudaEventElapsedTime(&p->last_ms, h->ev0, h->ev1));
    return check_device_status(h);
}

int sddmm_coo_sort_rows_gpu(sddmm_handle_t h, int64_t *M, int64_t *N, int64_t nnz, int32_t *rows, int32_t *cols,
                            float *vals, int transpose)
{
    if (!h || !M || !N || nnz < 0 || nnz >= INT32_MAX || (nnz > 0 && (!rows || !cols || !vals))) return SDDMM_INVALID_ARG;
    if (nnz > 0) {
        CUDA_TRY(h, cudaSetDevice(h->device));
        cudaStream_t s = h->stream;
        const bool idx_dev = is_device_ptr(rows), val_dev = is_device_ptr(vals);
        if (idx_dev != is_device_ptr(cols)) {
            h->last_error = "sddmm_coo_sort_rows_gpu: rows and cols must both be host or both be device arrays";
            return SDDMM_INVALID_ARG;
        }
        struct Tmp {
            void *p[3] = {nullptr, nullptr, nullptr};
            ~Tmp() { for (void *q : p) if (q) cudaFree(q); }
        } tmp;
        const size_t bytes = 4 * (size_t)nnz;
        int32_t *d_rows = rows, *d_cols = cols;
        float *d_vals = vals;
        if (!idx_dev) {
            CUDA_TRY(h, cudaMalloc(&tmp.p[0], bytes));
            CUDA_TRY(h, cudaMalloc(&tmp.p[1], bytes));
            d_rows = (int32_t *)tmp.p[0];
            d_cols = (int32_t *)tmp.p[1];
            CUDA_TRY(h, cudaMemcpyAsync(d_rows, rows, bytes, cudaMemcpyHostToDevice, s));
            CUDA_TRY(h, cudaMemcpyAsync(d_cols, cols, bytes, cudaMemcpyHostToDevice, s));
        }
        if (!val_dev) {
            CUDA_TRY(h, cudaMalloc(&tmp.p[2], bytes));
            d_vals = (float *)tmp.p[2];
            CUDA_TRY(h, cudaMemcpyAsync(d_vals, vals, bytes, cudaMemcpyHostToDevice, s));
        }
        // transposing: the reference sorts whole (col, row, val) tuples and then swaps the roles
        // (util.h:88-104): the old columns become the rows of the result
        if (transpose) CUDA_TRY(h, sort_coo(d_cols, d_rows, d_vals, nnz, true, s));
        else CUDA_TRY(h, sort_coo(d_rows, d_cols, d_vals, nnz, false, s));
        const int32_t *new_rows = transpose ? d_cols : d_rows, *new_cols = transpose ? d_rows : d_cols;
        if (!idx_dev) {
            CUDA_TRY(h, cudaMemcpyAsync(rows, new_rows, bytes, cudaMemcpyDeviceToHost, s));
            CUDA_TRY(h, cudaMemcpyAsync(cols, new_cols, bytes, cudaMemcpyDeviceToHost, s));
        } else if (transpose) {
            // device arrays: exchange the contents of rows and cols through a scratch copy
            CUDA_TRY(h, cudaMalloc(&tmp.p[0], bytes));
            CUDA_TRY(h, cudaMemcpyAsync(tmp.p[0], rows, bytes, cudaMemcpyDeviceToDevice, s));
            CUDA_TRY(h, cudaMemcpyAsync(rows, cols, bytes, cudaMemcpyDeviceToDevice, s));
            CUDA_TRY(h, cudaMemcpyAsync(cols, tmp.p[0], bytes, cudaMemcpyDeviceToDevice, s));
        }
        if (!val_dev) CUDA_TRY(h, cudaMemcpyAsync(vals, d_vals, bytes, cudaMemcpyDeviceToHost, s));
        CUDA_TRY(h, cudaStreamSynchronize(s));
    }
    if (transpose) std::swap(*M, *N);
    return SDDMM_OK;
}

int sddmm_plan_used_lines(sddmm_plan_t p, int which, const int32_t **d_ids, int64_t *n)
{
    if (!p || !d_ids || !n || (which != 0 && which != 1)) return SDDMM_INVALID_ARG;
    sddmm_handle_s *h = p->h;
    *d_ids = nullptr;
    *n = 0;
    if (p->nnz == 0) return SDDMM_OK;
    CUDA_TRY(h, cudaSetDevice(h->device));
    if (which == 0) {
        if (!p->d_used_rows) {
            CUDA_TRY(h, build_used_row_list(p->d_row_ptr, p->M, &p->d_used_rows, &p->n_used_rows, h->stream));
            p->device_bytes += (int64_t)sizeof(int32_t) * p->n_used_rows;
        }
        *d_ids = p->d_used_rows;
        *n = p->n_used_rows;
    } else {
        if (!p->d_used_cols) {
            CUDA_TRY(h, build_used_col_list(p->d_cols, p->nnz, p->N, &p->d_used_cols, &p->n_used_cols, h->stream));
            p->device_bytes += (int64_t)sizeof(int32_t) * p->n_used_cols;
        }
        *d_ids = p->d_used_cols;
        *n = p->n_used_cols;
    }
    return SDDMM_OK;
}

int sddmm_upload_rows(sddmm_handle_t h, const float *host, float *dev, const int32_t *d_row_ids, int64_t n_rows, int K,
                      void *cuda_stream)
{
    if (!h || n_rows < 0) return SDDMM_INVALID_ARG;
    int st = check_k(K);
    if (st != SDDMM_OK) return st;
    if (n_rows == 0) return SDDMM_OK;
    if (!host || !dev || !d_row_ids) return SDDMM_INVALID_ARG;
    CUDA_TRY(h, cudaSetDevice(h->device));
    const float *mapped = mapped_host_ptr(host);
    if (!mapped) {
        h->last_error = "sddmm_upload_rows needs page-locked, mapped host memory (cudaHostAlloc / cudaHostRegister)";
        return SDDMM_INVALID_ARG;
    }
    if (!is_device_ptr(dev) || !is_device_ptr(d_row_ids) || (((uintptr_t)mapped | (uintptr_t)dev) & 15u) != 0) {
        h->last_error = "sddmm_upload_rows: dev and d_row_ids must be device memory, both arrays 16-byte aligned";
        return SDDMM_INVALID_ARG;
    }
    LAUNCH_TRY(h, launch_upload_rows(mapped, dev, d_row_ids, n_rows, K, h->upload_ctas,
                                   cuda_stream ? (cudaStream_t)cuda_stream : h->stream));
    return SDDMM_OK;
}

int sddmm_last_transfer_bytes(sddmm_plan_t p, int64_t *h2d_bytes, int64_t *d2h_bytes)
{
    if (!p) return SDDMM_INVALID_ARG;
    if (h2d_bytes) *h2d_bytes = p->last_h2d_bytes;
    if (d2h_bytes) *d2h_bytes = p->last_d2h_bytes;
    return SDDMM_OK;
}

int sddmm_kernel_launches(sddmm_handle_t h, int64_t *n)
{
    if (!h || !n) return SDDMM_INVALID_ARG;
    *n = h->n_launches;
    return SDDMM_OK;
}

const char *sddmm_last_kernel_name(sddmm_plan_t p) { return p ? p->last_kernel : ""; }

int sddmm_sync(sddmm_handle_t h)
{
    if (!h) return SDDMM_INVALID_ARG;
    CUDA_TRY(h, cudaSetDevice(h->device));
    CUDA_TRY(h, cudaMemcpyAsync(h->h_status, h->d_status, sizeof(int), cudaMemcpyDeviceToHost, h->stream));
    CUDA_TRY(h, cudaStreamSynchronize(h->stream));
    return check_device_status(h);
}

int sddmm_check_result(sddmm_plan_t p, const float *W, const float *H, const float *Sval, const float *P,
                       int64_t stride, double tol, double *max_scaled_err, int64_t *n_checked, int64_t *n_bad)
{
    if (!p || stride < 1 || !(tol > 0)) return SDDMM_INVALID_ARG;
    sddmm_handle_s *h = p->h;
    if (max_scaled_err) *max_scaled_err = 0.0;
    if (n_checked) *n_checked = 0;
    if (n_bad) *n_bad = 0;
    if (p->nnz == 0) return SDDMM_OK;
    if (!W || !H || !P) return SDDMM_INVALID_ARG;
    CUDA_TRY(h, cudaSetDevice(h->device));
    // host arrays are staged for this call only
    struct Tmp {
        void *p[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
        ~Tmp() { for (void *q : p) if (q) cudaFree(q); }
    } tmp;
    auto stage = [&](int slot, const float *src, size_t count, const float **dst) -> cudaError_t {
        if (!src || is_device_ptr(src)) { *dst = src; return cudaSuccess; }
        cudaError_t e = cudaMalloc(&tmp.p[slot], sizeof(float) * (count ? count : 1));
        if (e != cudaSuccess) return e;
        *dst = (const float *)tmp.p[slot];
        return cudaMemcpyAsync(tmp.p[slot], src, sizeof(float) * count, cudaMemcpyHostToDevice, h->stream);
    };
    const float *dW, *dH, *dS, *dP;
    CUDA_TRY(h, stage(0, W, (size_t)p->M * p->K, &dW));
    CUDA_TRY(h, stage(1, H, (size_t)p->N * p->K, &dH));
    CUDA_TRY(h, stage(2, Sval, (size_t)p->nnz, &dS));
    CUDA_TRY(h, stage(3, P, (size_t)p->nnz, &dP));
    CheckResult host{};
    CUDA_TRY(h, cudaMalloc(&tmp.p[4], sizeof(CheckResult)));
    CheckResult *d_out = (CheckResult *)tmp.p[4];
    cudaError_t e = launch_check_result(p->d_rows, p->d_cols, dS, dW, dH, dP, p->nnz, p->K, stride, tol, d_out, h->sm_count,
                                        h->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&host, d_out, sizeof(host), cudaMemcpyDeviceToHost, h->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
    if (e != cudaSuccess) return fail_cuda(h, e, "sddmm_check_result");
    if (max_scaled_err) *max_scaled_err = host.max_scaled_err;
    if (n_checked) *n_checked = (int64_t)host.n_checked;
    if (n_bad) *n_bad = (int64_t)host.n_bad;
    return SDDMM_OK;
}

namespace {

// Tasks of the SpMM kernels, built once per plan from the row pointer (host side: one pass over M + 1 offsets).
int ensure_spmm_tasks(sddmm_plan_s *p)
{
    if (p->n_spmm_tasks >= 0) return SDDMM_OK;
    sddmm_handle_s *h = p->h;
    std::vector<int64_t> rp;
    std::vector<SpmmTask> tasks;
    std::vector<SpmmLongRow> long_rows;
    try {
        rp.resize((size_t)p->M + 1);
    } catch (const std::bad_alloc &) {
        return SDDMM_OUT_OF_MEMORY;
    }
    CUDA_TRY(h, cudaMemcpyAsync(rp.data(), p->d_row_ptr, sizeof(int64_t) * rp.size(), cudaMemcpyDeviceToHost, h->stream));
    CUDA_TRY(h, cudaStreamSynchronize(h->stream));
    int64_t slots = 0;
    try {
        build_spmm_tasks(rp.data(), p->M, tasks, long_rows, &slots);
    } catch (const std::bad_alloc &) {
        return SDDMM_OUT_OF_MEMORY;
    }
    CUDA_TRY(h, dev_alloc(p, &p->d_spmm_tasks, tasks.size()));
    CUDA_TRY(h, dev_alloc(p, &p->d_spmm_long, long_rows.size()));
    CUDA_TRY(h, dev_alloc(p, &p->d_spmm_scratch, (size_t)slots * p->K));
    if (!tasks.empty())
        CUDA_TRY(h, cudaMemcpyAsync(p->d_spmm_tasks, tasks.data(), sizeof(SpmmTask) * tasks.size(), cudaMemcpyHostToDevice, h->stream));
    if (!long_rows.empty())
        CUDA_TRY(h, cudaMemcpyAsync(p->d_spmm_long, long_rows.data(), sizeof(SpmmLongRow) * long_rows.size(),
                                    cudaMemcpyHostToDevice, h->stream));
    CUDA_TRY(h, cudaStreamSynchronize(h->stream));
    p->n_spmm_tasks = (int64_t)tasks.size();
    p->n_spmm_long = (int64_t)long_rows.size();
    p->n_spmm_slots = slots;
    return SDDMM_OK;
}

// The ring form's plan data: row groups (device), tasks over groups (host from the groups' row offsets).
int ensure_spmm_ring(sddmm_plan_s *p)
{
    if (p->n_spmr_tasks >= 0) return SDDMM_OK;
    sddmm_handle_s *h = p->h;
    std::vector<int64_t> gstart;
    std::vector<SpmmTask> tasks;
    std::vector<SpmmLongRow> long_rows;
    int64_t slots = 0;
    try {
        CUDA_TRY(h, build_row_groups(p->d_rows, p->d_cols, p->d_row_ptr, p->nnz, p->M, spmm_ring_group_slots(p->K), &p->row_groups,
                                     &gstart, h->stream));
        build_spmm_tasks(gstart.data(), p->M, tasks, long_rows, &slots, /*groups per task*/ 256);
    } catch (const std::bad_alloc &) {
        return SDDMM_OUT_OF_MEMORY;
    }
    p->device_bytes += (int64_t)(p->row_groups.n_groups * (8 * p->row_groups.B + 4));
    CUDA_TRY(h, dev_alloc(p, &p->d_spmr_tasks, tasks.size()));
    CUDA_TRY(h, dev_alloc(p, &p->d_spmr_long, long_rows.size()));
    CUDA_TRY(h, dev_alloc(p, &p->d_spmr_scratch, (size_t)slots * p->K));
    if (!tasks.empty())
        CUDA_TRY(h, cudaMemcpyAsync(p->d_spmr_tasks, tasks.data(), sizeof(SpmmTask) * tasks.size(), cudaMemcpyHostToDevice, h->stream));
    if (!long_rows.empty())
        CUDA_TRY(h, cudaMemcpyAsync(p->d_spmr_long, long_rows.data(), sizeof(SpmmLongRow) * long_rows.size(),
                                    cudaMemcpyHostToDevice, h->stream));
    CUDA_TRY(h, cudaStreamSynchronize(h->stream));
    p->n_spmr_tasks = (int64_t)tasks.size();
    p->n_spmr_long = (int64_t)long_rows.size();
    return SDDMM_OK;
}

// Y = P H (fused: P = S o (W H^T) on the fly).  Host arrays are staged for the call.
int run_spmm(sddmm_plan_s *p, bool fused, const float *W, const float *H, const float *pval, float *P_out, float *Y,
             uint32_t flags)
{
    sddmm_handle_s *h = p->h;
    if (!spmm_supports(p->K)) return SDDMM_K_UNSUPPORTED;
    if (!H || !Y || (fused && !W)) return SDDMM_INVALID_ARG;
    if (flags & ~(uint32_t)SDDMM_FLAG_ASYNC) return SDDMM_INVALID_ARG;
    CUDA_TRY(h, cudaSetDevice(h->device));
    // long rows on the shared-memory rings (SDDMM_SPMM_RING=0: the register-staged kernel for every K)
    bool ring = spmm_ring_supports(p->K) && p->nnz >= 65536;
    if (const char *env = std::getenv("SDDMM_SPMM_RING")) ring = ring && std::atoi(env) != 0;
    int st = ring ? ensure_spmm_ring(p) : ensure_spmm_tasks(p);
    if (st != SDDMM_OK) return st;
    cudaStream_t s = h->stream;
    struct Tmp {
        void *p[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
        ~Tmp() { for (void *q : p) if (q) cudaFree(q); }
    } tmp;
    auto stage_in = [&](int slot, const float *src, size_t count, const float **dst) -> cudaError_t {
        if (!src || is_device_ptr(src)) { *dst = src; return cudaSuccess; }
        cudaError_t e = cudaMalloc(&tmp.p[slot], sizeof(float) * (count ? count : 1));
        if (e != cudaSuccess) return e;
        *dst = (const float *)tmp.p[slot];
        return cudaMemcpyAsync(tmp.p[slot], src, sizeof(float) * count, cudaMemcpyHostToDevice, s);
    };
    const size_t mk = (size_t)p->M * p->K, nk = (size_t)p->N * p->K, nz = (size_t)p->nnz;
    const float *dW = nullptr, *dH = nullptr, *dV = nullptr;
    CUDA_TRY(h, stage_in(0, W, mk, &dW));
    CUDA_TRY(h, stage_in(1, H, nk, &dH));
    CUDA_TRY(h, stage_in(2, pval, nz, &dV));
    float *dY = Y, *dP = P_out;
    const bool y_dev = is_device_ptr(Y), p_dev = P_out ? is_device_ptr(P_out) : true;
    if ((flags & SDDMM_FLAG_ASYNC) && (!y_dev || !p_dev || tmp.p[0] || tmp.p[1] || tmp.p[2])) return SDDMM_INVALID_ARG;
    if (!y_dev) {
        CUDA_TRY(h, cudaMalloc(&tmp.p[3], sizeof(float) * (mk ? mk : 1)));
        dY = (float *)tmp.p[3];
    }
    if (P_out && !p_dev) {
        CUDA_TRY(h, cudaMalloc(&tmp.p[4], sizeof(float) * (nz ? nz : 1)));
        dP = (float *)tmp.p[4];
    }
    if ((((uintptr_t)dW | (uintptr_t)dH | (uintptr_t)dY) & 15u) != 0) {
        h->last_error = "W, H and Y must be 16-byte aligned on the device";
        return SDDMM_INVALID_ARG;
    }
    CUDA_TRY(h, cudaEventRecord(h->ev0, s));
    if (p->M > 0 && ring) {
        LAUNCH_TRY(h, launch_spmm_ring(fused, p->d_spmr_tasks, p->n_spmr_tasks, p->row_groups.pcols, p->row_groups.pidx,
                                       p->row_groups.grow, dV, dW, dH, dP, dY, p->d_spmr_scratch, p->K, h->d_work_counter,
                                       h->d_status, h->sm_count, s));
        LAUNCH_TRY(h, launch_spmm_fixup(p->d_spmr_long, p->n_spmr_long, p->d_spmr_scratch, dY, p->K, s));
    } else if (p->M > 0) {
        LAUNCH_TRY(h, launch_spmm(fused, p->d_spmm_tasks, p->n_spmm_tasks, p->d_spmm_long, p->n_spmm_long, p->d_row_ptr, p->d_cols,
                                  dV, dW, dH, dP, dY, p->d_spmm_scratch, p->K, h->d_work_counter, h->sm_count, s));
    }
    CUDA_TRY(h, cudaEventRecord(h->ev1, s));
    p->last_kernel = ring ? (fused ? "fused_sddmm_spmm_ring" : "spmm_ring") : (fused ? "fused_sddmm_spmm" : "spmm");
    if (!y_dev) CUDA_TRY(h, cudaMemcpyAsync(Y, dY, sizeof(float) * mk, cudaMemcpyDeviceToHost, s));
    if (P_out && !p_dev) CUDA_TRY(h, cudaMemcpyAsync(P_out, dP, sizeof(float) * nz, cudaMemcpyDeviceToHost, s));
    if (flags & SDDMM_FLAG_ASYNC) {
        p->last_ms = -1.f;
        return SDDMM_OK;
    }
    CUDA_TRY(h, cudaMemcpyAsync(h->h_status, h->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
    CUDA_TRY(h, cudaStreamSynchronize(s));
    CUDA_TRY(h, cudaEventElapsedTime(&p->last_ms, h->ev0, h->ev1));
    return check_device_status(h);
}

}  // namespace

int sddmm_spmm_execute(sddmm_plan_t p, const float *Pval, const float *H, float *Y, uint32_t flags)
{
    if (!p) return SDDMM_INVALID_ARG;
    return run_spmm(p, false, nullptr, H, Pval, nullptr, Y, flags);
}

int sddmm_fused_execute(sddmm_plan_t p, const float *W, const float *H, const float *Sval, float *P_out, float *Y,
                        uint32_t flags)
{
    if (!p) return SDDMM_INVALID_ARG;
    return run_spmm(p, true, W, H, Sval, P_out, Y, flags);
}

int sddmm_selftest_optin_cache(void)
{
    // host-only: the shared-memory opt-in cache must be keyed by device ordinal
    SmemOptinCache c;
    if (!c.needs(0, 1024) || !c.needs(1, 1024)) return SDDMM_INVALID_ARG;
    c.record(0, 4096);
    if (c.needs(0, 4096) || c.needs(0, 1024)) return SDDMM_INVALID_ARG;   // device 0 holds it
    if (!c.needs(1, 1024) || !c.needs(0, 8192)) return SDDMM_INVALID_ARG;  // device 1 does not; larger sizes do not either
    if (!c.needs(-1, 1) || !c.needs(SmemOptinCache::MAX_DEVICES, 1)) return SDDMM_INVALID_ARG;
    c.record(SmemOptinCache::MAX_DEVICES, 1);                               // out of table: never cached
    if (!c.needs(SmemOptinCache::MAX_DEVICES, 1)) return SDDMM_INVALID_ARG;
    return SDDMM_OK;
}

int sddmm_last_kernel_ms(sddmm_plan_t p, float *ms)
{
    if (!p || !ms) return SDDMM_INVALID_ARG;
    *ms = p->last_ms;
    return SDDMM_OK;
}

int sddmm_coo(sddmm_handle_t h, int64_t M, int64_t N, int64_t nnz, const int32_t *rows, const int32_t *cols,
              const float *Sval, const float *W, const float *H, int K, float *P)
{
    if (!h) return SDDMM_INVALID_ARG;
    if (M < 0 || N < 0 || nnz < 0) return SDDMM_INVALID_ARG;
    int st = check_k(K);
    if (st != SDDMM_OK) return st;
    if (nnz == 0) return SDDMM_OK;
    if (!rows || !cols || !W || !H || !P) return SDDMM_INVALID_ARG;
    CUDA_TRY(h, cudaSetDevice(h->device));
    cudaStream_t s = h->stream;
    // Everything that is not already on the device is staged for this call only,
    // as the reference does (sddmm.cu:38-73,147-150).
    struct Tmp {
        void *p[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
        ~Tmp() { for (void *q : p) if (q) cudaFree(q); }
    } tmp;
    auto stage = [&](int slot, const void *src, size_t bytes, const void **dst) -> cudaError_t {
        if (is_device_ptr(src)) { *dst = src; return cudaSuccess; }
        cudaError_t e = cudaMalloc(&tmp.p[slot], bytes);
        if (e != cudaSuccess) return e;
        *dst = tmp.p[slot];
        return cudaMemcpyAsync(tmp.p[slot], src, bytes, cudaMemcpyHostToDevice, s);
    };
    const void *dr, *dc, *dw, *dh, *ds = nullptr;
    CUDA_TRY(h, stage(0, rows, sizeof(int32_t) * nnz, &dr));
    CUDA_TRY(h, stage(1, cols, sizeof(int32_t) * nnz, &dc));
    CUDA_TRY(h, stage(2, W, sizeof(float) * (size_t)M * K, &dw));
    CUDA_TRY(h, stage(3, H, sizeof(float) * (size_t)N * K, &dh));
    if (Sval) CUDA_TRY(h, stage(4, Sval, sizeof(float) * nnz, &ds));
    float *dp = P;
    const bool p_dev = is_device_ptr(P);
    if (!p_dev) {
        CUDA_TRY(h, cudaMalloc(&tmp.p[5], sizeof(float) * nnz));
        dp = (float *)tmp.p[5];
    }
    CUDA_TRY(h, launch_gather((const int32_t *)dr, (const int32_t *)dc, (const float *)ds, (const float *)dw,
                              (const float *)dh, dp, nnz, K, h->sm_count, s));
    if (!p_dev) CUDA_TRY(h, cudaMemcpyAsync(P, dp, sizeof(float) * nnz, cudaMemcpyDeviceToHost, s));
    CUDA_TRY(h, cudaStreamSynchronize(s));
    return SDDMM_OK;
}

int sddmm_selftest_wait_timeout(sddmm_handle_t h)
{
    if (!h) return SDDMM_INVALID_ARG;
    CUDA_TRY(h, cudaSetDevice(h->device));
    cudaStream_t s = h->stream;
    CUDA_TRY(h, launch_wait_timeout_probe(h->d_status, s));
    CUDA_TRY(h, cudaMemcpyAsync(h->h_status, h->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
    CUDA_TRY(h, cudaStreamSynchronize(s));
    return check_device_status(h);
}

int sddmm_plan_get_info(sddmm_plan_t p, sddmm_plan_info *info)
{
    if (!p || !info) return SDDMM_INVALID_ARG;
    info->M = p->M; info->N = p->N; info->nnz = p->nnz; info->K = p->K;
    info->panel_rows = p->cfg.panel_rows;
    info->col_tile = p->col_tile;
    info->n_col_tiles = p->n_col_tiles;
    info->n_work_items = p->n_items;
    info->n_nonempty_rows = p->n_nonempty_rows;
    info->n_nonempty_cols = p->n_nonempty_cols;
    info->device_bytes = p->device_bytes;
    info->plan_ms = p->plan_ms;
    info->n_dense_cells = p->dense.n_cells;
    info->n_dense_nnz = p->dense.n_dense_nnz;
    info->n_hub_cols = p->n_hub_cols;
    return SDDMM_OK;
}

int sddmm_plan_count_cols(sddmm_plan_t p, int64_t *out)
{
    if (!p || !out) return SDDMM_INVALID_ARG;
    sddmm_handle_s *h = p->h;
    if (p->n_nonempty_cols < 0) {
        CUDA_TRY(h, cudaSetDevice(h->device));
        int64_t c = 0;
        CUDA_TRY(h, count_distinct_cols(p->d_cols, p->nnz, p->N, &c, h->stream));
        p->n_nonempty_cols = c;
    }
    *out = p->n_nonempty_cols;
    return SDDMM_OK;
}

int sddmm_plan_export_row_ptr(sddmm_plan_t p, int64_t *row_ptr)
{
    if (!p || !row_ptr) return SDDMM_INVALID_ARG;
    sddmm_handle_s *h = p->h;
    CUDA_TRY(h, cudaSetDevice(h->device));
    CUDA_TRY(h, cudaMemcpyAsync(row_ptr, p->d_row_ptr, sizeof(int64_t) * (size_t)(p->M + 1), cudaMemcpyDeviceToHost,
                                h->stream));
    CUDA_TRY(h, cudaStreamSynchronize(h->stream));
    return SDDMM_OK;
}

int sddmm_plan_export_tiling(sddmm_plan_t p, int panel_rows, int col_tile, int32_t *t_rows, int32_t *t_cols,
                             int32_t *tiled_ind, int32_t *lastIdx_tile, int32_t *lastIdx_block_tile,
                             int32_t *active_row, int32_t *n_actv_row, int32_t *max_active_row)
{
    if (!p || panel_rows <= 0 || col_tile <= 0) return SDDMM_INVALID_ARG;
    sddmm_handle_s *h = p->h;
    CUDA_TRY(h, cudaSetDevice(h->device));
    TilingTables t{t_rows, t_cols, tiled_ind, lastIdx_tile, lastIdx_block_tile, active_row, n_actv_row, max_active_row};
    CUDA_TRY(h, export_reference_tiling(p->d_rows, p->d_cols, p->nnz, p->M, p->N, panel_rows, col_tile, t, h->stream));
    return SDDMM_OK;
}

}  // extern "C"
