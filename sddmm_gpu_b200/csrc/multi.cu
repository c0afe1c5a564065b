// Multi-GPU layer of the C ABI: one rank per GPU (one process per GPU, or one
// host thread per GPU inside one process), nnz-balanced blocks of consecutive rows,
// H distributed over NCCL.
//
// Replaces the MPI program of the reference (HiPC18_mpi/sddmm.cu:139-351): there
// every rank redoes the whole preprocessing, uploads all of W and H and runs one
// column panel (make_CSC, HiPC18_mpi/util.h:100-135), MPI being used for barriers
// only.  Here rank r owns rows [cuts[r], cuts[r+1]) of S and W -- its nonzeros are
// one contiguous slice of the input, so the ranks' outputs concatenate to P in
// input order -- and H, the one operand every rank needs whole, travels over
// NVLink / NVSwitch into each GPU's own memory.  No kernel reads a peer's memory.
//
// H broadcast and compute overlap: H goes out in chunks of consecutive rows
// (= column ranges of S) on a communication stream; the rank's nonzeros are
// bucketed by the same column ranges (the plan's column-tile permutation) and the
// gather kernel of bucket i is ordered behind the arrival of chunk i by a CUDA
// event, while chunk i+1 is already on the wire.  Nothing waits on the device side
// for a peer: ordering is stream order plus NCCL's own synchronisation.
//
// NCCL is bound at run time (dlopen): an already loaded libnccl.so.2 is reused
// (e.g. the one a framework in the same process brought), else the system
// library is opened.  The single-GPU entry points never touch it.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "engine_internal.hpp"

// ---- the part of NCCL's C ABI that is used (stable across NCCL 2.x) -------------
extern "C" {
typedef struct ncclComm *ncclComm_t;
typedef struct {
    char internal[128];
} ncclUniqueId;
typedef int ncclResult_t;  // 0 = ncclSuccess
}
static_assert(sizeof(ncclUniqueId) == SDDMM_COMM_ID_BYTES, "unique id size");

namespace {

constexpr int NCCL_FLOAT32 = 7;

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int *) = nullptr;
    std::string error;
};

NcclApi *nccl_api()
{
    static NcclApi api;
    static bool tried = false;
    if (tried) return api.lib ? &api : nullptr;
    tried = true;
    const char *names[3] = {std::getenv("SDDMM_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
    void *lib = nullptr;
    for (const char *n : names)  // a copy that is already in the process first
        if (!lib && n && *n) lib = dlopen(n, RTLD_NOW | RTLD_NOLOAD);
    for (const char *n : names)
        if (!lib && n && *n) lib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
    if (!lib) {
        api.error = "libnccl.so.2 not found (set SDDMM_NCCL_LIBRARY)";
        return nullptr;
    }
    bool ok = true;
    auto sym = [&](const char *name) {
        void *p = dlsym(lib, name);
        if (!p) {
            ok = false;
            api.error = std::string("NCCL symbol missing: ") + name;
        }
        return p;
    };
    api.GetUniqueId = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))sym("ncclCommInitRank");
    api.CommDestroy = (decltype(api.CommDestroy))sym("ncclCommDestroy");
    api.Broadcast = (decltype(api.Broadcast))sym("ncclBroadcast");
    api.AllGather = (decltype(api.AllGather))sym("ncclAllGather");
    api.GroupStart = (decltype(api.GroupStart))sym("ncclGroupStart");
    api.GroupEnd = (decltype(api.GroupEnd))sym("ncclGroupEnd");
    api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
    api.GetVersion = (decltype(api.GetVersion))sym("ncclGetVersion");
    if (!ok) return nullptr;
    api.lib = lib;
    return &api;
}

}  // namespace

struct sddmm_comm_s {
    sddmm_handle_s *h = nullptr;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ev_begin = nullptr, ev_end = nullptr, ev_bcast_end = nullptr;
    std::vector<cudaEvent_t> chunk_done;
};

struct sddmm_dist_plan_s {
    sddmm_comm_s *c = nullptr;
    int64_t M = 0, N = 0, nnz = 0;
    int K = 0;
    std::vector<int64_t> cuts, nnz_cuts;
    int64_t row_begin = 0, row_end = 0, nnz_begin = 0, nnz_end = 0;
    sddmm_plan_t local = nullptr;    // this rank's row block, single column tile
    sddmm_plan_t chunked = nullptr;  // the same block bucketed by the column ranges of the H chunks
    int n_chunks = 1;
    int64_t chunk_cols = 0;
    std::vector<int64_t> tile_off;   // nonzero offsets of the buckets in the chunked plan's order
    int32_t *d_local_rows = nullptr;  // rows rebased to the block (when the caller's indices are device arrays)
    float t_bcast = -1.f, t_compute = -1.f, t_total = -1.f;
};

namespace {

int fail_nccl(sddmm_handle_s *h, ncclResult_t r, const char *what)
{
    NcclApi *a = nccl_api();
    h->last_error = std::string(what) + ": " + ((a && a->GetErrorString) ? a->GetErrorString(r) : "NCCL error");
    return SDDMM_NCCL_ERROR;
}
int fail_cuda_m(sddmm_handle_s *h, cudaError_t e, const char *what)
{
    h->last_error = std::string(what) + ": " + cudaGetErrorString(e);
    (void)cudaGetLastError();
    return e == cudaErrorMemoryAllocation ? SDDMM_OUT_OF_MEMORY : SDDMM_CUDA_ERROR;
}
#define CU_TRY(h, expr)                                              \
    do {                                                             \
        cudaError_t _e = (expr);                                     \
        if (_e != cudaSuccess) return fail_cuda_m((h), _e, #expr);   \
    } while (0)
#define NC_TRY(h, expr)                                  \
    do {                                                 \
        ncclResult_t _r = (expr);                        \
        if (_r != 0) return fail_nccl((h), _r, #expr);   \
    } while (0)

bool device_ptr(const void *p)
{
    cudaPointerAttributes a;
    if (!p || cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

__global__ void rebase_rows_kernel(const int32_t *__restrict__ rows, int32_t *__restrict__ out, int64_t n, int32_t base)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = rows[i] - base;
}

// first nonzero (tiled order: column tiles ascending) of every column tile: off[t] = lower bound of tile t
__global__ void tile_offsets_kernel(const int32_t *__restrict__ cols_t, int64_t nnz, int col_tile, int n_tiles, int64_t *off)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t > n_tiles) return;
    int64_t lo = 0, hi = nnz;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (cols_t[mid] / col_tile < t) lo = mid + 1;
        else hi = mid;
    }
    off[t] = lo;
}

}  // namespace

extern "C" {

int sddmm_comm_unique_id(void *id)
{
    if (!id) return SDDMM_INVALID_ARG;
    NcclApi *a = nccl_api();
    if (!a) return SDDMM_NCCL_ERROR;
    return a->GetUniqueId((ncclUniqueId *)id) == 0 ? SDDMM_OK : SDDMM_NCCL_ERROR;
}

int sddmm_comm_create(sddmm_handle_t h, const void *id, int rank, int world, sddmm_comm_t *out)
{
    if (!h || !out || !id || world < 1 || rank < 0 || rank >= world) return SDDMM_INVALID_ARG;
    *out = nullptr;
    NcclApi *a = world > 1 ? nccl_api() : nullptr;  // a single rank has nobody to talk to and needs no NCCL
    if (world > 1 && !a) {
        h->last_error = "NCCL is not available in this process";
        return SDDMM_NCCL_ERROR;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    sddmm_comm_s *c = new (std::nothrow) sddmm_comm_s;
    if (!c) return SDDMM_OUT_OF_MEMORY;
    c->h = h;
    c->rank = rank;
    c->world = world;
    if (world > 1) {
        ncclUniqueId uid;
        std::memcpy(&uid, id, sizeof(uid));
        ncclResult_t r = a->CommInitRank(&c->comm, world, uid, rank);
        if (r != 0) {
            delete c;
            return fail_nccl(h, r, "ncclCommInitRank");
        }
    }
    cudaError_t e = cudaStreamCreateWithFlags(&c->comm_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&c->ev_begin);
    if (e == cudaSuccess) e = cudaEventCreate(&c->ev_end);
    if (e == cudaSuccess) e = cudaEventCreate(&c->ev_bcast_end);
    if (e != cudaSuccess) {
        sddmm_comm_destroy(c);
        return fail_cuda_m(h, e, "sddmm_comm_create");
    }
    *out = c;
    return SDDMM_OK;
}

int sddmm_comm_destroy(sddmm_comm_t c)
{
    if (!c) return SDDMM_OK;
    cudaSetDevice(c->h->device);
    if (c->comm_stream) cudaStreamSynchronize(c->comm_stream);
    NcclApi *a = nccl_api();
    if (c->comm && a) a->CommDestroy(c->comm);
    if (c->comm_stream) cudaStreamDestroy(c->comm_stream);
    for (cudaEvent_t ev : {c->ev_begin, c->ev_end, c->ev_bcast_end})
        if (ev) cudaEventDestroy(ev);
    for (cudaEvent_t ev : c->chunk_done) cudaEventDestroy(ev);
    (void)cudaGetLastError();
    delete c;
    return SDDMM_OK;
}

int sddmm_comm_broadcast(sddmm_comm_t c, float *buf, int64_t count, int root, void *cuda_stream)
{
    if (!c || count < 0 || root < 0 || root >= c->world || (count > 0 && !buf)) return SDDMM_INVALID_ARG;
    if (c->world == 1 || count == 0) return SDDMM_OK;
    sddmm_handle_s *h = c->h;
    CU_TRY(h, cudaSetDevice(h->device));
    cudaStream_t s = cuda_stream ? (cudaStream_t)cuda_stream : h->stream;
    NC_TRY(h, nccl_api()->Broadcast(buf, buf, (size_t)count, NCCL_FLOAT32, root, c->comm, s));
    return SDDMM_OK;
}

int sddmm_comm_all_gather(sddmm_comm_t c, float *buf, int64_t count_per_rank, void *cuda_stream)
{
    if (!c || count_per_rank < 0 || (count_per_rank > 0 && !buf)) return SDDMM_INVALID_ARG;
    if (c->world == 1 || count_per_rank == 0) return SDDMM_OK;
    sddmm_handle_s *h = c->h;
    CU_TRY(h, cudaSetDevice(h->device));
    cudaStream_t s = cuda_stream ? (cudaStream_t)cuda_stream : h->stream;
    NC_TRY(h, nccl_api()->AllGather(buf + (size_t)c->rank * count_per_rank, buf, (size_t)count_per_rank, NCCL_FLOAT32, c->comm, s));
    return SDDMM_OK;
}

int sddmm_dist_plan_coo(sddmm_comm_t c, int64_t M, int64_t N, int64_t nnz, const int32_t *rows, const int32_t *cols, int K,
                        int panel_rows_hint, int h_chunks, uint32_t flags, sddmm_dist_plan_t *out)
{
    return sddmm_dist_plan_coo_shares(c, M, N, nnz, rows, cols, K, panel_rows_hint, h_chunks, nullptr, flags, out);
}

int sddmm_dist_plan_coo_shares(sddmm_comm_t c, int64_t M, int64_t N, int64_t nnz, const int32_t *rows, const int32_t *cols, int K,
                               int panel_rows_hint, int h_chunks, const double *rank_shares, uint32_t flags,
                               sddmm_dist_plan_t *out)
{
    if (!c || !out || M < 0 || N < 0 || nnz < 0 || (nnz > 0 && (!rows || !cols))) return SDDMM_INVALID_ARG;
    *out = nullptr;
    sddmm_handle_s *h = c->h;
    CU_TRY(h, cudaSetDevice(h->device));
    const bool dev_idx = (flags & SDDMM_PLAN_DEVICE_INDICES) != 0;
    if (dev_idx != device_ptr(rows) && nnz > 0) {
        h->last_error = "sddmm_dist_plan_coo: SDDMM_PLAN_DEVICE_INDICES does not match where rows[] lives";
        return SDDMM_INVALID_ARG;
    }
    sddmm_dist_plan_s *p = new (std::nothrow) sddmm_dist_plan_s;
    if (!p) return SDDMM_OUT_OF_MEMORY;
    p->c = c;
    p->M = M; p->N = N; p->nnz = nnz; p->K = K;
    p->cuts.assign((size_t)c->world + 1, 0);
    p->nnz_cuts.assign((size_t)c->world + 1, 0);
    auto bail = [&](int st) {
        sddmm_dist_plan_destroy(p);
        return st;
    };
    // the cuts are a function of the row indices alone: every rank computes the same ones
    std::vector<int32_t> host_rows;
    const int32_t *rows_h = rows;
    if (dev_idx && nnz > 0) {
        try {
            host_rows.resize((size_t)nnz);
        } catch (const std::bad_alloc &) {
            return bail(SDDMM_OUT_OF_MEMORY);
        }
        cudaError_t e = cudaMemcpyAsync(host_rows.data(), rows, sizeof(int32_t) * (size_t)nnz, cudaMemcpyDeviceToHost, h->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
        if (e != cudaSuccess) return bail(fail_cuda_m(h, e, "copying the row indices to the host"));
        rows_h = host_rows.data();
    }
    if (nnz > 0 && !sddmm_coo_is_row_sorted(nnz, rows_h)) return bail(SDDMM_UNSORTED_INPUT);
    int st = sddmm_partition_rows_shares(M, nnz, rows_h, c->world, 32, rank_shares, p->cuts.data(), p->nnz_cuts.data());
    if (st != SDDMM_OK) return bail(st);
    p->row_begin = p->cuts[c->rank];
    p->row_end = p->cuts[c->rank + 1];
    p->nnz_begin = p->nnz_cuts[c->rank];
    p->nnz_end = p->nnz_cuts[c->rank + 1];
    const int64_t ln = p->nnz_end - p->nnz_begin, lm = p->row_end - p->row_begin;

    // this rank's rows, rebased to its block
    const int32_t *lrows = nullptr, *lcols = cols ? cols + p->nnz_begin : nullptr;
    std::vector<int32_t> lrows_h;
    if (dev_idx) {
        cudaError_t e = cudaMalloc((void **)&p->d_local_rows, sizeof(int32_t) * (size_t)(ln ? ln : 1));
        if (e != cudaSuccess) return bail(fail_cuda_m(h, e, "cudaMalloc(local rows)"));
        if (ln > 0) {
            rebase_rows_kernel<<<(unsigned)std::min<int64_t>((ln + 255) / 256, 148 * 16), 256, 0, h->stream>>>(
                rows + p->nnz_begin, p->d_local_rows, ln, (int32_t)p->row_begin);
            e = cudaGetLastError();
            if (e != cudaSuccess) return bail(fail_cuda_m(h, e, "rebasing the row indices"));
        }
        lrows = p->d_local_rows;
    } else {
        try {
            lrows_h.resize((size_t)ln);
        } catch (const std::bad_alloc &) {
            return bail(SDDMM_OUT_OF_MEMORY);
        }
        for (int64_t i = 0; i < ln; ++i) lrows_h[(size_t)i] = rows[p->nnz_begin + i] - (int32_t)p->row_begin;
        lrows = lrows_h.data();
    }
    const uint32_t pf = (flags & (SDDMM_PLAN_DEVICE_INDICES | SDDMM_PLAN_SKIP_VALIDATION));
    st = sddmm_plan_coo(h, lm, N, ln, lrows, lcols, K, panel_rows_hint, 0, pf, &p->local);
    if (st != SDDMM_OK) return bail(st);

    // H chunks: consecutive rows of H = column ranges of S, a multiple of 32 columns each
    if (h_chunks < 1) h_chunks = 1;
    if (h_chunks > 64) h_chunks = 64;
    p->chunk_cols = N > 0 ? ((N + h_chunks - 1) / h_chunks + 31) / 32 * 32 : 32;
    p->n_chunks = N > 0 ? (int)((N + p->chunk_cols - 1) / p->chunk_cols) : 1;
    if ((c->world > 1 || (flags & SDDMM_PLAN_FORCE_H_CHUNKS)) && p->n_chunks > 1 && ln > 0) {
        st = sddmm_plan_coo(h, lm, N, ln, lrows, lcols, K, panel_rows_hint, (int)p->chunk_cols, pf | SDDMM_PLAN_SKIP_VALIDATION,
                            &p->chunked);
        if (st != SDDMM_OK) return bail(st);
        p->tile_off.assign((size_t)p->n_chunks + 1, 0);
        int64_t *d_off = nullptr;
        cudaError_t e = cudaMalloc((void **)&d_off, sizeof(int64_t) * (size_t)(p->n_chunks + 1));
        if (e == cudaSuccess) {
            tile_offsets_kernel<<<1, 128, 0, h->stream>>>(p->chunked->d_cols_t, ln, (int)p->chunk_cols, p->n_chunks, d_off);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(p->tile_off.data(), d_off, sizeof(int64_t) * (size_t)(p->n_chunks + 1), cudaMemcpyDeviceToHost,
                                h->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
        cudaFree(d_off);
        if (e != cudaSuccess) return bail(fail_cuda_m(h, e, "bucket offsets of the H chunks"));
    } else {
        p->n_chunks = 1;
        p->chunk_cols = N > 0 ? N : 1;
    }
    while ((int)c->chunk_done.size() < p->n_chunks) {
        cudaEvent_t ev = nullptr;
        cudaError_t e = cudaEventCreate(&ev);
        if (e != cudaSuccess) return bail(fail_cuda_m(h, e, "cudaEventCreate"));
        c->chunk_done.push_back(ev);
    }
    CU_TRY(h, cudaStreamSynchronize(h->stream));  // host staging vectors go out of scope
    *out = p;
    return SDDMM_OK;
}

int sddmm_dist_plan_destroy(sddmm_dist_plan_t p)
{
    if (!p) return SDDMM_OK;
    cudaSetDevice(p->c->h->device);
    if (p->local) sddmm_destroy_plan(p->local);
    if (p->chunked) sddmm_destroy_plan(p->chunked);
    if (p->d_local_rows) cudaFree(p->d_local_rows);
    (void)cudaGetLastError();
    delete p;
    return SDDMM_OK;
}

int sddmm_dist_plan_get_shard(sddmm_dist_plan_t p, int64_t *row_begin, int64_t *row_end, int64_t *nnz_begin, int64_t *nnz_end,
                              int32_t *n_chunks)
{
    if (!p) return SDDMM_INVALID_ARG;
    if (row_begin) *row_begin = p->row_begin;
    if (row_end) *row_end = p->row_end;
    if (nnz_begin) *nnz_begin = p->nnz_begin;
    if (nnz_end) *nnz_end = p->nnz_end;
    if (n_chunks) *n_chunks = p->n_chunks;
    return SDDMM_OK;
}

sddmm_plan_t sddmm_dist_plan_local(sddmm_dist_plan_t p) { return p ? p->local : nullptr; }

int sddmm_dist_execute(sddmm_dist_plan_t p, const float *W_local, float *H, const float *Sval_local, float *P_local, int root,
                       uint32_t flags)
{
    if (!p) return SDDMM_INVALID_ARG;
    sddmm_comm_s *c = p->c;
    sddmm_handle_s *h = c->h;
    if (root < 0 || root >= c->world) return SDDMM_INVALID_ARG;
    const uint32_t exec_flags = flags & ~(uint32_t)(SDDMM_DIST_H_RESIDENT | SDDMM_DIST_BROADCAST_ONLY);
    p->t_bcast = p->t_compute = p->t_total = -1.f;
    if ((flags & SDDMM_DIST_H_RESIDENT) || (c->world == 1 && !p->chunked)) {
        // H is in place on every rank: the path has no collective
        const int st = sddmm_execute(p->local, W_local, H, Sval_local, P_local, exec_flags);
        if (st == SDDMM_OK && !(exec_flags & SDDMM_FLAG_ASYNC)) {
            sddmm_last_kernel_ms(p->local, &p->t_compute);
            p->t_total = p->t_compute;
            p->t_bcast = 0.f;
        }
        return st;
    }
    if (!H || !device_ptr(H)) {
        h->last_error = "sddmm_dist_execute: H must be a device array of N x K floats on every rank";
        return SDDMM_INVALID_ARG;
    }
    const bool only_bcast = (flags & SDDMM_DIST_BROADCAST_ONLY) != 0;
    const int64_t ln = p->nnz_end - p->nnz_begin;
    if (!only_bcast && ln > 0 && (!W_local || !P_local || !device_ptr(W_local) || !device_ptr(P_local) ||
                                  (Sval_local && !device_ptr(Sval_local)))) {
        h->last_error = "sddmm_dist_execute: with the broadcast inside the call W, S values and P must be device arrays";
        return SDDMM_INVALID_ARG;
    }
    CU_TRY(h, cudaSetDevice(h->device));
    NcclApi *a = c->world > 1 ? nccl_api() : nullptr;
    cudaStream_t s = h->stream, cs = c->comm_stream;
    // the chunks go out behind everything already enqueued on the compute stream (H may still be read there)
    CU_TRY(h, cudaEventRecord(c->ev_begin, s));
    CU_TRY(h, cudaStreamWaitEvent(cs, c->ev_begin, 0));
    for (int i = 0; i < p->n_chunks; ++i) {
        const int64_t c0 = (int64_t)i * p->chunk_cols;
        const int64_t c1 = std::min<int64_t>(p->N, c0 + p->chunk_cols);
        float *piece = H + (size_t)c0 * p->K;
        if (c->world > 1) NC_TRY(h, a->Broadcast(piece, piece, (size_t)(c1 - c0) * p->K, NCCL_FLOAT32, root, c->comm, cs));
        CU_TRY(h, cudaEventRecord(c->chunk_done[i], cs));
    }
    CU_TRY(h, cudaEventRecord(c->ev_bcast_end, cs));
    const sddmm_plan_s *q = p->chunked;
    // (Leaving SMs free for the broadcast's kernels was tried -- 0, 16 and 32 of 148 -- and changed nothing:
    // when the broadcast slows down beside the bucket kernels it is for HBM bandwidth, not for SMs.)
    for (int i = 0; i < p->n_chunks; ++i) {
        CU_TRY(h, cudaStreamWaitEvent(s, c->chunk_done[i], 0));
        if (only_bcast || ln == 0) continue;
        if (!q) {  // a single chunk: the plain plan behind the whole broadcast
            const int st = sddmm_execute(p->local, W_local, H, Sval_local, P_local, exec_flags | SDDMM_FLAG_ASYNC);
            if (st != SDDMM_OK) return st;
            continue;
        }
        const int64_t o0 = p->tile_off[(size_t)i], cnt = p->tile_off[(size_t)i + 1] - o0;
        if (cnt <= 0) continue;
        const int32_t *cols_p = q->d_cols_hint ? q->d_cols_hint : q->d_cols_t;
        cudaError_t e;
        if (ring_supports(p->K)) {
            e = launch_ring(q->d_rows_t + o0, cols_p + o0, q->d_perm + o0, Sval_local, W_local, H, P_local, cnt, p->K,
                                q->d_cols_hint != nullptr, h->sm_count, h->d_work_counter, h->d_status, s);
            if (e != cudaSuccess) return fail_cuda_m(h, e, "launching the gather kernel of an H chunk");
            ++h->n_launches;
        } else {
            h->last_error = "sddmm_dist_execute: the chunked form needs K in {32, 64, 128, 256, 512, 1024}";
            return SDDMM_K_UNSUPPORTED;
        }
    }
    CU_TRY(h, cudaEventRecord(c->ev_end, s));
    if (exec_flags & SDDMM_FLAG_ASYNC) return SDDMM_OK;
    CU_TRY(h, cudaMemcpyAsync(h->h_status, h->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
    CU_TRY(h, cudaStreamSynchronize(s));
    CU_TRY(h, cudaEventElapsedTime(&p->t_total, c->ev_begin, c->ev_end));
    CU_TRY(h, cudaEventElapsedTime(&p->t_bcast, c->ev_begin, c->ev_bcast_end));
    if (*h->h_status != DEV_OK) {
        h->last_error = "a bounded device-side wait (mbarrier) gave up";
        *h->h_status = DEV_OK;
        cudaMemsetAsync(h->d_status, 0, sizeof(int), s);
        return SDDMM_DEVICE_TIMEOUT;
    }
    return SDDMM_OK;
}

int sddmm_dist_last_times(sddmm_dist_plan_t p, float *bcast_ms, float *compute_ms, float *total_ms)
{
    if (!p) return SDDMM_INVALID_ARG;
    if (bcast_ms) *bcast_ms = p->t_bcast;
    if (compute_ms) *compute_ms = p->t_compute;
    if (total_ms) *total_ms = p->t_total;
    return SDDMM_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// One process, several GPUs: one host thread per GPU, each a rank of the layer
// above.  This is what the command line's --gpus N uses; the reference's
// equivalent is `mpiexec -n P ./sddmm ...` (HiPC18_mpi/scripts/run_mpi.sh:14-22).
// ---------------------------------------------------------------------------
struct sddmm_multi_s {
    std::vector<int> devices;
    std::vector<sddmm_handle_t> handles;
    std::vector<sddmm_comm_t> comms;
    std::string last_error;
};

struct sddmm_multi_plan_s {
    sddmm_multi_s *m = nullptr;
    int64_t M = 0, N = 0, nnz = 0, n_pad = 0;  // n_pad: rows of the device copy of H, a multiple of the GPU count
    int K = 0;
    std::vector<sddmm_dist_plan_t> plans;
    std::vector<float *> dW, dH, dS, dP;
    float last_kernel_ms = -1.f;
};

namespace {

// Runs fn(rank) on one thread per rank and returns the first non-OK status.
template <class F>
int for_each_rank(int n, F fn)
{
    std::vector<int> st((size_t)n, SDDMM_OK);
    std::vector<std::thread> th;
    th.reserve((size_t)n);
    for (int r = 0; r < n; ++r) th.emplace_back([&, r] { st[(size_t)r] = fn(r); });
    for (auto &t : th) t.join();
    for (int r = 0; r < n; ++r)
        if (st[(size_t)r] != SDDMM_OK) return st[(size_t)r];
    return SDDMM_OK;
}

void note_error(sddmm_multi_s *m, int rank)
{
    m->last_error = "GPU " + std::to_string(m->devices[(size_t)rank]) + ": " + sddmm_last_error(m->handles[(size_t)rank]);
}

}  // namespace

extern "C" {

int sddmm_multi_create(const int *devices, int ndev, sddmm_multi_t *out)
{
    if (!out || ndev < 1 || ndev > 64) return SDDMM_INVALID_ARG;
    *out = nullptr;
    sddmm_multi_s *m = new (std::nothrow) sddmm_multi_s;
    if (!m) return SDDMM_OUT_OF_MEMORY;
    for (int r = 0; r < ndev; ++r) m->devices.push_back(devices ? devices[r] : r);
    m->handles.assign((size_t)ndev, nullptr);
    m->comms.assign((size_t)ndev, nullptr);
    for (int r = 0; r < ndev; ++r) {
        const int st = sddmm_create(&m->handles[(size_t)r], m->devices[(size_t)r]);
        if (st != SDDMM_OK) {
            sddmm_multi_destroy(m);
            return st;
        }
    }
    if (ndev > 1) {
        ncclUniqueId id;
        int st = sddmm_comm_unique_id(&id);
        if (st == SDDMM_OK)  // ncclCommInitRank returns when every rank has joined: one thread per rank
            st = for_each_rank(ndev, [&](int r) { return sddmm_comm_create(m->handles[(size_t)r], &id, r, ndev, &m->comms[(size_t)r]); });
        if (st != SDDMM_OK) {
            sddmm_multi_destroy(m);
            return st;
        }
    } else {
        ncclUniqueId id{};  // a one-rank communicator needs no rendezvous and no NCCL
        const int st = sddmm_comm_create(m->handles[0], &id, 0, 1, &m->comms[0]);
        if (st != SDDMM_OK) {
            sddmm_multi_destroy(m);
            return st;
        }
    }
    *out = m;
    return SDDMM_OK;
}

int sddmm_multi_destroy(sddmm_multi_t m)
{
    if (!m) return SDDMM_OK;
    for (sddmm_comm_t c : m->comms) sddmm_comm_destroy(c);
    for (sddmm_handle_t h : m->handles) sddmm_destroy(h);
    delete m;
    return SDDMM_OK;
}

const char *sddmm_multi_last_error(sddmm_multi_t m) { return m ? m->last_error.c_str() : ""; }

int sddmm_multi_plan_coo(sddmm_multi_t m, int64_t M, int64_t N, int64_t nnz, const int32_t *rows, const int32_t *cols, int K,
                         int panel_rows_hint, uint32_t flags, sddmm_multi_plan_t *out)
{
    if (!m || !out) return SDDMM_INVALID_ARG;
    *out = nullptr;
    if (flags & SDDMM_PLAN_DEVICE_INDICES) return SDDMM_INVALID_ARG;  // one host copy of the pattern serves every GPU
    const int n = (int)m->handles.size();
    sddmm_multi_plan_s *p = new (std::nothrow) sddmm_multi_plan_s;
    if (!p) return SDDMM_OUT_OF_MEMORY;
    p->m = m;
    p->M = M; p->N = N; p->nnz = nnz; p->K = K;
    p->n_pad = (N + n - 1) / n * n;
    p->plans.assign((size_t)n, nullptr);
    p->dW.assign((size_t)n, nullptr);
    p->dH.assign((size_t)n, nullptr);
    p->dS.assign((size_t)n, nullptr);
    p->dP.assign((size_t)n, nullptr);
    const int st = for_each_rank(n, [&](int r) {
        int s = sddmm_dist_plan_coo(m->comms[(size_t)r], M, N, nnz, rows, cols, K, panel_rows_hint, 1, flags, &p->plans[(size_t)r]);
        if (s != SDDMM_OK) return s;
        const sddmm_dist_plan_s *d = p->plans[(size_t)r];
        const size_t lm = (size_t)(d->row_end - d->row_begin), ln = (size_t)(d->nnz_end - d->nnz_begin);
        cudaError_t e = cudaSetDevice(m->devices[(size_t)r]);
        if (e == cudaSuccess) e = cudaMalloc((void **)&p->dW[(size_t)r], sizeof(float) * std::max<size_t>(lm * (size_t)K, 1));
        if (e == cudaSuccess) e = cudaMalloc((void **)&p->dH[(size_t)r], sizeof(float) * std::max<size_t>((size_t)p->n_pad * (size_t)K, 1));
        if (e == cudaSuccess) e = cudaMalloc((void **)&p->dS[(size_t)r], sizeof(float) * (ln ? ln : 1));
        if (e == cudaSuccess) e = cudaMalloc((void **)&p->dP[(size_t)r], sizeof(float) * (ln ? ln : 1));
        if (e != cudaSuccess) return fail_cuda_m(m->handles[(size_t)r], e, "allocating the operands of a GPU");
        return (int)SDDMM_OK;
    });
    if (st != SDDMM_OK) {
        for (int r = 0; r < n; ++r)
            if (*sddmm_last_error(m->handles[(size_t)r])) note_error(m, r);
        sddmm_multi_plan_destroy(p);
        return st;
    }
    *out = p;
    return SDDMM_OK;
}

int sddmm_multi_plan_destroy(sddmm_multi_plan_t p)
{
    if (!p) return SDDMM_OK;
    for (size_t r = 0; r < p->plans.size(); ++r) {
        cudaSetDevice(p->m->devices[r]);
        sddmm_dist_plan_destroy(p->plans[r]);
        cudaFree(p->dW[r]);
        cudaFree(p->dH[r]);
        cudaFree(p->dS[r]);
        cudaFree(p->dP[r]);
    }
    (void)cudaGetLastError();
    delete p;
    return SDDMM_OK;
}

int sddmm_multi_plan_get_cuts(sddmm_multi_plan_t p, int64_t *row_cuts, int64_t *nnz_cuts)
{
    if (!p || p->plans.empty()) return SDDMM_INVALID_ARG;
    const sddmm_dist_plan_s *d = p->plans[0];
    if (row_cuts) std::copy(d->cuts.begin(), d->cuts.end(), row_cuts);
    if (nnz_cuts) std::copy(d->nnz_cuts.begin(), d->nnz_cuts.end(), nnz_cuts);
    return SDDMM_OK;
}

int sddmm_multi_execute(sddmm_multi_plan_t p, const float *W, const float *H, const float *Sval, float *P, uint32_t flags)
{
    if (!p) return SDDMM_INVALID_ARG;
    if (p->nnz == 0) return SDDMM_OK;
    if (!W || !H || !P) return SDDMM_INVALID_ARG;
    if (device_ptr(W) || device_ptr(H) || device_ptr(P) || (Sval && device_ptr(Sval))) return SDDMM_INVALID_ARG;  // host arrays
    sddmm_multi_s *m = p->m;
    const int n = (int)p->plans.size();
    const int K = p->K;
    const int64_t slice = p->n_pad / n;  // rows of H every GPU uploads over its own PCIe link
    std::vector<float> kernel_ms((size_t)n, 0.f);
    const int st = for_each_rank(n, [&](int r) -> int {
        sddmm_handle_s *h = m->handles[(size_t)r];
        sddmm_dist_plan_s *d = p->plans[(size_t)r];
        CU_TRY(h, cudaSetDevice(h->device));
        cudaStream_t s = h->stream;
        const int64_t lm = d->row_end - d->row_begin, ln = d->nnz_end - d->nnz_begin;
        // All uploads first, the exchange after them: a copy from pageable host memory blocks its host thread
        // until the stream has caught up, and a thread that sits in such a call while its GPU's all-gather waits
        // for peers whose threads have not launched theirs yet is the classic way to stall every GPU of a
        // one-process job.  With the copies in front, no thread blocks between the collective's launches.
        const int64_t h0 = std::min<int64_t>(p->N, slice * r), h1 = std::min<int64_t>(p->N, slice * (r + 1));
        if (h1 > h0)
            CU_TRY(h, cudaMemcpyAsync(p->dH[(size_t)r] + (size_t)h0 * K, H + (size_t)h0 * K, sizeof(float) * (size_t)(h1 - h0) * K,
                                      cudaMemcpyHostToDevice, s));
        if (lm > 0)
            CU_TRY(h, cudaMemcpyAsync(p->dW[(size_t)r], W + (size_t)d->row_begin * K, sizeof(float) * (size_t)lm * K,
                                      cudaMemcpyHostToDevice, s));
        if (Sval && ln > 0)
            CU_TRY(h, cudaMemcpyAsync(p->dS[(size_t)r], Sval + d->nnz_begin, sizeof(float) * (size_t)ln, cudaMemcpyHostToDevice, s));
        if (n > 1) {
            const int cst = sddmm_comm_all_gather(m->comms[(size_t)r], p->dH[(size_t)r], slice * K, s);
            if (cst != SDDMM_OK) return cst;
        }
        if (ln > 0) {
            const int est = sddmm_dist_execute(d, p->dW[(size_t)r], p->dH[(size_t)r], Sval ? p->dS[(size_t)r] : nullptr,
                                               p->dP[(size_t)r], 0, flags | SDDMM_DIST_H_RESIDENT);
            if (est != SDDMM_OK) return est;
            sddmm_last_kernel_ms(d->local, &kernel_ms[(size_t)r]);
            CU_TRY(h, cudaMemcpyAsync(P + d->nnz_begin, p->dP[(size_t)r], sizeof(float) * (size_t)ln, cudaMemcpyDeviceToHost, s));
        }
        CU_TRY(h, cudaStreamSynchronize(s));
        return SDDMM_OK;
    });
    if (st != SDDMM_OK) {
        for (int r = 0; r < n; ++r)
            if (*sddmm_last_error(m->handles[(size_t)r])) note_error(m, r);
        return st;
    }
    p->last_kernel_ms = *std::max_element(kernel_ms.begin(), kernel_ms.end());
    return SDDMM_OK;
}

int sddmm_multi_last_kernel_ms(sddmm_multi_plan_t p, float *ms)
{
    if (!p || !ms) return SDDMM_INVALID_ARG;
    *ms = p->last_kernel_ms;
    return SDDMM_OK;
}

}  // extern "C"
