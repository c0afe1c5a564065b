// The step after SDDMM in its callers: Y = P * H with P on the sparsity pattern of S
// (SpMM), and the fused form Y = (S o (W H^T)) * H that never writes P to memory.
//
// The reference stops at SDDMM; its README motivates SDDMM as "a core component in
// reformulations of many machine learning algorithms" (README.md:1), where the
// sampled product is at once multiplied back into a dense factor.  These kernels
// have therefore no counterpart to be pinned to: the parity tests use a CPU loop of
// the same definition (oracle/sddmm_oracle.c, oracle_spmm*).
//
//     Y[r, :] = sum over the nonzeros i of row r of  p_i * H[col_i, :]
//     p_i     = Pval[i]                                    (SpMM; 1 when Pval is NULL)
//             = (sum_t W[r, t] H[col_i, t]) * Sval[i]      (fused; Sval NULL = 1)
//
// Shape.  Like the SDDMM gather kernels this is an integer-indexed gather bound by
// HBM / L2, not a GEMM: per nonzero one row of H (4K bytes) comes in, once, and is
// used twice in the fused form (for the dot product and for the update of Y).  A
// warp owns whole rows of S: all 32 lanes work on one nonzero, lane l holding the
// float4 pieces l, l + 32, ... of the H row, of the W row (fused) and of the Y row,
// so the dot product is one 5-step butterfly and the update needs no exchange at
// all; four nonzeros are in flight per warp (two at K > 512), indices one step ahead.
// Rows are dealt out as TASKS built once per plan on the host from the row pointer:
// runs of consecutive whole rows holding about 1024 nonzeros, and -- for rows longer
// than that -- pieces of one row whose partial sums go to a scratch slot each and are
// added up in a fixed order by a second, tiny kernel.  No atomics on Y: the result
// does not depend on scheduling.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <vector>

#include "common.cuh"
#include "device_utils.cuh"

namespace sddmm {

using namespace dev;

namespace {

constexpr int SPMM_TASK_NNZ = 1024;  // nonzeros a task aims for; longer rows are cut into pieces of this size
constexpr int SPMM_WARPS = 8;        // warps per CTA

// F = float4 pieces per lane (K <= 128 F floats ... K4 <= 32 F); FUSED: p_i from W and H
template <int F, bool FUSED>
__global__ void __launch_bounds__(SPMM_WARPS * 32)
spmm_rows_kernel(const SpmmTask *__restrict__ tasks, int64_t n_tasks, const int64_t *__restrict__ row_ptr,
                 const int32_t *__restrict__ cols, const float *__restrict__ pval, const float *__restrict__ W,
                 const float *__restrict__ H, float *__restrict__ P_out, float *__restrict__ Y, float *__restrict__ scratch,
                 int K4, unsigned long long *work_counter)
{
    // nonzeros in flight per warp.  Four (two for the longest rows): eight were measured slower at K = 256
    // (19.6 ms against 16.2 ms on the scale-22 R-MAT matrix) -- the registers they take cost a resident CTA
    constexpr int U = F >= 8 ? 2 : 4;
    const int lane = threadIdx.x & 31;
    const float4 *H4 = reinterpret_cast<const float4 *>(H);
    bool qv[F];
#pragma unroll
    for (int c = 0; c < F; ++c) qv[c] = lane + 32 * c < K4;

    // One row (or a piece of one): nonzeros [j0, j1) of row r; the sum goes to out (K floats).
    auto run_row = [&](int64_t j0, int64_t j1, int r, float *out) {
        float4 y[F], w[F];
#pragma unroll
        for (int c = 0; c < F; ++c) {
            y[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            w[c] = y[c];
            if (FUSED && qv[c]) w[c] = __ldg(reinterpret_cast<const float4 *>(W) + (int64_t)r * K4 + lane + 32 * c);
        }
        // lanes 0..U-1 hold the columns of the step's U nonzeros
        auto load_cols = [&](int64_t j) { return (lane < U && j + lane < j1) ? __ldcs(cols + j + lane) : 0; };
        int cnext = j0 < j1 ? load_cols(j0) : 0;
        for (int64_t j = j0; j < j1; j += U) {
            const int cmine = cnext;
            cnext = load_cols(j + U);
            float4 h[U][F];
#pragma unroll
            for (int i = 0; i < U; ++i) {
                const int ci = __shfl_sync(FULL, cmine, i);
                const bool live = j + i < j1;
#pragma unroll
                for (int c = 0; c < F; ++c)
                    h[i][c] = (live && qv[c]) ? ld_h(H4 + (int64_t)ci * K4 + lane + 32 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float p[U];
            if (FUSED) {
#pragma unroll
                for (int i = 0; i < U; ++i) {
                    float a = 0.f;
#pragma unroll
                    for (int c = 0; c < F; ++c) a = dot4(w[c], h[i][c], a);
                    p[i] = a;
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
                    for (int i = 0; i < U; ++i) p[i] += __shfl_xor_sync(FULL, p[i], off);
                }
                if (pval) {
                    const float s = (lane < U && j + lane < j1) ? __ldcs(pval + j + lane) : 0.f;
#pragma unroll
                    for (int i = 0; i < U; ++i) p[i] *= __shfl_sync(FULL, s, i);
                }
                if (P_out) {
                    float mine = p[0];
#pragma unroll
                    for (int i = 1; i < U; ++i) mine = lane == i ? p[i] : mine;
                    if (lane < U && j + lane < j1) __stcs(P_out + j + lane, mine);
                }
            } else {
                const float s = pval ? ((lane < U && j + lane < j1) ? __ldcs(pval + j + lane) : 0.f) : 1.f;
#pragma unroll
                for (int i = 0; i < U; ++i) p[i] = pval ? __shfl_sync(FULL, s, i) : 1.f;
            }
            // the nonzeros are added in their input order (dead ones carry h = 0)
#pragma unroll
            for (int i = 0; i < U; ++i) {
#pragma unroll
                for (int c = 0; c < F; ++c) {
                    y[c].x = fmaf(p[i], h[i][c].x, y[c].x);
                    y[c].y = fmaf(p[i], h[i][c].y, y[c].y);
                    y[c].z = fmaf(p[i], h[i][c].z, y[c].z);
                    y[c].w = fmaf(p[i], h[i][c].w, y[c].w);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < F; ++c)
            if (qv[c]) reinterpret_cast<float4 *>(out)[lane + 32 * c] = y[c];
    };

    for (;;) {
        unsigned long long t = 0;
        if (lane == 0) t = atomicAdd(work_counter, 1ull);
        t = __shfl_sync(FULL, t, 0);
        if ((int64_t)t >= n_tasks) break;
        const SpmmTask task = tasks[t];
        if (task.slot >= 0) {
            run_row(task.j0, task.j1, task.row_a, scratch + (int64_t)task.slot * K4 * 4);
        } else {
            for (int r = task.row_a; r < task.row_b; ++r)
                run_row(row_ptr[r], row_ptr[r + 1], r, Y + (int64_t)r * K4 * 4);
        }
    }
}

// Y[row] = sum of the row's scratch slots, in slot order.
__global__ void __launch_bounds__(256)
spmm_fixup_kernel(const SpmmLongRow *__restrict__ long_rows, int64_t n_long, const float *__restrict__ scratch,
                  float *__restrict__ Y, int K)
{
    for (int64_t i = blockIdx.x; i < n_long; i += gridDim.x) {
        const SpmmLongRow lr = long_rows[i];
        for (int t = threadIdx.x; t < K; t += blockDim.x) {
            float s = 0.f;
            for (int k = 0; k < lr.n_slots; ++k) s += scratch[((int64_t)lr.first_slot + k) * K + t];
            Y[(int64_t)lr.row * K + t] = s;
        }
    }
}

template <int F>
cudaError_t launch_rows(bool fused, const SpmmTask *tasks, int64_t n_tasks, const int64_t *row_ptr, const int32_t *cols,
                        const float *pval, const float *W, const float *H, float *P_out, float *Y, float *scratch, int K4,
                        unsigned long long *work_counter, int sm_count, cudaStream_t stream)
{
    int64_t blocks = (n_tasks + SPMM_WARPS - 1) / SPMM_WARPS;
    const int64_t cap = (int64_t)sm_count * 8;  // more than can be resident: the tasks are handed out by a counter
    if (blocks > cap) blocks = cap;
    if (fused)
        spmm_rows_kernel<F, true><<<(unsigned)blocks, SPMM_WARPS * 32, 0, stream>>>(tasks, n_tasks, row_ptr, cols, pval, W, H,
                                                                                   P_out, Y, scratch, K4, work_counter);
    else
        spmm_rows_kernel<F, false><<<(unsigned)blocks, SPMM_WARPS * 32, 0, stream>>>(tasks, n_tasks, row_ptr, cols, pval, W, H,
                                                                                    P_out, Y, scratch, K4, work_counter);
    return cudaGetLastError();
}

}  // namespace

void build_spmm_tasks(const int64_t *row_ptr_host, int64_t M, std::vector<SpmmTask> &tasks, std::vector<SpmmLongRow> &long_rows,
                      int64_t *n_slots, int64_t budget)
{
    if (budget <= 0) budget = SPMM_TASK_NNZ;
    tasks.clear();
    long_rows.clear();
    int64_t slots = 0;
    int64_t r = 0;
    while (r < M) {
        const int64_t n = row_ptr_host[r + 1] - row_ptr_host[r];
        if (n > budget) {
            // a long row: pieces of `budget` units, one scratch slot each
            SpmmLongRow lr;
            lr.row = (int32_t)r;
            lr.first_slot = (int32_t)slots;
            lr.n_slots = 0;
            for (int64_t j = row_ptr_host[r]; j < row_ptr_host[r + 1]; j += budget) {
                SpmmTask t;
                t.j0 = j;
                t.j1 = std::min<int64_t>(j + budget, row_ptr_host[r + 1]);
                t.row_a = (int32_t)r;
                t.row_b = (int32_t)r + 1;
                t.slot = (int32_t)slots++;
                t.pad = 0;
                tasks.push_back(t);
                ++lr.n_slots;
            }
            long_rows.push_back(lr);
            ++r;
            continue;
        }
        // a run of whole rows: until the next row would pass the budget (empty rows ride along; at most
        // 4096 rows per task so that long stretches of empty rows are shared out too)
        int64_t e = r, acc = 0;
        while (e < M && e - r < 4096) {
            const int64_t ne = row_ptr_host[e + 1] - row_ptr_host[e];
            if (ne > budget || (acc > 0 && acc + ne > budget)) break;
            acc += ne;
            ++e;
        }
        SpmmTask t;
        t.j0 = row_ptr_host[r];
        t.j1 = row_ptr_host[e];
        t.row_a = (int32_t)r;
        t.row_b = (int32_t)e;
        t.slot = -1;
        t.pad = 0;
        tasks.push_back(t);
        r = e;
    }
    *n_slots = slots;
}

bool spmm_supports(int K) { return K > 0 && K % 4 == 0 && K <= 1024; }

cudaError_t launch_spmm(bool fused, const SpmmTask *tasks, int64_t n_tasks, const SpmmLongRow *long_rows, int64_t n_long,
                        const int64_t *row_ptr, const int32_t *cols, const float *pval, const float *W, const float *H,
                        float *P_out, float *Y, float *scratch, int K, unsigned long long *work_counter, int sm_count,
                        cudaStream_t stream)
{
    if (n_tasks == 0) return cudaSuccess;
    cudaError_t e = cudaMemsetAsync(work_counter, 0, sizeof(unsigned long long), stream);
    if (e != cudaSuccess) return e;
    const int K4 = K / 4;
    const int F = (K4 + 31) / 32;
    if (F <= 1) e = launch_rows<1>(fused, tasks, n_tasks, row_ptr, cols, pval, W, H, P_out, Y, scratch, K4, work_counter, sm_count, stream);
    else if (F <= 2) e = launch_rows<2>(fused, tasks, n_tasks, row_ptr, cols, pval, W, H, P_out, Y, scratch, K4, work_counter, sm_count, stream);
    else if (F <= 4) e = launch_rows<4>(fused, tasks, n_tasks, row_ptr, cols, pval, W, H, P_out, Y, scratch, K4, work_counter, sm_count, stream);
    else if (F <= 8) e = launch_rows<8>(fused, tasks, n_tasks, row_ptr, cols, pval, W, H, P_out, Y, scratch, K4, work_counter, sm_count, stream);
    else return cudaErrorInvalidValue;
    if (e != cudaSuccess) return e;
    return launch_spmm_fixup(long_rows, n_long, scratch, Y, K, stream);
}

cudaError_t launch_spmm_fixup(const SpmmLongRow *long_rows, int64_t n_long, const float *scratch, float *Y, int K,
                              cudaStream_t stream)
{
    if (n_long <= 0) return cudaSuccess;
    spmm_fixup_kernel<<<(unsigned)std::min<int64_t>(n_long, 4096), 256, 0, stream>>>(long_rows, n_long, scratch, Y, K);
    return cudaGetLastError();
}

}  // namespace sddmm
