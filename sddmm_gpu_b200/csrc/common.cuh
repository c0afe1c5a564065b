// Shared declarations of the sm_100a SDDMM engine (internal; the public surface
// is include/sddmm_b200.h).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>
#include <string>
#include <vector>

#include "sddmm_b200.h"

namespace sddmm {

// One unit of work of the row-panel kernel: a run of consecutive nonzeros (in the
// plan's processing order) whose rows all lie in [row_begin, row_begin + n_rows),
// n_rows <= the plan's panel height, so that the W rows they touch fit one
// shared-memory panel.  Built on the device by the binning pass.
struct WorkItem {
    int64_t nnz_begin;   // first nonzero (processing order)
    int64_t list_begin;  // offset of the item's distinct rows in the plan's item-row list
    int32_t nnz_count;
    int32_t row_begin;   // smallest row of the item
    int32_t n_rows;      // number of distinct rows (entries of the item-row list)
    int32_t reserved;
};

// A dense cell of S: rows [row0, row0 + DENSE_CELL_ROWS) x columns [col0, col0 +
// DENSE_CELL_COLS) (clipped), whose `count` nonzeros start at `offset` in the
// plan's dense arrays.  cls 0: row0 indexes the list of compacted full rows;
// cls 1: col0 indexes the list of compacted full columns; cls 2: both are
// plain matrix coordinates.
constexpr int DENSE_CELL_ROWS = 128;
constexpr int DENSE_CELL_COLS = 64;
struct DenseCell {
    int64_t offset;
    int32_t row0, col0;
    int32_t count;
    int32_t cls;
};

// The opt-in to more than 48 KB of dynamic shared memory (cudaFuncSetAttribute) is a
// property of a kernel ON ONE DEVICE: a process that drives several GPUs must make it
// on each of them.  One cache per kernel instantiation remembers the largest size
// already granted, per device ordinal; devices beyond the table are never cached.
struct SmemOptinCache {
    static constexpr int MAX_DEVICES = 64;
    std::atomic<size_t> granted[MAX_DEVICES];
    SmemOptinCache() { for (auto &g : granted) g.store(0, std::memory_order_relaxed); }
    bool needs(int device, size_t bytes) const
    {
        return device < 0 || device >= MAX_DEVICES || bytes > granted[device].load(std::memory_order_acquire);
    }
    void record(int device, size_t bytes)
    {
        if (device >= 0 && device < MAX_DEVICES) granted[device].store(bytes, std::memory_order_release);
    }
};

// Makes the opt-in for `kern` on the current device unless `cache` says it holds.
template <class Kern>
inline cudaError_t optin_dynamic_smem(Kern kern, size_t bytes, SmemOptinCache &cache)
{
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (!cache.needs(device, bytes)) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) cache.record(device, bytes);
    return e;
}

// Device status word written by kernels whose bounded waits give up.
enum DeviceStatus : int { DEV_OK = 0, DEV_MBARRIER_TIMEOUT = 1 };

struct PanelConfig {
    int panel_rows;      // rows of W per staged panel
    int item_nnz;        // nonzero budget of one work item
    int threads;         // CTA size
    int ctas_per_sm;     // resident CTAs per SM the launch is sized for
    size_t smem_bytes;   // dynamic shared memory per CTA
};

// Chooses panel height / item budget / CTA shape for a given K and hint.
PanelConfig choose_panel_config(int K, int panel_rows_hint, int sm_count, size_t smem_optin);

// Planless kernel: every sub-warp group gathers its W row and H row from global
// memory.  rows/cols/P in the same (input) order.
cudaError_t launch_gather(const int32_t *rows, const int32_t *cols, const float *sval,
                          const float *W, const float *H, float *P, int64_t nnz, int K,
                          int sm_count, cudaStream_t stream);

// Row-panel kernel: persistent CTAs walk the work items; the W rows an item
// touches (item_rows lists them) are staged into shared memory with bulk
// asynchronous copies (TMA, double-buffered on mbarriers) by a producer warp,
// H rows are gathered with software-pipelined 128-bit loads.
// perm == nullptr: P[j] = result of processing-order nonzero j (sval indexed the
// same way).  perm != nullptr: result of j goes to P[perm[j]], scaled by sval[perm[j]].
cudaError_t launch_panel(const WorkItem *items, int64_t n_items, const int32_t *item_rows,
                         const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                         const float *W, const float *H, float *P, int K,
                         const PanelConfig &cfg, int sm_count, int *dev_status,
                         cudaStream_t stream);

// dst[r*K + t] = src[t*n + r]: a K-major operand (K x n) into the row-major layout (n x K) the kernels read.
cudaError_t launch_transpose_operand(const float *src_kmajor, float *dst_rowmajor, int64_t n, int K, cudaStream_t stream);

// Copies the listed rows (K floats each) of a row-major array in mapped, page-locked
// host memory to the same rows of a device array; the GPU reads the host memory.
cudaError_t launch_upload_rows(const float *mapped_host, float *dev, const int32_t *d_row_list, int64_t n_rows, int K,
                               int n_ctas, cudaStream_t stream);

// Ring kernel: H rows gathered by bulk asynchronous copies (TMA) into per-warp
// shared-memory rings, work handed out dynamically through *work_counter (one
// device word, zeroed by the launcher).  K must satisfy ring_supports(K)
// (32, 64, 128, 256, 512, 1024).
bool ring_supports(int K);
// cols_hinted: bit 31 of every column index marks a hub column (see build_hub_column_hints).
cudaError_t launch_ring(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                        const float *W, const float *H, float *P, int64_t nnz, int K, bool cols_hinted, int sm_count,
                        unsigned long long *work_counter, int *dev_status, cudaStream_t stream);

// Column-tile kernel: a tile of htile_cols(K) rows of H in shared memory, nonzeros in tiled order (column tiles
// ascending; tile_off[t] = first nonzero of tile t, n_tiles + 1 device entries from build_htile_offsets; perm = input
// position of a nonzero or null).  htile_cols(K) is 0 for an unsupported K (supported: 128, 256, 512); W and H must
// be 16-byte aligned.
int htile_cols(int K);
cudaError_t build_htile_offsets(const int32_t *cols_t, int64_t nnz, int col_tile, int n_tiles, int64_t *d_off,
                                cudaStream_t stream);
cudaError_t launch_htile(const int32_t *rows_t, const int32_t *cols_t, const int32_t *perm, const float *sval, const float *W,
                         const float *H, float *P, int64_t nnz, int64_t N, int K, int col_tile, const int64_t *tile_off,
                         int n_tiles, int sm_count, int *dev_status, cudaStream_t stream);

// The same TMA rings over operands stored in bfloat16 (rows of 2K bytes; products and sums in fp32):
// K = 256, 512, 1024 or 2048.  Opt-in, outside the fp32 tolerance contract.
bool ring_bf16_supports(int K);
cudaError_t launch_ring_bf16(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                             const void *W_bf16, const void *H_bf16, float *P, int64_t nnz, int K, bool cols_hinted, int sm_count,
                             unsigned long long *work_counter, int *dev_status, cudaStream_t stream);

// Dense-cell kernel: every dense cell is computed as the 128 x 64 block
// W[rows] * H[cols]^T -- fp32 FMAs, or (tensor) 3xTF32 on the tensor cores -- then
// the cell's nonzeros pick their entries: P[idx[i]] = block[rc[i]] (* sval[idx[i]]).
// Cells whose cls has bit 8 set are in row-mask form (row_mask / row_base, see DensePlan) and
// do not read idx / rc.
cudaError_t launch_dense_cells(const DenseCell *cells, int64_t n_cells, const int32_t *idx, const uint16_t *rc,
                               const unsigned long long *row_mask, const int32_t *row_base, const int32_t *dense_rows, int64_t n_dense_rows, const int32_t *dense_cols,
                               int64_t n_dense_cols, const float *sval, const float *W, const float *H, float *P,
                               int64_t M, int64_t N, int K, bool tensor, int sm_count, cudaStream_t stream);

// The same dense cells on tcgen05: MMAs issued by one thread from shared-memory descriptors, accumulator in
// tensor memory (3xTF32).  dev_status receives DEV_MBARRIER_TIMEOUT if a bounded wait gives up.
cudaError_t launch_dense_cells_tc(const DenseCell *cells, int64_t n_cells, const int32_t *idx, const uint16_t *rc,
                                  const unsigned long long *row_mask, const int32_t *row_base, const int32_t *dense_rows,
                                  int64_t n_dense_rows, const int32_t *dense_cols, int64_t n_dense_cols, const float *sval,
                                  const float *W, const float *H, float *P, int64_t M, int64_t N, int K, int sm_count,
                                  int *dev_status, cudaStream_t stream);

// Ring kernel for short rows (K = 32, 64, 128): the same per-warp rings filled with
// 16-byte cp.async copies; reached through launch_ring.
cudaError_t launch_ring_small(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                              const float *W, const float *H, float *P, int64_t nnz, int K, bool cols_hinted,
                              int sm_count, unsigned long long *work_counter, cudaStream_t stream);

// SpMM / fused SDDMM->SpMM over the plan's rows (spmm.cu).  A task is a run of whole rows
// [row_a, row_b) (slot < 0), or the nonzeros [j0, j1) of the long row row_a, summed into scratch slot `slot`.
struct SpmmTask {
    int64_t j0, j1;
    int32_t row_a, row_b;
    int32_t slot, pad;
};
struct SpmmLongRow {
    int32_t row, first_slot, n_slots;
};
bool spmm_supports(int K);  // K a multiple of 4, at most 1024
// Host: tasks and long-row table from the row pointer over all M rows; *n_slots = scratch slots (K floats each).
// `budget`: units (nonzeros, or groups when the offsets count groups) a task aims for; 0 = the default.
void build_spmm_tasks(const int64_t *row_ptr_host, int64_t M, std::vector<SpmmTask> &tasks, std::vector<SpmmLongRow> &long_rows,
                      int64_t *n_slots, int64_t budget = 0);
cudaError_t launch_spmm_fixup(const SpmmLongRow *long_rows, int64_t n_long, const float *scratch, float *Y, int K,
                              cudaStream_t stream);
// The same operations for K = 256, 512, 1024 on the shared-memory gather rings (spmm_ring.cu), over the plan's row
// groups (build_row_groups); tasks count GROUPS here (j0, j1 are group indices).
bool spmm_ring_supports(int K);
int spmm_ring_group_slots(int K);
cudaError_t launch_spmm_ring(bool fused, const SpmmTask *tasks, int64_t n_tasks, const int32_t *pcols, const int32_t *pidx,
                             const int32_t *grow, const float *pval, const float *W, const float *H, float *P_out, float *Y,
                             float *scratch, int K, unsigned long long *work_counter, int *dev_status, int sm_count,
                             cudaStream_t stream);
cudaError_t launch_spmm(bool fused, const SpmmTask *tasks, int64_t n_tasks, const SpmmLongRow *long_rows, int64_t n_long,
                        const int64_t *row_ptr, const int32_t *cols, const float *pval, const float *W, const float *H,
                        float *P_out, float *Y, float *scratch, int K, unsigned long long *work_counter, int sm_count,
                        cudaStream_t stream);

// float64 recomputation of every stride-th nonzero on the device (see check.cu).
struct CheckResult {
    unsigned long long n_checked;
    unsigned long long n_bad;      // sampled nonzeros with |P - ref| > tol * max(|ref|, A), or not finite
    double max_scaled_err;         // max |P - ref| / max(|ref|, A)
};
cudaError_t launch_check_result(const int32_t *rows, const int32_t *cols, const float *sval, const float *W, const float *H,
                                const float *P, int64_t nnz, int K, int64_t stride, double tol, CheckResult *d_out,
                                int sm_count, cudaStream_t stream);

// Self-test of the bounded-wait path: one warp waits (with a short poll limit) on
// an mbarrier that nothing ever arrives on, gives up, records DEV_MBARRIER_TIMEOUT
// in *dev_status and returns normally.  Nothing faults, traps or hangs.
cudaError_t launch_wait_timeout_probe(int *dev_status, cudaStream_t stream);

}  // namespace sddmm
