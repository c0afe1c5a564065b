// SDDMM compute kernels for sm_100a.
//
//   P[i] = dot(W[row_i, :], H[col_i, :]) [* S.val_i]      (fp32, K % 4 == 0)
//
// They replace comp_kernel_COO of the reference (HiPC18/src/kernel.h:2-52): one
// launch per call instead of n_col_tiles x K/k_slice launches, no read-modify-write
// of the result, 64-bit offsets, any K that is a multiple of 4.
//
// Work decomposition shared by both kernels.  A group of L lanes (L = 1..32, a
// power of two, L*4 floats cover min(K,128) floats) owns one nonzero at a time and
// processes B nonzeros per step, so a warp retires NB = B * (32/L) consecutive
// nonzeros per step.  All 128-bit H loads of a step are issued before the first
// use (B*C independent 16-byte loads per lane in flight).  The B partial sums of a
// lane are reduced with a transposed butterfly: the first log2(B) exchange rounds
// halve the number of live accumulators instead of keeping all of them, which
// costs B-1 + log2(L/B) shuffles per B nonzeros instead of B*log2(L).
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace sddmm {

using namespace dev;

namespace {

// ---------------------------------------------------------------------------
// Software-pipelined stream of warp steps.
//
// The nonzeros [begin, begin + count) are cut into chunks of NB consecutive
// nonzeros; warp `part` of `n_parts` takes a contiguous range of chunks.  The
// 128-bit H loads of chunk k+1 are issued before chunk k is consumed, and the
// row/column indices are fetched two chunks ahead, so that neither the index
// latency nor the gather latency is exposed between chunks: every warp keeps one
// or two chunks' worth of H rows (NB x K x 4 bytes each) in flight all the time.
//
// Consecutive chunks of a warp mostly lie in one row of S (rows are sorted and
// most nonzeros sit in long rows).  A chunk whose nonzeros all share a row takes
// that row of W from registers: it is (re)loaded only when the row changes, so
// the per-nonzero work is the H gather, K FMAs and the reduction.  Mixed chunks
// read W per nonzero (from the staged panel, or from global memory).
//
// The pipelined path is the predicate-free one: full chunks (NB valid nonzeros)
// of rows that one pass covers exactly (K == L*C*4).  The last, partial chunk
// and every other K take the general warp_step.
// ---------------------------------------------------------------------------
template <int B, int C>
struct StepBuf {
    float4 hv[B][C];
    int my_row;   // row of nonzero `lane` of the chunk (lanes >= NB mirror a valid one)
    int row0;     // row of the chunk's first nonzero
    bool single;  // every nonzero of the chunk lies in row0
};

template <int C>
struct WCache {
    float4 w[C];
    int row;  // row held in w, -1 if none
};

template <int L, int C, int B>
__device__ __forceinline__ void issue_h_loads(StepBuf<B, C> &buf, const char *__restrict__ H_lane,
                                              unsigned row_bytes, int my_row, int my_col, int lane)
{
    using S = Shape<L, C, B>;
    const int g = lane / L;
    buf.my_row = my_row;
    buf.row0 = __shfl_sync(FULL, my_row, 0);
    buf.single = __all_sync(FULL, my_row == buf.row0);
#pragma unroll
    for (int j = 0; j < B; ++j) {
        const unsigned cj = (unsigned)__shfl_sync(FULL, my_col, j * S::G + g);
        const float4 *hrow = reinterpret_cast<const float4 *>(H_lane + (size_t)cj * row_bytes);
#pragma unroll
        for (int c = 0; c < C; ++c) buf.hv[j][c] = ld_h(hrow + c * L);
    }
}

template <int L, int C, int B, bool W_IN_SMEM>
__device__ __forceinline__ float consume_step(const StepBuf<B, C> &buf, WCache<C> &wc,
                                              const char *__restrict__ W_lane, unsigned row_bytes, int lane)
{
    using S = Shape<L, C, B>;
    const int lig = lane & (L - 1);
    const int g = lane / L;
    float acc[B];
    // 32-bit offset inside a staged panel, 64-bit into the whole of W otherwise
    auto w_row_ptr = [&](unsigned r) {
        return reinterpret_cast<const float4 *>(W_IN_SMEM ? W_lane + r * row_bytes : W_lane + (size_t)r * row_bytes);
    };
    if (buf.single) {
        if (buf.row0 != wc.row) {
            const float4 *wrow = w_row_ptr((unsigned)buf.row0);
#pragma unroll
            for (int c = 0; c < C; ++c) wc.w[c] = W_IN_SMEM ? wrow[c * L] : __ldg(wrow + c * L);
            wc.row = buf.row0;
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            acc[j] = 0.f;
#pragma unroll
            for (int c = 0; c < C; ++c) acc[j] = dot4(wc.w[c], buf.hv[j][c], acc[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < B; ++j) {
            acc[j] = 0.f;
            const unsigned rj = (unsigned)__shfl_sync(FULL, buf.my_row, j * S::G + g);
            const float4 *wrow = w_row_ptr(rj);
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const float4 w = W_IN_SMEM ? wrow[c * L] : __ldg(wrow + c * L);
                acc[j] = dot4(w, buf.hv[j][c], acc[j]);
            }
        }
    }
    reduce_transposed<L, B>(acc, lig);
    const int t_j = lane / S::G, t_g = lane % S::G;
    const int src = t_g * L + (t_j & (B - 1)) * (L / B);
    return __shfl_sync(FULL, acc[0], src);
}

// store(off, n_valid, value): lane t < n_valid holds the result of nonzero begin + off + t.
// IdxT: int for the bounded range of a work item, int64_t for a whole matrix.
template <int L, int C, int B, bool W_IN_SMEM, class IdxT, class StoreFn>
__device__ __forceinline__ void warp_stream(const int32_t *__restrict__ rows, const int32_t *__restrict__ cols,
                                            int row_bias, const float *__restrict__ Wbase,
                                            const float *__restrict__ H, int64_t begin, IdxT count, IdxT part,
                                            IdxT n_parts, int K4, int lane, StoreFn store)
{
    using S = Shape<L, C, B>;
    const IdxT n_full = count / S::NB;
    const int tail = (int)(count - n_full * S::NB);
    rows += begin;
    cols += begin;
    if (tail > 0 && part == n_parts - 1) {  // the partial chunk
        const IdxT off = n_full * S::NB;
        int r = 0, c = 0;
        if (lane < tail) {
            r = __ldcs(rows + off + lane) - row_bias;
            c = __ldcs(cols + off + lane);
        }
        const float res = warp_step<L, C, B, W_IN_SMEM>(Wbase, H, r, c, tail, K4, lane);
        store(off, tail, res);
    }
    // this warp's contiguous share of the full chunks
    IdxT k = (IdxT)(((int64_t)n_full * part) / n_parts);
    const IdxT k_end = (IdxT)(((int64_t)n_full * (part + 1)) / n_parts);
    if (k >= k_end) return;
    if (K4 != S::STRIDE4) {  // rows that one pass does not cover exactly: general step, not pipelined
        for (; k < k_end; ++k) {
            const IdxT off = k * S::NB;
            int r = 0, c = 0;
            if (lane < S::NB) {
                r = __ldcs(rows + off + lane) - row_bias;
                c = __ldcs(cols + off + lane);
            }
            const float res = warp_step<L, C, B, W_IN_SMEM>(Wbase, H, r, c, S::NB, K4, lane);
            store(off, S::NB, res);
        }
        return;
    }

    const unsigned row_bytes = (unsigned)K4 * 16u;
    const int lig = lane & (L - 1);
    const char *H_lane = reinterpret_cast<const char *>(H) + lig * 16;
    const char *W_lane = reinterpret_cast<const char *>(Wbase) + lig * 16;
    const int il = lane & (S::NB - 1);  // lanes >= NB mirror a valid nonzero (NB is a power of two)
    auto load_raw = [&](IdxT kk, int &r, int &c) {
        // past the end the last chunk is read again (harmless, never consumed)
        if (kk >= k_end) kk = k_end - 1;
        r = __ldcs(rows + kk * S::NB + il) - row_bias;
        c = __ldcs(cols + kk * S::NB + il);
    };
    StepBuf<B, C> bufA, bufB;
    WCache<C> wc;
    wc.row = -1;
    int r_nx, c_nx;
    {
        int r0, c0;
        load_raw(k, r0, c0);
        load_raw(k + 1, r_nx, c_nx);
        issue_h_loads<L, C, B>(bufA, H_lane, row_bytes, r0, c0, lane);
    }
    while (true) {
        // bufA holds chunk k; (r_nx, c_nx) are the indices of chunk k + 1
        {
            const bool more = k + 1 < k_end;
            if (more) issue_h_loads<L, C, B>(bufB, H_lane, row_bytes, r_nx, c_nx, lane);
            load_raw(k + 2, r_nx, c_nx);
            const float res = consume_step<L, C, B, W_IN_SMEM>(bufA, wc, W_lane, row_bytes, lane);
            store(k * S::NB, S::NB, res);
            if (!more) break;
            ++k;
        }
        {
            const bool more = k + 1 < k_end;
            if (more) issue_h_loads<L, C, B>(bufA, H_lane, row_bytes, r_nx, c_nx, lane);
            load_raw(k + 2, r_nx, c_nx);
            const float res = consume_step<L, C, B, W_IN_SMEM>(bufB, wc, W_lane, row_bytes, lane);
            store(k * S::NB, S::NB, res);
            if (!more) break;
            ++k;
        }
    }
}

// ---------------------------------------------------------------------------
// Kernel A: planless gather.  Warps stride over the nonzeros; W rows come from
// global memory through L1 (row-sorted input makes consecutive nonzeros share them).
// ---------------------------------------------------------------------------
template <int L, int C, int B>
__global__ void __launch_bounds__(256)
sddmm_gather_kernel(const int32_t *__restrict__ rows, const int32_t *__restrict__ cols,
                    const float *__restrict__ sval, const float *__restrict__ W,
                    const float *__restrict__ H, float *__restrict__ P, int64_t nnz, int K4)
{
    using S = Shape<L, C, B>;
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    auto store = [&](int64_t off, int n_valid, float res) {
        if (lane < n_valid) {
            if (sval) res *= __ldcs(sval + off + lane);
            __stcs(P + off + lane, res);
        }
    };
    warp_stream<L, C, B, false, int64_t>(rows, cols, 0, W, H, 0, nnz, warp, n_warps, K4, lane, store);
}

// ---------------------------------------------------------------------------
// Kernel B: row-panel kernel.
//
// Persistent CTAs walk the work items (item = blockIdx.x, + gridDim.x, ...).
// One producer warp stages the W rows an item touches into one of two
// shared-memory panels with bulk asynchronous copies (TMA) -- slot = row -
// item.row_begin, one copy per distinct row -- always one item ahead of the
// NWARPS consumer warps.  full[b] (tx-count mbarrier) tells the consumers that
// panel b has landed, empty[b] (NWARPS arrivals) tells the producer that every
// consumer is done with it; nobody waits on a CTA-wide barrier inside the loop,
// so a warp that finishes its share of an item early moves on to the next one.
// Every wait is bounded; a wait that gives up raises DEV_MBARRIER_TIMEOUT and the
// CTA drains and returns.
// ---------------------------------------------------------------------------
struct PanelSmem {
    uint64_t full[2];
    uint64_t empty[2];
    int abort_flag;
};

__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, unsigned parity, volatile int *abort_flag)
{
    WaitClock clock;
    for (int it = 0; it < MBAR_SPIN_LIMIT; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255) == 255 && *abort_flag) return false;
        if (clock.expired(it)) return false;
    }
    return false;
}

template <int L, int C, int B, int NWARPS>
__global__ void __launch_bounds__((NWARPS + 1) * 32, 1)
sddmm_panel_kernel(const WorkItem *__restrict__ items, int64_t n_items,
                   const int32_t *__restrict__ item_rows, const int32_t *__restrict__ rows,
                   const int32_t *__restrict__ cols, const int32_t *__restrict__ perm,
                   const float *__restrict__ sval, const float *__restrict__ W,
                   const float *__restrict__ H, float *__restrict__ P, int K, int panel_floats,
                   int *dev_status)
{
    using S = Shape<L, C, B>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *wbuf = reinterpret_cast<float *>(smem_raw);  // 2 panels
    PanelSmem *sm = reinterpret_cast<PanelSmem *>(wbuf + 2 * (size_t)panel_floats);

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int K4 = K >> 2;

    if (threadIdx.x == 0) {
        mbar_init(&sm->full[0], 1);
        mbar_init(&sm->full[1], 1);
        mbar_init(&sm->empty[0], NWARPS);
        mbar_init(&sm->empty[1], NWARPS);
        sm->abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    volatile int *abort_flag = &sm->abort_flag;
    bool timed_out = false;

    if (warp == NWARPS) {
        // ---- producer warp ----
        const uint32_t row_bytes = (uint32_t)K * 4u;
        int n = 0;
        for (int64_t idx = blockIdx.x; idx < n_items; idx += gridDim.x, ++n) {
            const int b = n & 1;
            if (n >= 2) {  // panel b was last used by item n-2: wait until every consumer released it
                if (!wait_or_abort(&sm->empty[b], ((n - 2) >> 1) & 1u, abort_flag)) { timed_out = true; break; }
            }
            const WorkItem it = items[idx];
            float *buf = wbuf + (size_t)b * panel_floats;
            // it.reserved = offset of the item's distinct-row list, it.n_rows... see binning
            const int n_list = it.n_rows;
            for (int e = lane; e < n_list; e += 32) {
                const int r = __ldg(item_rows + it.list_begin + e);
                mbar_expect_tx(&sm->full[b], row_bytes);
                bulk_g2s(buf + (int64_t)(r - it.row_begin) * K, W + (int64_t)r * K, row_bytes, &sm->full[b]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->full[b]);
        }
        // before leaving, make sure every copy this warp issued has landed: the
        // consumers wait for them anyway, except on the abort path
        if (timed_out) {
            if (lane == 0) { *abort_flag = 1; atomicExch(dev_status, (int)DEV_MBARRIER_TIMEOUT); }
        }
    } else {
        // ---- consumer warps ----
        int n = 0;
        for (int64_t idx = blockIdx.x; idx < n_items; idx += gridDim.x, ++n) {
            const int b = n & 1;
            const WorkItem it = items[idx];
            if (!wait_or_abort(&sm->full[b], (n >> 1) & 1u, abort_flag)) { timed_out = true; break; }
            const float *wp = wbuf + (size_t)b * panel_floats;
            const int64_t begin = it.nnz_begin;
            auto store = [&](int off, int n_valid, float res) {
                if (lane < n_valid) {
                    const int64_t j = begin + off + lane;
                    if (perm) {
                        const int64_t dst = __ldcs(perm + j);
                        if (sval) res *= __ldg(sval + dst);
                        P[dst] = res;
                    } else {
                        if (sval) res *= __ldcs(sval + j);
                        __stcs(P + j, res);
                    }
                }
            };
            warp_stream<L, C, B, true, int>(rows, cols, it.row_begin, wp, H, begin, it.nnz_count, warp, NWARPS, K4,
                                            lane, store);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->empty[b]);
        }
        if (timed_out && lane == 0) { *abort_flag = 1; atomicExch(dev_status, (int)DEV_MBARRIER_TIMEOUT); }
    }
    // Copies may only still be in flight on the abort path (otherwise every
    // issued panel was waited for by the consumers).  Give them a bounded chance
    // to land before the CTA's shared memory is released.
    __syncthreads();
    if (sm->abort_flag && threadIdx.x < 2) {
        for (int p = 0; p < 2; ++p)
            for (int it = 0; it < (1 << 12); ++it)
                if (mbar_try_wait(&sm->full[threadIdx.x], (unsigned)p)) break;
    }
}

template <int L, int C, int B>
cudaError_t launch_gather_t(const int32_t *rows, const int32_t *cols, const float *sval, const float *W,
                            const float *H, float *P, int64_t nnz, int K, int sm_count,
                            cudaStream_t stream)
{
    using S = Shape<L, C, B>;
    const int threads = 256;
    const int64_t steps = (nnz + S::NB - 1) / S::NB;
    int64_t blocks = (steps + (threads / 32) - 1) / (threads / 32);
    const int64_t cap = (int64_t)sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    sddmm_gather_kernel<L, C, B><<<(unsigned)blocks, threads, 0, stream>>>(rows, cols, sval, W, H, P, nnz, K / 4);
    return cudaGetLastError();
}

constexpr int PANEL_WARPS = 15;  // consumer warps; with the producer warp 16 warps = 4 per SM sub-partition, 128 registers each

template <int L, int C, int B>
cudaError_t launch_panel_t(const WorkItem *items, int64_t n_items, const int32_t *item_rows, const int32_t *rows,
                           const int32_t *cols, const int32_t *perm, const float *sval,
                           const float *W, const float *H, float *P, int K, const PanelConfig &cfg,
                           int sm_count, int *dev_status, cudaStream_t stream)
{
    auto kern = sddmm_panel_kernel<L, C, B, PANEL_WARPS>;
    static SmemOptinCache optin;  // largest opt-in made so far for this instantiation, per device
    {
        cudaError_t e = optin_dynamic_smem(kern, cfg.smem_bytes, optin);
        if (e != cudaSuccess) return e;
    }
    int64_t blocks = (int64_t)sm_count * cfg.ctas_per_sm;
    if (blocks > n_items) blocks = n_items;
    if (blocks < 1) blocks = 1;
    const int panel_floats = cfg.panel_rows * K;
    kern<<<(unsigned)blocks, (PANEL_WARPS + 1) * 32, cfg.smem_bytes, stream>>>(items, n_items, item_rows, rows, cols,
                                                                             perm, sval, W, H, P, K, panel_floats,
                                                                             dev_status);
    return cudaGetLastError();
}

}  // namespace

// K -> (L, C, B): L lanes x C float4 per lane cover one pass over (part of) a row.
#define SDDMM_DISPATCH_K(K, CALL)                      \
    do {                                               \
        if ((K) <= 4) { CALL(1, 1, 1); }               \
        else if ((K) <= 8) { CALL(2, 1, 2); }          \
        else if ((K) <= 16) { CALL(4, 1, 4); }         \
        else if ((K) <= 32) { CALL(8, 1, 8); }         \
        else if ((K) <= 64) { CALL(16, 1, 8); }        \
        else if ((K) <= 128) { CALL(32, 1, 8); }       \
        else if ((K) <= 256) { CALL(32, 2, 4); }       \
        else if ((K) <= 512) { CALL(32, 4, 2); }       \
        else { CALL(32, 8, 1); }                       \
    } while (0)

cudaError_t launch_gather(const int32_t *rows, const int32_t *cols, const float *sval, const float *W,
                          const float *H, float *P, int64_t nnz, int K, int sm_count, cudaStream_t stream)
{
    if (nnz == 0) return cudaSuccess;
#define CALL(L, C, B) return launch_gather_t<L, C, B>(rows, cols, sval, W, H, P, nnz, K, sm_count, stream)
    SDDMM_DISPATCH_K(K, CALL);
#undef CALL
    return cudaSuccess;
}

cudaError_t launch_panel(const WorkItem *items, int64_t n_items, const int32_t *item_rows, const int32_t *rows,
                         const int32_t *cols, const int32_t *perm, const float *sval, const float *W, const float *H, float *P,
                         int K, const PanelConfig &cfg, int sm_count, int *dev_status, cudaStream_t stream)
{
    if (n_items == 0) return cudaSuccess;
#define CALL(L, C, B) \
    return launch_panel_t<L, C, B>(items, n_items, item_rows, rows, cols, perm, sval, W, H, P, K, cfg, sm_count, dev_status, stream)
    SDDMM_DISPATCH_K(K, CALL);
#undef CALL
    return cudaSuccess;
}

PanelConfig choose_panel_config(int K, int panel_rows_hint, int sm_count, size_t smem_optin)
{
    (void)sm_count;
    PanelConfig cfg;
    // One persistent CTA per SM: 15 consumer warps + 1 producer warp, two W
    // panels of up to 48 KB each (48 rows at K = 256).
    size_t panel_bytes = 48 * 1024;
    const size_t row_bytes = (size_t)K * 4;
    if (row_bytes * 2 > panel_bytes) panel_bytes = row_bytes * 2;  // at least two rows per panel
    int rows = (int)(panel_bytes / row_bytes);
    if (panel_rows_hint > 0 && panel_rows_hint < rows) rows = panel_rows_hint;
    if (rows < 1) rows = 1;
    cfg.panel_rows = rows;
    cfg.smem_bytes = 2 * (size_t)rows * row_bytes + 128;
    while (cfg.smem_bytes > smem_optin && cfg.panel_rows > 1) {
        cfg.panel_rows /= 2;
        cfg.smem_bytes = 2 * (size_t)cfg.panel_rows * row_bytes + 128;
    }
    cfg.threads = (PANEL_WARPS + 1) * 32;
    cfg.ctas_per_sm = 1;
    cfg.item_nnz = 4096;
    return cfg;
}

namespace {
// The wait that is meant to run out: same try_wait + back-off loop as the real
// kernels, with a poll limit of a few thousand (a few milliseconds at most).
__global__ void wait_timeout_probe_kernel(int *dev_status)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncwarp();
    bool done = false;
    for (int it = 0; it < 4096 && !done; ++it) {
        done = mbar_try_wait(&bar, 0);
        if (!done) __nanosleep(256);
    }
    if (!done && threadIdx.x == 0) atomicExch(dev_status, (int)DEV_MBARRIER_TIMEOUT);
}
}  // namespace

cudaError_t launch_wait_timeout_probe(int *dev_status, cudaStream_t stream)
{
    wait_timeout_probe_kernel<<<1, 32, 0, stream>>>(dev_status);
    return cudaGetLastError();
}

}  // namespace sddmm
