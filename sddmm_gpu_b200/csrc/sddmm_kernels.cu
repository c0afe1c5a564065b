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

namespace sddmm {

namespace {

constexpr unsigned FULL = 0xffffffffu;
// Upper bound on polls of an mbarrier before a CTA gives up and reports
// DEV_MBARRIER_TIMEOUT.  try_wait itself blocks for a hardware-defined slice, so
// this is far beyond any legitimate copy latency but still finite.
constexpr int MBAR_SPIN_LIMIT = 1 << 20;

__device__ __forceinline__ float4 ld_h(const float4 *p)
{
    // read-only path; H rows are the data worth keeping in L1/L2
    return __ldg(p);
}

__device__ __forceinline__ float dot4(float4 a, float4 b, float acc)
{
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
    return acc;
}

// Transposed butterfly over a group of L lanes holding B accumulators each
// (B <= L, both powers of two).  On return acc[0] of lane `lig` (lane in group)
// holds the complete sum of accumulator j = lig / (L/B); every lane of that
// L/B-lane cluster holds the same value.
template <int L, int B>
__device__ __forceinline__ void reduce_transposed(float (&acc)[B], int lig)
{
    int off = L >> 1;
#pragma unroll
    for (int half = B >> 1; half >= 1; half >>= 1) {
        const bool upper = (lig & off) != 0;
#pragma unroll
        for (int j = 0; j < half; ++j) {
            float send = upper ? acc[j] : acc[j + half];
            float keep = upper ? acc[j + half] : acc[j];
            acc[j] = keep + __shfl_xor_sync(FULL, send, off);
        }
        off >>= 1;
    }
#pragma unroll
    for (; off >= 1; off >>= 1) acc[0] += __shfl_xor_sync(FULL, acc[0], off);
}

// ---------------------------------------------------------------------------
// mbarrier / bulk-copy (TMA) primitives
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile(
        "{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, unsigned parity)
{
    for (int it = 0; it < MBAR_SPIN_LIMIT; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// 1-D bulk asynchronous copy global -> shared, completion counted in bytes on
// an mbarrier.  Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---------------------------------------------------------------------------
// One step of a warp: NB = B*G consecutive nonzeros starting at `base`
// (n_valid of them exist).  WSRC gives the W row of a nonzero.
// ---------------------------------------------------------------------------
template <int L, int C, int B>
struct Shape {
    static constexpr int G = 32 / L;       // nonzero groups per warp
    static constexpr int NB = B * G;       // nonzeros per warp step
    static constexpr int STRIDE4 = L * C;  // float4 chunks of a row per pass
    static_assert(B <= L, "transposed reduction needs B <= L");
    static_assert(NB <= 32, "index distribution uses one lane per nonzero");
};

template <int L, int C, int B, bool W_IN_SMEM>
__device__ __forceinline__ float warp_step(const float *__restrict__ Wbase,  // global W or smem panel
                                           const float *__restrict__ H, int my_row, int my_col,
                                           int n_valid, int K4, int lane)
{
    using S = Shape<L, C, B>;
    const int lig = lane & (L - 1);
    const int g = lane / L;
    float acc[B];
#pragma unroll
    for (int j = 0; j < B; ++j) acc[j] = 0.f;

    int rj[B], cj[B];
#pragma unroll
    for (int j = 0; j < B; ++j) {
        rj[j] = __shfl_sync(FULL, my_row, j * S::G + g);
        cj[j] = __shfl_sync(FULL, my_col, j * S::G + g);
    }

    for (int q0 = 0; q0 < K4; q0 += S::STRIDE4) {
        float4 hv[B][C];
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const float4 *hrow = reinterpret_cast<const float4 *>(H) + (int64_t)cj[j] * K4;
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const int q = q0 + c * L + lig;
                if (j * S::G < n_valid && q < K4) hv[j][c] = ld_h(hrow + q);
                else hv[j][c] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const float4 *wrow = reinterpret_cast<const float4 *>(Wbase) + (int64_t)rj[j] * K4;
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const int q = q0 + c * L + lig;
                if (j * S::G < n_valid && q < K4) {
                    float4 w = W_IN_SMEM ? wrow[q] : __ldg(wrow + q);
                    acc[j] = dot4(w, hv[j][c], acc[j]);
                }
            }
        }
    }
    reduce_transposed<L, B>(acc, lig);
    // route: lane t (< NB) takes the result of nonzero t = j*G + g
    const int t_j = lane / S::G, t_g = lane % S::G;
    const int src = t_g * L + (t_j & (B - 1)) * (L / B);
    return __shfl_sync(FULL, acc[0], src);
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
    for (int64_t base = warp * S::NB; base < nnz; base += n_warps * S::NB) {
        const int64_t rem = nnz - base;
        const int n_valid = rem < S::NB ? (int)rem : S::NB;
        int r = 0, c = 0;
        if (lane < n_valid) {
            r = __ldcs(rows + base + lane);
            c = __ldcs(cols + base + lane);
        }
        float res = warp_step<L, C, B, false>(W, H, r, c, n_valid, K4, lane);
        if (lane < n_valid) {
            if (sval) res *= __ldcs(sval + base + lane);
            __stcs(P + base + lane, res);
        }
    }
}

// ---------------------------------------------------------------------------
// Kernel B: row-panel kernel.
// ---------------------------------------------------------------------------
// Stage the W rows that the nonzeros [begin, begin+count) touch into `buf`
// (slot = row - row_begin), one bulk copy per distinct row, issued by the lanes
// of one warp.  Every lane posts the bytes it is about to copy with expect_tx
// before it issues them; lane 0 arrives last, so the phase cannot complete early.
__device__ __forceinline__ void stage_panel(const WorkItem &it, const int32_t *__restrict__ rows,
                                            const float *__restrict__ W, float *buf, uint64_t *bar,
                                            int K, int lane)
{
    const uint32_t row_bytes = (uint32_t)K * 4u;
    for (int o = lane; o < it.nnz_count; o += 32) {
        const int64_t i = it.nnz_begin + o;
        const int r = rows[i];
        const bool head = (o == 0) || (rows[i - 1] != r);
        if (head) {
            mbar_expect_tx(bar, row_bytes);
            bulk_g2s(buf + (int64_t)(r - it.row_begin) * K, W + (int64_t)r * K, row_bytes, bar);
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

template <int L, int C, int B, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
sddmm_panel_kernel(const WorkItem *__restrict__ items, int64_t n_items,
                   const int32_t *__restrict__ rows, const int32_t *__restrict__ cols,
                   const int32_t *__restrict__ perm, const float *__restrict__ sval,
                   const float *__restrict__ W, const float *__restrict__ H,
                   float *__restrict__ P, int K, int panel_floats, int *dev_status)
{
    using S = Shape<L, C, B>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *wbuf = reinterpret_cast<float *>(smem_raw);                               // 2 panels
    uint64_t *bars = reinterpret_cast<uint64_t *>(wbuf + 2 * (size_t)panel_floats);  // 2 barriers

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int K4 = K >> 2;

    if (threadIdx.x == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_fence_init();
    }
    __syncthreads();

    int64_t it_idx = blockIdx.x;
    if (warp == 0 && it_idx < n_items) {
        WorkItem it = items[it_idx];
        stage_panel(it, rows, W, wbuf, &bars[0], K, lane);
    }

    unsigned phase_bits = 0;   // bit b = parity of the next phase of buffer b
    bool next_issued = false;  // a prefetch into the other buffer is in flight
    bool aborted = false;
    int b = 0;
    for (; it_idx < n_items; it_idx += gridDim.x, b ^= 1) {
        const WorkItem it = items[it_idx];
        const int64_t next_idx = it_idx + gridDim.x;
        next_issued = next_idx < n_items;
        if (next_issued && warp == 0) {
            WorkItem nx = items[next_idx];
            stage_panel(nx, rows, W, wbuf + (size_t)(b ^ 1) * panel_floats, &bars[b ^ 1], K, lane);
        }
        const bool ok = mbar_wait_bounded(&bars[b], (phase_bits >> b) & 1u);
        if (__syncthreads_or(!ok)) {  // same decision in every thread
            aborted = true;
            break;
        }
        phase_bits ^= (1u << b);

        const float *wp = wbuf + (size_t)b * panel_floats;
        for (int off = warp * S::NB; off < it.nnz_count; off += NWARPS * S::NB) {
            const int rem = it.nnz_count - off;
            const int n_valid = rem < S::NB ? rem : S::NB;
            const int64_t base = it.nnz_begin + off;
            int r = 0, c = 0;
            if (lane < n_valid) {
                r = rows[base + lane] - it.row_begin;
                c = __ldcs(cols + base + lane);
            }
            float res = warp_step<L, C, B, true>(wp, H, r, c, n_valid, K4, lane);
            if (lane < n_valid) {
                if (perm) {
                    const int64_t dst = __ldcs(perm + base + lane);
                    if (sval) res *= __ldg(sval + dst);
                    P[dst] = res;
                } else {
                    if (sval) res *= __ldcs(sval + base + lane);
                    __stcs(P + base + lane, res);
                }
            }
        }
        __syncthreads();  // buffer b is free for the item after next
    }
    if (aborted) {
        // Report, then give the copies that may still be in flight (the panel that
        // timed out and the prefetch behind it) a bounded chance to land before
        // this CTA's shared memory is released.
        if (threadIdx.x == 0) atomicExch(dev_status, (int)DEV_MBARRIER_TIMEOUT);
        (void)mbar_wait_bounded(&bars[b], (phase_bits >> b) & 1u);
        if (next_issued) (void)mbar_wait_bounded(&bars[b ^ 1], (phase_bits >> (b ^ 1)) & 1u);
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

constexpr int PANEL_WARPS = 8;

template <int L, int C, int B>
cudaError_t launch_panel_t(const WorkItem *items, int64_t n_items, const int32_t *rows,
                           const int32_t *cols, const int32_t *perm, const float *sval,
                           const float *W, const float *H, float *P, int K, const PanelConfig &cfg,
                           int sm_count, int *dev_status, cudaStream_t stream)
{
    auto kern = sddmm_panel_kernel<L, C, B, PANEL_WARPS>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cfg.smem_bytes);
    if (e != cudaSuccess) return e;
    int64_t blocks = (int64_t)sm_count * cfg.ctas_per_sm;
    if (blocks > n_items) blocks = n_items;
    if (blocks < 1) blocks = 1;
    const int panel_floats = cfg.panel_rows * K;
    kern<<<(unsigned)blocks, PANEL_WARPS * 32, cfg.smem_bytes, stream>>>(items, n_items, rows, cols, perm, sval, W, H,
                                                                       P, K, panel_floats, dev_status);
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
        else if ((K) <= 64) { CALL(16, 1, 16); }       \
        else if ((K) <= 128) { CALL(32, 1, 16); }      \
        else if ((K) <= 256) { CALL(32, 2, 8); }       \
        else if ((K) <= 512) { CALL(32, 4, 4); }       \
        else { CALL(32, 8, 2); }                       \
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

cudaError_t launch_panel(const WorkItem *items, int64_t n_items, const int32_t *rows, const int32_t *cols,
                         const int32_t *perm, const float *sval, const float *W, const float *H, float *P,
                         int K, const PanelConfig &cfg, int sm_count, int *dev_status, cudaStream_t stream)
{
    if (n_items == 0) return cudaSuccess;
#define CALL(L, C, B) \
    return launch_panel_t<L, C, B>(items, n_items, rows, cols, perm, sval, W, H, P, K, cfg, sm_count, dev_status, stream)
    SDDMM_DISPATCH_K(K, CALL);
#undef CALL
    return cudaSuccess;
}

PanelConfig choose_panel_config(int K, int panel_rows_hint, int sm_count, size_t smem_optin)
{
    (void)sm_count;
    PanelConfig cfg;
    // Two W panels per CTA.  32 KB panels let three 8-warp CTAs share an SM
    // (3 x (64 KB + barriers) < 227 KB) while a panel still holds 32 rows at K = 256.
    size_t panel_bytes = 32 * 1024;
    const size_t row_bytes = (size_t)K * 4;
    if (row_bytes * 2 > panel_bytes) panel_bytes = row_bytes * 2;  // at least two rows per panel
    int rows = (int)(panel_bytes / row_bytes);
    if (panel_rows_hint > 0 && panel_rows_hint < rows) rows = panel_rows_hint;
    if (rows < 1) rows = 1;
    cfg.panel_rows = rows;
    cfg.smem_bytes = 2 * (size_t)rows * row_bytes + 64;
    while (cfg.smem_bytes > smem_optin && cfg.panel_rows > 1) {
        cfg.panel_rows /= 2;
        cfg.smem_bytes = 2 * (size_t)cfg.panel_rows * row_bytes + 64;
    }
    cfg.threads = PANEL_WARPS * 32;
    int per_sm = (int)((smem_optin + 1024) / (cfg.smem_bytes + 1024));
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 3) per_sm = 3;
    cfg.ctas_per_sm = per_sm;
    cfg.item_nnz = 2048;
    return cfg;
}

cudaError_t init_kernel_attributes(size_t) { return cudaSuccess; }

}  // namespace sddmm
