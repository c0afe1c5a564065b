// SpMM / fused SDDMM->SpMM for long rows (K = 256, 512, 1024) on the shared-memory
// gather rings of the SDDMM kernel.
//
//     Y[r, :] = sum over the nonzeros i of row r of  p_i * H[col_i, :]
//     p_i = Pval[i] (SpMM)   or   (sum_t W[r,t] H[col_i,t]) * Sval[i] (fused)
//
// Why a second form beside spmm.cu: there the H rows are staged in registers and a
// warp keeps 4 KB in flight; here every H row is one bulk copy (TMA) into a 4 KB
// ring slot counted on an mbarrier, two slots per warp in flight without a single
// register held for them -- the same reason the SDDMM ring kernel exists.
//
// Shape.  The rows of S are cut into GROUPS of B = 4096 / (4K) slots at plan time
// (build_row_groups): a row's last group is padded with slots that repeat a real
// column and carry index -1 (weight 0), so the B lane sets of a warp -- one per
// slot, LPN = 32 / B lanes each, every lane 8 float4 of its slot's H row -- always
// work on the SAME row of S.  Per group and lane set: the slot's H row comes from
// shared memory once into registers, is multiplied with the lane's share of the W
// row (fused; one log2(LPN)-step butterfly gives every lane of the set p_i), and
// p_i times the same registers is added to the lane's share of the Y row.  When a
// row ends (a bit in the group's row word, uniform over the warp) the B partial Y
// rows are added across the lane sets by shuffles and one set stores the row.
// Work comes as TASKS (spmm.cu): runs of whole rows, or pieces of a long row that
// go to scratch slots and are summed in slot order by spmm_fixup_kernel -- no
// atomics on Y, nothing depends on scheduling.  Rows of S without nonzeros inside a
// task's row range are written as zeros by the task's warp.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace sddmm {

using namespace dev;

namespace {

constexpr int SPR_WARPS = 16;
constexpr int SPR_NG = 3;       // ring slots per warp: two groups in flight while one is read
constexpr int SPR_SLOT = 4096;  // H bytes of one group

template <int C>
struct SpmmRingShape {
    static constexpr int ROW_BYTES = C * 512;
    static constexpr int B = SPR_SLOT / ROW_BYTES;  // slots of a group: 4, 2, 1
    static constexpr int LPN = 32 / B;              // lanes per slot: 8, 16, 32
    static constexpr int F = 8;                     // float4 per lane per row
    static_assert(LPN * F * 16 == ROW_BYTES && B * LPN == 32 && B >= 1, "group geometry");
};

template <int C, bool FUSED>
__global__ void __launch_bounds__(SPR_WARPS * 32, 1)
spmm_ring_kernel(const SpmmTask *__restrict__ tasks, int64_t n_tasks, const int32_t *__restrict__ pcols,
                 const int32_t *__restrict__ pidx, const int32_t *__restrict__ grow, const float *__restrict__ pval,
                 const float *__restrict__ W, const float *__restrict__ H, float *__restrict__ P_out, float *__restrict__ Y,
                 float *__restrict__ scratch, unsigned long long *work_counter, int *dev_status)
{
    using R = SpmmRingShape<C>;
    constexpr int B = R::B, LPN = R::LPN, F = R::F, NG = SPR_NG;
    constexpr int K = C * 128;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane / LPN;  // this lane's slot of a group
    const int l = lane % LPN;  // position inside the lane set
    unsigned char *ring = smem_raw + (size_t)warp * NG * SPR_SLOT;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw + (size_t)SPR_WARPS * NG * SPR_SLOT) + warp * NG;
    if (lane < NG) mbar_init(&bars[lane], 1);
    mbar_fence_init();
    __syncwarp();

    const char *Hb = reinterpret_cast<const char *>(H);
    const char *W_lane = reinterpret_cast<const char *>(W) + l * 16;
    unsigned s_issue = 0, s_cons = 0;  // next slot to issue into / to read
    unsigned phase = 0;                // bit s: parity of slot s's next completion
    unsigned in_flight = 0;
    bool timed_out = false;

    // the columns of a group's slots (lanes 0..B-1 hold one each), loaded an iteration before they are needed
    auto load_cols = [&](int64_t grp) { return (unsigned)__ldcs(pcols + grp * B + (lane < B ? lane : 0)); };
    auto issue = [&](unsigned cj) {
        uint64_t *bar = &bars[s_issue];
        if (lane == 0)
            asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                             smem_u32(bar)),
                         "r"((unsigned)SPR_SLOT)
                         : "memory");
        if (lane < B) bulk_g2s(ring + s_issue * SPR_SLOT + lane * R::ROW_BYTES, Hb + (size_t)cj * R::ROW_BYTES, R::ROW_BYTES, bar);
        s_issue = s_issue + 1 == NG ? 0 : s_issue + 1;
        ++in_flight;
    };
    // 1 KB .. 4 KB of zeros for a row of S that has no nonzero (the whole warp stores)
    auto zero_row = [&](int64_t r) {
        float4 *o = reinterpret_cast<float4 *>(Y + r * K);
        for (int q = lane; q < K / 4; q += 32) o[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    };

    while (!timed_out) {
        unsigned long long t = 0;
        if (lane == 0) t = atomicAdd(work_counter, 1ull);
        t = __shfl_sync(FULL, t, 0);
        if ((int64_t)t >= n_tasks) break;
        const SpmmTask task = tasks[t];
        const int64_t g0 = task.j0;
        const int n = (int)(task.j1 - task.j0);
        const bool piece = task.slot >= 0;  // a piece of one long row: its sum goes to a scratch slot
        int64_t prev_row = (int64_t)task.row_a - 1;  // last row of the task's range that has been written
        int cur_row = -1;
        float4 y[F], wc[F];
#pragma unroll
        for (int c = 0; c < F; ++c) y[c] = wc[c] = make_float4(0.f, 0.f, 0.f, 0.f);

        for (int i = 0; i < NG - 1 && i < n; ++i) issue(load_cols(g0 + i));
        unsigned cols_next = NG - 1 < n ? load_cols(g0 + NG - 1) : 0u;  // of the group the next iteration issues
        // Metadata two groups ahead, in two steps, so that no load waits for another inside an iteration: the
        // row word and this lane set's nonzero index of group q + 2, the weight (a load that needs the index)
        // of group q + 1.
        auto load_idx = [&](int q, int &rw, int &idx) {
            rw = __ldcs(grow + g0 + q);
            idx = __ldcs(pidx + (g0 + q) * B + g);
        };
        auto load_wgt = [&](int idx) { return idx >= 0 ? (pval ? __ldcs(pval + idx) : 1.f) : 0.f; };
        int rw_1 = 0, idx_1 = -1, rw_2 = 0, idx_2 = -1;  // groups q + 1 and q + 2
        float wgt_1 = 0.f;
        if (n > 0) load_idx(0, rw_1, idx_1);
        if (n > 1) load_idx(1, rw_2, idx_2);
        if (FUSED && n > 0 && lane < R::ROW_BYTES / 128) {
            // the task's first W row, and its second when the first row is one group long
            const char *Wb = reinterpret_cast<const char *>(W);
            asm volatile("prefetch.global.L2 [%0];" ::"l"(Wb + (size_t)(unsigned)(rw_1 & 0x7fffffff) * R::ROW_BYTES + lane * 128));
            if (n > 1 && ((rw_2 ^ rw_1) & 0x7fffffff) != 0)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(Wb + (size_t)(unsigned)(rw_2 & 0x7fffffff) * R::ROW_BYTES + lane * 128));
        }
        if (n > 0) wgt_1 = load_wgt(idx_1);

        for (int q = 0; q < n; ++q) {
            if (q + NG - 1 < n) issue(cols_next);
            if (q + NG < n) cols_next = load_cols(g0 + q + NG);
            const int rw = rw_1, idx = idx_1;
            const float wgt = wgt_1;
            rw_1 = rw_2;
            idx_1 = idx_2;
            if (q + 1 < n) wgt_1 = load_wgt(idx_1);
            if (q + 2 < n) {
                load_idx(q + 2, rw_2, idx_2);
                // the W row of a row of S that starts two groups from now: into L2 ahead of its use (the load
                // at the row's first group would otherwise stall the whole warp for a DRAM round trip)
                if (FUSED && ((rw_2 ^ rw_1) & 0x7fffffff) != 0 && lane < R::ROW_BYTES / 128)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char *>(W) +
                                                                  (size_t)(unsigned)(rw_2 & 0x7fffffff) * R::ROW_BYTES + lane * 128));
            }
            const int row = rw & 0x7fffffff;
            const bool last = piece ? (q == n - 1) : ((unsigned)rw >> 31) != 0;
            if (row != cur_row) {
                // a new row of S begins (uniform over the warp): rows skipped since the last one are empty
                if (!piece)
                    for (int64_t r = prev_row + 1; r < row; ++r) zero_row(r);
                cur_row = row;
                if (FUSED) {
                    const float4 *wrow = reinterpret_cast<const float4 *>(W_lane + (size_t)(unsigned)row * R::ROW_BYTES);
#pragma unroll
                    for (int c = 0; c < F; ++c) wc[c] = __ldg(wrow + c * LPN);
                }
            }
            const unsigned par = (phase >> s_cons) & 1u;
            if (!mbar_try_wait(&bars[s_cons], par) && !mbar_wait_bounded(&bars[s_cons], par)) {
                timed_out = true;
                break;
            }
            const float4 *srow = reinterpret_cast<const float4 *>(ring + s_cons * SPR_SLOT + g * R::ROW_BYTES) + l;
            float4 h[F];
#pragma unroll
            for (int c = 0; c < F; ++c) h[c] = srow[c * LPN];
            phase ^= 1u << s_cons;
            s_cons = s_cons + 1 == NG ? 0 : s_cons + 1;
            --in_flight;
            float p = wgt;
            if (FUSED) {
                float a = 0.f;
#pragma unroll
                for (int c = 0; c < F; ++c) a = dot4(wc[c], h[c], a);
#pragma unroll
                for (int off = LPN / 2; off >= 1; off >>= 1) a += __shfl_xor_sync(FULL, a, off);
                p = a * wgt;  // padding slots carry weight 0
                if (P_out && l == 0 && idx >= 0) __stcs(P_out + idx, p);
            }
#pragma unroll
            for (int c = 0; c < F; ++c) {
                y[c].x = fmaf(p, h[c].x, y[c].x);
                y[c].y = fmaf(p, h[c].y, y[c].y);
                y[c].z = fmaf(p, h[c].z, y[c].z);
                y[c].w = fmaf(p, h[c].w, y[c].w);
            }
            if (last) {
                // the row (or the piece) ends: add the B lane sets' partial rows and let set 0 store
#pragma unroll
                for (int off = LPN; off < 32; off <<= 1) {
#pragma unroll
                    for (int c = 0; c < F; ++c) {
                        y[c].x += __shfl_xor_sync(FULL, y[c].x, off);
                        y[c].y += __shfl_xor_sync(FULL, y[c].y, off);
                        y[c].z += __shfl_xor_sync(FULL, y[c].z, off);
                        y[c].w += __shfl_xor_sync(FULL, y[c].w, off);
                    }
                }
                float *out = piece ? scratch + (int64_t)task.slot * K : Y + (int64_t)row * K;
                if (g == 0) {
                    float4 *o = reinterpret_cast<float4 *>(out) + l;
#pragma unroll
                    for (int c = 0; c < F; ++c) o[c * LPN] = y[c];
                }
#pragma unroll
                for (int c = 0; c < F; ++c) y[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                prev_row = row;
                cur_row = -1;
            }
        }
        if (timed_out) break;
        if (!piece)
            for (int64_t r = prev_row + 1; r < task.row_b; ++r) zero_row(r);
    }
    if (timed_out) {
        if (lane == 0) atomicExch(dev_status, (int)DEV_MBARRIER_TIMEOUT);
        // copies issued but not read may still be landing in this warp's ring
        for (unsigned i = 0; i < in_flight && i < (unsigned)NG; ++i) {
            (void)mbar_wait_bounded(&bars[s_cons], (phase >> s_cons) & 1u);
            s_cons = s_cons + 1 == NG ? 0 : s_cons + 1;
        }
    }
}

template <int C>
cudaError_t launch_t(bool fused, const SpmmTask *tasks, int64_t n_tasks, const int32_t *pcols, const int32_t *pidx,
                     const int32_t *grow, const float *pval, const float *W, const float *H, float *P_out, float *Y,
                     float *scratch, unsigned long long *work_counter, int *dev_status, int sm_count, cudaStream_t stream)
{
    const size_t smem = (size_t)SPR_WARPS * SPR_NG * SPR_SLOT + (size_t)SPR_WARPS * SPR_NG * 8;
    static SmemOptinCache optin_f, optin_s;  // per instantiation and device
    cudaError_t e = fused ? optin_dynamic_smem(spmm_ring_kernel<C, true>, smem, optin_f)
                          : optin_dynamic_smem(spmm_ring_kernel<C, false>, smem, optin_s);
    if (e != cudaSuccess) return e;
    int64_t blocks = (n_tasks + SPR_WARPS - 1) / SPR_WARPS;
    if (blocks > sm_count) blocks = sm_count;
    if (fused)
        spmm_ring_kernel<C, true><<<(unsigned)blocks, SPR_WARPS * 32, smem, stream>>>(tasks, n_tasks, pcols, pidx, grow, pval, W,
                                                                                   H, P_out, Y, scratch, work_counter, dev_status);
    else
        spmm_ring_kernel<C, false><<<(unsigned)blocks, SPR_WARPS * 32, smem, stream>>>(tasks, n_tasks, pcols, pidx, grow, pval, W,
                                                                                    H, P_out, Y, scratch, work_counter, dev_status);
    return cudaGetLastError();
}

}  // namespace

bool spmm_ring_supports(int K) { return K == 256 || K == 512 || K == 1024; }
int spmm_ring_group_slots(int K) { return SPR_SLOT / (K * 4); }

cudaError_t launch_spmm_ring(bool fused, const SpmmTask *tasks, int64_t n_tasks, const int32_t *pcols, const int32_t *pidx,
                             const int32_t *grow, const float *pval, const float *W, const float *H, float *P_out, float *Y,
                             float *scratch, int K, unsigned long long *work_counter, int *dev_status, int sm_count,
                             cudaStream_t stream)
{
    if (n_tasks == 0) return cudaSuccess;
    cudaError_t e = cudaMemsetAsync(work_counter, 0, sizeof(unsigned long long), stream);
    if (e != cudaSuccess) return e;
    switch (K) {
    case 256: return launch_t<2>(fused, tasks, n_tasks, pcols, pidx, grow, pval, W, H, P_out, Y, scratch, work_counter, dev_status, sm_count, stream);
    case 512: return launch_t<4>(fused, tasks, n_tasks, pcols, pidx, grow, pval, W, H, P_out, Y, scratch, work_counter, dev_status, sm_count, stream);
    case 1024: return launch_t<8>(fused, tasks, n_tasks, pcols, pidx, grow, pval, W, H, P_out, Y, scratch, work_counter, dev_status, sm_count, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace sddmm
