// Ring kernel for short rows (K = 32, 64 and 128): the per-warp shared-memory ring of
// sddmm_ring.cu, filled with 16-byte asynchronous copies (cp.async) instead of
// one bulk copy per row.
//
// A row of 128 to 512 bytes is too small for a bulk copy of its own (the fixed
// cost per copy and per mbarrier phase dominates; measured on the scale-22 R-MAT
// matrix at K = 128: 4.2 ms with these copies against 5.2 ms with one bulk copy
// per row, while at K = 256 the bulk copies win), but the reason for the ring is
// the same as for long rows: gathers that land in shared memory hold no registers
// while they are in flight, so a warp can keep a whole 4 KB group (32 or 16 rows
// of H) outstanding while it works on the previous one.  Here every lane issues
// eight 16-byte copies per group (one warp instruction moves 512 bytes: 4 rows at
// K = 32, 2 rows at K = 64, 1 row at K = 128), closes the group with cp.async.commit_group and
// later waits for it with cp.async.wait_group -- a wait on the thread's own
// copies only, so there is nothing that could spin for ever and no mbarrier.
//
// Lane sets as in the long-row kernel: the 32 lanes are B = 4096/(4K) sets of
// LPN = 32/B lanes, one set per nonzero of the group (K = 32: every lane owns a
// nonzero and needs no shuffle at all; K = 64: two lanes per nonzero, one
// shuffle; K = 128: four lanes, two shuffles).  Each lane multiplies 8 float4 of its H row with its share of the W
// row, which stays in registers while consecutive nonzeros of the set lie in the
// same row of S.  Rows are padded in the slot (144 / 288 / 576 bytes) so that the
// 128-bit shared-memory loads of a quarter-warp fall into different banks.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace sddmm {

using namespace dev;

namespace {

constexpr int SR_WARPS = 24;
constexpr int SR_NG = 2;  // ring slots (groups) per warp

template <int RB>  // row bytes: 128 (K = 32), 256 (K = 64) or 512 (K = 128)
struct SmallShape {
    static constexpr int B = 4096 / RB;        // nonzeros per group: 32 / 16
    static constexpr int LPN = 32 / B;         // lanes per nonzero: 1 / 2
    static constexpr int F = RB / 16 / LPN;    // float4 per lane per row: 8
    static constexpr int PPR = RB / 16;        // 16-byte pieces per row: 8 / 16
    static constexpr int NCOPY = B * PPR / 32; // copy instructions per group: 8
    static constexpr int ROW_STRIDE = RB + (LPN < 8 ? 16 * LPN : 0);  // 144 / 288: conflict-free 128-bit loads
    static constexpr int SLOT_BYTES = (B * ROW_STRIDE + 127) / 128 * 128;
    static constexpr int K4 = RB / 16;
    static_assert(F == 8 && NCOPY == 8, "geometry");
};

__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16_hint(void *dst_smem, const void *src, uint64_t policy)
{
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src),
                 "l"(policy)
                 : "memory");
}

template <int RB, bool HAS_PERM, bool HAS_SVAL, bool HAS_HINT>
__global__ void __launch_bounds__(SR_WARPS * 32, 1)
sddmm_ring_small_kernel(const int32_t *__restrict__ rows, const int32_t *__restrict__ cols,
                        const int32_t *__restrict__ perm, const float *__restrict__ sval,
                        const float *__restrict__ W, const float *__restrict__ H, float *__restrict__ P,
                        int64_t nnz, int block_groups, unsigned long long *work_counter)
{
    using R = SmallShape<RB>;
    constexpr int B = R::B, LPN = R::LPN, F = R::F, NG = SR_NG;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane / LPN;  // which nonzero of a group this lane works on
    const int l = lane % LPN;  // position inside the lane set
    unsigned char *ring = smem_raw + (size_t)warp * NG * R::SLOT_BYTES;

    const int64_t n_groups = nnz / B;
    const int64_t n_blocks = (n_groups + block_groups - 1) / block_groups;
    const char *Hb = reinterpret_cast<const char *>(H);
    const char *W_lane = reinterpret_cast<const char *>(W) + l * 16;

    float4 wc[F];     // this lane's share of the W row of its lane set's current row of S
    int wc_row = -1;
    uint64_t pol_keep = 0, pol_drop = 0;
    if (HAS_HINT) {
        pol_keep = l2_policy_evict_last();
        pol_drop = l2_policy_evict_first();
    }
    unsigned s_issue = 0, s_cons = 0;

    // lane j < B holds the column of nonzero j of the group in c_mine
    auto issue = [&](int c_mine) {
        unsigned char *slot = ring + s_issue * R::SLOT_BYTES;
#pragma unroll
        for (int i = 0; i < R::NCOPY; ++i) {
            const int piece = i * 32 + lane;  // 16-byte piece of the group handled by this lane in copy i
            const int r = piece / R::PPR, part = piece % R::PPR;
            const unsigned cj = (unsigned)__shfl_sync(FULL, c_mine, r);
            void *dst = slot + r * R::ROW_STRIDE + part * 16;
            if (HAS_HINT)
                cp_async16_hint(dst, Hb + (size_t)(cj & 0x7fffffffu) * RB + part * 16, (cj >> 31) ? pol_keep : pol_drop);
            else
                cp_async16(dst, Hb + (size_t)cj * RB + part * 16);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        s_issue ^= 1u;
    };
    auto store = [&](int64_t j, float v) {
        if (HAS_PERM) {
            const int64_t dst = __ldcs(perm + j);
            if (HAS_SVAL) v *= __ldg(sval + dst);
            P[dst] = v;
        } else {
            if (HAS_SVAL) v *= __ldcs(sval + j);
            __stcs(P + j, v);
        }
    };
    auto load_w = [&](int r) {
        const float4 *wrow = reinterpret_cast<const float4 *>(W_lane + (size_t)(unsigned)r * RB);
#pragma unroll
        for (int c = 0; c < F; ++c) wc[c] = __ldg(wrow + c * LPN);
        wc_row = r;
    };

    while (true) {
        unsigned long long blk = 0;
        if (lane == 0) blk = atomicAdd(work_counter, 1ull);
        blk = __shfl_sync(FULL, blk, 0);
        if ((int64_t)blk > n_blocks) break;
        if ((int64_t)blk == n_blocks) {
            // the block after the last one is the partial group at the very end
            const int tail = (int)(nnz - n_groups * B);
            if (tail > 0) {
                const int64_t off = n_groups * B;
                int r = 0, c = 0;
                if (lane < tail) {
                    r = __ldcs(rows + off + lane);
                    c = __ldcs(cols + off + lane);
                    if (HAS_HINT) c &= 0x7fffffff;
                }
                // general predicated step: 8 (K = 32) or 16 (K = 64) lanes per nonzero, up to 32 / 16 nonzeros
                const float res = warp_step<(R::K4 < 32 ? R::K4 : 32), (R::K4 < 32 ? 1 : R::K4 / 32), (B < 8 ? B : 8), false>(
                    W, H, r, c, tail, R::K4, lane);
                if (lane < tail) store(off + lane, res);
            }
            continue;
        }
        const int64_t g0 = (int64_t)blk * block_groups;
        const int n = (int)((n_groups - g0) < block_groups ? (n_groups - g0) : block_groups);
        const int32_t *brow = rows + g0 * B + g;              // row of this lane set's nonzero in group q: brow[q * B]
        const int32_t *bcol = cols + g0 * B + (lane & (B - 1));  // column of nonzero `lane` of group q: bcol[q * B]
        auto clampq = [&](int q) { return q < n ? q : n - 1; };  // past the end the last group is re-read

        // prologue: one group in flight, W of the first group, indices one step ahead
        issue(__ldcs(bcol));
        int c_next = __ldcs(bcol + clampq(1) * B);  // columns of group q + 1
        {
            const int r0 = __ldcs(brow);
            if (r0 != wc_row) load_w(r0);
        }
        int r_next = __ldcs(brow + clampq(1) * B);  // row of group q + 1

        for (int q = 0; q < n; ++q) {
            const bool more = q + 1 < n;
            if (more) issue(c_next);  // group q + 1 goes into the slot freed by group q - 1
            c_next = __ldcs(bcol + clampq(q + 2) * B);
            const int r_fut = __ldcs(brow + clampq(q + 2) * B);
            // wait for this thread's copies of group q, then for everybody else's
            if (more) asm volatile("cp.async.wait_group 1;" ::: "memory");
            else asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncwarp();
            const float4 *srow = reinterpret_cast<const float4 *>(ring + s_cons * R::SLOT_BYTES + g * R::ROW_STRIDE) + l;
            s_cons ^= 1u;
            float acc = 0.f;
#pragma unroll
            for (int c = 0; c < F; ++c) acc = dot4(wc[c], srow[c * LPN], acc);
            __syncwarp();  // every lane has read the slot before the next issue overwrites it
            // W of the next group, fetched while this group is reduced and stored
            if (r_next != wc_row) load_w(r_next);
            r_next = r_fut;
#pragma unroll
            for (int off = LPN / 2; off >= 1; off >>= 1) acc += __shfl_xor_sync(FULL, acc, off);
            if (l == 0) store((g0 + q) * B + g, acc);
        }
    }
}

template <int RB, bool HAS_PERM, bool HAS_SVAL, bool HAS_HINT>
cudaError_t launch_small_tt(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                            const float *W, const float *H, float *P, int64_t nnz, int sm_count,
                            unsigned long long *work_counter, cudaStream_t stream)
{
    using R = SmallShape<RB>;
    const size_t smem = (size_t)SR_WARPS * SR_NG * R::SLOT_BYTES;
    auto kern = sddmm_ring_small_kernel<RB, HAS_PERM, HAS_SVAL, HAS_HINT>;
    static SmemOptinCache optin;  // one opt-in per instantiation and device
    cudaError_t e = optin_dynamic_smem(kern, smem, optin);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(work_counter, 0, sizeof(unsigned long long), stream);
    if (e != cudaSuccess) return e;
    const int64_t n_groups = nnz / R::B;
    int64_t bg = n_groups / ((int64_t)sm_count * SR_WARPS * 4);
    if (bg < 4) bg = 4;
    if (bg > 128) bg = 128;
    kern<<<(unsigned)sm_count, SR_WARPS * 32, smem, stream>>>(rows, cols, perm, sval, W, H, P, nnz, (int)bg, work_counter);
    return cudaGetLastError();
}

template <int RB>
cudaError_t launch_small_t(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                           const float *W, const float *H, float *P, int64_t nnz, bool cols_hinted, int sm_count,
                           unsigned long long *work_counter, cudaStream_t stream)
{
#define SR_GO(PERM, SVAL, HINT) \
    return launch_small_tt<RB, PERM, SVAL, HINT>(rows, cols, perm, sval, W, H, P, nnz, sm_count, work_counter, stream)
#define SR_GO2(PERM, SVAL)                        \
    do {                                          \
        if (cols_hinted) SR_GO(PERM, SVAL, true); \
        SR_GO(PERM, SVAL, false);                 \
    } while (0)
    if (perm) {
        if (sval) SR_GO2(true, true);
        SR_GO2(true, false);
    }
    if (sval) SR_GO2(false, true);
    SR_GO2(false, false);
#undef SR_GO2
#undef SR_GO
}

}  // namespace

cudaError_t launch_ring_small(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                              const float *W, const float *H, float *P, int64_t nnz, int K, bool cols_hinted,
                              int sm_count, unsigned long long *work_counter, cudaStream_t stream)
{
    if (nnz == 0) return cudaSuccess;
    if (K == 32)
        return launch_small_t<128>(rows, cols, perm, sval, W, H, P, nnz, cols_hinted, sm_count, work_counter, stream);
    if (K == 64)
        return launch_small_t<256>(rows, cols, perm, sval, W, H, P, nnz, cols_hinted, sm_count, work_counter, stream);
    if (K == 128)
        return launch_small_t<512>(rows, cols, perm, sval, W, H, P, nnz, cols_hinted, sm_count, work_counter, stream);
    return cudaErrorInvalidValue;
}

}  // namespace sddmm
