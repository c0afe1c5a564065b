// Ring kernel: H rows gathered by bulk asynchronous copies (TMA) into per-warp
// shared-memory rings.
//
// Why it exists.  On a power-law matrix most chunks of nonzeros contain at least
// one H row that misses L2, and a warp consumes its chunks in order, so its
// throughput is (bytes it keeps in flight) / (DRAM latency) whatever the L2 hit
// rate.  Gathering into registers caps the bytes in flight at a fraction of the
// register file.  Here every H row is one cp.async.bulk of K*4 bytes into a
// shared-memory slot, completion counted on an mbarrier, so an SM keeps
// NWARPS * (NG-1) * 4 KB (~128 KB) of gathers in flight without holding a single
// register for them, and the address arithmetic per 16 bytes disappears.
//
// Shape.  One persistent CTA per SM, NWARPS independent warps, no CTA-wide
// synchronisation after set-up.  A warp owns NG ring slots of one group each; a
// group is B = 4096 / (K*4) consecutive nonzeros (4 KB of H rows).  Work is
// handed out in blocks of BLOCK_GROUPS groups through a global counter
// (atomicAdd), in nonzero order, so concurrently running warps work on
// neighbouring rows of S.  Per group: lane t < B issues the copy of H[col_t],
// lane 0 arms the slot's mbarrier with the byte count; NG-1 groups later the
// warp waits on that mbarrier (bounded), reads the rows back with 128-bit
// shared-memory loads and multiplies with W.
//
// W.  Consecutive groups of a warp mostly lie in one row of S, whose W row lives
// in registers and is reloaded only when the row changes; groups that straddle
// rows load one W row per nonzero.  Both are fetched from global memory (L1/L2)
// one group ahead, right after the previous group's FMAs.
//
// Supported: K = 128 * C with C in {1, 2, 4, 8} (K = 128 ... 1024).
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace sddmm {

using namespace dev;

namespace {

#ifndef SDDMM_RING_WARPS
#define SDDMM_RING_WARPS 24
#endif
#ifndef SDDMM_RING_NG
#define SDDMM_RING_NG 2
#endif
#ifndef SDDMM_RING_GROUP_BYTES
#define SDDMM_RING_GROUP_BYTES 4096
#endif
constexpr int RING_WARPS = SDDMM_RING_WARPS;
constexpr int RING_NG = SDDMM_RING_NG;  // ring slots (groups) per warp
constexpr int RING_GROUP_BYTES = SDDMM_RING_GROUP_BYTES;
constexpr int RING_BLOCK_GROUPS = 128;  // groups per dynamically scheduled block

template <int C>
struct RingShape {
    static constexpr int ROW_BYTES = C * 512;
    static constexpr int SLOT_BYTES = RING_GROUP_BYTES > ROW_BYTES ? RING_GROUP_BYTES : ROW_BYTES;
    static constexpr int B = SLOT_BYTES / ROW_BYTES;  // nonzeros per group
    static_assert(B >= 1 && B <= 32, "group size");
};

template <int C, bool HAS_PERM, bool HAS_SVAL, bool HAS_HINT>
__global__ void __launch_bounds__(RING_WARPS * 32, 1)
sddmm_ring_kernel(const int32_t *__restrict__ rows, const int32_t *__restrict__ cols,
                  const int32_t *__restrict__ perm, const float *__restrict__ sval,
                  const float *__restrict__ W, const float *__restrict__ H, float *__restrict__ P,
                  int64_t nnz, unsigned long long *work_counter, int *dev_status)
{
    using R = RingShape<C>;
    constexpr int B = R::B;
    constexpr int NG = RING_NG;
    constexpr int K4 = 32 * C;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    // per warp: NG slots of one group each, then (after all rings) NG mbarriers per warp
    unsigned char *ring = smem_raw + (size_t)warp * NG * R::SLOT_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw + (size_t)RING_WARPS * NG * R::SLOT_BYTES) + warp * NG;
    if (lane < NG) mbar_init(&bars[lane], 1);
    mbar_fence_init();
    __syncwarp();

    const int64_t n_groups = nnz / B;  // full groups; the remainder is handled at the end
    const int64_t n_blocks = (n_groups + RING_BLOCK_GROUPS - 1) / RING_BLOCK_GROUPS;
    const char *Hb = reinterpret_cast<const char *>(H);
    const char *W_lane = reinterpret_cast<const char *>(W) + lane * 16;
    const int il = lane & (B - 1);  // lanes >= B mirror a valid nonzero of the group

    // Ring bookkeeping.  Issue and consume each walk the NG slots round-robin; a
    // slot's mbarrier phase flips every time the slot is reused, so the parity to
    // wait for is the number of completed walks of the consumer, modulo 2.
    unsigned s_issue = 0, s_cons = 0;  // next slot to issue into / to consume
    unsigned cons_parity = 0;          // parity of the consumer's current walk
    unsigned in_flight = 0;            // groups issued and not yet consumed
    bool timed_out = false;
    float4 wc[C];  // W row of a single-row group
    int wc_row = -1;
    // HAS_HINT: bit 31 of a column index marks a hub column (chosen by the plan so
    // that all hub rows of H fit a share of L2); its copy asks L2 to keep the row,
    // every other copy asks L2 to drop the row first.
    uint64_t pol_keep = 0, pol_drop = 0;
    if (HAS_HINT) {
        pol_keep = l2_policy_evict_last();
        pol_drop = l2_policy_evict_first();
    }

    // One lane arms the slot's mbarrier with the byte count and issues the B row
    // copies (column indices arrive by shuffle, so the issuing code is uniform).
    auto issue = [&](int c_mine) {
        unsigned char *slot = ring + s_issue * R::SLOT_BYTES;
        uint64_t *bar = &bars[s_issue];
        unsigned cj[B];
#pragma unroll
        for (int j = 0; j < B; ++j) cj[j] = (unsigned)__shfl_sync(FULL, c_mine, j);
        if (lane == 0) {
            asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                             smem_u32(bar)),
                         "r"((unsigned)(B * R::ROW_BYTES))
                         : "memory");
#pragma unroll
            for (int j = 0; j < B; ++j) {
                if (HAS_HINT) {
                    const unsigned col = cj[j] & 0x7fffffffu;
                    bulk_g2s_hint(slot + j * R::ROW_BYTES, Hb + (size_t)col * R::ROW_BYTES, R::ROW_BYTES, bar,
                                  (cj[j] >> 31) ? pol_keep : pol_drop);
                } else {
                    bulk_g2s(slot + j * R::ROW_BYTES, Hb + (size_t)cj[j] * R::ROW_BYTES, R::ROW_BYTES, bar);
                }
            }
        }
        s_issue = (s_issue + 1 == NG) ? 0 : s_issue + 1;
        ++in_flight;
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

    while (!timed_out) {
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
                const float res = warp_step<32, C, B, false>(W, H, r, c, tail, K4, lane);
                if (lane < tail) store(off + lane, res);
            }
            continue;
        }
        const int64_t g0 = (int64_t)blk * RING_BLOCK_GROUPS;
        const int n = (int)((n_groups - g0) < RING_BLOCK_GROUPS ? (n_groups - g0) : RING_BLOCK_GROUPS);
        const int32_t *brow = rows + g0 * B + il;
        const int32_t *bcol = cols + g0 * B + il;

        // (row, col) of nonzero `il` of group q of this block; past the end the last group is re-read
        auto load_idx = [&](int q, int &r, int &c) {
            const int qq = q < n ? q : n - 1;
            r = __ldcs(brow + qq * B);
            c = __ldcs(bcol + qq * B);
        };

        // index registers of the groups ahead: r_q[i], c_q[i] belong to group (current + i)
        int r_q[NG], c_q[NG];
#pragma unroll
        for (int i = 0; i < NG; ++i) load_idx(i, r_q[i], c_q[i]);
        // prologue: NG-1 groups in flight
#pragma unroll
        for (int i = 0; i < NG - 1; ++i)
            if (i < n) issue(c_q[i]);

        // W of the next group: a group whose nonzeros share one row keeps that row
        // of W in registers (fetched here, one group ahead, only when the row
        // changes); a group that straddles rows reads W per nonzero when consumed.
        auto prefetch_w = [&](int r_mine) {
            const int r0 = __shfl_sync(FULL, r_mine, 0);
            const bool single = __all_sync(FULL, r_mine == r0);
            if (single && r0 != wc_row) {
                const float4 *wrow = reinterpret_cast<const float4 *>(W_lane + (size_t)(unsigned)r0 * R::ROW_BYTES);
#pragma unroll
                for (int c = 0; c < C; ++c) wc[c] = __ldg(wrow + c * 32);
                wc_row = r0;
            }
            return single;
        };
        bool single = prefetch_w(r_q[0]);

        for (int q = 0; q < n; ++q) {
            // keep NG-1 groups in flight: group q + NG - 1 goes into the slot freed by group q - 1
            if (q + NG - 1 < n) issue(c_q[NG - 1]);
            // wait for group q
            if (!mbar_try_wait(&bars[s_cons], cons_parity) && !mbar_wait_bounded(&bars[s_cons], cons_parity)) {
                timed_out = true;
                break;
            }
            const float4 *slot = reinterpret_cast<const float4 *>(ring + s_cons * R::SLOT_BYTES) + lane;
            --in_flight;
            if (++s_cons == NG) {
                s_cons = 0;
                cons_parity ^= 1u;
            }
            float acc[B];
            if (single) {
#pragma unroll
                for (int j = 0; j < B; ++j) {
                    acc[j] = 0.f;
#pragma unroll
                    for (int c = 0; c < C; ++c) acc[j] = dot4(wc[c], slot[j * K4 + c * 32], acc[j]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < B; ++j) {
                    acc[j] = 0.f;
                    const unsigned rj = (unsigned)__shfl_sync(FULL, r_q[0], j);
                    const float4 *wrow = reinterpret_cast<const float4 *>(W_lane + (size_t)rj * R::ROW_BYTES);
#pragma unroll
                    for (int c = 0; c < C; ++c) acc[j] = dot4(__ldg(wrow + c * 32), slot[j * K4 + c * 32], acc[j]);
                }
            }
            // shift the index queue, fetch the indices of group q + NG, prefetch W of group q + 1
#pragma unroll
            for (int i = 0; i < NG - 1; ++i) {
                r_q[i] = r_q[i + 1];
                c_q[i] = c_q[i + 1];
            }
            load_idx(q + NG, r_q[NG - 1], c_q[NG - 1]);
            bool single_next = single;
            if (q + 1 < n) single_next = prefetch_w(r_q[0]);
            // reduce, route, store
            reduce_transposed<32, B>(acc, lane);
            const float res = __shfl_sync(FULL, acc[0], (lane & (B - 1)) * (32 / B));
            if (lane < B) store((g0 + q) * B + lane, res);
            single = single_next;
        }
    }
    if (timed_out) {
        if (lane == 0) atomicExch(dev_status, (int)DEV_MBARRIER_TIMEOUT);
        // copies issued but not consumed may still be landing in this warp's ring:
        // give each a bounded chance before the CTA's shared memory is released
        while (in_flight > 0) {
            (void)mbar_wait_bounded(&bars[s_cons], cons_parity);
            --in_flight;
            if (++s_cons == NG) {
                s_cons = 0;
                cons_parity ^= 1u;
            }
        }
    }
}

template <int C, bool HAS_PERM, bool HAS_SVAL, bool HAS_HINT>
cudaError_t launch_ring_tt(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                           const float *W, const float *H, float *P, int64_t nnz, int sm_count,
                           unsigned long long *work_counter, int *dev_status, cudaStream_t stream)
{
    const size_t smem = (size_t)RING_WARPS * RING_NG * RingShape<C>::SLOT_BYTES + (size_t)RING_WARPS * RING_NG * 8;
    auto kern = sddmm_ring_kernel<C, HAS_PERM, HAS_SVAL, HAS_HINT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(work_counter, 0, sizeof(unsigned long long), stream);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)sm_count, RING_WARPS * 32, smem, stream>>>(rows, cols, perm, sval, W, H, P, nnz, work_counter,
                                                                dev_status);
    return cudaGetLastError();
}

template <int C>
cudaError_t launch_ring_t(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                          const float *W, const float *H, float *P, int64_t nnz, bool cols_hinted, int sm_count,
                          unsigned long long *work_counter, int *dev_status, cudaStream_t stream)
{
#define RING_GO(PERM, SVAL, HINT)                                                                                   \
    return launch_ring_tt<C, PERM, SVAL, HINT>(rows, cols, perm, sval, W, H, P, nnz, sm_count, work_counter, dev_status, \
                                               stream)
#define RING_GO2(PERM, SVAL)              \
    do {                                  \
        if (cols_hinted) RING_GO(PERM, SVAL, true); \
        RING_GO(PERM, SVAL, false);       \
    } while (0)
    if (perm) {
        if (sval) RING_GO2(true, true);
        RING_GO2(true, false);
    }
    if (sval) RING_GO2(false, true);
    RING_GO2(false, false);
#undef RING_GO2
#undef RING_GO
}

}  // namespace

bool ring_supports(int K) { return K == 128 || K == 256 || K == 512 || K == 1024; }

cudaError_t launch_ring(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                        const float *W, const float *H, float *P, int64_t nnz, int K, bool cols_hinted, int sm_count,
                        unsigned long long *work_counter, int *dev_status, cudaStream_t stream)
{
    if (nnz == 0) return cudaSuccess;
    switch (K) {
    case 128: return launch_ring_t<1>(rows, cols, perm, sval, W, H, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    case 256: return launch_ring_t<2>(rows, cols, perm, sval, W, H, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    case 512: return launch_ring_t<4>(rows, cols, perm, sval, W, H, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    case 1024: return launch_ring_t<8>(rows, cols, perm, sval, W, H, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace sddmm
