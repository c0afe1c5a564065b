// Ring kernel: H rows gathered by bulk asynchronous copies (TMA) into per-warp
// shared-memory rings.
//
// Why it exists.  On a power-law matrix most chunks of nonzeros contain at least
// one H row that misses L2, and a warp consumes its chunks in order, so its
// throughput is (bytes it keeps in flight) / (DRAM latency) whatever the L2 hit
// rate.  Gathering into registers caps the bytes in flight at a fraction of the
// register file.  Here every H row is one cp.async.bulk of K*4 bytes into a
// shared-memory slot, completion counted on an mbarrier, so an SM keeps
// NWARPS * (NG-1) * 4 KB (~100 KB) of gathers in flight without holding a single
// register for them, and the address arithmetic per 16 bytes disappears.
//
// Shape.  One persistent CTA per SM, NWARPS independent warps, no CTA-wide
// synchronisation after set-up.  A warp owns NG ring slots of one group each; a
// group is B = 4096 / (K*4) consecutive nonzeros (4 KB of H rows).  Work is
// handed out in blocks of groups through a global counter (atomicAdd), in
// nonzero order, so concurrently running warps work on neighbouring rows of S.
// Per group: one lane arms the slot's mbarrier with the byte count and issues
// the B row copies; NG-1 groups later the warp waits on that mbarrier (bounded).
// The 32 lanes are B sets of 32/B lanes, one set per nonzero: every lane reads 8
// float4 of its nonzero's H row from shared memory, multiplies with its share of
// the W row, and the sets finish their dot products together with log2(32/B)
// __shfl_xor_sync steps.
//
// W.  Consecutive nonzeros handled by a lane set mostly lie in one row of S, so
// a lane keeps its share of that W row in registers and reloads it (from global
// memory, L1/L2) only when the row changes -- one group ahead, right after the
// previous group's FMAs.
//
// Used for K = 256, 512 and 1024 (C = 2, 4, 8); K = 32, 64 and 128 are served by
// the cp.async ring of sddmm_ring_small.cu through the same launcher.
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
constexpr int RING_WARPS = SDDMM_RING_WARPS;
constexpr int RING_NG = SDDMM_RING_NG;  // ring slots (groups) per warp
constexpr int RING_GROUP_BYTES = 4096;  // H bytes of one group

// Geometry for K = 128 * C floats per row.  A group is B rows of H (4 KB); the
// 32 lanes split into B sets of LPN lanes, one set per nonzero, and every lane
// handles F = 8 float4 of its nonzero's row, interleaved with the other lanes of
// its set (lane l takes float4 c*LPN + l), so that a 128-bit shared-memory load
// of a set covers LPN*16 consecutive bytes and the dot product is finished with
// log2(LPN) shuffles -- all B nonzeros of the group reduce at the same time.
template <int C>
struct RingShape {
    static constexpr int ROW_BYTES = C * 512;
    static constexpr int B = RING_GROUP_BYTES > ROW_BYTES ? RING_GROUP_BYTES / ROW_BYTES : 1;
    static constexpr int LPN = 32 / B;                   // lanes per nonzero
    static constexpr int F = ROW_BYTES / 16 / LPN;       // float4 per lane per row
    // with 4 lanes per row two rows share a quarter-warp: pad the row stride so
    // that their 64-byte pieces fall into different banks
    static constexpr int ROW_STRIDE = ROW_BYTES + (LPN == 4 ? 64 : 0);
    static constexpr int SLOT_BYTES = (B * ROW_STRIDE + 127) / 128 * 128;
    // Who issues the B row copies of a group: with four or more rows per group
    // lanes 0..B-1 issue one copy each in the same instruction; with one or two
    // rows lane 0 issues them one after the other (measured: K = 256 on a matrix
    // whose H fits L2 6.5 % faster with parallel issue, K = 512 on a matrix whose
    // H does not 4 % slower).
    static constexpr bool PAR_ISSUE = B >= 4;
    static_assert(B >= 1 && B <= 8 && LPN * B == 32, "group geometry");
};

// A 16-byte piece of a row: four fp32 values, or eight bfloat16 values (operand storage
// in bfloat16, products and sums in fp32: a bfloat16 is the upper half of an fp32, so
// widening is a shift or a mask).
template <bool BF16>
struct Piece {
    using T = float4;
    static __device__ __forceinline__ float dot(T a, T b, float acc) { return dot4(a, b, acc); }
};
template <>
struct Piece<true> {
    using T = uint4;
    static __device__ __forceinline__ float dot2(unsigned a, unsigned b, float acc)
    {
        acc = fmaf(__uint_as_float(a << 16), __uint_as_float(b << 16), acc);
        return fmaf(__uint_as_float(a & 0xffff0000u), __uint_as_float(b & 0xffff0000u), acc);
    }
    static __device__ __forceinline__ float dot(T a, T b, float acc)
    {
        acc = dot2(a.x, b.x, acc);
        acc = dot2(a.y, b.y, acc);
        acc = dot2(a.z, b.z, acc);
        return dot2(a.w, b.w, acc);
    }
};

// The column indices a lane needs to issue a group: its own one (parallel issue),
// or all B <= 2 of them (lane 0 issues; every lane loads the same vector).
template <int B, bool PAR>
struct GroupCols {
    int v[PAR ? 1 : B];
};
template <int B, bool PAR>
__device__ __forceinline__ GroupCols<B, PAR> load_group_cols(const int32_t *group, int lane)
{
    GroupCols<B, PAR> r;
    if constexpr (PAR) {
        r.v[0] = __ldcs(group + (lane & (B - 1)));
    } else if constexpr (B == 2) {
        const int2 t = __ldcs(reinterpret_cast<const int2 *>(group));
        r.v[0] = t.x;
        r.v[1] = t.y;
    } else {
        static_assert(B == 1, "serial issue is for one or two rows per group");
        r.v[0] = __ldcs(group);
    }
    return r;
}

// C: row bytes / 512.  BF16: W and H hold bfloat16 (K = 256 C), else fp32 (K = 128 C).
template <int C, bool HAS_PERM, bool HAS_SVAL, bool HAS_HINT, bool BF16 = false>
__global__ void __launch_bounds__(RING_WARPS * 32, 1)
sddmm_ring_kernel(const int32_t *__restrict__ rows, const int32_t *__restrict__ cols,
                  const int32_t *__restrict__ perm, const float *__restrict__ sval,
                  const void *__restrict__ W, const void *__restrict__ H, float *__restrict__ P,
                  int64_t nnz, int block_groups, unsigned long long *work_counter, int *dev_status)
{
    using R = RingShape<C>;
    using PT = typename Piece<BF16>::T;
    constexpr int B = R::B, LPN = R::LPN, F = R::F, NG = RING_NG;
    constexpr bool PAR = R::PAR_ISSUE;
    constexpr int K4 = 32 * C;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane / LPN;  // which nonzero of a group this lane works on
    const int l = lane % LPN;  // position inside the lane set
    // per warp: NG slots of one group each, then (after all rings) NG mbarriers per warp
    unsigned char *ring = smem_raw + (size_t)warp * NG * R::SLOT_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw + (size_t)RING_WARPS * NG * R::SLOT_BYTES) + warp * NG;
    if (lane < NG) mbar_init(&bars[lane], 1);
    mbar_fence_init();
    __syncwarp();

    const int64_t n_groups = nnz / B;  // full groups; the remainder is handled at the end
    const int64_t n_blocks = (n_groups + block_groups - 1) / block_groups;
    const char *Hb = reinterpret_cast<const char *>(H);
    const char *W_lane = reinterpret_cast<const char *>(W) + l * 16;

    // Ring bookkeeping.  Issue and consume each walk the NG slots round-robin; a
    // slot's mbarrier phase flips every time the slot is reused, so the parity to
    // wait for is the number of completed walks of the consumer, modulo 2.
    unsigned s_issue = 0, s_cons = 0;  // next slot to issue into / to consume
    unsigned cons_parity = 0;          // parity of the consumer's current walk
    unsigned in_flight = 0;            // groups issued and not yet consumed
    bool timed_out = false;
    PT wc[F];         // this lane's share of the W row of its lane set's current row of S
    int wc_row = -1;  // that row (-1: none)
    // HAS_HINT: bit 31 of a column index marks a hub column (chosen by the plan so
    // that all hub rows of H fit a share of L2); its copy asks L2 to keep the row,
    // every other copy asks L2 to drop the row first.
    uint64_t pol_keep = 0, pol_drop = 0;
    if (HAS_HINT) {
        pol_keep = l2_policy_evict_last();
        pol_drop = l2_policy_evict_first();
    }

    // Lane 0 arms the slot's mbarrier with the byte count of the whole group, then
    // the B row copies are issued (by lanes 0..B-1 together, or by lane 0 alone).
    // A copy that lands before the arming only drives the barrier's byte count
    // negative for a moment: the phase cannot complete before lane 0's arrival.
    auto copy_row = [&](unsigned char *dst, unsigned cj, uint64_t *bar) {
        if (HAS_HINT) {
            bulk_g2s_hint(dst, Hb + (size_t)(cj & 0x7fffffffu) * R::ROW_BYTES, R::ROW_BYTES, bar,
                          (cj >> 31) ? pol_keep : pol_drop);
        } else {
            bulk_g2s(dst, Hb + (size_t)cj * R::ROW_BYTES, R::ROW_BYTES, bar);
        }
    };
    auto issue = [&](const GroupCols<B, PAR> &gc) {
        unsigned char *slot = ring + s_issue * R::SLOT_BYTES;
        uint64_t *bar = &bars[s_issue];
        if (lane == 0)
            asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                             smem_u32(bar)),
                         "r"((unsigned)(B * R::ROW_BYTES))
                         : "memory");
        if constexpr (PAR) {
            if (lane < B) copy_row(slot + lane * R::ROW_STRIDE, (unsigned)gc.v[0], bar);
        } else {
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < B; ++j) copy_row(slot + j * R::ROW_STRIDE, (unsigned)gc.v[j], bar);
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
    auto load_w = [&](int r) {
        const PT *wrow = reinterpret_cast<const PT *>(W_lane + (size_t)(unsigned)r * R::ROW_BYTES);
#pragma unroll
        for (int c = 0; c < F; ++c) wc[c] = __ldg(wrow + c * LPN);
        wc_row = r;
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
                float res;
                if constexpr (BF16) {
                    // every tail nonzero by the whole warp: lane l takes the pieces l, l + 32, ... of both rows
                    res = 0.f;
                    for (int j = 0; j < tail; ++j) {
                        const int rj = __shfl_sync(FULL, r, j), cj = __shfl_sync(FULL, c, j);
                        const uint4 *w4 = reinterpret_cast<const uint4 *>(reinterpret_cast<const char *>(W) + (size_t)(unsigned)rj * R::ROW_BYTES);
                        const uint4 *h4 = reinterpret_cast<const uint4 *>(Hb + (size_t)(unsigned)cj * R::ROW_BYTES);
                        float a = 0.f;
                        for (int q = lane; q < R::ROW_BYTES / 16; q += 32) a = Piece<true>::dot(__ldg(w4 + q), __ldg(h4 + q), a);
#pragma unroll
                        for (int off2 = 16; off2 >= 1; off2 >>= 1) a += __shfl_xor_sync(FULL, a, off2);
                        if (lane == j) res = a;
                    }
                } else {
                    res = warp_step<32, C, B, false>(reinterpret_cast<const float *>(W), reinterpret_cast<const float *>(H), r, c,
                                                     tail, K4, lane);
                }
                if (lane < tail) store(off + lane, res);
            }
            continue;
        }
        const int64_t g0 = (int64_t)blk * block_groups;
        const int n = (int)((n_groups - g0) < block_groups ? (n_groups - g0) : block_groups);
        const int32_t *brow = rows + g0 * B + g;  // row of this lane set's nonzero in group q: brow[q * B]
        const int32_t *bcol = cols + g0 * B;      // the B columns of group q start at bcol + q * B
        auto clampq = [&](int q) { return q < n ? q : n - 1; };  // past the end the last group is re-read

        // prologue: NG-1 groups in flight, W of the first group, indices one step ahead
#pragma unroll
        for (int i = 0; i < NG - 1; ++i)
            if (i < n) issue(load_group_cols<B, PAR>(bcol + i * B, lane));
        auto cv = load_group_cols<B, PAR>(bcol + clampq(NG - 1) * B, lane);  // columns of group q + NG - 1
        {
            const int r0 = __ldcs(brow);
            if (r0 != wc_row) load_w(r0);
        }
        int r_next = __ldcs(brow + clampq(1) * B);  // row of group q + 1

        for (int q = 0; q < n; ++q) {
            // keep NG-1 groups in flight: group q + NG - 1 goes into the slot freed by group q - 1
            if (q + NG - 1 < n) issue(cv);
            cv = load_group_cols<B, PAR>(bcol + clampq(q + NG) * B, lane);
            const int r_fut = __ldcs(brow + clampq(q + 2) * B);
            // wait for group q
            if (!mbar_try_wait(&bars[s_cons], cons_parity) && !mbar_wait_bounded(&bars[s_cons], cons_parity)) {
                timed_out = true;
                break;
            }
            const PT *srow = reinterpret_cast<const PT *>(ring + s_cons * R::SLOT_BYTES + g * R::ROW_STRIDE) + l;
            --in_flight;
            if (++s_cons == NG) {
                s_cons = 0;
                cons_parity ^= 1u;
            }
            float acc = 0.f;
#pragma unroll
            for (int c = 0; c < F; ++c) acc = Piece<BF16>::dot(wc[c], srow[c * LPN], acc);
            // W of the next group, fetched while this group is reduced and stored
            if (r_next != wc_row) load_w(r_next);
            r_next = r_fut;
#pragma unroll
            for (int off = LPN / 2; off >= 1; off >>= 1) acc += __shfl_xor_sync(FULL, acc, off);
            if (l == 0) store((g0 + q) * B + g, acc);
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

template <int C, bool HAS_PERM, bool HAS_SVAL, bool HAS_HINT, bool BF16 = false>
cudaError_t launch_ring_tt(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                           const void *W, const void *H, float *P, int64_t nnz, int sm_count,
                           unsigned long long *work_counter, int *dev_status, cudaStream_t stream)
{
    using R = RingShape<C>;
    const size_t smem = (size_t)RING_WARPS * RING_NG * R::SLOT_BYTES + (size_t)RING_WARPS * RING_NG * 8;
    auto kern = sddmm_ring_kernel<C, HAS_PERM, HAS_SVAL, HAS_HINT, BF16>;
    static SmemOptinCache optin;  // one opt-in per instantiation and device
    cudaError_t e = optin_dynamic_smem(kern, smem, optin);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(work_counter, 0, sizeof(unsigned long long), stream);
    if (e != cudaSuccess) return e;
    // blocks of groups handed out dynamically: about four blocks per warp on small
    // inputs, never fewer than 4 groups (the ring drains between blocks; below ~100 k nonzeros
    // spreading the work over all warps matters more) or more than 128
    const int64_t n_groups = nnz / R::B;
    int64_t bg = n_groups / ((int64_t)sm_count * RING_WARPS * 4);
    if (bg < 4) bg = 4;
    if (bg > 128) bg = 128;
    kern<<<(unsigned)sm_count, RING_WARPS * 32, smem, stream>>>(rows, cols, perm, sval, W, H, P, nnz, (int)bg,
                                                                work_counter, dev_status);
    return cudaGetLastError();
}

template <int C, bool BF16 = false>
cudaError_t launch_ring_t(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                          const void *W, const void *H, float *P, int64_t nnz, bool cols_hinted, int sm_count,
                          unsigned long long *work_counter, int *dev_status, cudaStream_t stream)
{
#define RING_GO(PERM, SVAL, HINT)                                                                                         \
    return launch_ring_tt<C, PERM, SVAL, HINT, BF16>(rows, cols, perm, sval, W, H, P, nnz, sm_count, work_counter, dev_status, \
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

bool ring_supports(int K) { return K == 32 || K == 64 || K == 128 || K == 256 || K == 512 || K == 1024; }

cudaError_t launch_ring(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                        const float *W, const float *H, float *P, int64_t nnz, int K, bool cols_hinted, int sm_count,
                        unsigned long long *work_counter, int *dev_status, cudaStream_t stream)
{
    if (nnz == 0) return cudaSuccess;
    switch (K) {
    case 32:
    case 64:
    case 128:  // rows up to 512 bytes: the cp.async ring (measured faster than one bulk copy per row there)
        return launch_ring_small(rows, cols, perm, sval, W, H, P, nnz, K, cols_hinted, sm_count, work_counter, stream);
    case 256: return launch_ring_t<2>(rows, cols, perm, sval, W, H, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    case 512: return launch_ring_t<4>(rows, cols, perm, sval, W, H, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    case 1024: return launch_ring_t<8>(rows, cols, perm, sval, W, H, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    default: return cudaErrorInvalidValue;
    }
}

// bfloat16 operand storage (opt-in): rows of 2K bytes on the same rings, fp32 products and sums.
bool ring_bf16_supports(int K) { return K == 256 || K == 512 || K == 1024 || K == 2048; }

cudaError_t launch_ring_bf16(const int32_t *rows, const int32_t *cols, const int32_t *perm, const float *sval,
                             const void *W_bf16, const void *H_bf16, float *P, int64_t nnz, int K, bool cols_hinted, int sm_count,
                             unsigned long long *work_counter, int *dev_status, cudaStream_t stream)
{
    if (nnz == 0) return cudaSuccess;
    switch (K) {
    case 256: return launch_ring_t<1, true>(rows, cols, perm, sval, W_bf16, H_bf16, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    case 512: return launch_ring_t<2, true>(rows, cols, perm, sval, W_bf16, H_bf16, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    case 1024: return launch_ring_t<4, true>(rows, cols, perm, sval, W_bf16, H_bf16, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    case 2048: return launch_ring_t<8, true>(rows, cols, perm, sval, W_bf16, H_bf16, P, nnz, cols_hinted, sm_count, work_counter, dev_status, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace sddmm
