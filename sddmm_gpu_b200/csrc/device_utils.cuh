// Device-side building blocks shared by the SDDMM kernels: the transposed
// butterfly reduction, mbarrier / bulk-copy (TMA) wrappers and the general,
// fully predicated warp step.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace sddmm {
namespace dev {

constexpr unsigned FULL = 0xffffffffu;
// Upper bound on polls of an mbarrier before a CTA gives up and reports
// DEV_MBARRIER_TIMEOUT: the backstop behind the wall-clock budget of
// mbar_wait_bounded (MBAR_WAIT_BUDGET_NS), far beyond any legitimate copy latency.
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
__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Wall-clock budget of one bounded wait.  The poll count alone says little about
// time (every try_wait may block for a hardware-defined slice before it answers),
// so the loop also reads the nanosecond timer every 64 polls and gives up once the
// budget is spent; the poll limit stays as a backstop should the timer stand still.
#ifndef SDDMM_WAIT_BUDGET_MS
#define SDDMM_WAIT_BUDGET_MS 500
#endif
constexpr unsigned long long MBAR_WAIT_BUDGET_NS = SDDMM_WAIT_BUDGET_MS * 1000000ull;  // 0.5 s: a thousand times any legitimate wait
struct WaitClock {
    unsigned long long start = 0;
    __device__ __forceinline__ bool expired(int it, unsigned long long budget_ns = MBAR_WAIT_BUDGET_NS)
    {
        if ((it & 63) != 63) return false;
        const unsigned long long now = globaltimer_ns();
        if (start == 0) {
            start = now;
            return false;
        }
        return now - start > budget_ns;
    }
};
// Bounded wait: false when the limit ran out.  Polls back off with a short
// sleep so that a waiting warp does not take issue slots from working ones.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, unsigned parity)
{
    WaitClock clock;
#pragma unroll 1
    for (int it = 0; it < MBAR_SPIN_LIMIT; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(it < 16 ? 32 : 256);
        if (clock.expired(it)) return false;
    }
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
// The same copy with an L2 eviction-priority hint (a createpolicy descriptor).
__device__ __forceinline__ void bulk_g2s_hint(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar,
                                              uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_last()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
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


}  // namespace dev
}  // namespace sddmm
