// The "pick" phase of the dense-cell kernels: the finished 128 x 64 block of a cell sits in shared
// memory (row-major, `stride` floats per row) and the cell's nonzeros take their entries, scale them
// by S and store them to P at their input positions.  NT threads (a multiple of 32), tid in [0, NT).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace sddmm {

template <int NT = 256>
__device__ __forceinline__ void pick_block(const float *Ct, int stride, const DenseCell &dc, bool masked, int64_t cell,
                                           int tid, const int32_t *__restrict__ idx, const uint16_t *__restrict__ rc,
                                           const unsigned long long *__restrict__ row_mask,
                                           const int32_t *__restrict__ row_base, const float *__restrict__ sval,
                                           float *__restrict__ P)
{
    if (masked) {
        // Row r of the cell holds the columns of mask[r]; its nonzeros are consecutive in the input from
        // base[r] on, in column order, so the one in column c sits at base[r] + popc(mask[r] below bit c).
        // A warp takes four rows at a time, lane l the columns l and l + 32: the S loads and the P stores of
        // a row are one or two contiguous runs.
        const unsigned long long *cm = row_mask + cell * DENSE_CELL_ROWS;
        const int32_t *cb = row_base + cell * DENSE_CELL_ROWS;
        const int lane = tid & 31, warp = tid >> 5;
        const unsigned below = (1u << lane) - 1u;
        for (int r0 = warp * 4; r0 < DENSE_CELL_ROWS; r0 += NT / 8) {
            unsigned lo[4], hi[4];
            int32_t base[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const unsigned long long m = __ldg(cm + r0 + u);
                lo[u] = (unsigned)m;
                hi[u] = (unsigned)(m >> 32);
                base[u] = __ldg(cb + r0 + u);
            }
            float s_lo[4], s_hi[4];
            int32_t p_lo[4], p_hi[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                p_lo[u] = base[u] + __popc(lo[u] & below);
                p_hi[u] = base[u] + __popc(lo[u]) + __popc(hi[u] & below);
                s_lo[u] = s_hi[u] = 1.f;
                if (sval) {
                    if ((lo[u] >> lane) & 1u) s_lo[u] = __ldcs(sval + p_lo[u]);
                    if ((hi[u] >> lane) & 1u) s_hi[u] = __ldcs(sval + p_hi[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float *crow = Ct + (r0 + u) * stride;
                if ((lo[u] >> lane) & 1u) __stcs(P + p_lo[u], crow[lane] * s_lo[u]);
                if ((hi[u] >> lane) & 1u) __stcs(P + p_hi[u], crow[lane + 32] * s_hi[u]);
            }
        }
    } else {
        // per-nonzero lists: input index and (row, column) inside the cell
        const int32_t *cidx = idx + dc.offset;
        const uint16_t *crc = rc + dc.offset;
        int i = tid;
        for (; i + 3 * NT < dc.count; i += 4 * NT) {  // four independent nonzeros per thread and trip
            unsigned code[4];
            int32_t o[4];
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                code[u] = __ldcs(crc + i + u * NT);
                o[u] = __ldcs(cidx + i + u * NT);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                v[u] = Ct[(code[u] >> 8) * stride + (code[u] & 255u)];
                if (sval) v[u] *= __ldg(sval + o[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) P[o[u]] = v[u];
        }
        for (; i < dc.count; i += NT) {
            const unsigned code = crc[i];
            const int32_t o = cidx[i];
            float v = Ct[(code >> 8) * stride + (code & 255u)];
            if (sval) v *= __ldg(sval + o);
            P[o] = v;
        }
    }
}

}  // namespace sddmm
