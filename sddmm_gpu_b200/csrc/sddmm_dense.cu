// Dense-cell kernel.
//
// Where S is locally dense -- a band, fully populated "global" rows and columns
// of an attention mask, the hub core of a power-law matrix -- gathering one H row
// per nonzero wastes the reuse that is there: the 128 x 64 nonzeros of a full
// cell touch only 128 rows of W and 64 rows of H.  The plan's classification pass
// (binning.cu, build_dense_cells) hands such cells to this kernel, which computes
// the whole block W[row0 .. row0+128) * H[col0 .. col0+64)^T as a small dense
// product and then lets the cell's nonzeros pick their entries.
//
// The product is plain fp32 FMA, register-tiled (each of the 256 threads owns an
// 8 x 4 piece of the block; per k it reads 12 floats from shared memory for 32
// FMAs), so results carry ordinary fp32 rounding -- no reduced-precision tensor
// path is involved.  W and H are staged through shared memory in chunks of 32
// along K, transposed so that the inner loop reads 128-bit vectors; positions
// outside the matrix or beyond K are zero-filled.  After the last chunk the block
// is parked in shared memory and the cell's nonzeros (grouped by cell, row-major
// inside, by the plan) read block[r][c], scale by S and store to P at their
// input positions.
//
// This replaces, for those cells, the per-nonzero gathers of comp_kernel_COO
// (HiPC18/src/kernel.h:29-50); the nearest idea in the reference tree is the
// dense/sparse split of other_ideas/our_work/sparse_dense_split.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace sddmm {

namespace {

constexpr int DR = DENSE_CELL_ROWS;  // 128
constexpr int DC = DENSE_CELL_COLS;  // 64
constexpr int KC = 32;               // K chunk
constexpr int WT_STRIDE = DR + 4;    // floats; keeps rows 16-byte aligned, spreads banks
constexpr int HT_STRIDE = DC + 4;
constexpr int CT_STRIDE = DC + 1;
constexpr int WT_FLOATS = KC * WT_STRIDE;
constexpr int HT_FLOATS = KC * HT_STRIDE;
constexpr int SMEM_FLOATS = DR * CT_STRIDE;  // the block; the staging buffers alias its start
static_assert(WT_FLOATS + HT_FLOATS <= SMEM_FLOATS, "staging must fit under the block");
static_assert(DR == 128 && DC == 64, "thread tiling below assumes 128 x 64 cells and 256 threads");

__global__ void __launch_bounds__(256)
sddmm_dense_kernel(const DenseCell *__restrict__ cells, int64_t n_cells, const int32_t *__restrict__ idx,
                   const uint16_t *__restrict__ rc, const float *__restrict__ sval, const float *__restrict__ W,
                   const float *__restrict__ H, float *__restrict__ P, int64_t M, int64_t N, int K)
{
    __shared__ __align__(16) float smem[SMEM_FLOATS];
    float *Wt = smem;              // [KC][WT_STRIDE]: Wt[k][r] = W[row0 + r][k0 + k]
    float *Ht = smem + WT_FLOATS;  // [KC][HT_STRIDE]: Ht[k][c] = H[col0 + c][k0 + k]
    float *Ct = smem;              // [DR][CT_STRIDE], after the last chunk

    const int tid = threadIdx.x;
    const int ty = tid >> 4;  // rows ty*8 .. ty*8+7
    const int tx = tid & 15;  // cols tx*4 .. tx*4+3

    for (int64_t cell = blockIdx.x; cell < n_cells; cell += gridDim.x) {
        const DenseCell dc = cells[cell];
        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

        for (int k0 = 0; k0 < K; k0 += KC) {
            // stage W: 128 rows x 32 floats = 1024 float4, four per thread
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int f = tid + i * 256;
                const int r = f >> 3, kq = (f & 7) * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                const int64_t row = (int64_t)dc.row0 + r;
                if (row < M && k0 + kq < K) v = __ldg(reinterpret_cast<const float4 *>(W + row * K + k0 + kq));
                Wt[(kq + 0) * WT_STRIDE + r] = v.x;
                Wt[(kq + 1) * WT_STRIDE + r] = v.y;
                Wt[(kq + 2) * WT_STRIDE + r] = v.z;
                Wt[(kq + 3) * WT_STRIDE + r] = v.w;
            }
            // stage H: 64 rows x 32 floats = 512 float4, two per thread
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int f = tid + i * 256;
                const int c = f >> 3, kq = (f & 7) * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                const int64_t col = (int64_t)dc.col0 + c;
                if (col < N && k0 + kq < K) v = __ldg(reinterpret_cast<const float4 *>(H + col * K + k0 + kq));
                Ht[(kq + 0) * HT_STRIDE + c] = v.x;
                Ht[(kq + 1) * HT_STRIDE + c] = v.y;
                Ht[(kq + 2) * HT_STRIDE + c] = v.z;
                Ht[(kq + 3) * HT_STRIDE + c] = v.w;
            }
            __syncthreads();
#pragma unroll 8
            for (int k = 0; k < KC; ++k) {
                const float4 a0 = *reinterpret_cast<const float4 *>(Wt + k * WT_STRIDE + ty * 8);
                const float4 a1 = *reinterpret_cast<const float4 *>(Wt + k * WT_STRIDE + ty * 8 + 4);
                const float4 b = *reinterpret_cast<const float4 *>(Ht + k * HT_STRIDE + tx * 4);
                const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const float bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
            }
            __syncthreads();  // everyone is done with this chunk (and, after the last, with the staging area)
        }
        // park the block, then let the nonzeros pick their entries
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) Ct[(ty * 8 + i) * CT_STRIDE + tx * 4 + j] = acc[i][j];
        __syncthreads();
        const int32_t *cidx = idx + dc.offset;
        const uint16_t *crc = rc + dc.offset;
        for (int i = tid; i < dc.count; i += 256) {
            const unsigned code = crc[i];
            const int32_t o = cidx[i];
            float v = Ct[(code >> 8) * CT_STRIDE + (code & 255u)];
            if (sval) v *= __ldg(sval + o);
            P[o] = v;
        }
        __syncthreads();  // the block is overwritten by the next cell's staging
    }
}

}  // namespace

cudaError_t launch_dense_cells(const DenseCell *cells, int64_t n_cells, const int32_t *idx, const uint16_t *rc,
                               const float *sval, const float *W, const float *H, float *P, int64_t M, int64_t N,
                               int K, int sm_count, cudaStream_t stream)
{
    if (n_cells == 0) return cudaSuccess;
    int64_t blocks = (int64_t)sm_count * 4;
    if (blocks > n_cells) blocks = n_cells;
    sddmm_dense_kernel<<<(unsigned)blocks, 256, 0, stream>>>(cells, n_cells, idx, rc, sval, W, H, P, M, N, K);
    return cudaGetLastError();
}

}  // namespace sddmm
