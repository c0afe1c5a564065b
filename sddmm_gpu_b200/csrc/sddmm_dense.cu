// Dense-cell kernel.
//
// Where S is locally dense -- a band, fully populated "global" rows and columns
// of an attention mask, the hub core of a power-law matrix -- gathering one H row
// per nonzero wastes the reuse that is there: the 128 x 64 nonzeros of a full
// cell touch only 128 rows of W and 64 rows of H.  The plan's classification pass
// (binning.cu, build_dense_cells) hands such cells to this kernel, which computes
// the whole block W[row0 .. row0+128) * H[col0 .. col0+64)^T as a small dense
// product and then lets the cell's nonzeros pick their entries.  Full rows and
// full columns ("global" tokens) are compacted by the plan first, so a cell's
// rows or columns may come through an index list instead of being consecutive.
//
// The product runs either on the tensor cores as 3xTF32 (every fp32 operand split
// into a TF32 head and tail, three mma.sync.m16n8k8 per product, fp32
// accumulation: fp32-level accuracy) or as plain fp32 FMA, register-tiled (each
// of the 256 threads owns an 8 x 4 piece of the block; per four k it reads twelve
// float4 from shared memory for 128 FMAs).  W and H are staged through shared memory in chunks of 64
// along K with 16-byte asynchronous copies (cp.async), rows padded so that the
// inner loop's 128-bit loads are conflict-free; positions outside the matrix or
// beyond K are zero-filled.  After the last chunk the block
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
#include "dense_pick.cuh"

namespace sddmm {

namespace {

constexpr int DR = DENSE_CELL_ROWS;  // 128
constexpr int DC = DENSE_CELL_COLS;  // 64
constexpr int KC = 64;               // K chunk staged at a time
constexpr int KS = KC + 4;           // row stride of the staged operands (floats): 16-byte aligned rows, banks spread
constexpr int CT_STRIDE = DC + 8;  // 72: the tensor path parks its fragments with conflict-free 64-bit stores
constexpr int STAGE_FLOATS = (DR + DC) * KS;
constexpr int BLOCK_FLOATS = DR * CT_STRIDE;  // the finished block; aliases the staging area
constexpr int SMEM_FLOATS = STAGE_FLOATS > BLOCK_FLOATS ? STAGE_FLOATS : BLOCK_FLOATS;
static_assert(DR == 128 && DC == 64, "thread tiling below assumes 128 x 64 cells and 256 threads");

// 16-byte asynchronous copy global -> shared; src_bytes = 0 fills the 16 bytes with zeros.
__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src, int src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)),
                 "l"(src), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_wait_all()
{
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// 3xTF32: an fp32 value x is split into hi = tf32(x) and lo = tf32(x - hi); the
// product a*b is accumulated as lo_a*hi_b + hi_a*lo_b + hi_a*hi_b in fp32 by
// three tensor-core MMAs, which keeps the error of the products at the 2^-19
// level instead of TF32's 2^-11.
__device__ __forceinline__ void split_tf32(float x, uint32_t &hi, uint32_t &lo)
{
    // head = x with the 13 mantissa bits TF32 does not have cleared; tail = x - head, exact in fp32.
    // The tensor core reads only the TF32 bits of an operand register, so the tail needs no conversion of
    // its own: what it drops is below 2^-20 |x|.  Two instructions per operand instead of two conversions
    // and a subtraction.
    hi = __float_as_uint(x) & 0xffffe000u;
    lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// TENSOR = false: fp32 FMA, register tile 8 x 4 per thread.
// TENSOR = true : 3xTF32 on the tensor cores (mma.sync m16n8k8), warp tile 32 x 32.
template <bool TENSOR>
__global__ void __launch_bounds__(256, 3)
sddmm_dense_kernel(const DenseCell *__restrict__ cells, int64_t n_cells, const int32_t *__restrict__ idx,
                   const uint16_t *__restrict__ rc, const unsigned long long *__restrict__ row_mask,
                   const int32_t *__restrict__ row_base, const int32_t *__restrict__ dense_rows, int64_t n_dense_rows,
                   const int32_t *__restrict__ dense_cols, int64_t n_dense_cols, const float *__restrict__ sval,
                   const float *__restrict__ W, const float *__restrict__ H, float *__restrict__ P, int64_t M,
                   int64_t N, int K)
{
    extern __shared__ __align__(16) float smem[];
    float *Ws = smem;            // [DR][KS]: Ws[r][k] = W[row0 + r][k0 + k]
    float *Hs = smem + DR * KS;  // [DC][KS]: Hs[c][k] = H[col0 + c][k0 + k]
    float *Ct = smem;            // [DR][CT_STRIDE], after the last chunk

    const int tid = threadIdx.x;
    // thread (ty, tx) owns rows ty + 16 i (i < 8) and columns tx + 16 j (j < 4): neighbouring
    // threads read neighbouring rows of the staged operands, which keeps the 128-bit
    // shared-memory loads free of bank conflicts
    const int ty = tid >> 4;
    const int tx = tid & 15;

    for (int64_t cell = blockIdx.x; cell < n_cells; cell += gridDim.x) {
        DenseCell dc = cells[cell];
        const bool masked = (dc.cls & 0x100) != 0;  // row-mask form: no per-nonzero list
        dc.cls &= 0xff;
        float acc[8][4];  // FMA path: [row i][col j]; tensor path: [m-tile*4 + n-tile][fragment register]
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

        for (int k0 = 0; k0 < K; k0 += KC) {
            // stage W (128 x 64 floats = 2048 float4, eight per thread) and H (1024 float4, four per
            // thread); rows outside the matrix and k beyond K arrive as zeros
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int f = tid + i * 256;
                const int r = f >> 4, kq = (f & 15) * 4;
                int64_t row = (int64_t)dc.row0 + r;
                if (dc.cls == 0) row = row < n_dense_rows ? dense_rows[row] : M;  // compacted full rows
                const bool ok = row < M && k0 + kq < K;
                cp_async16(Ws + r * KS + kq, ok ? W + row * K + k0 + kq : W, ok ? 16 : 0);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int f = tid + i * 256;
                const int c = f >> 4, kq = (f & 15) * 4;
                int64_t col = (int64_t)dc.col0 + c;
                if (dc.cls == 1) col = col < n_dense_cols ? dense_cols[col] : N;  // compacted full columns
                const bool ok = col < N && k0 + kq < K;
                cp_async16(Hs + c * KS + kq, ok ? H + col * K + k0 + kq : H, ok ? 16 : 0);
            }
            cp_async_wait_all();
            __syncthreads();
            if constexpr (TENSOR) {
                // warp (wr, wc) of a 4 x 2 grid owns rows wr*32 .. +32 and columns wc*32 .. +32 of the block:
                // two m16 tiles x four n8 tiles.  Fragment element (row, k) sits at Ws[row][k], (k, n) at
                // Hs[n][k]; with a row stride of 68 floats the 32 lanes of a fragment load hit 32 banks.
                const int lane = tid & 31, warp = tid >> 5;
                const int wr = warp >> 1, wc = warp & 1;
                const int fr = lane >> 2, fk = lane & 3;
#pragma unroll 2
                for (int kk = 0; kk < KC; kk += 8) {
                    // B fragments of the four n8 tiles first, then one m16 tile of A at a time: 24 split
                    // operands live at once instead of 32, which keeps the kernel inside 80 registers
                    uint32_t b_hi[4][2], b_lo[4][2];
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        const float *p = Hs + (wc * 32 + nt * 8 + fr) * KS + kk + fk;
                        split_tf32(p[0], b_hi[nt][0], b_lo[nt][0]);
                        split_tf32(p[4], b_hi[nt][1], b_lo[nt][1]);
                    }
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        uint32_t a_hi[4], a_lo[4];
                        const float *p = Ws + (wr * 32 + mt * 16 + fr) * KS + kk + fk;
                        split_tf32(p[0], a_hi[0], a_lo[0]);
                        split_tf32(p[8 * KS], a_hi[1], a_lo[1]);
                        split_tf32(p[4], a_hi[2], a_lo[2]);
                        split_tf32(p[8 * KS + 4], a_hi[3], a_lo[3]);
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt) {
                            mma_tf32(acc[mt * 4 + nt], a_lo, b_hi[nt]);
                            mma_tf32(acc[mt * 4 + nt], a_hi, b_lo[nt]);
                            mma_tf32(acc[mt * 4 + nt], a_hi, b_hi[nt]);
                        }
                    }
                }
            } else {
#pragma unroll 2
                for (int kk = 0; kk < KC; kk += 4) {
                    float4 a[8], b[4];
    #pragma unroll
                    for (int i = 0; i < 8; ++i) a[i] = *reinterpret_cast<const float4 *>(Ws + (ty + 16 * i) * KS + kk);
    #pragma unroll
                    for (int j = 0; j < 4; ++j) b[j] = *reinterpret_cast<const float4 *>(Hs + (tx + 16 * j) * KS + kk);
    #pragma unroll
                    for (int i = 0; i < 8; ++i)
    #pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
                            acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
                            acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
                            acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
                        }
                }
}
            __syncthreads();  // everyone is done with this chunk (and, after the last, with the staging area)
        }
        // park the block, then let the nonzeros pick their entries
        if constexpr (TENSOR) {
            const int lane = tid & 31, warp = tid >> 5;
            const int wr = warp >> 1, wc = warp & 1;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int r = wr * 32 + mt * 16 + (lane >> 2), c = wc * 32 + nt * 8 + (lane & 3) * 2;
                    *reinterpret_cast<float2 *>(Ct + r * CT_STRIDE + c) = make_float2(acc[mt * 4 + nt][0], acc[mt * 4 + nt][1]);
                    *reinterpret_cast<float2 *>(Ct + (r + 8) * CT_STRIDE + c) = make_float2(acc[mt * 4 + nt][2], acc[mt * 4 + nt][3]);
                }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) Ct[(ty + 16 * i) * CT_STRIDE + tx + 16 * j] = acc[i][j];
        }
        __syncthreads();
        pick_block(Ct, CT_STRIDE, dc, masked, cell, tid, idx, rc, row_mask, row_base, sval, P);
        __syncthreads();  // the block is overwritten by the next cell's staging
    }
}

}  // namespace

cudaError_t launch_dense_cells(const DenseCell *cells, int64_t n_cells, const int32_t *idx, const uint16_t *rc,
                               const unsigned long long *row_mask, const int32_t *row_base, const int32_t *dense_rows, int64_t n_dense_rows, const int32_t *dense_cols,
                               int64_t n_dense_cols, const float *sval, const float *W, const float *H, float *P,
                               int64_t M, int64_t N, int K, bool tensor, int sm_count, cudaStream_t stream)
{
    if (n_cells == 0) return cudaSuccess;
    const size_t smem = sizeof(float) * SMEM_FLOATS;
    static SmemOptinCache optin_fma, optin_tensor;  // per device
    {
        cudaError_t e = optin_dynamic_smem(sddmm_dense_kernel<false>, smem, optin_fma);
        if (e == cudaSuccess) e = optin_dynamic_smem(sddmm_dense_kernel<true>, smem, optin_tensor);
        if (e != cudaSuccess) return e;
    }
    int64_t blocks = (int64_t)sm_count * 3;
    if (blocks > n_cells) blocks = n_cells;
    if (tensor)
        sddmm_dense_kernel<true><<<(unsigned)blocks, 256, smem, stream>>>(cells, n_cells, idx, rc, row_mask, row_base,
                                                                          dense_rows, n_dense_rows, dense_cols,
                                                                          n_dense_cols, sval, W, H, P, M, N, K);
    else
        sddmm_dense_kernel<false><<<(unsigned)blocks, 256, smem, stream>>>(cells, n_cells, idx, rc, row_mask, row_base,
                                                                           dense_rows, n_dense_rows, dense_cols,
                                                                           n_dense_cols, sval, W, H, P, M, N, K);
    return cudaGetLastError();
}

}  // namespace sddmm
