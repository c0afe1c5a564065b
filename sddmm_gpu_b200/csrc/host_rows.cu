// Row upload from mapped host memory: the GPU reads the listed rows of a
// row-major host array over PCIe and writes them to the same rows of a device
// array.  An SDDMM reads only the rows of W and H that a nonzero touches; on
// graph matrices close to half of the rows are untouched, and a plain
// cudaMemcpy of the whole array moves them all the same (the reference does,
// HiPC18/src/sddmm.cu:71-73).  The host array must be page-locked and mapped into
// the device's address space (every cudaHostAlloc / cudaHostRegister allocation
// is, under unified addressing); the caller checks that before launching.
//
// Few, small CTAs on purpose: the kernel is bound by the PCIe link, not by the
// SMs, and it shares the SMs with the SDDMM kernels of earlier chunks.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace sddmm {

namespace {

constexpr int UP_TPB = 256;
constexpr int UP_ROWS = 4;  // rows a warp moves together: 4 x 16 bytes in flight per lane

__global__ void __launch_bounds__(UP_TPB)
upload_rows_kernel(const char *__restrict__ src, char *__restrict__ dst, const int32_t *__restrict__ list,
                   int64_t n_rows, int row_bytes)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * UP_TPB + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * UP_TPB) >> 5;
    const int pieces = row_bytes >> 4;  // 16-byte pieces per row (row_bytes = 4K, K a multiple of 4)
    for (int64_t q = warp * UP_ROWS; q < n_rows; q += n_warps * UP_ROWS) {
        int64_t off[UP_ROWS];
#pragma unroll
        for (int j = 0; j < UP_ROWS; ++j)
            off[j] = q + j < n_rows ? (int64_t)__ldg(list + q + j) * row_bytes : -1;
        for (int c = lane; c < pieces; c += 32) {
            uint4 v[UP_ROWS];
#pragma unroll
            for (int j = 0; j < UP_ROWS; ++j)
                if (off[j] >= 0) v[j] = __ldcs(reinterpret_cast<const uint4 *>(src + off[j]) + c);
#pragma unroll
            for (int j = 0; j < UP_ROWS; ++j)
                if (off[j] >= 0) __stcs(reinterpret_cast<uint4 *>(dst + off[j]) + c, v[j]);
        }
    }
}

// 32 x 32 tiles through shared memory: coalesced reads along n, coalesced writes along K.
__global__ void __launch_bounds__(256)
transpose_operand_kernel(const float *__restrict__ src, float *__restrict__ dst, int64_t n, int K)
{
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8 threads
    const int64_t n_tiles_n = (n + 31) / 32;
    const int64_t n_tiles = n_tiles_n * ((K + 31) / 32);
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const int64_t r0 = (t % n_tiles_n) * 32;
        const int k0 = (int)(t / n_tiles_n) * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            const int k = k0 + ty + j;
            const int64_t r = r0 + tx;
            tile[ty + j][tx] = (k < K && r < n) ? src[(int64_t)k * n + r] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            const int64_t r = r0 + ty + j;
            const int k = k0 + tx;
            if (r < n && k < K) dst[r * K + k] = tile[tx][ty + j];
        }
        __syncthreads();
    }
}

}  // namespace

cudaError_t launch_transpose_operand(const float *src_kmajor, float *dst_rowmajor, int64_t n, int K, cudaStream_t stream)
{
    if (n == 0 || K == 0) return cudaSuccess;
    const int64_t n_tiles = ((n + 31) / 32) * ((K + 31) / 32);
    const unsigned grid = (unsigned)(n_tiles < 148 * 16 ? n_tiles : 148 * 16);
    transpose_operand_kernel<<<grid, 256, 0, stream>>>(src_kmajor, dst_rowmajor, n, K);
    return cudaGetLastError();
}

cudaError_t launch_upload_rows(const float *mapped_host, float *dev, const int32_t *d_row_list, int64_t n_rows, int K,
                               int n_ctas, cudaStream_t stream)
{
    if (n_rows == 0) return cudaSuccess;
    upload_rows_kernel<<<(unsigned)n_ctas, UP_TPB, 0, stream>>>(reinterpret_cast<const char *>(mapped_host),
                                                               reinterpret_cast<char *>(dev), d_row_list, n_rows, K * 4);
    return cudaGetLastError();
}

}  // namespace sddmm
