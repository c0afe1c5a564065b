// sddmm_count_cols_noalloc -- the one entry point of the library that never
// allocates.
//
// Who needs it.  Some hosts of this library are not allowed to create device
// memory at all: a serving process whose framework has already reserved the
// whole GPU for its own pool, a latency-critical loop that cannot afford the
// device-wide synchronisation cudaMalloc and cudaFree imply, or a plug-in that
// runs inside somebody else's callback where the CUDA allocator must not be
// entered.  Those callers still want N_nz (the number of distinct columns of S)
// to report the algorithmic bytes of an SDDMM; sddmm_plan_count_cols() gets it
// with a temporary cudaMalloc'ed mark array, this variant keeps the mark array
// in the library image instead.
//
// The scratch is one file-scope device array of fixed size (below): every GPU
// that loads the library holds SDDMM_NOALLOC_SCRATCH_BYTES of it until the
// process exits, and that size bounds the matrices the entry point accepts.
// It is shared by every call on a device and keeps whatever the last call left in
// it, so each call clears the part it is going to use first, and two calls that
// overlap on the same GPU (different streams or threads) would race on it.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdio>

#include "sddmm_b200.h"

namespace {

constexpr size_t HEADER_BYTES = 256;  // [0, 8): the count; the column marks follow
constexpr size_t SCRATCH_BYTES = HEADER_BYTES + (size_t)SDDMM_NOALLOC_MAX_COLS;
static_assert(SCRATCH_BYTES == SDDMM_NOALLOC_SCRATCH_BYTES, "header and source disagree on the scratch size");

// In host code this name is only a handle for cudaGetSymbolAddress(): it is not
// a device address and must never be handed to a kernel as one.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
// device address of the array, per device, once resolved (two threads making a device's first call
// both resolve the same address; the atomic only makes the publication well defined)
std::atomic<unsigned char *> g_scratch_addr[MAX_DEVICES];

void fail(char *errbuf, int len, const char *msg, cudaError_t e = cudaSuccess)
{
    if (!errbuf || len <= 0) return;
    if (e != cudaSuccess) std::snprintf(errbuf, (size_t)len, "%s: %s", msg, cudaGetErrorString(e));
    else std::snprintf(errbuf, (size_t)len, "%s", msg);
}

__global__ void noalloc_mark_kernel(const int32_t *__restrict__ cols, int64_t nnz, int64_t N, unsigned char *marks)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nnz; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = cols[i];
        if (c >= 0 && c < N) marks[c] = 1;  // an index outside the matrix is ignored, never written
    }
}

__global__ void noalloc_count_kernel(const unsigned char *__restrict__ marks, int64_t N, unsigned long long *count)
{
    unsigned long long c = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += (int64_t)gridDim.x * blockDim.x)
        c += marks[i];
    for (int o = 16; o; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0 && c) atomicAdd(count, c);
}

unsigned blocks_for(int64_t n)
{
    int64_t b = (n + 255) / 256;
    if (b > 148 * 16) b = 148 * 16;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace

extern "C" int sddmm_count_cols_noalloc(int device, const int32_t *d_cols, int64_t nnz, int64_t N, void *cuda_stream,
                                        int64_t *n_nonempty_cols, char *errbuf, int errbuf_len)
{
    if (errbuf && errbuf_len > 0) errbuf[0] = 0;
    if (!n_nonempty_cols || nnz < 0 || N < 0 || (nnz > 0 && !d_cols) || device < 0 || device >= MAX_DEVICES) {
        fail(errbuf, errbuf_len, "invalid argument");
        return SDDMM_INVALID_ARG;
    }
    if (N > (int64_t)SDDMM_NOALLOC_MAX_COLS) {
        char msg[160];
        std::snprintf(msg, sizeof(msg), "N = %lld exceeds SDDMM_NOALLOC_MAX_COLS = %lld: the built-in scratch cannot hold "
                      "one mark per column; use sddmm_plan_count_cols()", (long long)N, (long long)SDDMM_NOALLOC_MAX_COLS);
        fail(errbuf, errbuf_len, msg);
        return SDDMM_INVALID_ARG;
    }
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) {
        fail(errbuf, errbuf_len, "cudaSetDevice", e);
        (void)cudaGetLastError();
        return SDDMM_NO_DEVICE;
    }
    cudaStream_t s = (cudaStream_t)cuda_stream;
    {
        // the call hands back a number, so it ends by waiting for the stream: a stream that
        // is being captured cannot be waited for, and trying would break the capture
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        e = cudaStreamIsCapturing(s, &cap);
        if (e != cudaSuccess) {
            fail(errbuf, errbuf_len, "cudaStreamIsCapturing", e);
            (void)cudaGetLastError();
            return SDDMM_CUDA_ERROR;
        }
        if (cap != cudaStreamCaptureStatusNone) {
            fail(errbuf, errbuf_len, "sddmm_count_cols_noalloc waits for its result and cannot run on a capturing stream");
            return SDDMM_INVALID_ARG;
        }
    }
    // One-time set-up per device, with that device current: ask the runtime where
    // this device's copy of the array lives.  This is the part of the first call
    // that must not fall inside a stream capture.
    if (!g_scratch_addr[device].load(std::memory_order_acquire)) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            fail(errbuf, errbuf_len, "cudaGetSymbolAddress(scratch)", e);
            (void)cudaGetLastError();
            return SDDMM_CUDA_ERROR;
        }
        g_scratch_addr[device].store((unsigned char *)p, std::memory_order_release);
    }
    unsigned char *scratch = g_scratch_addr[device].load(std::memory_order_acquire);
    unsigned long long *count = (unsigned long long *)scratch;
    unsigned char *marks = scratch + HEADER_BYTES;

    // the previous call's count and marks are still there: clear what this call uses
    e = cudaMemsetAsync(scratch, 0, HEADER_BYTES + (size_t)N, s);
    if (e == cudaSuccess && nnz > 0) {
        noalloc_mark_kernel<<<blocks_for(nnz), 256, 0, s>>>(d_cols, nnz, N, marks);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess && N > 0) {
        noalloc_count_kernel<<<blocks_for(N), 256, 0, s>>>(marks, N, count);
        e = cudaGetLastError();
    }
    unsigned long long h = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&h, count, sizeof(h), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        fail(errbuf, errbuf_len, "counting columns", e);
        (void)cudaGetLastError();
        return SDDMM_CUDA_ERROR;
    }
    *n_nonempty_cols = (int64_t)h;
    return SDDMM_OK;
}
