// Device-side self-check of an SDDMM result: every sampled nonzero is recomputed in
// float64 (operands exact, products and sums in double) together with the magnitude
// scale A = sum_t |w_t h_t| (|s|), and |P - ref| is compared with tol * max(|ref|, A)
// -- the per-nonzero criterion the reference's in-line comparison approximates with
// an absolute bound (HiPC18_mpi/sddmm.cu:318-334).  It is a product-side sanity
// check for the command line (--check) and for multi-GPU runs where no host holds
// all of W; the parity tests use the CPU oracle instead.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace sddmm {

namespace {

__global__ void __launch_bounds__(256)
check_result_kernel(const int32_t *__restrict__ rows, const int32_t *__restrict__ cols, const float *__restrict__ sval,
                    const float *__restrict__ W, const float *__restrict__ H, const float *__restrict__ P, int64_t nnz,
                    int K, int64_t stride, double tol, CheckResult *out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int K4 = K >> 2;
    double worst = 0.0;
    unsigned long long bad = 0, checked = 0;
    for (int64_t i = warp * stride; i < nnz; i += n_warps * stride) {
        const float4 *w = reinterpret_cast<const float4 *>(W) + (int64_t)rows[i] * K4;
        const float4 *h = reinterpret_cast<const float4 *>(H) + (int64_t)cols[i] * K4;
        double s = 0.0, a = 0.0;
        for (int q = lane; q < K4; q += 32) {
            const float4 x = __ldg(w + q), y = __ldg(h + q);
            const double p0 = (double)x.x * y.x, p1 = (double)x.y * y.y, p2 = (double)x.z * y.z, p3 = (double)x.w * y.w;
            s += (p0 + p1) + (p2 + p3);
            a += (fabs(p0) + fabs(p1)) + (fabs(p2) + fabs(p3));
        }
        for (int o = 16; o; o >>= 1) {
            s += __shfl_xor_sync(0xffffffffu, s, o);
            a += __shfl_xor_sync(0xffffffffu, a, o);
        }
        if (lane == 0) {
            if (sval) {
                const double v = (double)sval[i];
                s *= v;
                a *= fabs(v);
            }
            const double got = (double)P[i];
            const double scale = fmax(fmax(fabs(s), a), 1e-300);
            const double err = fabs(got - s) / scale;
            ++checked;
            if (!(err <= tol)) ++bad;  // NaN counts as bad
            if (!(err <= worst)) worst = err == err ? err : 1e300;
        }
    }
    if (lane == 0 && checked) {
        atomicAdd(&out->n_checked, checked);
        if (bad) atomicAdd(&out->n_bad, bad);
        // doubles >= 0 order like their bit patterns
        atomicMax(reinterpret_cast<unsigned long long *>(&out->max_scaled_err), (unsigned long long)__double_as_longlong(worst));
    }
}

}  // namespace

cudaError_t launch_check_result(const int32_t *rows, const int32_t *cols, const float *sval, const float *W, const float *H,
                                const float *P, int64_t nnz, int K, int64_t stride, double tol, CheckResult *d_out,
                                int sm_count, cudaStream_t stream)
{
    cudaError_t e = cudaMemsetAsync(d_out, 0, sizeof(CheckResult), stream);
    if (e != cudaSuccess || nnz == 0) return e;
    if (stride < 1) stride = 1;
    check_result_kernel<<<(unsigned)(sm_count * 8), 256, 0, stream>>>(rows, cols, sval, W, H, P, nnz, K, stride, tol, d_out);
    return cudaGetLastError();
}

}  // namespace sddmm
