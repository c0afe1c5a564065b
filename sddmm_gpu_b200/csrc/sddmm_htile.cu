// Column-tile kernel for matrices with few columns: a tile of H rows lives in
// shared memory and every nonzero of that tile reads its H row from there.
//
// The reference's kernel keeps a tile of tile_size_X columns of H in shared memory
// and walks the nonzeros of that tile (HiPC18/src/sddmm.cu:70-170: comp_kernel_COO
// over the tiled order of util.h:286-372).  The same idea pays on B200 when the
// whole of H is a handful of tiles: 227 KB of shared memory hold 192 rows of
// K = 256, the gather then runs at shared-memory bandwidth (128 B / clock / SM)
// instead of the L2 -> SM rate of the ring kernel, and H crosses from L2 once per
// CTA and tile instead of once per nonzero.
//
// The nonzeros are in tiled order (column tiles ascending, rows ascending inside a
// tile; perm gives the input position).  The CTAs cut that order into equal
// contiguous ranges; a range lies in one tile or spans a few, and the CTA loads
// each tile it meets with bulk asynchronous copies (one per lane of warp 0,
// counted on one mbarrier).  Inside a range the warps take windows of 32 nonzeros
// round-robin: lane l holds the row, the input position and the S value of nonzero
// l and one packed word -- the byte offset of its H row in the tile, bit 0 set when
// its row differs from the row of the nonzero before it.  The window is processed
// 16 nonzeros at a time: one shuffle brings a nonzero's packed word to all lanes,
// the W row is in registers (reloaded when bit 0 says so: C float4 per lane), the
// H row is read from the tile as C conflict-free 128-bit loads per lane, the 16
// partial sums are reduced by one transposed butterfly (16 shuffles for 16
// nonzeros) and lane l stores nonzero l.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace sddmm {

using namespace dev;

namespace {

constexpr int HTILE_SMEM_BYTES = 196608;  // the tile: 192 rows of K = 256

template <int C, int NT>  // C float4 per lane: K = 128 C
__global__ void __launch_bounds__(NT, 1)
sddmm_htile_kernel(const int32_t *__restrict__ rows_t, const int32_t *__restrict__ cols_t, const int32_t *__restrict__ perm,
                   const float *__restrict__ sval, const float *__restrict__ W, const float *__restrict__ H,
                   float *__restrict__ P, int64_t nnz, int64_t N, int col_tile, const int64_t *__restrict__ tile_off,
                   int n_tiles, int *dev_status)
{
    constexpr int K = 128 * C, K4 = K / 4, NW = NT / 32;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ uint64_t bar;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const int64_t j_begin = nnz * blockIdx.x / gridDim.x, j_end = nnz * (blockIdx.x + 1) / gridDim.x;
    int t = 0;
    unsigned phase = 0;
    const float4 *W4 = reinterpret_cast<const float4 *>(W) + lane;
    const unsigned char *my_tile = smem_raw + lane * 16;  // this lane's 16 bytes of every 512-byte piece of a row
    for (int64_t j0 = j_begin; j0 < j_end;) {
        while (t + 1 < n_tiles && tile_off[t + 1] <= j0) ++t;  // the tile of nonzero j0 (empty tiles are skipped)
        const int64_t j1 = min(j_end, tile_off[t + 1]);
        const int64_t col0 = (int64_t)t * col_tile;
        const uint32_t bytes = (uint32_t)min((int64_t)col_tile, N - col0) * (uint32_t)(K * 4);
        __syncthreads();  // every warp has finished with the previous tile
        if (warp == 0) {
            if (lane == 0) {
                mbar_expect_tx(&bar, bytes);
                mbar_arrive(&bar);
            }
            __syncwarp();
            const uint32_t piece = (bytes + 511u) / 512u * 16u;  // a 32nd of the tile, in whole 16-byte units
            const uint32_t off = lane * piece;
            if (off < bytes)
                bulk_g2s(smem_raw + off, reinterpret_cast<const unsigned char *>(H + col0 * K) + off, min(piece, bytes - off), &bar);
        }
        bool ok = mbar_try_wait(&bar, phase) || mbar_wait_bounded(&bar, phase);
        if (!__syncthreads_and(ok)) {
            // a copy that did not arrive within the budget: report, give it one more budget to land (the
            // shared memory must not be released under a copy in flight) and leave
            if (tid == 0) atomicExch(dev_status, (int)DEV_MBARRIER_TIMEOUT);
            if (!ok) mbar_wait_bounded(&bar, phase);
            return;
        }
        phase ^= 1u;
        int cur = -1;  // the row whose W is in registers
        float4 w[C];
#pragma unroll
        for (int i = 0; i < C; ++i) w[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int64_t jb = j0 + 32 * warp; jb < j1; jb += 32 * NW) {
            const int64_t j = jb + lane;
            const int cnt = (int)min((int64_t)32, j1 - jb);
            const bool valid = lane < cnt;
            int r = 0;
            unsigned packed = 0;
            int64_t pm = 0;
            float sv = 1.f;
            if (valid) {
                r = __ldg(rows_t + j);
                packed = (unsigned)(__ldg(cols_t + j) - (int)col0) * (unsigned)(K * 4);
                pm = perm ? (int64_t)__ldg(perm + j) : j;
                if (sval) sv = __ldg(sval + pm);
            }
            // lanes past the end repeat the last nonzero's row (no reload) and read the tile's first row (discarded)
            const int r_last = __shfl_sync(FULL, r, cnt - 1);  // (every lane takes part in the shuffle)
            r = valid ? r : r_last;
            const int before = __shfl_up_sync(FULL, r, 1);
            packed |= (r != (lane == 0 ? cur : before)) ? 1u : 0u;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                if (16 * half >= cnt) break;
                float acc[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const unsigned pk = __shfl_sync(FULL, packed, 16 * half + k);
                    if (pk & 1u) {  // the same for all lanes: a new row
                        cur = __shfl_sync(FULL, r, 16 * half + k);
#pragma unroll
                        for (int i = 0; i < C; ++i) w[i] = __ldg(W4 + (int64_t)cur * K4 + i * 32);
                    }
                    const float4 *h = reinterpret_cast<const float4 *>(my_tile + (pk & ~1u));
                    float a = 0.f;
#pragma unroll
                    for (int i = 0; i < C; ++i) a = dot4(w[i], h[i * 32], a);
                    acc[k] = a;
                }
                reduce_transposed<32, 16>(acc, lane);  // the sum of nonzero k is now in lanes 2k, 2k + 1
                const float res = __shfl_sync(FULL, acc[0], 2 * (lane & 15));
                if (valid && (lane >> 4) == half) P[pm] = res * sv;
            }
            cur = __shfl_sync(FULL, r, 31);  // the last row of the window (also after an early exit of the loop)
        }
        j0 = j1;
    }
}

__global__ void htile_offsets_kernel(const int32_t *__restrict__ cols_t, int64_t nnz, int col_tile, int n_tiles, int64_t *off)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t > n_tiles) return;
    int64_t lo = 0, hi = nnz;
    while (lo < hi) {  // first nonzero of the tiled order whose tile is >= t
        const int64_t mid = (lo + hi) >> 1;
        if (cols_t[mid] / col_tile < t) lo = mid + 1;
        else hi = mid;
    }
    off[t] = lo;
}

template <int C, int NT>
cudaError_t launch_tt(const int32_t *rows_t, const int32_t *cols_t, const int32_t *perm, const float *sval, const float *W,
                      const float *H, float *P, int64_t nnz, int64_t N, int col_tile, const int64_t *tile_off, int n_tiles,
                      int sm_count, int *dev_status, cudaStream_t stream)
{
    static SmemOptinCache optin;  // per device
    const int smem = col_tile * 128 * C * 4;
    cudaError_t e = optin_dynamic_smem(sddmm_htile_kernel<C, NT>, smem, optin);
    if (e != cudaSuccess) return e;
    int64_t blocks = nnz / 1024;  // a CTA loads whole tiles: none for a handful of nonzeros
    if (blocks > sm_count) blocks = sm_count;
    if (blocks < 1) blocks = 1;
    sddmm_htile_kernel<C, NT><<<(unsigned)blocks, NT, smem, stream>>>(rows_t, cols_t, perm, sval, W, H, P, nnz, N, col_tile,
                                                                      tile_off, n_tiles, dev_status);
    return cudaGetLastError();
}

}  // namespace

int htile_cols(int K)
{
    if (K != 128 && K != 256 && K != 512) return 0;
    return HTILE_SMEM_BYTES / (K * 4);
}

cudaError_t build_htile_offsets(const int32_t *cols_t, int64_t nnz, int col_tile, int n_tiles, int64_t *d_off, cudaStream_t stream)
{
    htile_offsets_kernel<<<(n_tiles + 1 + 127) / 128, 128, 0, stream>>>(cols_t, nnz, col_tile, n_tiles, d_off);
    return cudaGetLastError();
}

cudaError_t launch_htile(const int32_t *rows_t, const int32_t *cols_t, const int32_t *perm, const float *sval, const float *W,
                         const float *H, float *P, int64_t nnz, int64_t N, int K, int col_tile, const int64_t *tile_off,
                         int n_tiles, int sm_count, int *dev_status, cudaStream_t stream)
{
    if (nnz == 0) return cudaSuccess;
    if (col_tile <= 0 || col_tile > htile_cols(K)) return cudaErrorInvalidValue;
    switch (K) {
    case 128: return launch_tt<1, 1024>(rows_t, cols_t, perm, sval, W, H, P, nnz, N, col_tile, tile_off, n_tiles, sm_count, dev_status, stream);
    // K = 256 with 1024 threads: the 64-register limit costs a few spilled words and is still the fastest
    // (config 2: 0.054 ms against 0.057 ms with 768 threads and 0.065 ms with 512)
    case 256: return launch_tt<2, 1024>(rows_t, cols_t, perm, sval, W, H, P, nnz, N, col_tile, tile_off, n_tiles, sm_count, dev_status, stream);
    case 512: return launch_tt<4, 512>(rows_t, cols_t, perm, sval, W, H, P, nnz, N, col_tile, tile_off, n_tiles, sm_count, dev_status, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace sddmm
