// Dense-cell kernel on the 5th-generation tensor cores (tcgen05, accumulator in
// tensor memory), warp-specialised.
//
// Same job as sddmm_dense_kernel: a dense cell of S is computed as the 128 x 64
// block W[rows] * H[cols]^T and the cell's nonzeros pick their entries.  Here
// the product is issued by ONE thread as tcgen05.mma instructions (M = 128,
// N = 64, K = 8 per instruction, kind::tf32) that read both operands from shared
// memory through matrix descriptors and accumulate into 64 columns of tensor
// memory (TMEM).  fp32-level accuracy comes from 3xTF32 as in the mma.sync
// variant: every operand is written to shared memory twice, as its TF32 head (x
// with the 13 low mantissa bits cleared) and its tail (x - head, exact), and
// every k-step issues tail*head + head*tail + head*head.  (The head tile is the
// raw fp32 data: the tensor core reads only the TF32 bits of an element.)
//
// One persistent CTA per SM, three roles that overlap through mbarriers:
//   warps 0-7   producers: copy W / H rows of a K chunk (32 k) into the head tiles of one
//               of three operand stages with cp.async, two chunks ahead (the raw fp32
//               data is the TF32 head as far as the tensor core is concerned), and
//               compute the tail tiles from them in shared memory;
//   warp  8     one thread issues the MMAs of a chunk when its stage is full and
//               commits them to the stage's "empty" barrier; after a cell's last
//               chunk it commits to the accumulator's "full" barrier;
//   warps 9-24  epilogue: read the finished block from TMEM (tcgen05.ld, a quarter row per
//               thread), release the accumulator (two of them alternate), park the
//               block in shared memory and let the cell's nonzeros pick their entries.
//
// Shared-memory operand layout (K-major, 128-byte swizzle): a tile of R rows x 32 k is R lines of
// 128 bytes, one per row, in groups of eight rows (1024 bytes, the descriptor's stride-dimension
// offset); inside a group the 16-byte piece c of row r sits at piece c ^ (r % 8) of the row's line --
// the layout a tile copy with the 128-byte swizzle would produce, and the one the tensor core reads
// without bank conflicts.  One instruction consumes 32 bytes of every row, so k-step s starts 32 s
// bytes into the tile.  Producer thread f writes bytes [16 f, 16 f + 16) of a tile, i.e. piece f % 8
// of row f / 8, which holds the four k from 4 ((f % 8) ^ (f / 8 % 8)) on: the eight lanes of a row
// read its 128 contiguous bytes in global memory and fill one 128-byte line of shared memory.
//
// Two forms.  General: every chunk of every cell brings its W and H tiles into one of three stages.  Runs
// (K <= 64): the CTAs take the cells four consecutive ones at a time, and the W tile (both chunks, head and tail:
// 64 KB, two buffers alternating) stays in shared memory for as long as the cells that follow belong to the same
// row block -- only H tiles go through the stages then, and the producers stage and split a third of the bytes.
//
// Every wait is bounded (mbarrier polls with a limit; on expiry the role sets the
// device status word and leaves its loop, the others run into their own limits),
// the only CTA-wide barriers are at the start and the end, and the TMEM columns
// are released on every path.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "common.cuh"
#include "dense_pick.cuh"
#include "device_utils.cuh"

namespace sddmm {

using namespace dev;

namespace {

constexpr int DR = DENSE_CELL_ROWS;  // 128 = M of the MMA = TMEM lanes
constexpr int DC = DENSE_CELL_COLS;  // 64  = N of the MMA = TMEM columns per accumulator
constexpr int KC = 32;               // K chunk of one operand stage
constexpr int STAGES = 3;
constexpr int A_TILE_BYTES = DR * KC * 4;  // 16 KB
constexpr int B_TILE_BYTES = DC * KC * 4;  // 8 KB
constexpr int STAGE_BYTES = 2 * A_TILE_BYTES + 2 * B_TILE_BYTES;  // head and tail tiles of both operands: 48 KB
constexpr int CT_STRIDE = DC + 4;          // floats per row of the parked block: the 128-bit stores of eight rows fall into different banks
constexpr int CT_BYTES = DR * CT_STRIDE * 4;
constexpr int TC_SMEM_BYTES = STAGES * STAGE_BYTES + CT_BYTES;  // 182,272 bytes
constexpr int N_PRODUCERS = 256, N_EPILOGUE = 512;
constexpr int MMA_WARP = N_PRODUCERS / 32, EPI_WARP0 = MMA_WARP + 1;
constexpr int TC_THREADS = N_PRODUCERS + 32 + N_EPILOGUE;  // 800
constexpr uint32_t TMEM_COLS = 2 * DC;  // two accumulators
constexpr uint32_t LBO = 16, SBO = 8 * KC * 4;  // leading offset unused by swizzled K-major tiles; 8 rows of 128 bytes
// What the epilogue needs to know about a cell before its product is there: fetched into shared memory two
// cells ahead.
constexpr int META_SLOTS = 4;
// "Runs" form (K <= 64, i.e. at most two chunks): the W tile of a cell stays in shared memory for all the cells of
// its row block that the CTA takes one after the other (a run); only H tiles go through the stages.
constexpr int RUN_DEAL = 4;                                   // consecutive cells a CTA takes at a time (2: 0.237 ms, 3: 0.232, 4: 0.227, 8: 0.235, 16: 0.259 on config 5)
constexpr int A_CHUNK_BYTES = 2 * A_TILE_BYTES;               // head and tail tile of one chunk of W: 32 KB
constexpr int A_BUF_BYTES = 2 * A_CHUNK_BYTES;                // both chunks: 64 KB, two such buffers alternate
constexpr int B_STAGE_BYTES = 2 * B_TILE_BYTES;               // head and tail tile of one chunk of H: 16 KB
constexpr int RUNS_SMEM_BYTES = 2 * A_BUF_BYTES + STAGES * B_STAGE_BYTES + CT_BYTES;  // 215,040 bytes
struct __align__(16) MetaSlot {
    unsigned long long mask[DENSE_CELL_ROWS];  // columns held by each cell row
    int32_t base[DENSE_CELL_ROWS];             // input index of each cell row's first nonzero
    int32_t cls;                               // DenseCell::cls (class, row-mask flag)
    int32_t pad[3];
};

// Shared-memory matrix descriptor: start address, leading / stride byte offsets (all >> 4), version 1,
// layout type 2 = 128-byte swizzle (bits 61-63).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor of kind::tf32: D = fp32 (bits 4-5 = 1), A = B = TF32 (bits 7-9, 10-12 = 2), both
// K-major (bits 15, 16 = 0), N >> 3 at bit 17, M >> 4 at bit 24.
constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(DC >> 3) << 17) | ((uint32_t)(DR >> 4) << 24);

__device__ __forceinline__ void mma_tf32_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(IDESC), "r"(accumulate)
        : "memory");
}

// tail = x - head(x) of four consecutive k of one row (head = x with the 13 low mantissa bits cleared), exact
__device__ __forceinline__ void tail_store(const float4 v, unsigned char *dst)
{
    float4 lo;
    lo.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
    lo.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
    lo.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
    lo.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
    *reinterpret_cast<float4 *>(dst) = lo;
}
// 16-byte asynchronous copy global -> shared; src_bytes = 0 fills the 16 bytes with zeros
__device__ __forceinline__ void cp_async16_zfill(void *dst_smem, const void *src, int src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(src_bytes) : "memory");
}

// barrier.cta.red.and over the 512 epilogue threads (named barrier 1): one answer for all of them
__device__ __forceinline__ bool epilogue_all(bool mine)
{
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbarrier.cta.red.and.pred q, 1, 512, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)mine)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("barrier.cta.sync 1, 512;" ::: "memory"); }

// A warp waits for a barrier phase: lane 0 polls (32 lanes polling one word cost 32 accesses of the shared-memory
// pipe per poll), the others take its answer; __shfl_sync orders the warp's memory accesses behind the wait.
__device__ __forceinline__ bool wait_bar(uint64_t *bar, unsigned parity)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = (mbar_try_wait(bar, parity) || mbar_wait_bounded(bar, parity)) ? 1 : 0;
    return __shfl_sync(FULL, ok, 0) != 0;
}

template <bool RUNS>
__global__ void __launch_bounds__(TC_THREADS, 1)
sddmm_dense_tc_kernel(const DenseCell *__restrict__ cells, int64_t n_cells, const int32_t *__restrict__ idx,
                      const uint16_t *__restrict__ rc, const unsigned long long *__restrict__ row_mask,
                      const int32_t *__restrict__ row_base, const int32_t *__restrict__ dense_rows, int64_t n_dense_rows,
                      const int32_t *__restrict__ dense_cols, int64_t n_dense_cols, const float *__restrict__ sval,
                      const float *__restrict__ W, const float *__restrict__ H, float *__restrict__ P, int64_t M,
                      int64_t N, int K, int *dev_status)
{
    extern __shared__ __align__(1024) unsigned char smem[];
    float *Ct = reinterpret_cast<float *>(smem + (RUNS ? 2 * A_BUF_BYTES + STAGES * B_STAGE_BYTES : STAGES * STAGE_BYTES));
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2], a_empty[2];
    // runs form: what the MMA warp has to know about chunk g (written by producer thread 0 before its warp arrives on
    // the chunk's full barrier): bit 0 = W buffer of the chunk's cell, bit 1 = the run ends with this chunk
    __shared__ uint32_t cinfo[8];
    __shared__ MetaSlot meta[META_SLOTS];
    __shared__ uint32_t tmem_holder;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], N_PRODUCERS / 32);  // one arrival per producer warp, after all its lanes' stores
            mbar_init(&empty_bar[s], 1);           // one tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);            // one tcgen05.commit
            mbar_init(&acc_empty[b], N_EPILOGUE / 32);  // one arrival per epilogue warp, after its tcgen05.ld
            mbar_init(&a_empty[b], 1);             // one tcgen05.commit after a run's last MMA
        }
        mbar_fence_init();
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_holder)),
                     "n"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_holder;
    const int n_chunks = (K + KC - 1) / KC;
    bool ok = true;
    // The cells of this CTA: dealt one at a time, or (runs form) RUN_DEAL consecutive cells of the (row block,
    // column block)-ordered list at a time; cell_of(i) is the i-th of them.
    constexpr int DEAL = RUNS ? RUN_DEAL : 1;
    int my_cells = 0;
    {
        const int64_t n_deals = (n_cells + DEAL - 1) / DEAL;
        if ((int64_t)blockIdx.x < n_deals) {
            const int64_t mine = (n_deals - blockIdx.x + gridDim.x - 1) / gridDim.x;
            const int64_t last = blockIdx.x + (mine - 1) * gridDim.x;  // my last deal; the list's last deal may be short
            my_cells = (int)(mine * DEAL - (last == n_deals - 1 ? n_deals * DEAL - n_cells : 0));
        }
    }
    auto cell_of = [&](int i) -> int64_t { return ((int64_t)(i / DEAL) * gridDim.x + blockIdx.x) * DEAL + i % DEAL; };

    if (warp < MMA_WARP) {
        // ---------------- producers ----------------
        // The head tile of an operand is the raw fp32 data (the tensor core reads only the TF32 bits of an
        // element), so it is brought in by 16-byte cp.async copies, two chunks ahead and without holding a
        // register; the tail tile (x minus its TF32 head, exact) is computed from the head tile in shared memory.
        // Thread f owns bytes [16 f, 16 f + 16) of every tile, so it only ever reads what it copied itself.
        const unsigned total = (unsigned)my_cells * (unsigned)n_chunks;
        // the k group of this thread's pieces, f = tid + 256 i: piece f % 8 of row f / 8 holds group (f % 8) ^ (f / 8 % 8)
        const int kq = ((tid & 7) ^ ((tid >> 3) & 7)) * 4;
        // issue cursor: cell, chunk and this thread's operand rows of that cell
        int icell = 0;  // number of the cell within this CTA
        int ichunk = 0;
        // runs form: the W tile in shared memory belongs to (row0, compacted or not) = a_key; run_no counts the runs
        int64_t a_key = -1;
        int run_no = -1;
        unsigned carries_a = 0;  // two bits per chunk g % 4: the chunk brought its part of a W tile; into which buffer
        unsigned gi = 0;
        const float *wrow[4], *hrow[2];
        bool new_run = true;  // the cell at the issue cursor starts a run
        auto load_rows = [&]() {
            const DenseCell dc = cells[cell_of(icell)];
            const int cls = dc.cls & 0xff;
            if (RUNS) {
                const int64_t key = ((int64_t)dc.row0 << 1) | (cls == 0 ? 1 : 0);
                new_run = key != a_key;
                a_key = key;
                if (new_run) ++run_no;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int f = tid + i * N_PRODUCERS;
                int64_t row = (int64_t)dc.row0 + (f >> 3);
                if (cls == 0) row = row < n_dense_rows ? dense_rows[row] : M;  // compacted full rows
                wrow[i] = row < M ? W + row * K + kq : nullptr;
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int f = tid + i * N_PRODUCERS;
                int64_t col = (int64_t)dc.col0 + (f >> 3);
                if (cls == 1) col = col < n_dense_cols ? dense_cols[col] : N;  // compacted full columns
                hrow[i] = col < N ? H + col * K + kq : nullptr;
            }
        };
        auto issue = [&]() -> bool {  // copies of chunk gi into its stage; false on a timed-out wait
            if (gi < total) {
                if (ichunk == 0) load_rows();
                const unsigned s = gi % STAGES, use = gi / STAGES;
                // the MMAs of the stage's previous use are done; one decision per warp
                if (!wait_bar(&empty_bar[s], (use & 1u) ^ 1u)) return false;
                // runs form, first chunk of a run: so are the MMAs of the run that used this W buffer before
                if (RUNS && new_run && ichunk == 0 && run_no >= 2 && !wait_bar(&a_empty[run_no & 1], (((run_no >> 1) - 1) & 1u)))
                    return false;
                unsigned char *st_a = RUNS ? smem + (run_no & 1) * A_BUF_BYTES + ichunk * A_CHUNK_BYTES : smem + s * STAGE_BYTES;
                unsigned char *st_b = RUNS ? smem + 2 * A_BUF_BYTES + s * B_STAGE_BYTES : smem + s * STAGE_BYTES + 2 * A_TILE_BYTES;
                const int k0 = ichunk * KC;
                const bool in_k = k0 + kq < K;  // rows outside the matrix and k beyond K arrive as zeros
                if (!RUNS || new_run) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const bool v = in_k && wrow[i];
                        cp_async16_zfill(st_a + (tid + i * N_PRODUCERS) * 16, v ? (const void *)(wrow[i] + k0) : (const void *)W, v ? 16 : 0);
                    }
                }
                if (RUNS) {
                    carries_a = (carries_a & ~(3u << (2 * (gi & 3)))) | (((new_run ? 1u : 0u) | ((unsigned)(run_no & 1) << 1)) << (2 * (gi & 3)));
                    // bit 0: W buffer; bit 1 (set later, when the next cell is known): the run ends with this chunk
                    if (tid == 0) cinfo[gi & 7] = (unsigned)(run_no & 1);
                    // the last chunk of the cell before this one ended a run if this cell starts one
                    if (tid == 0 && ichunk == 0 && new_run && gi > 0) cinfo[(gi - 1) & 7] |= 2u;
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const bool v = in_k && hrow[i];
                    cp_async16_zfill(st_b + (tid + i * N_PRODUCERS) * 16, v ? (const void *)(hrow[i] + k0) : (const void *)H, v ? 16 : 0);
                }
                if (++ichunk == n_chunks) {
                    ichunk = 0;
                    ++icell;
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");  // an empty group past the end keeps the count uniform
            ++gi;
            return true;
        };
        ok = issue() && issue();
        for (unsigned g = 0; g < total && ok; ++g) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");  // this thread's copies of chunk g have landed
            const unsigned slot = (carries_a >> (2 * (g & 3))) & 3u;
            unsigned char *st_a = RUNS ? smem + (slot >> 1) * A_BUF_BYTES + (g % (unsigned)n_chunks) * A_CHUNK_BYTES
                                       : smem + (g % STAGES) * STAGE_BYTES;
            unsigned char *st_b = RUNS ? smem + 2 * A_BUF_BYTES + (g % STAGES) * B_STAGE_BYTES
                                       : smem + (g % STAGES) * STAGE_BYTES + 2 * A_TILE_BYTES;
            if (!RUNS || (slot & 1u)) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int off = (tid + i * N_PRODUCERS) * 16;
                    tail_store(*reinterpret_cast<const float4 *>(st_a + off), st_a + A_TILE_BYTES + off);
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int off = (tid + i * N_PRODUCERS) * 16;
                tail_store(*reinterpret_cast<const float4 *>(st_b + off), st_b + B_TILE_BYTES + off);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // my copies and stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[g % STAGES]);
            // only now the copies of chunk g + 2: they need the stage of chunk g - 1, whose MMAs ran meanwhile
            if (!issue()) { ok = false; break; }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (warp == MMA_WARP) {
        // ---------------- MMA issue: the whole warp walks the loop, lane 0 issues ----------------
        unsigned g = 0, n_acc = 0;
        for (int i = 0; i < my_cells && ok; ++i) {
            const unsigned b = n_acc & 1u, use = n_acc >> 1;
            // the epilogue has read this accumulator
            if (!wait_bar(&acc_empty[b], (use & 1u) ^ 1u)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t d = tmem + b * DC;
            for (int c = 0; c < n_chunks; ++c) {
                const unsigned s = g % STAGES;
                if (!wait_bar(&full_bar[s], (g / STAGES) & 1u)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
                    const unsigned info = RUNS ? cinfo[g & 7] : 0u;
                    const uint32_t a_hi = RUNS ? smem_u32(smem + (info & 1u) * A_BUF_BYTES + c * A_CHUNK_BYTES) : smem_u32(smem + s * STAGE_BYTES);
                    const uint32_t a_lo = a_hi + A_TILE_BYTES;
                    const uint32_t b_hi = RUNS ? smem_u32(smem + 2 * A_BUF_BYTES + s * B_STAGE_BYTES) : a_hi + 2 * A_TILE_BYTES;
                    const uint32_t b_lo = b_hi + B_TILE_BYTES;
#pragma unroll
                    for (int ks = 0; ks < KC / 8; ++ks) {
                        const uint32_t o = ks * 32;  // eight k = 32 bytes of every row per instruction
                        const uint64_t dah = smem_desc(a_hi + o, LBO, SBO), dal = smem_desc(a_lo + o, LBO, SBO);
                        const uint64_t dbh = smem_desc(b_hi + o, LBO, SBO), dbl = smem_desc(b_lo + o, LBO, SBO);
                        mma_tf32_ss(d, dal, dbh, (c > 0 || ks > 0) ? 1u : 0u);  // a cell's very first MMA overwrites
                        mma_tf32_ss(d, dah, dbl, 1u);
                        mma_tf32_ss(d, dah, dbh, 1u);
                    }
                    // arrives when the MMAs issued so far have finished reading the stage
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                     smem_u32(&empty_bar[s]))
                                 : "memory");
                    // runs form: the run's W buffer is free once its last MMAs are done
                    if (RUNS && (info & 2u))
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                         smem_u32(&a_empty[info & 1u]))
                                     : "memory");
                }
                __syncwarp();
                ++g;
            }
            if (!ok) break;
            if (lane == 0)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 smem_u32(&acc_full[b]))
                             : "memory");
            __syncwarp();
            ++n_acc;
        }
    } else {
        // ---------------- epilogue ----------------
        // Sixteen warps.  Warp ew reads TMEM lanes 32 (warp % 4) .., columns 16 (ew / 4) .. + 16 of the finished
        // block and parks them; it then picks the block's rows 8 ew .. 8 ew + 7.  What does not depend on the product
        // runs ahead of it: a cell's row masks and base indices come into shared memory two cells early
        // (cp.async), its S values into registers one cell early.
        const int et = tid - EPI_WARP0 * 32;  // 0 .. 511
        const int ew = et >> 5;               // epilogue warp 0 .. 15
        const int quarter = warp & 3, cgroup = ew >> 2;
        const int row = quarter * 32 + lane;
        const unsigned below = (1u << lane) - 1u;
        // metadata of cell i of this CTA -> ring slot i % META_SLOTS, by 16-byte cp.async (97 threads take part)
        auto fetch_meta = [&](int i) {
            if (i < my_cells) {
                const int64_t c = cell_of(i);
                MetaSlot &m = meta[i % META_SLOTS];
                if (et < 64) cp_async16_zfill(&m.mask[et * 2], row_mask + c * DR + et * 2, 16);
                else if (et < 96) cp_async16_zfill(&m.base[(et - 64) * 4], row_base + c * DR + (et - 64) * 4, 16);
                else if (et == 96)
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(&m.cls)), "l"(&cells[c].cls) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        // S values of this warp's rows of cell i (row-mask form): lane l takes the columns l and l + 32 of a row; the
        // nonzero in column c sits at base + popc(mask below bit c)
        auto load_s = [&](int i, float (&s_lo)[8], float (&s_hi)[8]) {
            const MetaSlot &m = meta[i % META_SLOTS];
            const bool on = i < my_cells && (m.cls & 0x100) != 0 && sval != nullptr;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                s_lo[u] = s_hi[u] = 1.f;
                if (on) {
                    const unsigned long long mk = m.mask[ew * 8 + u];
                    const unsigned lo = (unsigned)mk, hi = (unsigned)(mk >> 32);
                    const int32_t bs = m.base[ew * 8 + u];
                    if ((lo >> lane) & 1u) s_lo[u] = __ldg(sval + bs + __popc(lo & below));
                    if ((hi >> lane) & 1u) s_hi[u] = __ldg(sval + bs + __popc(lo) + __popc(hi & below));
                }
            }
        };
        fetch_meta(0);
        fetch_meta(1);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        epilogue_sync();
        float s_lo[8], s_hi[8];
        load_s(0, s_lo, s_hi);
        unsigned n_acc = 0;
        for (int i = 0; i < my_cells; ++i) {
            const int64_t cell = cell_of(i);
            const MetaSlot &m = meta[i % META_SLOTS];
            const bool masked = (m.cls & 0x100) != 0;
            // two cells ahead: metadata; one cell ahead: S values -- neither depends on the product
            fetch_meta(i + 2);
            float n_lo[8], n_hi[8];
            load_s(i + 1, n_lo, n_hi);
            const unsigned b = n_acc & 1u;
            ok = epilogue_all(wait_bar(&acc_full[b], (n_acc >> 1) & 1u));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            {
                uint32_t v[16];
                const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + b * DC + cgroup * 16;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[b]);  // the accumulator may be overwritten: the next cell's MMAs run during the pick
                float *crow = Ct + row * CT_STRIDE + cgroup * 16;
#pragma unroll
                for (int c = 0; c < 16; c += 4)
                    *reinterpret_cast<float4 *>(crow + c) = make_float4(__uint_as_float(v[c]), __uint_as_float(v[c + 1]),
                                                                        __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
            }
            epilogue_sync();  // the block is parked
            if (masked) {
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const unsigned long long mk = m.mask[ew * 8 + u];
                    const unsigned lo = (unsigned)mk, hi = (unsigned)(mk >> 32);
                    const int32_t bs = m.base[ew * 8 + u];
                    const float *cr = Ct + (ew * 8 + u) * CT_STRIDE;
                    if ((lo >> lane) & 1u) P[bs + __popc(lo & below)] = cr[lane] * s_lo[u];
                    if ((hi >> lane) & 1u) P[bs + __popc(lo) + __popc(hi & below)] = cr[lane + 32] * s_hi[u];
                }
            } else {
                // per-nonzero lists, eight nonzeros per thread and trip, the loads of a trip grouped by dependency
                // level (codes and indices, then S values)
                const DenseCell dc = cells[cell];
                const int32_t *cidx = idx + dc.offset;
                const uint16_t *crc = rc + dc.offset;
                for (int i0 = 0; i0 < dc.count; i0 += 8 * N_EPILOGUE) {
                    unsigned code[8];
                    int32_t o[8];
                    float sv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int j = i0 + et + u * N_EPILOGUE;
                        code[u] = j < dc.count ? (unsigned)__ldcs(crc + j) : 0u;
                        o[u] = j < dc.count ? __ldcs(cidx + j) : -1;
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) sv[u] = (sval && o[u] >= 0) ? __ldg(sval + o[u]) : 1.f;
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (o[u] >= 0) P[o[u]] = Ct[(code[u] >> 8) * CT_STRIDE + (code[u] & 255u)] * sv[u];
                }
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");  // the metadata fetched at the top of this iteration
            epilogue_sync();  // ... is visible to everybody; and the next cell's block may overwrite this one
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                s_lo[u] = n_lo[u];
                s_hi[u] = n_hi[u];
            }
            ++n_acc;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    if (!ok && lane == 0) atomicExch(dev_status, (int)DEV_MBARRIER_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == MMA_WARP)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(TMEM_COLS) : "memory");
}

}  // namespace

cudaError_t launch_dense_cells_tc(const DenseCell *cells, int64_t n_cells, const int32_t *idx, const uint16_t *rc,
                                  const unsigned long long *row_mask, const int32_t *row_base, const int32_t *dense_rows,
                                  int64_t n_dense_rows, const int32_t *dense_cols, int64_t n_dense_cols, const float *sval,
                                  const float *W, const float *H, float *P, int64_t M, int64_t N, int K, int sm_count,
                                  int *dev_status, cudaStream_t stream)
{
    if (n_cells == 0) return cudaSuccess;
    int64_t blocks = sm_count;  // one persistent CTA per SM
    if (blocks > n_cells) blocks = n_cells;
    // K <= 64: the runs form (the W tile of a row block stays in shared memory across its cells), unless most cells
    // are cells of compacted full rows / columns -- their operands are shared by thousands of cells and sit in L2, the
    // staging is not what limits them, and the general form measures faster there (202 M-nonzero attention mask with
    // 1,311 global rows and columns: 0.839 ms against 0.874 ms; 80 global: 0.246 ms against 0.227 ms).
    // SDDMM_DENSE_RUNS=0 / 1 forces the general / the runs form.
    const char *runs_str = getenv("SDDMM_DENSE_RUNS");
    const int runs_env = runs_str ? atoi(runs_str) : -1;
    const int64_t compacted = ((n_dense_rows + DR - 1) / DR) * ((N + DC - 1) / DC) + ((n_dense_cols + DC - 1) / DC) * ((M + DR - 1) / DR);
    const bool runs = runs_env >= 0 ? runs_env != 0 : 2 * compacted < n_cells;
    if (K <= 2 * KC && runs) {
        static SmemOptinCache optin_runs;  // per device
        cudaError_t e = optin_dynamic_smem(sddmm_dense_tc_kernel<true>, RUNS_SMEM_BYTES, optin_runs);
        if (e != cudaSuccess) return e;
        sddmm_dense_tc_kernel<true><<<(unsigned)blocks, TC_THREADS, RUNS_SMEM_BYTES, stream>>>(
            cells, n_cells, idx, rc, row_mask, row_base, dense_rows, n_dense_rows, dense_cols, n_dense_cols, sval, W, H, P, M,
            N, K, dev_status);
        return cudaGetLastError();
    }
    static SmemOptinCache optin;  // per device
    {
        cudaError_t e = optin_dynamic_smem(sddmm_dense_tc_kernel<false>, TC_SMEM_BYTES, optin);
        if (e != cudaSuccess) return e;
    }
    sddmm_dense_tc_kernel<false><<<(unsigned)blocks, TC_THREADS, TC_SMEM_BYTES, stream>>>(
        cells, n_cells, idx, rc, row_mask, row_base, dense_rows, n_dense_rows, dense_cols, n_dense_cols, sval, W, H, P, M, N,
        K, dev_status);
    return cudaGetLastError();
}

}  // namespace sddmm
