/*
 * sddmm_b200 -- C ABI of the B200 (sm_100a) SDDMM engine.
 *
 *     P[i] = ( sum_{t<K} W[row_i*K + t] * H[col_i*K + t] ) [ * S.val_i ]
 *
 * for every nonzero i of a row-sorted sparse matrix S (M x N, COO, 0-based
 * int32 indices), W (M x K) and H (N x K) dense, row-major, fp32.  P is returned
 * in the order of the input nonzeros.
 *
 * Every entry point is a drop-in for one piece of the reference program
 * (isratnisa/SDDMM_GPU); the piece is cited above each declaration by its path
 * inside that project.  Plain pointers and sizes only: no C++ types cross this
 * boundary, nothing throws or aborts, every function returns a status code.
 *
 * A handle is bound to one CUDA device and is used by one host thread at a time
 * (the reference is single-threaded, HiPC18/src/sddmm.cu:32-151).  For several
 * GPUs run one handle per device (one process per GPU) and split S with
 * sddmm_partition_rows().
 */
#ifndef SDDMM_B200_H
#define SDDMM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SDDMM_API __attribute__((visibility("default")))

/* ---- status codes -------------------------------------------------------- */
enum {
    SDDMM_OK = 0,
    SDDMM_INVALID_ARG = 1,        /* NULL pointer, negative size, bad flag        */
    SDDMM_UNSORTED_INPUT = 2,     /* rows[] not non-decreasing                     */
    SDDMM_INDEX_OUT_OF_RANGE = 3, /* a row >= M or col >= N or negative index      */
    SDDMM_K_UNSUPPORTED = 4,      /* K <= 0, K % 4 != 0 or K > SDDMM_MAX_K         */
    SDDMM_CUDA_ERROR = 5,         /* see sddmm_last_error()                        */
    SDDMM_NCCL_ERROR = 6,
    SDDMM_OUT_OF_MEMORY = 7,
    SDDMM_DEVICE_TIMEOUT = 8,     /* a bounded device-side wait gave up            */
    SDDMM_IO_ERROR = 9,           /* file missing / unreadable / unwritable        */
    SDDMM_PARSE_ERROR = 10,       /* malformed Matrix Market text                  */
    SDDMM_NO_DEVICE = 11          /* no CUDA device: there is no CPU fallback      */
};

#define SDDMM_MAX_K 4096

/* ---- execute flags ------------------------------------------------------- */
#define SDDMM_FLAG_ASYNC        0x1u /* return after enqueue on the handle's stream (device pointers only) */
#define SDDMM_FLAG_TILED_ORDER  0x2u /* P in the plan's tiled order (what the reference's sddmm_GPU leaves in d_val, sddmm.cu:119) instead of input order */
#define SDDMM_FLAG_H_TRANSPOSED  0x4u /* H is given K-major, H_t[t*N + c] -- the layout make_HTasH builds (util.h:68-73) -- and is transposed on the device first */
#define SDDMM_FLAG_W_TRANSPOSED  0x8u /* W is given K-major, W_t[t*M + r] */
#define SDDMM_FLAG_KERNEL_GATHER 0x10u /* force the planless gather kernel */
#define SDDMM_FLAG_KERNEL_PANEL  0x20u /* force the TMA-staged row-panel kernel */
#define SDDMM_FLAG_KERNEL_RING   0x40u /* force the shared-memory gather-ring kernels (K = 32, 64, 128, 256, 512 or 1024) */

#define SDDMM_FLAG_OPERANDS_BF16 0x100u /* W and H point to bfloat16 arrays (row-major, 2 bytes per element; K = 256, 512,
                                          1024 or 2048); products and sums stay fp32.  Opt-in, outside the fp32 tolerance
                                          contract (operands carry 8 bits of mantissa); halves the bytes of every gather.
                                          Device arrays only; no counterpart in the reference, whose operands are fp32
                                          (HiPC18/src/sddmm.cu:32) */

/* ---- plan flags ---------------------------------------------------------- */
#define SDDMM_PLAN_SKIP_VALIDATION 0x1u /* trust sortedness and bounds (the reference checks neither) */
#define SDDMM_PLAN_DEVICE_INDICES  0x2u /* rows/cols are device pointers on the handle's device */
#define SDDMM_PLAN_FORCE_H_CHUNKS  0x4u /* sddmm_dist_plan_coo: build and use the column-bucketed form even with a single rank (exercises the overlapped execute on one GPU; the broadcasts are no-ops) */

typedef struct sddmm_handle_s *sddmm_handle_t;
typedef struct sddmm_plan_s *sddmm_plan_t;

/* Human-readable name of a status code (static storage). */
SDDMM_API const char *sddmm_status_string(int status);

/*
 * Replaces the implicit "device 0, fresh allocations and streams on every call"
 * set-up of sddmm_GPU (HiPC18/src/sddmm.cu:38-46,78-84).  Creates the compute
 * stream and the timing events once.  SDDMM_NO_DEVICE when no GPU is usable.
 */
SDDMM_API int sddmm_create(sddmm_handle_t *out, int device);
SDDMM_API int sddmm_destroy(sddmm_handle_t h);

/* Text of the last CUDA / parse error seen through this handle ("" if none). */
SDDMM_API const char *sddmm_last_error(sddmm_handle_t h);

/*
 * Run on a caller-owned CUDA stream (a cudaStream_t passed as void*) instead of
 * the handle's own; NULL restores the handle's stream (to launch on the legacy
 * default stream pass cudaStreamLegacy, not 0).  The reference launches on its
 * private stream[0] (sddmm.cu:81-84,102).
 */
SDDMM_API int sddmm_set_stream(sddmm_handle_t h, void *cuda_stream);

/*
 * Replaces make_CSR (HiPC18/src/util.h:131-153), the TiledMatrix constructor
 * (util.h:52-65), rewrite_matrix_1D (util.h:267-343) and the index uploads of
 * sddmm_GPU (sddmm.cu:41-64): validates the row-sorted COO (unless told not to),
 * copies the indices to the device once and runs the GPU binning pass (row
 * pointer over ALL rows -- empty rows are fine -- row-panel work items, and, when
 * col_tile_hint < N, the column-tile permutation).
 *
 *   panel_rows_hint : the CLI's argv[3] (rows of W per shared-memory panel,
 *                     "tile_sizeY"/actv_row_size in the reference, sddmm.cu:253-255);
 *                     clamped to what fits the sm_100a shared memory for this K;
 *                     <= 0 lets the engine choose.
 *   col_tile_hint   : the CLI's argv[4] (column-tile width, "tile_sizeX",
 *                     sddmm.cu:254); >= N or <= 0 means a single column tile,
 *                     i.e. the identity permutation.
 * The plan is reusable for any number of sddmm_execute() calls.
 */
SDDMM_API int sddmm_plan_coo(sddmm_handle_t h, int64_t M, int64_t N, int64_t nnz,
                             const int32_t *rows, const int32_t *cols, int K,
                             int panel_rows_hint, int col_tile_hint, uint32_t flags,
                             sddmm_plan_t *out);
SDDMM_API int sddmm_destroy_plan(sddmm_plan_t p);

/*
 * Replaces the W/H uploads, cudaMemset, launch loop and result download of
 * sddmm_GPU (HiPC18/src/sddmm.cu:53,71-73,93-119) and the kernel comp_kernel_COO
 * (HiPC18/src/kernel.h:2-52) -- one launch, no K-slicing.
 *
 *   W, H, P : host or device pointers (detected); host buffers are copied
 *             through plan-owned device staging inside the call.  With W in
 *             host memory and a large matrix (256 MB of W or more, a million
 *             nonzeros or more, ring-kernel K, single column tile) the call is
 *             pipelined: H first, then W rows and S values in up to 16 chunks of
 *             consecutive nonzeros, every chunk's kernel and the download of
 *             its part of P running behind the uploads of the later chunks on
 *             two internal streams; W rows that no nonzero touches between two
 *             chunks are not uploaded.  Results are bit-identical to the
 *             unpipelined call (SDDMM_PIPELINE=0 in the environment at
 *             sddmm_create() switches the pipeline off).  Pinned host buffers
 *             are needed for the copies to overlap.  In a pipelined call, W
 *             and H buffers that are page-locked and mapped (cudaHostAlloc,
 *             cudaHostRegister) are not copied whole: a kernel reads, over
 *             PCIe, exactly the rows of W and H that some nonzero touches (the
 *             reference uploads both arrays whole, sddmm.cu:71-73);
 *             SDDMM_SPARSE_UPLOAD=0 at sddmm_create() keeps cudaMemcpy.
 *   Sval    : NULL -> the unscaled dot product, as sddmm_CPU_COO and the
 *             reference kernel store it (sddmm.cu:192, kernel.h:48);
 *             else P[i] *= Sval[i], as sddmm_CPU_CSR does (sddmm.cu:171).
 * Synchronous unless SDDMM_FLAG_ASYNC (the reference waits on its stop event,
 * sddmm.cu:110).
 */
SDDMM_API int sddmm_execute(sddmm_plan_t p, const float *W, const float *H,
                            const float *Sval, float *P, uint32_t flags);

/*
 * The step after SDDMM in its callers (the reference stops at SDDMM; its README names SDDMM "a
 * core component in reformulations of many machine learning algorithms", README.md:1 -- there
 * the sampled product is multiplied straight back into a dense factor).  No counterpart in the
 * reference: parity is pinned to a CPU loop of the same definition, not to reference code.
 *
 *   sddmm_spmm_execute : Y[r, :] = sum over the nonzeros i of row r of Pval[i] * H[col_i, :]
 *                        (Pval NULL: all ones).  Y is M x K, every row written (empty rows: 0).
 *   sddmm_fused_execute: the same with Pval[i] = (sum_t W[r,t] H[col_i,t]) * Sval[i] computed on
 *                        the fly (Sval NULL: unscaled) -- P never goes to memory and every H row
 *                        is gathered once for both uses; P_out != NULL also stores P (input order).
 * K a multiple of 4 up to 1024 (SDDMM_K_UNSUPPORTED otherwise).  Pointers host or device (host
 * arrays are staged for the call); flags: 0 or SDDMM_FLAG_ASYNC (device pointers only).  Rows
 * are processed whole by one warp, long rows in pieces that are added in a fixed order: the
 * result does not depend on scheduling.  Works on the plan's input order (column tiles of the
 * plan are not used).  sddmm_last_kernel_ms() reports the kernels' time.
 */
SDDMM_API int sddmm_spmm_execute(sddmm_plan_t p, const float *Pval, const float *H, float *Y, uint32_t flags);
SDDMM_API int sddmm_fused_execute(sddmm_plan_t p, const float *W, const float *H, const float *Sval,
                                  float *P_out, float *Y, uint32_t flags);

/* Milliseconds of the kernels of the last synchronous sddmm_execute(), measured
 * with CUDA events on the compute stream -- the region the reference times and
 * prints as "Time for SDDMM with K = ..." (sddmm.cu:93,109-114).  For a pipelined
 * call (see sddmm_execute) it is the sum over the chunks' kernels; the waits for
 * uploads between them are not counted. */
SDDMM_API int sddmm_last_kernel_ms(sddmm_plan_t p, float *ms);

/* Which kernels the last sddmm_execute() on this plan launched: "ring", "ring_small",
 * "panel", "gather", "dense_tc+ring_small", ... (static storage).  The reference has one
 * kernel, comp_kernel_COO (HiPC18/src/kernel.h:2), and nothing to report. */
SDDMM_API const char *sddmm_last_kernel_name(sddmm_plan_t p);

/* Number of kernels sddmm_execute() and sddmm_upload_rows() have launched through this
 * handle since it was created (SDDMM kernels, row uploads, operand transpositions; plan-time
 * kernels are not counted).  The reference launches n_col_tiles * K/k_slice kernels per call
 * (HiPC18/src/sddmm.cu:95-108). */
SDDMM_API int sddmm_kernel_launches(sddmm_handle_t h, int64_t *n);

/*
 * Wait for everything enqueued on the handle's stream and report the device
 * status word: SDDMM_DEVICE_TIMEOUT if a bounded device-side wait of any earlier
 * call gave up -- the way to learn the outcome of SDDMM_FLAG_ASYNC calls.  The
 * reference's equivalent is cudaEventSynchronize(stop) (HiPC18/src/sddmm.cu:110).
 */
SDDMM_API int sddmm_sync(sddmm_handle_t h);

/*
 * Self-check of a result on the device: every stride-th nonzero is recomputed in
 * float64 and compared per nonzero with |P - ref| <= tol * max(|ref|, A),
 * A = sum_t |w_t h_t| (|s|).  W, H, Sval (or NULL) and P as passed to
 * sddmm_execute(): host or device arrays (host arrays are staged for the call).  Counterpart: the reference's in-line comparison of
 * the GPU result with its CPU result (HiPC18_mpi/sddmm.cu:318-334; absolute 1e-4).
 * Any of the three outputs may be NULL.
 */
SDDMM_API int sddmm_check_result(sddmm_plan_t p, const float *W, const float *H, const float *Sval,
                                 const float *P, int64_t stride, double tol, double *max_scaled_err,
                                 int64_t *n_checked, int64_t *n_bad);

/* Host-only self-test (no GPU needed): the per-kernel cache of shared-memory
 * opt-ins is keyed by device ordinal, so a second GPU in the same process makes
 * its own opt-in.  No counterpart in the reference (one GPU, static shared memory). */
SDDMM_API int sddmm_selftest_optin_cache(void);

/*
 * The rows of W (which = 0) or of H (which = 1) that an SDDMM over this plan
 * reads: ascending ids of the rows / columns of S that hold at least one
 * nonzero, as a device array owned by the plan (valid until the plan is
 * destroyed), built on first request.  Together with sddmm_upload_rows this
 * replaces the whole-array uploads of sddmm_GPU (HiPC18/src/sddmm.cu:71-73) for
 * callers that stage the operands themselves (e.g. one process per GPU).
 */
SDDMM_API int sddmm_plan_used_lines(sddmm_plan_t p, int which, const int32_t **d_ids, int64_t *n);

/*
 * Copy the listed rows of a row-major fp32 array with K columns from
 * page-locked, mapped host memory (cudaHostAlloc / cudaHostRegister) to the same
 * rows of a device array; a kernel reads the host rows over PCIe, so rows that
 * are not listed do not travel.  Stream-ordered on cuda_stream (a cudaStream_t
 * as void*; NULL = the handle's stream); returns after enqueueing.
 * SDDMM_INVALID_ARG when `host` is not mapped page-locked memory (nothing is
 * launched).  Counterpart in the reference: the cudaMemcpy of W and H
 * (sddmm.cu:71-73).
 */
SDDMM_API int sddmm_upload_rows(sddmm_handle_t h, const float *host, float *dev, const int32_t *d_row_ids,
                                int64_t n_rows, int K, void *cuda_stream);

/* Bytes the last sddmm_execute() moved host -> device and device -> host (0 for
 * operands that were already on the device).  The reference moves
 * 4K(M+N) + 12 nnz up and 4 nnz down on every call (sddmm.cu:50-73,119). */
SDDMM_API int sddmm_last_transfer_bytes(sddmm_plan_t p, int64_t *h2d_bytes, int64_t *d2h_bytes);

/*
 * One-shot form with the shape of the reference's sddmm_GPU(S, tS, P, W, H)
 * (HiPC18/src/sddmm.cu:32): all pointers host or device, nothing is kept between
 * calls, no plan.  Uses the planless gather kernel.
 */
SDDMM_API int sddmm_coo(sddmm_handle_t h, int64_t M, int64_t N, int64_t nnz,
                        const int32_t *rows, const int32_t *cols, const float *Sval,
                        const float *W, const float *H, int K, float *P);

/*
 * Self-test of the failure path (no counterpart in the reference, whose waits
 * are unbounded): launches one warp that waits, with a short poll limit, on a
 * barrier nothing arrives on.  The warp gives up after a few milliseconds and
 * the call returns SDDMM_DEVICE_TIMEOUT -- the status a real kernel reports when
 * one of its bounded waits runs out.  Nothing faults or hangs; the handle stays
 * usable.
 */
SDDMM_API int sddmm_selftest_wait_timeout(sddmm_handle_t h);

/* Sizes of what the binning pass built (test and reporting hook). */
typedef struct {
    int64_t M, N, nnz;
    int32_t K;
    int32_t panel_rows;     /* rows of W per staged panel actually used        */
    int32_t col_tile;       /* column-tile width actually used (N if single)   */
    int32_t n_col_tiles;
    int64_t n_work_items;
    int64_t n_nonempty_rows;
    int64_t n_nonempty_cols; /* -1 unless computed (sddmm_plan_count_cols)     */
    int64_t device_bytes;   /* device memory the plan owns                     */
    float plan_ms;          /* device time of the binning pass                 */
    int32_t reserved0;
    int64_t n_dense_cells;  /* 128 x 64 cells handed to the dense-cell kernel  */
    int64_t n_dense_nnz;    /* nonzeros inside them                            */
    int64_t n_hub_cols;     /* columns marked for L2 residency (ring kernel)   */
} sddmm_plan_info;
SDDMM_API int sddmm_plan_get_info(sddmm_plan_t p, sddmm_plan_info *info);

/* Number of distinct columns of S (N_nz of the algorithmic-bytes formula);
 * computed on the device on request and cached in the plan. */
SDDMM_API int sddmm_plan_count_cols(sddmm_plan_t p, int64_t *n_nonempty_cols);

/*
 * The same count for callers that may not allocate device memory (no
 * counterpart in the reference: it allocates and frees on every call).
 *
 * Meant for hosts that cannot enter the CUDA allocator: a process whose
 * framework already owns all device memory, a loop that cannot take the
 * device-wide synchronisation cudaMalloc/cudaFree imply, a plug-in running
 * inside another library's callback.  This entry point calls no cudaMalloc,
 * cudaFree or other allocating routine and needs no handle or plan: its scratch
 * (one mark per column plus a counter) is a fixed array inside the library image,
 * SDDMM_NOALLOC_SCRATCH_BYTES per GPU that loads the library, held until exit.
 *
 *   device   : CUDA device that owns d_cols; made current by the call.
 *   d_cols   : nnz column indices in device memory (any order); indices outside
 *              [0, N) are ignored.
 *   N        : number of columns; N > SDDMM_NOALLOC_MAX_COLS is rejected with
 *              SDDMM_INVALID_ARG and a message in errbuf (use
 *              sddmm_plan_count_cols for larger matrices).
 *   cuda_stream : cudaStream_t to run on (NULL = the default stream); the call
 *              returns after the count has been copied back, i.e. it waits for
 *              the stream, and is refused (SDDMM_INVALID_ARG) on a stream that
 *              is being captured.
 * The first call on each device also looks up the scratch array's device address;
 * make that first call outside any stream capture.  All calls on a device share
 * the scratch, which keeps the previous call's contents: every call clears what
 * it uses before it starts, and calls that overlap on one GPU (two streams or two
 * threads at once) race with each other -- serialise them.
 */
#define SDDMM_NOALLOC_MAX_COLS (8 * 1024 * 1024)
#define SDDMM_NOALLOC_SCRATCH_BYTES (SDDMM_NOALLOC_MAX_COLS + 256)
SDDMM_API int sddmm_count_cols_noalloc(int device, const int32_t *d_cols, int64_t nnz, int64_t N,
                                       void *cuda_stream, int64_t *n_nonempty_cols, char *errbuf,
                                       int errbuf_len);

/* Row pointer over all M rows (M + 1 int64 entries, host buffer), the GPU
 * replacement of make_CSR's row_ptr/row_holder pair (util.h:131-153). */
SDDMM_API int sddmm_plan_export_row_ptr(sddmm_plan_t p, int64_t *row_ptr);

/*
 * Test hook: the tables rewrite_matrix_1D (HiPC18/src/util.h:267-343) would
 * produce for the same (panel_rows, col_tile), computed by the GPU binning pass,
 * in the reference's layout and sizes (TiledMatrix constructor, util.h:52-65):
 *   t_rows, t_cols, tiled_ind : nnz each
 *   lastIdx_tile              : ntile_c + 1,              ntile_c = N/col_tile + 1
 *   lastIdx_block_tile        : (ntile_c + 1) * max_blk,  max_blk = M/panel_rows + 1
 *   active_row                : M * ntile_c
 *   n_actv_row                : ntile_c
 * All host buffers; any of them may be NULL to skip it.  panel_rows/col_tile are
 * the CLI's argv[3]/argv[4] taken literally (not clamped).
 */
SDDMM_API int sddmm_plan_export_tiling(sddmm_plan_t p, int panel_rows, int col_tile,
                                       int32_t *t_rows, int32_t *t_cols,
                                       int32_t *tiled_ind, int32_t *lastIdx_tile,
                                       int32_t *lastIdx_block_tile, int32_t *active_row,
                                       int32_t *n_actv_row, int32_t *max_active_row);

/*
 * Replaces the nnz-balanced cuts of make_CSC (HiPC18_mpi/util.h:100-135), over
 * ROWS instead of columns: cuts[g] .. cuts[g+1] is the row range of part g
 * (n_parts + 1 entries, cuts[0] = 0, cuts[n_parts] = M), each cut the first
 * multiple of align_rows whose prefix holds >= g*nnz/n_parts nonzeros.
 * nnz_cuts (n_parts + 1) receives the matching nonzero offsets.  Pure host code.
 */
SDDMM_API int sddmm_partition_rows(int64_t M, int64_t nnz, const int32_t *rows,
                                   int n_parts, int align_rows, int64_t *cuts,
                                   int64_t *nnz_cuts);

/*
 * The same cuts with a cost model instead of plain nonzero counts: a prefix
 * costs its nonzeros plus row_cost per non-empty row (a row of S costs one W row
 * however few nonzeros it has, so blocks of short rows are more expensive per
 * nonzero than blocks of long ones).  row_cost = 0 gives sddmm_partition_rows.
 * No counterpart in the reference beyond make_CSC's plain nnz balance.
 */
SDDMM_API int sddmm_partition_rows_weighted(int64_t M, int64_t nnz, const int32_t *rows, int n_parts,
                                            int align_rows, double row_cost, int64_t *cuts,
                                            int64_t *nnz_cuts);

/*
 * The same cuts for unequal parts: part g is to hold shares[g] / sum(shares) of the nonzeros
 * (shares NULL = equal parts = sddmm_partition_rows).  For row blocks that cost a different
 * time per nonzero on different GPUs -- e.g. shares proportional to each rank's measured
 * nonzeros per millisecond.  make_CSC has equal parts only (HiPC18_mpi/util.h:104).
 */
SDDMM_API int sddmm_partition_rows_shares(int64_t M, int64_t nnz, const int32_t *rows, int n_parts,
                                          int align_rows, const double *shares, int64_t *cuts,
                                          int64_t *nnz_cuts);

/* ---- several GPUs ---------------------------------------------------------------
 *
 * Replaces the MPI program of the reference (HiPC18_mpi/sddmm.cu:139-351, launched as
 * `mpiexec -n P -ppn 1 sddmm ...`, HiPC18_mpi/scripts/run_mpi.sh:14-22), which
 * partitions by columns in make_CSC (HiPC18_mpi/util.h:100-135), uploads all of W and H
 * on every rank (HiPC18_mpi/sddmm.cu:281-284) and uses MPI for barriers only.  Here a
 * rank owns an nnz-balanced block of consecutive ROWS (sddmm_partition_rows) and H
 * travels over NCCL (NVLink / NVSwitch) into every GPU's own memory.  NCCL is bound at
 * run time; without it these entry points return SDDMM_NCCL_ERROR and the
 * single-GPU ones are unaffected.
 *
 * Two forms: (1) one rank per process (or thread): sddmm_comm_* + sddmm_dist_*; the
 * caller carries the 128-byte id from rank 0 to the others (any channel: a file, a
 * socket, MPI, torch.distributed) as ncclGetUniqueId / ncclCommInitRank ask;
 * (2) one process driving all GPUs from host arrays: sddmm_multi_*.
 */
#define SDDMM_COMM_ID_BYTES 128
typedef struct sddmm_comm_s *sddmm_comm_t;
typedef struct sddmm_dist_plan_s *sddmm_dist_plan_t;

/* Fills id[SDDMM_COMM_ID_BYTES] (ncclGetUniqueId); call on one rank, hand the bytes to all. */
SDDMM_API int sddmm_comm_unique_id(void *id);
/* Joins the communicator on the handle's GPU (ncclCommInitRank; returns when all `world`
 * ranks have called).  Owns a communication stream next to the handle's compute stream. */
SDDMM_API int sddmm_comm_create(sddmm_handle_t h, const void *id, int rank, int world, sddmm_comm_t *out);
SDDMM_API int sddmm_comm_destroy(sddmm_comm_t c);
/* buf (count floats, device memory on every rank) <- root's buf; stream-ordered on
 * cuda_stream (NULL: the handle's stream).  The reference has no collective. */
SDDMM_API int sddmm_comm_broadcast(sddmm_comm_t c, float *buf, int64_t count, int root, void *cuda_stream);
/* In place: rank r holds floats [r * count_per_rank, (r+1) * count_per_rank) of buf;
 * afterwards every rank holds all world * count_per_rank (ncclAllGather). */
SDDMM_API int sddmm_comm_all_gather(sddmm_comm_t c, float *buf, int64_t count_per_rank, void *cuda_stream);

/*
 * This rank's part of a plan over the WHOLE matrix (every rank passes the same row-sorted
 * pattern, as every MPI rank of the reference parses the same file): rows are cut with
 * sddmm_partition_rows (32-row alignment), the rank's block is planned like
 * sddmm_plan_coo, and -- when h_chunks > 1 -- a second, column-bucketed plan is built
 * for the execute that overlaps the H broadcast (h_chunks column ranges of S = blocks of
 * consecutive rows of H).  flags: SDDMM_PLAN_*; with SDDMM_PLAN_DEVICE_INDICES rows and
 * cols are device arrays (borrowed for the life of the plan).
 */
SDDMM_API int sddmm_dist_plan_coo(sddmm_comm_t c, int64_t M, int64_t N, int64_t nnz, const int32_t *rows,
                                  const int32_t *cols, int K, int panel_rows_hint, int h_chunks, uint32_t flags,
                                  sddmm_dist_plan_t *out);
/* The same with unequal row blocks: rank r is given rank_shares[r] / sum of the nonzeros
 * (world entries, identical on every rank; NULL = equal).  Re-plan with shares proportional to
 * each rank's measured nonzeros per millisecond to even out blocks whose nonzeros cost
 * different times (short rows cost more per nonzero than long ones). */
SDDMM_API int sddmm_dist_plan_coo_shares(sddmm_comm_t c, int64_t M, int64_t N, int64_t nnz, const int32_t *rows,
                                         const int32_t *cols, int K, int panel_rows_hint, int h_chunks,
                                         const double *rank_shares, uint32_t flags, sddmm_dist_plan_t *out);
SDDMM_API int sddmm_dist_plan_destroy(sddmm_dist_plan_t p);
/* The rank's rows [row_begin, row_end) and nonzeros [nnz_begin, nnz_end) of the input, and
 * the number of H chunks in use.  Any output may be NULL. */
SDDMM_API int sddmm_dist_plan_get_shard(sddmm_dist_plan_t p, int64_t *row_begin, int64_t *row_end, int64_t *nnz_begin,
                                        int64_t *nnz_end, int32_t *n_chunks);
/* The rank's single-GPU plan (for sddmm_plan_get_info, sddmm_plan_count_cols, ...); owned by p. */
SDDMM_API sddmm_plan_t sddmm_dist_plan_local(sddmm_dist_plan_t p);

#define SDDMM_DIST_H_RESIDENT     0x10000u /* H is already complete on every rank: no collective, plain execute */
#define SDDMM_DIST_BROADCAST_ONLY 0x20000u /* only the chunked H broadcast (to time it on its own) */
/*
 * One SDDMM over the rank's block: W_local = the rank's rows of W, Sval_local / P_local =
 * its slice of the nonzeros, H = a device array of N x K floats on every rank.  Without
 * SDDMM_DIST_H_RESIDENT, root's H is broadcast inside the call in the plan's chunks on the
 * communication stream while the nonzeros of the column ranges already received are
 * computed (all operands must be device arrays).  SDDMM_FLAG_* as in sddmm_execute.
 */
SDDMM_API int sddmm_dist_execute(sddmm_dist_plan_t p, const float *W_local, float *H, const float *Sval_local,
                                 float *P_local, int root, uint32_t flags);
/* Of the last synchronous sddmm_dist_execute on this rank, in ms (CUDA events): the
 * broadcast (first chunk enqueued -> last chunk arrived), the kernels when H was resident,
 * and the whole call on the compute stream.  -1 where it does not apply. */
SDDMM_API int sddmm_dist_last_times(sddmm_dist_plan_t p, float *bcast_ms, float *compute_ms, float *total_ms);

typedef struct sddmm_multi_s *sddmm_multi_t;
typedef struct sddmm_multi_plan_s *sddmm_multi_plan_t;
/* One process, ndev GPUs (devices == NULL: 0 .. ndev-1): a handle, a host thread and a
 * communicator per GPU. */
SDDMM_API int sddmm_multi_create(const int *devices, int ndev, sddmm_multi_t *out);
SDDMM_API int sddmm_multi_destroy(sddmm_multi_t m);
SDDMM_API const char *sddmm_multi_last_error(sddmm_multi_t m);
/* Host pattern (row-sorted COO); allocates every GPU's operand buffers. */
SDDMM_API int sddmm_multi_plan_coo(sddmm_multi_t m, int64_t M, int64_t N, int64_t nnz, const int32_t *rows,
                                   const int32_t *cols, int K, int panel_rows_hint, uint32_t flags,
                                   sddmm_multi_plan_t *out);
SDDMM_API int sddmm_multi_plan_destroy(sddmm_multi_plan_t p);
/* row_cuts / nnz_cuts: ndev + 1 entries each (either may be NULL). */
SDDMM_API int sddmm_multi_plan_get_cuts(sddmm_multi_plan_t p, int64_t *row_cuts, int64_t *nnz_cuts);
/* W, H, Sval (or NULL), P: HOST arrays of the whole problem.  Every GPU uploads its rows
 * of W, its S values and 1/ndev of H over its own PCIe link; the H slices are exchanged
 * with one all-gather; P comes back in input order. */
SDDMM_API int sddmm_multi_execute(sddmm_multi_plan_t p, const float *W, const float *H, const float *Sval, float *P,
                                  uint32_t flags);
/* Slowest GPU's kernel time of the last sddmm_multi_execute, in ms. */
SDDMM_API int sddmm_multi_last_kernel_ms(sddmm_multi_plan_t p, float *ms);

/* ---- Matrix Market I/O (host) -------------------------------------------- */

/*
 * Replaces the loader in main (HiPC18/src/sddmm.cu:257-281): skips the banner
 * and comment lines, reads "M N nnz", then nnz triples "row col val" (1-based).
 * Accepts everything the reference accepts; additionally accepts a size line that
 * is the first line and `pattern` files (value 1.0), expands `symmetric` only on
 * request (sddmm_mtx_open_ex), and reports what the reference silently mis-parses as
 * SDDMM_PARSE_ERROR.  Two-call protocol: sddmm_mtx_open reads the file and
 * reports the sizes, sddmm_mtx_read copies into caller buffers and closes.
 */
typedef struct sddmm_mtx_s *sddmm_mtx_t;
SDDMM_API int sddmm_mtx_open(const char *path, sddmm_mtx_t *out, int64_t *M, int64_t *N,
                             int64_t *nnz, char *errbuf, int errbuf_len);
/*
 * The same reader with options, and with the formats found around the reference's
 * loaders: Matrix Market `general` / `symmetric` / `skew-symmetric`, fields
 * `real` / `integer` / `pattern`; the three sizes on one line or on three
 * (headerless bag-of-words "docword" files, which the reference's other readers
 * take with `fp >> n_rows >> n_cols >> nnz`,
 * other_ideas/our_work/sparse_dense_split/sddmm.cu:356); and the binary form
 * written by sddmm_coo_save_binary (recognised by its first bytes).
 *   SDDMM_MTX_EXPAND_SYMMETRIC : a symmetric file stores one triangle -- add the
 *       mirror image of every off-diagonal entry (negated for skew-symmetric).
 *       Without the flag the stored triangle is returned as is, which is what
 *       the reference does (it ignores the banner, sddmm.cu:257-261).
 *   SDDMM_MTX_SORT_ROWS : return the triples sorted by (row, col) (stable), as
 *       sddmm_plan_coo needs them; sorted input is left untouched.
 */
#define SDDMM_MTX_EXPAND_SYMMETRIC 0x1u
#define SDDMM_MTX_SORT_ROWS 0x2u
SDDMM_API int sddmm_mtx_open_ex(const char *path, uint32_t flags, sddmm_mtx_t *out, int64_t *M,
                                int64_t *N, int64_t *nnz, char *errbuf, int errbuf_len);
SDDMM_API int sddmm_mtx_read(sddmm_mtx_t f, int32_t *rows, int32_t *cols, float *vals);
/*
 * Binary form of a COO matrix (48-byte header with a checksum, then rows, cols
 * and, unless vals is NULL, values; little-endian, 0-based): the reference
 * re-parses the text file on every run (sddmm.cu:274-281), this loads at the
 * speed of the disk.  Read it back with sddmm_mtx_open / sddmm_mtx_open_ex.
 */
SDDMM_API int sddmm_coo_save_binary(const char *path, int64_t M, int64_t N, int64_t nnz,
                                    const int32_t *rows, const int32_t *cols, const float *vals);
SDDMM_API int sddmm_mtx_close(sddmm_mtx_t f);
/*
 * Seeded synthetic matrix instead of a file (the reference ships no dataset: its
 * dataset/ folder is empty and HiPC18/run.sh, scripts/ name public corpora that
 * must be fetched).  `spec` is one of
 *   uniform:M:N:density | zipf:M:N:nnz | rmat:scale:edge_factor | band:M:half_width:g
 *   | c1 | c2 | c3 | c4 | c5        (the five benchmark configurations)
 * optionally followed by ":seed=S".  The result is row-sorted (columns ascending
 * inside a row, no duplicates) and is read with sddmm_mtx_read / released with
 * sddmm_mtx_close like a parsed file.  Host code; deterministic for a given spec.
 */
SDDMM_API int sddmm_gen_open(const char *spec, sddmm_mtx_t *out, int64_t *M, int64_t *N,
                             int64_t *nnz, char *errbuf, int errbuf_len);
/* 0/1: whether the triples just read are sorted by row (what the engine needs). */
SDDMM_API int sddmm_coo_is_row_sorted(int64_t nnz, const int32_t *rows);
SDDMM_API int sddmm_mtx_write(const char *path, int64_t M, int64_t N, int64_t nnz,
                              const int32_t *rows, const int32_t *cols, const float *vals);

/*
 * Replaces unsorted_make_CSR (HiPC18/src/util.h:82-128), the README's "conversion
 * code from col sorted to row sorted".  In place, 0-based in and out.
 *   transpose = 1 : the reference's live behaviour -- sort by (col,row,val) and
 *                   swap the roles, i.e. emit S^T row-sorted; *M and *N swap.
 *   transpose = 0 : stable sort by (row, col) of S itself (the commented variant,
 *                   util.h:93).
 */
SDDMM_API int sddmm_coo_sort_rows(int64_t *M, int64_t *N, int64_t nnz, int32_t *rows,
                                  int32_t *cols, float *vals, int transpose);

/*
 * The same conversion on the GPU (radix sorts instead of std::sort; seconds become
 * milliseconds at 10^8 nonzeros).  Results are identical to sddmm_coo_sort_rows:
 * transpose = 0 keeps the input order of equal (row, col) pairs, transpose = 1
 * orders whole (col, row, val) tuples.  rows / cols / vals may be host or device
 * arrays (rows and cols both of the same kind); sorted in place.
 */
SDDMM_API int sddmm_coo_sort_rows_gpu(sddmm_handle_t h, int64_t *M, int64_t *N, int64_t nnz,
                                      int32_t *rows, int32_t *cols, float *vals, int transpose);

#ifdef __cplusplus
}
#endif
#endif /* SDDMM_B200_H */
