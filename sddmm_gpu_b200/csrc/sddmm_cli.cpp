// Drop-in command line of the reference program:
//
//     ./sddmm input.mtx K tile_size_X tile_size_Y [options]
//     ./sddmm gen:SPEC  K tile_size_X tile_size_Y [options]
//
// The second form takes a seeded synthetic matrix instead of a file (the
// reference ships no dataset): gen:c1 .. gen:c5 are the benchmark configurations,
// gen:uniform:M:N:density, gen:zipf:M:N:nnz, gen:rmat:scale:edge_factor and
// gen:band:M:half_width:g the generators behind them (see sddmm_gen_open).
//
// Same four positionals in the same order and with the meaning the reference's
// code gives them (HiPC18/src/sddmm.cu:251-255): argv[3] is the row-panel height
// (rows of W per shared-memory panel), argv[4] the column-tile width.  The same
// three stdout lines are printed (sddmm.cu:267, :282, :114) so that scripts
// scraping them keep working.  W and H are initialised as the reference does
// (util.h:75-81).  Everything runs on the GPU through the C ABI; there is no CPU
// path here.  Errors give a one-line message on stderr and a non-zero exit code
// instead of assert().
//
// Options (after the positionals):
//   --iters N          timed repetitions (default 1, as the reference); the
//                      printed time is the mean kernel time per repetition
//   --warmup N         untimed repetitions first (default 0)
//   --no-scale-by-s    store the unscaled dot product, as the reference's GPU
//                      and COO CPU paths do (default: P = S o (W H^T))
//   --gather           use the planless gather kernel
//   --device D         CUDA device (default 0)
//   --gpus N           split S into N nnz-balanced row blocks over GPUs 0 .. N-1 of this box (one host
//                      thread and one NCCL rank per GPU, H exchanged over NVLink); what the reference
//                      does with `mpiexec -n N` (HiPC18_mpi/scripts/run_mpi.sh).  The printed time is the
//                      slowest GPU's kernel time
//   --dump-p FILE      write P (float32, input nonzero order) to FILE
//   --json FILE        write a small JSON report: ms, GFLOP/s, the kernels that ran, plan sizes,
//                      GPU count, host cores and the roofline figures (algorithmic bytes of the
//                      call, achieved GB/s, and its fraction of --hbm-gbs when that is given)
//   --hbm-gbs X        HBM bandwidth to report the roofline fraction against (GB/s)
//   --check            recompute every nonzero in float64 on the GPU and compare per nonzero
//                      (|P - ref| <= 1e-4 max(|ref|, sum_t |w_t h_t| |s|)): the in-line check the
//                      reference's MPI program makes against its CPU result
//                      (HiPC18_mpi/sddmm.cu:318-334); a failed check exits non-zero
//   --seed S           W and H uniform in [0, 1) from a counter-based generator seeded with S
//                      instead of the reference's srand48(0) initialisation
//   --write-mtx FILE   write the input matrix as Matrix Market (e.g. to hand a
//                      generated matrix to another program)
//   --save-bin FILE    write the input matrix in the library's binary form, which
//                      loads without parsing (pass FILE as the input next time)
//   --sort             an input that is not sorted by row is sorted by (row, col) on
//                      the GPU instead of being refused
//   --expand-symmetric a `symmetric` Matrix Market file stores one triangle: add the other
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "sddmm_b200.h"

namespace {

int die(const char *what, int status, const char *detail)
{
    std::fprintf(stderr, "sddmm: %s: %s%s%s\n", what, sddmm_status_string(status), (detail && *detail) ? " - " : "",
                 detail ? detail : "");
    return status ? status : 1;
}

void initial(std::vector<float> &X, long n, int k)
{
    srand48(0L);  // W and H restart the same stream, as in the reference
    for (long i = 0; i < n * (long)k; ++i) X[(size_t)i] = (float)(0.1 * drand48());
}

// uniform [0, 1) from splitmix64(seed, stream, index): exact in fp32, the same on every host
void seeded(std::vector<float> &X, uint64_t seed, uint64_t stream)
{
    for (size_t i = 0; i < X.size(); ++i) {
        uint64_t z = seed * 0x9e3779b97f4a7c15ull + stream * 0xbf58476d1ce4e5b9ull + (uint64_t)i + 0x94d049bb133111ebull;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        z ^= z >> 31;
        X[i] = (float)(uint32_t)(z >> 40) * (1.0f / 16777216.0f);
    }
}

}  // namespace

int main(int argc, char **argv)
{
    if (argc < 5) {
        std::fprintf(stderr, "usage: %s input.mtx K tile_size_X tile_size_Y [--iters N] [--warmup N] "
                             "[--no-scale-by-s] [--gather] [--device D] [--dump-p FILE] [--json FILE] [--write-mtx FILE] [--save-bin FILE] [--gpus N] [--sort] [--expand-symmetric] [--check] [--seed S] [--hbm-gbs X]\n"
                             "       input may be gen:c1..c5 | gen:uniform:M:N:density | gen:zipf:M:N:nnz | "
                             "gen:rmat:scale:edge_factor | gen:band:M:half_width:g [:seed=S]\n", argv[0]);
        return 2;
    }
    const char *path = argv[1];
    const int K = std::atoi(argv[2]);
    const int panel_rows = std::atoi(argv[3]);  // tile_sizeY / actv_row_size in the reference
    const int col_tile = std::atoi(argv[4]);    // tile_sizeX in the reference
    int iters = 1, warmup = 0, device = 0, gpus = 1;
    bool scale = true, gather = false;
    const char *dump_p = nullptr, *json = nullptr, *write_mtx = nullptr, *save_bin = nullptr;
    bool sort_input = false, check = false, have_seed = false;
    unsigned long long seed = 0;
    double hbm_gbs = 0.0;
    uint32_t open_flags = 0;
    for (int i = 5; i < argc; ++i) {
        std::string a = argv[i];
        auto need = [&](const char *name) -> const char * {
            if (i + 1 >= argc) {
                std::fprintf(stderr, "sddmm: %s needs a value\n", name);
                std::exit(2);
            }
            return argv[++i];
        };
        if (a == "--iters") iters = std::atoi(need("--iters"));
        else if (a == "--warmup") warmup = std::atoi(need("--warmup"));
        else if (a == "--device") device = std::atoi(need("--device"));
        else if (a == "--gpus") gpus = std::atoi(need("--gpus"));
        else if (a == "--no-scale-by-s") scale = false;
        else if (a == "--scale-by-s") scale = true;
        else if (a == "--gather") gather = true;
        else if (a == "--dump-p") dump_p = need("--dump-p");
        else if (a == "--json") json = need("--json");
        else if (a == "--write-mtx") write_mtx = need("--write-mtx");
        else if (a == "--save-bin") save_bin = need("--save-bin");
        else if (a == "--sort") sort_input = true;
        else if (a == "--check") check = true;
        else if (a == "--hbm-gbs") hbm_gbs = std::atof(need("--hbm-gbs"));
        else if (a == "--seed") {
            seed = std::strtoull(need("--seed"), nullptr, 10);
            have_seed = true;
        }
        else if (a == "--expand-symmetric") open_flags |= SDDMM_MTX_EXPAND_SYMMETRIC;
        else {
            std::fprintf(stderr, "sddmm: unknown option %s\n", a.c_str());
            return 2;
        }
    }
    if (iters < 1) iters = 1;

    sddmm_mtx_t f = nullptr;
    int64_t M = 0, N = 0, nnz = 0;
    char err[256] = "";
    const bool generated = std::strncmp(path, "gen:", 4) == 0;
    int st = generated ? sddmm_gen_open(path + 4, &f, &M, &N, &nnz, err, sizeof(err))
                       : sddmm_mtx_open_ex(path, open_flags, &f, &M, &N, &nnz, err, sizeof(err));
    if (st != SDDMM_OK) return die(generated ? "generating input" : "reading input", st, err);
    std::printf("\nMatrix info:  rows: %lld, cols: %lld, nnz: %lld\n", (long long)M, (long long)N, (long long)nnz);
    std::vector<int32_t> rows((size_t)nnz), cols((size_t)nnz);
    std::vector<float> vals((size_t)nnz);
    st = sddmm_mtx_read(f, rows.data(), cols.data(), vals.data());
    if (st != SDDMM_OK) return die("reading input", st, "");
    std::printf("\nTilesize: X = %d, tilesize: Y = %d, TB: %d\n", col_tile, panel_rows, 512);  // BLOCKSIZE of the reference (util.h:19)
    sddmm_handle_t h = nullptr;
    st = sddmm_create(&h, device);
    if (st != SDDMM_OK) return die("creating the engine", st, "");
    if (!sddmm_coo_is_row_sorted(nnz, rows.data())) {
        if (!sort_input) {
            sddmm_destroy(h);
            return die("input", SDDMM_UNSORTED_INPUT, "pass --sort, or convert it with sddmm_coo_sort_rows first");
        }
        st = sddmm_coo_sort_rows_gpu(h, &M, &N, nnz, rows.data(), cols.data(), vals.data(), 0);
        if (st != SDDMM_OK) {
            int rc = die("sorting the input", st, sddmm_last_error(h));
            sddmm_destroy(h);
            return rc;
        }
    }
    if (write_mtx) {
        st = sddmm_mtx_write(write_mtx, M, N, nnz, rows.data(), cols.data(), vals.data());
        if (st != SDDMM_OK) return die("writing the matrix", st, write_mtx);
    }
    if (save_bin) {
        st = sddmm_coo_save_binary(save_bin, M, N, nnz, rows.data(), cols.data(), vals.data());
        if (st != SDDMM_OK) return die("writing the matrix", st, save_bin);
    }

    std::vector<float> W((size_t)M * K), H((size_t)N * K), P((size_t)nnz);
    if (K > 0 && have_seed) {
        seeded(W, seed, 1);
        seeded(H, seed, 2);
    } else if (K > 0) {
        initial(W, M, K);
        initial(H, N, K);
    }

    const uint32_t flags = gather ? SDDMM_FLAG_KERNEL_GATHER : 0u;
    const float *sval = scale ? vals.data() : nullptr;
    double multi_ms = -1.0;
    if (gpus > 1) {
        // several GPUs: one rank per GPU inside this process
        sddmm_multi_t multi = nullptr;
        st = sddmm_multi_create(nullptr, gpus, &multi);
        if (st != SDDMM_OK) {
            sddmm_destroy(h);
            return die("creating the multi-GPU engine", st, "");
        }
        sddmm_multi_plan_t mplan = nullptr;
        st = sddmm_multi_plan_coo(multi, M, N, nnz, rows.data(), cols.data(), K, panel_rows, 0, &mplan);
        double total = 0;
        for (int it = 0; st == SDDMM_OK && it < warmup + iters; ++it) {
            st = sddmm_multi_execute(mplan, W.data(), H.data(), sval, P.data(), flags);
            float ms1 = 0;
            sddmm_multi_last_kernel_ms(mplan, &ms1);
            if (it >= warmup) total += ms1;
        }
        if (st != SDDMM_OK) {
            int rc = die("running on several GPUs", st, sddmm_multi_last_error(multi));
            sddmm_multi_plan_destroy(mplan);
            sddmm_multi_destroy(multi);
            sddmm_destroy(h);
            return rc;
        }
        multi_ms = total / iters;
        sddmm_multi_plan_destroy(mplan);
        sddmm_multi_destroy(multi);
    }

    // the single-GPU plan: the whole run with one GPU; with several, what --check and the report read
    sddmm_plan_t plan = nullptr;
    st = sddmm_plan_coo(h, M, N, nnz, rows.data(), cols.data(), K, panel_rows, col_tile, 0, &plan);
    if (st != SDDMM_OK) {
        int rc = die("planning", st, sddmm_last_error(h));
        sddmm_destroy(h);
        return rc;
    }
    double total_ms = 0;
    // with several GPUs P already holds the result that is reported, dumped and checked
    for (int it = 0; it < (gpus > 1 ? 0 : warmup + iters); ++it) {
        st = sddmm_execute(plan, W.data(), H.data(), sval, P.data(), flags);
        if (st != SDDMM_OK) {
            int rc = die("executing", st, sddmm_last_error(h));
            sddmm_destroy_plan(plan);
            sddmm_destroy(h);
            return rc;
        }
        float ms = 0;
        sddmm_last_kernel_ms(plan, &ms);
        if (it >= warmup) total_ms += ms;
    }
    const double ms = gpus > 1 ? multi_ms : total_ms / iters;
    std::printf("\nTime for SDDMM with K = %d : %g ms\n", K, ms);

    sddmm_plan_info info;
    sddmm_plan_get_info(plan, &info);
    const std::string kernel_name = gpus > 1 ? "row blocks over several GPUs" : sddmm_last_kernel_name(plan);
    double check_err = -1.0;
    long long check_n = 0, check_bad = 0;
    if (check && nnz > 0) {
        int64_t n_checked = 0, n_bad = 0;
        st = sddmm_check_result(plan, W.data(), H.data(), sval, P.data(), 1, 1e-4, &check_err, &n_checked, &n_bad);
        if (st != SDDMM_OK) {
            int rc = die("checking", st, sddmm_last_error(h));
            sddmm_destroy_plan(plan);
            sddmm_destroy(h);
            return rc;
        }
        check_n = n_checked;
        check_bad = n_bad;
        std::fprintf(stderr, "sddmm: check: %lld nonzeros recomputed in float64, %lld out of tolerance, max scaled error %.3g\n",
                     check_n, check_bad, check_err);
    }
    if (dump_p) {
        FILE *o = std::fopen(dump_p, "wb");
        if (!o || std::fwrite(P.data(), sizeof(float), (size_t)nnz, o) != (size_t)nnz) return die("writing P", SDDMM_IO_ERROR, dump_p);
        std::fclose(o);
    }
    if (json) {
        FILE *o = std::fopen(json, "w");
        if (!o) return die("writing report", SDDMM_IO_ERROR, json);
        const double gflops = ms > 0 ? 2.0 * (double)nnz * K / (ms * 1e6) : 0.0;
        // algorithmic bytes of one call: every touched row of W and H once, per nonzero a column index, an S
        // value and a P store, plus the row pointer
        int64_t n_cols_used = 0;
        sddmm_plan_count_cols(plan, &n_cols_used);
        const double alg_bytes = 4.0 * K * (double)(info.n_nonempty_rows + n_cols_used) + 12.0 * (double)nnz + 4.0 * (double)(M + 1);
        const double achieved = ms > 0 ? alg_bytes / (ms * 1e6) : 0.0;
        std::fprintf(o, "{\"roofline\": {\"bound\": \"hbm\", \"algorithmic_bytes\": %.0f, \"achieved_gbs\": %.3f, \"peak_gbs\": %s, "
                        "\"frac\": %s}, \"gpus\": %d, \"host_cores\": %u, \"check\": {\"ran\": %s, \"n\": %lld, \"bad\": %lld, "
                        "\"max_scaled_err\": %.6g}, ",
                     alg_bytes, achieved, hbm_gbs > 0 ? std::to_string(hbm_gbs).c_str() : "null",
                     hbm_gbs > 0 ? std::to_string(achieved / hbm_gbs / gpus).c_str() : "null", gpus, std::thread::hardware_concurrency(),
                     check ? "true" : "false", check_n, check_bad, check_err);
        std::fprintf(o,
                     "\"rows\": %lld, \"cols\": %lld, \"nnz\": %lld, \"K\": %d, \"kernel_ms\": %.6f, "
                     "\"gflops\": %.3f, \"plan_ms\": %.4f, \"panel_rows\": %d, \"col_tile\": %d, "
                     "\"n_col_tiles\": %d, \"work_items\": %lld, \"nonempty_rows\": %lld, \"scale_by_s\": %s, "
                     "\"kernel\": \"%s\"}\n",
                     (long long)M, (long long)N, (long long)nnz, K, ms, gflops, info.plan_ms, info.panel_rows,
                     info.col_tile, info.n_col_tiles, (long long)info.n_work_items, (long long)info.n_nonempty_rows,
                     scale ? "true" : "false", kernel_name.c_str());
        std::fclose(o);
    }
    sddmm_destroy_plan(plan);
    sddmm_destroy(h);
    if (check && check_bad > 0) {
        std::fprintf(stderr, "sddmm: check failed\n");
        return 3;
    }
    return 0;
}
