"""Parity of the CUDA path with the CPU oracle, through the C ABI.

Oracle = oracle/sddmm_oracle.c (restatement of sddmm_CPU_COO / sddmm_CPU_CSR,
HiPC18/src/sddmm.cu:153-200).  Tolerance: 1e-4 relative per nonzero for the
values (fp32, reassociated sums); order and indices bit-exact.
"""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_parity, random_coo
from sddmm_gpu_b200 import api, synth

pytestmark = pytest.mark.gpu

KERNELS = {"panel": api.FLAG_KERNEL_PANEL, "gather": api.FLAG_KERNEL_GATHER, "ring": api.FLAG_KERNEL_RING}
RING_K = (32, 64, 128, 256, 512, 1024)
LONG_ROW_K = (256, 512, 1024)


def kernels_for(K):
    return [k for k in KERNELS if k != "ring" or K in RING_K]


def run_plan(engine, M, N, rows, cols, W, H, vals=None, flags=0, panel_rows=0, col_tile=0):
    plan = engine.plan_coo(M, N, rows, cols, W.shape[1], panel_rows, col_tile)
    P = np.full(rows.shape[0], np.nan, np.float32)
    plan.execute(W, H, P, vals, flags)
    info = plan.info()
    plan.close()
    return P, info


def test_hand_computable(engine):
    # 3 x 4, 5 nonzeros, K = 4, integer-valued operands -> exact results
    rows = np.array([0, 0, 1, 2, 2], np.int32)
    cols = np.array([0, 3, 1, 0, 2], np.int32)
    vals = np.array([1, 2, 3, 4, 5], np.float32)
    W = np.arange(12, dtype=np.float32).reshape(3, 4)
    H = (np.arange(16, dtype=np.float32).reshape(4, 4) % 5) - 2
    expect = np.array([(W[r] * H[c]).sum() for r, c in zip(rows, cols)], np.float32)
    for flag in (KERNELS["panel"], KERNELS["gather"], 0):
        P, _ = run_plan(engine, 3, 4, rows, cols, W, H, None, flag)
        assert np.array_equal(P, expect)
        P, _ = run_plan(engine, 3, 4, rows, cols, W, H, vals, flag)
        assert np.array_equal(P, expect * vals)


@pytest.mark.parametrize("kernel", list(KERNELS))
@pytest.mark.parametrize("K", [4, 8, 12, 16, 20, 32, 36, 64, 100, 128, 192, 256, 260, 512, 1024, 2048])
def test_every_k(engine, kernel, K):
    if kernel not in kernels_for(K):
        pytest.skip("the ring kernels cover K = 32, 64, 128, 256, 512, 1024")
    rng = np.random.default_rng(K)
    M, N = 257, 190
    rows, cols = random_coo(rng, M, N, 6000, empty_rows=[0, 5, 6, 7, 100, 256])
    vals = rng.standard_normal(rows.shape[0]).astype(np.float32)
    W = rng.standard_normal((M, K)).astype(np.float32)
    H = rng.standard_normal((N, K)).astype(np.float32)
    P, _ = run_plan(engine, M, N, rows, cols, W, H, vals, KERNELS[kernel])
    assert_parity(P, rows, cols, W, H, vals)
    P, _ = run_plan(engine, M, N, rows, cols, W, H, None, KERNELS[kernel])
    assert_parity(P, rows, cols, W, H, None)


@pytest.mark.parametrize("kernel", list(KERNELS))
def test_structure_edge_cases(engine, kernel):
    rng = np.random.default_rng(7)
    K = 128 if kernel == "ring" else 32
    flag = KERNELS[kernel]
    cases = []
    # nnz = 1, M = 1, N = 1, max column index, one row holding everything
    cases.append((1, 1, np.array([0], np.int32), np.array([0], np.int32)))
    cases.append((5, 9, np.array([4], np.int32), np.array([8], np.int32)))
    cases.append((1, 300, np.zeros(300, np.int32), np.arange(300, dtype=np.int32)))
    cases.append((300, 1, np.arange(300, dtype=np.int32), np.zeros(300, np.int32)))
    r, c = random_coo(rng, 64, 5000, 3000, hub_row=17)          # one hub row with all N columns
    cases.append((64, 5000, r, c))
    r, c = random_coo(rng, 3000, 64, 9000, empty_rows=range(0, 1000))   # empty rows at the start
    cases.append((3000, 64, r, c))
    r, c = random_coo(rng, 3000, 64, 9000, empty_rows=range(2000, 3000))  # ... at the end
    cases.append((3000, 64, r, c))
    for M, N, rows, cols in cases:
        W = rng.random((M, K), dtype=np.float32)
        H = rng.random((N, K), dtype=np.float32)
        P, info = run_plan(engine, M, N, rows, cols, W, H, None, flag)
        assert_parity(P, rows, cols, W, H)
        assert info.n_nonempty_rows == np.unique(rows).size


def test_empty_matrix(engine):
    plan = engine.plan_coo(10, 10, np.zeros(0, np.int32), np.zeros(0, np.int32), 8)
    W = np.ones((10, 8), np.float32)
    plan.execute(W, W, np.zeros(0, np.float32))
    assert plan.info().n_work_items == 0
    assert np.array_equal(plan.export_row_ptr(), np.zeros(11, np.int64))
    plan.close()


def test_row_ptr_and_counts(engine):
    rng = np.random.default_rng(3)
    M, N = 1000, 777
    rows, cols = random_coo(rng, M, N, 5000, empty_rows=[0, 1, 2, 500, 999])
    plan = engine.plan_coo(M, N, rows, cols, 16)
    rp = plan.export_row_ptr()
    expect = np.zeros(M + 1, np.int64)
    np.add.at(expect, rows.astype(np.int64) + 1, 1)
    assert np.array_equal(rp, np.cumsum(expect))
    assert plan.count_cols() == np.unique(cols).size
    plan.close()


def test_validation_errors(engine):
    W = np.zeros((4, 8), np.float32)
    rows = np.array([0, 2, 1], np.int32)
    cols = np.array([0, 1, 2], np.int32)
    with pytest.raises(api.SddmmError) as e:
        engine.plan_coo(4, 4, rows, cols, 8)
    assert e.value.status == api.UNSORTED_INPUT
    with pytest.raises(api.SddmmError) as e:
        engine.plan_coo(4, 4, np.array([0, 1, 4], np.int32), cols, 8)
    assert e.value.status == api.INDEX_OUT_OF_RANGE
    with pytest.raises(api.SddmmError) as e:
        engine.plan_coo(4, 4, np.array([0, 1, 2], np.int32), np.array([0, -1, 2], np.int32), 8)
    assert e.value.status == api.INDEX_OUT_OF_RANGE
    for K in (0, 3, 30, 4100):
        with pytest.raises(api.SddmmError) as e:
            engine.plan_coo(4, 4, np.array([0, 1, 2], np.int32), cols, K)
        assert e.value.status == api.K_UNSUPPORTED
    # the handle stays usable after an error
    plan = engine.plan_coo(4, 4, np.array([0, 1, 2], np.int32), cols, 8)
    P = np.zeros(3, np.float32)
    plan.execute(W, W, P)
    plan.close()


@pytest.mark.parametrize("K", [64, 128])
@pytest.mark.parametrize("col_tile,panel_rows", [(64, 16), (33, 7), (1, 1), (500, 192), (128, 0)])
def test_column_tiled_plan(engine, col_tile, panel_rows, K):
    # a multi-tile plan processes in the reference's tiled order and still
    # returns P in input order; TILED_ORDER returns what sddmm_GPU leaves in d_val
    rng = np.random.default_rng(11)
    M, N = 300, 200
    rows, cols = random_coo(rng, M, N, 5003)
    vals = rng.integers(1, 20, rows.shape[0]).astype(np.float32)
    W = rng.random((M, K), dtype=np.float32)
    H = rng.random((N, K), dtype=np.float32)
    P, info = run_plan(engine, M, N, rows, cols, W, H, vals, 0, panel_rows, col_tile)
    assert info.n_col_tiles == -(-N // col_tile)
    ref = assert_parity(P, rows, cols, W, H, vals)
    Pt, _ = run_plan(engine, M, N, rows, cols, W, H, None, api.FLAG_TILED_ORDER, panel_rows, col_tile)
    tiling = oracle.cpu.rewrite_matrix_1d(rows, cols, vals, M, N, max(panel_rows, 1), col_tile)
    P_unscaled, _ = run_plan(engine, M, N, rows, cols, W, H, None, 0, panel_rows, col_tile)
    assert np.array_equal(Pt, P_unscaled[tiling["tiled_ind"]])
    del ref


def test_device_pointers_and_stream(engine):
    p = synth.uniform_sparse(M=2048, N=1024, density=0.004, K=64, device="cuda")
    rows, cols, W, H, vals = p["rows"], p["cols"], p["W"], p["H"], p["vals"] * 3
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    engine.set_stream(side.cuda_stream)
    plan = engine.plan_coo(p["M"], p["N"], rows, cols, p["K"])
    P = torch.empty(rows.shape[0], device="cuda")
    with torch.cuda.stream(side):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        plan.execute(W, H, P, vals, api.FLAG_ASYNC)
        e1.record()
    side.synchronize()                  # only the caller's stream is waited for
    assert e0.elapsed_time(e1) > 0.0
    engine.set_stream(None)
    q = synth.to_numpy(p)
    assert_parity(P.cpu().numpy(), q["rows"], q["cols"], q["W"], q["H"], q["vals"] * 3)
    # one-shot form, host pointers
    P2 = np.zeros(rows.shape[0], np.float32)
    engine.sddmm_coo(p["M"], p["N"], q["rows"], q["cols"], q["W"], q["H"], p["K"], P2)
    assert_parity(P2, q["rows"], q["cols"], q["W"], q["H"])
    plan.close()


def test_calls_follow_torch_current_stream_without_manual_sync():
    """No torch.cuda.synchronize() around the calls: a handle that was not given a stream launches on
    torch's current stream, so it sees operands that are still being produced on that stream and the
    next torch operation on it sees the finished P."""
    h = api.Handle(0)
    try:
        p = synth.uniform_sparse(M=4096, N=4096, density=0.01, K=256, device="cuda")
        rows, cols = p["rows"], p["cols"]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            plan = h.plan_coo(p["M"], p["N"], rows, cols, p["K"])
            big = torch.randn(8192, 8192, device="cuda")
            for _ in range(4):
                big = big @ big * 1e-4                       # keeps the stream busy for a while
            W = torch.zeros_like(p["W"])
            W += p["W"] + big[0, 0] * 0                      # W is complete only after the matrix products
            P = torch.empty(rows.shape[0], device="cuda")
            plan.execute(W, p["H"], P, p["vals"], api.FLAG_ASYNC)
            total = P.double().sum()                         # enqueued right behind the kernel, same stream
            W.zero_()                                        # and the operand is overwritten straight after
            h.sync()                                         # waits for the stream and reads the device status word
            got_total = float(total)
        q = synth.to_numpy(p)
        ref = oracle.cpu.sddmm_coo(q["rows"], q["cols"], q["W"], q["H"], q["vals"])
        assert_parity(P.cpu().numpy(), q["rows"], q["cols"], q["W"], q["H"], q["vals"])
        assert abs(got_total - float(ref.astype(np.float64).sum())) <= 1e-3 * float(np.abs(ref).sum())
        assert plan.last_kernel_name() == "ring"
        # the device-side float64 self-check agrees, and notices a damaged result
        worst, n, bad = plan.check_result(p["W"], p["H"], P, p["vals"])
        assert n == rows.shape[0] and bad == 0 and worst <= 1e-4
        P[7] += 1.0
        worst, n, bad = plan.check_result(p["W"], p["H"], P, p["vals"], stride=1)
        assert bad == 1 and worst > 1e-4
        plan.close()
    finally:
        h.close()


def _scaled(problem_fn, **kw):
    return synth.to_numpy(problem_fn(device="cpu", **kw))


@pytest.mark.parametrize("name", ["c1", "c2", "c3_small", "c4_small", "c5_small"])
@pytest.mark.parametrize("kernel", list(KERNELS))
def test_benchmark_configs(engine, name, kernel):
    # config 1 and 2 at full size; 3, 4, 5 at sizes the oracle finishes in seconds
    if name == "c1":
        p = _scaled(synth.uniform_sparse)
    elif name == "c2":
        p = _scaled(synth.bag_of_words)
    elif name == "c3_small":
        p = _scaled(synth.rmat, scale=14, edge_factor=16, K=128)
    elif name == "c4_small":
        p = _scaled(synth.rmat, scale=15, edge_factor=24, K=256, seed=synth.SEEDS["c4"])
    else:
        p = _scaled(synth.attention_mask, M=4096, half_width=64, n_global=12, K=64)
    if kernel not in kernels_for(p["K"]):
        pytest.skip("the ring kernels cover K = 32, 64, 128, 256, 512, 1024")
    P, info = run_plan(engine, p["M"], p["N"], p["rows"], p["cols"], p["W"], p["H"], p["vals"], KERNELS[kernel],
                       p["panel_rows"], p["col_tile"])
    assert_parity(P, p["rows"], p["cols"], p["W"], p["H"], p["vals"])
    assert info.nnz == p["rows"].shape[0]


@pytest.mark.parametrize("K", LONG_ROW_K)
def test_long_row_ring_shapes(engine, K):
    """The TMA ring kernel (K = 256, 512, 1024) on inputs that exercise its edges: fewer nonzeros than one
    group, a last group that is not full, sizes around a block of groups, the column-tile permutation,
    scaled and unscaled."""
    rng = np.random.default_rng(100 + K)
    for M, N, nnz, col_tile in ((7, 9, 5, 0), (300, 200, 8191, 0), (300, 200, 8192, 0), (2000, 1500, 70001, 0),
                                (300, 200, 9000, 64)):
        rows, cols = random_coo(rng, M, N, nnz, empty_rows=[1, 2])
        vals = rng.standard_normal(rows.shape[0]).astype(np.float32)
        W = rng.standard_normal((M, K)).astype(np.float32)
        H = rng.standard_normal((N, K)).astype(np.float32)
        for sv in (vals, None):
            P, _ = run_plan(engine, M, N, rows, cols, W, H, sv, KERNELS["ring"], 0, col_tile)
            assert_parity(P, rows, cols, W, H, sv)


def test_repeatable_and_reusable_plan(engine):
    # same plan, different operands; identical calls give identical bits
    rng = np.random.default_rng(5)
    M, N, K = 500, 400, 128
    rows, cols = random_coo(rng, M, N, 20000)
    plan = engine.plan_coo(M, N, rows, cols, K)
    outs = []
    for seed in (1, 2, 1):
        r = np.random.default_rng(seed)
        W = r.standard_normal((M, K)).astype(np.float32)
        H = r.standard_normal((N, K)).astype(np.float32)
        P = np.zeros(rows.shape[0], np.float32)
        plan.execute(W, H, P)
        assert_parity(P, rows, cols, W, H)
        outs.append(P)
    assert np.array_equal(outs[0], outs[2])
    plan.close()


def test_linearity_at_scale(engine):
    # size-independent property on a larger input: SDDMM is linear in W
    p = synth.rmat(scale=18, edge_factor=16, K=128, device="cuda")
    plan = engine.plan_coo(p["M"], p["N"], p["rows"], p["cols"], p["K"])
    nnz = p["rows"].shape[0]
    P1, P2, P3 = (torch.empty(nnz, device="cuda") for _ in range(3))
    W2 = torch.randn_like(p["W"])
    plan.execute(p["W"], p["H"], P1)
    plan.execute(W2, p["H"], P2)
    plan.execute(p["W"] + W2, p["H"], P3)
    scale = (p["W"].abs().max() + W2.abs().max()) * p["H"].abs().max() * p["K"]
    assert float((P1 + P2 - P3).abs().max()) <= 1e-5 * float(scale)
    # and the kernels agree with each other to rounding
    for flag in KERNELS.values():
        P4 = torch.empty(nnz, device="cuda")
        plan.execute(p["W"], p["H"], P4, None, flag)
        assert float((P1 - P4).abs().max()) <= 1e-5 * float(scale)
    plan.close()


# ---- binning pass vs the reference's host tiling (bit-exact) ------------------

TILING_KEYS = ("rows", "cols", "tiled_ind", "lastIdx_tile", "lastIdx_block_tile", "active_row", "n_actv_row")


def _check_tiling(engine, M, N, rows, cols, pairs, expected=None):
    plan = engine.plan_coo(M, N, rows, cols, 8)
    for i, (pr, ct) in enumerate(pairs):
        got = plan.export_tiling(int(pr), int(ct))
        want = expected(i) if expected else oracle.cpu.rewrite_matrix_1d(rows, cols, None, M, N, int(pr), int(ct))
        for k in TILING_KEYS:
            assert np.array_equal(got[k], np.asarray(want[k])), (pr, ct, k)
        assert got["max_active_row"] == int(want["max_active_row"]), (pr, ct)
    plan.close()


def test_export_tiling_matches_reference_golden(engine):
    # the fixture holds what the reference's own make_CSR + rewrite_matrix_1D produced
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiling.npz"))
    M, N = int(g["M"]), int(g["N"])
    _check_tiling(engine, M, N, g["rows"], g["cols"], g["pairs"],
                  expected=lambda i: {k: g[f"t{i}_{k}"] for k in TILING_KEYS + ("max_active_row",)})


@pytest.mark.parametrize("seed", [0, 1])
def test_export_tiling_matches_oracle(engine, seed):
    rng = np.random.default_rng(seed)
    M, N = 517, 300
    rows, cols = random_coo(rng, M, N, 7001, empty_rows=[0, 3, 4, 100, 516] if seed else ())
    pairs = [(32, 4096), (16, 64), (7, 33), (192, 50000), (1, 1), (5, 300), (64, 100), (517, 299)]
    _check_tiling(engine, M, N, rows, cols, pairs)


def test_export_tiling_config1_and_2_shapes(engine):
    # the CLI pairs of the first two benchmark configurations: a single column tile, identity order
    p = synth.to_numpy(synth.uniform_sparse(device="cpu"))
    _check_tiling(engine, p["M"], p["N"], p["rows"], p["cols"], [(32, 4096)])
    p = synth.to_numpy(synth.bag_of_words(device="cpu"))
    _check_tiling(engine, p["M"], p["N"], p["rows"], p["cols"], [(192, 50000), (96, 50000), (24, 500)])


# ---- the drop-in command line -------------------------------------------------

def test_cli_prints_reference_lines_and_matches_oracle(tmp_path):
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(root, "sddmm_gpu_b200", "csrc", "sddmm")
    rng = np.random.default_rng(3)
    M, N, K = 200, 150, 32
    rows, cols = random_coo(rng, M, N, 3000)
    vals = rng.integers(1, 20, rows.shape[0]).astype(np.float32)
    mtx = str(tmp_path / "in.mtx")
    api.mtx_write(mtx, M, N, rows, cols, vals)
    out = str(tmp_path / "p.bin")
    for extra, sv in (([], vals), (["--no-scale-by-s"], None)):
        res = subprocess.run([exe, mtx, str(K), "192", "50000", "--dump-p", out, "--json", str(tmp_path / "r.json"),
                              "--check", "--hbm-gbs", "6500"] + extra, capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
        import json
        rep = json.load(open(tmp_path / "r.json"))
        assert rep["kernel"] == "panel" and rep["gpus"] == 1 and rep["host_cores"] >= 1   # 3000 nonzeros: the panel kernel
        assert rep["check"]["ran"] and rep["check"]["n"] == rows.shape[0] and rep["check"]["bad"] == 0
        assert rep["check"]["max_scaled_err"] <= 1e-4
        n_cols_used = np.unique(cols).size
        assert rep["roofline"]["algorithmic_bytes"] == 4 * K * (np.unique(rows).size + n_cols_used) + 12 * rows.shape[0] + 4 * (M + 1)
        assert abs(rep["roofline"]["frac"] - rep["roofline"]["achieved_gbs"] / 6500) < 1e-6
        lines = [l for l in res.stdout.splitlines() if l.strip()]
        assert lines[0] == f"Matrix info:  rows: {M}, cols: {N}, nnz: {rows.shape[0]}"
        assert lines[1] == "Tilesize: X = 50000, tilesize: Y = 192, TB: 512"   # the reference's line, verbatim (sddmm.cu:282)
        assert lines[2].startswith(f"Time for SDDMM with K = {K} : ") and lines[2].endswith(" ms")
        W = oracle.cpu.initial(M, K)     # the reference's operand initialisation
        H = oracle.cpu.initial(N, K)
        assert_parity(np.fromfile(out, np.float32), rows, cols, W, H, sv)
    # a generated input instead of a file: the matrix written by --write-mtx is the one that was computed on
    gen_mtx = str(tmp_path / "gen.mtx")
    res = subprocess.run([exe, "gen:rmat:11:12:seed=5", "64", "96", "50000", "--dump-p", out, "--write-mtx", gen_mtx],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    gM, gN, g_rows, g_cols, g_vals = api.mtx_read(gen_mtx)
    m2 = api.gen_matrix("rmat:11:12:seed=5")
    assert (gM, gN) == (2048, 2048) and np.array_equal(g_rows, m2[2]) and np.array_equal(g_cols, m2[3])
    assert res.stdout.splitlines()[1] == f"Matrix info:  rows: 2048, cols: 2048, nnz: {g_rows.size}"
    assert_parity(np.fromfile(out, np.float32), g_rows, g_cols, oracle.cpu.initial(gM, 64), oracle.cpu.initial(gN, 64), g_vals)
    # an input sorted by column: refused without --sort, sorted on the GPU with it; the binary form it saves
    # loads back to the same result
    order = np.lexsort((rows, cols))
    col_sorted = str(tmp_path / "colsorted.mtx")
    api.mtx_write(col_sorted, M, N, rows[order], cols[order], vals[order])
    bad = subprocess.run([exe, col_sorted, str(K), "192", "50000"], capture_output=True, text=True)
    assert bad.returncode != 0 and "not sorted by row" in bad.stderr
    binf, out2 = str(tmp_path / "m.sddmm"), str(tmp_path / "p2.bin")
    res = subprocess.run([exe, col_sorted, str(K), "192", "50000", "--sort", "--save-bin", binf, "--dump-p", out],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    assert_parity(np.fromfile(out, np.float32), rows, cols, oracle.cpu.initial(M, K), oracle.cpu.initial(N, K), vals)
    res = subprocess.run([exe, binf, str(K), "192", "50000", "--dump-p", out2], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    assert np.array_equal(np.fromfile(out, np.float32), np.fromfile(out2, np.float32))
    # errors: non-zero exit code and one line on stderr instead of an assert
    bad = subprocess.run([exe, "gen:nosuch", "32", "192", "50000"], capture_output=True, text=True)
    assert bad.returncode != 0 and bad.stderr.startswith("sddmm: ")
    bad = subprocess.run([exe, str(tmp_path / "missing.mtx"), "32", "192", "50000"], capture_output=True, text=True)
    assert bad.returncode != 0 and bad.stderr.startswith("sddmm: ")
    bad = subprocess.run([exe, mtx, "30", "192", "50000"], capture_output=True, text=True)
    assert bad.returncode != 0 and "K must be" in bad.stderr


# ---- dense cells: locally dense matrices split into dense blocks + gathered remainder ----

@pytest.mark.parametrize("K", [16, 64, 100, 256])
def test_dense_cell_path(engine, K):
    p = synth.to_numpy(synth.attention_mask(M=1100, half_width=96, n_global=7, K=K, device="cpu"))
    rng = np.random.default_rng(K)
    vals = rng.standard_normal(p["rows"].shape[0]).astype(np.float32)
    for sv in (vals, None):
        P, info = run_plan(engine, p["M"], p["N"], p["rows"], p["cols"], p["W"], p["H"], sv, 0)
        assert info.n_dense_cells > 0 and 0 < info.n_dense_nnz <= info.nnz
        assert_parity(P, p["rows"], p["cols"], p["W"], p["H"], sv)
    # a forced kernel bypasses the split and must agree
    P2, _ = run_plan(engine, p["M"], p["N"], p["rows"], p["cols"], p["W"], p["H"], vals, api.FLAG_KERNEL_GATHER)
    assert_parity(P2, p["rows"], p["cols"], p["W"], p["H"], vals)


def test_dense_cells_cover_everything_or_nothing(engine):
    # fully dense small matrix: the full cells are dense, the thin edge cells fall to the remainder
    M, N, K = 200, 130, 32
    rows = np.repeat(np.arange(M), N).astype(np.int32)
    cols = np.tile(np.arange(N), M).astype(np.int32)
    rng = np.random.default_rng(0)
    W = rng.standard_normal((M, K)).astype(np.float32)
    H = rng.standard_normal((N, K)).astype(np.float32)
    P, info = run_plan(engine, M, N, rows, cols, W, H, None, 0)
    assert info.n_dense_cells >= 2 and 128 * 128 <= info.n_dense_nnz < rows.shape[0]
    assert_parity(P, rows, cols, W, H)
    # sparse matrix with long rows but no dense cell: classification declines
    rows, cols = random_coo(rng, 64, 60000, 64 * 40)
    W = rng.standard_normal((64, K)).astype(np.float32)
    H = rng.standard_normal((60000, K)).astype(np.float32)
    P, info = run_plan(engine, 64, 60000, rows, cols, W, H, None, 0)
    assert info.n_dense_cells == 0
    assert_parity(P, rows, cols, W, H)


@pytest.mark.parametrize("name", ["c2", "c5_small"])
def test_benchmark_configs_default_path(engine, name):
    p = _scaled(synth.bag_of_words) if name == "c2" else _scaled(synth.attention_mask, M=4096, half_width=64, n_global=12, K=64)
    P, info = run_plan(engine, p["M"], p["N"], p["rows"], p["cols"], p["W"], p["H"], p["vals"], 0,
                       p["panel_rows"], p["col_tile"])
    assert_parity(P, p["rows"], p["cols"], p["W"], p["H"], p["vals"])


@pytest.mark.parametrize("runs", ["0", "1"])
@pytest.mark.parametrize("K", [16, 36, 64])
def test_dense_cell_forms(engine, K, runs, monkeypatch):
    # K <= 64: the general form of the tcgen05 dense-cell kernel and the one that keeps a row block's W tile in shared
    # memory across consecutive cells, on a band + global rows / columns mask (compacted and regular cells, runs of
    # several cells and of one)
    monkeypatch.setenv("SDDMM_DENSE_RUNS", runs)
    p = _scaled(synth.attention_mask, M=4096, half_width=96, n_global=20, K=K)
    P, info = run_plan(engine, p["M"], p["N"], p["rows"], p["cols"], p["W"], p["H"], p["vals"], 0)
    assert info.n_dense_nnz > 0
    assert_parity(P, p["rows"], p["cols"], p["W"], p["H"], p["vals"])


@pytest.mark.parametrize("K", [128, 256, 512])
@pytest.mark.parametrize("N", [150, 777, 1500])
def test_column_tile_kernel(engine, K, N, monkeypatch):
    # few columns, many nonzeros per column: tiles of H in shared memory (one tile, a ragged last tile, eight tiles
    # at K = 256); the dense-cell split is switched off so that the 42 % dense case takes this path as well
    monkeypatch.setenv("SDDMM_DENSE_CELLS", "0")
    rng = np.random.default_rng(K + N)
    M = 8000
    rows, cols = random_coo(rng, M, N, 500_000, empty_rows=(0, 17, M - 1))
    W = rng.standard_normal((M, K), dtype=np.float32)
    H = rng.standard_normal((N, K), dtype=np.float32)
    vals = rng.standard_normal(rows.shape[0], dtype=np.float32)
    plan = engine.plan_coo(M, N, rows, cols, K)
    P = np.full(rows.shape[0], np.nan, np.float32)
    plan.execute(W, H, P, vals, 0)
    assert plan.last_kernel_name() == "htile"
    assert_parity(P, rows, cols, W, H, vals)
    P2 = np.full(rows.shape[0], np.nan, np.float32)
    plan.execute(W, H, P2, None, api.FLAG_KERNEL_RING)    # the forced ring kernel on the same plan, S = 1
    assert plan.last_kernel_name().startswith("ring")
    assert_parity(P2, rows, cols, W, H, None)
    plan.close()


# ---- failure path: a bounded device wait that runs out ------------------------

def test_bounded_wait_reports_timeout_and_handle_survives(engine):
    # one warp waits on a barrier nothing sets, with a short limit; it gives up and the host
    # sees DEVICE_TIMEOUT.  No fault, trap or hang is involved; the context stays usable.
    assert engine.selftest_wait_timeout() == api.DEVICE_TIMEOUT
    assert "wait" in engine.last_error()
    rows = np.array([0, 1, 2], np.int32)
    cols = np.array([0, 1, 2], np.int32)
    W = np.ones((3, 128), np.float32)
    P, _ = run_plan(engine, 3, 3, rows, cols, W, W, None, 0)
    assert np.array_equal(P, np.full(3, 128.0, np.float32))


# ---- hub-column L2 hints (bit 31 of the plan's column copy) --------------------

@pytest.mark.parametrize("K", [32, 128, 256, 1024])
def test_hub_column_hints_do_not_change_results(engine, K, monkeypatch):
    # force the marks on a small matrix (the default only marks when H exceeds 64 MB): results must be
    # those of the unmarked plan bit for bit, and the oracle's within tolerance
    p = synth.to_numpy(synth.rmat(scale=12, edge_factor=24, K=K, device="cpu"))
    monkeypatch.setenv("SDDMM_L2_HUB_MB", "0")
    P0, info0 = run_plan(engine, p["M"], p["N"], p["rows"], p["cols"], p["W"], p["H"], p["vals"], api.FLAG_KERNEL_RING)
    monkeypatch.setenv("SDDMM_L2_HUB_MB", "1")
    P1, info1 = run_plan(engine, p["M"], p["N"], p["rows"], p["cols"], p["W"], p["H"], p["vals"], api.FLAG_KERNEL_RING)
    assert info0.n_hub_cols == 0
    if p["N"] * K * 4 > (1 << 20):
        assert info1.n_hub_cols > 0
    assert np.array_equal(P0, P1)
    assert_parity(P1, p["rows"], p["cols"], p["W"], p["H"], p["vals"])


# ---- opt-in bfloat16 operand storage -----------------------------------------------

@pytest.mark.parametrize("K", [256, 512, 1024, 2048])
def test_bf16_operand_storage(engine, K):
    """SDDMM_FLAG_OPERANDS_BF16: W and H stored in bfloat16, products and sums in fp32.  Its oracle is the same
    CPU loop run on the operands AFTER rounding to bfloat16 (every bfloat16 is an fp32, so the loop is
    unchanged); with that the usual tolerance applies, 1e-4 max(|ref|, A).  Against the unrounded fp32 operands
    the results differ by the operands' rounding (2^-9 relative each), which is why the flag is opt-in and
    outside the fp32 contract."""
    rng = np.random.default_rng(K)
    M, N = 700, 600
    rows, cols = random_coo(rng, M, N, 70_001, empty_rows=[0, 1, 699])
    vals = rng.standard_normal(rows.shape[0]).astype(np.float32)
    W32 = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda()
    H32 = torch.from_numpy(rng.standard_normal((N, K)).astype(np.float32)).cuda()
    W16, H16 = W32.to(torch.bfloat16), H32.to(torch.bfloat16)
    Wr, Hr = W16.float().cpu().numpy(), H16.float().cpu().numpy()      # what the kernel sees, as fp32
    for col_tile in (0, 128):
        plan = engine.plan_coo(M, N, rows, cols, K, 0, col_tile)
        for sv in (vals, None):
            P = torch.full((rows.shape[0],), float("nan"), device="cuda")
            dS = None if sv is None else torch.from_numpy(sv).cuda()
            plan.execute(W16, H16, P, dS, api.FLAG_OPERANDS_BF16)
            assert plan.last_kernel_name() == "ring (bf16 operands)"
            assert_parity(P.cpu().numpy(), rows, cols, Wr, Hr, sv)
        plan.close()
    # other K, host arrays or a second kernel flag are refused
    plan = engine.plan_coo(M, N, rows, cols, 128)
    with pytest.raises(api.SddmmError) as e:
        plan.execute(W16, H16, P, None, api.FLAG_OPERANDS_BF16)
    assert e.value.status == api.K_UNSUPPORTED
    plan.close()


# ---- host operands: pipelined upload / compute / download ----------------------

def test_host_operand_pipeline_matches_unpipelined(monkeypatch):
    # 256 MB of W triggers the chunked pipeline of sddmm_execute with host operands;
    # its result must equal the one-shot path bit for bit and the oracle within tolerance
    p = synth.to_numpy(synth.rmat(scale=18, edge_factor=6, K=256, device="cpu"))
    outs = []
    for pipeline in ("1", "0"):
        monkeypatch.setenv("SDDMM_PIPELINE", pipeline)
        h = api.Handle(0)
        P, _ = run_plan(h, p["M"], p["N"], p["rows"], p["cols"], p["W"], p["H"], p["vals"])
        P_unscaled, _ = run_plan(h, p["M"], p["N"], p["rows"], p["cols"], p["W"], p["H"], None)
        h.close()
        outs.append((P, P_unscaled))
    assert np.array_equal(outs[0][0], outs[1][0])
    assert np.array_equal(outs[0][1], outs[1][1])
    assert_parity(outs[0][0], p["rows"], p["cols"], p["W"], p["H"], p["vals"])


def test_pinned_host_operands_upload_only_touched_rows(monkeypatch):
    # page-locked W and H: the pipelined call reads just the rows a nonzero touches; the result must be the
    # pageable-memory result bit for bit, and the byte count must be the touched rows' (plus S)
    import torch
    p = synth.to_numpy(synth.rmat(scale=18, edge_factor=6, K=256, device="cpu"))
    K, nnz = 256, p["rows"].shape[0]
    h = api.Handle(0)
    plan = h.plan_coo(p["M"], p["N"], p["rows"], p["cols"], K)
    P_pageable = np.full(nnz, np.nan, np.float32)
    plan.execute(p["W"], p["H"], P_pageable, p["vals"])
    up_pageable, down = plan.last_transfer_bytes()
    Wp = torch.from_numpy(p["W"]).pin_memory()
    Hp = torch.from_numpy(p["H"]).pin_memory()
    Sp = torch.from_numpy(p["vals"]).pin_memory()
    Pp = torch.full((nnz,), float("nan")).pin_memory()
    plan.execute(Wp, Hp, Pp, Sp)
    up_pinned, down2 = plan.last_transfer_bytes()
    info = plan.info()
    n_cols = plan.count_cols()
    plan.close()
    h.close()
    assert down == down2 == 4 * nnz
    assert up_pinned == 4 * K * (info.n_nonempty_rows + n_cols) + 4 * nnz
    assert up_pinned < up_pageable <= 4 * K * (p["M"] + p["N"]) + 4 * nnz
    assert np.array_equal(Pp.numpy(), P_pageable)
    assert_parity(P_pageable, p["rows"], p["cols"], p["W"], p["H"], p["vals"])


def test_used_lines_and_row_upload(engine):
    import torch
    rng = np.random.default_rng(7)
    M, N, K = 300, 200, 36
    rows = np.sort(rng.choice(np.arange(0, M, 3), 900)).astype(np.int32)       # two rows of three stay empty
    cols = rng.choice(np.arange(1, N, 2), 900).astype(np.int32)                 # even columns stay empty
    plan = engine.plan_coo(M, N, rows, cols, K)
    for which, ids_ref, n_lines in ((0, np.unique(rows), M), (1, np.unique(cols), N)):
        ptr, n = plan.used_lines(which)
        assert n == ids_ref.size
        # the list lives in plan-owned device memory: it is checked through what the row upload moves
        host = torch.from_numpy(rng.standard_normal((n_lines, K)).astype(np.float32)).pin_memory()
        dev = torch.zeros((n_lines, K), device="cuda")
        engine.upload_rows(host, dev, ptr, n, K, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        got = dev.cpu().numpy()
        expect = np.zeros((n_lines, K), np.float32)
        expect[ids_ref] = host.numpy()[ids_ref]
        assert np.array_equal(got, expect)        # listed rows arrived, every other row untouched
    # pageable host memory is refused before anything is launched
    with pytest.raises(api.SddmmError):
        engine.upload_rows(np.zeros((M, K), np.float32), torch.zeros((M, K), device="cuda"), plan.used_lines(0)[0], 1, K)
    plan.close()


# ---- col-sorted -> row-sorted conversion on the GPU ------------------------------

@pytest.mark.parametrize("transpose", [False, True])
def test_gpu_coo_sort_equals_host_sort(engine, transpose):
    import torch
    rng = np.random.default_rng(11)
    M, N, nnz = 900, 1300, 60000
    rows = rng.integers(0, M, nnz).astype(np.int32)
    cols = rng.integers(0, N, nnz).astype(np.int32)
    rows[:2000], cols[:2000] = rows[2000:4000], cols[2000:4000]              # duplicates of (row, col) pairs
    vals = rng.standard_normal(nnz).astype(np.float32)
    order = np.lexsort((rows, cols))                                         # the reference's input: sorted by column
    rows, cols, vals = rows[order].copy(), cols[order].copy(), vals[order].copy()
    ref = api.coo_sort_rows(M, N, rows.copy(), cols.copy(), vals.copy(), transpose)
    r, c, v = rows.copy(), cols.copy(), vals.copy()
    m2, n2 = engine.coo_sort_rows(M, N, r, c, v, transpose)                  # host arrays, staged
    assert (m2, n2) == (ref[0], ref[1])
    assert np.array_equal(r, ref[2]) and np.array_equal(c, ref[3]) and np.array_equal(v, ref[4])
    rd, cd, vd = (torch.from_numpy(x.copy()).cuda() for x in (rows, cols, vals))
    engine.coo_sort_rows(M, N, rd, cd, vd, transpose)                        # device arrays, in place
    torch.cuda.synchronize()
    assert np.array_equal(rd.cpu().numpy(), ref[2]) and np.array_equal(cd.cpu().numpy(), ref[3])
    assert np.array_equal(vd.cpu().numpy(), ref[4])


def test_dense_cells_with_columns_unsorted_inside_rows(engine):
    # row-sorted input whose columns are shuffled inside every row: dense cells cannot use their row-mask
    # form (a row's nonzeros are not in column order) and take the per-nonzero lists; results must not change
    p = synth.to_numpy(synth.attention_mask(M=900, half_width=80, n_global=5, K=64, device="cpu"))
    rng = np.random.default_rng(5)
    rows, cols = p["rows"].copy(), p["cols"].copy()
    vals = rng.standard_normal(rows.shape[0]).astype(np.float32)
    P_sorted, info = run_plan(engine, p["M"], p["N"], rows, cols, p["W"], p["H"], vals)
    assert info.n_dense_cells > 0
    order = np.lexsort((rng.random(rows.shape[0]), rows))                    # random order inside each row
    r2, c2, v2 = rows[order], cols[order], vals[order]
    assert np.array_equal(r2, rows) and not np.array_equal(c2, cols)
    P_shuffled, info2 = run_plan(engine, p["M"], p["N"], r2, c2, p["W"], p["H"], v2)
    assert info2.n_dense_cells > 0
    assert_parity(P_shuffled, r2, c2, p["W"], p["H"], v2)
    inv = np.empty_like(order)
    inv[order] = np.arange(order.size)
    # the same values whatever the form (the gathered remainder may round differently with its neighbours)
    assert np.allclose(P_shuffled[inv], P_sorted, rtol=1e-5, atol=1e-5)


# ---- K-major operands (the layout the reference's make_HTasH builds) -------------

@pytest.mark.parametrize("K", [32, 100, 256])
def test_transposed_operands(engine, K):
    import torch
    rng = np.random.default_rng(K)
    M, N = 700, 450
    rows, cols = random_coo(rng, M, N, 9000, empty_rows=(0, 5, 699))
    W = rng.standard_normal((M, K)).astype(np.float32)
    H = rng.standard_normal((N, K)).astype(np.float32)
    vals = rng.standard_normal(rows.shape[0]).astype(np.float32)
    Wt, Ht = oracle.cpu.make_htash(W), oracle.cpu.make_htash(H)
    P_ref, _ = run_plan(engine, M, N, rows, cols, W, H, vals)
    assert_parity(P_ref, rows, cols, W, H, vals)
    plan = engine.plan_coo(M, N, rows, cols, K)
    for w_t, h_t in ((False, True), (True, False), (True, True)):
        flags = (api.FLAG_W_TRANSPOSED if w_t else 0) | (api.FLAG_H_TRANSPOSED if h_t else 0)
        P = np.full(rows.shape[0], np.nan, np.float32)
        plan.execute(Wt if w_t else W, Ht if h_t else H, P, vals, flags)           # host operands
        assert np.array_equal(P, P_ref)
        Wd = torch.from_numpy(np.ascontiguousarray(Wt if w_t else W)).cuda()
        Hd = torch.from_numpy(np.ascontiguousarray(Ht if h_t else H)).cuda()
        Pd = torch.full((rows.shape[0],), float("nan"), device="cuda")
        plan.execute(Wd, Hd, Pd, torch.from_numpy(vals).cuda(), flags)              # device operands
        torch.cuda.synchronize()
        assert np.array_equal(Pd.cpu().numpy(), P_ref)
    plan.close()


# ---- the three dense-cell kernels ---------------------------------------------------

@pytest.mark.parametrize("mode", ["2", "1", "0"])
@pytest.mark.parametrize("K", [16, 64, 100, 256])
def test_dense_cell_variants(monkeypatch, K, mode):
    # 2 = tcgen05 / tensor memory (the default), 1 = mma.sync, 0 = fp32 FMA
    monkeypatch.setenv("SDDMM_DENSE_TENSOR", mode)
    h = api.Handle(0)
    p = synth.to_numpy(synth.attention_mask(M=1100, half_width=96, n_global=7, K=K, device="cpu"))
    rng = np.random.default_rng(K)
    vals = rng.standard_normal(p["rows"].shape[0]).astype(np.float32)
    for sv in (vals, None):
        P, info = run_plan(h, p["M"], p["N"], p["rows"], p["cols"], p["W"], p["H"], sv, 0)
        assert info.n_dense_cells > 0 and 0 < info.n_dense_nnz <= info.nnz
        assert_parity(P, p["rows"], p["cols"], p["W"], p["H"], sv)
    # a plan reused for several calls: tensor memory is allocated and released by every launch
    plan = h.plan_coo(p["M"], p["N"], p["rows"], p["cols"], K)
    outs = []
    for _ in range(3):
        P = np.full(p["rows"].shape[0], np.nan, np.float32)
        plan.execute(p["W"], p["H"], P, vals)
        outs.append(P)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    plan.close()
    h.close()
