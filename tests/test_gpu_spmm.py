"""SpMM on the plan's pattern and the fused SDDMM->SpMM (sddmm_spmm_execute, sddmm_fused_execute) against
the CPU loops oracle_spmm / oracle_spmm_f64.  The reference has no such function, so these oracles are
pinned to their own definition only ("parity unpinned by the reference"); tolerance as for SDDMM:
|gpu - ref| <= 1e-4 max(|ref|, A) per entry of Y, A = sum_i |p_i H[c_i, t]| from the float64 loop."""
import numpy as np
import pytest
import torch

import oracle
from helpers import random_coo
from sddmm_gpu_b200 import api, synth

pytestmark = pytest.mark.gpu
TOL = 1e-4


def _check_y(Y, rows, cols, H, M, pvals, A_extra=None):
    ref = oracle.cpu.spmm(rows, cols, H, M, pvals).astype(np.float64)
    _, A = oracle.cpu.spmm_f64(rows, cols, H, M, None if pvals is None else pvals.astype(np.float64))
    if A_extra is not None:
        A = np.maximum(A, A_extra)
    Y = np.asarray(Y, np.float64)
    assert np.isfinite(Y).all()
    err = np.abs(Y - ref)
    bad = err > TOL * np.maximum(np.abs(ref), A) + 1e-30
    assert not bad.any(), f"{bad.sum()} of {Y.size} entries out of tolerance, worst {np.max(err / np.maximum(A, 1e-30))}"


@pytest.mark.parametrize("K", [4, 32, 64, 100, 128, 256, 260, 512, 1024])
def test_spmm_and_fused_every_k(engine, K):
    rng = np.random.default_rng(K)
    M, N = 300, 257
    rows, cols = random_coo(rng, M, N, 7000, empty_rows=[0, 5, 6, 299], hub_row=17)   # one row holds all N columns
    vals = rng.standard_normal(rows.shape[0]).astype(np.float32)
    W = rng.standard_normal((M, K)).astype(np.float32)
    H = rng.standard_normal((N, K)).astype(np.float32)
    plan = engine.plan_coo(M, N, rows, cols, K)
    # SpMM with given values, and with the bare pattern
    for pv in (vals, None):
        Y = np.full((M, K), np.nan, np.float32)
        plan.spmm(H, Y, pv)
        _check_y(Y, rows, cols, H, M, pv)
    assert plan.last_kernel_name() == "spmm"
    # fused: P = S o (W H^T) never stored ... and stored on request; Y agrees with SpMM over the oracle's P
    for sv in (vals, None):
        P_ref = oracle.cpu.sddmm_coo(rows, cols, W, H, sv)
        P64, A_p = oracle.cpu.sddmm_coo_f64(rows, cols, W, H, sv)
        # an error of 1e-4 A_p in a p_i moves Y by up to that times |H|: part of the scale
        _, A_from_p = oracle.cpu.spmm_f64(rows, cols, H, M, A_p)
        Y = np.full((M, K), np.nan, np.float32)
        P_out = np.full(rows.shape[0], np.nan, np.float32)
        plan.fused(W, H, Y, sv, P_out)
        assert np.all(np.abs(P_out.astype(np.float64) - P64) <= TOL * np.maximum(np.abs(P64), A_p))
        _check_y(Y, rows, cols, H, M, P_ref, A_extra=A_from_p)
        Y2 = np.full((M, K), np.nan, np.float32)
        plan.fused(W, H, Y2, sv)                      # without P_out: the same bits
        assert np.array_equal(Y, Y2)
    assert plan.last_kernel_name() == "fused_sddmm_spmm"
    plan.close()


@pytest.mark.parametrize("K", [256, 512, 1024])
def test_ring_form_for_long_rows(engine, K, monkeypatch):
    """K = 256, 512, 1024 and 65,536 nonzeros or more run on the shared-memory rings over padded row groups:
    empty rows at both ends and in the middle (written as zeros), rows of 1 .. B+1 nonzeros (padding), one row
    holding every column (cut into pieces and summed by the fix-up kernel); against the oracle, and against
    the register-staged kernel (SDDMM_SPMM_RING=0)."""
    rng = np.random.default_rng(7 * K)
    M, N = 900, 700
    rows, cols = random_coo(rng, M, N, 120_000, empty_rows=[0, 1, 2, 450, 451, 898, 899], hub_row=17)
    # a few very short rows
    keep = np.ones(rows.shape[0], bool)
    for r, n_keep in ((100, 1), (101, 2), (102, 3), (103, 5)):
        where = np.nonzero(rows == r)[0]
        keep[where[n_keep:]] = False
    rows, cols = rows[keep], cols[keep]
    vals = rng.standard_normal(rows.shape[0]).astype(np.float32)
    W = rng.standard_normal((M, K)).astype(np.float32)
    H = rng.standard_normal((N, K)).astype(np.float32)
    plan = engine.plan_coo(M, N, rows, cols, K)
    Y = np.full((M, K), np.nan, np.float32)
    plan.spmm(H, Y, vals)
    assert plan.last_kernel_name() == "spmm_ring"
    _check_y(Y, rows, cols, H, M, vals)
    P_ref = oracle.cpu.sddmm_coo(rows, cols, W, H, vals)
    P64, A_p = oracle.cpu.sddmm_coo_f64(rows, cols, W, H, vals)
    _, A_from_p = oracle.cpu.spmm_f64(rows, cols, H, M, A_p)
    Yf = np.full((M, K), np.nan, np.float32)
    P_out = np.full(rows.shape[0], np.nan, np.float32)
    plan.fused(W, H, Yf, vals, P_out)
    assert plan.last_kernel_name() == "fused_sddmm_spmm_ring"
    assert np.all(np.abs(P_out.astype(np.float64) - P64) <= TOL * np.maximum(np.abs(P64), A_p))
    _check_y(Yf, rows, cols, H, M, P_ref, A_extra=A_from_p)
    Yu = np.full((M, K), np.nan, np.float32)
    plan.fused(W, H, Yu, None)                       # unscaled
    _check_y(Yu, rows, cols, H, M, oracle.cpu.sddmm_coo(rows, cols, W, H), A_extra=oracle.cpu.spmm_f64(
        rows, cols, H, M, oracle.cpu.sddmm_coo_f64(rows, cols, W, H)[1])[1])
    plan.close()
    monkeypatch.setenv("SDDMM_SPMM_RING", "0")
    plan = engine.plan_coo(M, N, rows, cols, K)
    Y2 = np.full((M, K), np.nan, np.float32)
    plan.fused(W, H, Y2, vals)
    assert plan.last_kernel_name() == "fused_sddmm_spmm"
    _check_y(Y2, rows, cols, H, M, P_ref, A_extra=A_from_p)
    plan.close()


def test_spmm_unsupported_k_and_empty(engine):
    rows, cols = np.array([0, 1], np.int32), np.array([1, 0], np.int32)
    plan = engine.plan_coo(2, 2, rows, cols, 2048)
    H = np.ones((2, 2048), np.float32)
    with pytest.raises(api.SddmmError) as e:
        plan.spmm(H, np.zeros((2, 2048), np.float32))
    assert e.value.status == api.K_UNSUPPORTED
    plan.close()
    plan = engine.plan_coo(5, 4, np.zeros(0, np.int32), np.zeros(0, np.int32), 8)
    Y = np.full((5, 8), np.nan, np.float32)
    plan.spmm(np.ones((4, 8), np.float32), Y)
    assert np.array_equal(Y, np.zeros((5, 8), np.float32))          # every row written, empty rows are zero
    plan.close()


@pytest.mark.parametrize("name", ["c2", "c3_small", "c4_small", "c5_small"])
def test_fused_on_benchmark_shapes(engine, name):
    if name == "c2":
        p = synth.bag_of_words(device="cuda")
    elif name == "c3_small":
        p = synth.rmat(scale=14, edge_factor=16, K=128, device="cuda")
    elif name == "c4_small":
        p = synth.rmat(scale=15, edge_factor=24, K=256, seed=synth.SEEDS["c4"], device="cuda")   # hub rows: long-row pieces
    else:
        p = synth.attention_mask(M=4096, half_width=64, n_global=12, K=64, device="cuda")
    q = synth.to_numpy(p)
    M, K = p["M"], p["K"]
    plan = engine.plan_coo(M, p["N"], p["rows"], p["cols"], K)
    Y = torch.full((M, K), float("nan"), device="cuda")
    P = torch.full((q["rows"].shape[0],), float("nan"), device="cuda")
    plan.fused(p["W"], p["H"], Y, p["vals"], P)
    P_ref = oracle.cpu.sddmm_coo(q["rows"], q["cols"], q["W"], q["H"], q["vals"])
    P64, A_p = oracle.cpu.sddmm_coo_f64(q["rows"], q["cols"], q["W"], q["H"], q["vals"])
    assert np.all(np.abs(P.cpu().numpy().astype(np.float64) - P64) <= TOL * np.maximum(np.abs(P64), A_p))
    _, A_from_p = oracle.cpu.spmm_f64(q["rows"], q["cols"], q["H"], M, A_p)
    _check_y(Y.cpu().numpy(), q["rows"], q["cols"], q["H"], M, P_ref, A_extra=A_from_p)
    # the unfused pair through the same plan gives the same Y up to rounding of P
    P2 = torch.empty_like(P)
    plan.execute(p["W"], p["H"], P2, p["vals"])
    Y2 = torch.empty_like(Y)
    plan.spmm(p["H"], Y2, P2)
    _check_y(Y2.cpu().numpy(), q["rows"], q["cols"], q["H"], M, P_ref, A_extra=A_from_p)
    plan.close()
