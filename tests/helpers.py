"""Shared pieces of the parity tests."""
import numpy as np

import oracle

REL_TOL = 1e-4  # relative tolerance per nonzero (fp32, reassociated sums)


def random_coo(rng, M, N, nnz, empty_rows=(), hub_row=None):
    """Row-sorted COO without duplicates; optional empty rows / one hub row."""
    nnz = min(nnz, M * N)
    cells = rng.choice(M * N, nnz, replace=False)
    rows, cols = cells // N, cells % N
    keep = ~np.isin(rows, np.asarray(empty_rows, dtype=np.int64))
    rows, cols = rows[keep], cols[keep]
    if hub_row is not None:
        rows = np.concatenate([rows[rows != hub_row], np.full(N, hub_row)])
        cols = np.concatenate([cols[: rows.shape[0] - N], np.arange(N)])
    order = np.lexsort((cols, rows))
    return rows[order].astype(np.int32), cols[order].astype(np.int32)


def assert_parity(P_gpu, rows, cols, W, H, vals=None, tol=REL_TOL):
    """|gpu - ref| <= tol * max(|ref|, A), A = sum_t |w_t h_t| (|s|), ref = the CPU
    oracle (sequential fp32, as the reference); the well-conditioned nonzeros
    (|ref| >= 1e-2 A, i.e. fewer than two digits cancelled) must also meet the plain relative tolerance."""
    ref = oracle.cpu.sddmm_coo(rows, cols, W, H, vals)
    _, A = oracle.cpu.sddmm_coo_f64(rows, cols, W, H, vals)
    P_gpu = np.asarray(P_gpu, dtype=np.float64)
    ref64 = ref.astype(np.float64)
    assert np.isfinite(P_gpu).all(), f"{(~np.isfinite(P_gpu)).sum()} results are not finite (unwritten or NaN)"
    err = np.abs(P_gpu - ref64)
    bound = tol * np.maximum(np.abs(ref64), A)
    bad = np.nonzero(err > bound)[0]
    assert bad.size == 0, (f"{bad.size} of {ref.size} nonzeros out of tolerance; first {bad[:5]}: "
                           f"gpu {P_gpu[bad[:5]]} ref {ref64[bad[:5]]}")
    well = (np.abs(ref64) >= 1e-2 * A) & (np.abs(ref64) > 0)   # an exactly zero S value gives ref = A = 0
    if well.any():
        rel = err[well] / np.abs(ref64[well])
        assert rel.max() <= tol, f"max relative error {rel.max()} on well-conditioned nonzeros"
    return ref
