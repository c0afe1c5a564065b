"""Shared pieces of the parity tests."""
import numpy as np

import oracle

REL_TOL = 1e-4  # relative tolerance per nonzero (fp32, reassociated sums)
# A nonzero is "well-conditioned" when |ref| >= WELL_CONDITIONED * A, A = sum_t |w_t h_t| (|s|): fewer than two
# decimal digits cancelled.  The plain relative tolerance is asserted on those.  Why not 1e-3: an fp32 sum of K
# terms carries an error of about 0.5 eps sqrt(K/2) A / 0.8 sqrt(K) ~ 3e-8 A (rms; a few 1e-7 A in the tail of 10^5
# samples), so at |ref| = 1e-3 A the REFERENCE's own sequential fp32 loop is already off by up to ~2e-4 relative
# against float64 (tests/test_oracle_golden.py::test_fp32_reference_itself_misses_1e4_between_1e3_and_1e2 shows it).
# Nonzeros with 1e-3 A <= |ref| < 1e-2 A are therefore covered by the magnitude-scaled bound only; assert_parity
# returns how many there were (parity_stats) so that a run can print the count.
WELL_CONDITIONED = 1e-2
BAND_LOW = 1e-3
parity_stats = {"checked": 0, "well_conditioned": 0, "between_1e-3_and_1e-2": 0, "below_1e-3": 0}


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
    (|ref| >= 1e-2 A, i.e. fewer than two digits cancelled) must also meet the plain relative tolerance;
    see WELL_CONDITIONED above for the nonzeros between 1e-3 A and 1e-2 A."""
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
    well = (np.abs(ref64) >= WELL_CONDITIONED * A) & (np.abs(ref64) > 0)   # an exactly zero S value gives ref = A = 0
    band = (~well) & (np.abs(ref64) >= BAND_LOW * A) & (np.abs(ref64) > 0)
    parity_stats["checked"] += int(ref.size)
    parity_stats["well_conditioned"] += int(well.sum())
    parity_stats["between_1e-3_and_1e-2"] += int(band.sum())
    parity_stats["below_1e-3"] += int(ref.size - well.sum() - band.sum())
    if well.any():
        rel = err[well] / np.abs(ref64[well])
        assert rel.max() <= tol, f"max relative error {rel.max()} on well-conditioned nonzeros"
    return ref
