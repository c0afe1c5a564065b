"""Generates the golden fixtures of this directory from the REFERENCE ITSELF.

Run in a container that has the reference tree (the build recipe in oracle/
compiles its translation unit into oracle/_ref/libsddmm_ref.so):

    python tests/golden/make_golden.py

Each .npz holds the seeded inputs and what the reference's own functions
(HiPC18/src/sddmm.cu, util.h) returned for them.  The fixtures travel with the
repository; the reference does not have to be present to check against them.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402


def coo(rng, M, N, nnz, empty_rows=()):
    cells = np.sort(rng.choice(M * N, nnz, replace=False))
    rows, cols = cells // N, cells % N
    keep = ~np.isin(rows, np.asarray(empty_rows, dtype=np.int64))
    return rows[keep].astype(np.int32), cols[keep].astype(np.int32)


def main():
    ref = oracle.ref
    assert ref is not None, "oracle/_ref/libsddmm_ref.so is missing (run make -C oracle)"
    rng = np.random.default_rng(20181217)

    # 1. SDDMM values: sddmm_CPU_COO (unscaled) and sddmm_CPU_CSR (scaled by S)
    for tag, (M, N, K, nnz, dist) in {
        "uniform_k32": (96, 80, 32, 1201, "uniform"),
        "normal_k100": (64, 120, 100, 1999, "normal"),
        "counts_k256": (50, 40, 256, 777, "uniform"),
    }.items():
        rows, cols = coo(rng, M, N, nnz)
        vals = rng.integers(1, 21, rows.shape[0]).astype(np.float32)
        if dist == "uniform":
            W = rng.random((M, K), dtype=np.float32)
            H = rng.random((N, K), dtype=np.float32)
        else:
            W = (rng.standard_normal((M, K)) * 0.1).astype(np.float32)
            H = (rng.standard_normal((N, K)) * 0.1).astype(np.float32)
        row_ptr = np.zeros(M + 1, np.int64)
        np.add.at(row_ptr, rows.astype(np.int64) + 1, 1)
        row_ptr = np.cumsum(row_ptr)
        np.savez_compressed(
            os.path.join(HERE, f"sddmm_{tag}.npz"), M=M, N=N, K=K, rows=rows, cols=cols, vals=vals, W=W, H=H,
            row_ptr=row_ptr,
            P_coo=ref.sddmm_cpu_coo(rows, cols, vals, M, N, W, H),
            P_csr=ref.sddmm_cpu_csr(row_ptr.astype(np.int32), cols, vals, M, N, W, H))

    # 2. tiling tables: make_CSR + TiledMatrix + rewrite_matrix_1D for CLI (argv[3], argv[4]) pairs
    M, N, nnz = 120, 90, 1501
    rows, cols = coo(rng, M, N, nnz)
    vals = rng.integers(1, 21, rows.shape[0]).astype(np.float32)
    out = dict(M=M, N=N, rows=rows, cols=cols, vals=vals)
    pairs = [(32, 4096), (16, 30), (7, 33), (192, 50000), (1, 1), (24, 45)]
    out["pairs"] = np.array(pairs, np.int32)
    for i, (pr, ct) in enumerate(pairs):
        t = ref.rewrite_matrix_1d(rows, cols, vals, M, N, pr, ct)
        for k, v in t.items():
            out[f"t{i}_{k}"] = np.asarray(v)
    rp, rh = ref.make_csr(rows, M)
    out["csr_row_ptr"], out["csr_row_holder"] = rp, rh
    np.savez_compressed(os.path.join(HERE, "tiling.npz"), **out)

    # 3. dense operand init (srand48(0); 0.1*drand48())
    np.savez_compressed(os.path.join(HERE, "initial.npz"), X=ref.initial(40, 12))

    # 4. column-sorted -> row-sorted conversion (transposing, 1-based output, file dump)
    M, N, nnz = 70, 50, 601   # N <= M: the regime in which the reference keeps every entry
    rows, cols = coo(rng, M, N, nnz)
    vals = rng.integers(1, 21, rows.shape[0]).astype(np.float32)
    order = np.lexsort((rows, cols))
    r_in, c_in, v_in = rows[order], cols[order], vals[order]
    r_out, c_out, v_out, row_ptr, dump = ref.unsorted_make_csr(r_in, c_in, v_in, M, N)
    np.savez_compressed(os.path.join(HERE, "convert.npz"), M=M, N=N, rows_in=r_in, cols_in=c_in, vals_in=v_in,
                        rows_out=r_out, cols_out=c_out, vals_out=v_out, row_ptr=row_ptr,
                        dump_head=np.array(dump.splitlines()[:4]))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
