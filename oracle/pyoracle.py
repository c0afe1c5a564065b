"""ctypes bindings of the CPU oracle and of the reference-built checker.

Test infrastructure only (see ``oracle/__init__.py``).  Arrays are numpy,
C-contiguous; indices are int32 as in the reference's ``Matrix`` type
(HiPC18/src/util.h:21-31), values float32.
"""
import ctypes as C
import os
import subprocess
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_CPU_SO = os.path.join(_HERE, "liboracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libsddmm_ref.so")

_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(np.int64, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")


def build(verbose=False):
    """Compile liboracle.so and, if the reference tree is present, _ref/."""
    out = subprocess.run(["make", "-C", _HERE], capture_output=True, text=True)
    if verbose or out.returncode != 0:
        print(out.stdout, out.stderr)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed")


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _opt(a, ptr_type):
    """None -> NULL pointer, array -> its data pointer."""
    if a is None:
        return None
    return a.ctypes.data_as(ptr_type)


class CpuOracle:
    """The plain-C restatement (sddmm_oracle.c)."""

    def __init__(self, lib):
        self.lib = lib
        L = lib
        L.oracle_max_threads.restype = C.c_int
        L.oracle_sddmm_coo.restype = C.c_double
        L.oracle_sddmm_coo.argtypes = [_i32p, _i32p, C.c_int64, _f32p, _f32p, C.c_int, _f32p, C.c_int]
        L.oracle_sddmm_csr.restype = C.c_double
        L.oracle_sddmm_csr.argtypes = [_i64p, _i32p, _f32p, C.c_int64, _f32p, _f32p, C.c_int, _f32p, C.c_int]
        L.oracle_sddmm_coo_scaled.restype = C.c_double
        L.oracle_sddmm_coo_scaled.argtypes = [_i32p, _i32p, C.c_void_p, C.c_int64, _f32p, _f32p, C.c_int, _f32p, C.c_int]
        L.oracle_sddmm_coo_f64.restype = None
        L.oracle_sddmm_coo_f64.argtypes = [_i32p, _i32p, C.c_void_p, C.c_int64, _f32p, _f32p, C.c_int, _f64p, _f64p, C.c_int]
        L.oracle_initial.restype = None
        L.oracle_spmm.restype = None
        L.oracle_spmm.argtypes = [_i32p, _i32p, C.c_void_p, C.c_int64, C.c_int64, _f32p, C.c_int, _f32p, C.c_int]
        L.oracle_spmm_f64.restype = None
        L.oracle_spmm_f64.argtypes = [_i32p, _i32p, C.c_void_p, C.c_int64, C.c_int64, _f32p, C.c_int, _f64p, _f64p, C.c_int]
        L.oracle_initial.argtypes = [_f32p, C.c_int64, C.c_int]
        L.oracle_make_htash.restype = None
        L.oracle_make_htash.argtypes = [_f32p, _f32p, C.c_int64, C.c_int]
        L.oracle_make_csr.restype = C.c_int64
        L.oracle_make_csr.argtypes = [_i32p, C.c_int64, C.c_int64, _i32p, _i32p]
        L.oracle_rewrite_matrix_1d.restype = C.c_int32
        L.oracle_rewrite_matrix_1d.argtypes = [
            _i32p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, _i32p, _i32p, C.c_int64,
            C.c_int, C.c_int, _i32p, _i32p, _f32p, _i32p, _i32p, _i32p, _i32p, _i32p]
        L.oracle_unsorted_make_csr.restype = C.c_int64
        L.oracle_unsorted_make_csr.argtypes = [_i32p, _i32p, _f32p, C.c_int64, C.c_int64, C.c_int64, _i32p, C.c_int]
        L.oracle_make_csc_cuts.restype = C.c_int
        L.oracle_make_csc_cuts.argtypes = [_i32p, C.c_int64, C.c_int64, C.c_int, _i32p, _i32p]

    def max_threads(self):
        return int(self.lib.oracle_max_threads())

    def sddmm_coo(self, rows, cols, W, H, vals=None, threads=0, return_seconds=False):
        """P[i] = dot(W[rows[i]], H[cols[i]]) (* vals[i] when given)."""
        rows, cols, W, H = _i32(rows), _i32(cols), _f32(W), _f32(H)
        k = W.shape[1]
        P = np.empty(rows.shape[0], np.float32)
        if vals is None:
            s = self.lib.oracle_sddmm_coo(rows, cols, rows.shape[0], W, H, k, P, threads)
        else:
            vals = _f32(vals)
            s = self.lib.oracle_sddmm_coo_scaled(rows, cols, vals.ctypes.data, rows.shape[0], W, H, k, P, threads)
        return (P, s) if return_seconds else P

    def sddmm_csr(self, row_ptr, cols, vals, W, H, threads=0):
        row_ptr = np.ascontiguousarray(row_ptr, np.int64)
        cols, vals, W, H = _i32(cols), _f32(vals), _f32(W), _f32(H)
        P = np.empty(cols.shape[0], np.float32)
        self.lib.oracle_sddmm_csr(row_ptr, cols, vals, row_ptr.shape[0] - 1, W, H, W.shape[1], P, threads)
        return P

    def sddmm_coo_f64(self, rows, cols, W, H, vals=None, threads=0):
        """float64 result and the magnitude scale A = sum_t |w_t h_t| (|s|)."""
        rows, cols, W, H = _i32(rows), _i32(cols), _f32(W), _f32(H)
        n = rows.shape[0]
        P = np.empty(n, np.float64)
        A = np.empty(n, np.float64)
        vp = None
        if vals is not None:
            vals = _f32(vals)
            vp = vals.ctypes.data
        self.lib.oracle_sddmm_coo_f64(rows, cols, vp, n, W, H, W.shape[1], P, A, threads)
        return P, A

    def spmm(self, rows, cols, H, M, pvals=None, threads=0):
        """Y = P H on the pattern (rows sorted): fp32, nonzeros of a row added in input order.  No counterpart in
        the reference."""
        rows, cols, H = _i32(rows), _i32(cols), _f32(H)
        Y = np.empty((M, H.shape[1]), np.float32)
        pp = None
        if pvals is not None:
            pvals = _f32(pvals)
            pp = pvals.ctypes.data
        self.lib.oracle_spmm(rows, cols, pp, rows.shape[0], M, H, H.shape[1], Y, threads)
        return Y

    def spmm_f64(self, rows, cols, H, M, pvals64=None, threads=0):
        """float64 Y and the magnitude scale A[r, t] = sum_i |p_i H[c_i, t]| (pvals64: float64 or None)."""
        rows, cols, H = _i32(rows), _i32(cols), _f32(H)
        Y = np.empty((M, H.shape[1]), np.float64)
        A = np.empty((M, H.shape[1]), np.float64)
        pp = None
        if pvals64 is not None:
            pvals64 = np.ascontiguousarray(pvals64, np.float64)
            pp = pvals64.ctypes.data
        self.lib.oracle_spmm_f64(rows, cols, pp, rows.shape[0], M, H, H.shape[1], Y, A, threads)
        return Y, A

    def initial(self, n, k):
        X = np.empty((n, k), np.float32)
        self.lib.oracle_initial(X, n, k)
        return X

    def make_htash(self, H):
        """K-major copy of an (n, k) operand: the reference's make_HTasH."""
        H = _f32(H)
        n, k = H.shape
        Ht = np.empty((k, n), np.float32)
        self.lib.oracle_make_htash(H, Ht, n, k)
        return Ht

    def make_csr(self, rows, n_rows):
        rows = _i32(rows)
        row_ptr = np.empty(n_rows + 2, np.int32)
        row_holder = np.empty(n_rows + 1, np.int32)
        n_holder = self.lib.oracle_make_csr(rows, rows.shape[0], n_rows, row_ptr, row_holder)
        return row_ptr, row_holder, int(n_holder)

    def rewrite_matrix_1d(self, rows, cols, vals, n_rows, n_cols, panel_rows, col_tile):
        """Reference tiling tables for CLI arguments (argv[3]=panel_rows, argv[4]=col_tile)."""
        rows, cols = _i32(rows), _i32(cols)
        nnz = rows.shape[0]
        row_ptr, row_holder, n_holder = self.make_csr(rows, n_rows)
        ntile_c = n_cols // col_tile + 1
        max_blk = n_rows // panel_rows + 1
        out = dict(
            rows=np.zeros(nnz, np.int32), cols=np.zeros(nnz, np.int32),
            vals=np.zeros(nnz, np.float32), tiled_ind=np.zeros(nnz, np.int32),
            lastIdx_tile=np.zeros(ntile_c + 1, np.int32),
            lastIdx_block_tile=np.zeros((ntile_c + 1) * max_blk, np.int32),
            active_row=np.zeros(n_rows * ntile_c, np.int32),
            n_actv_row=np.zeros(ntile_c, np.int32))
        vp = None
        if vals is not None:
            vals = _f32(vals)
            vp = vals.ctypes.data
        mar = self.lib.oracle_rewrite_matrix_1d(
            cols, vp, nnz, n_rows, n_cols, row_ptr, row_holder, n_holder, col_tile, panel_rows,
            out["rows"], out["cols"], out["vals"], out["tiled_ind"], out["lastIdx_tile"],
            out["lastIdx_block_tile"], out["active_row"], out["n_actv_row"])
        out["max_active_row"] = int(mar)
        out["ntile_c"] = ntile_c
        out["max_active_block"] = max_blk
        return out

    def unsorted_make_csr(self, rows, cols, vals, n_rows, n_cols, transpose=True):
        rows, cols, vals = _i32(rows).copy(), _i32(cols).copy(), _f32(vals).copy()
        row_ptr = np.zeros(n_rows + 1, np.int32)
        n = self.lib.oracle_unsorted_make_csr(rows, cols, vals, rows.shape[0], n_rows, n_cols, row_ptr, int(transpose))
        return rows, cols, vals, row_ptr, int(n)

    def make_csc_cuts(self, cols, n_cols, n_p):
        cols = _i32(cols)
        cir = np.zeros(n_p + 2, np.int32)
        nir = np.zeros(n_p + 2, np.int32)
        t = self.lib.oracle_make_csc_cuts(cols, cols.shape[0], n_cols, n_p, cir, nir)
        return cir[:t].copy(), nir[:t].copy()


class RefChecker:
    """The reference's own code (HiPC18/src/sddmm.cu + util.h) through ref_bridge.cu."""

    def __init__(self, lib):
        self.lib = lib
        L = lib
        L.ref_sddmm_cpu_coo.restype = C.c_double
        L.ref_sddmm_cpu_coo.argtypes = [_i32p, _i32p, _f32p, C.c_long, C.c_long, C.c_long, _f32p, _f32p, C.c_int, _f32p]
        L.ref_coo_state_create.restype = C.c_void_p
        L.ref_coo_state_create.argtypes = [_i32p, _i32p, _f32p, C.c_long, C.c_long, C.c_long, _f32p, _f32p, C.c_int]
        L.ref_coo_state_run.restype = C.c_double
        L.ref_coo_state_run.argtypes = [C.c_void_p, C.c_long]
        L.ref_coo_state_result.restype = None
        L.ref_coo_state_result.argtypes = [C.c_void_p, _f32p, C.c_long]
        L.ref_coo_state_destroy.restype = None
        L.ref_coo_state_destroy.argtypes = [C.c_void_p]
        L.ref_sddmm_cpu_csr.restype = None
        L.ref_sddmm_cpu_csr.argtypes = [_i32p, _i32p, _f32p, C.c_long, C.c_long, C.c_long, _f32p, _f32p, C.c_int, _f32p]
        L.ref_initial.restype = None
        L.ref_initial.argtypes = [_f32p, C.c_long, C.c_int]
        if hasattr(L, "ref_make_htash"):
            L.ref_make_htash.restype = None
            L.ref_make_htash.argtypes = [_f32p, _f32p, C.c_long, C.c_int]
        L.ref_make_csr.restype = None
        L.ref_make_csr.argtypes = [_i32p, C.c_long, C.c_long, _i32p, _i32p]
        L.ref_rewrite_matrix_1d.restype = C.c_int
        L.ref_rewrite_matrix_1d.argtypes = [
            _i32p, _i32p, _f32p, C.c_long, C.c_long, C.c_long, C.c_int, C.c_int,
            _i32p, _i32p, _f32p, _i32p, _i32p, _i32p, _i32p, _i32p, _i32p]
        L.ref_unsorted_make_csr.restype = C.c_int
        L.ref_unsorted_make_csr.argtypes = [_i32p, _i32p, _f32p, C.c_long, C.c_long, C.c_long, _i32p, C.c_char_p]

    def sddmm_cpu_coo(self, rows, cols, vals, n_rows, n_cols, W, H):
        rows, cols, vals, W, H = _i32(rows), _i32(cols), _f32(vals), _f32(W), _f32(H)
        P = np.zeros(max(rows.shape[0], 1), np.float32)
        self.lib.ref_sddmm_cpu_coo(rows, cols, vals, rows.shape[0], n_rows, n_cols, W, H, W.shape[1], P)
        return P[:rows.shape[0]]

    def timed_cpu_coo(self, rows, cols, vals, n_rows, n_cols, W, H, repeats=3):
        """Best-of-`repeats` seconds of the reference's sddmm_CPU_COO over all the
        nonzeros, and of the same call over zero nonzeros (its by-value argument
        copies alone, which the reference's own timer excludes)."""
        rows, cols, vals, W, H = _i32(rows), _i32(cols), _f32(vals), _f32(W), _f32(H)
        st = self.lib.ref_coo_state_create(rows, cols, vals, rows.shape[0], n_rows, n_cols, W, H, W.shape[1])
        try:
            full = min(self.lib.ref_coo_state_run(st, rows.shape[0]) for _ in range(repeats))
            copy = min(self.lib.ref_coo_state_run(st, 0) for _ in range(repeats))
            P = np.zeros(max(rows.shape[0], 1), np.float32)
            self.lib.ref_coo_state_result(st, P, rows.shape[0])
        finally:
            self.lib.ref_coo_state_destroy(st)
        return full, copy, P[:rows.shape[0]]

    def sddmm_cpu_csr(self, row_ptr, cols, vals, n_rows, n_cols, W, H):
        row_ptr, cols, vals, W, H = _i32(row_ptr), _i32(cols), _f32(vals), _f32(W), _f32(H)
        P = np.zeros(max(cols.shape[0], 1), np.float32)
        self.lib.ref_sddmm_cpu_csr(row_ptr, cols, vals, cols.shape[0], n_rows, n_cols, W, H, W.shape[1], P)
        return P[:cols.shape[0]]

    def spmm(self, rows, cols, H, M, pvals=None, threads=0):
        """Y = P H on the pattern (rows sorted): fp32, nonzeros of a row added in input order.  No counterpart in
        the reference."""
        rows, cols, H = _i32(rows), _i32(cols), _f32(H)
        Y = np.empty((M, H.shape[1]), np.float32)
        pp = None
        if pvals is not None:
            pvals = _f32(pvals)
            pp = pvals.ctypes.data
        self.lib.oracle_spmm(rows, cols, pp, rows.shape[0], M, H, H.shape[1], Y, threads)
        return Y

    def spmm_f64(self, rows, cols, H, M, pvals64=None, threads=0):
        """float64 Y and the magnitude scale A[r, t] = sum_i |p_i H[c_i, t]| (pvals64: float64 or None)."""
        rows, cols, H = _i32(rows), _i32(cols), _f32(H)
        Y = np.empty((M, H.shape[1]), np.float64)
        A = np.empty((M, H.shape[1]), np.float64)
        pp = None
        if pvals64 is not None:
            pvals64 = np.ascontiguousarray(pvals64, np.float64)
            pp = pvals64.ctypes.data
        self.lib.oracle_spmm_f64(rows, cols, pp, rows.shape[0], M, H, H.shape[1], Y, A, threads)
        return Y, A

    def initial(self, n, k):
        X = np.empty((n, k), np.float32)
        self.lib.ref_initial(X, n, k)
        return X

    def make_htash(self, H):
        H = _f32(H)
        n, k = H.shape
        Ht = np.empty((k, n), np.float32)
        self.lib.ref_make_htash(H, Ht, n, k)
        return Ht

    def make_csr(self, rows, n_rows):
        rows = _i32(rows)
        row_ptr = np.zeros(n_rows + 2, np.int32)
        row_holder = np.zeros(n_rows + 1, np.int32)
        self.lib.ref_make_csr(rows, rows.shape[0], n_rows, row_ptr, row_holder)
        return row_ptr, row_holder

    def rewrite_matrix_1d(self, rows, cols, vals, n_rows, n_cols, panel_rows, col_tile):
        rows, cols, vals = _i32(rows), _i32(cols), _f32(vals)
        nnz = rows.shape[0]
        ntile_c = n_cols // col_tile + 1
        max_blk = n_rows // panel_rows + 1
        out = dict(
            rows=np.zeros(nnz, np.int32), cols=np.zeros(nnz, np.int32),
            vals=np.zeros(nnz, np.float32), tiled_ind=np.zeros(nnz, np.int32),
            lastIdx_tile=np.zeros(ntile_c + 1, np.int32),
            lastIdx_block_tile=np.zeros((ntile_c + 1) * max_blk, np.int32),
            active_row=np.zeros(n_rows * ntile_c, np.int32),
            n_actv_row=np.zeros(ntile_c, np.int32))
        sizes = np.zeros(2, np.int32)
        mar = self.lib.ref_rewrite_matrix_1d(
            rows, cols, vals, nnz, n_rows, n_cols, panel_rows, col_tile,
            out["rows"], out["cols"], out["vals"], out["tiled_ind"], out["lastIdx_tile"],
            out["lastIdx_block_tile"], out["active_row"], out["n_actv_row"], sizes)
        assert sizes[0] == ntile_c and sizes[1] == max_blk
        out["max_active_row"] = int(mar)
        out["ntile_c"] = ntile_c
        out["max_active_block"] = max_blk
        return out

    def unsorted_make_csr(self, rows, cols, vals, n_rows, n_cols):
        rows, cols, vals = _i32(rows).copy(), _i32(cols).copy(), _f32(vals).copy()
        row_ptr = np.zeros(n_rows + 1, np.int32)
        with tempfile.TemporaryDirectory() as d:
            rc = self.lib.ref_unsorted_make_csr(rows, cols, vals, rows.shape[0], n_rows, n_cols, row_ptr, d.encode())
            assert rc == 0
            with open(os.path.join(d, "nytimes_tans.txt")) as f:
                dump = f.read()
        return rows, cols, vals, row_ptr, dump


def load_cpu():
    if not os.path.exists(_CPU_SO):
        build()
    return CpuOracle(C.CDLL(_CPU_SO))


def load_ref():
    if not os.path.exists(_REF_SO):
        return None
    return RefChecker(C.CDLL(_REF_SO))
