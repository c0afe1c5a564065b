"""ctypes binding of ``libsddmm_b200.so`` -- the C ABI declared in
``include/sddmm_b200.h``.

This is the host-side mirror a Python caller uses; it adds nothing to the C ABI
except argument marshalling.  Pointers may be numpy arrays (host), torch tensors
(host or CUDA) or raw integer addresses.  There is no CPU fallback: without the
built library (or without a GPU, for the compute calls) everything here raises.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# SDDMM_B200_LIBRARY: another build of the same library (e.g. one compiled with different tuning macros)
LIB_PATH = os.environ.get("SDDMM_B200_LIBRARY") or os.path.join(_HERE, "csrc", "libsddmm_b200.so")

# status codes (include/sddmm_b200.h)
OK, INVALID_ARG, UNSORTED_INPUT, INDEX_OUT_OF_RANGE, K_UNSUPPORTED, CUDA_ERROR, NCCL_ERROR, \
    OUT_OF_MEMORY, DEVICE_TIMEOUT, IO_ERROR, PARSE_ERROR, NO_DEVICE = range(12)

FLAG_ASYNC = 0x1
FLAG_TILED_ORDER = 0x2
FLAG_H_TRANSPOSED = 0x4
FLAG_W_TRANSPOSED = 0x8
FLAG_KERNEL_GATHER = 0x10
FLAG_KERNEL_PANEL = 0x20
FLAG_KERNEL_RING = 0x40
FLAG_OPERANDS_BF16 = 0x100
PLAN_SKIP_VALIDATION = 0x1
PLAN_DEVICE_INDICES = 0x2
PLAN_FORCE_H_CHUNKS = 0x4

EXPORTED_SYMBOLS = [
    "sddmm_status_string", "sddmm_create", "sddmm_destroy", "sddmm_last_error", "sddmm_set_stream",
    "sddmm_plan_coo", "sddmm_destroy_plan", "sddmm_execute", "sddmm_last_kernel_ms", "sddmm_last_transfer_bytes", "sddmm_plan_used_lines", "sddmm_upload_rows", "sddmm_coo",
    "sddmm_selftest_wait_timeout", "sddmm_plan_get_info", "sddmm_plan_count_cols", "sddmm_count_cols_noalloc", "sddmm_plan_export_row_ptr",
    "sddmm_plan_export_tiling", "sddmm_partition_rows", "sddmm_partition_rows_weighted", "sddmm_mtx_open", "sddmm_mtx_read",
    "sddmm_spmm_execute", "sddmm_fused_execute", "sddmm_last_kernel_name", "sddmm_kernel_launches", "sddmm_sync", "sddmm_check_result", "sddmm_selftest_optin_cache",
    "sddmm_comm_unique_id", "sddmm_comm_create", "sddmm_comm_destroy", "sddmm_comm_broadcast", "sddmm_comm_all_gather",
    "sddmm_dist_plan_coo", "sddmm_dist_plan_coo_shares", "sddmm_partition_rows_shares", "sddmm_dist_plan_destroy", "sddmm_dist_plan_get_shard", "sddmm_dist_plan_local",
    "sddmm_dist_execute", "sddmm_dist_last_times", "sddmm_multi_create", "sddmm_multi_destroy", "sddmm_multi_last_error",
    "sddmm_multi_plan_coo", "sddmm_multi_plan_destroy", "sddmm_multi_plan_get_cuts", "sddmm_multi_execute",
    "sddmm_multi_last_kernel_ms",
    "sddmm_mtx_close", "sddmm_mtx_open_ex", "sddmm_coo_save_binary", "sddmm_coo_sort_rows_gpu", "sddmm_gen_open", "sddmm_coo_is_row_sorted", "sddmm_mtx_write", "sddmm_coo_sort_rows",
]


class SddmmError(RuntimeError):
    def __init__(self, status, detail=""):
        self.status = status
        msg = lib().sddmm_status_string(status).decode()
        super().__init__(f"sddmm status {status} ({msg})" + (f": {detail}" if detail else ""))


class PlanInfo(C.Structure):
    _fields_ = [("M", C.c_int64), ("N", C.c_int64), ("nnz", C.c_int64), ("K", C.c_int32),
                ("panel_rows", C.c_int32), ("col_tile", C.c_int32), ("n_col_tiles", C.c_int32),
                ("n_work_items", C.c_int64), ("n_nonempty_rows", C.c_int64),
                ("n_nonempty_cols", C.c_int64), ("device_bytes", C.c_int64), ("plan_ms", C.c_float),
                ("reserved0", C.c_int32), ("n_dense_cells", C.c_int64), ("n_dense_nnz", C.c_int64),
                ("n_hub_cols", C.c_int64)]


_lib = None


def lib():
    """The loaded shared library.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `make -C sddmm_gpu_b200/csrc` "
            "(or __graft_entry__.build()).  There is no CPU fallback.")
    L = C.CDLL(LIB_PATH)
    vp, i64, i32, u32 = C.c_void_p, C.c_int64, C.c_int32, C.c_uint32
    L.sddmm_status_string.restype = C.c_char_p
    L.sddmm_status_string.argtypes = [C.c_int]
    L.sddmm_create.argtypes = [C.POINTER(vp), C.c_int]
    L.sddmm_destroy.argtypes = [vp]
    L.sddmm_last_error.restype = C.c_char_p
    L.sddmm_last_error.argtypes = [vp]
    L.sddmm_set_stream.argtypes = [vp, vp]
    L.sddmm_plan_coo.argtypes = [vp, i64, i64, i64, vp, vp, C.c_int, C.c_int, C.c_int, u32, C.POINTER(vp)]
    L.sddmm_destroy_plan.argtypes = [vp]
    L.sddmm_execute.argtypes = [vp, vp, vp, vp, vp, u32]
    L.sddmm_last_kernel_ms.argtypes = [vp, C.POINTER(C.c_float)]
    L.sddmm_last_kernel_name.restype = C.c_char_p
    L.sddmm_last_kernel_name.argtypes = [vp]
    L.sddmm_spmm_execute.argtypes = [vp, vp, vp, vp, u32]
    L.sddmm_fused_execute.argtypes = [vp, vp, vp, vp, vp, vp, u32]
    L.sddmm_sync.argtypes = [vp]
    L.sddmm_kernel_launches.argtypes = [vp, C.POINTER(i64)]
    L.sddmm_check_result.argtypes = [vp, vp, vp, vp, vp, i64, C.c_double, C.POINTER(C.c_double), C.POINTER(i64),
                                     C.POINTER(i64)]
    L.sddmm_selftest_optin_cache.argtypes = []
    L.sddmm_comm_unique_id.argtypes = [vp]
    L.sddmm_comm_create.argtypes = [vp, vp, C.c_int, C.c_int, C.POINTER(vp)]
    L.sddmm_comm_destroy.argtypes = [vp]
    L.sddmm_comm_broadcast.argtypes = [vp, vp, i64, C.c_int, vp]
    L.sddmm_comm_all_gather.argtypes = [vp, vp, i64, vp]
    L.sddmm_dist_plan_coo.argtypes = [vp, i64, i64, i64, vp, vp, C.c_int, C.c_int, C.c_int, u32, C.POINTER(vp)]
    L.sddmm_dist_plan_coo_shares.argtypes = [vp, i64, i64, i64, vp, vp, C.c_int, C.c_int, C.c_int, vp, u32, C.POINTER(vp)]
    L.sddmm_partition_rows_shares.argtypes = [i64, i64, vp, C.c_int, C.c_int, vp, vp, vp]
    L.sddmm_dist_plan_destroy.argtypes = [vp]
    L.sddmm_dist_plan_get_shard.argtypes = [vp, C.POINTER(i64), C.POINTER(i64), C.POINTER(i64), C.POINTER(i64),
                                            C.POINTER(i32)]
    L.sddmm_dist_plan_local.restype = vp
    L.sddmm_dist_plan_local.argtypes = [vp]
    L.sddmm_dist_execute.argtypes = [vp, vp, vp, vp, vp, C.c_int, u32]
    L.sddmm_dist_last_times.argtypes = [vp, C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float)]
    L.sddmm_multi_create.argtypes = [vp, C.c_int, C.POINTER(vp)]
    L.sddmm_multi_destroy.argtypes = [vp]
    L.sddmm_multi_last_error.restype = C.c_char_p
    L.sddmm_multi_last_error.argtypes = [vp]
    L.sddmm_multi_plan_coo.argtypes = [vp, i64, i64, i64, vp, vp, C.c_int, C.c_int, u32, C.POINTER(vp)]
    L.sddmm_multi_plan_destroy.argtypes = [vp]
    L.sddmm_multi_plan_get_cuts.argtypes = [vp, vp, vp]
    L.sddmm_multi_execute.argtypes = [vp, vp, vp, vp, vp, u32]
    L.sddmm_multi_last_kernel_ms.argtypes = [vp, C.POINTER(C.c_float)]
    L.sddmm_last_transfer_bytes.argtypes = [vp, C.POINTER(i64), C.POINTER(i64)]
    L.sddmm_plan_used_lines.argtypes = [vp, C.c_int, C.POINTER(vp), C.POINTER(i64)]
    L.sddmm_upload_rows.argtypes = [vp, vp, vp, vp, i64, C.c_int, vp]
    L.sddmm_coo.argtypes = [vp, i64, i64, i64, vp, vp, vp, vp, vp, C.c_int, vp]
    L.sddmm_selftest_wait_timeout.argtypes = [vp]
    L.sddmm_plan_get_info.argtypes = [vp, C.POINTER(PlanInfo)]
    L.sddmm_plan_count_cols.argtypes = [vp, C.POINTER(i64)]
    L.sddmm_count_cols_noalloc.argtypes = [C.c_int, vp, i64, i64, vp, C.POINTER(i64), C.c_char_p, C.c_int]
    L.sddmm_plan_export_row_ptr.argtypes = [vp, vp]
    L.sddmm_plan_export_tiling.argtypes = [vp, C.c_int, C.c_int, vp, vp, vp, vp, vp, vp, vp, C.POINTER(i32)]
    L.sddmm_partition_rows.argtypes = [i64, i64, vp, C.c_int, C.c_int, vp, vp]
    L.sddmm_partition_rows_weighted.argtypes = [i64, i64, vp, C.c_int, C.c_int, C.c_double, vp, vp]
    L.sddmm_mtx_open.argtypes = [C.c_char_p, C.POINTER(vp), C.POINTER(i64), C.POINTER(i64), C.POINTER(i64),
                                 C.c_char_p, C.c_int]
    L.sddmm_mtx_open_ex.argtypes = [C.c_char_p, u32, C.POINTER(vp), C.POINTER(i64), C.POINTER(i64), C.POINTER(i64),
                                    C.c_char_p, C.c_int]
    L.sddmm_coo_save_binary.argtypes = [C.c_char_p, i64, i64, i64, vp, vp, vp]
    L.sddmm_coo_sort_rows_gpu.argtypes = [vp, C.POINTER(i64), C.POINTER(i64), i64, vp, vp, vp, C.c_int]
    L.sddmm_gen_open.argtypes = [C.c_char_p, C.POINTER(vp), C.POINTER(i64), C.POINTER(i64), C.POINTER(i64),
                                 C.c_char_p, C.c_int]
    L.sddmm_mtx_read.argtypes = [vp, vp, vp, vp]
    L.sddmm_mtx_close.argtypes = [vp]
    L.sddmm_coo_is_row_sorted.argtypes = [i64, vp]
    L.sddmm_mtx_write.argtypes = [C.c_char_p, i64, i64, i64, vp, vp, vp]
    L.sddmm_coo_sort_rows.argtypes = [C.POINTER(i64), C.POINTER(i64), i64, vp, vp, vp, C.c_int]
    for name in EXPORTED_SYMBOLS:
        fn = getattr(L, name)
        if fn.restype is C.c_int or fn.restype is None:
            fn.restype = C.c_int
    _lib = L
    return L


def _ptr(a):
    """Address of a numpy array / torch tensor / int / None."""
    if a is None:
        return None
    if isinstance(a, int):
        return a
    if isinstance(a, np.ndarray):
        if not a.flags["C_CONTIGUOUS"]:
            raise ValueError("array must be C-contiguous")
        return a.ctypes.data
    if hasattr(a, "data_ptr"):  # torch tensor
        if not a.is_contiguous():
            raise ValueError("tensor must be contiguous")
        return a.data_ptr()
    raise TypeError(f"cannot take the address of {type(a)}")


CUDA_STREAM_LEGACY = 0x1  # cudaStreamLegacy: the handle that names the legacy default stream explicitly


def _is_cuda_tensor(a):
    return hasattr(a, "is_cuda") and a.is_cuda


class Handle:
    """One engine instance bound to one CUDA device (sddmm_create).

    Stream ordering.  The engine launches on one CUDA stream.  Unless set_stream()
    has been called, every call that is given a CUDA torch tensor first points the
    engine at torch's CURRENT stream of the handle's device, so the call is ordered
    after the work that produced its inputs and before whatever the caller
    enqueues next on that stream -- no torch.cuda.synchronize() is needed around
    it.  After an explicit set_stream() the caller owns the ordering: inputs must
    be ready on that stream, and results are ready on it.  Calls with host arrays
    only run on the handle's own stream and return when the result is complete."""

    def __init__(self, device=0):
        self._h = C.c_void_p()
        st = lib().sddmm_create(C.byref(self._h), device)
        if st != OK:
            self._h = None
            raise SddmmError(st)
        self.device = device
        self._explicit_stream = False

    def _follow_torch_stream(self, *args):
        """Launch on torch's current stream when a CUDA tensor is among the arguments
        (and the caller has not chosen a stream)."""
        if self._explicit_stream or not any(_is_cuda_tensor(a) for a in args):
            return
        import torch
        s = torch.cuda.current_stream(self.device).cuda_stream
        self._check(lib().sddmm_set_stream(self._h, s if s else CUDA_STREAM_LEGACY))

    def close(self):
        if self._h:
            lib().sddmm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def last_error(self):
        return lib().sddmm_last_error(self._h).decode()

    def _check(self, st):
        if st != OK:
            raise SddmmError(st, self.last_error())

    def selftest_wait_timeout(self):
        """Status of a wait that is made to run out (expected: DEVICE_TIMEOUT)."""
        return lib().sddmm_selftest_wait_timeout(self._h)

    def set_stream(self, cuda_stream):
        """cuda_stream: integer cudaStream_t (e.g. torch.cuda.current_stream().cuda_stream) or None."""
        self._check(lib().sddmm_set_stream(self._h, cuda_stream))
        self._explicit_stream = cuda_stream is not None

    def kernel_launches(self):
        """Kernels launched through this handle by execute() / upload_rows() so far."""
        n = C.c_int64()
        self._check(lib().sddmm_kernel_launches(self._h, C.byref(n)))
        return n.value

    def sync(self):
        """Wait for the handle's stream; raises SddmmError(DEVICE_TIMEOUT) if a bounded device-side wait of
        an earlier (possibly FLAG_ASYNC) call gave up."""
        self._check(lib().sddmm_sync(self._h))

    def upload_rows(self, host, dev, d_row_ids, n_rows, K, cuda_stream=None):
        """Copy the listed rows of a pinned host array to the same rows of a device array (the GPU
        reads the host rows); `d_row_ids` is a device int32 tensor or a device address."""
        self._check(lib().sddmm_upload_rows(self._h, _ptr(host), _ptr(dev), _ptr(d_row_ids), n_rows, K,
                                            cuda_stream))

    def coo_sort_rows(self, M, N, rows, cols, vals, transpose=False):
        """sddmm_coo_sort_rows on the GPU, in place (numpy arrays or device tensors); returns (M, N)."""
        m, n = C.c_int64(M), C.c_int64(N)
        self._follow_torch_stream(rows, cols, vals)
        self._check(lib().sddmm_coo_sort_rows_gpu(self._h, C.byref(m), C.byref(n), rows.shape[0], _ptr(rows), _ptr(cols),
                                                  _ptr(vals), 1 if transpose else 0))
        return m.value, n.value

    def plan_coo(self, M, N, rows, cols, K, panel_rows_hint=0, col_tile_hint=0, flags=0, nnz=None):
        if nnz is None:
            nnz = int(rows.shape[0])
        is_dev = hasattr(rows, "is_cuda") and rows.is_cuda
        if is_dev:
            flags |= PLAN_DEVICE_INDICES
        p = C.c_void_p()
        self._follow_torch_stream(rows, cols)
        st = lib().sddmm_plan_coo(self._h, M, N, nnz, _ptr(rows), _ptr(cols), K, panel_rows_hint, col_tile_hint,
                                  flags, C.byref(p))
        self._check(st)
        keep = (rows, cols) if is_dev else None  # device indices are borrowed, keep them alive
        return Plan(self, p, nnz, keep)

    def sddmm_coo(self, M, N, rows, cols, W, H, K, P, Sval=None, nnz=None):
        if nnz is None:
            nnz = int(rows.shape[0])
        self._follow_torch_stream(rows, cols, W, H, P, Sval)
        self._check(lib().sddmm_coo(self._h, M, N, nnz, _ptr(rows), _ptr(cols), _ptr(Sval), _ptr(W), _ptr(H), K,
                                    _ptr(P)))


class Plan:
    """A binned sparsity pattern, reusable across executes (sddmm_plan_coo)."""

    def __init__(self, handle, p, nnz, keep):
        self.handle = handle
        self._p = p
        self.nnz = nnz
        self._keep = keep

    def close(self):
        if self._p:
            lib().sddmm_destroy_plan(self._p)
            self._p = None

    def __del__(self):
        try:
            if self.handle._h:
                self.close()
        except Exception:
            pass

    def execute(self, W, H, P, Sval=None, flags=0):
        self.handle._follow_torch_stream(W, H, P, Sval)
        self.handle._check(lib().sddmm_execute(self._p, _ptr(W), _ptr(H), _ptr(Sval), _ptr(P), flags))

    def spmm(self, H, Y, Pval=None, flags=0):
        """Y = P H on the plan's pattern (sddmm_spmm_execute); Pval None = all ones."""
        self.handle._follow_torch_stream(H, Y, Pval)
        self.handle._check(lib().sddmm_spmm_execute(self._p, _ptr(Pval), _ptr(H), _ptr(Y), flags))

    def fused(self, W, H, Y, Sval=None, P_out=None, flags=0):
        """Y = (S o (W H^T)) H without writing P (sddmm_fused_execute); P_out, if given, receives P."""
        self.handle._follow_torch_stream(W, H, Y, Sval, P_out)
        self.handle._check(lib().sddmm_fused_execute(self._p, _ptr(W), _ptr(H), _ptr(Sval), _ptr(P_out), _ptr(Y), flags))

    def last_kernel_name(self):
        return lib().sddmm_last_kernel_name(self._p).decode()

    def check_result(self, W, H, P, Sval=None, stride=1, tol=1e-4):
        """float64 recomputation of every stride-th nonzero on the device (sddmm_check_result):
        returns (max scaled error, nonzeros checked, nonzeros out of tolerance)."""
        worst, n, bad = C.c_double(), C.c_int64(), C.c_int64()
        self.handle._follow_torch_stream(W, H, P, Sval)
        self.handle._check(lib().sddmm_check_result(self._p, _ptr(W), _ptr(H), _ptr(Sval), _ptr(P), stride, tol,
                                                    C.byref(worst), C.byref(n), C.byref(bad)))
        return worst.value, n.value, bad.value

    def last_kernel_ms(self):
        ms = C.c_float()
        self.handle._check(lib().sddmm_last_kernel_ms(self._p, C.byref(ms)))
        return ms.value

    def used_lines(self, which):
        """(device address, count) of the plan's list of rows (which=0) / columns (which=1) of S
        that hold a nonzero: the rows of W / H the SDDMM reads.  Owned by the plan."""
        ptr, n = C.c_void_p(), C.c_int64(0)
        self.handle._check(lib().sddmm_plan_used_lines(self._p, which, C.byref(ptr), C.byref(n)))
        return ptr.value or 0, n.value

    def last_transfer_bytes(self):
        """(host->device, device->host) bytes moved by the last execute()."""
        up, down = C.c_int64(0), C.c_int64(0)
        self.handle._check(lib().sddmm_last_transfer_bytes(self._p, C.byref(up), C.byref(down)))
        return up.value, down.value

    def info(self):
        inf = PlanInfo()
        self.handle._check(lib().sddmm_plan_get_info(self._p, C.byref(inf)))
        return inf

    def count_cols(self):
        n = C.c_int64()
        self.handle._check(lib().sddmm_plan_count_cols(self._p, C.byref(n)))
        return n.value

    def export_row_ptr(self):
        inf = self.info()
        out = np.empty(inf.M + 1, np.int64)
        self.handle._check(lib().sddmm_plan_export_row_ptr(self._p, out.ctypes.data))
        return out

    def export_tiling(self, panel_rows, col_tile):
        inf = self.info()
        M, N, nnz = inf.M, inf.N, inf.nnz
        ntile_c = N // col_tile + 1
        max_blk = M // panel_rows + 1
        out = dict(
            rows=np.zeros(nnz, np.int32), cols=np.zeros(nnz, np.int32), tiled_ind=np.zeros(nnz, np.int32),
            lastIdx_tile=np.zeros(ntile_c + 1, np.int32),
            lastIdx_block_tile=np.zeros((ntile_c + 1) * max_blk, np.int32),
            active_row=np.zeros(M * ntile_c, np.int32), n_actv_row=np.zeros(ntile_c, np.int32))
        mar = C.c_int32()
        st = lib().sddmm_plan_export_tiling(
            self._p, panel_rows, col_tile, out["rows"].ctypes.data, out["cols"].ctypes.data,
            out["tiled_ind"].ctypes.data, out["lastIdx_tile"].ctypes.data,
            out["lastIdx_block_tile"].ctypes.data, out["active_row"].ctypes.data,
            out["n_actv_row"].ctypes.data, C.byref(mar))
        self.handle._check(st)
        out["max_active_row"] = mar.value
        out["ntile_c"] = ntile_c
        out["max_active_block"] = max_blk
        return out


COMM_ID_BYTES = 128
DIST_H_RESIDENT = 0x10000
DIST_BROADCAST_ONLY = 0x20000


def comm_unique_id():
    """128 bytes that rank 0 creates and every rank passes to Comm() (ncclGetUniqueId)."""
    buf = C.create_string_buffer(COMM_ID_BYTES)
    st = lib().sddmm_comm_unique_id(buf)
    if st != OK:
        raise SddmmError(st, "NCCL is not available in this process")
    return buf.raw


class Comm:
    """This rank's end of an NCCL communicator on the handle's GPU (sddmm_comm_create)."""

    def __init__(self, handle, unique_id, rank, world):
        self.handle, self.rank, self.world = handle, rank, world
        self._c = C.c_void_p()
        handle._check(lib().sddmm_comm_create(handle._h, unique_id, rank, world, C.byref(self._c)))

    def close(self):
        if self._c:
            lib().sddmm_comm_destroy(self._c)
            self._c = None

    def broadcast(self, buf, root=0, cuda_stream=None):
        self.handle._follow_torch_stream(buf)
        self.handle._check(lib().sddmm_comm_broadcast(self._c, _ptr(buf), buf.numel(), root, cuda_stream))

    def all_gather(self, buf, count_per_rank, cuda_stream=None):
        """In place: rank r's floats [r * count_per_rank, (r + 1) * count_per_rank) of buf go to every rank."""
        self.handle._follow_torch_stream(buf)
        self.handle._check(lib().sddmm_comm_all_gather(self._c, _ptr(buf), count_per_rank, cuda_stream))

    def plan_coo(self, M, N, rows, cols, K, panel_rows_hint=0, h_chunks=1, flags=0, rank_shares=None):
        """This rank's part of a plan over the whole matrix (sddmm_dist_plan_coo[_shares]); rank_shares: the
        fraction of the nonzeros every rank is to get (a sequence of `world` numbers, the same on every rank)."""
        is_dev = _is_cuda_tensor(rows)
        if is_dev:
            flags |= PLAN_DEVICE_INDICES
        p = C.c_void_p()
        shares = None
        if rank_shares is not None:
            shares = np.ascontiguousarray(rank_shares, np.float64)
            assert shares.shape[0] == self.world
        self.handle._follow_torch_stream(rows, cols)
        self.handle._check(lib().sddmm_dist_plan_coo_shares(self._c, M, N, int(rows.shape[0]), _ptr(rows), _ptr(cols), K,
                                                            panel_rows_hint, h_chunks, _ptr(shares), flags, C.byref(p)))
        return DistPlan(self, p, (rows, cols) if is_dev else None)


class DistPlan:
    def __init__(self, comm, p, keep):
        self.comm, self._p, self._keep = comm, p, keep
        rb, re_, nb, ne, nc = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64(), C.c_int32()
        comm.handle._check(lib().sddmm_dist_plan_get_shard(p, C.byref(rb), C.byref(re_), C.byref(nb), C.byref(ne),
                                                           C.byref(nc)))
        self.row_begin, self.row_end, self.nnz_begin, self.nnz_end = rb.value, re_.value, nb.value, ne.value
        self.n_chunks = nc.value
        # the rank's single-GPU plan, owned by the distributed plan (never closed on its own)
        self.local = Plan(comm.handle, C.c_void_p(lib().sddmm_dist_plan_local(p)), self.nnz_end - self.nnz_begin, None)
        self.local.close = lambda: None

    def close(self):
        if self._p:
            self.local._p = None
            lib().sddmm_dist_plan_destroy(self._p)
            self._p = None

    def execute(self, W_local, H, P_local, Sval_local=None, root=0, flags=0):
        """flags: FLAG_* | DIST_H_RESIDENT | DIST_BROADCAST_ONLY (sddmm_dist_execute)."""
        h = self.comm.handle
        h._follow_torch_stream(W_local, H, P_local, Sval_local)
        h._check(lib().sddmm_dist_execute(self._p, _ptr(W_local), _ptr(H), _ptr(Sval_local), _ptr(P_local), root, flags))

    def last_times(self):
        """(broadcast ms, kernel ms with H resident, whole call ms) of the last synchronous execute."""
        a, b, c = C.c_float(), C.c_float(), C.c_float()
        self.comm.handle._check(lib().sddmm_dist_last_times(self._p, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value


class MultiGpu:
    """One process driving several GPUs from host arrays (sddmm_multi_*)."""

    def __init__(self, devices):
        devices = list(devices)
        arr = (C.c_int * len(devices))(*devices)
        self._m = C.c_void_p()
        st = lib().sddmm_multi_create(arr, len(devices), C.byref(self._m))
        if st != OK:
            self._m = None
            raise SddmmError(st)
        self.devices = devices

    def _check(self, st):
        if st != OK:
            raise SddmmError(st, lib().sddmm_multi_last_error(self._m).decode())

    def close(self):
        if self._m:
            lib().sddmm_multi_destroy(self._m)
            self._m = None

    def plan_coo(self, M, N, rows, cols, K, panel_rows_hint=0, flags=0):
        p = C.c_void_p()
        self._check(lib().sddmm_multi_plan_coo(self._m, M, N, int(rows.shape[0]), _ptr(rows), _ptr(cols), K,
                                               panel_rows_hint, flags, C.byref(p)))
        return MultiPlan(self, p)


class MultiPlan:
    def __init__(self, multi, p):
        self.multi, self._p = multi, p

    def close(self):
        if self._p:
            lib().sddmm_multi_plan_destroy(self._p)
            self._p = None

    def cuts(self):
        n = len(self.multi.devices)
        rc, nc = np.zeros(n + 1, np.int64), np.zeros(n + 1, np.int64)
        self.multi._check(lib().sddmm_multi_plan_get_cuts(self._p, rc.ctypes.data, nc.ctypes.data))
        return rc, nc

    def execute(self, W, H, P, Sval=None, flags=0):
        """W, H, Sval, P: host arrays of the whole problem."""
        self.multi._check(lib().sddmm_multi_execute(self._p, _ptr(W), _ptr(H), _ptr(Sval), _ptr(P), flags))

    def last_kernel_ms(self):
        ms = C.c_float()
        self.multi._check(lib().sddmm_multi_last_kernel_ms(self._p, C.byref(ms)))
        return ms.value


NOALLOC_MAX_COLS = 8 * 1024 * 1024


def count_cols_noalloc(d_cols, N, device=0, cuda_stream=None, nnz=None):
    """Distinct columns among the device-resident column indices `d_cols`, computed
    without any device allocation (sddmm_count_cols_noalloc).  For callers that are
    not allowed to enter the CUDA allocator; N is limited to NOALLOC_MAX_COLS by the
    library's built-in scratch.  Calls on one GPU must not overlap."""
    if nnz is None:
        nnz = int(d_cols.shape[0])
    out = C.c_int64()
    err = C.create_string_buffer(256)
    st = lib().sddmm_count_cols_noalloc(device, _ptr(d_cols), nnz, N, cuda_stream, C.byref(out), err, 256)
    if st != OK:
        raise SddmmError(st, err.value.decode())
    return out.value


# ---- host-only helpers (no GPU needed) -------------------------------------

def partition_rows_shares(M, rows, shares, align_rows=1):
    """Row cuts for parts that are to hold shares[g] / sum(shares) of the nonzeros (sddmm_partition_rows_shares)."""
    rows = np.ascontiguousarray(rows, np.int32)
    shares = np.ascontiguousarray(shares, np.float64)
    n = shares.shape[0]
    cuts, nnz_cuts = np.zeros(n + 1, np.int64), np.zeros(n + 1, np.int64)
    st = lib().sddmm_partition_rows_shares(M, rows.shape[0], rows.ctypes.data, n, align_rows, shares.ctypes.data,
                                           cuts.ctypes.data, nnz_cuts.ctypes.data)
    if st != OK:
        raise SddmmError(st)
    return cuts, nnz_cuts


def partition_rows(M, rows, n_parts, align_rows=1, row_cost=0.0):
    rows = np.ascontiguousarray(rows, np.int32)
    cuts = np.zeros(n_parts + 1, np.int64)
    nnz_cuts = np.zeros(n_parts + 1, np.int64)
    st = lib().sddmm_partition_rows_weighted(M, rows.shape[0], rows.ctypes.data, n_parts, align_rows, float(row_cost),
                                             cuts.ctypes.data, nnz_cuts.ctypes.data)
    if st != OK:
        raise SddmmError(st)
    return cuts, nnz_cuts


MTX_EXPAND_SYMMETRIC = 0x1
MTX_SORT_ROWS = 0x2


def mtx_read(path, flags=0):
    """Returns (M, N, rows, cols, vals) with 0-based int32 indices.  Reads Matrix Market text,
    headerless docword triples and the binary form of coo_save_binary; flags: MTX_*."""
    f = C.c_void_p()
    M, N, nnz = C.c_int64(), C.c_int64(), C.c_int64()
    err = C.create_string_buffer(256)
    st = lib().sddmm_mtx_open_ex(os.fsencode(path), flags, C.byref(f), C.byref(M), C.byref(N), C.byref(nnz), err, 256)
    if st != OK:
        raise SddmmError(st, err.value.decode())
    rows = np.empty(nnz.value, np.int32)
    cols = np.empty(nnz.value, np.int32)
    vals = np.empty(nnz.value, np.float32)
    st = lib().sddmm_mtx_read(f, rows.ctypes.data, cols.ctypes.data, vals.ctypes.data)
    if st != OK:
        raise SddmmError(st)
    return M.value, N.value, rows, cols, vals


def coo_save_binary(path, M, N, rows, cols, vals=None):
    st = lib().sddmm_coo_save_binary(os.fsencode(path), M, N, rows.shape[0], _ptr(rows), _ptr(cols), _ptr(vals))
    if st != OK:
        raise SddmmError(st)


def gen_matrix(spec):
    """Seeded synthetic matrix (see sddmm_gen_open): (M, N, rows, cols, vals), row-sorted."""
    f = C.c_void_p()
    M, N, nnz = C.c_int64(), C.c_int64(), C.c_int64()
    err = C.create_string_buffer(256)
    st = lib().sddmm_gen_open(spec.encode(), C.byref(f), C.byref(M), C.byref(N), C.byref(nnz), err, 256)
    if st != OK:
        raise SddmmError(st, err.value.decode())
    rows = np.empty(nnz.value, np.int32)
    cols = np.empty(nnz.value, np.int32)
    vals = np.empty(nnz.value, np.float32)
    st = lib().sddmm_mtx_read(f, rows.ctypes.data, cols.ctypes.data, vals.ctypes.data)
    if st != OK:
        raise SddmmError(st)
    return M.value, N.value, rows, cols, vals


def mtx_write(path, M, N, rows, cols, vals=None):
    rows = np.ascontiguousarray(rows, np.int32)
    cols = np.ascontiguousarray(cols, np.int32)
    if vals is not None:
        vals = np.ascontiguousarray(vals, np.float32)
    st = lib().sddmm_mtx_write(os.fsencode(path), M, N, rows.shape[0], rows.ctypes.data, cols.ctypes.data,
                               _ptr(vals))
    if st != OK:
        raise SddmmError(st)


def coo_is_row_sorted(rows):
    rows = np.ascontiguousarray(rows, np.int32)
    return bool(lib().sddmm_coo_is_row_sorted(rows.shape[0], rows.ctypes.data))


def coo_sort_rows(M, N, rows, cols, vals, transpose=False):
    """Returns (M, N, rows, cols, vals) row-sorted; transpose=True emits S^T as the reference's converter does."""
    rows = np.ascontiguousarray(rows, np.int32).copy()
    cols = np.ascontiguousarray(cols, np.int32).copy()
    vals = np.ascontiguousarray(vals, np.float32).copy()
    m, n = C.c_int64(M), C.c_int64(N)
    st = lib().sddmm_coo_sort_rows(C.byref(m), C.byref(n), rows.shape[0], rows.ctypes.data, cols.ctypes.data,
                                   vals.ctypes.data, int(transpose))
    if st != OK:
        raise SddmmError(st)
    return m.value, n.value, rows, cols, vals
