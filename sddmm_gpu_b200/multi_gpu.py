"""Row-block sharding of one SDDMM across the GPUs of a box, one process per GPU.

Replaces the MPI variant of the reference (HiPC18_mpi/sddmm.cu:139-351,
HiPC18_mpi/util.h:100-135): there every rank parses the whole file, redoes the
whole preprocessing, uploads all of W and H and processes one nnz-balanced
COLUMN panel, with MPI used for barriers only.  Here S is cut into nnz-balanced
blocks of consecutive ROWS (so each rank's nonzeros are one contiguous slice of
the input and the concatenation of the ranks' outputs is P in input order), rank
r keeps only its rows of W, and H -- the one operand every rank needs whole -- is
broadcast once per H version over NCCL (NVLink / NVSwitch).  P stays sharded.

The collective is ``torch.distributed`` plumbing; the compute on each rank is the
same C-ABI plan/execute as on one GPU.  Nothing here computes on the CPU.
"""
import numpy as np
import torch
import torch.distributed as dist

from . import api


class RowShard:
    """What one rank owns: rows [row_begin, row_end), nonzeros [nnz_begin, nnz_end)."""

    def __init__(self, rank, world, cuts, nnz_cuts):
        self.rank, self.world = rank, world
        self.cuts, self.nnz_cuts = cuts, nnz_cuts
        self.row_begin, self.row_end = int(cuts[rank]), int(cuts[rank + 1])
        self.nnz_begin, self.nnz_end = int(nnz_cuts[rank]), int(nnz_cuts[rank + 1])

    @property
    def n_rows(self):
        return self.row_end - self.row_begin

    @property
    def nnz(self):
        return self.nnz_end - self.nnz_begin


def make_shard(M, rows_host, world, rank, align_rows=32, row_cost=0.0):
    """Balanced row cuts (sddmm_partition_rows_weighted) -> this rank's shard.
    rows_host: the row index of every nonzero (row-sorted), numpy int32.
    row_cost: extra cost of a non-empty row, in nonzeros (0 = balance nonzeros only)."""
    cuts, nnz_cuts = api.partition_rows(M, rows_host, world, align_rows, row_cost)
    return RowShard(rank, world, cuts, nnz_cuts)


def local_pattern(shard, rows, cols):
    """This rank's slice of the pattern with rows rebased to the shard (tensors or arrays)."""
    a, b = shard.nnz_begin, shard.nnz_end
    return rows[a:b] - shard.row_begin, cols[a:b]


def broadcast_h(H, src=0, group=None, chunks=1):
    """Broadcast H from `src` into every rank's own memory (in place).  With
    chunks > 1 the rows of H go out as that many separate collectives, so that
    work depending only on the early ones can be enqueued behind them."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return []
    handles = []
    n = H.shape[0]
    step = -(-n // chunks)
    for c0 in range(0, n, step):
        handles.append(dist.broadcast(H[c0:c0 + step], src=src, group=group, async_op=True))
    return handles


def exchange_h_slices(H_dev, rank, world, group=None):
    """Every rank holds rows [r*n/world, (r+1)*n/world) of H in its own copy H_dev;
    afterwards every copy is complete.  One all-gather (in place) when the slices have
    equal length, one broadcast per slice otherwise.  NVLink / NVSwitch traffic only."""
    if world == 1:
        return
    n = H_dev.shape[0]
    bounds = [(n * r) // world for r in range(world + 1)]
    if n % world == 0:
        dist.all_gather_into_tensor(H_dev, H_dev[bounds[rank]:bounds[rank + 1]], group=group)
        return
    for r in range(world):
        if bounds[r + 1] > bounds[r]:
            dist.broadcast(H_dev[bounds[r]:bounds[r + 1]], src=r, group=group)


def upload_h_sharded(H_dev, H_host_slice, rank, world, group=None):
    """Bring a host-resident H into every rank's device memory using all PCIe links:
    rank r copies its slice of H's rows from its pinned host memory to its GPU, then the
    slices are exchanged (exchange_h_slices).  H_dev is complete on return of the
    collectives (stream-ordered)."""
    a, b = h_slice_bounds(H_dev.shape[0], rank, world)
    H_dev[a:b].copy_(H_host_slice, non_blocking=True)
    exchange_h_slices(H_dev, rank, world, group)


def h_slice_bounds(n, rank, world):
    return (n * rank) // world, (n * (rank + 1)) // world


def gather_p(P_local, shard, group=None):
    """All ranks' P slices concatenated in input order (optional; P normally stays sharded)."""
    if not dist.is_initialized() or shard.world == 1:
        return P_local
    sizes = [int(shard.nnz_cuts[g + 1] - shard.nnz_cuts[g]) for g in range(shard.world)]
    # the shards differ in length, so every rank broadcasts its own slice
    out = torch.empty(sum(sizes), dtype=P_local.dtype, device=P_local.device)
    off = 0
    for g, n in enumerate(sizes):
        piece = out[off:off + n]
        if g == shard.rank:
            piece.copy_(P_local)
        if n > 0:
            dist.broadcast(piece, src=g, group=group)
        off += n
    return out


def used_h_rows_of_slice(cols_all, N, rank, world):
    """Ids, relative to this rank's slice of H's rows, of the H rows that any nonzero of
    the WHOLE matrix touches (`cols_all`: every column index of S, a device tensor): the
    rows of the slice worth uploading.  int32 device tensor, ascending."""
    a, b = h_slice_bounds(N, rank, world)
    used = torch.zeros(N, dtype=torch.bool, device=cols_all.device)
    used[cols_all.long()] = True
    return (torch.nonzero(used[a:b]).squeeze(1)).to(torch.int32).contiguous()


def host_step(plan, rank, world, W_host, H_host_slice, H_dev, P_host, Sval_host=None, flags=0, staging=None,
              h_slice_rows=None, comm=None, phases=None):
    """One SDDMM on this rank's row block with every operand in (pinned) host memory:
    this rank's rows of W, its 1/world slice of H's rows, its S values; P comes back to
    host memory.  Order on the rank's PCIe link: the H slice first, then W rows and S
    values (on a side stream) while the H slices are exchanged over NVLink on the current
    stream (which must be the stream the plan's handle launches on); the kernel starts
    when both are in place.  Only rows that a nonzero touches travel over PCIe: the rows
    of W from the plan's own list, the rows of the H slice from `h_slice_rows`
    (used_h_rows_of_slice; None uploads the whole slice).  `staging` (a dict the caller
    keeps) holds the device copies of W and S and the side stream between calls.
    `comm` (an api.Comm) exchanges the H slices through the C ABI's all-gather instead of torch.distributed
    when the slices have equal length.  `phases` (a dict) receives CUDA events around the phases of the step;
    phase_times() turns them into milliseconds after the step has completed."""
    staging = staging if staging is not None else {}
    handle, K = plan.handle, H_dev.shape[1]
    cur = torch.cuda.current_stream()
    side = staging.get("side")
    if side is None:
        side = staging["side"] = torch.cuda.Stream()
    def mark(name, stream):
        if phases is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            phases[name] = ev

    mark("begin", cur)
    a, b = h_slice_bounds(H_dev.shape[0], rank, world)
    if h_slice_rows is not None:
        handle.upload_rows(H_host_slice, H_dev[a:b], h_slice_rows, h_slice_rows.numel(), K, cur.cuda_stream)
    else:
        H_dev[a:b].copy_(H_host_slice, non_blocking=True)
    slice_up = torch.cuda.Event(enable_timing=phases is not None)
    slice_up.record(cur)
    if phases is not None:
        phases["h_slice_uploaded"] = slice_up

    def staged(name, host):
        t = staging.get(name)
        if t is None or t.shape != host.shape:
            t = staging[name] = torch.empty(host.shape, dtype=host.dtype, device=H_dev.device)
        return t

    side.wait_event(slice_up)
    with torch.cuda.stream(side):
        W_dev = staged("W", W_host)
        ids, n_ids = plan.used_lines(0)
        handle.upload_rows(W_host, W_dev, ids, n_ids, K, side.cuda_stream)
        S_dev = None
        if Sval_host is not None:
            S_dev = staged("S", Sval_host)
            S_dev.copy_(Sval_host, non_blocking=True)
        mark("w_uploaded", side)
    n = H_dev.shape[0]
    if comm is not None and world > 1 and n % world == 0:
        comm.all_gather(H_dev, (n // world) * K, cur.cuda_stream)
    else:
        exchange_h_slices(H_dev, rank, world)
    mark("h_exchanged", cur)
    cur.wait_stream(side)
    plan.execute(W_dev, H_dev, P_host, S_dev, flags)   # kernel and download of P; synchronous
    mark("end", cur)
    if phases is not None:
        phases["kernel_ms"] = plan.last_kernel_ms()
    n_h = h_slice_rows.numel() if h_slice_rows is not None else (b - a)
    return 4 * K * (n_ids + n_h) + (4 * Sval_host.numel() if Sval_host is not None else 0)   # bytes uploaded


def phase_times(phases):
    """Milliseconds of the phases of one host_step (after it has completed), on this rank: the upload of
    the rank's H slice, the exchange of the slices, the upload of W and S (runs beside the exchange, on the
    side stream, from the moment the H slice is up), the kernel, and what is left of the step after the
    later of exchange and W upload (kernel + download of P)."""
    b, e = phases["begin"], phases["end"]
    up, ex, w = phases["h_slice_uploaded"], phases["h_exchanged"], phases["w_uploaded"]
    total = b.elapsed_time(e)
    t_ex, t_w = b.elapsed_time(ex), b.elapsed_time(w)
    return {"h_slice_upload_ms": b.elapsed_time(up), "h_exchange_ms": up.elapsed_time(ex),
            "w_s_upload_ms": up.elapsed_time(w), "kernel_ms": phases["kernel_ms"],
            "p_download_and_sync_ms": total - max(t_ex, t_w) - phases["kernel_ms"], "total_ms": total}


class ShardedSddmm:
    """One rank's plan over its row block.  execute() takes this rank's W rows,
    the full (already broadcast) H and returns this rank's slice of P."""

    def __init__(self, handle, M, N, rows, cols, K, rows_host=None, world=None, rank=None, panel_rows_hint=0,
                 col_tile_hint=0, align_rows=32):
        world = world if world is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        rank = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
        if rows_host is None:
            rows_host = rows.cpu().numpy() if hasattr(rows, "cpu") else np.asarray(rows)
        self.shard = make_shard(M, rows_host, world, rank, align_rows)
        lr, lc = local_pattern(self.shard, rows, cols)
        if hasattr(lr, "contiguous"):
            lr, lc = lr.contiguous(), lc.contiguous()
        else:
            lr, lc = np.ascontiguousarray(lr), np.ascontiguousarray(lc)
        self.plan = handle.plan_coo(self.shard.n_rows, N, lr, lc, K, panel_rows_hint, col_tile_hint)
        self.K = K

    def execute(self, W_local, H, P_local, Sval_local=None, flags=0):
        self.plan.execute(W_local, H, P_local, Sval_local, flags)

    def execute_from_host(self, W_host, H_host_slice, H_dev, P_host, Sval_host=None, flags=0, h_slice_rows=None):
        """execute() with every operand in pinned host memory (see host_step)."""
        if not hasattr(self, "_staging"):
            self._staging = {}
        return host_step(self.plan, self.shard.rank, self.shard.world, W_host, H_host_slice, H_dev, P_host, Sval_host,
                         flags, self._staging, h_slice_rows)

    def close(self):
        self.plan.close()
