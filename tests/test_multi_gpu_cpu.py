"""The N > 1 path on CPU: two gloo ranks shard S by nnz-balanced row blocks,
broadcast H, run the CPU oracle in place of the kernel on each shard and gather
P; the concatenation must equal the unsharded result bit for bit (each output
depends only on its own W row and H row, so sharding cannot change a value)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_problem():
    rng = np.random.default_rng(42)
    M, N, K = 700, 260, 24
    deg = (rng.pareto(1.1, M) * 4).astype(np.int64).clip(0, N)
    deg[rng.choice(M, 200, replace=False)] = 0
    deg[5] = N                                   # one hub row
    rows = np.repeat(np.arange(M), deg).astype(np.int32)
    cols = np.concatenate([np.sort(rng.choice(N, d, replace=False)) for d in deg]).astype(np.int32)
    vals = rng.standard_normal(rows.shape[0]).astype(np.float32)
    W = rng.standard_normal((M, K)).astype(np.float32)
    H = rng.standard_normal((N, K)).astype(np.float32)
    return M, N, K, rows, cols, vals, W, H


def _worker(rank, world, port, out_path):
    sys.path.insert(0, ROOT)
    import oracle
    from sddmm_gpu_b200 import multi_gpu
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    M, N, K, rows, cols, vals, W, H = _make_problem()
    shard = multi_gpu.make_shard(M, rows, world, rank, align_rows=8)
    l_rows, l_cols = multi_gpu.local_pattern(shard, rows, cols)
    # only rank 0 owns H; the others receive it
    Ht = torch.from_numpy(H.copy() if rank == 0 else np.zeros_like(H))
    for hnd in multi_gpu.broadcast_h(Ht, src=0, chunks=3):
        hnd.wait()
    assert np.array_equal(Ht.numpy(), H)
    W_local = W[shard.row_begin:shard.row_end]
    P_local = oracle.cpu.sddmm_coo(np.ascontiguousarray(l_rows), np.ascontiguousarray(l_cols), W_local, Ht.numpy(),
                                   vals[shard.nnz_begin:shard.nnz_end])
    P = multi_gpu.gather_p(torch.from_numpy(P_local), shard)
    if rank == 0:
        np.save(out_path, P.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_result(tmp_path):
    sys.path.insert(0, ROOT)
    import oracle
    out = str(tmp_path / "p.npy")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    M, N, K, rows, cols, vals, W, H = _make_problem()
    full = oracle.cpu.sddmm_coo(rows, cols, W, H, vals)
    assert np.array_equal(np.load(out), full)


def test_shards_cover_the_matrix_without_overlap():
    from sddmm_gpu_b200 import multi_gpu
    M, N, K, rows, cols, vals, W, H = _make_problem()
    for world in (1, 2, 3, 4, 8):
        shards = [multi_gpu.make_shard(M, rows, world, r, align_rows=8) for r in range(world)]
        assert shards[0].row_begin == 0 and shards[-1].row_end == M
        assert shards[0].nnz_begin == 0 and shards[-1].nnz_end == rows.shape[0]
        for a, b in zip(shards, shards[1:]):
            assert a.row_end == b.row_begin and a.nnz_end == b.nnz_begin
        for s in shards:
            lr, lc = multi_gpu.local_pattern(s, rows, cols)
            assert lr.shape[0] == s.nnz and (s.nnz == 0 or (lr.min() >= 0 and lr.max() < s.n_rows))


def _h_exchange_worker(rank, world, port, n_rows):
    sys.path.insert(0, ROOT)
    from sddmm_gpu_b200 import multi_gpu
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    K = 12
    H = torch.arange(n_rows * K, dtype=torch.float32).reshape(n_rows, K)
    a, b = multi_gpu.h_slice_bounds(n_rows, rank, world)
    H_mine = torch.full_like(H, -1.0)            # nothing but this rank's slice is known beforehand
    multi_gpu.upload_h_sharded(H_mine, H[a:b].clone(), rank, world)
    assert torch.equal(H_mine, H), f"rank {rank}: H not assembled"
    dist.barrier()
    dist.destroy_process_group()


def test_h_slices_are_assembled_on_every_rank():
    # equal slices take the all-gather, ragged ones a broadcast per slice
    for n_rows in (64, 61):
        mp.spawn(_h_exchange_worker, args=(2, _free_port(), n_rows), nprocs=2, join=True)


def test_partition_by_shares():
    """sddmm_partition_rows_shares: unequal parts, aligned cuts, every nonzero in exactly one part; equal
    shares give the plain partition; a zero share gives an empty part."""
    from sddmm_gpu_b200 import api
    rng = np.random.default_rng(9)
    M, nnz = 5000, 60_000
    rows = np.sort(rng.integers(0, M, nnz)).astype(np.int32)
    cuts, nz = api.partition_rows_shares(M, rows, [1, 1, 1, 1], align_rows=32)
    c0, n0 = api.partition_rows(M, rows, 4, 32)
    assert np.array_equal(cuts, c0) and np.array_equal(nz, n0)
    shares = np.array([4.0, 1.0, 0.0, 3.0])
    cuts, nz = api.partition_rows_shares(M, rows, shares, align_rows=32)
    assert cuts[0] == 0 and cuts[-1] == M and nz[0] == 0 and nz[-1] == nnz
    assert np.all(np.diff(cuts) >= 0) and np.all(cuts[1:-1] % 32 == 0)
    got = np.diff(nz) / nnz
    assert np.all(np.abs(got - shares / shares.sum()) < 0.02)        # within a few rows of the target
    assert nz[2] == nz[3] or got[2] < 0.02                            # the zero share is (nearly) empty
    for g in range(4):                                                # the cuts and the offsets agree
        assert np.all((rows[nz[g]:nz[g + 1]] >= cuts[g]) & (rows[nz[g]:nz[g + 1]] < cuts[g + 1]))
    with pytest.raises(api.SddmmError):
        api.partition_rows_shares(M, rows, [0.0, 0.0])
