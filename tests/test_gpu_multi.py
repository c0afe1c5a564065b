"""The multi-GPU layer of the C ABI (sddmm_comm_*, sddmm_dist_*, sddmm_multi_*) on however many GPUs are
visible: with one GPU the one-rank forms and the column-bucketed execute (broadcasts are no-ops); with two or
more, one process driving all GPUs and one process per GPU with the H broadcast overlapped.  Results are
compared with the CPU oracle (oracle/sddmm_oracle.c), tolerance 1e-4 as in tests/helpers.py."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import assert_parity, random_coo
from sddmm_gpu_b200 import api

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _problem(seed, M, N, nnz, K):
    rng = np.random.default_rng(seed)
    rows, cols = random_coo(rng, M, N, nnz, empty_rows=[0, 3, M - 1])
    vals = rng.standard_normal(rows.shape[0]).astype(np.float32)
    W = rng.standard_normal((M, K)).astype(np.float32)
    H = rng.standard_normal((N, K)).astype(np.float32)
    return rows, cols, vals, W, H


@pytest.mark.parametrize("K", [64, 256])
def test_one_process_all_gpus(K):
    """sddmm_multi_*: host arrays in, P in input order out; every visible GPU count from 1 up (two handles on
    two devices in one process each make their own shared-memory opt-in)."""
    n_all = torch.cuda.device_count()
    M, N = 3000, 2500
    rows, cols, vals, W, H = _problem(K, M, N, 90_000, K)
    for n in sorted({1, min(2, n_all), n_all}):
        multi = api.MultiGpu(range(n))
        plan = multi.plan_coo(M, N, rows, cols, K)
        rc, nc = plan.cuts()
        assert rc[0] == 0 and rc[-1] == M and nc[0] == 0 and nc[-1] == rows.shape[0]
        assert np.all(np.diff(nc) >= 0) and np.all(rc[1:-1] % 32 == 0)
        for sv in (vals, None):
            P = np.full(rows.shape[0], np.nan, np.float32)
            plan.execute(W, H, P, sv)
            assert_parity(P, rows, cols, W, H, sv)
        assert plan.last_kernel_ms() > 0
        plan.close()
        multi.close()


@pytest.mark.parametrize("K", [128, 256])
def test_column_bucketed_execute_on_one_rank(engine, K):
    """sddmm_dist_*: a one-rank communicator (no NCCL needed); the plan is forced into the column-bucketed
    form that the overlapped H broadcast uses, with 5 chunks that do not divide N."""
    M, N = 2000, 3001
    rows, cols, vals, W, H = _problem(100 + K, M, N, 120_000, K)
    comm = api.Comm(engine, b"\0" * api.COMM_ID_BYTES, 0, 1)
    d_rows, d_cols = torch.from_numpy(rows).cuda(), torch.from_numpy(cols).cuda()
    for idx in ((rows, cols), (d_rows, d_cols)):
        plan = comm.plan_coo(M, N, idx[0], idx[1], K, h_chunks=5, flags=api.PLAN_FORCE_H_CHUNKS)
        assert plan.n_chunks == 5 and (plan.row_begin, plan.row_end) == (0, M) and plan.nnz_end == rows.shape[0]
        dW, dH, dS = torch.from_numpy(W).cuda(), torch.from_numpy(H).cuda(), torch.from_numpy(vals).cuda()
        for sv, dsv in ((vals, dS), (None, None)):
            P = torch.full((rows.shape[0],), float("nan"), device="cuda")
            plan.execute(dW, dH, P, dsv)                               # bucketed, one launch per chunk
            assert_parity(P.cpu().numpy(), rows, cols, W, H, sv)
            t_bcast, _, t_total = plan.last_times()
            assert t_total > 0 and t_bcast >= 0
            P2 = torch.full_like(P, float("nan"))
            plan.execute(dW, dH, P2, dsv, flags=api.DIST_H_RESIDENT)   # the plain plan
            assert_parity(P2.cpu().numpy(), rows, cols, W, H, sv)
        assert plan.local.info().nnz == rows.shape[0]
        plan.close()
    comm.close()


_RANK_SCRIPT = r"""
import os, sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import numpy as np, torch, torch.distributed as dist
from sddmm_gpu_b200 import api
from helpers import assert_parity, random_coo
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo")                      # the id travels over any channel; here a CPU broadcast
ids = [api.comm_unique_id() if rank == 0 else None]
dist.broadcast_object_list(ids, src=0)
h = api.Handle(rank)
comm = api.Comm(h, ids[0], rank, world)
rng = np.random.default_rng(5)
M, N, K = 4000, 3500, 256
rows, cols = random_coo(rng, M, N, 200_000)
vals = rng.standard_normal(rows.shape[0]).astype(np.float32)
W = rng.standard_normal((M, K)).astype(np.float32)
H = rng.standard_normal((N, K)).astype(np.float32)
plan = comm.plan_coo(M, N, rows, cols, K, h_chunks=4)
a, b = plan.nnz_begin, plan.nnz_end
dW = torch.from_numpy(W[plan.row_begin:plan.row_end]).cuda()
dS = torch.from_numpy(vals[a:b]).cuda()
dH = torch.from_numpy(H).cuda() if rank == 0 else torch.zeros((N, K), device="cuda")   # only the root holds H
P = torch.full((b - a,), float("nan"), device="cuda")
plan.execute(dW, dH, P, dS, root=0)                  # chunked broadcast overlapped with the bucketed kernels
lr = rows[a:b] - plan.row_begin
assert_parity(P.cpu().numpy(), lr, cols[a:b], W[plan.row_begin:plan.row_end], H, vals[a:b])
assert torch.equal(dH.cpu(), torch.from_numpy(H))    # every rank now holds H
P.fill_(float("nan"))
plan.execute(dW, dH, P, dS, flags=api.DIST_H_RESIDENT)
assert_parity(P.cpu().numpy(), lr, cols[a:b], W[plan.row_begin:plan.row_end], H, vals[a:b])
plan.close(); comm.close(); h.close()
dist.barrier(); dist.destroy_process_group()
open(os.path.join(sys.argv[2], f"rank{rank}.ok"), "w").write("ok")
"""


def test_one_process_per_gpu_overlapped_broadcast(tmp_path):
    """Two ranks as child processes on two GPUs: NCCL communicator from the C ABI, H on the root only,
    broadcast in 4 chunks overlapped with the bucketed kernels; each rank checks its slice against the oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script), ROOT, str(tmp_path)],
                         capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert (tmp_path / "rank0.ok").exists() and (tmp_path / "rank1.ok").exists()
