"""Seeded synthetic inputs with the shapes, sizes and value distributions of the
benchmark configurations.  They stand in for the public datasets the reference's
scripts name but do not ship (bag-of-words corpora, SuiteSparse/SNAP graphs); no
record of any dataset is reproduced here.

Everything is generated with torch on the requested device (CPU for the tests,
CUDA for the full-size benchmark) from an explicit seed, so a run is reproducible
on a given device type.  The CPU oracle and the GPU kernels always consume the
same bytes: whatever is generated is handed to both.

A problem is a dict: M, N, K, rows, cols (int32, row-sorted, columns ascending
within a row), vals, W (M x K), H (N x K) (float32), name, panel_rows, col_tile
(the CLI's argv[3], argv[4] for the configuration).
"""
import math

import torch

SEEDS = {"c1": 1001, "c2": 1002, "c3": 1003, "c4": 1004, "c5": 1005}


def _gen(seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _finish(name, M, N, K, keys, vals_fn, wh_fn, device, seed, panel_rows, col_tile):
    """keys: sorted unique int64 cell ids row*N + col."""
    rows = torch.div(keys, N, rounding_mode="floor").to(torch.int32)
    cols = (keys - rows.to(torch.int64) * N).to(torch.int32)
    nnz = rows.shape[0]
    vals = vals_fn(nnz, _gen(seed + 40, device))
    W = wh_fn((M, K), _gen(seed + 10, device))
    H = wh_fn((N, K), _gen(seed + 20, device))
    return dict(name=name, M=M, N=N, K=K, rows=rows.contiguous(), cols=cols.contiguous(), vals=vals, W=W, H=H,
                panel_rows=panel_rows, col_tile=col_tile)


def uniform_sparse(M=4096, N=4096, density=0.001, K=32, seed=SEEDS["c1"], device="cpu"):
    """Config 1: uniformly random cells without replacement, S = 1, W/H uniform[0,1)."""
    nnz = int(math.floor(density * M * N))
    g = _gen(seed + 30, device)
    keys = torch.randperm(M * N, generator=g, device=device)[:nnz].to(torch.int64).sort().values
    return _finish("c1_uniform", M, N, K, keys,
                   lambda n, gg: torch.ones(n, dtype=torch.float32, device=device),
                   lambda s, gg: torch.rand(s, generator=gg, device=device, dtype=torch.float32),
                   device, seed, 32, 4096)


def bag_of_words(M=12419, N=1500, nnz=746316, K=256, seed=SEEDS["c2"], device="cpu"):
    """Config 2: row lengths ~ Zipf(1.1) over a random row permutation (scaled to hit
    nnz exactly, each <= N), columns per row drawn without replacement with
    popularity ~ Zipf(1.0), integer values 1..20, W/H uniform[0,1)."""
    g = _gen(seed + 30, device)
    rank = torch.arange(1, M + 1, device=device, dtype=torch.float64)
    w = rank.pow(-1.1)
    w = w[torch.randperm(M, generator=g, device=device)]
    lengths = torch.clamp(torch.floor(w / w.sum() * nnz), max=N).to(torch.int64)
    # hand the remainder out one by one to the rows with room, heaviest first
    while int(lengths.sum()) < nnz:
        room = (lengths < N).nonzero().flatten()
        order = room[torch.argsort(w[room], descending=True)]
        take = order[: nnz - int(lengths.sum())]
        lengths[take] += 1
    pop = torch.arange(1, N + 1, device=device, dtype=torch.float64).pow(-1.0)
    pop = pop[torch.randperm(N, generator=g, device=device)]
    logp = pop.log().to(torch.float32)
    key_chunks = []
    step = 2048
    for r0 in range(0, M, step):
        r1 = min(M, r0 + step)
        # Gumbel top-k = weighted sampling without replacement
        u = torch.rand((r1 - r0, N), generator=g, device=device, dtype=torch.float32).clamp_(1e-20, 1.0)
        score = logp[None, :] - torch.log(-torch.log(u))
        order = torch.argsort(score, dim=1, descending=True)
        take = torch.arange(N, device=device)[None, :] < lengths[r0:r1, None]
        rr = torch.arange(r0, r1, device=device, dtype=torch.int64)[:, None].expand(-1, N)
        key_chunks.append((rr * N + order)[take])
    keys = torch.cat(key_chunks).sort().values
    assert keys.shape[0] == nnz
    return _finish("c2_bagofwords", M, N, K, keys,
                   lambda n, gg: torch.randint(1, 21, (n,), generator=gg, device=device).to(torch.float32),
                   lambda s, gg: torch.rand(s, generator=gg, device=device, dtype=torch.float32),
                   device, seed, 192, 50000)


def rmat(scale=20, edge_factor=16, K=128, abcd=(0.57, 0.19, 0.19, 0.05), seed=SEEDS["c3"], device="cpu",
         name="c3_rmat", chunk=1 << 24):
    """Configs 3 and 4: R-MAT edges, duplicates removed, values normal(0,1),
    W/H normal(0, sigma=0.1)."""
    M = N = 1 << scale
    E = edge_factor * M
    a, b, c, _ = abcd
    g = _gen(seed + 30, device)
    parts = []
    for e0 in range(0, E, chunk):
        n = min(chunk, E - e0)
        r = torch.zeros(n, dtype=torch.int64, device=device)
        col = torch.zeros(n, dtype=torch.int64, device=device)
        for _ in range(scale):
            u = torch.rand(n, generator=g, device=device, dtype=torch.float32)
            rbit = (u >= a + b).to(torch.int64)                       # quadrants c, d
            cbit = (((u >= a) & (u < a + b)) | (u >= a + b + c)).to(torch.int64)  # quadrants b, d
            r = (r << 1) | rbit
            col = (col << 1) | cbit
        parts.append(torch.unique(r * N + col))
    keys = torch.unique(torch.cat(parts)) if len(parts) > 1 else parts[0]
    del parts
    return _finish(name, M, N, K, keys,
                   lambda n, gg: torch.randn(n, generator=gg, device=device, dtype=torch.float32),
                   lambda s, gg: torch.randn(s, generator=gg, device=device, dtype=torch.float32) * 0.1,
                   device, seed, 192, 1 << 30)


def rmat_c4(K=256, device="cpu", scale=22, edge_factor=24):
    return rmat(scale=scale, edge_factor=edge_factor, K=K, seed=SEEDS["c4"], device=device, name="c4_rmat")


def attention_mask(M=65536, half_width=256, n_global=80, K=64, seed=SEEDS["c5"], device="cpu"):
    """Config 5: band |i-j| <= half_width plus n_global fully dense rows and
    columns at seeded positions; S = 1, W = Q and H = K normal(0,1)."""
    N = M
    g = _gen(seed + 30, device)
    glob = torch.randperm(M, generator=g, device=device)[:n_global].to(torch.int64).sort().values
    parts = []
    step = 4096
    offs = torch.arange(-half_width, half_width + 1, device=device, dtype=torch.int64)
    for r0 in range(0, M, step):
        rr = torch.arange(r0, min(M, r0 + step), device=device, dtype=torch.int64)
        cc = rr[:, None] + offs[None, :]
        ok = (cc >= 0) & (cc < N)
        parts.append((rr[:, None] * N + cc)[ok])
    if n_global > 0:
        allc = torch.arange(N, device=device, dtype=torch.int64)
        parts.append((glob[:, None] * N + allc[None, :]).flatten())   # global rows
        parts.append((allc[:, None] * N + glob[None, :]).flatten())   # global columns
    keys = torch.unique(torch.cat(parts))
    del parts
    return _finish("c5_attention", M, N, K, keys,
                   lambda n, gg: torch.ones(n, dtype=torch.float32, device=device),
                   lambda s, gg: torch.randn(s, generator=gg, device=device, dtype=torch.float32),
                   device, seed, 128, 1 << 30)


def to_numpy(problem):
    """Host numpy copies of the tensors of a problem (for the CPU oracle)."""
    out = dict(problem)
    for k in ("rows", "cols", "vals", "W", "H"):
        out[k] = problem[k].detach().cpu().numpy()
    return out


def algorithmic_bytes(M, nnz, K, m_nz, n_nz):
    """Compulsory traffic of one SDDMM call: every touched W and H row once, per
    nonzero a column index, an S value and a P store, plus a row pointer array."""
    return 4 * K * (m_nz + n_nz) + 12 * nnz + 4 * (M + 1)
