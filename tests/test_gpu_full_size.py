"""The benchmark configurations at FULL size on the GPU, checked through properties that do not
need the oracle to run over the whole matrix: the oracle on a random sample of the nonzeros (their W
and H rows brought to the host), linearity in W, agreement between kernels, and the checksum of P
against the checksum of the sample-independent row sums it implies."""
import numpy as np
import pytest
import torch

import oracle
from helpers import WELL_CONDITIONED, parity_stats
from sddmm_gpu_b200 import api, synth

pytestmark = pytest.mark.gpu


def _sample_check(p, P, n_sample, seed, pick=None):
    """The CPU oracle on n_sample random nonzeros (rows/cols compacted so that only the touched
    operand rows leave the device)."""
    nnz = p["rows"].shape[0]
    g = torch.Generator(device="cpu").manual_seed(seed)
    if pick is None:
        pick = torch.randint(0, nnz, (n_sample,), generator=g).to(p["rows"].device)
    r, c = p["rows"][pick].long(), p["cols"][pick].long()
    ur, ri = torch.unique(r, return_inverse=True)
    uc, ci = torch.unique(c, return_inverse=True)
    Ws, Hs = p["W"][ur].cpu().numpy(), p["H"][uc].cpu().numpy()
    vals = p["vals"][pick].cpu().numpy()
    rows_s, cols_s = ri.cpu().numpy().astype(np.int32), ci.cpu().numpy().astype(np.int32)
    ref = oracle.cpu.sddmm_coo(rows_s, cols_s, Ws, Hs, vals)
    _, A = oracle.cpu.sddmm_coo_f64(rows_s, cols_s, Ws, Hs, vals)
    got = P[pick].cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    err = np.abs(got - ref)
    assert (err <= 1e-4 * np.maximum(np.abs(ref), A)).all(), f"max scaled error {np.max(err / np.maximum(A, 1e-30))}"
    # plain relative tolerance on the well-conditioned samples (threshold: tests/helpers.py)
    well = (np.abs(ref) >= WELL_CONDITIONED * A) & (np.abs(ref) > 0)
    assert well.any()
    rel = err[well] / np.abs(ref[well])
    assert rel.max() <= 1e-4, f"max relative error {rel.max()} on {int(well.sum())} well-conditioned samples"
    parity_stats["checked"] += int(ref.size)
    parity_stats["well_conditioned"] += int(well.sum())
    band = (~well) & (np.abs(ref) >= 1e-3 * A)
    parity_stats["between_1e-3_and_1e-2"] += int(band.sum())
    parity_stats["below_1e-3"] += int(ref.size - well.sum() - band.sum())


@pytest.mark.parametrize("name", ["c3", "c4", "c4_K512", "c4_K1024", "c5", "c5b"])
def test_full_size_configuration(engine, name):
    if name == "c3":
        p = synth.rmat(device="cuda")                       # scale 20, 16 M draws, K = 128
    elif name.startswith("c4"):
        # scale 22, 100 M draws; K = 512 and 1024 take offsets past 2^31 (M K = 2^31, 2^32) and 34 GB of operands
        p = synth.rmat_c4(K=int(name.split("_K")[1]) if "_K" in name else 256, device="cuda")
    elif name == "c5b":
        p = synth.attention_mask(n_global=1311, device="cuda")   # the "2 % global rows and columns" reading: 202 M nonzeros
    else:
        p = synth.attention_mask(device="cuda")             # 65,536 x 65,536, band 256 + 80 global, K = 64
    nnz = p["rows"].shape[0]
    torch.cuda.synchronize()
    plan = engine.plan_coo(p["M"], p["N"], p["rows"], p["cols"], p["K"])
    P = torch.full((nnz,), float("nan"), device="cuda")
    torch.cuda.synchronize()
    plan.execute(p["W"], p["H"], P, p["vals"])
    torch.cuda.synchronize()
    assert bool(torch.isfinite(P).all())                    # every nonzero was written
    _sample_check(p, P, 200_000, seed=1)
    if name in ("c4_K512", "c4_K1024"):
        # the 64 longest rows in full, as well as the random sample (hub rows are where a lane set keeps its W row longest)
        deg = torch.bincount(p["rows"], minlength=p["M"])
        top = torch.topk(deg, 64).indices
        sel = torch.nonzero(torch.isin(p["rows"], top.to(p["rows"].dtype))).squeeze(1)
        _sample_check(p, P, 0, seed=2, pick=sel[torch.randperm(sel.numel(), device=sel.device)[:300_000]])
        # and agreement with the panel kernel on everything; linearity is covered at K = 256
        P4 = torch.empty_like(P)
        plan.execute(p["W"], p["H"], P4, p["vals"], api.FLAG_KERNEL_PANEL)
        bound = 1e-5 * float(p["W"].abs().max() * p["H"].abs().max() * p["K"] * p["vals"].abs().max())
        assert float((P - P4).abs().max()) <= bound
        plan.close()
        return

    # linearity in W (S fixed): sddmm(W1 + W2) = sddmm(W1) + sddmm(W2) up to rounding
    W2 = torch.randn_like(p["W"]) * p["W"].std()
    P2, P3 = torch.empty_like(P), torch.empty_like(P)
    torch.cuda.synchronize()                               # the engine launches on its own stream
    plan.execute(W2, p["H"], P2, p["vals"])
    W2 += p["W"]
    torch.cuda.synchronize()
    plan.execute(W2, p["H"], P3, p["vals"])
    torch.cuda.synchronize()
    del W2
    bound = 1e-5 * float(p["W"].abs().max() * 3 * p["H"].abs().max() * p["K"] * p["vals"].abs().max())
    assert float((P + P2 - P3).abs().max()) <= bound

    # another kernel on the same plan agrees to rounding, and its checksum with it
    P4 = torch.empty_like(P)
    torch.cuda.synchronize()
    plan.execute(p["W"], p["H"], P4, p["vals"], api.FLAG_KERNEL_PANEL)
    torch.cuda.synchronize()
    assert float((P - P4).abs().max()) <= bound
    assert abs(float(P.double().sum() - P4.double().sum())) <= bound * nnz ** 0.5
    plan.close()
