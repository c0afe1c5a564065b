#!/usr/bin/env python
"""Benchmark of the SDDMM hot path: P = S o (W H^T) on a row-sorted sparse S.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c4|c3|c2|c1|c5] [--k K]

A step is one SDDMM over the whole synthetic matrix.  The default workload is
the power-law R-MAT matrix of scale 22 with ~100 M nonzeros at K = 256.  Rank 0
prints ONE JSON line:

  value        GFLOP/s (2*nnz*K / t) of the whole job, operands resident in HBM,
               t from CUDA events on the launching stream, max over ranks;
  roofline     compulsory bytes of one call / kernel time against the measured
               HBM copy bandwidth (MEASURED_PEAKS.json), plus DRAM traffic from
               the committed ncu capture when one exists for the workload;
  e2e          the same metric through the C ABI with HOST buffers: W, H, S values
               copied to the device and P copied back inside the timed region;
  cpu_baseline the CPU SDDMM (OpenMP, all host cores) on a bounded sample.

--impl reference times the reference's own CPU SDDMM (its sddmm_CPU_COO compiled
from the reference tree when that library was built, else the C port) on the
same workload, sampled; rank 0 only.

Multi-GPU: launched by torchrun, one rank per GPU.  S is cut into nnz-balanced
row blocks (strong scaling: the matrix is fixed), each rank holds its rows of W
and a full copy of H, which rank 0 broadcasts once over NCCL before the timed
region (its time is reported as h_broadcast_ms).  In the e2e figure every rank
uploads 1/N of H from its own pinned host slice and the slices are exchanged
over NVLink inside the timed region.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "cusparse"],
                    help="ours; the reference's CPU SDDMM; or cuSPARSE's SDDMM as a labelled library comparator")
    ap.add_argument("--workload", default="c4", choices=["c1", "c2", "c3", "c4", "c5", "c5b"])
    ap.add_argument("--k", type=int, default=0, help="override K of the workload")
    ap.add_argument("--scale", type=int, default=0, help="override the R-MAT scale (c3/c4), for quick runs")
    ap.add_argument("--kernel", default="auto", choices=["auto", "ring", "panel", "gather"])
    ap.add_argument("--col-tile", type=int, default=0, help="column-tile width passed to the plan (argv[4] of the CLI)")
    ap.add_argument("--op", default="sddmm", choices=["sddmm", "sddmm_bf16", "fused"],
                    help="sddmm: the benchmark proper.  sddmm_bf16 / fused: a short device-resident timing of the opt-in "
                         "bfloat16-operand SDDMM or of the fused SDDMM->SpMM on the chosen workload (one GPU), one JSON line")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-rebalance", action="store_true", help="N > 1: keep the equal-nonzero row blocks")
    ap.add_argument("--no-also", action="store_true", help="skip the short runs of the other configurations")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="target CPU time of the baseline sample")
    return ap.parse_args()


def make_problem(args, device):
    from sddmm_gpu_b200 import synth
    w = args.workload
    if w == "c1":
        p = synth.uniform_sparse(K=args.k or 32, device=device)
        name = "c1_uniform_4096x4096_d0.001"
    elif w == "c2":
        p = synth.bag_of_words(K=args.k or 256, device=device)
        name = "c2_bagofwords_12419x1500_nnz746316"
    elif w == "c3":
        s = args.scale or 20
        p = synth.rmat(scale=s, edge_factor=16, K=args.k or 128, device=device)
        name = f"c3_rmat_scale{s}_ef16"
    elif w == "c4":
        s = args.scale or 22
        p = synth.rmat_c4(K=args.k or 256, device=device, scale=s)
        name = f"c4_rmat_scale{s}_ef24"
    elif w == "c5b":
        # the "2 % of rows and columns are global" reading of the same configuration: 1311 global rows / columns
        p = synth.attention_mask(n_global=1311, K=args.k or 64, device=device)
        name = "c5b_attention_65536_band256_g1311"
    else:
        p = synth.attention_mask(K=args.k or 64, device=device)
        name = "c5_attention_65536_band256_g80"
    p["workload"] = f"{name}_K{p['K']}"
    return p


class ClockSampler:
    """Samples SM clock and clock-event reasons through NVML while a region runs (read-only)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.dev, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.dev)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic(workload, kernel):
    """The committed ncu DRAM-traffic record of the dominant kernel for this workload, if any
    (profiles/dram_bytes.json: bytes per launch, the duration ncu saw, how it was captured)."""
    try:
        table = json.load(open(os.path.join(ROOT, "profiles", "dram_bytes.json")))["captures"]
    except Exception:
        return None
    for rec in table:
        if rec["workload"] == workload and rec["kernel"] == kernel:
            return rec
    return None


def sample_blocks(nnz, n_sample, n_blocks=64):
    """Indices of n_blocks evenly spaced runs of consecutive nonzeros, n_sample in total."""
    n_sample = min(n_sample, nnz)
    n_blocks = max(1, min(n_blocks, n_sample))
    blen = n_sample // n_blocks
    starts = (np.arange(n_blocks, dtype=np.int64) * (nnz - blen)) // max(n_blocks - 1, 1)
    return (starts[:, None] + np.arange(blen, dtype=np.int64)[None, :]).reshape(-1)


def build_cpu_sample(rows_h, cols_h, vals_h, W_of_rows, nnz, n_sample):
    """Sample of the workload for the CPU legs: blocks of consecutive nonzeros, the W
    rows they touch compacted (same reuse pattern, small copy), H whole."""
    idx = sample_blocks(nnz, n_sample)
    r, c, v = rows_h[idx], cols_h[idx], vals_h[idx]
    uniq, inv = np.unique(r, return_inverse=True)
    Ws = W_of_rows(uniq)
    return inv.astype(np.int32), np.ascontiguousarray(c), np.ascontiguousarray(v), Ws, idx.shape[0]


def oracle_sample_check(rows_d, cols_d, vals_d, W_d, H_d, results, n_sample=262_144, n_blocks=256):
    """Worst scaled error |P - ref| / max(|ref|, A) of the given result arrays (device or host
    tensors, aligned with rows_d) against the CPU oracle (sequential fp32, as the reference; A from its
    float64 companion) on n_sample nonzeros taken as evenly spaced blocks over the WHOLE slice.  Only
    the W and H rows the sample touches leave the device."""
    import oracle
    nnz = int(rows_d.shape[0])
    if nnz == 0:
        return 0.0, 0
    idx = torch.from_numpy(sample_blocks(nnz, min(nnz, n_sample), n_blocks)).to(rows_d.device)
    r, c = rows_d[idx].long(), cols_d[idx].long()
    ur, ri = torch.unique(r, return_inverse=True)
    uc, ci = torch.unique(c, return_inverse=True)
    Ws, Hs = W_d[ur].cpu().numpy(), H_d[uc].cpu().numpy()
    v = vals_d[idx].cpu().numpy()
    rs, cs = ri.cpu().numpy().astype(np.int32), ci.cpu().numpy().astype(np.int32)
    ref = oracle.cpu.sddmm_coo(rs, cs, Ws, Hs, v).astype(np.float64)
    _, A = oracle.cpu.sddmm_coo_f64(rs, cs, Ws, Hs, v)
    denom = np.maximum(np.maximum(np.abs(ref), A), 1e-30)
    worst = 0.0
    idx_h = idx.cpu()
    for res in results:
        got = (res[idx] if res.is_cuda else res[idx_h]).cpu().numpy().astype(np.float64)
        err = np.abs(got - ref) / denom
        worst = max(worst, float(np.max(np.where(np.isfinite(err), err, np.inf))))
    return worst, int(idx.shape[0])


def quick_run(handle, p, peak, steps=5, warmup=3, bf16=False):
    """A short device-resident timing of one configuration: plan, warm-up, `steps` timed executes
    (CUDA events on the launching stream), a sampled oracle check.  bf16: the opt-in bfloat16 operand
    storage (fp32 accumulate), checked against the oracle on the rounded operands."""
    from sddmm_gpu_b200 import api, synth
    nnz = int(p["rows"].shape[0])
    if bf16:
        p = dict(p)
        p["W16"], p["H16"] = p["W"].to(torch.bfloat16), p["H"].to(torch.bfloat16)
        p["W"], p["H"] = p["W16"].float(), p["H16"].float()     # what the kernel sees, for the oracle
    Wk, Hk = (p["W16"], p["H16"]) if bf16 else (p["W"], p["H"])
    xflag = api.FLAG_OPERANDS_BF16 if bf16 else 0
    # planned twice: the first plan of a process also pays for loading the binning kernels and for fresh
    # device allocations; plan_ms below is the second plan's
    handle.plan_coo(p["M"], p["N"], p["rows"], p["cols"], p["K"], p.get("panel_rows", 0), p.get("col_tile", 0)).close()
    plan = handle.plan_coo(p["M"], p["N"], p["rows"], p["cols"], p["K"], p.get("panel_rows", 0), p.get("col_tile", 0))
    info = plan.info()
    P = torch.empty(nnz, device=p["rows"].device, dtype=torch.float32)
    for _ in range(warmup):
        plan.execute(Wk, Hk, P, p["vals"], api.FLAG_ASYNC | xflag)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record()
    for i in range(steps):
        plan.execute(Wk, Hk, P, p["vals"], api.FLAG_ASYNC | xflag)
        evs[i + 1].record()
    handle.sync()
    ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    mean_ms = sum(ms) / len(ms)
    alg = synth.algorithmic_bytes(p["M"], nnz, p["K"], info.n_nonempty_rows, plan.count_cols())
    if bf16:   # operand rows are half as long
        alg -= 2 * p["K"] * (info.n_nonempty_rows + plan.count_cols())
    worst, n_checked = oracle_sample_check(p["rows"], p["cols"], p["vals"], p["W"], p["H"], [P], 65_536, 64)
    out = {"workload": p["workload"], "nnz": nnz, "K": p["K"], "ms_per_step": mean_ms, "ms_min": min(ms),
           "gflops": 2.0 * nnz * p["K"] / (mean_ms * 1e-3) / 1e9, "algorithmic_bytes": alg,
           "frac": alg / (mean_ms * 1e-3) / 1e9 / peak, "kernel": plan.last_kernel_name(),
           "dense_cell_share": (info.n_dense_nnz / nnz) if nnz else 0.0, "plan_ms": info.plan_ms,
           "parity_max_scaled_err": worst, "parity_n_checked": n_checked, "steps": steps}
    if bf16:
        out["operands"] = "bf16 storage, fp32 accumulate (opt-in, outside the fp32 tolerance contract; oracle on rounded operands)"
    plan.close()
    return out


def quick_run_fused(handle, p, peak, steps=5, warmup=3):
    """The fused SDDMM->SpMM (Y = (S o (W H^T)) H, P never stored) and the unfused pair (SDDMM, then SpMM over the
    stored P) on one configuration; algorithmic bytes of the fused form: every touched row of W and H once, Y
    written once (all M rows), per nonzero a column index and an S value, the row pointer."""
    from sddmm_gpu_b200 import api
    nnz, M, K = int(p["rows"].shape[0]), p["M"], p["K"]
    plan = handle.plan_coo(M, p["N"], p["rows"], p["cols"], K)
    info = plan.info()
    dev = p["rows"].device
    Y = torch.empty((M, K), device=dev, dtype=torch.float32)
    P = torch.empty(nnz, device=dev, dtype=torch.float32)

    def timed(fn):
        for _ in range(warmup):
            fn()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        evs[0].record()
        for i in range(steps):
            fn()
            evs[i + 1].record()
        handle.sync()
        return sum(evs[i].elapsed_time(evs[i + 1]) for i in range(steps)) / steps

    t_fused = timed(lambda: plan.fused(p["W"], p["H"], Y, p["vals"], None, api.FLAG_ASYNC))
    Yf = Y.clone()

    def pair():
        plan.execute(p["W"], p["H"], P, p["vals"], api.FLAG_ASYNC)
        plan.spmm(p["H"], Y, P, api.FLAG_ASYNC)

    t_pair = timed(pair)
    # the two routes agree up to the rounding of P (the fused form is checked against the CPU loops in the tests)
    scale = float(Y.abs().max()) + 1e-30
    diff = float((Y - Yf).abs().max()) / scale
    n_nz = plan.count_cols()
    alg = 4 * K * (info.n_nonempty_rows + n_nz) + 4 * K * M + 8 * nnz + 8 * (M + 1)
    out = {"workload": p["workload"], "op": "fused_sddmm_spmm", "nnz": nnz, "K": K, "ms_per_step": t_fused,
           "unfused_pair_ms": t_pair, "gflops": 4.0 * nnz * K / (t_fused * 1e-3) / 1e9, "algorithmic_bytes": alg,
           "frac": alg / (t_fused * 1e-3) / 1e9 / peak, "kernel": "fused_sddmm_spmm",
           "max_diff_vs_unfused_pair_rel_to_max": diff, "steps": steps}
    plan.close()
    return out


def run_also(handle, device, peak, c4_pattern, args):
    """The other benchmark configurations and config 4's K sweep, a few steps each, so that
    one default run shows every configuration's time and roofline fraction (frac = algorithmic bytes /
    time / measured HBM peak; recomputable from the entry)."""
    from sddmm_gpu_b200 import synth
    out = []

    def go(make, compare=False, bf16=False):
        p = make()
        try:
            out.append(quick_run(handle, p, peak, bf16=bf16))
            if compare:
                # same operands through cuSPARSE's SDDMM: a library comparator beside this entry's time
                try:
                    ms, _ = cusparse_sddmm_ms(p)
                    out[-1]["comparators"] = {"cusparse_ms": ms, "what": "cusparseSDDMM via torch.sparse.sampled_addmm, "
                                                                        "CSR fp32, then values * S"}
                except Exception as ex:
                    out[-1]["comparators"] = {"cusparse_ms": None, "error": str(ex)[:160]}
        except Exception as ex:  # a failure here must not lose the headline line
            out.append({"workload": p.get("workload", "?"), "error": str(ex)[:200]})
        del p
        torch.cuda.empty_cache()

    def named(p, name):
        p["workload"] = f"{name}_K{p['K']}"
        return p

    if c4_pattern is not None:
        rows, cols, vals, M, N = c4_pattern
        for K in (32, 64, 128, 512, 1024):   # the K sweep of config 4 (K = 256 is the headline and follows below)
            def make(K=K):
                g = torch.Generator(device=device)
                g.manual_seed(synth.SEEDS["c4"] + K)
                return dict(M=M, N=N, K=K, rows=rows, cols=cols, vals=vals, workload=f"c4_rmat_scale22_ef24_K{K}",
                            W=torch.randn((M, K), generator=g, device=device) * 0.1,
                            H=torch.randn((N, K), generator=g, device=device) * 0.1, panel_rows=192, col_tile=1 << 30)
            go(make)
    if c4_pattern is not None:
        rows, cols, vals, M, N = c4_pattern

        def make_fused():
            g = torch.Generator(device=device)
            g.manual_seed(synth.SEEDS["c4"] + 256)
            return dict(M=M, N=N, K=256, rows=rows, cols=cols, vals=vals, workload="c4_rmat_scale22_ef24_K256",
                        W=torch.randn((M, 256), generator=g, device=device) * 0.1,
                        H=torch.randn((N, 256), generator=g, device=device) * 0.1)
        go(make_fused, compare=True)            # config 4 at K = 256 once more, beside cuSPARSE on the same operands
        go(make_fused, bf16=True)               # and with the operands stored in bfloat16
        pf = make_fused()
        try:
            out.append(quick_run_fused(handle, pf, peak))
        except Exception as ex:
            out.append({"workload": pf["workload"], "op": "fused_sddmm_spmm", "error": str(ex)[:200]})
        del pf
        torch.cuda.empty_cache()
    go(lambda: named(synth.uniform_sparse(device=device), "c1_uniform_4096x4096_d0.001"))
    go(lambda: named(synth.bag_of_words(device=device), "c2_bagofwords_12419x1500_nnz746316"), compare=True)
    go(lambda: named(synth.rmat(device=device), "c3_rmat_scale20_ef16"), compare=True)
    go(lambda: named(synth.attention_mask(device=device), "c5_attention_65536_band256_g80"))
    go(lambda: named(synth.attention_mask(n_global=1311, device=device), "c5b_attention_65536_band256_g1311"))
    return out


def cpu_port_rate(r, c, W, H, K, seconds):
    """GFLOP/s of the C port (OpenMP, all cores) on a sample sized for ~`seconds`."""
    import oracle
    probe = min(r.shape[0], 200_000)
    _, t = oracle.cpu.sddmm_coo(r[:probe], c[:probe], W, H, return_seconds=True)
    _, t = oracle.cpu.sddmm_coo(r[:probe], c[:probe], W, H, return_seconds=True)
    n = int(min(r.shape[0], max(probe, probe * seconds / max(t, 1e-6))))
    best = None
    for _ in range(2):
        _, t = oracle.cpu.sddmm_coo(r[:n], c[:n], W, H, return_seconds=True)
        best = t if best is None else min(best, t)
    return 2.0 * n * K / best / 1e9, n, oracle.cpu.max_threads()


def run_reference(args, rank):
    """--impl reference: the reference's CPU SDDMM on the host cores, rank 0 only."""
    if rank != 0:
        return
    import oracle
    device = "cuda" if torch.cuda.is_available() else "cpu"
    p = make_problem(args, device)
    K, nnz, M, N = p["K"], int(p["rows"].shape[0]), p["M"], p["N"]
    rows_h, cols_h, vals_h = (p[k].cpu().numpy() for k in ("rows", "cols", "vals"))
    H_h = p["H"].cpu().numpy()
    Wt = p["W"]
    # The sample depends on the workload only (never on a timing probe or on OMP_NUM_THREADS), so that every
    # launch of this arm -- alone or as rank 0 under torchrun, on any box -- times the same nonzeros:
    # all of them up to 60 GFLOP per step, else that many in 64 evenly spaced blocks.
    n_step = int(min(nnz, max(200_000, 60e9 / (2.0 * K))))
    r, c, v, Ws, _ = build_cpu_sample(rows_h, cols_h, vals_h,
                                      lambda u: Wt[torch.from_numpy(u).to(Wt.device)].cpu().numpy(), nnz, n_step)
    n_step = min(n_step, r.shape[0])
    r, c, v = r[:n_step], c[:n_step], v[:n_step]
    del p
    times = []
    if oracle.ref is not None:
        kind, cores = "reference", 28  # the reference forces 28 OpenMP threads (sddmm.cu:184)
        st = oracle.ref.lib.ref_coo_state_create(r, c, v, n_step, Ws.shape[0], N, Ws, H_h, K)
        copy_s = min(oracle.ref.lib.ref_coo_state_run(st, 0) for _ in range(3))
        for i in range(args.warmup + args.steps):
            t = oracle.ref.lib.ref_coo_state_run(st, n_step) - copy_s
            if i >= args.warmup:
                times.append(max(t, 1e-9))
        oracle.ref.lib.ref_coo_state_destroy(st)
        note = (f"{n_step} nonzeros in 64 evenly spaced blocks ({100.0 * n_step / nnz:.2f}% of nnz), W rows "
                f"compacted, H whole; sddmm_CPU_COO by-value argument copies ({copy_s:.2f} s per call) subtracted, "
                f"as its own timer excludes them")
    else:
        kind, cores = "port", os.cpu_count() or 1   # all host cores, whatever OMP_NUM_THREADS the launcher set
        for i in range(args.warmup + args.steps):
            _, t = oracle.cpu.sddmm_coo(r, c, Ws, H_h, return_seconds=True, threads=cores)
            if i >= args.warmup:
                times.append(t)
        note = f"{n_step} nonzeros in 64 evenly spaced blocks ({100.0 * n_step / nnz:.2f}% of nnz), W rows compacted, H whole"
    ms = 1e3 * sum(times) / len(times)
    value = 2.0 * n_step * K / (ms * 1e-3) / 1e9
    line = {
        "impl": "reference", "metric": "SDDMM GFLOP/s (2*nnz*K)", "value": value, "unit": "GFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": p_workload(args), "M": M, "N": N, "nnz": nnz, "K": K},
        "cpu_baseline": {"value": value, "unit": "GFLOP/s", "cores": cores, "kind": kind, "sample": note,
                         "host_cores": os.cpu_count()},
        "e2e": {"value": value, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cusparse_sddmm_ms(p, steps=3, warmup=2):
    """Milliseconds per SDDMM of cuSPARSE's kernel (torch.sparse.sampled_addmm on the CSR pattern, then * S) on the
    operands of problem p: a labelled library comparator, nothing of this repository runs in it."""
    device = p["rows"].device
    M, N, nnz = p["M"], p["N"], int(p["rows"].shape[0])
    crow = torch.zeros(M + 1, dtype=torch.int64, device=device)
    crow[1:] = torch.cumsum(torch.bincount(p["rows"], minlength=M), 0)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        pattern = torch.sparse_csr_tensor(crow.to(torch.int32), p["cols"], torch.zeros(nnz, device=device), size=(M, N))
    Ht = p["H"].t()

    def step():
        return torch.sparse.sampled_addmm(pattern, p["W"], Ht, beta=0.0, alpha=1.0).values() * p["vals"]

    for _ in range(warmup):
        res = step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        res = step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps, res


def run_cusparse(args, rank):
    """--impl cusparse: cuSPARSE's SDDMM (through torch.sparse.sampled_addmm on a CSR pattern) on the same
    synthetic operands, one GPU, rank 0.  A labelled LIBRARY comparator: it says how a vendor kernel does on
    the workload; it is neither the product nor the oracle."""
    if rank != 0:
        return
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "cusparse", "unavailable": "no CUDA device"}), flush=True)
        return
    device = torch.device("cuda", 0)
    p = make_problem(args, device)
    M, N, K = p["M"], p["N"], p["K"]
    rows, cols, vals, W, H = p["rows"], p["cols"], p["vals"], p["W"], p["H"]
    nnz = int(rows.shape[0])
    try:
        crow = torch.zeros(M + 1, dtype=torch.int64, device=device)
        crow[1:] = torch.cumsum(torch.bincount(rows, minlength=M), 0)
        # cuSPARSE's SDDMM computes alpha (A B) o spy(C) + beta C: the pattern only; S's values are applied afterwards
        pattern = torch.sparse_csr_tensor(crow.to(torch.int32), cols, torch.zeros(nnz, device=device), size=(M, N))
        Ht = H.t()   # a view: op(B) = H^T, no copy of H
        steps, warmup = args.steps, max(args.warmup, 3)

        def step():
            out = torch.sparse.sampled_addmm(pattern, W, Ht, beta=0.0, alpha=1.0)
            return out.values() * vals

        for _ in range(warmup):
            res = step()
        torch.cuda.synchronize()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        evs[0].record()
        for i in range(steps):
            res = step()
            evs[i + 1].record()
        torch.cuda.synchronize()
        ms = sum(evs[i].elapsed_time(evs[i + 1]) for i in range(steps)) / steps
        worst, n_checked = oracle_sample_check(rows, cols, vals, W, H, [res], 65_536, 64)
        line = {"impl": "cusparse", "metric": "SDDMM GFLOP/s (2*nnz*K)", "value": 2.0 * nnz * K / (ms * 1e-3) / 1e9,
                "unit": "GFLOP/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
                "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                "config": {"workload": p["workload"], "M": M, "N": N, "nnz": nnz, "K": K},
                "library": "cusparseSDDMM via torch.sparse.sampled_addmm (CSR, fp32), then values * S",
                "parity_max_scaled_err": worst, "parity_n_checked": n_checked}
    except Exception as ex:
        line = {"impl": "cusparse", "unavailable": str(ex)[:300]}
    print(json.dumps(line), flush=True)


def p_workload(args):
    K = args.k or {"c1": 32, "c2": 256, "c3": 128, "c4": 256, "c5": 64, "c5b": 64}[args.workload]
    s3, s4 = args.scale or 20, args.scale or 22
    return {"c1": "c1_uniform_4096x4096_d0.001", "c2": "c2_bagofwords_12419x1500_nnz746316",
            "c3": f"c3_rmat_scale{s3}_ef16", "c4": f"c4_rmat_scale{s4}_ef24",
            "c5": "c5_attention_65536_band256_g80", "c5b": "c5b_attention_65536_band256_g1311"}[args.workload] + f"_K{K}"


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.impl == "cusparse":
        run_cusparse(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU fallback")
    from sddmm_gpu_b200 import api, multi_gpu, synth
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    p = make_problem(args, device)
    M, N, K = p["M"], p["N"], p["K"]
    rows, cols, vals, W, H = p["rows"], p["cols"], p["vals"], p["W"], p["H"]
    nnz = int(rows.shape[0])
    handle = api.Handle(local_rank)
    if args.op != "sddmm":
        # the neighbouring operations: not the headline metric, one short timing each
        if world > 1:
            raise SystemExit("--op sddmm_bf16 / fused run on one GPU")
        peak, _ = hbm_peak()
        steps = max(args.steps, 3)
        out = quick_run_fused(handle, p, peak, steps) if args.op == "fused" else quick_run(handle, p, peak, steps, bf16=True)
        out.update({"op": args.op, "unit": "GFLOP/s", "value": out["gflops"], "n_gpus": 1, "data": "synthetic"})
        print(json.dumps(out), flush=True)
        handle.close()
        return
    # Everything below runs on one explicit (non-default) torch stream that the
    # engine is told to launch on, so that torch's CUDA events see its kernels.
    stream = torch.cuda.Stream(device=device)
    torch.cuda.set_stream(stream)
    handle.set_stream(stream.cuda_stream)
    kflag = {"auto": 0, "ring": api.FLAG_KERNEL_RING, "panel": api.FLAG_KERNEL_PANEL,
             "gather": api.FLAG_KERNEL_GATHER}[args.kernel]

    # ---- sharding through the C ABI (identity at one GPU) --------------------------
    # Every rank holds the whole pattern; sddmm_dist_plan_coo cuts it into nnz-balanced row blocks and plans
    # this rank's block (plus, at N > 1, the column-bucketed form used while H is being broadcast).
    comm = None
    if world > 1:
        ids = [api.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)          # plumbing: 128 bytes from rank 0 to everybody
        comm = api.Comm(handle, ids[0], rank, world)
    else:
        comm = api.Comm(handle, b"\0" * api.COMM_ID_BYTES, 0, 1)
    H_CHUNKS = 8
    dplan = comm.plan_coo(M, N, rows, cols, K, p["panel_rows"], h_chunks=H_CHUNKS)

    def take_shard(dp):
        a_, b_ = dp.nnz_begin, dp.nnz_end
        return (a_, b_, dp.row_begin, dp.row_end, (rows[a_:b_] - dp.row_begin).contiguous(), cols[a_:b_].contiguous(),
                vals[a_:b_].contiguous(), W[dp.row_begin:dp.row_end].contiguous() if world > 1 else W)

    a, b, row_begin, row_end, l_rows, l_cols, l_vals, l_W = take_shard(dplan)
    plan = dplan.local
    rows_host = rows.cpu().numpy() if (world == 1 and not args.no_cpu) else None
    h_bcast_ms = 0.0
    bcast = None
    rebalance = None
    if world > 1:
        if rank != 0:
            H.zero_()  # only rank 0's copy counts; everyone else receives it
        dist.barrier()
        torch.cuda.synchronize()
        for _ in range(2):   # the first collective of a communicator also sets up its channels: time the second
            dplan.execute(l_W, H, None, l_vals, root=0, flags=api.DIST_BROADCAST_ONLY)   # H arrives in H_CHUNKS pieces
            h_bcast_ms = dplan.last_times()[0]
            dist.barrier()
        # Equal nonzeros are not equal time: blocks of short rows cost more per nonzero (more W rows, colder
        # columns).  Measure every rank's nonzeros per millisecond on the equal split, re-cut the rows in
        # proportion (sddmm_dist_plan_coo_shares), and keep the new split -- part of set-up, like the plan.
        if not args.no_rebalance:
            history = []
            for _ in range(2):
                Pt = torch.empty(b - a, device=device, dtype=torch.float32)
                for _ in range(2):
                    plan.execute(l_W, H, Pt, l_vals, kflag | api.FLAG_ASYNC)
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(4):
                    plan.execute(l_W, H, Pt, l_vals, kflag | api.FLAG_ASYNC)
                e1.record()
                torch.cuda.synchronize()
                mine = torch.tensor([e0.elapsed_time(e1) / 4, float(b - a)], device=device, dtype=torch.float64)
                every = [torch.zeros_like(mine) for _ in range(world)]
                dist.all_gather(every, mine)
                t_r = np.array([float(x[0].item()) for x in every])
                n_r = np.array([float(x[1].item()) for x in every])
                history.append({"rank_ms": [round(x, 4) for x in t_r.tolist()], "rank_nnz": [int(x) for x in n_r.tolist()]})
                del Pt
                if t_r.max() / t_r.min() < 1.03:
                    break
                shares = n_r / t_r
                dplan.close()
                dplan = comm.plan_coo(M, N, rows, cols, K, p["panel_rows"], h_chunks=H_CHUNKS, rank_shares=shares)
                a, b, row_begin, row_end, l_rows, l_cols, l_vals, l_W = take_shard(dplan)
                plan = dplan.local
            rebalance = {"what": "row blocks re-cut in proportion to each rank's measured nonzeros per millisecond",
                         "rounds": history}
        del W
    info = plan.info()
    m_nz_local = info.n_nonempty_rows
    n_nz_local = plan.count_cols()
    P = torch.empty(b - a, device=device, dtype=torch.float32)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    launches_before = handle.kernel_launches()
    # ---- device-resident timing ------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        plan.execute(l_W, H, P, l_vals, kflag | api.FLAG_ASYNC)
    barrier()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    with ClockSampler(local_rank) as clocks:
        evs[0].record()
        for i in range(args.steps):
            plan.execute(l_W, H, P, l_vals, kflag | api.FLAG_ASYNC)
            evs[i + 1].record()
        barrier()
    step_ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    total_ms = evs[0].elapsed_time(evs[-1])
    t = torch.tensor([total_ms], device=device, dtype=torch.float64)
    rank_ms = [total_ms / args.steps]
    if world > 1:
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        rank_ms = [float(x.item()) / args.steps for x in every]
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms_max = float(t.item())
    ms_per_step = total_ms_max / args.steps
    value = 2.0 * nnz * K / (ms_per_step * 1e-3) / 1e9

    kernel_name = plan.last_kernel_name()   # what actually ran: ring, ring_small, panel, gather, dense_*+...
    # ---- roofline of the dominant kernel (this rank's launch) -------------------
    peak, peak_kind = hbm_peak()
    alg_bytes = synth.algorithmic_bytes(row_end - row_begin, b - a, K, m_nz_local, n_nz_local)
    kernel_ms = statistics.mean(step_ms)
    achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
    capture = ncu_traffic(p["workload"], kernel_name) if world == 1 else None
    traffic = capture["dram_bytes_per_launch"] if capture else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "peak_source": peak_kind, "algorithmic_bytes": alg_bytes,
                "kernel_ms": kernel_ms, "kernel_ms_min": min(step_ms), "kernel_ms_median": statistics.median(step_ms),
                "frac_of_nominal_8000": achieved / 8000.0,
                "kernel": kernel_name}
    if capture:
        # measured: the capture's bytes over the capture's own duration.  The same bytes over THIS run's
        # kernel time is an estimate (another GPU, another day) and is labelled as one.
        roofline["traffic_source"] = capture["source"]
        roofline["traffic_scaled_from"] = capture.get("scaled_from")
        roofline["dram_frac_at_capture"] = traffic / (capture["ncu_duration_ms"] * 1e-3) / 1e9 / peak
        roofline["dram_frac_estimate_live"] = traffic / (kernel_ms * 1e-3) / 1e9 / peak
        roofline["traffic_ratio"] = traffic / alg_bytes
    gather_bytes = 4 * K * (b - a) + 4 * K * m_nz_local + 12 * (b - a) + 4 * (row_end - row_begin + 1)
    roofline["gather_model_bytes"] = gather_bytes
    roofline["gather_model_gbs"] = gather_bytes / (kernel_ms * 1e-3) / 1e9

    # ---- H broadcast overlapped with compute (N > 1): the timing protocol's t_compute + t_bcastH ----
    if world > 1:
        t_tot, t_bc = [], []
        for i in range(1 + max(3, min(args.steps, 5))):
            barrier()
            dplan.execute(l_W, H, P, l_vals, root=0)          # chunked broadcast + bucketed kernels, synchronous
            tb, _, tt = dplan.last_times()
            if i > 0:
                t_tot.append(tt)
                t_bc.append(tb)
        tv = torch.tensor([sum(t_tot) / len(t_tot), sum(t_bc) / len(t_bc), h_bcast_ms], device=device, dtype=torch.float64)
        dist.all_reduce(tv, op=dist.ReduceOp.MAX)
        bcast = {"h_bytes": 4 * N * K, "chunks": dplan.n_chunks, "t_bcast_ms": float(tv[2].item()),
                 "t_bcast_inside_overlapped_call_ms": float(tv[1].item()), "t_compute_ms": ms_per_step,
                 "t_compute_plus_bcast_ms": float(tv[0].item()),
                 "overlap_ratio": float(tv[0].item()) / max(ms_per_step, float(tv[2].item())),
                 "how": "max over ranks, CUDA events on each rank's compute stream; root's H goes out in column-range "
                        "chunks on a communication stream, each chunk's nonzero bucket is computed as soon as it lands"}

    # ---- end to end through the C ABI with host buffers -------------------------
    e2e = None
    hW = hH = hS = hP = None
    if not args.no_e2e:
        try:
            hW = torch.empty(l_W.shape, dtype=torch.float32, pin_memory=True).copy_(l_W)
            hS = torch.empty(l_vals.shape, dtype=torch.float32, pin_memory=True).copy_(l_vals)
            hP = torch.empty(P.shape, dtype=torch.float32, pin_memory=True)
            # host copy of H: whole on one GPU; with several ranks each pins 1/world of the rows
            h0, h1 = multi_gpu.h_slice_bounds(N, rank, world)
            hH = torch.empty((h1 - h0, K), dtype=torch.float32, pin_memory=True).copy_(H[h0:h1])
            torch.cuda.synchronize()

            staging = {}
            up_bytes = [0]
            h_rows = multi_gpu.used_h_rows_of_slice(cols, N, rank, world) if world > 1 else None
            phases = {} if world > 1 else None
            torch.cuda.synchronize()

            def e2e_step():
                if world == 1:
                    plan.execute(hW, hH, hP, hS, kflag)         # H2D W, H, S; kernel; D2H P; synchronous
                else:
                    # every rank uploads its slice of H over its own PCIe link and the slices are exchanged
                    # over NVLink while the rank's W rows and S values are uploaded; kernel; D2H P
                    up_bytes[0] = multi_gpu.host_step(plan, rank, world, hW, hH, H, hP, hS, kflag, staging, h_rows,
                                                      comm=comm, phases=phases)

            n_e2e = max(3, min(args.steps, 5))
            for _ in range(2):
                e2e_step()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n_e2e):
                e2e_step()
            e1.record()
            barrier()
            te = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(te, op=dist.ReduceOp.MAX)
            e2e_ms = float(te.item()) / n_e2e
            if world == 1:
                h2d, d2h = plan.last_transfer_bytes()          # what the call moved (untouched W/H rows do not travel)
            else:
                h2d = up_bytes[0]
                d2h = 4 * P.numel()
            operand = 4 * (l_W.numel() + l_vals.numel() + hH.numel())
            tb = torch.tensor([h2d, d2h, operand], device=device, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(tb, op=dist.ReduceOp.SUM)
            e2e = {"value": 2.0 * nnz * K / (e2e_ms * 1e-3) / 1e9, "unit": "GFLOP/s",
                   "h2d_bytes_per_step": int(tb[0].item()), "d2h_bytes_per_step": int(tb[1].item()),
                   "ms_per_step": e2e_ms, "steps": n_e2e, "host_memory": "pinned",
                   "outside_the_step": "the plan (binning pass, plan_ms) and the upload of the 8 nnz bytes of row and "
                                       "column indices it keeps; the reference uploads indices inside sddmm_GPU",
                   "operand_bytes": int(tb[2].item())}
            if phases:
                # the last step's phases, each the max over ranks (they overlap: W/S upload runs beside the exchange)
                ph = multi_gpu.phase_times(phases)
                keys = sorted(ph)
                tph = torch.tensor([ph[k] for k in keys], device=device, dtype=torch.float64)
                dist.all_reduce(tph, op=dist.ReduceOp.MAX)
                e2e["phases_ms_max_over_ranks"] = {k: round(float(v), 3) for k, v in zip(keys, tph.tolist())}
            # the host copy of the result is the one that is checked below
            P_check = hP
        except RuntimeError as ex:  # e.g. pinned allocation refused
            e2e = {"value": None, "unit": "GFLOP/s", "error": str(ex)[:200]}
            P_check = None
    else:
        P_check = None

    # ---- parity with the CPU oracle, every rank, every world size ---------------
    # >= 262,144 nonzeros in 256 evenly spaced blocks over the rank's whole slice; both the device-resident
    # result and the host result of the end-to-end step are checked; a disagreement ends the run non-zero.
    handle.sync()                                   # also reads the device status word of the FLAG_ASYNC calls
    results = [P] + ([P_check] if P_check is not None else [])
    worst, n_checked = oracle_sample_check(l_rows, l_cols, l_vals, l_W, H, results)
    tp = torch.tensor([worst], device=device, dtype=torch.float64)
    per_rank = [worst]
    n_total = torch.tensor([n_checked], device=device, dtype=torch.int64)
    if world > 1:
        every = [torch.zeros_like(tp) for _ in range(world)]
        dist.all_gather(every, tp)
        per_rank = [float(x.item()) for x in every]
        dist.all_reduce(n_total, op=dist.ReduceOp.SUM)
    parity = {"max_scaled_err": max(per_rank), "n_checked": int(n_total.item()), "per_rank": per_rank,
              "checked": "P resident" + (" and P from the end-to-end step" if P_check is not None else ""),
              "tolerance": 1e-4, "oracle": "oracle/sddmm_oracle.c (fp32 sequential) + float64 magnitude scale"}
    parity_failed = not (parity["max_scaled_err"] <= 1e-4)

    # ---- CPU baseline on a bounded sample (rank 0, one GPU) ----------------------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cols_h, vals_h = cols.cpu().numpy(), vals.cpu().numpy()
        H_h = H.cpu().numpy()
        r, c, v, Ws, n_s = build_cpu_sample(rows_host, cols_h, vals_h,
                                            lambda u: l_W[torch.from_numpy(u).to(device)].cpu().numpy(), nnz,
                                            min(nnz, 40_000_000))
        gflops, n_used, cores = cpu_port_rate(r, c, Ws, H_h, K, args.cpu_seconds)
        cpu_baseline = {"value": gflops, "unit": "GFLOP/s", "cores": cores, "kind": "port",
                        "sample": f"{n_used} nonzeros ({100.0 * n_used / nnz:.2f}% of nnz) from 64 evenly spaced "
                                  f"blocks, W rows compacted, H whole; best of 2"}
        del r, c, v, Ws, H_h, cols_h, vals_h

    launches_main = handle.kernel_launches() - launches_before

    # ---- the other configurations, briefly (one GPU) ----------------------------
    also = None
    if rank == 0 and world == 1 and not args.no_also and not parity_failed:
        c4_pattern = (rows, cols, vals, M, N) if (args.workload == "c4" and not args.scale) else None
        del W, H, l_W, P, hW, hH, hS, hP, P_check, results, l_rows, l_cols, l_vals
        for key in ("W", "H", "rows", "cols", "vals"):
            p.pop(key, None)
        dplan.close()
        dplan = None
        torch.cuda.empty_cache()
        also = run_also(handle, device, peak, c4_pattern, args)

    if rank == 0:
        line = {
            "metric": "SDDMM GFLOP/s (2*nnz*K)", "value": value, "unit": "GFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": p["workload"], "M": M, "N": N, "nnz": nnz, "K": K,
                       "l2": "inputs larger than L2 (no flush)" if 4 * K * (M + N) > 200e6 else "inputs fit L2",
                       "parallelism": f"nnz-balanced row blocks x{world}", "kernel": kernel_name,
                       "panel_rows": info.panel_rows, "work_items": info.n_work_items,
                       "plan_ms": info.plan_ms, "h_broadcast_ms": h_bcast_ms,
                       "rank_ms_per_step": [round(x, 4) for x in rank_ms], "rebalance": rebalance,
                       "dense_cells": info.n_dense_cells, "dense_cell_nnz": info.n_dense_nnz,
                       "hub_columns": info.n_hub_cols},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "parity": parity, "h_broadcast": bcast,
            # counted by the library: kernels launched by sddmm_execute / sddmm_upload_rows on this rank from the
            # first warm-up step to the end of the end-to-end steps (timed steps: one SDDMM kernel each, two when
            # the plan split S into dense cells and a remainder)
            "gpu_launches": launches_main,
            "gpu_launches_timed_steps": args.steps * (2 if (info.n_dense_cells > 0 and args.kernel == "auto") else 1),
            "clocks": clocks.summary(),
        }
        if also is not None:
            line["also"] = also
        print(json.dumps(line), flush=True)
    if parity_failed:
        sys.stderr.write(f"bench.py: GPU result disagrees with the CPU oracle: {parity}\n")
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        raise SystemExit(3)
    if plan is not None:
        handle.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
