#!/usr/bin/env python
"""Bench of the merge-path CSR SpMM hot path: SpMM GFLOP/s = 2*nnz*dim / t.

    python bench.py [--gpus N --steps K --warmup W]            this library (one rank per GPU)
    python bench.py --impl reference ...                       host-CPU arm (see below)
    python bench.py --impl reference-gpu ...                   the reference's CUDA kernels on the GPU
    python bench.py --impl baselines ...                       every reported GPU baseline on one GPU

Workload (seeded, synthetic; stands in for the reference's public graph suite): an R-MAT graph
with 2^21 nodes per GPU and average degree 32 (~67M non-zeros per GPU), GCN-normalised fp32
values, B with `dim` = 64 fp32 columns uniform in [-1,1).  With N GPUs the graph has 2^21*N nodes,
A is cut into N row slabs of equal weighted item count, B is replicated, each rank multiplies its slab
(weak scaling, no collective on the data path).  One step = one SpMM of the whole matrix.  The line also
carries "check" (sampled rows of the C that the timed steps wrote, against fp64), a roofline with bounds
that can read <= 1 (compulsory HBM bytes, measured DRAM traffic, L2 -> SM gather rate from a probe kernel),
"e2e" through the host-buffer call (at one GPU also "e2e.scaled_call": the same product with the two GCN factor vectors
in place of a value per non-zero, as the reference program uploads it), and "c5_strong": the fixed 2^24-node, degree-64 graph at dim 32 cut over
the same N GPUs (strong scaling).

The reference has no CPU SpMM (its hot path is CUDA); the host arm that `--impl reference` times is
the oracle's OpenMP CSR loop on all host cores (kind "port").  The reference's own kernels,
compiled unmodified into oracle/_ref/, are timed on the GPU by `--impl reference-gpu`, and the
default run embeds that number as "reference_gpu" so both baselines sit beside the result.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu", "baselines"])
    ap.add_argument("--scale", type=int, default=21, help="log2 of nodes per GPU")
    ap.add_argument("--avg-degree", type=int, default=32)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--cost", type=int, default=0, help="merge items per chunk (0 = the default of this build)")
    ap.add_argument("--tpw", type=int, default=1, help="threads_per_warp, accepted as the reference's CLI does")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f16"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--chunks-per-unit", type=int, default=0)
    ap.add_argument("--unroll", type=int, default=0)
    ap.add_argument("--no-bulk", action="store_true")
    ap.add_argument("--block", type=int, default=0, help="threads per tile block (0 = automatic)")
    ap.add_argument("--fused", type=int, default=-1, help="cross-tile fix-up inside the tile kernel: 1, 0, -1 = automatic")
    ap.add_argument("--e2e-steps", type=int, default=3, help="timed host-buffer calls (at least 1)")
    ap.add_argument("--skip-baselines", action="store_true", help="leave out cpu_baseline and reference_gpu (tuning runs)")
    ap.add_argument("--balance", default="items", choices=["nnz", "items"], help="row slabs of equal non-zeros or equal rows+non-zeros")
    ap.add_argument("--row-weight", type=int, default=4, help="cost of a row in non-zeros for --balance items")
    ap.add_argument("--strong", action="store_true", help="keep the graph fixed as N grows (strong scaling) instead of 2^scale nodes per GPU")
    ap.add_argument("--gather-c", action="store_true", help="also time the NCCL replication of C (one broadcast per slab, N > 1)")
    ap.add_argument("--no-c5", action="store_true", help="leave out the strong-scaling object on the 2^24-node graph (tuning runs)")
    ap.add_argument("--c5-scale", type=int, default=24)
    ap.add_argument("--c5-degree", type=int, default=64)
    ap.add_argument("--c5-dim", type=int, default=32)
    ap.add_argument("--c5-steps", type=int, default=20)
    ap.add_argument("--c5-sweep", type=int, nargs="*", default=[16, 64, 128], help="other widths timed on the same slabs (the configuration's dim sweep)")
    ap.add_argument("--walk", type=int, default=-1, help="1: a warp walks a unit (mps_plan_set_walk), 0: a lane group per unit, -1: automatic")
    ap.add_argument("--slab", default="", help="R/N: on one GPU, the workload of rank R of an N-GPU run (graph of 2^scale * N nodes, slab R of N) - for profiling")
    ap.add_argument("--no-probe", action="store_true", help="leave out the gather-rate probe (roofline.l2_peak_gbs)")
    return ap.parse_args()


DEFAULT_COST = 16


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 50 ms while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw"

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for i, nm in enumerate(names):
                if len(r) > 2 + i and r[2 + i].lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(local)
    return rank, world, local


def barrier(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    import torch
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_ranks(x: float, world: int):
    import torch
    if world == 1:
        return [round(x, 4)]
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    out = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [round(float(o.item()), 4) for o in out]


def sum_over_ranks(x: float, world: int) -> float:
    import torch
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def check_product(rp, col, val, B, C_out, half, seed=0, n_random=4096, n_long=32):
    """Looks at what was timed: >= 4096 random rows and the longest rows of C_out against an fp64 product formed with
    torch's own gather / index_add (none of this library's kernels).  max_scaled_err = max |d| / (1e-6 + tol * scale),
    scale = sum_k |a_ik b_kj| (fp16: at least |ref|), tol = 1e-5 fp32 / 1e-2 fp16; ok means <= 1."""
    import torch
    dev = C_out.device
    n = rp.numel() - 1
    tol = 1e-2 if half else 1e-5
    lens = (rp[1:] - rp[:-1]).long()
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    rows = torch.unique(torch.cat([torch.randperm(max(n, 1), generator=g)[:n_random].to(dev), torch.topk(lens, min(n_long, n)).indices,
                                   torch.tensor([0, n - 1], device=dev)]))
    l = lens[rows]
    total = int(l.sum().item())
    seg = torch.repeat_interleave(torch.arange(rows.numel(), device=dev), l)
    start = torch.cumsum(l, 0) - l
    idx = rp[rows].long()[seg] + (torch.arange(total, device=dev) - start[seg])
    dim = B.shape[1]
    ref = torch.zeros((rows.numel(), dim), dtype=torch.float64, device=dev)
    scale = torch.zeros_like(ref)
    step = max(1, (1 << 24) // dim)
    for a in range(0, total, step):
        k = idx[a:a + step]
        b = B[col[k].long()].double()
        v = val[k].double()[:, None] if val is not None else 1.0
        ref.index_add_(0, seg[a:a + step], v * b)
        scale.index_add_(0, seg[a:a + step], (v * b).abs())
    if half:
        scale = torch.maximum(scale, ref.abs())
    got = C_out[rows].double()
    err = (got - ref).abs()
    worst = float((err / (1e-6 + tol * scale)).max().item()) if total else 0.0
    finite = bool(torch.isfinite(got).all().item())
    return {"rows": int(rows.numel()), "nnz": total, "max_scaled_err": round(worst, 4), "tol": tol, "ok": bool(finite and worst <= 1.0),
            "against": "fp64 product of the sampled rows (torch gather + index_add), after the timed region"}


def gather_rates(mps, dev, row_bytes, B=None, col=None):
    """The rates the multiply's gather can be held against (mps_gather_probe): random whole rows of `row_bytes`
    out of a 32 MB table (L2 -> SM) and out of a 4 GiB table (HBM, ~3 % L2 hits), 128-bit loads, GB/s; and, when the
    row width allows, the multiply's own stream - the rows of B that col_idx names, in its order - fetched by a kernel
    that does nothing else (mps_gather_probe_stream)."""
    import torch
    exact = row_bytes in (32, 64, 128, 256, 512)
    row_bytes = min(512, max(32, 1 << (int(row_bytes) - 1).bit_length()))
    out = {}
    if exact and B is not None and col is not None and col.numel() > 0:
        out["stream"] = round(max(mps.gather_probe_stream(B, row_bytes, col) for _ in range(3)), 1)
    for name, size in (("l2", 32 << 20), ("hbm", 4 << 30)):
        table = torch.zeros(size, dtype=torch.uint8, device=dev)
        best = 0.0
        for _ in range(3):
            best = max(best, mps.gather_probe(table, row_bytes, 1 << 25))
        out[name] = round(best, 1)
        del table
    torch.cuda.empty_cache()
    return out, row_bytes


def build_workload(args, world, rank, dev):
    """Whole graph on this rank's GPU (same bits on every rank), then this rank's row slab."""
    import torch
    from mergepath_spmm_b200 import graphs
    mps = entry.load_package()
    scale = total_scale(args, world)
    cut, piece = world, rank
    if args.slab and world == 1:  # one rank's share of a larger run, alone on this GPU
        piece, cut = (int(v) for v in args.slab.split("/"))
        scale = total_scale(args, cut)
    rp, col = graphs.rmat_csr(scale, args.avg_degree, args.seed, device=dev)
    n, nnz = rp.numel() - 1, col.numel()
    half = args.dtype == "f16"
    val = graphs.gcn_values(rp, col, "f16" if half else "f32")
    if cut > 1:
        bounds = mps.slab_bounds(rp.cpu().numpy(), cut, args.balance, args.row_weight)
        r0, r1 = int(bounds[piece]), int(bounds[piece + 1])
        k0, k1 = int(rp[r0].item()), int(rp[r1].item())
        s_rp = (rp[r0:r1 + 1] - k0).contiguous()
        s_col, s_val = col[k0:k1].clone(), val[k0:k1].clone()
        del rp, col, val
    else:
        r0, r1, s_rp, s_col, s_val = 0, n, rp, col, val
    torch.cuda.empty_cache()
    if half:
        B = graphs.dense_normal_f16(n, args.dim, args.seed + 1, device=dev)
    else:
        B = graphs.dense_uniform(n, args.dim, args.seed + 1, device=dev)
    return dict(n=n, nnz=nnz, scale=scale, r0=r0, r1=r1, slab_nnz=int(s_col.numel()), rp=s_rp, col=s_col, val=s_val, B=B, half=half)


def total_scale(args, world):
    if args.strong:
        return args.scale
    lg = int(round(np.log2(world)))
    assert 1 << lg == world, "--gpus must be a power of two"
    return args.scale + lg


def workload_name(args, world):
    if args.slab and world == 1:
        piece, cut = (int(v) for v in args.slab.split("/"))
        return f"rmat{total_scale(args, cut)}_deg{args.avg_degree}_gcn_{args.dtype}_dim{args.dim}_slab{piece}of{cut}"
    return f"rmat{total_scale(args, world)}_deg{args.avg_degree}_gcn_{args.dtype}_dim{args.dim}"


def time_multiplies(plan, w, C_out, steps, world, local=None):
    """`steps` multiplies timed by CUDA events on the launching stream between two barriers; returns this rank's
    milliseconds (whole region) and the clock sampler (None when local is None)."""
    import torch
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    clocks = None
    if local is not None:
        clocks = ClockSampler(local)
        clocks.__enter__()
    ev0.record()
    for _ in range(steps):
        plan.spmm(w["rp"], w["col"], w["val"], w["B"], out=C_out)
    ev1.record()
    barrier(world)
    if clocks is not None:
        clocks.__exit__()
    return ev0.elapsed_time(ev1), clocks


def kernel_pass(plan, w, C_out, steps):
    """A second, separately reported pass with an event pair around every tile-kernel launch (mps_plan_profile): the
    dominant kernel's mean duration.  Kept out of the headline region, whose steps carry no extra events."""
    plan.profile(True)
    for _ in range(min(steps, 256)):
        plan.spmm(w["rp"], w["col"], w["val"], w["B"], out=C_out)
    tile_ms, launches = plan.profile_read()
    plan.profile(False)
    return tile_ms / max(launches, 1), launches


def roofline_of(mps, args, w, n_slab, nnz_slab, dt, tile_ms_avg, ms_step, rates, probe_row_bytes, workload):
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    s_el = 2 if w["half"] else 4
    dim = w["B"].shape[1]
    alg = mps.algorithmic_bytes(n_slab, nnz_slab, dim, dt, True)
    # every operand once: row_ptr, col_idx, val, B (all its rows), C - what HBM has to move at least
    compulsory = 4 * (n_slab + 1) + nnz_slab * (4 + s_el) + (w["n"] + n_slab) * dim * s_el
    gathered = nnz_slab * dim * s_el
    t = tile_ms_avg * 1e-3
    r = {"bound": "hbm", "achieved": round(alg / t / 1e9, 1), "peak": peak, "unit": "GB/s", "frac": round(alg / t / 1e9 / peak, 4),
         "traffic": None, "kernel": "spmm_tile_kernel", "kernel_ms": round(tile_ms_avg, 4), "algorithmic_bytes": alg,
         "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback 6650 GB/s",
         "step_frac": round(alg / (ms_step * 1e-3) / 1e9 / peak, 4),
         "note": "frac charges every gathered row of B to HBM (the contract's byte count) and exceeds 1 when the L2 serves the gather; "
                 "compulsory_frac, dram_frac and l2_frac are fractions of a peak each",
         "compulsory_bytes": compulsory, "compulsory_frac": round(compulsory / t / 1e9 / peak, 4),
         "gathered_bytes": gathered, "gathered_gbs": round(gathered / t / 1e9, 1)}
    fracs = {"hbm_compulsory": r["compulsory_frac"]}
    if rates:
        r["l2_peak_gbs"] = rates["l2"]
        r["hbm_gather_gbs"] = rates["hbm"]
        r["probe"] = f"mps_gather_probe, random rows of {probe_row_bytes} B, 128-bit loads: 32 MB table (L2) and 4 GiB table (HBM)"
        r["l2_frac"] = round(gathered / t / 1e9 / rates["l2"], 4)
        fracs["l2_gather"] = r["l2_frac"]
        if "stream" in rates:
            # the same rows in the same order, fetched by a kernel that only fetches: what this index stream allows
            r["stream_gather_gbs"] = rates["stream"]
            r["stream_frac"] = round(gathered / t / 1e9 / rates["stream"], 4)
            fracs["own_stream_gather"] = r["stream_frac"]
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        try:
            tj = json.load(open(tpath)).get(workload)
            if tj:
                # DRAM bytes of one launch from the committed ncu capture of this workload
                r["traffic"] = tj["dram_bytes_per_launch"]
                r["traffic_source"] = tj.get("source")
                r["dram_frac"] = round(tj["dram_bytes_per_launch"] / t / 1e9 / peak, 4)
                r["l2_hit_rate"] = tj.get("l2_hit_rate")
                fracs["hbm_measured_traffic"] = r["dram_frac"]
        except Exception:
            pass
    r["nearest_bound"] = max(fracs, key=fracs.get)
    r["nearest_bound_frac"] = fracs[r["nearest_bound"]]
    return r


def e2e_through_host_call(mps, args, w, world, rank, dev, cost, dt, n_slab, nnz_slab):
    """The same metric through the host-buffer C-ABI call: pinned host inputs in, C in pinned host memory out, every
    copy inside the timed region.  One rank: mps_spmm_host.  Several ranks: every rank uploads 1/N of B's rows, an
    NCCL all-gather completes B over NVLink, and mps_spmm_host_resident_b uploads the rank's slab of A meanwhile."""
    import torch
    from mergepath_spmm_b200 import graphs, multi
    elem = 2 if w["half"] else 4
    d = {k: w[k] for k in ("rp", "col", "val")}   # this rank's slab of A on the device (for the check afterwards)
    slabs = "the slabs of the device-timed run"
    if world > 1:
        # a rank's call is bound by its own PCIe link: 4 + s bytes up per non-zero, dim * s bytes down per row.  The slabs
        # that balance the kernel (nnz + 4 rows) give one rank up to 47x the rows of another; for this call A is cut
        # on link bytes instead (same matrix, same product)
        row_w = max(1, args.dim * elem // (4 + elem))
        rp, col = graphs.rmat_csr(w["scale"], args.avg_degree, args.seed, device=dev)
        val = graphs.gcn_values(rp, col, "f16" if w["half"] else "f32")
        bounds = mps.slab_bounds(rp.cpu().numpy(), world, "items", row_w)
        r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
        k0, k1 = int(rp[r0].item()), int(rp[r1].item())
        d = {"rp": (rp[r0:r1 + 1] - k0).contiguous(), "col": col[k0:k1].clone(), "val": val[k0:k1].clone()}
        del rp, col, val
        torch.cuda.empty_cache()
        n_slab, nnz_slab = r1 - r0, int(d["col"].numel())
        slabs = f"balanced on link bytes: nnz + {row_w} rows"
    h = {k: (d[k].cpu().pin_memory() if d[k] is not None else None) for k in ("rp", "col", "val")}
    h_C = torch.empty((n_slab, args.dim), dtype=w["B"].dtype).pin_memory()
    if world == 1:
        h["B"] = w["B"].cpu().pin_memory()

        def call():
            mps.capi.check(mps.capi.lib().mps_spmm_host(n_slab, w["n"], nnz_slab, args.dim, dt, cost, args.tpw, C.c_void_p(h["rp"].data_ptr()),
                                                        C.c_void_p(h["col"].data_ptr()), C.c_void_p(h["val"].data_ptr()),
                                                        C.c_void_p(h["B"].data_ptr()), C.c_void_p(h_C.data_ptr())))
    else:
        b0, b1, blk = multi.b_block(w["n"], rank, world)
        h["B"] = w["B"][b0:b1].cpu().pin_memory()
        d_B = torch.empty((world * blk, args.dim), dtype=w["B"].dtype, device=dev)

        def call():
            whole = multi.replicate_b(h["B"], w["n"], out=d_B)
            mps.spmm_host_resident_b(h["rp"], h["col"], h["val"], whole, h_C, cost=cost, threads_per_warp=args.tpw)
    steps = max(1, args.e2e_steps)
    call()  # warm: workspace allocation, communicator
    barrier(world)
    t0 = time.perf_counter()
    for _ in range(steps):
        call()
    t_mine = time.perf_counter() - t0   # this rank's calls alone (each is blocking); the job's time includes the barrier
    barrier(world)
    e2e_s = max_over_ranks((time.perf_counter() - t0) / steps, world)
    e2e_rank_s = t_mine / steps
    h2d = sum(h[k].numel() * h[k].element_size() for k in h if h[k] is not None)
    d2h = h_C.numel() * h_C.element_size()
    chk = check_product(d["rp"], d["col"], d["val"], w["B"], h_C.to(dev), w["half"], seed=100 + rank)   # the C that came back to the host
    ok = bool(min_over_ranks(1.0 if chk["ok"] else 0.0, world) > 0.5)
    scaled = None
    if world == 1 and not w["half"] and not args.slab:
        # the same GCN product with the two factor vectors (degree^-1/2) instead of a value per non-zero - the shape of
        # the reference program, which uploads one number per node and forms the values in the kernel
        deg = (d["rp"][1:] - d["rp"][:-1]).to(torch.float64)
        h_s = (1.0 / torch.sqrt(deg)).to(torch.float32).cpu().pin_memory()
        h_C2 = torch.full_like(h_C, float("nan")).pin_memory()

        def call_scaled():
            mps.spmm_host_scaled(h["rp"], h["col"], h_s, h_s, h["B"], out=h_C2, cost=cost, threads_per_warp=args.tpw)
        call_scaled()
        t1 = time.perf_counter()
        for _ in range(steps):
            call_scaled()
        s_s = (time.perf_counter() - t1) / steps
        chk2 = check_product(d["rp"], d["col"], d["val"], w["B"], h_C2.to(dev), False, seed=200)
        scaled = {"call": "mps_spmm_host_scaled (row and column factors instead of a value per non-zero)", "ms_per_step": round(s_s * 1e3, 3),
                  "value": round(2.0 * w["nnz"] * args.dim / s_s / 1e9, 2), "unit": "GFLOP/s",
                  "h2d_bytes_per_step": int(sum(h[k].numel() * h[k].element_size() for k in ("rp", "col", "B")) + 2 * h_s.numel() * 4),
                  "d2h_bytes_per_step": int(d2h), "check_ok": bool(chk2["ok"])}
        del h_C2
    mps.capi.lib().mps_host_workspace_release()
    host = {k: (h[k].numpy() if h[k] is not None else None) for k in h} if world == 1 else None
    flop_nnz = nnz_slab if (args.slab and world == 1) else w["nnz"]
    return {"value": round(2.0 * flop_nnz * args.dim / e2e_s / 1e9, 2), "unit": "GFLOP/s", "h2d_bytes_per_step": int(sum_over_ranks(h2d, world)),
            "d2h_bytes_per_step": int(sum_over_ranks(d2h, world)), "ms_per_step": round(e2e_s * 1e3, 3), "steps": steps,
            "b_replication": "each rank uploads 1/N of B, NCCL all-gather over NVLink" if world > 1 else "one upload", "slabs": slabs,
            "per_rank_ms": all_ranks(e2e_rank_s * 1e3, world),
            "check": {"ok": ok, "max_scaled_err": max_over_ranks(chk["max_scaled_err"], world), "rows": int(sum_over_ranks(chk["rows"], world))},
            **({"scaled_call": scaled} if scaled else {})}, host


def c5_strong(mps, args, world, rank, dev):
    """Configuration 5 in the driver's record: the 2^24-node, degree-64 R-MAT graph (fixed size), cut into `world`
    item-balanced row slabs, B replicated, dim 32; each rank multiplies its slab.  Strong scaling: 8-GPU / 1-GPU time."""
    import torch
    from mergepath_spmm_b200 import graphs
    torch.cuda.empty_cache()
    t0 = time.perf_counter()
    dim = args.c5_dim
    built, why = True, ""
    try:
        rp, col = graphs.rmat_csr(args.c5_scale, args.c5_degree, args.seed, device=dev)
        n, nnz = rp.numel() - 1, col.numel()
        val = graphs.gcn_values(rp, col, "f32")
        if world > 1:
            bounds = mps.slab_bounds(rp.cpu().numpy(), world, "items", args.row_weight)
            r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
            k0, k1 = int(rp[r0].item()), int(rp[r1].item())
            s_rp, s_col, s_val = (rp[r0:r1 + 1] - k0).contiguous(), col[k0:k1].clone(), val[k0:k1].clone()
            del rp, col, val
        else:
            r0, r1, s_rp, s_col, s_val = 0, n, rp, col, val
        torch.cuda.empty_cache()
        B = graphs.dense_uniform(n, dim, args.seed + 1, device=dev)
        torch.cuda.synchronize()
        n_slab, nnz_slab = r1 - r0, s_col.numel()
        plan = mps.Plan(n_slab, nnz_slab, dim, mps.F32, args.cost or DEFAULT_COST, args.tpw, device=dev)
        plan.partition(s_rp)
    except (torch.cuda.OutOfMemoryError, mps.MpsError) as e:
        built, why = False, str(e)[:160]
    # every rank takes the same branch: one that could not build must not leave the others waiting in a collective
    if min_over_ranks(1.0 if built else 0.0, world) < 0.5:
        torch.cuda.empty_cache()
        return {"unavailable": "a rank could not build the workload" + (": " + why if why else "")}
    build_s = time.perf_counter() - t0
    C_out = torch.empty((n_slab, dim), dtype=torch.float32, device=dev)
    w = dict(rp=s_rp, col=s_col, val=s_val, B=B, half=False, n=n, nnz=nnz)
    for _ in range(3):
        plan.spmm(s_rp, s_col, s_val, B, out=C_out)
    plan.sync_check()
    C_out.fill_(float("nan"))
    ms_mine, _ = time_multiplies(plan, w, C_out, args.c5_steps, world)
    plan.sync_check()
    ms_step = max_over_ranks(ms_mine, world) / args.c5_steps
    check = check_product(s_rp, s_col, s_val, B, C_out, False, seed=rank)
    info = plan.info()
    plan.close()
    # the other widths of the configuration's sweep on the same slabs (fewer steps; each with its own look at C)
    sweep = {}
    for d2 in [d for d in args.c5_sweep if d != dim]:
        del B, C_out
        torch.cuda.empty_cache()
        B = graphs.dense_uniform(n, d2, args.seed + 1, device=dev)
        C_out = torch.full((n_slab, d2), float("nan"), dtype=torch.float32, device=dev)
        p2 = mps.Plan(n_slab, nnz_slab, d2, mps.F32, args.cost or DEFAULT_COST, args.tpw, device=dev)
        p2.partition(s_rp)
        w2 = dict(rp=s_rp, col=s_col, val=s_val, B=B)
        for _ in range(3):
            p2.spmm(s_rp, s_col, s_val, B, out=C_out)
        steps2 = max(3, args.c5_steps // 2)
        ms2, _ = time_multiplies(p2, w2, C_out, steps2, world)
        p2.sync_check()
        p2.close()
        ms2 = max_over_ranks(ms2, world) / steps2
        c2 = check_product(s_rp, s_col, s_val, B, C_out, False, seed=rank + d2, n_random=1024, n_long=8)
        sweep[str(d2)] = {"ms_per_step": round(ms2, 4), "value": round(2.0 * nnz * d2 / (ms2 * 1e-3) / 1e9, 2),
                          "check_ok": bool(min_over_ranks(1.0 if c2["ok"] else 0.0, world) > 0.5)}
    alg = mps.algorithmic_bytes(n_slab, nnz_slab, dim, mps.F32, True)
    out = {"workload": f"rmat{args.c5_scale}_deg{args.c5_degree}_gcn_f32_dim{dim}", "scaling": "strong", "dim_sweep": sweep, "nodes": n, "nnz": nnz, "dim": dim,
           "n_gpus": world, "steps": args.c5_steps, "ms_per_step": round(ms_step, 4), "value": round(2.0 * nnz * dim / (ms_step * 1e-3) / 1e9, 2),
           "unit": "GFLOP/s", "per_rank_ms": all_ranks(ms_mine / args.c5_steps, world), "per_rank_nnz": [int(v) for v in all_ranks(float(nnz_slab), world)],
           "per_rank_rows": [int(v) for v in all_ranks(float(n_slab), world)], "tiles": info["n_tiles"], "long_rows": info["long_rows"],
           "hbm_algorithmic_gbs": round(sum_over_ranks(alg, world) / (ms_step * 1e-3) / 1e9, 1),
           "check": {"ok": bool(min_over_ranks(1.0 if check["ok"] else 0.0, world) > 0.5), "rows": int(sum_over_ranks(check["rows"], world)),
                     "max_scaled_err": max_over_ranks(check["max_scaled_err"], world), "tol": check["tol"], "against": check["against"]},
           "graph_build_s": round(max_over_ranks(build_s, world), 1)}
    del plan, C_out, B, s_rp, s_col, s_val, w
    torch.cuda.empty_cache()
    return out


def min_over_ranks(x: float, world: int) -> float:
    return -max_over_ranks(-x, world)


def run_ours(args):
    import torch
    rank, world, local = dist_setup(args)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run"
    dev = torch.device("cuda", local)
    mps = entry.load_package()
    cost = args.cost or DEFAULT_COST
    w = build_workload(args, world, rank, dev)
    n_slab, nnz_slab = w["r1"] - w["r0"], w["col"].numel()
    dt = mps.F16 if w["half"] else mps.F32
    plan = mps.Plan(n_slab, nnz_slab, args.dim, dt, cost, args.tpw, device=dev)
    if args.chunks_per_unit or args.unroll or args.no_bulk or args.block or args.fused >= 0:
        plan.tune(args.chunks_per_unit, args.unroll, not args.no_bulk, args.block, args.fused)
    if args.walk >= 0:
        plan.set_walk(args.walk)
    partition_first_ms = partition_ms = 0.0
    for i in range(2):  # the first call also loads the library's kernels onto the device
        t0 = time.perf_counter()
        plan.partition(w["rp"])
        torch.cuda.synchronize()
        partition_ms = (time.perf_counter() - t0) * 1e3
        if i == 0:
            partition_first_ms = partition_ms
    info = plan.info()
    C_out = torch.empty((n_slab, args.dim), dtype=w["B"].dtype, device=dev)

    for _ in range(max(args.warmup, 3)):
        plan.spmm(w["rp"], w["col"], w["val"], w["B"], out=C_out)
    plan.sync_check()
    C_out.fill_(float("nan"))  # what the check below reads was written by the timed steps

    # ---- timed region: K steps, CUDA events on the launching stream, barrier + sync on both sides ----
    ms_mine, clocks = time_multiplies(plan, w, C_out, args.steps, world, local)
    ms_total = max_over_ranks(ms_mine, world)
    per_rank_ms = all_ranks(ms_mine / args.steps, world)
    plan.sync_check()
    ms_step = ms_total / args.steps
    flops = 2.0 * (nnz_slab if (args.slab and world == 1) else w["nnz"]) * args.dim
    value = flops / (ms_step * 1e-3) / 1e9

    # ---- a look at what was timed (outside the timed region), every rank ----
    chk = check_product(w["rp"], w["col"], w["val"], w["B"], C_out, w["half"], seed=rank)
    check = {"ok": bool(min_over_ranks(1.0 if chk["ok"] else 0.0, world) > 0.5), "rows": int(sum_over_ranks(chk["rows"], world)),
             "max_scaled_err": max_over_ranks(chk["max_scaled_err"], world), "tol": chk["tol"], "against": chk["against"], "ranks": world}

    # ---- roofline of the dominant kernel (the tile kernel), this rank's slab ----
    tile_ms_avg, tile_launches = kernel_pass(plan, w, C_out, args.steps)
    rates, probe_row = (None, 0) if args.no_probe else gather_rates(mps, dev, args.dim * (2 if w["half"] else 4), w["B"], w["col"])
    roofline = roofline_of(mps, args, w, n_slab, nnz_slab, dt, tile_ms_avg, ms_step, rates, probe_row, workload_name(args, world))
    roofline["kernel_pass_launches"] = tile_launches

    # ---- end to end through the host-buffer C-ABI call ----
    e2e, host = e2e_through_host_call(mps, args, w, world, rank, dev, cost, dt, n_slab, nnz_slab)

    out = {
        "metric": "SpMM GFLOP/s (2*nnz*dim/t)", "value": round(value, 2), "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong" if args.strong else "weak",
        "vs_baseline": None, "dtype": "f16 storage / f32 accumulate" if w["half"] else "f32", "data": "synthetic",
        "config": {"workload": workload_name(args, world), "nodes": w["n"], "nnz": w["nnz"], "dim": args.dim, "cost": cost,
                   "threads_per_warp": info["threads_per_warp"], "values": "gcn", "parallelism": f"row-slabs x{world} ({args.balance}-balanced, row weight {args.row_weight}), B replicated", "per_rank_ms": per_rank_ms, "per_rank_rows": [int(v) for v in all_ranks(float(n_slab), world)], "per_rank_nnz": [int(v) for v in all_ranks(float(nnz_slab), world)],
                   "l2": "inputs larger than L2 (B and A each > 126 MB)", "unit_items": info["unit_items"], "units_per_tile": info["units_per_tile"], "groups_per_unit": info["groups_per_unit"],
                   "items_per_chunk": info["items_per_chunk"], "unroll": info["unroll"], "block_threads": info["block_threads"], "tiles": info["n_tiles"],
                   "long_rows": info["long_rows"]},
        "check": check, "roofline": roofline, "e2e": e2e, "gpu_launches": args.steps * info["kernels_per_call"],
        "clocks": clocks.summary(), "partition_ms": round(partition_ms, 3), "partition_first_call_ms": round(partition_first_ms, 3),
        "hbm_algorithmic_gbs": round(sum_over_ranks(roofline["algorithmic_bytes"], world) / (ms_step * 1e-3) / 1e9, 1),
    }

    if args.gather_c and world > 1:
        out["gather_c"] = time_gather_c(w, args, world, rank, dev, C_out)

    if rank == 0 and world == 1 and not args.skip_baselines:
        out["cpu_baseline"] = cpu_baseline(host, args.dim, w["nnz"], w["half"])
        try:
            out["reference_gpu"] = reference_gpu_both(w, args, dev)
        except Exception as e:  # the checker being absent must not lose the bench line
            out["reference_gpu"] = {"unavailable": str(e)[:200]}
    plan.close()
    del plan, C_out, host
    w.clear()
    torch.cuda.empty_cache()

    if not args.no_c5:
        out["c5_strong"] = c5_strong(mps, args, world, rank, dev)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def time_gather_c(w, args, world, rank, dev, c_slab):
    """Optional replicated C: one NCCL broadcast per slab straight into place (slab heights differ up to 47x, so
    nothing is padded); GB/s on the bytes of C that each rank receives."""
    import torch
    from mergepath_spmm_b200 import multi
    import torch.distributed as dist
    rows = torch.tensor([w["r1"] - w["r0"]], device=dev)
    allrows = [torch.zeros_like(rows) for _ in range(world)]
    dist.all_gather(allrows, rows)
    bounds = np.concatenate([[0], np.cumsum([int(r.item()) for r in allrows])])
    full = torch.empty((int(bounds[-1]), args.dim), dtype=c_slab.dtype, device=dev)
    for _ in range(2):
        multi.gather_c(c_slab, bounds, out=full)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    e0.record()
    for _ in range(5):
        multi.gather_c(c_slab, bounds, out=full)
    e1.record()
    barrier(world)
    ms = max_over_ranks(e0.elapsed_time(e1) / 5, world)
    received = (full.numel() - c_slab.numel()) * full.element_size()
    return {"ms": round(ms, 3), "bytes_received_per_rank": int(received), "gbs_per_rank": round(received / (ms * 1e-3) / 1e9, 1),
            "how": "one broadcast per slab, no padding"}


def cpu_baseline(host, dim, nnz, half):
    """The oracle's OpenMP fp32 CSR loop on all host cores, whole workload, 1 warm-up + best of 3."""
    orc = entry.load_oracle()
    val = host["val"].astype(np.float32) if half else host["val"]
    B = host["B"].astype(np.float32) if half else host["B"]
    out = np.empty((len(host["rp"]) - 1, dim), np.float32)
    threads = len(os.sched_getaffinity(0))  # explicit: launchers such as torchrun export OMP_NUM_THREADS=1
    _, cores = orc.spmm_f32_omp(host["rp"], host["col"], val, B, out=out, threads=threads)
    best = float("inf")
    t_all = time.perf_counter()
    for _ in range(3):
        t0 = time.perf_counter()
        orc.spmm_f32_omp(host["rp"], host["col"], val, B, out=out, threads=threads)
        best = min(best, time.perf_counter() - t0)
        if time.perf_counter() - t_all > 25:
            break
    return {"value": round(2.0 * nnz * dim / best / 1e9, 3), "unit": "GFLOP/s", "cores": int(cores), "kind": "port",
            "sample": "the whole workload (one full SpMM), best of up to 3 after 1 warm-up", "ms_per_step": round(best * 1e3, 2)}


def _ref_lib(half):
    path = os.path.join(ROOT, "oracle", "_ref", "libref_mergepath_f16.so" if half else "libref_mergepath_f32.so")
    if not os.path.exists(path):
        raise RuntimeError("oracle/_ref is not built")
    lib = C.CDLL(path)
    lib.refh_launch.argtypes = [C.c_void_p] * 5 + [C.POINTER(C.c_void_p)] + [C.c_int] * 4
    return lib


def reference_gpu(w, args, dev, steps=5, cost=8):
    """The reference's own kernel (spmm_merge_path / _64, unmodified) on the same graph and B, driven as
    its main() drives it: schedule for `cost`, degrees == 1 (unit values - the only setting in which it
    is a correct SpMM), 256-thread blocks, sync after each launch.  Kernel time by CUDA events."""
    import torch
    mps = entry.load_package()
    lib = _ref_lib(w["half"])
    n, nnz, dim = w["rp"].numel() - 1, w["col"].numel(), args.dim
    if (n + 1) * dim >= 2 ** 31:
        raise RuntimeError("reference index arithmetic is 32-bit: (N+1)*dim overflows")
    p, _ = mps.chunk_count(n, nnz, cost)
    six = mps.schedule_device(w["rp"], p)
    padded = torch.zeros((6, p + 64), dtype=torch.int32, device=dev)
    padded[:, :p] = six
    del six
    deg = torch.ones(n + 1, dtype=torch.int32, device=dev)
    B1 = torch.zeros((n + 1, dim), dtype=w["B"].dtype, device=dev)
    B1[:n] = w["B"]
    Cr = torch.zeros((n + 1, dim), dtype=w["B"].dtype, device=dev)
    ptrs = (C.c_void_p * 6)(*[padded[i].data_ptr() for i in range(6)])
    tpw = max(1, min(args.tpw, 32 // dim)) if dim <= 32 else 1
    times = []
    for i in range(steps + 1):
        Cr.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        rc = lib.refh_launch(Cr.data_ptr(), B1.data_ptr(), w["rp"].data_ptr(), w["col"].data_ptr(), deg.data_ptr(), ptrs, n, dim, p, tpw)
        e1.record()
        torch.cuda.synchronize()
        if rc != 0:
            raise RuntimeError(f"reference launch returned CUDA error {rc}")
        if i:
            times.append(e0.elapsed_time(e1))
    ms = float(np.median(times))
    return {"kernel": "spmm_merge_path_64" if dim > 32 else "spmm_merge_path", "value": round(2.0 * nnz * dim / (ms * 1e-3) / 1e9, 2),
            "unit": "GFLOP/s", "ms_per_step": round(ms, 4), "cost": cost, "threads_per_warp": tpw, "values": "unit (degrees == 1)",
            "steps": steps}


def reference_gpu_both(w, args, dev):
    """The reference's kernel at cost 8 (the value configuration 1 names) and at the best of its four costs on this
    graph (cost 32), both in the line."""
    r8 = reference_gpu(w, args, dev, steps=5, cost=8)
    r32 = reference_gpu(w, args, dev, steps=5, cost=32)
    best = r32 if r32["ms_per_step"] <= r8["ms_per_step"] else r8
    out = dict(r8)
    out["best"] = {"cost": best["cost"], "ms_per_step": best["ms_per_step"], "value": best["value"], "unit": "GFLOP/s",
                   "of_costs": [4, 8, 16, 32], "note": "cost 4 and 16 are slower than 32 on this graph (bench.py --impl baselines)"}
    return out


def _lib(name):
    path = os.path.join(ROOT, "oracle", "_ref", name)
    if not os.path.exists(path):
        raise RuntimeError(f"oracle/_ref/{name} is not built")
    return C.CDLL(path)


def _timed(fn, steps, before=None):
    import torch
    times = []
    for i in range(steps + 1):
        if before:
            before()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        rc = fn()
        e1.record()
        torch.cuda.synchronize()
        if rc != 0:
            raise RuntimeError(f"launch returned {rc}")
        if i:
            times.append(e0.elapsed_time(e1))
    return float(np.median(times))


def run_baselines(args):
    """Reported baselines on one GPU, same graph and B as the default workload, unit values (the
    reference programs have none): the reference merge-path kernels, its row_wise and nz_splitting
    programs' kernels (unmodified, from oracle/_ref), cuSPARSE row- and column-major set up as the
    reference's cusparse_spmm_{row,col}.cu do, and this library with unit values.  One JSON line."""
    import torch
    rank, world, local = dist_setup(args)
    if rank != 0:
        return
    dev = torch.device("cuda", local)
    mps = entry.load_package()
    w = build_workload(args, 1, 0, dev)
    n, nnz, dim = w["n"], w["nnz"], args.dim
    vp, ci = C.c_void_p, C.c_int
    flops = 2.0 * nnz * dim
    res = {}

    def rec(name, ms, **kw):
        res[name] = {"ms": round(ms, 4), "gflops": round(flops / ms / 1e6, 1), **kw}

    steps = max(min(args.steps, 10), 1)
    # this library, unit values and GCN values
    plan = mps.Plan(n, nnz, dim, mps.F16 if w["half"] else mps.F32, args.cost or DEFAULT_COST, args.tpw, device=dev)
    plan.partition(w["rp"])
    Cm = torch.empty((n, dim), dtype=w["B"].dtype, device=dev)
    for name, val in (("this_library_unit_values", None), ("this_library_gcn_values", w["val"])):
        for _ in range(3):
            plan.spmm(w["rp"], w["col"], val, w["B"], out=Cm)
        rec(name, _timed(lambda: (plan.spmm(w["rp"], w["col"], val, w["B"], out=Cm), 0)[1], steps), cost=args.cost or DEFAULT_COST)
    plan.close()
    del Cm
    # reference merge-path kernel at each cost of the configured sweep
    # (the fp16 reference kernels add split rows with fp16 atomics and take seconds per launch at small costs on a
    # power-law graph - 4.3 s at cost 8, dim 128 - so only the two largest costs are run for fp16)
    for cost in ((16, 32) if w["half"] else (4, 8, 16, 32)):
        try:
            r = reference_gpu(w, args, dev, steps=1 if w["half"] else 3, cost=cost)
            rec(f"reference_mergepath_cost{cost}", r["ms_per_step"], kernel=r["kernel"])
        except Exception as e:
            res[f"reference_mergepath_cost{cost}"] = {"unavailable": str(e)[:160]}
    if w["half"]:  # the other baselines are fp32 programs; the fp16 table has this library and MergePathSpMM_fp16 only
        print(json.dumps({"impl": "baselines", "metric": "SpMM GFLOP/s (2*nnz*dim/t)", "unit": "GFLOP/s", "n_gpus": 1,
                          "config": {"workload": workload_name(args, 1), "nodes": n, "nnz": nnz, "dim": dim, "values": "unit unless named",
                                     "reference": "MergePathSpMM_fp16 kernels (fp16 accumulation)"}, "results": res}), flush=True)
        return
    deg = torch.ones(n + 1, dtype=torch.int32, device=dev)
    B1 = torch.zeros((n + 1, dim), dtype=torch.float32, device=dev)
    B1[:n] = w["B"]
    Cr = torch.zeros((n + 1, dim), dtype=torch.float32, device=dev)
    if (n + 1) * dim < 2 ** 31:
        # row_wise: dim <= 32 only
        try:
            if dim > 32:
                raise RuntimeError("row_wise computes one column per lane: dim <= 32 only (src/row_wise.cu:222)")
            lib = _lib("libref_row_wise.so")
            lib.baseh_row_wise.argtypes = [vp] * 5 + [ci] * 3
            nw = max(n // 8, 1)
            rec("reference_row_wise", _timed(lambda: lib.baseh_row_wise(Cr.data_ptr(), B1.data_ptr(), w["rp"].data_ptr(), w["col"].data_ptr(),
                                                                        deg.data_ptr(), n, dim, nw), 3), num_warps=nw)
        except Exception as e:
            res["reference_row_wise"] = {"unavailable": str(e)[:160]}
        # nz_splitting (GNNAdvisor-opt)
        try:
            if dim <= 32:
                # src/nz_splitting.cu:412-424: the dim <= 32 kernel guards with warpId < num_parts although each warp
                # takes 32/dim parts, so the last block reads part_pointers/part2Node up to 8*(32/dim) entries past
                # their end and then row data at whatever index it found there.  With the arrays sized as the
                # reference's main() sizes them this raised an illegal memory access on a B200; not run again.
                raise RuntimeError("reference kernel reads past its part arrays for dim <= 32 (guard at nz_splitting.cu:412); "
                                   "faulted with an illegal memory access on B200, not run again")
            lib = _lib("libref_nz_splitting.so")
            part = min(dim, 32)
            i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
            lib.baseh_nz_count.argtypes = [i32p, ci, ci]
            lib.baseh_nz_build.argtypes = [i32p, ci, ci, ci, i32p, i32p]
            lib.baseh_nz_launch.argtypes = [vp] * 7 + [ci] * 4
            h_rp = w["rp"].cpu().numpy()
            num_parts = lib.baseh_nz_count(h_rp, n, part)
            pp, p2n = np.zeros(num_parts + 1, np.int32), np.zeros(num_parts, np.int32)
            lib.baseh_nz_build(h_rp, n, part, num_parts, pp, p2n)
            d_pp, d_p2n = torch.from_numpy(pp).to(dev), torch.from_numpy(p2n).to(dev)
            rec("reference_nz_splitting", _timed(lambda: lib.baseh_nz_launch(Cr.data_ptr(), B1.data_ptr(), w["rp"].data_ptr(), w["col"].data_ptr(),
                                                                             deg.data_ptr(), d_pp.data_ptr(), d_p2n.data_ptr(), n, dim, num_parts, part),
                                                 3, before=Cr.zero_), part_size=part, num_parts=int(num_parts))
            del d_pp, d_p2n
        except Exception as e:
            res["reference_nz_splitting"] = {"unavailable": str(e)[:160]}
    del B1, Cr, deg
    # cuSPARSE, row- and column-major dense operands, values = 1
    try:
        lib = _lib("libcusparse_baseline.so")
        lib.cush_spmm.argtypes = [ci] * 4 + [vp] * 5 + [ci, ci, ci, C.POINTER(C.c_float)]
        ones = torch.ones(nnz, dtype=torch.float32, device=dev)
        Cc = torch.empty((n, dim), dtype=torch.float32, device=dev)
        Bt = w["B"].t().contiguous()
        runs = [("cusparse_row_major", 0, 0, w["B"], "CUSPARSE_SPMM_ALG_DEFAULT"), ("cusparse_col_major", 1, 0, Bt, "CUSPARSE_SPMM_ALG_DEFAULT"),
                ("cusparse_row_major_csr_alg2_preprocessed", 0, 2, w["B"], "CUSPARSE_SPMM_CSR_ALG2 + preprocess"),
                ("cusparse_row_major_csr_alg3_preprocessed", 0, 3, w["B"], "CUSPARSE_SPMM_CSR_ALG3 + preprocess"),
                ("cusparse_col_major_csr_alg1_preprocessed", 1, 1, Bt, "CUSPARSE_SPMM_CSR_ALG1 + preprocess")]
        for name, colmajor, alg, Bop, label in runs:
            ms = C.c_float()
            rc = lib.cush_spmm(n, n, nnz, dim, w["rp"].data_ptr(), w["col"].data_ptr(), ones.data_ptr(), Bop.data_ptr(), Cc.data_ptr(),
                               colmajor, alg, steps, C.byref(ms))
            if rc != 0:
                res[name] = {"unavailable": f"cusparse step {rc} failed"}
            else:
                rec(name, ms.value, alg=label)
    except Exception as e:
        res["cusparse"] = {"unavailable": str(e)[:160]}
    print(json.dumps({"impl": "baselines", "metric": "SpMM GFLOP/s (2*nnz*dim/t)", "unit": "GFLOP/s", "n_gpus": 1,
                      "config": {"workload": workload_name(args, 1), "nodes": n, "nnz": nnz, "dim": dim, "values": "unit unless named"},
                      "results": res}), flush=True)


def run_reference_gpu(args):
    import torch
    rank, world, local = dist_setup(args)
    if rank != 0:
        return
    dev = torch.device("cuda", local)
    w = build_workload(args, 1, 0, dev)
    try:
        r = reference_gpu(w, args, dev, steps=max(args.steps, 1), cost=args.cost or 8)
    except Exception as e:
        print(json.dumps({"impl": "reference-gpu", "unavailable": str(e)[:200]}), flush=True)
        return
    print(json.dumps({"impl": "reference-gpu", "metric": "SpMM GFLOP/s (2*nnz*dim/t)", **r, "n_gpus": 1,
                      "config": {"workload": workload_name(args, 1), "nodes": w["n"], "nnz": w["nnz"], "dim": args.dim}}), flush=True)


def run_reference_cpu(args):
    """Host arm: the OpenMP CSR loop of the oracle on all host cores, one step = one SpMM over the WHOLE workload of
    this library's arm at the same N (R-MAT scale 21 + log2 N: 0.1 s per step at scale 21, under a second at 24)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    entry.load_package()
    from mergepath_spmm_b200 import graphs
    orc = entry.load_oracle()
    import torch
    scale = total_scale(args, max(world, args.gpus))
    half = args.dtype == "f16"
    try:
        if torch.cuda.is_available():  # the graph generator is faster on the device; the multiply below is host-only
            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
            rp, col = graphs.rmat_csr(scale, args.avg_degree, args.seed, device=dev)
            val = graphs.gcn_values(rp, col).cpu().numpy()
            rp, col = rp.cpu().numpy(), col.cpu().numpy()
            torch.cuda.empty_cache()
        else:
            rp, col = graphs.rmat_csr(scale, args.avg_degree, args.seed)
            val = graphs.gcn_values(rp, col)
        n, nnz = len(rp) - 1, len(col)
        B = graphs.dense_uniform(n, args.dim, args.seed + 1)
        out = np.empty((n, args.dim), np.float32)
    except MemoryError as e:
        print(json.dumps({"impl": "reference", "unavailable": f"host memory: the scale-{scale} workload does not fit ({e})"}), flush=True)
        return
    cores = 1
    threads = len(os.sched_getaffinity(0))  # explicit: launchers such as torchrun export OMP_NUM_THREADS=1
    for _ in range(max(args.warmup, 1)):
        _, cores = orc.spmm_f32_omp(rp, col, val, B, out=out, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.spmm_f32_omp(rp, col, val, B, out=out, threads=threads)
    s = (time.perf_counter() - t0) / args.steps
    v = round(2.0 * nnz * args.dim / s / 1e9, 3)
    sample = f"the whole workload: R-MAT scale {scale}, avg degree {args.avg_degree}, {nnz} nnz, dim {args.dim}, one full SpMM per step"
    print(json.dumps({
        "impl": "reference", "metric": "SpMM GFLOP/s (2*nnz*dim/t)", "value": v, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": round(s * 1e3, 3), "higher_is_better": True,
        "scaling": "strong" if args.strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args, max(world, args.gpus)), "nodes": n, "nnz": nnz, "dim": args.dim, "cost": args.cost or DEFAULT_COST,
                   "threads_per_warp": args.tpw, "values": "gcn", "l2": "inputs larger than L2 (B and A each > 126 MB)",
                   "parallelism": f"{cores} host threads, rows split at equal non-zero counts",
                   "fp16_note": "fp16 storage is multiplied as fp32 on the host" if half else None},
        "cpu_baseline": {"value": v, "unit": "GFLOP/s", "cores": int(cores), "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU SpMM; this is the oracle's OpenMP CSR loop. Its CUDA kernels: --impl reference-gpu",
    }), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_cpu(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    elif args.impl == "baselines":
        run_baselines(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
