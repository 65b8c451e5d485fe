#!/usr/bin/env python
"""Benchmark of the fused 3S path: ms/call and edge-GFLOP/s (4*d*H*nnz useful flops per call).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg4] [--impl ours|reference]

One "step" is one fused forward call over the whole graph (all row windows, all heads).
``--impl ours``      times this package: ``value`` with Q/K/V resident in HBM (C-ABI launch, CUDA
                     events), ``e2e`` through the reference-shaped ``F3S`` op from pinned host
                     buffers (H2D of Q/K/V and D2H of the output inside the timed region).
``--impl reference`` times the reference's CPU sparse-attention path (gather-SDDMM, segment
                     softmax, scatter-SpMM; a plain-torch port of its PyTorch-Geometric route, see
                     oracle/attention_oracle.py) on a bounded sample of the same workload with all
                     host threads.
With N > 1 (launched by torchrun, one rank per GPU) the row windows are sharded by TC-block count,
K and V are all-gathered over NCCL (one collective, overlapped with the kernel's first launch) inside
the timed region, and the time is the max over ranks.  The line also carries sub-records for the two
workloads that really run from HBM (``other_workloads``: the molecule batch and the 1 M-node 8-head
graph at N = 1; the latter, with its exchange inside the step, at N > 1).
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {"cfg1": 1, "cfg2": 2, "cfg3": 3, "cfg4": 4, "cfg5": 5}
SCALE_DIVISOR = 8.0  # 1/sqrt(64)
L2_FLUSH_BYTES = 256 << 20


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg4", choices=sorted(WORKLOADS))
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload (profiling / debugging)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-cuda", action="store_true", help="skip timing the rebuilt reference kernel")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true", help="skip the cfg3 / cfg5 sub-records")
    ap.add_argument("--no-parity-check", action="store_true", help="skip the sampled comparison with the oracle")
    ap.add_argument("--reference-seconds", type=float, default=600.0,
                    help="--impl reference: wall-clock budget for warm-up + timed steps; the full workload is "
                         "timed when it fits, a bounded sample of it otherwise")
    ap.add_argument("--backward", action="store_true",
                    help="also time the training path (forward with log-sum-exp output, backward), 1 GPU only")
    ap.add_argument("--e2e-chunks", type=int, default=4, help="row chunks of the host-to-host pipeline")
    ap.add_argument("--head-chunks", type=int, default=4,
                    help="row chunks of the head-sharded pipeline (kernel of one chunk overlaps the exchange of others)")
    ap.add_argument("--score-stage", action="store_true",
                    help="1 GPU, one head: also time the score stage alone on tcgen05.mma / tensor memory "
                         "(f3s_sddmm_umma) against the fused kernel with and without its score dump")
    ap.add_argument("--collective", default="auto", choices=["auto", "nccl", "multimem"],
                    help="multi-GPU row sharding: the K/V all-gather through NCCL or through NVSwitch multicast "
                         "(torch symmetric memory); auto = multicast when it can be set up, else NCCL")
    ap.add_argument("--two-phase", action="store_true",
                    help="multi-GPU row sharding: overlap the all-gather with a first kernel launch on the rank's own "
                         "columns (default: collective, then one launch)")
    ap.add_argument("--kv-capped", action="store_true",
                    help="head pipeline: run the K+V all-to-all on the capped communicator too (default: uncapped)")
    ap.add_argument("--reserve-sms", type=int, default=32,
                    help="multi-GPU, overlapped schemes (head pipeline, --two-phase): SMs the fused kernel leaves to the "
                         "collectives' kernels while both run")
    ap.add_argument("--nccl-max-ctas", type=int, default=32,
                    help="multi-GPU, overlapped schemes: cap on NCCL's CTAs per collective in the process group those "
                         "schemes use (0: NCCL's default); the plain all-gather of row sharding is never capped")
    ap.add_argument("--reorder", default="none", choices=["none", "degree"],
                    help="relabel the nodes before building TC blocks (fused3s_b200.reorder); the default "
                         "benchmark keeps the generator's order")
    ap.add_argument("--sharding", default="auto", choices=["auto", "rows", "heads", "heads-resident"],
                    help="multi-GPU scheme: auto = heads over GPUs when the head count divides evenly, else row "
                         "windows + K/V all-gather; heads / heads-resident = with / without the all-to-all of "
                         "row-sharded inputs inside the step")
    ap.add_argument("--min-warmup-seconds", type=float, default=1.0,
                    help="single-GPU runs keep warming up until this much time has passed (clock sampling)")
    return ap.parse_args()


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json: stream copy)"
    return 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50", "-i",
                 str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t0 = time.perf_counter()  # nvidia-smi needs a moment to attach: wait for its first sample
            while not self.rows and time.perf_counter() - t0 < 5.0:
                time.sleep(0.05)
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        hi = [s for s in sm if s >= 0.5 * max(sm)]  # samples taken under load
        return {"sm_mhz": float(np.median(hi)), "sm_max_mhz": float(max(mx)), "samples": len(sm),
                "reasons": sorted(reasons)}


def algorithmic_bytes(n, heads, d, sum_u, n_tcb, n_rw, bw=16):
    """Bytes one call must move: Q once (fp16), output once (fp32), one K and one V row (fp16) per
    (row window, distinct column) pair and head, plus the TC-block metadata read once."""
    feat = heads * d * (2 * n + 4 * n + 2 * 2 * sum_u)
    meta = 4 * (n_rw + 1) + 4 * n_rw + 4 * bw * n_tcb + (16 * bw // 8) * n_tcb
    return feat + meta


def compulsory_bytes(n, heads, d, n_tcb, n_rw, bw=16):
    """What DRAM has to move even with a perfect cache: Q, K, V and the output once, the metadata once."""
    return heads * d * (2 * n + 2 * 2 * n + 4 * n) + 4 * (n_rw + 1) + 4 * n_rw + 4 * bw * n_tcb + (16 * bw // 8) * n_tcb


def distinct_window_columns(rowptr_t, colidx_t, n):
    """sum over windows of distinct columns, on the device (exact integer work)."""
    import torch

    deg = (rowptr_t[1:] - rowptr_t[:-1]).long()
    rows = torch.repeat_interleave(torch.arange(n, device=rowptr_t.device), deg)
    key = (rows // 16) * (1 << 32) + colidx_t.long()
    return int(torch.unique(key).numel())


def sharding_note(args, heads):
    """One string for both arms (their ``config`` entries have to be identical)."""
    if args.gpus == 1:
        return "single GPU"
    mode = args.sharding
    if mode == "auto" or heads % args.gpus != 0:
        mode = "heads" if (args.sharding == "auto" and heads > 1 and heads % args.gpus == 0) else "rows"
    if mode == "rows":
        return ("row windows by TC-block count; K and V all-gathered by one collective inside every step "
                f"(--collective {args.collective}: auto = NVSwitch multicast through torch symmetric memory from 8 ranks "
                "on when available, else NCCL)" +
                (", overlapped with a first kernel launch on the rank's own columns" if args.two_phase else
                 ", then one kernel launch"))
    if mode == "heads-resident":
        return f"{heads // args.gpus} of {heads} heads per GPU, Q/K/V already head-sharded: no communication"
    return (f"{heads // args.gpus} of {heads} heads per GPU; row-sharded Q/K/V -> all-to-all (K+V in one, Q by row "
            "pieces) -> kernel per piece -> all-to-all of the output pieces, all inside every step and overlapped")


def workload_config(args, g):
    return {"workload": f"{g.name} (N={g.num_nodes}, nnz={g.nnz}, heads={g.heads}, d={g.dim}, fp16 Q/K/V ~N(0,1), "
                        f"score divisor {SCALE_DIVISOR})" + (f" scaled x{args.scale}" if args.scale != 1.0 else ""),
            "l2": f"L2 flushed: a {L2_FLUSH_BYTES >> 20} MiB buffer is written between timed steps"
                  + ("; the inputs are larger than L2 as well (more than 126 MB of TC-block metadata)"
                     if g.nnz >= 30_000_000 else ""),
            "sharding": sharding_note(args, g.heads),
            "node_order": "generator order" if args.reorder == "none" else "descending degree (reorder.py)"}


def _cpu_rows_for_budget(g, edges_budget):
    ptr = g.rowptr.astype(np.int64)
    r1 = int(np.searchsorted(ptr, max(1, edges_budget), side="right"))
    r1 = max(16, min(r1, g.num_nodes))
    return r1, int(ptr[r1])


def cpu_baseline(g, q, k, v, seconds=15.0, threads=None):
    """The CPU sparse-attention path (oracle/attention_oracle.py::edge_attention, the plain-torch port of the
    reference's PyTorch-Geometric route) on the first rows of the workload: a sample sized, from a short
    probe, to take about ``seconds`` of CPU time; the whole workload if that fits."""
    import torch

    from oracle import attention_oracle as ao

    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    r_probe, e_probe = _cpu_rows_for_budget(g, 1_000_000 // max(1, g.heads))
    ao.edge_attention(g.rowptr, g.colidx, q, k, v, SCALE_DIVISOR, row_begin=0, row_end=min(r_probe, 256))  # warm-up
    t0 = time.perf_counter()
    ao.edge_attention(g.rowptr, g.colidx, q, k, v, SCALE_DIVISOR, row_begin=0, row_end=r_probe)
    rate = e_probe / max(1e-6, time.perf_counter() - t0)  # edges per second
    r1, edges = _cpu_rows_for_budget(g, int(rate * seconds))
    t0 = time.perf_counter()
    ao.edge_attention(g.rowptr, g.colidx, q, k, v, SCALE_DIVISOR, row_begin=0, row_end=r1)
    dt = time.perf_counter() - t0
    gflops = 4.0 * g.dim * g.heads * edges / dt / 1e9
    return {"value": gflops, "unit": "GFLOP/s", "cores": threads, "kind": "port",
            "sample": f"rows [0,{r1}) of {g.name}: {edges} of {g.nnz} edges x {g.heads} head(s), {dt:.2f} s, "
                      f"torch {threads} threads, fp32 gather-SDDMM/segment-softmax/scatter-SpMM",
            "ms_full_call_extrapolated": dt * 1e3 * g.nnz / max(1, edges)}


def run_reference_arm(args, g, q, k, v):
    """--impl reference: the CPU path, W warm-up and K timed steps.  A step is the WHOLE workload when
    W + K of them fit the time budget (``ms_per_step`` is then a measured full call); otherwise a step is
    the largest prefix of rows that fits, ``ms_per_step`` is the measured time of that sample and the
    full-call figure is given separately as an extrapolation."""
    import torch

    from oracle import attention_oracle as ao

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    r_probe, e_probe = _cpu_rows_for_budget(g, 2_000_000 // max(1, g.heads))
    ao.edge_attention(g.rowptr, g.colidx, q, k, v, SCALE_DIVISOR, row_begin=0, row_end=min(r_probe, 256))
    t0 = time.perf_counter()
    ao.edge_attention(g.rowptr, g.colidx, q, k, v, SCALE_DIVISOR, row_begin=0, row_end=r_probe)
    rate = e_probe / max(1e-6, time.perf_counter() - t0)
    calls = args.steps + args.warmup
    per_step_budget = args.reference_seconds / max(1, calls)
    full = g.nnz / rate <= per_step_budget
    r1, edges = (g.num_nodes, g.nnz) if full else _cpu_rows_for_budget(g, int(rate * per_step_budget))
    for _ in range(args.warmup):
        ao.edge_attention(g.rowptr, g.colidx, q, k, v, SCALE_DIVISOR, row_begin=0, row_end=r1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ao.edge_attention(g.rowptr, g.colidx, q, k, v, SCALE_DIVISOR, row_begin=0, row_end=r1)
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    gflops = 4.0 * g.dim * g.heads * edges / dt / 1e9
    sample = (f"the whole workload per step ({edges} edges x {g.heads} head(s))" if full else
              f"rows [0,{r1}) of {g.name} per step: {edges} of {g.nnz} edges x {g.heads} head(s); ms_per_step is the "
              "measured time of that sample")
    line = {
        "impl": "reference", "metric": "edge_gflops", "value": gflops, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": workload_config(args, g),
        "cpu_baseline": {"value": gflops, "unit": "GFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gflops, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "full_workload_per_step": bool(full),
    }
    if not full:
        line["ms_full_call_extrapolated"] = dt * 1e3 * g.nnz / max(1, edges)
    return line

class Bench:
    """Timing context of one process: device, world, L2 flush buffer."""

    def __init__(self, dev, world):
        import torch

        self.dev, self.world = dev, world
        self.flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)

    def timed(self, fn, steps):
        """ms of ``steps`` calls of fn, each behind an L2 flush, CUDA events on the current stream;
        barrier + synchronize on both sides; with several ranks the max over ranks, step by step."""
        import torch
        import torch.distributed as dist

        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        for a, b in ev:
            self.flush.fill_(1)
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
        ms = np.array([a.elapsed_time(b) for a, b in ev])
        local = ms.copy()
        if self.world > 1:
            t = torch.tensor(ms, device=self.dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.cpu().numpy()
        return ms, local


def parity_check(g, q_h, k_h, v_h, out, row_begin, row_end, seed, blocks=4):
    """Sampled comparison of device output rows [row_begin, row_end) with the CPU oracle: ``blocks`` blocks
    of 64 rows (and, with several heads, one sampled head each).  Returns (ok, worst max-abs, worst mean-rel)."""
    from oracle import attention_oracle as ao

    rng = np.random.default_rng(seed)
    ok, worst_abs, worst_rel = True, 0.0, 0.0
    span = max(1, row_end - row_begin - 64)
    for _ in range(blocks):
        r0 = row_begin + int(rng.integers(0, span)) // 16 * 16
        r1 = min(row_end, r0 + 64)
        if g.heads > 1:
            h = int(rng.integers(0, g.heads))
            want = ao.edge_attention(g.rowptr, g.colidx, q_h[:, h], k_h[:, h], v_h[:, h], SCALE_DIVISOR,
                                     row_begin=r0, row_end=r1)
            got = out[r0 - row_begin:r1 - row_begin, h].float().cpu()
        else:
            want = ao.edge_attention(g.rowptr, g.colidx, q_h, k_h, v_h, SCALE_DIVISOR, row_begin=r0, row_end=r1)
            got = out[r0 - row_begin:r1 - row_begin].float().cpu()
        m = ao.compare(got, want)
        worst_abs, worst_rel = max(worst_abs, m["max_abs"]), max(worst_rel, m["mean_rel"])
        ok = ok and m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL
    return ok, worst_abs, worst_rel


def roofline_record(b_alg, b_min, kern_ms, peak, peak_src, traffic, kv_bytes, l2_gather_gbs, gather_bytes, kernel,
                    hbm_gather_gbs=None):
    """The HBM fraction the contract asks for, plus the two measured ceilings that actually bind a gather
    kernel: this package's probe kernel gathers 128-byte rows at random ids from a table of the size of
    K + V (L2-resident case) and from a 2 GiB table (HBM case).  ``frac_mixed`` compares the kernel time with
    gathered bytes / gather ceiling + streamed bytes (Q, output, metadata) / copy rate."""
    achieved = b_alg / (kern_ms * 1e-3) / 1e9
    rec = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
           "traffic": traffic, "peak_source": peak_src, "algorithmic_bytes_per_call": b_alg, "kernel": kernel,
           "frac_dram_compulsory": b_min / (kern_ms * 1e-3) / 1e9 / peak,
           "compulsory_bytes_per_call": b_min, "gathered_bytes_per_call": gather_bytes}
    l2_resident = kv_bytes < 100e6
    rec["bound_effective"] = "l2" if l2_resident else "hbm"
    if l2_gather_gbs is not None:
        rec["l2_peak_gbs"] = l2_gather_gbs
        rec["frac_l2"] = gather_bytes / (kern_ms * 1e-3) / 1e9 / l2_gather_gbs
    if hbm_gather_gbs is not None:
        rec["hbm_gather_peak_gbs"] = hbm_gather_gbs
    ceiling = l2_gather_gbs if l2_resident else hbm_gather_gbs
    if ceiling:
        t_roof = gather_bytes / ceiling / 1e6 + (b_alg - gather_bytes) / peak / 1e6  # ms
        rec["t_roof_mixed_ms"] = t_roof
        rec["frac_mixed"] = t_roof / kern_ms
    rec["gather_peak_source"] = ("f3s_probe_gather_rows (this package): 128-byte rows at seeded random ids, loads only, "
                                 "best of 5, same process; table = size of K + V of one head (L2) / 2 GiB (HBM)")
    rec["note"] = ("frac = algorithmic bytes / kernel time / measured HBM copy rate. K + V of a head fit the L2 cache, so "
                   "the gathers never reach DRAM and frac may exceed 1; frac_l2 and frac_mixed (against the measured L2 "
                   "gather rate) say how far the kernel is from the roof that binds" if l2_resident else
                   "frac = algorithmic bytes / kernel time / measured HBM copy rate. K + V of a head exceed the L2 cache; "
                   "random 128-byte rows come from HBM slower than a copy streams, hence frac_mixed against the measured "
                   "HBM gather rate (above 1 when part of the gathers still hit L2)")
    return rec


def time_rebuilt_reference(tcb, n, q, k, v, graph=None):
    """The reference's own best kernel (f3s_1tb1rw_scheduled_permuteV_scaleQK, rebuilt for sm_100a by
    oracle/build_ref.py) on the same device arrays; its own event time, median of 10 after 3 warm-ups,
    as scripts/baseline_comp/baseline_comp_kernel_only.py:230-238 measures it.  It has one head per call:
    with several heads it is called once per head on contiguous copies and the medians are added."""
    import torch

    try:
        from oracle import build_ref

        ref = build_ref.load("F3S_ref")
    except Exception as e:
        return {"unavailable": f"{e}"}
    if ref is None:
        return {"unavailable": "oracle/_ref not built"}
    d = q.shape[-1]
    heads = q.shape[1] if q.dim() == 3 else 1

    def pad(x):  # its kernels read all 16 rows of the last window
        buf = torch.zeros(((n + 15) // 16 * 16, d), dtype=x.dtype, device=x.device)
        buf[:n] = x
        return buf[:n]

    total = 0.0
    for h in range(heads):
        qd, kd, vd = (pad(x if heads == 1 else x[:, h]) for x in (q, k, v))
        ts = []
        for i in range(13 if heads == 1 else 6):
            t, _, _ = ref.f3s_1tb1rw_scheduled_permuteV_scaleQK(tcb["rowWindowOffset"], tcb["sortedRowWindows"],
                                                                tcb["sparseAToXidx"], tcb["tcbBitMap"], n, qd, kd, vd,
                                                                SCALE_DIVISOR, 8)
            if i >= 3:
                ts.append(float(t))
        total += float(np.median(ts))
    res = {"ms_median": total, "op": "f3s_1tb1rw_scheduled_permuteV_scaleQK, nWarpPerBlock=8"
                                     + ("" if heads == 1 else f", {heads} calls (one per head)")}
    if graph is not None:
        # the reference's own preprocessing on the same CSR (it prints to stdout: silenced here so that
        # this process still prints exactly one JSON line)
        rp_t, ci_t = graph
        nrw = (n + 15) // 16
        dev = q.device
        ms = []
        for _ in range(2):
            bp = torch.zeros(nrw, dtype=torch.int32, device=dev)
            e2c = torch.zeros(ci_t.numel(), dtype=torch.int32, device=dev)
            e2r = torch.zeros(ci_t.numel(), dtype=torch.int32, device=dev)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            with _silence_stdout():
                ref.preprocess_gpu(ci_t, rp_t, n, 16, 16, bp, e2c, e2r)
                torch.cuda.synchronize()
            ms.append((time.perf_counter() - t0) * 1e3)
        res["preprocess_ms"] = float(min(ms))
    return res


class _silence_stdout:
    """Temporarily point file descriptor 1 at /dev/null (C-level printf of the reference extension)."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        self.null = os.open(os.devnull, os.O_WRONLY)
        os.dup2(self.null, 1)

    def __exit__(self, *exc):
        os.dup2(self.saved, 1)
        os.close(self.null)
        os.close(self.saved)

def kernel_name(d, n_tcb, n_rw, direct):
    if direct:
        return "f3s::fwd_kernel_coop (one-launch mode for small problems)"
    if d == 64 and 2 * n_tcb >= 16 * n_rw:
        return "f3s::fwd_kernel_split<12> (d = 64, separate K and V rings)"
    return "f3s::fwd_kernel (combined K+V stages: short row windows / head dims other than 64)"


def traffic_for(workload):
    tj = ROOT / "profiles" / "traffic.json"
    if tj.exists():
        try:
            return json.loads(tj.read_text()).get(workload)
        except Exception:
            return None
    return None


def single_gpu_subrecord(bench, cfg, args, steps):
    """One other workload on one GPU, device-resident inputs: ms per call, edge-GFLOP/s, roofline, the
    rebuilt reference kernel on the same arrays, sampled parity.  Shorter than the headline record: no
    end-to-end leg, no CPU leg."""
    import torch

    from fused3s_b200 import cabi, graphs

    dev = bench.dev
    g = graphs.make_config(cfg, device=dev, scale=args.scale)
    q_h, k_h, v_h = graphs.make_features(g)
    n, heads, d = g.num_nodes, g.heads, g.dim
    rp_t, ci_t = torch.from_numpy(g.rowptr).to(dev), torch.from_numpy(g.colidx).to(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pre = []
    for _ in range(2):
        tcb = None
        e0.record()
        tcb = cabi.preprocess(ci_t, rp_t, n, 16)
        e1.record()
        torch.cuda.synchronize()
        pre.append(e0.elapsed_time(e1))
    qd, kd, vd = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    plan = cabi.ForwardPlan(tcb, n, qd, kd, vd, SCALE_DIVISOR)
    for _ in range(5):
        plan.launch()
    torch.cuda.synchronize()
    l0 = cabi.lib().f3s_kernel_launch_count()
    ms, _ = bench.timed(plan.launch, steps)
    launches = int(cabi.lib().f3s_kernel_launch_count() - l0)
    plan.status()
    n_rw = (n + 15) // 16
    sum_u = distinct_window_columns(rp_t, ci_t, n)
    b_alg = algorithmic_bytes(n, heads, d, sum_u, tcb["nTCB"], n_rw)
    b_min = compulsory_bytes(n, heads, d, tcb["nTCB"], n_rw)
    peak, peak_src = measured_peaks()
    kv_bytes = 2 * n * d * 2  # K + V of ONE head: heads are processed one after the other by every warp
    l2 = cabi.gather_rate_gbs(kv_bytes, dev) if kv_bytes < 100e6 else None
    hbm_g = cabi.gather_rate_gbs(2 << 30, dev, n_ids=1 << 23)
    t = float(ms.mean())
    rec = {"workload": workload_config(args, g)["workload"], "ms_per_step": t, "ms_per_step_median": float(np.median(ms)),
           "edge_gflops": 4.0 * d * heads * g.nnz / (t * 1e-3) / 1e9, "steps": steps, "gpu_launches": launches,
           "preprocess_ms": float(min(pre)), "tcb": {"nTCB": tcb["nTCB"], "sumU": sum_u, "nRW": n_rw},
           "roofline": roofline_record(b_alg, b_min, t, peak, peak_src, traffic_for(f"cfg{cfg}"), kv_bytes, l2,
                                       heads * d * 4 * sum_u, kernel_name(d, tcb["nTCB"], n_rw, plan.ws_bytes <= 256),
                                       hbm_g)}
    if not args.no_ref_cuda:
        rec["reference_cuda_rebuilt"] = time_rebuilt_reference(tcb, n, qd, kd, vd)
    if not args.no_parity_check:
        ok, ma, mr = parity_check(g, q_h, k_h, v_h, plan.out, 0, n, seed=cfg)
        rec["parity_check"] = "ok" if ok else "FAILED"
        rec["parity_worst"] = {"max_abs": ma, "mean_rel": mr}
    del plan, qd, kd, vd, tcb
    torch.cuda.empty_cache()
    return rec


def multi_gpu_heads_subrecord(bench, cfg, args, steps, rank, world, group=None):
    """The multi-head workload with the heads divided over the ranks and row-sharded producers and
    consumers: the step holds the all-to-all of Q/K/V, the kernel and the all-to-all of the output."""
    import torch
    import torch.distributed as dist

    from fused3s_b200 import cabi, graphs, sharding

    dev = bench.dev
    g = graphs.make_config(cfg, device=dev, scale=args.scale)
    q_h, k_h, v_h = graphs.make_features(g)
    n, heads, d = g.num_nodes, g.heads, g.dim
    if heads % world != 0:
        return {"unavailable": f"{heads} heads do not divide over {world} GPUs"}
    attn = sharding.HeadShardedPipeline(g.rowptr, g.colidx, n, heads, rank, world, dev, chunks=args.head_chunks,
                                        reserve_sms=args.reserve_sms, group=group,
                                        kv_group=group if args.kv_capped else None)
    rb, re_ = attn.row_begin, attn.row_end
    q_x = attn.to_exchange_layout(q_h[rb:re_].to(dev))
    kv_x = attn.kv_to_exchange_layout(k_h[rb:re_].to(dev), v_h[rb:re_].to(dev))
    step = lambda: attn.forward(q_x, kv_x, SCALE_DIVISOR)
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    ms, local = bench.timed(step, steps)
    t = float(ms.mean())
    out = attn.from_exchange_layout(step())
    torch.cuda.synchronize()
    rec = {"workload": workload_config(args, g)["workload"], "ms_per_step": t, "ms_per_step_median": float(np.median(ms)),
           "edge_gflops": 4.0 * d * heads * g.nnz / (t * 1e-3) / 1e9, "steps": steps,
           "scheme": attn.describe(), "exchange_inside_step": True}
    if not args.no_parity_check:
        ok, ma, mr = parity_check(g, q_h, k_h, v_h, out, attn.row_begin, attn.row_end, seed=100 + rank)
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        rec["parity_check"] = "ok" if int(flag) == 1 else "FAILED"
    kern, _ = bench.timed(lambda: attn.kernel_only(SCALE_DIVISOR), steps)
    rec["kernel_only_ms"] = float(kern.mean())
    del attn
    torch.cuda.empty_cache()
    return rec


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = WORKLOADS[args.workload]

    import torch

    from fused3s_b200 import graphs

    # torchrun pins every rank to one host thread; the seeded feature tensors are drawn on the host
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // max(1, world)))

    if args.impl == "reference":
        if rank != 0:
            return
        g = graphs.make_config(cfg, device="cuda" if torch.cuda.is_available() else None, scale=args.scale)
        q, k, v = graphs.make_features(g)
        print(json.dumps(run_reference_arm(args, g, q, k, v)), flush=True)
        return

    assert torch.cuda.is_available(), "bench.py --impl ours needs a CUDA device (there is no CPU fallback)"
    import torch.distributed as dist

    from fused3s_b200 import cabi, import_f3s, sharding

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    overlap_group = None
    if world > 1:
        # a rank that never joins ends the others' collectives with an error after this long (torch's NCCL
        # watchdog), instead of leaving them waiting for ever
        import datetime

        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
        if args.nccl_max_ctas > 0:  # collectives that share the GPU with the fused kernel: a narrow communicator
            opts = dist.ProcessGroupNCCL.Options()
            opts.config.max_ctas = args.nccl_max_ctas
            overlap_group = dist.new_group(ranks=list(range(world)), backend="nccl", pg_options=opts,
                                           timeout=datetime.timedelta(seconds=300))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    bench = Bench(dev, world)
    lib = cabi.lib()

    t_gen = time.perf_counter()
    g = graphs.make_config(cfg, device=dev, scale=args.scale)
    q_h, k_h, v_h = graphs.make_features(g)
    if args.reorder == "degree":
        from fused3s_b200 import reorder

        perm = reorder.degree_order(g.rowptr)
        g.rowptr, g.colidx = reorder.permute_csr(g.rowptr, g.colidx, perm, device=dev)
        q_h, k_h, v_h = (reorder.apply(perm, x) for x in (q_h, k_h, v_h))
    t_gen = time.perf_counter() - t_gen
    n, heads, d = g.num_nodes, g.heads, g.dim

    mode = args.sharding
    if mode == "auto":
        mode = "heads" if (heads > 1 and world > 1 and heads % world == 0) else "rows"
    if world == 1 or heads % world != 0:
        mode = "rows"
    cabi.preprocess(torch.zeros(0, dtype=torch.int32, device=dev), torch.zeros(17, dtype=torch.int32, device=dev),
                    16, 16)  # loads the library and warms the allocator
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    F3S = None if args.no_e2e else import_f3s()
    pipe = pipe2 = None
    ref_args = None
    balance = None

    if mode == "rows":
        rp_full = torch.from_numpy(g.rowptr).to(dev)
        ci_full = torch.from_numpy(g.colidx).to(dev)
        weights = None
        if world > 1:  # TC blocks per window of the whole graph: what the partition is balanced by
            weights = cabi.window_tcb_counts(ci_full, rp_full, n).cpu().numpy()
        shard = sharding.make_shard(g.rowptr, g.colidx, n, rank, world, window_weight=weights, local_last=world > 1 and args.two_phase)
        del rp_full, ci_full
        rp_t = torch.from_numpy(shard.rowptr).to(dev)
        ci_t = torch.from_numpy(shard.padded_colidx()).to(dev)
        pre_ms = []
        for _ in range(2):  # the first call also pays for the allocator's first device allocations of these sizes
            tcb = None
            e0.record()
            tcb = cabi.preprocess(ci_t, rp_t, shard.num_rows, 16, num_cols=shard.padded_cols)
            e1.record()
            torch.cuda.synchronize()
            pre_ms.append(e0.elapsed_time(e1))
        preprocess_ms = min(pre_ms)
        n_tcb_local = tcb["nTCB"]
        sum_u_local = distinct_window_columns(rp_t, ci_t, shard.num_rows)
        totals_are_partial = True
        r0, r1 = shard.row_begin, shard.row_end
        q_pin = q_h[r0:r1].contiguous().pin_memory()
        k_pin = k_h[r0:r1].contiguous().pin_memory()
        v_pin = v_h[r0:r1].contiguous().pin_memory()
        q_loc = q_pin.to(dev)
        attn = sharding.ShardedAttention(shard, dev, 16, tcb=tcb, two_phase=args.two_phase, reserve_sms=args.reserve_sms,
                                         collective=args.collective)
        if world > 1:  # the local K/V rows live in the send block of the all-gather
            k_loc, v_loc = attn.send_buffers(q_loc)
            k_loc[: r1 - r0].copy_(k_pin)
            v_loc[: r1 - r0].copy_(v_pin)
        else:
            k_loc, v_loc = k_pin.to(dev), v_pin.to(dev)

        def step_device():
            if world > 1:
                return attn.forward(q_loc, k_loc, v_loc, SCALE_DIVISOR)
            return attn.forward_local(q_loc, k_loc, v_loc, SCALE_DIVISOR)

        def make_kernel_only():
            if world == 1:
                return None
            kf, vf = attn.gather_kv(k_loc, v_loc)
            return lambda: attn.forward_local(q_loc, kf, vf, SCALE_DIVISOR)

        out_rows = r1 - r0
        out_pin = None if args.no_e2e else torch.empty(
            (out_rows, heads, d) if heads > 1 else (out_rows, d), dtype=torch.float32).pin_memory()

        def step_e2e():
            if world > 1:  # host rows -> send block -> all-gather + two-phase kernel -> host rows
                k_loc[: r1 - r0].copy_(k_pin, non_blocking=True)
                v_loc[: r1 - r0].copy_(v_pin, non_blocking=True)
                q_loc.copy_(q_pin, non_blocking=True)
                out = attn.forward(q_loc, k_loc, v_loc, SCALE_DIVISOR)
            else:
                qd = q_pin.to(dev, non_blocking=True)
                kd = k_pin.to(dev, non_blocking=True)
                vd = v_pin.to(dev, non_blocking=True)
                _, out, _ = F3S.f3s_1tb1rw_scheduled_permuteV_scaleQK(
                    tcb["rowWindowOffset"], tcb["sortedRowWindows"], tcb["sparseAToXidx"], tcb["tcbBitMap"], r1 - r0,
                    qd, kd, vd, SCALE_DIVISOR, 8)
            out_pin.copy_(out, non_blocking=True)

        # single GPU: the same host-to-host call through the pipelined public API (chunked row windows,
        # copies overlapped with the kernel on three streams)
        if world == 1 and not args.no_e2e:
            from fused3s_b200.host_pipeline import HostPipelinedAttention

            pipe = HostPipelinedAttention(g.rowptr, g.colidx, n, heads, d, dev, chunks=args.e2e_chunks, kv_halves=False)
            pipe2 = HostPipelinedAttention(g.rowptr, g.colidx, n, heads, d, dev, chunks=args.e2e_chunks, kv_halves=True)
            if not pipe2.kv_halves:  # the two-launch forward does not apply to this workload
                pipe2 = None

        def step_e2e_pipelined():
            pipe.forward(q_pin, k_pin, v_pin, out_pin, SCALE_DIVISOR)

        def step_e2e_pipelined_halves():
            pipe2.forward(q_pin, k_pin, v_pin, out_pin, SCALE_DIVISOR)

        e2e_api = ("F3S.f3s_1tb1rw_scheduled_permuteV_scaleQK" if world == 1
                   else "fused3s_b200.sharding.ShardedAttention.forward")
        if world == 1:
            ref_args = (tcb, n, q_loc, k_loc, v_loc, (rp_t, ci_t))
        get_out = lambda: step_device()
        out_range = (r0, r1)
    else:
        # ---- heads divided over the ranks; every rank runs all row windows for heads/world heads
        rp_t = torch.from_numpy(g.rowptr).to(dev)
        ci_t = torch.from_numpy(g.colidx).to(dev)
        hp = sharding.HeadShardedPipeline(g.rowptr, g.colidx, n, heads, rank, world, dev, chunks=args.head_chunks,
                                          reserve_sms=args.reserve_sms, group=overlap_group,
                                          kv_group=overlap_group if args.kv_capped else None)
        preprocess_ms = hp.preprocess_ms
        n_tcb_local = hp.n_tcb
        sum_u_local = distinct_window_columns(rp_t, ci_t, n)
        totals_are_partial = False
        rb, re_ = hp.row_begin, hp.row_end
        q_pin, k_pin, v_pin = (x[rb:re_].contiguous().pin_memory() for x in (q_h, k_h, v_h))
        q_x = hp.to_exchange_layout(q_pin.to(dev))
        kv_x = hp.kv_to_exchange_layout(k_pin.to(dev), v_pin.to(dev))
        if mode == "heads-resident":
            hl = heads // world
            hs = slice(rank * hl, (rank + 1) * hl)
            q_hd, k_hd, v_hd = (x[:, hs].contiguous().to(dev) for x in (q_h, k_h, v_h))
            res = sharding.HeadShardedAttention(g.rowptr, g.colidx, n, heads, rank, world, dev)

            def step_device():
                return res.forward_resident(q_hd, k_hd, v_hd, SCALE_DIVISOR)
        else:
            def step_device():
                return hp.forward(q_x, kv_x, SCALE_DIVISOR)

        def make_kernel_only():
            return lambda: hp.kernel_only(SCALE_DIVISOR)

        out_pin = None if args.no_e2e else torch.empty((re_ - rb, heads, d), dtype=torch.float32).pin_memory()

        def step_e2e():  # host row shards in, host row shards out (layout conversions included)
            qx = hp.to_exchange_layout(q_pin.to(dev, non_blocking=True))
            kvx = hp.kv_to_exchange_layout(k_pin.to(dev, non_blocking=True), v_pin.to(dev, non_blocking=True))
            out_pin.copy_(hp.from_exchange_layout(hp.forward(qx, kvx, SCALE_DIVISOR)), non_blocking=True)

        e2e_api = "fused3s_b200.sharding.HeadShardedPipeline.forward"
        get_out = (lambda: hp.from_exchange_layout(hp.forward(q_x, kv_x, SCALE_DIVISOR))) \
            if mode == "heads" else None
        out_range = (rb, re_)
    h2d_bytes = int(3 * q_h.numel() * 2)

    # the clock sampler covers warm-up and the timed loops; warm-up lasts at least a second so that
    # nvidia-smi (one sample per 50 ms) sees the GPU under this kernel's load
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    warm_steps = max(args.warmup, 3) + (30 if world > 1 else 0)  # ranks must agree on the count
    t_warm = time.perf_counter()
    done = 0
    while done < warm_steps or (world == 1 and time.perf_counter() - t_warm < args.min_warmup_seconds):
        step_device()
        done += 1
        if done % 8 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    if world > 1 and args.min_warmup_seconds > 0:
        # several ranks: the number of further warm-up steps that fills the same time is agreed on first
        spent = torch.tensor([(time.perf_counter() - t_warm) / max(1, done)], device=dev, dtype=torch.float64)
        dist.all_reduce(spent, op=dist.ReduceOp.MAX)
        extra = int(min(20000, max(0.0, args.min_warmup_seconds - float(spent) * done) / max(1e-6, float(spent))))
        for i in range(extra):
            step_device()
            if i % 64 == 63:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
    launches0 = lib.f3s_kernel_launch_count()
    ms_steps, _ = bench.timed(step_device, args.steps)
    gpu_launches = int(lib.f3s_kernel_launch_count() - launches0)  # counted by the library, this rank
    # kernel-only time with every input already where the kernel needs it (pure kernel scaling)
    kernel_only = make_kernel_only()
    if kernel_only is not None:
        ms_kernel, ms_kernel_local = bench.timed(kernel_only, args.steps)
    else:
        ms_kernel, ms_kernel_local = ms_steps, ms_steps
    clocks = sampler.stop() if rank == 0 else None
    if world > 1 and mode == "rows":  # the parts of the step, each timed alone
        ms_ag, _ = bench.timed(attn._all_gather, args.steps)
        parts = {"all_gather_alone_ms": float(ms_ag.mean()), "collective": attn.collective_used}
        if attn._phased is not None:
            ph = attn._phased
            ms_2p, _ = bench.timed(lambda: (ph.launch_phase(1), ph.launch_phase(2)), args.steps)
            parts["two_launches_without_collective_ms"] = float(ms_2p.mean())
    else:
        parts = None
    if world > 1:  # per-rank kernel time: how well the partition balances
        t = torch.tensor([float(ms_kernel_local.mean())], device=dev, dtype=torch.float64)
        allt = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        per_rank = [float(x) for x in allt]
        balance = {"kernel_ms_per_rank_min": min(per_rank), "kernel_ms_per_rank_max": max(per_rank),
                   "kernel_ms_per_rank": per_rank}

    # ---- sampled parity of what the timed step produced (every rank checks rows of its own)
    parity = None
    if not args.no_parity_check and get_out is not None:
        out_dev = get_out()
        torch.cuda.synchronize()
        ok, ma, mr = parity_check(g, q_h, k_h, v_h, out_dev, out_range[0], out_range[1], seed=1000 + rank)
        flag = torch.tensor([1 if ok else 0], device=dev)
        worst = torch.tensor([ma, mr], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        parity = {"result": "ok" if int(flag) == 1 else "FAILED", "max_abs": float(worst[0]), "mean_rel": float(worst[1]),
                  "what": "4 sampled 64-row blocks of every rank's output rows against the CPU oracle "
                          "(bars: max-abs 2e-2, mean-rel 1e-3)"}
        del out_dev

    # ---- end to end through the public API, host buffers in and out
    e2e = None
    if not args.no_e2e:
        for _ in range(2):
            step_e2e()
        ms_e2e, _ = bench.timed(step_e2e, max(3, min(args.steps, 10)))
        flops = 4.0 * d * heads * g.nnz
        e2e = {"value": flops / (ms_e2e.mean() * 1e-3) / 1e9, "unit": "GFLOP/s", "ms_per_step": float(ms_e2e.mean()),
               "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": int(n * heads * d * 4), "api": e2e_api,
               "note": "pinned host Q/K/V in, pinned host output out, collectives included"}
        if pipe is not None:
            for _ in range(2):
                step_e2e_pipelined()
            ms_pipe, _ = bench.timed(step_e2e_pipelined, max(3, min(args.steps, 10)))
            # both public calls stay on record; the headline is the faster one (the pipeline pays off once
            # the transfers are long enough to hide behind the kernel)
            e2e["f3s_op_ms_per_step"] = e2e["ms_per_step"]
            e2e["pipelined_ms_per_step"] = float(ms_pipe.mean())
            best_ms, best_api = float(ms_pipe.mean()), (f"fused3s_b200.host_pipeline.HostPipelinedAttention.forward "
                                                        f"({len(pipe.plans)} row chunks)")
            if pipe2 is not None:  # K and V in two halves, every chunk as the two-launch forward
                for _ in range(2):
                    step_e2e_pipelined_halves()
                ms_h, _ = bench.timed(step_e2e_pipelined_halves, max(3, min(args.steps, 10)))
                e2e["pipelined_kv_halves_ms_per_step"] = float(ms_h.mean())
                if ms_h.mean() < best_ms:
                    best_ms, best_api = float(ms_h.mean()), best_api[:-1] + ", K/V in two halves, two launches per chunk)"
            if best_ms < ms_e2e.mean():
                e2e.update(value=flops / (best_ms * 1e-3) / 1e9, ms_per_step=best_ms, api=best_api,
                           note="pinned host Q/K/V in, pinned host output out; copies overlap the kernel; "
                                "f3s_op_ms_per_step is the same transfer done around one F3S op call")

    # ---- the score stage on the 5th-generation tensor cores, beside the fused kernel (optional)
    score_stage = None
    if args.score_stage and world == 1 and mode == "rows" and heads == 1 and d == 64:
        dump = torch.empty(tcb["nTCB"] * 256, dtype=torch.float32, device=dev)
        plan_dump = cabi.ForwardPlan(tcb, n, q_loc, k_loc, v_loc, SCALE_DIVISOR, sddmm_out=dump)
        ws_u = torch.empty(64, dtype=torch.uint8, device=dev)

        def umma_call():  # the C entry point itself: no status read-back inside the timed region
            cabi.check(lib.f3s_sddmm_umma(tcb["rowWindowOffset"].data_ptr(), tcb["sparseAToXidx"].data_ptr(),
                                          tcb["tcbBitMap"].data_ptr(), n, tcb["rowWindowOffset"].numel() - 1,
                                          tcb["nTCB"], 16, d, d, q_loc.data_ptr(), d, k_loc.data_ptr(), dump.data_ptr(),
                                          ws_u.data_ptr(), 64, torch.cuda.current_stream().cuda_stream))

        for _ in range(3):
            plan_dump.launch(), umma_call()
        st = max(3, min(args.steps, 10))
        (ms_d, _), (ms_u, _) = bench.timed(plan_dump.launch, st), bench.timed(umma_call, st)
        cabi.check(lib.f3s_forward_status(ws_u.data_ptr(), None, torch.cuda.current_stream().cuda_stream))
        score_stage = {"fused_kernel_ms": float(ms_steps.mean()), "fused_kernel_with_score_dump_ms": float(ms_d.mean()),
                       "score_stage_tcgen05_ms": float(ms_u.mean()), "score_dump_bytes": int(dump.numel() * 4),
                       "note": "f3s_sddmm_umma computes only S = Q K^T (masked) and writes the dump; the fused kernel "
                               "with dump computes softmax and P V as well"}
        del dump, plan_dump

    # ---- training path (optional): forward that also returns the row log-sum-exp, then dQ/dK/dV
    training = None
    if args.backward and world == 1 and mode == "rows":
        tr_ms = []
        for _ in range(2):  # the first call also pays for one-time allocations inside torch's sort
            e0.record()
            rp_tr, ci_tr = cabi.transpose_csr(rp_t, ci_t, n)
            e1.record()
            torch.cuda.synchronize()
            tr_ms.append(e0.elapsed_time(e1))
        transpose_ms = min(tr_ms)
        e0.record()
        tcb_tr = cabi.preprocess(ci_tr, rp_tr, n, 16)
        e1.record()
        torch.cuda.synchronize()
        d_out = torch.randn(q_loc.shape, device=dev, dtype=torch.float32)
        out_l, lse_l = cabi.forward_lse(tcb, n, q_loc, k_loc, v_loc, SCALE_DIVISOR)
        fl = lambda: cabi.forward_lse(tcb, n, q_loc, k_loc, v_loc, SCALE_DIVISOR)
        bw = lambda: cabi.backward(tcb, tcb_tr, n, q_loc, k_loc, v_loc, out_l, lse_l, d_out, SCALE_DIVISOR,
                                   grad_dtype=torch.float16)
        for _ in range(3):
            fl(), bw()
        st = max(3, min(args.steps, 10))
        (ms_fl, _), (ms_bw, _) = bench.timed(fl, st), bench.timed(bw, st)
        training = {"forward_lse_ms": float(ms_fl.mean()), "backward_ms": float(ms_bw.mean()),
                    "backward_edge_gflops": 10.0 * d * heads * g.nnz / (ms_bw.mean() * 1e-3) / 1e9,
                    "transpose_csr_ms": transpose_ms, "transposed_preprocess_ms": e0.elapsed_time(e1),
                    "nTCB_transposed": tcb_tr["nTCB"], "grad_dtype": "fp16",
                    "note": "backward = prepare kernel + dQ launch on the graph's TC blocks + dK/dV launch(es) on the "
                            "transposed graph's; useful flops counted as 5 products of 2*d per edge"}
        del out_l, lse_l, d_out, tcb_tr

    # ---- whole-job numbers
    tot = torch.tensor([n_tcb_local, sum_u_local, preprocess_ms], device=dev, dtype=torch.float64)
    if world > 1:
        mx = tot.clone()
        if totals_are_partial:
            dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        preprocess_ms = float(mx[2])
    n_tcb, sum_u = int(tot[0]), int(tot[1])

    # ---- the L2 ceiling for the gathers, measured here with this package's own probe kernel
    kv_bytes = 2 * n * d * 2  # K + V of one head (heads are walked one after the other)
    l2_gbs = cabi.gather_rate_gbs(kv_bytes, dev) if (rank == 0 and kv_bytes < 100e6) else None
    hbm_gather_gbs = cabi.gather_rate_gbs(2 << 30, dev, n_ids=1 << 23) if rank == 0 else None

    # ---- the other workloads (every rank takes part in the multi-GPU one)
    others = None
    if not args.no_other_workloads and args.scale == 1.0 and args.workload == "cfg4":
        others = {}
        sub_steps = max(5, min(args.steps, 20))
        # this workload's device buffers are no longer needed
        if world == 1:
            others["cfg3"] = single_gpu_subrecord(bench, 3, args, sub_steps)
            others["cfg5"] = single_gpu_subrecord(bench, 5, args, sub_steps)
        else:
            others["cfg5"] = multi_gpu_heads_subrecord(bench, 5, args, sub_steps, rank, world, overlap_group)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    flops = 4.0 * d * heads * g.nnz
    ms = float(ms_steps.mean())
    n_rw = (n + 15) // 16
    b_alg = algorithmic_bytes(n, heads, d, sum_u, n_tcb, n_rw)
    b_min = compulsory_bytes(n, heads, d, n_tcb, n_rw)
    peak, peak_src = measured_peaks()
    kern_ms = float(ms_kernel.mean())
    traffic = traffic_for(args.workload)
    roof = roofline_record(b_alg / world, b_min / world, kern_ms, peak, peak_src, traffic, kv_bytes, l2_gbs,
                           heads * d * 4 * sum_u / world,
                           kernel_name(d, n_tcb_local, (out_range[1] - out_range[0] + 15) // 16, False),
                           hbm_gather_gbs)
    roof["per_gpu"] = "bytes of one rank (1/n_gpus of the job) over the kernel-only time"
    line = {
        "metric": "edge_gflops", "value": flops / (ms * 1e-3) / 1e9, "unit": "GFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "ms_per_step_median": float(np.median(ms_steps)), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp16 operands, fp32 accumulate", "data": "synthetic",
        "config": workload_config(args, g),
        "kernel_only_ms": kern_ms,
        "preprocess_ms": preprocess_ms, "preprocess_note": "CSR -> all TC-block arrays incl. the one device->host "
        "read of the TCB count and the output allocations; best of 2 calls (rows mode)", "graph_build_s": t_gen,
        "tcb": {"nTCB": n_tcb, "sumU": sum_u, "nRW": n_rw},
        "roofline": roof,
        "e2e": e2e,
        "gpu_launches": gpu_launches,
        "gpu_launches_note": "kernels of this package launched by rank 0 inside the timed region, counted by the "
                             "library (f3s_kernel_launch_count)",
        "clocks": clocks,
    }
    if parity is not None:
        line["parity_check"] = parity["result"]
        line["parity"] = parity
    if balance is not None:
        line["balance"] = balance
    if parts is not None:
        line["step_parts"] = parts
    if others is not None:
        line["other_workloads"] = others
    if training is not None:
        line["training"] = training
    if score_stage is not None:
        line["score_stage"] = score_stage
    if world == 1 and not args.no_ref_cuda and ref_args is not None:
        line["reference_cuda_rebuilt"] = time_rebuilt_reference(*ref_args)
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(g, q_h, k_h, v_h)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
