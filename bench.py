#!/usr/bin/env python
"""Benchmark of the token-sampling stage: sampled tokens/s at B=256 x V=151936 fp32.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config c1|c2|c3|c4|c5] [--rows R] [--kernel-only]

One step is one pass of the sampler over one logit block. The default workload is the
benchmark configuration the metric is quoted on (c3: 256 rows of 151936 logits, per-row
settings: temperature U[0,1.5] with every 16th row greedy, top-k from {0,1,20,50,100}, top-p
U[0.5,1], repetition penalty U[1,1.3] over 256-token windows). With N GPUs the 256 rows are
sharded over the ranks (rows are independent: no collective; strong scaling); the value is the
256 rows times the steps over the slowest rank's device time. A `weak` sub-record times 256
rows on every rank as well. `--config c5` is the vocab-sharded case (needs --gpus 2, 4 or 8).
Prints one JSON line on rank 0.

`--impl reference` times the CPU restatement of the reference's own sampler on the host cores
(the reference itself is Mojo and cannot run here) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sampled tokens/s at B=256xV=151936 fp32"
NBUF = 3  # distinct logit blocks rotated between steps so that no step finds its rows in L2
L2_BYTES = 126 * 1024 * 1024


def workload(config: str, rows: int | None = None):
    from molla_b200 import workloads as W
    make = {"c1": W.config1, "c2": W.config2, "c3": W.config3, "c4": W.config4, "c5": W.config5}[config]
    return make() if rows is None else make(B=rows)


def algorithmic_bytes(w, top_n: int = 0, logprob: bool = False) -> int:
    """One read of the logits + the windows + ~48 B of settings per row + the token ids
    (+ the logprob outputs where they are asked for)."""
    B, V = w["logits"].shape
    out = 4 * B + (4 * B * (1 + 2 * top_n) if (logprob or top_n) else 0)
    return 4 * B * V + 8 * int(w["hist_off"][-1]) + 48 * B + out


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.rows = []
        self._stop = threading.Event()
        self._t = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.idx)], capture_output=True, text=True, timeout=5).stdout
                for line in out.strip().splitlines():
                    self.rows.append([x.strip() for x in line.split(",")])
            except Exception:
                pass
            self._stop.wait(0.05)

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_rate(w, rows: int, threads: int, seconds_target: float) -> tuple[float, int]:
    """Rows per second of the CPU restatement (oracle/) with the reference's own costs (the linear
    window scan per vocabulary entry, full heapsorts) on the first `rows` rows of `w`."""
    from oracle import pyoracle as O
    from molla_b200 import workloads as W
    best, used = None, min(rows, w["B"])
    t_all = time.time()
    for _ in range(3):
        sub = W.slice_rows(w, 0, used)
        kw = {k: sub[k] for k in W.SAMPLER_KEYS}
        t0 = time.perf_counter()
        O.pick_batch(sub["logits"], **kw, faithful_cost=True, nthreads=threads)
        dt = time.perf_counter() - t0
        best = used / dt if best is None else max(best, used / dt)
        if time.time() - t_all > seconds_target:
            break
        if dt < seconds_target / 6 and used < w["B"]:
            used = min(w["B"], used * 2)  # grow the sample while it stays cheap
    return best, used


def cpu_baseline(w, seconds_target: float = 12.0):
    """The reference samples every row on its one runner thread (batch.mojo:509-511, serve.mojo:122):
    the single-thread figure is what it does today; the all-core figure is what its loop could do."""
    cores = host_cores()
    allc, used = cpu_rate(w, max(cores, 8), cores, seconds_target)
    one, used1 = cpu_rate(w, 2, 1, seconds_target / 3)
    return {"value": allc, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"first {used} of {w['B']} rows of the same workload on all {cores} host threads "
                      "(rows are independent); faithful O(V*window) penalty scan and full heapsorts",
            "single_thread": {"value": one, "unit": "tokens/s", "cores": 1,
                              "sample": f"first {used1} rows on one thread, as the reference's runner thread samples"}}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import pyoracle as O
    from molla_b200 import workloads as W
    O.build()
    cores = host_cores()
    cfg = args.config if args.config != "c5" else "c5"
    full = workload(cfg)
    rows = max(8, min(full["B"], 2 * cores))
    w = W.slice_rows(full, 0, rows)  # the first rows of the very workload the GPU arm samples
    kw = {k: w[k] for k in W.SAMPLER_KEYS}
    for _ in range(args.warmup):
        O.pick_batch(w["logits"], **kw, faithful_cost=True, nthreads=cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.pick_batch(w["logits"], **kw, faithful_cost=True, nthreads=cores)
    dt = time.perf_counter() - t0
    value = rows * args.steps / dt
    sample = (f"first {rows} of the {full['B']} rows of the GPU arm's workload per step (rows are independent, so "
              f"rows/s of a sample is the rate), {cores} host threads; CPU restatement of sample.mojo "
              "(the Mojo reference cannot run here)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": full["name"], "rows_timed_per_step": rows, "rows_of_workload": full["B"]},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def exactness_report(w, tokens, status, sample_rows: int = 48):
    """Rows of the timed workload compared with the CPU checker outside the timed region: how many
    the library refused, how many carry a tie flag, how many the checker places within 1e-6 of a
    CDF edge, and how many differ without any of those reasons (must be none)."""
    from oracle import pyoracle as O
    from molla_b200 import capi, workloads as W
    n = min(sample_rows, w["B"])
    sub = W.slice_rows(w, 0, n)
    ref = O.pick_batch(sub["logits"], **{k: sub[k] for k in W.SAMPLER_KEYS})
    st = status[:n].astype(np.uint32)
    tok = tokens[:n]
    tie = ((st & np.uint32(capi.ROW_TIE_BITS)) != 0) | ((ref["flags"] & 7) != 0)
    edge = (ref["flags"] & O.FLAG_CDF_EDGE) != 0
    mism = tok != ref["tokens"]
    allst = status.astype(np.uint32)
    return {"rows_compared_with_cpu": int(n), "mismatches": int(mism.sum()),
            "tie_flagged": int(tie.sum()), "cdf_edge": int(edge.sum()),
            "unexplained": int((mism & ~tie & ~edge).sum()),
            "refused_rows_of_all": int(((allst & np.uint32(capi.ROW_UNSUPPORTED)) != 0).sum()),
            "error_rows_of_all": int(((allst & np.uint32(capi.ROW_ERROR_BITS)) != 0).sum()),
            "sums": "softmax denominator, kept mass and draw target bit-exact (tests/test_parity_gpu.py)"}


def roofline(abytes: int, ms_step: float, kernel: str, traffic_key: str | None):
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    src = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
    achieved = abytes / (ms_step / 1e3) / 1e9
    traffic = None
    if traffic_key:  # a figure captured with ncu for exactly this kernel and workload, or nothing
        try:
            traffic = json.load(open(os.path.join(ROOT, "profiles", "traffic.json"))).get(traffic_key, {}).get("bytes")
        except Exception:
            pass
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": traffic, "peak_source": src, "frac_of_8TBs_nominal": achieved / 8000.0,
            "algorithmic_bytes_per_launch": abytes, "kernel": kernel, "avg_launch_ms": ms_step}


def n_blocks(block_bytes: int) -> int:
    """Distinct logit blocks rotated through the steps: enough that their total is well above the
    L2 (a step never finds its rows there), within reason for tiny blocks."""
    return int(min(64, max(NBUF, -(-int(2.2 * L2_BYTES) // max(block_bytes, 1)) + 1)))


class Timed:
    """One workload resident on the device, ready to be stepped."""

    def __init__(self, w, dev, top_n=0, logprob=False):
        import torch
        from molla_b200 import sampler as S
        self.S, self.torch, self.w, self.dev = S, torch, w, dev
        self.B, self.V = w["logits"].shape
        self.top_n, self.logprob = top_n, logprob
        self.p = S.upload_params(w, dev)          # per-row settings: uploaded once, resident, not re-sent per step
        first = torch.from_numpy(w["logits"]).to(dev)
        self.nbuf = n_blocks(first.numel() * 4)
        self.bufs = [first] + [torch.roll(first, shifts=i * 7 + 1, dims=0).contiguous() for i in range(1, self.nbuf)]
        self.ws = S.Workspace(self.B, self.V, top_n, dev)
        self.out = {"tokens": torch.empty(self.B, dtype=torch.int32, device=dev),
                    "row_status": torch.empty(self.B, dtype=torch.int32, device=dev)}

    def step(self, i):
        return self.S.sample_batch(self.bufs[i % self.nbuf], self.p, workspace=self.ws, out=self.out,
                                   top_n=self.top_n, want_logprob=self.logprob)

    def run(self, steps, warmup, barrier):
        torch = self.torch
        for i in range(max(warmup, 3)):
            self.step(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            self.step(i)
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    def first_block_results(self):
        self.step(0)
        self.torch.cuda.synchronize()
        return self.out["tokens"].cpu().numpy(), self.out["row_status"].cpu().numpy()

    def launches_per_step(self):
        sms = self.torch.cuda.get_device_properties(self.dev).multi_processor_count
        # thread blocks per row (the smallest cluster whose blocks hold 38400 logits each); the kernel
        # that ranks the rows runs when not all rows can start at once
        groups = next(g for g in (1, 2, 4, 8, 8) if self.V <= 38400 * g or g == 8)
        return 1 + (1 if self.B * groups > sms else 0) + (1 if (self.logprob or self.top_n) else 0)


def measure_e2e(w, dev, steps, barrier, top_n=0, logprob=False):
    """The same step through the host-buffer entry point: pinned host block in (host-to-device copy
    inside the timed region), host tokens out."""
    import torch
    from molla_b200 import sampler as S
    hb = S.HostBlock(w, dev, top_n=top_n, want_logprob=logprob)
    for _ in range(2):
        S.sample_batch_host(hb)
    barrier()
    t0 = time.perf_counter()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(steps):
        S.sample_batch_host(hb)
    e3.record()
    barrier()
    return max(e2.elapsed_time(e3), 1e3 * (time.perf_counter() - t0)), hb.h2d_bytes, hb.d2h_bytes


def run_ours(args):
    import torch
    import torch.distributed as dist
    from molla_b200 import capi, sharded, workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampling kernels have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    capi.lib()  # fail loudly here if the library is missing

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(*vals):
        if world == 1:
            return list(vals)
        t = torch.tensor(vals, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t]

    if args.config == "c5":
        return run_c5(args, world, rank, dev, barrier, max_over_ranks)

    full = workload(args.config, args.rows)
    B_total, V = full["logits"].shape
    top_n = int(full.get("top_n", 0))
    logprob = top_n > 0
    lo, hi = sharded.row_range(rank, world, B_total)     # this rank's rows of the one workload
    mine = W.slice_rows(full, lo, hi)
    steps = args.steps

    t = Timed(mine, dev, top_n, logprob)
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
        time.sleep(0.2)
    ms = t.run(steps, args.warmup, barrier)
    repeats = [t.run(steps, 0, barrier) / steps for _ in range(3)] if not args.kernel_only else []
    tok, st = t.first_block_results()
    launches = t.launches_per_step()
    nbuf = t.nbuf
    e2e_ms = e2e_steps = h2d = d2h = None
    if not args.kernel_only:
        e2e_steps = max(3, min(steps, 10))
        e2e_ms, h2d, d2h = measure_e2e(mine, dev, e2e_steps, barrier, top_n, logprob)
    clk = clocks.stop() if rank == 0 else None
    del t
    torch.cuda.empty_cache()

    weak_ms = None
    if world > 1 and not args.kernel_only:   # every rank all the rows: the weak-scaling figure of earlier records
        tw = Timed(full, dev, top_n, logprob)
        weak_ms = tw.run(steps, args.warmup, barrier)
        del tw
        torch.cuda.empty_cache()

    bad = int(np.sum((st.astype(np.uint32) & np.uint32(capi.ROW_ERROR_BITS)) != 0))
    ms, e2e_max, weak_max, bad_all = (max_over_ranks(ms, e2e_ms or 0.0, weak_ms or 0.0, 0.0)[:3] + [bad])
    if world > 1:
        b = torch.tensor([bad], device=dev)
        dist.all_reduce(b)
        bad_all = int(b[0])

    if rank == 0:
        ms_step = ms / steps
        abytes_rank = algorithmic_bytes(mine, top_n, logprob)   # the slowest rank's launch streams its own rows
        line = {
            "metric": METRIC, "value": B_total * steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": full["name"], "rows_total": B_total, "rows_per_gpu": hi - lo, "vocab": V,
                       "sharding": "rows of the one workload split over the ranks, no collective",
                       "l2": f"{nbuf} distinct {4 * (hi - lo) * V / 1e6:.0f} MB logit blocks rotated per rank "
                             f"({nbuf * 4 * (hi - lo) * V / 1e6:.0f} MB against a 126 MB L2)",
                       "params": "per-row settings, windows and draw counters resident on the device, uploaded once "
                                 "outside the timed region (the decode loop keeps them there)",
                       "timed_region_ms": ms, "ms_per_step_of_3_more_runs": repeats},
            "roofline": roofline(abytes_rank, ms_step, "sample_rows_cluster_kernel",
                                 f"sample_rows_cluster_kernel:{args.config}" if args.rows is None else None),
            "e2e": None if e2e_ms is None else {
                "value": B_total * e2e_steps / (e2e_max / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_max / e2e_steps, "steps": e2e_steps,
                "bytes_are": "per rank"},
            "gpu_launches": steps * launches,
            "clocks": clk,
        }
        if weak_ms is not None:
            line["weak"] = {"scaling": "weak", "rows_per_gpu": B_total, "ms_per_step": weak_max / steps,
                            "value": world * B_total * steps / (weak_max / 1e3), "unit": "tokens/s"}
        if not args.kernel_only:
            ex = exactness_report(mine, tok, st)
            ex["error_rows_all_ranks"] = bad_all
            line["config"]["exactness"] = ex
        else:
            line["config"]["exactness"] = {"error_rows_all_ranks": bad_all}
        if world == 1 and not args.kernel_only:
            line["cpu_baseline"] = cpu_baseline(full)
            if args.config == "c3" and args.rows is None:
                line["configs"] = other_configs(dev, barrier)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def other_configs(dev, barrier):
    """The other single-GPU benchmark configurations, briefly: ms per step, tokens/s, GB/s of
    algorithmic bytes, fraction of the measured HBM peak."""
    import torch
    out = {}
    for cfg, steps in (("c1", 200), ("c2", 50), ("c4", 8)):
        w = workload(cfg)
        top_n = int(w.get("top_n", 0))
        t = Timed(w, dev, top_n, top_n > 0)
        ms = t.run(steps, 3, barrier) / steps
        rf = roofline(algorithmic_bytes(w, top_n, top_n > 0), ms, "sample_rows_cluster_kernel", None)
        out[cfg] = {"workload": w["name"], "ms_per_step": ms, "tokens_per_s": w["B"] / (ms / 1e3),
                    "achieved_GBs": rf["achieved"], "frac_of_measured_peak": rf["frac"],
                    "launches_per_step": t.launches_per_step(), "blocks_rotated": t.nbuf}
        del t
        torch.cuda.empty_cache()
    out["c5"] = "vocab-sharded: python bench.py --config c5 --gpus 8 (under torchrun)"
    return out


def run_c5(args, world, rank, dev, barrier, max_over_ranks):
    """The vocab-sharded configuration: every rank holds a contiguous slice of each row's columns and
    one `molla_sample_sharded_step` per step runs the stages and the all-gathers between them."""
    import torch
    import torch.distributed as dist
    from molla_b200 import capi, sampler as S, sharded
    if world < 2:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "unavailable": "config c5 is the vocab-sharded case: run it under "
                              "torchrun with --gpus 2, 4 or 8"}))
        return 0
    w = workload("c5", args.rows)
    B, V = w["logits"].shape
    Vs = V // world
    nbuf = n_blocks(4 * B * Vs)
    first = torch.from_numpy(np.ascontiguousarray(w["logits"][:, rank * Vs:(rank + 1) * Vs])).to(dev)
    bufs = [first] + [torch.roll(first, shifts=i * 7 + 1, dims=1).contiguous() for i in range(1, nbuf)]
    p = S.upload_params(w, dev)
    sh = sharded.NcclShardedSampler(B, Vs, rank * Vs, V, rank, world, dev, sharded.share_over_torch_distributed())
    for i in range(max(args.warmup, 3)):
        sh.step(bufs[i % nbuf], p)
    barrier()
    clocks = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        sh.step(bufs[i % nbuf], p)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clk = clocks.stop() if rank == 0 else None
    tok, st = sh.step(bufs[0], p)
    torch.cuda.synchronize()
    st = st.cpu().numpy().astype(np.uint32)
    tok = tok.cpu().numpy()
    wire = sh.wire_bytes
    (ms,) = max_over_ranks(ms)
    if rank == 0:
        ms_step = ms / args.steps
        ab = 4 * B * Vs + 8 * int(w["hist_off"][-1]) + 52 * B   # this rank's slice, once
        line = {
            "metric": "sampled tokens/s, vocab-sharded (config 5)", "value": B * args.steps / (ms / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": w["name"], "rows": B, "vocab": V, "columns_per_gpu": Vs,
                       "exchange": dict(wire, collectives="three NCCL all-gathers per step (summaries, list lengths, lists)"),
                       "exactness": exactness_report(w, tok, st)},
            "roofline": roofline(ab, ms_step, "sample_rows_kernel (stages a, b, c)", None),
            "e2e": None, "gpu_launches": args.steps * 6, "clocks": clk,
        }
        print(json.dumps(line))
    sh.close()
    dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300, help="timed steps (300 steps of the default workload are about 0.1 s)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c3", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--rows", type=int, default=None, help="a workload of this many rows instead (profiler captures)")
    ap.add_argument("--kernel-only", action="store_true", help="skip the end-to-end, CPU and exactness legs")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.steps > 40:
            args.steps = 40   # a bounded sample: every step is seconds of host work
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
