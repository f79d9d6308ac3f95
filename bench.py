#!/usr/bin/env python
"""Benchmark of the hot path: BinnedSelectKnn + AccumulateKnn on 200k-hit events.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (synthetic, seeded): a batch of ``--events`` (default 64) events of 200k hits each from the
shower-plus-noise generator (4 coordinates, K = 64 neighbours incl. the hit itself, F = 64 float32
features).  A step is one pass of the path over the batch: BinnedSelectKnn (grid, binning, sort,
search, mapping back) followed by AccumulateKnn with exp(-10 d^2) weights (mean | max, and the
arg-max indices).  With N GPUs the events are split evenly over the ranks (whole events, no
collective on the data path); the total work is fixed, so the scaling is "strong".

One JSON line is printed by rank 0.  ``value`` is hits/s with the inputs resident in device memory,
``e2e`` the same through host buffers (pinned host -> device copies of coordinates, features and
row splits, device -> host copy of the accumulated features inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "hits/sec for BinnedSelectKnn+AccumulateKnn at 200k-hit events"
UNIT = "hits/s"
# DRAM traffic per hit of the two main kernels at K = F = 64, 4 coordinates, from the ncu capture
# summarised in profiles/select_knn_and_accumulate_2events_full.md (traffic grows with the hits).
ACC_DRAM_BYTES_PER_HIT = 1972
KNN_DRAM_BYTES_PER_HIT = 438
KNN_ISSUE_ACTIVE_PCT = 90.4
KNN_WARP_INSTR_PER_QUERY = 5715


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--events", type=int, default=64)
    p.add_argument("--hits", type=int, default=200000)
    p.add_argument("--neighbours", type=int, default=64)
    p.add_argument("--features", type=int, default=64)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-kernel-times", action="store_true")
    return p.parse_args()


def workload_config(a):
    return {"workload": f"{a.events} events x {a.hits} hits, shower+noise generator, 4 coordinates "
                        f"(3 binned), K={a.neighbours}, F={a.features}, float32",
            "events": a.events, "hits_per_event": a.hits, "K": a.neighbours, "F": a.features,
            "coord_dims": 4, "sharding": "whole events per rank, no collective",
            "l2": "inputs larger than L2 (no explicit flush)"}


def make_events(a, event_ids):
    from hgcalml_b200 import synth
    coords = [synth.shower_event(a.hits, dims=4, seed=500 + e) for e in event_ids]
    feats = [np.random.default_rng(700000 + e).standard_normal((a.hits, a.features), dtype=np.float32)
             for e in event_ids]
    row_splits = (np.arange(len(event_ids) + 1) * a.hits).astype(np.int32)
    return np.concatenate(coords), np.concatenate(feats), row_splits


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, t_begin=None, t_end=None):
        """Samples taken between the two wall-clock times (all of them when none fall inside: the
        sampler runs from the warm-up on, so those are under the same load)."""
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            for line in open(self.path):
                c = [x.strip() for x in line.split(",")]
                if len(c) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(c[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    rows.append((ts, float(c[1]), float(c[2]), c[5:9]))
                except ValueError:
                    continue
            os.unlink(self.path)
        except Exception:
            pass
        inside = [r for r in rows if t_begin is not None and t_begin <= r[0] <= t_end]
        use = inside or rows
        reasons = set()
        for r in use:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if use:
            out.update(sm_mhz=float(np.median([r[1] for r in use])), sm_max_mhz=float(max(r[2] for r in use)),
                       reasons=sorted(reasons), samples=len(use), samples_in_timed_region=len(inside))
        return out


# ------------------------------------------------------------------------------------ reference arm
def _ref_backend():
    from oracle import oracle as O
    if O.have("ref"):
        return O, "ref", "reference"
    return O, "port", "port"


def cpu_path_event(O, backend, coords, feats, row_splits, K, n_threads=1, pool=None):
    """The reference's CPU path for one batch (wrapper glue in numpy, ops from the CPU library),
    optionally with queries / rows spread over threads; see oracle.knn_accumulate_path."""
    return O.knn_accumulate_path(K, coords, feats, row_splits, n_threads=n_threads, pool=pool, backend=backend)


def run_reference_arm(a):
    """Times the reference's own CPU implementation of the path on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from concurrent.futures import ThreadPoolExecutor
    O, backend, kind = _ref_backend()
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    n_threads = max(1, min(cores, 64))
    pool = ThreadPoolExecutor(n_threads)
    sample_events = 1
    coords, feats, rs = make_events(a, list(range(sample_events)))
    for _ in range(a.warmup):
        cpu_path_event(O, backend, coords, feats, rs, a.neighbours, n_threads, pool)
    t0 = time.perf_counter()
    for _ in range(a.steps):
        cpu_path_event(O, backend, coords, feats, rs, a.neighbours, n_threads, pool)
    dt = time.perf_counter() - t0
    hits = sample_events * a.hits * a.steps
    value = hits / dt
    sample = (f"{sample_events} event of {a.hits} hits per step (of the {a.events}-event batch); queries split over "
              f"{n_threads} threads via the op's direction input, AccumulateKnn over row slices")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": 1e3 * dt / a.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(a),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": n_threads, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def cpu_baseline(a):
    """One event on one host core through the reference's CPU path (a reported baseline, not a target)."""
    O, backend, kind = _ref_backend()
    coords, feats, rs = make_events(a, [0])
    t0 = time.perf_counter()
    cpu_path_event(O, backend, coords, feats, rs, a.neighbours, 1)
    dt = time.perf_counter() - t0
    return {"value": a.hits / dt, "unit": UNIT, "cores": 1, "kind": kind,
            "sample": f"1 event of {a.hits} hits, single thread, {dt:.1f} s"}


# ------------------------------------------------------------------------------------------ our arm
def main():
    a = parse()
    if a.impl == "reference":
        run_reference_arm(a)
        return

    import torch
    import torch.distributed as dist
    from hgcalml_b200 import _capi
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn
    from hgcalml_b200.accknn_op import AccumulateKnn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    K, F = a.neighbours, a.features
    from hgcalml_b200.sharding import shard_events
    first, last = shard_events(np.arange(a.events + 1) * a.hits, world)[rank]
    my_events = list(range(first, last))
    coords_h, feats_h, rs_h = make_events(a, my_events)
    n = coords_h.shape[0]
    coords_p = torch.from_numpy(coords_h).pin_memory()
    feats_p = torch.from_numpy(feats_h).pin_memory()
    rs_p = torch.from_numpy(rs_h).pin_memory()
    out_p = torch.empty((n, 2 * F), dtype=torch.float32).pin_memory()

    coords = coords_p.to(dev)
    feats = feats_p.to(dev)
    rs = rs_p.to(dev)

    def step():
        idx, d2, sorting = BinnedSelectKnn(K, coords, rs, return_sorting=True)
        out, maxidx = AccumulateKnn(d2, feats, idx, order=sorting, distance_scale=10.)
        return out

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(a.warmup, 1)):
        step()
    barrier()
    t_begin = time.time()
    launches0 = _capi.lib.hgc_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(a.steps):
        step()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = _capi.lib.hgc_launch_count() - launches0
    clocks = sampler.stop(t_begin, time.time()) if rank == 0 else None

    kernel_times = None
    if rank == 0 and not a.no_kernel_times:
        kernel_times = measure_kernels(torch, dev, coords, feats, rs, K, F)

    # end to end: host buffers in, accumulated features out, copies inside the timed region.  The
    # public host-buffer entry cuts the batch into chunks of whole events and overlaps the PCIe
    # copies of neighbouring chunks with the kernels (three streams, double-buffered inputs).
    from hgcalml_b200.pipeline import KnnAccumulatePipeline
    del coords, feats
    torch.cuda.empty_cache()
    pipe = KnnAccumulatePipeline(K, dev, events_per_chunk=2, distance_scale=10.)

    def e2e_step():
        pipe.run(coords_p, feats_p, rs_h, out_p)

    e2e_step()
    barrier()
    e2e_steps = max(1, min(a.steps, 3))
    ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev2.record()
    for _ in range(e2e_steps):
        e2e_step()
    ev3.record()
    barrier()
    e2e_ms = ev2.elapsed_time(ev3)

    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    total_hits = a.events * a.hits

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"
        line = {"metric": METRIC, "value": total_hits * a.steps / (ms * 1e-3), "unit": UNIT,
                "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": workload_config(a), "clocks": clocks,
                "gpu_launches": int(launches),
                "e2e": {"value": total_hits * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": int(coords_p.numel() * 4 + feats_p.numel() * 4 + rs_p.numel() * 4),
                        "d2h_bytes_per_step": int(out_p.numel() * 4), "steps": e2e_steps,
                        "result": "accumulated features [N, 2F]",
                        "api": "hgcalml_b200.pipeline.KnnAccumulatePipeline.run (chunks of whole events, copies overlapped with kernels)"}}
        if kernel_times:
            acc_bytes = n * (8 * K + 16 * F)
            knn_bytes = n * (4 * 4 + 4 + 4 * 4 + 8 * K)
            acc = {"kernel": "accumulate_vec_kernel", "bound": "hbm",
                   "achieved": acc_bytes / (kernel_times["accumulate_ms"] * 1e-3) / 1e9, "peak": hbm_peak,
                   "unit": "GB/s", "peak_kind": peak_kind, "traffic": int(n * ACC_DRAM_BYTES_PER_HIT) if (K, F) == (64, 64) else None,
                   "traffic_source": "ncu dram__bytes_read+write of a 400k-hit launch, scaled by hits",
                   "ms_per_launch": kernel_times["accumulate_ms"], "algorithmic_bytes": acc_bytes}
            acc["frac"] = acc["achieved"] / hbm_peak
            knn = {"kernel": "select_knn_kernel", "bound": "hbm",
                   "achieved": knn_bytes / (kernel_times["select_knn_ms"] * 1e-3) / 1e9, "peak": hbm_peak,
                   "unit": "GB/s", "peak_kind": peak_kind, "traffic": int(n * KNN_DRAM_BYTES_PER_HIT) if (K, F) == (64, 64) else None,
                   "traffic_source": "ncu dram__bytes_read+write of a 400k-hit launch, scaled by hits",
                   "ms_per_launch": kernel_times["select_knn_ms"], "algorithmic_bytes": knn_bytes,
                   "note": "the search is bound by instruction issue (sorting networks on shuffles), not by "
                           "HBM; the HBM figure is reported because it is the dominant kernel by time",
                   # what bounds it instead, from the ncu capture of a 400k-hit launch (profiles/): issue
                   # slots in use, and warp instructions per query against the SMs' issue rate at the
                   # sampled clock
                   "issue": {"ncu_issue_active_pct": KNN_ISSUE_ACTIVE_PCT,
                             "ncu_warp_instructions_per_query": KNN_WARP_INSTR_PER_QUERY,
                             "issue_bound_ms": n * KNN_WARP_INSTR_PER_QUERY
                                               / (148 * 4 * float((clocks or {}).get("sm_mhz") or 1965.0) * 1e6) * 1e3
                             if (K, F) == (64, 64) else None}}
            knn["frac"] = knn["achieved"] / hbm_peak
            dominant = knn if kernel_times["select_knn_ms"] >= kernel_times["accumulate_ms"] else acc
            line["roofline"] = dominant
            line["roofline_kernels"] = {"select_knn": knn, "accumulate_knn": acc}
            line["stage_ms"] = kernel_times
        if not a.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(a)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def measure_kernels(torch, dev, coords, feats, rs, K, F, reps=3):
    """Per-launch durations of the two main kernels with CUDA events on the launching stream:
    AccumulateKnn is a single kernel; the search kernel is timed through the op-level entry on
    bin-sorted inputs (its only other launch is the small coordinate packing kernel)."""
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn, _BinnedSelectKnn
    from hgcalml_b200.accknn_op import AccumulateKnn
    from hgcalml_b200.bin_by_coordinates_op import BinByCoordinates

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    idx, d2, sorting = BinnedSelectKnn(K, coords, rs, return_sorting=True)
    acc_ms = timed(lambda: AccumulateKnn(d2, feats, idx, order=sorting, distance_scale=10.))
    acc_unordered_ms = timed(lambda: AccumulateKnn(d2, feats, idx, distance_scale=10.))
    wrapper_ms = timed(lambda: BinnedSelectKnn(K, coords, rs))
    # op-level search on bin-sorted inputs
    n_first = int(rs[1].item())
    nb0 = int(min(max(int((np.float32(n_first) / np.float32(K / 32)) ** np.float32(1 / 3)), 5), 30))
    dbin, flat, nb, bw, nper = BinByCoordinates(coords[:, :3].contiguous(), rs, n_bins=nb0)
    order = torch.sort(flat, stable=True).indices
    sc, sb, sdb = coords[order].contiguous(), flat[order].contiguous(), dbin[order].contiguous()
    bb = torch.cat([torch.zeros(1, dtype=torch.int32, device=dev), nper.cumsum(0).to(torch.int32)])
    knn_ms = timed(lambda: _BinnedSelectKnn(K, sc, sb, sdb, bb, nb, bw))
    return {"accumulate_ms": acc_ms, "accumulate_unordered_ms": acc_unordered_ms,
            "select_knn_ms": knn_ms, "binned_select_knn_wrapper_ms": wrapper_ms}


if __name__ == "__main__":
    main()
