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
# Counters of the two main kernels at K = F = 64, 4 coordinates, from one ncu capture of a 400k-hit
# launch each (the DRAM traffic grows in proportion to the hits); this is their only copy.
NCU = {
    "accumulate_knn": {"dram_bytes_per_hit": 1782, "algorithmic_bytes_per_hit": 1536},
    "accumulate_knn_no_argmax": {"dram_bytes_per_hit": 1314, "algorithmic_bytes_per_hit": 1280},
    "select_knn": {"dram_bytes_per_hit": 433, "issue_active_pct": 90.4, "warp_instructions_per_query": 5715},
}


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
    p.add_argument("--no-kernel-times", action="store_true",
                   help="skip the per-kernel, single-event and configuration 3/4 measurements")
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
def device_timed(torch, fn, reps):
    """Average duration of fn in ms, CUDA events on the current stream, one untimed call first."""
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


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
        # the two ops with all their outputs: neighbour indices and distances, [mean | max], arg-max indices
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

    extra = None
    if rank == 0 and not a.no_kernel_times:
        extra = measure_kernels(torch, dev, coords, feats, rs, K, F)
        if world == 1:
            extra["single_event"] = measure_single_event(torch, dev, coords, feats, coords_p, feats_p, a, K, F)

    # end to end: host buffers in, accumulated features out, copies inside the timed region.  The
    # public host-buffer entry cuts the batch into chunks of whole events and overlaps the PCIe
    # copies of neighbouring chunks with the kernels (three streams, double-buffered inputs); each
    # call returns with its result rows in host memory.  At least eight chunks per rank, so that
    # filling and draining the three stages stays a small part of a call.
    from hgcalml_b200.pipeline import KnnAccumulatePipeline
    del coords, feats
    torch.cuda.empty_cache()
    events_per_chunk = 2 if len(my_events) >= 16 else 1
    pipe = KnnAccumulatePipeline(K, dev, events_per_chunk=events_per_chunk, distance_scale=10.)

    def timed_e2e(copies_only):
        pipe.run(coords_p, feats_p, rs_h, out_p, copies_only=copies_only)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            pipe.run(coords_p, feats_p, rs_h, out_p, copies_only=copies_only)
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    e2e_ms = timed_e2e(False)
    copy_ms = timed_e2e(True)

    t = torch.tensor([ms, e2e_ms, copy_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, copy_ms = float(t[0]), float(t[1]), float(t[2])
    total_hits = a.events * a.hits

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"
        h2d = int(coords_p.numel() * 4 + feats_p.numel() * 4 + rs_p.numel() * 4)
        d2h = int(out_p.numel() * 4)
        e2e_value = total_hits * a.steps / (e2e_ms * 1e-3)
        copy_value = total_hits * a.steps / (copy_ms * 1e-3)
        line = {"metric": METRIC, "value": total_hits * a.steps / (ms * 1e-3), "unit": UNIT,
                "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": workload_config(a), "clocks": clocks,
                "gpu_launches": int(launches),
                "e2e": {"value": e2e_value, "unit": UNIT,
                        "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": a.steps,
                        "ms_per_step": e2e_ms / a.steps,
                        "result": "accumulated features [N, 2F] in host memory when each call returns",
                        "api": "hgcalml_b200.pipeline.KnnAccumulatePipeline.run (chunks of whole events, "
                               "copies overlapped with kernels)",
                        "events_per_chunk": events_per_chunk,
                        # the same chunks, buffers, streams and copies with the two ops left out: what the
                        # transfers alone allow on this host, and how close the full call comes to it
                        "copy_only": {"value": copy_value, "unit": UNIT, "ms_per_step": copy_ms / a.steps,
                                      "host_gb_per_s": (h2d + d2h) * world * a.steps / (copy_ms * 1e-3) / 1e9},
                        "pipeline_efficiency": e2e_value / copy_value}}
        if extra:
            kt = extra["stage_ms"]
            sm_mhz = float((clocks or {}).get("sm_mhz") or 1965.0)
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            full = (K, F) == (64, 64)

            def hbm(ms_, bytes_per_hit, dram_per_hit):
                ach = n * bytes_per_hit / (ms_ * 1e-3) / 1e9
                return {"bound": "hbm", "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak,
                        "peak_kind": peak_kind, "ms_per_launch": ms_, "algorithmic_bytes": n * bytes_per_hit,
                        "traffic": int(n * dram_per_hit) if (full and dram_per_hit) else None,
                        "traffic_source": "ncu dram__bytes_read+write of a 400k-hit launch, scaled by hits"}

            acc = dict(hbm(kt["accumulate_ms"], 8 * K + 16 * F, NCU["accumulate_knn"]["dram_bytes_per_hit"]),
                       kernel="accumulate kernel, arg-max indices written")
            acc_na = dict(hbm(kt["accumulate_no_argmax_ms"], 8 * K + 12 * F,
                              NCU["accumulate_knn_no_argmax"]["dram_bytes_per_hit"]),
                          kernel="accumulate kernel, [mean | max] only (what the host-buffer entry runs)")
            knn_hbm = hbm(kt["select_knn_ms"], 4 * 4 + 4 + 4 * 4 + 8 * K, NCU["select_knn"]["dram_bytes_per_hit"])
            # The search is bound by instruction issue, not by memory: its roofline is the warp
            # instructions it needs per query (ncu) against the issue slots of the SMs at the clock
            # sampled during the run; the HBM view is kept beside it.
            instr = NCU["select_knn"]["warp_instructions_per_query"]
            issue_peak = sms * 4 * sm_mhz * 1e6 / 1e9
            issue_ach = n * instr / (kt["select_knn_ms"] * 1e-3) / 1e9 if full else None
            knn = {"kernel": "select_knn_kernel", "bound": "issue", "achieved": issue_ach, "peak": issue_peak,
                   "unit": "G warp-instructions/s", "frac": issue_ach / issue_peak if full else None,
                   "ms_per_launch": kt["select_knn_ms"],
                   "ncu_issue_active_pct": NCU["select_knn"]["issue_active_pct"] if full else None,
                   "ncu_warp_instructions_per_query": instr if full else None,
                   "traffic": knn_hbm["traffic"], "hbm": knn_hbm}
            dominant = knn if kt["select_knn_ms"] >= kt["accumulate_ms"] else acc
            line["roofline"] = dominant
            line["roofline_kernels"] = {"select_knn": knn, "accumulate_knn": acc, "accumulate_knn_no_argmax": acc_na}
            line["stage_ms"] = kt
            if "single_event" in extra:
                line["single_event"] = extra["single_event"]
            if world == 1:
                line["configs"] = measure_other_configs(torch, dev, K, F, not a.no_cpu_baseline)
        if not a.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(a)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def measure_kernels(torch, dev, coords, feats, rs, K, F, reps=3):
    """Per-launch durations of the two main kernels with CUDA events on the launching stream:
    AccumulateKnn is a single kernel; the search kernel is timed through the op-level entry on
    bin-sorted inputs (its only other launches are the small packing and bounding-box kernels)."""
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn, _BinnedSelectKnn
    from hgcalml_b200.accknn_op import AccumulateKnn
    from hgcalml_b200.bin_by_coordinates_op import BinByCoordinates

    def timed(fn):
        return device_timed(torch, fn, reps)

    idx, d2, sorting = BinnedSelectKnn(K, coords, rs, return_sorting=True)
    acc_ms = timed(lambda: AccumulateKnn(d2, feats, idx, order=sorting, distance_scale=10.))
    acc_na_ms = timed(lambda: AccumulateKnn(d2, feats, idx, order=sorting, distance_scale=10., with_max_idxs=False))
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
    return {"stage_ms": {"accumulate_ms": acc_ms, "accumulate_no_argmax_ms": acc_na_ms,
                         "accumulate_unordered_ms": acc_unordered_ms,
                         "select_knn_ms": knn_ms, "binned_select_knn_wrapper_ms": wrapper_ms}}


def measure_single_event(torch, dev, coords, feats, coords_p, feats_p, a, K, F, reps=20):
    """What a predict loop with batch size 1 runs: one 200k-hit event per call.  Device-timed per
    call, launches per call, the share of the two main kernels, and the same through host buffers."""
    from hgcalml_b200 import _capi
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn
    from hgcalml_b200.accknn_op import AccumulateKnn
    from hgcalml_b200.pipeline import KnnAccumulatePipeline
    n1 = a.hits
    c1, f1 = coords[:n1].contiguous(), feats[:n1].contiguous()
    rs1 = torch.tensor([0, n1], dtype=torch.int32, device=dev)

    def call():
        idx, d2, sorting = BinnedSelectKnn(K, c1, rs1, return_sorting=True)
        return AccumulateKnn(d2, f1, idx, order=sorting, distance_scale=10., with_max_idxs=False)

    l0 = _capi.lib.hgc_launch_count()
    call()
    launches = int(_capi.lib.hgc_launch_count() - l0)
    call_ms = device_timed(torch, call, reps)
    idx, d2, sorting = BinnedSelectKnn(K, c1, rs1, return_sorting=True)
    knn_ms = device_timed(torch, lambda: BinnedSelectKnn(K, c1, rs1, return_sorting=True), reps)
    acc_ms = device_timed(torch, lambda: AccumulateKnn(d2, f1, idx, order=sorting, distance_scale=10.,
                                                       with_max_idxs=False), reps)
    # host buffers: wall clock around blocking calls (each returns with its rows in host memory)
    pipe = KnnAccumulatePipeline(K, dev, events_per_chunk=1, distance_scale=10.)
    cp, fp = coords_p[:n1], feats_p[:n1]
    out = torch.empty((n1, 2 * F), dtype=torch.float32).pin_memory()
    rs_h = np.array([0, n1], np.int64)
    pipe.run(cp, fp, rs_h, out)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(reps):
        pipe.run(cp, fp, rs_h, out)
    host_ms = (time.perf_counter() - t0) / reps * 1e3
    return {"hits": n1, "call_ms": call_ms, "hits_per_s": n1 / (call_ms * 1e-3), "launches_per_call": launches,
            "binned_select_knn_ms": knn_ms, "accumulate_ms": acc_ms,
            "e2e_call_ms": host_ms, "e2e_hits_per_s": n1 / (host_ms * 1e-3),
            "note": "call = BinnedSelectKnn wrapper + AccumulateKnn ([mean | max]) on one event, device-timed back "
                    "to back; e2e = the host-buffer entry, wall clock per blocking call"}


def measure_other_configs(torch, dev, K, F, with_cpu):
    """Configurations 3 and 4 of the benchmark description, device-timed: the GravNet-style stack of
    four blocks on one 200k-hit event, and AssignToCondensates on 4 x 200k hits."""
    from hgcalml_b200 import synth
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn
    from hgcalml_b200.accknn_op import AccumulateKnn
    from hgcalml_b200.assign_condensate_op import BuildAndAssignCondensatesBinned
    out = {}
    n = 200000
    x0 = torch.as_tensor(np.random.default_rng(300).standard_normal((n, 64), dtype=np.float32), device=dev)
    rs = torch.tensor([0, n], dtype=torch.int32, device=dev)
    weights = [tuple(torch.as_tensor(w, device=dev) for w in synth.gravnet_weights(b)) for b in range(4)]

    def stack():
        x = x0
        for wc, wo in weights:
            coords = (x @ wc).contiguous()
            idx, d2, sorting = BinnedSelectKnn(64, coords, rs, return_sorting=True)
            acc, _ = AccumulateKnn(d2, x, idx, order=sorting, distance_scale=10., with_max_idxs=False)
            x = torch.relu(torch.cat([x, acc], dim=1) @ wo).contiguous()
        return x

    out["cfg3_gravnet_stack"] = {"ms": device_timed(torch, stack, 3), "hits": n, "blocks": 4,
                                 "note": "4 x (dense 64->4, BinnedSelectKnn K=64, AccumulateKnn F=64, dense 192->64 + "
                                         "ReLU); the dense layers are library GEMMs"}
    cc, beta, rsc = synth.condensation_batch(4, 200000, 500, 3, 0.1, seed=400)
    dist = np.full_like(beta, 0.5)
    t = [torch.as_tensor(v, device=dev) for v in (cc, beta, dist, rsc)]
    cfg4 = {"hits": int(len(cc)), "events": 4}
    for amb, tag in ((True, "max_beta"), (False, "min_distance")):
        res = BuildAndAssignCondensatesBinned(t[0], t[1], t[2], t[3], 0.1, assign_by_max_beta=amb)
        cfg4[tag] = {"wrapper_ms": device_timed(
            torch, lambda: BuildAndAssignCondensatesBinned(t[0], t[1], t[2], t[3], 0.1, assign_by_max_beta=amb), 5),
            "n_condensates": int(res[4][-1].item())}
        if with_cpu:
            cfg4[tag].update(cpu_condensates(cc, beta, dist, rsc, amb))
    out["cfg4_condensates"] = cfg4
    return out


def cpu_condensates(cc, beta, dist, rs, amb):
    """Configuration 4 through the reference's CPU op on one host core (part of the CPU baseline)."""
    O, backend, kind = _ref_backend()
    t0 = time.perf_counter()
    _, op_in, _ = O.BuildAndAssignCondensatesBinned(cc, beta, dist, rs, 0.1, assign_by_max_beta=amb,
                                                    return_op_io=True, backend=backend)
    wrapper = time.perf_counter() - t0
    t0 = time.perf_counter()
    O.op_binned_assign_to_condensates(**op_in, backend=backend)
    op = time.perf_counter() - t0
    return {"cpu_wrapper_ms": wrapper * 1e3, "cpu_op_ms": op * 1e3, "cpu_kind": kind, "cpu_cores": 1}


if __name__ == "__main__":
    main()
