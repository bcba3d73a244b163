#!/usr/bin/env python
"""Benchmark of the neighbor-search + KDE path (workload: 16 clouds x 100 000 surface points,
radius 0.05, KDE bandwidth 0.01) through the reference-shaped operator API.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = bounding boxes -> grid size -> keys -> stable sort (+ gathers) -> cell table ->
radius search (count, scan, store) -> KDE, for one batch of 16 clouds.  With N > 1 every rank
runs its own 16 clouds (clouds are independent, there is no collective on the data path) and
the reported value is the sum over ranks divided by the slowest rank's time.

Prints one JSON line.  `value` is measured with the inputs resident on the device; `e2e`
repeats the step with pinned host inputs copied in and the per-point results copied back inside
the timed region.  `--impl reference` times the CPU restatement of the reference algorithm
(oracle/, C + OpenMP, all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CLOUDS_PER_RANK = 16
POINTS_PER_CLOUD = 100000
RADIUS = 0.05
BANDWIDTH = 0.01
MAX_PAIRS_PER_CALL = (1 << 31) - 1  # int32 CSR offsets of the reference format


# ---- synthetic clouds --------------------------------------------------------------------------
def _rotation(rs):
    q, r = np.linalg.qr(rs.normal(size=(3, 3)))
    return q * np.sign(np.diag(r))


def surface_cloud(cloud_id, num_pts):
    """Points on the surfaces of 1-8 random primitives (sphere / box / plane patch, scale 0.1-0.5,
    centres in the unit cube) plus N(0, 0.002) jitter; seeded by the cloud id."""
    rs = np.random.RandomState(1000 + cloud_id)
    k = rs.randint(1, 9)
    kinds = rs.randint(0, 3, size=k)
    scales = rs.uniform(0.1, 0.5, size=k)
    centres = rs.uniform(0.0, 1.0, size=(k, 3))
    areas = np.where(kinds == 0, 4 * np.pi * scales ** 2, np.where(kinds == 1, 24 * scales ** 2, 4 * scales ** 2))
    counts = np.floor(areas / areas.sum() * num_pts).astype(np.int64)
    counts[np.argmax(counts)] += num_pts - counts.sum()
    parts = []
    for i in range(k):
        n, s = int(counts[i]), scales[i]
        if kinds[i] == 0:
            v = rs.normal(size=(n, 3))
            p = v / np.linalg.norm(v, axis=1, keepdims=True) * s
        elif kinds[i] == 1:
            p = rs.uniform(-s, s, size=(n, 3))
            axis = rs.randint(0, 3, size=n)
            p[np.arange(n), axis] = np.where(rs.rand(n) < 0.5, -s, s)
            p = p @ _rotation(rs).T
        else:
            p = np.concatenate([rs.uniform(-s, s, size=(n, 2)), np.zeros((n, 1))], 1) @ _rotation(rs).T
        parts.append(p + centres[i])
    pts = np.concatenate(parts, 0) + rs.normal(0.0, 0.002, size=(num_pts, 3))
    return pts.astype(np.float32)


def make_batch(first_cloud, num_clouds, num_pts=POINTS_PER_CLOUD):
    pts = np.concatenate([surface_cloud(first_cloud + i, num_pts) for i in range(num_clouds)], 0)
    batch_ids = np.repeat(np.arange(num_clouds, dtype=np.int32), num_pts)
    return pts, batch_ids


# ---- clocks -------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while a timed
    region runs."""
    BAD = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20}
    NOTED = {"sw_power_cap": 0x4}

    def __init__(self, device_index, period=0.02):
        super().__init__(daemon=True)
        self.period, self.samples, self.reasons, self.max_mhz = period, [], set(), None
        self._stop_evt = threading.Event()
        self.handle = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.handle = None

    def run(self):
        if self.handle is None:
            return
        while not self._stop_evt.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.handle, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for name, bit in list(self.BAD.items()) + list(self.NOTED.items()):
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def finish(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join()
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ---- the step on the GPU -----------------------------------------------------------------------
STAGES = ["bounding_box", "grid_size", "keys", "sort", "cell_table", "neighbors_count", "neighbors_store", "kde"]


class Step:
    """One pass of the hot path over one batch, through pccnn_lib_b200.ops, with a CUDA-event pair
    around every stage (recorded on the current stream, which is the stream the kernels run on)."""

    def __init__(self, num_batches, device):
        import torch
        from pccnn_lib_b200 import ops
        self.torch, self.ops = torch, ops
        self.num_batches = num_batches
        self.cell = torch.full((3,), RADIUS, dtype=torch.float32, device=device)
        self.bw = torch.full((3,), BANDWIDTH, dtype=torch.float32, device=device)
        self.events = []
        self.record = False

    def _mark(self):
        if not self.record:
            return None
        e = self.torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def run(self, pts, batch_ids):
        ops = self.ops
        marks = [self._mark()]
        mn, mx = ops.bounding_box(pts, batch_ids, self.num_batches)
        marks.append(self._mark())
        nc = ops.grid_num_cells(mn, mx, self.cell)
        marks.append(self._mark())
        keys = ops.compute_keys(pts, batch_ids, mn, nc, self.cell)
        marks.append(self._mark())
        skeys, sids, spts = ops.sort_keys(keys, 64, pts)
        marks.append(self._mark())
        shape = [self.num_batches] + nc[0:2].tolist() + [2]
        ds = ops.build_grid_ds(skeys, nc, shape)
        marks.append(self._mark())
        state = ops.find_neighbors_count(spts, skeys, spts, skeys, ds, nc, self.cell, 0)
        marks.append(self._mark())
        neigh, start_ids = ops.find_neighbors_store(state)
        marks.append(self._mark())
        pdf = ops.compute_pdf(3, self.bw, spts, neigh, start_ids)
        marks.append(self._mark())
        if self.record:
            self.events.append(marks)
        return pdf, start_ids, sids, neigh.shape[0]

    def stage_ms(self):
        """Mean duration of every stage over the recorded steps (call after a synchronize)."""
        out = {}
        for i, name in enumerate(STAGES):
            out[name] = float(np.mean([m[i].elapsed_time(m[i + 1]) for m in self.events]))
        return out


def split_for_int32(step, pts, batch_ids, num_clouds):
    """Largest equal split of the batch whose neighbor lists fit int32 offsets (the reference's
    CSR format): returns the list of (first_cloud, num_clouds) sub-batches."""
    import torch
    parts = 1
    while True:
        per = (num_clouds + parts - 1) // parts
        ok = True
        for first in range(0, num_clouds, per):
            sel = (batch_ids >= first) & (batch_ids < first + per)
            try:
                step.num_batches = min(per, num_clouds - first)
                step.run(pts[sel].contiguous(), (batch_ids[sel] - first).contiguous())
            except RuntimeError as e:
                if "int32" in str(e):
                    ok = False
                    break
                raise
        torch.cuda.synchronize()
        if ok:
            return [(first, min(per, num_clouds - first)) for first in range(0, num_clouds, per)]
        parts *= 2
        if parts > num_clouds:
            raise RuntimeError("a single cloud exceeds the int32 neighbor-list limit")


def run_b200(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    from pccnn_lib_b200 import _capi  # noqa: F401  (fails loudly if the CUDA library is missing)

    # Host data: this rank's clouds, in pinned memory for the end-to-end arm.
    h_pts, h_ids = make_batch(rank * CLOUDS_PER_RANK, CLOUDS_PER_RANK)
    hp = torch.from_numpy(h_pts).pin_memory()
    hb = torch.from_numpy(h_ids).pin_memory()
    d_pts, d_ids = hp.to(device), hb.to(device)

    step = Step(CLOUDS_PER_RANK, device)
    parts = split_for_int32(step, d_pts, d_ids, CLOUDS_PER_RANK)  # also the first warm-up pass
    subs = []
    for first, count in parts:
        sel = (d_ids >= first) & (d_ids < first + count)
        hsel = (hb >= first) & (hb < first + count)
        subs.append(dict(count=count, pts=d_pts[sel].contiguous(), ids=(d_ids[sel] - first).contiguous(),
                         h_pts=hp[hsel].contiguous().pin_memory(), h_ids=(hb[hsel] - first).contiguous().pin_memory()))

    def one_step(resident):
        pairs = 0
        for sub in subs:
            step.num_batches = sub["count"]
            if resident:
                pdf, start_ids, sids, t = step.run(sub["pts"], sub["ids"])
            else:
                p = sub["h_pts"].to(device, non_blocking=True)
                b = sub["h_ids"].to(device, non_blocking=True)
                pdf, start_ids, sids, t = step.run(p, b)
                sub["out_pdf"].copy_(pdf, non_blocking=True)
                sub["out_ends"].copy_(start_ids, non_blocking=True)
                sub["out_perm"].copy_(sids, non_blocking=True)
            pairs += t
        return pairs

    for sub in subs:
        n = sub["pts"].shape[0]
        sub["out_pdf"] = torch.empty((n,), dtype=torch.float32).pin_memory()
        sub["out_ends"] = torch.empty((n,), dtype=torch.int32).pin_memory()
        sub["out_perm"] = torch.empty((n,), dtype=torch.int64).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(resident, steps, warmup, sample_clocks):
        for _ in range(warmup):
            one_step(resident)
        step.events, step.record = [], resident
        barrier()
        sampler = ClockSampler(local_rank) if sample_clocks else None
        if sampler:
            sampler.start()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        pairs = 0
        for _ in range(steps):
            pairs += one_step(resident)
        t1.record()
        torch.cuda.synchronize()
        clocks = sampler.finish() if sampler else None
        barrier()
        step.record = False
        ms = t0.elapsed_time(t1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            p = torch.tensor([pairs], dtype=torch.float64, device=device)
            dist.all_reduce(p, op=dist.ReduceOp.SUM)
            pairs = float(p.item())
        return pairs, ms, clocks

    warm = max(args.warmup, 3)
    pairs, ms, clocks = timed(True, args.steps, warm, True)
    stage_ms = step.stage_ms()
    e_pairs, e_ms, _ = timed(False, args.steps, warm, False)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"

    n_pts = CLOUDS_PER_RANK * POINTS_PER_CLOUD
    t_rank = pairs / world / args.steps  # pairs of one step on one rank
    # Algorithmic bytes per launch: 8 B per pair written (store) / read (KDE) plus the per-point streams.
    algo = {
        "neighbors_store": 8.0 * t_rank + n_pts * (12 + 8 + 4),
        "neighbors_count": n_pts * (12 + 8 + 4),
        "kde": 8.0 * t_rank + n_pts * (12 + 4 + 4),
    }
    # every stage runs once per sub-batch; events bracket one sub-batch, so scale by their number
    n_sub = len(subs)
    dominant = max(("neighbors_count", "neighbors_store", "kde"), key=lambda k: stage_ms[k])
    dom_ms = stage_ms[dominant] * n_sub
    achieved = algo[dominant] / (dom_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": dominant, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "peak_source": peak_src, "traffic": None,
                "ms_per_launch_set": round(dom_ms, 4),
                "stage_ms": {k: round(v * n_sub, 4) for k, v in stage_ms.items()}}

    cpu = None if args.no_cpu else cpu_baseline_sample()

    h2d = sum(s["h_pts"].numel() * 4 + s["h_ids"].numel() * 4 for s in subs)
    d2h = sum(s["out_pdf"].numel() * 4 + s["out_ends"].numel() * 4 + s["out_perm"].numel() * 8 for s in subs)
    line = {
        "metric": "neighbor pairs/s (radius search + KDE)", "value": pairs / (ms * 1e-3), "unit": "pairs/s",
        "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32+i32/i64",
        "data": "synthetic",
        "config": {"workload": "neighbor search + KDE: %d clouds x 100k surface points per GPU, radius 0.05, "
                               "int32 CSR, fp32 KDE bandwidth 0.01" % CLOUDS_PER_RANK,
                   "clouds_per_gpu": CLOUDS_PER_RANK, "points_per_cloud": POINTS_PER_CLOUD,
                   "pairs_per_step_per_gpu": t_rank, "neighbors_per_point": t_rank / n_pts,
                   "sub_batches_for_int32_offsets": n_sub, "l2": "inputs larger than L2 (neighbor list)",
                   "library_kernels": "cub radix sort and scan"},
        "clocks": clocks,
        "e2e": {"value": e_pairs / (e_ms * 1e-3), "unit": "pairs/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e_ms / args.steps,
                "result": "per-point pdf, CSR end offsets and sort permutation copied to pinned host memory"},
        "gpu_launches": 12 * n_sub * args.steps,
        "roofline": roofline,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---- CPU arm ------------------------------------------------------------------------------------
def cpu_step(pts, batch_ids, num_clouds):
    """The same step on the CPU oracle.  Returns the number of neighbor pairs."""
    from oracle import oracle
    cell = np.full((3,), RADIUS, np.float32)
    g = oracle.build_grid(pts, batch_ids, num_clouds, cell)
    neigh, start_ids = oracle.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"],
                                             g["grid_ds"], g["num_cells"], cell, 0)
    oracle.compute_pdf(3, np.full((3,), BANDWIDTH, np.float32), g["sorted_pts"], neigh, start_ids)
    return neigh.shape[0]


def cpu_baseline_sample(num_clouds=None):
    num_clouds = num_clouds or CLOUDS_PER_RANK
    cores = len(os.sched_getaffinity(0))
    pts, ids = make_batch(0, num_clouds)
    t0 = time.perf_counter()
    pairs = cpu_step(pts, ids, num_clouds)
    dt = time.perf_counter() - t0
    return {"value": pairs / dt, "unit": "pairs/s", "cores": cores, "kind": "port",
            "sample": "one step over %d of the 16 clouds (%d points, %d pairs) in %.2f s, C + OpenMP restatement"
                      % (num_clouds, pts.shape[0], pairs, dt)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    num_clouds = 8  # half of the batch per step keeps the default run within a couple of minutes
    pts, ids = make_batch(0, num_clouds)
    for _ in range(max(args.warmup, 1)):
        cpu_step(pts, ids, num_clouds)
    t0 = time.perf_counter()
    pairs = 0
    for _ in range(args.steps):
        pairs += cpu_step(pts, ids, num_clouds)
    dt = time.perf_counter() - t0
    value = pairs / dt
    line = {
        "impl": "reference", "metric": "neighbor pairs/s (radius search + KDE)", "value": value, "unit": "pairs/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32+i32/i64", "data": "synthetic",
        "config": {"workload": "neighbor search + KDE: 16 clouds x 100k surface points per GPU, radius 0.05, "
                               "int32 CSR, fp32 KDE bandwidth 0.01",
                   "note": "the reference has no CPU implementation; this is the C + OpenMP restatement of its "
                           "algorithm on the host cores, each step a %d-cloud sample of the batch" % num_clouds},
        "cpu_baseline": {"value": value, "unit": "pairs/s", "cores": cores, "kind": "port",
                         "sample": "%d clouds x %d points per step" % (num_clouds, POINTS_PER_CLOUD)},
        "e2e": {"value": value, "unit": "pairs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--clouds", type=int, default=CLOUDS_PER_RANK,
                    help="clouds per GPU (default: the full workload; smaller values are for profiler captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiler captures)")
    args = ap.parse_args()
    globals()["CLOUDS_PER_RANK"] = args.clouds
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
