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
# DRAM bytes per neighbor pair of the three heavy kernels, from one ncu capture of a 6-cloud case
# (profiles/neighbors_kernel_pdf_kernel_6clouds_ncu.md); traffic grows in proportion to the pairs.
NCU_DRAM_BYTES_PER_PAIR = {"neighbors_store": 10.04, "neighbors_count": 0.11, "kde": 8.10}


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
        cells = nc.tolist()  # the one small device-to-host read the reference's wrapper also does
        key_bits = max(1, int(np.ceil(np.log2(float(self.num_batches) * cells[0] * cells[1] * cells[2] + 1))))
        skeys, sids, spts = ops.sort_keys(keys, key_bits, pts)
        marks.append(self._mark())
        shape = [self.num_batches] + cells[0:2] + [2]
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
    # Every rank draws the same 16 clouds, so per-GPU work is identical at every N (weak scaling).
    h_pts, h_ids = make_batch(0, CLOUDS_PER_RANK)
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

    # End-to-end arm: the inputs of every sub-batch come from pinned host memory and its results go back to
    # pinned host memory, every step, inside the timed region.  The copies run on two side streams so that the
    # upload of the next sub-batch and the download of the previous one overlap the kernels of the current one
    # (events order the hand-over between the streams; tensors stay referenced until their copies have run).
    copy_in, copy_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    pending = {"uploads": {}, "downloads": []}

    def upload(job):
        sub = subs[job % len(subs)]
        with torch.cuda.stream(copy_in):
            p = sub["h_pts"].to(device, non_blocking=True)
            b = sub["h_ids"].to(device, non_blocking=True)
            done = torch.cuda.Event()
            done.record(copy_in)
        pending["uploads"][job] = (p, b, done)

    def download(sub, pdf, start_ids, sids):
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(ready)
            sub["out_pdf"].copy_(pdf, non_blocking=True)
            sub["out_ends"].copy_(start_ids, non_blocking=True)
            sub["out_perm"].copy_(sids, non_blocking=True)
            done = torch.cuda.Event()
            done.record(copy_out)
        # the device tensors stay referenced until their copies have run
        pending["downloads"] = [d for d in pending["downloads"] if not d[0].query()] + [(done, pdf, start_ids, sids)]

    def one_step(resident, step_index=0, last=True):
        pairs = 0
        for si, sub in enumerate(subs):
            step.num_batches = sub["count"]
            if resident:
                pdf, start_ids, sids, t = step.run(sub["pts"], sub["ids"])
            else:
                job = step_index * len(subs) + si
                if job not in pending["uploads"]:
                    upload(job)
                p, b, done = pending["uploads"].pop(job)
                torch.cuda.current_stream().wait_event(done)
                p.record_stream(torch.cuda.current_stream())
                b.record_stream(torch.cuda.current_stream())
                if not (last and si == len(subs) - 1):
                    upload(job + 1)  # travels while this sub-batch is computed
                pdf, start_ids, sids, t = step.run(p, b)
                download(sub, pdf, start_ids, sids)
            pairs += t
        return pairs

    def drain():
        copy_out.synchronize()
        pending["downloads"] = []
        pending["uploads"] = {}

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
        for i in range(warmup):
            one_step(resident, i, i == warmup - 1)
        drain()
        step.events, step.record = [], resident
        barrier()
        sampler = ClockSampler(local_rank) if sample_clocks else None
        if sampler:
            sampler.start()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        pairs = 0
        for i in range(steps):
            pairs += one_step(resident, i, i == steps - 1)
        if not resident:
            torch.cuda.current_stream().wait_stream(copy_out)  # the last results are on the host before the clock stops
        t1.record()
        torch.cuda.synchronize()
        drain()
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
    local_pairs = one_step(True)  # this rank's pairs per step
    pairs, ms, clocks = timed(True, args.steps, warm, True)
    stage_ms = step.stage_ms()
    e_pairs, e_ms, _ = timed(False, args.steps, warm, False)
    # what reached the host through the pipelined copies is what a resident run computes
    step.num_batches = subs[-1]["count"]
    chk_pdf, chk_ends, chk_perm, _ = step.run(subs[-1]["pts"], subs[-1]["ids"])
    e2e_verified = bool(torch.equal(chk_pdf.cpu(), subs[-1]["out_pdf"]) and torch.equal(chk_ends.cpu(), subs[-1]["out_ends"])
                        and torch.equal(chk_perm.cpu(), subs[-1]["out_perm"]))

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"

    # Secondary number: the class-level route to the same density, Pointcloud.compute_pdf, which searches
    # within 4 bandwidths with at most 300 neighbors per point (pccnn_lib/pc/Pointcloud.py:81-109).
    import pccnn_lib_b200 as lib
    pc = lib.pc.Pointcloud(d_pts, d_ids)
    bw3 = np.full((3,), BANDWIDTH, np.float32)
    for _ in range(2):
        pc.compute_pdf(bw3)
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(3):
        pc.compute_pdf(bw3)
    c1.record()
    torch.cuda.synchronize()
    class_pdf_ms = c0.elapsed_time(c1) / 3

    n_pts = CLOUDS_PER_RANK * POINTS_PER_CLOUD
    t_rank = float(local_pairs)  # pairs of one step on this rank
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
                "frac": round(achieved / peak, 4), "peak_source": peak_src,
                "traffic": round(NCU_DRAM_BYTES_PER_PAIR[dominant] * t_rank), "algorithmic_bytes": round(algo[dominant]),
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
                   "pointcloud_compute_pdf_ms": round(class_pdf_ms, 3), "sub_batches_for_int32_offsets": n_sub, "l2": "inputs larger than L2 (neighbor list)",
                   "library_kernels": "cub radix sort and scan",
                   "sharding": "every rank processes its own batch of 16 clouds (same seeds on every rank); no collective on the data path"},
        "clocks": clocks,
        "e2e": {"value": e_pairs / (e_ms * 1e-3), "unit": "pairs/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e_ms / args.steps,
                "result": "per-point pdf, CSR end offsets and sort permutation copied to pinned host memory",
                "host_results_equal_resident_run": e2e_verified,
                "pipelining": "uploads of the next and downloads of the previous sub-batch overlap the kernels of the "
                              "current one (two copy streams); all copies inside the timed region"},
        "gpu_launches": 12 * n_sub * args.steps,
        "roofline": roofline,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---- convolution workloads (the other configurations of the baseline; run with --workload) ------
def scene_cloud(seed, num_pts):
    """Room-like scene: floor and four walls of a 20 x 20 x 3 m box plus 50-200 primitives resting
    on the floor, sampling density modulated 1-4x by a smooth field over (x, y)."""
    rs = np.random.RandomState(5000 + seed)
    parts = []
    n_struct = num_pts // 2
    per = n_struct // 5
    xy = rs.uniform(0, 20, size=(per, 2))
    parts.append(np.concatenate([xy, np.zeros((per, 1))], 1))
    for wall in range(4):
        u, h = rs.uniform(0, 20, size=(per, 1)), rs.uniform(0, 3, size=(per, 1))
        fixed = np.full((per, 1), 0.0 if wall % 2 == 0 else 20.0)
        parts.append(np.concatenate([u, fixed, h] if wall < 2 else [fixed, u, h], 1))
    k = rs.randint(50, 201)
    n_obj = num_pts - 5 * per
    counts = np.full(k, n_obj // k)
    counts[0] += n_obj - counts.sum()
    for i in range(k):
        s = rs.uniform(0.2, 1.5)
        c = np.array([rs.uniform(1, 19), rs.uniform(1, 19), s])
        v = rs.normal(size=(int(counts[i]), 3))
        if rs.rand() < 0.5:
            p = v / np.linalg.norm(v, axis=1, keepdims=True) * s
        else:
            p = rs.uniform(-s, s, size=(int(counts[i]), 3))
            ax = rs.randint(0, 3, size=int(counts[i]))
            p[np.arange(int(counts[i])), ax] = np.where(rs.rand(int(counts[i])) < 0.5, -s, s)
        parts.append(p + c)
    pts = np.concatenate(parts, 0)
    # density field: keep a point with probability field/4, then resample to the requested size
    field = 2.5 + 1.5 * np.sin(pts[:, 0] * 0.3) * np.cos(pts[:, 1] * 0.3)
    keep = rs.rand(pts.shape[0]) < field / 4.0
    pts = pts[keep]
    pts = pts[rs.randint(0, pts.shape[0], size=num_pts)] + rs.normal(0, 0.004, size=(num_pts, 3))
    return pts.astype(np.float32)


CONV_WORKLOADS = {
    # name: (description, builder kwargs)
    "kpconv_cfg0": dict(desc="KPConv single layer forward: 1 cloud x 4096 uniform points, Cin 16, Cout 32, 16 kernel "
                             "points, radius 0.1", kind="kp", clouds=1, pts=4096, gen="cube", radius=0.1, cin=16,
                        cout=32, k=16, backward=False, pool=None),
    "mcconv_cfg2": dict(desc="MCConv forward+backward: 32 clouds x 32768 surface points, outputs Poisson-disk radius "
                             "0.03, conv radius 0.075, Cin 64, Cout 128, hidden 16, pdf bandwidth 0.015", kind="mc",
                        clouds=32, pts=32768, gen="surface", radius=0.075, cin=64, cout=128, k=16, backward=True,
                        pool=0.03, bw=0.015),
    "kpconv_scene": dict(desc="KPConv forward+backward on one room-like scene of 2M points, radius 0.1 m, Cin 128, "
                              "Cout 128, 16 kernel points (one GPU's share of the large-scene configuration)",
                         kind="kp", clouds=1, pts=2000000, gen="scene", radius=0.1, cin=128, cout=128, k=16,
                         backward=True, pool=None),
    "mcconv_scene": dict(desc="MCConv forward+backward on one room-like scene of 2M points, radius 0.1 m, Cin 128, "
                              "Cout 128, hidden 16, pdf bandwidth 0.02 m", kind="mc", clouds=1, pts=2000000,
                         gen="scene", radius=0.1, cin=128, cout=128, k=16, backward=True, pool=None, bw=0.02),
}


def run_conv_workload(args):
    import torch
    import pccnn_lib_b200 as lib
    from pccnn_lib_b200 import ops
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    w = dict(CONV_WORKLOADS[args.workload])
    if args.points:
        w["pts"] = args.points  # smaller instance of the same workload, for profiler captures
        w["desc"] += " [reduced to %d points per cloud]" % args.points
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    rs = np.random.RandomState(77)
    if w["gen"] == "cube":
        pts = np.random.RandomState(1000).rand(w["pts"], 3).astype(np.float32)
        ids = np.zeros(w["pts"], np.int32)
    elif w["gen"] == "surface":
        pts, ids = make_batch(0, w["clouds"], w["pts"])
    else:
        pts, ids = scene_cloud(0, w["pts"]), np.zeros(w["pts"], np.int32)
    radius = np.full((3,), w["radius"], np.float32)
    if args.presort:
        # store the cloud in grid-cell order (what a spatially coherent scan or a previous pooling
        # stage would deliver); neighbor rows of nearby samples then hit in L2
        tmp = lib.pc.Pointcloud(pts, ids, device=device)
        g0 = lib.pc.Grid(tmp, lib.pc.BoundingBox(tmp), radius)
        g0.compute_cell_ids()
        order = g0.sorted_ids_.cpu().numpy()
        pts, ids = np.ascontiguousarray(pts[order]), np.ascontiguousarray(ids[order])
    pc = lib.pc.Pointcloud(pts, ids, device=device)
    t0 = time.perf_counter()
    pc_out = pc
    if w["pool"]:
        pool = lib.pc.PointPooling(pc, np.full((3,), w["pool"], np.float32))
        pc_out = lib.pc.Pointcloud(pool.pool_tensor(pc.pts_), pool.pool_tensor(pc.batch_ids_))
    bb = lib.pc.BoundingBox(pc)
    grid = lib.pc.Grid(pc, bb, radius)
    grid.compute_cell_ids()
    grid.build_ds()
    nb = lib.pc.Neighborhood(grid, pc_out, 0)
    pdf = None
    if w["kind"] == "mc":
        pc.compute_pdf(np.full((3,), w["bw"], np.float32))
        pdf = (pc.pts_unnorm_pdf_ * float(np.prod(radius))).contiguous()
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t0
    n, m, t = pts.shape[0], pc_out.pts_.shape[0], nb.neighbors_.shape[0]
    cin, cout, k = w["cin"], w["cout"], w["k"]
    feats = torch.as_tensor(rs.normal(size=(n, cin)).astype(np.float32), device=device)
    rad = torch.as_tensor(radius, device=device)
    grads = torch.as_tensor(rs.normal(size=(m, cout)).astype(np.float32), device=device)
    if args.impl == "reference_gpu":
        import importlib.util
        so = os.path.join(ROOT, "oracle", "_ref", "pccnn_lib_ops.so")
        if not os.path.exists(so):
            print(json.dumps({"impl": "reference_gpu", "unavailable": "oracle/_ref/pccnn_lib_ops.so has not been built"}))
            return
        spec = importlib.util.spec_from_file_location("pccnn_lib_ops", so)
        ops = importlib.util.module_from_spec(spec)  # the reference's operators under the same names
        spec.loader.exec_module(ops)
    if w["kind"] == "kp":
        kp, sigma = prepare_kernel_points(3, k)
        kpts = torch.as_tensor(kp, device=device)
        weights = torch.as_tensor(rs.normal(0, np.sqrt(1.0 / (15 * cin)), size=(k * cin, cout)).astype(np.float32), device=device)
        fwd = lambda: ops.kp_conv(pc.pts_, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, rad, kpts, sigma, weights)
        bwd = lambda: ops.kp_conv_grads(pc.pts_, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, rad, kpts, sigma, weights, grads)
    else:
        axis = torch.as_tensor(rs.normal(0, np.sqrt(1 / 3.0), size=(3, k)).astype(np.float32), device=device)
        bias = torch.zeros((1, k), dtype=torch.float32, device=device)
        weights = torch.as_tensor(rs.normal(0, np.sqrt(1.0 / (cin * k)), size=(1, k * cin, cout)).astype(np.float32), device=device)
        fwd = lambda: ops.mc_conv(pc.pts_, pdf, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, rad, axis, bias, weights)
        bwd = lambda: ops.mc_conv_grads(pc.pts_, pdf, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, rad, axis, bias, weights, grads)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    warm = max(args.warmup, 3)
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    fwd_ms = timed(fwd, args.steps, warm)
    bwd_ms = timed(bwd, args.steps, warm) if w["backward"] else 0.0
    clocks = sampler.finish()
    if args.impl == "reference_gpu":
        step_ms = fwd_ms + bwd_ms
        print(json.dumps({"impl": "reference_gpu", "metric": "conv-layer points/s", "value": m / (step_ms * 1e-3),
                          "unit": "points/s", "ms_per_step": step_ms, "clocks": clocks,
                          "config": {"workload": w["desc"], "forward_ms": fwd_ms, "backward_ms": bwd_ms, "samples": m,
                                     "pairs": t, "note": "unmodified reference kernels + cuBLAS, built for sm_100"}}))
        return
    # the contraction alone, on the same shapes, for the tensor-core roofline
    from pccnn_lib_b200 import ops
    inner = cin * k
    rows = min(m, 1 << 17)
    kpad = (inner + 63) // 64 * 64
    a32 = torch.randn(rows, kpad, device=device)
    b32 = torch.randn(cout, kpad, device=device)
    a_hi, b_hi = a32.to(torch.bfloat16), b32.to(torch.bfloat16)
    a_lo, b_lo = (a32 - a_hi.float()).to(torch.bfloat16), (b32 - b_hi.float()).to(torch.bfloat16)
    c_out = torch.empty((rows, cout), dtype=torch.float32, device=device)
    st = torch.zeros((1,), dtype=torch.int32, device=device)
    gemm_ms = timed(lambda: ops.gemm_bf16(a_hi, b_hi, a_lo, b_lo, out=c_out, status=st), max(args.steps, 20), warm)
    assert int(st.item()) == 0
    # three bf16 products per output element are executed; all of them are counted as tensor-core work
    flops = 2.0 * rows * kpad * cout * 3
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    tc_peak = float(json.load(open(peaks_path))["bf16_tflops"]) if os.path.exists(peaks_path) else 1590.0
    step_ms = fwd_ms + bwd_ms
    line = {
        "metric": "conv-layer points/s (%s)" % ("forward+backward" if w["backward"] else "forward"),
        "value": m / (step_ms * 1e-3), "unit": "points/s", "n_gpus": 1, "steps": args.steps, "warmup": warm,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (bf16 hi/lo split on tensor cores, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": w["desc"], "point_order": "grid-cell order" if args.presort else "random", "points": n, "samples": m, "pairs": t, "neighbors_per_sample": t / max(m, 1),
                   "forward_ms": fwd_ms, "backward_ms": bwd_ms, "setup_s_untimed": setup_s,
                   "useful_contraction_flop_per_step": 2.0 * m * inner * cout * (3 if w["backward"] else 1),
                   "projection_flop_per_step": 2.0 * t * inner * (2 if w["backward"] else 1)},
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "gemm_bf16_kernel<BN, split> alone (three bf16 products per element, all counted)",
                     "achieved": round(flops / (gemm_ms * 1e-3) / 1e12, 2), "peak": tc_peak, "unit": "TFLOP/s",
                     "frac": round(flops / (gemm_ms * 1e-3) / 1e12 / tc_peak, 4), "traffic": None,
                     "rows": int(rows), "inner": int(kpad), "cols": int(cout), "ms": gemm_ms,
                     "useful_fp32_equivalent_tflops": round(flops / 3 / (gemm_ms * 1e-3) / 1e12, 2)},
    }
    # CPU baseline for the layer-sized forward workload: the torch composition that mirrors the reference's
    # ATen host code (index_select, broadcast ops, index_add_, matmul) on all host cores, float32.
    if w["kind"] == "kp" and not w["backward"] and t * k * cin <= (1 << 28) and not args.no_cpu:
        from oracle import conv_oracle
        host = [x.cpu() for x in (pc.pts_, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, rad, kpts, weights)]
        conv_oracle.kp_conv(host[0], host[1], host[2], host[3], host[4], host[5], host[6], sigma, host[7], dtype=torch.float32)
        reps, c0 = 5, time.perf_counter()
        for _ in range(reps):
            conv_oracle.kp_conv(host[0], host[1], host[2], host[3], host[4], host[5], host[6], sigma, host[7],
                                dtype=torch.float32)
        cpu_s = (time.perf_counter() - c0) / reps
        line["cpu_baseline"] = {"value": m / cpu_s, "unit": "points/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": "the whole layer, %d forward passes of the torch-CPU restatement, %.2f ms each"
                                          % (reps, cpu_s * 1e3)}
    print(json.dumps(line))


def run_pooling_workload(args):
    """Poisson-disk pooling of the encoder's first level (64 clouds x 50k surface points, radius 0.02), both routes:
    the reference's pair of operators (full self-neighborhood, then the list-based sampling) and the list-free
    sampling on the grid.  One step = grid front end + sampling; the two selections are compared."""
    import torch
    from pccnn_lib_b200 import ops
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    clouds = args.clouds if args.clouds != CLOUDS_PER_RANK else 64
    pts, ids = make_batch(0, clouds, args.points or 50000)
    d_pts, d_ids = torch.as_tensor(pts, device=device), torch.as_tensor(ids, device=device)
    cell = torch.full((3,), 0.02, dtype=torch.float32, device=device)

    def event():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    rows = []
    for i in range(max(args.warmup, 3) + args.steps):
        m = [event()]
        g = ops.grid_front_end(d_pts, d_ids, clouds, cell)
        m.append(event())
        nb, st = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"], g["grid_ds"],
                                    g["num_cells"], cell, 0)
        m.append(event())
        by_list = ops.poisson_disk_sampling(g["sorted_keys"], nb, st, g["num_cells"])
        m.append(event())
        by_grid = ops.poisson_disk_sampling_grid(g["sorted_pts"], g["sorted_keys"], g["grid_ds"], g["num_cells"], cell)
        m.append(event())
        torch.cuda.synchronize()
        if i >= max(args.warmup, 3):
            rows.append([m[j].elapsed_time(m[j + 1]) for j in range(4)])
    same = bool(torch.equal(by_list, by_grid))
    front, search, listed, gridded = [float(np.mean([r[j] for r in rows])) for j in range(4)]
    print(json.dumps({
        "metric": "pooled points/s (Poisson-disk pooling, list-free route)", "value": pts.shape[0] / ((front + gridded) * 1e-3),
        "unit": "points/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": front + gridded,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32+i32/i64", "data": "synthetic",
        "config": {"workload": run_pooling_workload.__doc__.split("\n")[0], "points": int(pts.shape[0]),
                   "pairs_of_the_self_neighborhood": int(nb.shape[0]), "selected": int(by_grid.shape[0]),
                   "grid_front_end_ms": front, "search_ms": search, "list_based_sampling_ms": listed,
                   "list_free_sampling_ms": gridded, "selections_identical": same}}))


def run_encoder_workload(args):
    """KPConv 5-level encoder, inference, bf16 features and weights with fp32 accumulation: 64 clouds x 50k
    surface points, Poisson-disk radii 0.02 ... 0.32, convolution radius 2.5 x the sampling radius, channels
    3-64-128-256-512-1024, 16 kernel points.  No normalisation or activation between levels (the reference
    ships no model).  One step = all poolings, neighborhoods and convolutions of the five levels."""
    import torch
    import pccnn_lib_b200 as lib
    from pccnn_lib_b200 import ops
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    clouds = args.clouds if args.clouds != CLOUDS_PER_RANK or args.clouds == 64 else 64
    num_pts = args.points or 50000
    pts, ids = make_batch(0, clouds, num_pts)
    rs = np.random.RandomState(3)
    channels = [3, 64, 128, 256, 512, 1024]
    kp, sigma = prepare_kernel_points(3, 16)
    kpts = torch.as_tensor(kp, device=device)
    weights = [torch.as_tensor(rs.normal(0, np.sqrt(2.0 / (channels[l] * 16)), size=(16 * channels[l], channels[l + 1]))
                               .astype(np.float32), device=device).to(torch.bfloat16) for l in range(5)]
    feats0 = torch.as_tensor(rs.normal(size=(pts.shape[0], 3)).astype(np.float32), device=device).to(torch.bfloat16)
    d_pts, d_ids = torch.as_tensor(pts, device=device), torch.as_tensor(ids, device=device)
    stats = {}

    def step(record=False):
        pc, feats = lib.pc.Pointcloud(d_pts, d_ids), feats0
        conv_ms, geo = [], []
        for level in range(5):
            r_pool = 0.02 * (2 ** level)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
            pool = lib.pc.PointPooling(pc, np.full((3,), r_pool, np.float32))
            pc_out = lib.pc.Pointcloud(pool.pool_tensor(pc.pts_), pool.pool_tensor(pc.batch_ids_))
            ev[1].record()
            radius = torch.full((3,), 2.5 * r_pool, dtype=torch.float32, device=device)
            grid = lib.pc.Grid(pc, lib.pc.BoundingBox(pc), radius)
            grid.compute_cell_ids()
            grid.build_ds()
            nb = lib.pc.Neighborhood(grid, pc_out, 0)
            ev[2].record()
            geo.append(ev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            feats = ops.kp_conv(pc.pts_, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, radius, kpts, sigma,
                                weights[level])
            e1.record()
            if record:
                stats.setdefault("levels", []).append(dict(points=int(pc.pts_.shape[0]), samples=int(pc_out.pts_.shape[0]),
                                                           pairs=int(nb.neighbors_.shape[0])))
            conv_ms.append((e0, e1))
            pc = pc_out
        return feats, (conv_ms, geo)

    step(record=True)
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    marks = []
    for _ in range(args.steps):
        out, conv_ms = step()
        marks.append(conv_ms)
    t1.record()
    torch.cuda.synchronize()
    clocks = sampler.finish()
    ms = t0.elapsed_time(t1) / args.steps
    conv = [float(np.mean([m[0][l][0].elapsed_time(m[0][l][1]) for m in marks])) for l in range(5)]
    pooling = [float(np.mean([m[1][l][0].elapsed_time(m[1][l][1]) for m in marks])) for l in range(5)]
    neighborhoods = [float(np.mean([m[1][l][1].elapsed_time(m[1][l][2]) for m in marks])) for l in range(5)]
    flops = sum(2.0 * lv["samples"] * 16 * channels[l] * channels[l + 1] for l, lv in enumerate(stats["levels"]))
    print(json.dumps({
        "metric": "conv-layer points/s (5-level KPConv encoder, inference)", "value": pts.shape[0] / (ms * 1e-3),
        "unit": "points/s", "n_gpus": 1, "steps": args.steps, "warmup": warm, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": run_encoder_workload.__doc__.split("  One step")[0].replace("\n    ", " "),
                   "clouds": clouds, "points_per_cloud": num_pts, "levels": stats["levels"], "conv_ms_per_level": conv,
                   "conv_ms_total": sum(conv), "geometry_ms": ms - sum(conv),
                   "pooling_ms_per_level": pooling, "neighborhood_ms_per_level": neighborhoods, "contraction_flop_per_step": flops,
                   "finite_output": bool(torch.isfinite(out.float()).all())},
        "clocks": clocks}))


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
    from oracle import oracle
    num_clouds = num_clouds or CLOUDS_PER_RANK
    cores = oracle.set_threads(len(os.sched_getaffinity(0)))  # a launcher may have capped OMP_NUM_THREADS
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
    from oracle import oracle
    cores = oracle.set_threads(len(os.sched_getaffinity(0)))  # a launcher may have capped OMP_NUM_THREADS
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


def run_reference_gpu(args):
    """Second comparator: the reference's own (generic SIMT) kernels, compiled unmodified for sm_100 by
    oracle/build_reference.py, on the same workload and GPU.  Not the contract's reference arm (that
    one is the CPU); printed with impl = "reference_gpu"."""
    import importlib.util
    import torch
    so = os.path.join(ROOT, "oracle", "_ref", "pccnn_lib_ops.so")
    if not os.path.exists(so):
        print(json.dumps({"impl": "reference_gpu", "unavailable": "oracle/_ref/pccnn_lib_ops.so has not been built"}))
        return
    spec = importlib.util.spec_from_file_location("pccnn_lib_ops", so)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    device = torch.device("cuda", 0)
    pts_h, ids_h = make_batch(0, CLOUDS_PER_RANK)
    pts, ids = torch.as_tensor(pts_h, device=device), torch.as_tensor(ids_h, device=device)
    cell = torch.full((3,), RADIUS, dtype=torch.float32, device=device)
    bw = torch.full((3,), BANDWIDTH, dtype=torch.float32, device=device)

    def step():
        # the caller-side code of the reference (pc/BoundingBox.py, pc/Grid.py, pc/Neighborhood.py) with torch ops
        idx = ids.to(torch.int64).unsqueeze(1).expand(-1, 3)
        mx = torch.full((CLOUDS_PER_RANK, 3), -float("inf"), device=device).scatter_reduce(0, idx, pts, "amax") + 1e-6
        mn = torch.full((CLOUDS_PER_RANK, 3), float("inf"), device=device).scatter_reduce(0, idx, pts, "amin") - 1e-6
        nc = torch.max(((mx - mn) / cell).to(torch.int32) + 1, dim=0)[0]
        keys = ref.compute_keys(pts, ids, mn, nc, cell)
        order = torch.argsort(keys)
        skeys = torch.index_select(keys, 0, order)
        spts = torch.index_select(pts, 0, order)
        ds = ref.build_grid_ds(skeys, nc, [CLOUDS_PER_RANK] + nc[0:2].tolist() + [2])
        neigh, ends = ref.find_neighbors(spts, skeys, spts, skeys, ds, nc, cell, 0)
        pdf = ref.compute_pdf(3, bw, spts, neigh, ends)
        return neigh.shape[0], pdf

    for _ in range(max(args.warmup, 1)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pairs = 0
    for _ in range(args.steps):
        pairs += step()[0]
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    print(json.dumps({"impl": "reference_gpu", "metric": "neighbor pairs/s (radius search + KDE)",
                      "value": pairs / (ms * 1e-3), "unit": "pairs/s", "n_gpus": 1, "steps": args.steps,
                      "ms_per_step": ms / args.steps, "higher_is_better": True,
                      "config": {"workload": "neighbor search + KDE: %d clouds x 100k surface points, radius 0.05"
                                             % CLOUDS_PER_RANK,
                                 "note": "unmodified reference kernels built for sm_100 (generic SIMT), torch ops for "
                                         "bbox / argsort / gathers as in the reference's Python classes"}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference_gpu"])
    ap.add_argument("--clouds", type=int, default=CLOUDS_PER_RANK,
                    help="clouds per GPU (default: the full workload; smaller values are for profiler captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiler captures)")
    ap.add_argument("--points", type=int, default=0,
                    help="convolution workloads: points per cloud (default: the workload's own size)")
    ap.add_argument("--presort", action="store_true",
                    help="convolution workloads: store the points in grid-cell order instead of random order")
    ap.add_argument("--workload", default="neighbors_kde", choices=["neighbors_kde", "kpconv_encoder_cfg3", "pooling_cfg3_level1"] + sorted(CONV_WORKLOADS),
                    help="neighbors_kde is the headline workload; the others time one convolution layer")
    args = ap.parse_args()
    globals()["CLOUDS_PER_RANK"] = args.clouds
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference_gpu" and args.workload != "neighbors_kde":
        run_conv_workload(args)
    elif args.impl == "reference_gpu":
        run_reference_gpu(args)
    elif args.workload == "pooling_cfg3_level1":
        run_pooling_workload(args)
    elif args.workload == "kpconv_encoder_cfg3":
        run_encoder_workload(args)
    elif args.workload != "neighbors_kde":
        run_conv_workload(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
