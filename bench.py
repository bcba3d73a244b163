#!/usr/bin/env python
"""Benchmark of the point-convolution hot path through the reference-shaped operator API.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference|reference_gpu] [--workload NAME]

Headline (the JSON line's `value`): neighbor search + KDE on 16 clouds x 100 000 surface points per GPU, radius
0.05, KDE bandwidth 0.01.  One step = bounding boxes -> grid size -> keys -> stable sort (+ gathers) -> cell table
-> radius search (count, scan, store) -> KDE for one batch.  With N GPUs the batch is 16 N distinct clouds
(every 16 consecutive ids hold the same mix of primitives, drawn anew), dealt to the ranks by an estimate of their
neighbor pairs (clouds are independent: no collective on the data path); the value is all pairs divided by the
slowest rank's time.

The same line carries, under `secondary`, the convolution configurations (conv-layer points/s): the single-layer
KPConv forward on 4096 points, MCConv forward+backward on 32 x 32k points with Poisson-disk pooled outputs, the
5-level bf16 KPConv encoder on 64 x 50k points, and a KPConv+MCConv layer pair forward+backward on a 2M-point
scene per GPU -- each with its own CUDA-event time, clocks, an end-to-end figure from pinned host memory, a
layer-level tensor-core roofline and a CPU baseline on a stated sample.  With N > 1 the batches are split by cloud
(the scene configuration runs one scene per GPU) and the backward configurations sum their parameter gradients with
NCCL on a side stream that starts as soon as the weight gradient is final.

`--impl reference` times the CPU restatement of the reference algorithm (oracle/, C + OpenMP, all host threads) on
the headline configuration.  `--workload NAME` runs one configuration alone (profiler captures).
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
CLOUDS_PER_RANK_DEFAULT = 16  # the surface sampler repeats its recipes with this period (not changed by --clouds)
POINTS_PER_CLOUD = 100000
RADIUS = 0.05
BANDWIDTH = 0.01
# DRAM bytes per neighbor pair of the heavy kernels, from one ncu capture of a 6-cloud case of this workload
# (dram__bytes_read.sum + dram__bytes_write.sum per launch, divided by the pairs of that launch); the traffic of
# these kernels grows in proportion to the pairs.
NCU_DRAM_BYTES_PER_PAIR = {"neighbors_store": 10.04, "neighbors_count": 0.11, "neighbors": 8.2, "kde": 8.10}


# ---- synthetic clouds --------------------------------------------------------------------------
def _rotation(rs):
    q, r = np.linalg.qr(rs.normal(size=(3, 3)))
    return q * np.sign(np.diag(r))


def surface_cloud(cloud_id, num_pts):
    """Points on the surfaces of 1-8 random primitives (sphere / box / plane patch, scale 0.1-0.5,
    centres in the unit cube) plus N(0, 0.002) jitter; seeded by the cloud id.  Clouds 16 and up repeat the
    primitives of cloud (id mod 16) with points, orientations and jitter drawn anew, so that every 16 consecutive
    clouds -- what one GPU gets under weak scaling -- hold the same mix of sparse and dense clouds."""
    rs = np.random.RandomState(1000 + cloud_id % CLOUDS_PER_RANK_DEFAULT)
    k = rs.randint(1, 9)
    kinds = rs.randint(0, 3, size=k)
    scales = rs.uniform(0.1, 0.5, size=k)
    centres = rs.uniform(0.0, 1.0, size=(k, 3))
    if cloud_id >= CLOUDS_PER_RANK_DEFAULT:
        rs = np.random.RandomState(1000 + cloud_id)
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


def make_batch(first_cloud, num_clouds, num_pts=POINTS_PER_CLOUD, cloud_ids=None):
    """Clouds first_cloud ... first_cloud + num_clouds - 1 of the surface sampler (or the listed cloud ids) as one
    batch with batch ids 0 ... num_clouds - 1."""
    cloud_ids = list(range(first_cloud, first_cloud + num_clouds)) if cloud_ids is None else list(cloud_ids)
    pts = np.concatenate([surface_cloud(c, num_pts) for c in cloud_ids], 0)
    batch_ids = np.repeat(np.arange(len(cloud_ids), dtype=np.int32), num_pts)
    return pts, batch_ids


def estimate_pairs(cloud_id, num_pts=POINTS_PER_CLOUD, radius=RADIUS, probe=10000):
    """Neighbor pairs a cloud of the surface sampler will produce at `num_pts` points, estimated from a
    `probe`-point draw of the same cloud: pairs ~ sum over cells of n_cell * (points in the 27-cell stencil) *
    (ball volume / stencil volume), scaled by (num_pts / probe)^2.  Used to balance the partition of a batch."""
    p = surface_cloud(cloud_id, probe)
    c = np.floor((p - p.min(0)) / radius).astype(np.int64) + 1
    dims = c.max(0) + 2
    hist = np.zeros(dims, np.float64)
    np.add.at(hist, (c[:, 0], c[:, 1], c[:, 2]), 1.0)
    box = np.zeros_like(hist)
    for dx in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dz in (-1, 0, 1):
                box += np.roll(hist, (dx, dy, dz), axis=(0, 1, 2))
    return float((hist * box).sum() * (4.0 / 3.0 * np.pi / 27.0) * (num_pts / float(probe)) ** 2)


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


# ---- clocks, peaks, ranks -----------------------------------------------------------------------
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


def measured_peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, source) from the file the harness measured on this pool, else the stated
    fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def bind_to_gpu_numa_node(device_index):
    """Restricts this process to the CPUs next to its GPU (the PCI device's local_cpulist), so that the pinned
    host buffers it allocates afterwards are first touched, and therefore placed, on that NUMA node.  Best effort:
    returns the CPU count used, or None when the topology cannot be read."""
    try:
        import torch
        props = torch.cuda.get_device_properties(device_index)
        bus = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        text = open("/sys/bus/pci/devices/%s/local_cpulist" % bus).read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return len(allowed)
    except Exception:
        return None


class Ranks(object):
    """One process per GPU (torchrun); every collective used by the bench itself lives here."""

    def __init__(self):
        import torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        self.numa_cpus = bind_to_gpu_numa_node(self.local_rank) if self.world > 1 else None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.device)

    def barrier(self):
        import torch
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def _reduce(self, value, op):
        if self.world == 1:
            return float(value)
        import torch
        import torch.distributed as dist
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=getattr(dist.ReduceOp, op))
        return float(t.item())

    def max(self, value):
        return self._reduce(value, "MAX")

    def sum(self, value):
        return self._reduce(value, "SUM")

    def gather(self, value):
        if self.world == 1:
            return [float(value)]
        import torch
        import torch.distributed as dist
        t = torch.zeros((self.world,), dtype=torch.float64, device=self.device)
        t[self.rank] = float(value)
        dist.all_reduce(t)
        return [float(v) for v in t.tolist()]

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


def device_timed(fn, steps, warmup, ranks=None, clocks_device=None):
    """Mean milliseconds of fn() over `steps` calls after `warmup` untimed ones, CUDA events on the current stream,
    a barrier + synchronize on both sides, the maximum over the ranks.  Returns (ms, clocks or None)."""
    import torch
    for _ in range(warmup):
        fn()
    if ranks is not None:
        ranks.barrier()
    else:
        torch.cuda.synchronize()
    sampler = ClockSampler(clocks_device) if clocks_device is not None else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.finish() if sampler else None
    ms = e0.elapsed_time(e1) / steps
    if ranks is not None:
        ranks.barrier()
        ms = ranks.max(ms)
    return ms, clocks


# ---- headline: neighbor search + KDE ---------------------------------------------------------------
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
        self.keep = None  # (sorted points, neighbor list, ends) of the last run, when asked for

    def _mark(self):
        if not self.record:
            return None
        e = self.torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def run(self, pts, batch_ids, keep=False):
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
        self.keep = (spts, neigh, start_ids) if keep else None
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


def list_checksum(neighbors):
    """Order-sensitive 64-bit checksum of a [T, 2] int32 list (wrap-around arithmetic): the same on a numpy
    array and on a CUDA tensor."""
    import torch
    if isinstance(neighbors, np.ndarray):
        t = neighbors.shape[0]
        with np.errstate(over="ignore"):
            w = (np.arange(t, dtype=np.uint64) % np.uint64(65521)) + np.uint64(1)
            v = neighbors[:, 0].astype(np.uint64) * np.uint64(1000003) + neighbors[:, 1].astype(np.uint64)
            return int((v * w).sum(dtype=np.uint64))
    t = neighbors.shape[0]
    w = (torch.arange(t, dtype=torch.int64, device=neighbors.device) % 65521) + 1
    v = neighbors[:, 0].to(torch.int64) * 1000003 + neighbors[:, 1].to(torch.int64)
    return int((v * w).sum().item()) & 0xFFFFFFFFFFFFFFFF


def run_neighbors_kde(args, R):
    """The headline workload.  Returns the JSON line as a dict on rank 0 (None elsewhere)."""
    import torch
    from pccnn_lib_b200 import parallel
    device = R.device

    # The global batch of 16 N clouds, dealt to the ranks by estimated pairs; this rank's clouds on the host
    # (pinned, for the end-to-end arm) and on the device.
    total_clouds = CLOUDS_PER_RANK * R.world
    if R.world > 1:
        weights = [estimate_pairs(c) for c in range(total_clouds)]
        cloud_ids = parallel.assign_clouds(weights, R.world)[R.rank]
    else:
        cloud_ids = list(range(total_clouds))
    my_clouds = len(cloud_ids)
    h_pts, h_ids = make_batch(0, 0, cloud_ids=cloud_ids)
    hp = torch.from_numpy(h_pts).pin_memory()
    hb = torch.from_numpy(h_ids).pin_memory()
    d_pts, d_ids = hp.to(device), hb.to(device)

    step = Step(my_clouds, device)
    parts = split_for_int32(step, d_pts, d_ids, my_clouds)  # also the first warm-up pass
    subs = []
    for first, count in parts:
        sel = (d_ids >= first) & (d_ids < first + count)
        hsel = (hb >= first) & (hb < first + count)
        subs.append(dict(first=first, count=count, pts=d_pts[sel].contiguous(), ids=(d_ids[sel] - first).contiguous(),
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

    def timed(resident, steps, warmup, sample_clocks):
        for i in range(warmup):
            one_step(resident, i, i == warmup - 1)
        drain()
        step.events, step.record = [], resident
        R.barrier()
        sampler = ClockSampler(R.local_rank) if sample_clocks else None
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
        R.barrier()
        step.record = False
        my_ms = t0.elapsed_time(t1)
        return R.sum(pairs), R.max(my_ms), clocks, my_ms

    warm = max(args.warmup, 3)
    local_pairs = one_step(True)  # this rank's pairs per step
    pairs, ms, clocks, my_ms = timed(True, args.steps, warm, True)
    stage_ms = step.stage_ms()
    e_pairs, e_ms, _, my_e_ms = timed(False, args.steps, warm, False)
    rank_ms = R.gather(my_ms / args.steps)
    rank_pairs = R.gather(local_pairs)
    # what reached the host through the pipelined copies is what a resident run computes
    step.num_batches = subs[-1]["count"]
    chk_pdf, chk_ends, chk_perm, _ = step.run(subs[-1]["pts"], subs[-1]["ids"])
    e2e_verified = bool(torch.equal(chk_pdf.cpu(), subs[-1]["out_pdf"]) and torch.equal(chk_ends.cpu(), subs[-1]["out_ends"])
                        and torch.equal(chk_perm.cpu(), subs[-1]["out_perm"]))

    # KDE gradients on the last sub-batch's list (not part of the step: the configuration is search + KDE)
    from pccnn_lib_b200 import ops
    step.run(subs[-1]["pts"], subs[-1]["ids"], keep=True)
    spts, neigh, ends = step.keep
    w_up = torch.randn(spts.shape[0], device=device)
    # the list is the uncapped neighborhood of the points in themselves: the one-pass gradient applies; the general
    # operator (what a capped or foreign list needs) is timed beside it and must agree
    grads_ms, _ = device_timed(lambda: ops.compute_pdf_grads(3, step.bw, spts, neigh, ends, w_up,
                                                             full_self_neighborhood=True), 5, 2)
    grads_general_ms, _ = device_timed(lambda: ops.compute_pdf_grads(3, step.bw, spts, neigh, ends, w_up), 3, 1)
    g_one = ops.compute_pdf_grads(3, step.bw, spts, neigh, ends, w_up, full_self_neighborhood=True)
    g_gen = ops.compute_pdf_grads(3, step.bw, spts, neigh, ends, w_up)
    grads_agree = bool((g_one - g_gen).abs().max() <= 2e-5 * g_gen.abs().max())
    del g_one, g_gen
    grads_pairs, grads_pts = int(neigh.shape[0]), int(spts.shape[0])

    # results of a resident run of every sub-batch, for the comparison with the CPU leg
    gpu_results = None
    if R.world == 1 and not args.no_cpu:
        gpu_results = []
        for sub in subs:
            step.num_batches = sub["count"]
            pdf, s_ends, _, _ = step.run(sub["pts"], sub["ids"], keep=True)
            gpu_results.append(dict(first=sub["first"], count=sub["count"], pdf=pdf.cpu().numpy(),
                                    ends=s_ends.cpu().numpy(), checksum=list_checksum(step.keep[1])))
    step.keep = None
    del spts, neigh, ends, w_up

    if R.rank != 0:
        return None

    peak, _, peak_src = measured_peaks()

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
    del pc

    n_pts = my_clouds * POINTS_PER_CLOUD
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
    search_ms = (stage_ms["neighbors_count"] + stage_ms["neighbors_store"]) * n_sub
    search_bytes = 8.0 * t_rank + n_pts * (12 + 8) * 2 + 4.0 * n_pts
    kde_gbs = algo["kde"] / (stage_ms["kde"] * n_sub * 1e-3) / 1e9
    grads_bytes = 8.0 * grads_pairs + 32.0 * grads_pts
    roofline = {"bound": "hbm", "kernel": dominant, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "peak_source": peak_src,
                "traffic": round(NCU_DRAM_BYTES_PER_PAIR[dominant] * t_rank), "algorithmic_bytes": round(algo[dominant]),
                "ms_per_launch_set": round(dom_ms, 4),
                "stage_ms": {k: round(v * n_sub, 4) for k, v in stage_ms.items()},
                "find_neighbors_operator": {"ms": round(search_ms, 4), "algorithmic_bytes": round(search_bytes),
                                            "achieved": round(search_bytes / (search_ms * 1e-3) / 1e9, 1),
                                            "frac": round(search_bytes / (search_ms * 1e-3) / 1e9 / peak, 4)},
                "compute_pdf": {"achieved": round(kde_gbs, 1), "frac": round(kde_gbs / peak, 4)},
                "compute_pdf_grads": {"ms": round(grads_ms, 4), "pairs": grads_pairs, "algorithmic_bytes": round(grads_bytes),
                                      "achieved": round(grads_bytes / (grads_ms * 1e-3) / 1e9, 1),
                                      "frac": round(grads_bytes / (grads_ms * 1e-3) / 1e9 / peak, 4),
                                      "kernel": "one pass per point over the full self-neighborhood",
                                      "general_operator_ms": round(grads_general_ms, 4),
                                      "general_operator_frac": round(grads_bytes / (grads_general_ms * 1e-3) / 1e9 / peak, 4),
                                      "agree_2e-5": grads_agree}}

    cpu, parity = None, None
    if gpu_results is not None:
        cpu, parity = cpu_baseline_sample(h_pts, h_ids, gpu_results)

    h2d = sum(s["h_pts"].numel() * 4 + s["h_ids"].numel() * 4 for s in subs)
    d2h = sum(s["out_pdf"].numel() * 4 + s["out_ends"].numel() * 4 + s["out_perm"].numel() * 8 for s in subs)
    mean_ms = float(np.mean(rank_ms))
    # neighbors per point of this rank's clouds, from the CSR ends the end-to-end run left in host memory
    per_point = np.concatenate([np.diff(s["out_ends"].numpy().astype(np.int64), prepend=0) for s in subs])
    quantiles = {name: int(v) for name, v in zip(["min", "p10", "p50", "p90", "p99", "max"],
                                                  np.percentile(per_point, [0, 10, 50, 90, 99, 100]))}
    line = {
        "metric": "neighbor pairs/s (radius search + KDE)", "value": pairs / (ms * 1e-3), "unit": "pairs/s",
        "n_gpus": R.world, "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32+i32/i64",
        "data": "synthetic",
        "config": {"workload": "neighbor search + KDE: %d clouds x 100k surface points per GPU, radius 0.05, "
                               "int32 CSR, fp32 KDE bandwidth 0.01" % CLOUDS_PER_RANK,
                   "clouds_total": total_clouds, "points_per_cloud": POINTS_PER_CLOUD,
                   "pairs_per_step_rank0": t_rank, "neighbors_per_point_rank0": t_rank / n_pts,
                   "neighbors_per_point_quantiles_rank0": quantiles,
                   "pointcloud_compute_pdf_ms": round(class_pdf_ms, 3), "sub_batches_for_int32_offsets": n_sub,
                   "l2": "inputs larger than L2 (neighbor list)", "library_kernels": "cub radix sort and scan",
                   "sharding": "one batch of 16 N distinct clouds (every 16 consecutive ids repeat the same primitives with "
                               "new points) dealt to the ranks by estimated neighbor pairs, heaviest first "
                               "(parallel.assign_clouds); every rank runs the whole pipeline on its clouds; no collective "
                               "on the data path",
                   "clouds_rank0": cloud_ids,
                   "rank_ms_per_step": [round(v, 4) for v in rank_ms], "rank_pairs_per_step": rank_pairs,
                   "imbalance_max_over_mean": round(max(rank_ms) / mean_ms, 4) if mean_ms > 0 else None,
                   "numa_local_cpus": R.numa_cpus},
        "clocks": clocks,
        "e2e": {"value": e_pairs / (e_ms * 1e-3), "unit": "pairs/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e_ms / args.steps,
                "result": "per-point pdf, CSR end offsets and sort permutation copied to pinned host memory",
                "host_results_equal_resident_run": e2e_verified,
                "pipelining": "uploads of the next and downloads of the previous sub-batch overlap the kernels of the "
                              "current one (two copy streams); all copies inside the timed region"},
        # kernels of this library per sub-batch and step (cub's sort and scan kernels not counted): box init and
        # accumulate, cells per axis, keys, iota, gather, cell table; tile estimate + iota, count, clamp; tile estimate
        # + iota, store; point padding, density
        "gpu_launches": 16 * n_sub * args.steps,
        "roofline": roofline,
        "cpu_baseline": cpu,
        "parity_checked": parity,
    }
    return line


# ---- CPU arm of the headline ---------------------------------------------------------------------
def cpu_step(pts, batch_ids, num_clouds, with_points=False):
    """The same step on the CPU oracle.  Returns (neighbor list, end offsets, density) in sorted point order
    (and the sorted points when asked)."""
    from oracle import oracle
    cell = np.full((3,), RADIUS, np.float32)
    g = oracle.build_grid(pts, batch_ids, num_clouds, cell)
    neigh, start_ids = oracle.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"],
                                             g["grid_ds"], g["num_cells"], cell, 0)
    pdf = oracle.compute_pdf(3, np.full((3,), BANDWIDTH, np.float32), g["sorted_pts"], neigh, start_ids)
    if with_points:
        return neigh, start_ids, pdf, g["sorted_pts"]
    return neigh, start_ids, pdf


def pdf_float64(sorted_pts, neigh, ends, which):
    """The density of the points `which` evaluated in float64 from a neighbor list (compute_pdf/compute_pdf.cu:56-75
    of the reference, same constants), as the yardstick for two float32 summations in different orders."""
    ibw = 1.0 / np.float64(np.float32(BANDWIDTH))
    scale = ibw ** 3 / (2.0 * 3.1415) ** 1.5
    out = np.zeros((len(which),), np.float64)
    for i, m in enumerate(which):
        lo = int(ends[m - 1]) if m > 0 else 0
        d = (sorted_pts[neigh[lo:int(ends[m]), 0]].astype(np.float64) - sorted_pts[m].astype(np.float64)) * ibw
        out[i] = scale * np.exp(-0.5 * (d * d).sum(1)).sum()
    return out


def cpu_baseline_sample(pts, ids, gpu_results):
    """One step of the CPU restatement over the same sub-batches the GPU ran, timed, and compared with the GPU's
    results: CSR end offsets exactly, the neighbor list through an order-sensitive checksum, the density within
    1e-5 of a float64 evaluation on a sample of points (and within 1e-4 of the restatement everywhere: both sum
    thousands of float32 terms per point, in different orders)."""
    from oracle import oracle
    cores = oracle.set_threads(len(os.sched_getaffinity(0)))  # a launcher may have capped OMP_NUM_THREADS
    pairs, dt, ok, detail = 0, 0.0, True, []
    for res in gpu_results:
        sel = (ids >= res["first"]) & (ids < res["first"] + res["count"])
        p, b = np.ascontiguousarray(pts[sel]), np.ascontiguousarray(ids[sel] - res["first"])
        t0 = time.perf_counter()
        neigh, ends, pdf, g_sorted = cpu_step(p, b, res["count"], with_points=True)
        dt += time.perf_counter() - t0
        pairs += neigh.shape[0]
        same_ends = bool(np.array_equal(ends, res["ends"]))
        same_list = list_checksum(neigh) == res["checksum"]
        which = np.random.RandomState(5).randint(0, p.shape[0], size=512)
        exact = pdf_float64(g_sorted, neigh, ends, which)
        gpu_err = float(np.abs(res["pdf"][which] - exact).max() / np.abs(exact).max()) if same_ends else None
        gpu_rel = float((np.abs(res["pdf"][which] - exact) / exact).max()) if same_ends else None
        cpu_rel = float((np.abs(pdf[which] - exact) / exact).max())
        everywhere = float((np.abs(res["pdf"] - pdf) / np.abs(pdf)).max()) if same_ends else None
        same_pdf = bool(same_ends and gpu_rel <= 1e-5 and everywhere <= 1e-4)
        detail.append({"csr_ends_equal": same_ends, "list_checksum_equal": same_list,
                       "pdf_gpu_vs_float64_max_rel_512_points": gpu_rel, "pdf_cpu_port_vs_float64_max_rel": cpu_rel,
                       "pdf_gpu_vs_cpu_port_max_rel_all_points": everywhere, "pdf_ok": same_pdf})
        ok = ok and same_ends and same_list and same_pdf
    cpu = {"value": pairs / dt, "unit": "pairs/s", "cores": cores, "kind": "port",
           "sample": "one step over all %d clouds (%d points, %d pairs) in %.2f s, C + OpenMP restatement; its list, "
                     "end offsets and density compared with the GPU's" % (int(ids.max()) + 1, pts.shape[0], pairs, dt),
           "comparison": detail}
    return cpu, ok


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from oracle import oracle
    cores = oracle.set_threads(len(os.sched_getaffinity(0)))  # a launcher may have capped OMP_NUM_THREADS
    num_clouds = CLOUDS_PER_RANK
    pts, ids = make_batch(0, num_clouds)
    # a step is the whole 16-cloud batch, about two seconds on 16 cores
    steps, warmup = args.steps, max(args.warmup, 1)
    for _ in range(warmup):
        cpu_step(pts, ids, num_clouds)
    t0 = time.perf_counter()
    pairs = 0
    for _ in range(steps):
        pairs += cpu_step(pts, ids, num_clouds)[0].shape[0]
    dt = time.perf_counter() - t0
    value = pairs / dt
    line = {
        "impl": "reference", "metric": "neighbor pairs/s (radius search + KDE)", "value": value, "unit": "pairs/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": dt / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32+i32/i64", "data": "synthetic",
        "config": {"workload": "neighbor search + KDE: %d clouds x 100k surface points per GPU, radius 0.05, "
                               "int32 CSR, fp32 KDE bandwidth 0.01" % CLOUDS_PER_RANK,
                   "note": "the reference has no CPU implementation; this is the C + OpenMP restatement of its "
                           "algorithm on the host cores, each step the whole %d-cloud batch" % num_clouds},
        "cpu_baseline": {"value": value, "unit": "pairs/s", "cores": cores, "kind": "port",
                         "sample": "%d clouds x %d points per step, %d steps" % (num_clouds, POINTS_PER_CLOUD, steps)},
        "e2e": {"value": value, "unit": "pairs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(json.dumps(line))


# ---- convolution configurations ------------------------------------------------------------------
CONV_WORKLOADS = {
    "kpconv_cfg0": dict(desc="KPConv single layer forward: 1 cloud x 4096 uniform points, Cin 16, Cout 32, 16 kernel "
                             "points, radius 0.1", layers=[("kp", 16, 32)], clouds=1, pts=4096, gen="cube", radius=0.1,
                        k=16, backward=False, pool=None, shard="none"),
    "mcconv_cfg2": dict(desc="MCConv forward+backward: 32 clouds x 32768 surface points, outputs Poisson-disk radius "
                             "0.03, conv radius 0.075, Cin 64, Cout 128, hidden 16, pdf bandwidth 0.015",
                        layers=[("mc", 64, 128)], clouds=32, pts=32768, gen="surface", radius=0.075, k=16,
                        backward=True, pool=0.03, bw=0.015, shard="clouds"),
    "kpconv_scene": dict(desc="KPConv forward+backward on one room-like scene of 2M points, radius 0.1 m, Cin 128, "
                              "Cout 128, 16 kernel points", layers=[("kp", 128, 128)], clouds=1, pts=2000000,
                         gen="scene", radius=0.1, k=16, backward=True, pool=None, shard="scenes"),
    "mcconv_scene": dict(desc="MCConv forward+backward on one room-like scene of 2M points, radius 0.1 m, Cin 128, "
                              "Cout 128, hidden 16, pdf bandwidth 0.02 m", layers=[("mc", 128, 128)], clouds=1,
                         pts=2000000, gen="scene", radius=0.1, k=16, backward=True, pool=None, bw=0.02, shard="scenes"),
    "scene_pair_cfg4": dict(desc="KPConv + MCConv layer pair forward+backward on one room-like scene of 2M points per "
                                 "GPU, radius 0.1 m, Cin = Cout = 128, 16 kernel points / hidden 16, pdf bandwidth 0.02 m",
                            layers=[("kp", 128, 128), ("mc", 128, 128)], clouds=1, pts=2000000, gen="scene", radius=0.1,
                            k=16, backward=True, pool=None, bw=0.02, shard="scenes"),
}
LIST_FREE_MAX_SAMPLES = 16384  # encoder levels up to this many output points use the list-free convolution
SECONDARY = ["kpconv_cfg0", "mcconv_cfg2", "kpconv_encoder_cfg3", "scene_pair_cfg4"]


class GradientSum(object):
    """Sum of parameter gradients over the ranks on a communication stream of its own (NCCL): the weight gradient
    as soon as the backward operator has recorded that it is final, the small parameter gradients when the operator
    has finished.  Device times of the collectives and of what the compute stream had to wait for at the end."""

    def __init__(self, R):
        import torch
        self.R, self.stream = R, torch.cuda.Stream(device=R.device)
        self.marks, self.enabled = [], R.world > 1

    def new_event(self):
        import torch
        if not self.enabled:
            return None
        e = torch.cuda.Event()
        e.record()
        return e

    def _sum(self, tensors, after_event):
        import torch
        import torch.distributed as dist
        with torch.cuda.stream(self.stream):
            if after_event is not None:
                self.stream.wait_event(after_event)
            else:
                self.stream.wait_stream(torch.cuda.current_stream(self.R.device))
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for t in tensors:
                t.record_stream(self.stream)
            if len(tensors) == 1:
                dist.all_reduce(tensors[0])
            else:
                flat = torch.cat([t.reshape(-1) for t in tensors])
                dist.all_reduce(flat)
                off = 0
                for t in tensors:
                    t.copy_(flat[off:off + t.numel()].reshape(t.shape))
                    off += t.numel()
            b.record()
            self.marks.append((a, b))

    def weights(self, d_w, event):
        if self.enabled:
            self._sum([d_w], event)

    def small(self, tensors):
        if self.enabled:
            self._sum(list(tensors), None)

    def finish(self):
        """Makes the compute stream wait for the collectives; returns the events that bracket the wait."""
        import torch
        if not self.enabled:
            return None
        cur = torch.cuda.current_stream(self.R.device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        cur.wait_stream(self.stream)
        b.record()
        return a, b


def _conv_host_data(w, R):
    """This rank's clouds of a convolution workload on the host: (pts, ids, clouds)."""
    if w["gen"] == "cube":
        return np.random.RandomState(1000).rand(w["pts"], 3).astype(np.float32), np.zeros(w["pts"], np.int32), 1
    if w["gen"] == "scene":
        # Weak scaling with equal work: every rank gets the same room, turned by a multiple of 90 degrees about its
        # centre (mirrored from the fifth rank on) and shifted by a fraction of a cell, i.e. different coordinates,
        # another alignment to the grid, the same neighborhoods.
        pts = scene_cloud(0, w["pts"])
        if R.rank > 0:
            x, y = pts[:, 0] - 10.0, pts[:, 1] - 10.0
            if R.rank >= 4:
                x = -x
            for _ in range(R.rank % 4):
                x, y = -y, x
            shift = np.float32(0.013 * R.rank)
            pts = np.stack([x + 10.0 + shift, y + 10.0 + shift, pts[:, 2]], 1).astype(np.float32)
        return np.ascontiguousarray(pts), np.zeros(w["pts"], np.int32), 1
    from pccnn_lib_b200 import parallel
    lo, hi = parallel.shard_clouds([w["pts"]] * w["clouds"], R.world, R.rank)
    pts, ids = make_batch(lo, hi - lo, w["pts"])
    return pts, ids, hi - lo


def conv_entry(name, args, R, steps=None, with_gemm_alone=True):
    """One convolution configuration: resident time of the layer(s), end-to-end time from pinned host memory
    (geometry included), layer-level roofline, CPU baseline on a sample (single GPU only)."""
    import torch
    import pccnn_lib_b200 as lib
    from pccnn_lib_b200 import ops
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    w = dict(CONV_WORKLOADS[name])
    if args.points:
        w["pts"] = args.points  # smaller instance of the same workload, for profiler captures
        w["desc"] += " [reduced to %d points per cloud]" % args.points
    if w["shard"] == "none" and R.world > 1:
        return {"workload": name, "skipped": "a single cloud does not shard; measured at 1 GPU"}
    device = R.device
    steps = steps or (args.steps if args.exact_steps else max(args.steps, 10))
    warm = args.warmup if args.exact_steps else max(args.warmup, 3)
    rs = np.random.RandomState(77 + R.rank)
    pts, ids, clouds = _conv_host_data(w, R)
    radius = np.full((3,), w["radius"], np.float32)
    if args.presort:
        # store the cloud in grid-cell order (what a spatially coherent scan or a previous pooling stage would
        # deliver); neighbor rows of nearby samples then sit close together in memory
        tmp = lib.pc.Pointcloud(pts, ids, device=R.device)
        g0 = lib.pc.Grid(tmp, lib.pc.BoundingBox(tmp), radius)
        g0.compute_cell_ids()
        order = g0.sorted_ids_.cpu().numpy()
        pts, ids = np.ascontiguousarray(pts[order]), np.ascontiguousarray(ids[order])
        w["desc"] += " [points stored in grid-cell order]"
        del tmp, g0
    k = w["k"]
    n = pts.shape[0]
    cin0 = w["layers"][0][1]
    cout_last = w["layers"][-1][2]
    h_pts, h_ids = torch.from_numpy(pts).pin_memory(), torch.from_numpy(ids).pin_memory()
    h_feats = torch.from_numpy(rs.normal(size=(n, cin0)).astype(np.float32)).pin_memory()
    rad = torch.as_tensor(radius, device=device)

    def geometry(d_pts, d_ids):
        """Everything a layer needs besides features: output points, neighborhood, density."""
        pc = lib.pc.Pointcloud(d_pts, d_ids)
        pc._batch_size_host = clouds
        pc_out = pc
        if w["pool"]:
            pool = lib.pc.PointPooling(pc, np.full((3,), w["pool"], np.float32))
            pc_out = lib.pc.Pointcloud(pool.pool_tensor(pc.pts_), pool.pool_tensor(pc.batch_ids_))
            pc_out._batch_size_host = clouds
        grid = lib.pc.Grid(pc, lib.pc.BoundingBox(pc), radius)
        grid.compute_cell_ids()
        grid.build_ds()
        nb = lib.pc.Neighborhood(grid, pc_out, 0)
        pdf = None
        if any(kind == "mc" for kind, _, _ in w["layers"]):
            pc.compute_pdf(np.full((3,), w["bw"], np.float32))
            pdf = (pc.pts_unnorm_pdf_ * float(np.prod(radius))).contiguous()
        return dict(pc=pc, pc_out=pc_out, nb=nb, pdf=pdf)

    # parameters of the layers (same on every rank, as after a broadcast)
    prs = np.random.RandomState(7)
    params = []
    for kind, cin, cout in w["layers"]:
        if kind == "kp":
            kp, sigma = prepare_kernel_points(3, k)
            params.append(dict(kind="kp", cin=cin, cout=cout, kpts=torch.as_tensor(kp, device=device), sigma=sigma,
                               weights=torch.as_tensor(prs.normal(0, np.sqrt(1.0 / (15 * cin)), size=(k * cin, cout))
                                                       .astype(np.float32), device=device)))
        else:
            params.append(dict(kind="mc", cin=cin, cout=cout,
                               axis=torch.as_tensor(prs.normal(0, np.sqrt(1 / 3.0), size=(3, k)).astype(np.float32), device=device),
                               bias=torch.zeros((1, k), dtype=torch.float32, device=device),
                               weights=torch.as_tensor(prs.normal(0, np.sqrt(1.0 / (cin * k)), size=(1, k * cin, cout))
                                                       .astype(np.float32), device=device)))
    gsum = GradientSum(R)

    def forward(geo, feats):
        acts = [feats]
        for p in params:
            a = (geo["pc"].pts_, acts[-1], geo["pc_out"].pts_, geo["nb"].neighbors_, geo["nb"].start_ids_, rad)
            if p["kind"] == "kp":
                acts.append(ops.kp_conv(*a, p["kpts"], p["sigma"], p["weights"]))
            else:
                acts.append(ops.mc_conv(a[0], geo["pdf"], *a[1:], p["axis"], p["bias"], p["weights"]))
        return acts

    def backward(geo, acts, grads):
        """Backward through the layers in reverse; parameter gradients are summed over the ranks as they appear."""
        g, out = grads, []
        for p, x in zip(reversed(params), reversed(acts[:-1])):
            a = (geo["pc"].pts_, x, geo["pc_out"].pts_, geo["nb"].neighbors_, geo["nb"].start_ids_, rad)
            ev = gsum.new_event()
            if p["kind"] == "kp":
                r = ops.kp_conv_grads(*a, p["kpts"], p["sigma"], p["weights"], g, weight_grads_event=ev)
                small = [r[2]]
            else:
                r = ops.mc_conv_grads(a[0], geo["pdf"], *a[1:], p["axis"], p["bias"], p["weights"], g,
                                      weight_grads_event=ev)
                small = [r[2], r[3]]
            gsum.weights(r[0], ev)
            gsum.small(small)
            out.append(r)
            g = r[1]
        return out

    d_pts, d_ids = h_pts.to(device), h_ids.to(device)
    t0 = time.perf_counter()
    geo = geometry(d_pts, d_ids)
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t0
    m, t = int(geo["pc_out"].pts_.shape[0]), int(geo["nb"].neighbors_.shape[0])
    feats = h_feats.to(device)
    h_grads = torch.from_numpy(rs.normal(size=(m, cout_last)).astype(np.float32)).pin_memory() if w["backward"] else None
    grads = h_grads.to(device) if w["backward"] else None
    wait_marks = []

    def step():
        acts = forward(geo, feats)
        if w["backward"]:
            r = backward(geo, acts, grads)
            wm = gsum.finish()
            if wm:
                wait_marks.append(wm)
            return acts[-1], r
        return acts[-1], None

    ms, clocks = device_timed(step, steps, warm, R, R.local_rank)
    fwd_ms, _ = device_timed(lambda: forward(geo, feats), max(3, steps // 2), 1, R)
    torch.cuda.synchronize()
    allreduce = None
    if gsum.enabled and w["backward"]:
        per_step = len(gsum.marks) // (steps + warm + 0) if gsum.marks else 0
        recent = gsum.marks[-steps * max(per_step, 1):]
        coll_us = 1e3 * sum(a.elapsed_time(b) for a, b in recent) / steps
        exposed_us = 1e3 * sum(a.elapsed_time(b) for a, b in wait_marks[-steps:]) / steps
        allreduce = {"backend": "nccl", "ranks": R.world, "collectives_per_step": per_step,
                     "bytes_per_step": int(sum(p["weights"].numel() * 4 for p in params)),
                     "device_us_per_step": round(R.max(coll_us), 1), "exposed_us_per_step": round(R.max(exposed_us), 1),
                     "overlap": "weight gradients are summed on a side stream from the moment the backward operator "
                                "records them final; the wait of the compute stream at the end of the step is the exposed part. "
                                "Both figures include waiting for the slowest rank to reach the collective (the ranks' "
                                "clouds differ), not only the transfer"}
    gsum.marks, wait_marks = [], []

    # ---- end to end: points, features and upstream gradients from pinned host memory, geometry rebuilt, output and
    # weight gradients back to pinned host memory, all inside the timed region
    h_out = torch.empty((m, cout_last), dtype=torch.float32).pin_memory()
    h_dw = [torch.empty(tuple(p["weights"].shape), dtype=torch.float32).pin_memory() for p in params]

    def e2e_step():
        p_d, i_d = h_pts.to(device, non_blocking=True), h_ids.to(device, non_blocking=True)
        f_d = h_feats.to(device, non_blocking=True)
        g_d = h_grads.to(device, non_blocking=True) if w["backward"] else None
        geo2 = geometry(p_d, i_d)
        acts = forward(geo2, f_d)
        h_out.copy_(acts[-1], non_blocking=True)
        if w["backward"]:
            r = backward(geo2, acts, g_d)
            gsum.finish()
            for dst, layer in zip(h_dw, reversed(r)):
                dst.copy_(layer[0], non_blocking=True)

    e2e_steps = max(3, min(steps, 10))
    e2e_ms, _ = device_timed(e2e_step, e2e_steps, 2, R)
    gsum.marks = []
    h2d = h_pts.numel() * 4 + h_ids.numel() * 4 + h_feats.numel() * 4 + (h_grads.numel() * 4 if w["backward"] else 0)
    d2h = h_out.numel() * 4 + (sum(x.numel() * 4 for x in h_dw) if w["backward"] else 0)

    total_m = R.sum(m)
    total_t = R.sum(t)
    mult = 3 if w["backward"] else 1
    useful = sum(2.0 * m * k * cin * cout for _, cin, cout in w["layers"]) * mult
    _, tc_peak, peak_src = measured_peaks()
    entry = {
        "workload": name, "metric": "conv-layer points/s (%s)" % ("forward+backward" if w["backward"] else "forward"),
        "value": total_m / (ms * 1e-3), "unit": "points/s", "n_gpus": R.world, "steps": steps, "warmup": warm,
        "ms_per_step": ms, "dtype": "f32 (bf16 hi/lo split on tensor cores, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": w["desc"], "points_rank0": n, "samples_rank0": m, "pairs_rank0": t,
                   "samples_total": total_m, "pairs_total": total_t, "neighbors_per_sample": t / max(m, 1),
                   "forward_ms": fwd_ms, "backward_ms": ms - fwd_ms if w["backward"] else 0.0,
                   "setup_s_untimed": setup_s,
                   "sharding": {"none": "single cloud", "clouds": "clouds split over the ranks (parallel.shard_clouds)",
                                "scenes": "one scene per rank (the same room, turned and shifted)"}[w["shard"]]},
        "clocks": clocks,
        "e2e": {"value": total_m / (e2e_ms * 1e-3), "unit": "points/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "includes": "upload of points, batch ids, features%s; %sgrid, neighborhood%s; the layer(s); download of "
                            "the output%s" % (", upstream gradients" if w["backward"] else "",
                                              "Poisson-disk pooling, " if w["pool"] else "",
                                              ", density" if geo["pdf"] is not None else "",
                                              " and weight gradients" if w["backward"] else "")},
        "roofline": {"bound": "tensor", "level": "layer", "useful_flop_per_step": useful,
                     "formula": "2*M*K*Cin*Cout per layer%s" % (" x3 with backward" if w["backward"] else ""),
                     "achieved": round(useful / (ms * 1e-3) / 1e12, 3), "peak": tc_peak, "unit": "TFLOP/s",
                     "frac": round(useful / (ms * 1e-3) / 1e12 / tc_peak, 5), "peak_source": peak_src, "traffic": None},
    }
    if allreduce:
        entry["allreduce"] = allreduce
    if with_gemm_alone and R.rank == 0:
        entry["roofline"]["contraction_alone"] = gemm_alone(w["layers"][0][1] * k, w["layers"][0][2], min(m, 1 << 17),
                                                            device, tc_peak)
    if R.world == 1 and not args.no_cpu:
        entry["cpu_baseline"], entry["parity_checked"] = cpu_conv_sample(w, params, geo, forward(geo, feats), grads, k)
    del geo, feats, grads
    torch.cuda.empty_cache()
    return entry


def gemm_alone(inner, cout, rows, device, tc_peak):
    """The tensor-core contraction alone on the layer's shape (three bf16 products per element, all counted)."""
    import torch
    from pccnn_lib_b200 import ops
    kpad = (inner + 63) // 64 * 64
    a32 = torch.randn(rows, kpad, device=device)
    b32 = torch.randn(cout, kpad, device=device)
    a_hi, b_hi = a32.to(torch.bfloat16), b32.to(torch.bfloat16)
    a_lo, b_lo = (a32 - a_hi.float()).to(torch.bfloat16), (b32 - b_hi.float()).to(torch.bfloat16)
    c_out = torch.empty((rows, cout), dtype=torch.float32, device=device)
    st = torch.zeros((1,), dtype=torch.int32, device=device)
    ms, _ = device_timed(lambda: ops.gemm_bf16(a_hi, b_hi, a_lo, b_lo, out=c_out, status=st), 20, 3)
    flops = 2.0 * rows * kpad * cout * 3
    return {"kernel": "gemm_bf16 (hi/lo split) alone", "rows": int(rows), "inner": int(kpad), "cols": int(cout), "ms": ms,
            "status": int(st.item()), "achieved": round(flops / (ms * 1e-3) / 1e12, 2),
            "frac": round(flops / (ms * 1e-3) / 1e12 / tc_peak, 4),
            "useful_fp32_equivalent_tflops": round(flops / 3 / (ms * 1e-3) / 1e12, 2)}


def cpu_conv_sample(w, params, geo, acts, grads, k, budget=1 << 26):
    """CPU baseline of a convolution configuration: the torch composition that mirrors the reference's ATen host code
    (index_select, broadcast ops, index_add_, matmul; oracle/conv_oracle.py in float32, all host cores) on the first
    samples of the workload -- as many as keep the [pairs, Cin, K] temporary within `budget` elements -- forward
    and, where the configuration has one, backward.  `acts` are the GPU's activations (input features, then the output
    of every layer): each layer is run on the CPU with the input the GPU gave it, and the GPU's output rows of those
    samples are compared with the CPU's."""
    import torch
    from oracle import conv_oracle
    nb, ends = geo["nb"].neighbors_, geo["nb"].start_ids_
    cin_max = max(p["cin"] for p in params)
    max_pairs = max(1, budget // (cin_max * k))
    ends_h = ends.cpu().numpy()
    s = int(np.searchsorted(ends_h, max_pairs, side="right"))
    s = max(1, min(s, ends_h.shape[0]))
    t_s = int(ends_h[s - 1])
    rows = nb[:t_s].cpu().numpy()
    uniq, inv = np.unique(rows[:, 0], return_inverse=True)
    rows_c = np.stack([inv.astype(np.int32), rows[:, 1]], 1)
    idx = torch.as_tensor(uniq.astype(np.int64), device=acts[0].device)
    sub_pts = geo["pc"].pts_[idx].cpu()
    sub_samples = geo["pc_out"].pts_[:s].cpu()
    sub_pdf = geo["pdf"][idx].cpu() if geo["pdf"] is not None else None
    radii = torch.full((3,), float(w["radius"]))
    xs = [a[idx].float().cpu() for a in acts[:-1]]
    g = grads[:s].cpu() if grads is not None else None
    host = [{kk: (v.cpu() if torch.is_tensor(v) else v) for kk, v in p.items()} for p in params]

    def run():
        # the sample subset has no neighborhoods of its own neighbors, so a chain of layers is run layer by layer, each
        # on the rows of the GPU's input to that layer (same arithmetic per layer as in the chain)
        outs = []
        for p, xin in zip(host, xs):
            if p["kind"] == "kp":
                o = conv_oracle.kp_conv(sub_pts, xin, sub_samples, rows_c, ends_h[:s], radii, p["kpts"], p["sigma"],
                                        p["weights"], dtype=torch.float32)
                if g is not None:
                    gg = g if g.shape[1] == p["cout"] else torch.randn(s, p["cout"])
                    conv_oracle.kp_conv_grads(sub_pts, xin, sub_samples, rows_c, ends_h[:s], radii, p["kpts"], p["sigma"],
                                              p["weights"], gg, dtype=torch.float32)
            else:
                o = conv_oracle.mc_conv(sub_pts, sub_pdf, xin, sub_samples, rows_c, ends_h[:s], radii, p["axis"],
                                        p["bias"], p["weights"], dtype=torch.float32)
                if g is not None:
                    gg = g if g.shape[1] == p["cout"] else torch.randn(s, p["cout"])
                    conv_oracle.mc_conv_grads(sub_pts, sub_pdf, xin, sub_samples, rows_c, ends_h[:s], radii, p["axis"],
                                              p["bias"], p["weights"], gg, dtype=torch.float32)
            outs.append(o)
        return outs

    run()
    reps, t0 = 3, time.perf_counter()
    for _ in range(reps):
        outs = run()
    dt = (time.perf_counter() - t0) / reps
    parity = True
    for o, a in zip(outs, acts[1:]):
        ref, got = o.numpy(), a[:s].float().cpu().numpy()
        scale = max(1.0, float(np.abs(ref).max()))
        parity = parity and bool(np.isclose(ref / scale, got / scale, rtol=1e-4, atol=1e-4).all())
    cpu = {"value": s / dt, "unit": "points/s", "cores": torch.get_num_threads(), "kind": "port",
           "sample": "the first %d samples (%d pairs, %d distinct neighbors) of the workload, %s, %d passes of the "
                     "torch-CPU restatement in float32, %.1f ms each%s"
                     % (s, t_s, uniq.shape[0], "forward+backward" if g is not None else "forward", reps, dt * 1e3,
                        "; every layer on the GPU's input to it, its output compared with the GPU's rows (isclose 1e-4 "
                        "of the output scale)")}
    return cpu, parity


def encoder_entry(args, R):
    """KPConv 5-level encoder, inference, bf16 features and weights with fp32 accumulation: 64 clouds x 50k
    surface points, Poisson-disk radii 0.02 ... 0.32, convolution radius 2.5 x the sampling radius, channels
    3-64-128-256-512-1024, 16 kernel points.  No normalisation or activation between levels (the reference
    ships no model).  One step = all poolings, neighborhoods and convolutions of the five levels."""
    import torch
    import pccnn_lib_b200 as lib
    from pccnn_lib_b200 import ops, parallel
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    device = R.device
    total_clouds = args.clouds if args.clouds not in (CLOUDS_PER_RANK,) else 64
    num_pts = args.points or 50000
    lo, hi = parallel.shard_clouds([num_pts] * total_clouds, R.world, R.rank)
    clouds = hi - lo
    pts, ids = make_batch(lo, clouds, num_pts)
    rs = np.random.RandomState(3)
    channels = [3, 64, 128, 256, 512, 1024]
    kp, sigma = prepare_kernel_points(3, 16)
    kpts = torch.as_tensor(kp, device=device)
    w32 = [rs.normal(0, np.sqrt(2.0 / (channels[l] * 16)), size=(16 * channels[l], channels[l + 1])).astype(np.float32)
           for l in range(5)]
    weights = [torch.as_tensor(x, device=device).to(torch.bfloat16) for x in w32]
    f32 = np.random.RandomState(30 + R.rank).normal(size=(pts.shape[0], 3)).astype(np.float32)
    h_pts, h_ids = torch.from_numpy(pts).pin_memory(), torch.from_numpy(ids).pin_memory()
    h_feats = torch.from_numpy(f32).to(torch.bfloat16).pin_memory()
    d_pts, d_ids, feats0 = h_pts.to(device), h_ids.to(device), h_feats.to(device)
    stats = {}

    def step(p_d=None, i_d=None, f_d=None, record=False, list_free=True):
        pc = lib.pc.Pointcloud(d_pts if p_d is None else p_d, d_ids if i_d is None else i_d)
        pc._batch_size_host = clouds
        feats = feats0 if f_d is None else f_d
        conv_ms, geo = [], []
        for level in range(5):
            r_pool = 0.02 * (2 ** level)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
            pool = lib.pc.PointPooling(pc, np.full((3,), r_pool, np.float32))
            pc_out = lib.pc.Pointcloud(pool.pool_tensor(pc.pts_), pool.pool_tensor(pc.batch_ids_))
            pc_out._batch_size_host = clouds
            ev[1].record()
            radius = torch.full((3,), 2.5 * r_pool, dtype=torch.float32, device=device)
            grid = lib.pc.Grid(pc, lib.pc.BoundingBox(pc), radius)
            grid.compute_cell_ids()
            grid.build_ds()
            # inference needs no neighbor list: at the small levels, where a level costs what its launches and host
            # round trips cost, the convolution searches the grid in its own kernel instead
            free = list_free and not record and pc_out.pts_.shape[0] <= LIST_FREE_MAX_SAMPLES
            nb = lib.pc.GridNeighborhood(grid, pc_out) if free else lib.pc.Neighborhood(grid, pc_out, 0)
            ev[2].record()
            geo.append(ev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if nb.neighbors_ is None:
                feats = ops.kp_conv_grid(grid.sorted_pts_, grid.sorted_cell_ids_, grid.sorted_ids_, feats, pc_out.pts_,
                                         nb.sample_cell_ids_, grid.grid_ds_, grid.num_cells_, grid.cell_size_, kpts, sigma,
                                         weights[level])
            else:
                feats = ops.kp_conv(pc.pts_, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, radius, kpts, sigma,
                                    weights[level])
            e1.record()
            if record:
                stats.setdefault("levels", []).append(dict(points=int(pc.pts_.shape[0]), samples=int(pc_out.pts_.shape[0]),
                                                           pairs=int(nb.neighbors_.shape[0])))
            conv_ms.append((e0, e1))
            pc = pc_out
        if record:
            stats["last_batch_ids"] = pc.batch_ids_
        return feats, (conv_ms, geo)

    out_listed, _ = step(record=True)
    out, _ = step()
    same = float((out.float() - out_listed.float()).abs().max() / out_listed.float().abs().max())
    steps, warm = (args.steps, args.warmup) if args.exact_steps else (max(args.steps, 10), max(args.warmup, 3))
    listed_ms, _ = device_timed(lambda: step(list_free=False), max(3, steps // 2), 2, R)
    marks = []

    def timed_step():
        marks.append(step()[1])

    ms, clocks = device_timed(timed_step, steps, warm, R, R.local_rank)
    marks = marks[-steps:]
    conv = [float(np.mean([m[0][l][0].elapsed_time(m[0][l][1]) for m in marks])) for l in range(5)]
    pooling = [float(np.mean([m[1][l][0].elapsed_time(m[1][l][1]) for m in marks])) for l in range(5)]
    neighborhoods = [float(np.mean([m[1][l][1].elapsed_time(m[1][l][2]) for m in marks])) for l in range(5)]
    flops = sum(2.0 * lv["samples"] * 16 * channels[l] * channels[l + 1] for l, lv in enumerate(stats["levels"]))
    conv_total = sum(conv)

    h_out = torch.empty(tuple(out.shape), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        f, _ = step(h_pts.to(device, non_blocking=True), h_ids.to(device, non_blocking=True),
                    h_feats.to(device, non_blocking=True))
        h_out.copy_(f, non_blocking=True)

    e2e_ms, _ = device_timed(e2e_step, max(3, min(steps, 10)), 2, R)
    total_pts = R.sum(pts.shape[0])
    _, tc_peak, peak_src = measured_peaks()
    entry = {
        "workload": "kpconv_encoder_cfg3", "metric": "conv-layer points/s (5-level KPConv encoder, inference; input points per second)",
        "value": total_pts / (ms * 1e-3), "unit": "points/s", "n_gpus": R.world, "steps": steps, "warmup": warm,
        "ms_per_step": ms, "dtype": "bf16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": encoder_entry.__doc__.split("  One step")[0].replace("\n    ", " "),
                   "clouds_total": total_clouds, "clouds_rank0": clouds, "points_per_cloud": num_pts,
                   "levels_rank0": stats["levels"], "conv_ms_per_level": conv, "conv_ms_total": conv_total,
                   "geometry_ms": ms - conv_total, "pooling_ms_per_level": pooling,
                   "neighborhood_ms_per_level": neighborhoods,
                   "finite_output": bool(torch.isfinite(out.float()).all()),
                   "route": "levels with at most %d output points run without a neighbor list (the convolution searches the "
                            "grid in its own kernel, ops.kp_conv_grid); larger levels build the list" % LIST_FREE_MAX_SAMPLES,
                   "with_neighbor_lists_ms_per_step": listed_ms,
                   "max_rel_difference_between_the_two_routes": same,
                   "sharding": "clouds split over the ranks (parallel.shard_clouds)"},
        "clocks": clocks,
        "e2e": {"value": total_pts / (e2e_ms * 1e-3), "unit": "points/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h_pts.numel() * 4 + h_ids.numel() * 4 + h_feats.numel() * 2,
                "d2h_bytes_per_step": h_out.numel() * 2,
                "includes": "upload of points, batch ids and input features; the five levels; download of the last level's features"},
        "roofline": {"bound": "tensor", "level": "layers (the five convolutions, geometry excluded)",
                     "useful_flop_per_step": flops, "formula": "sum over levels of 2*M*K*Cin*Cout",
                     "achieved": round(flops / (conv_total * 1e-3) / 1e12, 3), "peak": tc_peak, "unit": "TFLOP/s",
                     "frac": round(flops / (conv_total * 1e-3) / 1e12 / tc_peak, 5), "peak_source": peak_src,
                     "traffic": None,
                     "whole_step_frac": round(flops / (ms * 1e-3) / 1e12 / tc_peak, 5)},
    }
    if R.world == 1 and not args.no_cpu:
        # the CPU leg gets the values the GPU got (features and weights as rounded to bf16), so that what is left
        # between the two results is the rounding of the activations to bf16 after every level
        cpu, x = cpu_encoder_sample(pts[:num_pts], h_feats[:num_pts].float().numpy(), kp, sigma,
                                    [wt.float().cpu().numpy() for wt in weights], channels)
        rows0 = int((stats["last_batch_ids"] == 0).sum().item())
        rel = (float((out[:rows0].float().cpu() - x).abs().max() / x.abs().max()) if rows0 == x.shape[0] else None)
        cpu["sample"] += ("; its last level (%d points x %d channels) compared with the GPU's rows of that cloud: "
                          "largest difference %s of the largest value (bound 2e-2: bf16 activations on the GPU)"
                          % (x.shape[0], x.shape[1], "%.2e" % rel if rel is not None else "n/a, %d rows on the GPU" % rows0))
        entry["cpu_baseline"], entry["parity_checked"] = cpu, bool(rel is not None and rel <= 2e-2)
    del d_pts, d_ids, feats0, out
    torch.cuda.empty_cache()
    return entry


def cpu_encoder_sample(pts, feats, kp, sigma, weights, channels, chunk=1 << 15):
    """The five encoder levels of ONE cloud on the host cores: grid, search and Poisson-disk selection with the C +
    OpenMP restatement, the convolutions as the torch composition of the reference's host code in float32, the
    projection summed over chunks of pairs (index_add_) so that the [pairs, Cin, K] temporary stays small."""
    import torch
    from oracle import oracle
    oracle.set_threads(len(os.sched_getaffinity(0)))
    t0 = time.perf_counter()
    ids = np.zeros((pts.shape[0],), np.int32)
    x = torch.from_numpy(feats)
    kpt = torch.from_numpy(kp)
    for level in range(5):
        r_pool = np.float32(0.02 * (2 ** level))
        cell = np.full((3,), r_pool, np.float32)
        g = oracle.build_grid(pts, ids, 1, cell)
        nbp, ep = oracle.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"], g["grid_ds"],
                                        g["num_cells"], cell, 0)
        sel = g["sorted_ids"][oracle.poisson_disk_sampling(g["sorted_keys"], nbp, ep, g["num_cells"]).reshape(-1)]
        samples = np.ascontiguousarray(pts[sel])
        sids = np.zeros((samples.shape[0],), np.int32)
        rad = np.full((3,), 2.5 * r_pool, np.float32)
        g2 = oracle.build_grid(pts, ids, 1, rad)
        skeys = oracle.compute_keys(samples, sids, g2["aabb_min"], g2["num_cells"], rad)
        nb, ends = oracle.find_neighbors(g2["sorted_pts"], g2["sorted_keys"], samples, skeys, g2["grid_ds"],
                                         g2["num_cells"], rad, 0)
        n0 = torch.from_numpy(g2["sorted_ids"][nb[:, 0]].astype(np.int64))
        n1 = torch.from_numpy(nb[:, 1].astype(np.int64))
        p_t, s_t = torch.from_numpy(pts), torch.from_numpy(samples)
        cin = channels[level]
        proj = torch.zeros((samples.shape[0], cin, 16), dtype=torch.float32)
        for a in range(0, n0.shape[0], chunk):
            i0, i1 = n0[a:a + chunk], n1[a:a + chunk]
            d = (p_t[i0] - s_t[i1]) / torch.from_numpy(rad)
            dist = torch.linalg.norm(d.unsqueeze(1) - kpt.unsqueeze(0), dim=-1)
            basis = torch.clamp(1.0 - dist / sigma, 0.0, 1.0)
            proj.index_add_(0, i1, x[i0].unsqueeze(2) * basis.unsqueeze(1))
        x = proj.reshape(samples.shape[0], -1) @ torch.from_numpy(weights[level])
        pts, ids = samples, sids
    dt = time.perf_counter() - t0
    return {"value": feats.shape[0] / dt, "unit": "points/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": "one of the 64 clouds (%d points) through all five levels in %.2f s: C + OpenMP grid / search / "
                      "sampling, torch-CPU float32 convolutions" % (feats.shape[0], dt)}, x


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
    emit(json.dumps({
        "metric": "pooled points/s (Poisson-disk pooling, list-free route)", "value": pts.shape[0] / ((front + gridded) * 1e-3),
        "unit": "points/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": front + gridded,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32+i32/i64", "data": "synthetic",
        "config": {"workload": run_pooling_workload.__doc__.split("\n")[0], "points": int(pts.shape[0]),
                   "pairs_of_the_self_neighborhood": int(nb.shape[0]), "selected": int(by_grid.shape[0]),
                   "grid_front_end_ms": front, "search_ms": search, "list_based_sampling_ms": listed,
                   "list_free_sampling_ms": gridded, "selections_identical": same}}))


# ---- the reference's own kernels on the same GPU (extra comparator) ------------------------------
def run_reference_gpu(args):
    """Second comparator: the reference's own (generic SIMT) kernels, compiled unmodified for sm_100 by
    oracle/build_reference.py, on the same workload and GPU.  Not the contract's reference arm (that
    one is the CPU); printed with impl = "reference_gpu"."""
    import importlib.util
    import torch
    so = os.path.join(ROOT, "oracle", "_ref", "pccnn_lib_ops.so")
    if not os.path.exists(so):
        emit(json.dumps({"impl": "reference_gpu", "unavailable": "oracle/_ref/pccnn_lib_ops.so has not been built"}))
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
    emit(json.dumps({"impl": "reference_gpu", "metric": "neighbor pairs/s (radius search + KDE)",
                      "value": pairs / (ms * 1e-3), "unit": "pairs/s", "n_gpus": 1, "steps": args.steps,
                      "ms_per_step": ms / args.steps, "higher_is_better": True,
                      "config": {"workload": "neighbor search + KDE: %d clouds x 100k surface points, radius 0.05"
                                             % CLOUDS_PER_RANK,
                                 "note": "unmodified reference kernels built for sm_100 (generic SIMT), torch ops for "
                                         "bbox / argsort / gathers as in the reference's Python classes"}}))


def run_reference_gpu_conv(args):
    """A single-layer convolution workload on the reference's own kernels (built by oracle/build_reference.py)."""
    import importlib.util
    import torch
    import pccnn_lib_b200 as lib
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    so = os.path.join(ROOT, "oracle", "_ref", "pccnn_lib_ops.so")
    if not os.path.exists(so):
        emit(json.dumps({"impl": "reference_gpu", "unavailable": "oracle/_ref/pccnn_lib_ops.so has not been built"}))
        return
    spec = importlib.util.spec_from_file_location("pccnn_lib_ops", so)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    w = dict(CONV_WORKLOADS[args.workload])
    if len(w["layers"]) != 1:
        emit(json.dumps({"impl": "reference_gpu", "unavailable": "single-layer workloads only"}))
        return
    if args.points:
        w["pts"] = args.points
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)

    class _One(object):
        rank, world = 0, 1
    pts, ids, clouds = _conv_host_data(w, _One)
    radius = np.full((3,), w["radius"], np.float32)
    pc = lib.pc.Pointcloud(pts, ids, device=device)
    pc_out = pc
    if w["pool"]:
        pool = lib.pc.PointPooling(pc, np.full((3,), w["pool"], np.float32))
        pc_out = lib.pc.Pointcloud(pool.pool_tensor(pc.pts_), pool.pool_tensor(pc.batch_ids_))
    grid = lib.pc.Grid(pc, lib.pc.BoundingBox(pc), radius)
    grid.compute_cell_ids()
    grid.build_ds()
    nb = lib.pc.Neighborhood(grid, pc_out, 0)
    kind, cin, cout = w["layers"][0]
    k = w["k"]
    rs = np.random.RandomState(77)
    n, m = pts.shape[0], pc_out.pts_.shape[0]
    feats = torch.as_tensor(rs.normal(size=(n, cin)).astype(np.float32), device=device)
    grads = torch.as_tensor(rs.normal(size=(m, cout)).astype(np.float32), device=device)
    rad = torch.as_tensor(radius, device=device)
    if kind == "kp":
        kp, sigma = prepare_kernel_points(3, k)
        kpts = torch.as_tensor(kp, device=device)
        weights = torch.as_tensor(rs.normal(0, np.sqrt(1.0 / (15 * cin)), size=(k * cin, cout)).astype(np.float32), device=device)
        fwd = lambda: ref.kp_conv(pc.pts_, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, rad, kpts, sigma, weights)
        bwd = lambda: ref.kp_conv_grads(pc.pts_, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, rad, kpts, sigma, weights, grads)
    else:
        pc.compute_pdf(np.full((3,), w["bw"], np.float32))
        pdf = (pc.pts_unnorm_pdf_ * float(np.prod(radius))).contiguous()
        axis = torch.as_tensor(rs.normal(0, np.sqrt(1 / 3.0), size=(3, k)).astype(np.float32), device=device)
        bias = torch.zeros((1, k), dtype=torch.float32, device=device)
        weights = torch.as_tensor(rs.normal(0, np.sqrt(1.0 / (cin * k)), size=(1, k * cin, cout)).astype(np.float32), device=device)
        fwd = lambda: ref.mc_conv(pc.pts_, pdf, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, rad, axis, bias, weights)
        bwd = lambda: ref.mc_conv_grads(pc.pts_, pdf, feats, pc_out.pts_, nb.neighbors_, nb.start_ids_, rad, axis, bias, weights, grads)
    fwd_ms, _ = device_timed(fwd, args.steps, max(args.warmup, 1))
    bwd_ms = device_timed(bwd, args.steps, max(args.warmup, 1))[0] if w["backward"] else 0.0
    step_ms = fwd_ms + bwd_ms
    emit(json.dumps({"impl": "reference_gpu", "metric": "conv-layer points/s", "value": m / (step_ms * 1e-3),
                      "unit": "points/s", "ms_per_step": step_ms,
                      "config": {"workload": w["desc"], "forward_ms": fwd_ms, "backward_ms": bwd_ms, "samples": m,
                                 "pairs": int(nb.neighbors_.shape[0]),
                                 "note": "unmodified reference kernels + cuBLAS, built for sm_100"}}))


def run_b200(args):
    import torch
    from pccnn_lib_b200 import _capi  # noqa: F401  (fails loudly if the CUDA library is missing)
    R = Ranks()
    if args.workload != "neighbors_kde":
        entry = encoder_entry(args, R) if args.workload == "kpconv_encoder_cfg3" else conv_entry(args.workload, args, R)
        if R.rank == 0:
            entry.update({"higher_is_better": True, "scaling": "weak", "vs_baseline": None})
            emit(json.dumps(entry))
        R.close()
        return
    line = run_neighbors_kde(args, R)
    torch.cuda.empty_cache()
    secondary = []
    if not args.no_secondary:
        for name in SECONDARY:
            try:
                entry = encoder_entry(args, R) if name == "kpconv_encoder_cfg3" else conv_entry(name, args, R)
            except Exception as e:  # keep the headline even if one configuration fails
                entry = {"workload": name, "error": "%s: %s" % (type(e).__name__, str(e)[:300])}
                torch.cuda.empty_cache()
            secondary.append(entry)
    if R.rank == 0:
        line["secondary"] = secondary
        emit(json.dumps(line))
    R.close()


_RESULT_FD = None


def keep_stdout_for_the_result():
    """From here on everything any library writes to file descriptor 1 (NCCL's version line, for one) goes to stderr;
    the result line alone is written to what stdout was."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(text):
    if _RESULT_FD is None:
        print(text)
        return
    sys.stdout.flush()
    os.write(_RESULT_FD, (text + "\n").encode())


def main():
    keep_stdout_for_the_result()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference_gpu"])
    ap.add_argument("--clouds", type=int, default=CLOUDS_PER_RANK,
                    help="clouds per GPU (default: the full workload; smaller values are for profiler captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs (profiler captures)")
    ap.add_argument("--no-secondary", action="store_true", help="headline workload only (profiler captures)")
    ap.add_argument("--exact-steps", action="store_true",
                    help="convolution workloads: run exactly --steps / --warmup instead of at least 10 / 3 (profiler captures)")
    ap.add_argument("--points", type=int, default=0,
                    help="convolution workloads: points per cloud (default: the workload's own size)")
    ap.add_argument("--presort", action="store_true",
                    help="convolution workloads: store the points in grid-cell order instead of the sampler's random order")
    ap.add_argument("--workload", default="neighbors_kde",
                    choices=["neighbors_kde", "kpconv_encoder_cfg3", "pooling_cfg3_level1"] + sorted(CONV_WORKLOADS),
                    help="neighbors_kde is the headline workload (with the convolution configurations as `secondary`); "
                         "any other name runs that configuration alone")
    args = ap.parse_args()
    globals()["CLOUDS_PER_RANK"] = args.clouds
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference_gpu" and args.workload != "neighbors_kde":
        run_reference_gpu_conv(args)
    elif args.impl == "reference_gpu":
        run_reference_gpu(args)
    elif args.workload == "pooling_cfg3_level1":
        run_pooling_workload(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
