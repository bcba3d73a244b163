"""Data parallelism over independent clouds.

The reference is single-process.  Clouds of a batch never interact (keys embed the batch id,
shared/grid_utils.cuh:93 of the reference; the search clamps key windows to the cloud,
find_neighbors/find_ranges_grid_ds.cu:100-105), so a batch is split by cloud across one process
per GPU and the whole pipeline runs locally.  The only exchange is the sum of parameter gradients
after a backward pass.
"""
import torch
import torch.distributed as dist


def shard_clouds(points_per_cloud, world_size, rank):
    """Contiguous range of cloud ids for `rank`, balanced by point count.

    `points_per_cloud` is a sequence of sizes; returns (first_cloud, last_cloud_exclusive).
    Every cloud belongs to exactly one rank and ranges follow rank order.
    """
    sizes = [int(s) for s in points_per_cloud]
    total = float(sum(sizes))
    bounds = [0]
    acc, cloud = 0.0, 0
    for r in range(1, world_size):
        target = total * r / world_size
        while cloud < len(sizes) and acc + sizes[cloud] / 2.0 <= target:
            acc += sizes[cloud]
            cloud += 1
        # leave at least one cloud for every remaining rank when there are enough clouds
        cloud = min(cloud, max(bounds[-1], len(sizes) - (world_size - r)))
        bounds.append(cloud)
    bounds.append(len(sizes))
    return bounds[rank], bounds[rank + 1]


def assign_clouds(weights, world_size):
    """Clouds to ranks by estimated work, without the contiguity of shard_clouds: heaviest cloud first, each to
    the rank with the least work so far (longest-processing-time rule), which keeps one unusually dense cloud
    from dragging its neighbors in id order onto the same rank.  Returns one ascending list of cloud ids per
    rank; deterministic (ties go to the lower rank and the lower cloud id), so every rank computes the same plan.
    """
    order = sorted(range(len(weights)), key=lambda c: (-float(weights[c]), c))
    loads = [0.0] * world_size
    plan = [[] for _ in range(world_size)]
    for c in order:
        r = min(range(world_size), key=lambda i: (loads[i], i))
        plan[r].append(c)
        loads[r] += float(weights[c])
    return [sorted(p) for p in plan]


def rebase_batch_ids(batch_ids, first_cloud):
    """Batch ids of a shard renumbered from zero (each rank builds its own grid)."""
    return batch_ids - first_cloud


def allreduce_grads(tensors, group=None, average=False):
    """Sum (or average) gradient tensors over all ranks in one flat bucket, in place.

    The gradients that need it are small (KPConv dW [K*Cin, Cout], dKernelPts; MCConv dW, dAxis,
    dBias: about a megabyte together), so one collective per backward pass is latency-bound and a
    single bucket is the right shape.  Returns the work handle's result for chaining; tensors of
    `None` are skipped.
    """
    live = [t for t in tensors if t is not None]
    if not live or not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return live
    flat = torch.cat([t.reshape(-1).to(torch.float32) for t in live])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    if average:
        flat /= dist.get_world_size(group)
    offset = 0
    for t in live:
        n = t.numel()
        t.copy_(flat[offset:offset + n].reshape(t.shape).to(t.dtype))
        offset += n
    return live
