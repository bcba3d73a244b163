"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world size 2): cloud sharding and the
gradient allreduce.  The data path itself has no collective."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pccnn_lib_b200 import parallel


def test_shards_cover_every_cloud_once_and_balance_points():
    sizes = [100000] * 16
    for world in (1, 2, 4, 8):
        ranges = [parallel.shard_clouds(sizes, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == 16
        assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))
        assert all(hi - lo == 16 // world for lo, hi in ranges)
    ragged = [5, 100, 7, 300, 12, 90, 250, 40]
    ranges = [parallel.shard_clouds(ragged, 3, r) for r in range(3)]
    covered = [c for lo, hi in ranges for c in range(lo, hi)]
    assert covered == list(range(len(ragged))) and all(hi > lo for lo, hi in ranges)
    loads = [sum(ragged[lo:hi]) for lo, hi in ranges]
    assert max(loads) <= 2.0 * sum(ragged) / 3


def test_work_balanced_assignment_covers_every_cloud_once():
    weights = [48.0] * 15 + [420.0] + [30.0] * 16  # one cloud with nine times the work of the others
    for world in (1, 2, 4, 8):
        plan = parallel.assign_clouds(weights, world)
        assert sorted(c for p in plan for c in p) == list(range(len(weights)))
        loads = [sum(weights[c] for c in p) for p in plan]
        # no rank exceeds the larger of the mean load (+ one light cloud) and the heaviest single cloud
        assert max(loads) <= max(sum(weights) / world + 48.0, 420.0)
    assert parallel.assign_clouds(weights, 4) == parallel.assign_clouds(list(weights), 4)  # deterministic


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rs = np.random.RandomState(100 + rank)
        grads = [torch.as_tensor(rs.randn(256, 32).astype(np.float32)), None,
                 torch.as_tensor(rs.randn(16, 3).astype(np.float32)), torch.as_tensor(rs.randn(1, 16).astype(np.float32))]
        parallel.allreduce_grads(grads)
        # every rank also reports how many clouds it would process
        lo, hi = parallel.shard_clouds([1000] * 6, world, rank)
        torch.save(dict(grads=[g for g in grads if g is not None], clouds=(lo, hi)), os.path.join(out_dir, "r%d.pt" % rank))
    finally:
        dist.destroy_process_group()


def test_gradient_allreduce_on_two_gloo_ranks(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    results = [torch.load(os.path.join(str(tmp_path), "r%d.pt" % r)) for r in range(world)]
    # rebuild the per-rank inputs exactly as the workers drew them
    per_rank = []
    for r in range(world):
        rs = np.random.RandomState(100 + r)
        per_rank.append([rs.randn(256, 32).astype(np.float32), rs.randn(16, 3).astype(np.float32),
                         rs.randn(1, 16).astype(np.float32)])
    for i in range(3):
        want = per_rank[0][i] + per_rank[1][i]
        for r in range(world):
            assert np.allclose(results[r]["grads"][i].numpy(), want, rtol=0, atol=1e-6)
    assert results[0]["clouds"] == (0, 3) and results[1]["clouds"] == (3, 6)
