"""Host-side pieces of bench.py that the measured numbers rest on: the synthetic samplers under weak scaling and the
rule that stdout carries the result line alone."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_every_sixteen_clouds_repeat_the_same_mix_with_new_points():
    # clouds 16 and up take the primitives of cloud (id mod 16): same extent and density, other points
    for c in (3, 13):
        a, b = bench.surface_cloud(c, 4000), bench.surface_cloud(c + 16, 4000)
        assert a.shape == b.shape == (4000, 3) and a.dtype == np.float32
        assert not np.array_equal(a, b)
    # cloud 13 is one small sphere: its copy has the same size (the orientations of boxes and patches are drawn anew,
    # so clouds made of those keep their primitives but not their extent)
    a, b = bench.surface_cloud(13, 4000), bench.surface_cloud(29, 4000)
    assert np.allclose(a.max(0) - a.min(0), b.max(0) - b.min(0), rtol=0.05)
    first = [bench.estimate_pairs(c, probe=4000) for c in range(16)]
    second = [bench.estimate_pairs(c + 16, probe=4000) for c in range(16)]
    assert np.allclose(first, second, rtol=0.25)
    assert abs(sum(first) - sum(second)) <= 0.05 * sum(first)  # a rank's batch carries the work of the one-GPU batch
    assert max(first) > 5 * np.median(first)                    # ... including its one dense cloud


def test_the_first_sixteen_clouds_are_seeded_by_their_id_alone():
    a = bench.surface_cloud(7, 1000)
    assert np.array_equal(a, bench.surface_cloud(7, 1000))
    assert not np.array_equal(a, bench.surface_cloud(8, 1000))
    pts, ids = bench.make_batch(0, 3, 500)
    assert pts.shape == (1500, 3) and ids.tolist() == [0] * 500 + [1] * 500 + [2] * 500
    assert np.array_equal(pts[500:1000], bench.surface_cloud(1, 500))


def test_stdout_carries_the_result_line_alone():
    # whatever a library prints to file descriptor 1 during the run goes to stderr; the JSON line is written to what
    # stdout was when the program started
    code = ("import os, sys, json; sys.path.insert(0, %r); import bench; bench.keep_stdout_for_the_result(); "
            "os.write(1, b'noise from a library\\n'); print('python-level noise'); bench.emit(json.dumps({'ok': 1}))" % ROOT)
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stderr
    assert res.stdout.strip().splitlines() == ['{"ok": 1}']
    assert json.loads(res.stdout) == {"ok": 1}
    assert "noise from a library" in res.stderr and "python-level noise" in res.stderr
