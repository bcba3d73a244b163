"""Builds convolution test cases the way the reference's unit tests do
(unit_test/test_kpconv.py:14-57, unit_test/test_mcconv.py:14-60 of phermosilla/pccnn_lib):
clouds from the golden fixture, uniform features seeded with the case's rnd_seed, neighborhoods
of every point in its own cloud, parameters drawn like the layers' reset_parameters."""
import numpy as np

from conftest import ref_case
from oracle import oracle
from test_oracle_pins import oracle_neighborhood, oracle_pdf

KP_CASES = [dict(seed=33, batch=4, n=100, dims=3, cin=32, cout=64, k=16, radius=0.25),
            dict(seed=33, batch=4, n=250, dims=3, cin=32, cout=4, k=16, radius=0.125),
            dict(seed=33, batch=4, n=250, dims=2, cin=32, cout=4, k=8, radius=0.125),
            dict(seed=33, batch=4, n=250, dims=4, cin=32, cout=4, k=16, radius=0.25)]
MC_CASES = [dict(seed=33, batch=4, n=100, dims=3, cin=32, cout=64, k=16, radius=0.25, bw=0.1),
            dict(seed=33, batch=4, n=250, dims=3, cin=32, cout=4, k=16, radius=0.125, bw=0.1),
            dict(seed=33, batch=4, n=250, dims=2, cin=32, cout=4, k=16, radius=0.125, bw=0.1),
            dict(seed=33, batch=4, n=250, dims=4, cin=32, cout=4, k=16, radius=0.25, bw=0.1),
            dict(seed=34, batch=2, n=300, dims=3, cin=3, cout=8, k=16, radius=0.2, bw=0.1)]
# shapes the reference cannot run: odd kernel-point count, channels not a multiple of 8, pooled samples
EXTRA_KP_CASES = [dict(seed=5, batch=3, n=400, dims=3, cin=3, cout=64, k=16, radius=0.2),
                  dict(seed=6, batch=2, n=300, dims=3, cin=20, cout=10, k=15, radius=0.2),
                  dict(seed=7, batch=2, n=500, dims=3, cin=70, cout=130, k=32, radius=0.15, pooled=True),
                  dict(seed=8, batch=2, n=300, dims=3, cin=16, cout=300, k=64, radius=0.2),
                  # narrow inputs (Cin * K <= 64 slots): the lanes-as-neighbors projection
                  dict(seed=9, batch=2, n=300, dims=3, cin=2, cout=12, k=15, radius=0.2),
                  dict(seed=10, batch=2, n=300, dims=2, cin=1, cout=8, k=64, radius=0.2),
                  dict(seed=11, batch=2, n=300, dims=3, cin=5, cout=8, k=8, radius=0.2)]


def base_case(clouds, c, normal_feats=False):
    pts, batch_ids = ref_case(clouds, c["batch"], c["n"], c["dims"])
    rs = np.random.RandomState(c["seed"])
    feats = (rs.normal(size=(pts.shape[0], c["cin"])) if normal_feats
             else rs.uniform(0.0, 1.0, size=(pts.shape[0], c["cin"]))).astype(np.float32)
    samples, sample_b = pts, batch_ids
    if c.get("pooled"):
        pick = np.sort(rs.permutation(pts.shape[0])[: pts.shape[0] // 3])
        samples, sample_b = pts[pick], batch_ids[pick]
    neigh, start_ids, _ = oracle_neighborhood(pts, batch_ids, c["batch"], c["radius"], 0, samples, sample_b)
    out = dict(pts=pts, batch_ids=batch_ids, samples=samples, sample_batch_ids=sample_b, feats=feats, neighbors=neigh,
               start_ids=start_ids,
               radii=np.full((c["dims"],), c["radius"], np.float32), rs=rs)
    return out


def kp_case(clouds, c, normal_feats=False, shrink=False):
    """`shrink` is for gradient comparisons only: the shell point(s) closest to the centre lie at distance
    exactly sigma from it in the reference's tables, so every self pair (offset 0) sits on the kink of the
    clamp, where float32 and float64 evaluations of the derivative pick different sides; pulling the shell
    points in a little moves the kink away.  The forward is continuous there, so forward cases use the
    table as the layers do."""
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    out = base_case(clouds, c, normal_feats)
    k = c["k"]
    table_k = k if k in (8, 16, 32, 64) else 16
    kpts, sigma = prepare_kernel_points(c["dims"], table_k)
    if shrink:
        kpts = kpts * np.random.RandomState(1).uniform(0.85, 0.99, size=(kpts.shape[0], 1)).astype(np.float32)
    out["kernel_pts"], out["sigma"] = np.ascontiguousarray(kpts[:k]), sigma
    out["weights"] = out["rs"].normal(0.0, np.sqrt(2.0 / (c["cin"] * k)), size=(k * c["cin"], c["cout"])).astype(np.float32)
    return out


def mc_case(clouds, c, normal_feats=False, num_mlps=1):
    out = base_case(clouds, c, normal_feats)
    _, unnorm, _, _ = oracle_pdf(out["pts"], out["batch_ids"], c["batch"], c["bw"])
    out["pdf"] = (unnorm * np.prod(out["radii"])).astype(np.float32)
    h = c["k"]
    rs = out["rs"]
    out["axis"] = rs.normal(0.0, np.sqrt(1.0 / c["dims"]), size=(c["dims"], h * num_mlps)).astype(np.float32)
    out["bias"] = rs.normal(0.0, 0.1, size=(1, h * num_mlps)).astype(np.float32)
    out["weights"] = rs.normal(0.0, np.sqrt(1.0 / (c["cin"] * h)),
                               size=(num_mlps, h * c["cin"], c["cout"] // num_mlps)).astype(np.float32)
    return out
