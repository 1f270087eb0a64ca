"""Seeded synthetic range-voxel scans that stand in for LiDAR sweeps.

The reference's fixtures are four reduced KITTI velodyne scans and its tests voxelise them on the
CPU; no dataset is available here, so every measurement and parity case uses scans drawn from the
column-occupancy / bins-per-column / depth distributions listed in ``CONFIGS`` below.  Output is the
range-voxel format of ``sphconv/tensor.py:33-125``: ``feature [NNZ,C]``, ``z_idx int32 [NNZ]``
(ascending inside a column) and ``z_ptr int32 [B,H,W]``, an *inclusive* prefix sum over (b,h,w)
row-major (``src/sphconv/tensor.cu:107-109``).
"""
import math

import numpy as np

# name -> workload description.  shape is [H (beams), W (azimuth), D (depth bins)], i.e. the list
# the reference's Python code calls spatial_shape_DWH (shape[2] is the compressed axis).
CONFIGS = {
    "cfg1": dict(id=1, B=1, shape=[32, 128, 64], occ=0.85, nbins="uniform", nmax=3, depth="uniform", C=16,
                 dtype="fp32", net="subm16"),
    "cfg2": dict(id=2, B=4, shape=[64, 512, 128], occ=0.90, nbins="geometric", nmax=4, depth="uniform", C=32,
                 dtype="fp16", net="down32_64"),
    "cfg3": dict(id=3, B=8, shape=[64, 512, 256], occ=0.90, nbins="uniform", nmax=4, depth="lognormal", C=4,
                 dtype="fp16", net="encoder8"),
    "cfg4": dict(id=4, B=16, shape=[64, 512, 256], occ=0.90, nbins="uniform", nmax=4, depth="lognormal", C=4,
                 dtype="bf16", net="encoder8"),
    "cfg5": dict(id=5, B=64, shape=[64, 2048, 256], occ=0.90, nbins="uniform", nmax=4, depth="lognormal", C=4,
                 dtype="int8", net="encoder8"),
}

# SECOND-style middle encoder: (subm?, iC, oC, stride, indice_key)
ENCODER8 = [
    (True, 4, 16, 1, "subm0"), (True, 16, 16, 1, "subm0"),
    (False, 16, 32, 2, None), (True, 32, 32, 1, "subm1"), (True, 32, 32, 1, "subm1"),
    (False, 32, 64, 2, None), (True, 64, 64, 1, "subm2"), (True, 64, 64, 1, "subm2"),
]


def _draw_bins(rng, ncol, nmax, D, depth):
    """[ncol, nmax] candidate bins; every row holds distinct values when depth == 'uniform'."""
    if depth == "uniform":
        bins = rng.integers(0, D, size=(ncol, nmax))
        while True:
            srt = np.sort(bins, axis=1)
            bad = (srt[:, 1:] == srt[:, :-1]).any(axis=1)
            if not bad.any():
                return bins
            bins[bad] = rng.integers(0, D, size=(int(bad.sum()), nmax))
    # distance ~ LogNormal(ln 20 m, 0.6), rejected outside [0, 80) m, mapped linearly onto D bins
    r = rng.lognormal(mean=math.log(20.0), sigma=0.6, size=(ncol, nmax))
    while True:
        bad = r >= 80.0
        if not bad.any():
            break
        r[bad] = rng.lognormal(mean=math.log(20.0), sigma=0.6, size=int(bad.sum()))
    return np.floor(r / 80.0 * D).astype(np.int64)


def make_scan(cfg, scan_id):
    """One scan: (counts [H*W] int64, z values [nnz] int64 ascending per column)."""
    H, W, D = cfg["shape"]
    rng = np.random.default_rng(cfg["id"] * 1000 + scan_id)
    ncol = H * W
    occupied = rng.random(ncol) < cfg["occ"]
    nmax = cfg["nmax"]
    if cfg["nbins"] == "uniform":
        n = rng.integers(1, nmax + 1, size=ncol)
    else:  # truncated geometric(p=0.5) on 1..nmax
        p = np.array([0.5 ** j for j in range(1, nmax + 1)])
        n = rng.choice(np.arange(1, nmax + 1), size=ncol, p=p / p.sum())
    n = np.where(occupied, n, 0)
    bins = _draw_bins(rng, ncol, nmax, D, cfg["depth"])
    keep = np.arange(nmax)[None, :] < n[:, None]
    # encode (column, bin) keys, drop duplicates inside a column (lognormal draws can collide)
    key = (np.arange(ncol, dtype=np.int64)[:, None] * D + bins)[keep]
    key = np.unique(key)
    counts = np.bincount(key // D, minlength=ncol)
    return counts, key % D


def make_batch(name_or_cfg, batch=None, first_scan=0, channels=None, feature_seed=None):
    """Range-voxel batch of ``batch`` scans starting at scan id ``first_scan``.
    Returns dict(feature float32 [NNZ,C], z_idx int32 [NNZ], z_ptr int32 [B,H,W], B, shape)."""
    cfg = CONFIGS[name_or_cfg] if isinstance(name_or_cfg, str) else name_or_cfg
    B = cfg["B"] if batch is None else batch
    C = cfg["C"] if channels is None else channels
    H, W, D = cfg["shape"]
    counts, zs = [], []
    for s in range(B):
        c, z = make_scan(cfg, first_scan + s)
        counts.append(c)
        zs.append(z)
    counts = np.concatenate(counts)
    z_idx = np.concatenate(zs).astype(np.int32)
    z_ptr = np.cumsum(counts).astype(np.int32).reshape(B, H, W)
    frng = np.random.default_rng((cfg["id"] * 1000 + first_scan) * 7919 + 17 if feature_seed is None else feature_seed)
    feature = frng.standard_normal((z_idx.shape[0], C), dtype=np.float32)
    return dict(feature=feature, z_idx=z_idx, z_ptr=z_ptr, B=B, shape=[H, W, D])


def make_weight(ksize, iC, oC, seed):
    """[k0,k1,k2,iC,oC] float32, uniform(-b, b) with the bound the reference's initialiser produces:
    kaiming_uniform_(a=sqrt(5)) whose fan_in is size(-1) * receptive field = oC*KV
    (sphconv/utils/__init__.py:57-77,91-124), i.e. b = 1/sqrt(oC*KV)."""
    kv = int(np.prod(ksize))
    bound = 1.0 / math.sqrt(oC * kv)
    rng = np.random.default_rng(seed)
    return rng.uniform(-bound, bound, size=(*ksize, iC, oC)).astype(np.float32)


def make_random_occupancy(rng, B, shape, density, sort_columns=True):
    """Small random case for tests: each (b,h,w,d) cell active with probability ``density``.
    sort_columns=False shuffles the order inside every column (what init_tensor may produce)."""
    H, W, D = shape
    occ = rng.random((B, H, W, D)) < density
    counts = occ.sum(axis=3).reshape(-1)
    z_ptr = np.cumsum(counts).astype(np.int32).reshape(B, H, W)
    z_idx = np.nonzero(occ)[3].astype(np.int32)
    if not sort_columns:
        start = 0
        for c in counts:
            seg = z_idx[start:start + c]
            rng.shuffle(seg)
            start += c
    return z_idx, z_ptr


def make_point_cloud(rng, n_points, sph_range=(6.0, -45.0, 87.5, 70.4, 45.0, 100.0), margin=0.04, degenerate=3):
    """Seeded stand-in for one LiDAR sweep: float32 [n_points, 4] = (x, y, z, intensity).

    Directions are uniform over the angular window of `sph_range` = (r0, phi0, theta0, r1, phi1, theta1) in
    degrees, widened by `margin` on every side so that some points fall outside the grid, ranges are log-normal
    (most returns near), and the points come in azimuth order like a spinning sensor's.  A few degenerate points
    (the origin, points on the z axis: undefined azimuth) exercise the not-a-number path of the transforms."""
    r0, p0, t0, r1, p1, t1 = [float(v) for v in sph_range]
    n = int(n_points)
    phi = np.radians(np.sort(rng.uniform(p0 - margin * (p1 - p0), p1 + margin * (p1 - p0), n)))
    theta = np.radians(rng.uniform(t0 - margin * (t1 - t0), t1 + margin * (t1 - t0), n))
    r = np.exp(rng.normal(math.log(3.0 * r0), 0.7, n)).clip(0.5 * r0, 1.1 * r1)
    pts = np.stack([r * np.sin(theta) * np.cos(phi), r * np.sin(theta) * np.sin(phi), r * np.cos(theta),
                    rng.uniform(0.0, 1.0, n)], 1).astype(np.float32)
    for j in range(min(int(degenerate), n)):
        pts[(j * 7919) % n, :3] = (0.0, 0.0, 0.0 if j == 0 else float(j))
    return pts
