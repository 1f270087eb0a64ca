"""CPU tests of oracle/voxelize_np.py: against vectors recorded from the reference's own host voxeliser
(tests/golden/voxelize_ref.npz, written by tests/golden/make_voxelize_golden.py) and, where the reference tree and
its compiled module are present, against that module run live on more cases."""
import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

from oracle import build_ref, voxelize_np  # noqa: E402
from sphconv_b200 import synthetic  # noqa: E402
import make_voxelize_golden as gold  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden", "voxelize_ref.npz")


def check_case(points, ref, system, grid, mp, mv, am, own_transform):
    rng6 = voxelize_np.system_range(gold.CART_RANGE, gold.SPH_RANGE, system)
    np.testing.assert_array_equal(rng6, ref["sys_range"])
    sys_pts = voxelize_np.system_points(points, system)
    # same numpy functions as the reference uses -> bit-identical, not-a-number entries included
    np.testing.assert_array_equal(sys_pts, ref["sys_pts"])
    r = voxelize_np.points_to_voxel(points, sys_pts if own_transform else ref["sys_pts"], rng6, grid, mp, mv, am)
    np.testing.assert_array_equal(r["coordinates"], ref["coordinates"])
    np.testing.assert_array_equal(r["num_points_per_voxel"], ref["num_points_per_voxel"])
    np.testing.assert_array_equal(r["voxels"], ref["voxels"])
    assert r["voxel_num"] == ref["voxels"].shape[0] <= mv


def test_oracle_matches_recorded_reference_outputs():
    data = np.load(GOLDEN)
    for ci, (system, n, grid, mp, mv, am) in enumerate(gold.CASES):
        ref = {k: data["c%d_%s" % (ci, k)] for k in ("sys_pts", "sys_range", "voxels", "coordinates",
                                                      "num_points_per_voxel")}
        pts = data["c%d_points" % ci]
        np.testing.assert_array_equal(pts, synthetic.make_point_cloud(np.random.default_rng(9100 + ci), n,
                                                                      gold.SPH_RANGE))
        check_case(pts, ref, system, grid, mp, mv, am, own_transform=True)
    assert any(data["c%d_voxels" % ci].shape[0] == c[4] for ci, c in enumerate(gold.CASES)), "no early stop covered"


@pytest.mark.skipif(build_ref.utils_lib_path() is None or
                    not os.path.exists(os.path.join(build_ref.REFERENCE_ROOT, "sphconv/utils/coord_transform.py")),
                    reason="reference tree / compiled host voxeliser not present")
def test_oracle_matches_live_reference():
    utils = build_ref.load_utils()
    transforms = gold.reference_transforms()
    rng = np.random.default_rng(77)
    for trial in range(24):
        system = voxelize_np.SYSTEMS[trial % 6]
        n = int(rng.integers(1, 6000))
        grid = [int(v) for v in rng.integers(1, 48, 3)]
        mp = int(rng.integers(1, 7))
        mv = int(rng.integers(1, 400)) if trial % 3 == 0 else 24000
        am = trial % 3
        pts = synthetic.make_point_cloud(rng, n, gold.SPH_RANGE, degenerate=trial % 4)
        if trial % 5 == 0:
            pts = pts[rng.permutation(n)]                       # no azimuth order
        ref = gold.run_reference(utils, transforms, pts, system, grid, mp, mv, am)
        check_case(pts, ref, system, grid, mp, mv, am, own_transform=True)


def test_simple_voxel_and_range_voxel_layout():
    rng = np.random.default_rng(5)
    grid = [12, 20, 6]
    scans = [synthetic.make_point_cloud(rng, n, gold.SPH_RANGE) for n in (900, 1, 1400)]
    scan_ptr = np.cumsum([0] + [s.shape[0] for s in scans])
    pts = np.concatenate(scans, 0)
    rng6 = voxelize_np.system_range(gold.CART_RANGE, gold.SPH_RANGE, "spherical")
    feat, z_idx, z_ptr, coord, num = voxelize_np.to_range_voxel(pts, scan_ptr, rng6, grid, 2, 24000, "spherical")
    assert z_ptr.shape == (3, grid[2], grid[1]) and z_ptr.reshape(-1)[-1] == feat.shape[0] == coord.shape[0]
    # rows are sorted by (b, c0, c1, c2) and z_idx is the depth cell
    key = ((coord[:, 0].astype(np.int64) * grid[2] + coord[:, 1]) * grid[1] + coord[:, 2]) * grid[0] + coord[:, 3]
    assert (np.diff(key) > 0).all()
    np.testing.assert_array_equal(z_idx, coord[:, 3])
    # the feature of a voxel is the mean of its first (at most two) points in sweep order
    sys_pts = voxelize_np.system_points(pts, "spherical")
    c0, c1, c2, valid = voxelize_np.cells_of(sys_pts, rng6, grid)
    for row in rng.integers(0, feat.shape[0], 40):
        b, a0, a1, a2 = coord[row]
        lo, hi = scan_ptr[b], scan_ptr[b + 1]
        hit = np.nonzero(valid[lo:hi] & (c0[lo:hi] == a0) & (c1[lo:hi] == a1) & (c2[lo:hi] == a2))[0][:2] + lo
        assert num[row] == hit.shape[0]
        np.testing.assert_array_equal(feat[row], pts[hit].sum(0, dtype=np.float32) / np.float32(hit.shape[0]))
