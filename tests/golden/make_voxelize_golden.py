"""Records outputs of the reference's OWN host voxeliser as golden vectors for oracle/voxelize_np.py.

    python tests/golden/make_voxelize_golden.py <output directory>      # writes voxelize_ref.npz

Runs on the CPU.  The compiled module is oracle/_ref/sphconv_utils (src/utils/all.cpp of the reference, built by
oracle/build_ref.py); the coordinate transforms are the reference's sphconv/utils/coord_transform.py, loaded by file
path from the reference tree named by REFERENCE_ROOT.  Around them this script does what
sphconv/utils/voxelize.py:122-219 (points_to_voxel_v2) does: allocate the output arrays, transform, call
points_to_voxel_3d, cut the arrays at voxel_num.  Inputs are seeded synthetic sweeps (sphconv_b200.synthetic)."""
import importlib.util
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import build_ref  # noqa: E402
from sphconv_b200 import synthetic  # noqa: E402

CART_RANGE = [6, -40, -3, 70.4, 40, 1]               # sphconv/datagen.py:84-85
SPH_RANGE = [6, -45, 87.5, 70.4, 45, 100]
# (system, points, resolution (first, second, third coordinate), max_points, max_voxels, append_mode)
CASES = [
    ("spherical", 1800, [16, 32, 8], 2, 24000, 0),
    ("spherical", 1800, [16, 32, 8], 2, 500, 0),      # the walk stops early
    ("l-spherical", 1500, [32, 24, 6], 1, 24000, 0),
    ("cylinder", 1500, [12, 40, 5], 3, 24000, 1),
    ("l-cylinder", 1500, [20, 16, 7], 5, 300, 2),
    ("hybrid", 1500, [24, 24, 4], 2, 24000, 0),
    ("l-hybrid", 1500, [9, 33, 11], 4, 24000, 1),
]


def reference_transforms():
    path = os.path.join(build_ref.REFERENCE_ROOT, "sphconv/utils/coord_transform.py")
    spec = importlib.util.spec_from_file_location("ref_coord_transform", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.transform_funcs


def run_reference(utils, transforms, points, system, grid, max_points, max_voxels, append_mode):
    cart = np.array(CART_RANGE, dtype=np.float32)
    sph = np.array(SPH_RANGE, dtype=np.float32)
    C = points.shape[1] + (3 if append_mode == 1 else 0)
    voxels = np.zeros((max_voxels, max_points, C), dtype=points.dtype)
    mask = np.zeros((max_voxels, max_points), dtype=points.dtype)
    coors = np.zeros((max_voxels, 3), dtype=np.int32)
    num = np.zeros((max_voxels,), dtype=np.int32)
    lookup = np.full(tuple(grid[::-1]), -1, dtype=np.int32)
    with np.errstate(all="ignore"):
        sys_pts, sys_range = transforms[system](points, cart, sph)
    n = utils.points_to_voxel_3d(points, sys_pts, voxels, mask, coors, num, lookup, sys_range, grid, max_points,
                                 max_voxels, append_mode)
    assert (lookup == -1).all()
    return dict(sys_pts=sys_pts, sys_range=np.asarray(sys_range, dtype=np.float32), voxels=voxels[:n],
                coordinates=coors[:n], num_points_per_voxel=num[:n], mask=mask[:n])


def main(out_dir):
    utils = build_ref.load_utils()
    assert utils is not None, "oracle/_ref/sphconv_utils is not built"
    transforms = reference_transforms()
    store = {}
    for ci, (system, n, grid, mp, mv, am) in enumerate(CASES):
        rng = np.random.default_rng(9100 + ci)
        pts = synthetic.make_point_cloud(rng, n, SPH_RANGE)
        r = run_reference(utils, transforms, pts, system, grid, mp, mv, am)
        store["c%d_points" % ci] = pts
        for k, v in r.items():
            if k != "mask":
                store["c%d_%s" % (ci, k)] = v
        print(ci, system, "voxels", r["voxels"].shape[0], "max pts", int(r["num_points_per_voxel"].max()))
    np.savez_compressed(os.path.join(out_dir, "voxelize_ref.npz"), **store)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
