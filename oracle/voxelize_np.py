"""CPU restatement of the reference's host voxeliser (test infrastructure: imported only by tests/ and by the
script that writes tests/golden/voxelize_*.npz).

    system_points      sphconv/utils/coord_transform.py:8-127   xyz -> (r | log r | d | log d, phi, theta | z)
    points_to_voxel    include/point2voxel.h:411-511            binning, first-come voxel numbering, point cap
    simple_voxel       sphconv/vfe.py:223-228                   mean of the kept points of a voxel
    to_range_voxel     the three above + init_tensor (src/sphconv/tensor.cu:78-127) for a batch of scans

Pinned against the reference's own compiled module (oracle/_ref/sphconv_utils, built by oracle/build_ref.py from
src/utils/all.cpp) in tests/test_voxelize_oracle.py and through tests/golden/voxelize_*.npz.

The reference walks the points in order: a point outside the grid is skipped; the first point of a new cell
numbers the voxel; when that would be voxel number max_voxels the walk STOPS (later points of existing voxels are
lost too, point2voxel.h:465-466); a voxel keeps its first max_points points.  Everything is float32 arithmetic
(points are float32, ranges are std::vector<float>): cell = floor((coordinate - low) / cell_size) with
cell_size = (high - low) / cells, each operation rounded to float32.
"""
import numpy as np

from . import tensor_np

SYSTEMS = ("spherical", "l-spherical", "cylinder", "l-cylinder", "hybrid", "l-hybrid")


def system_range(cart_range, sph_range, system):
    """float32 [6]: (low0, low1, low2, high0, high1, high2) of the system's three coordinates."""
    c = np.asarray(cart_range, dtype=np.float32)
    s = np.asarray(sph_range, dtype=np.float32)
    first = (np.log(s[0]), np.log(s[3])) if system.startswith("l-") else (s[0], s[3])
    third = (c[2], c[5]) if system.endswith("cylinder") else (np.radians(s[2]), np.radians(s[5]))
    return np.array([first[0], np.radians(s[1]), third[0], first[1], np.radians(s[4]), third[1]], dtype=np.float32)


def system_points(points, system):
    """[N,4] in the dtype of `points`: the three system coordinates and the intensity."""
    if system not in SYSTEMS:
        raise ValueError("unknown coordinate system %r" % (system,))
    p = np.asarray(points)
    x, y, z = p[:, 0], p[:, 1], p[:, 2]
    with np.errstate(all="ignore"):
        x2y2 = x * x + y * y
        planar = np.sqrt(x2y2)
        radial = np.sqrt(x2y2 + z * z)
        phi = np.arcsin(y / planar)
        base = system[2:] if system.startswith("l-") else system
        first = radial if base == "spherical" else planar
        if system.startswith("l-"):
            first = np.log(first)
        third = z if base == "cylinder" else np.arccos(z / radial)
    return np.stack([first, phi, third, p[:, 3]], 1).astype(p.dtype)


def cells_of(sys_pts, sys_range, grid):
    """(c0, c1, c2, valid): c0 from the third coordinate (grid[2] cells), c1 from the second, c2 from the first."""
    rng = np.asarray(sys_range, dtype=np.float32)
    g = [int(v) for v in grid]
    out, valid = [], np.ones(sys_pts.shape[0], dtype=bool)
    with np.errstate(all="ignore"):
        for axis in (2, 1, 0):
            size = np.float32(rng[3 + axis] - rng[axis]) / np.float32(g[axis])
            f = np.floor((sys_pts[:, axis].astype(np.float32) - rng[axis]) / size)
            ok = (f >= 0) & (f < g[axis])          # NaN and +-inf fail, as their int conversion does in the reference
            valid &= ok
            out.append(np.where(ok, f, 0).astype(np.int64))
    return out[0], out[1], out[2], valid


def point_features(points, sys_pts, append_mode):
    if append_mode == 0:
        return np.asarray(points)
    if append_mode == 1:
        return np.concatenate([points, sys_pts[:, :3]], 1)
    if append_mode == 2:
        return np.concatenate([sys_pts[:, :3], points[:, 3:4]], 1)
    raise ValueError("append_mode must be 0, 1 or 2")


def points_to_voxel(points, sys_pts, sys_range, grid, max_points, max_voxels, append_mode=0):
    """-> dict(voxels [V,max_points,C], coordinates int32 [V,3], num_points_per_voxel int32 [V], kept: point indices
    [V,max_points] or -1), voxels in the order their first point appears."""
    points = np.asarray(points)
    g = [int(v) for v in grid]
    c0, c1, c2, valid = cells_of(sys_pts, sys_range, g)
    idx = np.nonzero(valid)[0]
    cell = (c0[idx] * g[1] + c1[idx]) * g[0] + c2[idx]
    _, first_pos = np.unique(cell, return_index=True)
    first_pos.sort()
    if first_pos.shape[0] > max_voxels:                  # the walk stops at the point that would open one voxel more
        idx = idx[:first_pos[max_voxels]]
        cell = cell[:first_pos[max_voxels]]
        first_pos = first_pos[:max_voxels]
    uniq, inverse = np.unique(cell, return_inverse=True)
    ordinal_of_uniq = np.empty(uniq.shape[0], dtype=np.int64)
    ordinal_of_uniq[np.searchsorted(uniq, cell[first_pos])] = np.arange(first_pos.shape[0])
    vox = ordinal_of_uniq[inverse]                       # voxel number of every kept point
    V = first_pos.shape[0]
    order = np.argsort(vox, kind="stable")
    starts = np.searchsorted(vox[order], np.arange(V))
    rank = np.arange(order.shape[0]) - starts[vox[order]]
    keep = rank < max_points
    feats = point_features(points, np.asarray(sys_pts), append_mode)
    voxels = np.zeros((V, max_points, feats.shape[1]), dtype=points.dtype)
    kept = np.full((V, max_points), -1, dtype=np.int64)
    voxels[vox[order][keep], rank[keep]] = feats[idx[order][keep]]
    kept[vox[order][keep], rank[keep]] = idx[order][keep]
    counts = np.minimum(np.bincount(vox, minlength=V), max_points).astype(np.int32)
    fp = idx[first_pos]
    coords = np.stack([c0[fp], c1[fp], c2[fp]], 1).astype(np.int32).reshape(V, 3)
    return {"voxels": voxels, "coordinates": coords, "num_points_per_voxel": counts, "kept": kept, "voxel_num": V}


def simple_voxel(voxels, num_points):
    """Sum of the (zero padded) point slots in slot order, divided by the count."""
    total = np.zeros((voxels.shape[0], voxels.shape[2]), dtype=voxels.dtype)
    for j in range(voxels.shape[1]):
        total = total + voxels[:, j]
    return total / num_points.astype(voxels.dtype).reshape(-1, 1)


def to_range_voxel(points, scan_ptr, sys_range, grid, max_points, max_voxels, system=None, sys_pts=None,
                   append_mode=0):
    """Batch of scans (points[scan_ptr[b]:scan_ptr[b+1]]) -> (feature [NNZ,C], z_idx, z_ptr [B,grid[2],grid[1]],
    coordinates [NNZ,4] = (b, c0, c1, c2) and num_points [NNZ], all in range-voxel row order).  init_tensor reads the
    coordinate rows as they are (src/sphconv/tensor.cu:30-33): columns are (b, c0, c1), the depth is c2, so the
    tensor is [grid[2], grid[1]] columns of grid[0] depth cells."""
    points = np.asarray(points)
    if sys_pts is None:
        sys_pts = system_points(points, system)
    feats, coords, nums = [], [], []
    B = len(scan_ptr) - 1
    for b in range(B):
        lo, hi = int(scan_ptr[b]), int(scan_ptr[b + 1])
        r = points_to_voxel(points[lo:hi], sys_pts[lo:hi], sys_range, grid, max_points, max_voxels, append_mode)
        feats.append(simple_voxel(r["voxels"], r["num_points_per_voxel"]))
        coords.append(np.concatenate([np.full((r["voxel_num"], 1), b, dtype=np.int32), r["coordinates"]], 1))
        nums.append(r["num_points_per_voxel"])
    feat = np.concatenate(feats, 0)
    coord = np.concatenate(coords, 0)
    num = np.concatenate(nums, 0)
    g = [int(v) for v in grid]
    f2, z_idx, z_ptr, perm = tensor_np.init_tensor(feat, coord, B, (g[2], g[1], g[0]))
    order = np.argsort(perm)
    return f2, z_idx, z_ptr, coord[order], num[order]
