"""Points -> range-voxel on the GPU (through the C ABI) against the CPU restatement of the reference's host voxeliser.

Cells, kept points, z_idx / z_ptr, coordinates and point counts are compared bit for bit: the oracle bins the very
system coordinates the GPU computed.  The feature (a float32 mean) is bit-exact for at most two kept points per voxel
(one addition, one division, both correctly rounded) and within 1e-6 relative beyond.  The transforms use CUDA's
asinf / acosf / logf against numpy's: tolerance 4 float32 ulps, written below."""
import numpy as np
import pytest
import torch

from oracle import voxelize_np
from sphconv_b200 import VoxelGenerator, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CART_RANGE = [6, -40, -3, 70.4, 40, 1]
SPH_RANGE = [6, -45, 87.5, 70.4, 45, 100]


def _scans(rng, sizes, shuffle=False, degenerate=3):
    scans = [synthetic.make_point_cloud(rng, n, SPH_RANGE, degenerate=degenerate) for n in sizes]
    if shuffle:
        scans = [s[rng.permutation(s.shape[0])] for s in scans]
    scan_ptr = np.cumsum([0] + [s.shape[0] for s in scans]).astype(np.int32)
    pts = np.concatenate(scans, 0) if scans else np.zeros((0, 4), np.float32)
    return pts, scan_ptr


def _check(gen, pts, scan_ptr, exact_mean):
    pts_d = torch.as_tensor(pts, device=DEV)
    sys_d = gen.transform(pts_d)
    r = gen.generate(pts_d, torch.as_tensor(scan_ptr), system_points=sys_d)
    torch.cuda.synchronize()
    sys_pts = sys_d.cpu().numpy()
    feat, z_idx, z_ptr, coord, num = voxelize_np.to_range_voxel(
        pts, scan_ptr, gen.system_range, gen.grid_size, gen.max_num_points, gen.max_voxels, sys_pts=sys_pts,
        append_mode=gen.append_mode)
    assert r["voxel_num"] == feat.shape[0]
    np.testing.assert_array_equal(r["z_ptr"].cpu().numpy(), z_ptr)
    np.testing.assert_array_equal(r["z_idx"].cpu().numpy(), z_idx)
    np.testing.assert_array_equal(r["coordinates"].cpu().numpy(), coord)
    np.testing.assert_array_equal(r["num_points_per_voxel"].cpu().numpy(), num)
    got = r["feature"].cpu().numpy()
    assert got.shape == feat.shape
    if exact_mean:
        np.testing.assert_array_equal(got, feat)
    else:
        np.testing.assert_allclose(got, feat, rtol=1e-6, atol=1e-7)
    return r


@pytest.mark.parametrize("system", list(voxelize_np.SYSTEMS))
def test_transform_matches_numpy(system):
    rng = np.random.default_rng(3)
    pts, _ = _scans(rng, [20000])
    gen = VoxelGenerator(CART_RANGE, SPH_RANGE, 2, 24000, [16, 16, 16], system)
    np.testing.assert_array_equal(gen.system_range, voxelize_np.system_range(CART_RANGE, SPH_RANGE, system))
    got = gen.transform(torch.as_tensor(pts, device=DEV)).cpu().numpy()
    want = voxelize_np.system_points(pts, system)
    np.testing.assert_array_equal(np.isnan(got), np.isnan(want))
    np.testing.assert_array_equal(got[np.isinf(want)], want[np.isinf(want)])       # log of a zero range
    ok = np.isfinite(want)
    ulp = np.spacing(np.abs(want[ok]).astype(np.float32))
    assert (np.abs(got[ok] - want[ok]) <= 4 * ulp).all()
    np.testing.assert_array_equal(got[:, 3], pts[:, 3])


@pytest.mark.parametrize("system,grid,max_points,max_voxels,append_mode,sizes", [
    ("spherical", [16, 32, 8], 2, 24000, 0, [1800]),
    ("spherical", [16, 32, 8], 2, 500, 0, [1800, 2500, 300]),          # two scans stop early, one does not
    ("spherical", [256, 512, 64], 2, 24000, 0, [30000, 25000]),
    ("l-spherical", [70, 24, 6], 1, 24000, 0, [1500, 0, 900]),         # an empty scan; depth beyond 64 cells
    ("cylinder", [12, 40, 5], 3, 24000, 1, [1500, 1500]),
    ("l-cylinder", [20, 16, 7], 5, 300, 2, [1500]),
    ("hybrid", [24, 24, 4], 2, 1, 0, [400, 400]),                      # a single voxel per scan
    ("l-hybrid", [9, 33, 11], 4, 24000, 1, [1500, 7]),
    ("spherical", [1, 1, 1], 64, 24000, 0, [700]),                     # everything in one voxel, 64 points kept
])
def test_voxels_match_oracle(system, grid, max_points, max_voxels, append_mode, sizes):
    rng = np.random.default_rng(len(sizes) * 100 + max_points)
    pts, scan_ptr = _scans(rng, sizes)
    gen = VoxelGenerator(CART_RANGE, SPH_RANGE, max_points, max_voxels, grid, system, append_mode)
    r = _check(gen, pts, scan_ptr, exact_mean=max_points <= 2)
    assert r["voxel_num"] > 0


def test_point_order_decides():
    """The same points in another order keep other points and (under max_voxels) other voxels: both follow the oracle."""
    rng = np.random.default_rng(11)
    pts, scan_ptr = _scans(rng, [5000, 5000], shuffle=True)
    gen = VoxelGenerator(CART_RANGE, SPH_RANGE, 1, 900, [32, 64, 16], "spherical")
    a = _check(gen, pts, scan_ptr, True)
    rev = np.concatenate([pts[:5000][::-1], pts[5000:][::-1]], 0).copy()
    b = _check(gen, rev, scan_ptr, True)
    assert a["voxel_num"] == b["voxel_num"] == 1800
    assert not torch.equal(a["coordinates"], b["coordinates"])


def test_extra_point_features_and_no_points():
    rng = np.random.default_rng(5)
    pts, scan_ptr = _scans(rng, [3000])
    pts = np.concatenate([pts, rng.standard_normal((3000, 3)).astype(np.float32)], 1)      # 7 features per point
    gen = VoxelGenerator(CART_RANGE, SPH_RANGE, 2, 24000, [32, 32, 8], "spherical", append_mode=1)
    r = _check(gen, pts, scan_ptr, True)
    assert r["feature"].shape[1] == 10
    empty = gen.generate(torch.zeros((0, 7), device=DEV), torch.tensor([0, 0, 0], dtype=torch.int32))
    assert empty["voxel_num"] == 0 and int(empty["z_ptr"].abs().sum()) == 0 and empty["z_ptr"].shape == (2, 8, 32)
    outside = np.tile(np.array([[-5.0, 0.0, 0.0, 1.0, 0, 0, 0]], np.float32), (10, 1))       # behind the sensor
    assert gen.generate(torch.as_tensor(outside, device=DEV))["voxel_num"] == 0


def test_tensor_feeds_the_encoder():
    """to_tensor gives what SparseConvTensor(indices=...) gives from the oracle's voxel list."""
    from sphconv_b200 import SparseConvTensor, SubMConv3d
    rng = np.random.default_rng(8)
    pts, scan_ptr = _scans(rng, [20000, 15000])
    gen = VoxelGenerator(CART_RANGE, SPH_RANGE, 2, 24000, [64, 128, 16], "spherical")
    t = gen.to_tensor(torch.as_tensor(pts, device=DEV), torch.as_tensor(scan_ptr))
    r = gen.generate(torch.as_tensor(pts, device=DEV), torch.as_tensor(scan_ptr))
    t2 = SparseConvTensor(r["feature"], gen.spatial_shape, 2, indices=r["coordinates"])
    assert torch.equal(t.z_idx, t2.z_idx) and torch.equal(t.z_ptr, t2.z_ptr) and torch.equal(t.feature, t2.feature)
    conv = SubMConv3d(4, 16, 3, bias=False).to(DEV)
    out = conv(t)
    assert out.feature.shape == (t.feature.shape[0], 16) and torch.isfinite(out.feature).all()


def test_against_the_reference_module():
    """The reference's own compiled host voxeliser (oracle/_ref/sphconv_utils, when it was built) walks the system
    coordinates the GPU computed; its voxel list, reordered to range-voxel rows, must equal the GPU's."""
    from oracle import build_ref
    utils = build_ref.load_utils()
    if utils is None:
        pytest.skip("oracle/_ref/sphconv_utils is not built")
    rng = np.random.default_rng(21)
    for system, grid, mp, mv in [("spherical", [256, 512, 64], 2, 24000), ("l-hybrid", [40, 60, 9], 2, 800)]:
        pts, scan_ptr = _scans(rng, [40000])
        gen = VoxelGenerator(CART_RANGE, SPH_RANGE, mp, mv, grid, system)
        pts_d = torch.as_tensor(pts, device=DEV)
        sys_d = gen.transform(pts_d)
        r = gen.generate(pts_d, torch.as_tensor(scan_ptr), system_points=sys_d)
        voxels = np.zeros((mv, mp, 4), np.float32)
        mask = np.zeros((mv, mp), np.float32)
        coors = np.zeros((mv, 3), np.int32)
        num = np.zeros((mv,), np.int32)
        lookup = np.full(tuple(grid[::-1]), -1, np.int32)
        nv = utils.points_to_voxel_3d(pts, sys_d.cpu().numpy(), voxels, mask, coors, num, lookup, gen.system_range,
                                      grid, mp, mv, 0)
        assert nv == r["voxel_num"]
        mean = voxels[:nv].sum(1) / num[:nv, None].astype(np.float32)
        key = (coors[:nv, 0].astype(np.int64) * grid[1] + coors[:nv, 1]) * grid[0] + coors[:nv, 2]
        order = np.argsort(key)
        np.testing.assert_array_equal(r["coordinates"].cpu().numpy()[:, 1:], coors[:nv][order])
        np.testing.assert_array_equal(r["num_points_per_voxel"].cpu().numpy(), num[:nv][order])
        np.testing.assert_array_equal(r["feature"].cpu().numpy(), mean[order])
