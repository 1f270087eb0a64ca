"""Points -> range-voxel tensor on the GPU.

Host mirror of the reference's voxel generator for a given resolution (``VoxelGeneratorV3``,
sphconv/utils/voxel_generator.py:6-70, with ``points_to_voxel_v2``, sphconv/utils/voxelize.py:122-219) fused with
the mean of the kept points (``SimpleVoxel``, sphconv/vfe.py:210-228) and with ``init_tensor``: what
``VoxelizationVFE.generate`` + ``merge_batch_torch`` + ``SparseConvTensor(...)`` do in the reference's tests
(sphconv/datagen.py:77-108, test/common.py:33-59), for a whole batch of scans in a few kernel launches.

Differences from the reference, all on purpose: the points are a CUDA tensor (a batch is one tensor plus
``scan_ptr``); voxels come out in range-voxel row order (ascending b, c0, c1, c2), not in first-come order; the
per-voxel point lists (``voxels`` [V, max_points, C]) are not materialised, only their mean is.  Which points a
voxel keeps, which voxels survive ``max_voxels`` and every cell index are the reference's.
"""
import ctypes
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _capi as C
from .tensor import SparseConvTensor

SYSTEMS = {"spherical": 0, "l-spherical": 1, "cylinder": 2, "l-cylinder": 3, "hybrid": 4, "l-hybrid": 5}


def system_range(point_cloud_range: Sequence[float], point_cloud_sphere_range: Sequence[float],
                 coord_system: str) -> np.ndarray:
    """float32 [6] bounds of the three system coordinates, as the reference's transform functions return them
    (sphconv/utils/coord_transform.py:17-23 and the five siblings): degrees -> radians, logarithm of the range
    bounds for the l- systems, the Cartesian z bounds for the cylinders.  All in float32, like the reference."""
    c = np.asarray(point_cloud_range, dtype=np.float32)
    s = np.asarray(point_cloud_sphere_range, dtype=np.float32)
    logarithmic = coord_system.startswith("l-")
    first = (np.log(s[0]), np.log(s[3])) if logarithmic else (s[0], s[3])
    third = (c[2], c[5]) if coord_system.endswith("cylinder") else (np.radians(s[2]), np.radians(s[5]))
    return np.array([first[0], np.radians(s[1]), third[0], first[1], np.radians(s[4]), third[1]], dtype=np.float32)


class VoxelGenerator:
    """``VoxelGenerator(point_cloud_range, point_cloud_sphere_range, max_num_points, max_voxels, resolution_HWD,
    coord_system)``: the arguments of the reference's VoxelGeneratorV3 that its resolution path reads.
    ``resolution_HWD`` = cells along the (first, second, third) system coordinate, e.g. (r, phi, theta)."""

    def __init__(self, point_cloud_range, point_cloud_sphere_range, max_num_points: int, max_voxels: int = 30000,
                 resolution_HWD: Optional[List[int]] = None, coord_system: str = "spherical", append_mode: int = 0):
        if resolution_HWD is None:
            raise ValueError("resolution_HWD is required (the cell-size path of the reference is not provided)")
        if coord_system not in SYSTEMS:
            raise ValueError("unknown coord_system %r" % (coord_system,))    # the reference prints and exits
        self.coord_system = coord_system
        self.grid_size = [int(v) for v in resolution_HWD]
        self.max_num_points = int(max_num_points)
        self.max_voxels = int(max_voxels)
        self.append_mode = int(append_mode)
        self.system_range = system_range(point_cloud_range, point_cloud_sphere_range, coord_system)

    @property
    def spatial_shape(self) -> List[int]:
        """[s0, s1, s2] of the tensor ``to_tensor`` returns (what the reference calls spatial_shape_DWH)."""
        g = self.grid_size
        return [g[2], g[1], g[0]]

    def _grid(self, B: int) -> C.VoxelGrid:
        g = C.VoxelGrid()
        g.B = B
        for i in range(3):
            g.cells[i] = self.grid_size[i]
        for i in range(6):
            g.range[i] = float(self.system_range[i])
        g.max_points, g.max_voxels, g.append_mode = self.max_num_points, self.max_voxels, self.append_mode
        return g

    def transform(self, points: torch.Tensor) -> torch.Tensor:
        """[N,4] system coordinates + intensity of the points (coord_transform.py of the reference)."""
        C.require_cuda(points)
        if points.dtype != torch.float32 or points.dim() != 2 or points.shape[1] < 4:
            raise RuntimeError("points must be a float32 tensor [N, >=4]")
        sys_pts = torch.empty((points.shape[0], 4), dtype=torch.float32, device=points.device)
        with torch.cuda.device(points.device):
            C.check(C.lib().sph_voxel_transform(C.ptr(points), points.shape[1], points.shape[0],
                                                SYSTEMS[self.coord_system], C.ptr(sys_pts),
                                                C.stream_ptr(points.device)))
        return sys_pts

    def generate(self, points: torch.Tensor, scan_ptr: Optional[torch.Tensor] = None,
                 system_points: Optional[torch.Tensor] = None, with_coordinates: bool = True) -> dict:
        """points float32 [N, F] on the device; scan_ptr int32 [B+1] (device or host; None = one scan).
        Returns feature [NNZ, C], z_idx, z_ptr [B, s0, s1], coordinates int32 [NNZ,4] = (b, c0, c1, c2),
        num_points_per_voxel int32 [NNZ], voxel_num, batch_size, spatial_shape."""
        C.require_cuda(points)
        dev = points.device
        n = points.shape[0]
        if scan_ptr is None:
            scan_ptr = torch.tensor([0, n], dtype=torch.int32)
        B = scan_ptr.shape[0] - 1
        scan_dev = scan_ptr.to(device=dev, dtype=torch.int32).contiguous()
        sys_pts = self.transform(points) if system_points is None else system_points
        C.require_cuda(sys_pts)
        if sys_pts.dtype != torch.float32 or tuple(sys_pts.shape) != (n, 4):
            raise RuntimeError("system_points must be float32 [N, 4]")
        lib = C.lib()
        grid = self._grid(B)
        s = self.spatial_shape
        nbytes = C.check(lib.sph_voxelize_scratch_bytes(ctypes.byref(grid), n))
        scratch = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
        z_ptr = torch.empty((B, s[0], s[1]), dtype=torch.int32, device=dev)
        nnz = ctypes.c_int32(0)
        with torch.cuda.device(dev):
            st = C.stream_ptr(dev)
            C.check(lib.sph_voxelize_count(C.ptr(sys_pts), C.ptr(scan_dev), n, ctypes.byref(grid), C.ptr(scratch),
                                           C.ptr(z_ptr), ctypes.byref(nnz), st))
            nnz = int(nnz.value)
            n_feat = C.check(lib.sph_voxel_feature_count(points.shape[1], self.append_mode))
            feature = torch.empty((nnz, n_feat), dtype=torch.float32, device=dev)
            z_idx = torch.empty((nnz,), dtype=torch.int32, device=dev)
            coords = torch.empty((nnz, 4), dtype=torch.int32, device=dev) if with_coordinates else None
            num = torch.empty((nnz,), dtype=torch.int32, device=dev) if with_coordinates else None
            C.check(lib.sph_voxelize_fill(C.ptr(points), points.shape[1], C.ptr(sys_pts), C.ptr(scan_dev), n,
                                          ctypes.byref(grid), C.ptr(scratch), nnz, C.ptr(feature), C.ptr(z_idx),
                                          C.ptr(coords), C.ptr(num), st))
        return {"feature": feature, "z_idx": z_idx, "z_ptr": z_ptr, "coordinates": coords,
                "num_points_per_voxel": num, "voxel_num": nnz, "batch_size": B, "spatial_shape": s}

    def to_tensor(self, points: torch.Tensor, scan_ptr: Optional[torch.Tensor] = None,
                  dtype: Optional[torch.dtype] = None) -> SparseConvTensor:
        """The SparseConvTensor the encoder takes, straight from the points."""
        r = self.generate(points, scan_ptr, with_coordinates=False)
        feature = r["feature"] if dtype is None else r["feature"].to(dtype)
        return SparseConvTensor(feature, r["spatial_shape"], r["batch_size"], z_idx=r["z_idx"], z_ptr=r["z_ptr"])
