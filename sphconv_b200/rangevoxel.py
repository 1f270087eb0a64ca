"""The reference's legacy ``RangeVoxel`` container and its two helpers, kept so that code written against
``sphconv.RangeVoxel`` / ``sphconv.xyz2RangeVoxel`` / ``sphconv.merge_rangevoxel_batch`` still imports and runs
(ref: sphconv/rangevoxel.py:5-59, sphconv/data.py:29-148, exported at sphconv/__init__.py:2-4).

This is NOT the range-voxel format of the convolution path (that is ``SparseConvTensor``: feature [NNZ,C], z_idx,
z_ptr).  A ``RangeVoxel`` is a dense range image with up to T voxels per pixel:
feature [B,C,T,H,W], depth int [B,T,H,W] (depth bin of each slot), thick int [B,H,W] (slots in use per pixel),
shape = (B,C,D,H,W).  The convolution modules never take one; ``to_sparse()`` converts it to a ``SparseConvTensor``
so that it can enter the path.  Host-side data preparation: plain torch / numpy, no kernels of its own."""
from typing import List, Sequence

import numpy as np
import torch


class RangeVoxel:
    def __init__(self, feature: torch.Tensor, depth: torch.Tensor, thick: torch.Tensor, shape: Sequence[int]):
        B, C, D, H, W = shape
        if tuple(feature.shape[:2]) != (B, C) or tuple(feature.shape[3:]) != (H, W):
            raise AssertionError("feature %s does not match shape %s" % (tuple(feature.shape), tuple(shape)))
        if tuple(depth.shape) != (B, feature.shape[2], H, W):
            raise AssertionError("depth %s must be [B,T,H,W] with T = %d" % (tuple(depth.shape), feature.shape[2]))
        if tuple(thick.shape) != (B, H, W):
            raise AssertionError("thick %s must be [B,H,W]" % (tuple(thick.shape),))
        self.feature, self.depth, self.thick, self.shape = feature, depth, thick, tuple(shape)
        self.indice_dict = {}

    def cuda(self):
        self.feature, self.depth, self.thick = self.feature.cuda(), self.depth.cuda(), self.thick.cuda()
        return self

    def find_indice_pair(self, key):
        return None if key is None else self.indice_dict.get(key)

    def _slots(self):
        """(b, t, h, w) of every slot in use, ordered by (b, h, w, t)."""
        B, C, D, H, W = self.shape
        T = self.feature.shape[2]
        used = torch.arange(T, device=self.thick.device).view(1, 1, 1, T) < self.thick.unsqueeze(-1)   # [B,H,W,T]
        b, h, w, t = torch.nonzero(used, as_tuple=True)
        return b, t, h, w

    def dense(self, device=None):
        """Dense [B,C,D,H,W] tensor with every used slot's features at its depth bin."""
        B, C, D, H, W = self.shape
        b, t, h, w = self._slots()
        d = self.depth[b, t, h, w].long()
        out = torch.zeros((B, C, D, H, W), dtype=self.feature.dtype, device=self.feature.device)
        out[b, :, d, h, w] = self.feature[b, :, t, h, w]
        return out if device is None else out.to(device)

    def to_sparse(self):
        """The same voxels as a ``SparseConvTensor`` (columns = (b,h,w), compressed axis = depth), slots of a pixel
        sorted by depth as the rule kernels' column index wants them."""
        from .tensor import SparseConvTensor
        B, C, D, H, W = self.shape
        b, t, h, w = self._slots()
        d = self.depth[b, t, h, w].long()
        col = (b * H + h) * W + w
        order = torch.argsort(col * D + d)
        z_idx = d[order].to(torch.int32)
        z_ptr = torch.cumsum(torch.bincount(col, minlength=B * H * W), 0).to(torch.int32).view(B, H, W)
        feat = self.feature[b, :, t, h, w][order].contiguous()
        return SparseConvTensor(feat, [H, W, D], B, z_idx=z_idx.contiguous(), z_ptr=z_ptr.contiguous())


def xyz2RangeVoxel(points, v_res=64, h_res=512, d_res=512, v_range=(87.5, 103.4), h_range=(-45, 45),
                   d_range=(6, 70.4), log=True, verbose=False, device=None) -> RangeVoxel:
    """One LiDAR frame [M, NDim] (x, y, z, ...) -> RangeVoxel with T = 1, B = 1 and spatial shape
    [D, H, W] = [d_res, v_res, h_res]; indices outside a range are clamped to its border and a later point overwrites an
    earlier one in the same pixel (ref: sphconv/data.py:29-131)."""
    pts = np.asarray(points)
    x, y, z = pts[:, 0], pts[:, 1], pts[:, 2]
    planar = x * x + y * y
    r = np.sqrt(planar + z * z)
    theta, phi = np.arccos(z / r), np.arcsin(y / np.sqrt(planar))

    def cell(v, lo, hi, n):
        return np.clip(((v - lo) / ((hi - lo) / n)).astype(int), 0, n - 1)

    ti = cell(theta, np.radians(v_range[0]), np.radians(v_range[1]), v_res)
    pi = cell(phi, np.radians(h_range[0]), np.radians(h_range[1]), h_res)
    rr, lo, hi = (np.log(r), np.log(d_range[0]), np.log(d_range[1])) if log else (r, d_range[0], d_range[1])
    di = np.clip((rr - lo) / ((hi - lo) / d_res), 0, d_res - 1).astype(np.int32)
    C = pts.shape[1]
    feature = torch.zeros((1, C, 1, v_res, h_res))
    feature[0, :, 0, ti, pi] = torch.from_numpy(np.ascontiguousarray(pts.T)).float()
    depth = torch.zeros((1, 1, v_res, h_res), dtype=torch.int32)
    depth[0, 0, ti, pi] = torch.from_numpy(di)
    thick = torch.zeros((1, v_res, h_res), dtype=torch.int32)
    thick[0, ti, pi] = 1
    rv = RangeVoxel(feature, depth, thick, shape=(1, C, d_res, v_res, h_res))
    return rv if device is None else RangeVoxel(feature.to(device), depth.to(device), thick.to(device), rv.shape)


def merge_rangevoxel_batch(voxel_list: List[RangeVoxel]) -> RangeVoxel:
    """Frames of equal shape -> one batch, on the device the frames are on (ref: sphconv/data.py:136-148)."""
    first = voxel_list[0]
    shape = (len(voxel_list),) + tuple(first.shape[1:])
    return RangeVoxel(torch.cat([v.feature for v in voxel_list], 0), torch.cat([v.depth for v in voxel_list], 0),
                      torch.cat([v.thick for v in voxel_list], 0), shape)
