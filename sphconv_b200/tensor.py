"""The range-voxel sparse tensor (ref: sphconv/tensor.py)."""
from typing import List, Optional

import torch

from .functional import InitTensorFunction, ToDenseFunction


class SparseTensorBase:
    """Plain holder of the range-voxel fields (ref: sphconv/tensor.py:7-30)."""

    def __init__(self, B: int, D: int, W: int, H: int, C: int, device, dtype, itype, feature, z_idx, z_ptr):
        self.B, self.D, self.W, self.H, self.C = B, D, W, H, C
        self.device, self.dtype, self.itype = device, dtype, itype
        self.feature, self.z_idx, self.z_ptr = feature, z_idx, z_ptr


class SparseConvTensor(SparseTensorBase):
    """feature [NNZ,C], z_idx int32 [NNZ], z_ptr int32 [B,s0,s1] (inclusive flat prefix), rule_cache.

    ref: sphconv/tensor.py:33-125.  `spatial_shape_DWH` is [s0, s1, s2]: s0, s1 are the dense axes z_ptr is
    indexed by, s2 the compressed axis whose coordinate z_idx stores; they land in the attributes
    D, W, H in that order, exactly as in the reference.  Build it either from z_idx + z_ptr or from COO
    `indices` [NNZ,4] = (b, s0, s1, s2)."""

    def __init__(self, raw_feature: torch.Tensor, spatial_shape_DWH: List[int], batch_size: int,
                 indices: Optional[torch.Tensor] = None, z_idx: Optional[torch.Tensor] = None,
                 z_ptr: Optional[torch.Tensor] = None):
        self.rule_cache = {}
        self.requires_grad = False
        s0, s1, s2 = spatial_shape_DWH[0], spatial_shape_DWH[1], spatial_shape_DWH[2]
        if z_idx is not None and z_ptr is not None:
            super().__init__(batch_size, s0, s1, s2, raw_feature.shape[-1], raw_feature.device, raw_feature.dtype,
                             z_idx.dtype, raw_feature, z_idx, z_ptr)
            return
        if indices is None:
            raise ValueError("either (z_idx, z_ptr) or indices must be given")
        assert indices.dtype == torch.int32
        assert indices.dim() == 2 and indices.shape[1] == 4
        assert raw_feature.dim() == 2 and raw_feature.shape[0] == indices.shape[0]
        assert raw_feature.device == indices.device
        super().__init__(batch_size, s0, s1, s2, raw_feature.shape[-1], raw_feature.device, raw_feature.dtype,
                         indices.dtype, None, None, None)
        self.feature, self.z_idx, self.z_ptr = InitTensorFunction.apply(
            raw_feature, indices, self.B, [self.D, self.W, self.H])

    @property
    def shape(self):
        return [self.B, self.C, self.D, self.H, self.W]

    def find_rule(self, key: str):
        if key is None:
            return None
        return self.rule_cache.get(key)

    def dense(self, device=None):
        """Dense tensor [B, C, s0, s1, s2]."""
        return ToDenseFunction.apply(self.feature, self.z_idx, self.z_ptr, self.shape)
