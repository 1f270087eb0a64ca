"""sphconv_b200: the sphconv rule-generation + rule-driven sparse convolution path for B200 (sm_100a).

Same public names as the reference package (sphconv/__init__.py): import it as
``import sphconv_b200 as sphconv``, or import the alias package ``sphconv`` beside it.  All compute runs in the CUDA library behind
``include/sphconv_b200.h``; importing works without a GPU, calling an op without the built library raises.
"""
from .conv import Conv3d, SparseConv3d, SubMConv3d
from .modules import Sequential, SparseSequential, SphModule
from .tensor import SparseConvTensor
from .sphconv_cuda import config
from ._capi import check_status
from .pipeline import ScanPipeline
from .voxelize import VoxelGenerator
from .rangevoxel import RangeVoxel, merge_rangevoxel_batch, xyz2RangeVoxel

__all__ = ["ScanPipeline", "VoxelGenerator", "Conv3d", "SparseConv3d", "SubMConv3d", "Sequential", "SparseSequential", "SphModule",
           "SparseConvTensor", "config", "check_status", "RangeVoxel", "xyz2RangeVoxel", "merge_rangevoxel_batch"]
