"""`import sphconv` resolves to this implementation: every name the reference package exports
(sphconv/__init__.py:1-4) and the submodules its users import; the legacy RangeVoxel container converts to the
range-voxel tensor of the convolution path.  CPU only (no op is called)."""
import numpy as np
import torch


def test_reference_names_resolve():
    import sphconv
    import sphconv_b200
    for name in ("Conv3d", "SparseConv3d", "SubMConv3d", "RangeVoxel", "Sequential", "SparseSequential", "VoxelGenerator",
                 "xyz2RangeVoxel", "merge_rangevoxel_batch", "SparseConvTensor"):
        assert getattr(sphconv, name) is getattr(sphconv_b200, name), name
    from sphconv.tensor import SparseConvTensor
    from sphconv.functional import ConvFunction, InitTensorFunction, ToDenseFunction  # noqa: F401
    from sphconv.conv import Conv3d
    from sphconv.modules import Sequential
    from sphconv.utils import out_spatial
    from sphconv import sphconv_cuda
    assert SparseConvTensor is sphconv_b200.SparseConvTensor and Conv3d is sphconv_b200.Conv3d
    assert Sequential is sphconv_b200.Sequential
    assert out_spatial([8, 8, 8], [3, 3, 3], [2, 2, 2], [1, 1, 1]) == [4, 4, 4]
    for op in ("init_tensor", "init_tensor_backward", "to_dense", "to_dense_backward", "get_rules_subm", "get_rules",
               "rule_conv", "rule_conv_backward", "rule_conv_d_feature"):      # src/sphconv/all.cpp:18-31
        assert callable(getattr(sphconv_cuda, op)), op


def test_rangevoxel_roundtrip():
    from sphconv import RangeVoxel, merge_rangevoxel_batch, xyz2RangeVoxel
    rng = np.random.default_rng(0)
    frames = []
    for i in range(2):
        pts = np.c_[rng.uniform(10, 40, 400), rng.uniform(-5, 5, 400), rng.uniform(-2, 1, 400),
                    rng.uniform(0.1, 1, 400)].astype(np.float32)
        frames.append(xyz2RangeVoxel(pts, 16, 32, 24))
    rv = merge_rangevoxel_batch(frames)
    assert isinstance(rv, RangeVoxel) and rv.shape == (2, 4, 24, 16, 32)
    dense = rv.dense()
    assert dense.shape == (2, 4, 24, 16, 32)
    sp = rv.to_sparse()
    n = int(rv.thick.sum())
    assert sp.feature.shape == (n, 4) and int(sp.z_ptr.reshape(-1)[-1]) == n and sp.z_idx.shape[0] == n
    # every row of the sparse tensor sits where the dense image has it
    zp = sp.z_ptr.reshape(-1).long()
    col = torch.repeat_interleave(torch.arange(zp.shape[0]), torch.diff(zp, prepend=torch.zeros(1, dtype=torch.long)))
    b, h, w = col // (16 * 32), (col // 32) % 16, col % 32
    assert torch.equal(dense[b, :, sp.z_idx.long(), h, w], sp.feature)
    assert rv.find_indice_pair(None) is None and rv.find_indice_pair("k") is None
    try:
        RangeVoxel(rv.feature, rv.depth, rv.thick[:, :-1], rv.shape)
        raise RuntimeError("shape check missing")
    except AssertionError:
        pass
