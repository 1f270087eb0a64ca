"""The CPU restatement of the COO / range-voxel / dense operations against a direct construction of the dense image."""
import numpy as np

from oracle import tensor_np


def _coo(rng, B, shape, dens):
    occ = rng.random((B, *shape)) < dens
    idx = np.stack(np.nonzero(occ), axis=1).astype(np.int32)
    rng.shuffle(idx)
    return idx


def test_init_tensor_and_dense_image():
    rng = np.random.default_rng(3)
    B, shape, C = 3, [5, 6, 37], 4
    idx = _coo(rng, B, shape, 0.25)
    feat = rng.standard_normal((idx.shape[0], C)).astype(np.float32)
    f2, z_idx, z_ptr, perm = tensor_np.init_tensor(feat, idx, B, shape)
    # permutation: COO row n sits at row perm[n]
    assert (f2[perm] == feat).all() and sorted(perm.tolist()) == list(range(idx.shape[0]))
    # z_ptr is the inclusive prefix of the column counts, columns hold ascending depths
    counts = np.zeros((B, shape[0], shape[1]), dtype=np.int64)
    np.add.at(counts, (idx[:, 0], idx[:, 1], idx[:, 2]), 1)
    assert (z_ptr.reshape(-1) == np.cumsum(counts.reshape(-1))).all()
    starts = np.concatenate([[0], z_ptr.reshape(-1)[:-1]])
    for s, e in zip(starts, z_ptr.reshape(-1)):
        assert (np.diff(z_idx[s:e]) > 0).all()
    # dense image = direct scatter of the COO rows
    want = np.zeros((B, *shape, C), dtype=np.float32)
    want[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]] = feat
    dense = tensor_np.to_dense(f2, z_idx, z_ptr, B, shape)
    assert (dense == want).all()
    # the two backwards are the transposes of the forwards
    g = rng.standard_normal(dense.shape).astype(np.float32)
    rows_g = tensor_np.to_dense_backward(g, z_idx, z_ptr)
    assert (rows_g == g[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]][np.argsort(perm)]).all()
    assert (tensor_np.init_tensor_backward(rows_g, perm) == g[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]]).all()


def test_empty_and_single():
    f2, z_idx, z_ptr, perm = tensor_np.init_tensor(np.zeros((0, 3), np.float32), np.zeros((0, 4), np.int32), 2, [2, 3, 4])
    assert f2.shape == (0, 3) and z_idx.shape == (0,) and (z_ptr == 0).all() and perm.shape == (0,)
    f2, z_idx, z_ptr, perm = tensor_np.init_tensor(np.ones((1, 2), np.float32), np.array([[1, 1, 2, 3]], np.int32), 2, [2, 3, 4])
    assert z_idx.tolist() == [3] and z_ptr.reshape(-1).tolist() == [0] * 11 + [1]
