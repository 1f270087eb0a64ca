"""CPU restatement of the reference's tensor operations next to the convolution path (test infrastructure: imported
only by tests/).

    init_tensor            src/sphconv/tensor.cu:78-127   COO (b, s0, s1, s2) rows -> range-voxel
    init_tensor_backward   src/sphconv/tensor.cu:147-162  gradient back to the COO row order
    to_dense               src/sphconv/tensor.cu:222-264  range-voxel rows -> dense [B, s0, s1, s2, C]
    to_dense_backward      src/sphconv/tensor.cu:266-309  dense gradient -> rows

The reference counts the voxels of every (b, s0, s1) column with a dense grid, takes the inclusive prefix as z_ptr
(tensor.cu:96-109) and hands out the rows of a column in the arrival order of an atomic counter (tensor.cu:55-76), so
the order inside a column is not defined; this restatement, like the CUDA implementation it checks, uses ascending
depth.  Everything else (z_ptr, the set of (column, depth) per row, the dense image) is defined uniquely.
"""
import numpy as np


def init_tensor(feature, indices_bzyx, B, shape):
    """-> (feature', z_idx int32 [NNZ], z_ptr int32 [B,s0,s1], permutation int32 [NNZ]: new row of COO row n)."""
    H, W, D = [int(v) for v in shape]
    idx = np.asarray(indices_bzyx, dtype=np.int64)
    col = (idx[:, 0] * H + idx[:, 1]) * W + idx[:, 2]
    order = np.argsort(col * D + idx[:, 3], kind="stable")
    permutation = np.empty(idx.shape[0], dtype=np.int32)
    permutation[order] = np.arange(idx.shape[0], dtype=np.int32)
    counts = np.bincount(col, minlength=B * H * W)
    z_ptr = np.cumsum(counts).astype(np.int32).reshape(B, H, W)
    return np.asarray(feature)[order], idx[order, 3].astype(np.int32), z_ptr, permutation


def init_tensor_backward(d_feature_out, permutation):
    return np.asarray(d_feature_out)[np.asarray(permutation, dtype=np.int64)]


def row_columns(z_ptr):
    zp = np.asarray(z_ptr).reshape(-1).astype(np.int64)
    return np.repeat(np.arange(zp.shape[0]), np.diff(zp, prepend=0))


def to_dense(feature, z_idx, z_ptr, B, shape):
    """-> dense [B, s0, s1, s2, C], zero where no voxel."""
    H, W, D = [int(v) for v in shape]
    feature = np.asarray(feature)
    out = np.zeros((B * H * W, D, feature.shape[1]), dtype=feature.dtype)
    out[row_columns(z_ptr), np.asarray(z_idx, dtype=np.int64)] = feature
    return out.reshape(B, H, W, D, feature.shape[1])


def to_dense_backward(d_dense, z_idx, z_ptr):
    d = np.asarray(d_dense)
    B, H, W, D, C = d.shape
    return d.reshape(B * H * W, D, C)[row_columns(z_ptr), np.asarray(z_idx, dtype=np.int64)]
