"""Dense torch conv3d ground truth, built the way the reference's own tests build it.

Test infrastructure; never imported by the product.

* densify: ``SparseConvTensor.dense()`` layout [B, C, s0, s1, s2] (sphconv/functional.py:83-95, src/sphconv/tensor.cu:164-191)
* strided conv: ``conv3d(dense, W.permute(4,3,0,1,2), stride, padding)`` (test/test_grad.py:29-36, test/test_rules.py:49-55)
* submanifold: same with padding k//2, output kept only at the active input sites (sphconv/conv.py:150-153,210)

This is also the CPU baseline the benchmark times: the reference has no CPU implementation of the path,
its tests use this dense construction as their check.
"""
import numpy as np
import torch

from .rules_np import row_coords


def densify(feature, z_idx, z_ptr, B, shape):
    """[NNZ,C] rows -> dense [B,C,s0,s1,s2] float tensor."""
    H, W, D = shape
    f = torch.as_tensor(np.asarray(feature))
    b, x, y, z = row_coords(z_idx, z_ptr, B, H, W)
    dense = torch.zeros((B, H, W, D, f.shape[1]), dtype=f.dtype)
    dense[torch.as_tensor(b), torch.as_tensor(x), torch.as_tensor(y), torch.as_tensor(z)] = f
    return dense.permute(0, 4, 1, 2, 3).contiguous()


def gather_rows(dense, z_idx, z_ptr, B, shape):
    """dense [B,C,s0,s1,s2] -> rows [NNZ,C] at the sites of (z_idx, z_ptr)."""
    H, W, D = shape
    b, x, y, z = row_coords(z_idx, z_ptr, B, H, W)
    return dense[torch.as_tensor(b), :, torch.as_tensor(x), torch.as_tensor(y), torch.as_tensor(z)]


def occupancy_after_conv(z_idx, z_ptr, B, shape, ksize, stride, padding, dilation=(1, 1, 1)):
    """Output occupancy as test/test_rules.py:14-60 computes it: conv3d of ones != 0."""
    ones = np.ones((np.asarray(z_idx).shape[0], 1), dtype=np.float32)
    dense = densify(ones, z_idx, z_ptr, B, shape)
    w = torch.ones((1, 1, *ksize), dtype=torch.float32)
    out = torch.nn.functional.conv3d(dense, w, None, tuple(stride), tuple(padding), tuple(dilation))
    return (out != 0)[:, 0]


def dense_conv(feature, weight5, z_idx, z_ptr, B, shape, stride, padding, dtype=torch.float64, dilation=(1, 1, 1)):
    """Dense forward.  weight5 is [k0,k1,k2,iC,oC] (sphconv/conv.py:64-65).  Returns dense [B,oC,o0,o1,o2]."""
    dense = densify(np.asarray(feature), z_idx, z_ptr, B, shape).to(dtype)
    w = torch.as_tensor(np.asarray(weight5)).to(dtype).permute(4, 3, 0, 1, 2).contiguous()
    return torch.nn.functional.conv3d(dense, w, None, tuple(stride), tuple(padding), tuple(dilation))


def dense_conv_grads(feature, weight5, d_out_dense_fn, z_idx, z_ptr, B, shape, stride, padding, dtype=torch.float64,
                     dilation=(1, 1, 1)):
    """Forward + autograd through the dense conv (test/test_grad.py:7-36).
    d_out_dense_fn(y_dense) -> upstream gradient tensor of y's shape.
    Returns (y_dense, d_feature_rows [NNZ,iC], d_weight [k0,k1,k2,iC,oC])."""
    f = torch.as_tensor(np.asarray(feature)).to(dtype).requires_grad_(True)
    H, W, D = shape
    b, x, y, z = [torch.as_tensor(a) for a in row_coords(z_idx, z_ptr, B, H, W)]
    dense = torch.zeros((B, H, W, D, f.shape[1]), dtype=dtype)
    dense = dense.index_put((b, x, y, z), f).permute(0, 4, 1, 2, 3)
    w = torch.as_tensor(np.asarray(weight5)).to(dtype).permute(4, 3, 0, 1, 2).contiguous().requires_grad_(True)
    yd = torch.nn.functional.conv3d(dense, w, None, tuple(stride), tuple(padding), tuple(dilation))
    yd.backward(d_out_dense_fn(yd.detach()))
    return yd.detach(), f.grad, w.grad.permute(2, 3, 4, 1, 0).contiguous()


def encoder_dense_forward(feature, z_idx, z_ptr, B, shape, layers, params, threads=None):
    """Dense fp32 forward of a stack of 3x3x3 layers the way the reference's tests check single layers:
    conv3d on the densified grid, submanifold outputs masked to the active sites, then bias + ReLU.
    layers: [(subm, iC, oC, stride, key)], params: [(weight5, bias)].  Returns the dense output
    [B, oC, o0, o1, o2] and the final occupancy mask."""
    if threads:
        torch.set_num_threads(threads)
    x = densify(np.asarray(feature, dtype=np.float32), z_idx, z_ptr, B, shape)
    mask = densify(np.ones((np.asarray(z_idx).shape[0], 1), np.float32), z_idx, z_ptr, B, shape) != 0
    ones_w = torch.ones((1, 1, 3, 3, 3))
    for (subm, iC, oC, stride, key), (w5, bias) in zip(layers, params):
        w = torch.as_tensor(np.asarray(w5, dtype=np.float32)).permute(4, 3, 0, 1, 2).contiguous()
        b = torch.as_tensor(np.asarray(bias, dtype=np.float32))
        if subm:
            x = torch.nn.functional.conv3d(x, w, None, 1, 1)
        else:
            x = torch.nn.functional.conv3d(x, w, None, stride, 1)
            mask = torch.nn.functional.conv3d(mask.float(), ones_w, None, stride, 1) != 0
        x = torch.relu(x + b.view(1, -1, 1, 1, 1)) * mask
    return x, mask
