"""Dilated convolution (extension: the reference accepts `dilation` but its kernels ignore it,
src/sphconv/rules.cu:40-41, while its out_spatial sizes the output for a dilated kernel,
sphconv/utils/__init__.py:40-42).  Kernel offset k reads input o*stride - padding + k*dilation.

Rules bit-exact against the CPU oracle (itself pinned to dense conv3d with dilation in tests/test_oracle.py) through
both rule paths (column index / per-column scans), features against the oracle and the module against dense conv3d."""
import numpy as np
import pytest
import torch

import sphconv_b200 as sphconv
from oracle import conv_np, dense_ref, rules_np
from sphconv_b200 import check_status, synthetic
from sphconv_b200 import sphconv_cuda as ops

from gpu_util import DEV, assert_rules_equal, assert_tables_match, to_dev

pytestmark = pytest.mark.gpu

CASES = [
    # kernel, stride, padding, dilation, submanifold
    ([3, 3, 3], [1, 1, 1], [2, 2, 2], [2, 2, 2], True),
    ([3, 3, 3], [1, 1, 1], [3, 1, 2], [3, 1, 2], True),
    ([3, 3, 3], [2, 2, 2], [2, 2, 2], [2, 2, 2], False),
    ([3, 3, 3], [2, 1, 2], [1, 2, 3], [1, 2, 3], False),
    ([2, 3, 2], [1, 2, 1], [1, 2, 0], [3, 2, 1], False),
    ([3, 3, 5], [1, 1, 2], [0, 1, 4], [1, 1, 2], False),
]


@pytest.mark.parametrize("ks,st,pd,dl,subm", CASES)
@pytest.mark.parametrize("dens", [0.02, 0.35])
def test_dilated_rules_match_oracle(ks, st, pd, dl, subm, dens):
    rng = np.random.default_rng(31)
    B, shape = 3, [9, 11, 70]          # 70 depth bins: the column index spans three words
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, dens)
    osh = list(shape) if subm else rules_np.out_spatial(shape, ks, st, pd, dl)
    zi, zp = to_dev(z_idx, z_ptr)
    fn_g, fn_o = (ops.get_rules_subm, rules_np.get_rules_subm) if subm else (ops.get_rules, rules_np.get_rules)
    with torch.enable_grad():
        oz_idx, oz_ptr, rules, rule_size = fn_g(zi, zp, B, shape, osh, ks, st, pd, dl, [2, 2])
    res = fn_o(z_idx, z_ptr, B, shape, osh, ks, st, pd, dl, [2, 2], padded=False)
    assert_rules_equal(res, oz_idx, oz_ptr, rules, rule_size)
    assert_tables_match(res, rules, z_idx.shape[0], oz_idx.shape[0])
    assert check_status() == 0


def test_dilated_rules_unsorted_columns():
    """Columns stored out of depth order take the per-column scan path."""
    rng = np.random.default_rng(32)
    B, shape = 2, [6, 7, 40]
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3)
    zp_flat = np.asarray(z_ptr).reshape(-1)
    z_idx = np.array(z_idx)
    start = 0
    for end in zp_flat:                 # reverse every column
        z_idx[start:end] = z_idx[start:end][::-1]
        start = end
    ks, st, pd, dl = [3, 3, 3], [2, 2, 2], [2, 2, 2], [2, 2, 2]
    osh = rules_np.out_spatial(shape, ks, st, pd, dl)
    zi, zp = to_dev(z_idx, z_ptr)
    oz_idx, oz_ptr, rules, rule_size = ops.get_rules(zi, zp, B, shape, osh, ks, st, pd, dl, [2, 2])
    res = rules_np.get_rules(z_idx, z_ptr, B, shape, osh, ks, st, pd, dl, [2, 2], padded=False)
    assert_rules_equal(res, oz_idx, oz_ptr, rules, rule_size)
    assert check_status() == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.float16, 1e-2)])
@pytest.mark.parametrize("subm", [True, False])
def test_dilated_module_vs_dense_conv3d(dtype, tol, subm):
    """Conv3d / SubMConv3d with dilation 2 against torch's dense conv3d with the same dilation (forward, input and
    weight gradients), the check the reference's tests use for undilated layers (test/test_grad.py:7-36)."""
    rng = np.random.default_rng(33)
    B, shape, iC, oC = 2, [8, 10, 12], 16, 32
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3)
    feat = rng.standard_normal((z_idx.shape[0], iC)).astype(np.float32)
    if subm:
        m = sphconv.SubMConv3d(iC, oC, 3, dilation=2).to(DEV)
        st, pd = [1, 1, 1], [2, 2, 2]
        assert tuple(m.padding) == (2, 2, 2)
    else:
        m = sphconv.Conv3d(iC, oC, 3, stride=2, padding=2, dilation=2).to(DEV)
        st, pd = [2, 2, 2], [2, 2, 2]
    if dtype != torch.float32:
        m = m.to(dtype)
    f = torch.as_tensor(feat, device=DEV).to(dtype).requires_grad_(True)
    x = sphconv.SparseConvTensor(f, shape, B, z_idx=torch.as_tensor(z_idx, device=DEV), z_ptr=torch.as_tensor(z_ptr, device=DEV))
    y = m(x)
    osh = list(shape) if subm else rules_np.out_spatial(shape, [3, 3, 3], st, pd, [2, 2, 2])
    assert [y.D, y.W, y.H] == osh
    w5 = m.weight.detach().float().cpu().numpy()
    f_r = f.detach().float().cpu().numpy()
    up = torch.as_tensor(rng.standard_normal((B, oC, *osh)))
    if subm:        # gradient only flows from the active output sites
        mask = dense_ref.densify(np.ones((z_idx.shape[0], 1), np.float32), z_idx, z_ptr, B, shape) != 0
        up = up * mask
    yd, dfeat, dw5 = dense_ref.dense_conv_grads(f_r, w5, lambda t: up, z_idx, z_ptr, B, shape, st, pd, dilation=[2, 2, 2])
    oz_idx, oz_ptr = y.z_idx.cpu().numpy(), y.z_ptr.cpu().numpy()
    want = dense_ref.gather_rows(yd, oz_idx, oz_ptr, B, osh).numpy()
    got = y.feature.detach().double().cpu().numpy()
    assert (np.abs(got - want) <= tol * np.maximum(np.abs(want), 1)).all()
    if not subm:    # the output pattern is exactly where the dense result can be non-zero
        occ = dense_ref.occupancy_after_conv(z_idx, z_ptr, B, shape, [3, 3, 3], st, pd, [2, 2, 2])
        mine = dense_ref.densify(np.ones((oz_idx.shape[0], 1), np.float32), oz_idx, oz_ptr, B, osh)[:, 0] != 0
        assert (occ == mine).all()
    g_rows = dense_ref.gather_rows(up, oz_idx, oz_ptr, B, osh)
    y.feature.backward(g_rows.to(DEV).to(dtype))
    dx = f.grad.double().cpu().numpy()
    assert (np.abs(dx - dfeat.numpy()) <= tol * np.maximum(np.abs(dfeat.numpy()), 1)).all()
    dw = m.weight.grad.double().cpu().numpy()
    assert np.abs(dw - dw5.numpy()).max() <= tol * max(np.abs(dw5.numpy()).max(), 1)
    assert check_status() == 0
