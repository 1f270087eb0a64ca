"""COO -> range-voxel and range-voxel <-> dense on the GPU (through the C ABI) against the CPU restatement, for every
dtype and for row widths that exercise the 16- / 4- / 2- / 1-byte copy paths."""
import numpy as np
import pytest
import torch

from oracle import tensor_np
from sphconv_b200 import check_status
from sphconv_b200 import sphconv_cuda as ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _coo(rng, B, shape, dens):
    occ = rng.random((B, *shape)) < dens
    idx = np.stack(np.nonzero(occ), axis=1).astype(np.int32)
    rng.shuffle(idx)
    return idx


@pytest.mark.parametrize("dtype,C", [(torch.float32, 4), (torch.float32, 5), (torch.float16, 8), (torch.float16, 3),
                                     (torch.bfloat16, 64), (torch.int8, 7), (torch.int8, 32), (torch.float64, 2)])
def test_ops_match_oracle(dtype, C):
    rng = np.random.default_rng(C + 1)
    B, shape = 3, [6, 9, 70]
    idx = _coo(rng, B, shape, 0.2)
    if dtype == torch.int8:
        feat = torch.as_tensor(rng.integers(-100, 100, (idx.shape[0], C)), dtype=dtype)
    else:
        feat = torch.as_tensor(rng.standard_normal((idx.shape[0], C))).to(dtype)
    want_f, want_zi, want_zp, want_perm = tensor_np.init_tensor(feat.view(torch.uint8).numpy().reshape(idx.shape[0], -1),
                                                                idx, B, shape)
    f2, z_idx, z_ptr, perm = ops.init_tensor(feat.to(DEV), torch.as_tensor(idx, device=DEV), B, shape)
    assert (z_idx.cpu().numpy() == want_zi).all() and (z_ptr.cpu().numpy() == want_zp).all()
    assert (perm.cpu().numpy() == want_perm).all()
    assert (f2.cpu().view(torch.uint8).numpy().reshape(idx.shape[0], -1) == want_f).all()
    dense = torch.zeros((B, *shape, C), dtype=dtype, device=DEV)
    ops.to_dense(f2, z_idx, z_ptr, shape[2], dense)
    want_dense = tensor_np.to_dense(want_f, want_zi, want_zp, B, shape)
    assert (dense.cpu().view(torch.uint8).numpy().reshape(want_dense.shape) == want_dense).all()
    # backwards (pure row moves: bit-exact for every dtype)
    g = dense * 0 + torch.as_tensor(rng.integers(-3, 4, tuple(dense.shape)), device=DEV).to(dtype)
    rows_g = ops.to_dense_backward(g, z_idx, z_ptr)
    want_rows_g = tensor_np.to_dense_backward(g.cpu().view(torch.uint8).numpy().reshape(want_dense.shape), want_zi, want_zp)
    assert (rows_g.cpu().view(torch.uint8).numpy().reshape(want_rows_g.shape) == want_rows_g).all()
    back = ops.init_tensor_backward(rows_g, perm)
    want_back = tensor_np.init_tensor_backward(want_rows_g, want_perm)
    assert (back.cpu().view(torch.uint8).numpy().reshape(want_back.shape) == want_back).all()
    assert check_status() == 0


def test_empty_and_bad_coordinates():
    f2, z_idx, z_ptr, perm = ops.init_tensor(torch.zeros((0, 4), device=DEV), torch.zeros((0, 4), dtype=torch.int32, device=DEV),
                                             2, [3, 4, 5])
    assert f2.shape == (0, 4) and (z_ptr.cpu().numpy() == 0).all()
    idx = torch.tensor([[0, 1, 2, 3], [0, 1, 2, 9], [5, 0, 0, 0]], dtype=torch.int32, device=DEV)   # two rows out of range
    f2, z_idx, z_ptr, perm = ops.init_tensor(torch.ones((3, 2), device=DEV), idx, 2, [3, 4, 5])
    assert perm.cpu().tolist() == [0, -1, -1] and int(z_ptr.reshape(-1)[-1]) == 1
    with pytest.raises(RuntimeError):      # SPH_STATUS_BAD_INDEX is reported (and cleared) by the status read
        check_status()
    assert check_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("C,n", [(16, 1000), (64, 12345), (32, 7), (128, 300)])
def test_epilogue_backward(dtype, C, n):
    """Gradient mask of relu(acc + bias) and the bias gradient in one pass, against the torch expressions."""
    g = torch.Generator(device=DEV).manual_seed(C + n)
    out = torch.relu(torch.randn((n, C), generator=g, device=DEV)).to(dtype)
    d_out = torch.randn((n, C), generator=g, device=DEV).to(dtype)
    for relu in (True, False):
        d_pre, d_bias = ops.epilogue_backward(d_out, out, relu, True)
        want = torch.where(out > 0, d_out, torch.zeros((), dtype=dtype, device=DEV)) if relu else d_out
        assert torch.equal(d_pre, want)
        ref = want.double().sum(0)
        assert torch.allclose(d_bias.double(), ref, rtol=1e-4, atol=1e-3 * max(1.0, float(ref.abs().max())))
    d_pre, d_bias = ops.epilogue_backward(d_out, out, True, False)
    assert d_bias is None and torch.equal(d_pre, torch.where(out > 0, d_out, torch.zeros((), dtype=dtype, device=DEV)))
