"""The pair-compacting CUDA-core kernel (narrow rows of a sparse first level, small fp32 layers) against the CPU oracle,
through the same entry point as every other convolution: shapes the tensor-core kernels do not take route to it.

Cases: 4/8/16/32 channels in and out, fp16 / bf16 / fp32, submanifold and strided tables, nearly empty and completely
full grids (a full grid lists 27 items per row: every batch of 32 items is followed by a remainder, and consecutive
offsets name the same output row inside one pass), a kernel volume above 32 (the table is read in several groups),
output row counts that are not a multiple of 32, the fused epilogue with every output dtype, and dgrad (the flipped
table of a submanifold layer, the transposed table of a strided one)."""
import numpy as np
import pytest
import torch

from oracle import conv_np
from sphconv_b200 import check_status
from sphconv_b200 import sphconv_cuda as ops

from gpu_util import DEV
from test_gpu_conv import TOL, _close, _setup

pytestmark = pytest.mark.gpu

NARROW = [(4, 16), (16, 4), (8, 16), (4, 32), (32, 4), (8, 8), (4, 4)]


@pytest.mark.parametrize("iC,oC", NARROW)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("subm,dens", [(True, 0.02), (True, 0.3), (True, 1.0), (False, 0.05), (False, 1.0)])
def test_forward_narrow_rows(iC, oC, dtype, subm, dens):
    B, shape = 2, [9, 21, 13]
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, subm, dens, 31, iC, oC, dtype)
    out = ops.rule_conv(feat, w, rules, rule_size, n_out)
    assert out.dtype == dtype and tuple(out.shape) == (n_out, oC)
    ref = conv_np.conv_forward(feat.double().cpu().numpy(), w.double().cpu().numpy(), pairs, n_out)
    _close(out, ref, TOL[dtype])
    assert check_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("subm,ks", [(True, (5, 3, 3)), (False, (3, 5, 3)), (True, (5, 5, 5))])
def test_forward_kernel_volume_above_32(dtype, subm, ks):
    B, shape = 1, [8, 14, 12]
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, subm, 0.4, 32, 4, 16, dtype, ks=ks)
    out = ops.rule_conv(feat, w, rules, rule_size, n_out)
    ref = conv_np.conv_forward(feat.double().cpu().numpy(), w.double().cpu().numpy(), pairs, n_out)
    _close(out, ref, TOL[dtype])
    assert check_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("iC,oC", [(4, 16), (16, 4), (8, 32)])
def test_epilogue_and_out_dtype(dtype, out_dtype, iC, oC):
    B, shape = 1, [8, 16, 12]
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, True, 0.3, 33, iC, oC, dtype)
    bias = torch.as_tensor(rng.standard_normal(oC), dtype=torch.float32, device=DEV)
    scale = torch.as_tensor(rng.uniform(0.5, 2, size=oC), dtype=torch.float32, device=DEV)
    out = ops.rule_conv(feat, w, rules, rule_size, n_out, scale=scale, bias=bias, relu=True, out_dtype=out_dtype)
    ref = conv_np.conv_forward(feat.double().cpu().numpy(), w.double().cpu().numpy(), pairs, n_out)
    ref = np.maximum(ref * scale.double().cpu().numpy() + bias.double().cpu().numpy(), 0)
    assert out.dtype == out_dtype
    _close(out, ref, max(TOL[dtype], TOL[out_dtype]))
    assert check_status() == 0


@pytest.mark.parametrize("iC,oC", [(4, 16), (16, 8)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("subm", [True, False])
def test_dgrad_narrow_rows(iC, oC, dtype, subm):
    B, shape = 2, [9, 21, 13]
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, subm, 0.3, 34, iC, oC, dtype)
    dout = torch.as_tensor(rng.standard_normal((n_out, oC)), dtype=torch.float32, device=DEV).to(dtype)
    dfeat = ops.rule_conv_d_feature(dout, w.permute(0, 2, 1).contiguous(), rules, rule_size, [1, 1], n_in)
    assert tuple(dfeat.shape) == (n_in, iC)
    ref = conv_np.conv_dgrad(dout.double().cpu().numpy(), w.double().cpu().numpy(), pairs, n_in)
    _close(dfeat, ref, TOL[dtype])
    assert check_status() == 0


@pytest.mark.parametrize("iC,oC", [(4, 16), (16, 16), (16, 32), (8, 8), (16, 4)])
@pytest.mark.parametrize("subm,dens", [(True, 0.05), (True, 1.0), (False, 0.3)])
def test_int8_narrow_rows_exact(iC, oC, subm, dens):
    """int8 rows narrower than 32 bytes: products summed in fp32 (exact below 2^24), integer oracle, then the quantised
    epilogue with int8 output."""
    B, shape = 2, [9, 21, 13]
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, subm, dens, 35, iC, oC, torch.int8)
    out = ops.rule_conv(feat, w, rules, rule_size, n_out)
    ref = conv_np.conv_forward(feat.cpu().numpy(), w.cpu().numpy(), pairs, n_out, dtype=np.int64)
    assert out.dtype == torch.float32
    assert (out.cpu().numpy().astype(np.int64) == ref).all()
    scale = torch.as_tensor(rng.uniform(1e-4, 3e-4, size=oC), dtype=torch.float32, device=DEV)
    bias = torch.as_tensor(rng.uniform(-20, 20, size=oC), dtype=torch.float32, device=DEV)
    q = ops.rule_conv(feat, w, rules, rule_size, n_out, scale=scale, bias=bias, relu=True, out_dtype=torch.int8)
    want = np.maximum(ref.astype(np.float32) * scale.cpu().numpy() + bias.cpu().numpy(), 0)
    want = np.clip(np.rint(want), -127, 127).astype(np.int8)
    diff = np.abs(q.cpu().numpy().astype(np.int32) - want.astype(np.int32))
    assert q.dtype == torch.int8 and diff.max() <= 1 and (diff != 0).mean() < 1e-3   # ties at .5 may round differently
    assert check_status() == 0


@pytest.mark.parametrize("iC,oC", [(4, 16), (16, 4), (8, 8), (4, 4), (16, 32), (32, 16)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("subm,dens,ks", [(True, 0.05, (3, 3, 3)), (True, 1.0, (3, 3, 3)), (False, 0.3, (3, 3, 3)),
                                          (True, 0.4, (5, 3, 3))])
def test_wgrad_narrow_rows(iC, oC, dtype, subm, dens, ks):
    """Weight gradient of the narrow layers (the pair-compacting walk where the tensor-core kernel does not take the
    shape; 16x32 / 32x16 take it in fp32 only) against the float64 oracle, fp32 accumulation checked in place."""
    B, shape = 2, [9, 17, 13]
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, subm, dens, 36, iC, oC, dtype, ks=ks)
    dout = torch.as_tensor(rng.standard_normal((n_out, oC)), dtype=torch.float32, device=DEV).to(dtype)
    kv = w.shape[0]
    buf = torch.full((kv, iC, oC), 0.5, dtype=torch.float32, device=DEV)
    ops.rule_conv_d_weight(feat, dout, rules, rule_size, out=buf, accumulate=True)      # adds to what the buffer holds
    ref = conv_np.conv_wgrad(feat.double().cpu().numpy(), dout.double().cpu().numpy(), pairs, kv)
    got = buf.double().cpu().numpy() - 0.5
    scale = max(np.abs(ref).max(), 1.0)
    assert np.abs(got - ref).max() <= TOL[dtype] * scale
    assert check_status() == 0
