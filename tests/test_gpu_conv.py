"""Rule-driven convolution on the GPU (forward, dgrad, wgrad) against the CPU oracle.

Tolerances: fp32 |y - ref| <= 1e-4 * max(|ref|, 1); fp16 / bf16 1e-2 * max(|ref|, 1) against the
oracle evaluated in float64 on the same 16-bit-rounded operands; int8 exact (integer accumulation)
against the integer oracle.  Channel sweep follows test/test_conv.py of the reference (4->4 ... 64->64,
oC = 5, batch 1 and 8, submanifold and strided)."""
import numpy as np
import pytest
import torch

from oracle import conv_np, rules_np
from sphconv_b200 import check_status, synthetic
from sphconv_b200 import sphconv_cuda as ops

from gpu_util import DEV, gpu_rules, oracle_rules

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.float16: 1e-2, torch.bfloat16: 1e-2}


def _close(got, ref, tol):
    got = got.double().cpu().numpy()
    err = np.abs(got - ref)
    bound = tol * np.maximum(np.abs(ref), 1.0)
    assert (err <= bound).all(), "max err %g (bound %g at that element)" % (err.max(), bound.reshape(-1)[err.argmax()])


def _setup(B, shape, subm, dens, seed, iC, oC, dtype, ks=(3, 3, 3), stride=2):
    rng = np.random.default_rng(seed)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, dens)
    ks = list(ks)
    st, pd = ([1, 1, 1], [k // 2 for k in ks]) if subm else ([stride] * 3, [1, 1, 1])
    with torch.enable_grad():
        zi, zp, osh, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, [2, 2], subm)
    res = oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, [2, 2], subm)
    pairs = rules_np.canonical_from_table(res)
    kv = int(np.prod(ks))
    if dtype == torch.int8:
        feat = torch.as_tensor(rng.integers(-127, 128, size=(z_idx.shape[0], iC)), dtype=torch.int8, device=DEV)
        w = torch.as_tensor(rng.integers(-127, 128, size=(kv, iC, oC)), dtype=torch.int8, device=DEV)
    else:
        feat = torch.as_tensor(rng.standard_normal((z_idx.shape[0], iC)), dtype=torch.float32, device=DEV).to(dtype)
        w = torch.as_tensor(rng.uniform(-1, 1, size=(kv, iC, oC)) / np.sqrt(iC * 4), dtype=torch.float32, device=DEV).to(dtype)
    return rng, feat, w, rules, rule_size, pairs, z_idx.shape[0], oz_idx.shape[0]


CH = [(4, 4), (8, 8), (16, 16), (32, 32), (64, 64), (16, 32), (32, 64), (64, 32), (16, 5), (5, 16), (3, 7), (128, 128)]


@pytest.mark.parametrize("iC,oC", CH)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("subm", [True, False])
def test_forward(iC, oC, dtype, subm):
    B, shape = 2, [10, 24, 16]
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, subm, 0.25, 5, iC, oC, dtype)
    out = ops.rule_conv(feat, w, rules, rule_size, n_out)
    assert out.dtype == dtype and tuple(out.shape) == (n_out, oC)
    ref = conv_np.conv_forward(feat.double().cpu().numpy(), w.double().cpu().numpy(), pairs, n_out)
    _close(out, ref, TOL[dtype])
    assert check_status() == 0


@pytest.mark.parametrize("iC,oC", [(16, 16), (32, 64), (64, 64), (32, 16), (5, 16)])
@pytest.mark.parametrize("subm", [True, False])
def test_forward_int8_exact(iC, oC, subm):
    B, shape = 2, [10, 24, 16]
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, subm, 0.25, 6, iC, oC, torch.int8)
    out = ops.rule_conv(feat, w, rules, rule_size, n_out)            # float32 = exact integer sums
    ref = conv_np.conv_forward(feat.cpu().numpy(), w.cpu().numpy(), pairs, n_out, dtype=np.int64)
    assert out.dtype == torch.float32
    assert (out.cpu().numpy().astype(np.int64) == ref).all()
    # quantised epilogue: per-channel scale + bias + ReLU, int8 output with round-to-nearest and saturation at +-127
    scale = torch.as_tensor(rng.uniform(1e-4, 3e-4, size=oC), dtype=torch.float32, device=DEV)
    bias = torch.as_tensor(rng.uniform(-20, 20, size=oC), dtype=torch.float32, device=DEV)
    q = ops.rule_conv(feat, w, rules, rule_size, n_out, scale=scale, bias=bias, relu=True, out_dtype=torch.int8)
    want = np.maximum(ref.astype(np.float32) * scale.cpu().numpy() + bias.cpu().numpy(), 0)
    want = np.clip(np.rint(want), -127, 127).astype(np.int8)
    diff = np.abs(q.cpu().numpy().astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3      # ties at .5 may round differently in float32


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("iC,oC", [(16, 16), (64, 64), (16, 5), (32, 32), (32, 128)])
def test_forward_epilogue_and_out_dtype(dtype, iC, oC):
    B, shape = 1, [8, 16, 12]
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, True, 0.3, 8, iC, oC, dtype)
    bias = torch.as_tensor(rng.standard_normal(oC), dtype=torch.float32, device=DEV)
    scale = torch.as_tensor(rng.uniform(0.5, 2, size=oC), dtype=torch.float32, device=DEV)
    out = ops.rule_conv(feat, w, rules, rule_size, n_out, scale=scale, bias=bias, relu=True, out_dtype=torch.float32)
    ref = conv_np.conv_forward(feat.double().cpu().numpy(), w.double().cpu().numpy(), pairs, n_out)
    ref = np.maximum(ref * scale.double().cpu().numpy() + bias.double().cpu().numpy(), 0)
    assert out.dtype == torch.float32
    _close(out, ref, TOL[dtype])


@pytest.mark.parametrize("iC,oC", [(4, 4), (16, 16), (32, 64), (64, 64), (16, 5)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("subm,ks", [(True, (3, 3, 3)), (False, (3, 3, 3)), (True, (2, 2, 2)), (False, (2, 3, 2))])
def test_backward(iC, oC, dtype, subm, ks):
    B, shape = 2, [9, 14, 12]
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, subm, 0.3, 9, iC, oC, dtype, ks=ks)
    dout = torch.as_tensor(rng.standard_normal((n_out, oC)), dtype=torch.float32, device=DEV).to(dtype)
    kv = w.shape[0]
    d_feature, d_weight = ops.rule_conv_backward(dout, feat, w.permute(0, 2, 1).contiguous(), rules, rule_size,
                                                 [1, 1])
    assert tuple(d_feature.shape) == (n_in, iC) and tuple(d_weight.shape) == (kv, iC, oC)
    ref_dx = conv_np.conv_dgrad(dout.double().cpu().numpy(), w.double().cpu().numpy(), pairs, n_in)
    ref_dw = conv_np.conv_wgrad(feat.double().cpu().numpy(), dout.double().cpu().numpy(), pairs, kv)
    _close(d_feature, ref_dx, TOL[dtype])
    # weight gradient is accumulated in fp32 and returned in the feature dtype; bound relative to the largest entry
    got = d_weight.double().cpu().numpy()
    scale = max(np.abs(ref_dw).max(), 1.0)
    assert np.abs(got - ref_dw).max() <= TOL[dtype] * scale
    assert check_status() == 0


def test_foreign_rules_forward_and_backward():
    """Rules that did not come from this library (a clone drops the attached tables): every op converts them."""
    B, shape, iC, oC = 2, [8, 12, 10], 16, 16
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, False, 0.3, 12, iC, oC, torch.float16)
    r2, s2 = rules.clone(), rule_size.clone()
    out = ops.rule_conv(feat, w, r2, s2, n_out)
    assert torch.equal(out, ops.rule_conv(feat, w, rules, rule_size, n_out))
    dout = torch.as_tensor(rng.standard_normal((n_out, oC)), dtype=torch.float16, device=DEV)
    r3 = rules.clone()
    a = ops.rule_conv_backward(dout, feat, w.permute(0, 2, 1).contiguous(), r3, s2, [1, 1])
    b = ops.rule_conv_backward(dout, feat, w.permute(0, 2, 1).contiguous(), rules, rule_size, [1, 1])
    assert torch.equal(a[0], b[0])
    assert torch.allclose(a[1].float(), b[1].float(), rtol=1e-2, atol=1e-2)


def test_large_magnitudes():
    """test/test_stable.py of the reference: inputs and weights of magnitude ~100 (fp32 path, relative bound)."""
    B, shape, iC, oC = 1, [8, 12, 10], 64, 64
    rng, feat, w, rules, rule_size, pairs, n_in, n_out = _setup(B, shape, False, 0.3, 13, iC, oC, torch.float32)
    feat = feat * 100
    w = w * 100
    out = ops.rule_conv(feat, w, rules, rule_size, n_out)
    ref = conv_np.conv_forward(feat.double().cpu().numpy(), w.double().cpu().numpy(), pairs, n_out)
    assert np.abs(out.double().cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()


def test_tensor_core_path_is_selected():
    from sphconv_b200 import _capi as C
    lib = C.lib()
    assert lib.sph_conv_uses_tensor_cores(C.SPH_F16, 64, 64) == 1
    assert lib.sph_conv_uses_tensor_cores(C.SPH_BF16, 16, 32) == 1
    assert lib.sph_conv_uses_tensor_cores(C.SPH_I8, 32, 64) == 1
    assert lib.sph_conv_uses_tensor_cores(C.SPH_F32, 64, 64) == 0
    assert lib.sph_conv_uses_tensor_cores(C.SPH_F16, 4, 16) == 0
    # narrow rows of the first layer and small fp32 layers: the pair-compacting CUDA-core kernel
    assert lib.sph_conv_uses_pair_kernel(C.SPH_F16, 4, 16) == 1
    assert lib.sph_conv_uses_pair_kernel(C.SPH_F32, 16, 16) == 1
    assert lib.sph_conv_uses_pair_kernel(C.SPH_F16, 64, 64) == 0
    assert lib.sph_conv_uses_pair_kernel(C.SPH_F16, 5, 16) == 0


@pytest.mark.parametrize("dtype,iC,oC", [(torch.float16, 64, 64), (torch.bfloat16, 32, 64), (torch.int8, 64, 64),
                                         (torch.float16, 16, 16)])
def test_forward_many_blocks(dtype, iC, oC):
    """Enough output rows for several row blocks per CTA (persistent loop, both accumulator buffers, ring wrap)."""
    cfg = dict(synthetic.CONFIGS["cfg2"])
    b = synthetic.make_batch(cfg, batch=2)
    z_idx, z_ptr, shape = b["z_idx"], b["z_ptr"], cfg["shape"]
    zi, zp, osh, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, 2, shape, [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2], True)
    res = oracle_rules(z_idx, z_ptr, 2, shape, [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2], True)
    pairs = rules_np.canonical_from_table(res)
    rng = np.random.default_rng(21)
    n = z_idx.shape[0]
    if dtype == torch.int8:
        feat = torch.as_tensor(rng.integers(-127, 128, size=(n, iC)), dtype=torch.int8, device=DEV)
        w = torch.as_tensor(rng.integers(-127, 128, size=(27, iC, oC)), dtype=torch.int8, device=DEV)
        out = ops.rule_conv(feat, w, rules, rule_size, n)
        ref = conv_np.conv_forward(feat.cpu().numpy(), w.cpu().numpy(), pairs, n, dtype=np.int64)
        assert (out.cpu().numpy().astype(np.int64) == ref).all()
    else:
        feat = torch.as_tensor(rng.standard_normal((n, iC)), dtype=torch.float32, device=DEV).to(dtype)
        w = torch.as_tensor(rng.uniform(-1, 1, size=(27, iC, oC)) / np.sqrt(iC * 4), dtype=torch.float32, device=DEV).to(dtype)
        out = ops.rule_conv(feat, w, rules, rule_size, n)
        ref = conv_np.conv_forward(feat.double().cpu().numpy(), w.double().cpu().numpy(), pairs, n)
        _close(out, ref, TOL[dtype])
    assert check_status() == 0
