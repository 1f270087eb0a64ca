"""The 8-layer SECOND-style encoder end to end on the GPU: fp16 and bf16 inference against the fp32 dense
conv3d stack (rel-L2 <= 1e-2), training gradients against autograd through the dense stack, and the int8
variant against fp32 (rel-L2 <= 1e-1 after eight requantised layers, the stated bound)."""
import numpy as np
import pytest
import torch

import sphconv_b200 as sphconv
from oracle import dense_ref
from sphconv_b200 import quant, synthetic
from sphconv_b200.encoder import build_encoder8, encoder8_parameters

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SMALL = dict(id=3, B=2, shape=[16, 32, 64], occ=0.9, nbins="uniform", nmax=4, depth="lognormal", C=4)


def _batch(B=2):
    b = synthetic.make_batch(SMALL, batch=B)
    return b


def _tensor(b, dtype, requires_grad=False):
    f = torch.as_tensor(b["feature"], device=DEV).to(dtype)
    if requires_grad:
        f.requires_grad_(True)
    return sphconv.SparseConvTensor(f, b["shape"], b["B"], z_idx=torch.as_tensor(b["z_idx"], device=DEV),
                                    z_ptr=torch.as_tensor(b["z_ptr"], device=DEV))


def _rel_l2(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_encoder_inference_vs_dense(dtype):
    b = _batch()
    net = build_encoder8(dtype=dtype, device=DEV).eval()
    with torch.no_grad():
        y = net(_tensor(b, dtype))
    # fp32 dense stack fed the same 16-bit-rounded weights and inputs
    params = [(m.weight.detach().float().cpu().numpy(), m.bias.detach().float().cpu().numpy())
              for m in net._modules.values()]
    feat = torch.as_tensor(b["feature"]).to(dtype).float().numpy()
    ref, mask = dense_ref.encoder_dense_forward(feat, b["z_idx"], b["z_ptr"], b["B"], b["shape"], synthetic.ENCODER8, params)
    got = y.dense().float().cpu()
    assert got.shape == ref.shape
    assert ((got != 0) <= mask).all()
    assert _rel_l2(got, ref) <= 1e-2
    assert sphconv.check_status() == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-3), (torch.bfloat16, 1e-1)])
def test_encoder_training_step_vs_dense_autograd(dtype, tol):
    """Forward + backward of all eight layers against autograd through the dense fp32 stack on the same
    (rounded) parameters.  fp32 must agree tightly.  For bf16 the per-layer 1e-2 bound is checked in
    test_gpu_conv.py; across eight layers a rounded activation near zero can flip a ReLU and reroute a gradient
    path, so the end-to-end bound is looser."""
    b = _batch(1)
    net = build_encoder8(dtype=dtype, device=DEV).train()
    x = _tensor(b, dtype, requires_grad=True)
    y = net(x)
    g = torch.as_tensor(np.random.default_rng(1).standard_normal(tuple(y.feature.shape)), device=DEV).to(dtype)
    y.feature.backward(g)
    ws = [m.weight.detach().float().cpu().requires_grad_(True) for m in net._modules.values()]
    bs = [m.bias.detach().float().cpu().requires_grad_(True) for m in net._modules.values()]
    feat = torch.as_tensor(b["feature"]).to(dtype).float().requires_grad_(True)
    B, shape = b["B"], b["shape"]
    from oracle.rules_np import row_coords
    bb, xx, yy, zz = [torch.as_tensor(a) for a in row_coords(b["z_idx"], b["z_ptr"], B, *shape[:2])]
    d = torch.zeros((B, shape[0], shape[1], shape[2], 4)).index_put((bb, xx, yy, zz), feat).permute(0, 4, 1, 2, 3)
    mask = torch.zeros((B, 1, *shape)).index_put((bb, torch.zeros_like(bb), xx, yy, zz), torch.ones(bb.shape[0])) != 0
    for (subm, iC, oC, stride, key), w, bias in zip(synthetic.ENCODER8, ws, bs):
        wd = w.permute(4, 3, 0, 1, 2)
        if subm:
            d = torch.nn.functional.conv3d(d, wd, None, 1, 1)
        else:
            d = torch.nn.functional.conv3d(d, wd, None, stride, 1)
            mask = torch.nn.functional.conv3d(mask.float(), torch.ones((1, 1, 3, 3, 3)), None, stride, 1) != 0
        d = torch.relu(d + bias.view(1, -1, 1, 1, 1)) * mask
    gd = sphconv.SparseConvTensor(g.float(), [y.D, y.W, y.H], B, z_idx=y.z_idx, z_ptr=y.z_ptr).dense().cpu()
    d.backward(gd)
    errs = {"y": _rel_l2(y.dense().float().cpu(), d.detach()), "dx": _rel_l2(x.feature.grad.float().cpu(), feat.grad)}
    for li, (m, w) in enumerate(zip(net._modules.values(), ws)):
        errs["dw%d" % li] = _rel_l2(m.weight.grad.float().cpu(), w.grad)
    assert max(errs.values()) <= tol, errs
    assert sphconv.check_status() == 0


def test_master_gradient_buffer_keeps_fp32_weight_gradients():
    """bf16 training with a sharding.GradBuffer attached: the wgrad kernels accumulate into the flat fp32 buffer (no
    `.grad` comes through autograd, nothing is rounded to bf16), two backward passes add up, and the buffer equals the
    fp32 result of the op called directly on the same operands."""
    from sphconv_b200 import sharding
    b = _batch(1)
    net = build_encoder8(dtype=torch.bfloat16, device=DEV).train()
    gb = sharding.GradBuffer(net.parameters())
    caught = []
    import sphconv_b200.functional as F
    orig = F.rule_conv_d_weight

    def spy(feature, d_out, rules, rule_size, **kw):
        caught.append(orig(feature, d_out, rules, rule_size))      # the same operands, into a fresh fp32 tensor
        return orig(feature, d_out, rules, rule_size, **kw)
    F.rule_conv_d_weight = spy
    try:
        for rep in range(2):
            x = _tensor(b, torch.bfloat16, requires_grad=True)
            y = net(x)
            g = torch.as_tensor(np.random.default_rng(1).standard_normal(tuple(y.feature.shape)), device=DEV).bfloat16()
            y.feature.backward(g)
    finally:
        F.rule_conv_d_weight = orig
    mods = list(net._modules.values())
    assert all(m.weight.grad is None and m.bias.grad is None for m in mods)
    assert len(caught) == 16
    for li, m in enumerate(mods):               # backward visits the layers last to first
        direct = caught[len(mods) - 1 - li] + caught[2 * len(mods) - 1 - li]
        got = m.weight._sph_master_grad.view(27, m.in_channels, m.out_channels)
        assert got.dtype == torch.float32
        assert _rel_l2(got, direct) <= 1e-5, li
        assert float(m.bias._sph_master_grad.abs().sum()) > 0
    gb.to_grads()
    assert all(m.weight.grad.dtype == torch.bfloat16 for m in mods)
    gb.detach()
    assert sphconv.check_status() == 0


def test_int8_encoder_vs_fp32():
    b = _batch()
    net32 = build_encoder8(dtype=torch.float32, device=DEV).eval()
    with torch.no_grad():
        qenc = quant.quantize_encoder(net32, _tensor(_batch(1), torch.float32))
        x = _tensor(b, torch.float32)
        ref = net32(_tensor(b, torch.float32))
        xq = sphconv.SparseConvTensor(qenc.quantize_input(x.feature), b["shape"], b["B"], z_idx=x.z_idx, z_ptr=x.z_ptr)
        y = qenc(xq)
    assert y.feature.dtype == torch.float32 and y.feature.shape == ref.feature.shape
    assert torch.equal(y.z_idx, ref.z_idx)
    assert _rel_l2(y.feature, ref.feature) <= 1e-1
    assert sphconv.check_status() == 0
