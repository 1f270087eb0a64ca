"""Module-level API (SparseConvTensor, SubMConv3d, Conv3d, Sequential, autograd) against dense torch conv3d,
the ground truth of the reference's test/test_module.py, test/test_grad.py and test/test_util.py."""
import numpy as np
import pytest
import torch

import sphconv_b200 as sphconv
from oracle import dense_ref
from sphconv_b200 import synthetic

from gpu_util import DEV

pytestmark = pytest.mark.gpu


def _coo(rng, B, shape, dens):
    occ = rng.random((B, *shape)) < dens
    idx = np.stack(np.nonzero(occ), axis=1).astype(np.int32)
    rng.shuffle(idx)                       # COO rows in arbitrary order
    return idx


def test_init_tensor_and_dense_roundtrip():
    rng = np.random.default_rng(0)
    B, shape, C = 3, [6, 7, 9], 5
    idx = _coo(rng, B, shape, 0.3)
    feat = rng.standard_normal((idx.shape[0], C)).astype(np.float32)
    t = sphconv.SparseConvTensor(torch.as_tensor(feat, device=DEV), shape, B, indices=torch.as_tensor(idx, device=DEV))
    # the reference's shape property is [B, C, D, H, W] with (D, W, H) = (s0, s1, s2) (sphconv/tensor.py:104-106)
    assert t.shape == [B, C, shape[0], shape[2], shape[1]]
    dense = t.dense().cpu()
    want = torch.zeros((B, C, *shape))
    want[idx[:, 0], :, idx[:, 1], idx[:, 2], idx[:, 3]] = torch.as_tensor(feat)
    assert torch.equal(dense, want)
    zp = t.z_ptr.cpu().numpy().reshape(-1)
    assert zp[-1] == idx.shape[0] and (np.diff(zp) >= 0).all()
    # gradient flows through dense() and the COO reorder back to the raw rows
    raw = torch.as_tensor(feat, device=DEV).requires_grad_(True)
    t2 = sphconv.SparseConvTensor(raw, shape, B, indices=torch.as_tensor(idx, device=DEV))
    g = torch.as_tensor(rng.standard_normal((B, C, *shape)).astype(np.float32), device=DEV)
    (t2.dense() * g).sum().backward()
    want_g = g.cpu()[idx[:, 0], :, idx[:, 1], idx[:, 2], idx[:, 3]]
    assert torch.allclose(raw.grad.cpu(), want_g)


@pytest.mark.parametrize("subm", [True, False])
@pytest.mark.parametrize("iC,oC", [(4, 16), (16, 16), (32, 64)])
def test_module_forward_backward_vs_dense(subm, iC, oC):
    rng = np.random.default_rng(1)
    B, shape = 2, [8, 10, 12]
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3)
    feat = rng.standard_normal((z_idx.shape[0], iC)).astype(np.float32)
    if subm:
        layer = sphconv.SubMConv3d(iC, oC, 3, bias=False).to(DEV)
        st, pd = [1, 1, 1], [1, 1, 1]
    else:
        layer = sphconv.Conv3d(iC, oC, 3, stride=2, padding=1, bias=False).to(DEV)
        st, pd = [2, 2, 2], [1, 1, 1]
    f = torch.as_tensor(feat, device=DEV).requires_grad_(True)
    x = sphconv.SparseConvTensor(f, shape, B, z_idx=torch.as_tensor(z_idx, device=DEV), z_ptr=torch.as_tensor(z_ptr, device=DEV))
    y = layer(x)
    yd = y.dense()
    w5 = layer.weight.detach().cpu().numpy()
    up = rng.standard_normal(tuple(yd.shape)).astype(np.float32)
    if subm:   # gradient only at active sites
        mask = (dense_ref.densify(np.ones((z_idx.shape[0], 1), np.float32), z_idx, z_ptr, B, shape) != 0).numpy()
        up = up * mask
    (yd * torch.as_tensor(up, device=DEV)).sum().backward()
    ref_y, ref_dx, ref_dw = dense_ref.dense_conv_grads(feat, w5, lambda t: torch.as_tensor(up).double(), z_idx, z_ptr,
                                                       B, shape, st, pd)
    if subm:
        ref_y = ref_y * torch.as_tensor(mask)
    assert torch.allclose(yd.cpu().double(), ref_y, atol=1e-4)
    assert torch.allclose(f.grad.cpu().double(), ref_dx, atol=1e-4)
    assert torch.allclose(layer.weight.grad.cpu().double(), ref_dw, atol=1e-3)


def test_sequential_rule_cache_and_dense_modules():
    rng = np.random.default_rng(2)
    B, shape = 2, [8, 10, 12]
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3)
    feat = torch.as_tensor(rng.standard_normal((z_idx.shape[0], 4)).astype(np.float32), device=DEV)
    net = sphconv.Sequential(
        sphconv.SubMConv3d(4, 16, 3, indice_key="subm0"), torch.nn.ReLU(),
        sphconv.SubMConv3d(16, 16, 3, indice_key="subm0"), torch.nn.ReLU(),
        sphconv.SparseConv3d(16, 32, 3, stride=2, padding=1),
    ).to(DEV)
    x = sphconv.SparseConvTensor(feat, shape, B, z_idx=torch.as_tensor(z_idx, device=DEV), z_ptr=torch.as_tensor(z_ptr, device=DEV))
    with torch.no_grad():
        y = net(x)
    assert "subm0" in y.rule_cache and len(y.rule_cache) == 1
    assert y.feature.shape[1] == 32 and [y.D, y.W, y.H] == [4, 5, 6]
    # dense reference of the same stack
    d = dense_ref.densify(feat.cpu().numpy(), z_idx, z_ptr, B, shape)
    mask = dense_ref.densify(np.ones((z_idx.shape[0], 1), np.float32), z_idx, z_ptr, B, shape) != 0
    convs = [m for m in net._modules.values() if isinstance(m, sphconv.Conv3d)]
    for i, m in enumerate(convs):
        w = m.weight.detach().cpu().permute(4, 3, 0, 1, 2).contiguous()
        if m.subm:
            d = torch.relu(torch.nn.functional.conv3d(d, w, None, 1, 1)) * mask
        else:
            d = torch.nn.functional.conv3d(d, w, None, 2, 1)
    assert torch.allclose(y.dense().cpu(), d, atol=1e-4)


def test_fused_bias_relu_extension_matches_unfused():
    rng = np.random.default_rng(3)
    B, shape = 1, [8, 10, 12]
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3)
    feat = torch.as_tensor(rng.standard_normal((z_idx.shape[0], 16)).astype(np.float32), device=DEV).half()
    layer = sphconv.SubMConv3d(16, 32, 3, bias=True, apply_bias=True, activation='relu').to(DEV).half()
    plain = sphconv.SubMConv3d(16, 32, 3, bias=True).to(DEV).half()
    plain.load_state_dict(layer.state_dict())
    mk = lambda: sphconv.SparseConvTensor(feat, shape, B, z_idx=torch.as_tensor(z_idx, device=DEV), z_ptr=torch.as_tensor(z_ptr, device=DEV))
    with torch.no_grad():
        fused = layer(mk()).feature
        ref = torch.relu(plain(mk()).feature.float() + plain.bias.float())
    assert torch.allclose(fused.float(), ref, atol=2e-2, rtol=1e-2)
    # the reference applies no bias by default (sphconv/conv.py:182-185)
    with torch.no_grad():
        assert not torch.allclose(plain(mk()).feature.float(), ref)


def test_sequential_starts_strided_rules_ahead():
    """Sequential enqueues the first step of a strided layer's rule generation before the submanifold layer in front
    of it runs; outputs and rules are those of the layers called one by one."""
    from sphconv_b200 import sphconv_cuda as ops
    rng = np.random.default_rng(31)
    B, shape = 2, [12, 20, 16]
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.25)
    feat = torch.as_tensor(rng.standard_normal((z_idx.shape[0], 16)), dtype=torch.float16, device=DEV)
    zi, zp = torch.as_tensor(z_idx, device=DEV), torch.as_tensor(z_ptr, device=DEV)
    torch.manual_seed(3)
    net = sphconv.Sequential(
        sphconv.SubMConv3d(16, 16, 3, indice_key="a", name="s0"),
        torch.nn.ReLU(),
        sphconv.SparseConv3d(16, 32, 3, stride=2, padding=1, name="d0"),
        sphconv.SubMConv3d(32, 32, 3, indice_key="b", name="s1"),
        sphconv.SparseConv3d(32, 32, 3, stride=2, padding=1, name="d1"),
    ).to(DEV).half().eval()
    calls = []
    real_begin = ops.get_rules_begin

    def spy(*a, **k):
        calls.append(a[0])
        return real_begin(*a, **k)

    ops.get_rules_begin = spy
    try:
        with torch.no_grad():
            x = sphconv.SparseConvTensor(feat, shape, B, z_idx=zi, z_ptr=zp)
            y = net(x)
            assert len(calls) == 2                      # one per strided layer, none repeated by get_rules
            assert not any(isinstance(k, tuple) for k in y.rule_cache)     # the handles were consumed
            t = sphconv.SparseConvTensor(feat, shape, B, z_idx=zi, z_ptr=zp)
            for m in net:
                if isinstance(m, torch.nn.ReLU):
                    t.feature = m(t.feature)
                else:
                    t = m(t)
            assert len(calls) == 4                      # called one by one: get_rules runs both steps itself
    finally:
        ops.get_rules_begin = real_begin
    assert torch.equal(y.z_idx, t.z_idx) and torch.equal(y.z_ptr, t.z_ptr) and torch.equal(y.feature, t.feature)
    sphconv.check_status()
    # the handle API itself: a mismatching handle is ignored, a matching one is used
    geom = (zi, zp, B, shape, [6, 10, 8], [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1], [2, 2])
    want = ops.get_rules(*geom)
    pend = ops.get_rules_begin(*geom)
    got = ops.get_rules(*geom, pending=pend)
    other = ops.get_rules(zi.clone(), zp, *geom[2:], pending=ops.get_rules_begin(*geom))
    for a, b, c in zip(want, got, other):
        assert torch.equal(a, b) and torch.equal(a, c)


def test_module_rules_written_beside_the_convolution():
    """The module path writes the reference-format pair lists on a side stream while the convolution runs; once the
    layer has returned they are complete on the caller's stream and equal those of the plain ops."""
    from sphconv_b200 import sphconv_cuda as ops
    rng = np.random.default_rng(17)
    B, shape = 3, [10, 14, 12]
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3, False)        # unsorted columns too
    feat = torch.as_tensor(rng.standard_normal((z_idx.shape[0], 16)), dtype=torch.float16, device=DEV)
    zi, zp = torch.as_tensor(z_idx, device=DEV), torch.as_tensor(z_ptr, device=DEV)
    sub = sphconv.SubMConv3d(16, 16, 3, indice_key="k").to(DEV).half().eval()
    down = sphconv.SparseConv3d(16, 32, 3, stride=2, padding=1, indice_key="d").to(DEV).half().eval()

    def canon(rules, rule_size):
        r, n = rules.cpu().numpy(), rule_size.cpu().numpy()
        out = {}
        for t in range(r.shape[0]):
            for k in range(r.shape[1]):
                m = min(int(n[t, k]), r.shape[3])
                out[(t, k)] = sorted(zip(r[t, k, 0, :m].tolist(), r[t, k, 1, :m].tolist()))
        return n, out

    for flag in (True, False):
        ops.config.overlap_rule_lists = flag
        try:
            with torch.no_grad():
                x = sphconv.SparseConvTensor(feat, shape, B, z_idx=zi, z_ptr=zp)
                y = down(sub(x))
                # a kernel of the caller's on the current stream, right behind the layers, already sees the lists
                _, _, rules_s, size_s, _ = x.rule_cache["k"]
                _, _, rules_d, size_d, _ = y.rule_cache["d"]
                snap = (rules_s.clone(), size_s.clone(), rules_d.clone(), size_d.clone())
            assert getattr(rules_s, "_sph_ready", None) is None and getattr(rules_d, "_sph_ready", None) is None
        finally:
            ops.config.overlap_rule_lists = True
        want_s = ops.get_rules_subm(zi, zp, B, shape, shape, [3] * 3, [1] * 3, [1] * 3, [1] * 3, [2, 2])
        want_d = ops.get_rules(zi, zp, B, shape, [5, 7, 6], [3] * 3, [2] * 3, [1] * 3, [1] * 3, [2, 2])
        for (r, n), (wr, wn) in (((snap[0], snap[1]), (want_s[2], want_s[3])), ((snap[2], snap[3]), (want_d[2], want_d[3]))):
            n_got, got = canon(r, n)
            n_want, want = canon(wr, wn)
            assert (n_got == n_want).all() and got == want
    sphconv.check_status()
