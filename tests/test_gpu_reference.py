"""This library against the reference's OWN CUDA kernels on the same inputs, on the GPU.
The reference build (oracle/_ref, see oracle/build_ref.py) travels with the repository when it was built
where the reference sources are mounted; the tests skip when it is absent."""
import numpy as np
import pytest
import torch

from oracle import build_ref, rules_np
from sphconv_b200 import synthetic
from sphconv_b200 import sphconv_cuda as ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ref():
    mod = build_ref.load()
    if mod is None:
        pytest.skip("reference build oracle/_ref is not present")
    return mod


def _both(ref, subm, z_idx, z_ptr, B, shape, ks, st, pd, tile):
    osh = list(shape) if subm else rules_np.out_spatial(shape, ks, st, pd)
    zi = torch.as_tensor(z_idx, device=DEV)
    zp = torch.as_tensor(z_ptr, device=DEV)
    name = "get_rules_subm" if subm else "get_rules"
    a = getattr(ref, name)(zi, zp, B, shape, osh, ks, st, pd, [1, 1, 1], tile)
    with torch.enable_grad():
        b = getattr(ops, name)(zi, zp, B, shape, osh, ks, st, pd, [1, 1, 1], tile)
    torch.cuda.synchronize()
    return a, b, osh


@pytest.mark.parametrize("subm,B,shape,ks,st,pd,dens", [
    (True, 2, [12, 20, 16], [3, 3, 3], [1, 1, 1], [1, 1, 1], 0.2),
    (True, 8, [8, 8, 8], [3, 3, 1], [1, 1, 1], [1, 1, 0], 0.3),
    (False, 4, [12, 20, 16], [3, 3, 3], [2, 2, 2], [1, 1, 1], 0.2),
    (False, 1, [9, 7, 11], [2, 2, 2], [2, 2, 2], [0, 0, 0], 0.4),
    (False, 3, [10, 10, 10], [3, 3, 3], [1, 1, 1], [0, 0, 0], 0.15),
])
def test_rules_identical_to_reference_kernels(ref, subm, B, shape, ks, st, pd, dens):
    rng = np.random.default_rng(31)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, dens)
    (r_ozi, r_ozp, r_rules, r_size), (m_ozi, m_ozp, m_rules, m_size), _ = _both(ref, subm, z_idx, z_ptr, B, shape, ks,
                                                                               st, pd, [2, 2])
    assert r_rules.shape == m_rules.shape                  # same tile_n_max heuristic
    assert torch.equal(r_size, m_size)
    assert torch.equal(r_ozp.reshape(-1), m_ozp.reshape(-1))
    assert torch.equal(r_ozi, m_ozi)                       # output numbering identical without sorting
    a = rules_np.canonical_pairs(r_rules.cpu().numpy(), r_size.cpu().numpy())
    b = rules_np.canonical_pairs(m_rules.cpu().numpy(), m_size.cpu().numpy())
    assert (a == b).all()                                  # per-(tile,k) pair multisets


def test_rules_identical_on_cfg1_scan(ref):
    cfg = synthetic.CONFIGS["cfg1"]
    b = synthetic.make_batch("cfg1", batch=1)
    (r_ozi, r_ozp, r_rules, r_size), (m_ozi, m_ozp, m_rules, m_size), _ = _both(
        ref, True, b["z_idx"], b["z_ptr"], 1, cfg["shape"], [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2])
    assert torch.equal(r_size, m_size)
    a = rules_np.canonical_pairs(r_rules.cpu().numpy(), r_size.cpu().numpy())
    c = rules_np.canonical_pairs(m_rules.cpu().numpy(), m_size.cpu().numpy())
    assert (a == c).all()


@pytest.mark.parametrize("subm,iC,oC", [(True, 16, 16), (False, 32, 64), (True, 64, 64), (False, 4, 5)])
def test_conv_matches_reference_kernels_fp32(ref, subm, iC, oC):
    """fp32 forward / dgrad / wgrad of the reference's CUTLASS SIMT kernels vs this library, 1e-4 relative."""
    if not ref.has_conv:
        pytest.skip("reference rule_conv.cu was not built")
    rng = np.random.default_rng(77)
    B, shape = 2, [10, 12, 8]
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.25)
    st, pd = ([1, 1, 1], [1, 1, 1]) if subm else ([2, 2, 2], [1, 1, 1])
    (r_ozi, r_ozp, r_rules, r_size), (m_ozi, m_ozp, m_rules, m_size), osh = _both(ref, subm, z_idx, z_ptr, B, shape,
                                                                                 [3, 3, 3], st, pd, [2, 2])
    n_in, n_out = z_idx.shape[0], r_ozi.shape[0]
    feat = torch.as_tensor(rng.standard_normal((n_in, iC)), dtype=torch.float32, device=DEV)
    w = torch.as_tensor(rng.uniform(-1, 1, size=(27, iC, oC)) / np.sqrt(iC * 4), dtype=torch.float32, device=DEV)
    dout = torch.as_tensor(rng.standard_normal((n_out, oC)), dtype=torch.float32, device=DEV)
    tg = [-(-osh[0] // 2), -(-osh[1] // 2)]
    y_ref = ref.rule_conv(feat, w, r_rules, r_size, n_out)
    dx_ref, dw_ref = ref.rule_conv_backward(dout, feat, w.permute(0, 2, 1).contiguous(), r_rules, r_size, tg)
    # ours, fed with the REFERENCE's rule tensors (no attached tables: exercises the conversion path)
    y = ops.rule_conv(feat, w, r_rules, r_size, n_out)
    dx, dw = ops.rule_conv_backward(dout, feat, w.permute(0, 2, 1).contiguous(), r_rules, r_size, tg)
    torch.cuda.synchronize()
    for got, want in ((y, y_ref), (dx, dx_ref), (dw, dw_ref)):
        bound = 1e-4 * torch.clamp(want.abs().max(), min=1.0)
        assert (got - want).abs().max() <= bound


def test_init_tensor_and_to_dense_match_reference_kernels(ref):
    """The reference's init_tensor / to_dense (fp32 only; the order inside a column is its atomics' arrival order, so rows
    are compared per column as sets and through the dense image)."""
    rng = np.random.default_rng(17)
    B, shape, C = 3, [7, 9, 40], 6
    occ = rng.random((B, *shape)) < 0.2
    idx = np.stack(np.nonzero(occ), axis=1).astype(np.int32)
    rng.shuffle(idx)
    feat = torch.as_tensor(rng.standard_normal((idx.shape[0], C)).astype(np.float32), device=DEV)
    didx = torch.as_tensor(idx, device=DEV)
    r_f, r_zi, r_zp, r_perm = ref.init_tensor(feat, didx, B, shape)
    m_f, m_zi, m_zp, m_perm = ops.init_tensor(feat, didx, B, shape)
    torch.cuda.synchronize()
    assert torch.equal(r_zp.reshape(-1), m_zp.reshape(-1))
    # both permutations place row n inside its column's range, and moved the row there
    assert torch.equal(r_f[r_perm.long()], feat) and torch.equal(m_f[m_perm.long()], feat)
    assert torch.equal(r_zi[r_perm.long()], didx[:, 3]) and torch.equal(m_zi[m_perm.long()], didx[:, 3])
    r_dense = torch.zeros((B, *shape, C), device=DEV)
    m_dense = torch.zeros((B, *shape, C), device=DEV)
    ref.to_dense(r_f, r_zi, r_zp, shape[2], r_dense)
    ops.to_dense(m_f, m_zi, m_zp, shape[2], m_dense)
    torch.cuda.synchronize()
    assert torch.equal(r_dense, m_dense)
