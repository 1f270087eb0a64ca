"""The CPU oracle against itself (loop restatement vs vectorised) and against the dense conv3d
construction the reference's tests use (test/test_rules.py:14-60, test/test_grad.py:7-36)."""
import numpy as np
import pytest
import torch

from oracle import conv_np, dense_ref, rules_loops, rules_np
from sphconv_b200 import synthetic

CASES = [
    # B, shape, ksize, stride, padding, tile, density
    (1, [4, 4, 4], [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2], 0.4),
    (2, [5, 7, 6], [3, 3, 3], [2, 2, 2], [1, 1, 1], [2, 2], 0.3),
    (3, [6, 5, 8], [2, 3, 2], [1, 2, 1], [0, 1, 0], [2, 2], 0.35),
    (1, [8, 8, 8], [1, 1, 1], [1, 1, 1], [0, 0, 0], [2, 2], 0.2),
    (2, [7, 9, 5], [3, 3, 1], [1, 1, 1], [1, 1, 0], [3, 2], 0.3),
    (2, [9, 6, 10], [3, 3, 3], [2, 1, 2], [0, 1, 1], [2, 4], 0.25),
    (8, [4, 6, 4], [2, 2, 2], [2, 2, 2], [0, 0, 0], [2, 2], 0.5),
]


def _case(i, sort_columns=True):
    B, shape, ks, st, pd, tile, dens = CASES[i]
    rng = np.random.default_rng(100 + i)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, dens, sort_columns)
    return B, shape, ks, st, pd, tile, z_idx, z_ptr, rng


def test_tile_n_max_formula():
    # src/sphconv/rules.cu:21-28: (int)(B*tH*tW*D*sparsity*2 + 64) & ~15
    assert rules_loops.heuristic_tile_n_max(4, 4, 1, 32, 128, 64, 7000) == (int(1 * 4 * 4 * 64 * (7000 / (32 * 128 * 64)) * 2 + 64) & ~15)
    assert rules_loops.heuristic_tile_n_max(4, 4, 1, 8, 8, 8, 0) == 64
    assert rules_loops.in_tile_size(2, 2, 3) == 5
    assert rules_np.out_spatial([64, 512, 128], [3, 3, 3], [2, 2, 2], [1, 1, 1]) == [32, 256, 64]
    assert rules_np.out_spatial([9, 6, 10], [3, 3, 3], [2, 1, 2], [0, 1, 1]) == [4, 6, 5]


@pytest.mark.parametrize("i", range(len(CASES)))
@pytest.mark.parametrize("sort_columns", [True, False])
def test_strided_loops_vs_np(i, sort_columns):
    B, shape, ks, st, pd, tile, z_idx, z_ptr, _ = _case(i, sort_columns)
    osh = rules_np.out_spatial(shape, ks, st, pd)
    oz_idx, oz_ptr, rules, rule_size = rules_loops.get_rules(z_idx, z_ptr, B, shape, osh, ks, st, pd, [1, 1, 1], tile)
    res = rules_np.get_rules(z_idx, z_ptr, B, shape, osh, ks, st, pd, [1, 1, 1], tile)
    assert (oz_idx == res["oz_idx"]).all() and (oz_ptr == res["oz_ptr"]).all()
    assert (rule_size == res["rule_size"]).all()
    assert (rules_np.canonical_pairs(rules, rule_size) == rules_np.canonical_from_table(res)).all()
    assert (rules_np.canonical_pairs(res["rules"], res["rule_size"]) == rules_np.canonical_from_table(res)).all()
    # occupancy == conv3d(ones) != 0 (test/test_rules.py:14-60)
    occ = dense_ref.occupancy_after_conv(z_idx, z_ptr, B, shape, ks, st, pd)
    mine = dense_ref.densify(np.ones((oz_idx.shape[0], 1), np.float32), oz_idx, oz_ptr, B, osh)[:, 0] != 0
    assert (occ == mine).all()


@pytest.mark.parametrize("i", [0, 3, 4])
@pytest.mark.parametrize("sort_columns", [True, False])
def test_subm_loops_vs_np(i, sort_columns):
    B, shape, ks, st, pd, tile, z_idx, z_ptr, _ = _case(i, sort_columns)
    pd = [k // 2 for k in ks]
    _, _, rules, rule_size = rules_loops.get_rules_subm(z_idx, z_ptr, B, shape, shape, ks, [1, 1, 1], pd, [1, 1, 1], tile)
    res = rules_np.get_rules_subm(z_idx, z_ptr, B, shape, shape, ks, [1, 1, 1], pd, [1, 1, 1], tile)
    assert (rule_size == res["rule_size"]).all()
    assert (rules_np.canonical_pairs(rules, rule_size) == rules_np.canonical_from_table(res)).all()


def test_subm_even_kernel_loops_vs_np():
    rng = np.random.default_rng(5)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, 2, [5, 5, 5], 0.4)
    ks, pd = [2, 2, 2], [1, 1, 1]
    _, _, rules, rule_size = rules_loops.get_rules_subm(z_idx, z_ptr, 2, [5, 5, 5], [5, 5, 5], ks, [1, 1, 1], pd, [1, 1, 1], [2, 2])
    res = rules_np.get_rules_subm(z_idx, z_ptr, 2, [5, 5, 5], [5, 5, 5], ks, [1, 1, 1], pd, [1, 1, 1], [2, 2])
    assert (rules_np.canonical_pairs(rules, rule_size) == rules_np.canonical_from_table(res)).all()


@pytest.mark.parametrize("i", [1, 2, 5, 6])
def test_strided_conv_vs_dense(i):
    B, shape, ks, st, pd, tile, z_idx, z_ptr, rng = _case(i)
    iC, oC = 3, 5
    osh = rules_np.out_spatial(shape, ks, st, pd)
    res = rules_np.get_rules(z_idx, z_ptr, B, shape, osh, ks, st, pd, [1, 1, 1], tile, padded=False)
    pairs = rules_np.canonical_from_table(res)
    feat = rng.standard_normal((z_idx.shape[0], iC))
    w5 = rng.standard_normal((*ks, iC, oC))
    out = conv_np.conv_forward(feat, w5.reshape(-1, iC, oC), pairs, res["oz_idx"].shape[0])
    up = torch.as_tensor(rng.standard_normal((B, oC, *osh)))
    yd, dfeat, dw5 = dense_ref.dense_conv_grads(feat, w5, lambda y: up, z_idx, z_ptr, B, shape, st, pd)
    mine = dense_ref.densify(out, res["oz_idx"], res["oz_ptr"], B, osh)
    assert torch.allclose(mine, yd, atol=1e-10)
    d_out = dense_ref.gather_rows(up, res["oz_idx"], res["oz_ptr"], B, osh).numpy()
    dx = conv_np.conv_dgrad(d_out, w5.reshape(-1, iC, oC), pairs, z_idx.shape[0])
    dw = conv_np.conv_wgrad(feat, d_out, pairs, int(np.prod(ks)))
    assert np.allclose(dx, dfeat.numpy(), atol=1e-10)
    assert np.allclose(dw.reshape(*ks, iC, oC), dw5.numpy(), atol=1e-10)


@pytest.mark.parametrize("ks", [[3, 3, 3], [2, 2, 2], [3, 1, 3]])
def test_subm_conv_vs_masked_dense(ks):
    # even kernels: the reference's pair geometry o = i + k//2 - k stays inside the input shape while
    # conv3d(padding=k//2) yields shape+1; compare on the common leading block.
    rng = np.random.default_rng(11)
    B, shape = 2, [6, 5, 7]
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.35)
    pd = [k // 2 for k in ks]
    iC, oC = 4, 3
    res = rules_np.get_rules_subm(z_idx, z_ptr, B, shape, shape, ks, [1, 1, 1], pd, [1, 1, 1], [2, 2], padded=False)
    pairs = rules_np.canonical_from_table(res)
    feat = rng.standard_normal((z_idx.shape[0], iC))
    w5 = rng.standard_normal((*ks, iC, oC))
    out = conv_np.conv_forward(feat, w5.reshape(-1, iC, oC), pairs, z_idx.shape[0])
    yd = dense_ref.dense_conv(feat, w5, z_idx, z_ptr, B, shape, [1, 1, 1], pd)[:, :, :shape[0], :shape[1], :shape[2]]
    want = dense_ref.gather_rows(yd, z_idx, z_ptr, B, shape).numpy()
    assert np.allclose(out, want, atol=1e-10)


@pytest.mark.parametrize("ks,st,pd,dl", [([3, 3, 3], [1, 1, 1], [2, 2, 2], [2, 2, 2]), ([3, 3, 3], [2, 2, 2], [2, 1, 3], [2, 1, 3]),
                                         ([2, 3, 2], [1, 2, 1], [1, 2, 0], [3, 2, 1])])
def test_dilated_conv_vs_dense(ks, st, pd, dl):
    """Dilation != 1: offset k reads input o*s - pad + k*d (the reference has no consistent behaviour to copy: its
    kernels ignore the argument, its out_spatial honours it).  Pinned here against dense conv3d with the same
    dilation: output shape, occupancy, forward, dgrad, wgrad; and loops == numpy."""
    rng = np.random.default_rng(17)
    B, shape = 2, [7, 6, 9]
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3)
    osh = rules_np.out_spatial(shape, ks, st, pd, dl)
    oz_idx, oz_ptr, rules, rule_size = rules_loops.get_rules(z_idx, z_ptr, B, shape, osh, ks, st, pd, dl, [2, 2])
    res = rules_np.get_rules(z_idx, z_ptr, B, shape, osh, ks, st, pd, dl, [2, 2])
    assert (oz_idx == res["oz_idx"]).all() and (oz_ptr == res["oz_ptr"]).all() and (rule_size == res["rule_size"]).all()
    assert (rules_np.canonical_pairs(rules, rule_size) == rules_np.canonical_from_table(res)).all()
    occ = dense_ref.occupancy_after_conv(z_idx, z_ptr, B, shape, ks, st, pd, dl)
    assert list(occ.shape[1:]) == osh
    mine = dense_ref.densify(np.ones((oz_idx.shape[0], 1), np.float32), oz_idx, oz_ptr, B, osh)[:, 0] != 0
    assert (occ == mine).all()
    iC, oC = 3, 4
    pairs = rules_np.canonical_from_table(res)
    feat = rng.standard_normal((z_idx.shape[0], iC))
    w5 = rng.standard_normal((*ks, iC, oC))
    out = conv_np.conv_forward(feat, w5.reshape(-1, iC, oC), pairs, res["oz_idx"].shape[0])
    up = torch.as_tensor(rng.standard_normal((B, oC, *osh)))
    yd, dfeat, dw5 = dense_ref.dense_conv_grads(feat, w5, lambda y: up, z_idx, z_ptr, B, shape, st, pd, dilation=dl)
    assert torch.allclose(dense_ref.densify(out, res["oz_idx"], res["oz_ptr"], B, osh), yd, atol=1e-10)
    d_out = dense_ref.gather_rows(up, res["oz_idx"], res["oz_ptr"], B, osh).numpy()
    assert np.allclose(conv_np.conv_dgrad(d_out, w5.reshape(-1, iC, oC), pairs, z_idx.shape[0]), dfeat.numpy(), atol=1e-10)
    assert np.allclose(conv_np.conv_wgrad(feat, d_out, pairs, int(np.prod(ks))).reshape(*ks, iC, oC), dw5.numpy(), atol=1e-10)
    if st == [1, 1, 1] and all(p == d * (k // 2) for p, d, k in zip(pd, dl, ks)):
        # submanifold with the "same" padding of a dilated kernel: d * (k // 2)
        rs = rules_np.get_rules_subm(z_idx, z_ptr, B, shape, shape, ks, st, pd, dl, [2, 2], padded=False)
        _, _, rl, rsz = rules_loops.get_rules_subm(z_idx, z_ptr, B, shape, shape, ks, st, pd, dl, [2, 2])
        assert (rules_np.canonical_pairs(rl, rsz) == rules_np.canonical_from_table(rs)).all()
        o2 = conv_np.conv_forward(feat, w5.reshape(-1, iC, oC), rules_np.canonical_from_table(rs), z_idx.shape[0])
        want = dense_ref.gather_rows(dense_ref.dense_conv(feat, w5, z_idx, z_ptr, B, shape, st, pd, dilation=dl),
                                     z_idx, z_ptr, B, shape).numpy()
        assert np.allclose(o2, want, atol=1e-10)


def test_synthetic_configs_are_wellformed():
    for name in ["cfg1", "cfg2", "cfg3"]:
        cfg = synthetic.CONFIGS[name]
        b = synthetic.make_batch(name, batch=1)
        H, W, D = cfg["shape"]
        zp = b["z_ptr"].reshape(-1)
        counts = np.diff(np.concatenate([[0], zp]))
        assert zp[-1] == b["z_idx"].shape[0] and counts.min() >= 0 and counts.max() <= cfg["nmax"]
        assert 0 <= b["z_idx"].min() and b["z_idx"].max() < D
        occ = (counts > 0).mean()
        assert abs(occ - cfg["occ"]) < 0.02
        # ascending and distinct inside each column
        col = np.repeat(np.arange(zp.shape[0]), counts)
        same = col[1:] == col[:-1]
        assert (np.diff(b["z_idx"].astype(np.int64))[same] > 0).all()
    again = synthetic.make_batch("cfg1", batch=1)
    assert (again["z_idx"] == synthetic.make_batch("cfg1", batch=1)["z_idx"]).all()
