"""Rule generation on the GPU against the CPU oracle: bit-exact rule_size, pair multisets per (tile,k),
oz_idx and oz_ptr.  Shapes follow the reference's test/test_rules.py (small literal cases, kernels 1-3,
strides 1-2, paddings 0-1, batch 1-8, non-cubic shapes) with seeded random occupancies."""
import itertools

import numpy as np
import pytest
import torch

from oracle import rules_np
from sphconv_b200 import check_status, synthetic
from sphconv_b200 import sphconv_cuda as ops

from gpu_util import assert_rules_equal, assert_tables_match, gpu_rules, oracle_rules, to_dev
from test_oracle import CASES

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("i", range(len(CASES)))
@pytest.mark.parametrize("sort_columns", [True, False])
def test_strided_small(i, sort_columns):
    B, shape, ks, st, pd, tile, dens = CASES[i]
    rng = np.random.default_rng(100 + i)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, dens, sort_columns)
    with torch.enable_grad():
        zi, zp, osh, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, False)
    res = oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, False)
    assert_rules_equal(res, oz_idx, oz_ptr, rules, rule_size)
    assert_tables_match(res, rules, z_idx.shape[0], oz_idx.shape[0])
    assert rules._sph.nbr_t is not None
    assert check_status() & 1 == 0


@pytest.mark.parametrize("ks", [[3, 3, 3], [1, 1, 1], [3, 3, 1], [2, 2, 2], [3, 1, 3], [5, 5, 5]])
@pytest.mark.parametrize("sort_columns", [True, False])
def test_subm_small(ks, sort_columns):
    B, shape, tile = 3, [7, 9, 6], [2, 2]
    rng = np.random.default_rng(7)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3, sort_columns)
    pd = [k // 2 for k in ks]
    zi, zp, osh, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, ks, [1, 1, 1], pd, tile, True)
    assert oz_idx is zi and oz_ptr is zp           # same objects, as the reference returns them
    res = oracle_rules(z_idx, z_ptr, B, shape, ks, [1, 1, 1], pd, tile, True)
    assert_rules_equal(res, oz_idx, oz_ptr.reshape(B, *shape[:2]), rules, rule_size)
    assert_tables_match(res, rules, z_idx.shape[0], z_idx.shape[0])


def test_exhaustive_2x2x2():
    """Every occupancy of a 2x2x2 grid, batch 2 (second scan = complement), subm 3x3x3 and strided k2 s2 / k3 s2 p1."""
    shape = [2, 2, 2]
    for code in range(256):
        occ = np.array([(code >> b) & 1 for b in range(8)], dtype=bool).reshape(1, 2, 2, 2)
        occ = np.concatenate([occ, ~occ], axis=0)
        counts = occ.sum(axis=3).reshape(-1)
        z_ptr = np.cumsum(counts).astype(np.int32).reshape(2, 2, 2)
        z_idx = np.nonzero(occ)[3].astype(np.int32)
        for subm, ks, st, pd in [(True, [3, 3, 3], [1, 1, 1], [1, 1, 1]), (False, [2, 2, 2], [2, 2, 2], [0, 0, 0]),
                                 (False, [3, 3, 3], [2, 2, 2], [1, 1, 1])]:
            _, _, _, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, 2, shape, ks, st, pd, [2, 2], subm)
            res = oracle_rules(z_idx, z_ptr, 2, shape, ks, st, pd, [2, 2], subm)
            assert_rules_equal(res, oz_idx, oz_ptr.reshape(res["oz_ptr"].shape), rules, rule_size, check_padding=False)


def test_empty_and_single():
    shape, ks = [4, 4, 4], [3, 3, 3]
    z_ptr = np.zeros((1, 4, 4), np.int32)
    z_idx = np.zeros((0,), np.int32)
    for subm, st, pd in [(True, [1, 1, 1], [1, 1, 1]), (False, [2, 2, 2], [1, 1, 1])]:
        _, _, _, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, 1, shape, ks, st, pd, [2, 2], subm)
        assert int(rule_size.sum()) == 0 and oz_idx.shape[0] == 0
    occ = np.zeros((1, 4, 4, 4), bool)
    occ[0, 3, 3, 3] = True
    z_ptr = np.cumsum(occ.sum(axis=3).reshape(-1)).astype(np.int32).reshape(1, 4, 4)
    z_idx = np.array([3], np.int32)
    for subm, st, pd in [(True, [1, 1, 1], [1, 1, 1]), (False, [2, 2, 2], [1, 1, 1]), (False, [1, 1, 1], [0, 0, 0])]:
        _, _, _, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, 1, shape, ks, st, pd, [2, 2], subm)
        res = oracle_rules(z_idx, z_ptr, 1, shape, ks, st, pd, [2, 2], subm)
        assert_rules_equal(res, oz_idx, oz_ptr.reshape(res["oz_ptr"].shape), rules, rule_size)


def test_full_columns_and_big_tiles():
    """Dense grid (every depth bin active: maximum column length) and tiles larger than the grid."""
    B, shape = 2, [5, 6, 40]
    occ = np.ones((B, *shape), bool)
    z_ptr = np.cumsum(occ.sum(axis=3).reshape(-1)).astype(np.int32).reshape(B, 5, 6)
    z_idx = np.nonzero(occ)[3].astype(np.int32)
    for subm, ks, st, pd, tile in [(True, [3, 3, 3], [1, 1, 1], [1, 1, 1], [8, 8]),
                                   (False, [3, 3, 3], [2, 2, 2], [1, 1, 1], [2, 2]),
                                   (False, [3, 3, 3], [1, 1, 1], [0, 0, 0], [4, 3])]:
        _, _, _, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
        res = oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
        assert_rules_equal(res, oz_idx, oz_ptr.reshape(res["oz_ptr"].shape), rules, rule_size, check_padding=False)


def test_overflow_is_flagged_and_tables_stay_exact():
    """A tile_n_max overflow drops pairs from `rules` exactly like the reference (src/sphconv/rules.cu:217-224:
    rule_size keeps counting) and raises the status bit; the neighbour tables are not limited."""
    B, shape = 1, [16, 16, 64]
    occ = np.zeros((B, *shape), bool)
    occ[0, :2, :2, :] = True      # one dense tile in an otherwise empty grid: the sparsity heuristic underestimates
    z_ptr = np.cumsum(occ.sum(axis=3).reshape(-1)).astype(np.int32).reshape(B, 16, 16)
    z_idx = np.nonzero(occ)[3].astype(np.int32)
    check_status()
    _, _, _, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2], True)
    res = oracle_rules(z_idx, z_ptr, B, shape, [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2], True)
    assert res["rule_size"].max() > rules.shape[3]
    assert check_status() & 1
    assert (rule_size.cpu().numpy() == res["rule_size"]).all()
    assert_tables_match(res, rules, z_idx.shape[0], z_idx.shape[0])


@pytest.mark.parametrize("subm", [True, False])
def test_exact_rule_capacity_never_overflows(subm):
    """config.exact_rule_capacity: tile_n_max is the longest list (counted first), so the input that overflows the
    reference's heuristic capacity keeps every pair and raises no status bit."""
    from sphconv_b200 import sphconv_cuda as ops
    B, shape = 2, [16, 16, 64]
    occ = np.zeros((B, *shape), bool)
    occ[:, :2, :2, :] = True
    occ[1, 7, 9, 3] = True
    z_ptr = np.cumsum(occ.sum(axis=3).reshape(-1)).astype(np.int32).reshape(B, 16, 16)
    z_idx = np.nonzero(occ)[3].astype(np.int32)
    ks, st, pd = ([3, 3, 3], [1, 1, 1], [1, 1, 1]) if subm else ([3, 3, 3], [2, 2, 2], [1, 1, 1])
    res = oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, [2, 2], subm)
    check_status()
    ops.config.exact_rule_capacity = True
    try:
        _, _, _, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, [2, 2], subm)
    finally:
        ops.config.exact_rule_capacity = False
    assert check_status() == 0
    if subm:
        assert res["rule_size"].max() > res["tile_n_max"], "the case must overflow the heuristic capacity"
    assert rules.shape[3] == res["rule_size"].max()
    rs, r = rule_size.cpu().numpy(), rules.cpu().numpy()
    assert (rs == res["rule_size"]).all()
    got = set()
    for t, k in zip(*np.nonzero(rs)):
        n = rs[t, k]
        got.update((int(k), int(i), int(o)) for i, o in zip(r[t, k, 0, :n], r[t, k, 1, :n]))
    want = set(zip(res["k"].tolist(), res["in"].tolist(), res["out"].tolist()))
    assert got == want and len(want) == int(rs.sum())
    assert_tables_match(res, rules, z_idx.shape[0], oz_idx.shape[0])


@pytest.mark.parametrize("name,batch", [("cfg1", 1), ("cfg2", 4), ("cfg3", 2)])
def test_config_first_layer(name, batch):
    """BASELINE configs at full per-scan size: first layer's rule set (cfg1 SubM; cfg2 strided; cfg3 SubM)."""
    cfg = synthetic.CONFIGS[name]
    b = synthetic.make_batch(name, batch=batch)
    subm = name != "cfg2"
    ks = [3, 3, 3]
    st, pd = ([1, 1, 1], [1, 1, 1]) if subm else ([2, 2, 2], [1, 1, 1])
    _, _, _, oz_idx, oz_ptr, rules, rule_size = gpu_rules(b["z_idx"], b["z_ptr"], batch, cfg["shape"], ks, st, pd, [2, 2], subm)
    res = oracle_rules(b["z_idx"], b["z_ptr"], batch, cfg["shape"], ks, st, pd, [2, 2], subm)
    assert (rule_size.cpu().numpy() == res["rule_size"]).all()
    assert (oz_idx.cpu().numpy() == res["oz_idx"]).all() and (oz_ptr.cpu().numpy() == res["oz_ptr"]).all()
    assert res["rule_size"].max() <= rules.shape[3], "heuristic tile_n_max overflowed on a BASELINE config"
    assert_tables_match(res, rules, b["z_idx"].shape[0], oz_idx.shape[0])
    # pair multisets via the attached tables (the padded tensor is GB-scale here); lists themselves on a sample of tiles
    r = rules[:64].cpu().numpy()
    rs = rule_size[:64].cpu().numpy()
    got = rules_np.canonical_pairs(r, rs)
    full = rules_np.canonical_from_table(res)
    assert (got == full[full[:, 0] < 64]).all()


def test_encoder_rule_chain_cfg3():
    """Rule sets of the whole 8-layer encoder on one cfg3 scan: each level's oz_idx/oz_ptr feed the next."""
    cfg = synthetic.CONFIGS["cfg3"]
    b = synthetic.make_batch("cfg3", batch=1)
    z_idx, z_ptr, shape = b["z_idx"], b["z_ptr"], list(cfg["shape"])
    seen = set()
    for subm, iC, oC, stride, key in synthetic.ENCODER8:
        if key is not None and key in seen:
            continue
        seen.add(key)
        st, pd = [stride] * 3, [1, 1, 1]
        _, _, osh, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, 1, shape, [3, 3, 3], st, pd, [2, 2], subm)
        res = oracle_rules(z_idx, z_ptr, 1, shape, [3, 3, 3], st, pd, [2, 2], subm)
        assert (rule_size.cpu().numpy() == res["rule_size"]).all()
        assert (oz_idx.cpu().numpy() == res["oz_idx"]).all()
        assert (oz_ptr.cpu().numpy().reshape(-1) == res["oz_ptr"].reshape(-1)).all()
        assert_tables_match(res, rules, z_idx.shape[0], oz_idx.shape[0])
        if not subm:
            z_idx, z_ptr, shape = res["oz_idx"], res["oz_ptr"], osh


def test_deterministic_and_foreign_rules():
    """Two runs give identical tensors (list order included); a cloned rules tensor (no attached tables)
    converts to the same tables."""
    B, shape = 4, [8, 12, 16]
    rng = np.random.default_rng(3)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.2)
    a = gpu_rules(z_idx, z_ptr, B, shape, [3, 3, 3], [2, 2, 2], [1, 1, 1], [2, 2], False)
    b = gpu_rules(z_idx, z_ptr, B, shape, [3, 3, 3], [2, 2, 2], [1, 1, 1], [2, 2], False)
    for x, y in zip(a[3:], b[3:]):
        assert torch.equal(x, y)
    rules, rule_size = a[5], a[6]
    clone = rules.clone()
    assert not hasattr(clone, "_sph")
    tb = ops._tables_for(clone, rule_size, z_idx.shape[0], a[3].shape[0], need_t=True)
    assert torch.equal(tb.nbr, rules._sph.nbr)
    res = oracle_rules(z_idx, z_ptr, B, shape, [3, 3, 3], [2, 2, 2], [1, 1, 1], [2, 2], False)
    assert_tables_match(res, clone, z_idx.shape[0], a[3].shape[0])
    assert check_status() == 0


def test_bad_arguments_raise():
    zi, zp = to_dev(np.zeros(0, np.int32), np.zeros((1, 4, 4), np.int32))
    with pytest.raises(RuntimeError):
        ops.get_rules(zi, zp, 1, [4, 4, 4], [2, 2, 2], [3, 3, 3], [2, 2, 2], [1, 1, 1], [0, 1, 1], [2, 2])   # dilation 0
    with pytest.raises(RuntimeError):
        ops.get_rules_subm(zi, zp, 1, [4, 4, 4], [2, 2, 2], [3, 3, 3], [1, 1, 1], [1, 1, 1], [1, 1, 1], [2, 2])  # shape
    with pytest.raises(RuntimeError):
        ops.get_rules(zi.cpu(), zp.cpu(), 1, [4, 4, 4], [2, 2, 2], [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1], [2, 2])


@pytest.mark.parametrize("dens", [0.002, 0.05, 0.6])
@pytest.mark.parametrize("subm", [True, False])
def test_index_and_scan_paths_agree(dens, subm):
    """Nearly empty grids take the per-column scan kernels (no column index is built), denser ones the row-parallel
    kernels on the index; both must give the oracle's rules."""
    B, shape, tile = 2, [12, 20, 96], [2, 2]
    rng = np.random.default_rng(int(dens * 1000) + (7 if subm else 0))
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, dens, True)
    ks, st, pd = ([3, 3, 3], [1, 1, 1], [1, 1, 1]) if subm else ([3, 3, 3], [2, 2, 2], [1, 1, 1])
    _, _, _, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
    res = oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
    assert_rules_equal(res, oz_idx, oz_ptr.reshape(res["oz_ptr"].shape), rules, rule_size)
    assert_tables_match(res, rules, z_idx.shape[0], oz_idx.shape[0])


@pytest.mark.parametrize("ks,st,pd", [([7, 7, 7], [1, 1, 1], [3, 3, 3]), ([3, 3, 7], [2, 2, 6], [1, 1, 3]),
                                      ([2, 2, 2], [2, 2, 2], [0, 0, 0]), ([3, 3, 5], [1, 2, 4], [1, 1, 2])])
def test_large_kernels_and_strides(ks, st, pd):
    """Kernel extents up to 7 and depth strides beyond what the bit-parallel pattern kernel handles."""
    B, shape, tile = 2, [9, 11, 70], [2, 2]
    rng = np.random.default_rng(sum(ks) * 10 + sum(st))
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.15, True)
    subm = st == [1, 1, 1]
    _, _, _, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
    res = oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
    assert_rules_equal(res, oz_idx, oz_ptr.reshape(res["oz_ptr"].shape), rules, rule_size)
    assert_tables_match(res, rules, z_idx.shape[0], oz_idx.shape[0])


@pytest.mark.parametrize("subm", [True, False])
def test_tables_without_rule_lists(subm):
    """config.materialize_rules = False: no rules / rule_size, the neighbour tables alone, still exact."""
    B, shape, tile = 3, [10, 14, 40], [2, 2]
    rng = np.random.default_rng(11)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.2, True)
    ks, st, pd = ([3, 3, 3], [1, 1, 1], [1, 1, 1]) if subm else ([3, 3, 3], [2, 2, 2], [1, 1, 1])
    ops.config.materialize_rules = False
    try:
        with torch.enable_grad():
            _, _, _, oz_idx, oz_ptr, tables, none = gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
    finally:
        ops.config.materialize_rules = True
    assert none is None
    res = oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
    assert (oz_idx.cpu().numpy() == res["oz_idx"]).all()
    KV = res["rule_size"].shape[1]
    want = np.full((KV, oz_idx.shape[0]), -1, dtype=np.int64)
    want[res["k"], res["out"]] = res["in"]
    assert (tables.nbr.cpu().numpy() == want).all()
    if not subm:
        want_t = np.full((KV, z_idx.shape[0]), -1, dtype=np.int64)
        want_t[res["k"], res["in"]] = res["out"]
        assert (tables.nbr_t.cpu().numpy() == want_t).all()


@pytest.mark.parametrize("subm", [True, False])
def test_deep_grid(subm):
    """More than 256 depth bins: the column index is built by the kernel that works in global memory."""
    B, shape, tile = 2, [6, 10, 300], [2, 2]
    rng = np.random.default_rng(5)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.1, True)
    ks, st, pd = ([3, 3, 3], [1, 1, 1], [1, 1, 1]) if subm else ([3, 3, 3], [2, 2, 2], [1, 1, 1])
    _, _, _, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
    res = oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
    assert_rules_equal(res, oz_idx, oz_ptr.reshape(res["oz_ptr"].shape), rules, rule_size)
    assert_tables_match(res, rules, z_idx.shape[0], oz_idx.shape[0])


@pytest.mark.parametrize("depth", [3, 5, 31, 32, 33, 63, 64, 65, 66, 100, 129, 256])
@pytest.mark.parametrize("dens", [0.15, 1.0])
def test_stride2_depth_pattern_word_boundaries(depth, dens):
    """The usual stride-2, 3-deep, padding-1 layer at depths around the 32-bin word boundaries of the column index: the
    output pattern (oz_idx, oz_ptr), the pair lists and the tables against the oracle, sparse and completely full."""
    B, shape, tile = 2, [5, 6, depth], [2, 2]
    rng = np.random.default_rng(900 + depth)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, dens)
    ks, st, pd = [3, 3, 3], [2, 2, 2], [1, 1, 1]
    zi, zp, osh, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, False)
    res = oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, False)
    assert_rules_equal(res, oz_idx, oz_ptr, rules, rule_size)
    assert_tables_match(res, rules, z_idx.shape[0], oz_idx.shape[0])
    assert check_status() & 1 == 0


@pytest.mark.parametrize("subm", [True, False])
def test_more_runs_per_tile_than_one_staging_pass(subm):
    """150 scans in the batch: a tile of 2 x 2 columns then has 300 (batch, tile row) runs, more than the pair-list kernels
    stage at a time (128), so they go through a tile in several passes."""
    B, shape, tile = 150, [4, 6, 9], [2, 2]
    rng = np.random.default_rng(77)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.4)
    ks = [3, 3, 3]
    st, pd = ([1, 1, 1], [1, 1, 1]) if subm else ([2, 2, 2], [1, 1, 1])
    zi, zp, osh, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
    res = oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm)
    if subm:
        oz_ptr = oz_ptr.reshape(B, *shape[:2])
    assert_rules_equal(res, oz_idx, oz_ptr, rules, rule_size)
    assert_tables_match(res, rules, z_idx.shape[0], oz_idx.shape[0])
    assert check_status() & 1 == 0
