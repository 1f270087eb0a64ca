"""The CPU oracle against golden vectors recorded from the reference's own CUDA kernels on a B200
(tests/golden/ref_rules.npz, ref_conv.npz; produced by tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from oracle import conv_np, rules_np

HERE = os.path.dirname(os.path.abspath(__file__))
sys_path_golden = os.path.join(HERE, "golden")


def _load(name):
    path = os.path.join(sys_path_golden, name)
    if not os.path.exists(path):
        pytest.skip("golden file %s not recorded yet" % name)
    return np.load(path)


def _cases():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(sys_path_golden, "make_golden.py"))
    # only the case tables are needed; avoid importing torch-heavy parts by parsing lazily
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.RULE_CASES, mod.CONV_CASES


def test_rule_oracle_matches_reference_kernels():
    g = _load("ref_rules.npz")
    rule_cases, _ = _cases()
    for ci, (subm, B, shape, ks, st, pd, tile, dens, srt) in enumerate(rule_cases):
        z_idx, z_ptr = g["c%d_z_idx" % ci], g["c%d_z_ptr" % ci]
        osh = list(shape) if subm else rules_np.out_spatial(shape, ks, st, pd)
        fn = rules_np.get_rules_subm if subm else rules_np.get_rules
        res = fn(z_idx, z_ptr, B, shape, osh, ks, st, pd, [1, 1, 1], tile, padded=False)
        assert res["tile_n_max"] == int(g["c%d_tile_n_max" % ci])
        assert (res["rule_size"] == g["c%d_rule_size" % ci]).all()
        assert (rules_np.canonical_from_table(res) == g["c%d_pairs" % ci]).all()
        assert (res["oz_idx"] == g["c%d_oz_idx" % ci]).all()
        assert (res["oz_ptr"].reshape(-1) == g["c%d_oz_ptr" % ci].reshape(-1)).all()


def test_conv_oracle_matches_reference_kernels():
    g = _load("ref_conv.npz")
    r = _load("ref_rules.npz")
    _, conv_cases = _cases()
    for ci, iC, oC in conv_cases:
        tag = "v%d_%d_%d" % (ci, iC, oC)
        pairs = r["c%d_pairs" % ci]
        feat, w, dout = g[tag + "_feat"], g[tag + "_w"], g[tag + "_dout"]
        n_out = r["c%d_oz_idx" % ci].shape[0]
        y = conv_np.conv_forward(feat, w, pairs, n_out)
        dx = conv_np.conv_dgrad(dout, w, pairs, feat.shape[0])
        dw = conv_np.conv_wgrad(feat, dout, pairs, w.shape[0])
        for got, want in ((y, g[tag + "_y"]), (dx, g[tag + "_dx"]), (dw, g[tag + "_dw"])):
            assert np.abs(got - want).max() <= 1e-4 * max(np.abs(want).max(), 1.0)   # reference arithmetic is fp32
