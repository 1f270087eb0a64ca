"""Parity at the size of the five benchmark configurations (per scan), CUDA path against the CPU oracle.

What the small-grid tests cannot show: many tiles per persistent CTA across every layer of the stack (both
accumulator buffers, the stage ring wrapping many times), 32-bit row arithmetic at millions of rows x 27 offsets,
the heuristic list capacity on full-size grids, and exact int8 accumulation on the widest grid.

Tolerances: rules bit-exact; fp32 |y - ref| <= 1e-4 * max(|ref|, 1); fp16 / bf16 1e-2 * max(|ref|, 1) against the
float64 oracle on the same rounded operands; int8 exact.  The reference runs its own suites at scan size too
(test/test_grad.py:565-636, test/test_conv.py:119-363)."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import conv_np, dense_ref, rules_np
from sphconv_b200 import _capi as C
from sphconv_b200 import check_status, synthetic
from sphconv_b200 import sphconv_cuda as ops
from sphconv_b200.encoder import encoder8_parameters

from gpu_util import DEV, assert_tables_match, gpu_rules, oracle_rules

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-4, torch.float16: 1e-2, torch.bfloat16: 1e-2}


def _close(got, ref, tol, what):
    got = got.double().cpu().numpy()
    err = np.abs(got - ref)
    bound = tol * np.maximum(np.abs(ref), 1.0)
    assert (err <= bound).all(), "%s: max err %g (bound %g there)" % (what, err.max(), bound.reshape(-1)[err.argmax()])


def _close_global(got, ref, tol, what):
    got = got.double().cpu().numpy()
    assert np.abs(got - ref).max() <= tol * max(np.abs(ref).max(), 1.0), what


def _table_rules(z_idx, z_ptr, B, shape, stride, subm):
    """Rule set without the padded reference-format tensor (GB-sized on the wide grids): neighbour tables from the
    op, list lengths from the count-only mode of sph_rule_lists.  Returns (tables, rule_size, oz_idx, oz_ptr, osh)."""
    ops.config.materialize_rules = False
    try:
        with torch.enable_grad():       # also builds the transposed table of a strided set
            zi, zp, osh, oz_idx, oz_ptr, tables, _ = gpu_rules(z_idx, z_ptr, B, shape, [3, 3, 3], [stride] * 3,
                                                                [1, 1, 1], [2, 2], subm)
    finally:
        ops.config.materialize_rules = True
    g = C.make_geom(B, shape, osh, [3, 3, 3], [stride] * 3, [1, 1, 1], [2, 2])
    n_tile = C.check(C.lib().sph_num_tiles(ctypes.byref(g)))
    rule_size = torch.empty((n_tile, 27), dtype=torch.int32, device=DEV)
    C.check(C.lib().sph_rule_lists(C.ptr(oz_ptr), ctypes.byref(g), oz_idx.shape[0], C.ptr(tables.nbr), 0, None,
                                   C.ptr(rule_size), 0, C.ptr(C.status_tensor(torch.device(DEV))),
                                   C.stream_ptr(torch.device(DEV))))
    tnm = C.check(C.lib().sph_tile_n_max(ctypes.byref(g), z_idx.shape[0]))
    return tables, rule_size, oz_idx, oz_ptr, osh, tnm


def _assert_tables(res, tb, n_in, n_out):
    want = np.full((27, n_out), -1, dtype=np.int32)
    want[res["k"], res["out"]] = res["in"]
    assert (tb.nbr.cpu().numpy() == want).all()
    if tb.nbr_t is not None:
        want_t = np.full((27, n_in), -1, dtype=np.int32)
        want_t[res["k"], res["in"]] = res["out"]
        assert (tb.nbr_t.cpu().numpy() == want_t).all()


def test_cfg1_full_config_fp32_vs_dense_conv3d():
    """configs[0] exactly: one SubM 16->16 fp32 layer on the 32x128x64 grid, batch 1, against the dense conv3d of
    the reference's own tests evaluated in float64 and read back at the active sites."""
    cfg = synthetic.CONFIGS["cfg1"]
    b = synthetic.make_batch("cfg1", batch=1)
    shape = cfg["shape"]
    zi, zp, osh, oz_idx, oz_ptr, rules, rule_size = gpu_rules(b["z_idx"], b["z_ptr"], 1, shape, [3, 3, 3], [1, 1, 1],
                                                               [1, 1, 1], [2, 2], True)
    res = oracle_rules(b["z_idx"], b["z_ptr"], 1, shape, [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2], True)
    assert (rule_size.cpu().numpy() == res["rule_size"]).all()
    assert (rules_np.canonical_pairs(rules.cpu().numpy(), rule_size.cpu().numpy()) == rules_np.canonical_from_table(res)).all()
    w5 = synthetic.make_weight([3, 3, 3], 16, 16, 1234)
    feat = torch.as_tensor(b["feature"], device=DEV)
    w = torch.as_tensor(w5, device=DEV).reshape(27, 16, 16)
    out = ops.rule_conv(feat, w, rules, rule_size, feat.shape[0])
    dense = dense_ref.dense_conv(b["feature"], w5, b["z_idx"], b["z_ptr"], 1, shape, [1, 1, 1], [1, 1, 1])
    ref = dense_ref.gather_rows(dense, b["z_idx"], b["z_ptr"], 1, shape).numpy()
    _close(out, ref, 1e-4, "cfg1 forward")
    assert check_status() == 0


def test_cfg2_full_config_fp16_forward_backward():
    """configs[1] exactly: Conv3d 32->64, stride 2, padding 1, fp16, batch 4 on 64x512x128: rules bit-exact, forward,
    dgrad and wgrad within 1e-2 of the float64 oracle on the same fp16 operands."""
    cfg = synthetic.CONFIGS["cfg2"]
    B, shape = 4, cfg["shape"]
    b = synthetic.make_batch("cfg2", batch=B)
    with torch.enable_grad():
        zi, zp, osh, oz_idx, oz_ptr, rules, rule_size = gpu_rules(b["z_idx"], b["z_ptr"], B, shape, [3, 3, 3],
                                                                   [2, 2, 2], [1, 1, 1], [2, 2], False)
    res = oracle_rules(b["z_idx"], b["z_ptr"], B, shape, [3, 3, 3], [2, 2, 2], [1, 1, 1], [2, 2], False)
    assert (rule_size.cpu().numpy() == res["rule_size"]).all()
    assert (oz_idx.cpu().numpy() == res["oz_idx"]).all() and (oz_ptr.cpu().numpy() == res["oz_ptr"]).all()
    n_in, n_out = b["z_idx"].shape[0], oz_idx.shape[0]
    assert_tables_match(res, rules, n_in, n_out)
    pairs = rules_np.canonical_from_table(res)
    rng = np.random.default_rng(2)
    feat = torch.as_tensor(b["feature"], device=DEV).half()
    w = torch.as_tensor(synthetic.make_weight([3, 3, 3], 32, 64, 1236), device=DEV).reshape(27, 32, 64).half()
    out = ops.rule_conv(feat, w, rules, rule_size, n_out)
    f64, w64 = feat.double().cpu().numpy(), w.double().cpu().numpy()
    _close(out, conv_np.conv_forward(f64, w64, pairs, n_out), 1e-2, "cfg2 forward")
    dout = torch.as_tensor(rng.standard_normal((n_out, 64)), dtype=torch.float32, device=DEV).half()
    dx, dw = ops.rule_conv_backward(dout, feat, w.permute(0, 2, 1).contiguous(), rules, rule_size, [16, 128])
    d64 = dout.double().cpu().numpy()
    _close(dx, conv_np.conv_dgrad(d64, w64, pairs, n_in), 1e-2, "cfg2 dgrad")
    dw32 = ops.rule_conv_d_weight(feat, dout, rules, rule_size)
    _close_global(dw32, conv_np.conv_wgrad(f64, d64, pairs, 27), 1e-2, "cfg2 wgrad (fp32 result)")
    _close_global(dw, conv_np.conv_wgrad(f64, d64, pairs, 27), 1e-2, "cfg2 wgrad")
    assert check_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_cfg3_full_size_scan_all_layers(dtype):
    """One full-size cfg3 / cfg4 scan (64x512x256) through all 8 layers.  Every level's rule set is compared with the
    oracle bit for bit; every layer's forward (fused bias + ReLU), dgrad and wgrad are compared with the sparse
    float64 oracle fed the GPU's own input of that layer, so an error cannot hide behind the layers before it."""
    cfg = synthetic.CONFIGS["cfg3"]
    b = synthetic.make_batch("cfg3", batch=1, first_scan=3)
    z_idx, z_ptr, shape = b["z_idx"], b["z_ptr"], list(cfg["shape"])
    x = torch.as_tensor(b["feature"], device=DEV).to(dtype)
    params = encoder8_parameters()
    rng = np.random.default_rng(8)
    cache = {}
    for li, ((subm, iC, oC, stride, key), (w5, bias)) in enumerate(zip(synthetic.ENCODER8, params)):
        if key is not None and key in cache:
            rules, rule_size, pairs, n_in, n_out, oz_idx_np, oz_ptr_np, osh = cache[key]
        else:
            with torch.enable_grad():
                _, _, osh, oz_idx, oz_ptr, rules, rule_size = gpu_rules(z_idx, z_ptr, 1, shape, [3, 3, 3], [stride] * 3,
                                                                        [1, 1, 1], [2, 2], subm)
            res = oracle_rules(z_idx, z_ptr, 1, shape, [3, 3, 3], [stride] * 3, [1, 1, 1], [2, 2], subm)
            assert (rule_size.cpu().numpy() == res["rule_size"]).all(), "L%d rule_size" % li
            assert (oz_idx.cpu().numpy() == res["oz_idx"]).all() and \
                (oz_ptr.cpu().numpy().reshape(-1) == res["oz_ptr"].reshape(-1)).all(), "L%d output pattern" % li
            assert res["rule_size"].max() <= rules.shape[3], "L%d: heuristic capacity overflowed" % li
            n_in, n_out = z_idx.shape[0], oz_idx.shape[0]
            assert_tables_match(res, rules, n_in, n_out)
            pairs = rules_np.canonical_from_table(res)
            oz_idx_np, oz_ptr_np = res["oz_idx"], res["oz_ptr"]
            if key is not None:
                cache[key] = (rules, rule_size, pairs, n_in, n_out, oz_idx_np, oz_ptr_np, osh)
        w = torch.as_tensor(w5, device=DEV).reshape(27, iC, oC).to(dtype)
        bias_t = torch.as_tensor(bias, device=DEV)
        y = ops.rule_conv(x, w, rules, rule_size, n_out, bias=bias_t, relu=True)
        x64, w64 = x.double().cpu().numpy(), w.double().cpu().numpy()
        ref = np.maximum(conv_np.conv_forward(x64, w64, pairs, n_out) + bias.astype(np.float64), 0.0)
        _close(y, ref, TOL[dtype], "L%d forward" % li)
        dout = torch.as_tensor(rng.standard_normal((n_out, oC)), dtype=torch.float32, device=DEV).to(dtype)
        dx, dw = ops.rule_conv_backward(dout, x, w.permute(0, 2, 1).contiguous(), rules, rule_size, [1, 1])
        d64 = dout.double().cpu().numpy()
        _close(dx, conv_np.conv_dgrad(d64, w64, pairs, n_in), TOL[dtype], "L%d dgrad" % li)
        _close_global(ops.rule_conv_d_weight(x, dout, rules, rule_size), conv_np.conv_wgrad(x64, d64, pairs, 27),
                      TOL[dtype], "L%d wgrad" % li)
        x = y
        if not subm:
            z_idx, z_ptr, shape = oz_idx_np, oz_ptr_np, osh
    assert check_status() == 0


def test_cfg5_wide_grid_rules_and_int8():
    """The 64x2048x256 grid of configs[4], two scans: first-level SubM rule set, the strided set behind it and the
    SubM set of the next level (neighbour tables, list lengths, output pattern bit-exact; the heuristic list
    capacity not exceeded), then an int8 32->32 convolution on that level, exact against the integer oracle."""
    cfg = synthetic.CONFIGS["cfg5"]
    B, shape = 2, list(cfg["shape"])
    b = synthetic.make_batch("cfg5", batch=B)
    z_idx, z_ptr = b["z_idx"], b["z_ptr"]
    # level 0: submanifold
    tb, rule_size, oz_idx, oz_ptr, osh, tnm = _table_rules(z_idx, z_ptr, B, shape, 1, True)
    res = oracle_rules(z_idx, z_ptr, B, shape, [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2], True)
    assert (rule_size.cpu().numpy() == res["rule_size"]).all()
    assert res["rule_size"].max() <= tnm == res["tile_n_max"]
    _assert_tables(res, tb, z_idx.shape[0], z_idx.shape[0])
    # level 0 -> 1: strided
    tb, rule_size, oz_idx, oz_ptr, osh, tnm = _table_rules(z_idx, z_ptr, B, shape, 2, False)
    res = oracle_rules(z_idx, z_ptr, B, shape, [3, 3, 3], [2, 2, 2], [1, 1, 1], [2, 2], False)
    assert (oz_idx.cpu().numpy() == res["oz_idx"]).all() and (oz_ptr.cpu().numpy() == res["oz_ptr"]).all()
    assert (rule_size.cpu().numpy() == res["rule_size"]).all()
    assert res["rule_size"].max() <= tnm == res["tile_n_max"]
    _assert_tables(res, tb, z_idx.shape[0], oz_idx.shape[0])
    # level 1: submanifold on 32x1024x128, int8 convolution
    z_idx1, z_ptr1, shape1 = res["oz_idx"], res["oz_ptr"], osh
    tb, rule_size, _, _, _, tnm = _table_rules(z_idx1, z_ptr1, B, shape1, 1, True)
    res1 = oracle_rules(z_idx1, z_ptr1, B, shape1, [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2], True)
    assert (rule_size.cpu().numpy() == res1["rule_size"]).all()
    assert res1["rule_size"].max() <= tnm == res1["tile_n_max"]
    n = z_idx1.shape[0]
    _assert_tables(res1, tb, n, n)
    rng = np.random.default_rng(55)
    feat = torch.as_tensor(rng.integers(-127, 128, size=(n, 32)), dtype=torch.int8, device=DEV)
    w = torch.as_tensor(rng.integers(-127, 128, size=(27, 32, 32)), dtype=torch.int8, device=DEV)
    out = ops.rule_conv(feat, w, tb, None, n)                # float32 output of the exact int32 sums
    assert C.lib().sph_conv_uses_tensor_cores(C.SPH_I8, 32, 32) == 1
    # float64 holds these sums exactly (|sum| <= 27 * 32 * 127^2 < 2^53) and runs through BLAS
    ref = conv_np.conv_forward(feat.cpu().numpy(), w.cpu().numpy(), rules_np.canonical_from_table(res1), n)
    assert (out.double().cpu().numpy() == ref).all()
    assert check_status() == 0
