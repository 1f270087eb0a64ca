"""CPU-only checks of the C-ABI library: it loads, exports every symbol the header declares, and its
host-side geometry helpers agree with the oracle.  No device code is called."""
import ctypes
import os
import re

import numpy as np
import pytest

from oracle import rules_loops, rules_np
from sphconv_b200 import _capi as C
from sphconv_b200 import build as sph_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    sph_build.build()
    return C.lib()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "sphconv_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(sph_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(C.SIGNATURES), "ctypes table and header disagree: %s" % (declared ^ set(C.SIGNATURES))
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.sph_version() >= 100


def test_out_spatial_and_tile_n_max_match_oracle(lib):
    rng = np.random.default_rng(0)
    arr = lambda v: (ctypes.c_int32 * 3)(*[int(x) for x in v])
    for _ in range(200):
        shape = rng.integers(1, 70, size=3)
        ks = rng.integers(1, 4, size=3)
        st = np.minimum(rng.integers(1, 3, size=3), ks)
        pd = rng.integers(0, 2, size=3)
        out = arr([0, 0, 0])
        assert lib.sph_out_spatial(arr(shape), arr(ks), arr(st), arr(pd), None, out) == 0
        want = rules_np.out_spatial(list(shape), list(ks), list(st), list(pd))
        assert list(out) == want
        dl = rng.integers(1, 4, size=3) if _ % 2 else np.ones(3, dtype=np.int64)   # every other case dilated
        assert lib.sph_out_spatial(arr(shape), arr(ks), arr(st), arr(pd), arr(dl), out) == 0
        want = rules_np.out_spatial(list(shape), list(ks), list(st), list(pd), list(dl))
        assert list(out) == want
        if min(want) < 1:
            continue
        B = int(rng.integers(1, 9))
        tile = rng.integers(1, 5, size=2)
        nnz = int(rng.integers(0, B * int(np.prod(shape)) + 1))
        g = C.make_geom(B, shape, want, ks, st, pd, tile, dl)
        got = lib.sph_tile_n_max(ctypes.byref(g), nnz)
        ref = rules_loops.heuristic_tile_n_max(rules_loops.in_tile_size(int(tile[0]), int(st[0]), int(ks[0]), int(dl[0])),
                                               rules_loops.in_tile_size(int(tile[1]), int(st[1]), int(ks[1]), int(dl[1])),
                                               B, int(shape[0]), int(shape[1]), int(shape[2]), nnz)
        assert got == ref
        assert lib.sph_num_tiles(ctypes.byref(g)) == rules_loops.div_up(want[0], int(tile[0])) * rules_loops.div_up(want[1], int(tile[1]))


def test_errors_are_reported_not_fatal(lib):
    g = C.make_geom(0, [4, 4, 4], [4, 4, 4], [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2])
    assert lib.sph_num_tiles(ctypes.byref(g)) == -1
    assert b"batch" in lib.sph_last_error()
    g = C.make_geom(1, [4, 4, 4], [4, 4, 4], [8, 8, 8], [1, 1, 1], [1, 1, 1], [2, 2])
    assert lib.sph_num_tiles(ctypes.byref(g)) == -4
    with pytest.raises(RuntimeError):
        C.check(-1)


def test_ops_refuse_cpu_tensors():
    import torch
    from sphconv_b200 import sphconv_cuda as ops
    zi = torch.zeros(0, dtype=torch.int32)
    zp = torch.zeros((1, 4, 4), dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.get_rules_subm(zi, zp, 1, [4, 4, 4], [4, 4, 4], [3, 3, 3], [1, 1, 1], [1, 1, 1], [1, 1, 1], [2, 2])


def test_kernel_selection_predicates(lib):
    """Which convolution kernel a shape gets (host-side answers; 27 offsets assumed)."""
    tc, pair = lib.sph_conv_uses_tensor_cores, lib.sph_conv_uses_pair_kernel
    # rows of 32 to 256 bytes: tensor cores, never the pair kernel
    for dt, k, n in [(C.SPH_F16, 16, 16), (C.SPH_F16, 32, 32), (C.SPH_BF16, 64, 64), (C.SPH_I8, 32, 32), (C.SPH_I8, 64, 64)]:
        assert tc(dt, k, n) == 1 and pair(dt, k, n) == 0
    # narrower rows of 4 / 8 / 16 / 32 channels and small fp32 layers: the pair-compacting kernel
    for dt, k, n in [(C.SPH_F16, 4, 16), (C.SPH_F16, 8, 8), (C.SPH_BF16, 4, 32), (C.SPH_F32, 16, 16), (C.SPH_F32, 4, 4),
                     (C.SPH_I8, 4, 16), (C.SPH_I8, 16, 16), (C.SPH_I8, 16, 32)]:
        assert tc(dt, k, n) == 0 and pair(dt, k, n) == 1
    # odd channel counts and filters beyond its shared memory: the row-walking kernel
    for dt, k, n in [(C.SPH_F16, 5, 16), (C.SPH_F32, 32, 32), (C.SPH_F32, 64, 64), (C.SPH_F16, 4, 64)]:
        assert tc(dt, k, n) == 0 and pair(dt, k, n) == 0
    # weight gradient: 1 = tensor cores, 2 = the pair-compacting walk, 0 = the general CUDA-core kernel
    wk = lib.sph_conv_wgrad_kernel
    assert wk(C.SPH_BF16, 32, 32) == 1 and wk(C.SPH_F16, 16, 16) == 1 and wk(C.SPH_F16, 64, 64) == 1
    assert wk(C.SPH_BF16, 4, 16) == 2 and wk(C.SPH_F32, 16, 16) == 2 and wk(C.SPH_F32, 16, 32) == 2
    assert wk(C.SPH_F32, 64, 64) == 0 and wk(C.SPH_F16, 5, 16) == 0 and wk(C.SPH_I8, 16, 16) == 0
