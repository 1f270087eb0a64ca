"""sph_rules_subm_static: the allocation-free entry point for callers that cannot hand the library scratch
memory (host applications that own the allocator, no-malloc real-time loops, runtimes whose buffers cannot be
lent out).  Its scratch is a fixed array inside the library, so this test calls it straight through the C ABI,
twice in a row on different inputs (the array keeps the previous call's contents and must be rebuilt), and
requires bit-identical rules, rule sizes and neighbour tables to sph_rules_subm with caller scratch."""
import ctypes

import numpy as np
import pytest
import torch

from sphconv_b200 import _capi as C
from sphconv_b200 import synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(lib, fn_static, z_idx, z_ptr, B, shape):
    zi = torch.as_tensor(z_idx, dtype=torch.int32, device=DEV)
    zp = torch.as_tensor(z_ptr, dtype=torch.int32, device=DEV)
    nnz = zi.shape[0]
    g = C.make_geom(B, shape, shape, [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2])
    n_tile = C.check(lib.sph_num_tiles(ctypes.byref(g)))
    tnm = C.check(lib.sph_tile_n_max(ctypes.byref(g), nnz))
    outs = []
    for static in (False, True):
        rules = torch.full((n_tile, 27, 2, tnm), -7, dtype=torch.int32, device=DEV)
        rule_size = torch.full((n_tile, 27), -7, dtype=torch.int32, device=DEV)
        nbr = torch.full((27, nnz), -7, dtype=torch.int32, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        st = C.stream_ptr(torch.device(DEV))
        if static:
            C.check(fn_static(C.ptr(zi), C.ptr(zp), nnz, ctypes.byref(g), tnm, C.ptr(rules), C.ptr(rule_size),
                              C.ptr(nbr), 1, C.ptr(status), st))
        else:
            need = C.check(lib.sph_rules_subm_scratch_bytes(ctypes.byref(g), nnz))
            assert need > 0, "the case must exercise the scratch-using path"
            scratch = torch.empty(need, dtype=torch.uint8, device=DEV)
            C.check(lib.sph_rules_subm(C.ptr(zi), C.ptr(zp), nnz, ctypes.byref(g), C.ptr(scratch), tnm, C.ptr(rules),
                                       C.ptr(rule_size), C.ptr(nbr), 1, C.ptr(status), st))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        outs.append((rules, rule_size, nbr))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    assert int(outs[1][1].sum()) > 0


def test_static_scratch_entry_point_matches_twice_in_a_row():
    lib = C.lib()
    fn = lib.sph_rules_subm_static
    rng = np.random.default_rng(42)
    # long columns (about 19 and 13 voxels per column) so that the depth index, i.e. the scratch, is used
    a = synthetic.make_random_occupancy(rng, 2, [8, 12, 64], 0.30)
    b = synthetic.make_random_occupancy(rng, 3, [6, 10, 48], 0.27)
    _run(lib, fn, a[0], a[1], 2, [8, 12, 64])
    _run(lib, fn, b[0], b[1], 3, [6, 10, 48])
    _run(lib, fn, a[0], a[1], 2, [8, 12, 64])


def test_static_scratch_entry_point_allocates_nothing():
    """Free device memory as the driver reports it is the same before and after a series of calls (outputs are
    allocated beforehand; the first call, which looks up the array's address, has already happened)."""
    lib = C.lib()
    rng = np.random.default_rng(7)
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, 2, [8, 12, 64], 0.30)
    zi = torch.as_tensor(z_idx, dtype=torch.int32, device=DEV)
    zp = torch.as_tensor(z_ptr, dtype=torch.int32, device=DEV)
    nnz = zi.shape[0]
    g = C.make_geom(2, [8, 12, 64], [8, 12, 64], [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2])
    n_tile = C.check(lib.sph_num_tiles(ctypes.byref(g)))
    tnm = C.check(lib.sph_tile_n_max(ctypes.byref(g), nnz))
    rules = torch.empty((n_tile, 27, 2, tnm), dtype=torch.int32, device=DEV)
    rule_size = torch.empty((n_tile, 27), dtype=torch.int32, device=DEV)
    nbr = torch.empty((27, nnz), dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = C.stream_ptr(torch.device(DEV))
    call = lambda: C.check(lib.sph_rules_subm_static(C.ptr(zi), C.ptr(zp), nnz, ctypes.byref(g), tnm, C.ptr(rules),
                                                     C.ptr(rule_size), C.ptr(nbr), 1, C.ptr(status), st))
    call()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert int(status.item()) == 0


def test_static_scratch_entry_point_rejects_oversized_inputs():
    lib = C.lib()
    # 64 x 2048 x 2048 columns x 8 words x 8 bytes of index is far beyond the built-in 8 MiB
    g = C.make_geom(8, [2048, 2048, 256], [2048, 2048, 256], [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2])
    nnz = 3 * 8 * 2048 * 2048
    need = lib.sph_rules_subm_scratch_bytes(ctypes.byref(g), nnz)
    assert need > 8 * 1024 * 1024
    dummy = torch.zeros(16, dtype=torch.int32, device=DEV)
    rc = lib.sph_rules_subm_static(C.ptr(dummy), C.ptr(dummy), nnz, ctypes.byref(g), 64, None, None, C.ptr(dummy), 0,
                                   None, C.stream_ptr(torch.device(DEV)))
    assert rc == -4
    msg = lib.sph_last_error().decode()
    assert "scratch" in msg and str(8 * 1024 * 1024) in msg
