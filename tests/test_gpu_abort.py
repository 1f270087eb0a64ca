"""The bounded waits of the tensor-core convolution kernel: when a pipeline stage never becomes full, every role
leaves its loop, copies in flight are drained, tensor memory is freed, the launch returns and the status word carries
SPH_STATUS_TIMEOUT; the context stays usable and the next launch is correct.

The failure is made on purpose only in a test-only build of the library (`libsphconv_b200_hooks.so`,
sphconv_b200/build.py: conv_tc.cu compiled with -DSPH_TEST_HOOKS): there the wait limit is about 10 ms and
`sph_test_withhold_arrival(1)` makes one gather thread skip its arrival for the second stage.  Nothing faults, traps or
spins without a bound."""
import ctypes
import os

import numpy as np
import pytest
import torch

from sphconv_b200 import _capi as C
from sphconv_b200 import build as sph_build

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _hooks_lib():
    if not os.path.exists(sph_build.HOOKS_LIB):
        pytest.skip("test-hooks library not built (python -m sphconv_b200.build)")
    h = ctypes.CDLL(sph_build.HOOKS_LIB)
    for name in ("sph_pack_weight", "sph_conv_gather", "sph_packed_weight_bytes"):
        fn = getattr(h, name)
        fn.restype, fn.argtypes = C.SIGNATURES[name]
    h.sph_test_withhold_arrival.restype = None
    h.sph_test_withhold_arrival.argtypes = [ctypes.c_int]
    return h


def test_withheld_arrival_times_out_cleanly():
    h = _hooks_lib()
    dev = torch.device(DEV)
    rng = np.random.default_rng(3)
    n, K, N, kv = 4096, 64, 64, 27                 # 16 tiles of 256 rows, 27 stages each
    rows = torch.as_tensor(rng.standard_normal((n, K)), dtype=torch.float32, device=DEV).half()
    w = torch.as_tensor(rng.uniform(-.1, .1, (kv, K, N)), dtype=torch.float32, device=DEV).half()
    nbr = torch.as_tensor(rng.integers(-1, n, size=(kv, n)), dtype=torch.int32, device=DEV)
    packed = torch.empty(h.sph_packed_weight_bytes(C.SPH_F16, kv, K, N), dtype=torch.uint8, device=DEV)
    st = C.stream_ptr(dev)
    assert h.sph_pack_weight(C.ptr(w), C.SPH_F16, kv, K, N, C.ptr(packed), st) == 0
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def run():
        out = torch.zeros((n, N), dtype=torch.float16, device=DEV)
        rc = h.sph_conv_gather(C.ptr(rows), C.SPH_F16, n, C.ptr(w), C.ptr(packed), C.ptr(nbr), n, kv, K, N, 0, None, None,
                               0, C.ptr(out), C.SPH_F16, C.ptr(status), st)
        assert rc == 0
        torch.cuda.synchronize()
        return out

    good = run()
    assert int(status.item()) == 0
    h.sph_test_withhold_arrival(1)
    try:
        run()                                       # returns: the kernel gives up after its wait limit
        assert int(status.item()) & C.STATUS_TIMEOUT
    finally:
        h.sph_test_withhold_arrival(0)
    status.zero_()
    again = run()                                   # the context is intact and the kernel works again
    assert int(status.item()) == 0
    assert torch.equal(again, good)
    ref = torch.zeros((n, N), dtype=torch.float32, device=DEV)
    for k in range(kv):
        idx = nbr[k].long()
        m = idx >= 0
        ref[m] += rows.float()[idx[m]] @ w[k].float()
    assert ((good.float() - ref).abs() <= 1e-2 * ref.abs().clamp_min(1)).all()
