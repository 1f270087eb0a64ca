"""Records outputs of the reference's OWN CUDA kernels (oracle/_ref, built from the unmodified reference
sources by oracle/build_ref.py) as golden vectors for the CPU tests.  Needs a CUDA device.

    python tests/golden/make_golden.py <output directory>      # writes ref_rules.npz (and ref_conv.npz)

The committed tests/golden/*.npz were produced by this script on a B200.  Cases are seeded random
occupancies in the shapes the reference's tests use (test/test_rules.py: kernels 1-3, strides 1-2,
paddings 0-1, batch 1-8, non-cubic shapes, tile [2,2])."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import build_ref, rules_np  # noqa: E402
from sphconv_b200 import synthetic  # noqa: E402

# (subm, B, shape, ksize, stride, padding, tile, density, sorted columns)
RULE_CASES = [
    (True, 1, [4, 4, 4], [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2], 0.4, True),
    (True, 3, [7, 9, 6], [3, 3, 3], [1, 1, 1], [1, 1, 1], [2, 2], 0.3, True),
    (True, 2, [6, 5, 8], [3, 1, 3], [1, 1, 1], [1, 0, 1], [2, 2], 0.35, False),
    (True, 8, [8, 8, 8], [1, 1, 1], [1, 1, 1], [0, 0, 0], [2, 2], 0.2, True),
    (False, 2, [5, 7, 6], [3, 3, 3], [2, 2, 2], [1, 1, 1], [2, 2], 0.3, True),
    (False, 3, [6, 5, 8], [2, 3, 2], [1, 2, 1], [0, 1, 0], [2, 2], 0.35, True),
    (False, 2, [9, 6, 10], [3, 3, 3], [2, 1, 2], [0, 1, 1], [2, 4], 0.25, False),
    (False, 8, [4, 6, 4], [2, 2, 2], [2, 2, 2], [0, 0, 0], [2, 2], 0.5, True),
    (False, 1, [16, 24, 12], [3, 3, 3], [2, 2, 2], [1, 1, 1], [2, 2], 0.15, True),
]
CONV_CASES = [(0, 16, 16), (4, 32, 64), (1, 4, 5), (8, 64, 64)]   # (rule case, iC, oC), fp32 as the reference


def main(out_dir):
    ref = build_ref.load()
    assert ref is not None, "oracle/_ref is not built"
    dev = "cuda:0"
    store = {}
    kept = {}
    for ci, (subm, B, shape, ks, st, pd, tile, dens, srt) in enumerate(RULE_CASES):
        rng = np.random.default_rng(7000 + ci)
        z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, dens, srt)
        osh = list(shape) if subm else rules_np.out_spatial(shape, ks, st, pd)
        zi = torch.as_tensor(z_idx, device=dev)
        zp = torch.as_tensor(z_ptr, device=dev)
        fn = ref.get_rules_subm if subm else ref.get_rules
        oz_idx, oz_ptr, rules, rule_size = fn(zi, zp, B, shape, osh, ks, st, pd, [1, 1, 1], tile)
        torch.cuda.synchronize()
        rs = rule_size.cpu().numpy()
        assert rs.max() <= rules.shape[3], "reference overflowed its own tile_n_max; pick another case"
        store["c%d_z_idx" % ci] = z_idx
        store["c%d_z_ptr" % ci] = z_ptr
        store["c%d_oz_idx" % ci] = oz_idx.cpu().numpy()
        store["c%d_oz_ptr" % ci] = oz_ptr.cpu().numpy()
        store["c%d_rule_size" % ci] = rs
        store["c%d_tile_n_max" % ci] = np.int64(rules.shape[3])
        store["c%d_pairs" % ci] = rules_np.canonical_pairs(rules.cpu().numpy(), rs).astype(np.int32)
        kept[ci] = (zi, zp, oz_idx, rules, rule_size, z_idx.shape[0])
    np.savez_compressed(os.path.join(out_dir, "ref_rules.npz"), **store)
    print("wrote ref_rules.npz (%d cases)" % len(RULE_CASES))
    if not ref.has_conv or "--no-conv" in sys.argv:
        return
    cstore = {}
    for ci, iC, oC in CONV_CASES:
        zi, zp, oz_idx, rules, rule_size, nnz = kept[ci]
        rng = np.random.default_rng(9000 + ci)
        kv = int(np.prod(RULE_CASES[ci][3]))
        feat = rng.standard_normal((nnz, iC)).astype(np.float32)
        w = (rng.uniform(-1, 1, size=(kv, iC, oC)) / np.sqrt(iC * 4)).astype(np.float32)
        n_out = oz_idx.shape[0]
        dout = rng.standard_normal((n_out, oC)).astype(np.float32)
        f, wt, g = [torch.as_tensor(a, device=dev) for a in (feat, w, dout)]
        y = ref.rule_conv(f, wt, rules, rule_size, n_out)
        tg = [-(-s // t) for s, t in zip((RULE_CASES[ci][2] if RULE_CASES[ci][0] else
                                          rules_np.out_spatial(RULE_CASES[ci][2], *RULE_CASES[ci][3:6]))[:2], RULE_CASES[ci][6])]
        dx, dw = ref.rule_conv_backward(g, f, wt.permute(0, 2, 1).contiguous(), rules, rule_size, tg)
        torch.cuda.synchronize()
        tag = "v%d_%d_%d" % (ci, iC, oC)
        for name, arr in (("feat", feat), ("w", w), ("dout", dout), ("y", y.cpu().numpy()), ("dx", dx.cpu().numpy()),
                          ("dw", dw.cpu().numpy())):
            cstore["%s_%s" % (tag, name)] = arr
    np.savez_compressed(os.path.join(out_dir, "ref_conv.npz"), **cstore)
    print("wrote ref_conv.npz (%d cases)" % len(CONV_CASES))


if __name__ == "__main__":
    out = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--") else os.path.dirname(os.path.abspath(__file__))
    os.makedirs(out, exist_ok=True)
    main(out)
