"""Helpers shared by the GPU parity tests (everything goes through the C ABI via sphconv_b200.sphconv_cuda)."""
import numpy as np
import torch

from oracle import rules_np
from sphconv_b200 import sphconv_cuda as ops

DEV = "cuda:0"


def to_dev(z_idx, z_ptr):
    return (torch.as_tensor(np.ascontiguousarray(z_idx), dtype=torch.int32, device=DEV),
            torch.as_tensor(np.ascontiguousarray(z_ptr), dtype=torch.int32, device=DEV))


def gpu_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm):
    zi, zp = to_dev(z_idx, z_ptr)
    osh = list(shape) if subm else rules_np.out_spatial(shape, ks, st, pd)
    fn = ops.get_rules_subm if subm else ops.get_rules
    oz_idx, oz_ptr, rules, rule_size = fn(zi, zp, B, list(shape), osh, list(ks), list(st), list(pd), [1, 1, 1], list(tile))
    return zi, zp, osh, oz_idx, oz_ptr, rules, rule_size


def oracle_rules(z_idx, z_ptr, B, shape, ks, st, pd, tile, subm, padded=False):
    osh = list(shape) if subm else rules_np.out_spatial(shape, ks, st, pd)
    fn = rules_np.get_rules_subm if subm else rules_np.get_rules
    return fn(z_idx, z_ptr, B, shape, osh, ks, st, pd, [1, 1, 1], tile, padded=padded)


def assert_rules_equal(res, oz_idx, oz_ptr, rules, rule_size, check_padding=True):
    """Bit-exact parity: rule_size elementwise, per-(tile,k) pair multisets after canonical sort,
    oz_idx / oz_ptr without sorting."""
    rs = rule_size.cpu().numpy()
    assert rs.shape == res["rule_size"].shape
    assert (rs == res["rule_size"]).all()
    r = rules.cpu().numpy()
    assert r.shape[3] == res["tile_n_max"]
    assert (rules_np.canonical_pairs(r, rs) == rules_np.canonical_from_table(res)).all()
    assert (oz_idx.cpu().numpy() == res["oz_idx"]).all()
    assert (oz_ptr.cpu().numpy() == res["oz_ptr"]).all()
    if check_padding and ops.config.fill_unused_rules:
        slot = np.arange(r.shape[3])[None, None, None, :]
        unused = slot >= rs[:, :, None, None]
        assert (r[np.broadcast_to(unused, r.shape)] == -1).all()


def assert_tables_match(res, rules, n_in, n_out):
    """The neighbour tables attached to `rules` hold exactly the oracle's pairs."""
    tb = rules._sph
    KV = res["rule_size"].shape[1]
    want = np.full((KV, n_out), -1, dtype=np.int64)
    want[res["k"], res["out"]] = res["in"]
    assert (tb.nbr.cpu().numpy() == want).all()
    if tb.nbr_t is not None:
        want_t = np.full((KV, n_in), -1, dtype=np.int64)
        want_t[res["k"], res["in"]] = res["out"]
        assert (tb.nbr_t.cpu().numpy() == want_t).all()
