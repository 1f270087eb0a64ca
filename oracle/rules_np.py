"""Vectorised numpy restatement of the reference rule generation (any size).

Test infrastructure; never imported by the product.  Same algorithm as ``rules_loops`` (which
mirrors ``src/sphconv/rules.cu`` loop for loop) with the per-thread loops replaced by array
operations.  ``tests/test_oracle.py`` checks the two against each other and against the dense
conv3d occupancy construction of the reference's tests.

Geometry (src/sphconv/rules.cu:36-45,124-133,186-198): offset ``k -> (kH,kW,kD) = (k/(KW*KD), (k/KD)%KW, k%KD)``;
an input voxel at ``i`` pairs with output ``o = (i + pad - k)/s`` iff the division is exact and ``o`` is inside the
output shape; the pair goes to list ``(tile(o), k)`` with ``tile = (oX/tH)*ceil(oW/tW) + oY/tW``
(include/sphconv/debug_utils.h:37-42).
"""
import numpy as np

from .rules_loops import div_up, heuristic_tile_n_max, in_tile_size


def out_spatial(in_spatial, ksize, stride, padding, dilation=(1, 1, 1)):
    """sphconv/utils/__init__.py:27-44 (floor((i + 2p - d(k-1) - 1)/s + 1))."""
    return [int(np.floor((i + 2 * p - d * (k - 1) - 1) / s + 1))
            for i, k, s, p, d in zip(in_spatial, ksize, stride, padding, dilation)]


def row_coords(z_idx, z_ptr, B, H, W):
    """(b, x, y, z) of every feature row from the flat inclusive prefix z_ptr
    (src/sphconv/tensor.cu:107-109; column start = previous flat element, src/sphconv/rules.cu:72-74)."""
    zp = np.asarray(z_ptr, dtype=np.int64).reshape(-1)
    counts = np.diff(np.concatenate([[0], zp]))
    col = np.repeat(np.arange(zp.shape[0], dtype=np.int64), counts)
    b = col // (H * W)
    x = (col // W) % H
    y = col % W
    z = np.asarray(z_idx, dtype=np.int64).reshape(-1)
    assert z.shape[0] == col.shape[0], "z_idx length must equal z_ptr[-1]"
    return b, x, y, z


def _candidates(b, x, y, z, out_shape, ksize, stride, padding, dilation=(1, 1, 1)):
    """All (input row, k) whose output coordinate is inside the output shape.
    Yields per offset k: rows (int64 index array), ox, oy, oz.
    The reference's kernels ignore `dilation` (src/sphconv/rules.cu:36-45) while its Python out_spatial honours it
    (sphconv/utils/__init__.py:40-42), so it has no consistent behaviour for dilation != 1; here offset k reads input
    i = o*s - pad + k*d, the definition out_spatial implies (dense conv3d with dilation).  d = 1 is the reference."""
    oH, oW, oD = out_shape
    KH, KW, KD = ksize
    for k in range(KH * KW * KD):
        kh, kw, kd = k // (KW * KD), (k // KD) % KW, k % KD
        nx = x + padding[0] - kh * dilation[0]
        ny = y + padding[1] - kw * dilation[1]
        nz = z + padding[2] - kd * dilation[2]
        ok = (nx >= 0) & (ny >= 0) & (nz >= 0)
        ok &= (nx % stride[0] == 0) & (ny % stride[1] == 0) & (nz % stride[2] == 0)
        ox, oy, oz = nx // stride[0], ny // stride[1], nz // stride[2]
        ok &= (ox < oH) & (oy < oW) & (oz < oD)
        rows = np.nonzero(ok)[0]
        yield k, rows, ox[rows], oy[rows], oz[rows]


def _finish(pairs_k, n_tile, KV, tnm, padded):
    """Pack per-offset pair arrays into (rule_size, sorted pair table, optional padded rules tensor)."""
    tiles = np.concatenate([p[0] for p in pairs_k]) if pairs_k else np.zeros(0, np.int64)
    ks = np.concatenate([np.full(p[0].shape[0], k, np.int64) for k, p in enumerate(pairs_k)]) if pairs_k else tiles
    ins = np.concatenate([p[1] for p in pairs_k]) if pairs_k else tiles
    outs = np.concatenate([p[2] for p in pairs_k]) if pairs_k else tiles
    order = np.lexsort((outs, ins, ks, tiles))
    tiles, ks, ins, outs = tiles[order], ks[order], ins[order], outs[order]
    lst = tiles * KV + ks
    rule_size = np.bincount(lst, minlength=n_tile * KV).astype(np.int32).reshape(n_tile, KV)
    res = {"rule_size": rule_size, "tile": tiles, "k": ks, "in": ins, "out": outs, "tile_n_max": tnm}
    if padded:
        rules = np.full((n_tile, KV, 2, tnm), -1, dtype=np.int32)
        start = np.concatenate([[0], np.cumsum(rule_size.reshape(-1))])[:-1]
        slot = np.arange(lst.shape[0]) - start[lst]
        keep = slot < tnm                                    # overflow: pair dropped (src/sphconv/rules.cu:217-224)
        rules[tiles[keep], ks[keep], 0, slot[keep]] = ins[keep]
        rules[tiles[keep], ks[keep], 1, slot[keep]] = outs[keep]
        res["rules"] = rules
    return res


def get_rules_subm(z_idx, z_ptr, B, shape, out_shape, ksize, stride, padding, dilation, tile, padded=True):
    """src/sphconv/rules.cu:326-390.  Returns a dict: rule_size [NTile,KV], the canonical pair table
    (tile,k,in,out sorted), tile_n_max, and (padded=True) rules [NTile,KV,2,tile_n_max] filled with -1."""
    H, W, D = shape
    oH, oW, oD = out_shape
    b, x, y, z = row_coords(z_idx, z_ptr, B, H, W)
    key_in = ((b * oH + x) * oW + y) * oD + z                  # the dense grid of rules.cu:339-347, as keys
    order = np.argsort(key_in, kind="stable")
    key_sorted = key_in[order]
    KV = ksize[0] * ksize[1] * ksize[2]
    tgw = div_up(oW, tile[1])
    n_tile = div_up(oH, tile[0]) * tgw
    tnm = heuristic_tile_n_max(in_tile_size(tile[0], stride[0], ksize[0], dilation[0]),
                               in_tile_size(tile[1], stride[1], ksize[1], dilation[1]), B, H, W, D, z.shape[0])
    pairs_k = []
    for k, rows, ox, oy, oz in _candidates(b, x, y, z, out_shape, ksize, stride, padding, dilation):
        key = ((b[rows] * oH + ox) * oW + oy) * oD + oz
        pos = np.searchsorted(key_sorted, key)
        pos_c = np.minimum(pos, max(key_sorted.shape[0] - 1, 0))
        hit = (key_sorted[pos_c] == key) if key_sorted.shape[0] else np.zeros(key.shape, bool)
        out_row = order[pos_c[hit]]                            # grid value = row id of the active site (rules.cu:290-292)
        t = (ox[hit] // tile[0]) * tgw + oy[hit] // tile[1]
        pairs_k.append((t, rows[hit], out_row))
    res = _finish(pairs_k, n_tile, KV, tnm, padded)
    res["oz_idx"] = np.asarray(z_idx, dtype=np.int32).reshape(-1)     # same objects returned (rules.cu:389)
    res["oz_ptr"] = np.asarray(z_ptr, dtype=np.int32).reshape(B, H, W)
    return res


def get_rules(z_idx, z_ptr, B, shape, out_shape, ksize, stride, padding, dilation, tile, padded=True):
    """src/sphconv/rules.cu:405-486.  Output rows are numbered in ascending (b,oX,oY,oZ) (rules.cu:434-443)."""
    H, W, D = shape
    oH, oW, oD = out_shape
    b, x, y, z = row_coords(z_idx, z_ptr, B, H, W)
    KV = ksize[0] * ksize[1] * ksize[2]
    tgw = div_up(oW, tile[1])
    n_tile = div_up(oH, tile[0]) * tgw
    tnm = heuristic_tile_n_max(in_tile_size(tile[0], stride[0], ksize[0], dilation[0]),
                               in_tile_size(tile[1], stride[1], ksize[1], dilation[1]), B, H, W, D, z.shape[0])
    cand = []
    for k, rows, ox, oy, oz in _candidates(b, x, y, z, out_shape, ksize, stride, padding, dilation):
        key = ((b[rows] * oH + ox) * oW + oy) * oD + oz
        cand.append((rows, ox, oy, key))
    all_keys = np.concatenate([c[3] for c in cand]) if cand else np.zeros(0, np.int64)
    out_keys = np.unique(all_keys)                             # ascending key == ascending (b,oX,oY,oZ)
    oz_idx = (out_keys % oD).astype(np.int32)
    col = out_keys // oD
    counts = np.bincount(col, minlength=B * oH * oW)
    oz_ptr = np.cumsum(counts).astype(np.int32).reshape(B, oH, oW)
    pairs_k = []
    for rows, ox, oy, key in cand:
        out_row = np.searchsorted(out_keys, key)
        t = (ox // tile[0]) * tgw + oy // tile[1]
        pairs_k.append((t, rows, out_row))
    res = _finish(pairs_k, n_tile, KV, tnm, padded)
    res["oz_idx"] = oz_idx
    res["oz_ptr"] = oz_ptr
    return res


def canonical_pairs(rules, rule_size):
    """Sorted (tile, k, in, out) table of a padded rules tensor, reading only the first
    rule_size[tile,k] entries of each list (the parity definition: per-list multisets)."""
    rules = np.asarray(rules)
    rule_size = np.asarray(rule_size)
    n_tile, KV, _, tnm = rules.shape
    slot = np.arange(tnm)[None, None, :]
    valid = slot < np.minimum(rule_size, tnm)[:, :, None]
    t, k, s = np.nonzero(valid)
    ins = rules[t, k, 0, s].astype(np.int64)
    outs = rules[t, k, 1, s].astype(np.int64)
    order = np.lexsort((outs, ins, k, t))
    return np.stack([t[order], k[order], ins[order], outs[order]], axis=1)


def canonical_from_table(res):
    """Same table from the dict returned by get_rules*/get_rules_subm (already sorted)."""
    return np.stack([res["tile"], res["k"], res["in"], res["out"]], axis=1)
