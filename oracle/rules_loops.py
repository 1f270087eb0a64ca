"""Loop-for-loop CPU restatement of the reference rule generation (small cases only).

Test infrastructure; never imported by the product.  Every function names the reference
lines it follows (paths relative to the reference project).  The CUDA thread grid of each
reference kernel becomes explicit Python loops over (x, y, k); the dense ``grid`` tensor of
the reference is kept as a numpy array so the control flow can be compared line by line.

The order of pairs inside one (tile, k) list is arrival order of atomics in the reference and
therefore unspecified; here it is the loop order.  Compare lists after sorting.
"""
import numpy as np


def div_up(x, y):
    """include/sphconv/debug_utils.h:17-20"""
    return (x + y - 1) // y


def linear_tile_idx(tile0, tile1, x, y, tile_grid_w):
    """include/sphconv/debug_utils.h:37-42"""
    return (x // tile0) * tile_grid_w + (y // tile1)


def in_tile_size(out_tile, stride, ksize, dilation=1):
    """src/sphconv/rules.cu:30-34 (dilation = 1 there: a dilated kernel spans dilation * (ksize - 1) + 1 inputs)."""
    assert stride <= ksize
    return stride * (out_tile - 1) + dilation * (ksize - 1) + 1


def heuristic_tile_n_max(in_tile_h, in_tile_w, B, H, W, D, nnz):
    """src/sphconv/rules.cu:21-28 (double arithmetic, truncation, then clear the low 4 bits)."""
    sparsity = float(nnz) / float(B * H * W * D)
    size = B * in_tile_h * in_tile_w * D * sparsity * 2
    return int(size + 64) & ~15


def c_rem(a, b):
    """C '%' (sign follows the dividend)."""
    r = abs(a) % abs(b)
    return -r if a < 0 else r


def c_div(a, b):
    """C '/' (truncation toward zero)."""
    q = abs(a) // abs(b)
    return -q if (a < 0) != (b < 0) else q


def out_coord(k, x, s, pad, d=1):
    """src/sphconv/rules.cu:36-45.  The reference ignores dilation here (d = 1); for d != 1 offset k reads input
    o*s - pad + k*d, the definition its own out_spatial implies (sphconv/utils/__init__.py:40-42)."""
    if c_rem(x + pad - k * d, s) == 0:
        return c_div(x + pad - k * d, s)
    return -1


def _col_range(zp_flat, b, x, y, H, W):
    """Column [start, end): src/sphconv/rules.cu:72-74,137-138 (flat inclusive prefix)."""
    c = (b * H + x) * W + y
    end = int(zp_flat[c])
    start = 0 if c == 0 else int(zp_flat[c - 1])
    return start, end


def get_rules_subm(z_idx, z_ptr, B, shape, out_shape, ksize, stride, padding, dilation, tile):
    """src/sphconv/rules.cu:326-390 with kernels 55-82 and 234-311."""
    H, W, D = shape
    oH, oW, oD = out_shape
    KH, KW, KD = ksize
    zp = np.asarray(z_ptr).reshape(-1)
    zi = np.asarray(z_idx).reshape(-1)
    nnz = zi.shape[0]
    grid = np.full((B, oH, oW, oD), -1, dtype=np.int64)         # rules.cu:339-340
    for x in range(H):                                          # prepareSubMGridKernel 55-82
        for y in range(W):
            for b in range(B):
                s, e = _col_range(zp, b, x, y, H, W)
                for pos in range(s, e):
                    grid[b, x, y, zi[pos]] = pos
    KV = KH * KW * KD
    n_tile = div_up(oH, tile[0]) * div_up(oW, tile[1])          # rules.cu:353
    tnm = heuristic_tile_n_max(in_tile_size(tile[0], stride[0], KH, dilation[0]),
                               in_tile_size(tile[1], stride[1], KW, dilation[1]), B, H, W, D, nnz)                 # rules.cu:356-359
    rules = np.full((n_tile, KV, 2, tnm), -1, dtype=np.int32)   # rules.cu:364-366
    rule_size = np.zeros((n_tile, KV), dtype=np.int32)          # rules.cu:368-369
    tgw = div_up(oW, tile[1])
    for k in range(KV):                                         # getSubMRulesKernel 234-311
        kh, kw, kd = k // (KW * KD), (k // KD) % KW, k % KD
        for x in range(H):
            ox = out_coord(kh, x, stride[0], padding[0], dilation[0])
            if ox < 0 or ox >= oH:
                continue
            for y in range(W):
                oy = out_coord(kw, y, stride[1], padding[1], dilation[1])
                if oy < 0 or oy >= oW:
                    continue
                t = linear_tile_idx(tile[0], tile[1], ox, oy, tgw)
                for b in range(B):
                    s, e = _col_range(zp, b, x, y, H, W)
                    for gin in range(s, e):
                        oz = out_coord(kd, int(zi[gin]), stride[2], padding[2], dilation[2])
                        if oz < 0 or oz >= oD:
                            continue
                        gout = grid[b, ox, oy, oz]
                        if gout < 0:
                            continue
                        c = rule_size[t, k]
                        rule_size[t, k] += 1
                        if c < tnm:
                            rules[t, k, 0, c] = gin
                            rules[t, k, 1, c] = gout
    return zi.astype(np.int32), np.asarray(z_ptr, dtype=np.int32), rules, rule_size


def get_rules(z_idx, z_ptr, B, shape, out_shape, ksize, stride, padding, dilation, tile):
    """src/sphconv/rules.cu:405-486 with kernels 98-150 and 156-228 and the scans 434-443."""
    H, W, D = shape
    oH, oW, oD = out_shape
    KH, KW, KD = ksize
    zp = np.asarray(z_ptr).reshape(-1)
    zi = np.asarray(z_idx).reshape(-1)
    nnz = zi.shape[0]
    KV = KH * KW * KD
    grid = np.zeros((B, oH, oW, oD), dtype=np.int64)            # rules.cu:417-418
    for k in range(KV):                                         # prepareGridKernel 98-150
        kh, kw, kd = k // (KW * KD), (k // KD) % KW, k % KD
        for x in range(H):
            ox = out_coord(kh, x, stride[0], padding[0], dilation[0])
            if ox < 0 or ox >= oH:
                continue
            for y in range(W):
                oy = out_coord(kw, y, stride[1], padding[1], dilation[1])
                if oy < 0 or oy >= oW:
                    continue
                for b in range(B):
                    s, e = _col_range(zp, b, x, y, H, W)
                    for pos in range(s, e):
                        oz = out_coord(kd, int(zi[pos]), stride[2], padding[2], dilation[2])
                        if oz < 0 or oz >= oD:
                            continue
                        grid[b, ox, oy, oz] = 1
    grid = np.cumsum(grid, axis=3)                              # rules.cu:434
    oz_ptr = np.cumsum(grid[:, :, :, -1].reshape(-1)).reshape(B, oH, oW)   # rules.cu:438-439
    excl = np.roll(oz_ptr.reshape(-1), 1)                       # rules.cu:441-442
    excl[0] = 0
    grid = grid + excl.reshape(B, oH, oW, 1)                    # rules.cu:443 (1-based global out row)
    n_tile = div_up(oH, tile[0]) * div_up(oW, tile[1])
    tnm = heuristic_tile_n_max(in_tile_size(tile[0], stride[0], KH, dilation[0]),
                               in_tile_size(tile[1], stride[1], KW, dilation[1]), B, H, W, D, nnz)
    rules = np.full((n_tile, KV, 2, tnm), -1, dtype=np.int32)
    rule_size = np.zeros((n_tile, KV), dtype=np.int32)
    out_nnz = int(oz_ptr.reshape(-1)[-1]) if oz_ptr.size else 0  # rules.cu:461
    oz_idx = np.zeros((out_nnz,), dtype=np.int32)
    tgw = div_up(oW, tile[1])
    for k in range(KV):                                         # getOzIndicesAndRulesKernel 156-228
        kh, kw, kd = k // (KW * KD), (k // KD) % KW, k % KD
        for x in range(H):
            ox = out_coord(kh, x, stride[0], padding[0], dilation[0])
            if ox < 0 or ox >= oH:
                continue
            for y in range(W):
                oy = out_coord(kw, y, stride[1], padding[1], dilation[1])
                if oy < 0 or oy >= oW:
                    continue
                t = linear_tile_idx(tile[0], tile[1], ox, oy, tgw)
                for b in range(B):
                    s, e = _col_range(zp, b, x, y, H, W)
                    for gin in range(s, e):
                        oz = out_coord(kd, int(zi[gin]), stride[2], padding[2], dilation[2])
                        if oz < 0 or oz >= oD:
                            continue
                        gout = int(grid[b, ox, oy, oz]) - 1
                        c = rule_size[t, k]
                        rule_size[t, k] += 1
                        if c < tnm:
                            rules[t, k, 0, c] = gin
                            rules[t, k, 1, c] = gout
                        oz_idx[gout] = oz
    return oz_idx, oz_ptr.astype(np.int32), rules, rule_size
