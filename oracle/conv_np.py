"""CPU restatement of the rule-driven sparse convolution (forward, dgrad, wgrad).

Test infrastructure; never imported by the product.

* forward  ``out[o,:] = sum_k sum_{(i,o) in rule k} feat[i,:] @ W[k]``
  (include/sphconv/rule_conv_kernel.cu.h:96-152; output zero-initialised, src/sphconv/rule_conv.cu:302-304)
* dgrad    ``dX[i,:] = sum_k sum_{(i,o)} dY[o,:] @ W[k]^T``
  (src/sphconv/rule_conv.cu:520-575; the Python caller transposes the weight, sphconv/functional.py:70-74)
* wgrad    ``dW[k] = sum_{(i,o) in rule k} feat[i,:]^T dY[o,:]`` summed over tiles
  (src/sphconv/rule_conv.cu:469-518, the per-tile partials are summed at line 517)

``pairs`` is the canonical table [(tile, k, in, out)] from ``rules_np``; arithmetic is float64 unless asked otherwise.

Inside one kernel offset k the map input row <-> output row is one-to-one (an output voxel and an offset name
exactly one input voxel, src/sphconv/rules.cu:124-133), so the scatter of one offset has no repeated target and is a
plain indexed add; ``np.add.at`` is kept behind ``unique_per_k=False`` for pair tables that do not come from rules.
"""
import numpy as np


def _scatter_add(dst, idx, val, unique):
    if unique:
        dst[idx] += val
    else:
        np.add.at(dst, idx, val)


def _by_k(pairs, KV):
    pairs = np.asarray(pairs)
    for k in range(KV):
        sel = pairs[:, 1] == k
        if sel.any():
            yield k, pairs[sel, 2], pairs[sel, 3]


def conv_forward(feature, weight, pairs, out_nnz, dtype=np.float64, unique_per_k=True):
    """feature [NNZ,iC], weight [KV,iC,oC] -> [out_nnz,oC]."""
    f = np.asarray(feature, dtype=dtype)
    w = np.asarray(weight, dtype=dtype)
    out = np.zeros((out_nnz, w.shape[2]), dtype=dtype)
    for k, i, o in _by_k(pairs, w.shape[0]):
        _scatter_add(out, o, f[i] @ w[k], unique_per_k)
    return out


def conv_dgrad(d_out, weight, pairs, nnz, dtype=np.float64, unique_per_k=True):
    """d_out [outNNZ,oC], weight [KV,iC,oC] (un-transposed) -> d_feature [nnz,iC]."""
    g = np.asarray(d_out, dtype=dtype)
    w = np.asarray(weight, dtype=dtype)
    dx = np.zeros((nnz, w.shape[1]), dtype=dtype)
    for k, i, o in _by_k(pairs, w.shape[0]):
        _scatter_add(dx, i, g[o] @ w[k].T, unique_per_k)
    return dx


def conv_wgrad(feature, d_out, pairs, KV, dtype=np.float64):
    """-> d_weight [KV,iC,oC]."""
    f = np.asarray(feature, dtype=dtype)
    g = np.asarray(d_out, dtype=dtype)
    dw = np.zeros((KV, f.shape[1], g.shape[1]), dtype=dtype)
    for k, i, o in _by_k(pairs, KV):
        dw[k] = f[i].T @ g[o]
    return dw
