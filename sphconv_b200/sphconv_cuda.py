"""The nine operators of the reference's ``sphconv.sphconv_cuda`` pybind module
(``src/sphconv/all.cpp:14-38``), same names, argument order and return values, over the C ABI.

Differences a caller can see, all documented:
  * feature dtypes fp32, fp16, bf16 and int8 are accepted (the reference hard-codes float);
  * pairs inside one (tile,k) list come in a deterministic order (the reference's is atomics order);
  * entries of ``rules`` past ``rule_size`` are -1 only when ``config.fill_unused_rules`` is set
    (no consumer reads them, ``include/sphconv/iterator.cu.h:173-177``);
  * errors raise ``RuntimeError`` instead of ``printf``/``exit``;
  * ``dilation`` is honoured: kernel offset k reads input o*stride - padding + k*dilation.  The reference's kernels
    ignore the argument (src/sphconv/rules.cu:40-41) while its ``out_spatial`` sizes the output for a dilated kernel
    (sphconv/utils/__init__.py:40-42); dilation 1, the only value its tests use, behaves identically.

``get_rules*`` attach the neighbour tables the convolution kernels read to the returned ``rules``
tensor (attribute ``_sph``).  Rules without it - cloned, loaded from disk, made elsewhere - are
converted on first use and the result is cached on the tensor until it is modified in place.
"""
import ctypes
from typing import List, Optional

import torch

from . import _capi as C


class config:
    """Process-wide switches."""
    fill_unused_rules = True   # -1 padding of `rules` as the reference (rules.cu:364-366)
    materialize_rules = True   # False: module path skips the padded `rules` tensor (rules/rule_size come back None)
    transposed_table = None    # None: build the dgrad table when grad mode is on; True/False forces it
    overlap_rule_lists = True  # module path: write the reference-format pair lists on a side stream, beside the conv
    exact_rule_capacity = False  # True: tile_n_max = the longest list (two passes + a host read), never an overflow


class _Tables:
    """Neighbour tables of one rule set.  nbr[k, o] = input row or -1; nbr_t[k, i] = output row or -1."""
    __slots__ = ("nbr", "nbr_t", "n_in", "n_out", "version", "symmetric")

    def __init__(self, nbr, nbr_t, n_in, n_out, version, symmetric):
        self.nbr, self.nbr_t, self.n_in, self.n_out = nbr, nbr_t, n_in, n_out
        self.version, self.symmetric = version, symmetric


def _want_transposed():
    if config.transposed_table is None:
        return torch.is_grad_enabled()
    return bool(config.transposed_table)


def _check_common(zIndices, zPtr, dilation):
    C.require_cuda(zIndices, zPtr)
    if zIndices.dtype != torch.int32 or zPtr.dtype != torch.int32:
        raise RuntimeError("z_idx and z_ptr must be int32")
    if any(int(d) < 1 for d in dilation):
        raise RuntimeError("dilation must be positive")


_side_streams = {}


def _side_stream(dev):
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    st = _side_streams.get(key)
    if st is None:
        st = torch.cuda.Stream(torch.device("cuda", key))
        _side_streams[key] = st
    return st


def _lists_beside(dev, g, oz_ptr, out_nnz, nbr, tnm, rules, rule_size):
    """The pair lists of a rule set whose table has been enqueued on the current stream, on the side stream: the
    convolution kernels read the table only, so they can run while the lists are written.  `rules` carries the
    event that marks the lists complete until `_join_lists` has ordered the current stream behind it."""
    main = torch.cuda.current_stream(dev)
    side = _side_stream(dev)
    tables_done = torch.cuda.Event()
    tables_done.record(main)
    side.wait_event(tables_done)
    from . import profiling
    with torch.cuda.device(dev), profiling.section("lists:" + profiling.current_rule_tag, stream=side):
        C.check(C.lib().sph_rule_lists(C.ptr(oz_ptr), ctypes.byref(g), out_nnz, C.ptr(nbr), tnm, C.ptr(rules),
                                       C.ptr(rule_size), int(config.fill_unused_rules), C.ptr(C.status_tensor(dev)),
                                       ctypes.c_void_p(side.cuda_stream)))
    lists_done = torch.cuda.Event()
    lists_done.record(side)
    for t in (rules, rule_size, nbr, oz_ptr):
        t.record_stream(side)
    rules._sph_ready = lists_done


def _join_lists(rules):
    """Orders the current stream behind the side-stream work that fills `rules` (if any is outstanding).  Called
    by every op right AFTER it has enqueued its own kernel, so that kernel overlaps the lists and everything the
    caller enqueues later sees them complete."""
    ev = getattr(rules, "_sph_ready", None) if isinstance(rules, torch.Tensor) else None
    if ev is not None:
        torch.cuda.current_stream(rules.device).wait_event(ev)
        rules._sph_ready = None


def _exact_lists(dev, g, oz_ptr, out_nnz, nbr, n_tile, kv):
    """rules / rule_size sized by the longest list: count, read the maximum, allocate, fill (all on the current
    stream).  The reference's heuristic capacity (rules.cu:21-28) can be too small, and then pairs are lost."""
    lib = C.lib()
    rule_size = torch.empty((n_tile, kv), dtype=torch.int32, device=dev)
    status = C.status_tensor(dev)
    with torch.cuda.device(dev):
        st = C.stream_ptr(dev)
        C.check(lib.sph_rule_lists(C.ptr(oz_ptr), ctypes.byref(g), out_nnz, C.ptr(nbr), 0, None, C.ptr(rule_size), 0,
                                   C.ptr(status), st))
        tnm = max(1, int(rule_size.max().item())) if rule_size.numel() else 1
        rules = torch.empty((n_tile, kv, 2, tnm), dtype=torch.int32, device=dev)
        C.check(lib.sph_rule_lists(C.ptr(oz_ptr), ctypes.byref(g), out_nnz, C.ptr(nbr), tnm, C.ptr(rules),
                                   C.ptr(rule_size), int(config.fill_unused_rules), C.ptr(status), st))
    return rules, rule_size


def get_rules_subm(zIndices: torch.Tensor, zPtr: torch.Tensor, batchSize: int, spatialShape: List[int],
                   outSpatialShape: List[int], kernelSize: List[int], stride: List[int], padding: List[int],
                   dilation: List[int], tileSize: List[int], defer_lists: bool = False):
    """ref: get_rules_subm, src/sphconv/rules.cu:326-390.  Returns [zIndices, zPtr, rules, ruleSize]
    (the first two are the input objects, as in the reference).  `defer_lists` (extension, used by the modules):
    rules / ruleSize are written on a side stream and are complete on the current stream only after one of the
    rule_conv* ops has been called with them."""
    _check_common(zIndices, zPtr, dilation)
    lib = C.lib()
    dev = zIndices.device
    nnz = zIndices.shape[0]
    g = C.make_geom(batchSize, spatialShape, outSpatialShape, kernelSize, stride, padding, tileSize, dilation)
    kv = int(kernelSize[0]) * int(kernelSize[1]) * int(kernelSize[2])
    n_tile = C.check(lib.sph_num_tiles(ctypes.byref(g)))
    rules = rule_size = None
    tnm = 0
    exact = config.materialize_rules and config.exact_rule_capacity
    if config.materialize_rules and not exact:
        tnm = C.check(lib.sph_tile_n_max(ctypes.byref(g), nnz))
        rules = torch.empty((n_tile, kv, 2, tnm), dtype=torch.int32, device=dev)
        rule_size = torch.empty((n_tile, kv), dtype=torch.int32, device=dev)
    nbr = torch.empty((kv, nnz), dtype=torch.int32, device=dev)
    scratch_bytes = C.check(lib.sph_rules_subm_scratch_bytes(ctypes.byref(g), nnz))
    scratch = torch.empty((scratch_bytes,), dtype=torch.uint8, device=dev) if scratch_bytes else None
    defer = bool(defer_lists) and config.overlap_rule_lists and rules is not None and nnz > 0
    with torch.cuda.device(dev):
        C.check(lib.sph_rules_subm(C.ptr(zIndices), C.ptr(zPtr), nnz, ctypes.byref(g), C.ptr(scratch), tnm,
                                   None if defer else C.ptr(rules), None if defer else C.ptr(rule_size), C.ptr(nbr),
                                   int(config.fill_unused_rules), C.ptr(C.status_tensor(dev)), C.stream_ptr(dev)))
    if defer:
        _lists_beside(dev, g, zPtr, nnz, nbr, tnm, rules, rule_size)
    if exact:
        rules, rule_size = _exact_lists(dev, g, zPtr, nnz, nbr, n_tile, kv)
    symmetric = all(int(k) % 2 == 1 and int(p) == int(d) * (int(k) // 2) and int(s) == 1
                    for k, p, s, d in zip(kernelSize, padding, stride, dilation))
    tables = _Tables(nbr, None, nnz, nnz, rules._version if rules is not None else 0, symmetric)
    if rules is not None:
        rules._sph = tables
        return [zIndices, zPtr, rules, rule_size]
    return [zIndices, zPtr, tables, None]


class PendingRules:
    """Step 1 of a strided rule set (output sparsity pattern) that has been enqueued but whose row count has not been
    read yet; `get_rules(..., pending=...)` completes it."""
    __slots__ = ("z_idx", "z_ptr", "key", "geom", "scratch", "oz_ptr", "d_count", "count_word", "event")

    def matches(self, zIndices, zPtr, key):
        return self.z_idx is zIndices and self.z_ptr is zPtr and self.key == key


def _geom_key(batchSize, spatialShape, outSpatialShape, kernelSize, stride, padding, tileSize, dilation=(1, 1, 1)):
    return (int(batchSize),) + tuple(int(v) for seq in (spatialShape, outSpatialShape, kernelSize, stride, padding,
                                                        tileSize, dilation) for v in seq)


def get_rules_begin(zIndices: torch.Tensor, zPtr: torch.Tensor, batchSize: int, spatialShape: List[int],
                    outSpatialShape: List[int], kernelSize: List[int], stride: List[int], padding: List[int],
                    dilation: List[int], tileSize: List[int]) -> PendingRules:
    """Enqueues step 1 of get_rules without waiting for the row count.  Work enqueued after this call (the
    convolution of the previous layer, say) keeps the GPU busy while the host later waits for the count."""
    _check_common(zIndices, zPtr, dilation)
    lib = C.lib()
    dev = zIndices.device
    nnz = zIndices.shape[0]
    p = PendingRules()
    p.z_idx, p.z_ptr = zIndices, zPtr
    p.key = _geom_key(batchSize, spatialShape, outSpatialShape, kernelSize, stride, padding, tileSize, dilation)
    p.geom = C.make_geom(batchSize, spatialShape, outSpatialShape, kernelSize, stride, padding, tileSize, dilation)
    scratch_bytes = C.check(lib.sph_rules_strided_scratch_bytes(ctypes.byref(p.geom), nnz))
    p.scratch = torch.empty((scratch_bytes,), dtype=torch.uint8, device=dev)
    p.oz_ptr = torch.empty((batchSize, int(outSpatialShape[0]), int(outSpatialShape[1])), dtype=torch.int32, device=dev)
    p.d_count = torch.empty((1,), dtype=torch.int32, device=dev)
    word = ctypes.c_void_p(0)
    with torch.cuda.device(dev):
        C.check(lib.sph_rules_strided_count_async(C.ptr(zIndices), C.ptr(zPtr), nnz, ctypes.byref(p.geom),
                                                  C.ptr(p.scratch), C.ptr(p.oz_ptr), C.ptr(p.d_count),
                                                  ctypes.byref(word), C.stream_ptr(dev)))
        p.event = torch.cuda.Event()
        p.event.record(torch.cuda.current_stream(dev))
    p.count_word = word.value
    return p


def get_rules(zIndices: torch.Tensor, zPtr: torch.Tensor, batchSize: int, spatialShape: List[int],
              outSpatialShape: List[int], kernelSize: List[int], stride: List[int], padding: List[int],
              dilation: List[int], tileSize: List[int], pending: Optional[PendingRules] = None,
              defer_lists: bool = False):
    """ref: get_rules, src/sphconv/rules.cu:405-486.  Returns [ozIndices, ozPtr, rules, ruleSize].
    `pending` (extension): the result of get_rules_begin on the same arguments; step 1 is then not run again.
    `defer_lists` (extension): as for get_rules_subm."""
    key = _geom_key(batchSize, spatialShape, outSpatialShape, kernelSize, stride, padding, tileSize, dilation)
    if pending is None or not pending.matches(zIndices, zPtr, key):
        pending = get_rules_begin(zIndices, zPtr, batchSize, spatialShape, outSpatialShape, kernelSize, stride,
                                  padding, dilation, tileSize)
    lib = C.lib()
    dev = zIndices.device
    nnz = zIndices.shape[0]
    g = pending.geom
    kv = int(kernelSize[0]) * int(kernelSize[1]) * int(kernelSize[2])
    n_tile = C.check(lib.sph_num_tiles(ctypes.byref(g)))
    scratch, oz_ptr = pending.scratch, pending.oz_ptr
    status = C.status_tensor(dev)
    pending.event.synchronize()      # the same device -> host read the reference does at rules.cu:461
    out_nnz = int(ctypes.c_int32.from_address(pending.count_word).value)
    with torch.cuda.device(dev):
        st = C.stream_ptr(dev)
        oz_idx = torch.empty((out_nnz,), dtype=torch.int32, device=dev)
        rules = rule_size = None
        tnm = 0
        exact = config.materialize_rules and config.exact_rule_capacity
        if config.materialize_rules and not exact:
            tnm = C.check(lib.sph_tile_n_max(ctypes.byref(g), nnz))
            rules = torch.empty((n_tile, kv, 2, tnm), dtype=torch.int32, device=dev)
            rule_size = torch.empty((n_tile, kv), dtype=torch.int32, device=dev)
        nbr = torch.empty((kv, out_nnz), dtype=torch.int32, device=dev)
        nbr_t = torch.empty((kv, nnz), dtype=torch.int32, device=dev) if _want_transposed() else None
        defer = bool(defer_lists) and config.overlap_rule_lists and rules is not None and out_nnz > 0
        C.check(lib.sph_rules_strided_fill(C.ptr(zIndices), C.ptr(zPtr), nnz, ctypes.byref(g), C.ptr(scratch),
                                           C.ptr(oz_ptr), out_nnz, tnm, C.ptr(oz_idx),
                                           None if defer else C.ptr(rules), None if defer else C.ptr(rule_size),
                                           C.ptr(nbr), C.ptr(nbr_t), int(config.fill_unused_rules), C.ptr(status), st))
    if defer:
        _lists_beside(dev, g, oz_ptr, out_nnz, nbr, tnm, rules, rule_size)
    if exact:
        rules, rule_size = _exact_lists(dev, g, oz_ptr, out_nnz, nbr, n_tile, kv)
    tables = _Tables(nbr, nbr_t, nnz, out_nnz, rules._version if rules is not None else 0, False)
    if rules is not None:
        rules._sph = tables
        return [oz_idx, oz_ptr, rules, rule_size]
    return [oz_idx, oz_ptr, tables, None]


def _tables_for(rules, rule_size, n_in: int, n_out: int, need_t: bool) -> _Tables:
    """Neighbour tables of a rule set: the ones attached by get_rules*, or a conversion of the
    reference-format tensors (cached on `rules`)."""
    if isinstance(rules, _Tables):
        tb = rules
    else:
        tb = getattr(rules, "_sph", None)
        if tb is not None and (tb.version != rules._version or tb.n_in != n_in or tb.n_out != n_out):
            tb = None
    if tb is not None and (not need_t or tb.nbr_t is not None or tb.symmetric):
        return tb
    if isinstance(rules, _Tables):
        raise RuntimeError("this rule set was generated without the transposed table; enable grad mode (or "
                           "config.transposed_table) before generating rules that backward will use")
    C.require_cuda(rules, rule_size)
    lib = C.lib()
    dev = rules.device
    n_tile, kv, _, tnm = rules.shape
    nbr = tb.nbr if tb is not None else torch.empty((kv, n_out), dtype=torch.int32, device=dev)
    nbr_t = torch.empty((kv, n_in), dtype=torch.int32, device=dev) if need_t else None
    with torch.cuda.device(dev):
        C.check(lib.sph_rules_to_nbr(C.ptr(rules), C.ptr(rule_size), n_tile, kv, tnm, n_in, n_out,
                                     None if tb is not None else C.ptr(nbr), C.ptr(nbr_t),
                                     C.ptr(C.status_tensor(dev)), C.stream_ptr(dev)))
    new = _Tables(nbr, nbr_t, n_in, n_out, rules._version, tb.symmetric if tb is not None else False)
    rules._sph = new
    return new


def _packed_weight(weight: torch.Tensor):
    """UMMA image of a [KV, K, N] weight, or None when the CUDA-core kernel will run.  Cached on the tensor."""
    code = C.DTYPE_CODE[weight.dtype]
    kv, k_ch, n_ch = weight.shape
    lib = C.lib()
    nbytes = lib.sph_packed_weight_bytes(code, kv, k_ch, n_ch)
    if nbytes <= 0:
        return None
    cached = getattr(weight, "_sph_packed", None)
    if cached is not None and cached[0] == weight._version:
        return cached[1]
    packed = torch.empty((nbytes,), dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        C.check(lib.sph_pack_weight(C.ptr(weight), code, kv, k_ch, n_ch, C.ptr(packed), C.stream_ptr(weight.device)))
    weight._sph_packed = (weight._version, packed)
    return packed


def _gather(rows, weight, nbr, n_out, flip_k, scale, bias, relu, out_dtype):
    C.require_cuda(rows, weight, nbr, scale, bias)
    if rows.dtype not in C.DTYPE_CODE:
        raise RuntimeError("unsupported feature dtype %s" % rows.dtype)
    if weight.dtype != rows.dtype:
        raise RuntimeError("feature (%s) and weight (%s) dtypes differ" % (rows.dtype, weight.dtype))
    kv, k_ch, n_ch = weight.shape
    if rows.dim() != 2 or rows.shape[1] != k_ch:
        raise RuntimeError("feature has %d channels, weight expects %d" % (rows.shape[-1], k_ch))
    if out_dtype is None:
        out_dtype = torch.float32 if rows.dtype == torch.int8 else rows.dtype
    dev = rows.device
    out = torch.empty((n_out, n_ch), dtype=out_dtype, device=dev)
    if n_out == 0:
        return out
    packed = _packed_weight(weight)
    for v in (scale, bias):
        if v is not None and (v.dtype != torch.float32 or v.numel() != n_ch):
            raise RuntimeError("scale / bias must be float32 [out_channels]")
    with torch.cuda.device(dev):
        C.check(C.lib().sph_conv_gather(C.ptr(rows), C.DTYPE_CODE[rows.dtype], rows.shape[0], C.ptr(weight),
                                        C.ptr(packed), C.ptr(nbr), n_out, kv, k_ch, n_ch, int(bool(flip_k)),
                                        C.ptr(scale), C.ptr(bias), int(bool(relu)), C.ptr(out),
                                        C.DTYPE_CODE[out_dtype], C.ptr(C.status_tensor(dev)), C.stream_ptr(dev)))
    return out


def rule_conv(feature: torch.Tensor, weight: torch.Tensor, rules, ruleSize, outNNZ: int, *,
              scale: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, relu: bool = False,
              out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """ref: rule_conv, src/sphconv/rule_conv.cu:286-336.  feature [NNZ,iC], weight [KV,iC,oC] ->
    [outNNZ,oC].  Keyword arguments are extensions (fused epilogue relu(acc*scale + bias), output dtype)."""
    tb = _tables_for(rules, ruleSize, feature.shape[0], int(outNNZ), need_t=False)
    out = _gather(feature, weight, tb.nbr, int(outNNZ), False, scale, bias, relu, out_dtype)
    if getattr(rules, "_sph_ready", None) is not None:
        from . import profiling
        profiling.mark_stop()          # a timed section around this call ends with the kernel, not with the join
    _join_lists(rules)
    return out


def rule_conv_d_feature(feature: torch.Tensor, weight: torch.Tensor, rules, ruleSize,
                        tile_grid_shape: List[int], outNNZ: int) -> torch.Tensor:
    """ref: rule_conv_d_feature, src/sphconv/rule_conv.cu:520-575.  `feature` is the upstream gradient
    [outNNZ_fwd, oC], `weight` the [KV,oC,iC] transpose, `outNNZ` the number of input rows; returns [outNNZ, iC].
    tile_grid_shape is accepted for signature compatibility (the reference needs it for its 9-colour launches)."""
    n_in = int(outNNZ)
    tb = _tables_for(rules, ruleSize, n_in, feature.shape[0], need_t=True)
    if tb.nbr_t is not None:
        return _gather(feature, weight, tb.nbr_t, n_in, False, None, None, False, None)
    # odd-kernel submanifold layer: (i,o) at k  <=>  (o,i) at KV-1-k, so the forward table serves
    return _gather(feature, weight, tb.nbr, n_in, True, None, None, False, None)


def rule_conv_d_weight(feature: torch.Tensor, d_featureOut: torch.Tensor, rules, ruleSize, *,
                       out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """ref: rule_conv_d_weight, src/sphconv/rule_conv.cu:469-518.  Returns float32 [KV,iC,oC].
    Keyword arguments are extensions: `out` is a caller-owned contiguous float32 [KV,iC,oC] tensor (e.g. a slice
    of a flat gradient buffer) the kernel writes instead of a fresh one; with `accumulate` it adds to what is there."""
    C.require_cuda(feature, d_featureOut, out)
    if feature.dtype != d_featureOut.dtype:
        raise RuntimeError("feature and gradient dtypes differ")
    tb = _tables_for(rules, ruleSize, feature.shape[0], d_featureOut.shape[0], need_t=False)
    kv = tb.nbr.shape[0]
    k_ch, n_ch = feature.shape[1], d_featureOut.shape[1]
    dev = feature.device
    if out is None:
        dw = torch.empty((kv, k_ch, n_ch), dtype=torch.float32, device=dev)
        accumulate = False
    else:
        if out.dtype != torch.float32 or out.numel() != kv * k_ch * n_ch:
            raise RuntimeError("out must be float32 with %d x %d x %d elements" % (kv, k_ch, n_ch))
        dw = out
    with torch.cuda.device(dev):
        C.check(C.lib().sph_conv_wgrad(C.ptr(feature), C.ptr(d_featureOut), C.DTYPE_CODE[feature.dtype],
                                       feature.shape[0], C.ptr(tb.nbr), d_featureOut.shape[0], kv, k_ch, n_ch,
                                       C.ptr(dw), 0 if accumulate else 1, C.ptr(C.status_tensor(dev)),
                                       C.stream_ptr(dev)))
    _join_lists(rules)
    return dw


def rule_conv_backward(d_featureOut: torch.Tensor, feature: torch.Tensor, weight: torch.Tensor, rules, ruleSize,
                       tile_grid_shape: List[int]):
    """ref: rule_conv_backward, src/sphconv/rule_conv.cu:577-597.  `weight` is [KV,oC,iC].
    Returns [d_feature [NNZ,iC], d_weight [KV,iC,oC]] in the dtype of `feature`."""
    d_featureOut = d_featureOut.contiguous()
    d_feature = rule_conv_d_feature(d_featureOut, weight, rules, ruleSize, tile_grid_shape, feature.shape[0])
    d_weight = rule_conv_d_weight(feature, d_featureOut, rules, ruleSize).to(feature.dtype)
    return [d_feature, d_weight]


# ---- tensor ops on either side of the path: COO -> range-voxel, range-voxel <-> dense -----------------------

def _shape3(spatialShape):
    return (ctypes.c_int32 * 3)(*[int(v) for v in spatialShape])


def init_tensor(feature: torch.Tensor, indicesBZYX: torch.Tensor, batchSize: int, spatialShape: List[int]):
    """ref: init_tensor, src/sphconv/tensor.cu:78-127.  COO (b, s0, s1, s2) -> range-voxel.
    Returns [feature', zIndices, zPtr, permutation] with permutation[n] = new row of input row n.
    Rows inside a column are ordered by depth (the reference's order is atomics arrival order).  Any dtype."""
    C.require_cuda(feature, indicesBZYX)
    if indicesBZYX.dim() != 2 or indicesBZYX.shape[1] != 4 or indicesBZYX.is_floating_point():
        raise RuntimeError("indices must be an integer tensor [NNZ, 4]")
    if feature.dim() != 2 or feature.shape[0] != indicesBZYX.shape[0]:
        raise RuntimeError("feature must be [NNZ, C] with one row per index")
    lib = C.lib()
    dev = feature.device
    feature = feature.contiguous()
    idx = indicesBZYX.to(torch.int32).contiguous()
    nnz = feature.shape[0]
    shape = _shape3(spatialShape)
    out = torch.empty_like(feature)
    z_idx = torch.empty((nnz,), dtype=torch.int32, device=dev)
    z_ptr = torch.empty((int(batchSize), int(spatialShape[0]), int(spatialShape[1])), dtype=torch.int32, device=dev)
    perm = torch.empty((nnz,), dtype=torch.int32, device=dev)
    nbytes = C.check(lib.sph_init_tensor_scratch_bytes(int(batchSize), shape))
    scratch = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        C.check(lib.sph_init_tensor(C.ptr(feature), feature.shape[1] * feature.element_size(), nnz, C.ptr(idx),
                                    int(batchSize), shape, C.ptr(scratch), C.ptr(out), C.ptr(z_idx), C.ptr(z_ptr),
                                    C.ptr(perm), C.ptr(C.status_tensor(dev)), C.stream_ptr(dev)))
    return [out, z_idx, z_ptr, perm]


def init_tensor_backward(d_featureOut: torch.Tensor, permutation: torch.Tensor) -> torch.Tensor:
    """ref: init_tensor_backward, src/sphconv/tensor.cu:147-162: d_feature[n] = d_featureOut[permutation[n]]."""
    C.require_cuda(d_featureOut, permutation)
    d = d_featureOut.contiguous()
    perm = permutation.contiguous()
    if perm.dtype != torch.int32:
        raise RuntimeError("permutation must be int32")
    out = torch.empty_like(d)
    with torch.cuda.device(d.device):
        C.check(C.lib().sph_permute_rows(C.ptr(d), d.shape[1] * d.element_size(), d.shape[0], C.ptr(perm), 1, C.ptr(out),
                                         C.stream_ptr(d.device)))
    return out


def to_dense(feature: torch.Tensor, zIndices: torch.Tensor, zPtr: torch.Tensor, D: int, out: torch.Tensor):
    """ref: to_dense, src/sphconv/tensor.cu:222-264.  Fills out [B,H,W,D,C] in place and returns it.
    The integer argument is unused, as in the reference kernel, which takes every size from `out`."""
    C.require_cuda(feature, zIndices, zPtr, out)
    if not out.is_contiguous() or out.dim() != 5 or out.dtype != feature.dtype or out.shape[4] != feature.shape[1]:
        raise RuntimeError("out must be a contiguous [B,H,W,D,C] tensor of the feature dtype")
    f = feature.contiguous()
    with torch.cuda.device(f.device):
        C.check(C.lib().sph_to_dense(C.ptr(f), f.shape[1] * f.element_size(), f.shape[0], C.ptr(zIndices.contiguous()),
                                     C.ptr(zPtr.contiguous()), out.shape[0], _shape3(out.shape[1:4]), C.ptr(out), 0,
                                     C.ptr(C.status_tensor(f.device)), C.stream_ptr(f.device)))
    return out


def to_dense_backward(d_featureOut: torch.Tensor, zIndices: torch.Tensor, zPtr: torch.Tensor) -> torch.Tensor:
    """ref: to_dense_backward, src/sphconv/tensor.cu:266-309.  d_featureOut [B,H,W,D,C] -> [NNZ,C]."""
    C.require_cuda(d_featureOut, zIndices, zPtr)
    d = d_featureOut.contiguous()
    nnz = zIndices.shape[0]
    out = torch.empty((nnz, d.shape[4]), dtype=d.dtype, device=d.device)
    with torch.cuda.device(d.device):
        C.check(C.lib().sph_to_dense(C.ptr(out), d.shape[4] * d.element_size(), nnz, C.ptr(zIndices.contiguous()),
                                     C.ptr(zPtr.contiguous()), d.shape[0], _shape3(d.shape[1:4]), C.ptr(d), 1,
                                     C.ptr(C.status_tensor(d.device)), C.stream_ptr(d.device)))
    return out


def epilogue_backward(d_out: torch.Tensor, out: Optional[torch.Tensor], relu: bool, need_bias: bool):
    """Backward of the fused epilogue relu(acc + bias) (extension, no reference counterpart): returns
    (d_pre, d_bias fp32 [C] or None) with d_pre = d_out masked by (out > 0) when `relu`."""
    d_out = d_out.contiguous()
    out = None if out is None else out.contiguous()
    C.require_cuda(d_out, out)
    n, ch = d_out.shape
    if d_out.dtype not in (torch.float32, torch.float16, torch.bfloat16) or ch > 256:
        raise RuntimeError("epilogue_backward: float32 / float16 / bfloat16 gradients with at most 256 channels")
    dev = d_out.device
    d_pre = torch.empty_like(d_out) if relu else None
    d_bias = torch.empty((ch,), dtype=torch.float32, device=dev) if need_bias else None
    if d_pre is None and d_bias is None:
        return d_out, None
    with torch.cuda.device(dev):
        C.check(C.lib().sph_epilogue_backward(C.ptr(d_out), C.ptr(out) if relu else None,
                                              C.DTYPE_CODE[d_out.dtype], n, ch, int(bool(relu)), C.ptr(d_pre),
                                              C.ptr(d_bias), C.stream_ptr(dev)))
    return (d_pre if relu else d_out), d_bias
