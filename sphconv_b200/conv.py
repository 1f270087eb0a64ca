"""Sparse convolution modules (ref: sphconv/conv.py)."""
import math
from typing import List, Optional

import torch
import torch.nn as nn

from . import profiling
from . import sphconv_cuda as ops
from .functional import ConvFunction
from .modules import SphModule
from .tensor import SparseConvTensor
from .utils import _calculate_fan_in_and_fan_out, _triple, kaiming_uniform_, out_spatial


def divUp(x, y):
    return (x + y - 1) // y


def get_tile_grid_shape(out_spatial_shape_DWH: List[int], tile_size: List[int]) -> List[int]:
    """ref: sphconv/conv.py:32-38"""
    return [divUp(out_spatial_shape_DWH[0], tile_size[0]), divUp(out_spatial_shape_DWH[1], tile_size[1])]


class Convolution(SphModule):
    """Base class: owns weight [k0,k1,k2,iC,oC] and the optional bias (ref: sphconv/conv.py:40-96)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: List[int], stride: List[int],
                 padding: List[int], dilation: List[int], groups: int, tile_size: List[int], bias: bool, subm: bool,
                 name: str, indice_key: Optional[str] = None, **kwargs):
        super().__init__(**kwargs)
        # attribute and parameter names are the reference's (state_dict and user code read them)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.dilation = kernel_size, stride, padding, dilation
        self.groups, self.tile_size, self.subm = groups, tile_size, subm
        self.indice_key, self.name = indice_key, name
        self.weight = nn.Parameter(torch.empty((*kernel_size, in_channels, out_channels)))
        self.register_parameter('bias', nn.Parameter(torch.empty(out_channels)) if bias else None)
        self.reset_parameters()

    def reset_parameters(self):
        """Kaiming-uniform weight with a = sqrt(5) and a bias uniform in +-1/sqrt(fan_in), the fan computed the way the
        reference's initialiser computes it for the [k0,k1,k2,iC,oC] layout (sphconv/utils/__init__.py:57-124)."""
        kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in = _calculate_fan_in_and_fan_out(self.weight)[0]
            nn.init.uniform_(self.bias, -1.0 / math.sqrt(fan_in), 1.0 / math.sqrt(fan_in))

    def extra_repr(self):
        parts = ["{}, {}".format(self.in_channels, self.out_channels), "kernel_size={}".format(self.kernel_size),
                 "stride={}".format(self.stride)]
        if any(p != 0 for p in self.padding):
            parts.append("padding={}".format(self.padding))
        if any(d != 1 for d in self.dilation):
            parts.append("dilation={}".format(self.dilation))
        if self.groups != 1:
            parts.append("groups={}".format(self.groups))
        if self.bias is None:
            parts.append("bias=False")
        if self.subm:
            parts.append("subm=True")
        return ", ".join(parts)


class Conv3d(Convolution):
    """3-D sparse convolution on range-voxel tensors (ref: sphconv/conv.py:99-193).

    Reference behaviour is the default: the bias parameter exists but is not applied
    (sphconv/conv.py:182-185).  Two opt-in extensions: `apply_bias=True` adds it and
    `activation='relu'` applies ReLU; without grad both are fused into the kernel's epilogue."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, padding=0, dilation=1, groups=1,
                 bias=False, subm=False, tile_size=[2, 2], indice_key=None, name=None, apply_bias=False,
                 activation=None, **kwargs):
        kernel_size = _triple(kernel_size)
        stride = _triple(stride)
        padding = _triple(padding)
        dilation = _triple(dilation)
        assert groups == 1, "groups not supported yet"
        assert activation in (None, 'relu')
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, tile_size, bias,
                         subm, name, indice_key=indice_key, **kwargs)
        self.apply_bias = apply_bias
        self.activation = activation

    def _rules(self, input: SparseConvTensor, in_shape, out_shape):
        args = (input.z_idx, input.z_ptr, input.B, in_shape, out_shape, self.kernel_size, self.stride, self.padding,
                self.dilation, self.tile_size)
        # defer_lists: the reference-format pair lists are written on a side stream while this layer's convolution,
        # which reads the neighbour table only, runs; rule_conv orders the stream behind them again
        if self.subm:
            oz_idx, oz_ptr, rules, rule_size = ops.get_rules_subm(*args, defer_lists=True)
        else:
            pending = input.rule_cache.pop(("pending", id(self)), None)
            oz_idx, oz_ptr, rules, rule_size = ops.get_rules(*args, pending=pending, defer_lists=True)
        return oz_idx, oz_ptr, rules, rule_size, get_tile_grid_shape(out_shape, self.tile_size)

    def _rule_meta(self, input, in_shape, out_shape):
        """Sizes a timed rule-generation section carries (for byte accounting by whoever reads the timings)."""
        tg = get_tile_grid_shape(out_shape, self.tile_size)
        return dict(subm=self.subm, n_in=input.feature.shape[0], B=input.B, in_shape=list(in_shape),
                    out_shape=list(out_shape), n_tile=tg[0] * tg[1],
                    kv=self.kernel_size[0] * self.kernel_size[1] * self.kernel_size[2])

    def begin_rules(self, input: SparseConvTensor):
        """Extension used by Sequential: enqueue the first step of this (strided) layer's rule generation on a tensor
        that has the geometry this layer will see - the input of the submanifold layer in front of it - so that
        the layer in front runs on the GPU while the host waits for the output row count.  The handle travels in
        the tensor's rule cache, which the layers of a stack share."""
        if self.subm or (self.indice_key is not None and input.find_rule(self.indice_key) is not None):
            return
        in_shape = [input.D, input.W, input.H]
        out_shape = out_spatial(in_shape, self.kernel_size, self.stride, self.padding, self.dilation)
        tag = self.name or "conv{}_{}".format(self.in_channels, self.weight.shape[4])
        with profiling.section("rules:" + tag, **self._rule_meta(input, in_shape, out_shape)):
            input.rule_cache[("pending", id(self))] = ops.get_rules_begin(
                input.z_idx, input.z_ptr, input.B, in_shape, out_shape, self.kernel_size, self.stride, self.padding,
                self.dilation, self.tile_size)

    def forward(self, input: SparseConvTensor):
        batch_size, in_channels = input.B, input.C
        out_channels = self.weight.shape[4]
        assert self.in_channels == in_channels, \
            "input channel does not match Expect: {}, got {}".format(self.in_channels, in_channels)
        in_shape = [input.D, input.W, input.H]
        out_shape = in_shape
        if not self.subm:
            out_shape = out_spatial(in_shape, self.kernel_size, self.stride, self.padding, self.dilation)

        tag = self.name or "{}{}_{}".format("subm" if self.subm else "conv", in_channels, out_channels)
        datas = input.find_rule(self.indice_key) if self.indice_key is not None else None
        if datas is None:
            profiling.current_rule_tag = tag
            with profiling.section("rules:" + tag, **self._rule_meta(input, in_shape, out_shape)):
                datas = self._rules(input, in_shape, out_shape)
            if self.indice_key is not None:
                input.rule_cache[self.indice_key] = datas
        oz_idx, oz_ptr, rules, rule_size, tile_grid_shape = datas
        self.rule_size = rule_size

        weight = self.weight.view((-1, in_channels, out_channels))
        if weight.dtype != input.feature.dtype and input.feature.dtype != torch.int8:
            weight = weight.to(input.feature.dtype)
        bias = self.bias if (self.apply_bias and self.bias is not None) else None
        needs_grad = torch.is_grad_enabled() and (input.feature.requires_grad or self.weight.requires_grad)
        if needs_grad:
            profiling.current_tag = tag
            # bias and activation run in the kernel's epilogue in training too (extension arguments of ConvFunction)
            mw = getattr(self.weight, "_sph_master_grad", None)      # slices of a sharding.GradBuffer, if attached
            mb = getattr(bias, "_sph_master_grad", None) if bias is not None else None
            master = None if mw is None and mb is None else \
                (None if mw is None else mw.view(-1, in_channels, out_channels), mb)
            out_feature = ConvFunction.apply(input.feature, weight, rules, rule_size, tile_grid_shape,
                                             oz_idx.shape[0], bias, self.activation == 'relu', master)
        else:
            weight = self._cached_packed(weight)
            with profiling.section("conv:" + tag, iC=in_channels, oC=out_channels, n_in=input.feature.shape[0],
                                   n_out=oz_idx.shape[0], esize=input.feature.element_size()):
                profiling.count_pairs("conv:" + tag, rules)
                out_feature = ops.rule_conv(input.feature, weight, rules, rule_size, oz_idx.shape[0],
                                            bias=None if bias is None else bias.detach().float(),
                                            relu=self.activation == 'relu')
        out_tensor = SparseConvTensor(out_feature, out_shape, batch_size, z_ptr=oz_ptr, z_idx=oz_idx)
        out_tensor.rule_cache = input.rule_cache
        return out_tensor

    def _cached_packed(self, weight):
        """Inference: keep the tensor-core weight image across calls while the parameter is unchanged."""
        key = (self.weight._version, self.weight.data_ptr(), weight.dtype)
        cached = getattr(self, "_w_cache", None)
        if cached is not None and cached[0] == key:
            return cached[1]
        w = weight.detach().contiguous()
        ops._packed_weight(w)
        self._w_cache = (key, w)
        return w


SparseConv3d = Conv3d


class SubMConv3d(Conv3d):
    """Submanifold convolution: output sites = input sites, padding forced to k//2 (ref: sphconv/conv.py:200-210)."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, padding=0, dilation=1, groups=1,
                 bias=False, subm=False, indice_key=None, **kwargs):
        super().__init__(in_channels, out_channels, kernel_size, subm=True, stride=stride, padding=padding,
                         dilation=dilation, groups=groups, bias=bias, indice_key=indice_key, **kwargs)
        # the reference forces k // 2; for a dilated kernel the padding that keeps the geometry is d * (k // 2)
        self.padding = tuple([d * (k // 2) for k, d in zip(self.kernel_size, self.dilation)])
