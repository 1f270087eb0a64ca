"""Autograd glue, same classes and call signatures as the reference's sphconv/functional.py."""
from typing import List

import torch

from . import profiling
from .sphconv_cuda import (epilogue_backward, init_tensor, init_tensor_backward, rule_conv, rule_conv_d_feature,
                           rule_conv_d_weight, to_dense, to_dense_backward)


class ConvFunction(torch.autograd.Function):
    """Rule-driven sparse 3-D convolution (ref: sphconv/functional.py:12-78).

    forward(feature [NNZ,iC], weight [KV,iC,oC], rules, rule_size, tile_grid_shape, outNNZ) -> [outNNZ,oC]
    backward returns (d_feature, d_weight, None, None, None, None).

    Two optional trailing arguments (extensions): ``bias`` [oC] and ``relu``.  With them the kernel's epilogue
    computes relu(acc + bias) in fp32 before the single rounding to the output dtype, and backward masks the incoming
    gradient with (output > 0) and returns the bias gradient, so a training step needs no separate bias-add and
    activation passes over the output.  ``master`` (extension): (d_weight fp32 [KV,iC,oC] or None, d_bias fp32 [oC]
    or None) slices of a caller-owned fp32 gradient buffer (sharding.GradBuffer); backward then ACCUMULATES the fp32
    gradients there and returns None for them, so nothing is rounded to the feature dtype on the way."""

    @staticmethod
    def forward(ctx, feature: torch.Tensor, weight: torch.Tensor, rules, rule_size, tile_grid_shape: List[int],
                outNNZ: int, bias=None, relu: bool = False, master=None):
        ctx.tile_grid_shape = tile_grid_shape
        ctx.master = master if master is not None else (None, None)
        ctx.tag = profiling.current_tag
        ctx.relu = bool(relu)
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        with profiling.section("conv:" + ctx.tag, iC=weight.shape[1], oC=weight.shape[2], n_in=feature.shape[0],
                               n_out=int(outNNZ), esize=feature.element_size()):
            profiling.count_pairs("conv:" + ctx.tag, rules)
            out = rule_conv(feature, weight, rules, rule_size, outNNZ,
                            bias=None if bias is None else bias.detach().float(), relu=ctx.relu)
        extra = (out,) if ctx.relu else ()
        if isinstance(rules, torch.Tensor):
            ctx.save_for_backward(feature, weight, rules, rule_size, *extra)
            ctx.rule_obj = None
        else:  # rule set generated without the padded tensor: keep the table object itself
            ctx.save_for_backward(feature, weight, *extra)
            ctx.rule_obj = rules
        return out

    @staticmethod
    def backward(ctx, d_featureOut: torch.Tensor):
        saved = ctx.saved_tensors
        out = saved[-1] if ctx.relu else None
        if ctx.rule_obj is None:
            feature, weight, rules, rule_size = saved[:4]
        else:
            feature, weight = saved[:2]
            rules, rule_size = ctx.rule_obj, None
        # the ops take the [KV,oC,iC] transpose, as in the reference (sphconv/functional.py:70-74); this is
        # rule_conv_backward (src/sphconv/rule_conv.cu:577-597) spelled out so the two halves can be timed
        d_out = d_featureOut.contiguous()
        d_bias = None
        if ctx.relu or ctx.has_bias:    # gradient mask and bias gradient in one pass over the rows
            d_out, d_bias = epilogue_backward(d_out, out, ctx.relu, ctx.has_bias)
            if d_bias is not None:
                if ctx.master[1] is not None:
                    ctx.master[1].add_(d_bias)
                    d_bias = None
                else:
                    d_bias = d_bias.to(ctx.bias_dtype)
        meta = dict(iC=weight.shape[1], oC=weight.shape[2], n_in=feature.shape[0], n_out=d_out.shape[0],
                    esize=feature.element_size())
        with profiling.section("dgrad:" + ctx.tag, **meta):
            d_feature = rule_conv_d_feature(d_out, weight.permute(0, 2, 1).contiguous(), rules, rule_size,
                                            ctx.tile_grid_shape, feature.shape[0])
        with profiling.section("wgrad:" + ctx.tag, **meta):
            if ctx.master[0] is not None:
                rule_conv_d_weight(feature, d_out, rules, rule_size, out=ctx.master[0], accumulate=True)
                d_weight = None
            else:
                d_weight = rule_conv_d_weight(feature, d_out, rules, rule_size).to(feature.dtype)
        return d_feature, d_weight, None, None, None, None, d_bias, None, None


class ToDenseFunction(torch.autograd.Function):
    """[NNZ,C] rows -> dense [B,C,s0,s1,s2] (ref: sphconv/functional.py:81-106)."""

    @staticmethod
    def forward(ctx, feature: torch.Tensor, z_idx: torch.Tensor, z_ptr: torch.Tensor, shape: List[int]):
        ctx.save_for_backward(z_idx, z_ptr)
        B, C, D, H, W = shape  # the reference's names; the dense layout is [B, s0, s1, s2, C]
        res = torch.zeros((B, D, W, H, C), device=feature.device, dtype=feature.dtype)
        to_dense(feature, z_idx, z_ptr, D, res)
        return res.permute((0, 4, 1, 2, 3)).contiguous()

    @staticmethod
    def backward(ctx, d_featureOut):
        z_idx, z_ptr = ctx.saved_tensors
        d_feature = to_dense_backward(d_featureOut.permute((0, 2, 3, 4, 1)).contiguous(), z_idx, z_ptr)
        return d_feature, None, None, None


class InitTensorFunction(torch.autograd.Function):
    """COO -> range-voxel (ref: sphconv/functional.py:109-131)."""

    @staticmethod
    def forward(ctx, raw_feature: torch.Tensor, indices_bzyx: torch.Tensor, batchsize: int,
                spatial_shape_HWD: List[int]):
        feature_out, zidx, zptr, permutation = init_tensor(raw_feature, indices_bzyx, batchsize, spatial_shape_HWD)
        ctx.save_for_backward(permutation)
        ctx.mark_non_differentiable(zidx, zptr)
        return feature_out, zidx, zptr

    @staticmethod
    def backward(ctx, d_featureOut, d_zidx, d_zptr):
        permutation, = ctx.saved_tensors
        return init_tensor_backward(d_featureOut, permutation), None, None, None
