"""int8 inference variant of a stack of sparse convolutions (per-channel symmetric scales, int32 accumulation).

Quantisation scheme.  Activations entering layer l are int8 with one scale per input channel,
x ~ q_x * s_x[ic].  A per-input-channel scale cannot be pulled out of the sum over ic, so it is folded into
the weights first, W'[k,ic,oc] = W[k,ic,oc] * s_x[ic]; W' is then quantised with one scale per output
channel, W' ~ q_w * s_w[oc].  The kernel accumulates q_x * q_w exactly in int32 and its epilogue computes
relu(acc * scale[oc] + bias[oc]) with scale = s_w / s_y and bias = b / s_y, where s_y is the next layer's input
scale (int8 output), or s_y = 1 for the last layer (float output).  Activation scales come from the per-channel
absolute maxima of a float calibration pass."""
from typing import List

import torch

from . import profiling
from . import sphconv_cuda as ops
from .conv import Conv3d, get_tile_grid_shape
from .modules import Sequential
from .tensor import SparseConvTensor
from .utils import out_spatial

QMAX = 127.0


def _absmax_per_channel(x: torch.Tensor) -> torch.Tensor:
    if x.shape[0] == 0:
        return torch.ones(x.shape[1], device=x.device)
    return x.float().abs().amax(dim=0).clamp_min(1e-8)


class QuantConv:
    """One quantised layer: geometry and rule cache behaviour of the float module, int8 weight, fused epilogue."""

    def __init__(self, conv: Conv3d, weight_q: torch.Tensor, scale: torch.Tensor, bias: torch.Tensor, relu: bool,
                 out_dtype: torch.dtype):
        self.conv, self.weight_q, self.scale, self.bias, self.relu, self.out_dtype = conv, weight_q, scale, bias, relu, out_dtype
        ops._packed_weight(weight_q)

    def __call__(self, x: SparseConvTensor) -> SparseConvTensor:
        c = self.conv
        in_shape = [x.D, x.W, x.H]
        out_shape = in_shape if c.subm else out_spatial(in_shape, c.kernel_size, c.stride, c.padding, c.dilation)
        tag = c.name or "{}{}_{}".format("subm" if c.subm else "conv", c.in_channels, c.out_channels)
        datas = x.find_rule(c.indice_key) if c.indice_key is not None else None
        if datas is None:
            profiling.current_rule_tag = tag
            with profiling.section("rules:" + tag, **c._rule_meta(x, in_shape, out_shape)):
                datas = c._rules(x, in_shape, out_shape)
            if c.indice_key is not None:
                x.rule_cache[c.indice_key] = datas
        oz_idx, oz_ptr, rules, rule_size, _ = datas
        with profiling.section("conv:" + tag, iC=c.in_channels, oC=c.out_channels, n_in=x.feature.shape[0],
                               n_out=oz_idx.shape[0], esize=1, k_ch=self.weight_q.shape[1], n_ch=self.weight_q.shape[2]):
            profiling.count_pairs("conv:" + tag, rules)
            y = ops.rule_conv(x.feature, self.weight_q, rules, rule_size, oz_idx.shape[0], scale=self.scale,
                              bias=self.bias, relu=self.relu, out_dtype=self.out_dtype)
        out = SparseConvTensor(y, out_shape, x.B, z_ptr=oz_ptr, z_idx=oz_idx)
        out.rule_cache = x.rule_cache
        return out


class QuantEncoder:
    """Chain of QuantConv layers; `quantize_input` turns float features into the first layer's int8 input."""

    def __init__(self, layers: List[QuantConv], in_scale: torch.Tensor, in_channels_padded: int):
        self.layers, self.in_scale, self.in_channels_padded = layers, in_scale, in_channels_padded

    def quantize_input(self, feature: torch.Tensor) -> torch.Tensor:
        """float [n, C] -> int8 [n, C padded to the first layer's input width] (zeros in the padding)."""
        q = torch.round(feature.float() / self.in_scale).clamp_(-QMAX, QMAX).to(torch.int8)
        out = torch.zeros((q.shape[0], self.in_channels_padded), dtype=torch.int8, device=q.device)
        out[:, :q.shape[1]] = q
        return out

    def __call__(self, x: SparseConvTensor) -> SparseConvTensor:
        for layer in self.layers:
            x = layer(x)
        return x


@torch.no_grad()
def quantize_encoder(net: Sequential, calib: SparseConvTensor) -> QuantEncoder:
    """Builds the int8 encoder from a float Sequential of Conv3d layers (bias + ReLU as configured on the
    modules) and one float calibration batch."""
    convs = [m for m in net._modules.values() if isinstance(m, Conv3d)]
    assert len(convs) == len(net._modules), "quantize_encoder expects a stack of sparse convolutions only"
    # calibration pass: per-channel |max| of every layer's input
    acts = []
    x = calib
    for m in convs:
        acts.append(_absmax_per_channel(x.feature))
        x = m(x)
    # Channel counts at the layer boundaries.  The tensor-core kernel wants int8 rows of at least 32 bytes (one kind::i8
    # instruction consumes 32 channels), so counts are padded to a multiple of 32 with zero weights: a padded output channel
    # computes relu(0) = 0 and the next layer's padded input channels carry zero weights.  A layer with narrower rows keeps
    # them (padded to 4, 8 or 16 only) where the pair-compacting CUDA-core kernel takes the pair of widths: the first,
    # sparse levels then move a quarter of the bytes.
    from . import _capi as C
    lib = C.lib()
    pad32 = lambda c: max(32, (c + 31) // 32 * 32)
    narrow = lambda c: 4 if c <= 4 else 8 if c <= 8 else 16 if c <= 16 else pad32(c)
    chans = [convs[0].in_channels] + [m.out_channels for m in convs]
    width = [narrow(c) for c in chans]
    width[-1] = chans[-1]                                             # the last layer's output is not padded
    for li in range(len(convs) - 1, -1, -1):
        if width[li] < 32 and not lib.sph_conv_uses_pair_kernel(C.SPH_I8, width[li], width[li + 1]):
            width[li] = pad32(chans[li])
    layers = []
    for li, m in enumerate(convs):
        last = li == len(convs) - 1
        iC, oC = m.in_channels, m.out_channels
        iP, oP = width[li], width[li + 1]
        s_x = acts[li] / QMAX                                         # [iC]
        w = m.weight.detach().float().reshape(-1, iC, oC) * s_x.view(1, -1, 1)
        s_w = w.abs().amax(dim=(0, 1)).clamp_min(1e-12) / QMAX       # [oC]
        w_q = torch.zeros((w.shape[0], iP, oP), dtype=torch.int8, device=w.device)
        w_q[:, :iC, :oC] = torch.round(w / s_w.view(1, 1, -1)).clamp_(-QMAX, QMAX).to(torch.int8)
        bias = m.bias.detach().float() if (m.apply_bias and m.bias is not None) else torch.zeros_like(s_w)
        s_y = torch.ones_like(s_w) if last else acts[li + 1] / QMAX
        scale = torch.ones(oP, device=w.device)
        bias_p = torch.zeros(oP, device=w.device)
        scale[:oC] = s_w / s_y
        bias_p[:oC] = bias / s_y
        layers.append(QuantConv(m, w_q.contiguous(), scale.contiguous(), bias_p.contiguous(), m.activation == 'relu',
                                torch.float32 if last else torch.int8))
    return QuantEncoder(layers, acts[0] / QMAX, width[0])
