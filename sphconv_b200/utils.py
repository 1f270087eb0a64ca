"""Small helpers with the reference's semantics (sphconv/utils/__init__.py)."""
import math
from collections.abc import Iterable
from itertools import repeat
from typing import List

import torch
from torch.nn.init import calculate_gain


def out_spatial(in_spatial: List[int], kernel_size: List[int], stride: List[int], padding: List[int],
                dilation: List[int] = [1, 1, 1]) -> List[int]:
    """floor((i + 2p - d(k-1) - 1)/s + 1) per axis (sphconv/utils/__init__.py:27-44)."""
    return [math.floor((i + 2 * p - d * (k - 1) - 1) / s + 1)
            for i, k, s, p, d in zip(in_spatial, kernel_size, stride, padding, dilation)]


def _triple(x):
    """A single number repeated three times, an iterable unchanged (sphconv/utils/__init__.py:47-51)."""
    if isinstance(x, Iterable):
        return x
    return tuple(repeat(x, 3))


def _calculate_fan_in_and_fan_out(tensor):
    """Fans of a [..., iC, oC] weight exactly as the reference computes them
    (sphconv/utils/__init__.py:57-77): fan_in uses size(-1), fan_out size(-2)."""
    if tensor.ndimension() < 2:
        raise ValueError("Fan in and fan out can not be computed for tensor with fewer than 2 dimensions")
    receptive = tensor[..., 0, 0].numel() if tensor.dim() > 2 else 1
    return tensor.size(-1) * receptive, tensor.size(-2) * receptive


def kaiming_uniform_(tensor, a=0, mode='fan_in', nonlinearity='leaky_relu'):
    """He-uniform initialisation with the fans above (sphconv/utils/__init__.py:91-124)."""
    mode = mode.lower()
    if mode not in ('fan_in', 'fan_out'):
        raise ValueError("Mode {} not supported, please use one of ['fan_in', 'fan_out']".format(mode))
    fan_in, fan_out = _calculate_fan_in_and_fan_out(tensor)
    fan = fan_in if mode == 'fan_in' else fan_out
    bound = math.sqrt(3.0) * calculate_gain(nonlinearity, a) / math.sqrt(fan)
    with torch.no_grad():
        return tensor.uniform_(-bound, bound)
