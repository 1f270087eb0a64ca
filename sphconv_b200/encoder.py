"""The SECOND-style 8-layer sparse middle encoder used by the benchmark configurations:
SubM 4->16, SubM 16->16, Conv s2 16->32, SubM 32->32 x2, Conv s2 32->64, SubM 64->64 x2; all 3x3x3,
BatchNorm folded into a per-channel bias, ReLU.  The two layers of each SubM pair share an indice_key, so
five rule sets serve eight layers (the reference caches rules per indice_key, sphconv/conv.py:159-171)."""
import numpy as np
import torch

from . import synthetic
from .conv import Conv3d, SubMConv3d
from .modules import Sequential


def encoder8_parameters(seed=1234):
    """[(weight [3,3,3,iC,oC] float32, bias [oC] float32)] for the eight layers, seeded."""
    params = []
    for li, (subm, iC, oC, stride, key) in enumerate(synthetic.ENCODER8):
        w = synthetic.make_weight([3, 3, 3], iC, oC, seed + li)
        b = np.random.default_rng(seed + 100 + li).normal(0.0, 0.1, size=oC).astype(np.float32)
        params.append((w, b))
    return params


def build_encoder8(dtype=torch.float16, device="cuda", seed=1234, fused=True):
    """Sequential of the eight layers.  fused=True: bias + ReLU run in the convolution's epilogue (inference);
    fused=False: plain reference-style layers followed by nothing (bias/ReLU left to the caller)."""
    layers = []
    for li, ((subm, iC, oC, stride, key), (w, b)) in enumerate(zip(synthetic.ENCODER8, encoder8_parameters(seed))):
        kw = dict(bias=True, apply_bias=fused, activation='relu' if fused else None, name="L%d" % li)
        if subm:
            m = SubMConv3d(iC, oC, 3, indice_key=key, **kw)
        else:
            m = Conv3d(iC, oC, 3, stride=stride, padding=1, **kw)
        with torch.no_grad():
            m.weight.copy_(torch.as_tensor(w))
            m.bias.copy_(torch.as_tensor(b))
        layers.append(m)
    net = Sequential(*layers).to(device)
    if dtype in (torch.float16, torch.bfloat16):
        net = net.to(dtype)
    return net
