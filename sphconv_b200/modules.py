"""Module containers (ref: sphconv/modules.py)."""
from collections import OrderedDict

import torch
from torch import nn


class SphModule(nn.Module):
    """Marker base: subclasses receive a SparseConvTensor inside Sequential (ref: sphconv/modules.py:35-40)."""

    def __init__(self, **kwargs):
        super().__init__(**kwargs)


def is_sph_module(module):
    return isinstance(module, SphModule)


def is_sparse_conv(module):
    from .conv import Convolution
    return isinstance(module, Convolution)


class Sequential(SphModule):
    """Sequential container that hands the sparse tensor to sparse modules and only `.feature` to dense
    ones such as BatchNorm1d / ReLU (ref: sphconv/modules.py:43-128)."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        # accepted forms, as torch.nn.Sequential plus named keyword modules: Sequential(m0, m1, ...),
        # Sequential(OrderedDict(name=module, ...)), Sequential(m0, name=module, ...)
        named = list(args[0].items()) if len(args) == 1 and isinstance(args[0], OrderedDict) \
            else [(str(i), m) for i, m in enumerate(args)]
        for name, module in named + list(kwargs.items()):
            if name in self._modules:
                raise ValueError("module name '{}' given twice".format(name))
            self.add_module(name, module)

    def __len__(self):
        return len(self._modules)

    def __getitem__(self, idx):
        n = len(self)
        if not -n <= idx < n:
            raise IndexError("index {} is out of range".format(idx))
        return list(self._modules.values())[idx % n]

    def add(self, module, name=None):
        """Appends a module under `name` (default: its position)."""
        name = str(len(self._modules)) if name is None else name
        if name in self._modules:
            raise KeyError("module name '{}' exists".format(name))
        self.add_module(name, module)

    def forward(self, input):
        from .conv import Conv3d, SubMConv3d
        from .tensor import SparseConvTensor
        nvtx = torch.cuda.nvtx if torch.cuda.is_available() else None
        items = list(self._modules.items())
        for pos, (k, module) in enumerate(items):
            if is_sph_module(module):
                assert isinstance(input, SparseConvTensor)
                if isinstance(module, Conv3d) and module.subm:
                    # a submanifold layer keeps the geometry: the strided layer behind it can start finding its
                    # output pattern now, and this layer's convolution covers the host's wait for the row count
                    nxt = next((m for _, m in items[pos + 1:] if is_sph_module(m)), None)
                    if isinstance(nxt, Conv3d) and not nxt.subm:
                        nxt.begin_rules(input)
                if nvtx is not None:
                    tag = "SubMConv3d" if isinstance(module, SubMConv3d) else \
                        "Conv3d" if isinstance(module, Conv3d) else "layer"
                    nvtx.range_push("{}:{}".format(tag, k))
                input = module(input)
                if nvtx is not None:
                    nvtx.range_pop()
            elif isinstance(input, SparseConvTensor):
                input.feature = module(input.feature)
            else:
                input = module(input)
        return input


SparseSequential = Sequential
