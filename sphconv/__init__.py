"""``import sphconv`` for code written against the reference package: every name it exports
(sphconv/__init__.py:1-4 of the reference) and its submodules ``sphconv.tensor``, ``sphconv.functional``,
``sphconv.conv``, ``sphconv.modules``, ``sphconv.utils``, ``sphconv.sphconv_cuda`` and ``sphconv.rangevoxel`` resolve
to the B200 implementation in ``sphconv_b200``.  Nothing is implemented here."""
import importlib
import sys

import sphconv_b200 as _impl
from sphconv_b200 import *  # noqa: F401,F403
from sphconv_b200 import __all__  # noqa: F401

for _name in ("tensor", "functional", "conv", "modules", "utils", "sphconv_cuda", "rangevoxel", "voxelize", "quant",
              "sharding", "pipeline"):
    _mod = importlib.import_module("sphconv_b200." + _name)
    sys.modules[__name__ + "." + _name] = _mod
    globals()[_name] = _mod
