"""ctypes binding of the C ABI declared in include/sphconv_b200.h.

The shared library is built in-tree by ``python -m sphconv_b200.build`` (or ``__graft_entry__.build()``)
into ``sphconv_b200/_lib/libsphconv_b200.so``.  There is no fallback: if the library is missing, every op
raises.  torch is used only for device memory and the current stream.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lib", "libsphconv_b200.so")

SPH_F32, SPH_F16, SPH_BF16, SPH_I8 = 0, 1, 2, 3
STATUS_RULE_OVERFLOW, STATUS_BAD_INDEX, STATUS_TIMEOUT = 1, 2, 4

DTYPE_CODE = {torch.float32: SPH_F32, torch.float16: SPH_F16, torch.bfloat16: SPH_BF16, torch.int8: SPH_I8}

c_i32p = ctypes.POINTER(ctypes.c_int32)
vp = ctypes.c_void_p
i64 = ctypes.c_int64
i32 = ctypes.c_int32
cint = ctypes.c_int


class Geom(ctypes.Structure):
    """struct sph_geom"""
    _fields_ = [("B", i32), ("in_shape", i32 * 3), ("out_shape", i32 * 3), ("ksize", i32 * 3),
                ("stride", i32 * 3), ("padding", i32 * 3), ("tile", i32 * 2), ("dilation", i32 * 3)]


class VoxelGrid(ctypes.Structure):
    """struct sph_voxel_grid"""
    _fields_ = [("B", i32), ("cells", i32 * 3), ("range", ctypes.c_float * 6), ("max_points", i32),
                ("max_voxels", i32), ("append_mode", i32)]


# name -> (restype, argtypes); exactly the symbols include/sphconv_b200.h declares
SIGNATURES = {
    "sph_last_error": (ctypes.c_char_p, []),
    "sph_version": (cint, []),
    "sph_kernel_launches": (i64, []),
    "sph_out_spatial": (cint, [c_i32p, c_i32p, c_i32p, c_i32p, c_i32p, c_i32p]),
    "sph_tile_n_max": (cint, [ctypes.POINTER(Geom), i64]),
    "sph_num_tiles": (cint, [ctypes.POINTER(Geom)]),
    "sph_rules_subm_scratch_bytes": (i64, [ctypes.POINTER(Geom), i64]),
    "sph_rules_subm": (cint, [vp, vp, i64, ctypes.POINTER(Geom), vp, i32, vp, vp, vp, cint, vp, vp]),
    "sph_rules_subm_static": (cint, [vp, vp, i64, ctypes.POINTER(Geom), i32, vp, vp, vp, cint, vp, vp]),
    "sph_rules_strided_scratch_bytes": (i64, [ctypes.POINTER(Geom), i64]),
    "sph_rules_strided_count": (cint, [vp, vp, i64, ctypes.POINTER(Geom), vp, vp, vp, c_i32p, vp]),
    "sph_rules_strided_count_async": (cint, [vp, vp, i64, ctypes.POINTER(Geom), vp, vp, vp,
                                             ctypes.POINTER(ctypes.c_void_p), vp]),
    "sph_rules_strided_fill": (cint, [vp, vp, i64, ctypes.POINTER(Geom), vp, vp, i64, i32, vp, vp, vp, vp, vp, cint,
                                      vp, vp]),
    "sph_rule_lists": (cint, [vp, ctypes.POINTER(Geom), i64, vp, i32, vp, vp, cint, vp, vp]),
    "sph_rules_to_nbr": (cint, [vp, vp, i32, i32, i32, i64, i64, vp, vp, vp, vp]),
    "sph_packed_weight_bytes": (i64, [cint, i32, i32, i32]),
    "sph_pack_weight": (cint, [vp, cint, i32, i32, i32, vp, vp]),
    "sph_conv_uses_tensor_cores": (cint, [cint, i32, i32]),
    "sph_conv_uses_pair_kernel": (cint, [cint, i32, i32]),
    "sph_conv_wgrad_kernel": (cint, [cint, i32, i32]),
    "sph_conv_gather": (cint, [vp, cint, i64, vp, vp, vp, i64, i32, i32, i32, cint, vp, vp, cint, vp, cint, vp, vp]),
    "sph_conv_wgrad": (cint, [vp, vp, cint, i64, vp, i64, i32, i32, i32, vp, cint, vp, vp]),
    "sph_init_tensor_scratch_bytes": (i64, [i32, c_i32p]),
    "sph_init_tensor": (cint, [vp, i32, i64, vp, i32, c_i32p, vp, vp, vp, vp, vp, vp, vp]),
    "sph_permute_rows": (cint, [vp, i32, i64, vp, cint, vp, vp]),
    "sph_to_dense": (cint, [vp, i32, i64, vp, vp, i32, c_i32p, vp, cint, vp, vp]),
    "sph_epilogue_backward": (cint, [vp, vp, cint, i64, i32, cint, vp, vp, vp]),
    "sph_voxel_transform": (cint, [vp, i32, i64, cint, vp, vp]),
    "sph_voxel_feature_count": (cint, [i32, cint]),
    "sph_voxelize_scratch_bytes": (i64, [ctypes.POINTER(VoxelGrid), i64]),
    "sph_voxelize_count": (cint, [vp, vp, i64, ctypes.POINTER(VoxelGrid), vp, vp, c_i32p, vp]),
    "sph_voxelize_fill": (cint, [vp, i32, vp, vp, i64, ctypes.POINTER(VoxelGrid), vp, i64, vp, vp, vp, vp, vp]),
}

_lib = None


def lib():
    """The loaded library; raises RuntimeError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "sphconv_b200: CUDA library %s is missing - build it with `python -m sphconv_b200.build`; "
                "there is no CPU or PyTorch fallback" % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc):
    if rc < 0:
        raise RuntimeError("sphconv_b200: %s (code %d)" % (lib().sph_last_error().decode(), rc))
    return rc


def make_geom(B, in_shape, out_shape, ksize, stride, padding, tile, dilation=(1, 1, 1)):
    g = Geom()
    g.B = int(B)
    for i in range(3):
        g.in_shape[i] = int(in_shape[i])
        g.out_shape[i] = int(out_shape[i])
        g.ksize[i] = int(ksize[i])
        g.stride[i] = int(stride[i])
        g.padding[i] = int(padding[i])
        g.dilation[i] = int(dilation[i])
    g.tile[0], g.tile[1] = int(tile[0]), int(tile[1])
    return g


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("sphconv_b200 ops run on CUDA tensors only (got a %s tensor); there is no CPU path"
                               % t.device.type)
        if t is not None and not t.is_contiguous():
            raise RuntimeError("sphconv_b200 ops need contiguous tensors")


_status = {}


def status_tensor(device):
    """Per-device int32 status word the kernels OR error bits into."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = t
    return t


def check_status(device=None, reset=True, ignore_overflow=True):
    """Synchronising read of the device status word; raises on BAD_INDEX / TIMEOUT.
    Rule-list overflow is the reference's silent-drop case (src/sphconv/rules.cu:217-224) and only
    raises when ignore_overflow is False."""
    dev = torch.cuda.current_device() if device is None else device
    t = status_tensor(dev)
    v = int(t.item())
    if reset and v:
        t.zero_()
    if v & STATUS_TIMEOUT:
        raise RuntimeError("sphconv_b200: a bounded device-side wait ran out (status %d)" % v)
    if v & STATUS_BAD_INDEX:
        raise RuntimeError("sphconv_b200: an index outside its valid range was met (status %d)" % v)
    if (v & STATUS_RULE_OVERFLOW) and not ignore_overflow:
        raise RuntimeError("sphconv_b200: a rule list exceeded tile_n_max (status %d)" % v)
    return v
