"""Builds the reference's own CUDA implementation of the path as a checker: oracle/_ref/sphconv_ref*.so.

Sources are compiled where they lie in the reference tree (the directory named by the environment variable
REFERENCE_ROOT, else a directory "reference" beside this repository):
src/sphconv/rules.cu and src/sphconv/tensor.cu unmodified, plus - when a CUTLASS header tree is found -
src/sphconv/rule_conv.cu.  The reference pins no CUTLASS version (its submodule directory is empty); the
only copy on this machine is a 4.x tree whose MmaPipelined calls `iterator.clear_mask(bool)`, so the build
puts a temporary copy of include/sphconv/iterator.cu.h with that one method taking the flag on the include path
(the temporary copy is deleted afterwards; nothing of the reference is stored in this repository).

A second, CPU-only module is built from the reference's host voxeliser (src/utils/all.cpp + include/point2voxel.h,
pybind11, g++): oracle/_ref/sphconv_utils*.so.  It runs without a GPU and pins oracle/voxelize_np.py.

    python -m oracle.build_ref            # builds if the reference tree is present, else does nothing
"""
import glob
import os
import re
import shutil
import subprocess
import sys
import sysconfig
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# The reference tree: the directory the environment names, else a checkout called "reference" beside this repository.
REFERENCE_ROOT = os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _cutlass_include():
    import site
    for base in site.getsitepackages():
        for rel in ("flashinfer/data/cutlass/include", "tilelang/3rdparty/cutlass/include"):
            p = os.path.join(base, rel)
            if os.path.exists(os.path.join(p, "cutlass", "cutlass.h")):
                return p
    return None


def lib_path():
    hits = glob.glob(os.path.join(OUT, "sphconv_ref*.so"))
    return hits[0] if hits else None


def build(with_conv=True, verbose=False):
    from torch.utils import cpp_extension
    os.makedirs(OUT, exist_ok=True)
    ref = REFERENCE_ROOT
    inc = ["-I" + os.path.join(ref, "include")]
    for p in cpp_extension.include_paths("cuda") if hasattr(cpp_extension, "include_paths") else []:
        inc.append("-I" + p)
    inc.append("-I" + sysconfig.get_paths()["include"])
    common = ["-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-DTORCH_EXTENSION_NAME=sphconv_ref",
              "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1", "--expt-relaxed-constexpr",
              "-Wno-deprecated-gpu-targets", "-w"]
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    tmp = tempfile.mkdtemp(prefix="sphref_")
    objs, procs = [], []
    try:
        sources = [(os.path.join(ref, "src/sphconv/rules.cu"), []), (os.path.join(ref, "src/sphconv/tensor.cu"), [])]
        cutlass = _cutlass_include() if with_conv else None
        if cutlass:
            shim = os.path.join(tmp, "shim", "sphconv")
            os.makedirs(shim)
            text = open(os.path.join(ref, "include/sphconv/iterator.cu.h")).read()
            # CUTLASS 2.x called `if (k_iterations <= 1) it.clear_mask();`, 4.x calls `it.clear_mask(k_iterations <= 1)`:
            # same behaviour needs the flag to guard the body
            text, n_sub = re.subn(r"void\s+clear_mask\s*\(\s*\)\s*\{",
                                  "void clear_mask(bool enable = true)\n    {\n        if (!enable) return;", text)
            assert n_sub == 6, "unexpected number of clear_mask definitions: %d" % n_sub
            open(os.path.join(shim, "iterator.cu.h"), "w").write(text)
            sources.append((os.path.join(ref, "src/sphconv/rule_conv.cu"),
                            ["-I" + os.path.join(tmp, "shim"), "-I" + cutlass]))
        sources.append((os.path.join(HERE, "ref_binding.cpp"), ["-DSPH_REF_WITH_CONV"] if cutlass else []))
        for src, extra in sources:
            obj = os.path.join(tmp, os.path.basename(src) + ".o")
            cmd = [nvcc, *ARCH, *common, *extra, *inc, "-x", "cu", "-c", src, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
            objs.append(obj)
        failed = []
        for src, pr in procs:
            out, _ = pr.communicate()
            if pr.returncode != 0:
                failed.append(src)
                sys.stderr.write("[build_ref] %s failed:\n%s\n" % (src, out[-3000:]))
            elif verbose:
                sys.stderr.write(out)
        if failed:
            if cutlass and any("rule_conv" in f for f in failed) and len(failed) == 1:
                sys.stderr.write("[build_ref] retrying without the reference's rule_conv.cu\n")
                return build(with_conv=False, verbose=verbose)
            raise RuntimeError("reference build failed: %s" % failed)
        import torch
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        target = os.path.join(OUT, "sphconv_ref" + sysconfig.get_config_var("EXT_SUFFIX"))
        subprocess.check_call([nvcc, "-shared", "-o", target, *objs, "-L" + torch_lib, "-ltorch", "-ltorch_cpu",
                               "-ltorch_cuda", "-lc10", "-lc10_cuda", "-ltorch_python", "-lcudart",
                               "-Xlinker", "-rpath," + torch_lib])
        return target
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def build_if_possible():
    """Build when the reference tree is mounted and the library is missing; never raises for an absent tree."""
    if lib_path() is not None:
        return lib_path()
    if not os.path.exists(os.path.join(REFERENCE_ROOT, "src/sphconv/rules.cu")):
        return None
    try:
        return build()
    except Exception as e:  # the checker is optional: the oracle itself never depends on it
        sys.stderr.write("[build_ref] not built: %s\n" % e)
        return None


def utils_lib_path():
    hits = glob.glob(os.path.join(OUT, "sphconv_utils*.so"))
    return hits[0] if hits else None


def build_utils():
    """The reference's host voxeliser (pybind11 module `sphconv_utils`), compiled from its own two files."""
    import pybind11
    os.makedirs(OUT, exist_ok=True)
    target = os.path.join(OUT, "sphconv_utils" + sysconfig.get_config_var("EXT_SUFFIX"))
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-shared", "-fPIC", "-w",
           "-I" + os.path.join(REFERENCE_ROOT, "include"), "-I" + pybind11.get_include(),
           "-I" + sysconfig.get_paths()["include"], os.path.join(REFERENCE_ROOT, "src/utils/all.cpp"), "-o", target]
    subprocess.check_call(cmd)
    return target


def build_utils_if_possible():
    if utils_lib_path() is not None:
        return utils_lib_path()
    if not os.path.exists(os.path.join(REFERENCE_ROOT, "src/utils/all.cpp")):
        return None
    try:
        return build_utils()
    except Exception as e:
        sys.stderr.write("[build_ref] host voxeliser not built: %s\n" % e)
        return None


def load_utils():
    """Import the reference's host voxeliser module (CPU only) or return None."""
    path = utils_lib_path()
    if path is None:
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("sphconv_utils", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load():
    """Import the built module (needs CUDA at call time, not at import time) or return None."""
    path = lib_path()
    if path is None:
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)
    spec = importlib.util.spec_from_file_location("sphconv_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build_if_possible())
    print(build_utils_if_possible())
