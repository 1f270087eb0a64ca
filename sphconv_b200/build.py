"""Builds the C-ABI CUDA library in-tree: sphconv_b200/_lib/libsphconv_b200.so (sm_100a only).

    python -m sphconv_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "_lib")
LIB = os.path.join(LIBDIR, "libsphconv_b200.so")
SOURCES = ["rules.cu", "conv_generic.cu", "conv_sparse.cu", "conv_tc.cu", "conv_tc_rows.cu", "conv_wgrad_tc.cu", "tensor_ops.cu", "voxelize.cu", "capi.cu"]
# the explicit -gencode pair is required: the sm_100a shorthand does not enable tcgen05 in ptxas
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _nvcc():
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "sphconv_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


HOOKS_LIB = os.path.join(LIBDIR, "libsphconv_b200_hooks.so")


def build_test_hooks(force=False):
    """A second library for the test of the bounded waits only: the same sources, with conv_tc.cu compiled with
    -DSPH_TEST_HOOKS (a 10 ms wait limit and the entry point sph_test_withhold_arrival).  The shipped library holds
    none of it.  Returns the path."""
    build(force=force)
    src = os.path.join(CSRC, "conv_tc.cu")
    if not force and os.path.exists(HOOKS_LIB) and os.path.getmtime(HOOKS_LIB) >= os.path.getmtime(LIB):
        return HOOKS_LIB
    flags = [f for f in NVCC_FLAGS if not f.startswith("--use_fast_math")]
    obj = os.path.join(LIBDIR, "conv_tc_hooks.o")
    subprocess.check_call([_nvcc(), *flags, "-DSPH_TEST_HOOKS", "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c", src,
                           "-o", obj], stdout=subprocess.DEVNULL, stderr=subprocess.STDOUT)
    objs = [os.path.join(LIBDIR, s_.replace(".cu", ".o")) for s_ in SOURCES if s_ != "conv_tc.cu"] + [obj]
    subprocess.check_call([_nvcc(), "-shared", "-o", HOOKS_LIB, *objs, "-lcudart"])
    return HOOKS_LIB


def build(force=False, verbose=False):
    """Compile every .cu into one shared library; returns its path."""
    if not force and not _stale():
        return LIB
    os.makedirs(LIBDIR, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if not f.startswith("--use_fast_math")]
    if verbose:
        flags += ["-Xptxas", "-v"]
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(LIBDIR, src.replace(".cu", ".o"))
        cmd = [_nvcc(), *flags, "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write("[%s]\n%s\n" % (src, out))
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([_nvcc(), "-shared", "-o", LIB, *objs, "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_test_hooks(force="--force" in sys.argv))
