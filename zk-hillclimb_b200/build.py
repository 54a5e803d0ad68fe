"""Compile the CUDA library in-tree for sm_100a.

    python zk-hillclimb_b200/build.py [--force] [--verbose]

Produces zk-hillclimb_b200/libzkh.so from csrc/*.cu with nvcc.  The library has
no Python or torch dependency; it is what the C ABI in include/zkh.h names.
Also builds zk-hillclimb_b200/zkh_p3_selftest, zkh_p3_gadgets_selftest, the layer prover zkh_p3_layer and the driver executable zkob_p3fc
from host/*.cpp with g++: the C++ host side (include/zkh_p3.hpp, zkh_p3_verify.hpp) linked against the library.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libzkh.so")
SELFTEST = os.path.join(HERE, "zkh_p3_selftest")
GADGETS_SELFTEST = os.path.join(HERE, "zkh_p3_gadgets_selftest")
DRIVER = os.path.join(HERE, "zkob_p3fc")
LAYER = os.path.join(HERE, "zkh_p3_layer")
FC_DRIVER = os.path.join(HERE, "zkob_fc")
RESCALE_DRIVER = os.path.join(HERE, "zkob_rescale")
BATCH_DRIVER = os.path.join(HERE, "zkob_batchopen")
SKIP_DRIVER = os.path.join(HERE, "zkob_skip")
GLU_DRIVER = os.path.join(HERE, "zkob_glu")
HEADSLICE_DRIVER = os.path.join(HERE, "zkob_headslice")
HEADMERGE_DRIVER = os.path.join(HERE, "zkob_headmerge")
ROPE_DRIVER = os.path.join(HERE, "zkob_rope")
SOFTMAX_DRIVER = os.path.join(HERE, "zkob_softmax")
RMSNORM_DRIVER = os.path.join(HERE, "zkob_rmsnorm")
SOFTMAX8_DRIVER = os.path.join(HERE, "zkob_softmax8")
ROWMAX_DRIVER = os.path.join(HERE, "zkob_rowmax")
HOSTMATH = os.path.join(HERE, "zkob_hostmath")
INCLUDE = os.path.abspath(os.path.join(HERE, "..", "include"))
NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        [os.path.join(HERE, "..", "include", "zkh.h"), os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build_selftest(force=False):
    """The C++ host programs over the C ABI; linked with an rpath beside the library."""
    for name, exe in (("p3_selftest.cpp", SELFTEST), ("p3_gadgets_selftest.cpp", GADGETS_SELFTEST), ("zkob_p3fc.cpp", DRIVER),
                      ("p3_layer_main.cpp", LAYER), ("zkob_fc.cpp", FC_DRIVER), ("zkob_rescale.cpp", RESCALE_DRIVER), ("zkob_batchopen.cpp", BATCH_DRIVER), ("zkob_skip.cpp", SKIP_DRIVER), ("zkob_glu.cpp", GLU_DRIVER), ("zkob_headslice.cpp", HEADSLICE_DRIVER),
                      ("zkob_headmerge.cpp", HEADMERGE_DRIVER), ("zkob_rope.cpp", ROPE_DRIVER), ("zkob_softmax.cpp", SOFTMAX_DRIVER),
                      ("zkob_rmsnorm.cpp", RMSNORM_DRIVER), ("zkob_softmax8.cpp", SOFTMAX8_DRIVER),
                      ("zkob_rowmax.cpp", ROWMAX_DRIVER), ("zkob_hostmath.cpp", HOSTMATH)):
        src = os.path.join(HERE, "host", name)
        deps = [src, os.path.join(INCLUDE, "zkh.h"), os.path.join(INCLUDE, "zkh_p3.hpp"), os.path.join(INCLUDE, "zkh_p3_verify.hpp"),
                os.path.join(INCLUDE, "zkh_p3_layer.hpp"), os.path.join(HERE, "host", "zkob_common.hpp"), LIB]
        if not force and os.path.exists(exe) and all(os.path.getmtime(d) <= os.path.getmtime(exe) for d in deps):
            continue
        subprocess.check_call([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-Wall", "-pthread", "-I", INCLUDE, src, "-o", exe,
                               "-L", HERE, "-lzkh", "-Wl,-rpath,$ORIGIN"])
    return SELFTEST


def build(force=False, verbose=False):
    build_lib(force, verbose)
    build_selftest(force)
    return LIB


def build_lib(force=False, verbose=False):
    if not force and not stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for src in sources():
        obj = os.path.join(HERE, "build", os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write("== %s\n%s\n" % (os.path.basename(src), out))
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc, "-shared", "-o", LIB] + objs +
                          ["-gencode", "arch=compute_100a,code=sm_100a"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
