"""Build recipe for the native parts of the package (run here on CPU; nvcc cross-compiles sm_100a).

    python -m armnn_b200.build            # libb200k.so (+ the Arm NN backend plugin when the Arm NN
                                          #   headers are reachable through $ARMNN_ROOT)

Artefacts are written in-tree next to the sources and are git-ignored:
    armnn_b200/libb200k.so                 the kernel library (C ABI of include/b200k.h)
    armnn_b200/backend/Nv_B200Acc_backend.so   the IBackendInternal plugin (needs Arm NN headers)

The Arm NN source tree (headers only are needed) is found through the environment variable ARMNN_ROOT.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200k.so")
PLUGIN_DIR = os.path.join(HERE, "backend")
PLUGIN = os.path.join(PLUGIN_DIR, "Nv_B200Acc_backend.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-fmad=false", "-Xcompiler", "-fPIC"]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n%s\n%s" % (" ".join(cmd), r.stdout))
    return r.stdout


def build_kernels(force=False, verbose=False):
    """Compile every .cu under csrc/ into objects and link libb200k.so."""
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(ROOT, "include", "b200k.h")]
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            cmd = ["nvcc"] + NVCC_FLAGS + ["-c", s, "-o", o]
            if verbose:
                print(" ".join(cmd), flush=True)
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), out))
    if force or procs or _newer(LIB, objs):
        _run(["nvcc", "-shared", "-o", LIB] + objs, verbose)
    return LIB


def armnn_root():
    """Location of an Arm NN source tree (headers only are needed): $ARMNN_ROOT, or None."""
    cand = os.environ.get("ARMNN_ROOT")
    if cand and os.path.isfile(os.path.join(cand, "include", "armnn", "backends", "IBackendInternal.hpp")):
        return cand
    return None


def build_plugin(force=False, verbose=False):
    """Compile the Arm NN backend plugin against the Arm NN headers; skipped when they are absent."""
    root = armnn_root()
    # B200RegistryInitializer.cpp belongs to the in-tree (static) build only: the runtime registers a dynamic backend itself
    srcs = sorted(f for f in glob.glob(os.path.join(PLUGIN_DIR, "*.cpp")) if not f.endswith("B200RegistryInitializer.cpp"))
    if root is None or not srcs:
        return None
    hdrs = glob.glob(os.path.join(PLUGIN_DIR, "*.hpp")) + glob.glob(os.path.join(PLUGIN_DIR, "workloads", "*.hpp")) + \
        [os.path.join(ROOT, "include", "b200k.h")]
    if not (force or _newer(PLUGIN, srcs + hdrs + [LIB])):
        return PLUGIN
    incs = ["include", "profiling", "profiling/common/include", "profiling/client/include", "src/armnn",
            "src/armnnUtils", "src/backends", "src/profiling", "third-party"]
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-w", "-DNDEBUG", "-o", PLUGIN] + srcs + \
        ["-I" + os.path.join(root, i) for i in incs] + \
        ["-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include", "-I" + PLUGIN_DIR,
         "-L" + HERE, "-lb200k", "-Wl,-rpath,$ORIGIN/..", "-L/usr/local/cuda/lib64", "-lcudart"]
    _run(cmd, verbose)
    return PLUGIN


def armnn_lib_dir():
    """Directory with a built libarmnn.so: $ARMNN_LIB_DIR, else oracle/_ref of this repository."""
    return os.environ.get("ARMNN_LIB_DIR") or os.path.join(ROOT, "oracle", "_ref")


def build_host_binding(force=False, verbose=False):
    """armnn_b200/host/libarmnn_capi.so: the C binding of the Arm NN runtime API that armnn_b200.armnn_host loads.
    Needs the Arm NN headers ($ARMNN_ROOT) and a libarmnn.so to link against; skipped otherwise."""
    root, libdir = armnn_root(), armnn_lib_dir()
    src = os.path.join(HERE, "host", "armnn_capi.cpp")
    out = os.path.join(HERE, "host", "libarmnn_capi.so")
    if root is None or not os.path.exists(os.path.join(libdir, "libarmnn.so")):
        return None
    if not (force or _newer(out, [src, os.path.join(ROOT, "include", "b200k.h"), os.path.join(libdir, "libarmnn.so")])):
        return out
    incs = ["include", "profiling", "profiling/common/include", "profiling/client/include"]
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-w", "-DNDEBUG", "-o", out, src] + \
        ["-I" + os.path.join(root, i) for i in incs] + ["-L" + libdir, "-larmnn", "-Wl,-rpath,$ORIGIN/" + os.path.relpath(libdir, os.path.join(HERE, "host")), "-lpthread"]
    _run(cmd, verbose)
    return out


def build_all(force=False, verbose=False):
    build_kernels(force, verbose)
    build_plugin(force, verbose)
    build_host_binding(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built", LIB)
