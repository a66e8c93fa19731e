"""Builds the in-tree native libraries with nvcc for sm_100a.

    python -m ogle_b200.build            # build what is out of date
    python -m ogle_b200.build --force    # rebuild everything

Outputs (next to this file, git-ignored, shipped with the source tree):
    libogle_cuda.so   the CUDA kernels and the C ABI of include/ogle_cuda.h
    libogle_rt.so     the C++ host runtime (dlx loading, kernel registry, session)
                      and the C ABI of include/ogle_runtime.h; links libogle_cuda.so
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# /usr/bin/g++ is the full distribution compiler; the CXX the image exports is a
# trimmed copy without OpenMP.
HOST_CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd):
    print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build_cuda(force=False, verbose_ptxas=False):
    kdir = os.path.join(CSRC, "kernels")
    srcs = sorted(glob.glob(os.path.join(kdir, "*.cu")))
    deps = srcs + glob.glob(os.path.join(kdir, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, deps):
            cmd = [NVCC, "-ccbin", HOST_CXX, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
                   "-I", INCLUDE, "-I", kdir] + ARCH + (["-Xptxas", "-v"] if verbose_ptxas else []) + ["-c", s, "-o", o]
            print(" ".join(cmd), flush=True)
            procs.append((s, subprocess.Popen(cmd)))
    for s, p in procs:
        if p.wait() != 0:
            raise RuntimeError(f"nvcc failed on {s}")
    out = os.path.join(HERE, "libogle_cuda.so")
    if force or procs or _newer(out, objs):
        _run([NVCC, "-ccbin", HOST_CXX, "-shared", "-o", out] + objs + ARCH + ["-lcudart", "-Xlinker", "-rpath,$ORIGIN"])
    return out


def build_runtime(force=False):
    rdir = os.path.join(CSRC, "runtime")
    srcs = sorted(glob.glob(os.path.join(rdir, "*.cc")))
    if not srcs:
        return None
    deps = srcs + glob.glob(os.path.join(rdir, "*.h")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    out = os.path.join(HERE, "libogle_rt.so")
    if force or _newer(out, deps + [os.path.join(HERE, "libogle_cuda.so")]):
        _run([HOST_CXX, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-Wno-sign-compare", "-pthread",
              "-I", INCLUDE, "-I", rdir, "-I", "/usr/local/cuda/include"] + srcs +
             ["-o", out, "-L", HERE, "-logle_cuda", "-L", "/usr/local/cuda/lib64", "-lcudart",
              "-Wl,-rpath,$ORIGIN", "-Wl,--no-as-needed"])
    return out


def build_tools(force=False):
    """The headless run/profile program (csrc/tools/ogle_profile.cc) -> ogle_b200/ogle_profile."""
    src = os.path.join(CSRC, "tools", "ogle_profile.cc")
    if not os.path.exists(src):
        return None
    rdir = os.path.join(CSRC, "runtime")
    out = os.path.join(HERE, "ogle_profile")
    if force or _newer(out, [src, os.path.join(HERE, "libogle_rt.so")]):
        _run([HOST_CXX, "-O2", "-std=c++17", "-Wall", "-Wno-sign-compare", "-I", INCLUDE, "-I", rdir, src, "-o", out,
              "-L", HERE, "-logle_rt", "-logle_cuda", "-L", "/usr/local/cuda/lib64", "-lcudart",
              "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,/usr/local/cuda/lib64"])
    return out


def build_all(force=False, verbose_ptxas=False):
    a = build_cuda(force, verbose_ptxas)
    b = build_runtime(force)
    build_tools(force)
    return a, b


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose_ptxas="--ptxas" in sys.argv)
