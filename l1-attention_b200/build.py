"""Build everything in this directory, in place, for sm_100a.

  libl1attn_b200.so                 CUDA kernels + the C ABI of include/l1attn_b200.h (nvcc; no torch)
  l1attn_cuda_drv.so                pybind/torch drivers with the reference's module names
  l1attn_sparse_cuda_drv.so         (cuda/setup.py:13-33 of the reference builds the same three
  l1attn_sparse_bidi_cuda_drv.so     modules), each a thin layer that calls the C ABI

Usage:  python build.py [--force] [--no-drivers]
nvcc cross-compiles, so no GPU is needed to build.  The objects stay beside the sources
(they are git-ignored) so a copy of the tree carries them.
"""
import argparse
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INC = os.path.join(ROOT, "include")
LIB = os.path.join(HERE, "libl1attn_b200.so")
CU_SOURCES = ["dense_fwd.cu", "dense_fwd_tma.cu", "dense_bwd.cu", "dense_bwd_tma.cu", "dense_bwd_sv.cu", "dense_ties.cu", "dense_softmax_v.cu", "sparse.cu", "coo.cu", "capi.cu", "tma.cu"]
DRIVERS = ["l1attn_cuda_drv", "l1attn_sparse_cuda_drv", "l1attn_sparse_bidi_cuda_drv"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def nvcc():
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def build_lib(force=False, verbose=False):
    srcs = [os.path.join(CSRC, s) for s in CU_SOURCES]
    deps = srcs + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(INC, "*.h"))
    if not force and not _newer(LIB, deps):
        return LIB
    objs = []
    procs = []
    for s in srcs:
        o = s[:-3] + ".o"
        objs.append(o)
        cmd = [nvcc()] + NVCC_FLAGS + ["-I", INC, "-I", CSRC, "-c", s, "-o", o]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s" % (s, out))
        if verbose:
            print(out)
    subprocess.run([nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs + ["-lcudart", "-Xlinker", "-soname=libl1attn_b200.so"], check=True)
    return LIB


def build_drivers(force=False):
    """The pybind layer needs torch headers; it links against libl1attn_b200.so with an $ORIGIN rpath."""
    import ctypes
    from torch.utils.cpp_extension import load
    ctypes.CDLL(build_lib(), mode=ctypes.RTLD_GLOBAL)  # so that load()'s trial dlopen of each driver resolves it
    deps = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(INC, "*.h"))
    for name in DRIVERS:
        so = os.path.join(HERE, name + ".so")
        src = os.path.join(CSRC, name + ".cpp")
        if not force and not _newer(so, deps + [src]):
            continue
        bdir = os.path.join(HERE, "build", name)
        os.makedirs(bdir, exist_ok=True)
        load(name=name, sources=[src], build_directory=bdir, with_cuda=True, is_python_module=False,
             extra_cflags=["-O2", "-I" + INC, "-I" + CSRC],
             extra_ldflags=["-L" + HERE, "-ll1attn_b200", "-Wl,-rpath,'$$ORIGIN'"], verbose=False)
        built = glob.glob(os.path.join(bdir, name + "*.so"))[0]
        shutil.copy(built, so)
        shutil.rmtree(bdir, ignore_errors=True)
    return [os.path.join(HERE, n + ".so") for n in DRIVERS]


def build_all(force=False, drivers=True, verbose=False):
    build_lib(force, verbose)
    if drivers:
        build_drivers(force)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--no-drivers", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    build_all(a.force, not a.no_drivers, a.verbose)
    print("built:", LIB)
