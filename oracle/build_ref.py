"""Compile the reference's own sources, where they lie, into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  Nothing the library ships imports this file or the
objects it produces; they are the checker (parity tests) and the CPU / reference
arm of the benchmark.

What is built (all from the unmodified files of the reference checkout, whose
location is given by --ref or the L1ATTN_REFERENCE environment variable):

  cpp/l1attn_drv.cpp               -> _ref/l1attn_drv_cpp.so           (fp64 CPU loops)
  cpp/l1attn_sparse_drv.cpp        -> _ref/l1attn_sparse_drv.so
  cpp/l1attn_sparse_bidi_drv.cpp   -> _ref/l1attn_sparse_bidi_drv.so
  cuda/l1attn_cuda_drv.cpp + cuda/l1attn_cuda_kernel.cu
                                   -> _ref/ref_l1attn_cuda_drv.so      (reference GPU kernels, sm_100)
  cuda/l1attn_sparse_cuda_drv.cpp + cuda/l1attn_sparse_cuda_kernel.cu
                                   -> _ref/ref_l1attn_sparse_cuda_drv.so
  cuda/l1attn_sparse_bidi_cuda_drv.cpp + cuda/l1attn_sparse_cuda_kernel.cu
                                   -> _ref/ref_l1attn_sparse_bidi_cuda_drv.so

The CUDA modules get a `ref_` prefix because the product exports pybind modules
with the reference's own names; PYBIND11_MODULE(TORCH_EXTENSION_NAME, ...) in the
reference drivers takes its name from the build, so renaming needs no source edit.
Flags mirror cpp/setup.py (-O2 via sysconfig) and cuda/setup.py:4-10.

No source file is copied: the compiler reads the reference tree directly and
only objects / shared libraries land under oracle/_ref/.
"""
import argparse
import os
import shutil
import sys
import glob

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

CPP_MODULES = {
    "l1attn_drv_cpp": ["cpp/l1attn_drv.cpp"],
    "l1attn_sparse_drv": ["cpp/l1attn_sparse_drv.cpp"],
    "l1attn_sparse_bidi_drv": ["cpp/l1attn_sparse_bidi_drv.cpp"],
}
CUDA_MODULES = {
    "ref_l1attn_cuda_drv": ["cuda/l1attn_cuda_drv.cpp", "cuda/l1attn_cuda_kernel.cu"],
    "ref_l1attn_sparse_cuda_drv": ["cuda/l1attn_sparse_cuda_drv.cpp", "cuda/l1attn_sparse_cuda_kernel.cu"],
    "ref_l1attn_sparse_bidi_cuda_drv": ["cuda/l1attn_sparse_bidi_cuda_drv.cpp", "cuda/l1attn_sparse_cuda_kernel.cu"],
}
# cuda/setup.py:4-10 of the reference
REF_NVCC_FLAGS = ["-O3", "-std=c++17", "--expt-relaxed-constexpr", "--expt-extended-lambda", "--use_fast_math"]


def built(name):
    return os.path.exists(os.path.join(OUT, name + ".so"))


def build_one(name, sources, ref, cuda):
    from torch.utils.cpp_extension import load
    bdir = os.path.join(OUT, "build_" + name)
    os.makedirs(bdir, exist_ok=True)
    kwargs = dict(name=name, sources=[os.path.join(ref, s) for s in sources], build_directory=bdir,
                  extra_cflags=["-O2"], verbose=False)
    if cuda:
        os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
        kwargs["extra_cuda_cflags"] = REF_NVCC_FLAGS
    load(**kwargs)
    so = glob.glob(os.path.join(bdir, name + "*.so"))[0]
    shutil.copy(so, os.path.join(OUT, name + ".so"))
    shutil.rmtree(bdir, ignore_errors=True)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("L1ATTN_REFERENCE", ""))
    ap.add_argument("--only", choices=["cpp", "cuda", "all"], default="all")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    if not a.ref or not os.path.isdir(os.path.join(a.ref, "cpp")):
        print("build_ref: no reference checkout given (--ref / L1ATTN_REFERENCE); nothing built")
        return 0
    os.makedirs(OUT, exist_ok=True)
    todo = []
    if a.only in ("cpp", "all"):
        todo += [(n, s, False) for n, s in CPP_MODULES.items()]
    if a.only in ("cuda", "all"):
        todo += [(n, s, True) for n, s in CUDA_MODULES.items()]
    for name, srcs, cuda in todo:
        if built(name) and not a.force:
            print("build_ref: %s already built" % name)
            continue
        print("build_ref: building %s" % name, flush=True)
        build_one(name, srcs, a.ref, cuda)
    return 0


if __name__ == "__main__":
    sys.exit(main())
