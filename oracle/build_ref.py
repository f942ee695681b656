"""Builds oracle/_ref/libref_sched_meta.so: the reference's OWN tile-scheduler metadata kernel and split-KV combine kernel
(csrc/smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.cu and csrc/smxx/decode/combine/combine.cu, compiled
unmodified from a FlashMLA checkout, with the reference's own compiler flags) behind the C entry points of
oracle/ref_sched_shim.cu, for sm_100a.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  The parity tests load the library when it exists and compare this
repository's scheduler and combine kernels (and the scheduler's CPU restatement) with it.

Usage:  python oracle/build_ref.py <path-to-FlashMLA-checkout>

The reference source needs two things outside its own files: its `kerutils` headers (in the checkout) and CUTLASS, whose
submodule is absent from the checkout; the CUTLASS headers that ship inside an installed Python package (flashinfer or
tilelang) are used instead.  Only helper-level CUTLASS is involved (ceil_div, numeric types, CuTe index arithmetic).  The
reference's attention kernels are NOT built or run this way: they wait on barriers without a time limit, and a version
mismatch of the CUTLASS headers could leave such a wait unserved on a shared GPU.
Returns / prints the path of the library, or None when a prerequisite is missing."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libref_sched_meta.so")


def cutlass_include():
    for pkg, rel in (("flashinfer", "data/cutlass/include"), ("tilelang", "3rdparty/cutlass/include")):
        try:
            mod = __import__(pkg)
        except Exception:
            continue
        p = os.path.join(os.path.dirname(mod.__file__), rel)
        if os.path.exists(os.path.join(p, "cutlass", "fast_math.h")):
            return p
    return None


def build(ref_root):
    src = os.path.join(ref_root, "csrc/smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.cu")
    src_combine = os.path.join(ref_root, "csrc/smxx/decode/combine/combine.cu")
    cut = cutlass_include()
    if not os.path.exists(src) or not os.path.exists(src_combine) or cut is None:
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    # (the flags of the reference's setup.py:108-123 that change generated code)
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++20", "-DNDEBUG", "-D_USE_MATH_DEFINES",
           "--expt-relaxed-constexpr", "--expt-extended-lambda", "--use_fast_math", "-lineinfo", "-Wno-deprecated-declarations",
           "-Xcompiler", "-fPIC", "-shared",
           "-I", os.path.join(ref_root, "csrc"), "-I", os.path.join(ref_root, "csrc/kerutils/include"), "-I", cut,
           src, src_combine, os.path.join(HERE, "ref_sched_shim.cu"), "-o", LIB, "-lcudart"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(sys.argv[1]))
