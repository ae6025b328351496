"""Compile the UNMODIFIED reference extension (test infrastructure only).

The reference (`latentCall145/channels-last-groupnorm`, package `gnnhwc`) JIT-builds one
library from `src/gnnhwc/csrc/custom_gn.cpp` + `src/gnnhwc/csrc/gn_kernel.cu`
(`src/gnnhwc/custom_gn.py:7-27`).  This script compiles exactly those two files, where they
lie in the reference checkout, with the reference's own compiler flags plus an sm_100a
target, and writes the result to `oracle/_ref/gn_op.so`.  No reference source is copied.

The library registers `torch.ops.gnop.fwd / bwd` (`custom_gn.cpp:91-94`).  It is CUDA-only,
so it can only be *executed* on a GPU machine; it is used there by the GPU parity tests, by
`tests/golden/make_golden.py` and by the reference-timing leg of `bench.py`.  Nothing in the
shipped package may load it.

Usage:  python oracle/build_ref.py [path-to-reference-checkout]
"""
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_LIB = os.path.join(OUT_DIR, "gn_op.so")


def reference_sources(ref_root):
    csrc = os.path.join(ref_root, "src", "gnnhwc", "csrc")
    return os.path.join(csrc, "custom_gn.cpp"), os.path.join(csrc, "gn_kernel.cu")


def build(ref_root, force=False, verbose=True):
    """Returns the path of the built library, or None when the reference checkout is absent."""
    cpp, cu = reference_sources(ref_root)
    if not (os.path.isfile(cpp) and os.path.isfile(cu)):
        return OUT_LIB if os.path.isfile(OUT_LIB) else None
    if os.path.isfile(OUT_LIB) and not force:
        newest_src = max(os.path.getmtime(cpp), os.path.getmtime(cu))
        if os.path.getmtime(OUT_LIB) >= newest_src:
            return OUT_LIB
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT_DIR, exist_ok=True)
    inc = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.dirname(cu)]:
        inc += ["-I", p]
    torch_lib = ce.library_paths()[0]
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    common = ["-DTORCH_EXTENSION_NAME=gn_op", "-DTORCH_API_INCLUDE_EXTENSION_H", "-std=c++17"]
    obj_cpp = os.path.join(OUT_DIR, "custom_gn.o")
    obj_cu = os.path.join(OUT_DIR, "gn_kernel.o")
    # host flags of the reference: src/gnnhwc/custom_gn.py:20-24 (-march=native is dropped:
    # the library is built on one machine and run on another)
    cmd_cpp = ["g++", "-c", cpp, "-o", obj_cpp, "-fPIC", "-Ofast", "-funroll-all-loops"] + common + inc
    # device flags of the reference: src/gnnhwc/custom_gn.py:13-19, plus the sm_100a target
    cmd_cu = [nvcc, "-c", cu, "-o", obj_cu, "-Xcompiler", "-fPIC", "-O3",
              "-gencode", "arch=compute_100a,code=sm_100a",
              "-use_fast_math", "-extra-device-vectorization", "-extended-lambda", "-lineinfo",
              "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
              "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
              "--expt-relaxed-constexpr"] + common + inc
    cmd_ld = ["g++", "-shared", obj_cpp, obj_cu, "-o", OUT_LIB, "-L", torch_lib,
              "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
              "-L", "/usr/local/cuda/lib64", "-lcudart"]
    procs = []
    for cmd in (cmd_cpp, cmd_cu):
        if verbose:
            print("+", " ".join(cmd), flush=True)
        procs.append(subprocess.Popen(cmd))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("reference compile step failed")
    if verbose:
        print("+", " ".join(cmd_ld), flush=True)
    subprocess.check_call(cmd_ld)
    for o in (obj_cpp, obj_cu):
        os.remove(o)
    return OUT_LIB


if __name__ == "__main__":
    # default: a checkout of the reference beside this repository
    root = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--") else os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    lib = build(root, force="--force" in sys.argv)
    print("reference library:", lib)
