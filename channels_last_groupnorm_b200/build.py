"""Ahead-of-time build of the two native libraries, in-tree under `lib/`.

  lib/libgnb200.so      hand-written sm_100a CUDA kernels + planner + C ABI (include/gnb200.h);
                        depends only on the CUDA runtime (linked statically), not on torch
  lib/gnb200_torch.so   C++ torch binding (torch.ops.gnb200.*) over that C ABI

The reference JIT-compiles its extension on first import (src/gnnhwc/custom_gn.py:7-27); here the
libraries are built once (`python -m channels_last_groupnorm_b200.build`) and loaded from disk.
nvcc cross-compiles for sm_100a, so no GPU is needed to build.
"""
import hashlib
import os
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
INCLUDE_DIR = os.path.join(os.path.dirname(PKG_DIR), "include")
CORE_LIB = os.path.join(LIB_DIR, "libgnb200.so")
TORCH_LIB = os.path.join(LIB_DIR, "gnb200_torch.so")

CUDA_SOURCES = ["gn_fwd.cu", "gn_bwd.cu", "gn_wave.cu", "gn_nchw.cu", "gn_f64.cu", "gn_plan.cu", "gn_capi.cu", "gn_static_scratch.cu"]
CUDA_HEADERS = ["gn_common.cuh", "gn_math.cuh", "gn_peer.cuh", "gn_kernels.h", os.path.join(INCLUDE_DIR, "gnb200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return os.path.join(home, "bin", "nvcc")


def _digest(paths):
    """Content hash of source files (modification times do not survive copying a checkout)."""
    h = hashlib.sha256()
    for p in paths:
        full = p if os.path.isabs(p) else os.path.join(CSRC, p)
        with open(full, "rb") as f:
            h.update(f.read())
        h.update(b"\0")
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _stamp_path(lib_path):
    return lib_path + ".stamp"


def _stamp_matches(lib_path, digest):
    if not os.path.exists(lib_path) or not os.path.exists(_stamp_path(lib_path)):
        return False
    with open(_stamp_path(lib_path)) as f:
        return f.read().strip() == digest


def _write_stamp(lib_path, digest):
    with open(_stamp_path(lib_path), "w") as f:
        f.write(digest + "\n")


def _core_digest():
    return _digest(CUDA_SOURCES + CUDA_HEADERS)


def _torch_digest():
    return _digest(["gn_torch.cpp", os.path.join(INCLUDE_DIR, "gnb200.h")])


def core_is_stale():
    return not _stamp_matches(CORE_LIB, _core_digest())


def torch_is_stale():
    return not _stamp_matches(TORCH_LIB, _torch_digest())


def build_core(verbose=False, extra_flags=()):
    os.makedirs(LIB_DIR, exist_ok=True)
    objs, procs = [], []
    for src in CUDA_SOURCES:
        obj = os.path.join(LIB_DIR, src.replace(".cu", ".o"))
        cmd = [_nvcc()] + NVCC_FLAGS + list(extra_flags) + ["-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            print("+", " ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out.strip():
            print(out)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s" % (src, out))
    cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
           "-o", CORE_LIB] + objs
    if verbose:
        print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    for o in objs:
        os.remove(o)
    _write_stamp(CORE_LIB, _core_digest())
    return CORE_LIB


def build_torch(verbose=False):
    from torch.utils import cpp_extension as ce

    os.makedirs(LIB_DIR, exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]:
        inc += ["-isystem", p]
    torch_lib = ce.library_paths()[0]
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", os.path.join(CSRC, "gn_torch.cpp"), "-o", TORCH_LIB,
           "-DTORCH_API_INCLUDE_EXTENSION_H"] + inc + [
        "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
        "-L", LIB_DIR, "-lgnb200", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    if verbose:
        print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    _write_stamp(TORCH_LIB, _torch_digest())
    return TORCH_LIB


def build_all(force=False, verbose=False):
    """Builds whatever is missing or older than its sources. Returns the two library paths."""
    if force or core_is_stale():
        build_core(verbose)
    if force or torch_is_stale():
        build_torch(verbose)
    return CORE_LIB, TORCH_LIB


if __name__ == "__main__":
    libs = build_all(force="--force" in sys.argv, verbose=True)
    print("built:", *libs)
