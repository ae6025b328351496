"""TEST INFRASTRUCTURE ONLY - the checker, never the product path.

Two independent CPU oracles for channels-last GroupNorm + activation, forward and backward:

* `oracle_c`     - the plain-C double-precision restatement of the reference algorithm
                   (oracle/gn_oracle.c, built by oracle/Makefile), called through ctypes;
* `oracle_torch` - `torch.nn.functional.group_norm` followed by the torch activation on CPU in
                   fp64, gradients by autograd.  This is the oracle the reference's own tests use
                   (test/check_outputs.py:91-92,104 of latentCall145/channels-last-groupnorm, there
                   on CUDA) and the one the build's target names.

plus the seeded synthetic-input generator shared by tests, smoke and benchmark, and the error
metric / tolerances.  Only tests/, the smoke run and the benchmark's CPU-baseline leg may import
this module.
"""
import ctypes
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "libgn_oracle.so")

ACT_NAMES = ["identity", "relu", "silu", "gelu", "gelu_tanh"]
ACT_CODES = {"identity": 0, "relu": 1, "silu": 2, "swish": 2, "gelu": 3, "gelu_tanh": 4}

# max-abs error relative to max(1, max|oracle|): 1e-5 for fp32 tensors, 1e-2 for 16-bit tensors,
# 1e-10 for fp64 tensors
TOLERANCE = {torch.float32: 1e-5, torch.float16: 1e-2, torch.bfloat16: 1e-2, torch.float64: 1e-10}

_lib = None


def build(force=False):
    """Compiles oracle/gn_oracle.c with the Makefile beside it (gcc, no CUDA)."""
    src = os.path.join(HERE, "gn_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", HERE, "-B", "_build/libgn_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(LIB_PATH)
        dp = ctypes.POINTER(ctypes.c_double)
        lib.gn_oracle_fwd.restype = None
        lib.gn_oracle_fwd.argtypes = [dp, dp, dp, ctypes.c_long, ctypes.c_long, ctypes.c_long, ctypes.c_long,
                                      ctypes.c_double, ctypes.c_int, dp, dp, dp]
        lib.gn_oracle_bwd.restype = None
        lib.gn_oracle_bwd.argtypes = [dp, dp, dp, dp, dp, dp, ctypes.c_long, ctypes.c_long, ctypes.c_long,
                                      ctypes.c_long, ctypes.c_int, dp, dp, dp]
        _lib = lib
    return _lib


def _dp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))


def _nhwc64(t):
    """(N, C, *spatial) tensor of any float dtype -> contiguous float64 numpy array (N, R, C)."""
    n, c = t.shape[0], t.shape[1]
    return np.ascontiguousarray(
        t.detach().cpu().to(torch.float64).reshape(n, c, -1).permute(0, 2, 1).contiguous().numpy())


def _from_nhwc(a, shape):
    n, c = shape[0], shape[1]
    return torch.from_numpy(a).permute(0, 2, 1).reshape(n, c, *shape[2:])


def oracle_c(x, gamma, beta, dy, G, eps, act, threads=1):
    """C oracle. x, dy: (N, C, *spatial) tensors (any float dtype; values are up-cast to fp64).

    Returns dict of fp64 CPU tensors: y, dx (shape of x), dgamma, dbeta (C), mean, rstd (N, G).
    dy may be None (forward only).  `threads` > 1 splits the batch over Python threads
    (ctypes releases the GIL); results are independent of the split except for the summation
    order of dgamma / dbeta over the batch.
    """
    lib = _load()
    act = ACT_CODES[act] if isinstance(act, str) else int(act)
    xs = _nhwc64(x)
    N, R, C = xs.shape
    ga = np.ascontiguousarray(gamma.detach().cpu().to(torch.float64).numpy())
    be = np.ascontiguousarray(beta.detach().cpu().to(torch.float64).numpy())
    dys = _nhwc64(dy) if dy is not None else None
    y = np.empty_like(xs)
    mean = np.empty((N, G), dtype=np.float64)
    rstd = np.empty((N, G), dtype=np.float64)
    dx = np.empty_like(xs) if dys is not None else None
    threads = max(1, min(int(threads), N))
    bounds = np.linspace(0, N, threads + 1).astype(int)
    dgs = np.zeros((threads, C))
    dbs = np.zeros((threads, C))

    def work(i):
        a, b = int(bounds[i]), int(bounds[i + 1])
        if b <= a:
            return
        lib.gn_oracle_fwd(_dp(xs[a:b]), _dp(ga), _dp(be), b - a, R, C, G, float(eps), act,
                          _dp(y[a:b]), _dp(mean[a:b]), _dp(rstd[a:b]))
        if dys is not None:
            lib.gn_oracle_bwd(_dp(dys[a:b]), _dp(xs[a:b]), _dp(ga), _dp(be), _dp(mean[a:b]), _dp(rstd[a:b]),
                              b - a, R, C, G, act, _dp(dx[a:b]), _dp(dgs[i]), _dp(dbs[i]))

    if threads == 1:
        work(0)
    else:
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(work, range(threads)))
    out = {"y": _from_nhwc(y, x.shape), "mean": torch.from_numpy(mean), "rstd": torch.from_numpy(rstd)}
    if dys is not None:
        out["dx"] = _from_nhwc(dx, x.shape)
        out["dgamma"] = torch.from_numpy(dgs.sum(0))
        out["dbeta"] = torch.from_numpy(dbs.sum(0))
    return out


def torch_activation(act):
    act = ACT_NAMES[act] if not isinstance(act, str) else act
    return {
        "identity": lambda t: t,
        "relu": F.relu,
        "silu": F.silu,
        "swish": F.silu,
        "gelu": F.gelu,
        "gelu_tanh": lambda t: F.gelu(t, approximate="tanh"),
    }[act]


def oracle_torch(x, gamma, beta, dy, G, eps, act, dtype=torch.float64):
    """torch CPU oracle: act(F.group_norm(x)) in `dtype` (fp64 by default), gradients by autograd."""
    xs = x.detach().cpu().to(dtype).requires_grad_(dy is not None)
    ga = gamma.detach().cpu().to(dtype).requires_grad_(dy is not None)
    be = beta.detach().cpu().to(dtype).requires_grad_(dy is not None)
    y = torch_activation(act)(F.group_norm(xs, G, ga, be, eps))
    out = {"y": y.detach()}
    if dy is not None:
        dx, dg, db = torch.autograd.grad(y, (xs, ga, be), dy.detach().cpu().to(dtype))
        out.update(dx=dx, dgamma=dg, dbeta=db)
    return out


def rel_err(actual, expected):
    """max|a - b| / max(1, max|b|) with b the oracle (fp64)."""
    a = actual.detach().cpu().to(torch.float64)
    b = expected.detach().cpu().to(torch.float64)
    if b.numel() == 0:
        return 0.0
    return float((a - b).abs().max() / max(1.0, float(b.abs().max())))


# ------------------------------------------------------------------------------------------------
# seeded synthetic inputs
# ------------------------------------------------------------------------------------------------
def make_inputs(N, C, spatial, dtype, seed=0, x_dist="normal", x_scale=1.0, device="cpu"):
    """x, gamma, beta, dy drawn on CPU in fp32 from one generator in that order, then cast.

    x ~ N(0, x_scale^2) or U(-3, 3); gamma ~ U(0.5, 1.5); beta ~ N(0, 0.1^2); dy ~ N(0, 1).
    x and dy are returned as (N, C, *spatial) tensors with NHWC (channels-last) storage.
    """
    g = torch.Generator().manual_seed(seed)
    shape_nhwc = (N, *spatial, C)
    if x_dist == "uniform3":
        x = torch.rand(shape_nhwc, generator=g) * 6.0 - 3.0
    else:
        x = torch.randn(shape_nhwc, generator=g) * x_scale
    gamma = torch.rand(C, generator=g) + 0.5
    beta = torch.randn(C, generator=g) * 0.1
    dy = torch.randn(shape_nhwc, generator=g)
    perm = (0, len(shape_nhwc) - 1, *range(1, len(shape_nhwc) - 1))
    x = x.to(dtype).to(device).permute(*perm)
    dy = dy.to(dtype).to(device).permute(*perm)
    return x, gamma.to(dtype).to(device), beta.to(dtype).to(device), dy
