"""Loads the native libraries and exposes the C ABI through ctypes.

There is no Python, PyTorch-eager or CPU fallback anywhere in this package: if the libraries
cannot be loaded (or built from the in-tree sources), importing the package raises.
"""
import ctypes
import os

import torch

from . import build as _build

_c_int64 = ctypes.c_int64
_c_void_p = ctypes.c_void_p

DTYPE_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _load():
    try:
        core_path, torch_path = _build.build_all()
    except Exception as exc:  # pragma: no cover - depends on the toolchain of the machine
        if not (os.path.exists(_build.CORE_LIB) and os.path.exists(_build.TORCH_LIB)):
            raise ImportError(
                "channels_last_groupnorm_b200: the native libraries are missing and could not be built "
                "(run `python -m channels_last_groupnorm_b200.build`): %s" % exc) from exc
        core_path, torch_path = _build.CORE_LIB, _build.TORCH_LIB
    core = ctypes.CDLL(core_path, mode=ctypes.RTLD_GLOBAL)
    torch.ops.load_library(torch_path)
    return core


lib = _load()

lib.gnb200_version.restype = ctypes.c_int
lib.gnb200_last_error.restype = ctypes.c_char_p
lib.gnb200_act_code.restype = ctypes.c_int
lib.gnb200_act_code.argtypes = [ctypes.c_char_p]
for _name in ("gnb200_fwd_workspace_bytes", "gnb200_bwd_workspace_bytes"):
    getattr(lib, _name).restype = ctypes.c_size_t
    getattr(lib, _name).argtypes = [_c_int64, _c_int64, _c_int64, _c_int64, ctypes.c_int]
lib.gnb200_fwd.restype = ctypes.c_int
lib.gnb200_fwd.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int64, _c_int64, _c_int64, _c_int64,
                           ctypes.c_double, ctypes.c_int, ctypes.c_int, _c_void_p, _c_void_p, _c_void_p,
                           _c_void_p, ctypes.c_size_t, _c_void_p]
lib.gnb200_bwd.restype = ctypes.c_int
lib.gnb200_bwd.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                           _c_int64, _c_int64, _c_int64, _c_int64, ctypes.c_int, ctypes.c_int,
                           _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, ctypes.c_size_t, _c_void_p]
lib.gnb200_peer_exchange_bytes.restype = ctypes.c_size_t
lib.gnb200_peer_exchange_bytes.argtypes = [_c_int64, ctypes.c_int]
lib.gnb200_bwd_peer.restype = ctypes.c_int
lib.gnb200_bwd_peer.argtypes = lib.gnb200_bwd.argtypes[:-1] + [ctypes.POINTER(_c_void_p), ctypes.c_int, ctypes.c_int,
                                                                _c_void_p]
lib.gnb200_bwd_peer_push.restype = ctypes.c_int
lib.gnb200_bwd_peer_push.argtypes = lib.gnb200_bwd.argtypes[:14] + [_c_void_p, ctypes.c_size_t, ctypes.POINTER(_c_void_p),
                                                                    ctypes.c_int, ctypes.c_int, _c_void_p]
for _name in ("gnb200_allreduce_param_grads", "gnb200_peer_collect"):
    getattr(lib, _name).restype = ctypes.c_int
    getattr(lib, _name).argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int64, ctypes.c_int,
                                    ctypes.POINTER(_c_void_p), ctypes.c_int, ctypes.c_int, _c_void_p]
lib.gnb200_bwd_static_scratch.restype = ctypes.c_int
lib.gnb200_bwd_static_scratch.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                          _c_int64, _c_int64, _c_int64, _c_int64, ctypes.c_int, ctypes.c_int,
                                          _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p]
STATIC_SCRATCH_BYTES = 4 << 20
for _name in ("gnb200_fwd_nchw_workspace_bytes", "gnb200_bwd_nchw_workspace_bytes"):
    getattr(lib, _name).restype = ctypes.c_size_t
    getattr(lib, _name).argtypes = [_c_int64, _c_int64, _c_int64, _c_int64, ctypes.c_int]
lib.gnb200_fwd_nchw.restype = ctypes.c_int
lib.gnb200_fwd_nchw.argtypes = lib.gnb200_fwd.argtypes
lib.gnb200_bwd_nchw.restype = ctypes.c_int
lib.gnb200_bwd_nchw.argtypes = lib.gnb200_bwd.argtypes
lib.gnb200_bwd_f64_workspace_bytes.restype = ctypes.c_size_t
lib.gnb200_bwd_f64_workspace_bytes.argtypes = [_c_int64, _c_int64, _c_int64, _c_int64]
lib.gnb200_fwd_f64.restype = ctypes.c_int
lib.gnb200_fwd_f64.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int64, _c_int64, _c_int64, _c_int64,
                               ctypes.c_double, ctypes.c_int, ctypes.c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p]
lib.gnb200_bwd_f64.restype = ctypes.c_int
lib.gnb200_bwd_f64.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                               _c_int64, _c_int64, _c_int64, _c_int64, ctypes.c_int, ctypes.c_int,
                               _c_void_p, _c_void_p, _c_void_p, _c_void_p, ctypes.c_size_t, _c_void_p]
LAYOUT_NHWC, LAYOUT_NCHW = 0, 1
lib.gnb200_describe_plan.restype = ctypes.c_int
lib.gnb200_describe_plan.argtypes = [_c_int64, _c_int64, _c_int64, _c_int64, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_char_p, ctypes.c_int]
lib.gnb200_launch_count.restype = ctypes.c_int
lib.gnb200_launch_count.argtypes = [_c_int64, _c_int64, _c_int64, _c_int64, ctypes.c_int, ctypes.c_int]


class Gnb200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status, message):
        super().__init__("%s (status %d)" % (message, status))
        self.status = status


def check(status):
    if status != 0:
        raise Gnb200Error(status, lib.gnb200_last_error().decode())


def describe_plan(N, R, C, G, dtype, direction):
    """Text description of the launch plan for a problem (direction 0 = forward, 1 = backward)."""
    buf = ctypes.create_string_buffer(512)
    lib.gnb200_describe_plan(N, R, C, G, DTYPE_CODES[dtype], direction, buf, 512)
    return buf.value.decode()


lib.gnb200_wait_timeouts.restype = ctypes.c_longlong
lib.gnb200_wait_timeouts.argtypes = []
lib.gnb200_clear_wait_timeouts.restype = ctypes.c_int
lib.gnb200_clear_wait_timeouts.argtypes = []
lib.gnb200_selftest_exchange_timeout.restype = ctypes.c_int
lib.gnb200_selftest_exchange_timeout.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int64, _c_int64, _c_int64, _c_int64,
                                                 ctypes.c_double, ctypes.c_int, ctypes.c_int, _c_void_p, _c_void_p,
                                                 _c_void_p, _c_void_p]
ERR_EXCHANGE_TIMEOUT = -5


def wait_timeouts():
    """Exchange waits of the fused kernels that gave up on the current device (0 in a healthy run)."""
    v = lib.gnb200_wait_timeouts()
    if v < 0:
        raise Gnb200Error(int(v), lib.gnb200_last_error().decode())
    return int(v)


def clear_wait_timeouts():
    """Resets the give-up count and re-arms the entry points after GNB200_ERR_EXCHANGE_TIMEOUT."""
    check(lib.gnb200_clear_wait_timeouts())


def launch_count(N, R, C, G, dtype, direction):
    return lib.gnb200_launch_count(N, R, C, G, DTYPE_CODES[dtype], direction)


def _ptr(t):
    return None if t is None else t.data_ptr()


def fwd_raw(x_nhwc, gamma, beta, G, eps, act, y=None, workspace=None, stream=None):
    """Calls gnb200_fwd on torch CUDA tensors by raw pointer (used by tests and benchmarks).

    x_nhwc: contiguous (N, R, C) tensor.  Returns (y, mean, rstd).  `workspace`, if given, is a
    uint8 tensor that is reused instead of allocating one.
    """
    N, R, C = x_nhwc.shape
    code = DTYPE_CODES[x_nhwc.dtype]
    if y is None:
        y = torch.empty_like(x_nhwc)
    mean = torch.empty((N, G), device=x_nhwc.device, dtype=torch.float32)
    rstd = torch.empty((N, G), device=x_nhwc.device, dtype=torch.float32)
    need = lib.gnb200_fwd_workspace_bytes(N, R, C, G, code)
    if workspace is None and need:
        workspace = torch.empty(need, device=x_nhwc.device, dtype=torch.uint8)
    s = torch.cuda.current_stream(x_nhwc.device).cuda_stream if stream is None else stream
    check(lib.gnb200_fwd(_ptr(x_nhwc), _ptr(gamma), _ptr(beta), N, R, C, G, float(eps), int(act), code,
                         _ptr(y), _ptr(mean), _ptr(rstd), _ptr(workspace) if need else None,
                         workspace.numel() if (need and workspace is not None) else 0, s))
    return y, mean, rstd


def bwd_raw(dy_nhwc, x_nhwc, gamma, beta, mean, rstd, G, act, dx=None, workspace=None, stream=None,
            typed=True):
    """Calls gnb200_bwd by raw pointer. Returns (dx, dparam_f32[2, C], dgamma, dbeta)."""
    N, R, C = x_nhwc.shape
    code = DTYPE_CODES[x_nhwc.dtype]
    if dx is None:
        dx = torch.empty_like(x_nhwc)
    dparam = torch.empty((2, C), device=x_nhwc.device, dtype=torch.float32)
    dgamma = torch.empty(C, device=x_nhwc.device, dtype=x_nhwc.dtype) if typed else None
    dbeta = torch.empty(C, device=x_nhwc.device, dtype=x_nhwc.dtype) if typed else None
    need = lib.gnb200_bwd_workspace_bytes(N, R, C, G, code)
    if workspace is None and need:
        workspace = torch.empty(need, device=x_nhwc.device, dtype=torch.uint8)
    s = torch.cuda.current_stream(x_nhwc.device).cuda_stream if stream is None else stream
    check(lib.gnb200_bwd(_ptr(dy_nhwc), _ptr(x_nhwc), _ptr(gamma), _ptr(beta), _ptr(mean), _ptr(rstd),
                         N, R, C, G, int(act), code, _ptr(dx), _ptr(dparam), _ptr(dgamma), _ptr(dbeta),
                         _ptr(workspace) if need else None,
                         workspace.numel() if (need and workspace is not None) else 0, s))
    return dx, dparam, dgamma, dbeta


def peer_exchange_bytes(num_channels, world):
    """Bytes of one rank's exchange buffer for gnb200_bwd_peer / gnb200_allreduce_param_grads."""
    return int(lib.gnb200_peer_exchange_bytes(int(num_channels), int(world)))


def _peer_table(peer_ptrs):
    return (_c_void_p * len(peer_ptrs))(*[int(p) for p in peer_ptrs])


def bwd_peer_raw(dy_nhwc, x_nhwc, gamma, beta, mean, rstd, G, act, peer_ptrs, rank, dx=None, dparam=None,
                 workspace=None, stream=None, collect=True):
    """Calls gnb200_bwd_peer (collect=True: [dgamma | dbeta] summed over the ranks inside the call) or
    gnb200_bwd_peer_push (collect=False: this rank's sums are posted; peer_collect_raw sums them later).
    peer_ptrs[q] = address of rank q's exchange buffer in this process.  Returns (dx, dparam_f32[2, C])."""
    N, R, C = x_nhwc.shape
    code = DTYPE_CODES[x_nhwc.dtype]
    if dx is None:
        dx = torch.empty_like(x_nhwc)
    if dparam is None:
        dparam = torch.empty((2, C), device=x_nhwc.device, dtype=torch.float32)
    need = lib.gnb200_bwd_workspace_bytes(N, R, C, G, code)
    if workspace is None and need:
        workspace = torch.empty(need, device=x_nhwc.device, dtype=torch.uint8)
    s = torch.cuda.current_stream(x_nhwc.device).cuda_stream if stream is None else stream
    ws_args = (_ptr(workspace) if need else None, workspace.numel() if (need and workspace is not None) else 0)
    if collect:
        check(lib.gnb200_bwd_peer(_ptr(dy_nhwc), _ptr(x_nhwc), _ptr(gamma), _ptr(beta), _ptr(mean), _ptr(rstd),
                                  N, R, C, G, int(act), code, _ptr(dx), _ptr(dparam), None, None, *ws_args,
                                  _peer_table(peer_ptrs), int(rank), len(peer_ptrs), s))
    else:
        check(lib.gnb200_bwd_peer_push(_ptr(dy_nhwc), _ptr(x_nhwc), _ptr(gamma), _ptr(beta), _ptr(mean), _ptr(rstd),
                                       N, R, C, G, int(act), code, _ptr(dx), _ptr(dparam), *ws_args,
                                       _peer_table(peer_ptrs), int(rank), len(peer_ptrs), s))
    return dx, dparam


def peer_collect_raw(dparam, peer_ptrs, rank, stream=None):
    """Calls gnb200_peer_collect: dparam (float32 [2, C]) receives the sums over the ranks of the oldest push
    that has not been collected yet."""
    C = dparam.shape[1]
    s = torch.cuda.current_stream(dparam.device).cuda_stream if stream is None else stream
    check(lib.gnb200_peer_collect(_ptr(dparam), None, None, C, 0, _peer_table(peer_ptrs), int(rank), len(peer_ptrs), s))
    return dparam


def allreduce_param_grads_peer_raw(dparam, peer_ptrs, rank, stream=None):
    """Calls gnb200_allreduce_param_grads in place on a float32 [2, C] buffer."""
    C = dparam.shape[1]
    s = torch.cuda.current_stream(dparam.device).cuda_stream if stream is None else stream
    check(lib.gnb200_allreduce_param_grads(_ptr(dparam), None, None, C, 0, _peer_table(peer_ptrs), int(rank),
                                           len(peer_ptrs), s))
    return dparam


def bwd_static_scratch_raw(dy_nhwc, x_nhwc, gamma, beta, mean, rstd, G, act, dx, dparam, dgamma, dbeta, stream=None):
    """Calls gnb200_bwd_static_scratch on preallocated outputs (the entry point itself allocates nothing)."""
    N, R, C = x_nhwc.shape
    s = torch.cuda.current_stream(x_nhwc.device).cuda_stream if stream is None else stream
    check(lib.gnb200_bwd_static_scratch(_ptr(dy_nhwc), _ptr(x_nhwc), _ptr(gamma), _ptr(beta), _ptr(mean), _ptr(rstd),
                                        N, R, C, G, int(act), DTYPE_CODES[x_nhwc.dtype], _ptr(dx), _ptr(dparam),
                                        _ptr(dgamma), _ptr(dbeta), s))


def fwd_nchw_raw(x_nchw, gamma, beta, G, eps, act, stream=None):
    """Calls gnb200_fwd_nchw. x_nchw: contiguous (N, C, R) tensor. Returns (y, mean, rstd)."""
    N, C, R = x_nchw.shape
    code = DTYPE_CODES[x_nchw.dtype]
    y = torch.empty_like(x_nchw)
    mean = torch.empty((N, G), device=x_nchw.device, dtype=torch.float32)
    rstd = torch.empty((N, G), device=x_nchw.device, dtype=torch.float32)
    need = lib.gnb200_fwd_nchw_workspace_bytes(N, R, C, G, code)
    ws = torch.empty(max(need, 16), device=x_nchw.device, dtype=torch.uint8)
    s = torch.cuda.current_stream(x_nchw.device).cuda_stream if stream is None else stream
    check(lib.gnb200_fwd_nchw(_ptr(x_nchw), _ptr(gamma), _ptr(beta), N, R, C, G, float(eps), int(act), code,
                              _ptr(y), _ptr(mean), _ptr(rstd), _ptr(ws), ws.numel(), s))
    return y, mean, rstd


def bwd_nchw_raw(dy_nchw, x_nchw, gamma, beta, mean, rstd, G, act, stream=None):
    """Calls gnb200_bwd_nchw. Returns (dx, dparam_f32[2, C], dgamma, dbeta)."""
    N, C, R = x_nchw.shape
    code = DTYPE_CODES[x_nchw.dtype]
    dx = torch.empty_like(x_nchw)
    dparam = torch.empty((2, C), device=x_nchw.device, dtype=torch.float32)
    dgamma = torch.empty(C, device=x_nchw.device, dtype=x_nchw.dtype)
    dbeta = torch.empty(C, device=x_nchw.device, dtype=x_nchw.dtype)
    need = lib.gnb200_bwd_nchw_workspace_bytes(N, R, C, G, code)
    ws = torch.empty(max(need, 16), device=x_nchw.device, dtype=torch.uint8)
    s = torch.cuda.current_stream(x_nchw.device).cuda_stream if stream is None else stream
    check(lib.gnb200_bwd_nchw(_ptr(dy_nchw), _ptr(x_nchw), _ptr(gamma), _ptr(beta), _ptr(mean), _ptr(rstd),
                              N, R, C, G, int(act), code, _ptr(dx), _ptr(dparam), _ptr(dgamma), _ptr(dbeta),
                              _ptr(ws), ws.numel(), s))
    return dx, dparam, dgamma, dbeta


def fwd_f64_raw(x, gamma, beta, G, eps, act, channels_last, stream=None):
    """Calls gnb200_fwd_f64. x: contiguous (N, R, C) tensor if channels_last else contiguous (N, C, R)."""
    if channels_last:
        N, R, C = x.shape
    else:
        N, C, R = x.shape
    y = torch.empty_like(x)
    mean = torch.empty((N, G), device=x.device, dtype=torch.float64)
    rstd = torch.empty((N, G), device=x.device, dtype=torch.float64)
    s = torch.cuda.current_stream(x.device).cuda_stream if stream is None else stream
    check(lib.gnb200_fwd_f64(_ptr(x), _ptr(gamma), _ptr(beta), N, R, C, G, float(eps), int(act),
                             LAYOUT_NHWC if channels_last else LAYOUT_NCHW, _ptr(y), _ptr(mean), _ptr(rstd), s))
    return y, mean, rstd


def bwd_f64_raw(dy, x, gamma, beta, mean, rstd, G, act, channels_last, stream=None):
    """Calls gnb200_bwd_f64. Returns (dx, dgamma, dbeta), all float64."""
    if channels_last:
        N, R, C = x.shape
    else:
        N, C, R = x.shape
    dx = torch.empty_like(x)
    dgamma = torch.empty(C, device=x.device, dtype=torch.float64)
    dbeta = torch.empty(C, device=x.device, dtype=torch.float64)
    need = lib.gnb200_bwd_f64_workspace_bytes(N, R, C, G)
    ws = torch.empty(max(need, 16), device=x.device, dtype=torch.uint8)
    s = torch.cuda.current_stream(x.device).cuda_stream if stream is None else stream
    check(lib.gnb200_bwd_f64(_ptr(dy), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(mean), _ptr(rstd), N, R, C, G, int(act),
                             LAYOUT_NHWC if channels_last else LAYOUT_NCHW, _ptr(dx), _ptr(dgamma), _ptr(dbeta),
                             _ptr(ws), ws.numel(), s))
    return dx, dgamma, dbeta
