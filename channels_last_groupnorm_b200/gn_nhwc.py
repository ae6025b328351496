"""Host-side mirror of the reference's operator interface.

`GN_NHWC` and `GN_NHWC_Func` keep the names, argument meaning and call pattern of
src/gnnhwc/custom_gn.py:29-90 of latentCall145/channels-last-groupnorm, so a model written
against `gnnhwc` only has to change its import.  What differs, on purpose:

* inputs whose channel stride is not 1 (channels-first): the reference hands them to
  `F.group_norm` + activation (custom_gn.py:75-79); here they go to native channels-first kernels
  (csrc/gn_nchw.cu) - no permute, no torch fallback - and come back in the input's layout.  CPU
  tensors raise `ValueError`.  Everything that runs goes through the sm_100a kernels.
* fp64 tensors run on a plain double-precision path (csrc/gn_f64.cu), statistics in fp64.
* backward accepts any rank >= 3 (the reference's `dy.contiguous(memory_format=channels_last)`
  only works for rank 4, custom_gn.py:44).
* parameters whose dtype differs from the input's (fp32 weight / bias with fp16 / bf16
  activations, the autocast convention; the reference raises on the mismatch,
  custom_gn.cpp:35-36) are rounded to the input dtype for the kernels; their gradients are taken
  from the fp32 sums the backward kernels write and returned in the parameters' dtype.
* the module is not excluded from dynamo (the reference decorates `forward` with
  `torch._dynamo.disable`, custom_gn.py:63): the ops have fake-tensor kernels and an autograd
  formula (`_compile.py`), so `torch.compile` traces through them.
* `process_group`: for batch-sharded data-parallel training the packed fp32 `[dgamma | dbeta]`
  buffer written by the backward kernels is summed across the ranks; forward needs no
  communication.  A `torch.distributed` process group means one NCCL all-reduce in backward; a
  `dist.PeerExchange` (ranks on the GPUs of one node) means that the backward kernels exchange
  and sum the gradients themselves through peer-mapped memory, with no library collective.
"""
import torch
import torch.nn as nn

from . import _native  # noqa: F401  (loads the libraries; raises if they are missing)
from . import dist as _dist

ACTIVATION_CODES = {
    "identity": 0,
    "relu": 1,
    "swish": 2,
    "silu": 2,
    "gelu": 3,
    "gelu_tanh": 4,
}


def _is_channels_last(t: torch.Tensor) -> bool:
    """The reference's layout rule (custom_gn.py:68): unit channel stride means channels-last."""
    return t.stride(1) == 1 or t.shape[1] == 1


def _as_nhwc_flat(t: torch.Tensor) -> torch.Tensor:
    """(N, C, *spatial) tensor with NHWC-contiguous storage -> (N, C, R) view with strides (R*C, 1, C).

    Copies only when the storage is not already NHWC-contiguous.
    """
    n, c = t.shape[0], t.shape[1]
    inner = tuple(range(2, t.ndim))
    nhwc = t.permute(0, *inner, 1)
    if not nhwc.is_contiguous():
        nhwc = nhwc.contiguous()
    return nhwc.reshape(n, -1, c).permute(0, 2, 1)


def _as_nchw_flat(t: torch.Tensor) -> torch.Tensor:
    """(N, C, *spatial) tensor -> contiguous (N, C, R) view; copies only when it is not contiguous
    (the reference calls x.contiguous() on this branch too, custom_gn.py:76)."""
    return t.contiguous().reshape(t.shape[0], t.shape[1], -1)


class GN_NHWC_Func(torch.autograd.Function):
    """apply(X, weight, bias, G, eps, activation_code[, process_group]) -> Y

    Same positional signature as the reference Function (custom_gn.py:30-31); the optional
    seventh argument is the process group whose ranks share the parameter gradients.
    """

    @staticmethod
    def forward(ctx, X, weight, bias, G, eps, activation, process_group=None):
        if isinstance(process_group, _dist.PeerExchange) and process_group.num_channels != (X.shape[1] if X.ndim > 1 else -1):
            # the exchange buffers are laid out for one channel count: a mismatch would write outside them
            raise ValueError("GN_NHWC_Func: the PeerExchange was made for %d channels, X has %d"
                             % (process_group.num_channels, (X.shape[1] if X.ndim > 1 else -1)))
        if not X.is_cuda:
            raise ValueError("GN_NHWC_Func: X must be a CUDA tensor; this package has no CPU path")
        if X.ndim < 3:
            raise ValueError("GN_NHWC_Func: X must have shape (N, C, *spatial) with at least one spatial dim")
        ctx.x_shape = X.shape
        ctx.channels_last = _is_channels_last(X)
        X_flat = _as_nhwc_flat(X) if ctx.channels_last else _as_nchw_flat(X)
        ctx.param_dtypes = (weight.dtype, bias.dtype)
        if weight.dtype != X.dtype:
            weight = weight.to(X.dtype)
        if bias.dtype != X.dtype:
            bias = bias.to(X.dtype)
        Y, means, rstds = torch.ops.gnb200.fwd(X_flat, weight, bias, int(G), float(eps), int(activation))
        ctx.save_for_backward(X_flat, weight, bias, means, rstds)
        ctx.G = int(G)
        ctx.activation = int(activation)
        ctx.process_group = process_group
        return _restore_shape(Y, ctx.x_shape, ctx.channels_last)

    @staticmethod
    def backward(ctx, dy):
        X_flat, weight, bias, means, rstds = ctx.saved_tensors
        dy_flat = _as_nhwc_flat(dy) if ctx.channels_last else _as_nchw_flat(dy)
        if dy_flat.dtype != X_flat.dtype:
            dy_flat = dy_flat.to(X_flat.dtype)
        w_dtype, b_dtype = ctx.param_dtypes
        same = w_dtype == X_flat.dtype and b_dtype == X_flat.dtype
        if ctx.process_group is None and same:
            dx, dgamma, dbeta = torch.ops.gnb200.bwd(dy_flat, X_flat, weight, bias, means, rstds, ctx.G, ctx.activation)
        elif isinstance(ctx.process_group, _dist.PeerExchange) and X_flat.dtype != torch.float64:
            # ranks on the GPUs of one node: the sum over the ranks happens inside the backward kernels
            px = ctx.process_group
            dx, dparam = torch.ops.gnb200.bwd_f32_peer(dy_flat, X_flat, weight, bias, means, rstds, ctx.G, ctx.activation,
                                                       px.peer_ptrs, px.rank)
            dgamma, dbeta = dparam[0].to(w_dtype), dparam[1].to(b_dtype)
        else:
            dx, dparam = torch.ops.gnb200.bwd_f32(dy_flat, X_flat, weight, bias, means, rstds, ctx.G, ctx.activation)
            if isinstance(ctx.process_group, _dist.PeerExchange):
                _dist.allreduce_param_grads(dparam, ctx.process_group.group)  # fp64: library collective
            elif ctx.process_group is not None:
                _dist.allreduce_param_grads(dparam, ctx.process_group)
            dgamma, dbeta = dparam[0].to(w_dtype), dparam[1].to(b_dtype)
        return _restore_shape(dx, ctx.x_shape, ctx.channels_last), dgamma, dbeta, None, None, None, None


def _restore_shape(flat: torch.Tensor, shape, channels_last=True) -> torch.Tensor:
    """(N, C, R) view -> (N, C, *spatial) view over the same storage (NHWC or NCHW)."""
    n, c = shape[0], shape[1]
    spatial = tuple(shape[2:])
    if not channels_last:
        return flat.reshape(n, c, *spatial)
    nhwc = flat.permute(0, 2, 1).reshape(n, *spatial, c)
    return nhwc.permute(0, nhwc.ndim - 1, *range(1, nhwc.ndim - 1))


class GN_NHWC(nn.GroupNorm):
    """`nn.GroupNorm` with a fused activation for channels-last inputs.

    GN_NHWC(num_groups, num_channels, activation='identity', eps=1e-5, affine=True, device=None,
    dtype=None, process_group=None).  `activation` is one of identity, relu, silu (alias swish),
    gelu, gelu_tanh; an unknown name raises KeyError like the reference (custom_gn.py:52-61).
    state_dict keys are those of `nn.GroupNorm` (`weight`, `bias`).  `process_group`: a
    torch.distributed process group or a `dist.PeerExchange` whose ranks share the parameter gradients.
    """

    def __init__(self, num_groups: int, num_channels: int, activation="identity", process_group=None, **kwargs):
        super().__init__(num_groups, num_channels, **kwargs)
        self.activation = activation
        self.act_code = ACTIVATION_CODES[activation]
        self.process_group = process_group

    def forward(self, x):
        if not x.is_cuda:
            raise ValueError("GN_NHWC: input must be a CUDA tensor; this package has no CPU path")
        if x.ndim < 3 or x.shape[1] != self.num_channels:
            raise ValueError("GN_NHWC: expected input of shape (N, %d, *spatial), got %s"
                             % (self.num_channels, tuple(x.shape)))
        if self.affine:
            w, b = self.weight, self.bias
        else:
            w = torch.ones((self.num_channels,), device=x.device, dtype=x.dtype)
            b = torch.zeros((self.num_channels,), device=x.device, dtype=x.dtype)
        return GN_NHWC_Func.apply(x, w, b, self.num_groups, self.eps, self.act_code, self.process_group)

    def extra_repr(self):
        return "{num_groups}, {num_channels}, eps={eps}, affine={affine}, activation={activation}".format(
            **self.__dict__)
