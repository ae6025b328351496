"""Fake-tensor kernels and the autograd formula of torch.ops.gnb200.*.

The reference registers its two ops without a Meta kernel or an autograd formula and disables
dynamo on the module (src/gnnhwc/custom_gn.py:63, its README lists torch.compile support as to
do).  With the registrations below the ops can be traced: `torch.compile` sees the output shapes
and strides without running a kernel, and `torch.ops.gnb200.fwd` is differentiable on its own
(its backward is `torch.ops.gnb200.bwd`).
"""
import torch


def _like(X):
    """Same sizes and storage order as X (channels-last or channels-first)."""
    n, c, r = X.shape
    if X.stride(1) == 1 or c == 1:
        return X.new_empty((n, r, c)).permute(0, 2, 1)
    return X.new_empty((n, c, r))


def _stats_dtype(X):
    return torch.float64 if X.dtype == torch.float64 else torch.float32


@torch.library.register_fake("gnb200::fwd")
def _fwd_fake(X, weight, bias, G, eps, act):
    n = X.shape[0]
    stats = X.new_empty((n, G), dtype=_stats_dtype(X))
    return _like(X), stats, torch.empty_like(stats)


@torch.library.register_fake("gnb200::bwd")
def _bwd_fake(dy, X, weight, bias, means, rstds, G, act):
    return _like(X), torch.empty_like(weight), torch.empty_like(bias)


@torch.library.register_fake("gnb200::bwd_f32")
def _bwd_f32_fake(dy, X, weight, bias, means, rstds, G, act):
    return _like(X), X.new_empty((2, X.shape[1]), dtype=_stats_dtype(X))


@torch.library.register_fake("gnb200::bwd_f32_peer")
def _bwd_f32_peer_fake(dy, X, weight, bias, means, rstds, G, act, peer_ptrs, rank):
    return _like(X), X.new_empty((2, X.shape[1]), dtype=_stats_dtype(X))


def _fwd_setup_context(ctx, inputs, output):
    X, weight, bias, G, eps, act = inputs
    _, means, rstds = output
    ctx.save_for_backward(X, weight, bias, means, rstds)
    ctx.G = G
    ctx.act = act


def _fwd_backward(ctx, dY, dmeans, drstds):
    X, weight, bias, means, rstds = ctx.saved_tensors
    # the kernels want dy in the storage order of X
    if X.stride(1) == 1 or X.shape[1] == 1:
        dy = dY.permute(0, 2, 1).contiguous().permute(0, 2, 1)
    else:
        dy = dY.contiguous()
    dx, dgamma, dbeta = torch.ops.gnb200.bwd(dy, X, weight, bias, means, rstds, ctx.G, ctx.act)
    return dx, dgamma, dbeta, None, None, None


torch.library.register_autograd("gnb200::fwd", _fwd_backward, setup_context=_fwd_setup_context)
