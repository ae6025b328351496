"""Batch-sharded data parallelism for GroupNorm.

GroupNorm statistics are per (sample, group), so splitting the batch dimension N over ranks needs
no communication in forward, and in backward only the parameter gradients sum over samples:
one all-reduce of the packed fp32 `[dgamma | dbeta]` buffer (2 * C floats).  The reference has no
multi-GPU code; this module is the host logic of that extension and is backend-agnostic
(NCCL on GPUs, gloo in the CPU tests).
"""
import os

import torch
import torch.distributed as dist


def shard_bounds(n_total: int, rank: int, world_size: int):
    """Half-open sample range [lo, hi) of `rank` when n_total samples are split evenly.

    The split must be exact: a ragged split would give ranks different amounts of work and the
    benchmark configuration (N = 64 over 1/2/4/8 ranks) never needs it.
    """
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError("shard_bounds: rank %d is not in [0, %d)" % (rank, world_size))
    if n_total % world_size != 0:
        raise ValueError("shard_bounds: batch of %d samples does not split evenly over %d ranks"
                         % (n_total, world_size))
    per = n_total // world_size
    return rank * per, (rank + 1) * per


def shard_batch(t: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """This rank's samples of a global (N, ...) tensor (a view, no copy)."""
    lo, hi = shard_bounds(t.shape[0], rank, world_size)
    return t[lo:hi]


# (process group, num_channels) pairs whose ranks have been found to agree
_AGREED = set()


def _check_channels_once(num_channels: int, group, world: int):
    """Host-side check that every rank of `group` brings the same number of channels, done the
    first time a (group, num_channels) pair is seen: a mismatch raises on all ranks instead of
    hanging or corrupting the reduction.  Later calls with the same pair skip the (pickled,
    host-synchronising) exchange; the all-reduce itself costs microseconds."""
    key = (id(group) if group is not None else None, int(num_channels))
    if key in _AGREED:
        return
    sizes = [None] * world
    dist.all_gather_object(sizes, int(num_channels), group=group)
    if len(set(sizes)) != 1:
        raise RuntimeError("allreduce_param_grads: ranks disagree on num_channels: %s" % sizes)
    _AGREED.add(key)


def allreduce_param_grads(dparam_f32: torch.Tensor, group=None) -> torch.Tensor:
    """Sums the packed fp32 [2, C] parameter-gradient buffer over the ranks of `group`, in place.

    The first call for a (group, C) pair checks on the host that all ranks agree on C before the
    collective is issued.
    """
    if dparam_f32.dtype not in (torch.float32, torch.float64) or dparam_f32.ndim != 2 or dparam_f32.shape[0] != 2:
        raise ValueError("allreduce_param_grads: expected a float32 (float64 for fp64 inputs) [2, C] tensor, got %s %s"
                         % (dparam_f32.dtype, tuple(dparam_f32.shape)))
    if not dist.is_available() or not dist.is_initialized():
        return dparam_f32
    world = dist.get_world_size(group)
    if world == 1:
        return dparam_f32
    _check_channels_once(dparam_f32.shape[1], group, world)
    dist.all_reduce(dparam_f32, op=dist.ReduceOp.SUM, group=group)
    return dparam_f32


class PeerExchange:
    """Exchange buffers for the in-kernel all-reduce of [dgamma | dbeta] over the GPUs of ONE node
    (`gnb200_bwd_peer`): every rank of `group` allocates a zeroed buffer of
    `gnb200_peer_exchange_bytes(num_channels, world)` bytes in symmetric memory and maps the other
    ranks' buffers, so that the backward kernels can store into them directly over NVLink.

    Collective: every rank of the group must construct it at the same point.  One object belongs to
    one (group, num_channels) pair and the ranks must make the same sequence of backward calls with
    it.  The kernels wait about a second for one another; ranks that run further apart than that
    should use the NCCL path (`allreduce_param_grads`).  Only plain peer stores and loads are used:
    the buffers are never bound to a multicast object.
    """

    def __init__(self, num_channels: int, group=None, device=None):
        if not dist.is_available() or not dist.is_initialized():
            raise RuntimeError("PeerExchange: torch.distributed is not initialised")
        # this package only uses peer pointers; keep the allocator from creating multicast bindings
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        from . import _native

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.num_channels = int(num_channels)
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        _check_channels_once(self.num_channels, self.group, self.world)
        nbytes = _native.peer_exchange_bytes(self.num_channels, self.world)
        if nbytes == 0:
            raise ValueError("PeerExchange: %d channels over %d ranks is outside the supported range (1 .. 16 ranks)"
                             % (self.num_channels, self.world))
        self.buffer = symm_mem.empty(nbytes // 4, dtype=torch.float32, device=device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.peer_ptrs) != self.world or self.peer_ptrs[self.rank] != self.buffer.data_ptr():
            raise RuntimeError("PeerExchange: the symmetric-memory handle does not describe this group")
        # every buffer is zero before any rank's kernel can store into it
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def _check(self, dparam_f32, who):
        if dparam_f32.dtype != torch.float32 or tuple(dparam_f32.shape) != (2, self.num_channels):
            raise ValueError("PeerExchange.%s: expected a float32 [2, %d] tensor, got %s %s"
                             % (who, self.num_channels, dparam_f32.dtype, tuple(dparam_f32.shape)))

    def allreduce_(self, dparam_f32: torch.Tensor) -> torch.Tensor:
        """In-place sum of a float32 [2, C] buffer over the ranks (`gnb200_allreduce_param_grads`)."""
        from . import _native

        self._check(dparam_f32, "allreduce_")
        return _native.allreduce_param_grads_peer_raw(dparam_f32, self.peer_ptrs, self.rank)

    def collect_(self, dparam_f32: torch.Tensor) -> torch.Tensor:
        """Writes the sums over the ranks of the oldest push that has not been collected yet
        (`gnb200_bwd_peer_push` ... `gnb200_peer_collect`) into a float32 [2, C] buffer."""
        from . import _native

        self._check(dparam_f32, "collect_")
        return _native.peer_collect_raw(dparam_f32, self.peer_ptrs, self.rank)
