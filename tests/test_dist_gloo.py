"""World-size-2 gloo test of the batch-sharding host logic (CPU).

Each rank takes its half of the seeded global batch, obtains its local packed [dgamma | dbeta]
from the oracle (the CUDA kernels are not available on CPU; what is under test is the sharding and
the collective), all-reduces it with the package's helper and compares against the full-batch
oracle.  A second scenario checks that a channel-count mismatch raises on every rank instead of
hanging.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gn_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, scenario, ret):
    from channels_last_groupnorm_b200 import dist as gd

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, C, sp, G, act = 4, 24, (5, 3), 3, "gelu"
        x, ga, be, dy = O.make_inputs(N, C, sp, torch.float32, seed=0)
        if scenario == "sum":
            xs, dys = gd.shard_batch(x, rank, world), gd.shard_batch(dy, rank, world)
            local = O.oracle_c(xs, ga, be, dys, G, 1e-5, act)
            packed = torch.stack([local["dgamma"], local["dbeta"]]).float()
            again = packed.clone()
            gd.allreduce_param_grads(packed)
            # the ranks' agreement on C is checked once per (group, C); the second call skips it
            assert len(gd._AGREED) == 1
            gd.allreduce_param_grads(again)
            assert len(gd._AGREED) == 1 and torch.equal(again, packed)
            full = O.oracle_c(x, ga, be, dy, G, 1e-5, act)
            ok = (O.rel_err(packed[0], full["dgamma"]) < 1e-5 and O.rel_err(packed[1], full["dbeta"]) < 1e-5
                  and O.rel_err(local["dx"], gd.shard_batch(full["dx"], rank, world)) < 1e-12
                  and O.rel_err(local["y"], gd.shard_batch(full["y"], rank, world)) < 1e-12)
            ret[rank] = bool(ok)
        else:  # mismatch: rank 1 brings a different channel count
            packed = torch.zeros(2, C + rank)
            try:
                gd.allreduce_param_grads(packed)
                ret[rank] = False
            except RuntimeError as e:
                ret[rank] = "disagree" in str(e)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("scenario", ["sum", "mismatch"])
def test_sharded_param_grads_gloo(scenario):
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), scenario, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_shard_bounds():
    from channels_last_groupnorm_b200 import dist as gd

    assert [gd.shard_bounds(64, r, 8) for r in (0, 7)] == [(0, 8), (56, 64)]
    assert gd.shard_bounds(64, 0, 1) == (0, 64)
    with pytest.raises(ValueError):
        gd.shard_bounds(10, 0, 4)
    with pytest.raises(ValueError):
        gd.shard_bounds(8, 4, 4)
    with pytest.raises(ValueError):
        gd.allreduce_param_grads(torch.zeros(3, 4))
