"""In-kernel all-reduce of [dgamma | dbeta] over the GPUs of one node (gnb200_bwd_peer, gnb200_bwd_peer_push +
gnb200_peer_collect, gnb200_allreduce_param_grads, dist.PeerExchange), one process per GPU.

Kernels that wait for one another must not share a GPU, so this test needs at least two devices and is
skipped otherwise (bench.py's parity_check covers the same ground whenever it runs on several GPUs).  Each
rank takes its shard of a seeded global batch; the peer-summed gradients must equal the NCCL-summed ones
and the full-batch oracle within tolerance, be bit-identical on all ranks and between the three ways of
calling the exchange, for a channel count that fills whole 32-channel blocks and one that does not, and
through the module with process_group=PeerExchange.
"""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    import datetime

    # a short timeout: if a rank fails, the others' next collective ends with an error instead of hanging
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    try:
        import channels_last_groupnorm_b200 as pkg
        from channels_last_groupnorm_b200 import _native as nt
        from channels_last_groupnorm_b200 import dist as gd
        from oracle import gn_oracle as O

        problems = []
        for (N, C, sp, G, act, dtype) in [(2 * world, 64, (6, 10), 8, "silu", torch.float16),
                                          (world, 40, (7, 5), 8, "gelu", torch.float32),
                                          (world, 320, (8, 8), 32, "silu", torch.bfloat16)]:
            x, ga, be, dy = O.make_inputs(N, C, sp, dtype, seed=3)
            want = O.oracle_c(x, ga, be, dy, G, 1e-5, act, threads=2)
            px = gd.PeerExchange(C)
            code = O.ACT_CODES[act]
            R = sp[0] * sp[1]
            flat = lambda t: t.cuda().permute(0, 2, 3, 1).reshape(t.shape[0], R, C).contiguous()  # noqa: E731
            xs, dys = flat(gd.shard_batch(x, rank, world)), flat(gd.shard_batch(dy, rank, world))
            gd_, bd_ = ga.cuda(), be.cuda()
            _, mean, rstd = nt.fwd_raw(xs, gd_, bd_, G, 1e-5, code)
            _, local, _, _ = nt.bwd_raw(dys, xs, gd_, bd_, mean, rstd, G, code)
            ref = local.clone()
            dist.all_reduce(ref)
            tol = O.TOLERANCE[dtype]
            full = torch.stack([want["dgamma"], want["dbeta"]]).float().cuda()
            assert O.rel_err(ref, full) <= tol
            # one call
            _, fused = nt.bwd_peer_raw(dys, xs, gd_, bd_, mean, rstd, G, code, px.peer_ptrs, px.rank)
            assert O.rel_err(fused, ref) <= 1e-6 and O.rel_err(fused, full) <= tol
            first = fused.clone()
            dist.broadcast(first, src=0)
            assert torch.equal(first, fused), "ranks differ"
            # the exchange alone, on the sums of the plain backward (whose kernel adds the samples with 32 row
            # lanes where the exchanging one uses 8: the same numbers up to the order of fp32 additions)
            assert O.rel_err(px.allreduce_(local.clone()), fused) <= 1e-6
            # push and collect apart, two pushes outstanding, three rounds (slot reuse and acknowledgements)
            for _ in range(3):
                for _ in range(2):
                    _, loc = nt.bwd_peer_raw(dys, xs, gd_, bd_, mean, rstd, G, code, px.peer_ptrs, px.rank, collect=False)
                    assert O.rel_err(loc, local) <= 1e-6
                for _ in range(2):
                    assert torch.equal(px.collect_(torch.empty_like(fused)), fused)
            # the module
            m = pkg.GN_NHWC(G, C, activation=act, eps=1e-5, process_group=px).cuda().to(dtype)
            with torch.no_grad():
                m.weight.copy_(ga)
                m.bias.copy_(be)
            xin = gd.shard_batch(x, rank, world).cuda().to(memory_format=torch.channels_last).requires_grad_(True)
            m(xin).backward(gd.shard_batch(dy, rank, world).cuda().to(memory_format=torch.channels_last))
            assert O.rel_err(m.weight.grad, want["dgamma"]) <= tol and O.rel_err(m.bias.grad, want["dbeta"]) <= tol
            problems.append(px)  # keep the buffers alive until every rank is through
        torch.cuda.synchronize()
        assert nt.wait_timeouts() == 0
        dist.barrier()
        ret[rank] = "ok"
    except Exception as exc:  # pragma: no cover - reported to the parent
        import traceback

        ret[rank] = "".join(traceback.format_exception(type(exc), exc, exc.__traceback__))[-2000:]
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs one GPU per rank (kernels that wait for one another must not share a GPU)")
def test_peer_exchange_matches_nccl_and_oracle():
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(ret.get(r) == "ok" for r in range(world)), dict(ret)
