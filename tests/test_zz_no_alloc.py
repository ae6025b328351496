"""GPU test of gnb200_bwd_static_scratch, the backward entry point for callers that are not allowed
to allocate device memory (plugins of a runtime that owns every buffer, real-time loops, code under
a stream capture, thin FFI bindings): it must give the same gradients as gnb200_bwd, which gets its
scratch from the caller, call after call, because all calls share one built-in scratch array.

Collected last on purpose: a run that stops at the first failure has then already run every other test.
"""
import pytest
import torch

from oracle import gn_oracle as O

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _flat(t):
    n, c = t.shape[0], t.shape[1]
    return t.permute(0, *range(2, t.ndim), 1).reshape(n, -1, c)


@pytest.mark.parametrize("shape,dt,act,force", [
    ((4, 256, (16, 16), 32), "bfloat16", "gelu", ""),          # fused plan: per-sample channel sums in scratch
    ((2, 64, (24, 24), 8), "float32", "silu", "twopass"),      # multi-kernel plan: tile partials in scratch
])
def test_static_scratch_backward_matches_workspace_backward(shape, dt, act, force, monkeypatch):
    assert torch.cuda.is_available()
    from channels_last_groupnorm_b200 import _native as nt

    if force:
        monkeypatch.setenv("GNB200_FORCE_PATH", force)
    N, C, sp, G = shape
    code = O.ACT_CODES[act]
    tol = O.TOLERANCE[DT[dt]]
    for call in range(2):  # two calls in a row, different inputs: the array keeps the first call's contents
        x, ga, be, dy = O.make_inputs(N, C, sp, DT[dt], seed=10 + call)
        xd, dyd, gd, bd = _flat(x.cuda()), _flat(dy.cuda()), ga.cuda(), be.cuda()
        _, mean, rstd = nt.fwd_raw(xd, gd, bd, G, 1e-5, code)
        want_dx, want_dparam, want_dg, want_db = nt.bwd_raw(dyd, xd, gd, bd, mean, rstd, G, code)
        dx = torch.empty_like(xd)
        dparam = torch.empty((2, C), device="cuda", dtype=torch.float32)
        dg = torch.empty(C, device="cuda", dtype=DT[dt])
        db = torch.empty(C, device="cuda", dtype=DT[dt])
        nt.bwd_static_scratch_raw(dyd, xd, gd, bd, mean, rstd, G, code, dx, dparam, dg, db)
        torch.cuda.synchronize()
        for got, want in ((dx, want_dx), (dparam, want_dparam), (dg, want_dg), (db, want_db)):
            assert O.rel_err(got, want) <= tol
        # and against the CPU oracle, so that both entry points cannot be wrong together
        ref = O.oracle_c(x, ga, be, dy, G, 1e-5, act)
        assert O.rel_err(dx.reshape(N, *sp, C).permute(0, 3, 1, 2), ref["dx"]) <= tol
        assert O.rel_err(dparam[0], ref["dgamma"]) <= tol and O.rel_err(dparam[1], ref["dbeta"]) <= tol


def test_static_scratch_rejects_problems_beyond_its_array():
    from channels_last_groupnorm_b200 import _native as nt

    N, R, C, G = 8192, 64, 256, 32  # the plan keeps 2 * N * C floats = 16 MiB of channel sums
    assert nt.lib.gnb200_bwd_workspace_bytes(N, R, C, G, 2) > nt.STATIC_SCRATCH_BYTES
    # real buffers of the stated sizes (268 MB per tensor): the call must refuse before it launches,
    # but if that check ever regressed the kernels would still only touch memory they may touch
    x = torch.zeros((N, R, C), dtype=torch.bfloat16, device="cuda")
    dy = torch.zeros_like(x)
    dx = torch.empty_like(x)
    ga = torch.ones(C, dtype=torch.bfloat16, device="cuda")
    be = torch.zeros(C, dtype=torch.bfloat16, device="cuda")
    mean = torch.zeros((N, G), device="cuda")
    rstd = torch.ones((N, G), device="cuda")
    dparam = torch.empty((2, C), device="cuda")
    rc = nt.lib.gnb200_bwd_static_scratch(dy.data_ptr(), x.data_ptr(), ga.data_ptr(), be.data_ptr(), mean.data_ptr(),
                                          rstd.data_ptr(), N, R, C, G, 0, 2, dx.data_ptr(), dparam.data_ptr(), None,
                                          None, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == -2
    msg = nt.lib.gnb200_last_error().decode()
    assert "scratch" in msg and str(nt.STATIC_SCRATCH_BYTES) in msg
