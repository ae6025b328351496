"""GPU parity tests (B200): the CUDA path, called through the C ABI, against the CPU oracles.

Tolerances (max-abs error relative to max(1, max|oracle|)): 1e-5 for fp32 tensors, 1e-2 for
fp16 / bf16 tensors, on y, dx, dgamma and dbeta.
"""
import glob
import os

import pytest
import torch

from oracle import gn_oracle as O

from .cases import CFG1, CFG2, CFG3, CFG4, CFG5, REFERENCE_CUSTOM, REFERENCE_TRAILING

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REF_LIB = os.path.join(os.path.dirname(GOLDEN_DIR), "..", "oracle", "_ref", "gn_op.so")


@pytest.fixture(scope="module")
def nt():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from channels_last_groupnorm_b200 import _native

    return _native


def _flat(t):
    """(N, C, *spatial) channels-last tensor -> contiguous (N, R, C) view of the same storage."""
    n, c = t.shape[0], t.shape[1]
    nhwc = t.permute(0, *range(2, t.ndim), 1)
    assert nhwc.is_contiguous()
    return nhwc.reshape(n, -1, c)


def _unflat(a, shape):
    n, c = shape[0], shape[1]
    return a.reshape(n, *shape[2:], c).permute(0, len(shape) - 1, *range(1, len(shape) - 1))


def run_cabi(nt, x, ga, be, dy, G, eps, act):
    """Forward + backward through gnb200_fwd / gnb200_bwd; returns logical-shape tensors."""
    code = O.ACT_CODES[act]
    xd, gd, bd = x.cuda(), ga.cuda(), be.cuda()
    y, mean, rstd = nt.fwd_raw(_flat(xd), gd, bd, G, eps, code)
    out = {"y": _unflat(y, x.shape), "mean": mean, "rstd": rstd}
    if dy is not None:
        dx, dparam, dgamma, dbeta = nt.bwd_raw(_flat(dy.cuda()), _flat(xd), gd, bd, mean, rstd, G, code)
        out.update(dx=_unflat(dx, x.shape), dgamma=dgamma, dbeta=dbeta, dparam=dparam)
    torch.cuda.synchronize()
    return out


def check_against(out, want, dtype, keys=("y", "dx", "dgamma", "dbeta"), scale=1.0):
    tol = O.TOLERANCE[dtype] * scale
    errs = {k: O.rel_err(out[k], want[k]) for k in keys if k in want and k in out}
    bad = {k: e for k, e in errs.items() if not e <= tol}
    assert not bad, "error above %.1e: %s (all: %s)" % (tol, bad, errs)
    return errs


def _case_inputs(case, seed=0):
    N, C, sp, G, eps, act, dt, dist, scale = case
    x, ga, be, dy = O.make_inputs(N, C, sp, DT[dt], seed=seed, x_dist=dist, x_scale=scale)
    return x, ga, be, dy, G, eps, act, DT[dt]


def _id(case):
    N, C, sp, G, eps, act, dt = case[:7]
    return "%s-%s-%dx%dx%s-g%d" % (dt, act, N, C, "x".join(map(str, sp)), G)


# ------------------------------------------------------------------------------------------------
# benchmark configurations at sizes the CPU oracle finishes in seconds
# ------------------------------------------------------------------------------------------------
SMALL_CASES = [CFG1] + CFG2 + CFG3[:1] + CFG4[:1] + CFG5


@pytest.mark.parametrize("path", ["auto", "twopass", "wave"])
@pytest.mark.parametrize("case", SMALL_CASES, ids=_id)
def test_baseline_configs_against_oracle(nt, case, path, monkeypatch):
    if path != "auto":  # force the multi-kernel plan / the wave plan (where the shape allows it)
        monkeypatch.setenv("GNB200_FORCE_PATH", path)
    x, ga, be, dy, G, eps, act, dtype = _case_inputs(case)
    out = run_cabi(nt, x, ga, be, dy, G, eps, act)
    big = x.numel() > 2_000_000
    want = O.oracle_torch(x, ga, be, dy, G, eps, act) if big else O.oracle_c(x, ga, be, dy, G, eps, act, threads=4)
    check_against(out, want, dtype)
    if not big:  # saved statistics are part of the contract between fwd and bwd
        assert O.rel_err(out["mean"], want["mean"]) < 1e-5
        assert O.rel_err(out["rstd"] / want["rstd"].cuda().float(), torch.ones_like(want["rstd"])) < 1e-5
    # packed fp32 gradient buffer == typed outputs before rounding
    assert O.rel_err(out["dparam"][0], want["dgamma"]) <= O.TOLERANCE[dtype]
    assert O.rel_err(out["dparam"][1], want["dbeta"]) <= O.TOLERANCE[dtype]


@pytest.mark.parametrize("path", ["auto", "twopass"])
def test_chained_launches_change_no_bit(nt, path, monkeypatch):
    """Kernels after the first of a call are launched as programmatic dependents of their predecessor
    (they may become resident early and wait for it on the device).  With GNB200_CHAIN=0 they are
    launched in plain stream order; the results must be the same bits, also when calls follow each
    other back to back."""
    if path != "auto":
        monkeypatch.setenv("GNB200_FORCE_PATH", path)
    x, ga, be, dy, G, eps, act, dtype = _case_inputs(CFG4[0])
    outs = []
    for chain in ("1", "0"):
        monkeypatch.setenv("GNB200_CHAIN", chain)
        for _ in range(3):
            out = run_cabi(nt, x, ga, be, dy, G, eps, act)
        outs.append(out)
    for k in ("y", "dx", "mean", "rstd", "dparam", "dgamma", "dbeta"):
        assert torch.equal(outs[0][k], outs[1][k]), k


def test_peer_entry_points_with_one_rank_are_the_plain_backward(nt):
    """gnb200_bwd_peer / gnb200_bwd_peer_push / gnb200_peer_collect / gnb200_allreduce_param_grads with a single
    rank exchange nothing: same bits as gnb200_bwd, buffers untouched by the exchange calls.  (With several
    ranks the exchange is checked on the hardware by bench.py's parity_check, which needs one GPU per rank.)"""
    x, ga, be, dy, G, eps, act, dtype = _case_inputs(CFG4[0])
    code = O.ACT_CODES[act]
    xd, gd, bd, dyd = _flat(x.cuda()), ga.cuda(), be.cuda(), _flat(dy.cuda())
    y, mean, rstd = nt.fwd_raw(xd, gd, bd, G, eps, code)
    dx, dparam, _, _ = nt.bwd_raw(dyd, xd, gd, bd, mean, rstd, G, code)
    buf = torch.zeros(nt.peer_exchange_bytes(x.shape[1], 1) // 4, dtype=torch.float32, device="cuda")
    ptrs = [buf.data_ptr()]
    for collect in (True, False):
        dx2, dparam2 = nt.bwd_peer_raw(dyd, xd, gd, bd, mean, rstd, G, code, ptrs, 0, collect=collect)
        assert torch.equal(dx, dx2) and torch.equal(dparam, dparam2)
    keep = dparam.clone()
    nt.peer_collect_raw(dparam, ptrs, 0)
    nt.allreduce_param_grads_peer_raw(dparam, ptrs, 0)
    torch.cuda.synchronize()
    assert torch.equal(dparam, keep) and int(buf.abs().sum().item()) == 0
    assert nt.wait_timeouts() == 0


@pytest.mark.parametrize("act", O.ACT_NAMES)
@pytest.mark.parametrize("dt", ["float32", "float16", "bfloat16"])
def test_every_activation_and_dtype(nt, act, dt):
    x, ga, be, dy = O.make_inputs(3, 48, (9, 11), DT[dt], seed=2, x_dist="uniform3")
    out = run_cabi(nt, x, ga, be, dy, 6, 1e-5, act)
    check_against(out, O.oracle_c(x, ga, be, dy, 6, 1e-5, act), DT[dt])


@pytest.mark.parametrize("shape", REFERENCE_CUSTOM, ids=lambda s: "%dx%dx%s-g%d" % (s[0], s[1], "x".join(map(str, s[2])), s[3]))
@pytest.mark.parametrize("dt", ["float32", "bfloat16"])
def test_reference_custom_shapes(nt, shape, dt):
    N, C, sp, G = shape
    x, ga, be, dy = O.make_inputs(N, C, sp, DT[dt], seed=1)
    out = run_cabi(nt, x, ga, be, dy, G, 1e-5, "identity")
    check_against(out, O.oracle_c(x, ga, be, dy, G, 1e-5, "identity", threads=4), DT[dt])


# ------------------------------------------------------------------------------------------------
# full-size configurations: checked on the device against torch's fp64 GroupNorm (CUDA), which is
# itself checked against the CPU oracle at the small sizes above
# ------------------------------------------------------------------------------------------------
def _cuda_fp64_reference(x, ga, be, dy, G, eps, act):
    xs = x.double().requires_grad_(True)
    g = ga.double().requires_grad_(True)
    b = be.double().requires_grad_(True)
    y = O.torch_activation(act)(torch.nn.functional.group_norm(xs, G, g, b, eps))
    dx, dg, db = torch.autograd.grad(y, (xs, g, b), dy.double())
    return {"y": y.detach(), "dx": dx, "dgamma": dg, "dbeta": db}


def test_cuda_fp64_reference_agrees_with_cpu_oracle(nt):
    x, ga, be, dy, G, eps, act, dtype = _case_inputs(CFG5[0])
    a = _cuda_fp64_reference(x.cuda(), ga.cuda(), be.cuda(), dy.cuda(), G, eps, act)
    b = O.oracle_c(x, ga, be, dy, G, eps, act)
    for k in ("y", "dx", "dgamma", "dbeta"):
        assert O.rel_err(a[k], b[k]) < 1e-10


# (configuration, forced plan): every full-size configuration with the planner's choice, and the 1024-px
# VAE shapes with the smallest and the largest slab also with each of the multi-pass plans forced
FULL_SIZE = [(c, "auto") for c in CFG3[1:] + CFG4[1:]] + [(c, p) for c in (CFG3[1], CFG3[3]) for p in ("wave", "twopass")]


@pytest.mark.parametrize("case,path", FULL_SIZE, ids=lambda v: v if isinstance(v, str) else _id(v))
def test_full_size_configs_on_device(nt, case, path, monkeypatch):
    if path != "auto":
        monkeypatch.setenv("GNB200_FORCE_PATH", path)
    N, C, sp, G, eps, act, dt, dist, scale = case
    gen = torch.Generator(device="cuda").manual_seed(0)
    shape = (N, *sp, C)
    x = (torch.randn(shape, device="cuda", generator=gen) * scale).to(DT[dt]).permute(0, 3, 1, 2)
    dy = torch.randn(shape, device="cuda", generator=gen).to(DT[dt]).permute(0, 3, 1, 2)
    ga = (torch.rand(C, device="cuda", generator=gen) + 0.5).to(DT[dt])
    be = (torch.randn(C, device="cuda", generator=gen) * 0.1).to(DT[dt])
    out = run_cabi(nt, x, ga, be, dy, G, eps, act)
    want = _cuda_fp64_reference(x, ga, be, dy, G, eps, act)
    check_against(out, want, DT[dt])
    # size-independent property: with identity activation and gamma=1, beta=0 every
    # (sample, group) slab of y has mean 0 and variance 1
    one, zero = torch.ones_like(ga), torch.zeros_like(be)
    y = run_cabi(nt, x, one, zero, None, G, eps, "identity")["y"]
    slabs = y.float().reshape(N, G, C // G, -1)
    assert slabs.mean((2, 3)).abs().max() < 2e-3
    assert (slabs.var((2, 3), correction=0) - 1).abs().max() < 5e-3


# ------------------------------------------------------------------------------------------------
# robustness of the statistics and of the plumbing
# ------------------------------------------------------------------------------------------------
def test_large_mean_small_variance_fp32(nt):
    g = torch.Generator().manual_seed(3)
    x = (300.0 + 0.05 * torch.randn(2, 16, 16, 32, generator=g)).permute(0, 3, 1, 2)
    ga, be = torch.ones(32), torch.zeros(32)
    dy = torch.randn(2, 16, 16, 32, generator=g).permute(0, 3, 1, 2)
    for path in ("auto", "twopass"):
        if path == "twopass":
            os.environ["GNB200_FORCE_PATH"] = "twopass"
        try:
            out = run_cabi(nt, x, ga, be, dy, 4, 1e-5, "identity")
        finally:
            os.environ.pop("GNB200_FORCE_PATH", None)
        want = O.oracle_c(x, ga, be, dy, 4, 1e-5, "identity")
        # inputs near 300 carry an fp32 rounding of 3e-5 against a spread of 0.05: allow 1e-3
        check_against(out, want, torch.float32, scale=100.0)


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
def test_large_mean_small_variance_16bit(nt, dt):
    # 16-bit statistics use shifted sums (s = sum(x - K), q = sum((x - K)^2) about the thread's
    # first row): values quantised around a large mean must not cancel.  The oracle sees the
    # same quantised inputs.
    g = torch.Generator().manual_seed(5)
    base = 60.0 if dt == "float16" else 100.0
    x = (base + 2.0 * torch.randn(3, 24, 24, 64, generator=g)).to(DT[dt]).permute(0, 3, 1, 2)
    ga = (torch.rand(64, generator=g) + 0.5).to(DT[dt])
    be = (0.1 * torch.randn(64, generator=g)).to(DT[dt])
    dy = torch.randn(3, 24, 24, 64, generator=g).to(DT[dt]).permute(0, 3, 1, 2)
    want = O.oracle_c(x, ga, be, dy, 8, 1e-5, "silu")
    for path in ("auto", "twopass"):
        if path == "twopass":
            os.environ["GNB200_FORCE_PATH"] = "twopass"
        try:
            out = run_cabi(nt, x, ga, be, dy, 8, 1e-5, "silu")
        finally:
            os.environ.pop("GNB200_FORCE_PATH", None)
        check_against(out, want, DT[dt])
        # the statistics themselves: mean to 1e-3 relative, rstd to 2e-3 relative
        xf = x.double().reshape(3, 8, 8, -1)
        mu = xf.mean((2, 3))
        rs = 1.0 / torch.sqrt(xf.var((2, 3), correction=0) + 1e-5)
        assert ((out["mean"].cpu().double() - mu).abs() / mu.abs()).max() < 1e-3
        assert ((out["rstd"].cpu().double() - rs).abs() / rs).max() < 2e-3


@pytest.mark.parametrize("case", [
    # (N, C, spatial, G, dtype, act): more (sample, column block) items than resident clusters, so
    # every cluster of the fused forward kernel walks through several items and refills its tile
    (96, 320, (32, 32), 32, "float16", "silu"),      # D = 10: vectors straddle groups
    (40, 256, (64, 64), 32, "bfloat16", "gelu"),     # items not a multiple of the cluster count
    (24, 128, (96, 96), 16, "float32", "relu"),      # fp32 (Welford) statistics
    (150, 64, (48, 48), 64, "float16", "identity"),  # instance-norm-like: D = 1, scalar groups
], ids=lambda c: "%dx%dx%s-g%d-%s-%s" % (c[0], c[1], "x".join(map(str, c[2])), c[3], c[4], c[5]))
def test_persistent_clusters_over_many_items(nt, case):
    N, C, sp, G, dt, act = case
    gen = torch.Generator(device="cuda").manual_seed(1)
    shape = (N, *sp, C)
    # a different offset per sample and channel, so that an item computed with another item's
    # statistics or rows cannot pass
    off = torch.randn(N, 1, 1, C, device="cuda", generator=gen) * 2.0
    x = (torch.randn(shape, device="cuda", generator=gen) + off).to(DT[dt]).permute(0, 3, 1, 2)
    dy = torch.randn(shape, device="cuda", generator=gen).to(DT[dt]).permute(0, 3, 1, 2)
    ga = (torch.rand(C, device="cuda", generator=gen) + 0.5).to(DT[dt])
    be = (torch.randn(C, device="cuda", generator=gen) * 0.1).to(DT[dt])
    assert " fused " in nt.describe_plan(N, sp[0] * sp[1], C, G, DT[dt], 0)
    out = run_cabi(nt, x, ga, be, dy, G, 1e-5, act)
    want = _cuda_fp64_reference(x, ga, be, dy, G, 1e-5, act)
    check_against(out, want, DT[dt])
    again = run_cabi(nt, x, ga, be, dy, G, 1e-5, act)
    for k in ("y", "dx", "dparam", "mean", "rstd"):
        assert torch.equal(out[k], again[k]), k


def test_dependent_calls_back_to_back(nt):
    # A chain in which each call consumes the previous call's output (forward feeding forward, dx
    # feeding the next backward), issued without any host synchronisation: the persistent forward
    # kernel, the backward kernel and the parameter-gradient kernel follow each other on the stream.
    # The chain must give bit-identical results when run twice and when replayed from a CUDA graph.
    N, C, sp, G = 8, 128, (24, 24), 16
    x, ga, be, dy = O.make_inputs(N, C, sp, torch.bfloat16, seed=21)
    xf, dyf, gad, bed = _flat(x.cuda()), _flat(dy.cuda()), ga.cuda(), be.cuda()

    def chain():
        cur, grads = xf, dyf
        for _ in range(6):
            y, mean, rstd = nt.fwd_raw(cur, gad, bed, G, 1e-5, 2)
            dx, dparam, _, _ = nt.bwd_raw(grads, cur, gad, bed, mean, rstd, G, 2)
            cur, grads = y, dx
        return cur.clone(), grads.clone(), dparam.clone()

    want = chain()
    torch.cuda.synchronize()
    got = chain()
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain()  # warm-up on the capture stream
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            captured = chain()
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(captured, want):
        assert torch.equal(a, b)


def test_no_exchange_wait_gave_up(nt):
    # the bounded waits of the cluster exchange count the times they gave up; any count means that
    # a kernel carried on with meaningless statistics
    x, ga, be, dy, G, eps, act, dtype = _case_inputs(CFG4[0])
    run_cabi(nt, x, ga, be, dy, G, eps, act)
    assert nt.wait_timeouts() == 0


def test_exchange_wait_that_runs_out_is_reported_and_recoverable(nt):
    # The give-up path of the bounded waits, provoked on the host side only: the self-test entry
    # point runs the fused forward with a limit of about a millisecond while one rank of every
    # cluster withholds its contribution.  Every CTA still pushes before it waits and exits after
    # its wait ran out: nothing hangs or faults.
    N, C, sp, G = 2, 64, (64, 64), 8
    assert " fused " in nt.describe_plan(N, sp[0] * sp[1], C, G, torch.bfloat16, 0)
    x, ga, be, dy = O.make_inputs(N, C, sp, torch.bfloat16, seed=31)
    xf, gd, bd = _flat(x.cuda()), ga.cuda(), be.cuda()
    y = torch.zeros_like(xf)
    mean = torch.zeros((N, G), device="cuda")
    rstd = torch.zeros((N, G), device="cuda")
    assert nt.wait_timeouts() == 0
    try:
        nt.check(nt.lib.gnb200_selftest_exchange_timeout(
            xf.data_ptr(), gd.data_ptr(), bd.data_ptr(), N, sp[0] * sp[1], C, G, 1e-5, 2, 2,
            y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()  # the call returns and the GPU still answers
        assert nt.wait_timeouts() > 0
        # the failure is visible in the data ...
        assert torch.isnan(mean).all() and torch.isnan(rstd).all() and torch.isnan(y.float()).all()
        # ... and in the status of the next call, which launches nothing
        out = torch.full_like(xf, 3.0)
        rc = nt.lib.gnb200_fwd(xf.data_ptr(), gd.data_ptr(), bd.data_ptr(), N, sp[0] * sp[1], C, G, 1e-5, 2, 2,
                               out.data_ptr(), mean.data_ptr(), rstd.data_ptr(), None, 0,
                               torch.cuda.current_stream().cuda_stream)
        assert rc == nt.ERR_EXCHANGE_TIMEOUT and "gave up" in nt.lib.gnb200_last_error().decode()
        torch.cuda.synchronize()
        assert (out == 3.0).all()
    finally:
        nt.clear_wait_timeouts()
    assert nt.wait_timeouts() == 0
    # after re-arming, the same problem runs normally
    got = run_cabi(nt, x, ga, be, dy, G, 1e-5, "silu")
    check_against(got, O.oracle_c(x, ga, be, dy, G, 1e-5, "silu", threads=4), torch.bfloat16)
    assert nt.wait_timeouts() == 0


def test_unaligned_parameters_use_the_scalar_path(nt):
    # gamma / beta that are contiguous but start off a 16-byte boundary (a slice of a flat parameter
    # buffer): the vector kernels would read them with 16-byte loads, so such calls must take the
    # scalar instantiation.  x and dy stay aligned.
    N, C, sp, G = 2, 64, (9, 7), 8
    for dt in (torch.float16, torch.float32):
        x, ga, be, dy = O.make_inputs(N, C, sp, dt, seed=6)
        want = O.oracle_c(x, ga, be, dy, G, 1e-5, "gelu")
        flat = torch.empty(2 * C + 8, dtype=dt, device="cuda")
        gd, bd = flat[3:3 + C], flat[3 + C:3 + 2 * C]
        gd.copy_(ga)
        bd.copy_(be)
        assert gd.data_ptr() % 16 != 0 and gd.is_contiguous()
        xd = x.cuda()
        y, mean, rstd = nt.fwd_raw(_flat(xd), gd, bd, G, 1e-5, 3)
        dx, dparam, dgamma, dbeta = nt.bwd_raw(_flat(dy.cuda()), _flat(xd), gd, bd, mean, rstd, G, 3)
        torch.cuda.synchronize()
        got = {"y": _unflat(y, x.shape), "dx": _unflat(dx, x.shape), "dgamma": dgamma, "dbeta": dbeta}
        check_against(got, want, dt)


def test_gelu_derivative_of_huge_preactivations_is_finite(nt):
    # |yh| of a few 1e4 (large gamma): the packed half-precision derivative must give 1 / 0 like the
    # fp32 formula, not inf * 0 = NaN
    N, C, sp, G = 2, 32, (8, 8), 4
    for act in ("gelu_tanh", "gelu"):
        x, ga, be, dy = O.make_inputs(N, C, sp, torch.bfloat16, seed=14)
        ga = (ga.float() * 16000.0).to(torch.bfloat16)
        out = run_cabi(nt, x, ga, be, dy, G, 1e-5, act)
        want = O.oracle_c(x, ga, be, dy, G, 1e-5, act)
        for k in ("y", "dx", "dgamma", "dbeta"):
            assert torch.isfinite(out[k].float()).all(), (act, k)
        check_against(out, want, torch.bfloat16)


def test_misaligned_pointers_use_the_scalar_path(nt):
    N, C, sp, G = 2, 24, (5, 7), 3
    x, ga, be, dy = O.make_inputs(N, C, sp, torch.float16, seed=4)
    want = O.oracle_c(x, ga, be, dy, G, 1e-5, "silu")

    def shifted(t):  # same values, storage starts 2 bytes past a 16-byte boundary
        buf = torch.empty(t.numel() + 8, dtype=t.dtype, device="cuda")
        v = buf[1:1 + t.numel()].view(N, *sp, C)
        v.copy_(t.cuda().permute(0, 2, 3, 1))
        assert v.data_ptr() % 16 != 0
        return v.permute(0, 3, 1, 2)

    out = run_cabi(nt, shifted(x), ga, be, shifted(dy), G, 1e-5, "silu")
    check_against(out, want, torch.float16)


def test_results_are_bitwise_reproducible(nt):
    for case in (CFG4[0], CFG5[4], CFG3[0]):
        x, ga, be, dy, G, eps, act, dtype = _case_inputs(case)
        a = run_cabi(nt, x, ga, be, dy, G, eps, act)
        b = run_cabi(nt, x, ga, be, dy, G, eps, act)
        for k in ("y", "dx", "dparam", "mean", "rstd"):
            assert torch.equal(a[k], b[k]), k


def test_output_buffers_are_not_overrun(nt):
    # canary-padded outputs: nothing outside [0, numel) may be written
    N, C, sp, G = 3, 40, (17, 33), 8
    x, ga, be, dy = O.make_inputs(N, C, sp, torch.bfloat16, seed=0, x_dist="uniform3")
    xf, dyf = _flat(x.cuda()), _flat(dy.cuda())
    pad = 64
    for path in ("auto", "twopass"):
        if path == "twopass":
            os.environ["GNB200_FORCE_PATH"] = "twopass"
        try:
            ybuf = torch.full((xf.numel() + 2 * pad,), 7.0, dtype=x.dtype, device="cuda")
            y = ybuf[pad:pad + xf.numel()].view(xf.shape)
            _, mean, rstd = nt.fwd_raw(xf, ga.cuda(), be.cuda(), G, 1e-5, 4, y=y)
            dbuf = torch.full((xf.numel() + 2 * pad,), 7.0, dtype=x.dtype, device="cuda")
            dx = dbuf[pad:pad + xf.numel()].view(xf.shape)
            nt.bwd_raw(dyf, xf, ga.cuda(), be.cuda(), mean, rstd, G, 4, dx=dx)
            torch.cuda.synchronize()
        finally:
            os.environ.pop("GNB200_FORCE_PATH", None)
        for buf in (ybuf, dbuf):
            assert (buf[:pad] == 7).all() and (buf[-pad:] == 7).all()


# ------------------------------------------------------------------------------------------------
# the reference-facing Python interface (module + autograd Function + torch ops)
# ------------------------------------------------------------------------------------------------
def test_module_forward_backward_matches_oracle(nt):
    import channels_last_groupnorm_b200 as pkg

    for dt, act in (("float32", "gelu_tanh"), ("float16", "silu"), ("bfloat16", "gelu")):
        N, C, sp, G = 2, 64, (12, 10), 8
        x, ga, be, dy = O.make_inputs(N, C, sp, DT[dt], seed=7)
        m = pkg.GN_NHWC(G, C, activation=act).cuda().to(DT[dt])
        with torch.no_grad():
            m.weight.copy_(ga)
            m.bias.copy_(be)
        xd = x.cuda().requires_grad_(True)
        y = m(xd)
        assert y.shape == x.shape and y.stride() == xd.stride()
        y.backward(dy.cuda())
        want = O.oracle_c(x, ga, be, dy, G, 1e-5, act)
        got = {"y": y.detach(), "dx": xd.grad, "dgamma": m.weight.grad, "dbeta": m.bias.grad}
        check_against(got, want, DT[dt])
        assert xd.grad.stride() == xd.stride()


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
def test_module_with_fp32_parameters_and_16bit_input(nt, dt):
    # the autocast convention: fp32 weight / bias, 16-bit activations.  The kernels see the
    # parameters rounded to the activation dtype; gradients come back in fp32.
    import channels_last_groupnorm_b200 as pkg

    N, C, sp, G = 3, 64, (12, 20), 8
    x, ga, be, dy = O.make_inputs(N, C, sp, torch.float32, seed=11)
    x, dy = x.to(DT[dt]), dy.to(DT[dt])
    m = pkg.GN_NHWC(G, C, activation="silu", eps=1e-5).cuda()
    with torch.no_grad():
        m.weight.copy_(ga)
        m.bias.copy_(be)
    assert m.weight.dtype == torch.float32
    xin = x.cuda().to(memory_format=torch.channels_last).requires_grad_(True)
    y = m(xin)
    assert y.dtype == DT[dt]
    y.backward(dy.cuda().to(memory_format=torch.channels_last))
    assert m.weight.grad.dtype == torch.float32 and m.bias.grad.dtype == torch.float32
    want = O.oracle_c(x, ga.to(DT[dt]), be.to(DT[dt]), dy, G, 1e-5, "silu")
    got = {"y": y.detach(), "dx": xin.grad, "dgamma": m.weight.grad, "dbeta": m.bias.grad}
    check_against(got, want, DT[dt])


def test_forward_op_is_differentiable_on_its_own(nt):
    # torch.ops.gnb200.fwd carries an autograd formula (its backward is torch.ops.gnb200.bwd)
    N, C, sp, G = 2, 32, (9, 11), 4
    x, ga, be, dy = O.make_inputs(N, C, sp, torch.float32, seed=12)
    want = O.oracle_c(x, ga, be, dy, G, 1e-5, "gelu")
    X = _flat(x.cuda()).permute(0, 2, 1).requires_grad_(True)
    w, b = ga.cuda().requires_grad_(True), be.cuda().requires_grad_(True)
    Y, _, _ = torch.ops.gnb200.fwd(X, w, b, G, 1e-5, O.ACT_CODES["gelu"])
    dX, dw, db = torch.autograd.grad(Y, (X, w, b), _flat(dy.cuda()).permute(0, 2, 1))
    got = {"y": _unflat(Y.detach().permute(0, 2, 1), x.shape), "dx": _unflat(dX.permute(0, 2, 1), x.shape),
           "dgamma": dw, "dbeta": db}
    check_against(got, want, torch.float32)


def test_module_under_torch_compile(nt):
    import channels_last_groupnorm_b200 as pkg

    N, C, sp, G = 2, 64, (16, 16), 8
    x, ga, be, dy = O.make_inputs(N, C, sp, torch.float16, seed=13)
    want = O.oracle_c(x, ga, be, dy, G, 1e-5, "silu")
    m = pkg.GN_NHWC(G, C, activation="silu").cuda().half()
    with torch.no_grad():
        m.weight.copy_(ga)
        m.bias.copy_(be)

    def step(t):
        return m(t * 1.0) + 0.0

    compiled = torch.compile(step)
    xin = x.cuda().to(memory_format=torch.channels_last).requires_grad_(True)
    y = compiled(xin)
    y.backward(dy.cuda().to(memory_format=torch.channels_last))
    got = {"y": y.detach(), "dx": xin.grad, "dgamma": m.weight.grad, "dbeta": m.bias.grad}
    check_against(got, want, torch.float16)


def test_module_affine_false_and_state_dict(nt):
    import channels_last_groupnorm_b200 as pkg

    x, _, _, _ = O.make_inputs(2, 32, (6, 6), torch.float32, seed=8)
    m = pkg.GN_NHWC(4, 32, affine=False, activation="relu").cuda()
    y = m(x.cuda())
    want = O.oracle_c(x, torch.ones(32), torch.zeros(32), None, 4, 1e-5, "relu")
    assert O.rel_err(y, want["y"]) < 1e-5
    ref = torch.nn.GroupNorm(4, 32).cuda()
    m2 = pkg.GN_NHWC(4, 32).cuda()
    m2.load_state_dict(ref.state_dict())
    xc = x.cuda()
    assert O.rel_err(m2(xc), ref(xc.contiguous())) < 1e-5


def test_module_accepts_channels_first(nt):
    # the reference sends such inputs to torch's group_norm; here they take the native NCHW kernels
    # (tests/test_nchw_f64_gpu.py covers them in depth)
    import channels_last_groupnorm_b200 as pkg

    m = pkg.GN_NHWC(4, 32).cuda()
    x = torch.randn(2, 32, 6, 6, device="cuda")
    y = m(x)
    assert y.is_contiguous() and O.rel_err(y, torch.nn.functional.group_norm(x, 4, m.weight, m.bias, m.eps)) < 1e-5


@pytest.mark.parametrize("N,C,R_list", REFERENCE_TRAILING)
def test_trailing_dims_like_reference(nt, N, C, R_list):
    """Rank 3..6 inputs with stride(1) == 1, then successive flattening (test/trailing_dims.py:7-33)."""
    import channels_last_groupnorm_b200 as pkg

    R_list = list(R_list)
    g = torch.Generator().manual_seed(0)
    x = torch.randn((N, *R_list, C), generator=g).cuda()
    x = x.permute(0, -1, *range(1, len(R_list) + 1))
    for dtype in (torch.half, torch.float):
        m = pkg.GN_NHWC(32, C).cuda().to(dtype)
        ref = torch.nn.GroupNorm(32, C).cuda().to(dtype)
        y_ref = ref(x.to(dtype))
        rl = list(R_list)
        xx = x
        while True:
            y = m(xx.to(dtype))
            assert torch.nn.functional.mse_loss(y.float(), y_ref.float().view(N, C, *rl)) < 1e-6
            if len(rl) == 1:
                break
            last = rl.pop(-1)
            rl[-1] *= last
            xx = xx.reshape(N, C, *rl)


def test_pseudo_channels_last_inputs(nt):
    """x.stride(1) == 1 but inner dims permuted (test/trailing_dims.py:35-63): values must match."""
    import channels_last_groupnorm_b200 as pkg

    B, C, G = 2, 32, 8
    for dtype in (torch.half, torch.float):
        m = pkg.GN_NHWC(G, C).cuda().to(dtype)
        ref = torch.nn.GroupNorm(G, C).cuda().to(dtype)
        for inner in ((3, 5), (3, 5, 7), (3, 5, 7, 11)):
            x = torch.randn((B, *inner, C), device="cuda")
            x = x.permute(0, -1, *range(len(inner), 0, -1)).to(dtype)
            assert x.stride(1) == 1
            assert torch.nn.functional.mse_loss(m(x).float(), ref(x).float()) < 1e-6


def test_backward_of_rank3_and_rank5_inputs(nt):
    import channels_last_groupnorm_b200 as pkg

    for sp in ((20,), (3, 4, 5)):
        x, ga, be, dy = O.make_inputs(2, 16, sp, torch.float32, seed=9)
        m = pkg.GN_NHWC(4, 16, activation="silu").cuda()
        with torch.no_grad():
            m.weight.copy_(ga)
            m.bias.copy_(be)
        xd = x.cuda().requires_grad_(True)
        m(xd).backward(dy.cuda())
        want = O.oracle_c(x, ga, be, dy, 4, 1e-5, "silu")
        check_against({"dx": xd.grad, "dgamma": m.weight.grad, "dbeta": m.bias.grad}, want, torch.float32,
                      keys=("dx", "dgamma", "dbeta"))


def test_torch_op_validation_errors(nt):
    x = torch.randn(2, 16, 8, device="cuda").permute(0, 2, 1)  # (N=2, C=8, R=16) view of NHWC storage
    w, b = torch.ones(8, device="cuda"), torch.zeros(8, device="cuda")
    with pytest.raises(RuntimeError, match="divisible"):
        torch.ops.gnb200.fwd(x, w, b, 3, 1e-5, 0)
    with pytest.raises(RuntimeError, match="dtype"):
        torch.ops.gnb200.fwd(x, w.half(), b, 2, 1e-5, 0)
    with pytest.raises(RuntimeError, match="channels-last"):  # neither channels-last nor contiguous
        torch.ops.gnb200.fwd(torch.randn(2, 8, 32, device="cuda")[:, :, ::2], w, b, 2, 1e-5, 0)
    with pytest.raises(RuntimeError, match="dtype"):
        torch.ops.gnb200.fwd(x.to(torch.int32), w, b, 2, 1e-5, 0)


# ------------------------------------------------------------------------------------------------
# against the reference itself
# ------------------------------------------------------------------------------------------------
def _golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN_DIR, "*.pt")))


@pytest.mark.parametrize("path", _golden_files(), ids=[os.path.basename(p) for p in _golden_files()])
def test_against_recorded_reference_outputs(nt, path):
    g = torch.load(path)
    meta = g["meta"]
    dtype = DT[meta["dtype"]]
    if "x" in g:
        x, ga, be, dy = g["x"], g["gamma"], g["beta"], g["dy"]
    else:
        x, ga, be, dy = O.make_inputs(meta["N"], meta["C"], tuple(meta["spatial"]), dtype, seed=meta["seed"],
                                      x_dist=meta["x_dist"], x_scale=meta["x_scale"])
    out = run_cabi(nt, x, ga, be, dy, meta["G"], meta["eps"], meta["act"])
    idx = g.get("sample_index")
    # the reference runs with -use_fast_math and 16-bit statistics: its own distance to fp64 is
    # up to ~1e-4 (fp32) / ~1e-2 (16-bit); allow that on top of our tolerance
    slack = {"float32": 1e-4, "float16": 2e-2, "bfloat16": 1e-1}[meta["dtype"]]
    for k in ("y", "dx", "dgamma", "dbeta"):
        got = out[k]
        if idx is not None and k in ("y", "dx"):
            got = got.cpu().flatten()[idx]
        assert O.rel_err(got, g["ref_" + k]) < slack, k


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="reference extension not built (oracle/build_ref.py)")
def test_against_live_reference_extension(nt):
    """Same inputs through the unmodified reference kernels and through ours, on this GPU."""
    torch.ops.load_library(REF_LIB)
    for case in (CFG1, CFG2[1], CFG4[0], CFG5[1]):
        x, ga, be, dy, G, eps, act, dtype = _case_inputs(case)
        xd, gd, bd, dd = x.cuda(), ga.cuda(), be.cuda(), dy.cuda()
        x_flat = xd.view(xd.shape[0], xd.shape[1], -1)
        code = O.ACT_CODES[act]
        y_r, means, rstds = torch.ops.gnop.fwd(x_flat, gd, bd, G, eps, code)
        dx_r, dg_r, db_r = torch.ops.gnop.bwd(dd.view(x_flat.shape), x_flat, gd, bd, means, rstds, G, code)
        ref = {"y": y_r.view(x.shape), "dx": dx_r.view(x.shape), "dgamma": dg_r, "dbeta": db_r}
        ours = run_cabi(nt, x, ga, be, dy, G, eps, act)
        want = O.oracle_torch(x, ga, be, dy, G, eps, act)
        ours_err = check_against(ours, want, dtype)
        ref_err = {k: O.rel_err(ref[k], want[k]) for k in ours_err}
        print("\n%s ours %s\n%s ref  %s" % (_id(case), ours_err, " " * len(_id(case)), ref_err))
        loose = 1e-3 if dtype == torch.float32 else 1e-1
        assert all(e < loose for e in ref_err.values()), ref_err
