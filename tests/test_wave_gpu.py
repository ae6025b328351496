"""GPU parity tests of the wave plan: forward and backward as one persistent cooperative kernel each,
rows moved by TMA, slabs merged by the CTA that delivers the last partial (csrc/gn_wave.cu).

The plan is forced with GNB200_FORCE_PATH=wave; small L2 budgets and grids force several waves,
several units per CTA and several chunks per slab at sizes the CPU oracle finishes in seconds.
Tolerances as everywhere: 1e-5 (fp32), 1e-2 (fp16 / bf16), max-abs error relative to max(1, max|oracle|).
"""
import pytest
import torch

from oracle import gn_oracle as O

from .test_parity_gpu import DT, _cuda_fp64_reference, _flat, check_against, run_cabi

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nt():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from channels_last_groupnorm_b200 import _native

    return _native


CASES = [
    # (N, C, spatial, G, dtype, act, env)
    (2, 256, (96, 96), 32, "float16", "silu", {"GNB200_WAVE_MB": "1"}),                      # 16 waves of one slab
    (2, 256, (96, 96), 32, "bfloat16", "gelu", {"GNB200_WAVE_MB": "1", "GNB200_WAVE_GRID": "7"}),  # 5+ units per CTA
    (3, 128, (40, 56), 32, "float32", "gelu_tanh", {"GNB200_WAVE_GRID": "5"}),               # fp32: Welford, xh form
    (2, 320, (33, 47), 32, "float16", "silu", {}),                                             # D = 10: vectors straddle groups
    (2, 320, (33, 47), 32, "bfloat16", "relu", {"GNB200_WAVE_CW": "40", "GNB200_WAVE_KR": "2"}),  # 5 vectors per row
    (1, 64, (57, 31), 64, "float32", "identity", {"GNB200_WAVE_KR": "2", "GNB200_WAVE_STAGES": "2"}),  # D = 1
    (5, 512, (24, 24), 32, "bfloat16", "gelu_tanh", {"GNB200_WAVE_MB": "2", "GNB200_WAVE_STAGES": "5"}),
    (1, 96, (7, 7), 3, "float32", "relu", {}),                                                 # one short chunk per slab
    (2, 256, (96, 96), 32, "float16", "gelu", {"GNB200_WAVE_MB": "1", "GNB200_WAVE_OVERLAP": "1"}),  # pass A of wave w+1 before pass B of w
    (3, 128, (40, 56), 32, "float32", "silu", {"GNB200_WAVE_MB": "1", "GNB200_WAVE_OVERLAP": "1", "GNB200_WAVE_GRID": "9"}),
    (2, 256, (96, 96), 32, "bfloat16", "silu", {"GNB200_WAVE_MB": "2", "GNB200_WAVE_TEAMS": "2"}),     # two teams take alternate waves
    (3, 128, (40, 56), 32, "float16", "gelu", {"GNB200_WAVE_MB": "2", "GNB200_WAVE_TEAMS": "3", "GNB200_WAVE_OVERLAP": "1"}),
    (5, 64, (33, 31), 8, "float32", "relu", {"GNB200_WAVE_MB": "1", "GNB200_WAVE_TEAMS": "3", "GNB200_WAVE_GRID": "7"}),
]


def _id(c):
    return "%dx%dx%s-g%d-%s-%s-%s" % (c[0], c[1], "x".join(map(str, c[2])), c[3], c[4], c[5],
                                     ",".join("%s=%s" % (k[7:], v) for k, v in c[6].items()) or "default")


@pytest.mark.parametrize("case", CASES, ids=_id)
def test_wave_plan_against_oracle(nt, case, monkeypatch):
    N, C, sp, G, dt, act, env = case
    monkeypatch.setenv("GNB200_FORCE_PATH", "wave")
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    R = sp[0] * sp[1]
    assert " wave " in nt.describe_plan(N, R, C, G, DT[dt], 0) and " wave " in nt.describe_plan(N, R, C, G, DT[dt], 1)
    x, ga, be, dy = O.make_inputs(N, C, sp, DT[dt], seed=17, x_dist="uniform3")
    out = run_cabi(nt, x, ga, be, dy, G, 1e-5, act)
    want = O.oracle_c(x, ga, be, dy, G, 1e-5, act, threads=4)
    check_against(out, want, DT[dt])
    assert O.rel_err(out["mean"], want["mean"]) < 1e-5
    assert O.rel_err(out["rstd"] / want["rstd"].cuda().float(), torch.ones_like(want["rstd"])) < 1e-5
    assert O.rel_err(out["dparam"][0], want["dgamma"]) <= O.TOLERANCE[DT[dt]]
    assert O.rel_err(out["dparam"][1], want["dbeta"]) <= O.TOLERANCE[DT[dt]]
    again = run_cabi(nt, x, ga, be, dy, G, 1e-5, act)  # fixed summation order: bit-identical reruns
    for k in ("y", "dx", "dparam", "mean", "rstd"):
        assert torch.equal(out[k], again[k]), k
    assert nt.wait_timeouts() == 0


def test_wave_plan_with_many_samples_and_channels(nt, monkeypatch):
    # many slabs per wave and many rows of channel sums for the dgamma / dbeta reduction at the kernel's end
    N, C, sp, G = 160, 2048, (4, 4), 32
    monkeypatch.setenv("GNB200_FORCE_PATH", "wave")
    assert " wave " in nt.describe_plan(N, 16, C, G, torch.float16, 1)
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((N, *sp, C), device="cuda", generator=gen).half().permute(0, 3, 1, 2)
    dy = torch.randn((N, *sp, C), device="cuda", generator=gen).half().permute(0, 3, 1, 2)
    ga = (torch.rand(C, device="cuda", generator=gen) + 0.5).half()
    be = (torch.randn(C, device="cuda", generator=gen) * 0.1).half()
    out = run_cabi(nt, x, ga, be, dy, G, 1e-5, "silu")
    check_against(out, _cuda_fp64_reference(x, ga, be, dy, G, 1e-5, "silu"), torch.float16)


def test_wave_plan_matches_multi_kernel_plan_on_a_canary_padded_output(nt, monkeypatch):
    N, C, sp, G = 2, 128, (50, 30), 16
    x, ga, be, dy = O.make_inputs(N, C, sp, torch.bfloat16, seed=23)
    xf, dyf, gd, bd = _flat(x.cuda()), _flat(dy.cuda()), ga.cuda(), be.cuda()
    monkeypatch.setenv("GNB200_FORCE_PATH", "wave")
    pad = 64
    ybuf = torch.full((xf.numel() + 2 * pad,), 7.0, dtype=x.dtype, device="cuda")
    y = ybuf[pad:pad + xf.numel()].view(xf.shape)
    _, mean, rstd = nt.fwd_raw(xf, gd, bd, G, 1e-5, 3, y=y)
    dbuf = torch.full((xf.numel() + 2 * pad,), 7.0, dtype=x.dtype, device="cuda")
    dx = dbuf[pad:pad + xf.numel()].view(xf.shape)
    _, dparam, _, _ = nt.bwd_raw(dyf, xf, gd, bd, mean, rstd, G, 3, dx=dx)
    torch.cuda.synchronize()
    for buf in (ybuf, dbuf):
        assert (buf[:pad] == 7).all() and (buf[-pad:] == 7).all()
    monkeypatch.setenv("GNB200_FORCE_PATH", "twopass")
    y2, mean2, rstd2 = nt.fwd_raw(xf, gd, bd, G, 1e-5, 3)
    dx2, dparam2, _, _ = nt.bwd_raw(dyf, xf, gd, bd, mean2, rstd2, G, 3)
    torch.cuda.synchronize()
    assert O.rel_err(y, y2) <= 1e-2 and O.rel_err(dx, dx2) <= 1e-2 and O.rel_err(dparam, dparam2) <= 1e-2
    assert O.rel_err(mean, mean2) < 1e-5 and O.rel_err(rstd, rstd2) < 1e-4
