"""GPU parity tests of the channels-first (NCHW) kernels and of the double-precision path.

The reference sends channels-first inputs to torch's group_norm + activation
(src/gnnhwc/custom_gn.py:75-79) and instantiates its kernels for double
(src/gnnhwc/csrc/custom_gn.cpp:29-33); here both are native kernels behind the C ABI
(gnb200_fwd_nchw / gnb200_bwd_nchw, gnb200_fwd_f64 / gnb200_bwd_f64).  Shapes follow the
reference's own tests: test/nchw_nhwc_equal.py:7-25, test/trailing_dims.py:65-71,
test/check_outputs.py:161-185 (its fp64 CUSTOM_INPUTS).
Tolerances: 1e-5 (fp32), 1e-2 (fp16 / bf16), 1e-10 (fp64); max-abs error relative to max(1, max|oracle|).
"""
import pytest
import torch

from oracle import gn_oracle as O

from .cases import REFERENCE_CUSTOM
from .test_parity_gpu import DT, _cuda_fp64_reference, check_against

pytestmark = pytest.mark.gpu
DT = dict(DT, float64=torch.float64)


@pytest.fixture(scope="module")
def nt():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from channels_last_groupnorm_b200 import _native

    return _native


def run_nchw(nt, x, ga, be, dy, G, eps, act):
    """Forward + backward through gnb200_fwd_nchw / gnb200_bwd_nchw on NCHW-contiguous copies."""
    code = O.ACT_CODES[act]
    xd = x.cuda().contiguous()
    flat = xd.reshape(x.shape[0], x.shape[1], -1)
    gd, bd = ga.cuda(), be.cuda()
    y, mean, rstd = nt.fwd_nchw_raw(flat, gd, bd, G, eps, code)
    out = {"y": y.reshape(x.shape), "mean": mean, "rstd": rstd}
    if dy is not None:
        dyf = dy.cuda().contiguous().reshape(flat.shape)
        dx, dparam, dgamma, dbeta = nt.bwd_nchw_raw(dyf, flat, gd, bd, mean, rstd, G, code)
        out.update(dx=dx.reshape(x.shape), dgamma=dgamma, dbeta=dbeta, dparam=dparam)
    torch.cuda.synchronize()
    return out


NCHW_CASES = [
    # (N, C, spatial, G)
    (2, 128, (32, 32), 32),    # vector path, several chunks per slab
    (3, 40, (17, 33), 8),      # R = 561: odd, single-element path
    (8, 96, (7, 7), 3),        # tiny rows, large groups
    (4, 64, (56, 56), 64),     # one channel per group
    (2, 320, (16, 24), 32),    # D = 10
    (1, 16, (128, 160), 4),    # long channel rows: several pieces per row
]


@pytest.mark.parametrize("dt", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("shape", NCHW_CASES, ids=lambda s: "%dx%dx%s-g%d" % (s[0], s[1], "x".join(map(str, s[2])), s[3]))
def test_nchw_kernels_against_oracle(nt, shape, dt):
    N, C, sp, G = shape
    for act in ("silu", "gelu_tanh") if dt != "float32" else ("gelu", "relu"):
        x, ga, be, dy = O.make_inputs(N, C, sp, DT[dt], seed=41, x_dist="uniform3")
        out = run_nchw(nt, x, ga, be, dy, G, 1e-5, act)
        want = O.oracle_c(x, ga, be, dy, G, 1e-5, act, threads=4)
        check_against(out, want, DT[dt])
        assert O.rel_err(out["mean"], want["mean"]) < 1e-5
        assert O.rel_err(out["rstd"] / want["rstd"].cuda().float(), torch.ones_like(want["rstd"])) < 1e-5
        assert O.rel_err(out["dparam"][0], want["dgamma"]) <= O.TOLERANCE[DT[dt]]
        again = run_nchw(nt, x, ga, be, dy, G, 1e-5, act)
        for k in ("y", "dx", "dparam", "mean", "rstd"):
            assert torch.equal(out[k], again[k]), k


def test_nchw_chained_launches_change_no_bit(nt, monkeypatch):
    """GNB200_CHAIN=0 (plain stream order) and the default (programmatic dependent launches) give the same bits."""
    x, ga, be, dy = O.make_inputs(2, 128, (32, 32), torch.float16, seed=3)
    outs = []
    for chain in ("1", "0"):
        monkeypatch.setenv("GNB200_CHAIN", chain)
        for _ in range(3):
            out = run_nchw(nt, x, ga, be, dy, 32, 1e-5, "silu")
        outs.append(out)
    for k in ("y", "dx", "mean", "rstd", "dparam"):
        assert torch.equal(outs[0][k], outs[1][k]), k


@pytest.mark.parametrize("act", O.ACT_NAMES)
def test_nchw_every_activation(nt, act):
    for dt in ("float32", "float16", "bfloat16"):
        x, ga, be, dy = O.make_inputs(3, 48, (9, 16), DT[dt], seed=2, x_dist="uniform3")
        out = run_nchw(nt, x, ga, be, dy, 6, 1e-5, act)
        check_against(out, O.oracle_c(x, ga, be, dy, 6, 1e-5, act), DT[dt])


def test_nchw_and_nhwc_inputs_give_the_same_module_outputs(nt):
    """test/nchw_nhwc_equal.py of the reference: 1 x 128 x 256 x 256, G = 32, out and x.grad of the NCHW
    and the NHWC input agree (mean squared difference < 1e-6), for every activation and dtype."""
    import channels_last_groupnorm_b200 as pkg

    N, R, G, C = 1, 256, 32, 128
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((N, C, R, R), device="cuda", generator=gen)
    dy = torch.rand((N, C, R, R), device="cuda", generator=gen)
    for act in ("identity", "silu", "gelu", "gelu_tanh"):
        for dtype in (torch.half, torch.float, torch.double, torch.bfloat16):
            m = pkg.GN_NHWC(G, C, act).cuda().to(dtype)
            with torch.no_grad():
                m.weight.copy_(torch.rand(C, device="cuda", generator=gen) + 0.5)
                m.bias.copy_(torch.randn(C, device="cuda", generator=gen) * 0.1)
            x1 = x.to(dtype).clone().detach().requires_grad_(True)                                           # NCHW
            x2 = x.to(dtype).clone().to(memory_format=torch.channels_last).detach().requires_grad_(True)   # NHWC
            out1, out2 = m(x1), m(x2)
            assert out1.is_contiguous() and out2.stride(1) == 1
            out1.backward(dy.to(dtype))
            g1 = (m.weight.grad.clone(), m.bias.grad.clone())
            m.weight.grad = m.bias.grad = None
            out2.backward(dy.to(dtype).to(memory_format=torch.channels_last))
            tol = 1e-6 if dtype != torch.bfloat16 else 2e-4  # bf16 outputs of magnitude ~4 round to 1.6e-2
            assert (out1.float() - out2.float()).square().mean() < tol, (act, dtype)
            assert (x1.grad.float() - x2.grad.float()).square().mean() < tol, (act, dtype)
            assert O.rel_err(g1[0], m.weight.grad) < 2e-2 and O.rel_err(g1[1], m.bias.grad) < 2e-2
            if dtype == torch.float:  # and both agree with torch
                ref = O.torch_activation(act)(torch.nn.functional.group_norm(x, G, m.weight, m.bias, m.eps))
                assert O.rel_err(out1, ref) < 1e-5 and O.rel_err(out2, ref) < 1e-5


def test_pseudo_contiguous_inputs_like_reference(nt):
    """x.stride(-1) == 1 but not contiguous (test/trailing_dims.py:65-71): values must match nn.GroupNorm."""
    import channels_last_groupnorm_b200 as pkg

    B, C, G = 2, 32, 8
    for dtype in (torch.half, torch.float):
        m = pkg.GN_NHWC(G, C).cuda().to(dtype)
        ref = torch.nn.GroupNorm(G, C).cuda().to(dtype)
        for inner in ((3, 5), (3, 5, 7), (3, 5, 7, 11)):
            x = torch.randn((B, C, *inner), device="cuda")
            x = x.permute(0, 1, *range(len(inner), 1, -1), -1).to(dtype)
            assert x.stride(-1) == 1 and not x.is_contiguous() or len(inner) == 2
            assert torch.nn.functional.mse_loss(m(x).float(), ref(x).float()) < 1e-6


def test_module_backward_of_channels_first_inputs(nt):
    import channels_last_groupnorm_b200 as pkg

    for dt, act, sp in (("float32", "gelu_tanh", (12, 10)), ("float16", "silu", (8, 8, 4)), ("bfloat16", "gelu", (30,))):
        N, C, G = 2, 64, 8
        x, ga, be, dy = O.make_inputs(N, C, sp, DT[dt], seed=7)
        m = pkg.GN_NHWC(G, C, activation=act).cuda().to(DT[dt])
        with torch.no_grad():
            m.weight.copy_(ga)
            m.bias.copy_(be)
        xd = x.cuda().contiguous().requires_grad_(True)  # channels-first storage
        assert xd.stride(1) != 1
        y = m(xd)
        assert y.shape == x.shape and y.is_contiguous()
        y.backward(dy.cuda().contiguous())
        want = O.oracle_c(x, ga, be, dy, G, 1e-5, act)
        got = {"y": y.detach(), "dx": xd.grad, "dgamma": m.weight.grad, "dbeta": m.bias.grad}
        check_against(got, want, DT[dt])
        assert xd.grad.is_contiguous()


# ------------------------------------------------------------------------------------------------
# double precision
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("channels_last", [True, False], ids=["nhwc", "nchw"])
@pytest.mark.parametrize("shape", REFERENCE_CUSTOM, ids=lambda s: "%dx%dx%s-g%d" % (s[0], s[1], "x".join(map(str, s[2])), s[3]))
def test_fp64_reference_custom_shapes(nt, shape, channels_last):
    """The reference's fp64 CUSTOM_INPUTS (test/check_outputs.py:161-185) against the C oracle at 1e-10."""
    N, C, sp, G = shape
    act = O.ACT_NAMES[(N + C + G) % 5]
    x, ga, be, dy = O.make_inputs(N, C, sp, torch.float64, seed=1)
    xd, dyd = x.cuda(), dy.cuda()
    if channels_last:
        xf = xd.permute(0, 2, 3, 1).reshape(N, -1, C)
        dyf = dyd.permute(0, 2, 3, 1).reshape(N, -1, C)
    else:
        xf = xd.contiguous().reshape(N, C, -1)
        dyf = dyd.contiguous().reshape(N, C, -1)
    code = O.ACT_CODES[act]
    y, mean, rstd = nt.fwd_f64_raw(xf.contiguous(), ga.cuda(), be.cuda(), G, 1e-5, code, channels_last)
    dx, dgamma, dbeta = nt.bwd_f64_raw(dyf.contiguous(), xf.contiguous(), ga.cuda(), be.cuda(), mean, rstd, G, code,
                                      channels_last)
    torch.cuda.synchronize()
    if channels_last:
        y = y.reshape(N, *sp, C).permute(0, 3, 1, 2)
        dx = dx.reshape(N, *sp, C).permute(0, 3, 1, 2)
    else:
        y, dx = y.reshape(x.shape), dx.reshape(x.shape)
    want = O.oracle_c(x, ga, be, dy, G, 1e-5, act, threads=4)
    check_against({"y": y, "dx": dx, "dgamma": dgamma, "dbeta": dbeta}, want, torch.float64)
    assert O.rel_err(mean, want["mean"]) < 1e-12 and O.rel_err(rstd, want["rstd"]) < 1e-10


def test_fp64_module_and_ops(nt):
    import channels_last_groupnorm_b200 as pkg

    N, C, sp, G = 3, 40, (17, 33), 8
    for act in O.ACT_NAMES:
        x, ga, be, dy = O.make_inputs(N, C, sp, torch.float64, seed=5, x_dist="uniform3")
        want = O.oracle_c(x, ga, be, dy, G, 1e-5, act, threads=3)
        m = pkg.GN_NHWC(G, C, activation=act).cuda().double()
        with torch.no_grad():
            m.weight.copy_(ga)
            m.bias.copy_(be)
        for layout in ("nhwc", "nchw"):
            xd = x.cuda() if layout == "nhwc" else x.cuda().contiguous()
            xd = xd.detach().requires_grad_(True)
            m.weight.grad = m.bias.grad = None
            y = m(xd)
            assert y.dtype == torch.float64 and y.stride() == xd.stride()
            y.backward(dy.cuda())
            got = {"y": y.detach(), "dx": xd.grad, "dgamma": m.weight.grad, "dbeta": m.bias.grad}
            check_against(got, want, torch.float64)
