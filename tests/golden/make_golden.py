"""Records golden vectors from the UNMODIFIED reference extension.  Needs a CUDA GPU.

    python oracle/build_ref.py                      # where the reference checkout is present
    python tests/golden/make_golden.py --out tests/golden     # on the GPU machine

For each small case below the seeded inputs are generated (oracle.gn_oracle.make_inputs), pushed
through the reference's own ops `torch.ops.gnop.fwd / bwd` (src/gnnhwc/csrc/custom_gn.cpp:91-94 of
latentCall145/channels-last-groupnorm) exactly as its autograd Function does
(src/gnnhwc/custom_gn.py:30-47), and inputs + outputs are saved as one small `.pt` file per case.
tests/test_oracle.py then checks both CPU oracles against these files, and tests/test_parity_gpu.py
checks the new kernels against them.
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import gn_oracle as O  # noqa: E402

DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}

# name, N, C, spatial, G, eps, act, dtype, x distribution, x scale, subsample stride (0 = keep all)
CASES = [
    ("f32_identity_2x32x8x8_g8", 2, 32, (8, 8), 8, 1e-5, "identity", "float32", "normal", 1.0, 0),
    ("f32_gelu_tanh_2x24x5x7_g3", 2, 24, (5, 7), 3, 1e-5, "gelu_tanh", "float32", "uniform3", 1.0, 0),
    ("f32_relu_2x16x4x4_g16", 2, 16, (4, 4), 16, 1e-5, "relu", "float32", "uniform3", 1.0, 0),
    ("f32_gelu_3x40x17x33_g8", 3, 40, (17, 33), 8, 1e-5, "gelu", "float32", "uniform3", 1.0, 7),
    ("f16_silu_1x40x6x6_g4", 1, 40, (6, 6), 4, 1e-5, "silu", "float16", "normal", 1.0, 0),
    ("f16_silu_1x320x16x16_g32", 1, 320, (16, 16), 32, 1e-6, "silu", "float16", "normal", 2.0, 11),
    ("bf16_gelu_3x40x3x5_g8", 3, 40, (3, 5), 8, 1e-5, "gelu", "bfloat16", "normal", 1.0, 0),
    ("bf16_gelu_2x256x8x8_g32", 2, 256, (8, 8), 32, 1e-5, "gelu", "bfloat16", "normal", 1.0, 5),
    ("cfg1_f32_identity_2x128x32x32_g32", 2, 128, (32, 32), 32, 1e-5, "identity", "float32", "normal", 1.0, 97),
]


def run_reference(x, gamma, beta, dy, G, eps, act_code):
    """The reference's Function body: flatten to (N, C, R) views and call its two ops."""
    x_flat = x.view(x.shape[0], x.shape[1], -1)
    y, means, rstds = torch.ops.gnop.fwd(x_flat, gamma, beta, G, eps, act_code)
    dy_flat = dy.contiguous(memory_format=torch.channels_last).view(x_flat.shape) if dy.ndim == 4 else dy.view(x_flat.shape)
    dx, dgamma, dbeta = torch.ops.gnop.bwd(dy_flat, x_flat, gamma, beta, means, rstds, G, act_code)
    return y.view(x.shape), dx.view(x.shape), dgamma, dbeta


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden"))
    ap.add_argument("--lib", default=os.path.join(ROOT, "oracle", "_ref", "gn_op.so"))
    args = ap.parse_args()
    torch.ops.load_library(args.lib)
    os.makedirs(args.out, exist_ok=True)
    for name, N, C, sp, G, eps, act, dt, dist, scale, stride in CASES:
        x, ga, be, dy = O.make_inputs(N, C, sp, DT[dt], seed=0, x_dist=dist, x_scale=scale)
        xc, gc, bc, dc = x.cuda(), ga.cuda(), be.cuda(), dy.cuda()
        y, dx, dgamma, dbeta = run_reference(xc, gc, bc, dc, G, eps, O.ACT_CODES[act])
        torch.cuda.synchronize()
        rec = {
            "meta": {"N": N, "C": C, "spatial": list(sp), "G": G, "eps": eps, "act": act, "dtype": dt,
                     "seed": 0, "x_dist": dist, "x_scale": scale, "gpu": torch.cuda.get_device_name(0),
                     "torch": str(torch.__version__)},
            "x": x.clone(), "gamma": ga.clone(), "beta": be.clone(), "dy": dy.clone(),
            "ref_dgamma": dgamma.cpu(), "ref_dbeta": dbeta.cpu(),
        }
        if stride:
            idx = torch.arange(0, x.numel(), stride)
            rec["sample_index"] = idx
            rec["ref_y"] = y.cpu().flatten()[idx].clone()
            rec["ref_dx"] = dx.cpu().flatten()[idx].clone()
            if x.numel() > 20000:  # large case: inputs are regenerated from the seed, not stored
                for k in ("x", "gamma", "beta", "dy"):
                    rec.pop(k)
        else:
            rec["ref_y"] = y.cpu().clone()
            rec["ref_dx"] = dx.cpu().clone()
        torch.save(rec, os.path.join(args.out, name + ".pt"))
        o = O.oracle_torch(x, ga, be, dy, G, eps, act)
        want_y = o["y"].flatten()[rec["sample_index"]] if stride else o["y"]
        print("%-40s ref-vs-fp64: y %.2e  dgamma %.2e  dbeta %.2e" % (
            name, O.rel_err(rec["ref_y"], want_y), O.rel_err(dgamma, o["dgamma"]), O.rel_err(dbeta, o["dbeta"])))


if __name__ == "__main__":
    main()
