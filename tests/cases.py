"""Shapes shared by the CPU and GPU tests.

BASELINE_* are the benchmark configurations; REFERENCE_* re-use the shapes of the reference's own
test scripts (test/check_outputs.py:161-189, test/trailing_dims.py:9-14,52-56,
test/nchw_nhwc_equal.py:8, prof.py:20 of latentCall145/channels-last-groupnorm).
Tuples: (N, C, spatial, G, eps, activation, dtype-name, x distribution, x scale)
"""

CFG1 = (2, 128, (32, 32), 32, 1e-5, "identity", "float32", "normal", 1.0)

CFG2 = [
    (1, 320, (64, 64), 32, 1e-5, "silu", "float16", "normal", 1.0),
    (1, 640, (32, 32), 32, 1e-5, "silu", "float16", "normal", 1.0),
    (1, 1280, (16, 16), 32, 1e-5, "silu", "float16", "normal", 1.0),
    (1, 1280, (8, 8), 32, 1e-5, "silu", "float16", "normal", 1.0),
]

CFG3 = [
    (1, 512, (128, 128), 32, 1e-6, "silu", "float16", "normal", 2.0),
    (1, 512, (256, 256), 32, 1e-6, "silu", "float16", "normal", 2.0),
    (1, 256, (512, 512), 32, 1e-6, "silu", "float16", "normal", 2.0),
    (1, 128, (1024, 1024), 32, 1e-6, "silu", "float16", "normal", 2.0),
]

# per-rank batch of the sharded training configuration at 8 / 4 / 2 / 1 GPUs
CFG4 = [(n, 256, (64, 64), 32, 1e-5, "gelu", "bfloat16", "normal", 1.0) for n in (8, 16, 32, 64)]

CFG5 = [
    (N, C, sp, G, 1e-5, act, dt, "uniform3", 1.0)
    for (N, C, G, sp) in [(8, 96, 3, (7, 7)), (4, 64, 64, (56, 56)), (16, 2048, 32, (7, 7)), (3, 40, 8, (17, 33))]
    for act in ("gelu_tanh", "relu")
    for dt in ("float32", "bfloat16")
]

# shapes of the reference's CUSTOM_INPUTS (fp64 there; run here in the supported dtypes)
REFERENCE_CUSTOM = [
    (1, 1, (2, 2), 1), (2, 3909, (5, 5), 3), (1, 2062, (5, 5), 1031), (3, 4096, (7, 7), 4),
    (2, 160, (8, 8), 160), (1, 3, (7, 7), 1), (1, 1, (4, 4), 1), (1, 128, (8, 8), 8),
    (2, 1280, (8, 8), 32), (2, 640, (16, 16), 32), (2, 2560, (8, 8), 32), (2, 320, (32, 32), 32),
    (2, 1920, (16, 16), 32), (2, 960, (32, 32), 32), (8, 128, (64, 64), 32), (13, 2560, (8, 8), 4),
]

# rank-3..6 inputs of the reference's trailing-dims test (N, C, spatial list), G = 32
REFERENCE_TRAILING = [
    (1, 512, [1, 1, 1, 1]), (1, 256, [4, 2, 8, 1]), (1, 256, [7, 13, 19, 1]), (1, 128, [32, 1, 1, 1]),
    (1, 32, [32, 128, 32, 1]),
]
