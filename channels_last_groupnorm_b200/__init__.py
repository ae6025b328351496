"""B200-native channels-last GroupNorm with fused activation (drop-in for `gnnhwc`)."""
from .gn_nhwc import ACTIVATION_CODES, GN_NHWC, GN_NHWC_Func
from . import _compile  # noqa: F401  (fake-tensor kernels and autograd formula of torch.ops.gnb200.*)

__all__ = ["GN_NHWC", "GN_NHWC_Func", "ACTIVATION_CODES"]
