"""CPU tests of the host side: C ABI exports, argument validation, planner, module interface."""
import ctypes
import os
import re

import pytest
import torch

import channels_last_groupnorm_b200 as pkg
from channels_last_groupnorm_b200 import _native as nt
from channels_last_groupnorm_b200 import build as gnbuild


def _declared_functions(header_text):
    text = re.sub(r"/\*.*?\*/", "", header_text, flags=re.S)
    return sorted(set(re.findall(r"\b(gnb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(repo_root):
    header = open(os.path.join(repo_root, "include", "gnb200.h")).read()
    names = _declared_functions(header)
    assert {"gnb200_fwd", "gnb200_bwd", "gnb200_fwd_workspace_bytes", "gnb200_bwd_workspace_bytes"} <= set(names)
    lib = ctypes.CDLL(gnbuild.CORE_LIB)
    for name in names:
        assert hasattr(lib, name), "libgnb200.so does not export " + name


def test_core_library_does_not_link_torch():
    # the C ABI must be bindable without PyTorch: no libtorch / libc10 in the dynamic section
    with open(gnbuild.CORE_LIB, "rb") as f:
        blob = f.read()
    assert b"libtorch" not in blob and b"libc10" not in blob


def test_activation_codes_match_reference_table():
    # src/gnnhwc/custom_gn.py:52-59 of the reference
    want = {"identity": 0, "relu": 1, "swish": 2, "silu": 2, "gelu": 3, "gelu_tanh": 4}
    assert pkg.ACTIVATION_CODES == want
    for name, code in want.items():
        assert nt.lib.gnb200_act_code(name.encode()) == code
    assert nt.lib.gnb200_act_code(b"mish") == -1


_KEEP = []


def _buffer(nbytes):
    """A pointer for arguments that a refused call never dereferences.  With a GPU present it is a
    real device buffer of the stated size, so that a regression of the checks under test could not
    turn into a stray access; without one (the CPU test pass) nothing can be launched anyway."""
    if torch.cuda.is_available():
        t = torch.zeros(max(int(nbytes), 16), dtype=torch.uint8, device="cuda")
        _KEEP.append(t)
        return ctypes.c_void_p(t.data_ptr())
    return ctypes.c_void_p(16)


def test_invalid_arguments_are_rejected_before_any_cuda_call():
    f = nt.lib.gnb200_fwd
    one = _buffer(4096)  # validation fails before anything is launched
    assert f(one, one, one, 2, 4, 6, 4, 1e-5, 0, 0, one, one, one, None, 0, None) == -1  # C % G != 0
    assert "divisible" in nt.lib.gnb200_last_error().decode()
    assert f(one, one, one, 2, 4, 8, 4, 1e-5, 9, 0, one, one, one, None, 0, None) == -1  # bad activation
    assert f(one, one, one, 2, 4, 8, 4, 1e-5, 0, 7, one, one, one, None, 0, None) == -1  # bad dtype
    assert f(one, one, one, 0, 4, 8, 4, 1e-5, 0, 0, one, one, one, None, 0, None) == -1  # empty batch
    assert f(None, one, one, 2, 4, 8, 4, 1e-5, 0, 0, one, one, one, None, 0, None) == -1  # null x
    b = nt.lib.gnb200_bwd
    assert b(one, one, one, one, one, one, 2, 4, 8, 4, 0, 0, one, None, None, None, None, 0, None) == -1
    with pytest.raises(nt.Gnb200Error):
        nt.check(-1)


def test_peer_exchange_buffer_size_and_argument_checks():
    """The in-kernel all-reduce of [dgamma | dbeta]: two parities x world slots of 2 * C (value, number) pairs of
    8 bytes, world x blocks acknowledgement words and four counter words per block of 32 channels, rounded up
    to 256 bytes."""
    nbytes = nt.peer_exchange_bytes(256, 8)
    assert nbytes == (2 * 8 * 512 * 8 + (8 * 8 + 4 * 8) * 4 + 255) // 256 * 256
    assert nt.peer_exchange_bytes(256, 1) > 0 and nt.peer_exchange_bytes(40, 2) % 256 == 0
    assert nt.peer_exchange_bytes(256, 0) == 0 and nt.peer_exchange_bytes(256, 17) == 0 and nt.peer_exchange_bytes(0, 2) == 0
    one = _buffer(4096)
    table = (ctypes.c_void_p * 2)(one, one)
    f = nt.lib.gnb200_bwd_peer
    args = (one, one, one, one, one, one, 2, 4, 8, 4, 0, 0, one, one, None, None, None, 0)
    assert f(*args, table, 2, 2, None) == -1 and "rank 2 of 2" in nt.lib.gnb200_last_error().decode()
    assert f(*args, table, 0, 17, None) == -1
    assert f(*args, None, 0, 2, None) == -1 and "null table" in nt.lib.gnb200_last_error().decode()
    bad = (ctypes.c_void_p * 2)(one, None)
    assert f(*args, bad, 0, 2, None) == -1 and "rank 1" in nt.lib.gnb200_last_error().decode()
    push = nt.lib.gnb200_bwd_peer_push
    assert push(*args[:14], None, 0, table, 5, 2, None) == -1 and "rank 5 of 2" in nt.lib.gnb200_last_error().decode()
    for g in (nt.lib.gnb200_allreduce_param_grads, nt.lib.gnb200_peer_collect):
        assert g(one, None, None, 8, 9, table, 0, 2, None) == -1  # bad dtype code
        assert g(None, None, None, 8, 0, table, 0, 2, None) == -1  # null buffer
    _KEEP.clear()


def test_workspace_is_required_when_the_plan_needs_one():
    # a slab far too large for a cluster: multi-kernel path, scratch needed
    N, R, C, G = 1, 1 << 20, 128, 32
    need = nt.lib.gnb200_fwd_workspace_bytes(N, R, C, G, 1)
    assert need > 0
    one = _buffer(N * R * C * 2)
    rc = nt.lib.gnb200_fwd(one, one, one, N, R, C, G, 1e-5, 2, 1, one, one, one, None, 0, None)
    _KEEP.clear()
    assert rc == -2 and "workspace" in nt.lib.gnb200_last_error().decode()


@pytest.mark.parametrize("shape,dtype,path", [
    ((2, 1024, 128, 32), torch.float32, "fused"),
    ((64, 4096, 256, 32), torch.bfloat16, "fused"),
    ((1, 4096, 320, 32), torch.float16, "fused"),
    ((1, 1 << 20, 128, 32), torch.float16, "twopass"),
    ((1, 512 * 512, 256, 32), torch.float16, "twopass/wave"),
    ((2, 25, 3909, 3), torch.float32, "twopass"),
])
def test_planner_paths(shape, dtype, path):
    for direction in (0, 1):
        text = nt.describe_plan(*shape, dtype, direction)
        # "a/b": forward takes plan a, backward plan b (the wave plan is the default only in the backward
        # direction, where it measured faster than the multi-kernel plan)
        want = path.split("/")[direction] if "/" in path else path
        assert (" " + want + " ") in text, text
        fields = dict(kv.split("=") for kv in text.split()[2:])
        assert int(fields["threads"]) % 32 == 0 and int(fields["threads"]) <= 512
        assert int(fields["smem"]) <= 227 * 1024
        assert int(fields["cw"]) % int(fields["ve"]) == 0
        if want == "fused":
            assert int(fields["k"]) in (1, 2, 4, 8)
            D = shape[2] // shape[3]
            assert int(fields["cw"]) % D == 0  # a cluster owns whole groups
            assert nt.launch_count(*shape, dtype, direction) == (1 if direction == 0 else 2)


def test_planner_invariants_over_random_shapes():
    # every plan must fit the SM (shared memory, threads), keep whole groups inside a cluster's
    # column block, and never ask for more scratch than the workspace query reports
    import random

    rng = random.Random(7)
    codes = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
    for _ in range(400):
        G = rng.choice([1, 2, 3, 4, 8, 16, 32, 64])
        D = rng.choice([1, 2, 3, 4, 5, 8, 10, 16, 20, 40, 64])
        C = G * D
        R = rng.choice([1, 7, 49, 64, 255, 256, 1024, 3136, 4096, 16384, 65536, 1 << 20])
        N = rng.choice([1, 2, 3, 8, 64])
        dtype = rng.choice(list(codes))
        if N * R * C > 1 << 31:
            continue
        for direction in (0, 1):
            text = nt.describe_plan(N, R, C, G, dtype, direction)
            fields = dict(kv.split("=") for kv in text.split()[2:])
            threads, smem, cw, ve, k = (int(fields[x]) for x in ("threads", "smem", "cw", "ve", "k"))
            assert threads % 32 == 0 and 32 <= threads <= 512, text
            assert smem <= 227 * 1024, text
            assert cw % ve == 0 and int(fields["grid"]) >= 1, text
            if " fused " in text:
                assert cw % D == 0 and C % cw == 0 and k in (1, 2, 4, 8), text
                assert int(fields["rows"]) * k >= R, text
            query = nt.lib.gnb200_fwd_workspace_bytes if direction == 0 else nt.lib.gnb200_bwd_workspace_bytes
            assert int(fields["ws"]) <= query(N, R, C, G, codes[dtype]), text


def test_planner_env_override(monkeypatch):
    monkeypatch.setenv("GNB200_FORCE_PATH", "twopass")
    assert " twopass " in nt.describe_plan(2, 1024, 128, 32, torch.float32, 0)
    monkeypatch.delenv("GNB200_FORCE_PATH")
    assert " fused " in nt.describe_plan(2, 1024, 128, 32, torch.float32, 0)


def test_module_interface_matches_reference():
    m = pkg.GN_NHWC(32, 128, activation="silu", eps=1e-6)
    assert isinstance(m, torch.nn.GroupNorm)
    assert m.activation == "silu" and m.act_code == 2 and m.eps == 1e-6 and m.affine
    assert set(m.state_dict().keys()) == {"weight", "bias"}
    assert repr(m) == "GN_NHWC(32, 128, eps=1e-06, affine=True, activation=silu)"
    assert pkg.GN_NHWC(4, 8, activation="swish").act_code == 2
    with pytest.raises(KeyError):
        pkg.GN_NHWC(4, 8, activation="mish")
    plain = torch.nn.GroupNorm(32, 128)
    m.load_state_dict(plain.state_dict())  # checkpoints of nn.GroupNorm load unchanged
    assert pkg.GN_NHWC(4, 8, affine=False).weight is None


def test_module_refuses_cpu_and_channels_first_inputs():
    m = pkg.GN_NHWC(4, 8)
    with pytest.raises(ValueError, match="CUDA"):
        m(torch.randn(2, 8, 4, 4).to(memory_format=torch.channels_last))
    with pytest.raises(ValueError, match="CUDA"):
        pkg.GN_NHWC_Func.apply(torch.randn(2, 8, 4, 4), m.weight, m.bias, 4, 1e-5, 0)


def test_module_refuses_a_peer_exchange_made_for_another_channel_count():
    from channels_last_groupnorm_b200 import dist as gd

    px = object.__new__(gd.PeerExchange)  # no process group here: only the attribute the check reads
    px.num_channels = 16
    m = pkg.GN_NHWC(4, 8, process_group=px)
    with pytest.raises(ValueError, match="made for 16 channels"):
        pkg.GN_NHWC_Func.apply(torch.randn(2, 8, 4, 4), m.weight, m.bias, 4, 1e-5, 0, px)


def test_torch_ops_are_registered_with_reference_schemas():
    fwd = torch.ops.gnb200.fwd.default._schema
    bwd = torch.ops.gnb200.bwd.default._schema
    assert [a.type.kind() for a in fwd.arguments] == ["TensorType"] * 3 + ["IntType", "FloatType", "IntType"]
    assert len(fwd.returns) == 3
    assert [a.type.kind() for a in bwd.arguments] == ["TensorType"] * 6 + ["IntType", "IntType"]
    assert len(bwd.returns) == 3
    with pytest.raises(RuntimeError, match="CUDA"):
        torch.ops.gnb200.fwd(torch.randn(1, 8, 4).permute(0, 2, 1), torch.ones(8), torch.zeros(8), 2, 1e-5, 0)


def test_fake_tensor_kernels_describe_the_outputs():
    # shapes, strides and dtypes without a device: what torch.compile sees of the ops
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        X = torch.empty(2, 16, 8, dtype=torch.bfloat16, device="meta").permute(0, 2, 1)
        w = torch.empty(8, dtype=torch.bfloat16, device="meta")
        b = torch.empty(8, dtype=torch.bfloat16, device="meta")
        Y, means, rstds = torch.ops.gnb200.fwd(X, w, b, 2, 1e-5, 3)
        assert Y.shape == X.shape and Y.stride() == X.stride() and Y.dtype == X.dtype
        assert means.shape == (2, 2) and means.dtype == torch.float32 and rstds.shape == (2, 2)
        dX, dw, db = torch.ops.gnb200.bwd(Y, X, w, b, means, rstds, 2, 3)
        assert dX.stride() == X.stride() and dw.shape == (8,) and db.dtype == torch.bfloat16
        dX, dparam = torch.ops.gnb200.bwd_f32(Y, X, w, b, means, rstds, 2, 3)
        assert dparam.shape == (2, 8) and dparam.dtype == torch.float32
        dX, dparam = torch.ops.gnb200.bwd_f32_peer(Y, X, w, b, means, rstds, 2, 3, [1 << 20, 2 << 20], 1)
        assert dX.stride() == X.stride() and dparam.shape == (2, 8) and dparam.dtype == torch.float32
