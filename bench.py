#!/usr/bin/env python
"""Benchmark of the channels-last GroupNorm hot path on B200.

    python bench.py [--gpus N --steps K --warmup W]          # one JSON line (rank 0)
    python bench.py --impl reference ...                      # the CPU reference arm
    python bench.py --sweep [--out FILE]                      # every benchmark shape, one JSON line each

Workload of the headline line ("cfg4"): GroupNorm + GELU(erf), bf16, NHWC, global batch 64 of
256 x 64 x 64, 32 groups, eps 1e-5, forward + backward; the batch is split evenly over the ranks
(strong scaling) and the packed fp32 [dgamma | dbeta] buffer is summed over the ranks - by the
library's own kernels over peer-mapped memory or by an NCCL all-reduce (--collective; `auto` times
the arrangements, reports them under "collectives" and takes the fastest).  A step is one forward
+ one backward over the rank's samples.  Inputs are seeded synthetic tensors
(x ~ N(0,1), gamma ~ U(0.5,1.5), beta ~ N(0,0.01), dy ~ N(0,1)).

value      aggregate algorithmic bytes (5 * E * sizeof: read x, write y | read x, dy, write dx)
           of all ranks / max-over-ranks device time per step, inputs resident in HBM, through the
           C ABI (gnb200_fwd / gnb200_bwd).  Buffers rotate over enough copies that no step finds
           its inputs in L2.
e2e        same metric through the public module (GN_NHWC + autograd) with the step's x and dy
           copied from pinned host memory and y, dx, dgamma, dbeta copied back, all inside the
           timed region.
roofline   the backward call (the dominant kernel plus its 2-microsecond parameter-gradient
           kernel) and, as `roofline_fwd`, the forward kernel: algorithmic bytes / CUDA-event
           duration against the measured copy bandwidth in MEASURED_PEAKS.json.
cpu_baseline  torch.nn.functional.group_norm + activation on the host cores (channels_last, same
           dtype, autograd backward) on a bounded sample of the same workload.
parity_check  values of the sharded run, checked on this hardware before anything is timed (shard
           against full batch bit for bit, summed gradients against the full-batch ones, the
           in-kernel exchange in every form, the module, torch's fp64); a failure exits non-zero.
vae_sd_shapes  device times and roofline fractions of the VAE-decoder and SD-UNet shapes (1 GPU),
           cold (rotating buffers) and, labelled `_hot`, with one buffer set.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
DT_SHORT = {"float32": "f32", "float16": "f16", "bfloat16": "bf16"}
L2_BYTES = 126 * 1024 * 1024
FALLBACK_HBM_GBS = 6650.0

WORKLOADS = {
    # name: N, C, H, W, G, eps, act, dtype, x scale, backward?, x distribution
    "cfg1": (2, 128, 32, 32, 32, 1e-5, "identity", "float32", 1.0, True, "normal"),
    "cfg2_320x64": (1, 320, 64, 64, 32, 1e-5, "silu", "float16", 1.0, False, "normal"),
    "cfg2_640x32": (1, 640, 32, 32, 32, 1e-5, "silu", "float16", 1.0, False, "normal"),
    "cfg2_1280x16": (1, 1280, 16, 16, 32, 1e-5, "silu", "float16", 1.0, False, "normal"),
    "cfg2_1280x8": (1, 1280, 8, 8, 32, 1e-5, "silu", "float16", 1.0, False, "normal"),
    "cfg3_512x128": (1, 512, 128, 128, 32, 1e-6, "silu", "float16", 2.0, True, "normal"),
    "cfg3_512x256": (1, 512, 256, 256, 32, 1e-6, "silu", "float16", 2.0, True, "normal"),
    "cfg3_256x512": (1, 256, 512, 512, 32, 1e-6, "silu", "float16", 2.0, True, "normal"),
    "cfg3_128x1024": (1, 128, 1024, 1024, 32, 1e-6, "silu", "float16", 2.0, True, "normal"),
    "cfg4": (64, 256, 64, 64, 32, 1e-5, "gelu", "bfloat16", 1.0, True, "normal"),
    "cfg4_n32": (32, 256, 64, 64, 32, 1e-5, "gelu", "bfloat16", 1.0, True, "normal"),
    "cfg4_n16": (16, 256, 64, 64, 32, 1e-5, "gelu", "bfloat16", 1.0, True, "normal"),
    "cfg4_n8": (8, 256, 64, 64, 32, 1e-5, "gelu", "bfloat16", 1.0, True, "normal"),
    "cfg5_96x7_f32": (8, 96, 7, 7, 3, 1e-5, "gelu_tanh", "float32", 1.0, True, "uniform3"),
    "cfg5_64x56_f32": (4, 64, 56, 56, 64, 1e-5, "gelu_tanh", "float32", 1.0, True, "uniform3"),
    "cfg5_2048x7_f32": (16, 2048, 7, 7, 32, 1e-5, "relu", "float32", 1.0, True, "uniform3"),
    "cfg5_40x17x33_f32": (3, 40, 17, 33, 8, 1e-5, "gelu_tanh", "float32", 1.0, True, "uniform3"),
    "cfg5_2048x7_bf16": (16, 2048, 7, 7, 32, 1e-5, "gelu_tanh", "bfloat16", 1.0, True, "uniform3"),
    "cfg5_64x56_bf16": (4, 64, 56, 56, 64, 1e-5, "relu", "bfloat16", 1.0, True, "uniform3"),
}
HEADLINE = "cfg4"
ACT_CODES = {"identity": 0, "relu": 1, "silu": 2, "gelu": 3, "gelu_tanh": 4}


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------------------------------------
# seeded synthetic inputs (same generator order as the tests: x, gamma, beta, dy)
# ------------------------------------------------------------------------------------------------
def make_inputs(N, C, H, W, dtype, seed=0, x_scale=1.0, dist="normal"):
    g = torch.Generator().manual_seed(seed)
    if dist == "uniform3":
        x = torch.rand((N, H, W, C), generator=g) * 6.0 - 3.0
    else:
        x = torch.randn((N, H, W, C), generator=g) * x_scale
    gamma = torch.rand(C, generator=g) + 0.5
    beta = torch.randn(C, generator=g) * 0.1
    dy = torch.randn((N, H, W, C), generator=g)
    return x.to(dtype), gamma.to(dtype), beta.to(dtype), dy.to(dtype)  # NHWC-contiguous


def torch_act(name):
    import torch.nn.functional as F

    return {"identity": lambda t: t, "relu": F.relu, "silu": F.silu, "gelu": F.gelu,
            "gelu_tanh": lambda t: F.gelu(t, approximate="tanh")}[name]


# ------------------------------------------------------------------------------------------------
# clock sampling during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ts, line in self.lines:
            if t0 is not None and not (t0 - 0.02 <= ts <= t1 + 0.04):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:  # region shorter than one sample: fall back to everything that was seen
            return self.stop_all()
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}

    def stop_all(self):
        sm, mx = [], []
        for _, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": [], "samples": len(sm), "note": "timed region shorter than the sampling period"}


# ------------------------------------------------------------------------------------------------
# CPU arm: torch group_norm + activation on the host cores (bounded sample)
# ------------------------------------------------------------------------------------------------
def cpu_step_fn(wl, n_sample):
    import torch.nn.functional as F

    N, C, H, W, G, eps, act, dt, xs, bwd, dist = WORKLOADS[wl]
    dtype = DT[dt]
    x, ga, be, dy = make_inputs(n_sample, C, H, W, dtype, 0, xs, dist)
    x = x.permute(0, 3, 1, 2).requires_grad_(bwd)  # channels_last strides
    dy = dy.permute(0, 3, 1, 2)
    ga.requires_grad_(bwd)
    be.requires_grad_(bwd)
    fn = torch_act(act)

    def step():
        y = fn(F.group_norm(x, G, ga, be, eps))
        if bwd:
            torch.autograd.grad(y, (x, ga, be), dy)
        return y

    elems = n_sample * C * H * W
    alg_bytes = (5 if bwd else 2) * elems * x.element_size()
    return step, alg_bytes


def time_cpu(wl, n_sample, budget_s=12.0, min_iters=3, warmup=2):
    torch.set_num_threads(os.cpu_count() or 1)
    step, alg_bytes = cpu_step_fn(wl, n_sample)
    for _ in range(warmup):
        step()
    times = []
    t_end = time.time() + budget_s
    while len(times) < min_iters or (time.time() < t_end and len(times) < 200):
        t = time.perf_counter()
        step()
        times.append(time.perf_counter() - t)
    med = statistics.median(times)
    return alg_bytes / med / 1e9, med, len(times)


def reference_arm(args):
    """CPU reference arm: every step is a bounded sample of the headline workload on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = args.workload
    N, C, H, W, G, eps, act, dt, xs, bwd, dist = WORKLOADS[wl]
    n_sample = min(N, 8)
    torch.set_num_threads(os.cpu_count() or 1)
    step, alg_bytes = cpu_step_fn(wl, n_sample)
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt_s = (time.perf_counter() - t0) / args.steps
    value = alg_bytes / dt_s / 1e9
    sample = "%d of %d samples per step, torch.nn.functional.group_norm + %s, channels_last %s, autograd backward" % (
        n_sample, N, act, dt)
    line = {
        "impl": "reference", "metric": "gn_nhwc_fwd_bwd_achieved_GBps", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt_s * 1e3,
        "us_per_call_scaled_to_full_batch": dt_s * 1e6 * N / n_sample,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DT_SHORT[dt],
        "data": "synthetic", "config": workload_config(wl, args.gpus),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(wl, gpus):
    N, C, H, W, G, eps, act, dt, xs, bwd, dist = WORKLOADS[wl]
    return {"workload": "%s: GroupNorm+%s %s NHWC N=%d C=%d %dx%d G=%d eps=%g %s" % (
        wl, act, dt, N, C, H, W, G, eps, "fwd+bwd" if bwd else "fwd"),
        "global_batch": N, "per_gpu_batch": N // gpus, "parallelism": "batch-sharded x%d" % gpus,
        "l2_policy": "buffers rotate over copies totalling > 1 GiB, so inputs are never L2-resident"}


# ------------------------------------------------------------------------------------------------
# device arm
# ------------------------------------------------------------------------------------------------
class DeviceProblem:
    """Preallocated buffers for one workload on the current device, rotated to defeat L2 reuse."""

    def __init__(self, wl, n_local, x, ga, be, dy, min_total_bytes=1 << 30, peer=None, peer_mode="peer"):
        from channels_last_groupnorm_b200 import _native as nt

        self.nt = nt
        # dist.PeerExchange.  peer_mode "peer-inline": the backward posts [dgamma | dbeta] into the ranks' exchange
        # buffers from its own kernels and collects the sums in the same call; "peer": posts, and collects one step
        # later; "peer-side": plain backward, then the library's exchange kernel on a side stream (where the NCCL
        # variant runs its all-reduce)
        self.peer = peer
        self.peer_mode = peer_mode
        self.peer_inline = peer_mode == "peer-inline"
        self.peer_table = nt._peer_table(peer.peer_ptrs) if peer is not None else None
        N, C, H, W, G, eps, act, dt, xs, bwd, dist = WORKLOADS[wl]
        self.n, self.C, self.R, self.G, self.eps, self.act, self.bwd = n_local, C, H * W, G, eps, ACT_CODES[act], bwd
        self.dtype = DT[dt]
        self.code = nt.DTYPE_CODES[self.dtype]
        dev = torch.device("cuda", torch.cuda.current_device())
        per_set = x.numel() * x.element_size() * (4 if bwd else 2)
        self.nsets = max(2, min(64, -(-min_total_bytes // per_set)))
        self.sets = []
        for _ in range(self.nsets):
            s = {"x": x.to(dev).contiguous(), "y": torch.empty(x.shape, dtype=self.dtype, device=dev)}
            if bwd:
                s["dy"] = dy.to(dev).contiguous()
                s["dx"] = torch.empty(x.shape, dtype=self.dtype, device=dev)
            self.sets.append(s)
        self.ga, self.be = ga.to(dev), be.to(dev)
        self.mean = torch.empty((n_local, G), dtype=torch.float32, device=dev)
        self.rstd = torch.empty((n_local, G), dtype=torch.float32, device=dev)
        # two slots, so that the all-reduce of step i can overlap the kernels of step i+1
        self.dparams = [torch.empty((2, C), dtype=torch.float32, device=dev) for _ in range(2)]
        self.dparam = self.dparams[0]
        self.dgdb = [torch.empty((2, C), dtype=self.dtype, device=dev) for _ in range(2)]
        self.dgamma = torch.empty(C, dtype=self.dtype, device=dev)
        self.dbeta = torch.empty(C, dtype=self.dtype, device=dev)
        wf = nt.lib.gnb200_fwd_workspace_bytes(n_local, self.R, C, G, self.code)
        wb = nt.lib.gnb200_bwd_workspace_bytes(n_local, self.R, C, G, self.code)
        self.ws_f = torch.empty(max(wf, 16), dtype=torch.uint8, device=dev)
        self.ws_b = torch.empty(max(wb, 16), dtype=torch.uint8, device=dev)
        self.wf, self.wb = wf, wb
        self.elems = x.numel()
        self.esize = x.element_size()
        self.launches_fwd = nt.launch_count(n_local, self.R, C, G, self.dtype, 0)
        self.launches_bwd = nt.launch_count(n_local, self.R, C, G, self.dtype, 1) if bwd else 0

    def fwd(self, i, stream):
        s = self.sets[i % self.nsets]
        lib = self.nt.lib
        self.nt.check(lib.gnb200_fwd(s["x"].data_ptr(), self.ga.data_ptr(), self.be.data_ptr(), self.n, self.R, self.C,
                                     self.G, self.eps, self.act, self.code, s["y"].data_ptr(), self.mean.data_ptr(),
                                     self.rstd.data_ptr(), self.ws_f.data_ptr() if self.wf else None, self.wf, stream))

    def bwd_(self, i, stream, typed, slot=0, peer=False):
        s = self.sets[i % self.nsets]
        lib = self.nt.lib
        dparam = self.dparams[slot]
        if peer and self.peer_inline:
            self.nt.check(lib.gnb200_bwd_peer(s["dy"].data_ptr(), s["x"].data_ptr(), self.ga.data_ptr(), self.be.data_ptr(),
                                              self.mean.data_ptr(), self.rstd.data_ptr(), self.n, self.R, self.C, self.G,
                                              self.act, self.code, s["dx"].data_ptr(), dparam.data_ptr(),
                                              self.dgamma.data_ptr() if typed else None,
                                              self.dbeta.data_ptr() if typed else None,
                                              self.ws_b.data_ptr() if self.wb else None, self.wb,
                                              self.peer_table, self.peer.rank, self.peer.world, stream))
            return
        if peer:
            self.nt.check(lib.gnb200_bwd_peer_push(s["dy"].data_ptr(), s["x"].data_ptr(), self.ga.data_ptr(),
                                                   self.be.data_ptr(), self.mean.data_ptr(), self.rstd.data_ptr(), self.n,
                                                   self.R, self.C, self.G, self.act, self.code, s["dx"].data_ptr(),
                                                   dparam.data_ptr(), self.ws_b.data_ptr() if self.wb else None, self.wb,
                                                   self.peer_table, self.peer.rank, self.peer.world, stream))
            return
        self.nt.check(lib.gnb200_bwd(s["dy"].data_ptr(), s["x"].data_ptr(), self.ga.data_ptr(), self.be.data_ptr(),
                                     self.mean.data_ptr(), self.rstd.data_ptr(), self.n, self.R, self.C, self.G,
                                     self.act, self.code, s["dx"].data_ptr(), dparam.data_ptr(),
                                     self.dgamma.data_ptr() if typed else None,
                                     self.dbeta.data_ptr() if typed else None,
                                     self.ws_b.data_ptr() if self.wb else None, self.wb, stream))


def _collect(prob, slot, stream):
    """Sums over the ranks of the oldest posted gradients -> prob.dparams[slot] and the typed copies."""
    prob.nt.check(prob.nt.lib.gnb200_peer_collect(prob.dparams[slot].data_ptr(), prob.dgdb[slot][0].data_ptr(),
                                                  prob.dgdb[slot][1].data_ptr(), prob.C, prob.code, prob.peer_table,
                                                  prob.peer.rank, prob.peer.world, stream))


def _allreduce_peer(prob, slot, stream):
    """prob.dparams[slot] (this rank's sums) -> sums over the ranks, in place, plus the typed copies."""
    prob.nt.check(prob.nt.lib.gnb200_allreduce_param_grads(prob.dparams[slot].data_ptr(), prob.dgdb[slot][0].data_ptr(),
                                                           prob.dgdb[slot][1].data_ptr(), prob.C, prob.code,
                                                           prob.peer_table, prob.peer.rank, prob.peer.world, stream))


def _capture(fn, count):
    """Captures `count` calls fn(i) into one CUDA graph (on a side stream). Returns the graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(count):
            fn(i)
    torch.cuda.current_stream().wait_stream(side)
    return graph


kReplays = 9  # timed replays of the K-step graph


def _time_graph(graph, barrier):
    """Device time of one replay: barrier + synchronize on both sides, CUDA events around it."""
    barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    a.record()
    graph.replay()
    b.record()
    torch.cuda.synchronize()
    t1 = time.time()
    barrier()
    return a.elapsed_time(b) * 1e-3, (t0, t1)


def run_device_steps(prob, steps, warmup, world, barrier, use_graph=True):
    """Times exactly `steps` steps (forward, backward, all-reduce of the parameter gradients).

    Returns (seconds per step, max over ranks; mean forward seconds; mean backward seconds; wall
    interval of the timed region; how the loop was issued).  The K steps are captured once into a
    CUDA graph and replayed, so that host launch overhead does not enter the device time; the
    forward-only and backward-only graphs give the per-kernel durations for the roofline.  If
    capture is not possible the same loop runs eagerly with events around every call.
    """
    import torch.distributed as dist

    def cur():
        return torch.cuda.current_stream().cuda_stream

    side = torch.cuda.Stream() if world > 1 else None
    done = [None, None]  # per slot: event after which its all-reduced gradients are complete
    pending = [None]     # peer exchange: slot whose gradients are posted but not collected yet

    def one(i):
        """Forward, backward and - on more than one rank - the all-reduce of the packed fp32
        [dgamma | dbeta] buffer plus its cast to the tensor dtype.  The collective runs on a side
        stream and alternates between two buffers, so it overlaps the next step's kernels, as a
        gradient all-reduce overlaps the rest of a backward pass in training."""
        b = i & 1
        prob.fwd(i, cur())
        if prob.bwd and prob.peer is not None and prob.peer_mode != "peer-side":
            # the kernels of the backward post the gradients into every rank's exchange buffer (no library
            # collective); their sums are collected inside the same call, or - the default - one step later,
            # when every rank's contribution has long arrived, as a gradient all-reduce is awaited only before
            # the optimizer step
            prob.bwd_(i, cur(), typed=True, slot=b, peer=True)
            if not prob.peer_inline:
                if pending[0] is not None:
                    _collect(prob, pending[0], cur())
                pending[0] = b
        elif prob.bwd:
            if world > 1 and done[b] is not None:
                torch.cuda.current_stream().wait_event(done[b])  # slot b is free again
            prob.bwd_(i, cur(), typed=(world == 1), slot=b)
            if world > 1:
                ready = torch.cuda.Event()
                ready.record(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    side.wait_event(ready)
                    if prob.peer is not None:   # the library's own exchange kernel instead of NCCL + cast
                        _allreduce_peer(prob, b, side.cuda_stream)
                    else:
                        dist.all_reduce(prob.dparams[b])
                        prob.dgdb[b].copy_(prob.dparams[b])
                    done[b] = torch.cuda.Event()
                    done[b].record(side)

    def join():
        """Makes the current stream wait for the collectives still running on the side stream (NCCL), or
        collects the gradients posted last (peer exchange)."""
        if pending[0] is not None:
            _collect(prob, pending[0], cur())
            pending[0] = None
        for b in (0, 1):
            if done[b] is not None:
                torch.cuda.current_stream().wait_event(done[b])

    # the ranks enter together: the kernels of the in-kernel exchange wait only about a second for one another
    torch.cuda.synchronize()
    barrier()
    for i in range(warmup):
        one(i)
    join()
    torch.cuda.synchronize()
    done[0] = done[1] = None

    def reduce_max(v):
        if world > 1:
            t = torch.tensor([v], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return v

    if use_graph:
        try:
            def step_and_join(i):
                one(warmup + i)
                if i == steps - 1:
                    join()

            g_step = _capture(step_and_join, steps)
            done[0] = done[1] = None
            g_fwd = _capture(lambda i: prob.fwd(i, cur()), steps)
            g_bwd = _capture(lambda i: prob.bwd_(i, cur(), typed=True), steps) if prob.bwd else None
            for g in (g_step, g_fwd, g_bwd):  # one untimed replay each
                if g is not None:
                    g.replay()
            torch.cuda.synchronize()
            # the K-step graph is timed kReplays times, each replay bracketed on its own; the median
            # replay is reported and the clock sampler sees the whole sequence (tens of milliseconds)
            runs = [_time_graph(g_step, barrier) for _ in range(kReplays)]
            total = statistics.median(r[0] for r in runs)
            wall = (runs[0][1][0], runs[-1][1][1])
            fwd_t = statistics.median(_time_graph(g_fwd, barrier)[0] for _ in range(kReplays)) / steps
            bwd_t = (statistics.median(_time_graph(g_bwd, barrier)[0] for _ in range(kReplays)) / steps
                     if g_bwd is not None else 0.0)
            # the same K steps issued call by call (host launch overhead included), for comparison
            done[0] = done[1] = None
            barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(steps):
                one(warmup + i)
            join()
            e1.record()
            torch.cuda.synchronize()
            barrier()
            run_device_steps.eager_per_step = reduce_max(e0.elapsed_time(e1) * 1e-3 / steps)
            return reduce_max(total / steps), fwd_t, bwd_t, wall, "cuda-graph"
        except Exception as exc:  # pragma: no cover - depends on driver / NCCL capture support
            sys.stderr.write("bench: CUDA-graph capture failed (%s); timing the eager loop\n" % str(exc)[:200])
            torch.cuda.synchronize()

    barrier()
    torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    start.record()
    for i in range(steps):
        b = i & 1
        evs[i][0].record()
        prob.fwd(warmup + i, cur())
        evs[i][1].record()
        if prob.bwd and prob.peer is not None and prob.peer_mode != "peer-side":
            prob.bwd_(warmup + i, cur(), typed=True, slot=b, peer=True)
            evs[i][2].record()
            if not prob.peer_inline:
                if pending[0] is not None:
                    _collect(prob, pending[0], cur())
                pending[0] = b
        elif prob.bwd:
            if world > 1 and done[b] is not None:
                torch.cuda.current_stream().wait_event(done[b])
            prob.bwd_(warmup + i, cur(), typed=(world == 1), slot=b)
            evs[i][2].record()
            if world > 1:
                ready = torch.cuda.Event()
                ready.record(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    side.wait_event(ready)
                    if prob.peer is not None:
                        _allreduce_peer(prob, b, side.cuda_stream)
                    else:
                        dist.all_reduce(prob.dparams[b])
                        prob.dgdb[b].copy_(prob.dparams[b])
                    done[b] = torch.cuda.Event()
                    done[b].record(side)
    join()
    stop.record()
    torch.cuda.synchronize()
    t_wall1 = time.time()
    barrier()
    total = start.elapsed_time(stop) * 1e-3
    fwd_t = sum(e[0].elapsed_time(e[1]) for e in evs) * 1e-3 / steps
    bwd_t = sum(e[1].elapsed_time(e[2]) for e in evs) * 1e-3 / steps if prob.bwd else 0.0
    run_device_steps.eager_per_step = reduce_max(total / steps)
    return reduce_max(total / steps), fwd_t, bwd_t, (t_wall0, t_wall1), "eager"


run_device_steps.eager_per_step = None


def run_e2e(wl, n_local, x, ga, be, dy, steps, warmup, world, barrier, peer=None):
    """Public API (module + autograd) with host buffers; every step copies its x and dy from pinned
    host memory and its y, dx, dgamma, dbeta back, all inside the timed region.

    The three legs of a step run on three streams (copy-in, compute, copy-out) over two sets of
    device buffers, so the upload of step i+1 and the download of step i-1 overlap the kernels of
    step i, as in an input pipeline; every byte still crosses PCIe once per step.
    """
    import torch.distributed as dist

    import channels_last_groupnorm_b200 as pkg

    N, C, H, W, G, eps, act, dt, xs, bwd, dist_name = WORKLOADS[wl]
    dtype = DT[dt]
    dev = torch.device("cuda", torch.cuda.current_device())
    m = pkg.GN_NHWC(G, C, activation=act, eps=eps,
                    process_group=(peer if peer is not None else dist.group.WORLD if world > 1 else None)).to(dev).to(dtype)
    with torch.no_grad():
        m.weight.copy_(ga)
        m.bias.copy_(be)
    xh, dyh = x.pin_memory(), dy.pin_memory()
    yh = [torch.empty_like(xh).pin_memory() for _ in range(2)]
    dxh = [torch.empty_like(xh).pin_memory() for _ in range(2)]
    dgh = [torch.empty(C, dtype=dtype).pin_memory() for _ in range(2)]
    dbh = [torch.empty(C, dtype=dtype).pin_memory() for _ in range(2)]
    xd = [torch.empty(x.shape, dtype=dtype, device=dev) for _ in range(2)]
    dyd = [torch.empty(x.shape, dtype=dtype, device=dev) for _ in range(2)]
    s_in, s_comp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    used = [False, False]

    def one(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            if used[b]:
                s_in.wait_event(ev_comp[b])  # the device input buffers of this slot are free again
            xd[b].copy_(xh, non_blocking=True)
            if bwd:
                dyd[b].copy_(dyh, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(ev_in[b])
            xin = xd[b].permute(0, 3, 1, 2).detach().requires_grad_(bwd)
            y = m(xin)
            if bwd:
                m.weight.grad = None
                m.bias.grad = None
                y.backward(dyd[b].permute(0, 3, 1, 2))
            ev_comp[b].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])
            if used[b]:
                s_out.wait_event(ev_out[b])
            results = [(yh[b], y.detach().permute(0, 2, 3, 1))]
            if bwd:
                results += [(dxh[b], xin.grad.permute(0, 2, 3, 1)), (dgh[b], m.weight.grad), (dbh[b], m.bias.grad)]
            for host, devt in results:
                devt.record_stream(s_out)
                host.copy_(devt, non_blocking=True)
            ev_out[b].record(s_out)
        used[b] = True

    def drain():
        for st in (s_in, s_comp, s_out):
            torch.cuda.current_stream().wait_stream(st)

    torch.cuda.synchronize()
    barrier()  # the ranks enter together (allocating pinned memory takes a different time on every rank)
    for i in range(warmup):
        one(i)
    drain()
    barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for st in (s_in, s_comp, s_out):
        st.wait_event(start)
    for i in range(steps):
        one(warmup + i)
    drain()
    stop.record()
    torch.cuda.synchronize()
    barrier()
    per_step = start.elapsed_time(stop) * 1e-3 / steps
    if world > 1:
        t = torch.tensor([per_step], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        per_step = float(t.item())
    nbytes = x.numel() * x.element_size()
    h2d = nbytes * (2 if bwd else 1)
    d2h = nbytes * (2 if bwd else 1) + (2 * C * x.element_size() if bwd else 0)
    return per_step, h2d, d2h


def _geometry(plan_text):
    """The fields of a plan description that decide the arithmetic of one (sample, column block) slab."""
    keep = ("ve", "cw", "ncb", "ty", "threads", "rows", "chunks", "k")
    words = plan_text.split()
    fields = dict(w.split("=") for w in words[2:] if "=" in w)
    return (words[1],) + tuple(fields.get(k) for k in keep)


def _rel_err(a, b):
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / max(1.0, float(b.abs().max())))


def run_parity_check(wl, rank, world, x_full, ga, be, dy_full, lo, hi, peer=None):
    """Value check of the sharded run on this hardware, outside every timed region.

    Every rank runs the full global batch once on its own GPU, then its shard; the shard's y and dx must
    equal the matching samples of the full-batch run (bit for bit when both runs use the same slab
    geometry, else within the 16-bit tolerance), the all-reduced packed [dgamma | dbeta] of the shards
    must equal the full-batch one within tolerance, and so must the gradients that come out of the
    public module with process_group set.  The first samples of the shard are also compared with torch's
    fp64 group_norm + activation on the device.
    """
    import torch.distributed as dist

    import channels_last_groupnorm_b200 as pkg
    from channels_last_groupnorm_b200 import _native as nt

    N, C, H, W, G, eps, act, dt, xs, bwd, dist_name = WORKLOADS[wl]
    dtype = DT[dt]
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    dev = torch.device("cuda", torch.cuda.current_device())
    code = ACT_CODES[act]
    R = H * W
    xg, dyg = x_full.to(dev).reshape(N, R, C), dy_full.to(dev).reshape(N, R, C)
    gad, bed = ga.to(dev), be.to(dev)
    y_f, mean_f, rstd_f = nt.fwd_raw(xg, gad, bed, G, eps, code)
    errs, ok = {}, True
    same_geom = _geometry(nt.describe_plan(N, R, C, G, dtype, 0)) == _geometry(nt.describe_plan(hi - lo, R, C, G, dtype, 0))
    xs_, dys_ = xg[lo:hi].contiguous(), dyg[lo:hi].contiguous()
    y_s, mean_s, rstd_s = nt.fwd_raw(xs_, gad, bed, G, eps, code)
    bitwise = bool(torch.equal(y_s, y_f[lo:hi]))
    errs["y_shard_vs_full"] = _rel_err(y_s, y_f[lo:hi])
    if bwd:
        same_geom = same_geom and _geometry(nt.describe_plan(N, R, C, G, dtype, 1)) == _geometry(
            nt.describe_plan(hi - lo, R, C, G, dtype, 1))
        dx_f, dparam_f, _, _ = nt.bwd_raw(dyg, xg, gad, bed, mean_f, rstd_f, G, code)
        dx_s, dparam_s, _, _ = nt.bwd_raw(dys_, xs_, gad, bed, mean_s, rstd_s, G, code)
        bitwise = bitwise and bool(torch.equal(dx_s, dx_f[lo:hi]))
        errs["dx_shard_vs_full"] = _rel_err(dx_s, dx_f[lo:hi])
        if peer is not None:
            torch.cuda.synchronize()
            dist.barrier()  # the ranks enter the exchange together (its waits are bounded at about a second)
            # the in-kernel exchange: the summed gradients must equal the full-batch ones within tolerance, the
            # NCCL-summed ones closely, and be the same bits on every rank (they are added in rank order)
            _, dparam_p = nt.bwd_peer_raw(dys_, xs_, gad, bed, mean_s, rstd_s, G, code, peer.peer_ptrs, peer.rank)
            errs["dparam_peer_vs_full"] = _rel_err(dparam_p, dparam_f)
            first = dparam_p.clone()
            dist.broadcast(first, src=0)
            if not torch.equal(first, dparam_p):
                ok = False
                errs["dparam_peer_differs_between_ranks"] = _rel_err(dparam_p, first) + 1.0
            again = peer.allreduce_(dparam_s.clone())   # the exchange alone, on the local gradients
            errs["dparam_peer_standalone_vs_fused"] = _rel_err(again, dparam_p)
            # push and collect apart, two pushes outstanding (both slot parities), then a third round that has to
            # see the acknowledgements of the first: every collect must return the bits of the one-call form
            worst = 0.0
            for _ in range(2):
                locals_ = [nt.bwd_peer_raw(dys_, xs_, gad, bed, mean_s, rstd_s, G, code, peer.peer_ptrs, peer.rank,
                                           collect=False)[1] for _ in range(2)]
                worst = max(worst, max(_rel_err(t, dparam_s) for t in locals_))   # pushing leaves the local sums
                for _ in range(2):
                    got = peer.collect_(torch.empty_like(dparam_p))
                    worst = max(worst, 0.0 if torch.equal(got, dparam_p) else 1.0 + _rel_err(got, dparam_p))
            errs["dparam_peer_push_collect_vs_fused"] = worst
        if world > 1:
            dist.all_reduce(dparam_s)
        errs["dparam_allreduced_vs_full"] = _rel_err(dparam_s, dparam_f)
        # the public module with process_group: one step on the shard
        m = pkg.GN_NHWC(G, C, activation=act, eps=eps,
                        process_group=(peer if peer is not None else dist.group.WORLD if world > 1 else None)).to(dev).to(dtype)
        with torch.no_grad():
            m.weight.copy_(ga)
            m.bias.copy_(be)
        xin = xs_.reshape(hi - lo, H, W, C).permute(0, 3, 1, 2).detach().requires_grad_(True)
        ym = m(xin)
        ym.backward(dys_.reshape(hi - lo, H, W, C).permute(0, 3, 1, 2))
        errs["module_y_vs_full"] = _rel_err(ym.detach().permute(0, 2, 3, 1).reshape(hi - lo, R, C), y_f[lo:hi])
        errs["module_dx_vs_full"] = _rel_err(xin.grad.permute(0, 2, 3, 1).reshape(hi - lo, R, C), dx_f[lo:hi])
        errs["module_dgamma_vs_full"] = _rel_err(m.weight.grad, dparam_f[0])
        errs["module_dbeta_vs_full"] = _rel_err(m.bias.grad, dparam_f[1])
    # anchor: the first samples of the shard against torch's fp64 group_norm + activation on the device
    k = min(2, hi - lo)
    x64 = xs_[:k].double().reshape(k, H, W, C).permute(0, 3, 1, 2).requires_grad_(bwd)
    g64, b64 = gad.double().requires_grad_(bwd), bed.double().requires_grad_(bwd)
    y64 = torch_act(act)(torch.nn.functional.group_norm(x64, G, g64, b64, eps))
    errs["y_vs_fp64"] = _rel_err(y_s[:k], y64.detach().permute(0, 2, 3, 1).reshape(k, R, C))
    if bwd:
        dx64, = torch.autograd.grad(y64, (x64,), dys_[:k].double().reshape(k, H, W, C).permute(0, 3, 1, 2))
        errs["dx_vs_fp64"] = _rel_err(dx_s[:k], dx64.permute(0, 2, 3, 1).reshape(k, R, C))
    torch.cuda.synchronize()
    if same_geom and not bitwise:
        ok = False
    ok = ok and all(e <= tol for e in errs.values())
    ok = ok and nt.wait_timeouts() == 0
    if world > 1:
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(flag.item())
        worst = torch.tensor([errs[k_] for k_ in sorted(errs)], device=dev, dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        errs = {k_: float(v) for k_, v in zip(sorted(errs), worst.tolist())}
    return {"ok": ok, "ranks": world, "tolerance": tol, "same_slab_geometry": bool(same_geom),
            "shard_bitwise_equal_to_full_batch": bitwise, "max_rel_err": errs}


SHAPE_TABLE = ("cfg3_512x128", "cfg3_512x256", "cfg3_256x512", "cfg3_128x1024",
               "cfg2_320x64", "cfg2_640x32", "cfg2_1280x16", "cfg2_1280x8")


def shape_table(peak):
    """Device time of the VAE-decoder (cfg3) and SD-UNet (cfg2) shapes, same protocol as the headline:
    buffers rotating over > 1 GiB, 20 calls per CUDA graph, median of five replays."""
    from channels_last_groupnorm_b200 import _native as nt

    rows = []
    for wl in SHAPE_TABLE:
        N, C, H, W, G, eps, act, dt, xs, bwd, dist_name = WORKLOADS[wl]
        dtype = DT[dt]
        x, ga, be, dy = make_inputs(N, C, H, W, dtype, 0, xs, dist_name)
        prob = DeviceProblem(wl, N, x, ga, be, dy)
        E, es = x.numel(), x.element_size()
        cur = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
        t, _ = time_cuda(lambda i: prob.fwd(i, cur()))
        rec = {"workload": workload_config(wl, 1)["workload"], "us_fwd": t * 1e6, "frac_fwd": 2 * E * es / t / 1e9 / peak,
               "plan": nt.describe_plan(N, H * W, C, G, dtype, 0)}
        # hot mode: the same buffers every call, so whatever fits L2 stays there (labelled; not the headline)
        rec["us_fwd_hot"] = time_cuda(lambda i: prob.fwd(0, cur()))[0] * 1e6
        if bwd:
            t, _ = time_cuda(lambda i: prob.bwd_(i, cur(), True))
            rec.update(us_bwd=t * 1e6, frac_bwd=3 * E * es / t / 1e9 / peak,
                       plan_bwd=nt.describe_plan(N, H * W, C, G, dtype, 1))
            rec["us_bwd_hot"] = time_cuda(lambda i: prob.bwd_(0, cur(), True))[0] * 1e6
        rows.append(rec)
        del prob
        torch.cuda.empty_cache()
    return rows


def device_arm(args):
    with _StdoutToStderr():
        line = _device_arm(args)
    if line is not None:
        print(json.dumps(line), flush=True)


def _device_arm(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()

    from channels_last_groupnorm_b200 import _native as nt
    from channels_last_groupnorm_b200.dist import shard_bounds

    wl = args.workload
    N, C, H, W, G, eps, act, dt, xs, bwd, dist_name = WORKLOADS[wl]
    dtype = DT[dt]
    x, ga, be, dy = make_inputs(N, C, H, W, dtype, 0, xs, dist_name)  # the global seeded batch
    lo, hi = shard_bounds(N, rank, world)
    # more than one rank: the parameter gradients are summed inside the backward kernels over peer-mapped
    # exchange buffers (--collective peer-inline / peer / peer-side) or by an NCCL all-reduce on a side stream
    # (--collective nccl).  auto: the in-kernel exchange (collected inside the backward call, or by the library's
    # exchange kernel on a side stream, where the NCCL arrangement runs its all-reduce) and NCCL are timed, each with
    # the full protocol; the fastest gives the headline and all are reported ("collectives" in the line); the
    # in-kernel exchange is value-checked on the hardware in every case.
    peer, collective = None, ("none" if world == 1 else "nccl")
    if world > 1 and bwd and args.collective in ("auto", "peer", "peer-inline", "peer-side"):
        try:
            from channels_last_groupnorm_b200.dist import PeerExchange
            peer = PeerExchange(C)
            collective = args.collective if args.collective != "auto" else "peer-inline"
        except Exception as exc:
            if args.collective != "auto":
                raise
            sys.stderr.write("bench: no peer exchange (%s); using NCCL\n" % str(exc)[:300])
        # the choice must be the same on every rank
        flag = torch.tensor([1 if peer is not None else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            peer, collective = None, "nccl"
    parity = None if args.no_parity else run_parity_check(wl, rank, world, x, ga, be, dy, lo, hi, peer)
    torch.cuda.empty_cache()
    x, dy = x[lo:hi].contiguous(), dy[lo:hi].contiguous()
    n_local = hi - lo

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    collectives = {}
    modes = [collective]
    if args.collective == "auto" and peer is not None:
        modes = ["peer-inline", "peer-side", "nccl"]
    best = None
    for mode in modes:
        prob = DeviceProblem(wl, n_local, x, ga, be, dy, peer=(peer if mode.startswith("peer") else None), peer_mode=mode)
        res = run_device_steps(prob, args.steps, args.warmup, world, barrier, use_graph=not args.no_graph)
        eager = run_device_steps.eager_per_step
        del prob
        torch.cuda.empty_cache()
        collectives[mode] = {"us_per_call": res[0] * 1e6, "us_per_call_eager": eager * 1e6 if eager else None}
        if best is None or res[0] < best[0][0]:   # res[0] is the max over ranks: the same choice on every rank
            best = (res, eager, mode)
    (per_step, fwd_t, bwd_t, wall, issue_mode), run_device_steps.eager_per_step, collective = best
    clocks = sampler.stop(*wall) if rank == 0 else None
    e2e_steps = max(3, min(args.steps, 20))
    e2e_t, h2d, d2h = run_e2e(wl, n_local, x, ga, be, dy, e2e_steps, max(3, min(args.warmup, 5)), world, barrier, peer)

    if rank == 0:
        esize = x.element_size()
        elems_global = N * C * H * W
        elems_local = n_local * C * H * W
        alg_global = (5 if bwd else 2) * elems_global * esize
        peak, peak_kind = measured_hbm_peak()
        bwd_bytes = 3 * elems_local * esize
        fwd_bytes = 2 * elems_local * esize
        dom_bytes, dom_t, dom_name = (bwd_bytes, bwd_t, "backward") if bwd else (fwd_bytes, fwd_t, "forward")
        roof = {"bound": "hbm", "kernel": "%s (%s)" % (dom_name, nt.describe_plan(n_local, H * W, C, G, dtype, 1 if bwd else 0)),
                "achieved": dom_bytes / dom_t / 1e9, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": dom_bytes / dom_t / 1e9 / peak,
                "frac_of_8TBps_nominal": dom_bytes / dom_t / 1e9 / 8000.0,
                "traffic": ncu_traffic(dom_name, nt.describe_plan(n_local, H * W, C, G, dtype, 1 if bwd else 0)),
                "us_per_launch": dom_t * 1e6, "algorithmic_bytes": dom_bytes}
        roof_fwd = {"bound": "hbm", "kernel": "forward (%s)" % nt.describe_plan(n_local, H * W, C, G, dtype, 0),
                    "achieved": fwd_bytes / fwd_t / 1e9, "peak": peak, "unit": "GB/s",
                    "frac": fwd_bytes / fwd_t / 1e9 / peak, "frac_of_8TBps_nominal": fwd_bytes / fwd_t / 1e9 / 8000.0,
                    "traffic": ncu_traffic("forward", nt.describe_plan(n_local, H * W, C, G, dtype, 0)),
                    "us_per_launch": fwd_t * 1e6, "algorithmic_bytes": fwd_bytes}
        line = {
            "metric": "gn_nhwc_fwd_bwd_achieved_GBps", "value": alg_global / per_step / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
            "us_per_call": per_step * 1e6, "us_fwd": fwd_t * 1e6, "us_bwd": bwd_t * 1e6,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DT_SHORT[dt],
            "data": "synthetic", "config": dict(workload_config(wl, world), collective=collective),
            "frac_of_hbm_peak": alg_global / per_step / 1e9 / (peak * world),
            "roofline": roof, "roofline_fwd": roof_fwd,
            "e2e": {"value": alg_global / e2e_t / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_t * 1e3, "steps": e2e_steps,
                    "api": "GN_NHWC module + autograd, pinned host buffers; copy-in / compute / copy-out on three "
                           "streams, two buffer sets"},
            "gpu_launches": args.steps * (nt.launch_count(n_local, H * W, C, G, dtype, 0)
                                          + (nt.launch_count(n_local, H * W, C, G, dtype, 1) if bwd else 0)),
            "clocks": clocks, "issue": issue_mode,
            "us_per_call_eager": (run_device_steps.eager_per_step * 1e6 if run_device_steps.eager_per_step else None),
            # what the step costs beyond its two calls timed alone: the collective's exposed part and the
            # event dependencies between the streams
            "us_collective_exposed": (per_step - fwd_t - bwd_t) * 1e6,
            "collectives": collectives if world > 1 else None,
            "frac_of_8TBps_nominal": alg_global / per_step / 1e9 / (8000.0 * world),
            "parity_check": parity,
        }
        if world == 1 and not args.no_shapes:
            line["vae_sd_shapes"] = shape_table(peak)
        if world == 1 and not args.no_cpu:
            n_sample = min(N, 8)
            v, med, iters = time_cpu(wl, n_sample, budget_s=args.cpu_seconds)
            line["cpu_baseline"] = {
                "value": v, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                "ms_per_sample_step": med * 1e3, "iters": iters,
                "sample": "%d of %d samples, torch.nn.functional.group_norm + %s on CPU, channels_last %s, "
                          "autograd backward, median of %d runs (the sample's 17 MB per tensor may stay in the host's "
                          "L3, which flatters the CPU rate slightly)" % (n_sample, N, act, dt, iters)}
    else:
        line = None
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        if line is not None:
            print(json.dumps(line), flush=True)
        sys.stderr.write("bench: parity check failed: %s\n" % json.dumps(parity))
        sys.exit(1)
    return line


def ncu_traffic(direction, plan):
    """Per-launch DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel from
    the committed ncu summaries, profiles/traffic.json: a list of {"direction", "plan", "traffic",
    "source"} records.  The figure is only reported when the plan string of this run equals the one the
    capture was taken with (a changed launch plan means the capture no longer describes the kernel)."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            table = json.load(f)
    except Exception:
        return None
    for rec in table:
        if rec.get("direction") == direction and rec.get("plan") == plan:
            return rec.get("traffic")
    return None


# ------------------------------------------------------------------------------------------------
# sweep over every benchmark shape (1 GPU): ours vs torch CUDA vs reference kernels vs CPU
# ------------------------------------------------------------------------------------------------
def time_cuda(fn, iters=20, reps=5, warmup=5):
    """Median / min seconds per call of fn(i).  The `iters` calls are captured into one CUDA graph
    and replayed (device time without host launch overhead); falls back to an eager loop."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    graph = None
    try:
        graph = _capture(lambda i: fn(warmup + i), iters)
        graph.replay()
        torch.cuda.synchronize()
    except Exception:
        graph = None
        torch.cuda.synchronize()
    out = []
    k = warmup
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        if graph is not None:
            graph.replay()
        else:
            for _ in range(iters):
                fn(k)
                k += 1
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) * 1e-3 / iters)
    return statistics.median(out), min(out)


def sweep(args):
    from channels_last_groupnorm_b200 import _native as nt
    import torch.nn.functional as F

    torch.cuda.set_device(0)
    peak, peak_kind = measured_hbm_peak()
    ref_lib = os.path.join(ROOT, "oracle", "_ref", "gn_op.so")
    have_ref = os.path.exists(ref_lib) and not args.no_ref
    if have_ref:
        torch.ops.load_library(ref_lib)
    names = args.only.split(",") if args.only else list(WORKLOADS)
    out_f = open(args.out, "a") if args.out else None
    stream = torch.cuda.current_stream().cuda_stream
    for wl in names:
        N, C, H, W, G, eps, act, dt, xs, bwd, dist_name = WORKLOADS[wl]
        dtype = DT[dt]
        x, ga, be, dy = make_inputs(N, C, H, W, dtype, 0, xs, dist_name)
        prob = DeviceProblem(wl, N, x, ga, be, dy)
        esize = x.element_size()
        E = x.numel()
        rec = {"workload": wl, "config": workload_config(wl, 1)["workload"], "plan_fwd": nt.describe_plan(N, H * W, C, G, dtype, 0),
               "plan_bwd": nt.describe_plan(N, H * W, C, G, dtype, 1) if bwd else None, "nsets": prob.nsets,
               "peak_GBps": peak, "peak_kind": peak_kind}
        cur = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731  (the capture stream inside a graph)
        t, tmin = time_cuda(lambda i: prob.fwd(i, cur()))
        rec["ours_fwd_us"] = t * 1e6
        rec["ours_fwd_GBps"] = 2 * E * esize / t / 1e9
        rec["ours_fwd_frac"] = rec["ours_fwd_GBps"] / peak
        rec["ours_fwd_hot_us"] = time_cuda(lambda i: prob.fwd(0, cur()))[0] * 1e6  # hot mode: one buffer set
        if bwd:
            t, tmin = time_cuda(lambda i: prob.bwd_(i, cur(), True))
            rec["ours_bwd_us"] = t * 1e6
            rec["ours_bwd_GBps"] = 3 * E * esize / t / 1e9
            rec["ours_bwd_frac"] = rec["ours_bwd_GBps"] / peak
            rec["ours_bwd_hot_us"] = time_cuda(lambda i: prob.bwd_(0, cur(), True))[0] * 1e6
        # the same problem in channels-first storage through gnb200_fwd_nchw / gnb200_bwd_nchw
        if not args.no_nchw:
            code = ACT_CODES[act]
            nsets = len(prob.sets)
            xs_n = [s_["x"].permute(0, 3, 1, 2).contiguous().reshape(N, C, H * W) for s_ in prob.sets[:min(nsets, 4)]]
            g_n, b_n = prob.ga, prob.be
            t, _ = time_cuda(lambda i: nt.fwd_nchw_raw(xs_n[i % len(xs_n)], g_n, b_n, G, eps, code), iters=10, reps=3, warmup=3)
            rec["nchw_fwd_us"] = t * 1e6
            rec["nchw_fwd_frac"] = 2 * E * esize / t / 1e9 / peak
            if bwd:
                dys_n = [s_["dy"].permute(0, 3, 1, 2).contiguous().reshape(N, C, H * W) for s_ in prob.sets[:len(xs_n)]]
                _, mean_n, rstd_n = nt.fwd_nchw_raw(xs_n[0], g_n, b_n, G, eps, code)
                t, _ = time_cuda(lambda i: nt.bwd_nchw_raw(dys_n[i % len(xs_n)], xs_n[i % len(xs_n)], g_n, b_n, mean_n, rstd_n,
                                                           G, code), iters=10, reps=3, warmup=3)
                rec["nchw_bwd_us"] = t * 1e6
                rec["nchw_bwd_frac"] = 3 * E * esize / t / 1e9 / peak
                del dys_n
            del xs_n
        # torch CUDA group_norm + activation (context)
        fn = torch_act(act)
        sets = prob.sets
        gat, bet = prob.ga, prob.be

        def torch_fwd(i):
            s = sets[i % len(sets)]
            return fn(F.group_norm(s["x"].permute(0, 3, 1, 2), G, gat, bet, eps))

        try:
            t, _ = time_cuda(torch_fwd, iters=10, reps=3, warmup=3)
            rec["torch_cuda_fwd_us"] = t * 1e6
        except Exception as exc:  # pragma: no cover
            rec["torch_cuda_fwd_us"] = None
            rec["torch_cuda_error"] = str(exc)[:200]
        if have_ref:
            code = ACT_CODES[act]

            def ref_fwd(i):
                s = sets[i % len(sets)]
                xf = s["x"].view(N, H * W, C).permute(0, 2, 1)
                return torch.ops.gnop.fwd(xf, gat, bet, G, eps, code)

            t, _ = time_cuda(ref_fwd, iters=10, reps=3, warmup=3)
            rec["ref_fwd_us"] = t * 1e6
            if bwd:
                _, means, rstds = ref_fwd(0)

                def ref_bwd(i):
                    s = sets[i % len(sets)]
                    xf = s["x"].view(N, H * W, C).permute(0, 2, 1)
                    df = s["dy"].view(N, H * W, C).permute(0, 2, 1)
                    return torch.ops.gnop.bwd(df, xf, gat, bet, means, rstds, G, code)

                t, _ = time_cuda(ref_bwd, iters=10, reps=3, warmup=3)
                rec["ref_bwd_us"] = t * 1e6
        del prob, sets
        torch.cuda.empty_cache()
        if not args.no_cpu:
            n_sample = min(N, 8)
            v, med, iters = time_cpu(wl, n_sample, budget_s=2.0, min_iters=2, warmup=1)
            rec["cpu_us_scaled"] = med * 1e6 * N / n_sample
            rec["cpu_cores"] = torch.get_num_threads()
        print(json.dumps(rec), flush=True)
        if out_f:
            out_f.write(json.dumps(rec) + "\n")
            out_f.flush()


def profile_target(args):
    """A few plain calls of the hot path for ncu (`ncu ... python bench.py --workload W --profile 2`)."""
    torch.cuda.set_device(0)
    N, C, H, W, G, eps, act, dt, xs, bwd, dist_name = WORKLOADS[args.workload]
    x, ga, be, dy = make_inputs(N, C, H, W, DT[dt], 0, xs, dist_name)
    if args.nchw:  # the channels-first entry points on NCHW-contiguous copies of the same tensors
        from channels_last_groupnorm_b200 import _native as nt

        code = ACT_CODES[act]
        xn = x.cuda().permute(0, 3, 1, 2).contiguous().reshape(N, C, H * W)
        dn = dy.cuda().permute(0, 3, 1, 2).contiguous().reshape(N, C, H * W)
        gd, bd = ga.cuda(), be.cuda()
        for i in range(args.profile):
            y, mean, rstd = nt.fwd_nchw_raw(xn, gd, bd, G, eps, code)
            if bwd:
                nt.bwd_nchw_raw(dn, xn, gd, bd, mean, rstd, G, code)
        torch.cuda.synchronize()
        print("profiled", args.workload, "channels-first", args.profile, "calls")
        return
    prob = DeviceProblem(args.workload, N, x, ga, be, dy, min_total_bytes=1)
    stream = torch.cuda.current_stream().cuda_stream
    for i in range(args.profile):
        prob.fwd(i, stream)
        if bwd:
            prob.bwd_(i, stream, True)
    torch.cuda.synchronize()
    print("profiled", args.workload, args.profile, "calls")


class _StdoutToStderr:
    """While active, file descriptor 1 points at stderr, so that banners printed by libraries
    (NCCL prints its version) cannot end up next to the one JSON line this program owes stdout."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)
        return self

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        os.close(self.saved)
        return False


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=HEADLINE, choices=list(WORKLOADS))
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--only", default="")
    ap.add_argument("--out", default="")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-ref", action="store_true")
    ap.add_argument("--no-nchw", action="store_true", help="sweep: skip the channels-first entry points")
    ap.add_argument("--no-parity", action="store_true", help="skip the value check that precedes the timed runs")
    ap.add_argument("--no-shapes", action="store_true", help="skip the table of VAE / SD shapes (1 GPU only)")
    ap.add_argument("--collective", default="auto", choices=["auto", "peer", "peer-inline", "peer-side", "nccl"],
                    help="more than one GPU: the backward kernels post the parameter gradients into the ranks' exchange "
                         "buffers over peer memory and collect the sums inside the same call (peer-inline, the default "
                         "where symmetric memory can be set up), one step later (peer) or in the library's exchange kernel "
                         "on a side stream (peer-side); or an NCCL all-reduce on a side stream (nccl)")
    ap.add_argument("--no-graph", action="store_true", help="time the eager loop instead of a CUDA-graph replay")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--nchw", action="store_true", help="--profile: the channels-first entry points")
    ap.add_argument("--profile", type=int, default=0, metavar="CALLS",
                    help="profiling target: CALLS forward(+backward) calls of --workload through the C ABI, nothing else")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.profile > 0:
        return profile_target(args)
    if args.sweep:
        return sweep(args)
    if args.impl == "reference":
        return reference_arm(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        # launched without torchrun: re-launch one process per GPU on this node
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
               "--master-addr", "127.0.0.1", "--master-port", "29531"] + sys.argv
        raise SystemExit(subprocess.call(cmd))
    device_arm(args)


if __name__ == "__main__":
    main()
