"""Benchmark of the GLA hot path: chunk_gla forward+backward tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 2|3|4|5] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

A step is one forward+backward of ``chunk_gla`` with the reference harness loss
``hidden_final.sum() + out.sum()`` (gla.py:1336-1340) on seeded synthetic inputs.  The headline
(``--config 2``, the default) is the README shape (benchmark config 2: B=4, H=6, D=128, T=4096, bf16,
chunk 128, log_fgate = log_sigmoid(5 + N(0,1)) in float32); with N GPUs every rank runs that shape on its
own batch shard (batch x heads sharding needs no collective), so scaling is weak and ``value`` is the
whole-job tokens/s.  Rank 0 prints ONE JSON line.

Timed quantities of the headline:
  value      device-resident inputs, the C ABI called directly, one CUDA-graph replay per step, CUDA events
             around groups of ``inner_repeats`` steps (the timed region lasts about half a second), two
             rotating input/output sets so that no step finds its operands in L2.
  api_ms_per_step  the public Python operator (gla_jax_b200.chunk_gla + autograd) on device-resident inputs.
  e2e        the public operator with HOST pinned inputs: host->device copies of all five inputs and a
             device->host read of the scalar loss inside every timed step; the copies of step i+1 are
             issued on a copy stream while step i computes (a double-buffered input feed).
  roofline   the dominant kernel's time, from CUDA events the library records around each of its launches.
  cpu_baseline  the oracle's chunk path (torch CPU, float32) on a bounded sample.
The same line carries the other benchmark configurations, each measured at this run's N:
  cfg3  config 3 (B=32, H=16, D=128, T=8192, q,k,v/sqrt(128), zero initial state) with the batch split over
        the N ranks and no collective: strong scaling.
  cfg4  (N >= 2) config 4 (B=1, H=8, D=128, T=131072) with the sequence split over the N ranks
        (gla_jax_b200.sequence_parallel_chunk_gla over NCCL), beside one GPU's chunk_gla on the whole sequence.
  cfg5  (N = 1) config 5's per-GPU share at 8 GPUs (B=2, H=8, D=256, T=16384, sharp gates): chunk_gla and
        recurrent_gla.
``--config 3|4|5`` prints that configuration's block as a line of its own.
``--impl reference`` times the oracle's CPU chunk path alone (the reference itself needs jax 0.4.29 with
Pallas/Triton, which cannot be installed here; its CPU-runnable restatement is the oracle).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import re
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

CONFIGS = {
    2: dict(B=4, T=4096, H=6, D=128, C=128, shift=5.0, scale=1.0, zero_init=False,
            what="README shape: B=4,H=6,D=128,T=4096,chunk=128, bf16 q/k/v/hidden ~ N(0,1), f32 "
                 "log_fgate=log_sigmoid(5+N(0,1)) (benchmark config 2)"),
    3: dict(B=32, T=8192, H=16, D=128, C=128, shift=5.0, scale=128 ** -0.5, zero_init=True,
            what="training-scale layer: B=32,H=16,D=128,T=8192,chunk=128, bf16 q/k/v ~ N(0,1)/sqrt(128), zero "
                 "hidden_init, f32 log_fgate=log_sigmoid(5+N(0,1)) (benchmark config 3)"),
    4: dict(B=1, T=131072, H=8, D=128, C=128, shift=5.0, scale=1.0, zero_init=False,
            what="long context: B=1,H=8,D=128,T=131072,chunk=128, bf16 q/k/v/hidden ~ N(0,1), f32 "
                 "log_fgate=log_sigmoid(5+N(0,1)) (benchmark config 4)"),
    5: dict(B=16, T=16384, H=8, D=256, C=256, shift=0.0, scale=1.0, zero_init=False,
            what="sharp gates: B=16,H=8,D=256,T=16384,chunk=256, bf16 q/k/v/hidden ~ N(0,1), f32 "
                 "log_fgate=log_sigmoid(N(0,1)) (benchmark config 5)"),
}
CFG = CONFIGS[2]
METRIC = "chunk_gla fwd+bwd tokens/sec"


def flops_per_token_head(C, D):
    """Algorithmic matmul flops of chunk_gla fwd+bwd per token and head: 6CD + 12D^2."""
    return 6 * C * D + 12 * D * D


def bytes_per_token_head(D):
    """Compulsory HBM bytes per token and head, bf16 tensors + float32 gate: 34 D."""
    return 34 * D


def device_inputs(cfg, B, T, dev, seed):
    """Seeded inputs of a benchmark configuration generated on the device (one generator per tensor):
    (hidden_init, log_fgate, value, key, query), bf16 except the float32 gate."""
    import torch
    H, D = cfg["H"], cfg["D"]

    def normal(shape, s):
        gen = torch.Generator(device=dev).manual_seed(seed + s)
        return torch.randn(shape, generator=gen, device=dev, dtype=torch.float32)

    hidden = torch.zeros(B, H, D, D, device=dev) if cfg["zero_init"] else normal((B, H, D, D), 0)
    v, k, q = (normal((B, T, H, D), s) * cfg["scale"] for s in (1, 2, 3))
    g = torch.nn.functional.logsigmoid(cfg["shift"] + normal((B, T, H, D), 4))
    return [hidden.to(torch.bfloat16), g, v.to(torch.bfloat16), k.to(torch.bfloat16), q.to(torch.bfloat16)]


class AbiProblem:
    """One chunk_gla fwd+bwd problem driven through the C ABI on device-resident buffers."""

    def __init__(self, lib, dev, ins, C, impl, nsets=1):
        import torch
        from gla_jax_b200 import _lib
        self.lib, self._lib, self.dev, self.C, self.impl = lib, _lib, dev, C, impl
        self.B, self.T, self.H, self.D = ins[0][2].shape
        self.sets = []
        for (h, g, v, k, q) in ins:
            o = dict(hf=torch.empty_like(h), out=torch.empty_like(v), dh=torch.empty_like(h), dg=torch.empty_like(g),
                     dv=torch.empty_like(v), dk=torch.empty_like(v), dq=torch.empty_like(v), dhf=torch.ones_like(h),
                     dout=torch.ones_like(v))
            self.sets.append(((h, g, v, k, q), o))
        B, T, H, D = self.B, self.T, self.H, self.D
        dt = _lib.GLA_BF16
        self.saved = torch.empty(lib.gla_chunk_saved_bytes(B, T, H, D, C, dt, impl), dtype=torch.uint8, device=dev)
        n = max(lib.gla_chunk_fwd_workspace_bytes(B, T, H, D, C, dt, impl), lib.gla_chunk_bwd_workspace_bytes(B, T, H, D, C, dt, impl))
        self.ws = torch.empty(n, dtype=torch.uint8, device=dev)
        self.stream = torch.cuda.current_stream(dev).cuda_stream

    def step(self, i):
        lib, _lib = self.lib, self._lib
        (h, g, v, k, q), o = self.sets[i % len(self.sets)]
        B, T, H, D, C, dt = self.B, self.T, self.H, self.D, self.C, _lib.GLA_BF16
        st = lib.gla_chunk_fwd(self.stream, B, T, H, D, C, dt, self.impl, h.data_ptr(), g.data_ptr(), v.data_ptr(), k.data_ptr(),
                               q.data_ptr(), o["hf"].data_ptr(), o["out"].data_ptr(), self.saved.data_ptr(),
                               self.ws.data_ptr(), self.ws.numel())
        _lib.check(st, "gla_chunk_fwd")
        st = lib.gla_chunk_bwd(self.stream, B, T, H, D, C, dt, self.impl, g.data_ptr(), v.data_ptr(), k.data_ptr(), q.data_ptr(),
                               self.saved.data_ptr(), o["dhf"].data_ptr(), o["dout"].data_ptr(), o["dh"].data_ptr(),
                               o["dg"].data_ptr(), o["dv"].data_ptr(), o["dk"].data_ptr(), o["dq"].data_ptr(),
                               self.ws.data_ptr(), self.ws.numel())
        _lib.check(st, "gla_chunk_bwd")

    def capture(self):
        """One CUDA graph per input set (the library only enqueues work on the stream it is given)."""
        import torch
        graphs = []
        side = torch.cuda.Stream(device=self.dev)
        keep = self.stream
        for sidx in range(len(self.sets)):
            gph = torch.cuda.CUDAGraph()
            side.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(side):
                self.stream = side.cuda_stream
                with torch.cuda.graph(gph, stream=side):
                    self.step(sidx)
            graphs.append(gph)
        self.stream = keep
        torch.cuda.synchronize()
        return graphs

    def profile(self, steps):
        """Per-kernel (launches, total ms) over `steps` directly launched steps, from the library's own events."""
        lib = self.lib
        lib.gla_profile_enable(1)
        l0 = lib.gla_launch_count()
        for i in range(steps):
            self.step(i)
        import torch
        torch.cuda.synchronize()
        lib.gla_profile_enable(0)
        launches = lib.gla_launch_count() - l0
        buf = ctypes.create_string_buffer(1 << 16)
        lib.gla_profile_report(buf, len(buf))
        kern = {}
        for ln in buf.value.decode().strip().splitlines():
            name, n, ms = ln.split()
            kern[name] = (int(n), float(ms))
        return kern, launches


def timed(fn, K, barrier, repeats=1):
    """K event-bracketed groups of `repeats` calls of fn(i); returns total ms (sum over the groups)."""
    import torch
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    barrier()
    i = 0
    for a, b in evs:
        a.record()
        for _ in range(repeats):
            fn(i)
            i += 1
        b.record()
    barrier()
    return sum(a.elapsed_time(b) for a, b in evs)


def reduce_max(vals, dev, world):
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(vals), dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=float(d["hbm_gbs"]), tf_burst=float(d["bf16_tflops"]),
                    tf_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


def load_ncu_traffic():
    """DRAM bytes per launch of each kernel at the README shape, from the committed ncu summary
    (profiles/chunk_kernels_readme_shape_dram_traffic.md: table rows `| kernel | read MB | write MB | ...`)."""
    p = ROOT / "profiles" / "chunk_kernels_readme_shape_dram_traffic.md"
    out = {}
    if p.exists():
        for m in re.finditer(r"^\|\s*`?(\w+)`?\s*\|\s*([\d.]+)\s*\|\s*([\d.]+)\s*\|", p.read_text(), re.M):
            out[m.group(1)] = (float(m.group(2)) + float(m.group(3))) * 1e6
    return out


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.02)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# --------------------------------------------------------------------------------------------------
# CPU legs
# --------------------------------------------------------------------------------------------------
def cpu_baseline(seconds_budget=20.0, threads=None):
    """Oracle chunk path, forward + autograd backward, float32 torch-CPU, on single sequences of
    the benchmark shape (T=4096, H=6, D=128, chunk 128) until the budget is spent."""
    import torch
    from oracle import gla_oracle as O
    threads = threads or len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    T, H, D, C = CFG["T"], CFG["H"], CFG["D"], CFG["C"]
    h, g, v, k, q = O.make_inputs(1, T, H, D, torch.float32, seed=0)
    n, t0 = 0, time.perf_counter()
    while True:
        O.chunk_gla_cpu_fwd_bwd(h, g, v, k, q, C)
        n += 1
        el = time.perf_counter() - t0
        if el > seconds_budget or n >= 64:
            break
    return {"value": n * T / el, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{n} sequence(s) of T={T}, H={H}, D={D}, chunk={C}, float32, fwd+bwd, {el:.1f} s"}


def run_reference(args, rank, world):
    """The reference arm: the reference's CPU-runnable path (its jnp chunk algorithm restated in
    the oracle) on the host cores; rank 0 only."""
    if rank != 0:
        return
    import torch
    from oracle import gla_oracle as O
    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    T, H, D, C = CFG["T"], CFG["H"], CFG["D"], CFG["C"]
    h, g, v, k, q = O.make_inputs(1, T, H, D, torch.float32, seed=0)
    for _ in range(min(args.warmup, 1)):
        O.chunk_gla_cpu_fwd_bwd(h, g, v, k, q, C)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.chunk_gla_cpu_fwd_bwd(h, g, v, k, q, C)
    el = time.perf_counter() - t0
    val = args.steps * T / el
    sample = f"each step = one sequence (B=1 of the B={CFG['B']} workload): T={T}, H={H}, D={D}, chunk={C}, float32"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * el / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "README shape B=4,H=6,D=128,T=4096,chunk=128 (benchmark config 2); CPU sample B=1"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference needs jax==0.4.29 + Pallas/Triton (not installable here); this is its chunk "
                "algorithm restated with plain tensor ops (oracle/gla_oracle.py) on the host cores",
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# other ops (--op)
# --------------------------------------------------------------------------------------------------
def bench_layer(args, lib, dev, rank, world, local_rank, W, K):
    """The GLA layer around the op (projections, gate stage, chunk_gla, norm + output gate, projection), forward and
    backward, at the README op shape with d_model = H * D.  Reported: layer tokens/s and, per element-wise stage
    kernel, the achieved HBM bandwidth (algorithmic bytes: what the stage must read and write once)."""
    import torch
    import torch.distributed as dist
    from gla_jax_b200 import GLALayer
    B, T, H, D = 4, 4096, 6, 128
    d_model = H * D
    torch.manual_seed(1000 * rank + 3)
    layer = GLALayer(d_model, H, head_dim=D, chunk_size=128, device=dev, dtype=torch.bfloat16)
    xs = [torch.randn(B, T, d_model, device=dev).to(torch.bfloat16).requires_grad_(True) for _ in range(2)]

    def step(i):
        x = xs[i % 2]
        y, hf = layer(x)
        (y.float().sum() + hf.float().sum()).backward()
        x.grad = None
        layer.zero_grad(set_to_none=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(W):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        step(i)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches0 = lib.gla_launch_count()
    for i in range(K):
        step(i)
    barrier()
    launches = lib.gla_launch_count() - launches0
    # the four element-wise stage kernels, timed one by one through the C ABI on two rotating buffer sets
    # (2 x ~250 MB > L2); the backward of a layer step runs on autograd's own thread, so per-launch events
    # bracketed inside the library on this thread would only see the forward half
    from gla_jax_b200 import _lib
    n_el = B * T * H * D
    rows = B * T * H
    mkb = lambda: torch.randn(B, T, H, D, device=dev).to(torch.bfloat16)
    sets = [dict(z=mkb(), x=mkb(), gate=mkb(), dy=mkb(), y=mkb(), dx=mkb(), dgate=mkb(), dz=mkb(),
                 g=torch.empty(B, T, H, D, device=dev), dg=torch.randn(B, T, H, D, device=dev),
                 rstd=torch.empty(rows, device=dev)) for _ in range(2)]
    w = torch.ones(D, device=dev)
    dw = torch.empty(D, device=dev)
    ws_n = lib.gla_layer_headnorm_gate_bwd_workspace_bytes(rows, D)
    ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    BF = _lib.GLA_BF16
    calls = {
        "gate_fwd_kernel": lambda a: lib.gla_layer_gate_fwd(stream, n_el, BF, a["z"].data_ptr(), 1 / 16, a["g"].data_ptr()),
        "gate_bwd_kernel": lambda a: lib.gla_layer_gate_bwd(stream, n_el, BF, a["z"].data_ptr(), a["dg"].data_ptr(), 1 / 16,
                                                            a["dz"].data_ptr()),
        "headnorm_gate_fwd_kernel": lambda a: lib.gla_layer_headnorm_gate_fwd(
            stream, rows, D, BF, a["x"].data_ptr(), a["gate"].data_ptr(), w.data_ptr(), 1e-5, a["y"].data_ptr(),
            a["rstd"].data_ptr()),
        "headnorm_gate_bwd_kernel": lambda a: lib.gla_layer_headnorm_gate_bwd(
            stream, rows, D, BF, a["x"].data_ptr(), a["gate"].data_ptr(), w.data_ptr(), a["rstd"].data_ptr(),
            a["dy"].data_ptr(), a["dx"].data_ptr(), a["dgate"].data_ptr(), dw.data_ptr(), ws.data_ptr(), ws_n),
    }
    kern = {}
    for name, fn in calls.items():
        for i in range(4):
            _lib.check(fn(sets[i % 2]), name)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(2 * K)]
        for i, (a, b) in enumerate(evs):
            a.record()
            _lib.check(fn(sets[i % 2]), name)
            b.record()
        torch.cuda.synchronize()
        kern[name] = (len(evs), sum(a.elapsed_time(b) for a, b in evs))
    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    (ms_total,) = reduce_max([ms_total], dev, world)
    if rank == 0:
        peaks = load_peaks()
        stage_bytes = {"gate_fwd_kernel": 6, "gate_bwd_kernel": 8, "headnorm_gate_fwd_kernel": 6,
                       "headnorm_gate_bwd_kernel": 10}
        stages = {}
        for name, per_el in stage_bytes.items():
            if name in kern and kern[name][0]:
                per = kern[name][1] / kern[name][0] * 1e-3
                stages[name] = {"ms_per_launch": per * 1e3, "achieved_gbs": per_el * n_el / per / 1e9,
                                "frac_of_measured_copy": per_el * n_el / per / 1e9 / peaks["hbm"]}
        top = max(stages, key=lambda k: stages[k]["ms_per_launch"]) if stages else None
        print(json.dumps({
            "metric": "GLA layer fwd+bwd tokens/sec", "value": B * T * world * K / (ms_total * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"GLA layer: B={B},T={T},d_model={d_model},H={H},D={D},chunk=128, bf16 parameters "
                                   "and activations, float32 log_fgate; loss=y.sum()+hidden_final.sum()",
                       "l2": "2 rotating inputs; one step touches > 1 GB (L2 = 126 MB)", "launch": "plain launches"},
            "gpu_launches": launches, "clocks": sampler.summary(),
            "roofline": None if top is None else {
                "bound": "hbm", "kernel": top, "achieved": stages[top]["achieved_gbs"], "peak": peaks["hbm"],
                "unit": "GB/s", "frac": stages[top]["frac_of_measured_copy"], "traffic": None,
                "peak_source": peaks["source"]},
            "layer_stages": stages,
        }))


def bench_decode(args, lib, dev, rank, world, local_rank, W, K):
    """Single-token step: B requests x H heads advance one token per step; the (B,H,D,D) float32 states live on the
    device.  tokens/s = requests advanced per second; the step streams the state once in and once out."""
    import torch
    import torch.distributed as dist
    from gla_jax_b200 import decode_step, _lib
    B, H, D = 128, 16, 128
    gen = torch.Generator(device=dev).manual_seed(1000 * rank + 5)
    state = torch.randn(B, H, D, D, device=dev, generator=gen)                 # 134 MB > L2
    mk = lambda: torch.randn(B, H, D, device=dev, generator=gen).to(torch.bfloat16)
    g = torch.nn.functional.logsigmoid(5 + torch.randn(B, H, D, device=dev, generator=gen))
    v, k, q = mk(), mk(), mk()
    out = torch.empty(B, H, D, device=dev, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def step(_i=0):
        st = lib.gla_decode_step(stream, B, H, D, _lib.GLA_BF16, state.data_ptr(), g.data_ptr(), v.data_ptr(),
                                 k.data_ptr(), q.data_ptr(), out.data_ptr(), _lib.GLA_BF16)
        _lib.check(st, "gla_decode_step")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = lib.gla_launch_count()
    ms_total = timed(step, K, barrier)
    launches = lib.gla_launch_count() - launches0
    # end to end: this step's g, v, k, q from pinned host memory, its out back to the host
    host = [x.cpu().pin_memory() for x in (g, v, k, q)]
    hout = torch.empty(B, H, D, dtype=torch.bfloat16).pin_memory()
    h2d = sum(x.numel() * x.element_size() for x in host)

    def e2e_step(_i=0):
        gg, vv, kk, qq = (x.to(dev, non_blocking=True) for x in host)
        o = decode_step(state, gg, vv, kk, qq)
        hout.copy_(o, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()

    for _ in range(3):
        e2e_step()
    e2e_ms = timed(e2e_step, K, barrier)
    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    ms_total, e2e_ms = reduce_max([ms_total, e2e_ms], dev, world)
    if rank == 0:
        peaks = load_peaks()
        per = ms_total / K * 1e-3
        alg = 2 * 4 * D * D * B * H + B * H * D * (4 + 2 + 2 + 2 + 2)
        ach = alg / per / 1e9
        print(json.dumps({
            "metric": "decode step tokens/sec", "value": B * world * K / (ms_total * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"single-token step: {B} requests x {H} heads x D={D}, float32 states (134 MB per GPU, "
                                   "larger than L2), bf16 q/k/v/out, f32 log_fgate", "parallelism": f"request-shard x{world}"},
            "e2e": {"value": B * world * K / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": B * H * D * 2, "ms_per_step": e2e_ms / K},
            "gpu_launches": launches, "clocks": sampler.summary(),
            "roofline": {"bound": "hbm", "kernel": "decode_step_kernel", "achieved": ach, "peak": peaks["hbm"],
                         "unit": "GB/s", "frac": ach / peaks["hbm"], "traffic": None, "peak_source": peaks["source"],
                         "algorithmic": "state read + write 2*4*D*D B per (request, head) + q,k,v,out bf16 + g f32"},
        }))


def bench_scans(args, lib, dev, rank, world, local_rank, W, K):
    """The scan ops of ops.py on shapes of the chunk path and of long-sequence callers: achieved HBM GB/s against
    their algorithmic bytes (each element read once and written once)."""
    import torch
    from gla_jax_b200 import _lib
    stream = torch.cuda.current_stream(dev).cuda_stream
    peaks = load_peaks()
    res = {}

    def run(name, fn, alg_bytes, what):
        for _ in range(W):
            fn()
        ms = timed(lambda i: fn(), K, torch.cuda.synchronize)
        per = ms / K * 1e-3
        res[name] = {"ms_per_launch": per * 1e3, "achieved_gbs": alg_bytes / per / 1e9,
                     "frac_of_measured_copy": alg_bytes / per / 1e9 / peaks["hbm"], "algorithmic": what}

    # cumsum: log_fgate of the README shape seen as (B*N, C, H*D)... any (N, T, D): here (24, 4096, 128) x 2 sets > L2
    if args.op in ("cumsum", "scans"):
        N, T, D = 96, 4096, 128                      # 201 MB in + 201 MB out
        x = torch.randn(N, T, D, device=dev)
        y = torch.empty_like(x)
        run("cumsum_kernel", lambda: _lib.check(lib.gla_cumsum(stream, N, T, D, x.data_ptr(), None, y.data_ptr(), 0, 0, 0), "gla_cumsum"),
            2 * 4 * N * T * D, f"cumsum (N={N}, T={T}, D={D}) float32: 4 B in + 4 B out per element")
        N2, T2, D2 = 512, 128, 768                   # the chunk path's layout: (batch x chunks, chunk, heads x D)
        x2 = x.view(N2, T2, D2)
        y2 = y.view(N2, T2, D2)
        run("cumsum_kernel_chunk_layout", lambda: _lib.check(lib.gla_cumsum(stream, N2, T2, D2, x2.data_ptr(), None, y2.data_ptr(), 0, 0, 0), "gla_cumsum"),
            2 * 4 * N2 * T2 * D2, f"cumsum (N={N2}, T={T2}, D={D2}) float32: 4 B in + 4 B out per element")
    if args.op in ("rnn_scan", "scans"):
        batch, T, Kf, V = 24, 64, 128, 128           # 24 heads x 64 chunks of (128,128) float32 states: 100 MB in, 100 MB out
        g = -torch.rand(batch, T, Kf, device=dev) * 0.1
        kv = torch.randn(batch, T, Kf, V, device=dev)
        ol = torch.empty_like(g)
        os_ = torch.empty_like(kv)
        run("rnn_scan_kernel", lambda: _lib.check(lib.gla_rnn_scan(stream, batch, T, Kf, V, g.data_ptr(), kv.data_ptr(), None, None,
                                                                   ol.data_ptr(), os_.data_ptr(), 0, 0, 0), "gla_rnn_scan"),
            2 * 4 * batch * T * Kf * V, f"rnn scan ({batch} x T={T}, K={Kf}, V={V}) float32: state elements 4 B in + 4 B out")
        # a long axis with one row (what ops.py:396 rnn_recursive serves by recursion): segmented into runs
        T3 = 4096
        g3 = -torch.rand(1, T3, Kf, device=dev) * 0.1
        kv3 = torch.randn(1, T3, Kf, V, device=dev)
        ol3, os3 = torch.empty_like(g3), torch.empty_like(kv3)
        nws = lib.gla_rnn_scan_workspace_bytes(1, T3, Kf, V)
        ws3 = torch.empty(max(nws, 16), dtype=torch.uint8, device=dev)
        run("rnn_scan_kernel_long_axis", lambda: _lib.check(lib.gla_rnn_scan_ws(stream, 1, T3, Kf, V, g3.data_ptr(), kv3.data_ptr(), None, None,
                                                                                ol3.data_ptr(), os3.data_ptr(), 0, 0, 0, ws3.data_ptr(), nws), "gla_rnn_scan_ws"),
            2 * 4 * T3 * Kf * V, f"rnn scan (1 x T={T3}, K={Kf}, V={V}) float32 in runs: state elements 4 B in + 4 B out")
        run("rnn_scan_kernel_long_axis_single_walk", lambda: _lib.check(lib.gla_rnn_scan(stream, 1, T3, Kf, V, g3.data_ptr(), kv3.data_ptr(), None, None,
                                                                                         ol3.data_ptr(), os3.data_ptr(), 0, 0, 0), "gla_rnn_scan"),
            2 * 4 * T3 * Kf * V, f"rnn scan (1 x T={T3}, K={Kf}, V={V}) float32, one sequential walk (no scratch)")
    if rank == 0:
        top = "cumsum_kernel" if "cumsum_kernel" in res else next(iter(res))
        print(json.dumps({
            "metric": "scan ops achieved HBM GB/s", "value": res[top]["achieved_gbs"], "unit": "GB/s", "n_gpus": 1, "steps": K,
            "warmup": W, "ms_per_step": res[top]["ms_per_launch"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": res[top]["algorithmic"]},
            "roofline": {"bound": "hbm", "kernel": top, "achieved": res[top]["achieved_gbs"], "peak": peaks["hbm"],
                         "unit": "GB/s", "frac": res[top]["frac_of_measured_copy"], "traffic": None,
                         "peak_source": peaks["source"]},
            "scans": res}))


# --------------------------------------------------------------------------------------------------
# the other benchmark configurations
# --------------------------------------------------------------------------------------------------
def run_cfg3(lib, dev, rank, world, barrier, steps=5, warmup=2):
    """Config 3 with the batch split over the ranks (strong scaling, no collective on the data path)."""
    import torch
    from gla_jax_b200 import _lib
    from gla_jax_b200.parallel import shard_batch_heads
    cfg = CONFIGS[3]
    bs, hs = shard_batch_heads(cfg["B"], cfg["H"], world, rank)
    Bl = bs.stop - bs.start
    assert hs.stop - hs.start == cfg["H"]
    ins = [device_inputs(cfg, Bl, cfg["T"], dev, seed=3000 + 10 * rank)]
    prob = AbiProblem(lib, dev, ins, cfg["C"], _lib.IMPL_AUTO)
    for i in range(warmup):
        prob.step(i)
    ms = timed(prob.step, steps, barrier)
    kern, _ = prob.profile(1)
    wt = int(lib.gla_device_wait_timeouts())
    del prob, ins
    torch.cuda.empty_cache()
    (ms,) = reduce_max([ms], dev, world)
    per = ms / steps
    th = cfg["B"] * cfg["T"] * cfg["H"]
    peaks = load_peaks()
    return {"workload": cfg["what"], "parallelism": f"batch shard: {Bl} of {cfg['B']} sequences per GPU x {world}, no collectives",
            "scaling": "strong", "tokens_per_s": cfg["B"] * cfg["T"] / (per * 1e-3), "ms_per_step": per, "steps": steps,
            "hbm_frac_of_measured_copy": bytes_per_token_head(cfg["D"]) * th / world / (per * 1e-3) / (peaks["hbm"] * 1e9),
            "tensor_frac_of_burst_peak": flops_per_token_head(cfg["C"], cfg["D"]) * th / world / (per * 1e-3) / (peaks["tf_burst"] * 1e12),
            "state_path": "one_pass" if "tc_state_kernel" in kern else "two_kernels",
            "kernels_ms_per_step_rank0": {n: ms_ for n, (_, ms_) in sorted(kern.items(), key=lambda kv: -kv[1][1])},
            "device_wait_timeouts": wt}


def run_cfg4(lib, dev, rank, world, barrier, steps=5, warmup=2):
    """Config 4: one sequence of 131072 tokens split over the ranks (sequence parallel over NCCL), fwd+bwd through
    the public operator; beside it one GPU's chunk_gla on the whole sequence (rank 0), and their agreement."""
    import torch
    import torch.distributed as dist
    from gla_jax_b200 import chunk_gla
    from gla_jax_b200 import parallel as P
    from oracle import gla_oracle as O
    cfg = CONFIGS[4]
    T, C = cfg["T"], cfg["C"]
    L = T // world
    full = device_inputs(cfg, cfg["B"], T, dev, seed=4000)          # the same sequence on every rank (same seed)
    sl = slice(rank * L, (rank + 1) * L)
    h = full[0]
    mine = [x[:, sl].contiguous() for x in full[1:]]

    def sp_step(_i=0):
        leaves = [h.detach().requires_grad_(True)] + [x.detach().requires_grad_(True) for x in mine]
        hf, out = P.sequence_parallel_chunk_gla(*leaves, chunk_size=C)
        return hf, out, torch.autograd.grad(hf.float().sum() + out.float().sum(), leaves)

    for i in range(warmup):
        sp_step()
    ms = timed(sp_step, steps, barrier)
    hf_sp, out_sp, _ = sp_step()
    # The same step as ONE CUDA graph per rank (operator calls, NCCL all-gathers and the backward captured together):
    # at 4 and 8 ranks a rank's kernels take less time than Python needs to enqueue them, so the eager number above
    # measures the host; the replay measures the GPUs.  Every rank captures (collectives must be captured by all);
    # a rank whose capture fails tells the others, and nobody replays.
    graph_ms = graph_err = None
    try:
        leaves_g = [h.detach().requires_grad_(True)] + [x.detach().requires_grad_(True) for x in mine]
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        gph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            # thread-local capture mode: the process group's watchdog thread may query events meanwhile
            with torch.cuda.graph(gph, stream=side, capture_error_mode="thread_local"):
                hf_g, out_g = P.sequence_parallel_chunk_gla(*leaves_g, chunk_size=C)
                grads_g = torch.autograd.grad(hf_g.float().sum() + out_g.float().sum(), leaves_g)
        torch.cuda.synchronize()
        okflag = torch.ones(1, device=dev)
    except Exception as e:           # noqa: BLE001 - reported in the JSON line, the eager number stands
        graph_err = f"{type(e).__name__}: {e}"[:200]
        try:
            torch.cuda.synchronize()
        except Exception:            # noqa: BLE001
            pass
        okflag = torch.zeros(1, device=dev)
    dist.all_reduce(okflag, op=dist.ReduceOp.MIN)
    if float(okflag) > 0:
        for _ in range(warmup):
            gph.replay()
        graph_ms = timed(lambda i: gph.replay(), steps, barrier)
        graph_parity = O.rel_l2(out_sp.cpu(), out_g.cpu())
    # the exchange alone: the all-gathers and combine launches of a step, on tensors of the same size
    B, H, D = cfg["B"], cfg["H"], cfg["D"]
    Gl = torch.zeros(B, H, D, device=dev)
    Sl = torch.zeros(B, H, D, D, device=dev)
    ops = P.CudaOps()

    def exch(_i=0):
        # forward: one all-gather of the packed [G | S] record and one combine launch; backward: one all-gather of A
        # (G is kept from the forward) and one combine launch
        nG = Gl.numel()
        packed = P._all_gather(torch.cat([Gl.reshape(-1), Sl.reshape(-1)]), None)
        aG, aS = packed[:, :nG].unflatten(1, tuple(Gl.shape)), packed[:, nG:].unflatten(1, tuple(Sl.shape))
        ops.combine_both(aG, aS, rank, h, h.dtype, False)
        aA = P._all_gather(Sl, None)
        ops.combine_both(aG, aA, rank, h, h.dtype, True)

    exch()
    ms_ex = timed(exch, steps, barrier)
    single = parity = None
    if rank == 0:
        def one(_i=0):
            leaves = [x.detach().requires_grad_(True) for x in full]
            hf, out = chunk_gla(*leaves, chunk_size=C)
            return hf, out, torch.autograd.grad(hf.float().sum() + out.float().sum(), leaves)
        one()
        single = timed(one, 3, torch.cuda.synchronize) / 3
        hf1, out1, _ = one()
        parity = {"hidden_final_rel_l2": O.rel_l2(hf1.cpu(), hf_sp.cpu()),
                  "out_slice_rel_l2": O.rel_l2(out1[:, sl].cpu(), out_sp.cpu())}
    barrier()
    wt = int(lib.gla_device_wait_timeouts())
    ms, ms_ex = reduce_max([ms, ms_ex], dev, world)
    if graph_ms is not None:
        (graph_ms,) = reduce_max([graph_ms], dev, world)
    per = ms / steps
    return {"workload": cfg["what"], "parallelism": f"sequence split over {world} ranks ({L} tokens each), one all-gather of "
            f"(G, S) per direction over NCCL + local combine", "scaling": "strong",
            "tokens_per_s": cfg["B"] * T / (per * 1e-3), "ms_per_step": per, "steps": steps,
            "exchange_ms_per_step": ms_ex / steps, "single_gpu_whole_sequence_ms": single,
            "speedup_vs_single_gpu": None if single is None else single / per,
            "graph_replay_ms_per_step": None if graph_ms is None else graph_ms / steps,
            "graph_replay_speedup_vs_single_gpu": None if (single is None or graph_ms is None) else single / (graph_ms / steps),
            "graph_replay_out_rel_l2_vs_eager": None if graph_ms is None else graph_parity,
            "graph_capture_error": graph_err,
            "parity_vs_single_gpu": parity, "device_wait_timeouts": wt}


def run_cfg5(lib, dev, steps=3, warmup=2):
    """Config 5's per-GPU share at 8 GPUs (B=2 of 16): chunk_gla and recurrent_gla fwd+bwd through the C ABI."""
    import torch
    from gla_jax_b200 import _lib
    cfg = CONFIGS[5]
    Bl, T, H, D, C = 2, cfg["T"], cfg["H"], cfg["D"], cfg["C"]
    ins = [device_inputs(cfg, Bl, T, dev, seed=5000)]
    peaks = load_peaks()
    th = Bl * T * H
    out = {"workload": cfg["what"], "share": f"B={Bl} of {cfg['B']} sequences (one GPU's share at 8 GPUs)"}
    prob = AbiProblem(lib, dev, ins, C, _lib.IMPL_AUTO)
    for i in range(warmup):
        prob.step(i)
    per = timed(prob.step, steps, torch.cuda.synchronize) / steps
    kern, _ = prob.profile(1)
    out["chunk_gla"] = {"ms_per_step": per, "tokens_per_s": Bl * T / (per * 1e-3),
                        "hbm_frac_of_measured_copy": bytes_per_token_head(D) * th / (per * 1e-3) / (peaks["hbm"] * 1e9),
                        "tensor_frac_of_burst_peak": flops_per_token_head(C, D) * th / (per * 1e-3) / (peaks["tf_burst"] * 1e12),
                        "kernels_ms_per_step": {n: ms_ for n, (_, ms_) in sorted(kern.items(), key=lambda kv: -kv[1][1])}}
    (h, g, v, k, q), o = prob.sets[0]
    dt = _lib.GLA_BF16
    rws_n = lib.gla_recurrent_bwd_workspace_bytes(Bl, T, H, D, dt)
    rws = torch.empty(rws_n, dtype=torch.uint8, device=dev)
    stream = prob.stream

    def rec(_i=0):
        st = lib.gla_recurrent_fwd(stream, Bl, T, H, D, dt, h.data_ptr(), g.data_ptr(), v.data_ptr(), k.data_ptr(),
                                   q.data_ptr(), o["hf"].data_ptr(), o["out"].data_ptr(), dt, 0)
        _lib.check(st, "gla_recurrent_fwd")
        st = lib.gla_recurrent_bwd(stream, Bl, T, H, D, dt, h.data_ptr(), g.data_ptr(), v.data_ptr(), k.data_ptr(),
                                   q.data_ptr(), o["dhf"].data_ptr(), o["dout"].data_ptr(), dt, o["dh"].data_ptr(),
                                   o["dg"].data_ptr(), o["dv"].data_ptr(), o["dk"].data_ptr(), o["dq"].data_ptr(), 0,
                                   rws.data_ptr(), rws.numel())
        _lib.check(st, "gla_recurrent_bwd")

    rec()
    per = timed(rec, steps, torch.cuda.synchronize) / steps
    fp32_peak = 148 * 128 * 2 * 1.965e9          # FMA lanes x 2 flops x max SM clock
    out["recurrent_gla"] = {"ms_per_step": per, "tokens_per_s": Bl * T / (per * 1e-3),
                            "hbm_frac_of_measured_copy": bytes_per_token_head(D) * th / (per * 1e-3) / (peaks["hbm"] * 1e9),
                            "fp32_fma_frac": 17 * D * D * th / (per * 1e-3) / fp32_peak,
                            "algorithmic": "17 D^2 float32 flops per token-head (5 D^2 forward, 12 D^2 backward)"}
    out["device_wait_timeouts"] = int(lib.gla_device_wait_timeouts())
    del prob, ins
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5],
                    help="2: the headline line with the other configurations as blocks of it; 3, 4, 5: that block alone")
    ap.add_argument("--chunk-impl", default="auto", help="auto | fp32 | tcgen05, optionally with +options (see gla_b200.h)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler runs)")
    ap.add_argument("--no-graph", action="store_true", help="time plain launches instead of CUDA-graph replays")
    ap.add_argument("--no-extra", action="store_true", help="headline only: no api leg, no cfg3/cfg4/cfg5 blocks (profiler runs)")
    ap.add_argument("--op", default="chunk_gla", choices=["chunk_gla", "recurrent_gla", "decode", "layer", "cumsum", "rnn_scan", "scans"],
                    help="chunk_gla is the headline metric; recurrent_gla times the exact recurrence on the same shape; "
                         "decode times the single-token step with a persistent state; cumsum / rnn_scan / scans time the scan ops")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from gla_jax_b200 import _lib, chunk_gla
    from oracle import gla_oracle as O   # input generator and the cpu_baseline leg only

    lib = _lib.load()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    W = max(args.warmup, 3)
    K = args.steps

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def finish():
        if world > 1:
            dist.destroy_process_group()

    if args.op in ("decode", "layer", "cumsum", "rnn_scan", "scans"):
        fn = {"decode": bench_decode, "layer": bench_layer}.get(args.op, bench_scans)
        fn(args, lib, dev, rank, world, local_rank, W, K)
        return finish()
    if args.config != 2:
        blk = (run_cfg3(lib, dev, rank, world, barrier, steps=K, warmup=W) if args.config == 3 else
               run_cfg4(lib, dev, rank, world, barrier, steps=K, warmup=W) if args.config == 4 else
               run_cfg5(lib, dev, steps=K, warmup=W))
        if rank == 0:
            body = blk.get("chunk_gla", blk)
            print(json.dumps({"metric": METRIC, "value": body["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": K,
                              "warmup": W, "ms_per_step": body["ms_per_step"], "higher_is_better": True,
                              "scaling": blk.get("scaling", "weak"), "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                              "config": {"workload": blk["workload"]}, f"cfg{args.config}": blk}), flush=True)
        return finish()

    B, T, H, D, C = (CFG[x] for x in "BTHDC")
    impl = _lib.IMPL_BY_NAME[args.chunk_impl]
    dt = _lib.GLA_BF16

    # two rotating sets of inputs and outputs (each step touches > 400 MB, L2 is 126 MB)
    NSETS = 2
    ins = [[x.to(dev) for x in O.make_inputs(B, T, H, D, torch.bfloat16, seed=1000 * rank + 10 * s)] for s in range(NSETS)]
    prob = AbiProblem(lib, dev, ins, C, impl)
    stream = prob.stream

    rws_n = lib.gla_recurrent_bwd_workspace_bytes(B, T, H, D, dt)
    rws = torch.empty(rws_n if args.op == "recurrent_gla" else 16, dtype=torch.uint8, device=dev)

    def step_recurrent(i):
        (h, g, v, k, q), o = prob.sets[i % NSETS]
        st = lib.gla_recurrent_fwd(prob.stream, B, T, H, D, dt, h.data_ptr(), g.data_ptr(), v.data_ptr(), k.data_ptr(),
                                   q.data_ptr(), o["hf"].data_ptr(), o["out"].data_ptr(), dt, 0)
        _lib.check(st, "gla_recurrent_fwd")
        st = lib.gla_recurrent_bwd(prob.stream, B, T, H, D, dt, h.data_ptr(), g.data_ptr(), v.data_ptr(), k.data_ptr(),
                                   q.data_ptr(), o["dhf"].data_ptr(), o["dout"].data_ptr(), dt, o["dh"].data_ptr(),
                                   o["dg"].data_ptr(), o["dv"].data_ptr(), o["dk"].data_ptr(), o["dq"].data_ptr(), 0,
                                   rws.data_ptr(), rws.numel())
        _lib.check(st, "gla_recurrent_bwd")

    if args.op == "recurrent_gla":
        prob.step = step_recurrent
    step = prob.step

    for i in range(W):
        step(i)
    barrier()
    graphs = None
    if not args.no_graph:
        graphs = prob.capture()
        for i in range(2):
            graphs[i % NSETS].replay()
        barrier()
    run_one = (lambda i: graphs[i % NSETS].replay()) if graphs is not None else step
    # the timed region should last about half a second: K groups of `reps` steps, one event pair per group
    probe = timed(run_one, 2, barrier) / 2
    reps = 1 if args.no_extra else max(1, min(500, int(math.ceil(500.0 / max(K, 1) / max(probe, 1e-3)))))
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_total = timed(run_one, K, barrier, repeats=reps)
    # per-kernel times and the launch count come from K more steps launched directly (events cannot be
    # recorded inside a replayed graph); same kernels, same inputs
    kern, launches = prob.profile(K)

    # ---- the public operator on device-resident inputs ------------------------------------------
    api_ms = float("nan")
    if not args.no_extra and args.op == "chunk_gla":
        # the gradient of loss = hidden_final.sum() + out.sum() is asked for with its cotangents (ones) given
        # directly, so that the timed work is the operator's forward and backward and not the two reductions
        ones = [(torch.ones_like(x[0]), torch.ones_like(x[2])) for x in ins]

        def api_step(i):
            leaves = [x.detach().requires_grad_(True) for x in ins[i % NSETS]]
            hf, out = chunk_gla(*leaves, chunk_size=C, impl=args.chunk_impl)
            torch.autograd.grad((hf, out), leaves, ones[i % NSETS])
        for i in range(3):
            api_step(i)
        api_ms = timed(api_step, K, barrier, repeats=max(1, reps // 4))
        api_ms /= K * max(1, reps // 4)

    # ---- end to end through the public operator, host buffers in and a host read out -------
    host = [x.pin_memory() for x in O.make_inputs(B, T, H, D, torch.bfloat16, seed=1000 * rank + 77)]
    h2d = sum(x.numel() * x.element_size() for x in host)

    # The input feed is double-buffered the way a training loop's loader is: while step i computes, the
    # host->device copies of step i+1 run on a copy stream.  Every timed step still contains one full set of
    # copies (those of the next step; the last step's are issued and waited for too) and one host read.
    copy_stream = torch.cuda.Stream(device=dev)
    staged = [None, None]
    staged_ev = [torch.cuda.Event(), torch.cuda.Event()]

    def stage(slot):
        with torch.cuda.stream(copy_stream):
            staged[slot] = [x.to(dev, non_blocking=True) for x in host]
            staged_ev[slot].record(copy_stream)

    def e2e_step(i):
        cur = torch.cuda.current_stream(dev)
        copy_stream.wait_stream(cur)            # the buffers being replaced are no longer in use
        stage((i + 1) % 2)
        cur.wait_event(staged_ev[i % 2])
        leaves = [x.requires_grad_(True) for x in staged[i % 2]]
        for x in leaves:
            x.record_stream(cur)
        if args.op == "recurrent_gla":
            from gla_jax_b200 import recurrent_gla
            hf, out = recurrent_gla(*leaves)
        else:
            hf, out = chunk_gla(*leaves, chunk_size=C, impl=args.chunk_impl)
        loss = hf.float().sum() + out.float().sum()
        loss.backward()
        return float(loss.item())       # 4-byte device->host read; also orders the step

    e2e_ms = float("nan")
    if not args.no_e2e:
        stage(0)
        for i in range(3):
            e2e_step(i)
        barrier()
        e_evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
        for i in range(K):
            e_evs[i][0].record()
            e2e_step(i + 3)
            copy_stream.synchronize() if i == K - 1 else None    # the last step's copies end inside the region
            e_evs[i][1].record()
        barrier()
        e2e_ms = sum(a.elapsed_time(b) for a, b in e_evs)
    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    wait_timeouts = int(lib.gla_device_wait_timeouts())

    # ---- reduce over ranks: max time ---------------------------------------------------------
    ms_total, e2e_ms, api_ms = reduce_max([ms_total, e2e_ms, api_ms], dev, world)
    tokens_per_step = B * T * world
    nsteps = K * reps
    value = tokens_per_step * nsteps / (ms_total * 1e-3)
    e2e_val = tokens_per_step * K / (e2e_ms * 1e-3)

    extra = {}
    if not args.no_extra and args.op == "chunk_gla":
        del prob, ins, staged, graphs
        torch.cuda.empty_cache()
        extra["cfg3"] = run_cfg3(lib, dev, rank, world, barrier)
        if world >= 2:
            extra["cfg4"] = run_cfg4(lib, dev, rank, world, barrier)
        if world == 1:
            extra["cfg5"] = run_cfg5(lib, dev)

    if rank == 0:
        peaks = load_peaks()
        th = B * T * H                                   # token-heads per step per GPU
        step_s = ms_total * 1e-3 / nsteps
        # whole-step fractions (both rooflines of the path)
        tensor_frac = flops_per_token_head(C, D) * th / step_s / (peaks["tf_burst"] * 1e12)
        hbm_frac = bytes_per_token_head(D) * th / step_s / (peaks["hbm"] * 1e9)
        # dominant kernel: largest share of the recorded kernel time
        total_k = sum(ms for _, ms in kern.values()) or 1.0
        dom = max(kern, key=lambda n: kern[n][1]) if kern else None
        roof = None
        traffic = load_ncu_traffic() if args.op == "chunk_gla" else {}
        if dom:
            n_l, ms_l = kern[dom]
            per_launch_s = ms_l * 1e-3 / n_l
            alg = KERNEL_ALGORITHMIC.get(dom, KERNEL_ALGORITHMIC["_default"])(B, T, H, D, C)
            if alg["bound"] == "hbm":
                ach = alg["bytes"] / per_launch_s / 1e9
                roof = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peaks["hbm"], "unit": "GB/s",
                        "frac": ach / peaks["hbm"], "traffic": None}
            else:
                ach = alg["flops"] / per_launch_s / 1e12
                roof = {"bound": "tensor", "kernel": dom, "achieved": ach, "peak": peaks["tf_burst"],
                        "unit": "TFLOP/s", "frac": ach / peaks["tf_burst"], "traffic": None}
            # DRAM bytes per launch of this kernel at this exact shape, from the committed ncu capture
            # (summarised with its command under profiles/); null for kernels without one
            roof["traffic"] = traffic.get(dom)
            roof.update({"peak_source": peaks["source"], "launches": n_l, "ms_per_launch": 1e3 * per_launch_s,
                         "share_of_kernel_time": ms_l / total_k, "algorithmic": alg["what"]})
        line = {
            "metric": METRIC if args.op == "chunk_gla" else "recurrent_gla fwd+bwd tokens/sec", "value": value,
            "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_total / nsteps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "per GPU: " + CFG["what"] + "; loss=hidden_final.sum()+out.sum()",
                       "global_batch": B * world, "seq_len": T, "parallelism": f"batch-shard x{world}, no collectives",
                       "l2": f"{NSETS} rotating input/output sets; one step touches > 400 MB (L2 = 126 MB)",
                       "chunk_impl": args.chunk_impl,
                       "launch": "plain launches" if args.no_graph else "one CUDA graph replay per step"},
            "inner_repeats": reps, "timed_region_ms": ms_total,
            "api_ms_per_step": api_ms,
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms / K, "h2d_gbs_per_rank": h2d / (e2e_ms / K * 1e-3) / 1e9,
                    "host": "every rank stages its inputs from pinned host memory of the one NUMA node the GPUs share"},
            "gpu_launches": int(launches),
            "device_wait_timeouts": wait_timeouts,     # bounded device-side waits that gave up: must be 0
            "clocks": sampler.summary(),
            "roofline": roof,
            "step_fractions": {"tensor_frac_of_burst_peak": tensor_frac, "hbm_frac_of_measured_copy": hbm_frac,
                               "flops_per_step": flops_per_token_head(C, D) * th,
                               "compulsory_bytes_per_step": bytes_per_token_head(D) * th,
                               "ncu_dram_bytes_per_step": (sum(traffic.get(n, 0.0) for n in kern) if traffic and all(n in traffic for n in kern) else None)},
            "kernels": {n: {"launches": c, "ms_total": ms, "share": ms / total_k} for n, (c, ms) in
                        sorted(kern.items(), key=lambda kv: -kv[1][1])},
        }
        line.update(extra)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.cpu_seconds)
        print(json.dumps(line), flush=True)
    finish()


def _alg_simt_intra_bwd(B, T, H, D, C):
    th = B * T * H
    return {"bound": "hbm", "bytes": th * D * (2 + 2 + 4 + 4 + 4 + 2 + 2 + 4) + th * C * 4,
            "what": "q,k (bf16), lam, dqh, dkh (f32) in; dq, dk (bf16), dlam (f32) out; dP (f32 CxC per chunk) in"}


def _alg_simt_score(B, T, H, D, C):
    th = B * T * H
    return {"bound": "hbm", "bytes": th * D * (2 + 2 + 4) + th * C * 4,
            "what": "q,k (bf16), lam (f32) in; P (f32, C per token) out"}


def _alg_whole_step(B, T, H, D, C):
    th = B * T * H
    return {"bound": "hbm", "bytes": th * bytes_per_token_head(D), "what": "34*D bytes per token-head (whole step)"}


def _alg_tc_fwd(B, T, H, D, C):
    th = B * T * H
    return {"bound": "hbm", "bytes": th * 12 * D, "what": "forward: q,k,v (bf16) + log_fgate (f32) in, out (bf16): 12*D B per token-head"}


def _alg_tc_bwd(B, T, H, D, C):
    th = B * T * H
    return {"bound": "hbm", "bytes": th * 22 * D,
            "what": "backward: q,k,v,dout (bf16) + log_fgate (f32) in, dq,dk,dv (bf16) + dlog_fgate (f32) out: 22*D B per token-head"}


def _alg_tc_state(B, T, H, D, C):
    th = B * T * H
    return {"bound": "hbm", "bytes": th * (8 * D + 2 * D * D // C),
            "what": "chunk states: log_fgate (f32) + two bf16 operands in, one bf16 (D,D) state per chunk out: 8*D + 2*D*D/C B per token-head"}


KERNEL_ALGORITHMIC = {
    "simt_intra_bwd_kernel": _alg_simt_intra_bwd,
    "simt_score_kernel": _alg_simt_score,
    "tc_chunk_fwd_kernel": _alg_tc_fwd,
    "tc_chunk_bwd_kernel": _alg_tc_bwd,
    "tc_state_kernel": _alg_tc_state,
    "tc_dstate_scan_kernel": _alg_tc_state,
    "_default": _alg_whole_step,
}


if __name__ == "__main__":
    main()
