#!/usr/bin/env python
"""Benchmark of the W4A4 quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload ("qlinear-8b-m4096"): one step = the three Llama-3-8B linear shapes
(K, N) in {(4096, 4096), (4096, 14336), (14336, 4096)} at M = 4096 tokens, each as
sign-adjusted online Hadamard rotation + per-token int4 quantization (one fused kernel on
bf16 activations) followed by the W4A4 GEMM with fused dequant epilogue (fp16 output).
Inputs are seeded synthetic tensors (activations ~N(0,1) with 0.1 % of channels x100, uniform
int4 weight codes, fp16 scales).  Metric: TOP/s = 2*M*N*K summed over the three linears /
device time.  With N > 1 the group shares ONE problem and runs it tensor-parallel (Megatron
split: the (4096, 14336) linear by output columns, the other two by input channels with an
all-gather of the input shards and an int32 all-reduce of the partial sums): strong scaling;
the timed region is bracketed by a barrier and a device synchronise and the slowest rank's
time is used.  `rows_data_parallel` gives the same three linears with the token rows dealt
to the ranks instead (no collective), `decode_llama3_8b` / `decode_mixtral_8x7b_shape` the
full-model and sparse-stack decode at tensor / expert parallelism N.

The JSON line also carries: `roofline` (the tcgen05 GEMM against the int8 tensor peak,
measured here with torch._int_mm), `rotate_quant` (the fused kernels against the HBM copy
peak: per-launch events, the marginal cost inside the step, and back to back), `sustained`
(the step repeated for seconds, with the sampled SM clock), `e2e` (the same step through
the public API from pinned host buffers, copies timed), `cpu_baseline` (the reference's own
CPU fake-quant forward of the same step on a bounded row sample, or the oracle's restatement
of it when the reference's files are absent), `clocks` (NVML samples taken during the timed
region) and `gpu_launches`.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M_TOKENS = 4096
SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096)]  # (K, N)
NBUF = 2  # activation/output buffer sets rotated between steps (each set alone exceeds L2)


def ops_per_step(m=M_TOKENS):
    return sum(2 * m * n * k for k, n in SHAPES)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", 0), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.005):
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.period = period_s

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s), "power_w_max": round(max(self.power), 1) if self.power else None}


# ----------------------------------------------------------------------------- CPU arm

CPU_ROWS = 256   # token rows of the workload one CPU step processes (bounded sample of the 4096)


def workload_config(world: int) -> dict:
    """The `config` object both arms print."""
    par = "rows x1 (one GPU, no collective)" if world == 1 else \
        f"tensor-parallel x{world}: (4096,14336) column split, (14336,4096) and (4096,4096) row split with all-gather + int32 all-reduce"
    return {"workload": "qlinear-8b-m4096", "M": M_TOKENS, "shapes_KN": SHAPES, "activations": "bf16", "output": "fp16",
            "parallelism": par, "l2": f"inputs larger than L2: {NBUF} rotating buffer sets of 368 MB"}


class CpuArm:
    """The CPU statement of one step (rotation + sign + per-token int4 fake-quant + bf16 F.linear over the
    three linears) on CPU_ROWS token rows.  With the reference's files at hand (a checkout, or oracle/_ref/
    placed by build()) it is the reference's own ActQuantWrapper.forward (fake_quant/quant_utils.py:322-386),
    kind "reference"; otherwise the oracle's restatement of it, kind "port"."""

    def __init__(self, rows: int = CPU_ROWS):
        import oracle
        from oracle import fake_quant as fq
        from oracle import ref_shim
        from signrot_b200.functional.hadamard import get_hadK
        self.rows = rows
        self.threads = os.cpu_count() or 1
        torch.set_num_threads(self.threads)
        self.kind = "reference" if ref_shim.available() else "port"
        self.cases = []
        for k, n in SHAPES:
            c = fq.make_linear_case(rows, k, n, seed=0)
            hadK, K = get_hadK(k)
            w = (oracle.unpack_i4(c["w_packed"]).float() * c["w_scale"].float()).to(torch.bfloat16)
            case = {"x": c["x"], "sign": c["sign"], "hadK": hadK, "K": K, "w_deq": w}
            if self.kind == "reference":
                qu = ref_shim.module("quant_utils")
                lin = torch.nn.Linear(k, n, bias=False, dtype=torch.bfloat16)
                lin.weight.data = w              # RTN weights with the sign already folded
                wrp = qu.ActQuantWrapper(lin)
                wrp.quantizer.configure(bits=4, groupsize=-1, sym=True, clip_ratio=1.0)
                wrp.online_full_had, wrp.had_K, wrp.K = True, hadK, K
                wrp.had_adj_sign, wrp.had_adj_ready = c["sign"], True
                case["wrapper"] = wrp
            self.cases.append(case)
        self.oracle, self.fq = oracle, fq

    def step(self) -> float:
        t0 = time.perf_counter()
        with torch.no_grad():
            for c in self.cases:
                if self.kind == "reference":
                    c["wrapper"](c["x"])
                else:
                    y = self.oracle.rotate(c["x"], c["hadK"], c["K"], c["sign"])
                    torch.nn.functional.linear(self.fq.act_fake_quant(y, 1.0, True), c["w_deq"])
        return time.perf_counter() - t0

    def run(self, steps: int, warmup: int):
        """Mean seconds per step over exactly `steps` steps after `warmup` untimed ones."""
        for _ in range(max(1, warmup)):
            self.step()
        return sum(self.step() for _ in range(steps)) / steps

    def describe(self, steps: int) -> str:
        what = ("the reference's ActQuantWrapper.forward, fake-quant branch (Hadamard through a CPU stand-in for the "
                "fast_hadamard_transform library)" if self.kind == "reference" else "oracle restatement of the fake-quant forward")
        return f"{self.rows} of {M_TOKENS} token rows per linear per step, mean of {steps} steps; {what}"


def cpu_baseline(steps: int = 20, warmup: int = 3):
    arm = CpuArm()
    steps = max(3, min(steps, 40))
    sec = arm.run(steps, warmup)
    return {"value": round(ops_per_step(arm.rows) / sec / 1e12, 4), "unit": "TOP/s", "cores": arm.threads,
            "kind": arm.kind, "sample": arm.describe(steps)}


def run_reference_arm(args, rank, world):
    """The reference's CPU implementation of the path, timed on all host threads; each step is the same
    bounded row sample of the workload that `cpu_baseline` of the GPU arm uses."""
    if rank != 0:
        return
    steps = max(1, args.steps)
    arm = CpuArm()
    sec = arm.run(steps, min(args.warmup, 5))
    val = round(ops_per_step(arm.rows) / sec / 1e12, 4)
    print(json.dumps({
        "impl": "reference", "metric": "w4a4_qlinear_tops", "value": val, "unit": "TOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None,
        "dtype": "bf16 fake-quant (cpu)", "data": "synthetic", "config": workload_config(world),
        "cpu_baseline": {"value": val, "unit": "TOP/s", "cores": arm.threads, "kind": arm.kind, "sample": arm.describe(steps)},
        "e2e": {"value": val, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------- GPU arm

def make_linear_case(M, K, N, seed=0):
    """Seeded synthetic inputs of one linear: activations ~N(0,1) in bf16 with 0.1 % of the
    channels x100, int4 weight codes uniform in [-8, 7], fp16 weight scales ~U(0.001, 0.01), a
    random +-1 sign vector."""
    import math
    from signrot_b200.functional import pack_i4
    g = torch.Generator().manual_seed(seed * 1000003 + K * 31 + N)
    x = torch.randn((M, K), generator=g, dtype=torch.float32)
    gc = torch.Generator().manual_seed(1234 + K)
    ch = torch.randperm(K, generator=gc)[: max(1, math.ceil(K / 1000))]
    x[:, ch] *= 100.0
    codes = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int8)
    w_scale = (torch.rand((N, 1), generator=g) * 0.009 + 0.001).to(torch.float16)
    sign = (torch.randint(0, 2, (K,), generator=g) * 2 - 1).to(torch.int8)
    return {"x": x.to(torch.bfloat16), "w_packed": pack_i4(codes), "w_scale": w_scale, "sign": sign}


def measure_int8_peak(dev):
    """Dense int8 tensor-core rate of cuBLASLt on this GPU (torch._int_mm 8192^3, best of 10)."""
    n = 8192
    a = torch.randint(-8, 8, (n, n), dtype=torch.int8, device=dev)
    b = torch.randint(-8, 8, (n, n), dtype=torch.int8, device=dev)
    for _ in range(3):
        torch._int_mm(a, b)
    best = float("inf")
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return 2 * n ** 3 / (best * 1e-3) / 1e12


class QlinearStep:
    """One step of the workload on this rank: the three linears, each rotate+quant followed by the W4A4 GEMM.
    world == 1: straight through the C ABI.  world > 1: tensor-parallel over the group (Megatron split): the
    (4096, 14336) linear column-parallel (replicated input, N / world output columns per rank), the (14336, 4096)
    and (4096, 4096) linears row-parallel (K / world input channels per rank: all-gather of the fp16 input shards,
    full-row rotate+quant on every rank, K-slice GEMM to int32, int32 all-reduce, dequant)."""

    def __init__(self, rank, world, dev):
        from signrot_b200 import _lib, tp
        from signrot_b200.functional import kernel
        from signrot_b200.functional.hadamard import get_hadK
        self.lib, self._lib, self.kernel = _lib.load(), _lib, kernel
        self.rank, self.world, self.dev, self.M = rank, world, dev, M_TOKENS
        self.stream = torch.cuda.current_stream().cuda_stream
        self.weights, self.sets = [], []
        M = self.M
        for k, n in SHAPES:
            c = make_linear_case(M, k, n, seed=0 if world > 1 else rank)     # the group shares one problem
            hadK, K = get_hadK(k)
            w = {"w": c["w_packed"].to(dev), "ws": c["w_scale"].to(dev), "sign": c["sign"].to(dev),
                 "hadK": hadK.to(dev, torch.float16) if hadK is not None else None, "K": K, "k": k, "n": n,
                 "scale": kernel.had_scale(k), "x_host": c["x"].pin_memory()}
            if world > 1:
                if (k, n) == (4096, 14336):
                    w["mode"] = "column"
                    w["tp"] = tp.ColumnParallelLinear4bit(w["w"], w["ws"])
                else:
                    w["mode"] = "row"
                    w["tp"] = tp.RowParallelLinear4bit(w["w"], w["ws"], hadK=w["hadK"], K_had=K, sign=w["sign"])
                del w["w"]
            self.weights.append(w)
        for b in range(NBUF):
            one = []
            for w in self.weights:
                x = w["x_host"].to(dev)
                if b:
                    x = x.roll(b, 0).contiguous()
                if world > 1 and w["mode"] == "row":
                    x = x[:, w["tp"].begin:w["tp"].end].contiguous()        # this rank's input channels
                one.append({"x": x, "q": torch.empty((M, w["k"] // 2), dtype=torch.uint8, device=dev),
                            "s": torch.empty((M, 1), dtype=torch.float16, device=dev),
                            "out": torch.empty((M, w["n"]), dtype=torch.float16, device=dev) if world == 1 else None})
            self.sets.append(one)
        self.skip_rotate = False      # one GPU only: the step without its rotate+quant launches (codes of an earlier step)

    # ---- one GPU: raw C-ABI launches
    def rotate(self, w, b, stream=None):
        ptr = self._lib.ptr
        rc = self.lib.sr_rotate_quant(ptr(b["x"]), self._lib.SR_BF16, self.M, w["k"], ptr(w["hadK"]), w["K"], w["scale"],
                                      ptr(w["sign"]), None, 0, 1.0, 0, ptr(b["q"]), ptr(b["s"]), None, None,
                                      stream or self.stream)
        if rc:
            raise RuntimeError(self.lib.sr_last_error().decode())

    def gemm(self, w, b):
        ptr = self._lib.ptr
        rc = self.lib.sr_w4a4_linear(ptr(b["q"]), ptr(b["s"]), None, ptr(w["w"]), ptr(w["ws"]), None, None, self.M,
                                     w["n"], w["k"], ptr(b["out"]), self.stream)
        if rc:
            raise RuntimeError(self.lib.sr_last_error().decode())

    def run(self, i, ev=None):
        bufs = self.sets[i % NBUF]
        for j, (w, b) in enumerate(zip(self.weights, bufs)):
            if self.world == 1:
                if ev is not None:
                    ev[j][0].record()
                if not self.skip_rotate:
                    self.rotate(w, b)
                if ev is not None:
                    ev[j][1].record()
                self.gemm(w, b)
                if ev is not None:
                    ev[j][2].record()
            elif w["mode"] == "column":
                packed = self.kernel.rotate_quant(b["x"], w["hadK"], w["K"], sign=w["sign"])
                b["y"] = w["tp"].forward(packed)                      # [M, N / world], stays sharded
            else:
                b["y"] = w["tp"].forward(b["x"])                      # [M, N] on every rank

    def h2d_bytes(self):
        return sum(b["x"].numel() * 2 for b in self.sets[0])

    def d2h_bytes(self):
        return sum(self.M * w["n"] * 2 // self.world for w in self.weights)


def timed_steps(step, steps, world, dev, local_rank, evs=None):
    """Exactly `steps` steps between two events, bracketed by a barrier and a device synchronise; the slowest
    rank's device time.  Returns (ms, clock summary)."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local_rank) as clk:
        e0.record()
        for i in range(steps):
            step.run(i, evs.get(i) if evs else None)
        e1.record()
        torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = t.item()
    return ms, clk.summary()


def run_ours(args, rank, world, local_rank):
    import signrot_b200  # noqa: F401  (fails loudly when the library is missing)
    from signrot_b200 import _lib
    from signrot_b200.functional import kernel

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    M = M_TOKENS
    step = QlinearStep(rank, world, dev)
    weights, sets = step.weights, step.sets

    int8_peak = measure_int8_peak(dev) if rank == 0 else None
    for i in range(args.warmup):
        step.run(i)
    torch.cuda.synchronize()
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel reported a device-side failure during warm-up")

    # ---- timed region: exactly `steps` steps, device time.  On one GPU per-kernel events sit inside it on every
    # 8th step (an event record between two launches keeps the second kernel's set-up from overlapping the first
    # one's tail, so instrumenting every step would slow the thing being measured).
    ev_every = 8
    sampled = [i for i in range(args.steps) if i % ev_every == 0] if world == 1 else []
    evs = {i: [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in SHAPES] for i in sampled}
    ms, clocks = timed_steps(step, args.steps, world, dev, local_rank, evs)
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel reported a device-side failure during the timed region")

    # ---- the same step back to back for a few seconds: what the path sustains under the power cap, with the
    # SM clock sampled beside it (nothing about the GPU is changed; NVML is only read)
    sus_steps = max(args.steps, int(3000.0 / max(ms / args.steps, 1e-3)))
    sus_steps = min(sus_steps, 20000)
    sus_ms, sus_clocks = timed_steps(step, sus_steps, world, dev, local_rank)

    rot_ms = gemm_ms = rot_only_ms = None
    gemm_only_ms = None
    if world == 1:
        # the step without the rotate+quant launches (the GEMMs read the codes an earlier step left): the difference to the
        # full step is what the three fused kernels cost inside the step, launch gaps and dependent-launch overlap included,
        # with no event record perturbing the stream
        step.skip_rotate = True
        gemm_only_ms, _ = timed_steps(step, max(args.steps, 50), world, dev, local_rank)
        gemm_only_ms /= max(args.steps, 50)
        step.skip_rotate = False
        full_ms, _ = timed_steps(step, max(args.steps, 50), world, dev, local_rank)
        full_ms /= max(args.steps, 50)
        rot_ms = [sum(evs[i][j][0].elapsed_time(evs[i][j][1]) for i in sampled) / len(sampled) for j in range(3)]
        gemm_ms = [sum(evs[i][j][1].elapsed_time(evs[i][j][2]) for i in sampled) / len(sampled) for j in range(3)]
        # the rotation kernels back to back (no GEMM, no launch gap between dependent kernels): one CUDA graph of
        # 16 launches per shape over the rotating input sets, replayed once under CUDA events
        rot_only_ms = []
        try:
            for j, w in enumerate(weights):
                bufs = [sets[b][jj] for b in range(NBUF) for jj, ww in enumerate(weights) if ww["k"] == w["k"]]
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    for i in range(16):
                        step.rotate(w, bufs[i % len(bufs)], torch.cuda.current_stream().cuda_stream)
                gr.replay()
                torch.cuda.synchronize()
                g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                g0.record()
                gr.replay()
                g1.record()
                torch.cuda.synchronize()
                rot_only_ms.append(g0.elapsed_time(g1) / 16)
        except Exception:
            rot_only_ms = []

    # ---- end to end through the public API from pinned host memory.  Every step copies its inputs host -> device
    # and its outputs device -> host; the two directions of the link run at the same time (three streams: copy-in,
    # compute, copy-out, ordered by events, one device buffer per linear), as a serving loop would drive it.  With
    # several ranks every rank copies the input channels it owns and 1 / world of the output rows.
    s_in, s_comp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    x_host = []
    for w in weights:
        xh = w["x_host"]
        if world > 1 and w["mode"] == "row":
            xh = xh[:, w["tp"].begin:w["tp"].end].contiguous().pin_memory()
        x_host.append(xh)
    x_dev = [torch.empty_like(xh, device=dev) for xh in x_host]
    rows_out = M // world
    out_host = [torch.empty((rows_out, w["n"] // (world if world > 1 and w["mode"] == "column" else 1)),
                            dtype=torch.float16).pin_memory() for w in weights]
    ev_x_ready = [torch.cuda.Event() for _ in weights]
    ev_x_free = [torch.cuda.Event() for _ in weights]
    ev_y_ready = [torch.cuda.Event() for _ in weights]
    ev_y_done = [torch.cuda.Event() for _ in weights]
    y_keep = [None] * len(weights)

    def e2e_step():
        for j, (w, oh) in enumerate(zip(weights, out_host)):
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_x_free[j])
                x_dev[j].copy_(x_host[j], non_blocking=True)
                ev_x_ready[j].record(s_in)
            with torch.cuda.stream(s_comp):
                s_comp.wait_event(ev_x_ready[j])
                if world == 1:
                    pk = kernel.rotate_quant(x_dev[j], w["hadK"], w["K"], sign=w["sign"])
                    ev_x_free[j].record(s_comp)
                    s_comp.wait_event(ev_y_done[j])      # the previous result of this linear has left the device
                    y = kernel.w4a4_linear(pk, w["w"], w["ws"])
                elif w["mode"] == "column":
                    pk = kernel.rotate_quant(x_dev[j], w["hadK"], w["K"], sign=w["sign"])
                    ev_x_free[j].record(s_comp)
                    s_comp.wait_event(ev_y_done[j])
                    y = w["tp"].forward(pk)
                else:
                    s_comp.wait_event(ev_y_done[j])
                    y = w["tp"].forward(x_dev[j])
                    ev_x_free[j].record(s_comp)
                ev_y_ready[j].record(s_comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_y_ready[j])
                part = y if world == 1 else y[rank * rows_out:(rank + 1) * rows_out]
                oh.copy_(part, non_blocking=True)
                ev_y_done[j].record(s_out)
                y.record_stream(s_out)
            y_keep[j] = y
    e2e_steps = max(2, min(args.steps, 10))
    e2e_step()
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        e2e_s = t.item()
    h2d = sum(xh.numel() * 2 for xh in x_host)
    d2h = sum(oh.numel() * 2 for oh in out_host)
    del x_dev, y_keep, step, sets
    torch.cuda.empty_cache()

    # ---- several GPUs: the same three linears with the token rows dealt to the ranks instead (every rank its own
    # 4096 rows, no collective on the path), for comparison with the tensor-parallel step above
    dp_ms = None
    if world > 1:
        dp_step = QlinearStep(rank, 1, dev)
        for i in range(args.warmup):
            dp_step.run(i)
        dp_ms, _ = timed_steps(dp_step, args.steps, world, dev, local_rank)
        del dp_step
        torch.cuda.empty_cache()

    # ---- the full-model and sparse-stack configurations at this group size (decode tokens/s)
    extras = {}
    if not args.no_models:
        for key, fn in (("decode_llama3_8b", lambda: run_decode_model("decode_model_llama3_8b", {}, 8, 2048, 128, dev, world,
                                                                     quiet=True)),
                        ("decode_mixtral_8x7b_shape", lambda: run_decode_model(
                            "decode_model_mixtral_8x7b_shape",
                            {"num_local_experts": 8, "num_experts_per_tok": 2, "vocab_size": 32000}, 64, 64, 64, dev,
                            world, quiet=True, prefill_probe=4096))):
            try:
                extras[key] = fn()
            except Exception as exc:
                extras[key] = {"error": str(exc)[:300]}
            torch.cuda.empty_cache()

    if rank != 0:
        return
    pk_ = peaks()
    ops = ops_per_step()
    # one GPU: `world` is 1.  Several GPUs: the group shares ONE problem (strong scaling), so the job's work is `ops`.
    value = ops * args.steps / (ms * 1e-3) / 1e12
    sus_value = ops * sus_steps / (sus_ms * 1e-3) / 1e12
    out = {
        "metric": "w4a4_qlinear_tops", "value": round(value, 2), "unit": "TOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
        "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None,
        "dtype": "int4 codes, int8 tensor-core MMA, int32 accumulate", "data": "synthetic",
        "config": workload_config(world),
        "sustained": {"tops": round(sus_value, 2), "ms_per_step": round(sus_ms / sus_steps, 4), "steps": sus_steps,
                      "seconds": round(sus_ms * 1e-3, 2), "sm_mhz_median": sus_clocks.get("sm_mhz"),
                      "samples": sus_clocks.get("samples"), "reasons": sus_clocks.get("reasons"),
                      "power_w_max": sus_clocks.get("power_w_max"),
                      "tops_at_max_clock": (round(sus_value * sus_clocks["sm_max_mhz"] / sus_clocks["sm_mhz"], 2)
                                            if sus_clocks.get("sm_mhz") and sus_clocks.get("sm_max_mhz") else None),
                      "note": "the same step back to back; tops_at_max_clock scales by max / median sampled SM clock"},
        "e2e": {"value": round(ops * e2e_steps / e2e_s / 1e12, 3), "unit": "TOP/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "note": "bytes per rank" if world > 1 else "host buffers in, host buffers out"},
        "clocks": clocks,
    }
    if world == 1:
        gemm_ops = [2 * M * n * k for k, n in SHAPES]
        gemm_ach = sum(gemm_ops) / (sum(gemm_ms) * 1e-3) / 1e12
        rot_bytes = [M * k * 2 + M * k // 2 + M * 2 + k for k, _ in SHAPES]
        rot_ach = sum(rot_bytes) / (sum(rot_ms) * 1e-3) / 1e9
        sus_peak = 2 * pk_.get("bf16_tflops_sustained", 0) or None
        out["gpu_launches"] = 6 * args.steps
        out["config"]["kernel_events"] = f"per-kernel CUDA events on every {ev_every}th step of the timed region"
        out["roofline"] = {
            "kernel": "gemm_tc3_kernel (persistent tcgen05 cta_group::2 kind::i8, 256x256 tile per CTA pair, TMA-staged packed tiles, fused dequant)",
            "bound": "tensor", "achieved": round(gemm_ach, 1), "peak": round(int8_peak, 1), "unit": "TOP/s",
            "frac": round(gemm_ach / int8_peak, 4),
            "peak_source": "measured live: torch._int_mm 8192^3 int8, best of 10 (MEASURED_PEAKS.json has no int8 figure)",
            "peak_bf16_x2": round(2 * pk_["bf16_tflops"], 1), "frac_of_bf16_x2": round(gemm_ach / (2 * pk_["bf16_tflops"]), 4),
            "traffic": 123.3e6,
            "traffic_note": "bytes of DRAM traffic (42.0 MB read + 81.3 MB written) of one M=4096 K=4096 N=14336 launch, from one ncu capture "
                            "(profiles/gemm_tc3_kernel_m4096_k4096_n14336.md), not from this run; the launch's algorithmic "
                            "bytes are 155 MB: part of the fp16 output is still in L2 when the kernel ends",
            "per_shape_ms": [round(v, 4) for v in gemm_ms],
            "per_shape_tops": [round(o / (t * 1e-3) / 1e12, 1) for o, t in zip(gemm_ops, gemm_ms)]}
        # in the sustained run the step is GEMM-dominated; its whole-step rate against 2 x the sustained bf16 figure
        if sus_peak:
            out["sustained"]["step_frac_of_bf16_sustained_x2"] = round(sus_value / sus_peak, 4)
        marginal_ms = max(full_ms - gemm_only_ms, 1e-6)
        out["rotate_quant"] = {
            "kernel": "fused rotate+sign+quant (tcgen05 + TMA kernels for n = 4096 and n = 14336)", "bound": "hbm",
            "achieved": round(rot_ach, 1),
            "peak": pk_["hbm_gbs"], "unit": "GB/s", "frac": round(rot_ach / pk_["hbm_gbs"], 4),
            "peak_source": pk_["source"], "per_shape_ms": [round(v, 4) for v in rot_ms],
            "per_shape_gbs": [round(b / (t * 1e-3) / 1e9, 1) for b, t in zip(rot_bytes, rot_ms)],
            "note": "per-shape figures: CUDA events around each launch on every 8th step (an event record between two "
                    "launches removes the dependent-launch overlap, so these are upper bounds of the in-step cost)",
            "in_step_marginal": {"ms_per_step": round(marginal_ms, 4), "step_ms": round(full_ms, 4),
                                 "step_without_rotate_ms": round(gemm_only_ms, 4),
                                 "achieved": round(sum(rot_bytes) / (marginal_ms * 1e-3) / 1e9, 1),
                                 "frac": round(sum(rot_bytes) / (marginal_ms * 1e-3) / 1e9 / pk_["hbm_gbs"], 4),
                                 "note": "step time minus the time of the same step without its three rotate+quant launches"},
            "back_to_back": ({"per_shape_ms": [round(v, 4) for v in rot_only_ms],
                              "achieved": round(sum(rot_bytes) / (sum(rot_only_ms) * 1e-3) / 1e9, 1),
                              "frac": round(sum(rot_bytes) / (sum(rot_only_ms) * 1e-3) / 1e9 / pk_["hbm_gbs"], 4),
                              "note": "CUDA-graph replay of 16 launches per shape, inputs rotate over > 126 MB"}
                             if rot_only_ms and len(rot_only_ms) == 3 else None)}
    else:
        out["rows_data_parallel"] = {
            "value": round(world * ops * args.steps / (dp_ms * 1e-3) / 1e12, 2), "unit": "TOP/s",
            "ms_per_step": round(dp_ms / args.steps, 4), "scaling": "weak",
            "note": "every rank runs the one-GPU step on its own 4096 token rows (rows are independent: no collective); "
                    "the headline value above is the tensor-parallel step on ONE shared problem"}
        out["gpu_launches"] = 10 * args.steps      # per rank: 3 rotate+quant, 3 GEMM, 2 code-slice copies, 2 dequant
        out["roofline"] = {"kernel": "gemm_tc3_kernel on the per-rank shards", "bound": "tensor", "achieved": None,
                           "peak": round(int8_peak, 1), "unit": "TOP/s", "frac": None, "traffic": None,
                           "note": "per-kernel events are taken on one GPU only; at this size the step is bound by the "
                                   "int32 all-reduce and the fp16 all-gather of the row-parallel linears"}
    out.update(extras)
    if world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline(args.steps)
    print(json.dumps(out))


def run_kernel_case(name: str):
    """A few launches of ONE kernel on a real-size shape, for `ncu -k ... -c ...` captures
    (device memory stays below 1 GB, every launch works on buffers larger than L2 in total)."""
    import signrot_b200  # noqa: F401
    from signrot_b200.functional import kernel
    from signrot_b200.functional.hadamard import get_hadK
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    M = M_TOKENS
    if name in ("gemm", "gemm_small", "gemm_mid"):
        # gemm_mid: 256 rows against the (14336 -> 4096) projection: the CTA-pair kernel with K split four ways
        k, n = (14336, 4096) if name == "gemm_mid" else (4096, 14336)
        m = M if name == "gemm" else (256 if name == "gemm_mid" else 16)
        c = make_linear_case(m, k, n)
        hadK, K = get_hadK(k)
        pk = kernel.rotate_quant(c["x"].to(dev), hadK, K, sign=c["sign"].to(dev))
        w, ws = c["w_packed"].to(dev), c["w_scale"].to(dev)
        for _ in range(5):
            kernel.w4a4_linear(pk, w, ws)
    elif name in ("rotate4096", "rotate14336"):
        k = 4096 if name == "rotate4096" else 14336
        c = make_linear_case(M, k, 8)
        hadK, K = get_hadK(k)
        x, sg = c["x"].to(dev), c["sign"].to(dev)
        for _ in range(5):
            kernel.rotate_quant(x, hadK, K, sign=sg)
    elif name == "decode":
        from signrot_b200.transformers import kv_cache as kvc
        B, Hq, Hkv, T, page = 16, 32, 8, 4096, 256
        cache = kvc.MultiLayerPagedKVCache4Bit(B, page, T + 64, dev, 1, Hkv, 128, group_size=Hq // Hkv)
        g = torch.Generator().manual_seed(0)
        kk = torch.randn((B, T, Hkv, 128), generator=g).half().to(dev)
        cache.update(kk, kk, 0)
        q = torch.randn((B, 1, Hq, 128), generator=g).half().to(dev)
        for _ in range(5):
            attend = cache.update(kk[:, :1].contiguous(), kk[:, :1].contiguous(), 0)
            attend(q)
    elif name == "decode_layer":
        from signrot_b200.transformers import kv_cache as kvc
        B, Hq, Hkv, T, page = 16, 32, 8, 4096, 256
        cache = kvc.MultiLayerPagedKVCache4Bit(B, page, T + 64, dev, 1, Hkv, 128, group_size=Hq // Hkv)
        g = torch.Generator().manual_seed(0)
        kk = torch.randn((B, T, Hkv, 128), generator=g).half().to(dev)
        cache.update(kk, kk, 0)
        cache.refresh_specs()
        layer = build_decode_layer(cache, B, Hq, Hkv, dev)
        for _ in range(3):
            layer()
    else:
        raise SystemExit(f"unknown kernel case {name}")
    torch.cuda.synchronize()
    print(f"kernel case {name}: done")


def build_decode_layer(cache, B, Hq, Hkv, dev):
    """Closure running one decode step of a Llama-3-8B-shaped decoder layer (hidden 4096, FFN 14336,
    head_dim 128) on `cache` (already holding the context): RMSNorm, quantizer, q/k/v, RoPE, fused
    KV append, int4 decode attention, head-wise rotation + o_proj, RMSNorm, quantizer, gate/up,
    SwiGLU, had28 rotation + down_proj, residuals."""
    from signrot_b200 import nn as snn
    from signrot_b200.functional import kernel
    from signrot_b200.functional.hadamard import get_hadK
    hid, ffn, D = 4096, 14336, 128
    gen = torch.Generator().manual_seed(2)

    def qlin(k_, n_):
        m_ = snn.Linear4bit(k_, n_).to(dev)
        m_.weight.copy_(torch.randint(0, 256, (n_, k_ // 2), generator=gen, dtype=torch.uint8))
        m_.weight_scales = (torch.rand((n_, 1), generator=gen) * 0.5 / k_ + 0.5 / k_).half().to(dev)
        return m_
    lq, lk, lv, lo = qlin(hid, Hq * D), qlin(hid, Hkv * D), qlin(hid, Hkv * D), qlin(Hq * D, hid)
    lg, lu, ld = qlin(hid, ffn), qlin(hid, ffn), qlin(ffn, hid)
    norm, quant = snn.RMSNorm(hid, eps=1e-5).to(dev), snn.Quantizer()
    had28, K28 = get_hadK(ffn)
    had28 = had28.to(dev, torch.float16)
    sg_down = (torch.randint(0, 2, (ffn,), generator=gen) * 2 - 1).to(torch.int8).to(dev)
    ang = torch.rand((1, 1, D), generator=gen)
    cos, sin = torch.cos(ang).half().to(dev), torch.sin(ang).half().to(dev)   # [1, T = 1, D]
    xdec = torch.randn((B, 1, hid), generator=gen).half().to(dev)
    cache.freeze_specs(True)

    def decode_layer():
        h = norm(xdec)
        pkd = quant(h)
        qd_ = lq(pkd).view(B, 1, Hq, D)
        kd_ = lk(pkd).view(B, 1, Hkv, D)
        vd_ = lv(pkd).view(B, 1, Hkv, D)
        kernel.rope_qk(qd_, kd_, cos, sin)
        attend = cache.update(kd_, vd_, 0)
        a_ = attend(qd_).reshape(B, 1, Hq * D)
        x1 = xdec + lo(kernel.rotate_quant(a_, heads=Hq))
        pk2 = quant(norm(x1))
        mid = kernel.swiglu(lg(pk2), lu(pk2))
        return x1 + ld(kernel.rotate_quant(mid, had28, K28, sign=sg_down))
    return decode_layer


def _time_cuda(fn, iters=30, warmup=5, graph=True):
    """Mean device time of fn() in ms.  The launches are captured into one CUDA graph and replayed,
    so the host's per-call cost (tens of microseconds in Python) is not part of a small kernel's figure;
    callables that cannot be captured are timed launch by launch."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        try:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for _ in range(iters):
                    fn()
            gr.replay()
            torch.cuda.synchronize()
            e0.record()
            gr.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / iters
        except Exception:
            torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def run_sweep():
    """Secondary measurements (one JSON line each, not the headline): the fused-op sweep at M in
    {1, 16, 256, 4096} over the three Llama-3-8B linear shapes, int4-KV decode attention at batch 16 and
    context 4096, one Mixtral-shaped MoE block at 64 and 4096 tokens.  Each timing is the mean of 30 launches after 5
    warm-ups, replayed from a CUDA graph; small cases re-use L2-resident buffers, so they measure L2 behaviour."""
    import signrot_b200  # noqa: F401
    from signrot_b200.functional import kernel
    from signrot_b200.functional.hadamard import get_hadK
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm = peaks()["hbm_gbs"]
    for m in (1, 16, 256, 4096):
        for k, n in SHAPES:
            c = make_linear_case(m, k, n)
            hadK, K = get_hadK(k)
            x, sg, w, ws = c["x"].to(dev), c["sign"].to(dev), c["w_packed"].to(dev), c["w_scale"].to(dev)
            hk = hadK.to(dev, torch.float16) if hadK is not None else None
            pk = kernel.rotate_quant(x, hk, K, sign=sg)
            t_rot = _time_cuda(lambda: kernel.rotate_quant(x, hk, K, sign=sg))
            t_gemm = _time_cuda(lambda: kernel.w4a4_linear(pk, w, ws))
            rot_bytes = m * k * 2.5 + 2 * m + k
            w_bytes = n * k / 2 + m * k / 2 + 2 * m * n
            print(json.dumps({"case": "qlinear", "M": m, "K": k, "N": n,
                              "rotate_quant_us": round(t_rot * 1e3, 2),
                              "rotate_quant_gbs": round(rot_bytes / t_rot / 1e6, 1),
                              "gemm_us": round(t_gemm * 1e3, 2),
                              "gemm_tops": round(2 * m * n * k / t_gemm / 1e9, 1),
                              "gemm_gbs": round(w_bytes / t_gemm / 1e6, 1),
                              "gemm_frac_hbm": round(w_bytes / t_gemm / 1e6 / hbm, 3)}))
    # int4-KV GQA decode attention, B=16, ctx 4096, 32 q / 8 kv heads, page 256
    from signrot_b200.transformers import kv_cache as kvc
    B, Hq, Hkv, T, page = 16, 32, 8, 4096, 256
    cache = kvc.MultiLayerPagedKVCache4Bit(B, page, T + 64, dev, 1, Hkv, 128, group_size=Hq // Hkv)
    g = torch.Generator().manual_seed(0)
    kk = torch.randn((B, T, Hkv, 128), generator=g).half().to(dev)
    vv = torch.randn((B, T, Hkv, 128), generator=g).half().to(dev)
    t_fill = _time_cuda(lambda: (cache.reset(), cache.update(kk, vv, 0)), iters=5, warmup=1, graph=False)
    cache.reset()
    cache.update(kk, vv, 0)
    specs = cache.refresh_specs()
    q = torch.randn((B, Hq, 128), generator=g).half().to(dev)
    o = torch.empty_like(q)
    chunks, tmp = cache._stub.num_chunks, cache._stub.tmp
    t_dec = _time_cuda(lambda: kvc.batch_decode_i4(o, q, **specs, layer_idx=0, tmp=tmp, num_chunks=chunks,
                                                   hadamard_q=True))
    kv_bytes = B * T * Hkv * 68 * 2
    print(json.dumps({"case": "decode_attention_i4", "B": B, "ctx": T, "q_heads": Hq, "kv_heads": Hkv,
                      "chunks": chunks, "decode_us": round(t_dec * 1e3, 2),
                      "kv_gbs": round(kv_bytes / t_dec / 1e6, 1), "frac_hbm": round(kv_bytes / t_dec / 1e6 / hbm, 3),
                      "prefill_append_quant_us": round(t_fill * 1e3, 1)}))
    # one layer of the full model: decode step of a Llama-3-8B-shaped decoder layer, batch 16 at context 4096,
    # int4 weights + int4 paged KV cache, every operator from this package, replayed from one CUDA graph
    decode_layer = build_decode_layer(cache, B, Hq, Hkv, dev)
    hid, ffn, D = 4096, 14336, 128
    try:
        t_layer = _time_cuda(decode_layer, iters=20, warmup=3)
        w_bytes = (2 * hid * Hq * D + 2 * hid * Hkv * D + 3 * hid * ffn) / 2
        print(json.dumps({"case": "decode_step_llama3_8b_layer", "batch": B, "ctx": T, "layer_us": round(t_layer * 1e3, 1),
                          "weight_plus_kv_gbs": round((w_bytes + kv_bytes) / t_layer / 1e6, 1),
                          "tokens_per_s_32_layers": round(B / (32 * t_layer * 1e-3), 1),
                          "note": "one layer timed, 32 identical layers assumed; embeddings and lm_head not included"}))
    except Exception as e:  # the sweep is secondary: report and go on
        print(json.dumps({"case": "decode_step_llama3_8b_layer", "error": str(e)[:200]}))
    cache.freeze_specs(False)
    # one Mixtral-8x7B-shaped MoE block (8 experts, top-2, hidden 4096, ffn 14336)
    from signrot_b200 import nn as snn
    E, hid, ffn, top_k = 8, 4096, 14336, 2
    gen = torch.Generator().manual_seed(1)
    def wq(nn_, kk_):
        return torch.randint(0, 256, (E, nn_, kk_ // 2), generator=gen, dtype=torch.uint8).to(dev)
    def sc(nn_, kk_):
        return (torch.rand((E, nn_), generator=gen) * 0.5 / kk_ + 0.5 / kk_).half().to(dev)
    gate = torch.nn.Linear(hid, E, bias=False).half().to(dev)
    sign = (torch.randint(0, 2, (E, ffn), generator=gen) * 2 - 1).to(torch.int8).to(dev)
    blk = snn.SignRotMoEBlock(gate, top_k=top_k, norm_topk_prob=True, w_gate=wq(ffn, hid), s_gate=sc(ffn, hid),
                              w_up=wq(ffn, hid), s_up=sc(ffn, hid), w_down=wq(hid, ffn), s_down=sc(hid, ffn),
                              sign_down=sign)
    for tokens in (64, 4096):
        xm = torch.randn((1, tokens, hid), generator=gen).half().to(dev)
        t_moe = _time_cuda(lambda: blk(xm), iters=5 if tokens > 64 else 20, warmup=2)
        w_bytes = 3 * E * ffn * hid / 2
        print(json.dumps({"case": "moe_block", "tokens": tokens, "experts": E, "top_k": top_k,
                          "block_ms": round(t_moe, 3), "expert_weight_gbs": round(w_bytes / t_moe / 1e6, 1),
                          "tops": round(2 * 3 * tokens * top_k * ffn * hid / t_moe / 1e9, 1)}))
    del blk, cache
    torch.cuda.empty_cache()
    # the whole 32-layer stacks (dense and sparse) through the decode-graph glue
    for name, kw, bsz, prompt, steps in (
            ("decode_model_llama3_8b", {}, 8, 2048, 128),
            ("decode_model_mixtral_8x7b_shape", {"num_local_experts": 8, "num_experts_per_tok": 2, "vocab_size": 32000},
             64, 64, 64)):
        try:
            run_decode_model(name, kw, bsz, prompt, steps, dev)
        except Exception as e:
            print(json.dumps({"case": name, "error": str(e)[:300]}))


def run_decode_model(name, cfg_kwargs, bsz, prompt, steps, dev, world=1, quiet=False, prefill_probe=0):
    """Full decoder stack (the full-model and sparse-stack configurations): random-init int4 weights, int4 paged KV
    cache, prefill of `prompt` tokens per request, then `steps` decode steps replayed from one CUDA graph.
    world > 1: the stack is sharded over the process group first (`shard_decoder_`: attention tensor-parallel by
    heads, dense MLP tensor-parallel, sparse block expert-parallel; decode-size exchanges over peer memory, prefill
    through the collective library), timed as the slowest rank.  `prefill_probe`: also time one prefill of that many
    tokens for one request.  Returns (and prints unless `quiet`) a dict: decode tokens/s (bsz * steps / device time),
    prefill tokens/s, and the bytes of weights + cache a decode step must read against the measured HBM figure."""
    from signrot_b200.transformers import kernel_utils as ku
    hbm = peaks()["hbm_gbs"]
    cfg = ku.DecoderConfig(**cfg_kwargs)
    with torch.device(dev):
        model = ku.KernelDecoderModel(cfg)
    model = model.to(dev).random_init_(0)
    if world > 1:
        ku.shard_decoder_(model)
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(1000, 8000, (bsz, prompt), generator=gen).to(dev)
    cache = ku.build_paged_cache(model, bsz, prompt + steps + 8)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def slowest(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return t.item()

    with torch.no_grad():
        model(ids, past_key_values=cache, last_token_only=True)      # warm-up prefill (first-use costs)
        cache.reset()
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        e0.record()
        logits = model(ids, past_key_values=cache, last_token_only=True).logits
        e1.record()
        torch.cuda.synchronize()
        t_prefill = slowest(e0.elapsed_time(e1))
        tok = logits[:, -1:].argmax(-1)
        dec = ku.try_graph_decoder(model, cache, bsz)
        graphed = dec is not None
        for _ in range(3):                               # warm-up steps (they advance the cache like real ones)
            tok = (dec.step(tok) if graphed else model(tok, past_key_values=cache).logits)[:, -1:].argmax(-1)
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            tok = (dec.step(tok) if graphed else model(tok, past_key_values=cache).logits)[:, -1:].argmax(-1)
        e1.record()
        torch.cuda.synchronize()
        t_dec = slowest(e0.elapsed_time(e1)) / steps
        t_probe = None
        if prefill_probe:
            del cache, dec
            torch.cuda.empty_cache()
            probe_ids = torch.randint(1000, 8000, (1, prefill_probe), generator=gen).to(dev)
            pc = ku.build_paged_cache(model, 1, prefill_probe + 8)
            model(probe_ids, past_key_values=pc, last_token_only=True)
            pc.reset()
            if world > 1:
                torch.distributed.barrier()
            torch.cuda.synchronize()
            e0.record()
            model(probe_ids, past_key_values=pc, last_token_only=True)
            e1.record()
            torch.cuda.synchronize()
            t_probe = slowest(e0.elapsed_time(e1))
            del pc
    from signrot_b200 import _lib
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel gave up a bounded device-side wait")
    finite = bool(torch.isfinite(logits).all())
    full = ku.DecoderConfig(**cfg_kwargs)                # byte accounting on the unsharded geometry: the whole job
    hid, ffn, L = full.hidden_size, full.intermediate_size, full.num_hidden_layers
    attn_w = (2 * hid * full.num_attention_heads * full.head_dim + 2 * hid * full.num_key_value_heads * full.head_dim) / 2
    if full.num_local_experts:
        mlp_w = 3 * hid * ffn / 2 * min(full.num_local_experts, bsz * full.num_experts_per_tok)
    else:
        mlp_w = 3 * hid * ffn / 2
    ctx = prompt + 3 + steps / 2
    kv = bsz * ctx * full.num_key_value_heads * 68 * 2
    step_bytes = L * (attn_w + mlp_w + kv) + full.vocab_size * hid * 2 * world     # the fp16 head is replicated
    res = {"case": name, "n_gpus": world, "batch": bsz, "prefill_tokens": prompt, "decode_steps": steps, "layers": L,
           "experts": full.num_local_experts, "graph_replay": graphed, "finite": finite,
           "parallelism": "one GPU" if world == 1 else (f"attention tensor-parallel x{world}, " + (
               f"experts x{world}" if full.num_local_experts else f"MLP tensor-parallel x{world}")),
           "decode_ms_per_step": round(t_dec, 3), "decode_tok_s": round(bsz / t_dec * 1e3, 1),
           "prefill_ms": round(t_prefill, 1), "prefill_tok_s": round(bsz * prompt / t_prefill * 1e3, 1),
           "step_bytes_gb": round(step_bytes / 1e9, 3), "step_gbs_per_gpu": round(step_bytes / world / t_dec / 1e6, 1),
           "frac_hbm": round(step_bytes / world / t_dec / 1e6 / hbm, 3)}
    if t_probe is not None:
        res["prefill_probe_tokens"], res["prefill_probe_ms"] = prefill_probe, round(t_probe, 1)
        res["prefill_probe_tok_s"] = round(prefill_probe / t_probe * 1e3, 1)
    if not quiet:
        res["note"] = ("weights (every expert a step can touch), int4 KV at the mean context and the fp16 lm_head counted once "
                       "per step; prefill time is the second of two calls, dense prefill attention included")
        print(json.dumps(res))
    del model
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-models", action="store_true", help="skip the full-model / sparse-stack decode measurements")
    ap.add_argument("--sweep", action="store_true",
                    help="secondary measurements of the other configurations (JSON lines)")
    ap.add_argument("--kernel-case", default=None,
                    help="run a few launches of one kernel and exit (for ncu): gemm | gemm_small | gemm_mid | rotate4096 | decode_layer | "
                         "rotate14336 | decode")
    args = ap.parse_args()
    if args.kernel_case == "decode_model_small":
        # two Llama-3-8B-shaped layers, batch 8 at context 2048: three eager decode steps (launch lists)
        from signrot_b200.transformers import kernel_utils as ku
        dev = torch.device("cuda", 0)
        with torch.device(dev):
            model = ku.KernelDecoderModel(ku.DecoderConfig(num_hidden_layers=2, vocab_size=4096))
        model = model.to(dev).random_init_(0)
        cache = ku.build_paged_cache(model, 8, 2048 + 16)
        with torch.no_grad():
            model(torch.randint(0, 4096, (8, 2048), device=dev), past_key_values=cache, last_token_only=True)
            tok = torch.randint(0, 4096, (8, 1), device=dev)
            for _ in range(3):
                model(tok, past_key_values=cache)
        torch.cuda.synchronize()
        print("kernel case decode_model_small: done")
        return
    if args.kernel_case == "moe_decode":
        # one Mixtral-shaped sparse block, 64 tokens: three forwards (launch lists)
        from signrot_b200.transformers import kernel_utils as ku
        dev = torch.device("cuda", 0)
        with torch.device(dev):
            model = ku.KernelDecoderModel(ku.DecoderConfig(num_hidden_layers=1, vocab_size=4096, num_local_experts=8))
        model = model.to(dev).random_init_(0)
        blk = model.layers[0].mlp
        x = torch.randn((64, 1, 4096), device=dev).half()
        with torch.no_grad():
            for _ in range(3):
                blk(x)
        torch.cuda.synchronize()
        print("kernel case moe_decode: done")
        return
    if args.kernel_case == "decode_model":
        run_decode_model("decode_model_llama3_8b", {}, 8, 2048, 128, torch.device("cuda", 0))
        return
    if args.kernel_case:
        run_kernel_case(args.kernel_case)
        return
    if args.sweep:
        run_sweep()
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    run_ours(args, rank, world, local_rank)
    if world > 1:
        # Nothing is in flight after the barrier and the synchronise.  The process ends here instead of tearing the
        # communicator down: with CUDA graphs that captured work of this process group still referenced, the
        # tear-down of this collective-library version can block forever.
        torch.distributed.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
