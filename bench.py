#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extra]

Headline workload (N=1): causal prefill forward, bf16 in/out, B=4 H=32 L=4096 D=128, scale
1/sqrt(128), inputs N(0,1)*0.5 from a seed. One "step" is one forward pass over that batch. With
N>1 every rank runs the same batch on its own GPU (the (batch*head) axis shards with no collective,
so this is weak scaling: per-GPU work is fixed) and `value` is the whole-job rate.

Printed JSON (one line, rank 0): metric/value/unit as TFLOP/s of algorithmic work
(4*B*H*L*L*D/2 flop per step), `roofline` for the forward kernel against the measured dense bf16
peak, `e2e` (host buffers in pinned memory -> copy_to_device -> kernel -> copy_from_device through
the C ABI, all inside the timed region), `cpu_baseline` (the reference's own C operators composed
into attention, timed on the host cores on a bounded sample) and, at N=1, `extra` with the backward
and split-KV decode results.

`--impl reference` times only the CPU reference arm and prints the same line shape.
torch is used for device selection, input generation, events and torch.distributed plumbing; the
attention itself runs in this repo's CUDA library through its C ABI (ctypes).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(name="causal_prefill_fwd_bf16_B4_H32_L4096_D128", B=4, H=32, L=4096, D=128)
BWD_WORKLOAD = dict(name="causal_fwd_bwd_bf16_B2_H32_L8192_D128", B=2, H=32, L=8192, D=128)
DECODE_WORKLOAD = dict(name="decode_bf16_B64_H32_Lk32768_D128", B=64, H=32, Lk=32768, D=128)
NOMINAL_BF16_TFLOPS = 2250.0
NOMINAL_HBM_GBS = 8000.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ------------------------------------------------------------------------------------------------
# CPU reference arm
# ------------------------------------------------------------------------------------------------
def cpu_reference_sample(rows: int, slices: int, threads: int):
    """Times the composed reference attention (causal, L=4096, D=128) for the first `rows` query rows
    of `slices` independent (batch, head) slices, `threads` slices at a time. Returns seconds and
    which implementation ran ("reference": the reference's compiled C operators; "port": the C
    restatement)."""
    from oracle import cpu_oracle, ref_ops

    L, D = WORKLOAD["L"], WORKLOAD["D"]
    rng = np.random.default_rng(1234)
    q = (rng.standard_normal((slices, rows, D), dtype=np.float32) * 0.5)
    k = (rng.standard_normal((slices, L, D), dtype=np.float32) * 0.5)
    v = (rng.standard_normal((slices, L, D), dtype=np.float32) * 0.5)
    scale = 1.0 / math.sqrt(D)
    if ref_ops.available():
        kind = "reference"
        # rows [0, rows) of the causal problem: key j visible to row i iff j <= i (top-left rows of
        # the square mask), expressed the only way the reference can: an additive {0,-inf} mask.
        i = np.arange(rows)[:, None]
        j = np.arange(L)[None, :]
        mask = np.where(j > i, -np.inf, 0.0).astype(np.float32)

        def one(s):
            p, _, _ = ref_ops._probs(q[s], k[s], scale, mask)
            ref_ops._mm(p, v[s])

        t0 = time.perf_counter()
        if threads <= 1:
            for s in range(slices):
                one(s)
        else:
            ths = []
            nxt = iter(range(slices))
            lock = threading.Lock()

            def work():
                while True:
                    with lock:
                        s = next(nxt, None)
                    if s is None:
                        return
                    one(s)

            for _ in range(threads):
                th = threading.Thread(target=work)
                th.start()
                ths.append(th)
            for th in ths:
                th.join()
        return time.perf_counter() - t0, kind
    kind = "port"
    cpu_oracle.set_threads(threads)
    # the port's causal mask is bottom-right aligned; pass the first `rows` keys' worth of offset by
    # running non-causal over all L keys, which costs the reference path the same (it multiplies the
    # full rectangle either way).
    t0 = time.perf_counter()
    cpu_oracle.attention_fwd(q, k, v, scale, False)
    dt = time.perf_counter() - t0
    cpu_oracle.set_threads(1)
    return dt, kind


def cpu_baseline_value(rows: int, threads: int, repeats: int = 1):
    """TFLOP/s (algorithmic causal flops of the headline workload / extrapolated time) of the CPU
    reference on `threads` host threads, from a bounded sample."""
    B, H, L, D = (WORKLOAD[x] for x in "BHLD")
    slices = threads
    best = None
    for _ in range(repeats):
        dt, kind = cpu_reference_sample(rows, slices, threads)
        best = dt if best is None else min(best, dt)
    # The reference multiplies the full (rows x L) rectangle whatever the mask, so its time is
    # proportional to rows*slices; the whole workload has B*H slices of L rows.
    full_seconds = best * (L / rows) * (B * H / slices)
    flops = 4.0 * B * H * L * L * D / 2.0
    return dict(value=flops / full_seconds / 1e12, unit="TFLOP/s", cores=threads, kind=kind,
                sample=f"first {rows} query rows of {slices} (batch,head) slices of the headline workload "
                       f"({best:.2f} s measured, extrapolated x{(L / rows) * (B * H / slices):.0f})"), full_seconds


def host_threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return os.cpu_count() or 1


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = min(host_threads(), 64)
    rows = 256
    times = []
    kind = "port"
    for step in range(args.warmup + args.steps):
        dt, kind = cpu_reference_sample(rows, threads, threads)
        if step >= args.warmup:
            times.append(dt)
    B, H, L, D = (WORKLOAD[x] for x in "BHLD")
    mean = sum(times) / len(times)
    factor = (L / rows) * (B * H / threads)
    full_seconds = mean * factor
    flops = 4.0 * B * H * L * L * D / 2.0
    value = flops / full_seconds / 1e12
    sample = (f"each step: first {rows} query rows of {threads} (batch,head) slices on {threads} host threads "
              f"({mean:.3f} s/step measured), extrapolated x{factor:.0f} to the full batch")
    line = {
        "metric": "attention_causal_prefill_fwd_tflops", "value": value, "unit": "TFLOP/s", "impl": "reference",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": full_seconds * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "note": "reference CPU path computes in float32 with double-accumulated matmuls"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Polls NVML for SM clock and clock-event reasons of one GPU while the benchmark runs."""

    def __init__(self, torch_index: int):
        self.samples = []  # (t, sm_mhz, reasons_bitmask, power_w)
        self.max_mhz = None
        self._stop = threading.Event()
        self._th = None
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            import torch

            uuid = str(torch.cuda.get_device_properties(torch_index).uuid)
            self.h = None
            for i in range(pynvml.nvmlDeviceGetCount()):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                u = pynvml.nvmlDeviceGetUUID(h)
                u = u.decode() if isinstance(u, bytes) else u
                if uuid in u or u.replace("GPU-", "") == uuid:
                    self.h = h
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(torch_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                try:
                    power = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                except Exception:
                    power = 0.0
                self.samples.append((time.perf_counter(), mhz, reasons, power))
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self.nv is not None:
            self._th = threading.Thread(target=self._loop, daemon=True)
            self._th.start()

    def stop(self):
        self._stop.set()
        if self._th:
            self._th.join(timeout=1.0)

    def summary(self, t0: float, t1: float):
        if self.nv is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "window": "unavailable"}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        window = "timed_region"
        if len(inside) < 2:
            inside = self.samples
            window = "whole_gpu_phase"
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        mask = 0
        for s in inside:
            mask |= s[2]
        reasons = [n for n, bit in names.items() if mask & bit]
        return {"sm_mhz": float(np.median([s[1] for s in inside])), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "power_w_max": max(s[3] for s in inside), "samples": len(inside), "window": window}


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from ember_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the attention path")
    torch.cuda.set_device(local_rank)
    # stdout carries exactly one JSON line: anything a library prints there while the benchmark runs
    # (NCCL's version banner, for one) goes to stderr instead
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = _lib.lib()
    _lib.check(L.ember_set_device(local_rank))
    dev = torch.device("cuda", local_rank)
    # A stream of our own: the handle of torch's default stream is 0, which the C ABI reads as "use
    # the library's stream", and then the events below would not see the kernels.
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    assert stream.cuda_stream != 0
    sptr = ctypes.c_void_p(stream.cuda_stream)
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    from ember_b200 import synth

    B, H, S, D = (WORKLOAD[x] for x in "BHLD")
    scale = 1.0 / math.sqrt(D)
    # Inputs are keyed by the GLOBAL element index: the job is world x (B*H) units, rank r holds units
    # [r*B*H, (r+1)*B*H), and a unit's values do not depend on the number of ranks.
    BH = B * H
    u0 = rank * BH
    q, k, v = (synth.units_torch(torch, seed, u0, u0 + BH, S, D, dev, 0.5, torch.bfloat16).view(B, H, S, D)
               for seed in (1001, 1002, 1003))
    out = torch.empty_like(q)
    lse = torch.empty((B, H, S), device=dev, dtype=torch.float32)
    flops_step = 4.0 * B * H * S * S * D / 2.0

    def fwd():
        _lib.check(L.ember_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                         B * H, S, S, D, scale, 1, _lib.EMBER_BF16, sptr))

    sampler = ClockSampler(local_rank)
    sampler.start()
    # Generating the inputs is a few hundred elementwise launches; let the GPU idle for a moment so
    # that the short headline region starts from the same power state as a freshly started process.
    torch.cuda.synchronize()
    time.sleep(2.0)
    for _ in range(max(args.warmup, 3)):
        fwd()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.perf_counter()
    e0.record(stream)
    for _ in range(args.steps):
        fwd()
    e1.record(stream)
    barrier()
    t_wall1 = time.perf_counter()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    value = world * flops_step / (ms_step * 1e-3) / 1e12
    where = ctypes.c_int(0)
    _lib.check(L.ember_check_device_status(sptr, ctypes.byref(where)))
    sustained = run_sustained(torch, fwd, stream, sampler, ms_step, flops_step, world, peaks, barrier, max_over_ranks)
    identity = check_identity(L, _lib, torch, dist, synth, dev, sptr, out, lse, rank, world, BH, S, D, scale)

    # ---- end to end through the C ABI with host buffers (pinned), copies inside the timed region:
    # ember_attention_fwd_host takes host tensors (the reference's own calling pattern), streams the
    # (batch*head) units through device staging buffers and returns when the host result is complete
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty_like(hq).pin_memory()
    nbytes = hq.numel() * 2

    def e2e_step():
        _lib.check(L.ember_attention_fwd_host(hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), ho.data_ptr(), None, B * H, S, S,
                                              D, scale, 1, _lib.EMBER_BF16))

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = max_over_ranks((time.perf_counter() - t0) / e2e_steps)
    e2e_value = world * flops_step / e2e_s / 1e12
    e2e_ok = bool(torch.equal(ho.to(dev), out))
    # the same bytes moved with no kernel at all (both directions at once, on two streams): what the
    # host memory system and the PCIe link give THIS rank while the other ranks do the same
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    dq_, dk_, dv_ = (torch.empty_like(q) for _ in range(3))

    def copies():
        with torch.cuda.stream(s_in):
            dq_.copy_(hq, non_blocking=True)
            dk_.copy_(hk, non_blocking=True)
            dv_.copy_(hv, non_blocking=True)
        with torch.cuda.stream(s_out):
            ho.copy_(out, non_blocking=True)
        s_in.synchronize()
        s_out.synchronize()

    copies()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        copies()
    barrier()
    copy_only_s = max_over_ranks((time.perf_counter() - t0) / e2e_steps)
    del dq_, dk_, dv_
    sampler.stop()
    clocks = sampler.summary(t_wall0, t_wall1)

    line = {
        "metric": "attention_causal_prefill_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "per_gpu": True, "causal": True, "scale": scale,
                   "inputs": "approx. N(0,1)*0.5 keyed by the global element index (rank r holds units "
                             "[r*128, (r+1)*128) of a world*128-unit job), resident in HBM",
                   "identity_1_vs_n": identity,
                   "l2": "inputs (403 MB per step) larger than L2 (126 MB); no flush",
                   "idle_before_warmup_s": 2.0,
                   "kernel": L.ember_attention_kernel_name(0, S, S, D, 1).decode()},
        "roofline": {"bound": "tensor", "achieved": flops_step / (ms_step * 1e-3) / 1e12, "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": flops_step / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"],
                     # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the B=2 H=32 case
                     # (252.1 MB), scaled by the (batch*head) units of this launch: traffic grows in
                     # proportion because every head is an independent problem.
                     "traffic": 252.1e6 * (B * H) / 64.0, "traffic_unit": "bytes/launch",
                     "algorithmic_bytes": 4 * B * H * S * D * 2 + B * H * S * 4, "peak_source": peaks["source"] + " burst cuBLAS bf16",
                     "frac_of_nominal_2250": flops_step / (ms_step * 1e-3) / 1e12 / NOMINAL_BF16_TFLOPS,
                     "frac_of_sustained": flops_step / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"]},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": 3 * nbytes, "d2h_bytes_per_step": nbytes,
                "ms_per_step": e2e_s * 1e3, "steps": e2e_steps, "result_matches_device_run": e2e_ok,
                "copy_only_ms_per_step": copy_only_s * 1e3, "copy_only_h2d_gbs_per_rank": 3 * nbytes / copy_only_s / 1e9,
                "bound": "host-to-device copies (the copy-only figure is the floor of a step)"},
        "gpu_launches": args.steps,
        "clocks": clocks,
        "sustained": sustained,
    }

    if world > 1:
        line["gather"] = run_gather(L, _lib, torch, dist, dev, sptr, stream, out, rank, world)
    sweep = None
    if not args.no_extra:
        sweep = run_c5_sweep(L, _lib, torch, dist, dev, sptr, stream, rank, world, sampler)
    if rank == 0 and world == 1:
        cb, _ = cpu_baseline_value(rows=1024, threads=min(host_threads(), 64), repeats=1)
        # the reference is single-threaded (src/tensor/operators_cpu.c:47-67 has no parallel loop), so
        # its own figure is the one-thread one; the all-threads figure above runs independent slices
        one, _ = cpu_baseline_value(rows=512, threads=1, repeats=1)
        cb["single_thread"] = {"value": one["value"], "unit": "TFLOP/s", "cores": 1, "sample": one["sample"]}
        line["cpu_baseline"] = cb
        if not args.no_extra:
            line["extra"] = run_extras(L, _lib, torch, dev, sptr, stream, peaks)
    if sweep is not None:
        line.setdefault("extra", {})["scaling_sweep_fwd_bwd_128_heads"] = {
            "scaling": "strong", "note": "causal fwd+bwd, bf16, D=128, 128 (batch*head) units split over the GPUs",
            **sweep}
        # a compact copy where every reader of the line finds it: whole-job TFLOP/s and ms per length
        line["config"]["c5_strong"] = {
            "what": "causal fwd+bwd bf16 H=64 D=128, 128 (batch*head) units split over n_gpus (strong scaling)",
            **{key: {"tflops": round(val["tflops_total"], 1), "ms": round(val["ms_fwd_bwd"], 4),
                     "sm_mhz_min": min(val["sm_mhz_per_rank"]), "sm_mhz_max": max(val["sm_mhz_per_rank"])}
               for key, val in sweep.items() if key.startswith("L")},
            "identity_1_vs_n": sweep.get("identity_1_vs_n")}
    if world > 1:
        dist.destroy_process_group()
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    os.close(real_stdout)
    if rank == 0:
        print(json.dumps(line), flush=True)


def run_gather(L, _lib, torch, dist, dev, sptr, stream, out, rank, world):
    """The optional result gather (not on the data path): every rank's output slab into one full
    tensor on every rank with ember_gather_outputs (ncclAllGather over NVLink), timed on its own."""
    from ember_b200.comm import Communicator

    store = dist.PrefixStore("ember_bench_gather", dist.distributed_c10d._get_default_store())
    comm = Communicator(rank, world, store, timeout_s=120.0)
    nbytes = out.numel() * out.element_size()
    full = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device=dev)
    for _ in range(2):
        comm.gather_into(full.data_ptr(), out.data_ptr(), nbytes, sptr)
    dist.barrier()
    torch.cuda.synchronize()
    reps = 5
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(reps):
        comm.gather_into(full.data_ptr(), out.data_ptr(), nbytes, sptr)
    b.record(stream)
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / reps], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    # every slab of the gathered tensor carries its owner's checksum
    mine = torch.tensor([unit_checksum(torch, out.view(-1, out.shape[-2], out.shape[-1])[0])], dtype=torch.int64, device=dev)
    owners = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(owners, mine)
    ok = all(unit_checksum(torch, full[r].view(-1, out.shape[-2], out.shape[-1])[0]) == int(owners[r].item()) for r in range(world))
    ok = ok and bool(torch.equal(full[rank], out))
    comm.close()
    return {"ms": ms, "bytes_per_rank": nbytes, "bytes_total": world * nbytes, "algbw_gbs": world * nbytes / ms / 1e6,
            "busbw_gbs": (world - 1) * nbytes / ms / 1e6, "nvlink_measured_peer_gbs": 770.0, "result_ok": ok,
            "call": "ember_gather_outputs (ncclAllGather of equal slabs), timed apart from the attention step"}


def unit_checksum(torch, t):
    """A position-weighted 64-bit checksum of a tensor's bits (wrapping integer arithmetic)."""
    bits = t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32).reshape(-1).to(torch.int64)
    w = torch.arange(1, bits.numel() + 1, dtype=torch.int64, device=t.device)
    return int((bits * w).sum().item())


def check_identity(L, _lib, torch, dist, synth, dev, sptr, out, lse, rank, world, BH, S, D, scale):
    """Outside any timed region: does the result of a unit depend on which rank computed it, or on
    the shape of the launch it was part of? Every rank regenerates the FIRST unit of its right-hand
    neighbour's slab from the global generator, runs it as a launch of one unit, and the checksum of
    that output is compared with the checksum the owner took from its full launch (only the
    checksums travel). With one rank the neighbour is the rank itself."""
    nb = (rank + 1) % world
    g = nb * BH
    q1, k1, v1 = (synth.units_torch(torch, seed, g, g + 1, S, D, dev, 0.5, torch.bfloat16) for seed in (1001, 1002, 1003))
    o1 = torch.empty_like(q1)
    l1 = torch.empty((1, S), device=dev, dtype=torch.float32)
    _lib.check(L.ember_attention_fwd(q1.data_ptr(), k1.data_ptr(), v1.data_ptr(), o1.data_ptr(), l1.data_ptr(), 1, S, S, D,
                                     scale, 1, _lib.EMBER_BF16, sptr))
    torch.cuda.synchronize()
    mine = torch.tensor([unit_checksum(torch, out.view(BH, S, D)[0]), unit_checksum(torch, lse.view(BH, S)[0])],
                        dtype=torch.int64, device=dev)
    theirs = torch.tensor([unit_checksum(torch, o1[0]), unit_checksum(torch, l1[0])], dtype=torch.int64, device=dev)
    if world > 1:
        owners = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(owners, mine)
        ok = bool(torch.equal(owners[nb], theirs))
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(flag.item())
    else:
        ok = bool(torch.equal(mine, theirs))
    if not ok:
        raise SystemExit("bench.py: a unit computed alone differs from the same unit inside its owner's launch")
    return {"checked": True, "ok": ok, "how": "first unit of the next rank's slab recomputed as a one-unit launch; "
                                              "output and log-sum-exp checksums equal the owner's, bit for bit"}


def run_sustained(torch, fwd, stream, sampler, ms_step, flops_step, world, peaks, barrier, max_over_ranks):
    """A second, seconds-long timed region of back-to-back launches of the headline workload: the SM
    clock sinks under the power limit after the first tens of milliseconds, so this is the rate a
    long job sees. Reported beside the short-burst headline with the clock sampled inside the region
    (time x clock = cycles per step separates kernel changes from clock changes)."""
    n = max(50, int(2000.0 / max(ms_step, 1e-3)))
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record(stream)
    for _ in range(n):
        fwd()
    b.record(stream)
    barrier()
    t1 = time.perf_counter()
    ms = max_over_ranks(a.elapsed_time(b)) / n
    clk = sampler.summary(t0 + 0.25 * (t1 - t0), t1)  # the settled part of the region
    val = world * flops_step / (ms * 1e-3) / 1e12
    mhz = clk.get("sm_mhz")
    return {"value": val, "unit": "TFLOP/s", "steps": n, "ms_per_step": ms, "seconds": (t1 - t0),
            "frac_of_sustained_peak": val / world / peaks["bf16_tflops_sustained"],
            "peak_sustained": peaks["bf16_tflops_sustained"], "sm_mhz_median": mhz, "reasons": clk.get("reasons"),
            "power_w_max": clk.get("power_w_max"),
            "mcycles_per_step": (ms * 1e-3 * mhz) if mhz else None}


def run_c5_sweep(L, _lib, torch, dist, dev, sptr, stream, rank, world, sampler):
    """The strong-scaling configuration: causal forward+backward, bf16, 128 (batch*head) units with D=128 split over
    the ranks (strong scaling: the total work is fixed), L in {2048, 8192, 16384}. Every rank owns
    the contiguous slab shard_range(128, rank, world) of tensors generated from the global element
    index; no collective on the data path. Returns, per L, the whole-job TFLOP/s from the slowest
    rank's device time and the SM clock each rank saw. At L=2048 (cheap) every rank also computes ALL
    128 units, the single-GPU job, and checks outside the timed region that its slab of that result
    equals what it computed as a shard: bit for bit for O, LSE, dK and dV, and for dQ too when the
    deterministic backward is selected (the default backward adds dQ contributions in no fixed
    order; there dQ is compared to rounding)."""
    from ember_b200 import synth
    from ember_b200.shard import shard_range

    out = {}
    D, units = 128, 128
    b, e = shard_range(units, rank, world)
    scale = 1.0 / math.sqrt(D)

    def make(u0, u1, S):
        q, k, v = (synth.units_torch(torch, seed, u0, u1, S, D, dev, 0.5, torch.bfloat16) for seed in (501, 502, 503))
        do = synth.units_torch(torch, 504, u0, u1, S, D, dev, 1.0, torch.bfloat16)
        return q, k, v, do

    def run(q, k, v, do, S):
        bh = q.shape[0]
        o, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
        lse = torch.empty((bh, S), device=dev, dtype=torch.float32)
        wsn = L.ember_attention_workspace_bytes(_lib.EMBER_OP_BWD, bh, S, S, D, 1, 0)
        ws = torch.empty(max(wsn, 256), device=dev, dtype=torch.uint8)

        def step():
            _lib.check(L.ember_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), bh,
                                             S, S, D, scale, 1, 1, sptr))
            _lib.check(L.ember_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                             do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), bh, S, S, D,
                                             scale, 1, 1, ws.data_ptr(), wsn, sptr))
        return step, (o, lse, dq, dk, dv)

    for S in (2048, 8192, 16384):
        q, k, v, do = make(b, e, S)
        step, res = run(q, k, v, do, S)
        steps = {2048: 100, 8192: 20}.get(S, 6)  # each timed loop long enough for a few clock samples
        for _ in range(3):
            step()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, c = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        a.record(stream)
        for _ in range(steps):
            step()
        c.record(stream)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        ms = a.elapsed_time(c) / steps
        mhz = sampler.summary(t0, t1).get("sm_mhz") or 0.0
        mhz_all = [mhz]
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            g = [torch.empty(1, dtype=torch.float64, device=dev) for _ in range(world)]
            dist.all_gather(g, torch.tensor([mhz], dtype=torch.float64, device=dev))
            mhz_all = [float(x.item()) for x in g]
        total_flops = 3.5 * 4.0 * units * S * S * D / 2.0
        out[f"L{S}"] = {"ms_fwd_bwd": ms, "tflops_total": total_flops / ms / 1e9, "bh_per_gpu": e - b,
                        "sm_mhz_per_rank": mhz_all}
        if S == 2048:
            fq, fk, fv, fdo = (q, k, v, do) if world == 1 else make(0, units, S)
            if world == 1:
                # one GPU: the same units as a launch of a different shape (the second half alone)
                fq, fk, fv, fdo = (t[units // 2:] for t in (q, k, v, do))
                lo, hi = units // 2, units
            else:
                lo, hi = 0, units
            fstep, fres = run(fq, fk, fv, fdo, S)
            fstep()
            torch.cuda.synchronize()
            det = bool(L.ember_get_deterministic())
            ok = True
            for name, mine, full in zip(("o", "lse", "dq", "dk", "dv"), res, fres):
                ref = full[max(b, lo) - lo:min(e, hi) - lo]
                got = mine[max(b, lo) - b:min(e, hi) - b]
                if name == "dq" and not det:
                    ok = ok and bool(((got.float() - ref.float()).abs().max() <= 1e-2 * ref.float().abs().max()).item())
                else:
                    ok = ok and bool(torch.equal(got, ref))
            if world > 1:
                flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                ok = bool(flag.item())
            if not ok:
                raise SystemExit("bench.py: a rank's slab differs from the same slab of the single-GPU job")
            out["identity_1_vs_n"] = {"checked": True, "ok": ok, "L": S, "dq": "bit for bit" if det else "to rounding",
                                      "o_lse_dk_dv": "bit for bit"}
            del fq, fk, fv, fdo, fres
        del q, k, v, do, res
    return out


def run_extras(L, _lib, torch, dev, sptr, stream, peaks):
    """Backward (causal fwd+bwd workload) and split-KV decode, each with its own roofline entry."""
    extra = {}

    def timed(fn, steps, warm=3):
        # every extra is a short burst timed on its own: idle first, so that it does not inherit the
        # power state (a clock near 1.6 GHz) of the kernel measured before it
        torch.cuda.synchronize()
        time.sleep(1.0)
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(steps):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    # ---- backward
    B, H, S, D = (BWD_WORKLOAD[x] for x in "BHLD")
    scale = 1.0 / math.sqrt(D)
    gen = torch.Generator(device=dev).manual_seed(7)
    q, k, v = ((torch.randn((B, H, S, D), generator=gen, device=dev) * 0.5).to(torch.bfloat16) for _ in range(3))
    do = torch.randn((B, H, S, D), generator=gen, device=dev).to(torch.bfloat16)
    o = torch.empty_like(q)
    lse = torch.empty((B, H, S), device=dev, dtype=torch.float32)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    wsn = L.ember_attention_workspace_bytes(_lib.EMBER_OP_BWD, B * H, S, S, D, 1, 0)
    ws = torch.empty(wsn, device=dev, dtype=torch.uint8)

    def fwd():
        _lib.check(L.ember_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B * H,
                                         S, S, D, scale, 1, 1, sptr))

    def bwd():
        _lib.check(L.ember_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                         do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B * H, S, S, D,
                                         scale, 1, 1, ws.data_ptr(), wsn, sptr))

    fwd_flops = 4.0 * B * H * S * S * D / 2.0
    kern = L.ember_attention_kernel_name(_lib.EMBER_OP_BWD, S, S, D, 1).decode()
    ms_f = timed(fwd, 10)
    ms_b = timed(bwd, 10 if kern == "sm100_tcgen05" else 2, warm=1)
    extra["fwd_L8192"] = {"workload": BWD_WORKLOAD["name"], "ms": ms_f, "tflops": fwd_flops / ms_f / 1e9,
                          "frac_of_measured_peak": fwd_flops / ms_f / 1e9 / peaks["bf16_tflops"]}
    extra["bwd_L8192"] = {"workload": BWD_WORKLOAD["name"], "kernel": kern, "ms": ms_b,
                          "tflops": 2.5 * fwd_flops / ms_b / 1e9,
                          "frac_of_measured_peak": 2.5 * fwd_flops / ms_b / 1e9 / peaks["bf16_tflops"]}
    del q, k, v, do, o, dq, dk, dv, ws

    # ---- decode
    B, H, Lk, D = (DECODE_WORKLOAD[x] for x in ("B", "H", "Lk", "D"))
    scale = 1.0 / math.sqrt(D)
    kc = torch.empty((B, H, Lk, D), device=dev, dtype=torch.bfloat16)
    vc = torch.empty((B, H, Lk, D), device=dev, dtype=torch.bfloat16)
    for t in (kc, vc):  # fill in slabs to bound temporary memory
        for b in range(B):
            t[b] = (torch.randn((H, Lk, D), generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    qd = (torch.randn((B, H, 1, D), generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    od = torch.empty_like(qd)
    ld = torch.empty((B, H), device=dev, dtype=torch.float32)
    splits = L.ember_attention_decode_splits(B * H, Lk, D, 1)
    wsn = L.ember_attention_workspace_bytes(_lib.EMBER_OP_DECODE, B * H, 1, Lk, D, 1, 0)
    ws = torch.empty(max(wsn, 256), device=dev, dtype=torch.uint8)

    def dec():
        _lib.check(L.ember_attention_decode(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), od.data_ptr(), ld.data_ptr(),
                                            B * H, Lk, D, scale, 1, 0, ws.data_ptr(), wsn, sptr))

    ms_d = timed(dec, 10)
    nbytes = 2.0 * B * H * Lk * D * 2
    extra["decode"] = {"workload": DECODE_WORKLOAD["name"], "splits": splits, "ms": ms_d, "gbs": nbytes / ms_d / 1e6,
                       "roofline": {"bound": "hbm", "achieved": nbytes / ms_d / 1e6, "peak": peaks["hbm_gbs"],
                                    "unit": "GB/s", "frac": nbytes / ms_d / 1e6 / peaks["hbm_gbs"],
                                    "frac_of_nominal_8000": nbytes / ms_d / 1e6 / NOMINAL_HBM_GBS,
                                    "peak_source": peaks["source"] + " copy"}}
    # ---- the same decode step with grouped-query heads over a cache with spare capacity: 32 query
    # heads share 8 K/V heads, so the step streams a quarter of the cache bytes (the K/V of the first
    # 8 heads of the tensors above, read as a (B, 8, 4*Lk, D) cache filled to Lk rows)
    Hkv, cap = 8, 4 * Lk
    qg = qd.view(B, H, D)
    og = torch.empty_like(qg)
    wsn_g = L.ember_attention_decode_cache_workspace_bytes(B, H, Hkv, Lk, D, 0)
    ws_g = torch.empty(max(wsn_g, 256), device=dev, dtype=torch.uint8)

    def dec_gqa():
        _lib.check(L.ember_attention_decode_cache(qg.data_ptr(), kc.data_ptr(), vc.data_ptr(), og.data_ptr(), ld.data_ptr(), B, H,
                                                  Hkv, Lk, cap, D, scale, 1, None, None, 0, 0, 0, ws_g.data_ptr(), wsn_g, sptr))

    ms_g = timed(dec_gqa, 10)
    nbytes_g = 2.0 * B * Hkv * Lk * D * 2
    extra["decode_gqa"] = {"workload": f"decode_gqa_bf16_B{B}_Hq{H}_Hkv{Hkv}_Lk{Lk}_D{D}", "ms": ms_g, "gbs": nbytes_g / ms_g / 1e6,
                           "speedup_vs_per_head_cache": ms_d / ms_g,
                           "roofline": {"bound": "hbm", "achieved": nbytes_g / ms_g / 1e6, "peak": peaks["hbm_gbs"],
                                        "unit": "GB/s", "frac": nbytes_g / ms_g / 1e6 / peaks["hbm_gbs"],
                                        "peak_source": peaks["source"] + " copy"}}
    del kc, vc, ws, ws_g

    # ---- the projections either side of attention at the headline shape (E = H * D = 4096):
    # fused q/k/v projection writing (3, B, H, L, D), output projection reading (B, H, L, D)
    B, H, S, D = (WORKLOAD[x] for x in "BHLD")
    E, m = H * D, B * S
    x = torch.randn((m, E), generator=gen, device=dev).to(torch.bfloat16)
    proj = {}
    for name, n, xh, yh in (("qkv_projection", 3 * E, 0, H), ("output_projection", E, H, 0)):
        w = (torch.randn((E, n), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
        bias = torch.randn((n,), generator=gen, device=dev).to(torch.bfloat16)
        dy = torch.randn((m, n), generator=gen, device=dev).to(torch.bfloat16)
        y, dx, dw, db = torch.empty_like(dy), torch.empty_like(x), torch.empty_like(w), torch.empty_like(bias)

        def lin_f():
            _lib.check(L.ember_linear_fwd(x.data_ptr(), w.data_ptr(), bias.data_ptr(), y.data_ptr(), m, n, E, 1, xh, yh,
                                          S, D, sptr))

        def lin_b():
            _lib.check(L.ember_linear_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                                          db.data_ptr(), m, n, E, 1, xh, yh, S, D, sptr))

        ms_lf, ms_lb = timed(lin_f, 20), timed(lin_b, 10)
        fl = 2.0 * m * n * E
        proj[name] = {"m": m, "n": n, "k": E, "kernel": L.ember_linear_kernel_name(0, m, n, E, 1, xh, yh, S, D).decode(),
                      "fwd_ms": ms_lf, "fwd_tflops": fl / ms_lf / 1e9,
                      "fwd_frac_of_measured_peak": fl / ms_lf / 1e9 / peaks["bf16_tflops"],
                      "bwd_ms": ms_lb, "bwd_tflops": 2 * fl / ms_lb / 1e9,
                      "bwd_frac_of_measured_peak": 2 * fl / ms_lb / 1e9 / peaks["bf16_tflops"]}
        del w, bias, dy, y, dx, dw, db
    extra["projections"] = proj
    del x

    # ---- fused softmax (rows of attention-score length) and softmax cross-entropy (a vocabulary-
    # sized classifier head): HBM-bound, algorithmic bytes = one read and one write per element
    # (cross-entropy: logits and targets read, probabilities written)
    rows, cols = 65536, 4096
    xs = (torch.randn((rows, cols), generator=gen, device=dev) * 3).to(torch.bfloat16)
    ys = torch.empty_like(xs)

    def sm():
        _lib.check(L.ember_softmax_fwd(xs.data_ptr(), ys.data_ptr(), rows, cols, 1, 0, sptr))

    ms_s = timed(sm, 20)
    nb = 2.0 * rows * cols * 2
    extra["softmax"] = {"workload": f"softmax_bf16_rows{rows}_cols{cols}", "ms": ms_s, "gbs": nb / ms_s / 1e6,
                        "roofline": {"bound": "hbm", "achieved": nb / ms_s / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                     "frac": nb / ms_s / 1e6 / peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy"}}
    del xs, ys
    rows, cols = 8192, 32768
    pred = (torch.randn((rows, cols), generator=gen, device=dev) * 3).to(torch.bfloat16)
    tgt = torch.zeros((rows, cols), device=dev, dtype=torch.bfloat16)
    tgt[torch.arange(rows, device=dev), torch.randint(0, cols, (rows,), generator=gen, device=dev)] = 1
    probs, grad = torch.empty_like(pred), torch.empty_like(pred)
    loss = torch.zeros(1, device=dev, dtype=torch.float32)
    wn = L.ember_cross_entropy_workspace_bytes(rows)
    wsc = torch.empty(wn, device=dev, dtype=torch.uint8)

    def ce_f():
        _lib.check(L.ember_cross_entropy_fwd(pred.data_ptr(), tgt.data_ptr(), probs.data_ptr(), loss.data_ptr(), rows, cols,
                                             1, wsc.data_ptr(), wn, sptr))

    def ce_b():
        _lib.check(L.ember_cross_entropy_bwd(probs.data_ptr(), tgt.data_ptr(), grad.data_ptr(), rows, cols, 1, sptr))

    ms_cf, ms_cb = timed(ce_f, 10), timed(ce_b, 10)
    nb = 3.0 * rows * cols * 2
    extra["cross_entropy"] = {"workload": f"cross_entropy_bf16_rows{rows}_cols{cols}", "fwd_ms": ms_cf,
                              "fwd_gbs": nb / ms_cf / 1e6, "fwd_frac_of_measured_copy": nb / ms_cf / 1e6 / peaks["hbm_gbs"],
                              "bwd_ms": ms_cb, "bwd_gbs": nb / ms_cb / 1e6,
                              "bwd_frac_of_measured_copy": nb / ms_cb / 1e6 / peaks["hbm_gbs"], "loss": float(loss[0])}
    return extra


def run_profile_case(args):
    """A small single-kernel case for ncu captures (never a benchmark value): inputs larger than L2,
    a few hundred MB to a few GB on the device, `steps` launches after `warmup`."""
    import torch

    from ember_b200 import _lib

    torch.cuda.set_device(0)
    L = _lib.lib()
    _lib.check(L.ember_set_device(0))
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    sptr = ctypes.c_void_p(stream.cuda_stream)
    gen = torch.Generator(device=dev).manual_seed(3)
    D = 128
    scale = 1.0 / math.sqrt(D)
    if args.profile in ("fwd", "bwd"):
        B, H, S = 2, 32, 4096
        q, k, v, do = ((torch.randn((B, H, S, D), generator=gen, device=dev) * 0.5).to(torch.bfloat16) for _ in range(4))
        o, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
        lse = torch.empty((B, H, S), device=dev, dtype=torch.float32)
        wsn = L.ember_attention_workspace_bytes(_lib.EMBER_OP_BWD, B * H, S, S, D, 1, 0)
        ws = torch.empty(wsn, device=dev, dtype=torch.uint8)

        def fwd():
            _lib.check(L.ember_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                             B * H, S, S, D, scale, 1, 1, sptr))

        def bwd():
            _lib.check(L.ember_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                             do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B * H, S, S,
                                             D, scale, 1, 1, ws.data_ptr(), wsn, sptr))

        fwd()
        fn = fwd if args.profile == "fwd" else bwd
        work = 4.0 * B * H * S * S * D / 2.0 * (1.0 if args.profile == "fwd" else 2.5)
        unit, name = "TFLOP/s", f"causal_{args.profile}_bf16_B{B}_H{H}_L{S}_D{D}"
    elif args.profile == "decode_gqa":
        B, Hq, Hkv, Lk = 16, 32, 8, 32768  # 2.1 GB of cache, read once per step
        kc = (torch.randn((B, Hkv, Lk, D), generator=gen, device=dev) * 0.5).to(torch.bfloat16)
        vc = (torch.randn((B, Hkv, Lk, D), generator=gen, device=dev) * 0.5).to(torch.bfloat16)
        qd = (torch.randn((B, Hq, D), generator=gen, device=dev) * 0.5).to(torch.bfloat16)
        od = torch.empty_like(qd)
        ld = torch.empty((B, Hq), device=dev, dtype=torch.float32)
        wsn = L.ember_attention_decode_cache_workspace_bytes(B, Hq, Hkv, Lk, D, 0)
        ws = torch.empty(max(wsn, 256), device=dev, dtype=torch.uint8)

        def fn():
            _lib.check(L.ember_attention_decode_cache(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), od.data_ptr(),
                                                      ld.data_ptr(), B, Hq, Hkv, Lk, Lk, D, scale, 1, None, None, 0, 0, 0,
                                                      ws.data_ptr(), wsn, sptr))

        work = 2.0 * B * Hkv * Lk * D * 2
        unit, name = "GB/s", f"decode_gqa_bf16_B{B}_Hq{Hq}_Hkv{Hkv}_Lk{Lk}_D{D}"
    elif args.profile == "softmax":
        rows, cols = 32768, 4096  # 268 MB in, 268 MB out
        xs = (torch.randn((rows, cols), generator=gen, device=dev) * 3).to(torch.bfloat16)
        ys = torch.empty_like(xs)

        def fn():
            _lib.check(L.ember_softmax_fwd(xs.data_ptr(), ys.data_ptr(), rows, cols, 1, 0, sptr))

        work = 2.0 * rows * cols * 2
        unit, name = "GB/s", f"softmax_bf16_rows{rows}_cols{cols}"
    elif args.profile == "linear":
        m, n, k, heads = 8192, 6144, 2048, 16  # a q/k/v projection: x (8192, 2048) -> (3, 2, 16, 4096, 128)
        x = torch.randn((m, k), generator=gen, device=dev).to(torch.bfloat16)
        w = (torch.randn((k, n), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
        bias = torch.randn((n,), generator=gen, device=dev).to(torch.bfloat16)
        y = torch.empty((m, n), device=dev, dtype=torch.bfloat16)

        def fn():
            _lib.check(L.ember_linear_fwd(x.data_ptr(), w.data_ptr(), bias.data_ptr(), y.data_ptr(), m, n, k, 1, 0, heads,
                                          4096, D, sptr))

        work = 2.0 * m * n * k
        unit, name = "TFLOP/s", f"qkv_projection_bf16_m{m}_n{n}_k{k}"
    else:
        B, H, Lk = 8, 32, 32768
        kc = (torch.randn((B, H, Lk, D), generator=gen, device=dev) * 0.5).to(torch.bfloat16)
        vc = (torch.randn((B, H, Lk, D), generator=gen, device=dev) * 0.5).to(torch.bfloat16)
        qd = (torch.randn((B, H, 1, D), generator=gen, device=dev) * 0.5).to(torch.bfloat16)
        od = torch.empty_like(qd)
        ld = torch.empty((B, H), device=dev, dtype=torch.float32)
        wsn = L.ember_attention_workspace_bytes(_lib.EMBER_OP_DECODE, B * H, 1, Lk, D, 1, 0)
        ws = torch.empty(max(wsn, 256), device=dev, dtype=torch.uint8)

        def fn():
            _lib.check(L.ember_attention_decode(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), od.data_ptr(),
                                                ld.data_ptr(), B * H, Lk, D, scale, 1, 0, ws.data_ptr(), wsn, sptr))

        work = 2.0 * B * H * Lk * D * 2
        unit, name = "GB/s", f"decode_bf16_B{B}_H{H}_Lk{Lk}_D{D}"
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(args.steps):
        fn()
    b.record(stream)
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    rate = work / ms / (1e9 if unit == "TFLOP/s" else 1e6)
    print(json.dumps({"profile_case": name, "ms_per_launch": ms, "rate": rate, "unit": unit,
                      "note": "small case for profiler captures; not a benchmark value"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the backward and decode extras at N=1")
    ap.add_argument("--profile", choices=["fwd", "bwd", "decode", "decode_gqa", "linear", "softmax"], default=None,
                    help="run only a small single-kernel case (for ncu captures) and exit")
    args = ap.parse_args()
    if args.profile:
        if args.steps == 100 and args.warmup == 5:
            args.steps, args.warmup = 3, 2
        run_profile_case(args)
        return
    if args.impl == "reference":
        if args.steps == 100 and args.warmup == 5:  # defaults are sized for the GPU arm
            args.steps, args.warmup = 5, 1
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
