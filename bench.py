#!/usr/bin/env python
"""Benchmark of the QloraLinear hot path (benchmark configuration 2): one step = forward + backward of a
4096x4096 NF4 (block 64, double-quantised) QloraLinear with a rank-16 LoRA adapter over 8192 token
rows, bf16 activations, synthetic seeded data.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

For N > 1 launch with torchrun (one rank per GPU): token rows are sharded (every rank owns 8192
rows: weak scaling), W_q / A / B are replicated and only the LoRA gradients are all-reduced (NCCL).
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

OUT_DIM = IN_DIM = 4096
TOKENS = 8192
RANK_R, ALPHA = 16, 32.0
WORKLOAD = "QloraLinear fwd+bwd 4096x4096 (out x in), 8192 token rows/GPU, LoRA r=16 alpha=32, NF4 block 64 + double quant"
METRIC, UNIT = "qlora_linear_fwd_bwd_tokens_per_s", "tokens/s"
# DRAM bytes (read + write) of one weight-GEMM launch at this workload: dram__bytes_read.sum + dram__bytes_write.sum
# of an ncu capture of the same two kernels at this size (forward 130.8 MB, backward 113.0 MB; their average).
# A constant from that capture, not measured in the run.
GEMM_DRAM_TRAFFIC_PER_LAUNCH = 121.9e6
# SMs left to the NCCL kernels of the gradient exchange at N > 1 (NCCL_MAX_CTAS=2: two CTAs, possibly on two TPCs)
RESERVED_SMS = int(os.environ.get("QLC_BENCH_RESERVED_SMS", "4"))
# end-to-end leg: submissions kept in flight (each on its own set of pinned host buffers)
E2E_DEPTH = max(2, int(os.environ.get("QLC_BENCH_E2E_DEPTH", "2")))


def base_config(world):
    """The `config` object of a line: the same keys and values in the GPU arm and in the CPU reference arm."""
    return {"workload": WORKLOAD, "tokens_per_gpu": TOKENS, "global_tokens": world * TOKENS,
            "l2": "inputs+outputs per step (256 MiB) exceed the 126 MB L2; no explicit flush"}


def flops_fwd_bwd(m, n, k, r=0):
    """4·M·N·K + 2·M·r·(4K + 3N): forward 2MNK + 2Mr(K+N); backward 2MNK + 2Mr(3K+2N), counting
    the T1 recompute as qlora-core/src/qlora.rs:145 does."""
    return 4.0 * m * n * k + 2.0 * m * r * (4 * k + 3 * n)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tflops_burst=d["bf16_tflops"], tflops_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs (NVML every ~2 ms in a
    thread; falls back to `nvidia-smi -lms` when the NVML bindings are unavailable)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.samples, self.proc, self.stop_flag, self.thread = gpu_index, [], None, False, None
        self.max_mhz = None

    def start(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.gpu_index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if self.gpu_index < len(ids) and ids[self.gpu_index].isdigit():
                    idx = int(ids[self.gpu_index])
            h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                     "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                     "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                     "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons

            def loop():
                while not self.stop_flag:
                    try:
                        mhz = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                        bits = int(get_reasons(h))
                        self.samples.append((time.perf_counter(), mhz, {n for n, b in names.items() if bits & b}))
                    except Exception:
                        pass
                    time.sleep(0.002)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self._start_smi()

    def _start_smi(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)

            def pump():
                for line in self.proc.stdout:
                    f = [x.strip() for x in line.split(",")]
                    try:
                        self.max_mhz = float(f[2])
                        rs = {n for n, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9])
                              if v.lower().startswith("active")}
                        self.samples.append((time.perf_counter(), float(f[1]), rs))
                    except (ValueError, IndexError):
                        continue

            threading.Thread(target=pump, daemon=True).start()
        except Exception:
            self.proc = None

    def stop(self, t0, t1):
        time.sleep(0.02)
        self.stop_flag = True
        if self.proc:
            self.proc.terminate()
        inside = [(m, r) for t, m, r in self.samples if t0 <= t <= t1]
        if not inside:
            inside = [(m, r) for t, m, r in self.samples if t0 - 0.1 <= t <= t1 + 0.1]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples in the timed region"]}
        reasons = set()
        for _, r in inside:
            reasons |= r
        return {"sm_mhz": statistics.median(m for m, _ in inside), "sm_min_mhz": min(m for m, _ in inside),
                "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons), "samples": len(inside)}


# ---------------------------------------------------------------------------------------------
def cpu_reference_sample(seconds_target=12.0, max_rows=TOKENS):
    """Times the CPU restatement of qlora-core (oracle/qlora_oracle.c) on a bounded row sample of the
    workload: forward + backward for `rows` of the 8192 token rows, including the two dequantise()
    passes the reference performs per call.  Cost is exactly linear in the number of rows."""
    import numpy as np

    from oracle import c_oracle as orc

    orc.build()
    # every core this process may run on: under torchrun OMP_NUM_THREADS is preset to 1, which would leave the CPU
    # arm on one core; the oracle's loops take the thread count explicitly
    threads = max(orc.max_threads(), len(os.sched_getaffinity(0)))
    g = np.random.Generator(np.random.Philox(1))
    w = (g.standard_normal(OUT_DIM * IN_DIM) * 0.02).astype(np.float32)
    a = (np.random.Generator(np.random.Philox(2)).standard_normal(RANK_R * IN_DIM) / 64.0).astype(np.float32)
    b = (np.random.Generator(np.random.Philox(3)).standard_normal(OUT_DIM * RANK_R) * 0.01).astype(np.float32)
    q = orc.quantize_nf4(w, OUT_DIM, IN_DIM)

    def run(rows):
        x = np.random.Generator(np.random.Philox(4)).standard_normal(rows * IN_DIM).astype(np.float32)
        dy = np.random.Generator(np.random.Philox(5)).standard_normal(rows * OUT_DIM).astype(np.float32)
        t0 = time.perf_counter()
        wd = q.dequantize()  # qlora.rs:97
        orc.qlora_forward(x, rows, wd, OUT_DIM, IN_DIM, a, b, RANK_R, ALPHA, threads)
        wd = q.dequantize()  # qlora.rs:133
        orc.qlora_backward(x, dy, rows, wd, OUT_DIM, IN_DIM, a, b, RANK_R, ALPHA, threads)
        return time.perf_counter() - t0

    t1 = run(threads)  # one row per thread
    t4 = run(4 * threads)
    per_row = max((t4 - t1) / (3 * threads), 1e-6)
    fixed = max(t1 - per_row * threads, 0.0)  # the two dequantize passes do not depend on the row count
    rows = int(min(max_rows, max(threads, (seconds_target - fixed) / per_row)))
    rows = max(threads, rows // threads * threads)
    return run, rows, threads, fixed


def reference_arm(args, rank):
    if rank != 0:
        return
    run, rows, threads, _ = cpu_reference_sample(seconds_target=4.0)
    for _ in range(args.warmup):
        run(rows)
    times = [run(rows) for _ in range(args.steps)]
    t = sum(times) / len(times)
    val = rows / t
    sample = f"{rows} of {TOKENS} token rows per step (cost is linear in rows), fwd+bwd incl. 2 dequantize passes"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3 * TOKENS / rows, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": base_config(args.gpus),
        "reference": "C restatement of qlora-core (the Rust reference cannot be built here: no Rust toolchain); "
                     "ms_per_step is extrapolated linearly from the row sample to 8192 rows",
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
class Dist:
    """The process group of the run (NCCL through torch.distributed: barriers, the max over ranks, the broadcast of a
    communicator id) and the factory of the library's own communicators (qlc_comm_*), which carry the data path."""

    def __init__(self, rank, local_rank, world):
        import torch

        self.rank, self.local_rank, self.world = rank, local_rank, world
        self.dev = torch.device("cuda", local_rank)
        if world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        import torch

        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(self, x):
        import torch

        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def lib_comm(self, v, ctx):
        """A communicator of the library (NCCL loaded by libqlora_cuda itself) on `ctx`; rank 0's id travels through
        the process group."""
        import torch
        import torch.distributed as dist

        uid = torch.zeros(v.COMM_ID_BYTES, dtype=torch.uint8, device=self.dev)
        if self.rank == 0:
            uid = torch.frombuffer(bytearray(v.Comm.unique_id()), dtype=torch.uint8).to(self.dev)
        dist.broadcast(uid, 0)
        return v.Comm(ctx, self.world, self.rank, bytes(uid.cpu().numpy().tobytes()))

    def close(self):
        if self.world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


def timed_steps(dist_, ctx, ext, step, steps, warmup, finish=None, sample_clocks=True):
    """`warmup` untimed steps, then `steps` timed ones bracketed by a barrier + synchronize on both sides; CUDA
    events on the context's stream, maximum over ranks.  Returns (ms per step, clocks, launches)."""
    import torch

    for _ in range(warmup):
        step()
    if finish:
        finish()
    ctx.synchronize()
    dist_.barrier()
    sampler = ClockSampler(dist_.local_rank)
    if dist_.rank == 0 and sample_clocks:
        sampler.start()
        time.sleep(0.15)
    launches0 = ctx.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx.synchronize()
    dist_.barrier()
    t0 = time.perf_counter()
    e0.record(ext)
    for _ in range(steps):
        step()
    if finish:
        finish()
    e1.record(ext)
    ctx.synchronize()
    dist_.barrier()
    t1 = time.perf_counter()
    clocks = sampler.stop(t0, t1) if (dist_.rank == 0 and sample_clocks) else None
    ms = dist_.max_over_ranks(e0.elapsed_time(e1)) / steps
    return ms, clocks, int(ctx.launch_count - launches0)


def frac_of(value, peaks, key):
    return {"frac": value / peaks[key], "peak": peaks[key], "peak_source": f"{key}, {peaks['source']}"}


# ---------------------------------------------------------------------------------------------
def link_ceiling(dist_, nbytes_in, nbytes_out):
    """What this rank's host link carries when every rank copies at the same time: pinned host memory, one H2D and
    one D2H stream, `nbytes_in` in and `nbytes_out` out together (the byte counts of one end-to-end step).
    Returns GB/s per direction (the slowest rank's) while both directions are busy."""
    import torch

    dev = dist_.dev
    h_in = torch.empty(nbytes_in, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(nbytes_out, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(nbytes_in, dtype=torch.uint8, device=dev)
    d_out = torch.empty(nbytes_out, dtype=torch.uint8, device=dev)
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def both():
        with torch.cuda.stream(s_in):
            d_in.copy_(h_in, non_blocking=True)
        with torch.cuda.stream(s_out):
            h_out.copy_(d_out, non_blocking=True)

    for _ in range(2):
        both()
    dist_.barrier()
    t0 = time.perf_counter()
    n = 4
    for _ in range(n):
        both()
    dist_.barrier()
    dt = dist_.max_over_ranks(time.perf_counter() - t0) / n
    return {"seconds_per_step_of_copies": dt, "h2d_gbs_per_rank": nbytes_in / dt / 1e9, "d2h_gbs_per_rank": nbytes_out / dt / 1e9}


def ours_arm(args, dist_):
    import numpy as np
    import torch

    import vkqlora.rs_b200 as v

    rank, local_rank, world, dev = dist_.rank, dist_.local_rank, dist_.world, dist_.dev
    tf32 = args.precision == "tf32"
    ctx = v.GpuContext(local_rank)
    ctx.set_precision(v.PRECISION_TF32 if tf32 else v.PRECISION_BF16)
    ext = torch.cuda.ExternalStream(ctx.stream, device=dev)
    act_dtype, act_code = (torch.float32, v.DTYPE_F32) if tf32 else (torch.bfloat16, v.DTYPE_BF16)
    # the exchange step runs through the library's own communicator, on a context (stream) of its own
    cctx = lib_comm = cext = None
    if world > 1:
        cctx = v.GpuContext(local_rank)
        lib_comm = dist_.lib_comm(v, cctx)
        cext = torch.cuda.ExternalStream(cctx.stream, device=dev)
        # the exchange's collective overlaps the next GEMM: that GEMM's single wave of CTA pairs leaves it its SMs
        ctx.set_reserved_sms(RESERVED_SMS)

    # synthetic, seeded; W ~ N(0, 0.02), A ~ N(0, 1/64), B ~ N(0, 0.01), X, dY ~ N(0, 1) in bf16 (fp32 in TF32 mode)
    gen = torch.Generator(device=dev).manual_seed(1)
    w = torch.randn(OUT_DIM * IN_DIM, generator=gen, device=dev, dtype=torch.float32) * 0.02
    a = (torch.randn(RANK_R * IN_DIM, generator=gen, device=dev) / 64.0).cpu().numpy()
    b = (torch.randn(OUT_DIM * RANK_R, generator=gen, device=dev) * 0.01).cpu().numpy()
    torch.cuda.synchronize()
    q = v.QuantizedTensor.quantize_dev(w.data_ptr(), OUT_DIM, IN_DIM, v.QuantConfig(), ctx)
    ctx.synchronize()
    del w
    layer = v.QloraLinear.from_quantized(q, v.LoraAdapter(a, b, IN_DIM, OUT_DIM, RANK_R, ALPHA), ctx)
    gen.manual_seed(100 + rank)
    x = torch.randn(TOKENS, IN_DIM, generator=gen, device=dev).to(act_dtype)
    dy = torch.randn(TOKENS, OUT_DIM, generator=gen, device=dev).to(act_dtype)
    y = torch.empty(TOKENS, OUT_DIM, device=dev, dtype=act_dtype)
    dx = torch.empty(TOKENS, IN_DIM, device=dev, dtype=act_dtype)
    n_bucket = RANK_R * IN_DIM + OUT_DIM * RANK_R
    # Two gradient buckets used in turn: the exchange of step i reads one while the backward pass of step i + 1
    # writes the other, so no backward pass ever waits for an exchange (an optimiser would, one step later).
    buckets = [torch.zeros(n_bucket, device=dev, dtype=torch.float32) for _ in range(2)]
    torch.cuda.synchronize()

    done = torch.cuda.Event()
    joined = [torch.cuda.Event(), torch.cuda.Event()]
    in_flight = [False, False]
    count = [0]

    def step():
        # The exchange step (sum of the LoRA gradients over ranks: qlc_comm_allreduce_sum_f32, NCCL inside the
        # library) runs on the communicator context's stream and overlaps the following forward and backward
        # passes, as it would overlap the next layer's backward pass in a model; a backward pass waits for the
        # exchange that last read ITS bucket (two steps back) before it overwrites it.
        k = count[0] & 1
        count[0] += 1
        bk = buckets[k]
        layer.forward_dev(x.data_ptr(), TOKENS, y.data_ptr(), act_code)
        if in_flight[k]:
            ext.wait_event(joined[k])
        layer.backward_dev(x.data_ptr(), dy.data_ptr(), TOKENS, dx.data_ptr(), bk.data_ptr(),
                           bk.data_ptr() + 4 * RANK_R * IN_DIM, act_code)
        if world > 1:
            done.record(ext)
            cext.wait_event(done)
            lib_comm.allreduce_sum_f32(bk.data_ptr(), n_bucket)
            joined[k].record(cext)
            in_flight[k] = True

    def drain():  # the last exchanges belong to the timed region
        for k in range(2):
            if in_flight[k]:
                ext.wait_event(joined[k])

    ms_step, clocks, launches = timed_steps(dist_, ctx, ext, step, args.steps, args.warmup, finish=drain)
    value = world * TOKENS / (ms_step * 1e-3)

    # ---- per-kernel timing of the dominant kernel (the two weight GEMMs), live, with CUDA events on
    # the launching stream, over a second run of the same K steps
    ctx.profile_enable(True)
    for _ in range(args.steps):
        step()
    drain()
    ctx.synchronize()
    prof = [ctx.profile_read(s) for s in range(4)]
    ctx.profile_enable(False)
    peaks = measured_peaks()
    gemm_ms = prof[0][0] + prof[1][0]
    gemm_launches = prof[0][1] + prof[1][1]
    # algorithmic flops of one weight-GEMM launch: 2·M·N·K plus the rank-r update folded into it
    fl_launch = 2.0 * TOKENS * OUT_DIM * IN_DIM + 2.0 * TOKENS * RANK_R * OUT_DIM
    achieved = (fl_launch * gemm_launches / (gemm_ms * 1e-3) / 1e12) if gemm_ms > 0 else 0.0
    # the timed region is tens of milliseconds: the burst figure is the denominator; the sustained one beside it
    roofline = {
        "bound": "tensor", "kernel": "umma_gemm3_kernel (persistent paired-CTA tcgen05 weight GEMMs: forward Y and backward dX)",
        "achieved": achieved, "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
        "frac": achieved / peaks["tflops_burst"], "peak_source": f"bf16_tflops (burst), {peaks['source']}",
        "frac_sustained": achieved / peaks["tflops_sustained"], "peak_sustained": peaks["tflops_sustained"],
        "traffic": GEMM_DRAM_TRAFFIC_PER_LAUNCH,
        "traffic_unit": "bytes/launch (dram read+write of an ncu capture at this size; a constant, not measured in this run)",
        "algorithmic_bytes_per_launch": 2.0 * TOKENS * IN_DIM + 2.0 * TOKENS * OUT_DIM + 8654848.0,
        "avg_launch_ms": gemm_ms / max(gemm_launches, 1),
        "per_slot_ms_per_step": {name: prof[i][0] / args.steps for i, name in
                                 enumerate(("fwd_gemm", "bwd_dx_gemm", "lora_down", "token_grads_overlapping_bwd_dx_gemm"))},
    }
    tflops_step = flops_fwd_bwd(TOKENS, OUT_DIM, IN_DIM, RANK_R) / (ms_step * 1e-3) / 1e12

    # ---- end to end through the host-buffer C-ABI call (pinned host memory, copies inside the timed region)
    e2e = None
    if not args.no_e2e and not tf32:
        from vkqlora.rs_b200 import _lib

        # Two sets of pinned host buffers, two steps in flight: while step i's last results go out, step i + 1's
        # inputs already come in.  Every step still copies its own X and dY in and its own Y, dX and gradients out.
        def host_set():
            hs = dict(x=torch.empty(TOKENS * IN_DIM, dtype=torch.bfloat16).pin_memory(),
                      dy=torch.empty(TOKENS * OUT_DIM, dtype=torch.bfloat16).pin_memory(),
                      y=torch.empty(TOKENS * OUT_DIM, dtype=torch.bfloat16).pin_memory(),
                      gx=torch.empty(TOKENS * IN_DIM, dtype=torch.bfloat16).pin_memory(),
                      g=torch.empty(n_bucket, dtype=torch.float32).pin_memory())
            hs["x"].copy_(x.reshape(-1).cpu())
            hs["dy"].copy_(dy.reshape(-1).cpu())
            return hs

        depth = E2E_DEPTH
        sets = [host_set() for _ in range(depth)]
        bucket_ptr, _n = layer.grad_bucket()
        tickets = [None] * depth
        reduced = torch.cuda.Event()
        stepped = torch.cuda.Event()
        g_done = [torch.cuda.Event() for _ in range(depth)]
        e2e_count = [0]

        def e2e_wait(k):
            if tickets[k] is not None:
                ctx.wait(tickets[k])
                if world > 1:
                    g_done[k].synchronize()  # the summed gradients of that step have reached the host
                tickets[k] = None

        def e2e_step():
            k = e2e_count[0] % depth
            e2e_count[0] += 1
            e2e_wait(k)  # this buffer set's previous step has delivered: its results would be consumed here
            hs = sets[k]
            if world == 1:
                # X, dY in; Y, dX, grad_A, grad_B out: one call (X crosses the link once)
                tickets[k] = layer.forward_backward_host_async(
                    hs["x"].data_ptr(), hs["dy"].data_ptr(), TOKENS, v.DTYPE_BF16, hs["y"].data_ptr(), hs["gx"].data_ptr(),
                    hs["g"].data_ptr(), hs["g"].data_ptr() + 4 * RANK_R * IN_DIM)
            else:
                # the gradients stay in the layer's device bucket, are summed over the ranks by the library's
                # communicator (its own stream) and come to the host once, summed; the next step's compute must not
                # overwrite the bucket before that sum has read it
                if e2e_count[0] > 1:
                    ext.wait_event(reduced)
                tickets[k] = layer.forward_backward_host_async(
                    hs["x"].data_ptr(), hs["dy"].data_ptr(), TOKENS, v.DTYPE_BF16, hs["y"].data_ptr(), hs["gx"].data_ptr(),
                    None, None)
                stepped.record(ext)
                cext.wait_event(stepped)
                lib_comm.allreduce_sum_f32(bucket_ptr, n_bucket)
                cctx.copy_to_host(hs["g"].data_ptr(), bucket_ptr, 4 * n_bucket)
                reduced.record(cext)
                g_done[k].record(cext)

        def e2e_drain():
            for k in range(depth):
                e2e_wait(k)
            ctx.synchronize()
            if world > 1:
                cctx.synchronize()

        n_e2e = max(4, min(args.steps, 10))
        for _ in range(4):
            e2e_step()
        e2e_drain()
        dist_.barrier()
        te = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        e2e_drain()
        dist_.barrier()
        dt = dist_.max_over_ranks(time.perf_counter() - te)
        h2d = 2 * TOKENS * IN_DIM + 2 * TOKENS * OUT_DIM  # X once + dY, bf16
        d2h = 2 * TOKENS * OUT_DIM + 2 * TOKENS * IN_DIM + 4 * n_bucket
        e2e = {"value": world * TOKENS * n_e2e / dt, "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": n_e2e, "ms_per_step": dt / n_e2e * 1e3,
               "api": "qlc_qlora_forward_backward_host_async + qlc_ctx_wait (bf16 pinned host buffers; X, dY in, Y, dX, "
                      "grad_A, grad_B out; two steps in flight, each on its own buffer set)"
                      + ("" if world == 1 else " + qlc_comm_allreduce_sum_f32 on the layer's device bucket, summed gradients to the host")}
        del sets
        # the ceiling the host link sets: the same bytes as plain pinned copies, all ranks at once
        try:
            link = link_ceiling(dist_, h2d, d2h)
            link["e2e_ceiling_tokens_per_s"] = world * TOKENS / link["seconds_per_step_of_copies"]
            link["e2e_fraction_of_ceiling"] = e2e["value"] / link["e2e_ceiling_tokens_per_s"]
            e2e["host_link"] = link
        except Exception as exc:  # a diagnostic: never lose the line over it
            e2e["host_link"] = {"error": repr(exc)[:200]}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        run, rows, threads, _ = cpu_reference_sample(seconds_target=10.0)
        t = run(rows)
        cpu_baseline = {"value": rows / t, "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": f"{rows} of {TOKENS} token rows, fwd+bwd incl. 2 dequantize passes, {t:.1f} s, "
                                  f"C restatement of qlora-core with {threads} OpenMP threads (rows split across threads)"}

    # ---- the other workloads of the metric (quantise / dequantise GB/s, Adam, the projection stack, the model step)
    del x, dy, y, dx
    torch.cuda.empty_cache()
    secondary = None
    if not args.no_secondary and not tf32:
        secondary = {}
        sec_steps = max(3, min(args.steps, 10))

        def guarded(name, fn):
            try:
                secondary[name] = fn()
            except Exception as exc:  # a secondary number must never cost the headline line
                secondary[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            torch.cuda.empty_cache()
            dist_.barrier()

        if rank == 0:
            guarded("quant_sweep", lambda: measure_quant_sweep(v, dist_, [4096, 8192, 16384], sec_steps))
            guarded("adam_c3", lambda: measure_adam(v, dist_, ("resident", "resident_fast_math", "paged_4"), sec_steps))
        else:
            dist_.barrier()
            dist_.barrier()
        guarded("stack_c5", lambda: measure_stack(v, dist_, max(2, sec_steps // 2), 2))
        guarded("model_c4", lambda: measure_model(v, dist_, 5, 3, 0, with_e2e=False, with_cpu=False))

    if rank == 0:
        cfg = base_config(world)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "tf32" if tf32 else "bf16", "data": "synthetic", "config": cfg,
            "details": {"precision": "TF32 mode: fp32 activations, tf32 tensor-core operands" if tf32 else "bf16 operands, fp32 accumulate",
                        "parallelism": f"token rows sharded over {world} GPU(s); W_q/A/B replicated; LoRA gradients summed by the "
                                       "library's NCCL communicator (qlc_comm_allreduce_sum_f32) on a stream of its own",
                        "tflops_per_gpu": tflops_step, "flops_per_step_per_gpu": flops_fwd_bwd(TOKENS, OUT_DIM, IN_DIM, RANK_R)},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks, "secondary": secondary,
        }
        print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
C5_PROJECTIONS = (("q", 4096, 4096), ("k", 4096, 4096), ("v", 4096, 4096), ("o", 4096, 4096),
                  ("gate", 11008, 4096), ("up", 11008, 4096), ("down", 4096, 11008))  # (name, out, in)
C5_TOKENS, C5_RANK, C5_ALPHA = 65536, 64, 128.0
C5_WORKLOAD = ("Llama-7B projection stack (q,k,v,o 4096x4096; gate,up 11008x4096; down 4096x11008), "
               "NF4 block 64 + double quant, LoRA r=64 alpha=128 on all, 65536 token rows per step")


def measure_stack(v, dist_, steps, warmup):
    """benchmark configuration 5: the seven Llama-7B projections (q/k/v/o 4096x4096, gate/up 11008x4096, down
    4096x11008), NF4 + double quant, LoRA r=64 on all; 65536 token rows per step split evenly over the
    ranks (strong scaling); each projection is an independent QloraLinear fwd+bwd with its own bf16 X and
    dY.  The LoRA gradients of all projections live in one fp32 bucket (4 997 120 floats) that is summed over
    the ranks projection by projection, by the library's communicator on a stream of its own, while the next
    projection computes."""
    import torch

    rank, local_rank, world, dev = dist_.rank, dist_.local_rank, dist_.world, dist_.dev
    ctx = v.GpuContext(local_rank)
    ctx.set_precision(v.PRECISION_BF16)
    ext = torch.cuda.ExternalStream(ctx.stream, device=dev)
    cctx = lib_comm = cext = None
    if world > 1:
        cctx = v.GpuContext(local_rank)
        lib_comm = dist_.lib_comm(v, cctx)
        cext = torch.cuda.ExternalStream(cctx.stream, device=dev)
        # the exchange's collective overlaps the next GEMM: that GEMM's single wave of CTA pairs leaves it its SMs
        ctx.set_reserved_sms(RESERVED_SMS)
    rows = C5_TOKENS // world
    r = C5_RANK
    gen = torch.Generator(device=dev).manual_seed(1)
    n_bucket = sum(r * i + o * r for _, o, i in C5_PROJECTIONS)
    bucket = torch.zeros(n_bucket, device=dev, dtype=torch.float32)
    layers, off = [], 0
    for name, o, i in C5_PROJECTIONS:
        w = torch.randn(o * i, generator=gen, device=dev, dtype=torch.float32) * 0.02
        a = (torch.randn(r * i, generator=gen, device=dev) / (i ** 0.5)).cpu().numpy()
        b = (torch.randn(o * r, generator=gen, device=dev) * 0.01).cpu().numpy()
        torch.cuda.synchronize()
        q = v.QuantizedTensor.quantize_dev(w.data_ptr(), o, i, v.QuantConfig(), ctx)
        ctx.synchronize()
        del w
        layer = v.QloraLinear.from_quantized(q, v.LoraAdapter(a, b, i, o, r, C5_ALPHA), ctx)
        g = torch.Generator(device=dev).manual_seed(1000 * (len(layers) + 1) + rank)
        x = torch.randn(rows, i, generator=g, device=dev).to(torch.bfloat16)
        dy = torch.randn(rows, o, generator=g, device=dev).to(torch.bfloat16)
        y = torch.empty(rows, o, device=dev, dtype=torch.bfloat16)
        dx = torch.empty(rows, i, device=dev, dtype=torch.bfloat16)
        layers.append(dict(name=name, o=o, i=i, layer=layer, x=x, dy=dy, y=y, dx=dx, n=r * i + o * r,
                           ga=bucket.data_ptr() + 4 * off, gb=bucket.data_ptr() + 4 * (off + r * i)))
        off += r * i + o * r
    torch.cuda.synchronize()
    done = [torch.cuda.Event() for _ in layers]
    joined = torch.cuda.Event()

    def step():
        for k, p in enumerate(layers):
            p["layer"].forward_dev(p["x"].data_ptr(), rows, p["y"].data_ptr(), v.DTYPE_BF16)
            p["layer"].backward_dev(p["x"].data_ptr(), p["dy"].data_ptr(), rows, p["dx"].data_ptr(), p["ga"], p["gb"],
                                    v.DTYPE_BF16)
            if world > 1:  # the exchange step, overlapped with the next projection
                done[k].record(ext)
                cext.wait_event(done[k])
                lib_comm.allreduce_sum_f32(p["ga"], p["n"])
        if world > 1:
            joined.record(cext)
            ext.wait_event(joined)

    ms_step, clocks, launches = timed_steps(dist_, ctx, ext, step, steps, warmup)
    flops_rank = sum(flops_fwd_bwd(rows, o, i, r) for _, o, i in C5_PROJECTIONS)

    n_prof = min(steps, 3)
    ctx.profile_enable(True)
    for _ in range(n_prof):
        step()
    ctx.synchronize()
    prof = [ctx.profile_read(s) for s in range(4)]
    ctx.profile_enable(False)
    dist_.barrier()
    peaks = measured_peaks()
    gemm_ms = prof[0][0] + prof[1][0]
    gemm_flops = n_prof * sum(4.0 * rows * o * i + 2.0 * rows * r * (o + i) for _, o, i in C5_PROJECTIONS)
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    tfl = flops_rank / (ms_step * 1e-3) / 1e12
    # a step lasts tens of milliseconds and a run of them is seconds long: the sustained figure is the denominator
    return {
        "workload": C5_WORKLOAD, "scaling": "strong", "metric": METRIC, "value": C5_TOKENS / (ms_step * 1e-3), "unit": UNIT,
        "ms_per_step": ms_step, "steps": steps, "warmup": warmup, "tokens_per_gpu": rows, "global_tokens": C5_TOKENS,
        "tflops_per_gpu": tfl, "flops_per_step_per_gpu": flops_rank, **frac_of(tfl, peaks, "tflops_sustained"),
        "gemm_roofline": {"bound": "tensor", "kernel": "umma_gemm3_kernel (all projections, forward Y and backward dX)",
                          "achieved": achieved, "unit": "TFLOP/s", **frac_of(achieved, peaks, "tflops_sustained"),
                          "per_slot_ms_per_step": {name: prof[k][0] / n_prof for k, name in
                                                   enumerate(("fwd_gemm", "bwd_dx_gemm", "lora_down", "token_grads"))}},
        "parallelism": f"token rows sharded over {world} GPU(s); W_q/A/B replicated; per-projection sum of the LoRA gradient "
                       f"bucket ({n_bucket} floats) by the library's communicator on a stream of its own",
        "gpu_launches": launches, "clocks": clocks,
    }


def stack_arm(args, dist_):
    res = measure_stack(__import__("vkqlora.rs_b200", fromlist=["x"]), dist_, args.steps, args.warmup)
    if dist_.rank == 0:
        line = {"metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": dist_.world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": C5_WORKLOAD, "tokens_per_gpu": res["tokens_per_gpu"], "global_tokens": C5_TOKENS,
                           "l2": "inputs+outputs per projection exceed the 126 MB L2; no explicit flush"},
                "details": {k: res[k] for k in ("parallelism", "tflops_per_gpu", "flops_per_step_per_gpu")},
                "roofline": dict(res["gemm_roofline"], traffic=None), "cpu_baseline": None, "e2e": None,
                "gpu_launches": res["gpu_launches"], "clocks": res["clocks"]}
        print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
def model_cpu_baseline(cfg, r, alpha, seq_len=256):
    """The numpy restatement of qlora-model/src/llama.rs (oracle/np_llama.py) on a bounded sample of the model
    workload: one sequence of `seq_len` tokens, forward + cross-entropy + backward through all layers, with the
    host's BLAS threads.  Weights are plain fp32 (the reference dequantises once, llama.rs:106-114)."""
    import numpy as np

    from oracle import np_llama as nl

    ocfg = nl.LlamaConfig(hidden=cfg.hidden, layers=cfg.layers, heads=cfg.heads, kv_heads=cfg.kv_heads,
                          intermediate=cfg.intermediate, vocab=cfg.vocab)
    ref = nl.random_model(ocfg, seed=1, targets=("q", "v"), rank=r, alpha=alpha, scale=0.02)
    g = np.random.Generator(np.random.Philox(9))
    ids = g.integers(0, cfg.vocab, seq_len)
    targets = np.roll(ids, -1)
    t0 = time.perf_counter()
    logits = ref.forward(ids)
    _, dlogits = nl.softmax_cross_entropy(logits, targets)
    ref.backward(ids, dlogits)
    dt = time.perf_counter() - t0
    try:
        from threadpoolctl import threadpool_info
        threads = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        threads = os.cpu_count() or 1
    return {"value": seq_len / dt, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"1 sequence of {seq_len} tokens (of 16 x 512), forward + loss + backward through all {cfg.layers} layers, "
                      f"{dt:.1f} s, numpy restatement of llama.rs (backward re-runs the forward, as llama.rs:389-400 does)"}


def measure_model(v, dist_, steps, warmup, model_layers, with_e2e=True, with_cpu=True):
    """benchmark configuration 4: SmolLM-135M-shaped QLoRA training step, random init (no checkpoint is involved):
    30 Llama layers, hidden 576, 9 heads / 3 KV heads, MLP 1536 SwiGLU, vocab 49152, RMSNorm, RoPE; all linears
    NF4 block 64 + double quant, Q/V LoRA r=8 alpha=16; token ids uniform over the vocabulary, 16 sequences of
    512 tokens per GPU; one step = forward + cross-entropy + backward + 8-bit Adam (max_resident_pages=4: the
    optimiser state streams through pinned host memory).  N > 1 is data parallel, weak scaling: the same model on
    every rank, 16 sequences per rank, the adapter gradients summed over ranks inside the step."""
    import numpy as np
    import torch

    from vkqlora.rs_b200 import llama

    rank, local_rank, world = dist_.rank, dist_.local_rank, dist_.world
    ctx = v.GpuContext(local_rank)
    ctx.set_precision(v.PRECISION_BF16)
    peaks = measured_peaks()
    cfg = llama.LlamaConfig.smollm_135m()
    if model_layers:
        cfg = dataclasses.replace(cfg, layers=model_layers)
    n_seq, seq_len, r, alpha = 16, 512, 8, 16.0
    # N > 1 is data parallel: every rank holds the same model (same seed) and its own 16 sequences; the adapter
    # gradients are summed over ranks by the library's communicator inside the step (weak scaling).
    comm = dist_.lib_comm(v, ctx) if world > 1 else None
    g = np.random.Generator(np.random.Philox(4))
    nrm = lambda *shape, s=0.02: (g.standard_normal(shape) * s).astype(np.float32)
    model = llama.LlamaModel(cfg, nrm(cfg.vocab, cfg.hidden), np.ones(cfg.hidden, np.float32), ctx)
    n_adapter = 0
    for li in range(cfg.layers):
        ws = {k: nrm(*cfg.proj_dims(k)) for k in llama.KINDS}
        model.set_layer(li, np.ones(cfg.hidden, np.float32), np.ones(cfg.hidden, np.float32), ws)
        for k in ("q", "v"):
            o, i = cfg.proj_dims(k)
            model.attach_adapter(li, k, nrm(r, i), np.zeros((o, r), np.float32), r, alpha)  # B = 0 (llama.rs:229-230)
            n_adapter += r * i + o * r
    opt = v.Adam8bit(v.AdamConfig(max_resident_pages=4), ctx)
    g = np.random.Generator(np.random.Philox(1000 + rank))  # the data differs per rank
    ids = g.integers(0, cfg.vocab, n_seq * seq_len).astype(np.uint32)
    targets = np.roll(ids, -1).astype(np.uint32)
    tokens = n_seq * seq_len
    ext = torch.cuda.ExternalStream(ctx.stream, device=dist_.dev)

    def step(want_loss=False):
        return model.train_step(opt, ids, targets, n_seq, seq_len, want_loss=want_loss, comm=comm)

    first_loss = step(True)
    ms_step, clocks, launches = timed_steps(dist_, ctx, ext, step, steps, max(warmup - 1, 2))
    last_loss = step(True)
    # End to end: the same call, fresh host ids and targets every step (uploaded inside the call) and the mean loss
    # read back (the per-token losses cross the host link and are averaged on the host).
    e2e = None
    if with_e2e:  # every rank: with a communicator the step is a collective
        n_e2e = 5
        batches = [(g.integers(0, cfg.vocab, tokens).astype(np.uint32), g.integers(0, cfg.vocab, tokens).astype(np.uint32))
                   for _ in range(n_e2e)]
        ctx.synchronize()
        dist_.barrier()
        w0 = time.perf_counter()
        for bi, bt in batches:
            model.train_step(opt, bi, bt, n_seq, seq_len, want_loss=True, comm=comm)
        ctx.synchronize()
        dist_.barrier()
        dt = dist_.max_over_ranks(time.perf_counter() - w0)
        e2e = {"value": world * n_e2e * tokens / dt, "unit": UNIT, "h2d_bytes_per_step": 2 * tokens * 4,
               "d2h_bytes_per_step": tokens * 4, "steps": n_e2e,
               "api": "qlc_llama_train_step (host ids and targets in, mean loss out; wall clock around the calls)"}
    cpu_baseline = None
    if rank == 0 and world == 1 and with_cpu:
        cpu_baseline = model_cpu_baseline(cfg, r, alpha)
    # algorithmic flops of the step: linears fwd+bwd (4MNK + LoRA), tied head (4*T*V*h), attention (causal: 2*2*T*S/2*d*H fwd, 2.5x bwd)
    lin = sum(flops_fwd_bwd(tokens, *cfg.proj_dims(k), r if k in ("q", "v") else 0) for k in llama.KINDS) * cfg.layers
    head = 4.0 * tokens * cfg.vocab * cfg.hidden
    attn = 3.5 * (2.0 * 2.0 * tokens * (seq_len / 2.0) * 64 * cfg.heads) * cfg.layers
    tfl = (lin + head + attn) / (ms_step * 1e-3) / 1e12
    del model, opt
    return {
        "workload": f"SmolLM-135M-shaped QLoRA training step ({cfg.layers} layers, hidden 576, 9/3 heads, MLP 1536, vocab "
                    "49152), all linears NF4 block 64 + double quant, Q/V LoRA r=8 alpha=16, 16 x 512 tokens, "
                    "fwd + cross-entropy + bwd + paged 8-bit Adam",
        "scaling": "weak", "metric": "qlora_model_train_step_tokens_per_s", "value": world * tokens / (ms_step * 1e-3),
        "unit": UNIT, "ms_per_step": ms_step, "steps": steps, "warmup": warmup, "tokens_per_gpu": tokens,
        "trainable_parameters": n_adapter,
        "parallelism": ("1 GPU" if world == 1 else
                        f"data parallel over {world} GPUs: 16 sequences per GPU, adapter gradients summed by one "
                        "grouped NCCL all-reduce inside qlc_llama_train_step_dp"),
        "tflops_per_gpu": tfl, "flops_per_step": {"linears": lin, "lm_head": head, "attention": attn},
        # no single kernel dominates this step (weight GEMMs 43 % of the kernel time over 420 launches): the fraction is
        # stated for the whole step against the sustained tensor peak
        **frac_of(tfl, peaks, "tflops_sustained"),
        "loss_first_step": first_loss, "loss_after": last_loss, "e2e": e2e, "cpu_baseline": cpu_baseline,
        "gpu_launches": launches, "clocks": clocks,
    }


def model_arm(args, dist_):
    import vkqlora.rs_b200 as v

    res = measure_model(v, dist_, max(args.steps // 5, 5), args.warmup, args.model_layers, with_e2e=not args.no_e2e,
                        with_cpu=not args.no_cpu_baseline)
    if dist_.rank == 0:
        print(json.dumps({
            "metric": res["metric"], "value": res["value"], "unit": UNIT, "n_gpus": dist_.world, "steps": res["steps"],
            "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": res["workload"], "tokens_per_gpu": res["tokens_per_gpu"]},
            "details": {k: res[k] for k in ("trainable_parameters", "parallelism", "tflops_per_gpu", "flops_per_step",
                                            "loss_first_step", "loss_after")},
            "roofline": {"bound": "tensor", "kernel": "whole training step (all kernels)", "achieved": res["tflops_per_gpu"],
                         "peak": res["peak"], "unit": "TFLOP/s", "frac": res["frac"], "peak_source": res["peak_source"],
                         "traffic": None},
            "cpu_baseline": res["cpu_baseline"], "e2e": res["e2e"], "gpu_launches": res["gpu_launches"],
            "clocks": res["clocks"]}), flush=True)


# ---------------------------------------------------------------------------------------------
def measure_quant_sweep(v, dist_, sizes, iters):
    """Standalone quantize_nf4 / dequantize sweep (benchmark configuration 2b): GB/s of algorithmic bytes
    (quantize 4.51587 B/elem; dequantize 0.51587 + 4 (fp32) or + 2 (bf16) B/elem)."""
    import torch

    dev = dist_.dev
    ctx = v.GpuContext(dist_.local_rank)
    ext = torch.cuda.ExternalStream(ctx.stream, device=dev)
    peaks = measured_peaks()
    out = {}
    sampler = ClockSampler(dist_.local_rank)
    sampler.start()
    t_begin = time.perf_counter()
    for n_side in sizes:
        n = n_side * n_side
        copies = max(1, (512 << 20) // (4 * n))  # rotate inputs so every launch reads cold data
        ws = [torch.randn(n, device=dev, dtype=torch.float32) * 0.02 for _ in range(copies)]
        qs = [v.QuantizedTensor.quantize_dev(w.data_ptr(), n_side, n_side, v.QuantConfig(), ctx) for w in ws]
        # outputs rotate as well: a single 64 MiB output would stay in the 126 MB L2 from one launch to the next
        ofs = [torch.empty(n, device=dev, dtype=torch.float32) for _ in range(copies)]
        obs = [torch.empty(n, device=dev, dtype=torch.bfloat16) for _ in range(max(1, (512 << 20) // (2 * n)))]
        ctx.synchronize()
        torch.cuda.synchronize()

        def timed(fn, iters):
            for i in range(3):
                fn(i)
            ctx.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(ext)
            for i in range(iters):
                fn(i)
            e1.record(ext)
            ctx.synchronize()
            return e0.elapsed_time(e1) / iters * 1e-3

        it = max(iters, 2)
        if n_side <= 8192:
            it *= 4  # microsecond kernels: more launches per measurement
        tq = timed(lambda i: qs[i % copies].requantize_dev(ws[(i + 1) % copies].data_ptr()), it)
        for i in range(copies):  # restore: tensor i holds weights i again
            qs[i].requantize_dev(ws[i].data_ptr())
        tf = timed(lambda i: qs[i % copies].dequantize_dev(ofs[i % copies].data_ptr(), v.DTYPE_F32), it)
        tb = timed(lambda i: qs[i % copies].dequantize_dev(obs[i % len(obs)].data_ptr(), v.DTYPE_BF16), it)
        bq, bf_, bb = 4.515869140625 * n, 4.515869140625 * n, 2.515869140625 * n
        hb = peaks["hbm_gbs"]
        out[f"{n_side}x{n_side}"] = {
            "quantize_us": tq * 1e6, "quantize_gbs": bq / tq / 1e9, "quantize_frac": bq / tq / 1e9 / hb,
            "dequant_f32_us": tf * 1e6, "dequant_f32_gbs": bf_ / tf / 1e9, "dequant_f32_frac": bf_ / tf / 1e9 / hb,
            "dequant_bf16_us": tb * 1e6, "dequant_bf16_gbs": bb / tb / 1e9, "dequant_bf16_frac": bb / tb / 1e9 / hb,
            "launches_timed": it}
        del ws, qs, ofs, obs
        torch.cuda.empty_cache()
    clocks = sampler.stop(t_begin, time.perf_counter())
    return {"workload": "quantize_nf4 / dequantize sweep, fp32 weights ~N(0,0.02), block 64 + double quant",
            "unit": "GB/s of algorithmic bytes (quantize 4.51587 B/elem; dequantize 0.51587 + 4 (fp32) or + 2 (bf16) B/elem)",
            "l2": "inputs and outputs rotate over >= 512 MiB of distinct buffers each", "bound": "hbm", "peak": peaks["hbm_gbs"],
            "peak_source": f"hbm_gbs, {peaks['source']}", "sizes": out, "clocks": clocks}


def quant_sweep_arm(args, dist_):
    import vkqlora.rs_b200 as v

    res = measure_quant_sweep(v, dist_, [int(x) for x in args.sizes.split(",")], max(args.steps, 2))
    out = res["sizes"]
    big = out[max(out, key=lambda k: int(k.split("x")[0]))]
    print(json.dumps({"metric": "nf4_dequant_hbm_gbs", "value": big["dequant_f32_gbs"], "unit": "GB/s", "n_gpus": 1,
                      "steps": max(args.steps, 2), "warmup": 3, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": res["workload"], "l2": res["l2"]},
                      "roofline": {"bound": "hbm", "achieved": big["dequant_f32_gbs"], "peak": res["peak"], "unit": "GB/s",
                                   "frac": big["dequant_f32_gbs"] / res["peak"], "peak_source": res["peak_source"],
                                   "traffic": None},
                      "sweep": out, "clocks": res["clocks"]}), flush=True)


def measure_adam(v, dist_, variants, steps):
    """Paged 8-bit Adam (benchmark configuration 3): 112 tensors x 262144 fp32 (28 layers x Q/V x {A 64x4096, B 4096x64}),
    block 256, lr 1e-3, betas 0.9/0.999, eps 1e-8; once fully resident and once with max_resident_pages=4
    (every state page is evicted to pinned host memory each step).  Algorithmic traffic 16 B/elem + 16 B/block."""
    import torch

    dev = dist_.dev
    ctx = v.GpuContext(dist_.local_rank)
    ext = torch.cuda.ExternalStream(ctx.stream, device=dev)
    peaks = measured_peaks()
    n_t, numel = 112, 262144
    gen = torch.Generator(device=dev).manual_seed(6)
    params = [torch.randn(numel, generator=gen, device=dev) * 0.01 for _ in range(n_t)]
    grads = [torch.randn(numel, generator=gen, device=dev) * 0.01 for _ in range(n_t)]
    pp, gp, ll = [p.data_ptr() for p in params], [g.data_ptr() for g in grads], [numel] * n_t
    bytes_step = 16.0 * n_t * numel + 16.0 * n_t * (numel // 256)
    res = {}
    steps = max(steps, 2)
    all_variants = (("resident", None, False), ("resident_fast_math", None, True), ("paged_4", 4, False))
    sampler = ClockSampler(dist_.local_rank)
    sampler.start()
    t_begin = time.perf_counter()
    for name, pages, fast in [x for x in all_variants if x[0] in variants]:
        opt = v.Adam8bit(v.AdamConfig(max_resident_pages=pages), ctx)
        opt.set_fast_math(fast)
        for _ in range(5):
            opt.step_dev(pp, gp, ll)
        ctx.synchronize()
        torch.cuda.synchronize()
        n_steps = steps if pages else 4 * steps
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(ext)
        for _ in range(n_steps):
            opt.step_dev(pp, gp, ll)
        e1.record(ext)
        ctx.synchronize()
        wall = (time.perf_counter() - t0) / n_steps
        t = e0.elapsed_time(e1) / n_steps * 1e-3
        info = opt.paging_info()
        res[name] = {"us_per_step": t * 1e6, "wall_us_per_step": wall * 1e6, "gbs": bytes_step / t / 1e9,
                     "frac_of_hbm": bytes_step / t / 1e9 / peaks["hbm_gbs"], "steps_timed": n_steps,
                     "state_bytes": opt.state_bytes(), "device_state_bytes": info["device_bytes"],
                     "host_state_bytes": info["host_bytes"], "h2d_bytes_per_step": info["h2d_bytes_last_step"],
                     "d2h_bytes_per_step": info["d2h_bytes_last_step"],
                     "host_link_gbs_each_way": (info["h2d_bytes_last_step"] / t / 1e9) if pages else None}
        opt.close()
    clocks = sampler.stop(t_begin, time.perf_counter())
    return {"workload": "paged 8-bit Adam, 112 tensors x 262144 fp32, block 256 (exact = bit-identical to the CPU "
                        "restatement; fast_math = opt-in approximations within 1e-5; paged_4 = all state in pinned host memory)",
            "unit": "GB/s of algorithmic bytes (16 B/elem + 16 B/block = 471.6 MB per step)",
            "l2": "params+grads+state per step (0.47 GB) exceed the 126 MB L2", "bound": "hbm (paged_4: host link)",
            "peak": peaks["hbm_gbs"], "peak_source": f"hbm_gbs, {peaks['source']}", "variants": res, "clocks": clocks}


def adam_arm(args, dist_):
    import vkqlora.rs_b200 as v

    out = measure_adam(v, dist_, args.variants.split(","), args.steps)
    res = out["variants"]
    r = res.get("resident") or next(iter(res.values()))
    print(json.dumps({"metric": "adam8bit_step_hbm_gbs", "value": r["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": r["steps_timed"],
                      "warmup": 5, "ms_per_step": r["us_per_step"] / 1e3, "higher_is_better": True, "dtype": "f32",
                      "data": "synthetic", "config": {"workload": out["workload"], "l2": out["l2"]},
                      "roofline": {"bound": "hbm", "achieved": r["gbs"], "peak": out["peak"], "unit": "GB/s",
                                   "frac": r["gbs"] / out["peak"], "peak_source": out["peak_source"], "traffic": None},
                      "variants": res, "clocks": out["clocks"]}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qlora", choices=["qlora", "stack", "model", "quant_sweep", "adam"],
                    help="qlora = the headline step (default; its line also carries the other workloads under "
                         "`secondary`); the others run one of them alone")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "tf32"],
                    help="qlora workload: bf16 operands (default, the headline) or the TF32 mode")
    ap.add_argument("--sizes", default="4096,8192,16384", help="quant_sweep: square sizes to run")
    ap.add_argument("--variants", default="resident,resident_fast_math,paged_4", help="adam: variants to run")
    ap.add_argument("--model-layers", type=int, default=0,
                    help="model: number of decoder layers (0 = the configuration's 30); smaller values are for profiler "
                         "captures and are named in config.workload")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--no-secondary", action="store_true", help="qlora workload: skip the other workloads (profiling runs)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    # The exchange is a few MB per step: two NCCL channels carry it without taking SMs from the GEMM's waves; NVLS
    # (in-switch reduction) buys nothing at this size.  Both are defaults that the environment may override.
    os.environ.setdefault("NCCL_MAX_CTAS", "2")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch

    torch.cuda.set_device(local_rank)
    if args.workload in ("quant_sweep", "adam") and rank != 0:
        return
    dist_ = Dist(rank, local_rank, world if args.workload not in ("quant_sweep", "adam") else 1)
    try:
        if args.workload == "quant_sweep":
            quant_sweep_arm(args, dist_)
        elif args.workload == "adam":
            adam_arm(args, dist_)
        elif args.workload == "stack":
            stack_arm(args, dist_)
        elif args.workload == "model":
            model_arm(args, dist_)
        else:
            ours_arm(args, dist_)
    finally:
        dist_.close()


if __name__ == "__main__":
    main()
