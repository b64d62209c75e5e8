#!/usr/bin/env python
"""Benchmark of the Blaze quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c3|c4|c5]

Default workload (the one the metric is quoted on): MXFP8 GEMM M=N=K=8192 with fused bf16 bias + GELU(tanh) and bf16
output, synthetic seeded inputs.  With N GPUs (one process per GPU, launched by torch.distributed.run) the GEMM is
sharded along N with no data-path collective: every rank holds A and an 8192-column shard of B, so the global
problem is M=8192, N=8192*gpus, K=8192 (weak scaling).  One step = one pass of the hot path over that batch.

Prints ONE JSON line: `value` = whole-job TFLOPS with quantized operands resident in HBM; `e2e` = the same metric
through the acltensor* C API with the step's fp32 activations coming from pinned host memory and the bf16 result
going back to it (copies and on-device quantisation inside the timed region); `roofline` for the GEMM kernel against
the measured tensor peak; `cpu_baseline` = the reference-style CPU golden (de-quantise to float32, np.matmul,
epilogue, bf16) timed on this box's host cores.

`--impl reference` times that CPU golden alone, on the same config and metric.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, M, N, K, description)
    "c1": ("fp8", 256, 512, 1024, "FP8 1x128/128x128 GEMM 256x512x1024, bf16 out"),
    "c2": ("mx", 8192, 8192, 8192, "MXFP8 GEMM 8192^3 + bf16 bias + GELU(tanh), bf16 out"),
    "c3": ("mx4", 4096, 14336, 4096, "W4A8 MX GEMM 4096x14336x4096, bf16 out"),
    "c4": ("grouped", 32768, 768, 2048, "MoE grouped FP8 matmul G=128, K=2048, N=768, 32768 tokens"),
    "c5": ("fp8sk", 128, 7168, 18432, "stream-K decode FP8 GEMM M=128, N=7168, K=18432 + bf16 residual"),
    # beyond the five configurations: C2's shape with both operands MXFP4, on kind::mxf4
    "c6": ("mxf4", 8192, 8192, 8192, "MXFP4 x MXFP4 GEMM 8192^3 + bf16 bias + GELU(tanh), bf16 out"),
}


def algorithmic_bytes(kind, M, N, K, G=128):
    """Minimum HBM traffic: operands, scales, epilogue inputs and the output, each moved once."""
    if kind == "mx":
        return M * K + N * K + (M + N) * (K // 32) + 2 * N + 2 * M * N
    if kind == "mxf4":
        return M * K // 2 + N * K // 2 + (M + N) * (K // 32) + 2 * N + 2 * M * N
    if kind == "mx4":
        return M * K + N * K // 2 + (M + N) * (K // 32) + 2 * M * N
    if kind == "grouped":
        return M * K + G * N * K + 4 * M * (K // 128) + 4 * G * (K // 128) * (N // 128) + 8 * G + 2 * M * N
    kb, nb = -(-K // 128), -(-N // 128)
    extra = 2 * M * N if kind == "fp8sk" else 0
    return M * K + N * K + 4 * M * kb + 4 * kb * nb + 2 * M * N + extra


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and clock-event reasons through NVML (read-only queries) every few milliseconds on a
    thread while the timed region runs."""

    def __init__(self, gpu_index, period_s=0.005):
        self.gpu = gpu_index
        self.period = period_s
        self.samples = []
        self._stop = False
        self._thread = None
        self._max = None

    def start(self):
        try:
            import threading
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self._max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            return

        def loop():
            while not self._stop:
                try:
                    mhz = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                    reasons = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                    watts = pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0
                    self.samples.append((float(mhz), int(reasons), watts))
                except Exception:
                    pass
                time.sleep(self.period)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def _physical_index(self):
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            if self.gpu < len(ids) and ids[self.gpu].isdigit():
                return int(ids[self.gpu])
        return self.gpu

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": self._max, "reasons": [], "samples": 0, "power_w_max": None}
        if self._thread is None:
            return out
        self._stop = True
        self._thread.join(timeout=2)
        if not self.samples:
            return out
        import pynvml
        top = max(w for _, _, w in self.samples)
        busy = [x for x in self.samples if x[2] > 0.5 * top] or self.samples      # drop idle samples around the region
        names = (("hw_slowdown", pynvml.nvmlClocksEventReasonHwSlowdown),
                 ("hw_thermal_slowdown", pynvml.nvmlClocksEventReasonHwThermalSlowdown),
                 ("sw_thermal_slowdown", pynvml.nvmlClocksEventReasonSwThermalSlowdown),
                 ("sw_power_cap", pynvml.nvmlClocksEventReasonSwPowerCap))
        reasons = sorted({n for n, bit in names for _, r, _ in busy if r & bit})
        out.update(sm_mhz=float(np.median([m for m, _, _ in busy])), reasons=reasons, samples=len(busy),
                   power_w_max=round(top, 1))
        return out


# ---------------------------------------------------------------------------------------------------- CPU golden

def make_cpu_golden(workload):
    """Reference-style CPU golden (de-quantise to float32, np.matmul, epilogue, bf16) on a bounded sample of the
    workload: the first rows of A against the first rows of B (the first experts for the grouped workload), full K.
    Returns (run, flops, description)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import blaze_oracle as o
    try:
        # the launcher of multi-process runs pins OMP_NUM_THREADS to 1; the CPU golden is allowed every host core
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=len(os.sched_getaffinity(0)))
    except Exception:
        pass
    kind, M, N, K, desc = WORKLOADS[workload]
    cfg = int(workload[1:])
    if kind in ("mx", "mx4", "mxf4"):
        rows, cols = min(2048, M), min(4096, N)
        name = "e4m3" if kind == "mx" else "e2m1"
        name_a = "e2m1" if kind == "mxf4" else "e4m3"
        dense = kind in ("mx", "mxf4")                     # C2-style: N(0,1) weights, bias + GELU
        a = o.normal_f32(cfg, 0, (rows, K), 1.0)
        w = o.normal_f32(cfg, 1, (cols, K), 1.0 if dense else 0.02)
        bias = o.bf16_round(o.normal_f32(cfg, 2, (cols,), 0.1)) if dense else None
        act = o.ACT_GELU_TANH if dense else o.ACT_IDENTITY
        qa, sa = o.quant_mx(a, name_a)
        qb, sb = o.quant_mx(w, name)

        def run():
            da = o.dequant_mx(qa, sa, K, name_a, np.float32)
            db = o.dequant_mx(qb, sb, K, name, np.float32)
            return o.matmul_golden32(da, db, bias, act)
        what = f"{rows} rows of A x {cols} rows of B x K={K}"
        flops = 2.0 * rows * cols * K
    elif kind == "grouped":
        experts = 32
        group_rows = o.moe_group_rows()[:experts]
        rows = int(group_rows.sum())
        a = o.normal_f32(cfg, 0, (rows, K), 1.0)
        w = o.normal_f32(cfg, 1, (experts * N, K), 0.02)
        qa, sa = o.quant_fp8_1x128(a)
        qw = [o.quant_fp8_128x128(w[g * N:(g + 1) * N]) for g in range(experts)]

        def run():
            da = o.dequant_fp8_1x128(qa, sa, np.float32)
            db = np.stack([o.dequant_fp8_128x128(c, s, np.float32) for c, s in qw])
            return o.bf16_round(o.grouped_matmul_ref(da, db, group_rows, np.float32))
        what = f"the first {experts} experts ({rows} tokens) x N={N} x K={K}"
        flops = 2.0 * rows * N * K
    else:
        rows, cols = min(256, M), min(1024, N)
        a = o.normal_f32(cfg, 0, (rows, K), 1.0)
        w = o.normal_f32(cfg, 1, (cols, K), 0.02)
        residual = o.bf16_round(o.normal_f32(cfg, 3, (rows, cols), 1.0)) if kind == "fp8sk" else None
        qa, sa = o.quant_fp8_1x128(a)
        qb, sb = o.quant_fp8_128x128(w)

        def run():
            return o.matmul_golden32(o.dequant_fp8_1x128(qa, sa, np.float32), o.dequant_fp8_128x128(qb, sb, np.float32),
                                     None, o.ACT_IDENTITY, residual)
        what = f"{rows} rows of A x {cols} rows of B x K={K}"
        flops = 2.0 * rows * cols * K
    sample = f"{what} of '{desc}' per step: de-quantise to float32, np.matmul, epilogue, bf16"
    return run, flops, sample


def time_cpu_golden(run, repeats):
    run()                                            # warm-up (BLAS thread pool, page faults)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    return times


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, M, N, K, desc = WORKLOADS[args.workload]
    wl = args.workload
    cores = len(os.sched_getaffinity(0))
    run, flops, sample = make_cpu_golden(wl)
    for _ in range(max(1, min(args.warmup, 3))):
        run()
    times = []
    t_all = time.perf_counter()
    for _ in range(args.steps):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_all > 200:        # keep the whole run within a few minutes
            break
    ms = 1e3 * float(np.mean(times))
    value = flops / (ms * 1e-3) / 1e12
    line = {
        "impl": "reference", "metric": "quantized GEMM TFLOPS", "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
        "config": {"workload": WORKLOADS[wl][4], "M": M, "N": N, "K": K, "sharding": "none (CPU golden on rank 0)"},
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------- GPU arm

def gpu_arm(args):
    import torch
    import torch.distributed as dist
    from ops_tensor_b200 import host as H
    from ops_tensor_b200 import native, shard
    from ops_tensor_b200 import synthetic as o           # seeded input generators; the CPU oracle is not used here

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    native.lib()                                     # fails loudly if the CUDA library is missing

    kind, M, N, K, desc = WORKLOADS[args.workload]
    steps, warmup = args.steps, max(args.warmup, 3)
    cfg_id = int(args.workload[1])
    G = 128
    group_rows = None
    group_rows_host = None
    strong = args.shard == "strong" and world > 1
    flops_job = 2.0 * M * N * K * (1 if strong or world == 1 else world)     # whole-job flops per step
    sharding = f"N-sharded over {world} GPU(s), A replicated, no collective"
    if strong and kind == "grouped":
        # experts (or row ranges of oversized experts) dealt to ranks by token count; every rank computes its share
        pieces = shard.plan_experts(o.moe_group_rows(), world)[rank]
        group_rows_host = np.array([pc.rows for pc in pieces], dtype=np.int64)
        G = len(pieces)
        M = int(group_rows_host.sum())
        sharding = f"experts partitioned over {world} GPUs by token count (longest first), no collective"
    elif strong:
        n0, n1 = shard.n_shard(N, world, rank)
        N = n1 - n0
    elif kind == "grouped":
        group_rows_host = o.moe_group_rows()
    flops = 2.0 * M * N * K                                                  # this rank's flops per step

    # ---- inputs (seeded, generated on the host once) -----------------------------------------------------------
    a_host = torch.from_numpy(o.normal_f32(cfg_id, 0, (M, K), 1.0)).pin_memory()
    a_dev = a_host.to(dev, non_blocking=True)
    sigma_b = 1.0 if kind in ("mx", "mxf4") else 0.02
    b_rows = G * N if kind == "grouped" else N
    w_dev = torch.from_numpy(o.normal_f32(cfg_id, 1 + 16 * rank, (b_rows, K), sigma_b)).to(dev)
    bias = residual = None
    if kind in ("mx", "mxf4"):
        bias = torch.from_numpy(o.normal_f32(cfg_id, 2, (N,), 0.1)).to(dev).to(torch.bfloat16)   # nearest-even
    if kind == "fp8sk":
        residual = torch.from_numpy(o.normal_f32(cfg_id, 3, (M, N), 1.0)).to(dev).to(torch.bfloat16)

    a_dtype = H.R_4F_E2M1 if kind == "mxf4" else H.R_8F_E4M3
    if kind in ("mx", "mx4", "mxf4"):
        b_dtype = H.R_8F_E4M3 if kind == "mx" else H.R_4F_E2M1
        mode_a = mode_b = H.SCALE_MX_E8M0_VEC32
        qb, sb = H.quantize(w_dev, mode_b, b_dtype)
        plan = H.Contraction(M, N, K, scale_mode_a=mode_a, scale_mode_b=mode_b, a_dtype=a_dtype, b_dtype=b_dtype,
                             activation=H.OP_IDENTITY if kind == "mx4" else H.OP_GELU, bias=bias is not None,
                             b_is_static=True)
        launches_per_step = 2                        # scale re-tile of A + GEMM (B's pre-pass is reused)
    else:
        mode_a, mode_b = H.SCALE_FP32_1X128, H.SCALE_FP32_128X128
        if kind == "grouped":
            group_rows = torch.from_numpy(group_rows_host).to(dev)
            qb = torch.empty((G, N, K), dtype=torch.uint8, device=dev)
            sb = torch.empty((G, K // 128, N // 128), dtype=torch.float32, device=dev)
            for g in range(G):
                c, s = H.quantize(w_dev[g * N:(g + 1) * N], mode_b)
                qb[g].copy_(c)
                sb[g].copy_(s)
        else:
            qb, sb = H.quantize(w_dev, mode_b)
        plan = H.Contraction(M, N, K, scale_mode_a=mode_a, scale_mode_b=mode_b, groups=G if kind == "grouped" else 0,
                             residual=residual is not None)
        # a plan that asks for workspace runs stream-K: a kernel that zeroes the fix-up flags, then the GEMM
        launches_per_step = 2 if plan.workspace_bytes > 0 else 1
    del w_dev
    qa, sa = H.quantize(a_dev, mode_a, a_dtype)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    out_host = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    torch.cuda.synchronize()

    def step():
        plan(qa, sa, qb, sb, out, bias=bias, residual=residual, group_rows=group_rows)

    # End-to-end steps through the public API with HOST buffers.  Two pipelines are timed:
    #   "operands": every operand the contraction call takes (A codes and scales, B codes and scales, bias, residual,
    #               group list) starts each step in pinned host memory - the call the reference's operator API makes,
    #               with nothing assumed resident; a plan that does not treat B as static runs it;
    #   "fp32":     this step's fp32 activations start in pinned host memory and are quantised on the device first
    #               (weights resident, as in serving).
    # Both return the bf16 result to pinned host memory every step.  Copies in, compute and copies out run on three
    # streams over double buffers, so the copies of neighbouring steps overlap; every step still moves all of its
    # bytes inside the timed region.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    out2 = [out, torch.empty_like(out)]
    out_host2 = [out_host, torch.empty_like(out_host).pin_memory()]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_consumed = [torch.cuda.Event() for _ in range(2)]
    ev_computed = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    e2e_counter = [0]
    e2e_mode = ["operands"]

    dev_ops = {"a": qa, "sa": sa, "b": qb, "sb": sb}
    if bias is not None:
        dev_ops["bias"] = bias
    if residual is not None:
        dev_ops["residual"] = residual
    if group_rows is not None:
        dev_ops["group_rows"] = group_rows
    host_ops = {k: v.cpu().pin_memory() for k, v in dev_ops.items()}
    dev_ops2 = [dev_ops, {k: torch.empty_like(v) for k, v in dev_ops.items()}]
    a_dev2 = [a_dev, torch.empty_like(a_dev)]
    plan_e2e = plan
    if kind in ("mx", "mx4", "mxf4"):
        plan_e2e = H.Contraction(M, N, K, scale_mode_a=mode_a, scale_mode_b=mode_b, a_dtype=a_dtype, b_dtype=b_dtype,
                                 activation=H.OP_IDENTITY if kind == "mx4" else H.OP_GELU, bias=bias is not None,
                                 b_is_static=False)
    h2d_bytes = {"operands": sum(v.numel() * v.element_size() for v in host_ops.values()),
                 "fp32": a_host.numel() * 4}

    def step_e2e():
        i = e2e_counter[0]
        e2e_counter[0] += 1
        b = i & 1
        main = torch.cuda.current_stream()
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_consumed[b])           # the buffers' previous contents have been consumed
            if e2e_mode[0] == "operands":
                for k, v in host_ops.items():
                    dev_ops2[b][k].copy_(v, non_blocking=True)
            else:
                a_dev2[b].copy_(a_host, non_blocking=True)
            ev_in[b].record(s_in)
        main.wait_event(ev_in[b])
        if i >= 2:
            main.wait_event(ev_out[b])                    # the previous result in this buffer has left the device
        if e2e_mode[0] == "operands":
            d = dev_ops2[b]
            plan_e2e(d["a"], d["sa"], d["b"], d["sb"], out2[b], bias=d.get("bias"), residual=d.get("residual"),
                     group_rows=d.get("group_rows"))
            ev_consumed[b].record(main)
        else:
            qa2, sa2 = H.quantize(a_dev2[b], mode_a, a_dtype)
            ev_consumed[b].record(main)
            plan(qa2, sa2, qb, sb, out2[b], bias=bias, residual=residual, group_rows=group_rows)
        ev_computed[b].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_computed[b])
            out_host2[b].copy_(out2[b], non_blocking=True)
            ev_out[b].record(s_out)

    def drain_e2e():
        main = torch.cuda.current_stream()
        for b in range(2):
            main.wait_event(ev_out[b])

    def timed(fn, n):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        if fn is step_e2e:
            drain_e2e()                                   # the last copies back to the host are part of the region
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        return shard.max_over_ranks(e0.elapsed_time(e1), dev)

    sampler = ClockSampler(local_rank)
    if rank == 0 and not args.kernel_only:
        sampler.start()
        time.sleep(0.05)
    step()                                           # first call: module load, workspace allocation
    torch.cuda.synchronize()
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0.record()
    for _ in range(warmup):
        step()
    w1.record()
    torch.cuda.synchronize()
    # A short step (tens of microseconds) finishes its warm-up before the SM clock has left its idle state: keep
    # stepping, untimed, until the GPU has been busy for about 20 ms.  Long steps (C2) get exactly `warmup` steps.
    ramp_steps = 0
    warm_ms = w0.elapsed_time(w1)
    if warmup > 0 and warm_ms < 1.0:
        ramp_steps = min(5000, int(20.0 / max(warm_ms / warmup, 1e-3)))
        for _ in range(ramp_steps):
            step()
        torch.cuda.synchronize()
    total_ms = timed(step, steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = total_ms / steps
    # Optional: the same step followed by the one collective the path can need, an all-gather of the output shards,
    # either after the GEMM or chunk by chunk while the next chunk computes (reported beside the headline, not in it).
    gather_info = None
    if args.gather != "none" and world > 1 and kind in ("mx", "mx4", "mxf4"):
        ranges = shard.column_chunks(N, args.gather_chunks, 256)
        act = H.OP_IDENTITY if kind == "mx4" else H.OP_GELU
        chunk_plans = {r: H.Contraction(M, r[1] - r[0], K, scale_mode_a=mode_a, scale_mode_b=mode_b, a_dtype=a_dtype,
                                        b_dtype=b_dtype, activation=act, bias=bias is not None, b_is_static=True,
                                        sm_limit=args.gather_gemm_sms)
                       for r in ranges}
        whole = torch.empty((world * M, N), dtype=torch.bfloat16, device=dev)
        bufs = shard.gather_buffers(M, N, world, len(ranges), torch.bfloat16, dev, 256)
        peer = shard.PeerGatherBuffers(M, N, world, rank, len(ranges), torch.bfloat16, dev, 256) if args.gather == "peer" else None

        def run_chunk(c0, c1, o_):
            chunk_plans[(c0, c1)](qa, sa, qb[c0:c1], sb[c0:c1], o_, bias=None if bias is None else bias[c0:c1])

        fused = None
        if args.gather == "fused":
            # one full-width GEMM whose epilogue stores every tile to all ranks' gathered buffers (C ABI: peerD)
            fused = shard.PeerGatherBuffers(M, N, world, rank, 1, torch.bfloat16, dev, 256)
            f_kw = dict(b_elem=native.ELEM_E4M3 if kind == "mx" else native.ELEM_E2M1,
                        a_elem=native.ELEM_E2M1 if kind == "mxf4" else native.ELEM_E4M3, bias=bias,
                        activation=native.ACT_IDENTITY if kind == "mx4" else native.ACT_GELU_TANH)
            probe = native.mx_gemm_args(qa, sa, qb, sb, fused.gathered[0][rank],
                                        peer_outs=[s_ for s_ in fused.peer_slots[0] if s_ is not None], **f_kw)
            f_ws = torch.empty(max(native.mx_gemm_workspace_bytes(probe), 256), dtype=torch.uint8, device=dev)
            f_calls = [0]

            def run_fused(out_, peers):
                native.mx_gemm(qa, sa, qb, sb, out=out_, workspace=f_ws, peer_outs=peers,
                               reuse_b_prepass=f_calls[0] > 0, **f_kw)
                f_calls[0] += 1

        def step_gather():
            if args.gather == "fused":
                shard.gemm_gather_fused(run_fused, fused)
            elif args.gather == "after":
                step()
                dist.all_gather_into_tensor(whole, out)
            else:
                shard.gemm_gather_overlapped(run_chunk, M, N, world, chunks=len(ranges), dtype=torch.bfloat16,
                                             device=dev, multiple=256, assemble=False, buffers=bufs, peer_buffers=peer)

        for _ in range(warmup):
            step_gather()
        torch.cuda.synchronize()
        g_ms = timed(step_gather, steps) / steps
        gather_info = {"mode": args.gather, "chunks": 1 if args.gather in ("after", "fused") else len(ranges),
                       "gemm_sms": args.gather_gemm_sms or "all", "nccl_max_ctas": os.environ.get("NCCL_MAX_CTAS"),
                       "ms_per_step": g_ms, "gemm_only_ms_per_step": ms_per_step,
                       "gathered_bytes_per_rank": (world - 1) * M * N * 2}
    if args.gather in ("after", "fused") and world > 1 and kind == "fp8sk":
        # the decode GEMM: its output is small, so a separate all-gather is mostly launch latency
        whole = torch.empty((world * M, N), dtype=torch.bfloat16, device=dev)
        if args.gather == "fused":
            fused = shard.PeerGatherBuffers(M, N, world, rank, 1, torch.bfloat16, dev, 128)
            probe = native.fp8_gemm_args(qa, sa, qb, sb, fused.gathered[0][rank], residual=residual,
                                         peer_outs=[s_ for s_ in fused.peer_slots[0] if s_ is not None])
            f_ws = torch.empty(max(native.fp8_gemm_workspace_bytes(probe), 256), dtype=torch.uint8, device=dev)

        def step_gather():
            if args.gather == "fused":
                shard.gemm_gather_fused(lambda out_, peers: native.fp8_gemm(qa, sa, qb, sb, out=out_, workspace=f_ws,
                                                                            residual=residual, peer_outs=peers), fused)
            else:
                step()
                dist.all_gather_into_tensor(whole, out)

        for _ in range(max(warmup, 20)):
            step_gather()
        torch.cuda.synchronize()
        g_ms = timed(step_gather, steps) / steps
        gather_info = {"mode": args.gather, "chunks": 1, "ms_per_step": g_ms, "gemm_only_ms_per_step": ms_per_step,
                       "gathered_bytes_per_rank": (world - 1) * M * N * 2}
    e2e_ms = {"operands": float("nan"), "fp32": float("nan")}
    if not args.kernel_only:
        e2e_steps = max(4, min(steps, 20))
        for mode in ("operands", "fp32"):
            e2e_mode[0] = mode
            e2e_counter[0] = 0
            for _ in range(2):
                step_e2e()
            torch.cuda.synchronize()
            e2e_counter[0] = 0
            e2e_ms[mode] = timed(step_e2e, e2e_steps) / e2e_steps
    status = H.device_status()
    if plan_e2e is not plan:
        plan_e2e.close()
    plan.close()

    if rank == 0:
        peaks = measured_peaks()
        value = flops_job / (ms_per_step * 1e-3) / 1e12
        abytes = algorithmic_bytes(kind, M, N, K, G)
        tensor_bound = kind in ("mx", "mx4", "mxf4")
        if tensor_bound:
            # FP8 operands run at twice the bf16 MMA rate; the loop is timed back to back, so the burst figure
            # applies to short runs and the sustained one to runs of a second or more
            base = peaks["bf16_tflops_sustained"] if total_ms > 1000.0 else peaks["bf16_tflops"]
            peak = (4.0 if kind == "mxf4" else 2.0) * base      # FP4 x FP4 (kind::mxf4) runs at twice the FP8 rate
            achieved = flops / (ms_per_step * 1e-3) / 1e12
            unit = "TFLOP/s"
        else:
            peak = peaks["hbm_gbs"]
            achieved = abytes / (ms_per_step * 1e-3) / 1e9
            unit = "GB/s"
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tpath):
            with open(tpath) as f:
                traffic = json.load(f).get(args.workload)
        line = {
            "metric": "quantized GEMM TFLOPS", "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": "fp4" if kind == "mxf4" else "fp8", "data": "synthetic",
            "config": {"workload": desc, "M_rank0": M, "N_rank0": N, "K": K, "groups_rank0": G if kind == "grouped" else 0,
                       "job_flops_per_step": flops_job, "sharding": sharding,
                       "l2": "operands + output exceed the 126 MB L2" if abytes > 126e6 else "fits in L2 (latency config)",
                       "clock_ramp_steps": ramp_steps,
                       "pct_of_published_dense_fp8_peak": round(100.0 * value / world / 4500.0, 2),
                       **({"pct_of_published_dense_fp4_peak": round(100.0 * value / world / 9000.0, 2)}
                          if kind == "mxf4" else {})},
            "roofline": {"bound": "tensor" if tensor_bound else "hbm", "achieved": achieved, "peak": peak, "unit": unit,
                         "frac": achieved / peak, "traffic": traffic, "peak_source": peaks["source"],
                         "algorithmic_bytes": abytes, "flops": flops},
            "e2e": {"value": flops_job / (e2e_ms["operands"] * 1e-3) / 1e12, "unit": "TFLOPS",
                    "h2d_bytes_per_step": h2d_bytes["operands"], "d2h_bytes_per_step": out_host.numel() * 2,
                    "ms_per_step": e2e_ms["operands"],
                    "inputs": "all operands of the contraction call (A, B, scales, bias/residual/group list) from "
                              "pinned host memory every step; bf16 result back to pinned host memory",
                    "pipeline": "3 streams, double buffers"},
            "e2e_fp32_activations": {"value": flops_job / (e2e_ms["fp32"] * 1e-3) / 1e12, "unit": "TFLOPS",
                                     "h2d_bytes_per_step": h2d_bytes["fp32"],
                                     "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": e2e_ms["fp32"],
                                     "inputs": "fp32 activations from pinned host memory, quantised on the device; "
                                               "weights resident"},
            "gpu_launches": launches_per_step * steps,
            "clocks": clocks,
            **({"gather": gather_info} if gather_info else {}),
            "device_status": status,
        }
        if world == 1 and not args.kernel_only:
            run, cpu_flops, sample = make_cpu_golden(args.workload)
            times = time_cpu_golden(run, 3)
            line["cpu_baseline"] = {"value": cpu_flops / float(np.mean(times)) / 1e12, "unit": "TFLOPS",
                                    "cores": len(os.sched_getaffinity(0)), "kind": "port",
                                    "sample": sample + f"; mean of 3 runs, {np.mean(times):.2f} s each"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--shard", default="weak", choices=["weak", "strong"],
                    help="with N GPUs: weak = every GPU runs the whole single-GPU problem on its own shard of a "
                         "gpus-times larger N (default); strong = the single-GPU problem itself is split (along N, or by "
                         "expert for the grouped workload)")
    ap.add_argument("--gather", default="none", choices=["none", "after", "overlapped", "peer", "fused"],
                    help="N > 1, MX workloads: also time the step followed by / overlapped with an all-gather of the output")
    ap.add_argument("--gather-chunks", type=int, default=4)
    ap.add_argument("--gather-gemm-sms", type=int, default=0,
                    help="overlapped gather: SMs the chunk GEMMs may use (0 = all); the rest stay free for NCCL's CTAs")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (used for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = min(args.steps, 20)
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
