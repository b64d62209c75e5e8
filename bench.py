#!/usr/bin/env python
"""Benchmark of the Blaze quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c3|c4|c5|c6]

Headline workload (the one the metric is quoted on): MXFP8 GEMM M=N=K=8192 with fused bf16 bias + GELU(tanh) and bf16
output, synthetic seeded inputs; one step = one acltensorContract call over that batch.

One GPU: the headline line also carries `workloads`, one entry per other configuration (FP8 per-group 256x512x1024,
W4A8 MX 4096x14336x4096, MoE grouped matmul, the decode shape at M = 16 / 64 / 128), each timed by the same CUDA-event
loop with its own roofline and clock record, plus `library_fp8` (the vendor library's MXFP8 GEMM on the same codes, a
yardstick only) and `sustained` (two seconds of back-to-back steps).

N GPUs (one process per GPU, launched by torch.distributed.run): the single-GPU problem itself is split - dense GEMMs
along N (every rank keeps A and owns a range of B's rows), the grouped matmul by expert, balanced by token count -
with no collective on the data path ("scaling": "strong").  `value` is the whole 8192^3 job's TFLOPS over the slowest
rank's time.  `strong` lists every split workload with its own N=1-equivalent time measured in the same run (all
ranks run the whole problem, slowest rank) and the resulting efficiency; `gather` times the split GEMM whose epilogue
also stores every tile into the peers' gathered outputs, beside GEMM-then-all-gather, and checks both give the same
bits.  `--shard weak` keeps the older form (every rank runs the whole problem on its own weights).

`value` = TFLOPS with quantized operands resident in HBM; `e2e` = the same metric through the acltensor* C API with
every operand of the call in pinned host memory at the start of each step and the bf16 result returned to it (copies
inside the timed region); `roofline` for the GEMM kernel; `cpu_baseline` = the reference-style CPU golden (de-quantise
to float32, np.matmul, epilogue, bf16) timed on this box's host cores on a bounded sample.

`--impl reference` times that CPU golden alone, on the same config and metric.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
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
    # the unscaled GEMMs of the widened surface (single GPU; no end-to-end or CPU legs)
    "a8w8": ("int8", 8192, 8192, 8192, "INT8 x INT8 GEMM 8192^3, de-quantised on store, half out"),
    "bf16": ("bf16", 8192, 8192, 8192, "bf16 x bf16 GEMM 8192^3, bf16 out"),
}
TENSOR_BOUND = ("mx", "mx4", "mxf4")
L2_BYTES = 126e6


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
    thread while a timed region runs."""

    def __init__(self, gpu_index, period_s=0.002):
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
            return self

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
        return self

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
    Returns (run, flops of the sample, description, fraction of the workload's flops the sample covers)."""
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
    if kind in TENSOR_BOUND:
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
    return run, flops, sample, flops / (2.0 * M * N * K)


def time_cpu_golden(run, repeats):
    run()                                            # warm-up (BLAS thread pool, page faults)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    return times


def headline_config(wl, M, N, K, G, world, sharding, extra=None):
    """The `config` object both arms print: same keys, so the two lines can be compared field by field."""
    kind = WORKLOADS[wl][0]
    cfg = {"workload": WORKLOADS[wl][4], "M": M, "N": N, "K": K, "groups": G if kind == "grouped" else 0,
           "n_gpus": world, "sharding": sharding}
    if extra:
        cfg.update(extra)
    return cfg


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, M, N, K, desc = WORKLOADS[args.workload]
    wl = args.workload
    cores = len(os.sched_getaffinity(0))
    run, flops, sample, fraction = make_cpu_golden(wl)
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
        "steps": len(times), "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 and args.shard == "strong" else "weak",
        "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
        "config": headline_config(wl, M, N, K, 128, args.gpus, "none: the CPU golden runs on rank 0's host cores",
                                  {"sample_fraction": fraction,
                                   "rate": "value is the rate of the sample (its flops / its time); one step covers "
                                           "sample_fraction of the workload's flops"}),
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------- GPU arm

class Env:
    """What every part of the GPU arm needs: modules, device, rank."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        from ops_tensor_b200 import host as H
        from ops_tensor_b200 import native, shard
        from ops_tensor_b200 import synthetic as o           # seeded input generators; the CPU oracle is not used here
        self.torch, self.dist, self.H, self.native, self.shard, self.o = torch, dist, H, native, shard, o
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        native.lib()                                     # fails loudly if the CUDA library is missing


class Case:
    """One workload instance resident on this rank's GPU: quantized operands, a plan, and `step()`."""

    def __init__(self, env, wl, M=None):
        torch, H, o, dev = env.torch, env.H, env.o, env.dev
        self.env, self.wl = env, wl
        kind, M0, N, K, desc = WORKLOADS[wl]
        M = M or M0
        self.kind, self.M, self.N, self.K, self.desc = kind, M, N, K, desc
        self.G = 128 if kind == "grouped" else 0
        cfg = int(wl[1])
        self.a_host = torch.from_numpy(o.normal_f32(cfg, 0, (M, K), 1.0)).pin_memory()
        self.a_dev = self.a_host.to(dev, non_blocking=True)
        sigma_b = 1.0 if kind in ("mx", "mxf4") else 0.02
        b_rows = self.G * N if kind == "grouped" else N
        w_dev = torch.from_numpy(o.normal_f32(cfg, 1, (b_rows, K), sigma_b)).to(dev)
        self.bias = self.residual = self.group_rows = None
        self.group_rows_host = None
        if kind in ("mx", "mxf4"):
            self.bias = torch.from_numpy(o.normal_f32(cfg, 2, (N,), 0.1)).to(dev).to(torch.bfloat16)   # nearest-even
        if kind == "fp8sk":
            self.residual = torch.from_numpy(o.normal_f32(cfg, 3, (M, N), 1.0)).to(dev).to(torch.bfloat16)
        self.a_dtype = H.R_4F_E2M1 if kind == "mxf4" else H.R_8F_E4M3
        self.b_dtype = H.R_8F_E4M3
        if kind in TENSOR_BOUND:
            self.b_dtype = H.R_8F_E4M3 if kind == "mx" else H.R_4F_E2M1
            self.mode_a = self.mode_b = H.SCALE_MX_E8M0_VEC32
            self.qb, self.sb = H.quantize(w_dev, self.mode_b, self.b_dtype)
        else:
            self.mode_a, self.mode_b = H.SCALE_FP32_1X128, H.SCALE_FP32_128X128
            if kind == "grouped":
                self.group_rows_host = o.moe_group_rows()
                self.group_rows = torch.from_numpy(self.group_rows_host).to(dev)
                self.qb = torch.empty((self.G, N, K), dtype=torch.uint8, device=dev)
                self.sb = torch.empty((self.G, K // 128, N // 128), dtype=torch.float32, device=dev)
                for g in range(self.G):
                    c, s = H.quantize(w_dev[g * N:(g + 1) * N], self.mode_b)
                    self.qb[g].copy_(c)
                    self.sb[g].copy_(s)
            else:
                self.qb, self.sb = H.quantize(w_dev, self.mode_b)
        del w_dev
        self.qa, self.sa = H.quantize(self.a_dev, self.mode_a, self.a_dtype)
        self.out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        self.plans = []
        self._finish()

    def _plan(self, b_is_static=True):
        H = self.env.H
        if self.kind in TENSOR_BOUND:
            p = H.Contraction(self.M, self.N, self.K, scale_mode_a=self.mode_a, scale_mode_b=self.mode_b,
                              a_dtype=self.a_dtype, b_dtype=self.b_dtype,
                              activation=H.OP_IDENTITY if self.kind == "mx4" else H.OP_GELU, bias=self.bias is not None,
                              b_is_static=b_is_static)
        else:
            p = H.Contraction(self.M, self.N, self.K, scale_mode_a=self.mode_a, scale_mode_b=self.mode_b,
                              groups=self.G, residual=self.residual is not None, b_is_static=b_is_static)
        self.plans.append(p)
        return p

    def _finish(self):
        """Plan, launch count, flops and bytes of the operands as they are now; operand sets for L2 rotation."""
        torch = self.env.torch
        self.plan = self._plan()
        if self.kind in TENSOR_BOUND:
            self.launches = 2                        # scale re-tile of A + GEMM (B's pre-pass is reused)
        else:
            self.launches = 1                        # the GEMM alone, stream-K fix-up included
        self.flops = 2.0 * self.M * self.N * self.K
        self.abytes = algorithmic_bytes(self.kind, self.M, self.N, self.K, self.G or 128)
        base = {"qa": self.qa, "sa": self.sa, "qb": self.qb, "sb": self.sb, "out": self.out, "residual": self.residual}
        self.sets = [base]
        if self.kind not in TENSOR_BOUND and self.abytes < 2 * L2_BYTES and self.wl != "c1":
            # HBM-bound workload whose operands would stay in the 126 MB L2 from one step to the next: rotate among
            # copies of every operand so that each step streams its bytes from HBM
            copies = min(24, int(math.ceil(2.2 * L2_BYTES / self.abytes)))
            for _ in range(copies - 1):
                self.sets.append({k: (v.clone() if v is not None else None) for k, v in base.items()})
        self._i = 0
        torch.cuda.synchronize()

    def step(self):
        s = self.sets[self._i % len(self.sets)]
        self._i += 1
        self.plan(s["qa"], s["sa"], s["qb"], s["sb"], s["out"], bias=self.bias, residual=s["residual"],
                  group_rows=self.group_rows)

    def l2_note(self):
        if len(self.sets) > 1:
            return f"rotates among {len(self.sets)} copies of every operand ({self.abytes * len(self.sets) / 1e6:.0f} MB)"
        if self.abytes > L2_BYTES:
            return "operands + output exceed the 126 MB L2"
        if self.kind in TENSOR_BOUND:
            return "operands + output fit in the 126 MB L2; the kernel is tensor-bound"
        return "fits in L2 (latency-bound configuration)"

    # ---- shards of this case (strong scaling): operands are slices of the full problem's device tensors ----------
    def n_split(self, world, rank):
        """This rank's column range of the same problem: rows [n0, n1) of B, of its scales, of bias and residual."""
        torch, shard = self.env.torch, self.env.shard
        n0, n1 = shard.n_shard(self.N, world, rank)
        c = object.__new__(Case)
        c.__dict__.update({k: v for k, v in self.__dict__.items() if k not in ("plans", "plan", "sets")})
        c.plans = []
        c.N = n1 - n0
        c.qb = self.qb[n0:n1]
        c.sb = self.sb[n0:n1] if self.kind in TENSOR_BOUND else self.sb[:, n0 // 128:-(-n1 // 128)].contiguous()
        c.bias = None if self.bias is None else self.bias[n0:n1].contiguous()
        c.residual = None if self.residual is None else self.residual[:, n0:n1].contiguous()
        c.out = torch.empty((self.M, c.N), dtype=torch.bfloat16, device=self.env.dev)
        c.columns = (n0, n1)
        c._finish()
        return c

    def expert_split(self, world, rank):
        """This rank's experts (or row ranges of oversized experts), dealt longest-first by token count."""
        torch, shard = self.env.torch, self.env.shard
        pieces = shard.plan_experts(self.group_rows_host, world)[rank]
        starts = np.concatenate([[0], np.cumsum(self.group_rows_host)])
        rows = np.concatenate([np.arange(starts[p.expert] + p.row_begin, starts[p.expert] + p.row_end) for p in pieces])
        idx = torch.from_numpy(rows).to(self.env.dev)
        experts = torch.tensor([p.expert for p in pieces], device=self.env.dev)
        c = object.__new__(Case)
        c.__dict__.update({k: v for k, v in self.__dict__.items() if k not in ("plans", "plan", "sets")})
        c.plans = []
        c.qa, c.sa = self.qa.index_select(0, idx), self.sa.index_select(0, idx)
        c.qb, c.sb = self.qb.index_select(0, experts), self.sb.index_select(0, experts)
        c.group_rows_host = np.array([p.rows for p in pieces], dtype=np.int64)
        c.group_rows = torch.from_numpy(c.group_rows_host).to(self.env.dev)
        c.G = len(pieces)
        c.M = int(c.group_rows_host.sum())
        c.out = torch.empty((c.M, self.N), dtype=torch.bfloat16, device=self.env.dev)
        c.a_host = self.a_host[torch.from_numpy(rows)].pin_memory()
        c.a_dev = c.a_host.to(self.env.dev)
        c._finish()
        return c

    def close(self):
        for p in self.plans:
            p.close()
        self.plans = []


def timed_loop(env, fn, n, after=None):
    """n calls of fn between two CUDA events on the current stream, barrier + synchronize on both sides; milliseconds,
    the largest over the ranks."""
    torch, dist = env.torch, env.dist
    if env.world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    if after is not None:
        after()
    e1.record()
    torch.cuda.synchronize()
    if env.world > 1:
        dist.barrier()
    return env.shard.max_over_ranks(e0.elapsed_time(e1), env.dev)


def graph_of(env, step, count):
    """`count` consecutive steps recorded into one CUDA graph (the launch path allocates nothing and never
    synchronises, so it can be captured); replaying it takes the host's per-call cost out of the timed region."""
    torch = env.torch
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=env.dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=side):
            for _ in range(count):
                step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    return g


GRAPH_BELOW_MS = [0.2]          # steps shorter than this are replayed from a CUDA graph (0 with --no-graph)


def measure(env, step, steps, warmup, min_region_ms=40.0, graph_below_ms=None):
    """Warm-up, clock ramp, then `steps` timed steps (more when the region would be too short for the clock sampler to
    see it).  Steps shorter than `graph_below_ms` are replayed from a CUDA graph of several steps: with eight processes
    on one host the Python call path (tens of microseconds) would otherwise be what is timed.
    Returns (ms per step, steps timed, clock record, info)."""
    torch = env.torch
    if graph_below_ms is None:
        graph_below_ms = GRAPH_BELOW_MS[0]
    step()                                           # first call: module load, workspace allocation
    torch.cuda.synchronize()
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0.record()
    for _ in range(warmup):
        step()
    w1.record()
    torch.cuda.synchronize()
    per_step = max(w0.elapsed_time(w1) / max(warmup, 1), 1e-3)
    if env.world > 1:
        per_step = env.shard.max_over_ranks(per_step, env.dev)     # every rank takes the same decisions below
    n = steps
    if per_step * steps < min_region_ms:
        n = min(20000, int(math.ceil(min_region_ms / per_step)))
    fn, per_call, launch = step, 1, "one host call per step"
    if per_step < graph_below_ms:
        per_call = next(c for c in (25, 20, 10, 5, 4, 2, 1) if steps % c == 0) if n == steps else 25
        n = -(-n // per_call) * per_call
        graph = graph_of(env, step, per_call)
        fn = graph.replay
        launch = f"CUDA graph of {per_call} steps, replayed {n // per_call} times"
    # A short step (tens of microseconds) finishes its warm-up before the SM clock has left its idle state: keep
    # stepping, untimed, until the GPU has been busy for about 20 ms.  Long steps (C2) get exactly `warmup` steps.
    ramp_steps = 0
    if per_step * warmup < 1.0:
        ramp_steps = min(5000, int(20.0 / per_step))
        for _ in range(-(-ramp_steps // per_call)):
            fn()
        torch.cuda.synchronize()
    sampler = ClockSampler(env.local_rank).start() if env.rank == 0 else None
    if sampler is not None:
        time.sleep(0.01)
    total_ms = timed_loop(env, fn, n // per_call)
    clocks = sampler.stop() if sampler is not None else None
    return total_ms / n, n, clocks, {"clock_ramp_steps": ramp_steps, "launch": launch}


def traffic_of(name):
    """DRAM bytes of one launch of the workload's dominant kernel, from the committed ncu summaries (or None)."""
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(tpath):
        return None
    with open(tpath) as f:
        return json.load(f).get(name)


def roofline_of(case, ms, total_ms, peaks):
    tensor_bound = case.kind in TENSOR_BOUND
    if tensor_bound:
        # FP8 operands run at twice the bf16 MMA rate; the loop is timed back to back, so the burst figure applies
        # to short runs and the sustained one to runs of a second or more
        base = peaks["bf16_tflops_sustained"] if total_ms > 1000.0 else peaks["bf16_tflops"]
        peak = (4.0 if case.kind == "mxf4" else 2.0) * base      # FP4 x FP4 (kind::mxf4) runs at twice the FP8 rate
        achieved = case.flops / (ms * 1e-3) / 1e12
        unit = "TFLOP/s"
    else:
        peak = peaks["hbm_gbs"]
        achieved = case.abytes / (ms * 1e-3) / 1e9
        unit = "GB/s"
    traffic = traffic_of(case.wl) if case.M == WORKLOADS[case.wl][1] and case.N == WORKLOADS[case.wl][2] else None
    return {"bound": "tensor" if tensor_bound else "hbm", "achieved": achieved, "peak": peak, "unit": unit,
            "frac": achieved / peak, "traffic": traffic, "peak_source": peaks["source"],
            "peak_is": ("2 x measured bf16 tensor peak (no FP8 entry in MEASURED_PEAKS.json)" if tensor_bound
                        else "measured HBM copy bandwidth"),
            "algorithmic_bytes": case.abytes, "flops": case.flops}


def workload_entry(env, name, case, steps, warmup, peaks):
    ms, n, clocks, info = measure(env, case.step, steps, warmup)
    tf = case.flops / (ms * 1e-3) / 1e12
    return {"workload": name, "description": case.desc, "M": case.M, "N": case.N, "K": case.K, "groups": case.G,
            "ms_per_step": ms, "steps": n, "value": tf, "unit": "TFLOPS",
            "pct_of_published_dense_fp8_peak": round(100.0 * tf / 4500.0, 2),
            "roofline": roofline_of(case, ms, ms * n, peaks), "l2": case.l2_note(), "gpu_launches": case.launches * n,
            "clocks": clocks, **info}


def dense_entry(env, label, dtype_name, M, N, K, steps, warmup, peaks):
    """One of the unscaled GEMMs of the widened surface (INT8 A8W8 with per-tensor de-quantisation to half, or bf16
    with a bf16 result) on seeded random operands, timed like the other workloads; tensor-bound, so the roofline is
    the measured bf16 tensor peak (twice that for INT8, which runs at the 8-bit rate)."""
    torch, native, dev = env.torch, env.native, env.dev
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    if dtype_name == "int8":
        a = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev, generator=g)
        b = torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev, generator=g)
        scale = torch.full((1,), 0.01, dtype=torch.float32, device=dev)
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
        kw = dict(scale_a=scale, scale_b=scale)
        abytes, rate = M * K + N * K + 2 * M * N + 8, 2.0
        what = "INT8 x INT8 GEMM, int32 sums de-quantised on store (per-tensor scale), half out"
    else:
        a = torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)
        b = (torch.randn((N, K), device=dev, generator=g) * 0.05).to(torch.bfloat16)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        kw = {}
        abytes, rate = 2 * (M * K + N * K + M * N), 1.0
        what = "bf16 x bf16 GEMM, float32 accumulation, bf16 out"

    def step():
        native.dense_gemm(a, b, out=out, **kw)

    ms, n, clocks, info = measure(env, step, steps, warmup)
    flops = 2.0 * M * N * K
    tf = flops / (ms * 1e-3) / 1e12
    base = peaks["bf16_tflops_sustained"] if ms * n > 1000.0 else peaks["bf16_tflops"]
    return {"workload": label, "description": f"{what}, {M}x{N}x{K}", "M": M, "N": N, "K": K, "groups": 0,
            "ms_per_step": ms, "steps": n, "value": tf, "unit": "TFLOPS" if dtype_name != "int8" else "TOPS",
            "roofline": {"bound": "tensor", "achieved": tf, "peak": rate * base, "unit": "TFLOP/s", "frac": tf / (rate * base),
                         "traffic": traffic_of(label.split("_")[0]) if (M, N, K) == (8192, 8192, 8192) else None,
                         "peak_source": peaks["source"],
                         "peak_is": ("2 x " if rate == 2.0 else "") + "measured bf16 tensor peak",
                         "algorithmic_bytes": abytes, "flops": flops},
            "l2": "operands + output exceed the 126 MB L2" if abytes > L2_BYTES else "fits in L2",
            "gpu_launches": n, "clocks": clocks, **info}


def library_mxfp8(env, case, steps):
    """The vendor library's MXFP8 GEMM (torch._scaled_mm with E8M0 scales per 32 K) on this case's codes and scales:
    a yardstick beside our kernel, never part of the product path.  No bias or GELU: the library call has neither."""
    torch = env.torch
    if not hasattr(torch, "float8_e8m0fnu") or case.kind != "mx":
        return None

    def library_layout(scales):
        rows, groups = scales.shape
        t = scales.view(rows // 128, 4, 32, groups // 4, 4)
        return t.permute(0, 3, 2, 1, 4).contiguous().view(-1).view(torch.float8_e8m0fnu)

    try:
        a = case.qa.view(torch.float8_e4m3fn)
        b = case.qb.view(torch.float8_e4m3fn).t()
        sa, sb = library_layout(case.sa), library_layout(case.sb)

        def run():
            return torch._scaled_mm(a, b, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
        for _ in range(5):
            run()
        torch.cuda.synchronize()
        sampler = ClockSampler(env.local_rank).start()
        ms = timed_loop(env, run, steps) / steps
        clocks = sampler.stop()
    except Exception as exc:                         # this torch / cuBLASLt has no block-scaled FP8 GEMM
        return {"unavailable": repr(exc)[:200]}
    return {"what": "torch._scaled_mm, E4M3 x E4M3 with E8M0 scales per 32 K, bf16 out, same codes and scales; library "
                    "call timed as a yardstick only",
            "ms_per_step": ms, "value": case.flops / (ms * 1e-3) / 1e12, "unit": "TFLOPS", "steps": steps,
            "clocks": clocks}


def sustained_run(env, case, seconds=2.0):
    """Back-to-back steps for about `seconds`: the power-capped steady state, with time x median SM clock beside it."""
    torch = env.torch
    case.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        case.step()
    e1.record()
    torch.cuda.synchronize()
    n = max(20, int(seconds * 1e3 / max(e0.elapsed_time(e1) / 10, 1e-3)))
    sampler = ClockSampler(env.local_rank, 0.005).start()
    total = timed_loop(env, case.step, n)
    clocks = sampler.stop()
    ms = total / n
    out = {"seconds": total / 1e3, "steps": n, "ms_per_step": ms, "value": case.flops / (ms * 1e-3) / 1e12,
           "unit": "TFLOPS", "clocks": clocks}
    if clocks and clocks.get("sm_mhz"):
        out["ms_x_sm_ghz"] = ms * clocks["sm_mhz"] / 1e3           # SM cycles per step, in millions
    return out


class E2E:
    """End-to-end steps of one case through the public API with HOST buffers.  Two pipelines:
      "operands": every operand the contraction call takes (A codes and scales, B codes and scales, bias, residual,
                  group list) starts each step in pinned host memory - the call the reference's operator API makes,
                  with nothing assumed resident; a plan that does not treat B as static runs it;
      "fp32":     this step's fp32 activations start in pinned host memory and are quantised on the device first
                  (weights resident, as in serving).
    Both return the bf16 result to pinned host memory every step.  Copies in, compute and copies out run on three
    streams over double buffers, so the copies of neighbouring steps overlap; every step still moves all of its
    bytes inside the timed region."""

    def __init__(self, env, case):
        torch, dev = env.torch, env.dev
        self.env, self.case = env, case
        self.s_in, self.s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.out2 = [case.out, torch.empty_like(case.out)]
        self.out_host2 = [torch.empty(case.out.shape, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        self.ev = {k: [torch.cuda.Event() for _ in range(2)] for k in ("in", "consumed", "computed", "out")}
        self.counter = 0
        self.mode = "operands"
        dev_ops = {"a": case.qa, "sa": case.sa, "b": case.qb, "sb": case.sb}
        for k, v in (("bias", case.bias), ("residual", case.residual), ("group_rows", case.group_rows)):
            if v is not None:
                dev_ops[k] = v
        self.host_ops = {k: v.cpu().pin_memory() for k, v in dev_ops.items()}
        self.dev_ops2 = [dev_ops, {k: torch.empty_like(v) for k, v in dev_ops.items()}]
        self.a_dev2 = [case.a_dev, torch.empty_like(case.a_dev)]
        self.plan = case._plan(b_is_static=False)      # every operand arrives from the host each step: nothing is static
        self.h2d = {"operands": sum(v.numel() * v.element_size() for v in self.host_ops.values()),
                    "fp32": case.a_host.numel() * 4}
        self.d2h = case.out.numel() * 2

    def step(self):
        torch, H, case = self.env.torch, self.env.H, self.case
        i = self.counter
        self.counter += 1
        b = i & 1
        ev = self.ev
        main = torch.cuda.current_stream()
        with torch.cuda.stream(self.s_in):
            if i >= 2:
                self.s_in.wait_event(ev["consumed"][b])       # the buffers' previous contents have been consumed
            if self.mode == "operands":
                for k, v in self.host_ops.items():
                    self.dev_ops2[b][k].copy_(v, non_blocking=True)
            else:
                self.a_dev2[b].copy_(case.a_host, non_blocking=True)
            ev["in"][b].record(self.s_in)
        main.wait_event(ev["in"][b])
        if i >= 2:
            main.wait_event(ev["out"][b])                     # the previous result in this buffer has left the device
        if self.mode == "operands":
            d = self.dev_ops2[b]
            self.plan(d["a"], d["sa"], d["b"], d["sb"], self.out2[b], bias=d.get("bias"), residual=d.get("residual"),
                      group_rows=d.get("group_rows"))
            ev["consumed"][b].record(main)
        else:
            qa2, sa2 = H.quantize(self.a_dev2[b], case.mode_a, case.a_dtype)
            ev["consumed"][b].record(main)
            case.plan(qa2, sa2, case.qb, case.sb, self.out2[b], bias=case.bias, residual=case.residual,
                      group_rows=case.group_rows)
        ev["computed"][b].record(main)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(ev["computed"][b])
            self.out_host2[b].copy_(self.out2[b], non_blocking=True)
            ev["out"][b].record(self.s_out)

    def drain(self):
        main = self.env.torch.cuda.current_stream()
        for b in range(2):
            main.wait_event(self.ev["out"][b])

    def run(self, steps):
        torch = self.env.torch
        ms = {}
        for mode in ("operands", "fp32"):
            self.mode = mode
            self.counter = 0
            for _ in range(2):
                self.step()
            torch.cuda.synchronize()
            self.counter = 0
            ms[mode] = timed_loop(self.env, self.step, steps, after=self.drain) / steps   # last copies back included
        return ms


def gather_leg(env, full, part, steps, warmup, gemm_only_ms):
    """The split GEMM whose consumer needs the whole matrix on every rank: all-gather after the GEMM, against the GEMM
    whose epilogue stores every tile into the peers' gathered buffers as well (peer stores only; no load ever reads
    another GPU's memory).  Both must give the same bits."""
    torch, dist, native, shard = env.torch, env.dist, env.native, env.shard
    world, rank, dev = env.world, env.rank, env.dev
    M, N = part.M, part.N
    whole = torch.empty((world, M, N), dtype=torch.bfloat16, device=dev)

    def step_after():
        part.step()
        dist.all_gather_into_tensor(whole.view(world * M, N), part.out)

    for _ in range(warmup):
        step_after()
    after_ms = timed_loop(env, step_after, steps) / steps
    info = {"workload": part.wl, "M": M, "N_per_rank": N, "K": part.K, "gemm_only_ms": gemm_only_ms,
            "nccl_after_ms": after_ms, "gathered_bytes_per_rank": (world - 1) * M * N * 2}
    ok = torch.ones(1, device=dev)
    fused = None
    try:
        fused = shard.PeerGatherBuffers(M, N, world, rank, 1, torch.bfloat16, dev, 256)
    except Exception as exc:                             # no symmetric memory on this box
        info["fused_unavailable"] = repr(exc)[:200]
        ok.zero_()
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)            # every rank takes the same branch
    if ok.item() == 0 or fused is None:
        return info
    kw = dict(b_elem=native.ELEM_E4M3 if part.kind == "mx" else native.ELEM_E2M1,
              a_elem=native.ELEM_E2M1 if part.kind == "mxf4" else native.ELEM_E4M3, bias=part.bias,
              activation=native.ACT_IDENTITY if part.kind == "mx4" else native.ACT_GELU_TANH)
    peers = [s for s in fused.peer_slots[0] if s is not None]
    probe = native.mx_gemm_args(part.qa, part.sa, part.qb, part.sb, fused.gathered[0][rank], peer_outs=peers, **kw)
    ws = torch.empty(max(native.mx_gemm_workspace_bytes(probe), 256), dtype=torch.uint8, device=dev)
    calls = [0]

    def run_fused(out_, peer_outs):
        native.mx_gemm(part.qa, part.sa, part.qb, part.sb, out=out_, workspace=ws, peer_outs=peer_outs,
                       reuse_b_prepass=calls[0] > 0, **kw)
        calls[0] += 1

    def step_fused():
        shard.gemm_gather_fused(run_fused, fused)

    def step_fused_allreduce():
        shard.gemm_gather_fused(run_fused, fused, signal="allreduce")

    for _ in range(warmup):
        step_fused_allreduce()
    torch.cuda.synchronize()
    fused_allreduce_ms = timed_loop(env, step_fused_allreduce, steps) / steps
    for _ in range(warmup):
        step_fused()
    torch.cuda.synchronize()
    fused_ms = timed_loop(env, step_fused, steps) / steps
    step_after()
    step_fused()
    torch.cuda.synchronize()
    same = torch.equal(fused.gathered[0].view(torch.int16), whole.view(torch.int16))
    flag = torch.tensor([1.0 if same else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    info.update(fused_ms=fused_ms, fused_with_allreduce_signal_ms=fused_allreduce_ms, bit_equal=bool(flag.item() == 1.0),
                device_status=env.H.device_status(),
                how="epilogue TMA-stores every tile to the local and the peers' gathered buffers (symmetric memory); "
                    "closing signal: a step counter stored into the peers' flag arrays and a bounded wait on this GPU's own "
                    "(blazePeerSignal; peer stores and local loads only); fused_with_allreduce_signal_ms uses a "
                    "one-element all-reduce instead")
    return info


def decode_gather_leg(env, part, steps, warmup):
    """The split decode GEMM (C5, FP8 kernel) with the whole output on every rank: the shape where the closing signal's
    cost decides.  GEMM alone, GEMM + NCCL all-gather, and the fused form closed by the flag signal or by a one-element
    all-reduce; all must give the same bits."""
    torch, dist, native, shard = env.torch, env.dist, env.native, env.shard
    world, rank, dev = env.world, env.rank, env.dev
    M, N = part.M, part.N
    whole = torch.empty((world, M, N), dtype=torch.bfloat16, device=dev)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    try:
        fused = shard.PeerGatherBuffers(M, N, world, rank, 1, torch.bfloat16, dev, 128)
        ok = torch.ones(1, device=dev)
    except Exception as exc:                             # no symmetric memory on this box
        fused, ok = None, torch.zeros(1, device=dev)
        why = repr(exc)[:200]
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if ok.item() == 0 or fused is None:
        return {"workload": part.wl, "fused_unavailable": why if fused is None else "a peer has no symmetric memory"}

    def gemm(o, peers=None):
        native.fp8_gemm(part.qa, part.sa, part.qb, part.sb, out=o, residual=part.residual, peer_outs=peers)

    def step_after():
        gemm(out)
        dist.all_gather_into_tensor(whole.view(world * M, N), out)

    legs = {"gemm_only_ms": lambda: gemm(out), "nccl_after_ms": step_after,
            "fused_ms": lambda: shard.gemm_gather_fused(gemm, fused),
            "fused_with_allreduce_signal_ms": lambda: shard.gemm_gather_fused(gemm, fused, signal="allreduce")}
    info = {"workload": part.wl, "M": M, "N_per_rank": N, "K": part.K, "gathered_bytes_per_rank": (world - 1) * M * N * 2}
    n = max(steps, 100)
    for key, fn in legs.items():
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        info[key] = timed_loop(env, fn, n) / n
    step_after()
    shard.gemm_gather_fused(gemm, fused)
    torch.cuda.synchronize()
    same = torch.equal(fused.gathered[0].view(torch.int16), whole.view(torch.int16))
    flag = torch.tensor([1.0 if same else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    info.update(bit_equal=bool(flag.item() == 1.0), device_status=env.H.device_status(), steps=n,
                how="FP8 kernel: tiled output copies to D and, through a tensor map per peer, to every peer's gathered "
                    "buffer; closing signal blazePeerSignal")
    return info


def gpu_arm(args):
    env = Env()
    torch, dist, H = env.torch, env.dist, env.H
    world, rank = env.world, env.rank
    peaks = measured_peaks()
    steps, warmup = args.steps, max(args.warmup, 3)
    wl = args.workload
    strong = args.shard == "strong" and world > 1

    if WORKLOADS[wl][0] in ("int8", "bf16"):
        kind, M, N, K, desc = WORKLOADS[wl]
        e = dense_entry(env, wl, kind, M, N, K, steps, warmup, peaks)
        if rank == 0:
            print(json.dumps({"metric": "quantized GEMM TFLOPS", "value": e["value"], "unit": "TFLOPS", "n_gpus": 1,
                              "steps": e["steps"], "warmup": warmup, "ms_per_step": e["ms_per_step"],
                              "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                              "dtype": "int8" if kind == "int8" else "bf16", "data": "synthetic",
                              "config": headline_config(wl, M, N, K, 0, 1, "single GPU", {"l2": e["l2"], "launch": e["launch"]}),
                              "roofline": e["roofline"], "gpu_launches": e["gpu_launches"], "clocks": e["clocks"],
                              "device_status": H.device_status()}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    full = Case(env, wl)
    if not strong and world > 1:
        # weak form: every rank runs the whole problem on weights of its own (seeded by rank): N replicas
        pass
    case = full
    sharding = "single GPU"
    extra = {}
    strong_list = []
    if strong:
        case = full.expert_split(world, rank) if full.kind == "grouped" else full.n_split(world, rank)
        sharding = (f"the {WORKLOADS[wl][4]} problem split over {world} GPUs: "
                    + ("experts dealt by token count (longest first)" if full.kind == "grouped"
                       else "B's rows (output columns) in equal ranges, A replicated")
                    + ", no collective on the data path")
    elif world > 1:
        sharding = (f"{world} replicas: every GPU runs the whole problem (N-shards of a {world} times wider weight), no "
                    "collective; see --shard strong for the split of the problem itself")

    ms_per_step, n_timed, clocks, info = measure(env, case.step, steps, warmup, min_region_ms=0.0)
    total_ms = ms_per_step * n_timed
    flops_job = full.flops * (world if (world > 1 and not strong) else 1)

    if strong:
        # the same run's N=1-equivalent: every rank runs the whole problem, slowest rank counts
        for name in ([wl] + [w for w in ("c2", "c3", "c4", "c5") if w != wl] if not args.kernel_only else [wl]):
            f = full if name == wl else Case(env, name)
            p = case if name == wl else (f.expert_split(world, rank) if f.kind == "grouped" else f.n_split(world, rank))
            t_full, n1, clk1, info1 = measure(env, f.step, steps, warmup)
            # (the headline's own loop is exactly `steps` long; this one runs long enough for the clock sampler)
            t_part, nP, clkP, infoP = measure(env, p.step, steps, warmup)
            loads = None
            if f.kind == "grouped":
                loads = env.shard.plan_loads(env.shard.plan_experts(f.group_rows_host, world))
            strong_list.append({
                "workload": name, "description": f.desc, "split": "experts by token count" if f.kind == "grouped" else "N",
                "ms_per_step": t_part, "steps": nP, "value": f.flops / (t_part * 1e-3) / 1e12, "unit": "TFLOPS",
                "single_gpu_ms_per_step": t_full, "efficiency": t_full / (world * t_part),
                "rank0_shape": {"M": p.M, "N": p.N, "K": p.K, "groups": p.G},
                **({"tokens_per_rank": loads} if loads else {}),
                "l2": p.l2_note(), "launch": infoP["launch"], "single_gpu_launch": info1["launch"],
                "clocks": clkP, "single_gpu_clocks": clk1})
            if name != wl:
                p.close()
                f.close()
                del p, f
                torch.cuda.empty_cache()

    gather_info = None
    gather_decode = None
    if strong and full.kind in TENSOR_BOUND and not args.kernel_only and args.gather != "none":
        gather_info = gather_leg(env, full, case, max(5, min(steps, 50)), warmup, ms_per_step)
        # and the decode shape, where the closing signal's cost decides
        c5_full = Case(env, "c5")
        c5_part = c5_full.n_split(world, rank)
        gather_decode = decode_gather_leg(env, c5_part, steps, warmup)
        c5_part.close()
        c5_full.close()
        del c5_part, c5_full
        torch.cuda.empty_cache()

    e2e_ms = None
    e2e = None
    if not args.kernel_only:
        e2e = E2E(env, case)
        e2e_ms = e2e.run(max(4, min(steps, 20)))

    workloads = []
    library = sustained = None
    if world == 1 and not args.kernel_only and wl == "c2":
        library = library_mxfp8(env, full, max(5, min(steps, 50)))
        for name, m_rows in (("c1", None), ("c3", None), ("c4", None), ("c5", 16), ("c5", 64), ("c5", 128)):
            c = Case(env, name, m_rows)
            label = name if m_rows is None else f"{name}_m{m_rows}"
            workloads.append(workload_entry(env, label, c, steps, warmup, peaks))
            c.close()
            del c
            torch.cuda.empty_cache()
        # beyond the five configurations: the unscaled GEMMs the same API now serves
        workloads.append(dense_entry(env, "a8w8_8192", "int8", 8192, 8192, 8192, steps, warmup, peaks))
        workloads.append(dense_entry(env, "bf16_8192", "bf16", 8192, 8192, 8192, steps, warmup, peaks))
        sustained = sustained_run(env, full)           # last: it leaves the GPU at its power cap
    status = H.device_status()

    if rank == 0:
        value = flops_job / (ms_per_step * 1e-3) / 1e12
        roof = roofline_of(case, ms_per_step, total_ms, peaks)
        line = {
            "metric": "quantized GEMM TFLOPS", "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": n_timed,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if strong or world == 1 else "weak",
            "vs_baseline": None, "dtype": "fp4" if full.kind == "mxf4" else "fp8", "data": "synthetic",
            "config": headline_config(wl, full.M, full.N, full.K, full.G, world, sharding, {
                "rank0_shape": {"M": case.M, "N": case.N, "K": case.K, "groups": case.G},
                "job_flops_per_step": flops_job, "l2": case.l2_note(), **info,
                "pct_of_published_dense_fp8_peak": round(100.0 * value / world / 4500.0, 2),
                **({"pct_of_published_dense_fp4_peak": round(100.0 * value / world / 9000.0, 2)}
                   if full.kind == "mxf4" else {})}),
            "roofline": roof,
            "gpu_launches": case.launches * n_timed,
            "clocks": clocks,
            "device_status": status,
        }
        if strong_list and (not clocks or clocks.get("samples", 0) < 3):
            # the headline region is too short for the sampler: the same step's longer loop in `strong` has the record
            line["clocks"] = dict(strong_list[0]["clocks"] or {}, note="sampled during the longer loop of strong[0]")
        if e2e_ms is not None:
            line["e2e"] = {"value": flops_job / (e2e_ms["operands"] * 1e-3) / 1e12, "unit": "TFLOPS",
                           "h2d_bytes_per_step": e2e.h2d["operands"], "d2h_bytes_per_step": e2e.d2h,
                           "ms_per_step": e2e_ms["operands"],
                           "inputs": "all operands of the contraction call (A, B, scales, bias/residual/group list) "
                                     "from pinned host memory every step; bf16 result back to pinned host memory",
                           "pipeline": "3 streams, double buffers"}
            line["e2e_fp32_activations"] = {"value": flops_job / (e2e_ms["fp32"] * 1e-3) / 1e12, "unit": "TFLOPS",
                                            "h2d_bytes_per_step": e2e.h2d["fp32"], "d2h_bytes_per_step": e2e.d2h,
                                            "ms_per_step": e2e_ms["fp32"],
                                            "inputs": "fp32 activations from pinned host memory, quantised on the "
                                                      "device; weights resident"}
        if workloads:
            line["workloads"] = workloads
        if library:
            line["library_fp8"] = library
        if sustained:
            line["sustained"] = sustained
        if strong_list:
            line["strong"] = strong_list
        if gather_info:
            line["gather"] = gather_info
        if gather_decode:
            line["gather_decode"] = gather_decode
        if world == 1 and not args.kernel_only:
            run, cpu_flops, sample, fraction = make_cpu_golden(wl)
            times = time_cpu_golden(run, 3)
            line["cpu_baseline"] = {"value": cpu_flops / float(np.mean(times)) / 1e12, "unit": "TFLOPS",
                                    "cores": len(os.sched_getaffinity(0)), "kind": "port", "sample_fraction": fraction,
                                    "sample": sample + f"; mean of 3 runs, {np.mean(times):.2f} s each"}
        print(json.dumps(line), flush=True)
    if e2e is not None:
        del e2e
    case.close()
    if case is not full:
        full.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--shard", default="strong", choices=["weak", "strong"],
                    help="with N GPUs: strong = the single-GPU problem itself is split (along N, or by expert for the "
                         "grouped workload; default); weak = every GPU runs the whole problem (N replicas)")
    ap.add_argument("--gather", default="fused", choices=["none", "fused"],
                    help="N > 1, MX workloads: also time the split GEMM with its output gathered on every rank")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every step from the host even when it is short (profiler captures see plain launches)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the headline loop (used for profiler captures): no end-to-end, CPU or other-workload legs")
    args = ap.parse_args()
    if args.no_graph:
        GRAPH_BELOW_MS[0] = 0.0
    if args.impl == "reference":
        args.steps = min(args.steps, 20)
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
