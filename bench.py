#!/usr/bin/env python
"""Benchmark of the matmul hot path through the C ABI of libnova_b200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

A step is ONE pass of the contraction over one batch of seeded synthetic input.  The default workload
is the f16 batch_matmul configuration (batch 32 of 1024^3, fp32 accumulation, f16 output); the other
configurations are selectable with --workload.  Inputs are resident in HBM for `value`; `e2e` runs the
same contraction through nova_b200_gemm_host with pinned HOST buffers (H2D + kernel + D2H per step).
With N > 1 (torchrun, one rank per GPU) the batch index is sharded across ranks with no data-path
collective: every rank owns a full per-GPU batch (weak scaling) and the slowest rank sets the time.

`--impl reference` times the reference's own CPU lowering of the same contraction — the single-threaded
i/j/k loop nest its CPU pipeline emits, restated in oracle/nova_oracle.c — on this machine's host cores,
on a bounded row sample of the workload.  That is a reported baseline, not the target.

Rank 0 prints exactly one JSON line.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# name -> (description, dtype_ab, dtype_c, batch, M, N, K, epilogue)
WORKLOADS = {
    "c1": ("nova.matmul f32 512x512x512 (3xTF32)", "f32", "f32", 1, 512, 512, 512, None),
    "c2": ("linalg.batch_matmul f16 B=32 M=N=K=1024, fp32 accumulate, f16 out", "f16", "f16", 32, 1024, 1024, 1024, None),
    "c3": ("linear bf16 X[8192,4096] W[4096,11008] + bias, GELU(tanh), bf16 out", "bf16", "bf16", 1, 8192, 11008, 4096,
           "bias_gelu"),
    "c4": ("batch_matmul f16 Q[256,2048,128] K^T[256,128,2048], f16 out", "f16", "f16", 256, 2048, 2048, 128, None),
    "c4s": ("batch_matmul f16 Q[32,2048,128] K^T[32,128,2048] (C4 at one eighth of the batch, profiling-sized)", "f16", "f16", 32, 2048,
            2048, 128, None),
    "c5a": ("GEMM bf16 16384^3", "bf16", "bf16", 1, 16384, 16384, 16384, None),
    "c5b": ("GEMM bf16 ragged 1000x1000x999", "bf16", "bf16", 1, 1000, 1000, 999, None),
    "c5c": ("GEMM bf16 ragged 4095x11007x4097", "bf16", "bf16", 1, 4095, 11007, 4097, None),
}
# DRAM bytes one launch moves according to ncu (dram__bytes_read.sum + dram__bytes_write.sum), per workload;
# see profiles/.  None where no capture exists.
NCU_TRAFFIC_BYTES = {
    "c2": 173.7e6,      # 134.3 MB read + 39.4 MB written (part of the 67 MB output is still in L2 at kernel end)
    "c3": 468.5e6,      # 308.0 MB read + 160.5 MB written
    "c4": 8 * 243.4e6,  # captured on 32 of the 256 batches (c4s), scaled by 8: traffic is proportional to batches
    "c5c": 207.7e6,     # the contraction kernel: 140.2 MB read + 67.5 MB written (the re-pitch copy before it: 203.8 MB)
    # row kernels (reads match the inputs exactly; part of each output is still in L2 when the kernel ends)
    "ln": 92.3e6, "ln_bwd": 176.0e6, "softmax": 489.8e6, "sce": 3246.0e6, "sce_bwd": 3252.9e6, "gather": 209.2e6,
}


def load_peaks():
    path = os.path.join(HERE, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def algorithmic(w):
    _, dab, dc, B, M, N, K, epi = WORKLOADS[w]
    es = 4 if dab == "f32" else 2
    os_ = 4 if dc == "f32" else 2
    flops = 2.0 * B * M * N * K
    byts = es * B * (M * K + K * N) + os_ * B * M * N + (os_ * N if epi else 0)
    return flops, byts


def make_inputs_np(w, seed):
    """Seeded synthetic inputs with the configuration's shapes and distributions (numpy, storage bits)."""
    import numpy as np
    from oracle import oracle as O
    _, dab, dc, B, M, N, K, epi = WORKLOADS[w]
    rng = np.random.default_rng(seed)
    if w in ("c1", "c5a", "c5b", "c5c"):
        a = rng.uniform(-1, 1, (B, M, K)).astype(np.float32)
        b = rng.uniform(-1, 1, (B, K, N)).astype(np.float32)
    elif w == "c2":
        a = (rng.normal(size=(B, M, K)) / np.sqrt(K)).astype(np.float32)
        b = (rng.normal(size=(B, K, N)) / np.sqrt(K)).astype(np.float32)
    elif w == "c3":
        a = rng.normal(size=(B, M, K)).astype(np.float32)
        b = (rng.normal(size=(B, K, N)) * 0.02).astype(np.float32)
    else:
        a = rng.normal(size=(B, M, K)).astype(np.float32)
        b = rng.normal(size=(B, K, N)).astype(np.float32)
    bias = (rng.normal(size=N) * 0.02).astype(np.float32) if epi else None
    return O.to_bits(a, dab), O.to_bits(b, dab), (O.to_bits(bias, dc) if bias is not None else None)


# ---------------------------------------------------------------------------------------------- reference arm

def run_reference(args):
    """The reference's CPU path (restated): scalar i/j/k nest, C re-loaded every k, k unrolled x8, ONE thread
    (its pipeline has no OpenMP/async lowering: lib/Pipeline/Pipeline.cpp:135,157-165)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import numpy as np
    from oracle import oracle as O
    w = args.workload
    if w not in WORKLOADS:
        raise SystemExit("--impl reference times the contraction workloads only")
    desc, dab, dc, B, M, N, K, epi = WORKLOADS[w]
    # a bounded sample: one batch (c4: narrow K makes rows cheap) and a row slice sized for ~0.3 s per step
    rows = max(1, min(M, int(2.0e8 / (2.0 * N * K))))
    a, b, bias = make_inputs_np_small(w, rows)
    flops = 2.0 * rows * N * K
    def step():
        O.gemm_scalar_rows(a, b, dtype_in=dab, dtype_out=dc, bias=bias, act="gelu_tanh" if epi else "none",
                           row_begin=0, row_end=rows)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    tflops = flops / (ms * 1e-3) / 1e12
    sample = f"rows 0..{rows - 1} of the {B * M} (batch*M) output rows per step, full N and K; rate extrapolates linearly"
    line = {
        "impl": "reference", "metric": "batch-matmul/linear TFLOPS", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": dab, "data": "synthetic (seeded)",
        "config": {"workload": f"{w}: {desc}", "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": 1, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference = C restatement of the Nova CPU pipeline's single-threaded loop nest (oracle/nova_oracle.c); "
                "the MLIR reference itself cannot be built without LLVM 21",
    }
    print(json.dumps(line), flush=True)
    return 0


def make_inputs_np_small(w, rows):
    """First `rows` of the (batch*M) rows of the workload's A, and the matching B (first batch), seeded."""
    import numpy as np
    from oracle import oracle as O
    _, dab, dc, B, M, N, K, epi = WORKLOADS[w]
    rng = np.random.default_rng(1234)
    rows = min(rows, M)
    scale = 1.0 / np.sqrt(K) if w == "c2" else 1.0
    if w in ("c1", "c5a", "c5b", "c5c"):
        a = rng.uniform(-1, 1, (rows, K)).astype(np.float32)
        b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    else:
        a = (rng.normal(size=(rows, K)) * scale).astype(np.float32)
        b = (rng.normal(size=(K, N)) * (0.02 if w == "c3" else scale)).astype(np.float32)
    bias = (rng.normal(size=N) * 0.02).astype(np.float32) if epi else None
    return O.to_bits(a, dab), O.to_bits(b, dab), (O.to_bits(bias, dc) if bias is not None else None)


# ---------------------------------------------------------------------------------------------- clocks

class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
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
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ---------------------------------------------------------------------------------------------- GPU arm

def run_gpu(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from nova_compiler_b200 import _lib as L
    from nova_compiler_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = L.load()
    L.check(lib.nova_b200_init(local))

    w = args.workload
    desc, dab, dc, B, M, N, K, epi = WORKLOADS[w]
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
    flops, byts = algorithmic(w)

    def dev(arr, dt):
        t = torch.from_numpy(arr)
        if dt != "f32":
            t = t.view(torch.int16).view(tdt[dt])
        return t.cuda()

    # Batch-index sharding: rank r owns global batches [r*B, (r+1)*B); its inputs come from seed 1234 + r.
    a_np, b_np, bias_np = make_inputs_np(w, 1234 + rank)
    # Rotate over enough buffer sets that consecutive steps never find their operands in the 126 MB L2.
    n_sets = max(2, min(8, int(np.ceil(3 * 140e6 / byts)) + 1))
    sets = []
    for i in range(n_sets):
        a = dev(a_np, dab) if i == 0 else sets[0][0].clone()
        b = dev(b_np, dab) if i == 0 else sets[0][1].clone()
        c = torch.empty((B, M, N), dtype=tdt[dc], device="cuda")
        sets.append((a, b, c))
    bias = dev(bias_np, dc) if bias_np is not None else None
    act = "gelu" if epi else None

    def step(i):
        a, b, c = sets[i % n_sets]
        ops.gemm(a, b, bias=bias, act=act, out=c)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    # The launches of one pass over the buffer sets are captured into a CUDA graph and replayed: the host side
    # of a call (argument checks, three tensor-map encodings, the launch) costs more than the smallest
    # workloads' kernels.  EXACTLY args.steps steps run: whole replays, then the remainder as direct calls.
    graph = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(n_sets):
                    step(i)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()  # one untimed replay (n_sets more warm-up steps)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    if graph is not None:
        for _ in range(args.steps // n_sets):
            graph.replay()
        for i in range(args.steps % n_sets):
            step(i)
    else:
        for i in range(args.steps):
            step(i)
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    status = ops.device_status()
    if status != 0:
        raise SystemExit(f"device status 0x{status:x}: a bounded in-kernel wait gave up")
    value = world * flops / (ms_step * 1e-3) / 1e12
    per_gpu = flops / (ms_step * 1e-3) / 1e12

    # ---- end to end through the host-buffer C-ABI entry point (pinned host memory)
    g = L.GemmArgs()
    g.struct_size = C.sizeof(L.GemmArgs)
    g.dtype_ab, g.dtype_c = {"f32": L.F32, "f16": L.F16, "bf16": L.BF16}[dab], {"f32": L.F32, "f16": L.F16, "bf16": L.BF16}[dc]
    g.batch, g.M, g.N, g.K = B, M, N, K
    g.lda, g.ldb, g.ldc = K, N, N
    g.batch_stride_a, g.batch_stride_b, g.batch_stride_c = M * K, K * N, M * N
    ha = torch.from_numpy(a_np).pin_memory()
    hb = torch.from_numpy(b_np).pin_memory()
    hc = torch.empty((B, M, N), dtype=torch.float32 if dc == "f32" else torch.int16).pin_memory()
    g.A, g.B, g.C = ha.data_ptr(), hb.data_ptr(), hc.data_ptr()
    if bias_np is not None:
        hbias = torch.from_numpy(bias_np).pin_memory()
        g.bias, g.init, g.act = hbias.data_ptr(), L.INIT_BIAS_ROW, L.ACT_GELU_TANH
    e2e = None
    if not args.profile:
        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(2):
            L.check(lib.nova_b200_gemm_host(C.byref(g)))
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            L.check(lib.nova_b200_gemm_host(C.byref(g)))
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        t = torch.tensor([e2e_ms], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
        e2e = {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
               "steps": e2e_steps,
               "h2d_bytes_per_step": int(a_np.nbytes + b_np.nbytes + (bias_np.nbytes if bias_np is not None else 0)),
               "d2h_bytes_per_step": int(hc.numel() * hc.element_size()),
               "api": "nova_b200_gemm_host (pinned host buffers: H2D, kernel, D2H, sync every step)"}

    line = None
    if rank == 0:
        peaks, src = load_peaks()
        peak = peaks["bf16_tflops"]
        hbm = peaks["hbm_gbs"]
        ai = flops / byts
        bound = "tensor" if ai * hbm / 1e3 > peak else "hbm"
        if bound == "tensor":
            roof = {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak}
        else:
            gbs = byts / (ms_step * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm}
        roof.update({"traffic": NCU_TRAFFIC_BYTES.get(w), "peak_source": f"{src} (cuBLAS bf16 burst / copy bandwidth)",
                     "algorithmic_flops_per_launch": flops, "algorithmic_bytes_per_launch": byts,
                     "kernel_ms": ms_step, "frac_of_nominal_bf16_2250": per_gpu / NOMINAL_BF16_TFLOPS})
        # the contraction, plus one launch when operands go through scratch first (the f32 hi/lo split, or the
        # re-pitched copy of operands whose pitch no tensor map can describe)
        info = L.GemmPlanInfo()
        L.check(lib.nova_b200_gemm_plan(C.byref(g), C.byref(info)))
        launches_per_step = 2 if info.scratch_bytes > 0 else 1
        line = {
            "metric": "batch-matmul/linear TFLOPS", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": dab, "data": "synthetic (seeded, shapes and distributions of the config)",
            "config": {"workload": f"{w}: {desc}", "per_gpu_batch": B, "sharding": "batch index, no collective",
                       "l2": f"rotating {n_sets} buffer sets ({n_sets * byts / 1e6:.0f} MB) so operands never sit in L2",
                       "accumulate": "fp32",
                       "launch": "direct calls" if graph is None else f"CUDA graph of {n_sets} steps, replayed"},
            "impl": "nova_b200", "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "roofline": roof, "pct_of_bf16_dense_peak_nominal": 100.0 * per_gpu / NOMINAL_BF16_TFLOPS,
        }
        if world == 1 and not args.profile:
            line["cpu_baseline"] = cpu_baseline(w)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)
    return 0


def cpu_baseline(w, budget_s=12.0):
    """The reference's single-threaded CPU nest on a bounded row sample of the same workload (about 10 s)."""
    from oracle import oracle as O
    desc, dab, dc, B, M, N, K, epi = WORKLOADS[w]
    rows = max(1, min(M, int(1.0e8 / (2.0 * N * K)) or 1))
    a, b, bias = make_inputs_np_small(w, rows)
    done, t0 = 0, time.perf_counter()
    while True:
        O.gemm_scalar_rows(a, b, dtype_in=dab, dtype_out=dc, bias=bias, act="gelu_tanh" if epi else "none",
                           row_begin=0, row_end=rows)
        done += rows
        el = time.perf_counter() - t0
        if el > budget_s:
            break
    tflops = 2.0 * done * N * K / el / 1e12
    return {"value": tflops, "unit": "TFLOP/s", "cores": 1, "kind": "port",
            "sample": f"{done} output rows (repeats of rows 0..{rows - 1}) of {B * M}, full N and K, {el:.1f} s; "
                      "single-threaded scalar i/j/k nest as the reference's CPU pipeline emits it; extrapolates linearly"}


# HBM-bound companions of the contraction: name -> (description, dtype, rows, D)
ROW_WORKLOADS = {
    "ln": ("nova.layer_norm bf16 [8192, 4096] (the rows that feed the C3 linear)", "bf16", 8192, 4096),
    "softmax": ("nova.softmax f16 [65536, 2048] (attention-score rows, C4 layout, 32 of its 256 batches)", "f16", 65536, 2048),
    "gather": ("nova.gather bf16 table [50304, 4096], 16384 i32 ids (embedding lookup)", "bf16", 16384, 4096),
    "ln_bwd": ("nova.layer_norm_backward bf16 [8192, 4096] (dx, dgamma, dbeta from one read of gy and x)", "bf16", 8192, 4096),
    "sce": ("nova.sce f32 logits [8192, 50304], i16 targets (softmax + mean loss; the vocabulary rows of ltest/test.mlir)", "f32", 8192, 50304),
    "sce_bwd": ("nova.sce_backward f32 [8192, 50304]", "f32", 8192, 50304),
}


def run_rowop(args):
    """HBM roofline of the row-wise kernels: GB/s = (bytes read + bytes written) / event time."""
    import torch
    from nova_compiler_b200 import _lib as L
    from nova_compiler_b200 import ops
    torch.cuda.set_device(0)
    L.check(L.load().nova_b200_init(0))
    w = args.workload
    desc, dt, rows, D = ROW_WORKLOADS[w]
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[dt]
    es = 4 if dt == "f32" else 2
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    n_sets = 4  # rotate inputs so a step never finds its rows in L2
    if w == "gather":
        table = torch.randn(50304, D, device="cuda", generator=g).to(tdt)
        sets = [torch.randint(0, 50304, (rows,), device="cuda", generator=g).to(torch.int32) for _ in range(n_sets)]
        byts = 2 * rows * D * 2 + rows * 4
        fn = lambda i: ops.gather(table, sets[i % n_sets])
    elif w in ("sce", "sce_bwd"):
        n_sets = 2  # 1.65 GB per tensor
        sets = [torch.randn(rows, D, device="cuda", generator=g) * 3.0 for _ in range(n_sets)]
        tg = torch.randint(0, D, (rows,), device="cuda", generator=g).to(torch.int16)
        byts = 2 * rows * D * es + rows * 2
        if w == "sce":
            fn = lambda i: ops.sce(sets[i % n_sets], tg)
        else:
            sets = [ops.sce(x, tg)[0] for x in sets]
            fn = lambda i: ops.sce_backward(sets[i % n_sets], tg)
    elif w == "ln_bwd":
        sets = [torch.randn(rows, D, device="cuda", generator=g).to(tdt) for _ in range(n_sets)]
        gys = [torch.randn(rows, D, device="cuda", generator=g).to(tdt) for _ in range(n_sets)]
        gamma = torch.randn(D, device="cuda", generator=g).to(tdt)
        stats = [ops.layer_norm(x, gamma, gamma)[1:] for x in sets]
        byts = 3 * rows * D * es + 3 * D * es + 2 * rows * es
        fn = lambda i: ops.layer_norm_backward(gys[i % n_sets], sets[i % n_sets], gamma, *stats[i % n_sets])
    else:
        sets = [torch.randn(rows, D, device="cuda", generator=g).to(tdt) for _ in range(n_sets)]
        gamma = torch.randn(D, device="cuda", generator=g).to(tdt)
        beta = torch.randn(D, device="cuda", generator=g).to(tdt)
        byts = 2 * rows * D * 2 + (2 * D * 2 + 2 * rows * 2 if w == "ln" else 0)
        fn = (lambda i: ops.layer_norm(sets[i % n_sets], gamma, beta)) if w == "ln" else (lambda i: ops.softmax(sets[i % n_sets]))
    for i in range(max(args.warmup, 3)):
        fn(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    peaks, src = load_peaks()
    gbs = byts / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "row-op HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": dt, "data": "synthetic (seeded)", "impl": "nova_b200", "clocks": clocks,
        "gpu_launches": args.steps * {"ln_bwd": 2, "sce": 2}.get(w, 1),  # ln_bwd: + column-sum finish; sce: + loss kernel
        "config": {"workload": f"{w}: {desc}", "l2": f"rotating {n_sets} input sets; outputs are fresh allocations"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                     "traffic": NCU_TRAFFIC_BYTES.get(w), "peak_source": src, "algorithmic_bytes_per_launch": byts,
                     "frac_of_nominal_8000": gbs / 8000.0},
    }), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + sorted(ROW_WORKLOADS))
    ap.add_argument("--impl", default="nova_b200", choices=["nova_b200", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch every step with a direct call instead of replaying a CUDA graph")
    ap.add_argument("--profile", action="store_true",
                    help="device-resident leg only (no end-to-end leg, no CPU baseline): for captures under ncu")
    args = ap.parse_args()
    if args.profile:
        args.no_graph = True  # captures under ncu see plain kernel launches
    if args.impl == "reference":
        args.steps = args.steps or 10
        args.warmup = args.warmup if args.warmup is not None else 1
        return run_reference(args)
    if args.workload in ROW_WORKLOADS:
        args.steps = args.steps or 100
        args.warmup = args.warmup if args.warmup is not None else 5
        return run_rowop(args)
    args.steps = args.steps or (1000 if args.workload in ("c1", "c2", "c5b") else 200)
    args.warmup = args.warmup if args.warmup is not None else 10
    return run_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
