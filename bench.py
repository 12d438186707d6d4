#!/usr/bin/env python
"""Benchmark of the matmul hot path through the C ABI of libnova_b200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--only] [--impl reference]

A step is ONE pass of a contraction over one batch of seeded synthetic input.  The headline workload is the bf16
transformer linear layer (X[8192,4096] . W[4096,11008] + bias, GELU-tanh, fp32 accumulation, bf16 out); the same
JSON line carries a `workloads` object with one sub-record per remaining configuration (f32 512^3, f16 batch 32 x
1024^3, f16 attention scores 256 x 2048 x 2048 x 128, bf16 16384^3, the two ragged bf16 GEMMs) and per row kernel
(layer_norm, softmax, gather, layer_norm_backward), each with its own time, roofline fraction and clocks.
`--workload X` makes X the headline; `--only` drops the sub-records.

Inputs are resident in HBM for `value`; `e2e` runs the headline through nova_b200_gemm_host with pinned HOST
buffers (H2D + kernel + D2H inside the timed region).

With N > 1 (torchrun, one rank per GPU) every workload is ONE GLOBAL PROBLEM partitioned over the ranks with no
data-path collective: batched contractions by batch index (rank r owns a contiguous range of batches), single
GEMMs by 64-column-aligned N slabs (every rank holds A and reads its slab of B as a strided view).  value = global
FLOPs / the slowest rank's device time ("scaling": "strong").  The optional all-gather of the output slabs (NCCL +
one re-interleave kernel) is timed on its own and reported as `allgather_ms`, outside `value`.

`--impl reference` times the reference's own CPU lowering of the same contraction (the single-threaded i/j/k loop
nest its CPU pipeline emits, restated in oracle/nova_oracle.c) on this machine's host cores, on a bounded row
sample of the workload.  That is a reported baseline, not the target.

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

# name -> (description, dtype_ab, dtype_c, batch, M, N, K, epilogue, partition over ranks)
WORKLOADS = {
    "c1": ("nova.matmul f32 512x512x512 (3xTF32)", "f32", "f32", 1, 512, 512, 512, None, None),
    "c2": ("linalg.batch_matmul f16 B=32 M=N=K=1024, fp32 accumulate, f16 out", "f16", "f16", 32, 1024, 1024, 1024, None,
           "batch"),
    "c3": ("linear bf16 X[8192,4096] W[4096,11008] + bias, GELU(tanh), bf16 out", "bf16", "bf16", 1, 8192, 11008, 4096,
           "bias_gelu", "slab"),
    "c4": ("batch_matmul f16 Q[256,2048,128] K^T[256,128,2048], f16 out", "f16", "f16", 256, 2048, 2048, 128, None, "batch"),
    "c4s": ("batch_matmul f16 Q[32,2048,128] K^T[32,128,2048] (C4 at one eighth of the batch, profiling-sized)", "f16", "f16",
            32, 2048, 2048, 128, None, "batch"),
    "c5a": ("GEMM bf16 16384^3", "bf16", "bf16", 1, 16384, 16384, 16384, None, "slab"),
    "c5b": ("GEMM bf16 ragged 1000x1000x999", "bf16", "bf16", 1, 1000, 1000, 999, None, None),
    "c5c": ("GEMM bf16 ragged 4095x11007x4097", "bf16", "bf16", 1, 4095, 11007, 4097, None, None),
    "c5cp": ("GEMM bf16 ragged 4095x11007x4097 with B (the weight) prepared once: only A is re-pitched per call", "bf16", "bf16", 1,
             4095, 11007, 4097, None, None),
}
# default steps of a sub-record (the headline takes --steps)
SUB_STEPS = {"c1": 400, "c2": 400, "c3": 100, "c4": 60, "c4s": 100, "c5a": 12, "c5b": 400, "c5c": 100, "c5cp": 100}
# DRAM bytes one launch moves according to ncu (dram__bytes_read.sum + dram__bytes_write.sum), per workload at
# N = 1; see profiles/.  None where no capture exists.
NCU_TRAFFIC_BYTES = {
    "c2": 173.3e6,      # 134.3 MB read + 39.0 MB written (part of the 67 MB output is still in L2 at kernel end)
    "c3": 466.7e6,      # 306.1 MB read + 160.7 MB written
    "c4": 8 * 243.4e6,  # captured on 32 of the 256 batches (c4s), scaled by 8: traffic is proportional to batches
    "c4s": 243.4e6,
    "c5c": 207.7e6,     # the contraction kernel: 140.2 MB read + 67.5 MB written (the re-pitch copy before it: 203.8 MB)
    # row kernels (reads match the inputs exactly; part of each output is still in L2 when the kernel ends)
    "ln": 88.6e6, "ln_bwd": 182.1e6, "softmax": 488.6e6, "sce": 3246.0e6, "sce_bwd": 3252.9e6, "gather": 209.2e6,
}

# HBM-bound companions of the contraction: name -> (description, dtype, rows, D)
ROW_WORKLOADS = {
    "ln": ("nova.layer_norm bf16 [8192, 4096] (the rows that feed the C3 linear)", "bf16", 8192, 4096),
    "softmax": ("nova.softmax f16 [65536, 2048] (attention-score rows, C4 layout, 32 of its 256 batches)", "f16", 65536, 2048),
    "softmax8k": ("nova.softmax f16 [16384, 8192] (score rows of an 8192-token context)", "f16", 16384, 8192),
    "gather": ("nova.gather bf16 table [50304, 4096], 16384 i32 ids (embedding lookup)", "bf16", 16384, 4096),
    "ln_bwd": ("nova.layer_norm_backward bf16 [8192, 4096] (dx, dgamma, dbeta from one read of gy and x)", "bf16", 8192, 4096),
    "sce": ("nova.sce f32 logits [8192, 50304], i16 targets (softmax + mean loss; the vocabulary rows of ltest/test.mlir)", "f32", 8192, 50304),
    "sce_bwd": ("nova.sce_backward f32 [8192, 50304]", "f32", 8192, 50304),
}
# order: latency-bound and HBM-bound records first, the seconds of dense tensor work (which pull the part into its
# power cap) last; each record starts after a short idle so that it does not inherit the previous one's clocks
DEFAULT_SUBS = ["c1", "c5b", "ln", "softmax", "softmax8k", "gather", "ln_bwd", "sce", "sce_bwd", "c2", "c4", "c5c", "c5cp", "c5a"]
SUB_IDLE_S = 0.75


def load_peaks():
    path = os.path.join(HERE, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def algorithmic(w, batch=None, n=None):
    """(FLOPs, bytes) of one launch: one read of each input, one write of the output (B shared across the batch
    counts once per launch).  batch / n override the global extents (a rank's share)."""
    _, dab, dc, B, M, N, K, epi, _ = WORKLOADS[w]
    B = B if batch is None else batch
    N = N if n is None else n
    es = 4 if dab == "f32" else 2
    os_ = 4 if dc == "f32" else 2
    flops = 2.0 * B * M * N * K
    byts = es * B * (M * K + K * N) + os_ * B * M * N + (os_ * N if epi else 0)
    return flops, byts


# ---------------------------------------------------------------------------------------------- reference arm

def make_inputs_np_small(w, rows):
    """First `rows` of the (batch*M) rows of the workload's A, and the matching B (first batch), seeded."""
    import numpy as np
    from oracle import oracle as O
    _, dab, dc, B, M, N, K, epi, _ = WORKLOADS[w]
    rng = np.random.default_rng(1234)
    rows = min(rows, M)
    scale = 1.0 / np.sqrt(K) if w == "c2" else 1.0
    if w in ("c1", "c5a", "c5b", "c5c", "c5cp"):
        a = rng.uniform(-1, 1, (rows, K)).astype(np.float32)
        b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    else:
        a = (rng.normal(size=(rows, K)) * scale).astype(np.float32)
        b = (rng.normal(size=(K, N)) * (0.02 if w == "c3" else scale)).astype(np.float32)
    bias = (rng.normal(size=N) * 0.02).astype(np.float32) if epi else None
    return O.to_bits(a, dab), O.to_bits(b, dab), (O.to_bits(bias, dc) if bias is not None else None)


def run_reference(args):
    """The reference's CPU path (restated): scalar i/j/k nest, C re-loaded every k, k unrolled x8, ONE thread
    (its pipeline has no OpenMP/async lowering: lib/Pipeline/Pipeline.cpp:135,157-165)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle as O
    w = args.workload
    if w not in WORKLOADS:
        raise SystemExit("--impl reference times the contraction workloads only")
    desc, dab, dc, B, M, N, K, epi, _ = WORKLOADS[w]
    # a bounded sample: a row slice sized for ~0.3 s per step
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
        "scaling": "strong", "vs_baseline": None, "dtype": dab, "data": "synthetic (seeded)",
        "config": {"workload": f"{w}: {desc}", "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": 1, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference = C restatement of the Nova CPU pipeline's single-threaded loop nest (oracle/nova_oracle.c); "
                "the MLIR reference itself cannot be built without LLVM 21",
    }
    print(json.dumps(line), flush=True)
    return 0


def cpu_baseline(w, budget_s=12.0):
    """The reference's single-threaded CPU nest on a bounded row sample of the same workload (about 10 s)."""
    from oracle import oracle as O
    desc, dab, dc, B, M, N, K, epi, _ = WORKLOADS[w]
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

class Ctx:
    """Process-wide state of the GPU arm: rank layout, library handle, peaks."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        from nova_compiler_b200 import _lib as L
        self.torch, self.dist, self.L = torch, dist, L
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        torch.cuda.set_device(self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        self.lib = L.load()
        L.check(self.lib.nova_b200_init(self.local))
        self.peaks, self.peak_src = load_peaks()
        self.args = args

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        t = self.torch.tensor([float(v)], device="cuda", dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def _tdt(torch, name):
    return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[name]


def make_inputs(ctx, w, batch_range=None):
    """Seeded device inputs with the configuration's shapes and distributions.  Slab-partitioned workloads use
    the same seed on every rank (A and B are replicated; a rank reads its slab of B as a strided view);
    batch-partitioned ones draw only the rank's batches (seed offset by the first batch index)."""
    torch = ctx.torch
    _, dab, dc, B, M, N, K, epi, part = WORKLOADS[w]
    first, count = batch_range if batch_range is not None else (0, B)
    g = torch.Generator(device="cuda")
    g.manual_seed(1234 + first)
    dt, dtc = _tdt(torch, dab), _tdt(torch, dc)

    def uniform(shape):
        return (torch.rand(shape, device="cuda", generator=g, dtype=torch.float32) * 2 - 1).to(dt)

    def normal(shape, scale):
        return (torch.randn(shape, device="cuda", generator=g, dtype=torch.float32) * scale).to(dt)

    if w in ("c1", "c5a", "c5b", "c5c", "c5cp"):
        a, b = uniform((count, M, K)), uniform((count, K, N))
    elif w == "c2":
        a, b = normal((count, M, K), K ** -0.5), normal((count, K, N), K ** -0.5)
    elif w == "c3":
        a, b = normal((count, M, K), 1.0), normal((count, K, N), 0.02)
    else:
        a, b = normal((count, M, K), 1.0), normal((count, K, N), 1.0)
    bias = (torch.randn(N, device="cuda", generator=g, dtype=torch.float32) * 0.02).to(dtc) if epi else None
    return a, b, bias


def run_contraction(ctx, w, steps, warmup, headline=False):
    """One contraction workload: device-resident timing (graph replay unless --no-graph), roofline record, and for
    the headline the end-to-end and sustained legs."""
    import numpy as np
    from nova_compiler_b200 import ops, sharding
    torch, L, lib, args = ctx.torch, ctx.L, ctx.lib, ctx.args
    desc, dab, dc, B, M, N, K, epi, part = WORKLOADS[w]
    world, rank = ctx.world, ctx.rank
    if world > 1 and part is None:
        return None  # this workload has no partition the north star names: single-GPU record only
    # this rank's share of the global problem
    b0, bcount, n0, ncount = 0, B, 0, N
    if world > 1 and part == "batch":
        b0, bcount = sharding.batch_range(B, world, rank)
    if world > 1 and part == "slab":
        n0, ncount = sharding.column_slab(N, world, rank)
    g_flops, g_bytes = algorithmic(w)
    r_flops, r_bytes = algorithmic(w, batch=bcount, n=ncount)

    a0, b_full, bias_full = make_inputs(ctx, w, (b0, bcount))
    # Rotate over enough buffer sets that consecutive steps never find their operands in the 126 MB L2.
    n_sets = max(2, min(8, int(np.ceil(3 * 140e6 / max(r_bytes, 1))) + 1))
    sets = []
    prepared = []
    for i in range(n_sets):
        a = a0 if i == 0 else a0.clone()
        bf = b_full if i == 0 else b_full.clone()
        if w == "c5cp":  # the weight copied once to an aligned pitch, outside the timed region
            prepared.append(ops.PreparedOperand(bf[0]))
            bf = prepared[-1].tensor[None]
        bview = bf[:, :, n0:n0 + ncount]  # a column slab is a strided view: the row pitch stays N
        c = torch.empty((bcount, M, ncount), dtype=_tdt(torch, dc), device="cuda")
        sets.append((a, bview, c, bf))
    bias = bias_full[n0:n0 + ncount].contiguous() if bias_full is not None else None
    act = "gelu" if epi else None

    def step(i):
        a, b, c, _ = sets[i % n_sets]
        ops.gemm(a, b, bias=bias, act=act, out=c)

    # the same calls with the argument structs built once, as a compiled caller holds them: what a direct
    # (un-graphed) call costs through the C ABI itself, without the Python operator layer
    abi_args = []
    for a_, b_, c_, _ in sets:
        ga_ = L.GemmArgs()
        ga_.struct_size = C.sizeof(L.GemmArgs)
        ga_.dtype_ab = {"f32": L.F32, "f16": L.F16, "bf16": L.BF16}[dab]
        ga_.dtype_c = {"f32": L.F32, "f16": L.F16, "bf16": L.BF16}[dc]
        ga_.batch, ga_.M, ga_.N, ga_.K = max(bcount, 1), M, max(ncount, 1), K
        ga_.A, ga_.B, ga_.C = a_.data_ptr(), b_.data_ptr(), c_.data_ptr()
        ga_.lda, ga_.ldb, ga_.ldc = K, b_.stride(1), max(ncount, 1)
        ga_.batch_stride_a, ga_.batch_stride_b, ga_.batch_stride_c = M * K, K * b_.stride(1), M * max(ncount, 1)
        if bias is not None:
            ga_.init, ga_.bias, ga_.act = L.INIT_BIAS_ROW, bias.data_ptr(), L.ACT_GELU_TANH
        abi_args.append(ga_)

    def step_abi(i):
        L.check(lib.nova_b200_gemm(C.byref(abi_args[i % n_sets]), C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    if bcount == 0 or ncount == 0:
        def step(i):  # noqa: F811 - a rank that owns nothing still takes part in the barriers
            return None

    for i in range(max(warmup, 3)):
        step(i)
    ctx.barrier()
    # The launches of one pass over the buffer sets are captured into a CUDA graph and replayed; EXACTLY `steps`
    # steps run: whole replays, then the remainder as direct calls.
    graph = None
    if not args.no_graph and bcount and ncount:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(n_sets):
                step(i)  # the capturing stream's scratch must exist before the capture
        side.synchronize()
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(n_sets):
                    step(i)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()  # one untimed replay (n_sets more warm-up steps)

    def timed(n_steps, use_graph, fn=None):
        fn = fn or step
        ctx.barrier()
        sampler = ClockSampler(ctx.local)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx.barrier()
        e0.record()
        if use_graph and graph is not None:
            for _ in range(n_steps // n_sets):
                graph.replay()
            for i in range(n_steps % n_sets):
                fn(i)
        else:
            for i in range(n_steps):
                fn(i)
        e1.record()
        ctx.barrier()
        clocks = sampler.stop()
        return ctx.max_over_ranks(e0.elapsed_time(e1)) / n_steps, clocks

    ms_step, clocks = timed(steps, True)
    status = ops.device_status()
    if status != 0:
        raise SystemExit(f"device status 0x{status:x}: a bounded in-kernel wait gave up")
    value = g_flops / (ms_step * 1e-3) / 1e12          # whole job: the global problem / the slowest rank
    per_gpu = value / world

    peak, hbm = ctx.peaks["bf16_tflops"], ctx.peaks["hbm_gbs"]
    bound = "tensor" if (g_flops / g_bytes) * hbm / 1e3 > peak else "hbm"
    if bound == "tensor":
        roof = {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak}
    else:
        gbs = g_bytes / world / (ms_step * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm}
    roof.update({"traffic": NCU_TRAFFIC_BYTES.get(w) if world == 1 else None,
                 "peak_source": f"{ctx.peak_src} (cuBLAS bf16 burst / copy bandwidth), per GPU",
                 "algorithmic_flops_per_launch": r_flops, "algorithmic_bytes_per_launch": r_bytes,
                 "kernel_ms": ms_step, "frac_of_nominal_bf16_2250": per_gpu / NOMINAL_BF16_TFLOPS})

    # how this rank's call is executed
    ga = L.GemmArgs()
    ga.struct_size = C.sizeof(L.GemmArgs)
    code = {"f32": L.F32, "f16": L.F16, "bf16": L.BF16}
    ga.dtype_ab, ga.dtype_c = code[dab], code[dc]
    ga.batch, ga.M, ga.N, ga.K = max(bcount, 1), M, max(ncount, 1), K
    ga.lda, ga.ldb, ga.ldc = K, sets[0][1].stride(1), max(ncount, 1)
    ga.batch_stride_a, ga.batch_stride_b, ga.batch_stride_c = M * K, K * sets[0][1].stride(1), M * max(ncount, 1)
    ga.A, ga.B, ga.C = sets[0][0].data_ptr(), sets[0][1].data_ptr(), sets[0][2].data_ptr()
    info = L.GemmPlanInfo()
    L.check(lib.nova_b200_gemm_plan(C.byref(ga), C.byref(info)))
    # kernels per call: the contraction, a pre-pass when an operand goes through scratch (hi/lo split of f32, re-pitch),
    # and the reduce kernel when K runs as ranges (the plan then counts range x tile work units)
    base_tiles = ga.batch * ((ga.M + info.block_m - 1) // info.block_m) * ((ga.N + info.block_n - 1) // info.block_n)
    k_ranges = info.tiles // base_tiles if base_tiles and info.tiles % base_tiles == 0 else 1
    pre_pass = dab == "f32" or info.loader_a == 2 or info.loader_b == 2
    launches_per_step = 1 + (1 if pre_pass else 0) + (1 if k_ranges > 1 else 0)

    rec = {
        "workload": f"{w}: {desc}", "value": value, "unit": "TFLOP/s", "per_gpu": per_gpu, "ms_per_step": ms_step,
        "steps": steps, "dtype": dab, "roofline": roof, "clocks": clocks, "gpu_launches": launches_per_step * steps,
        "pct_of_bf16_dense_peak_nominal": 100.0 * per_gpu / NOMINAL_BF16_TFLOPS,
        "plan": {"tile": [info.block_m, info.block_n, info.block_k], "stages": info.stages, "grid": info.grid,
                 "tiles": info.tiles, "k_ranges": k_ranges, "loader_a": info.loader_a, "loader_b": info.loader_b, "store_c": info.store_c,
                 "repitch_bytes": int(info.scratch_bytes) if info.loader_a == 2 or info.loader_b == 2 else 0},
        "l2": f"rotating {n_sets} buffer sets ({n_sets * r_bytes / 1e6:.0f} MB per rank) so operands never sit in L2",
        "launch": "direct calls" if graph is None else f"CUDA graph of {n_sets} steps, replayed",
    }
    if world > 1:
        rec["partition"] = ({"by": "batch index", "per_rank_batches": [sharding.batch_range(B, world, r)[1] for r in range(world)]}
                            if part == "batch" else
                            {"by": "N-column slabs (64-column aligned), A replicated",
                             "per_rank_columns": [sharding.column_slab(N, world, r)[1] for r in range(world)]})
    # host cost of a call: the same steps as direct calls (no graph).  Small problems are where it shows.
    if graph is not None and (w in ("c1", "c5b") or headline) and world == 1:
        ms_direct, _ = timed(min(steps, 200), False, step_abi)
        rec["no_graph_ms_per_step"] = ms_direct
        rec["no_graph"] = "the same steps as direct nova_b200_gemm calls (argument structs built once), no CUDA graph"

    # the optional exchange: all ranks end with the whole row-major C (NCCL all-gather + one re-interleave kernel)
    if world > 1 and part == "slab" and not args.no_gather:
        c_slab = sets[0][2][0]
        full = sharding.gather_slabs(c_slab, N)  # warm-up (allocations, NCCL channels)
        ctx.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        e0.record()
        for _ in range(reps):
            full = sharding.gather_slabs(c_slab, N, out=full)
        e1.record()
        ctx.barrier()
        ag_ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / reps
        os_ = 4 if dc == "f32" else 2
        recv_bytes = M * (N - ncount) * os_
        rec["allgather_ms"] = ag_ms
        rec["allgather"] = {"ms": ag_ms, "bytes_received_per_rank": recv_bytes,
                            "gbs_per_rank": recv_bytes / (ag_ms * 1e-3) / 1e9,
                            "nvlink_peer_copy_gbs_measured": 770.0,
                            "how": "NCCL all_gather into [world, M, slab] staging + nova_b200_interleave_slabs; outside `value`"}
        del full
        # the fused form: the contraction's epilogue stores its slab into every rank's matrix (nova_b200_gemm_push);
        # a step is the whole exchange + contraction, to hold against ms_per_step + allgather_ms
        if (N * os_) % 16 == 0 and all(sharding.column_slab(N, world, r)[1] * os_ % 16 == 0 for r in range(world)):
            try:
                rec["allgather_fused"] = run_fused_push(ctx, sets[0], bias_full, act, M, N, ncount, os_, g_flops, steps, _tdt(torch, dc))
            except Exception as exc:  # peer mapping unavailable on this machine: the record says so, the run goes on
                rec["allgather_fused"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}

    if headline:
        if not args.profile:
            rec["e2e"] = run_e2e(ctx, w, sets[0], bias, (bcount, ncount), g_flops)
        if world == 1 and not args.profile and not args.no_sustained and graph is not None:
            rec["sustained"] = run_sustained(ctx, graph, n_sets, g_flops)
    del sets, graph
    for pr in prepared:
        pr.free()
    torch.cuda.empty_cache()
    return rec


def run_fused_push(ctx, set0, bias_full, act, M, N, ncount, os_, g_flops, steps, out_dtype):
    """The slab contraction whose epilogue stores into every rank's matrix (nova_b200_gemm_push): a step is the whole
    contraction + exchange, to hold against ms_per_step + allgather_ms."""
    from nova_compiler_b200 import sharding
    torch = ctx.torch
    pm = sharding.PeerMatrix(M, N, out_dtype)
    try:
        a2, b2 = set0[0][0], set0[3][0]
        for _ in range(3):
            sharding.slab_matmul_push(a2, b2, pm, bias=bias_full, act=act)
        ctx.barrier()
        reps = max(5, min(steps, 30))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            sharding.slab_matmul_push(a2, b2, pm, bias=bias_full, act=act)
        e1.record()
        ctx.barrier()
        push_ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / reps
    finally:
        pm.close()
    return {"ms_per_step": push_ms, "value": g_flops / (push_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "bytes_sent_per_rank": M * ncount * os_ * (ctx.world - 1),
            "how": "nova_b200_gemm_push: the epilogue stores every output box into the peers' matrices (plain stores over "
                   "NVLink), direct calls back to back; the whole C is on every rank when the step ends"}


def run_e2e(ctx, w, set0, bias, share, g_flops):
    """The same contraction through nova_b200_gemm_host: this rank's operands in pinned host memory, H2D + kernel +
    D2H + sync inside the timed region, every step."""
    torch, L, lib = ctx.torch, ctx.L, ctx.lib
    desc, dab, dc, B, M, N, K, epi, part = WORKLOADS[w]
    bcount, ncount = share
    if bcount == 0 or ncount == 0:
        ctx.barrier(); ctx.barrier()
        ctx.max_over_ranks(0.0)
        return None
    a, bview, c, _ = set0
    ha = a.cpu().pin_memory()
    hb = bview.contiguous().cpu().pin_memory()   # the host side holds the rank's slab of B on its own
    hc = torch.empty((bcount, M, ncount), dtype=c.dtype).pin_memory()
    g = L.GemmArgs()
    g.struct_size = C.sizeof(L.GemmArgs)
    code = {"f32": L.F32, "f16": L.F16, "bf16": L.BF16}
    g.dtype_ab, g.dtype_c = code[dab], code[dc]
    g.batch, g.M, g.N, g.K = bcount, M, ncount, K
    g.lda, g.ldb, g.ldc = K, ncount, ncount
    g.batch_stride_a, g.batch_stride_b, g.batch_stride_c = M * K, K * ncount, M * ncount
    g.A, g.B, g.C = ha.data_ptr(), hb.data_ptr(), hc.data_ptr()
    h2d = ha.numel() * ha.element_size() + hb.numel() * hb.element_size()
    if bias is not None:
        hbias = bias.cpu().pin_memory()
        g.bias, g.init, g.act = hbias.data_ptr(), L.INIT_BIAS_ROW, L.ACT_GELU_TANH
        h2d += hbias.numel() * hbias.element_size()
    d2h = hc.numel() * hc.element_size()
    e2e_steps = max(3, min(ctx.args.steps or 10, 10))
    for _ in range(2):
        L.check(lib.nova_b200_gemm_host(C.byref(g)))
    ctx.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        L.check(lib.nova_b200_gemm_host(C.byref(g)))
    torch.cuda.synchronize()
    own_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    ctx.barrier()
    e2e_ms = ctx.max_over_ranks(own_ms)
    return {"value": g_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
            "pcie_gbs_this_rank": (h2d + d2h) / (own_ms * 1e-3) / 1e9,
            "api": "nova_b200_gemm_host (pinned host buffers: H2D, kernel, D2H, sync every step); bytes are rank 0's share"}


def run_sustained(ctx, graph, n_sets, g_flops, seconds=2.5):
    """The headline launch looped for seconds (graph replays back to back) with the clocks sampled: the figure to
    hold against the sustained cuBLAS peak, where the burst number is held against the burst peak."""
    torch = ctx.torch
    torch.cuda.synchronize()
    sampler = ClockSampler(ctx.local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    n = 0
    e0.record()
    while time.perf_counter() - t0 < seconds:
        for _ in range(50):
            graph.replay()
        n += 50 * n_sets
        torch.cuda.synchronize()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / n
    tf = g_flops / (ms * 1e-3) / 1e12
    peak = ctx.peaks["bf16_tflops_sustained"]
    return {"value": tf, "unit": "TFLOP/s", "ms_per_step": ms, "steps": n, "seconds": e0.elapsed_time(e1) / 1e3,
            "clocks": clocks, "peak": peak, "frac": tf / peak, "peak_source": f"{ctx.peak_src} (cuBLAS bf16, seconds-long loop)"}


def run_ln_fold(ctx, steps=60):
    """nova.layer_norm feeding the headline linear + GELU: the two-kernel form (layer_norm writes y, the contraction
    reads it) against the folded form (row statistics in one read of x, the contraction consumes x itself).  Both
    timed as graph replays over rotating input sets; the record is the block's time, not a TFLOP/s figure."""
    from nova_compiler_b200 import ops
    torch = ctx.torch
    _, dab, dc, B, M, N, K, epi, _ = WORKLOADS["c3"]
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    dt = _tdt(torch, dab)
    n_sets = 3
    xs = [(torch.randn(M, K, device="cuda", generator=g)).to(dt) for _ in range(n_sets)]
    w = (torch.randn(K, N, device="cuda", generator=g) * 0.02).to(dt)
    bias = (torch.randn(N, device="cuda", generator=g) * 0.02).to(dt)
    gamma = (1.0 + 0.1 * torch.randn(K, device="cuda", generator=g)).to(dt)
    beta = (0.1 * torch.randn(K, device="cuda", generator=g)).to(dt)
    outs = [torch.empty(M, N, device="cuda", dtype=dt) for _ in range(n_sets)]
    folded = ops.LnFoldedLinear(w, gamma, beta, bias)

    def unfused(i):
        y, _, _ = ops.layer_norm(xs[i % n_sets], gamma, beta)
        ops.gemm(y[None], w[None], bias=bias, act="gelu", out=outs[i % n_sets][None])

    def fused(i):
        folded(xs[i % n_sets], act="gelu", out=outs[i % n_sets])

    res = {}
    for name, fn in (("layer_norm_then_linear_ms", unfused), ("folded_ms", fused)):
        for i in range(n_sets):
            fn(i)
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for i in range(n_sets):
                fn(i)
        side.synchronize()
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(n_sets):
                    fn(i)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        time.sleep(SUB_IDLE_S)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps // n_sets):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        res[name] = e0.elapsed_time(e1) / (steps // n_sets * n_sets)
        del graph
    es = 2
    res.update({"workload": "nova.layer_norm [8192, 4096] bf16 -> linear 4096 x 11008 + bias + GELU (the C3 block with its producer)",
                "hbm_bytes_saved_per_step": 2 * M * K * es - M * 8,
                "note": "folded: y is never written or read; kernels per step 2 (row statistics, contraction) in both forms"})
    return res


def run_graph_step(ctx, steps=20):
    """The reference's own GPT training-step graph (ltest/test.mlir: 8 x 1024 tokens, width 384, vocabulary 50304, f32:
    embedding gathers, a pre-norm FFN block, the vocabulary contraction, sparse cross entropy and the whole backward
    down to the embedding scatter-adds) run through the textual front-end, i.e. through the same C-ABI calls the
    lowering pass would emit.  The record is the step time; nothing is skipped or cached between steps."""
    from nova_compiler_b200.frontend import Module
    torch = ctx.torch
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tests", "golden", "ref_fixtures", "ltest__test.mlir")
    if not os.path.exists(path):
        return None
    m = Module(open(path).read())
    arg_sig, _ = m.signature("main")
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    V, T = 50304, 1024
    args = []
    for i, (dt, shape) in enumerate(arg_sig):
        if i in (0, 1):
            args.append(torch.randint(0, V, shape, device="cuda", generator=g).to(torch.int16))
        elif i in (2, 15):
            args.append(torch.arange(T, device="cuda", dtype=torch.int64).reshape(shape))
        elif i < 14:
            args.append((torch.rand(shape, device="cuda", generator=g) * 2 - 1) * 0.05 + (1.0 if i in (5, 11) else 0.0))
        else:
            args.append(torch.zeros(shape, device="cuda"))
    for _ in range(3):
        m.run("main", *args)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        m.run("main", *args)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    # the same step captured once into a CUDA graph (its intermediates become the graph's own allocations) and replayed
    graph_ms = None
    try:
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            m.run("main", *args)
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                m.run("main", *args)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        graph_ms = e0.elapsed_time(e1) / steps
        del graph
    except Exception as exc:  # capture is an extra: report why it was not possible
        graph_ms = f"not captured: {type(exc).__name__}: {str(exc)[:120]}"
        torch.cuda.synchronize()
    plan = m.plan("main").splitlines()[1:]
    kinds = [line.split()[0] for line in plan if line.strip()]
    flops = 2.0 * 8192 * 384 * 50304 * 3 + 2.0 * 8192 * 384 * 1536 * 2 * 3   # vocabulary and FFN contractions, forward + two backward each
    return {"workload": "ltest/test.mlir main: GPT training step, f32 (3xTF32 contractions), through nova_b200_module_run",
            "ms_per_step": ms, "graph_replay_ms_per_step": graph_ms, "steps": steps, "calls_per_step": len(kinds), "contractions_per_step": kinds.count("gemm"),
            "contraction_tflops": flops / (ms * 1e-3) / 1e12,
            "note": "direct calls (no CUDA graph), intermediates from cudaMallocAsync; contraction_tflops counts only the 2MNK of the nine contractions"}


def run_rowop(ctx, w, steps, warmup):
    """HBM roofline of the row-wise kernels: GB/s = (bytes read + bytes written) / event time."""
    from nova_compiler_b200 import ops
    torch = ctx.torch
    desc, dt, rows, D = ROW_WORKLOADS[w]
    tdt = _tdt(torch, dt)
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
    for i in range(max(warmup, 3)):
        fn(i)
    torch.cuda.synchronize()
    # one pass over the input sets captured into a CUDA graph and replayed, as for the contractions: the metric is
    # the kernels' HBM rate, and the host side of a call (allocations of the outputs, the ctypes call) is of the
    # same order as these kernels
    graph = None
    if not ctx.args.no_graph:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for i in range(n_sets):
                fn(i)
        side.synchronize()
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(n_sets):
                    fn(i)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
    sampler = ClockSampler(ctx.local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if graph is not None:
        for _ in range(steps // n_sets):
            graph.replay()
        for i in range(steps % n_sets):
            fn(i)
    else:
        for i in range(steps):
            fn(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    gbs = byts / (ms * 1e-3) / 1e9
    del sets
    torch.cuda.empty_cache()
    return {
        "workload": f"{w}: {desc}", "value": gbs, "unit": "GB/s", "ms_per_step": ms, "steps": steps, "dtype": dt,
        "clocks": clocks, "gpu_launches": steps * {"ln_bwd": 2, "sce": 2}.get(w, 1),  # + column-sum finish / loss kernel
        "l2": f"rotating {n_sets} input sets",
        "launch": "direct calls" if graph is None else f"CUDA graph of {n_sets} steps, replayed",
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": ctx.peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / ctx.peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get(w), "peak_source": ctx.peak_src,
                     "algorithmic_bytes_per_launch": byts, "frac_of_nominal_8000": gbs / 8000.0},
    }


def run_gpu(args):
    ctx = Ctx(args)
    head = args.workload
    if head in ROW_WORKLOADS:
        rec = run_rowop(ctx, head, args.steps or 100, args.warmup if args.warmup is not None else 5)
        line = {"metric": "row-op HBM GB/s", "value": rec["value"], "unit": "GB/s", "n_gpus": 1, "steps": rec["steps"],
                "warmup": max(args.warmup or 5, 3), "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": rec["dtype"], "data": "synthetic (seeded)",
                "impl": "nova_b200", "clocks": rec["clocks"], "gpu_launches": rec["gpu_launches"],
                "config": {"workload": rec["workload"], "l2": rec["l2"]}, "roofline": rec["roofline"]}
        print(json.dumps(line), flush=True)
        return 0
    steps = args.steps or SUB_STEPS[head]
    warmup = args.warmup if args.warmup is not None else 10
    rec = run_contraction(ctx, head, steps, warmup, headline=True)
    subs = {}
    if not args.only and not args.profile:
        for s in DEFAULT_SUBS:
            if s == head:
                continue
            ctx.torch.cuda.synchronize()
            time.sleep(SUB_IDLE_S)
            if s in WORKLOADS:
                r = run_contraction(ctx, s, SUB_STEPS[s], 5)
            elif ctx.world == 1:
                r = run_rowop(ctx, s, 60, 5)
            else:
                r = None  # row kernels are per-row independent: no multi-GPU partition is reported for them
            if r is not None:
                subs[s] = r
    ln_fold = None
    graph_step = None
    if not args.only and not args.profile and ctx.world == 1 and head == "c3":
        time.sleep(SUB_IDLE_S)
        ln_fold = run_ln_fold(ctx)
        time.sleep(SUB_IDLE_S)
        graph_step = run_graph_step(ctx)
    line = None
    if ctx.rank == 0:
        desc = WORKLOADS[head][0]
        part = WORKLOADS[head][8]
        line = {
            "metric": "batch-matmul/linear TFLOPS", "value": rec["value"], "unit": "TFLOP/s", "n_gpus": ctx.world,
            "steps": steps, "warmup": max(warmup, 3), "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": rec["dtype"],
            "data": "synthetic (seeded, shapes and distributions of the config)",
            "config": {"workload": f"{head}: {desc}",
                       "sub_records": f"each starts after {SUB_IDLE_S} s of idle; the headline runs first",
                       "partition": ("one GPU" if ctx.world == 1 else
                                     ("batch index, no collective" if part == "batch" else
                                      "N-column slabs of the one global GEMM, A replicated, no collective")),
                       "l2": rec["l2"], "accumulate": "fp32", "launch": rec["launch"]},
            "impl": "nova_b200", "clocks": rec["clocks"], "e2e": rec.get("e2e"), "gpu_launches": rec["gpu_launches"],
            "roofline": rec["roofline"], "pct_of_bf16_dense_peak_nominal": rec["pct_of_bf16_dense_peak_nominal"],
            "per_gpu": rec["per_gpu"], "plan": rec["plan"],
        }
        for k in ("sustained", "allgather_ms", "allgather", "allgather_fused", "partition", "no_graph_ms_per_step"):
            if k in rec:
                line[k] = rec[k]
        if subs:
            line["workloads"] = subs
        if ln_fold is not None:
            line["ln_fold"] = ln_fold
        if graph_step is not None:
            line["graph_step"] = graph_step
        if ctx.world == 1 and not args.profile and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(head)
    if ctx.world > 1:
        ctx.dist.barrier()
        ctx.dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS) + sorted(ROW_WORKLOADS))
    ap.add_argument("--impl", default="nova_b200", choices=["nova_b200", "reference"])
    ap.add_argument("--only", action="store_true", help="the headline workload only: no `workloads` sub-records")
    ap.add_argument("--no-graph", action="store_true", help="launch every step with a direct call instead of replaying a CUDA graph")
    ap.add_argument("--no-gather", action="store_true", help="skip the (separately timed) all-gather of slab-partitioned outputs")
    ap.add_argument("--no-sustained", action="store_true", help="skip the seconds-long sustained loop of the headline")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--profile", action="store_true",
                    help="device-resident leg of the headline only (no sub-records, end-to-end leg or CPU baseline): for captures under ncu")
    args = ap.parse_args()
    if args.profile:
        args.no_graph = True  # captures under ncu see plain kernel launches
    if args.impl == "reference":
        args.steps = args.steps or 10
        args.warmup = args.warmup if args.warmup is not None else 1
        return run_reference(args)
    return run_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
