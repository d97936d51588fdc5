#!/usr/bin/env python
"""Benchmark of the quantized mul_mat hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

A step is one pass of the hot path over one batch of synthetic input: on-the-fly activation quantization followed by
the quantized mul_mat. The default workload is benchmark configuration 2 (Q8_0 x Q8_0 prefill GEMM, W 11008 x 4096,
M = 512 tokens), the configuration the M = 512 half of the metric is quoted on; the line also carries a `decode` object
(the M = 1 half of the metric: configuration 1, the largest decode shape and the grouped q/k/v launch) and a `sharded`
object (the row-sharded configuration-5 shapes at this number of GPUs). `--workload` makes another configuration the
primary one (cfg1, cfg3-*, cfg4-*, cfg5-*).

Timing: W >= 3 untimed warm-up steps, then exactly K steps on the runtime's stream, timed with CUDA events on that
stream, bracketed by a barrier and a device synchronize, max over ranks. Every step reads a different copy of the
weights from a rotating pool larger than L2. On one GPU the steps are replayed from instantiated batches (CUDA graphs);
`value` is the device-resident throughput; `e2e` goes through the same public API with pinned host buffers, the
host->device copy of the activations and the device->host copy of the result inside the timed region.

With N > 1 (launched by torch.distributed.run):
  * the primary workload runs data-parallel over tokens: every rank holds the whole weight matrix and processes its own
    batch of M tokens, no exchange ("scaling": "weak"; a 47 MB matrix is not worth sharding, a step takes ~50 us);
  * the `sharded` object holds the shapes that are row-sharded over the ranks (configuration 5): every rank computes
    its slice of the output features and the ranks assemble the full [M][N] fp32 output on every rank, inside the timed
    region (strong scaling). `--exchange` selects how: "copy" (each rank's column block is pushed to the peers by the
    copy engines over NVLink, pipelined against the mul_mat of the next token chunk, closed by a flag barrier kernel),
    "fused" (the mul_mat kernels' epilogues store to every rank's output) or "nccl" (all-gather + permute).

`--impl reference` times the CPU implementation of the same path (the oracle: a C restatement of the ggml CPU
arithmetic, or for I2_S the reference's own CPU kernel) on the host cores, on a bounded sample of the workload; under
torch.distributed.run rank 0 alone runs it, with all host threads.
"""
from __future__ import annotations

import argparse
import ctypes
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

Q4_0, Q8_0, Q4_K, I2_S, Q6_K = 2, 8, 12, 36, 14
WORKLOADS = {
    # name: (type, M, N (a tuple: several matrices sharing the activation row, one launch), K, weight std, description)
    "cfg1": (Q4_0, 1, 4096, 4096, 0.02, "Q4_0 x Q8_0 decode GEMV 4096x4096 M=1"),
    "cfg2": (Q8_0, 512, 11008, 4096, 0.02, "Q8_0 x Q8_0 prefill GEMM 11008x4096 M=512"),
    "cfg3-qkvo-m1": (Q4_K, 1, 4096, 4096, 0.02, "Q4_K x Q8_K 4096x4096 M=1"),
    "cfg3-qkv-m1": (Q4_K, 1, (4096, 4096, 4096), 4096, 0.02, "Q4_K x Q8_K q,k,v 3 x 4096x4096 M=1, one launch"),
    "cfg3-gateup-m1": (Q4_K, 1, (11008, 11008), 4096, 0.02, "Q4_K x Q8_K gate,up 2 x 11008x4096 M=1, one launch"),
    "cfg3-gate-m1": (Q4_K, 1, 11008, 4096, 0.02, "Q4_K x Q8_K 11008x4096 M=1"),
    "cfg3-down-m1": (Q4_K, 1, 4096, 11008, 0.02, "Q4_K x Q8_K 4096x11008 M=1"),
    "cfg3-gate-m8": (Q4_K, 8, 11008, 4096, 0.02, "Q4_K x Q8_K 11008x4096 M=8"),
    "cfg3-gate-m512": (Q4_K, 512, 11008, 4096, 0.02, "Q4_K x Q8_K 11008x4096 M=512"),
    "cfg4-gate-m1": (I2_S, 1, 6912, 2560, 1.0, "I2_S x int8 6912x2560 M=1"),
    "cfg4-down-m1": (I2_S, 1, 2560, 6912, 1.0, "I2_S x int8 2560x6912 M=1"),
    "cfg4-gate-m128": (I2_S, 128, 6912, 2560, 1.0, "I2_S x int8 6912x2560 M=128"),
    "cfg5-up-m1": (Q4_K, 1, 28672, 8192, 0.01, "Q4_K x Q8_K 28672x8192 M=1"),
    "cfg5-down-m1": (Q4_K, 1, 8192, 28672, 0.01, "Q4_K x Q8_K 8192x28672 M=1"),
    "cfg5-up-m2048": (Q4_K, 2048, 28672, 8192, 0.01, "Q4_K x Q8_K 28672x8192 M=2048"),
    # not a BASELINE configuration: the Q6_K tensors a Q4_K_M model file carries (ffn_down of a llama-3-8B layer)
    "q6k-down-m1": (Q6_K, 1, 4096, 14336, 0.02, "Q6_K x Q8_K 4096x14336 M=1"),
    "q6k-down-m512": (Q6_K, 512, 4096, 14336, 0.02, "Q6_K x Q8_K 4096x14336 M=512 (ameva_mmtc_b8)"),
}
DECODE_LINES = ("cfg1", "cfg3-qkv-m1", "cfg3-down-m1", "cfg5-up-m1")      # the M = 1 half of the metric, in the default line
SHARDED_LINES = ("cfg5-up-m2048", "cfg5-up-m1")           # the row-sharded shapes, in every line
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel per launch, from the ncu captures summarised under
# profiles/ (bytes), by workload and kernel path
TRAFFIC = {("cfg2", "mmtc"): 57000000, ("cfg5-up-m2048", "mmtc"): 785200000, ("cfg3-gate-m8", "mmvm"): 25424896,
           ("cfg5-up-m1", "mmvs"): 136000000, ("cfg5-up-m1", "mmvq"): 136777216, ("q6k-down-m512", "mmtc"): 101992192}
GEMV_MAX_M = 8


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}


def n_list(N):
    return list(N) if isinstance(N, (tuple, list)) else [N]


def weight_bytes(t, N, K):
    n = sum(n_list(N))
    # (Q6_K: the 274 bytes per block the device layout holds; the ggml block has 210)
    return {Q4_0: 18 * n * K // 32, Q8_0: 34 * n * K // 32, Q4_K: 144 * n * K // 256, I2_S: n * K // 4,
            Q6_K: 274 * n * K // 256}[t]


def algorithmic_bytes(t, M, N, K):
    """packed weights (incl. scales) + fp32 activations read + fp32 output written, per pass."""
    return weight_bytes(t, N, K) + 4 * M * K + 4 * M * sum(n_list(N))


class ClockSampler:
    """Samples nvidia-smi while the timed region runs (reading only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.idx), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def make_inputs(t, M, N, K, std, seed=0):
    """Weights (one ggml block array per matrix of the workload), per-tensor scale, activations."""
    from helpers import make_acts, make_weights
    blocks, scale = [], 1.0
    for j, n in enumerate(n_list(N)):
        b, scale = make_weights(t, n, K, seed + 7 * j, std)
        blocks.append(b)
    return blocks, scale, make_acts(M, K, seed + 1)


def cpu_pass(t, blocks_list, scale, x, N, K, nthreads):
    """One pass of the path on the CPU (quantize activations once + one mul_mat per matrix); returns seconds."""
    import oracle
    M = x.shape[0]
    t0 = time.perf_counter()
    if t in (Q4_0, Q8_0):
        aq = oracle.quantize_q8_0(x)
        for blocks, n in zip(blocks_list, n_list(N)):
            (oracle.mul_mat_q4_0_q8_0 if t == Q4_0 else oracle.mul_mat_q8_0_q8_0)(blocks, aq, M, n, K, False, nthreads)
    elif t == Q4_K:
        aq = oracle.quantize_q8_K(x)
        for blocks, n in zip(blocks_list, n_list(N)):
            oracle.mul_mat_q4_K_q8_K(blocks, aq, M, n, K, False, nthreads)
    elif t == Q6_K:   # (the numpy restatement: one thread)
        from oracle import extra_types
        aq = oracle.quantize_q8_K(x)
        for blocks, n in zip(blocks_list, n_list(N)):
            extra_types.mul_mat_q6_K_q8_K(blocks, aq, M, n, K)
    else:
        q, dq, _ = oracle.quantize_i8_token(x)
        for blocks, n in zip(blocks_list, n_list(N)):
            if oracle.ref_available() and M == 1:   # the reference's own kernel (single vector per call)
                y = oracle.ref_vec_dot_i2_i8_s(blocks, q[0], n, K)
                y *= np.float32(dq[0]) * np.float32(scale)
            else:
                oracle.mul_mat_i2_s_i8(blocks, scale, q, dq, M, n, K, nthreads)
    return time.perf_counter() - t0


def unit_value(unit, t, M, N, K, seconds):
    if unit == "TFLOP/s":
        return 2.0 * M * sum(n_list(N)) * K / seconds / 1e12
    return algorithmic_bytes(t, M, N, K) / seconds / 1e9


def cpu_kind(t, M):
    import oracle
    return "reference" if (t == I2_S and M == 1 and oracle.ref_available()) else "port"


def cpu_build_note():
    import oracle
    return oracle.build_flavour() if hasattr(oracle, "build_flavour") else "portable -O3 build"


def parity_ties(t, x):
    from helpers import count_rounding_ties
    return {"convention": "nearest-even" if t != I2_S else "half-away (the scheme's only one)",
            "exact_half_values": count_rounding_ties(t, x), "values": int(x.size)}


def run_cpu_baseline(t, M, N, K, blocks, scale, x, unit, budget_s=12.0):
    """Times the CPU path on a bounded sample: the first Ms token rows, Ms sized from a probe so the timed pass costs
    roughly budget_s. Returns the cpu_baseline object."""
    import oracle
    kind = cpu_kind(t, M)
    cores = 1 if kind == "reference" else cpu_threads()
    with oracle.timing_build():
        dt = min(cpu_pass(t, blocks, scale, x[:1], N, K, cores) for _ in range(2))
        ms = int(max(1, min(M, budget_s / max(dt, 1e-6))))
        if ms > 1:
            dt = cpu_pass(t, blocks, scale, x[:ms], N, K, cores)
        else:
            reps = int(max(1, min(20, budget_s / max(dt, 1e-6))))
            dt = min(cpu_pass(t, blocks, scale, x[:1], N, K, cores) for _ in range(reps))
        note = cpu_build_note()
    return {"value": unit_value(unit, t, ms, N, K, dt), "unit": unit, "cores": cores, "kind": kind,
            "sample": f"{ms} of {M} token rows x all {sum(n_list(N))} weight rows, one pass, {dt * 1e3:.1f} ms", "build": note}


def workload_config(name):
    t, M, N, K, std, desc = WORKLOADS[name]
    return {"workload": f"{name}: {desc}", "M": M, "N": sum(n_list(N)), "K": K}


def reference_arm(args, name):
    t, M, N, K, std, desc = WORKLOADS[name]
    if int(os.environ.get("RANK", "0")) != 0:
        return
    unit = "TFLOP/s" if M > GEMV_MAX_M else "GB/s"
    import oracle
    blocks, scale, x = make_inputs(t, M, N, K, std)
    kind = cpu_kind(t, M)
    cores = 1 if kind == "reference" else cpu_threads()   # explicit: launchers set OMP_NUM_THREADS=1 for their ranks
    with oracle.timing_build():
        probe = min(cpu_pass(t, blocks, scale, x[:1], N, K, cores) for _ in range(2))
        per_step_budget = max(0.5, 60.0 / max(1, args.steps + args.warmup))
        ms = int(max(1, min(M, per_step_budget / max(probe, 1e-6))))
        for _ in range(args.warmup):
            cpu_pass(t, blocks, scale, x[:ms], N, K, cores)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            cpu_pass(t, blocks, scale, x[:ms], N, K, cores)
        dt = (time.perf_counter() - t0) / args.steps
        note = cpu_build_note()
    val = unit_value(unit, t, ms, N, K, dt)
    sample = f"{ms} of {M} token rows x all {sum(n_list(N))} weight rows per step"
    detail = {"sample": sample, "host": ("CPU restatement of the ggml CPU arithmetic" if kind == "port" else
                                         "reference's own ggml_vec_dot_i2_i8_s (scalar branch)") + ", " + note}
    print(json.dumps({
        "impl": "reference", "metric": metric_name(name), "value": val, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 dot, fp32 accumulate", "data": "synthetic",
        "config": workload_config(name), "config_detail": detail,
        "cpu_baseline": {"value": val, "unit": unit, "cores": cores, "kind": kind, "sample": sample, "build": note},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def metric_name(name):
    t, M, N, K, _, _ = WORKLOADS[name]
    return f"quant mul_mat TFLOPS (% tensor peak) at M={M}" if M > GEMV_MAX_M else \
        f"quant mul_mat GB/s (% of HBM) at M={M}"


class Env:
    """What every measurement shares: the process's rank, the runtime context, its stream as a torch stream."""

    def __init__(self, args):
        import torch
        self.args, self.torch = args, torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist
        self.pkg = importlib.import_module("ameva-compute_b200")
        self.rt, self.qmm, self.shard = self.pkg.runtime, self.pkg.qmm, self.pkg.shard
        self.ctx = self.rt.init()
        # the read-only probe is a measurement aid, not a runtime kernel: its own library adds it to the kernel table
        self.rt.load_library()
        measure = ctypes.CDLL(os.path.join(os.path.dirname(self.rt.LIB_PATH), "libac_b200_measure.so"), mode=ctypes.RTLD_GLOBAL)
        rc = measure.ac_b200_measure_register()
        if rc != 0:
            raise RuntimeError(f"ac_b200_measure_register failed with {rc}")
        self.stream = torch.cuda.ExternalStream(self.ctx.stream, device=torch.device("cuda", self.local_rank))

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        self.ctx.synchronize()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, seconds):
        if self.dist is None:
            return seconds
        tt = self.torch.tensor([seconds], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(tt, op=self.dist.ReduceOp.MAX)
        return float(tt.item())


class Measurement:
    """One workload on this process's GPU. mode: "single" (one GPU), "replicas" (N > 1, every rank the whole matrix and
    its own tokens, no exchange) or "sharded" (N > 1, weight rows split over the ranks, output assembled on every rank)."""

    def __init__(self, env: Env, name: str, mode: str):
        self.env, self.name, self.mode = env, name, mode
        args, rt, qmm, shard, ctx = env.args, env.rt, env.qmm, env.shard, env.ctx
        t, M, N, K, std, desc = WORKLOADS[name]
        self.t, self.M, self.N, self.K, self.desc = t, M, N, K, desc
        self.grouped = isinstance(N, tuple)
        self.Ntot = sum(n_list(N))
        self.unit = "TFLOP/s" if M > GEMV_MAX_M else "GB/s"
        world, rank = (env.world, env.rank) if mode == "sharded" else (1, 0)
        self.blocks, self.scale, self.x = make_inputs(t, M, N, K, std)
        if mode == "replicas":   # every rank its own batch of tokens
            from helpers import make_acts
            self.x = make_acts(M, K, 1 + env.rank)
        if self.grouped and mode == "sharded":
            raise SystemExit("grouped workloads are not sharded")
        n0 = n_list(N)[0]
        self.parts = shard.partition_rows(n0, world)
        self.row0, self.rows = self.parts[rank]
        self.pad = shard.padded_rows(n0, world)
        # rotating pool of weight copies larger than L2, so that no step finds its weights cached
        if self.grouped:
            my_blocks = self.blocks
            self.shard_bytes = weight_bytes(t, N, K)
        else:
            per_row = self.blocks[0].reshape(n0, -1).shape[1]
            my_blocks = [self.blocks[0].reshape(n0, per_row)[self.row0:self.row0 + self.rows]]
            self.shard_bytes = weight_bytes(t, max(self.rows, 1), K)
        self.pool_n = max(2, min(64, -(-2 * L2_BYTES // max(self.shard_bytes, 1)) + 1))
        streamed = {"auto": None, "register": False, "streamed": True, "mma": None}[args.gemv]
        mma = {"auto": None, "register": False, "streamed": False, "mma": True}[args.gemv]
        self.weights, self.mms = [], []
        for _ in range(self.pool_n):
            if self.grouped:
                ws = [qmm.QuantWeight.from_ggml(ctx, t, b, n, K, self.scale) for b, n in zip(my_blocks, n_list(N))]
                self.weights.append(ws)
                self.mms.append(qmm.MulMatGroup(ctx, ws, fused_quantize=args.fused_quantize))
            else:
                w = qmm.QuantWeight.from_ggml(ctx, t, my_blocks[0], self.rows, K, self.scale)
                self.weights.append([w])
                self.mms.append(qmm.MulMat(ctx, w, M, streamed=streamed, mma=mma if t == Q4_K else None,
                                           fused_quantize=args.fused_quantize and mma is not True,
                                           gemm_flags=args.gemm_flags))
        self.x_dev = ctx.buffer(data=self.x)
        self.probe_sink = ctx.buffer(64)
        self.launches_per_step = 0
        self.replay_cache = {}
        self.keep = []
        # output exchange of the sharded run
        self.exchange = "none"
        self.ex = None
        self.gathered_t = self.out_full_t = self.out_local_t = None
        tc_path = (not self.grouped) and M > GEMV_MAX_M and self.mms[0].tc_ok
        if mode == "sharded" and world > 1:
            want = args.exchange
            fused_ok = t != I2_S and (tc_path or (M <= GEMV_MAX_M and K % 256 == 0))
            if want == "fused" and not fused_ok:
                want = "nccl"
            self.exchange = want
        if self.exchange in ("fused", "copy"):
            self.ex = qmm.PeerExchange(ctx, rank, world, M * n0 * 4)
            handles = [None] * world
            env.dist.all_gather_object(handles, self.ex.handles())
            self.ex.connect(handles)
            self.out_buf, self.out_off, self.out_stride, self.out_cols = self.ex.out, self.row0 * 4, n0, n0
        elif self.grouped:
            self.out_bufs = [ctx.buffer(n * 4) for n in n_list(N)]
            self.out_buf, self.out_off, self.out_stride, self.out_cols = self.out_bufs[0], 0, n_list(N)[0], n_list(N)[0]
        else:
            self.out_buf, self.out_off, self.out_stride, self.out_cols = ctx.buffer(M * self.pad * 4), 0, self.pad, self.pad
        if self.exchange == "nccl":
            torch = env.torch
            self.out_local_t = torch.empty((M, self.pad), dtype=torch.float32, device="cuda")
            self.out_buf.destroy()
            self.out_buf = ctx.import_buffer(self.out_local_t.data_ptr(), self.out_local_t.numel() * 4)
            self.gathered_t = torch.empty((world, M, self.pad), dtype=torch.float32, device="cuda")
            self.out_full_t = torch.empty((M, n0), dtype=torch.float32, device="cuda")
        self.world, self.rank = world, rank
        self.exchange_on = True

    # ---- recording -------------------------------------------------------------------------------------------------
    def path(self):
        return self.mms[0].path

    def record_steps(self, batch, n, first, quantize=True):
        ctx = self.env.ctx
        if quantize == "read-probe":   # a plain read of each step's weight region instead of the step
            for i in range(n):
                for w in self.weights[(first + i) % self.pool_n]:
                    batch.dispatch(ctx.kernel("measure_read_probe"), [w.buf, self.probe_sink], [0, 0], (1, 1, 1))
            return
        for i in range(n):
            mm = self.mms[(first + i) % self.pool_n]
            before = batch.stats().dispatches if i == 0 else None
            if self.grouped:
                mm.record(batch, self.x_dev, self.out_bufs, quantize=bool(quantize) or mm.fq)
            elif self.ex and self.exchange == "copy" and self.exchange_on and self.M > GEMV_MAX_M:
                # chunks of token rows: the copy engines move chunk c to the peers while the tensor cores compute c + 1
                chunk = self.env.args.chunk_tokens
                for m0 in range(0, self.M, chunk):
                    mc = min(chunk, self.M - m0)
                    mm.record(batch, self.x_dev, self.out_buf, mc, x_offset=m0 * self.K * 4,
                              dst_offset=self.out_off + m0 * self.out_stride * 4, dst_stride=self.out_stride,
                              quantize=quantize)
                    self.ex.record_copy(batch, m0, mc, self.out_stride, self.row0, self.rows)
                self.ex.record_join(batch)
                self.ex.record_barrier(batch)
            else:
                fused = self.ex and self.exchange == "fused" and self.exchange_on
                mm.record(batch, self.x_dev, self.out_buf, self.M, dst_offset=self.out_off, dst_stride=self.out_stride,
                          quantize=quantize, peers=self.ex.peers if fused else None)
                if self.ex and self.exchange == "copy" and self.exchange_on:
                    self.ex.record_push(batch, self.M, self.out_stride, self.row0, self.rows)   # push + barrier
                elif fused:
                    self.ex.record_barrier(batch)
            if i == 0 and quantize is True:
                self.launches_per_step = batch.stats().dispatches - before

    def use_replay(self):
        # (the copy exchange forks copy queues off the stream at record time; its steps are submitted, not replayed)
        if self.exchange == "copy":
            return self.M <= GEMV_MAX_M and not self.env.args.no_replay
        return self.exchange in ("none", "fused") and not self.env.args.no_replay

    def graph_steps(self, n):
        """Steps per instantiated batch: all n of a short run in one (no launch of a graph inside the timed region but
        the first), else a multiple of the pool that keeps a graph at a few hundred launches."""
        if n <= 128:
            return n
        return self.pool_n * max(1, 96 // self.pool_n)

    def replay_batches(self, quantize, g, rem):
        """(graph of g consecutive steps, graph of the first `rem` steps): every step count replays. The steps of a graph
        cycle through the pool of weight copies."""
        ctx = self.env.ctx
        out = []
        for cnt in (g, rem):
            if not cnt:
                out.append(None)
                continue
            key = (quantize, cnt, self.exchange_on)
            if key not in self.replay_cache:
                rb = ctx.batch(max(64, cnt * 70), 0)
                self.record_steps(rb, cnt, 0, quantize)
                rb.instantiate()
                self.replay_cache[key] = rb
            out.append(self.replay_cache[key])
        return out[0], out[1]

    def gpu_steps(self, n, first, quantize=True, lead_in=False):
        """n steps on the device; returns the GPU seconds by CUDA events on the runtime's stream."""
        env, torch, ctx = self.env, self.env.torch, self.env.ctx
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if self.use_replay():
            g = self.graph_steps(n)
            full, rem = divmod(n, g)
            rb, tail = self.replay_batches(quantize, g, rem)   # instantiated before the timed region
            evs = []
            with torch.cuda.stream(env.stream):
                # untimed replays just ahead: the timed ones are enqueued while the GPU is still busy, so no launch
                # bubble sits behind the start event, and a short run starts as far into a busy period as a long one
                for _ in range(int(lead_in)):
                    evs.append((rb if full else tail).replay())
                start.record()
                for _ in range(full):
                    evs.append(rb.replay())
                if tail is not None:
                    evs.append(tail.replay())
                end.record()
            for ev in evs:
                ev.wait(600_000_000_000)
                ev.destroy()
            end.synchronize()
            return start.elapsed_time(end) / 1e3
        if self.exchange != "nccl":
            per_batch = max(1, min(n, 60000 // 70))   # a batch holds at most 65536 dispatches
            done, pending = 0, []
            with torch.cuda.stream(env.stream):
                start.record()
                while done < n:   # every batch is recorded and submitted before the first wait: the GPU never idles
                    cnt = min(per_batch, n - done)
                    batch = ctx.batch(max(64, cnt * 70), 0)
                    self.record_steps(batch, cnt, first + done, quantize)
                    pending.append((batch, batch.submit()))
                    done += cnt
                end.record()
            for bt, ev in pending:
                ev.wait(600_000_000_000)
                ev.destroy()
                bt.destroy()
            end.synchronize()
            return start.elapsed_time(end) / 1e3
        # all-gather exchange: compute on the runtime's stream, then the NCCL all-gather and the permute, in stream order
        dist, shard = env.dist, env.shard
        with torch.cuda.stream(env.stream):
            start.record()
            for i in range(n):
                batch = ctx.batch(128, 0)
                self.record_steps(batch, 1, first + i)
                batch.flush()
                dist.all_gather_into_tensor(self.gathered_t.view(self.world * self.M, self.pad), self.out_local_t)
                shard.assemble(self.gathered_t, self.parts, self.M, n_list(self.N)[0], self.out_full_t)
                self.keep.append(batch)
            end.record()
            end.synchronize()
        for b_ in self.keep:
            b_.destroy()
        self.keep.clear()
        return start.elapsed_time(end) / 1e3

    # ---- the measurements ------------------------------------------------------------------------------------------
    def lead_in_replays(self, steps):
        """Untimed replays of the timed graph enqueued directly ahead of the start event: about `lead_in_ms` of GPU work
        (from the step time of the untimed first launch of the graphs), at least one."""
        est = getattr(self, "step_estimate_s", None)
        ms = float(os.environ.get("AMEVA_BENCH_LEAD_IN_MS", "8"))
        if not est or ms <= 0:
            return 1
        g = self.graph_steps(steps)
        per_replay = est * (g if steps >= g else steps)
        return max(1, min(64, int(ms * 1e-3 / per_replay + 0.5)))

    def timed(self, steps, warmup):
        env = self.env
        self.gpu_steps(warmup, 0)
        if self.use_replay():   # the graphs of the timed run have been launched once before it is timed
            # (the same estimate on every rank: ranks that exchange outputs must enqueue the same number of replays)
            self.step_estimate_s = env.max_over_ranks(self.gpu_steps(steps, warmup) / steps)
        env.barrier()
        lead = self.lead_in_replays(steps) if self.use_replay() else 0
        t0 = time.perf_counter()
        gpu_s = self.gpu_steps(steps, warmup, lead_in=lead)
        env.barrier()
        g = self.graph_steps(steps)
        self.wall_steps = steps + lead * (g if steps >= g else steps)   # steps the host clock below covers
        self.wall_s = time.perf_counter() - t0
        return env.max_over_ranks(gpu_s)

    def roofline(self, steps, warmup, step_s):
        """Average launch duration of the dominant kernel, live: the mul_mat kernel alone (activations already quantized
        by the steps before), the same rotation of weight copies, back to back on the launching stream between two CUDA
        events; the quantize kernel's share is the rest of a step. A step that is one launch is timed as it is."""
        one_launch = self.path() in ("mmvq-fq", "mmvqg-fq")
        if self.use_replay():
            self.gpu_steps(steps, warmup + steps, quantize=True if one_launch else False)   # first launch of its graphs
        main_s = self.gpu_steps(steps, warmup + steps, quantize=True if one_launch else False,
                                lead_in=self.lead_in_replays(steps))
        main_ns = main_s / steps * 1e9
        quant_ns = max(0.0, step_s * 1e9 - main_ns)
        pk = peaks()
        t, M, N, K = self.t, self.M, self.N, self.K
        if self.unit == "TFLOP/s":
            ach = 2.0 * M * self.Ntot * K / (main_ns * 1e-9) / 1e12
            return {"bound": "tensor", "achieved": ach, "peak": pk["tflops"], "unit": "TFLOP/s",
                    "frac": ach / pk["tflops"], "traffic": TRAFFIC.get((self.name, self.path())),
                    "peak_source": pk["source"] + " bf16 burst", "kernel_us": main_ns / 1e3, "quant_us": quant_ns / 1e3}
        ach = algorithmic_bytes(t, M, N, K) / (main_ns * 1e-9) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
                "traffic": TRAFFIC.get((self.name, self.path())), "peak_source": pk["source"] + " copy",
                "kernel_us": main_ns / 1e3, "quant_us": quant_ns / 1e3}
        # what a kernel that only reads the same weight regions takes (same rotation, same timing): the ramp and the tail
        # of a launch this short keep a pure read well under the copy peak
        if self.use_replay():
            self.gpu_steps(steps, warmup + steps, quantize="read-probe")
        probe_s = self.gpu_steps(steps, warmup + steps, quantize="read-probe", lead_in=self.lead_in_replays(steps))
        roof["read_only_us"] = probe_s / steps * 1e6
        roof["read_only_gbs"] = sum(w.buf.size_bytes for w in self.weights[0]) / (probe_s / steps) / 1e9
        roof["frac_of_read_only"] = roof["read_only_us"] / roof["kernel_us"]
        return roof

    def read_result(self):
        """The last step's output on the host, [M][columns]."""
        if self.grouped:
            return np.concatenate([b.read(np.float32) for b in self.out_bufs]).reshape(1, -1)
        if self.exchange == "nccl":
            return self.out_full_t.cpu().numpy()
        return self.out_buf.read(np.float32, self.M * self.out_cols).reshape(self.M, self.out_cols)

    def parity(self, got):
        """First token rows x a sample of weight rows of the first and, when sharded, also of the last rank's shard, so a
        wrong kernel or exchange cannot post a number."""
        from helpers import max_normalised_error, oracle_mul_mat
        t, K = self.t, self.K
        ms = min(self.M, 4)
        worst = 0.0
        if self.grouped:
            col = 0
            for blocks, n in zip(self.blocks, n_list(self.N)):
                ns = min(n, 256)
                per_row = blocks.reshape(n, -1).shape[1]
                want, _, _ = oracle_mul_mat(t, np.ascontiguousarray(blocks.reshape(n, per_row)[:ns]), self.scale,
                                            self.x[:ms], ns, K, want_sums=False)
                worst = max(worst, max_normalised_error(got[:ms, col:col + ns], want))
                col += n
            return worst
        n0 = n_list(self.N)[0]
        allb = self.blocks[0].reshape(n0, -1)
        full = self.exchange != "none"
        spans = [(self.row0, min(self.rows, 512), self.row0 if full else 0)]
        if full:
            lr0, lrows = self.parts[-1]
            spans.append((lr0, min(lrows, 256), lr0))
        for g_row0, g_n, col0 in spans:
            want, _, _ = oracle_mul_mat(t, np.ascontiguousarray(allb[g_row0:g_row0 + g_n]), self.scale, self.x[:ms], g_n,
                                        K, want_sums=False)
            worst = max(worst, max_normalised_error(got[:ms, col0:col0 + g_n], want))
        return worst

    def e2e(self, steps):
        """End to end through the public API with host buffers: H2D of the activations, compute, D2H of the result, per
        step. One GPU per rank, software-pipelined when a step moves at least 1 MB: the activations of step i+1 travel
        host->device and the result of step i-1 device->host on two copy streams while step i computes (double-buffered
        device input and output imported into the runtime; events order the three streams)."""
        env, torch, ctx = self.env, self.env.torch, self.env.ctx
        M, K = self.M, self.K
        x_pin = torch.from_numpy(self.x).pin_memory()
        d2h_bytes = M * self.out_cols * 4 if not self.grouped else self.Ntot * 4
        y_pin = torch.empty((M, d2h_bytes // 4 // M), dtype=torch.float32).pin_memory()
        overlap = (self.exchange == "none" and not self.grouped and not env.args.no_overlap
                   and self.x.nbytes + d2h_bytes >= (1 << 20))
        if not overlap:
            mode = "sequential on the runtime's stream"

            def run(n, first):
                with torch.cuda.stream(env.stream):
                    for i in range(n):
                        self.x_dev.write_async(x_pin.data_ptr(), self.x.nbytes)
                        batch = ctx.batch(128, 0)
                        self.record_steps(batch, 1, first + i)
                        batch.flush()
                        self.keep.append(batch)
                        if self.exchange == "nccl":
                            env.dist.all_gather_into_tensor(self.gathered_t.view(self.world * M, self.pad), self.out_local_t)
                            env.shard.assemble(self.gathered_t, self.parts, M, n_list(self.N)[0], self.out_full_t)
                        if self.grouped:
                            off = 0
                            for b_, n_ in zip(self.out_bufs, n_list(self.N)):
                                b_.read_async(y_pin.data_ptr() + off, n_ * 4)
                                off += n_ * 4
                        else:
                            self.out_buf.read_async(y_pin.data_ptr(), d2h_bytes)
                ctx.synchronize()
                for bb in self.keep:
                    bb.destroy()
                self.keep.clear()
            cleanup = []
        else:
            mode = "pipelined: H2D, compute and D2H of neighbouring steps overlap on three streams"
            NBUF = 2
            x_t = [torch.empty((M, K), dtype=torch.float32, device="cuda") for _ in range(NBUF)]
            o_t = [torch.empty((M, self.out_cols), dtype=torch.float32, device="cuda") for _ in range(NBUF)]
            x_b = [ctx.import_buffer(tt_.data_ptr(), tt_.numel() * 4) for tt_ in x_t]
            o_b = [ctx.import_buffer(tt_.data_ptr(), tt_.numel() * 4) for tt_ in o_t]
            y_pins = [y_pin] + [torch.empty((M, self.out_cols), dtype=torch.float32).pin_memory() for _ in range(NBUF - 1)]
            s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
            cleanup = x_b + o_b

            def run(n, first):
                ev_cmp, ev_out = [None] * NBUF, [None] * NBUF
                for i in range(n):
                    b_ = i % NBUF
                    with torch.cuda.stream(s_in):
                        if ev_cmp[b_] is not None:
                            s_in.wait_event(ev_cmp[b_])          # the step that last read this input buffer has finished
                        x_t[b_].copy_(x_pin, non_blocking=True)
                        ev_in = torch.cuda.Event()
                        ev_in.record(s_in)
                    with torch.cuda.stream(env.stream):
                        env.stream.wait_event(ev_in)
                        if ev_out[b_] is not None:
                            env.stream.wait_event(ev_out[b_])    # the result that last used this output buffer is on the host
                        batch = ctx.batch(128, 0)
                        self.mms[(first + i) % self.pool_n].record(batch, x_b[b_], o_b[b_], M, dst_stride=self.out_stride)
                        batch.flush()
                        self.keep.append(batch)
                        ev_cmp[b_] = torch.cuda.Event()
                        ev_cmp[b_].record(env.stream)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(ev_cmp[b_])
                        y_pins[b_].copy_(o_t[b_], non_blocking=True)
                        ev_out[b_] = torch.cuda.Event()
                        ev_out[b_].record(s_out)
                torch.cuda.synchronize()
                ctx.synchronize()
                for bb in self.keep:
                    bb.destroy()
                self.keep.clear()

        run(3, 0)
        env.barrier()
        t0 = time.perf_counter()
        run(steps, 3)
        env.barrier()
        e2e_s = env.max_over_ranks(time.perf_counter() - t0)
        for ib in cleanup:
            ib.destroy()
        units = self.world_units()
        return {"value": unit_value(self.unit, self.t, self.M * units, self.N, self.K, e2e_s / steps), "unit": self.unit,
                "h2d_bytes_per_step": int(self.x.nbytes), "d2h_bytes_per_step": int(d2h_bytes),
                "ms_per_step": e2e_s / steps * 1e3, "mode": mode}, y_pin.numpy()

    def world_units(self):
        """How many independent batches one step of the whole job processes (replicas: one per rank)."""
        return self.env.world if self.mode == "replicas" else 1

    def destroy(self):
        for rb in self.replay_cache.values():
            rb.destroy()
        for mm in self.mms:
            mm.destroy()
        for ws in self.weights:
            for w in ws:
                w.destroy()
        self.x_dev.destroy()
        self.probe_sink.destroy()
        if self.ex:
            self.ex.destroy()
        elif self.grouped:
            for b in self.out_bufs:
                b.destroy()
        else:
            self.out_buf.destroy()


def sub_line(env, name, mode, steps, warmup, want_roof):
    """A compact record of one more workload for the `decode` / `sharded` objects of the line."""
    m = Measurement(env, name, mode)
    try:
        step_s = m.timed(steps, warmup) / steps
        t, M, N, K = m.t, m.M, m.N, m.K
        rec = {"workload": f"{name}: {m.desc}", "value": unit_value(m.unit, t, M, N, K, step_s), "unit": m.unit,
               "ms_per_step": step_s * 1e3, "steps": steps, "path": m.path(), "exchange": m.exchange}
        if want_roof and env.world == 1:
            r = m.roofline(steps, warmup, step_s)
            rec.update({k: r[k] for k in ("kernel_us", "frac", "achieved", "peak", "bound") if k in r})
            for k in ("read_only_us", "frac_of_read_only"):
                if k in r:
                    rec[k] = r[k]
        if mode == "sharded" and env.world > 1:
            # what crossed NVLink per rank and direction in a step: every other rank's share of the fp32 output comes in
            n0 = n_list(N)[0]
            in_bytes = 4 * M * (n0 - m.rows)
            rec["nvlink_in_bytes_per_rank"] = int(in_bytes)
            rec["nvlink_in_gbs_per_rank"] = in_bytes / step_s / 1e9
            m.exchange_on = False      # the same kernels on the rank's slice without the exchange: what the exchange costs
            rec["kernel_only_ms_per_step"] = m.timed(steps, warmup) / steps * 1e3
            m.exchange_on = True
        if env.rank == 0:
            rec["parity_max_normalised_error"] = m.parity(m.read_result())
            rec["parity_rounding_ties"] = parity_ties(m.t, m.x)
        return rec
    finally:
        env.barrier()
        m.destroy()


def layer_op_lines(env, steps=3):
    """The HBM-bound ops next to the mul_mat in a decoder (1 GPU): the f16 LM-head GEMV (BitNet-2B: 128256 x 2560) and
    token-generation attention over an f16 KV cache (32 heads on 8 KV heads of 128, one cache per layer, the layers'
    caches together larger than L2). Replayed batches of one launch per layer, CUDA events on the launching stream;
    `frac` is algorithmic bytes / time over the measured copy bandwidth."""
    import struct
    torch, ctx = env.torch, env.ctx
    pk = peaks()

    def fbits(v):
        return struct.unpack("<I", struct.pack("<f", float(v)))[0]

    def timed(record, launches):
        batch = ctx.batch(4 * launches + 8, 0)
        record(batch)
        batch.instantiate()
        secs = None
        try:
            for it in range(2 + steps):
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.stream(env.stream):
                    lead = batch.replay()
                    start.record()
                    evs = [batch.replay() for _ in range(steps)]
                    end.record()
                for ev in [lead] + evs:
                    ev.wait(600_000_000_000)
                    ev.destroy()
                end.synchronize()
                secs = start.elapsed_time(end) / 1e3 / (steps * launches)
        finally:
            batch.destroy()
        return secs

    out = {}
    rng = np.random.default_rng(0)
    # ---- LM head: one buffer of 657 MB, read once per launch ----
    n_rows, n_in, launches = 128256, 2560, 8
    W = (rng.standard_normal((n_rows, n_in), dtype=np.float32) * 0.02).astype(np.float16)
    x = rng.standard_normal(n_in).astype(np.float32)
    wb, xb, yb = ctx.buffer(data=W), ctx.buffer(data=x), ctx.buffer(n_rows * 4)
    kern = ctx.kernel("bitnet_gemv_f16_w4")
    s = timed(lambda b: [b.dispatch(kern, [wb, xb, yb], [n_in, n_rows, 0], (1, 1, 1)) for _ in range(launches)], launches)
    y = yb.read(np.float32)
    rows = rng.integers(0, n_rows, 512)
    want = W[rows].astype(np.float64) @ x.astype(np.float64)
    norm = np.abs(W[rows].astype(np.float64)) @ np.abs(x.astype(np.float64))
    nbytes = n_rows * n_in * 2 + n_in * 4 + n_rows * 4
    out["lm_head_f16"] = {"workload": f"f16 GEMV {n_rows}x{n_in} M=1 (bitnet_gemv_f16)", "us": s * 1e6,
                          "achieved": nbytes / s / 1e9, "unit": "GB/s", "peak": pk["hbm_gbs"], "frac": nbytes / s / 1e9 / pk["hbm_gbs"],
                          "parity_max_normalised_error": float(np.max(np.abs(y[rows] - want) / norm))}
    for b in (wb, xb, yb):
        b.destroy()
    del W
    # ---- attention at token generation ----
    D, n_head, n_head_kv, n_q = 128, 32, 8, 1
    fk = ctx.kernel("ameva_flash_attn")
    for label, n_kv, layers in (("flash_decode_4k", 4096, 32), ("flash_decode_32k", 32768, 4)):
        kv = (rng.standard_normal((n_head_kv, n_kv, D), dtype=np.float32)).astype(np.float16)
        ks = [ctx.buffer(data=kv) for _ in range(layers)]
        vs = [ctx.buffer(data=kv[::-1].copy()) for _ in range(layers)]
        q = rng.standard_normal((n_head, n_q, D)).astype(np.float32)
        mask = np.zeros((n_q, n_kv), np.float16)
        qb, mb, ob, pb = ctx.buffer(data=q), ctx.buffer(data=mask), ctx.buffer(n_q * n_head * D * 4), ctx.buffer(16 << 20)
        push = [D, D, n_kv, n_q, n_head, n_head_kv, 0x11, 1, 0, D, D * n_q, 0, D, D * n_kv, 0, D, D * n_kv, 0, n_kv, 0,
                1, 0, fbits(1.0 / np.sqrt(D)), 0, 0, 0, 0, 0, 0, 0, 0]
        s = timed(lambda b: [b.dispatch(fk, [qb, ks[i], vs[i], mb, ob, pb], push, (1, 1, 1)) for i in range(layers)], layers)
        got = ob.read(np.float32).reshape(n_q, n_head, D)
        kd, vd = kv.astype(np.float64), kv[::-1].astype(np.float64)
        worst = 0.0
        for h in (0, 13, 31):
            sc = (q[h, 0].astype(np.float64) @ kd[h // 4].T) / np.sqrt(D)
            p = np.exp(sc - sc.max())
            worst = max(worst, float(np.max(np.abs(got[0, h] - (p @ vd[h // 4]) / p.sum()))))
        nbytes = 2 * n_head_kv * n_kv * D * 2 + n_kv * 2 + q.nbytes + n_q * n_head * D * 4
        out[label] = {"workload": f"attention, 1 query x {n_kv} cached positions, {n_head} heads on {n_head_kv} KV heads of {D}, "
                                  f"f16 cache, {layers} caches in rotation ({layers * 2 * kv.nbytes / 1e6:.0f} MB)",
                      "us": s * 1e6, "achieved": nbytes / s / 1e9, "unit": "GB/s", "peak": pk["hbm_gbs"],
                      "frac": nbytes / s / 1e9 / pk["hbm_gbs"], "launches_per_step": 2, "parity_max_abs_error": worst}
        for b in ks + vs + [qb, mb, ob, pb]:
            b.destroy()
    # ---- attention over a prompt: 512 positions against themselves under a causal mask (tensor-bound, mma.sync) ----
    n_q = n_kv = 512
    kv = (rng.standard_normal((n_head_kv, n_kv, D), dtype=np.float32)).astype(np.float16)
    q = rng.standard_normal((n_head, n_q, D)).astype(np.float32)
    mask = np.triu(np.full((n_q, n_kv), -np.inf, np.float16), 1)
    kb, vb, qb, mb = ctx.buffer(data=kv), ctx.buffer(data=kv[::-1].copy()), ctx.buffer(data=q), ctx.buffer(data=mask)
    ob, pb = ctx.buffer(n_q * n_head * D * 4), ctx.buffer(16 << 20)
    push = [D, D, n_kv, n_q, n_head, n_head_kv, 0x11, 1, 0, D, D * n_q, 0, D, D * n_kv, 0, D, D * n_kv, 0, n_kv, 0,
            1, 0, fbits(1.0 / np.sqrt(D)), 0, 0, 0, 0, 0, 0, 0, 0]
    s = timed(lambda b: [b.dispatch(fk, [qb, kb, vb, mb, ob, pb], push, (1, 1, 1)) for _ in range(4)], 4)
    got = ob.read(np.float32).reshape(n_q, n_head, D)
    kd, vd = kv.astype(np.float64), kv[::-1].astype(np.float64)
    worst = 0.0
    for h, i in ((0, 0), (13, 200), (31, 511)):
        sc = (q[h, i].astype(np.float64) @ kd[h // 4, :i + 1].T) / np.sqrt(D)
        p = np.exp(sc - sc.max())
        worst = max(worst, float(np.max(np.abs(got[i, h] - (p @ vd[h // 4, :i + 1]) / p.sum()))))
    flops = 4.0 * n_head * D * (n_q * (n_q + 1) / 2)     # the unmasked half of both products
    out["flash_prompt_512"] = {"workload": f"attention, {n_q} query positions x {n_kv} keys, causal, {n_head} heads on "
                                           f"{n_head_kv} KV heads of {D}, f16 K / V", "us": s * 1e6,
                               "achieved": flops / s / 1e12, "unit": "TFLOP/s (unmasked products)",
                               "parity_max_abs_error": worst}
    for b in (kb, vb, qb, mb, ob, pb):
        b.destroy()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="leave the `decode` object out of the line")
    ap.add_argument("--no-sharded", action="store_true", help="leave the `sharded` object out of the line")
    ap.add_argument("--no-layer-ops", action="store_true", help="leave the `layer_ops` object out of the line")
    ap.add_argument("--sharded-primary", action="store_true",
                    help="N > 1: row-shard the primary workload too (strong scaling) instead of token-parallel replicas")
    ap.add_argument("--exchange", choices=["copy", "fused", "nccl"], default="fused",
                    help="how the ranks of a row-sharded mul_mat assemble the output (see the module docstring)")
    ap.add_argument("--chunk-tokens", type=int, default=256,
                    help="copy exchange, more than 8 token rows: token rows per mul_mat + copy chunk")
    ap.add_argument("--no-replay", action="store_true", help="one host launch per kernel instead of replayed batches")
    ap.add_argument("--no-overlap", action="store_true", help="e2e: copies and compute in sequence on one stream")
    ap.add_argument("--gemm-flags", type=int, default=0,
                    help="launch switches of the tensor-core GEMM (64: one tile per unit, 128: one accumulator per CTA pair)")
    ap.add_argument("--gemv", choices=["auto", "register", "streamed", "mma"], default="auto",
                    help="M <= 8: register-staged kernels (ameva_mmvq*), the one that stages the weight rows in shared "
                         "memory (ameva_mmvs_*), or the library's own choice")
    ap.add_argument("--fused-quantize", action="store_true",
                    help="M == 1, small projections: quantize inside the GEMV launch (ameva_mmv*_fq); in replayed batches "
                         "the two-kernel sequence measures as fast, it saves a host launch otherwise")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    name = args.workload
    if args.impl == "reference":
        reference_arm(args, name)
        return

    env = Env(args)
    world, rank = env.world, env.rank
    t, M, N, K, std, desc = WORKLOADS[name]
    mode = "single" if world == 1 else ("sharded" if args.sharded_primary else "replicas")
    m = Measurement(env, name, mode)
    units = m.world_units()

    sampler = ClockSampler(env.local_rank)
    sampler.start()
    gpu_s = m.timed(args.steps, args.warmup)   # warm-up, first launch of the timed graphs, then the timed region
    step_s = gpu_s / args.steps

    roof = m.roofline(args.steps, args.warmup, step_s) if world == 1 else None
    e2e, y_host = m.e2e(args.steps)
    clocks = sampler.stop()
    check = m.parity(y_host) if rank == 0 and m.rows else None

    decode = sharded = None
    sub_steps = 200   # (decode steps take microseconds: enough of them to amortise the replay launches, whatever --steps is)
    if not args.no_decode and world == 1 and name == "cfg2":
        decode = {w: sub_line(env, w, "single", sub_steps, 5, True) for w in DECODE_LINES}
    if not args.no_sharded and name == "cfg2":
        sharded = {w: sub_line(env, w, "sharded" if world > 1 else "single", max(10, min(sub_steps, 50)) if
                               WORKLOADS[w][1] > GEMV_MAX_M else sub_steps, 3, False) for w in SHARDED_LINES}
    layer_ops = None
    if not args.no_layer_ops and world == 1 and name == "cfg2":
        try:
            layer_ops = layer_op_lines(env)
        except Exception as e:   # (an aid beside the metric: its failure is reported, the line still goes out)
            layer_ops = {"error": repr(e)}

    if rank == 0:
        par = {"single": "single GPU",
               "replicas": f"data-parallel over tokens: {world} ranks, each with the whole weight matrix and its own batch of "
                           f"{M} tokens, no exchange",
               "sharded": f"weight rows sharded over {world} ranks, output assembled on every rank ({m.exchange})"}[mode]
        detail = ({"l2": f"rotating pool of {m.pool_n} weight copies ({m.pool_n * m.shard_bytes / 1e6:.0f} MB > L2) per rank",
                    "parallelism": par, "path": m.path(),
                    "launch": f"replayed batches (CUDA graphs of {m.graph_steps(args.steps)} steps, cycling the pool, + one of the remainder; the graphs are launched once untimed, and untimed replays (about 8 ms of them) are enqueued just ahead of the start event so that the timed ones are submitted while the GPU is busy)" if
                    m.use_replay() else "one host launch per kernel"})
        line = {
            "metric": metric_name(name), "value": unit_value(m.unit, t, M * units, N, K, step_s), "unit": m.unit,
            "n_gpus": env.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
            "higher_is_better": True, "scaling": "strong" if mode == "sharded" else "weak", "vs_baseline": None,
            "dtype": {"mmtc": "int8 (tcgen05 kind::i8, int32 accumulate)" if t == I2_S else
                      "f16 (tcgen05 kind::f16 on dequantized fp16 operands, fp32 accumulate in TMEM)"}.get(
                          m.path().split("+")[0], "int8 (dp4a, int32 per block, fp32 scale-accumulate)"),
            "data": "synthetic",
            "config": workload_config(name), "config_detail": detail,
            "wall_ms_per_step": m.wall_s / m.wall_steps * 1e3,
            "gpu_launches": m.launches_per_step * args.steps,
            "e2e": e2e,
            "clocks": clocks,
            "parity_max_normalised_error": check,
            # exact .5 values in this input's activation quantization (where nearest-even and half-away differ; the
            # kernels and the oracle share one switch, default nearest-even)
            "parity_rounding_ties": parity_ties(t, m.x),
        }
        if roof:
            line["roofline"] = roof
        if decode:
            line["decode"] = decode
        if sharded:
            line["sharded"] = sharded
        if layer_ops:
            line["layer_ops"] = layer_ops
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = run_cpu_baseline(t, M, N, K, m.blocks, m.scale, m.x, m.unit)
        print(json.dumps(line), flush=True)

    if env.dist is not None:   # nobody unmaps a buffer a peer may still be writing; and never hang after the line is out
        threading.Timer(60.0, lambda: os._exit(0)).start()
        env.barrier()
    m.destroy()
    env.ctx.destroy()
    if env.dist is not None:
        env.dist.destroy_process_group()
        os._exit(0)


if __name__ == "__main__":
    main()
