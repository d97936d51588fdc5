#!/usr/bin/env python
"""Benchmark of the quantized mul_mat hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

A step is one pass of the hot path over one batch of synthetic input: on-the-fly activation quantization followed by
the quantized mul_mat. The default workload is benchmark configuration 2 (Q8_0 x Q8_0 prefill GEMM, W 11008 x 4096,
M = 512 tokens); `--workload` selects another configuration (cfg1, cfg3-*, cfg4-*, cfg5-*).

Timing: W >= 3 untimed warm-up steps, then exactly K steps recorded into one batch on the runtime's stream and timed
with CUDA events on that stream, bracketed by a barrier and a device synchronize, max over ranks. Every step reads a
different copy of the weights from a rotating pool larger than L2. `value` is the device-resident throughput; `e2e` goes
through the same public API with host buffers (pinned), the host->device copy of the activations and the device->host
copy of the result inside the timed region.

With N > 1 (launched by torch.distributed.run) the weight rows are sharded over the ranks (strong scaling: the total
work is fixed). Every rank owns a full [M][N] output shared with the other ranks over CUDA IPC; the mul_mat's epilogue
stores the rank's rows into every rank's output over NVLink and a flag barrier kernel closes the step, so the exchange
is part of this library's kernels and of the timed region. Kernels without that epilogue (I2_S) fall
back to an NCCL all-gather of the fp32 output plus a permute, also inside the timed region.

`--impl reference` times the CPU implementation of the same path (the oracle: a C restatement of the ggml CPU
arithmetic, or for I2_S the reference's own CPU kernel) on the host cores, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
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

Q4_0, Q8_0, Q4_K, I2_S = 2, 8, 12, 36
WORKLOADS = {
    # name: (type, M, N, K, weight std, description)
    "cfg1": (Q4_0, 1, 4096, 4096, 0.02, "Q4_0 x Q8_0 decode GEMV 4096x4096 M=1"),
    "cfg2": (Q8_0, 512, 11008, 4096, 0.02, "Q8_0 x Q8_0 prefill GEMM 11008x4096 M=512"),
    "cfg3-qkvo-m1": (Q4_K, 1, 4096, 4096, 0.02, "Q4_K x Q8_K 4096x4096 M=1"),
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
}
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel per launch, from the ncu captures summarised under
# profiles/ (bytes), by workload and kernel path
TRAFFIC = {("cfg2", "mmtc"): 58200000, ("cfg5-up-m1", "mmvs"): 136000000, ("cfg5-up-m1", "mmvq"): 136777216}
GEMV_MAX_M = 8


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}


def weight_bytes(t, N, K):
    return {Q4_0: 18 * N * K // 32, Q8_0: 34 * N * K // 32, Q4_K: 144 * N * K // 256, I2_S: N * K // 4}[t]


def algorithmic_bytes(t, M, N, K):
    """packed weights (incl. scales) + fp32 activations read + fp32 output written, per pass."""
    return weight_bytes(t, N, K) + 4 * M * K + 4 * M * N


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
    from helpers import make_acts, make_weights
    blocks, scale = make_weights(t, N, K, seed, std)
    return blocks, scale, make_acts(M, K, seed + 1)


def cpu_pass(t, blocks, scale, x, N, K, nthreads=0):
    """One pass of the path on the CPU (quantize activations + mul_mat); returns seconds."""
    import oracle
    M = x.shape[0]
    t0 = time.perf_counter()
    if t in (Q4_0, Q8_0):
        aq = oracle.quantize_q8_0(x)
        (oracle.mul_mat_q4_0_q8_0 if t == Q4_0 else oracle.mul_mat_q8_0_q8_0)(blocks, aq, M, N, K, False, nthreads)
    elif t == Q4_K:
        oracle.mul_mat_q4_K_q8_K(blocks, oracle.quantize_q8_K(x), M, N, K, False, nthreads)
    else:
        q, dq, _ = oracle.quantize_i8_token(x)
        if oracle.ref_available() and M == 1:   # the reference's own kernel (single vector per call)
            y = oracle.ref_vec_dot_i2_i8_s(blocks, q[0], N, K)
            y *= np.float32(dq[0]) * np.float32(scale)
        else:
            oracle.mul_mat_i2_s_i8(blocks, scale, q, dq, M, N, K, nthreads)
    return time.perf_counter() - t0


def unit_value(unit, t, M, N, K, seconds):
    if unit == "TFLOP/s":
        return 2.0 * M * N * K / seconds / 1e12
    return algorithmic_bytes(t, M, N, K) / seconds / 1e9


def run_cpu_baseline(t, M, N, K, blocks, scale, x, unit, budget_s=15.0):
    """Times the CPU path on a bounded sample: the first Ms token rows, Ms sized from a probe so the timed pass costs
    roughly budget_s. Returns the cpu_baseline object."""
    import oracle
    kind = "reference" if (t == I2_S and M == 1 and oracle.ref_available()) else "port"
    cores = 1 if kind == "reference" else min(cpu_threads(), oracle.num_threads())
    probe_m = 1
    dt = cpu_pass(t, blocks, scale, x[:probe_m], N, K)
    dt = min(dt, cpu_pass(t, blocks, scale, x[:probe_m], N, K))
    ms = int(max(1, min(M, budget_s / max(dt, 1e-6))))
    if ms > 1:
        dt = cpu_pass(t, blocks, scale, x[:ms], N, K)
    else:
        reps = int(max(1, min(200, budget_s / max(dt, 1e-6))))
        dt = min(cpu_pass(t, blocks, scale, x[:1], N, K) for _ in range(min(reps, 20)))
    return {"value": unit_value(unit, t, ms, N, K, dt), "unit": unit, "cores": cores, "kind": kind,
            "sample": f"{ms} of {M} token rows x all {N} weight rows, one pass, {dt * 1e3:.1f} ms"}


def reference_arm(args, name):
    t, M, N, K, std, desc = WORKLOADS[name]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    unit = "TFLOP/s" if M > GEMV_MAX_M else "GB/s"
    import oracle
    blocks, scale, x = make_inputs(t, M, N, K, std)
    probe = min(cpu_pass(t, blocks, scale, x[:1], N, K) for _ in range(2))
    per_step_budget = max(0.5, 60.0 / max(1, args.steps + args.warmup))
    ms = int(max(1, min(M, per_step_budget / max(probe, 1e-6))))
    for _ in range(args.warmup):
        cpu_pass(t, blocks, scale, x[:ms], N, K)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(t, blocks, scale, x[:ms], N, K)
    dt = (time.perf_counter() - t0) / args.steps
    val = unit_value(unit, t, ms, N, K, dt)
    kind = "reference" if (t == I2_S and ms == 1 and oracle.ref_available()) else "port"
    cores = 1 if kind == "reference" else min(cpu_threads(), oracle.num_threads())
    sample = f"{ms} of {M} token rows x all {N} weight rows per step"
    print(json.dumps({
        "impl": "reference", "metric": metric_name(name), "value": val, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 dot, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"{name}: {desc}", "sample": sample, "host": "CPU restatement of the ggml CPU arithmetic"
                   if kind == "port" else "reference's own ggml_vec_dot_i2_i8_s (scalar branch)"},
        "cpu_baseline": {"value": val, "unit": unit, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def metric_name(name):
    t, M, N, K, _, _ = WORKLOADS[name]
    return f"quant mul_mat TFLOPS (% tensor peak) at M={M}" if M > GEMV_MAX_M else \
        f"quant mul_mat GB/s (% of HBM) at M={M}"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-replay", action="store_true", help="one host launch per kernel instead of replayed batches")
    ap.add_argument("--no-overlap", action="store_true", help="e2e: copies and compute in sequence on one stream")
    ap.add_argument("--gemv", choices=["auto", "register", "streamed"], default="auto",
                    help="M <= 8: register-staged kernels (ameva_mmvq*), the one that stages the weight rows in shared "
                         "memory (ameva_mmvs_*), or the library's own choice")
    ap.add_argument("--fused-quantize", action="store_true",
                    help="M == 1, small projections: quantize inside the GEMV launch (ameva_mmv*_fq)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    name = args.workload
    if args.impl == "reference":
        reference_arm(args, name)
        return

    t, M, N, K, std, desc = WORKLOADS[name]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    import torch
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    pkg = importlib.import_module("ameva-compute_b200")
    rt, qmm, shard = pkg.runtime, pkg.qmm, pkg.shard
    ctx = rt.init()
    ext_stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", local_rank))

    unit = "TFLOP/s" if M > GEMV_MAX_M else "GB/s"
    blocks, scale, x = make_inputs(t, M, N, K, std)
    parts = shard.partition_rows(N, world)
    row0, rows = parts[rank]
    pad = shard.padded_rows(N, world)
    per_row = blocks.reshape(N, -1).shape[1]
    my_blocks = blocks.reshape(N, per_row)[row0:row0 + rows]

    # rotating pool of weight copies larger than L2, so that no step finds its weights cached
    shard_bytes = weight_bytes(t, max(rows, 1), K)
    pool_n = max(2, min(64, -(-2 * L2_BYTES // max(shard_bytes, 1)) + 1))
    weights = [qmm.QuantWeight.from_ggml(ctx, t, my_blocks, rows, K, scale) for _ in range(pool_n)]
    mms = [qmm.MulMat(ctx, w, M, streamed={"auto": None, "register": False, "streamed": True}[args.gemv],
                      fused_quantize=args.fused_quantize) for w in weights]
    x_dev = ctx.buffer(data=x)

    # Output exchange of the sharded run. "peer": every rank owns a full [M][N] output; the mul_mat's epilogue stores
    # its rows into every rank's output over NVLink and a flag barrier closes the step (all inside this library's
    # kernels). "allgather": [M][rows] shards + NCCL all-gather + permute, for the kernels without the fused epilogue.
    tc_path = M > GEMV_MAX_M and mms[0].tc_ok
    exchange = "none"
    if world > 1:
        exchange = "peer" if (t != I2_S and (tc_path or (M <= GEMV_MAX_M and K % 256 == 0))) else "allgather"
    ex = None
    if exchange == "peer":
        ex = qmm.PeerExchange(ctx, rank, world, M * N * 4)
        handles = [None] * world
        dist.all_gather_object(handles, ex.handles())
        ex.connect(handles)
        out_buf, out_off, out_stride, out_cols = ex.out, row0 * 4, N, N
    else:
        out_buf, out_off, out_stride, out_cols = ctx.buffer(M * pad * 4), 0, pad, pad
    gathered_t = out_full_t = out_local_t = None
    if exchange == "allgather":
        out_local_t = torch.empty((M, pad), dtype=torch.float32, device="cuda")
        out_buf.destroy()
        out_buf = ctx.import_buffer(out_local_t.data_ptr(), out_local_t.numel() * 4)
        gathered_t = torch.empty((world, M, pad), dtype=torch.float32, device="cuda")
        out_full_t = torch.empty((M, N), dtype=torch.float32, device="cuda")

    launches_per_step = [0]
    batch_keep = []

    probe_sink = ctx.buffer(64)

    def record_steps(batch, n, first, quantize=True):
        if quantize == "read-probe":   # a plain read of each step's weight region instead of the step
            for i in range(n):
                batch.dispatch(ctx.kernel("ameva_read_probe"), [weights[(first + i) % pool_n].buf, probe_sink], [0, 0],
                               (1, 1, 1))
            return
        for i in range(n):
            mm = mms[(first + i) % pool_n]
            before = batch.stats().dispatches if i == 0 else None
            mm.record(batch, x_dev, out_buf, M, dst_offset=out_off, dst_stride=out_stride, quantize=quantize,
                      peers=ex.peers if ex else None)
            if ex:
                ex.record_barrier(batch)
            if i == 0 and quantize:
                launches_per_step[0] = batch.stats().dispatches - before

    # The steps are replayed from instantiated batches (CUDA graphs of pool_n consecutive steps, one per weight copy;
    # with peers each step ends in the flag barrier kernel, which counts its own epochs), so that a step of a few
    # microseconds is not bounded by one host launch per kernel; the timed region is bracketed by CUDA events on the
    # runtime's stream.
    use_replay = exchange != "allgather" and not args.no_replay
    replay_cache = {}

    def replay_batch(quantize):
        if quantize not in replay_cache:
            rb = ctx.batch(max(64, pool_n * 70), 0)
            record_steps(rb, pool_n, 0, quantize)
            rb.instantiate()
            replay_cache[quantize] = rb
        return replay_cache[quantize]

    def gpu_steps(n, first, flags=0, quantize=True):
        """n steps on the device; returns (gpu seconds by CUDA events on the runtime's stream, last batch)."""
        if use_replay and not flags:
            full, rem = divmod(n, pool_n)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            rb = replay_batch(quantize) if full else None
            tail = None
            if rem:
                tail = ctx.batch(max(64, rem * 70), 0)
                record_steps(tail, rem, 0, quantize)
            evs = []
            with torch.cuda.stream(ext_stream):
                start.record()
                for _ in range(full):
                    evs.append(rb.replay())
                if tail:
                    evs.append(tail.submit())
                end.record()
            for ev in evs:
                ev.wait(600_000_000_000)
                ev.destroy()
            end.synchronize()
            return start.elapsed_time(end) / 1e3, tail
        if exchange != "allgather":
            per_batch = n if flags else max(1, min(n, 60000 // 70))   # a batch holds at most 65536 dispatches
            gpu_s, done, batch = 0.0, 0, None
            pending = []
            while done < n:   # every batch is recorded and submitted before the first wait: the GPU never idles
                cnt = min(per_batch, n - done)
                batch = ctx.batch(max(64, cnt * 70), flags)
                record_steps(batch, cnt, first + done, quantize)
                pending.append((batch, batch.submit()))
                done += cnt
            for bt, ev in pending:
                ev.wait(600_000_000_000)
                gpu_s += ev.timing()[1] / 1e9
                ev.destroy()
                if bt is not batch:
                    bt.destroy()
            return gpu_s, batch
        # all-gather exchange: compute on the runtime's stream, then the NCCL all-gather and the permute, in stream order
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ext_stream):
            start.record()
            for i in range(n):
                batch = ctx.batch(128, 0)
                record_steps(batch, 1, first + i)
                batch.flush()
                dist.all_gather_into_tensor(gathered_t.view(world * M, pad), out_local_t)
                shard.assemble(gathered_t, parts, M, N, out_full_t)
                batch_keep.append(batch)
            end.record()
            end.synchronize()
        for b_ in batch_keep:
            b_.destroy()
        batch_keep.clear()
        return start.elapsed_time(end) / 1e3, None

    def barrier():
        if dist is not None:
            dist.barrier()
        ctx.synchronize()
        torch.cuda.synchronize()

    # warm-up
    _, b = gpu_steps(args.warmup, 0)
    if b:
        b.destroy()
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    t_wall0 = time.perf_counter()
    gpu_s, b = gpu_steps(args.steps, args.warmup)
    barrier()
    wall_s = time.perf_counter() - t_wall0
    if b:
        b.destroy()
    if dist is not None:
        tt = torch.tensor([gpu_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        gpu_s = float(tt.item())

    # average launch duration of the dominant kernel, live: the mul_mat kernel(s) alone (activations already quantized
    # by the steps above), the same rotation of weight copies, back to back on the launching stream between two CUDA
    # events; the quantize kernel's share is the rest of a step
    roof = None
    if world == 1:
        nprof = args.steps
        # (a step of the fused quantize+GEMV launch is that one kernel: it is timed as it is)
        main_s, pb = gpu_steps(nprof, args.warmup + args.steps, 0, quantize=mms[0].path == "mmvq-fq")
        if pb:
            pb.destroy()
        main_ns = main_s / nprof * 1e9
        quant_ns = max(0.0, gpu_s / args.steps * 1e9 - main_ns)
        pk = peaks()
        if unit == "TFLOP/s":
            ach = 2.0 * M * N * K / (main_ns * 1e-9) / 1e12
            roof = {"bound": "tensor", "achieved": ach, "peak": pk["tflops"], "unit": "TFLOP/s",
                    "frac": ach / pk["tflops"], "traffic": TRAFFIC.get((name, mms[0].path)),
                    "peak_source": pk["source"] + " bf16 burst", "kernel_us": main_ns / 1e3, "quant_us": quant_ns / 1e3}
        else:
            ach = algorithmic_bytes(t, M, N, K) / (main_ns * 1e-9) / 1e9
            roof = {"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
                    "traffic": TRAFFIC.get((name, mms[0].path)), "peak_source": pk["source"] + " copy", "kernel_us": main_ns / 1e3,
                    "quant_us": quant_ns / 1e3}
            # what a kernel that only reads the same weight regions (ameva_read_probe, same rotation, same timing)
            # takes: the ramp and the tail of a launch this short keep a pure read well under the copy peak
            probe_s, pb = gpu_steps(nprof, args.warmup + args.steps, 0, quantize="read-probe")
            if pb:
                pb.destroy()
            roof["read_only_us"] = probe_s / nprof * 1e6
            roof["read_only_gbs"] = weights[0].buf.size_bytes / (probe_s / nprof) / 1e9
            roof["frac_of_read_only"] = roof["read_only_us"] / roof["kernel_us"]

    # end to end through the public API with host buffers: H2D of the activations, compute, D2H of the result, per step
    x_pin = torch.from_numpy(x).pin_memory()
    d2h_bytes = M * out_cols * 4
    y_pin = torch.empty((M, out_cols), dtype=torch.float32).pin_memory()
    e2e_steps = args.steps

    def e2e_run(n, first):
        with torch.cuda.stream(ext_stream):
            for i in range(n):
                x_dev.write_async(x_pin.data_ptr(), x.nbytes)
                batch = ctx.batch(128, 0)
                record_steps(batch, 1, first + i)
                batch.flush()
                batch_keep.append(batch)
                if exchange == "allgather":
                    dist.all_gather_into_tensor(gathered_t.view(world * M, pad), out_local_t)
                    shard.assemble(gathered_t, parts, M, N, out_full_t)
                out_buf.read_async(y_pin.data_ptr(), d2h_bytes)
        ctx.synchronize()
        for bb in batch_keep:
            bb.destroy()
        batch_keep.clear()

    # One GPU: the same per-step work, software-pipelined. The activations of step i+1 travel host->device and the result
    # of step i-1 device->host on two copy streams while step i computes (double-buffered device input and output,
    # imported into the runtime with ac_b200_buffer_import; events order the three streams).
    e2e_mode = "sequential on the runtime's stream"
    overlap = exchange == "none" and not args.no_overlap and x.nbytes + d2h_bytes >= (1 << 20)   # else host-bound
    if overlap:
        e2e_mode = "pipelined: H2D, compute and D2H of neighbouring steps overlap on three streams"
        NBUF = 2
        x_t = [torch.empty((M, K), dtype=torch.float32, device="cuda") for _ in range(NBUF)]
        o_t = [torch.empty((M, out_cols), dtype=torch.float32, device="cuda") for _ in range(NBUF)]
        x_b = [ctx.import_buffer(tt_.data_ptr(), tt_.numel() * 4) for tt_ in x_t]
        o_b = [ctx.import_buffer(tt_.data_ptr(), tt_.numel() * 4) for tt_ in o_t]
        y_pins = [y_pin] + [torch.empty((M, out_cols), dtype=torch.float32).pin_memory() for _ in range(NBUF - 1)]
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

        def e2e_run(n, first):   # noqa: F811
            ev_cmp, ev_out = [None] * NBUF, [None] * NBUF
            for i in range(n):
                b_ = i % NBUF
                with torch.cuda.stream(s_in):
                    if ev_cmp[b_] is not None:
                        s_in.wait_event(ev_cmp[b_])          # the step that last read this input buffer has finished
                    x_t[b_].copy_(x_pin, non_blocking=True)
                    ev_in = torch.cuda.Event()
                    ev_in.record(s_in)
                with torch.cuda.stream(ext_stream):
                    ext_stream.wait_event(ev_in)
                    if ev_out[b_] is not None:
                        ext_stream.wait_event(ev_out[b_])    # the result that last used this output buffer is on the host
                    batch = ctx.batch(128, 0)
                    mms[(first + i) % pool_n].record(batch, x_b[b_], o_b[b_], M, dst_stride=out_stride)
                    batch.flush()
                    batch_keep.append(batch)
                    ev_cmp[b_] = torch.cuda.Event()
                    ev_cmp[b_].record(ext_stream)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[b_])
                    y_pins[b_].copy_(o_t[b_], non_blocking=True)
                    ev_out[b_] = torch.cuda.Event()
                    ev_out[b_].record(s_out)
            torch.cuda.synchronize()
            ctx.synchronize()
            for bb in batch_keep:
                bb.destroy()
            batch_keep.clear()

    e2e_run(3, 0)
    barrier()
    t0 = time.perf_counter()
    e2e_run(e2e_steps, 3)
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    if dist is not None:
        tt = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt.item())

    # parity spot check of what was timed (rank 0): first token rows x a sample of weight rows of the first and, when
    # sharded with the peer exchange, also of the last rank's shard, so a wrong kernel or exchange cannot post a number
    check = None
    if rank == 0 and rows:
        from helpers import max_normalised_error, oracle_mul_mat
        ms, ns = min(M, 4), min(rows, 512)
        got_all = y_pin.numpy()
        spans = [(row0, ns, 0 if exchange != "peer" else row0)]
        if exchange == "peer":
            lr0, lrows = parts[-1]
            spans.append((lr0, min(lrows, 256), lr0))
        check = 0.0
        allb = blocks.reshape(N, per_row)
        for g_row0, g_n, col0 in spans:
            want, _, _ = oracle_mul_mat(t, np.ascontiguousarray(allb[g_row0:g_row0 + g_n]), scale, x[:ms], g_n, K,
                                        want_sums=False)
            check = max(check, max_normalised_error(got_all[:ms, col0:col0 + g_n], want))

    if rank == 0:
        par = {"none": "single GPU",
               "peer": f"weight rows sharded over {world} ranks; the GEMM/GEMV epilogue stores each rank's rows into every "
                       "rank's [M][N] output over NVLink (peer memory) and a flag barrier kernel closes every step; no "
                       "collective library in the data path",
               "allgather": f"weight rows sharded over {world} ranks, NCCL all-gather of the fp32 output + permute inside "
                            "the timed region"}[exchange]
        line = {
            "metric": metric_name(name), "value": unit_value(unit, t, M, N, K, gpu_s / args.steps), "unit": unit,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": gpu_s / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"mmtc": "int8 (tcgen05 kind::i8, int32 accumulate)" if t == I2_S else
                      "f16 (tcgen05 kind::f16 on dequantized fp16 operands, fp32 accumulate in TMEM)"}.get(
                          mms[0].path.split("+")[0], "int8 (dp4a, int32 per block, fp32 scale-accumulate)"),
            "data": "synthetic",
            "config": {"workload": f"{name}: {desc}", "M": M, "N": N, "K": K,
                       "l2": f"rotating pool of {pool_n} weight copies ({pool_n * shard_bytes / 1e6:.0f} MB > L2) per rank",
                       "parallelism": par, "path": mms[0].path,
                       "launch": f"replayed batches (CUDA graphs of {pool_n} steps)" if use_replay else
                                 "one host launch per kernel"},
            "wall_ms_per_step": wall_s / args.steps * 1e3,
            "gpu_launches": launches_per_step[0] * args.steps,
            "e2e": {"value": unit_value(unit, t, M, N, K, e2e_s / e2e_steps), "unit": unit,
                    "h2d_bytes_per_step": int(x.nbytes), "d2h_bytes_per_step": int(d2h_bytes),
                    "ms_per_step": e2e_s / e2e_steps * 1e3, "mode": e2e_mode},
            "clocks": clocks,
            "parity_max_normalised_error": check,
        }
        if roof:
            line["roofline"] = roof
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = run_cpu_baseline(t, M, N, K, blocks, scale, x, unit)
        print(json.dumps(line), flush=True)

    if dist is not None:   # nobody unmaps a buffer a peer may still be writing; and never hang after the line is out
        threading.Timer(60.0, lambda: os._exit(0)).start()
        barrier()
    for rb in replay_cache.values():
        rb.destroy()
    if overlap:
        for ib in x_b + o_b:
            ib.destroy()
    for mm in mms:
        mm.destroy()
    for w in weights:
        w.destroy()
    x_dev.destroy()
    probe_sink.destroy()
    if ex:
        ex.destroy()
    else:
        out_buf.destroy()
    ctx.destroy()
    if dist is not None:
        dist.destroy_process_group()
        os._exit(0)


if __name__ == "__main__":
    main()
