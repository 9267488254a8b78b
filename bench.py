"""Benchmark of the quantized decode matmul path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

A "step" is one pass over every weight matmul of a Llama-8B-shaped decoder (32 layers
x {q,k,v,o,gate,up,down} + LM head, int4 / group 32, binary16 scales) with the norms, the
SiLU gate and the residual adds between them, for a batch of B token rows (bench_workload.py):
4.22 GB of packed weights stream from HBM once per step, which makes the inputs larger than L2
by construction (no flush needed).  With N > 1 (launched by torch.distributed.run, one rank per
GPU) the matmuls are tensor-parallel, column- then row-sharded with a sum over the ranks after
each row-parallel matmul; the total work is fixed, so scaling is "strong".

Prints ONE JSON line.  `value` is tok/s with inputs resident in HBM (device-timed);
`e2e` is the same metric through host buffers with a fence after every step (x copied in,
logits copied out, the host waits, as a decode loop must before it can pick the next token);
`roofline` relates the kernel's algorithmic bytes to its measured time; `parity` is a check of
this very run's outputs against the CPU oracle; `cpu_baseline` is the CPU oracle (the
reference's shader arithmetic restated in C) timed on this machine's host cores.

`--impl reference` times that CPU restatement alone.  The reference's own WGSL path
needs Deno + a WebGPU adapter, neither of which exists on these machines.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from bench_workload import DecodeConfig, reference_step, synth_norm, synth_weight  # noqa: E402


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return json.load(open(path)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def host_threads() -> int:
    """Cores this process may use.  torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm
    passes this count to the oracle explicitly so that it always uses the whole machine."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def workload_config(cfg: DecodeConfig, batch: int, world: int, **extra):
    """The `config` object: the same keys in the CUDA arm and in the CPU arm."""
    out = {
        "workload": f"{cfg.name}: {cfg.layers} layers x (rms_norm, q|k|v, o + residual, rms_norm, silu(gate)*up, "
                    f"down + residual) + rms_norm + lm_head, int4 g32, fp16 scales, batch {batch}"
                    + ("" if cfg.layers == 32 else " (REDUCED layer count: a profiling case, not the benchmark)"),
        "batch": batch, "activations": "f32", "parallelism": f"tp{world}",
        "weight_bytes": cfg.weight_bytes(),
        "l2": f"inputs larger than L2 ({cfg.weight_bytes() / 1e9:.1f} GB of weights per step)",
        "exchange": None, "replay": None,
    }
    out.update(extra)
    return out


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.lines = []
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [l.split(", ") for t, l in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l.split(", ") for _, l in self.lines]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_sample(cfg: DecodeConfig, batch: int, threads: int, steps: int):
    """Times the CPU restatement of the shader arithmetic (f32, sequential K, one f32 multiply
    per weight for the dequant) on full decode steps: one layer's seven matmuls and its norms,
    gate and adds run `layers` times (the same host weights stand in for every layer) plus the
    final norm and the LM head.  Returns (tok/s, seconds per step, sample description)."""
    import oracle
    mats = {}
    for name, k, n, _ in cfg.layer_matmuls() + [("lm_head", cfg.hidden, cfg.vocab, "col")]:
        payload, scale = synth_weight(0, "l0." + name if name != "lm_head" else name, n, k, cfg.group_size)
        mats[name] = (payload, scale.astype(np.float32), np.zeros(n, np.float32), n, k)
    gamma = synth_norm(0, "l0.norm1", cfg.hidden)
    x = np.random.default_rng(1).standard_normal((batch, cfg.hidden)).astype(np.float32)

    def lin(name, inp):
        payload, scale, bias, n, k = mats[name]
        return oracle.linear_i4(inp, payload, scale, bias, n, k, cfg.group_size, threads, f64=False)

    lin("k", x)  # warm the thread pool
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        h = x
        for _layer in range(cfg.layers):
            xn = oracle.rms_norm(h, gamma, cfg.eps)
            q = lin("q", xn)
            lin("k", xn)
            lin("v", xn)
            h = oracle.add(lin("o", q), h)
            xn = oracle.rms_norm(h, gamma, cfg.eps)
            act = oracle.silu_mul(lin("gate", xn), lin("up", xn))
            h = oracle.add(lin("down", act), h)
        lin("lm_head", oracle.rms_norm(h, gamma, cfg.eps))
        times.append(time.perf_counter() - t0)
    step_s = float(np.median(times))
    desc = (f"{steps} full decode steps ({cfg.layers} x 7 layer matmuls with norms, gate and adds + lm_head, "
            f"{cfg.weight_bytes() / 0.5625 / 1e6:.0f}M weights each; one layer's host weights reused for every layer) "
            f"on {threads} threads, f32 sequential-K shader arithmetic")
    return batch / step_s, step_s, desc


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = DecodeConfig(layers=args.layers)
    steps, warm = max(1, args.steps), max(0, args.warmup)
    import oracle
    oracle.build()
    threads = host_threads()
    if warm:
        cpu_sample(cfg, args.batch, threads, 1)
    timed_steps = min(steps, 10)  # each step is seconds of CPU work
    tok_s, step_s, desc = cpu_sample(cfg, args.batch, threads, timed_steps)
    line = {
        "impl": "reference", "metric": "decode_matmul_tok_per_s", "value": tok_s, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(cfg, args.batch, args.gpus,
                                  note="CPU restatement of the reference's WGSL arithmetic (Deno/WebGPU unavailable on this box)"),
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "timed_steps": timed_steps,  # at most 10 (each is seconds of CPU work); ms_per_step is their mean
    }
    print(json.dumps(line))


def synth_i8(n, k, seed):
    rng = np.random.default_rng(seed)
    q = rng.integers(-127, 128, size=(n, k), dtype=np.int16).astype(np.int8)
    s = (np.abs(rng.standard_normal(n).astype(np.float32)) * np.float32(0.02 / 127)).astype(np.float16)
    s[s == 0] = np.float16(6e-8)
    return q, s


def kernel_sweep(gpu, peak_gbs, peak_tf):
    """Kernel-only numbers for the other halves of the metric, measured after the timed region
    (N = 1 only): the int4 / int8 GEMV on single matrices (graph replay over distinct weight
    copies totalling more than L2, so every launch streams from HBM) and the prefill GEMM."""
    import torch
    out = {}

    def gemv(storage, k, n, m, dtype, a8=False, tc=False):
        if storage == "i4":
            data, scale = synth_weight(1, f"sweep.{n}x{k}", n, k)
        else:
            data, scale = synth_i8(n, k, 1)
        wbytes = data.nbytes + scale.nbytes
        copies = max(2, min(128, int(400e6 // wbytes) + 1))
        ws = [gpu.upload_weight(storage, data, scale, (n, k), 32 if storage == "i4" else 0) for _ in range(copies)]
        x = torch.randn(m, k, device="cuda").to(dtype)
        bias = torch.zeros(n, device="cuda")
        y = torch.empty(m, n, device="cuda")
        if a8:  # integer-dot form: int8 activations (quantised once, outside the timed launches)
            xq, xs = gpu.quantize_rows(x.float().contiguous())
            gpu.linear_a8(xq, xs, ws[0], bias, out=y)  # grows the context's scratch before the recording
        gpu.graph_begin()
        for w in ws:
            if a8:
                gpu.linear_a8(xq, xs, w, bias, out=y)
            elif tc:  # the same linear through the tcgen05 entry point (kq_linear_tc)
                gpu.linear_tc(x, [w], [bias], [y])
            else:
                gpu.linear(x, w, bias, out=y)
        g = gpu.graph_end()
        for _ in range(3):
            gpu.graph_launch(g)
        gpu.sync()
        times = []
        for _ in range(10):  # 10 replays x `copies` launches each: >= 50 timed launches per entry
            gpu.timer_start()
            gpu.graph_launch(g)
            times.append(gpu.timer_stop())
        best, median = min(times), sorted(times)[len(times) // 2]
        gpu.graph_free(g)
        for w in ws:
            w.free()
        alg = wbytes + m * k * (1 if a8 else x.element_size()) + m * n * 4
        us = best * 1e3 / copies
        return {"us": round(us, 3), "us_median": round(median * 1e3 / copies, 3), "GB/s": round(alg / us / 1e3, 1),
                "frac_of_8TB/s": round(alg / us / 1e3 / 8000, 3), "frac_of_measured_copy_peak": round(alg / us / 1e3 / peak_gbs, 3),
                "weights": "stream from HBM" if copies * wbytes > 200e6 else "L2-resident (the copies total less than L2)"}

    out["gemv_i4_m1_4096x4096_f32 (config 0)"] = gemv("i4", 4096, 4096, 1, torch.float32)
    out["gemv_i4_m1_1536x151936_f32 (config 1 lm head)"] = gemv("i4", 1536, 151936, 1, torch.float32)
    out["gemv_i8_m1_1536x151936_f32 (config 1 lm head)"] = gemv("i8", 1536, 151936, 1, torch.float32)
    for k, n in ((1536, 1536), (1536, 256), (1536, 8960), (8960, 1536)):  # config 1's projection shapes
        out[f"gemv_i4_m1_{k}x{n}_f32 (config 1)"] = gemv("i4", k, n, 1, torch.float32)
        out[f"gemv_i8_m1_{k}x{n}_f32 (config 1)"] = gemv("i8", k, n, 1, torch.float32)
    for n in (4096, 11008):  # config 2: the small-batch / verify shapes, binary16 activations
        for m in (1, 2, 4, 8, 16):
            out[f"gemv_i4_m{m}_4096x{n}_f16 (config 2)"] = gemv("i4", 4096, n, m, torch.float16)
    out["gemv_i4_m16_4096x11008_f32 (config 2 shape, f32 rows)"] = gemv("i4", 4096, 11008, 16, torch.float32)
    out["gemv_i4_m8_4096x11008_f16 through kq_linear_tc (tcgen05)"] = gemv("i4", 4096, 11008, 8, torch.float16, tc=True)
    out["gemv_i4_m16_4096x11008_f16 through kq_linear_tc (tcgen05)"] = gemv("i4", 4096, 11008, 16, torch.float16, tc=True)
    out["gemv_i4_m1_4096x128256_f32 (config 4 lm head)"] = gemv("i4", 4096, 128256, 1, torch.float32)
    out["w8a8_m1_1536x151936 (integer dot, config 1 lm head)"] = gemv("i8", 1536, 151936, 1, torch.float32, a8=True)
    out["w4a8_m1_4096x128256 (integer dot, config 4 lm head)"] = gemv("i4", 4096, 128256, 1, torch.float32, a8=True)
    out["w4a8_m8_4096x11008 (integer dot, config 2 shape)"] = gemv("i4", 4096, 11008, 8, torch.float32, a8=True)

    def gemm(m, k, n, dtype=torch.bfloat16, storage="i4"):
        if storage == "i4":
            data, scale = synth_weight(1, f"sweep.{n}x{k}", n, k)
        else:
            data, scale = synth_i8(n, k, 1)
        w = gpu.upload_weight(storage, data, scale, (n, k), 32 if storage == "i4" else 0)
        x = torch.randn(m, k, device="cuda").to(dtype)
        bias = torch.zeros(n, device="cuda")
        y = torch.empty(m, n, device="cuda")
        for _ in range(3):
            gpu.linear(x, w, bias, out=y)
        gpu.sync()
        best = 1e9
        for _ in range(8):
            gpu.timer_start()
            gpu.linear(x, w, bias, out=y)
            best = min(best, gpu.timer_stop())
        w.free()
        tf = 2.0 * m * n * k / best / 1e9
        return {"ms": round(best, 4), "TFLOP/s": round(tf, 1), "frac_of_measured_bf16_peak": round(tf / peak_tf, 3)}

    out["gemm_i4_bf16_m2048_4096x14336 (config 3)"] = gemm(2048, 4096, 14336)
    out["gemm_i4_bf16_m2048_14336x4096 (config 3)"] = gemm(2048, 14336, 4096)
    out["gemm_i4_bf16_m512_4096x14336 (config 3)"] = gemm(512, 4096, 14336)
    out["gemm_i4_bf16_m512_14336x4096 (config 3)"] = gemm(512, 14336, 4096)
    # the same shapes with f32 activations: operands carried as two bf16 numbers each (three MMAs per product)
    out["gemm_i4_f32_m2048_4096x14336 (config 3 shape, f32 rows)"] = gemm(2048, 4096, 14336, torch.float32)
    out["gemm_i4_f32_m2048_14336x4096 (config 3 shape, f32 rows)"] = gemm(2048, 14336, 4096, torch.float32)
    # int8 weights through the same tcgen05 kernel (bf16 rows)
    out["gemm_i8_bf16_m2048_4096x14336 (config 3 shape, int8 weights)"] = gemm(2048, 4096, 14336, storage="i8")
    out["gemm_i8_bf16_m2048_14336x4096 (config 3 shape, int8 weights)"] = gemm(2048, 14336, 4096, storage="i8")
    return out


def parity_gate(step, cfg, rank, world, dist, rows_per_rank=48):
    """This run's outputs against the CPU oracle: the hidden state after the last layer (the same
    on every rank) and a sample of each rank's logit columns.  Rank 0 runs the oracle chain
    (f64 accumulation, every weight re-made from its seed) and shares the expected values.
    Tolerance: |got - ref| <= 1e-5 * max(1, rms(ref)) + 1e-3 * |ref|."""
    import torch
    import oracle
    x = np.random.default_rng(7).standard_normal(step.host_x.shape).astype(np.float32)
    step.host_x[...] = x
    step.host_logits[...] = 0
    if world > 1:
        dist.barrier()
    step.run_host()
    step.sync()
    shard = cfg.vocab // world
    rows = np.concatenate([r * shard + np.sort(np.random.default_rng(11 + r).choice(shard, min(rows_per_rank, shard), replace=False))
                           for r in range(world)])
    t0 = time.time()
    if rank == 0:
        h_ref, logit_ref = reference_step(cfg, step.seed, x, rows, threads=host_threads())
        packed = np.concatenate([h_ref.reshape(-1), logit_ref.reshape(-1)]).astype(np.float32)
    else:
        packed = np.zeros(x.shape[0] * (cfg.hidden + len(rows)), np.float32)
    if world > 1:
        t = torch.from_numpy(packed).cuda()
        dist.broadcast(t, 0)
        packed = t.cpu().numpy()
    h_ref = packed[:x.shape[0] * cfg.hidden].reshape(x.shape[0], cfg.hidden)
    logit_ref = packed[x.shape[0] * cfg.hidden:].reshape(x.shape[0], len(rows))
    per = len(rows) // world
    mine = rows[rank * per:(rank + 1) * per] - rank * shard
    got_l = step.host_logits[:, mine]
    want_l = logit_ref[:, rank * per:(rank + 1) * per]
    got_h = step.h.cpu().numpy()

    def cmp(got, want):
        mag = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        rep = oracle.allclose(got, want, atol=1e-5 * max(1.0, mag), rtol=1e-3)
        return rep["pass"], rep["max_abs"], rep["max_rel"], mag

    ok_h, abs_h, rel_h, mag_h = cmp(got_h, h_ref)
    ok_l, abs_l, rel_l, mag_l = cmp(got_l, want_l)
    stats = np.array([float(ok_h and ok_l), -abs_h / max(mag_h, 1e-30), -abs_l / max(mag_l, 1e-30)], np.float64)
    if world > 1:
        t = torch.from_numpy(stats).cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        stats = t.cpu().numpy()
    return {"checked": int(got_h.size + got_l.size * world), "hidden_max_abs_over_rms": float(-stats[1]),
            "logits_max_abs_over_rms": float(-stats[2]), "logit_columns_per_rank": int(per),
            "max_abs": float(max(abs_h, abs_l)), "max_rel": float(max(rel_h, rel_l)),
            "tolerance": "1e-5 * max(1, rms(ref)) + 1e-3 * |ref| against the f64-accumulate CPU oracle, all ranks",
            "oracle_seconds": round(time.time() - t0, 1), "pass": bool(stats[0] > 0.5)}


def phase_table(gpu, step, cfg):
    """One profiled launch of the fused plan (kq_plan_profile): per kind of op, the median over
    CTAs and layers of the time spent in each phase, in microseconds."""
    stamps = gpu.plan_profile(step.plan).astype(np.float64)  # [cta, op, slot] ns
    names = ["q|k|v", "o", "gate*up", "down"]
    kinds = [names[i % 4] for i in range(4 * cfg.layers)] + ["lm_head"]
    begin, barrier, staged, first, consumed, end = (stamps[:, :, i] for i in range(6))
    last_arrival = begin.max(axis=0, keepdims=True)
    phases = {
        "wait_for_last_cta": np.maximum(last_arrival - begin, 0.0),
        "barrier_after_last_arrival": np.maximum(barrier - np.maximum(last_arrival, begin), 0.0),
        "stage_x": staged - barrier,
        "first_piece_wait": np.maximum(first - staged, 0.0),
        "weights": consumed - np.maximum(first, staged),
        "outputs": end - consumed,
        "op_total": end - begin,
    }
    table = {}
    for kind in names + ["lm_head"]:
        cols = [i for i, k in enumerate(kinds) if k == kind and i > 0]
        table[kind] = {name: round(float(np.median(val[:, cols])) / 1e3, 2) for name, val in phases.items()}
        table[kind]["ops"] = len(cols)
    span = float(end.max() - begin.min()) / 1e6
    return {"unit": "us (median over CTAs and ops of a kind; warp 0 of every CTA)", "kernel_ms": round(span, 4), "phases": table}


def run_cuda(args):
    # Libraries write banners to the process's stdout (NCCL's version line comes from native code);
    # rank 0's stdout must carry the one JSON line only, so everything else goes to stderr and the
    # line is written to the original descriptor at the end.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist

    import karume_b200 as kb
    from bench_workload import DecodeStep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = DecodeConfig(layers=args.layers)
    gpu = kb.acquire_gpu(local)
    fused = args.replay == "fused" and args.batch <= 2
    step = DecodeStep(gpu, cfg, args.batch, rank=rank, world=world, seed=0, fused=fused, exchange=args.exchange)
    step.record()
    rng = np.random.default_rng(1)
    step.host_x[...] = rng.standard_normal(step.host_x.shape).astype(np.float32)
    step.x.copy_(torch.from_numpy(step.host_x.copy()))
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(run, steps, fence_each=False):
        ev0 = torch.cuda.Event(enable_timing=True)
        ev1 = torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(step._stream):
            ev0.record()
        for _ in range(steps):
            run()
            if fence_each:
                step.sync()
        with torch.cuda.stream(step._stream):
            ev1.record()
        step.sync()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    warm = max(3, args.warmup)
    for _ in range(warm):
        step.run_device()
        step.run_host()
    step.sync()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    t0 = time.time()
    launches_before = gpu.launch_count
    ms_dev = timed(step.run_device, args.steps)
    launches = gpu.launch_count - launches_before
    if world > 1 and args.exchange == "nccl":  # a torch CUDA graph replays the launches; the library does not see them
        launches = step.kernels_per_step * args.steps
    ms_e2e = timed(step.run_host, args.steps, fence_each=True)
    ms_e2e_pipelined = timed(step.run_host, args.steps)
    # spread: repeat the K-step region until half a second has been timed
    rounds, spent = [], 0.0
    while spent < 500.0 and len(rounds) < 40:
        ms = timed(step.run_device, args.steps)
        rounds.append(ms / args.steps)
        spent += ms
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if rank == 0 else None

    parity = None if args.no_parity else parity_gate(step, cfg, rank, world, dist)
    logits_ok = bool(np.all(np.isfinite(step.host_logits)))
    per_step_ms = ms_dev / args.steps
    per_step_e2e = ms_e2e / args.steps
    tok_s = args.batch / (per_step_ms * 1e-3)
    tok_s_e2e = args.batch / (per_step_e2e * 1e-3)

    phases = None
    if args.phases and step.fused:
        # every rank runs the profiled launch (the fused kernel exchanges partial sums with its
        # peers); rank 0 reports its own CTAs
        barrier()
        phases = phase_table(gpu, step, cfg)
        barrier()

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        bytes_rank = cfg.algorithmic_bytes(args.batch, world)
        launches_per_step = step.kernels_per_step
        achieved = bytes_rank / (per_step_ms * 1e-3) / 1e9
        other_batch = None
        if world == 1 and not args.no_sweep and args.batch != 16:
            # the same resident weights at the other end of the batch range (device-timed, 5 steps)
            step16 = DecodeStep(gpu, cfg, 16, seed=0, fused=False, share_weights_with=step)
            step16.record()
            step16.x.normal_()
            for _ in range(3):
                step16.run_device()
            step16.sync()
            gpu.timer_start()
            for _ in range(5):
                step16.run_device()
            ms16 = gpu.timer_stop() / 5
            other_batch = {"batch": 16, "replay": "cuda graph of separate launches", "ms_per_step": ms16,
                           "tok_per_s": 16 / (ms16 * 1e-3), "GB/s": cfg.algorithmic_bytes(16, 1) / (ms16 * 1e-3) / 1e9}
            step16.close()
        sweep = None
        if world == 1 and not args.no_sweep:
            gpu.use_stream(torch.cuda.current_stream())
            sweep = kernel_sweep(gpu, float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"]))
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            import oracle
            oracle.build()
            threads = host_threads()
            tok_cpu, _, desc = cpu_sample(cfg, args.batch, threads, 3)
            cpu = {"value": tok_cpu, "unit": "tok/s", "cores": threads, "kind": "port", "sample": desc}
        line = {
            "metric": "decode_matmul_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": per_step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(cfg, args.batch, world, exchange=(args.exchange if world > 1 else None),
                                      replay="fused plan kernel" if step.fused else "cuda graph of separate launches"),
            "e2e": {"value": tok_s_e2e, "unit": "tok/s", "ms_per_step": per_step_e2e,
                    "fence": "host waits for the logits after every step",
                    "pipelined_tok_per_s": args.batch / (ms_e2e_pipelined / args.steps * 1e-3),
                    "h2d_bytes_per_step": int(step.x.numel() * 4),
                    "d2h_bytes_per_step": int(step.logits.numel() * 4)},
            "spread": {"rounds": len(rounds), "steps_per_round": args.steps, "ms_per_step_median": float(np.median(rounds)),
                       "ms_per_step_min": float(np.min(rounds)), "ms_per_step_max": float(np.max(rounds))},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "plan_pair_kernel" if step.fused else "qgemv_i4 per-launch kernels",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "frac_of_8tbs": achieved / 8000.0,
                         "launches_per_step": launches_per_step,
                         "algorithmic_bytes_per_launch": bytes_rank / max(1, launches_per_step),
                         # dram read+write of one launch: measured with ncu on a 2-layer, 1-GPU case of the
                         # same kernel (all of it weights, so it scales with the rank's weight bytes)
                         "traffic": (bytes_rank * 1.004) if step.fused else None,
                         "traffic_source": "ncu capture of the 2-layer 1-GPU case of the same kernel, scaled by this rank's weight bytes"
                                           if step.fused else None},
            "parity": parity,
            "plan_phases": phases,
            "cpu_baseline": cpu,
            "kernel_sweep": sweep,
            "other_batch": other_batch,
            "clocks": clocks,
            "finite_outputs": logits_ok,
        }
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        # Tearing down NCCL communicators that a CUDA graph still references can block;
        # everything is measured and printed, so synchronise, flush and leave.
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    step.close()
    gpu.destroy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="kq", choices=["kq", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the single-kernel GEMV / GEMM numbers")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of this run's outputs")
    ap.add_argument("--phases", action="store_true",
                    help="add a per-op phase table from one profiled launch of the fused plan (kq_plan_profile)")
    ap.add_argument("--exchange", default="kq", choices=["kq", "nccl"], help="sum over ranks used when --gpus > 1")
    ap.add_argument("--layers", type=int, default=32,
                    help="decoder layers; anything but 32 is a small case for profiler captures, not the benchmark")
    ap.add_argument("--replay", default="fused", choices=["fused", "graph"],
                    help="replay the step as one persistent plan kernel per rank (default, batch <= 2) or as a CUDA graph "
                         "of separate launches")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
