#!/usr/bin/env python
"""Benchmark of the matmul hot path: training tokens/s of the 33.49M-parameter decoder.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]
    python bench.py --only gemm|timeline|attention|decode|lmhead ...      (single-kernel programs, see --help)

Workload (N=1): one full training step -- forward, backward, gradient-norm clip, Adam -- of the
12-layer d_model-384 decoder at batch 8 x context 1024 with N(0, 0.02) weights and Zipf(1.1) token
ids (seed 1).  With N > 1 every rank runs that same per-GPU batch on its own Zipf stream (weak
scaling); the gradients are combined through the library's data-parallel step (tb_dp_step: NCCL over
NVLink, see include/turkce_b200.h).

One JSON line is printed by rank 0.  `value` is timed with the step's inputs already resident in
HBM; `e2e` is the same step through the public API with host token buffers, the host->device copy
of the ids and the device->host read of the loss inside the timed region.  Beside them, outside both
timed regions, the line carries sub-records for the other benchmark configurations:
  c1  one layer's four linear GEMMs (forward, dX, dW) in the three operand precisions: device time,
      TFLOP/s, error against the CPU oracle, and the reference's own tensor_matmul2d on the host cores
  tf32_step  the headline step with the linear-layer GEMMs in TF32 mode, with its own roofline
  c3  fused causal attention at B=16, H=6, T=1024, hd=64 (forward and backward)
  c4  batched decoding with a KV cache: 64 sequences, 128-token prompts, 128 greedy tokens
  c5  the data-parallel step with a fixed global batch of 128 x 1024 tokens (at every N)
  reference_gpu_trainer  the reference's own GPU trainer (its kernels compiled for sm_100a) on this GPU
  repro (N > 1)  the same two steps run twice from the same state, compared bit for bit

`--impl reference` times the reference's own CPU training step (its unmodified C sources compiled
into oracle/_ref/libref.so; the CPU port oracle/liboracle.so if that library is absent) on the host
cores, on a bounded sample of the same workload.
"""
import argparse
import hashlib
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(V=31769, D=384, H=6, L=12, F=1024)
BATCH, CONTEXT = 8, 1024
LR, BETA1, BETA2, ADAM_EPS, MAX_NORM = 6e-4, 0.9, 0.999, 1e-8, 1.0
METRIC, UNIT = "train tokens/s (33.5M-parameter decoder, batch 8 x context 1024 per GPU)", "tokens/s"
L2_BYTES = 126e6

# DRAM traffic of the GEMM launches of one training step (batch 8 x 1024), from one ncu capture of
# dram__bytes_read.sum + dram__bytes_write.sum over every gemm_bf16_kernel launch of a step.
GEMM_DRAM_TRAFFIC = {
    "bytes_per_step": 4956098816, "launches_per_step": 148,
    "source": "ncu dram__bytes_read.sum + dram__bytes_write.sum over the 148 gemm_bf16_kernel launches of one step "
              "(4.46 GB read + 0.50 GB written): profiles/gemm_bf16_kernel_dram_traffic_train_step.md",
}


def zipf_ids(n, vocab, seed):
    """Zipf(s=1.1) ranks over the vocabulary by inverse CDF on a seeded uniform stream."""
    rng = np.random.default_rng(seed)
    w = 1.0 / np.arange(1, vocab + 1, dtype=np.float64) ** 1.1
    cdf = np.cumsum(w / w.sum())
    return np.minimum(np.searchsorted(cdf, rng.random(n)), vocab - 1).astype(np.uint32)


def init_params(total, layout, seed=0):
    """N(0, 0.02) matrices, zero biases, unit norm weights (the reference's lm_init distribution)."""
    rng = np.random.default_rng(seed)
    p = (rng.standard_normal(total) * 0.02).astype(np.float32)
    off, num = layout
    last = len(off) - 1
    for i, (o, n) in enumerate(zip(off, num)):
        k = (i - 1) % 10 if 0 < i < last else -1
        if i == last or k in (0, 5):
            p[o:o + n] = 1.0
        elif k in (2, 4, 7, 9):
            p[o:o + n] = 0.0
    return p


def peaks():
    """Measured peaks of this pool's B200 (driver-written file), else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"burst": d.get("bf16_tflops", 1645.5), "sustained": d.get("bf16_tflops_sustained", 1364.9),
                "hbm": d.get("hbm_gbs", 6531.6), "src": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm": 6650.0, "src": "fallback"}


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, read through NVML from a thread every few
    milliseconds (nvidia-smi's 50 ms loop gives two samples for a 0.1 s timed region).  Reading only."""

    REASONS = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40, "sw_power_cap": 0x4}

    def __init__(self, gpu_index, period_s=0.004):
        self.samples = []           # (time, sm_mhz, reasons bitmask, watts)
        self.windows = []
        self.max_mhz = None
        self.period = period_s
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            # NVML counts physical GPUs; CUDA_VISIBLE_DEVICES may renumber them
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = gpu_index
            if vis:
                ids = [x.strip() for x in vis.split(",") if x.strip()]
                if gpu_index < len(ids) and ids[gpu_index].isdigit():
                    phys = int(ids[gpu_index])
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None

    def _run(self):
        nv, h = self._nvml, self._h
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                try:
                    why = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    why = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                watts = nv.nvmlDeviceGetPowerUsage(h) / 1e3
                self.samples.append((time.time(), float(mhz), int(why), watts))
            except Exception:
                pass
            time.sleep(self.period)

    def window(self, start, end):
        self.windows.append((start, end))

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0, "how": "NVML, one read per %d ms inside the timed regions" % int(self.period * 1e3)}
        if self._thread is None:
            return out
        self._stop.set()
        self._thread.join(timeout=2)
        sel = [s for s in self.samples if any(a <= s[0] <= b for a, b in self.windows)] if self.windows else self.samples
        if sel:
            mask = 0
            for s in sel:
                mask |= s[2]
            out.update({"sm_mhz": float(np.median([s[1] for s in sel])), "sm_min_mhz": float(min(s[1] for s in sel)),
                        "reasons": sorted(k for k, bit in self.REASONS.items() if mask & bit),
                        "power_w_max": float(max(s[3] for s in sel)), "samples": len(sel)})
        return out


class DevView:
    """Exposes a raw device buffer to torch through __cuda_array_interface__ (no copy)."""

    def __init__(self, ptr, count):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def graph_time_us(run, iters, replays=5):
    """Device time per call with the host out of the picture: `iters` calls captured into one CUDA
    graph on a side stream, the graph replayed and timed with events (mean over the replays)."""
    import torch
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        for i in range(min(iters, 3)):
            run(i)                               # everything lazily set up before the capture; warm-up
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=st):
            for i in range(iters):
                run(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (iters * replays)


# ------------------------------------------------------------------------------------- main arm

def run_ours(args):
    import torch
    import torch.distributed as dist
    from turkce_llm_b200 import lib
    from turkce_llm_b200.data_parallel import DataParallel
    from turkce_llm_b200.gpu_train import GRADS, AdamState, GpuTrainer

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs a torchrun launch with %d ranks" % (args.gpus, args.gpus))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    V, D, H, L, F = (MODEL[k] for k in "VDHLF")
    B, T = BATCH, CONTEXT
    if args.global_batch:
        rec = fixed_global_batch(args, rank, world, local, args.global_batch, args.steps, max(args.warmup, 3))
        if rank == 0:
            print(json.dumps(rec), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    g = GpuTrainer(V, D, H, L, F, T, B, 1e-5, device=local)
    p0 = init_params(g.total, g.param_layout(), seed=0)
    g.upload(p0)
    dp = DataParallel(g, rank, world, dist if world > 1 else None)
    opt = AdamState(LR, BETA1, BETA2, ADAM_EPS)
    # the trainer issues its work on a stream of its own; time and order everything on that stream
    ext = torch.cuda.ExternalStream(g.stream_ptr())
    torch.cuda.set_stream(ext)

    n_batches = 4
    stream = zipf_ids(n_batches * B * T + 1, V, seed=1 + 1000 * rank)
    batches = [(stream[i * B * T:(i + 1) * B * T].copy(), stream[i * B * T + 1:(i + 1) * B * T + 1].copy())
               for i in range(n_batches)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    warm = max(args.warmup, 3)
    # ---- device-resident leg: inputs already in HBM, no host transfer, no host sync per step
    sampler = ClockSampler(local) if rank == 0 else None
    g.set_inputs(*batches[0])
    for _ in range(warm):
        dp.step_resident(opt, MAX_NORM)
    barrier()
    launches0 = lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e0.record()
    for _ in range(args.steps):
        dp.step_resident(opt, MAX_NORM)
    e1.record()
    barrier()
    if sampler:
        sampler.window(w0, time.time())
    ms_value = max_over_ranks(e0.elapsed_time(e1))
    launches = lib.launch_count() - launches0
    loss_resident = g.read_loss()

    # ---- end-to-end leg: host ids in, loss out, every step
    for i in range(2):
        dp.step_host(batches[i % n_batches][0], batches[i % n_batches][1], opt, MAX_NORM)
    barrier()
    w0 = time.time()
    e0.record()
    loss = None
    for i in range(args.steps):
        loss, _ = dp.step_host(batches[i % n_batches][0], batches[i % n_batches][1], opt, MAX_NORM)
    e1.record()
    barrier()
    if sampler:
        sampler.window(w0, time.time())
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if sampler else None

    # ---- per-kernel timing of one step (CUDA events around every launch).  The stream is first held busy
    # for ~10 ms, so that the host has queued the whole step before the GPU starts on it: the events then
    # bracket the kernels back to back instead of the host's launch cost.
    with torch.cuda.stream(torch.cuda.ExternalStream(g.stream_ptr())):
        torch.cuda._sleep(20_000_000)
    lib.profile_begin()
    dp.step_resident(opt, MAX_NORM)
    prof = lib.profile_end(g.stream_ptr())
    torch.cuda.synchronize()

    repro = reproducibility(dp, g, p0, batches, opt.__class__, dist if world > 1 else None) if world > 1 else None

    tokens_per_step = B * T * world
    result = {
        "metric": METRIC, "value": tokens_per_step * args.steps / (ms_value / 1e3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": ms_value / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "single-B200 full training step of the 33,490,176-parameter decoder "
                               "(12 layers, d_model 384, 6 heads x 64, SwiGLU d_ff 1024, tied 31,769 vocab): "
                               "forward, backward, clip, Adam; bf16 tensor-core GEMMs, fp32 accumulation and master weights",
                   "per_gpu_batch": B, "context": T, "global_batch": B * world,
                   "parallelism": "dp%d" % world, "data_parallel": dp.describe(),
                   "l2": "no flush needed: one step streams about 5 GB of activations, 40x the 126 MB L2",
                   "token_ids": "Zipf(1.1) over the vocabulary, seed 1 (+1000*rank)"},
        "e2e": {"value": tokens_per_step * args.steps / (ms_e2e / 1e3), "unit": UNIT,
                "h2d_bytes_per_step": 2 * B * T * 4 + (6 * B * T + 2) * 4, "d2h_bytes_per_step": B * T * 4 + 8,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches),
        "final_loss": loss, "loss_resident": loss_resident,
    }
    if repro is not None:
        result["repro"] = repro
    if rank == 0:
        result["clocks"] = clocks
        result["roofline"] = roofline(prof, ms_value / args.steps, ms_value / 1e3, clocks)
        kern = {}
        for k, v in prof.items():
            name = k.split(":")[0]
            e = kern.setdefault(name, {"launches": 0, "ms": 0.0})
            e["launches"] += v["launches"]
            e["ms"] += v["ms"]
        result["kernels"] = {k: {"launches": v["launches"], "ms": round(v["ms"], 4)} for k, v in
                             sorted(kern.items(), key=lambda kv: -kv[1]["ms"])}
        if os.environ.get("TB_BENCH_GEMM_SHAPES"):
            result["gemm_shapes"] = {k: {"launches": v["launches"], "ms": round(v["ms"], 4),
                                         "tflops": round(v["flops"] / (v["ms"] * 1e-3) / 1e12, 1) if v["ms"] > 0 else 0}
                                     for k, v in sorted(prof.items(), key=lambda kv: -kv[1]["ms"])
                                     if k.startswith("gemm_")}
    dp.destroy()
    g.destroy()
    del g
    torch.cuda.set_stream(torch.cuda.default_stream())

    # ---- sub-records, all outside the timed regions above
    if not args.no_extras:
        c5_steps = 3 if world == 1 else 6
        c5 = fixed_global_batch(args, rank, world, local, 128, c5_steps, 2, with_sampler=False)
        if rank == 0:
            result["c5"] = {k: c5[k] for k in ("value", "unit", "ms_per_step", "steps", "warmup", "scaling", "config",
                                               "final_loss", "grad_norm", "gpu_launches")}
        if rank == 0 and world == 1:
            for name, fn in (("tf32_step", bench_tf32_step), ("c1", bench_c1), ("c3", bench_c3), ("c4", bench_c4),
                             ("reference_gpu_trainer", bench_reference_gpu_trainer),
                             ("cpu_baseline", cpu_baseline_port)):
                try:
                    result[name] = fn()
                except Exception as e:                      # a failed sub-record must not lose the headline
                    result[name] = {"error": "%s: %s" % (type(e).__name__, e)}
    if rank == 0:
        print(json.dumps(result), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def reproducibility(dp, g, p0, batches, AdamStateCls, dist):
    """Bitwise reproducibility across ranks as data: from the same start weights and zero optimiser state, the
    same two data-parallel steps are run twice; loss, gradient norm and a SHA-256 of the flat gradients and of
    the updated weights must come out bit-identical, on every rank."""
    import torch
    from turkce_llm_b200.gpu_train import GRADS, PARAMS, ADAM_M, ADAM_V
    zeros = np.zeros(g.total, np.float32)
    runs = []
    for _ in range(2):
        g.upload(p0)
        g.upload(zeros, ADAM_M)
        g.upload(zeros, ADAM_V)
        opt = AdamStateCls(LR, BETA1, BETA2, ADAM_EPS)
        out = []
        for i in range(2):
            loss, norm = dp.step_host(batches[i][0], batches[i][1], opt, MAX_NORM)
            out.append((np.float32(loss).tobytes().hex(), np.float64(norm).tobytes().hex()))
        out.append(hashlib.sha256(g.download(GRADS).tobytes()).hexdigest())
        out.append(hashlib.sha256(g.download(PARAMS).tobytes()).hexdigest())
        runs.append(out)
    same = [runs[0][i] == runs[1][i] for i in range(4)]
    flags = torch.tensor([1.0 if all(same[:2]) else 0.0, 1.0 if same[2] else 0.0, 1.0 if same[3] else 0.0], device="cuda")
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    # replicas must also agree with each other after the step: compare the weight hashes across ranks
    h = torch.tensor(list(bytes.fromhex(runs[0][3])), device="cuda", dtype=torch.float32)
    lo, hi = h.clone(), h.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    f = flags.cpu().numpy()
    return {"steps": 2, "loss_and_norm_bits_equal": bool(f[0] > 0.5), "grads_sha_equal": bool(f[1] > 0.5),
            "params_sha_equal": bool(f[2] > 0.5), "replicas_identical": bool(torch.equal(lo, hi)),
            "loss_bits": [r[0] for r in runs[0][:2]], "norm_bits": [r[1] for r in runs[0][:2]]}


def fixed_global_batch(args, rank, world, local, G, steps, warmup, with_sampler=True):
    """The data-parallel configuration with a FIXED global batch (strong scaling): G sequences of 1024 tokens per
    optimiser step, split over the ranks by sequence index and processed as micro-batches of 16 sequences whose
    gradients accumulate; the ranks' sums are combined once per optimiser step.  Every step draws its windows
    from a host token stream (pinned staging + H2D inside the timed region) and reads the loss back, so `value`
    and `e2e` are the same end-to-end measurement."""
    import torch
    import torch.distributed as dist
    from turkce_llm_b200 import lib
    from turkce_llm_b200.data_parallel import DataParallel, micro_batches, shard_sequences
    from turkce_llm_b200.gpu_train import AdamState, GpuTrainer, sample_batch

    V, D, H, L, F = (MODEL[k] for k in "VDHLF")
    T, micro = CONTEXT, 16
    first, count = shard_sequences(G, world, rank)
    plan = micro_batches(first, count, micro)
    g = GpuTrainer(V, D, H, L, F, T, micro, 1e-5, device=local)
    g.upload(init_params(g.total, g.param_layout(), seed=0))
    dp = DataParallel(g, rank, world, dist if world > 1 else None)
    opt = AdamState(LR, BETA1, BETA2, ADAM_EPS)
    torch.cuda.set_stream(torch.cuda.ExternalStream(g.stream_ptr()))
    tokens = zipf_ids(4_000_000, V, seed=4)          # the same stream on every rank: ranks differ by sequence index

    def one_step(s):
        batches = [sample_batch(tokens, T, c, 2026 + s, first_sequence=f) for f, c in plan]
        return dp.step_host_accumulate(batches, opt, MAX_NORM)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if (rank == 0 and with_sampler) else None
    for s in range(warmup):
        one_step(s)
    barrier()
    launches0 = lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e0.record()
    loss = norm = None
    for s in range(steps):
        loss, norm = one_step(100 + s)
    e1.record()
    barrier()
    if sampler:
        sampler.window(w0, time.time())
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    launches = lib.launch_count() - launches0
    value = G * T * steps / (ms / 1e3)
    describe = dp.describe()
    dp.destroy()
    g.destroy()
    torch.cuda.set_stream(torch.cuda.default_stream())
    return {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "data-parallel training of the 33,490,176-parameter decoder with a fixed global "
                               "batch: %d sequences x %d tokens per optimiser step, %d micro-batches of %d "
                               "sequences per rank, gradients combined once per step"
                               % (G, T, len(plan), micro),
                   "global_batch": G, "context": T, "parallelism": "dp%d" % world, "data_parallel": describe,
                   "l2": "no flush needed: a micro-batch streams about 10 GB, far beyond the 126 MB L2",
                   "token_ids": "Zipf(1.1) over the vocabulary, seed 4; windows drawn per global sequence index"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": len(plan) * (2 * micro * T * 4 + (6 * micro * T + 2) * 4),
                "d2h_bytes_per_step": len(plan) * (micro * T * 4 + 8), "ms_per_step": ms / steps},
        "gpu_launches": int(launches), "final_loss": loss, "grad_norm": norm,
        "clocks": sampler.stop() if sampler else None}


def roofline(prof, step_ms, timed_region_s, clocks):
    """Roofline of the dominant kernel (the tcgen05 GEMM): algorithmic flops of all its launches in one step
    / their summed duration.  Denominator: the measured BURST bf16 peak when the timed region is short and ran
    at full clock without a power cap, the measured SUSTAINED peak when it is seconds long or the power cap was
    seen; both fractions are printed."""
    pk = peaks()
    gemm = {"launches": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0}
    for name, v in prof.items():
        if name.startswith("gemm_bf16"):
            for k in gemm:
                gemm[k] += v[k]
    if gemm["ms"] <= 0:
        return None
    achieved = gemm["flops"] / (gemm["ms"] * 1e-3) / 1e12
    total_ms = sum(v["ms"] for v in prof.values())
    n_launches = sum(v["launches"] for v in prof.values())
    overhead_us, net_tflops = None, None
    if step_ms and n_launches and total_ms > step_ms:
        overhead_us = (total_ms - step_ms) * 1e3 / n_launches
        net_ms = gemm["ms"] - gemm["launches"] * overhead_us * 1e-3
        if net_ms > 0:
            net_tflops = gemm["flops"] / (net_ms * 1e-3) / 1e12
    capped = bool(clocks and "sw_power_cap" in (clocks.get("reasons") or []))
    use_sustained = capped or timed_region_s >= 2.0
    peak = pk["sustained"] if use_sustained else pk["burst"]
    traffic = None
    if GEMM_DRAM_TRAFFIC["bytes_per_step"] and GEMM_DRAM_TRAFFIC["launches_per_step"]:
        traffic = GEMM_DRAM_TRAFFIC["bytes_per_step"] / GEMM_DRAM_TRAFFIC["launches_per_step"]
    return {"bound": "tensor", "kernel": "gemm_bf16_kernel", "achieved": achieved, "peak": peak,
            "unit": "TFLOP/s", "frac": achieved / peak,
            "peak_source": "%s bf16 %s (MEASURED_PEAKS.json): timed region %.2f s, power cap %s"
                           % (pk["src"], "sustained" if use_sustained else "burst", timed_region_s,
                              "seen" if capped else "not seen"),
            "frac_of_burst_peak": achieved / pk["burst"], "frac_of_sustained_peak": achieved / pk["sustained"],
            "traffic": traffic, "traffic_source": GEMM_DRAM_TRAFFIC["source"],
            "traffic_bytes_per_step": GEMM_DRAM_TRAFFIC["bytes_per_step"],
            "launches_per_step": gemm["launches"], "ms_per_step": gemm["ms"],
            "share_of_step": gemm["ms"] / total_ms if total_ms > 0 else None,
            "algorithmic_gflop_per_step": gemm["flops"] / 1e9,
            "algorithmic_gbytes_per_step": gemm["bytes"] / 1e9,
            "algorithmic_bytes_per_launch": gemm["bytes"] / gemm["launches"],
            "achieved_gbs": gemm["bytes"] / (gemm["ms"] * 1e-3) / 1e9,
            # Events around every launch serialise the step (no overlap of one kernel's prologue with the
            # previous kernel's tail, no graph replay): the per-kernel times sum to more than the live step.
            # Spreading that excess evenly over the launches gives the GEMM time inside the live step.
            "event_overhead_us_per_launch": overhead_us,
            "achieved_net_of_event_overhead": net_tflops,
            "frac_net_of_event_overhead": net_tflops / peak if net_tflops else None}


# ------------------------------------------------------------------------------------- sub-records

C1_SHAPES = (("qkv", 384, 1152), ("out", 384, 384), ("gate_up", 384, 2048), ("down", 1024, 384))   # name, K, N


def _gemm_case(lib, torch, kind, M, N, K, precision, iters=20):
    """Device time of one GEMM through the float32 entry point (TF32, FP32 modes) or the native bf16 entry point
    (BF16: operands already packed, as the trainer keeps them), in a CUDA graph, on rotating operand sets larger
    than L2 together."""
    a_shape = (K, M) if kind == 2 else (M, K)
    b_shape = (N, K) if kind == 1 else (K, N)
    es = 2 if precision == lib.PREC_BF16 else 4
    per_set = es * (M * K + K * N) + 4 * M * N
    copies = int(min(24, max(2, L2_BYTES * 1.3 // per_set + 1)))
    gen = torch.Generator(device="cuda").manual_seed(7)
    dt = torch.bfloat16 if precision == lib.PREC_BF16 else torch.float32
    As = [torch.randn(a_shape, device="cuda", generator=gen).to(dt) for _ in range(copies)]
    Bs = [(torch.randn(b_shape, device="cuda", generator=gen) * 0.02).to(dt) for _ in range(copies)]
    Cs = [torch.empty(M, N, device="cuda") for _ in range(copies)]

    def run(i):
        j = i % copies
        if precision == lib.PREC_BF16:
            lib.gemm_bf16(kind, As[j], Bs[j], M, N, K, a_shape[1], b_shape[1], C32=Cs[j], ldc32=N)
        else:
            lib.gemm_f32(kind, As[j], Bs[j], Cs[j], M, N, K, a_shape[1], b_shape[1], N, precision=precision)
    us = graph_time_us(run, iters)
    lib.sync_check()
    return us, copies


def bench_c1():
    """One layer's four linear GEMMs at M = 4 x 256 tokens (and at M = 8192, the training step's token count),
    forward, dX and dW, in the three operand precisions: device time per call, TFLOP/s, and the largest error
    relative to max|want| against the CPU oracle on the seeded inputs of the parity tests; beside them the
    reference's own tensor_matmul2d + backward on the host cores (1 thread, 4 threads x 256 rows, all cores)."""
    import torch
    from oracle.pyoracle import Oracle
    from turkce_llm_b200 import lib
    lib.init(0)
    o = Oracle()
    o.set_threads(min(os.cpu_count() or 8, 64))
    pk = peaks()
    precisions = (("bf16", lib.PREC_BF16, 2e-2), ("tf32", lib.PREC_TF32, 5e-3), ("fp32", lib.PREC_FP32, 1e-5))
    forms = (("fwd", 0), ("dX", 1), ("dW", 2))
    rows = []
    rng = np.random.default_rng(0)
    worst = {p[0]: 0.0 for p in precisions}
    for name, K, N in C1_SHAPES:
        M = 1024
        X = rng.standard_normal((M, K)).astype(np.float32)
        W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        dY = rng.standard_normal((M, N)).astype(np.float32)
        for form, kind in forms:
            # (A, B, m, n, k) of this form as the entry point takes it
            A, Bm, m, n, k = {"fwd": (X, W, M, N, K), "dX": (dY, W, M, K, N), "dW": (X, dY, K, N, M)}[form]
            truth = o.gemm_f64(kind // 2, kind % 2, A, Bm, m, n, k).reshape(m, n)
            want32 = o.gemm(kind // 2, kind % 2, A, Bm, m, n, k).reshape(m, n)
            dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(Bm).cuda()
            for pname, prec, bound in precisions:
                C = torch.zeros(m, n, device="cuda")
                lib.gemm_f32(kind, dA, dB, C, m, n, k, A.shape[1], Bm.shape[1], n, precision=prec)
                lib.sync_check()
                got = C.cpu().numpy().astype(np.float64)
                ref = truth if pname == "fp32" else want32
                err = float(np.abs(got - ref).max() / np.abs(ref).max())
                worst[pname] = max(worst[pname], err)
                row = {"gemm": name, "form": form, "precision": pname, "M": m, "N": n, "K": k,
                       "max_rel_err": err, "bound": bound}
                for big in (False, True):
                    mm, nn, kk = (m, n, k)
                    if big:       # the same GEMM at the training step's 8192 tokens
                        mm, nn, kk = {"fwd": (8192, N, K), "dX": (8192, K, N), "dW": (K, N, 8192)}[form]
                    us, copies = _gemm_case(lib, torch, kind, mm, nn, kk, prec, iters=20 if big else 40)
                    tf = 2.0 * mm * nn * kk / us / 1e6
                    key = "tokens_8192" if big else "tokens_1024"
                    row[key] = {"us": round(us, 2), "tflops": round(tf, 1),
                                "frac_of_burst_bf16_peak": round(tf / pk["burst"], 4), "operand_sets": copies}
                rows.append(row)
    rec = {"workload": "one layer's linear GEMMs (QKV 384->1152, out 384->384, gate|up 384->2048, down 1024->384), "
                       "forward + dX + dW; X, dY ~ N(0,1), W ~ N(0,0.02), seed 0",
           "timing": "device time per call inside a CUDA graph, operand sets rotated so that together they exceed L2; "
                     "bf16: native bf16 entry point (operands packed once, as the trainer keeps them), "
                     "tf32 / fp32: float32 entry point, conversion kernels included",
           "tf32_peak_note": "no measured TF32 peak exists for this pool; fractions are of the measured burst bf16 peak "
                             "(nominal TF32 is half of bf16)",
           "worst_rel_err": worst, "error_metric": "max|got - want| / max|want| against the float32 CPU oracle "
                                                    "(float64 product for the fp32 mode)",
           "gemms": rows}
    try:
        rec["cpu_reference"] = c1_cpu_reference()
    except Exception as e:
        rec["cpu_reference"] = {"error": "%s: %s" % (type(e).__name__, e)}
    return rec


def c1_cpu_reference():
    """The reference's tensor_matmul2d + node_matmul2d backward (unmodified sources in oracle/_ref/libref.so) on
    the four layer GEMMs at M = 1024: one thread; four threads with one 256-row sequence each (the reference's
    one-sequence-per-thread scheme, training/data_parallel.c:126-140, each worker with its own weight gradient);
    and row blocks over all host cores."""
    from oracle import pyoracle
    if not os.path.exists(pyoracle.REF_SO):
        return {"unavailable": "oracle/_ref/libref.so is not built on this machine"}
    ref = pyoracle.Ref()
    cores = os.cpu_count() or 1
    rng = np.random.default_rng(0)
    M = 1024
    ops = []
    for name, K, N in C1_SHAPES:
        ops.append((rng.standard_normal((M, K)).astype(np.float32), (rng.standard_normal((K, N)) * 0.02).astype(np.float32),
                    rng.standard_normal((M, N)).astype(np.float32)))
    flops = sum(3 * 2.0 * M * x.shape[1] * w.shape[1] for x, w, _ in ops)

    def run(parts):
        t0 = time.time()
        for X, W, dY in ops:
            blocks = np.array_split(np.arange(M), parts)
            th = [threading.Thread(target=ref.matmul2d_fwd_bwd, args=(X[b[0]:b[-1] + 1], W, dY[b[0]:b[-1] + 1]))
                  for b in blocks if len(b)]
            for t in th:
                t.start()
            for t in th:
                t.join()
        return time.time() - t0
    out = {"code": "tensor_matmul2d + backward_matmul2d of the reference, gcc -std=c11 -O2", "host_cores": cores,
           "gflop": flops / 1e9, "cpu_model": cpu_model()}
    for label, parts in (("threads_1", 1), ("threads_4_x_256_rows", 4), ("all_cores_row_blocks", min(cores, 256))):
        sec = run(parts)
        out[label] = {"threads": parts, "seconds": round(sec, 3), "gflops": round(flops / sec / 1e9, 2)}
    return out


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def bench_c3():
    """Fused causal attention at B=16, H=6, T=1024, hd=64 (bf16): device time of the forward and backward
    kernels, and TFLOP/s of the causal-useful flops (lower triangle only: 2 products forward, 5 backward)."""
    import torch
    from turkce_llm_b200 import lib
    lib.init(0)
    B, H, T, hd = 16, 6, 1024, 64
    pk = peaks()
    gen = torch.Generator(device="cuda").manual_seed(2)
    sets = 4          # 4 x (Q, K, V, att, datt) = 4 x 63 MB > L2
    Q, K, V = ([torch.randn(B * H, T, hd, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(sets)] for _ in range(3))
    att = [torch.zeros(B * T, H * hd, device="cuda", dtype=torch.bfloat16) for _ in range(sets)]
    datt = [torch.randn(B * T, H * hd, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(sets)]
    lse = [torch.zeros(B * H, T, device="cuda") for _ in range(sets)]
    delta = torch.zeros(B * H, T, device="cuda")
    dQ, dK, dV = (torch.zeros(B * H, T, hd, device="cuda") for _ in range(3))
    scale = float(hd) ** -0.5
    for j in range(sets):
        lib.attention_fwd(Q[j], K[j], V[j], att[j], lse[j], B, H, T, hd, scale)
    f_us = graph_time_us(lambda i: lib.attention_fwd(Q[i % sets], K[i % sets], V[i % sets], att[i % sets], lse[i % sets],
                                                     B, H, T, hd, scale), 12)
    b_us = graph_time_us(lambda i: lib.attention_bwd(Q[i % sets], K[i % sets], V[i % sets], att[i % sets], datt[i % sets],
                                                     lse[i % sets], delta, dQ, dK, dV, B, H, T, hd, scale), 12)
    lib.sync_check()
    tri = float(B * H) * T * T * hd            # multiply-adds of one lower-triangular product (half of T*T*hd, x2 flops)
    f_tf, b_tf = 2 * tri / f_us / 1e6, 5 * tri / b_us / 1e6
    return {"workload": "B=16, H=6, T=1024, head dim 64, bf16; q, k, v ~ N(0,1), seed 2",
            "fwd": {"us": round(f_us, 1), "causal_useful_tflops": round(f_tf, 1), "frac_of_burst_bf16_peak": round(f_tf / pk["burst"], 4)},
            "bwd": {"us": round(b_us, 1), "causal_useful_tflops": round(b_tf, 1), "frac_of_burst_bf16_peak": round(b_tf / pk["burst"], 4),
                    "kernels": "delta + dK/dV + dQ (dS blocks handed from the dK/dV kernel to the dQ kernel: 5 triangular products)"},
            "algorithmic_mb_fwd": round(4 * B * H * T * hd * 2 / 1e6, 1),
            "timing": "device time per call inside a CUDA graph, 4 operand sets in rotation (252 MB > L2)"}


def bench_c4(S=64, prompt_len=128, n_new=128, with_lm_head=True):
    """Batched greedy decoding with a KV cache: 64 sequences, 128-token Zipf(1.1) prompts, 128 new tokens;
    random bf16 weights (seed 3).  HBM roofline: the step streams all weights once (66.9 MB) and the cache up to
    the current length (1.18 MB per position over all layers and sequences)."""
    import torch
    from turkce_llm_b200 import lib
    from turkce_llm_b200.decode import Decoder
    V, D, H, L, F = (MODEL[k] for k in "VDHLF")
    pk = peaks()
    dec = Decoder(V, D, H, L, F, S, prompt_len + n_new + 1)
    rng = np.random.default_rng(3)
    dec.upload((rng.standard_normal(dec.total) * 0.02).astype(np.float32))
    w = 1.0 / np.arange(1, V + 1, dtype=np.float64) ** 1.1
    cdf = np.cumsum(w / w.sum())
    prompts = np.minimum(np.searchsorted(cdf, rng.random((S, prompt_len))), V - 1).astype(np.uint32)
    st = torch.cuda.ExternalStream(dec.stream_ptr())
    dec.prefill(prompts)
    dec.generate(3)                      # eager step, capture, first replay
    dec.tokens(4)
    # the whole workload (prompt pass + 127 steps, 50 ms) once more as warm-up, so that the timed passes start on a
    # GPU that is already busy; then two timed passes back to back, their mean reported, clocks sampled over both
    dec.prefill(prompts)
    dec.generate(n_new - 1)
    sampler = ClockSampler(torch.cuda.current_device(), period_s=0.002)
    passes = 2
    e = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(passes)]
    launches0 = lib.launch_count()
    w0 = time.time()
    with torch.cuda.stream(st):
        for k in range(passes):
            e[k][0].record()
            dec.prefill(prompts)
            e[k][1].record()
            dec.generate(n_new - 1)
            e[k][2].record()
    toks = dec.tokens(n_new)
    sampler.window(w0, time.time())
    clocks = sampler.stop()
    launches = (lib.launch_count() - launches0) / passes
    pre_ms = sum(x[0].elapsed_time(x[1]) for x in e) / passes
    gen_ms = sum(x[1].elapsed_time(x[2]) for x in e) / passes
    step_us = gen_ms * 1e3 / (n_new - 1)
    dec.destroy()
    weight_bytes = 2.0 * (L * (D * 3 * D + D * D + D * 2 * F + F * D) + V * D)
    mean_len = prompt_len + (n_new - 1) / 2.0 + 1
    kv_bytes = S * L * 2 * mean_len * D * 2.0
    gbs = (weight_bytes + kv_bytes) / step_us / 1e3
    rec = {"workload": "%d sequences, %d-token Zipf(1.1) prompts, %d greedy tokens, cache length %d..%d; bf16 weights, seed 3"
                       % (S, prompt_len, n_new, prompt_len, prompt_len + n_new),
           "prefill_ms": round(pre_ms, 3), "prefill_tokens_per_s": round(S * prompt_len / pre_ms * 1e3),
           "decode_us_per_step": round(step_us, 1), "decode_tokens_per_s": round(S / step_us * 1e6),
           "algorithmic_mb_per_step": {"weights": round(weight_bytes / 1e6, 1), "kv_cache_mean": round(kv_bytes / 1e6, 1)},
           "achieved_gbs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / pk["hbm"], 4),
           "launches_per_token": round(launches / n_new, 1), "first_tokens": toks[0, :4].tolist(),
           "timing": "CUDA events on the decoder's stream; one untimed pass of the same workload, then the mean of 2 passes",
           "clocks": {k: clocks.get(k) for k in ("sm_mhz", "sm_min_mhz", "sm_max_mhz", "reasons", "samples")}}
    if with_lm_head:
        rec["lm_head"] = bench_lmhead()
    return rec


def bench_lmhead(S=64, V=31769, K=384, iters=40, copies=8):
    """Decode-time LM head [S, K] x [V, K]^T with the fused greedy choice.  `copies` tables are used in turn so
    that every launch streams its table from HBM (8 x 24.4 MB is larger than the 126 MB L2)."""
    import torch
    from turkce_llm_b200 import lib
    lib.init(0)
    pk = peaks()
    X = torch.randn(S, K, device="cuda").to(torch.bfloat16)
    Es = [(torch.randn(V, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
    tok = torch.zeros(S, device="cuda", dtype=torch.int32)
    for i in range(copies):
        lib.lmhead_argmax_bf16(X, Es[i], tok)
    lib.sync_check()
    want = (X.float() @ Es[copies - 1].float().t()).argmax(1).to(torch.int32)
    agree = int((want == tok).sum())
    nbytes = 2.0 * V * K + 2.0 * S * K
    gus = graph_time_us(lambda i: lib.lmhead_argmax_bf16(X, Es[i % copies], tok), iters)
    sus = graph_time_us(lambda i: lib.lmhead_argmax_bf16(X, Es[i % copies], tok, table_is_stable=True), iters)
    lib.sync_check()
    return {"shape": "[%d x %d] . [%d x %d]^T, fused argmax, logits never written" % (S, K, V, K),
            "us": round(gus, 2), "achieved_gbs": round(nbytes / gus / 1e3, 1), "frac_of_measured_hbm": round(nbytes / gus / 1e3 / pk["hbm"], 4),
            "us_table_stable": round(sus, 2), "achieved_gbs_table_stable": round(nbytes / sus / 1e3, 1),
            "frac_of_measured_hbm_table_stable": round(nbytes / sus / 1e3 / pk["hbm"], 4),
            "algorithmic_mb": round(nbytes / 1e6, 2), "tokens_agree_with_float32_product": "%d of %d" % (agree, S)}


def bench_reference_gpu_trainer(steps=8):
    """The reference's own GPU-resident trainer (model/gpu_train.c unmodified; the checker library
    oracle/_ref/librefgpu.so) on the same GPU and the same step, in a child process, twice: with its own 26 kernels
    compiled for sm_100a (the kernels this library replaces), and with the module in which its GEMM entries are this
    library's Driver-API cubin kernels (turkce_llm_b200/csrc/cubin/gemm_ref_abi.cu) and everything else is unchanged."""
    from oracle import ref_gpu
    if not ref_gpu.available():
        return {"unavailable": "oracle/_ref/librefgpu.so / train_kernels.cubin are not built on this machine"}
    V, D, H, L, F = (MODEL[k] for k in "VDHLF")
    out_rec = {}
    with tempfile.TemporaryDirectory() as tmp:
        tok = os.path.join(tmp, "tokens.npy")
        out = os.path.join(tmp, "out.json")
        np.save(tok, zipf_ids(400_000, V, 1))
        for key, module in (("own_kernels", ref_gpu.REFGPU_CUBIN), ("with_this_librarys_gemm_cubin", ref_gpu.REFGPU_TB_CUBIN)):
            if not os.path.exists(module):
                out_rec[key] = {"unavailable": os.path.basename(module) + " is not built on this machine"}
                continue
            runs = []
            for n in (2, 2 + steps):        # the difference of two runs leaves out context set-up and the first step
                r = ref_gpu.run_child(["trajectory", "--module", module, "--cfg", V, D, H, L, F, CONTEXT, BATCH, "--tokens", tok,
                                       "--steps", n, "--out", out], timeout=600)
                if r.returncode != 0:
                    runs = None
                    out_rec[key] = {"error": (r.stderr or r.stdout)[-400:]}
                    break
                runs.append(json.load(open(out)))
            if runs:
                sec = (runs[1]["seconds"] - runs[0]["seconds"]) / steps
                out_rec[key] = {"ms_per_step": round(sec * 1e3, 2), "tokens_per_s": round(BATCH * CONTEXT / sec),
                                "first_loss": runs[1]["losses"][0], "loss_after_%d_steps" % (2 + steps): runs[1]["losses"][-1]}
    out_rec["what"] = ("gpu_trainer_forward_backward + grad_norm + adam_step_scaled of the reference's unmodified host code, "
                       "batch 8 x 1024; %d steps (difference of a %d-step and a 2-step run)" % (steps, 2 + steps))
    if "ms_per_step" in out_rec.get("own_kernels", {}):
        out_rec["ms_per_step"] = out_rec["own_kernels"]["ms_per_step"]
        out_rec["tokens_per_s"] = out_rec["own_kernels"]["tokens_per_s"]
    return out_rec


def bench_tf32_step(steps=10):
    """The same training step with the linear-layer GEMMs in TF32 mode (float32 weights and activations read by
    the tensor cores as tf32): device-resident step time and the GEMM roofline against the TF32 peak.  No TF32 peak
    has been measured on this pool, so the denominator is half the measured burst bf16 peak (the nominal ratio)."""
    import torch
    from turkce_llm_b200 import lib
    from turkce_llm_b200.gpu_train import AdamState, GpuTrainer
    V, D, H, L, F = (MODEL[k] for k in "VDHLF")
    B, T = BATCH, CONTEXT
    pk = peaks()
    g = GpuTrainer(V, D, H, L, F, T, B, 1e-5, precision=lib.PREC_TF32)
    g.upload(init_params(g.total, g.param_layout(), seed=0))
    opt = AdamState(LR, BETA1, BETA2, ADAM_EPS)
    stream = zipf_ids(B * T + 1, V, seed=1)
    g.set_inputs(stream[:-1].copy(), stream[1:].copy())
    st = torch.cuda.ExternalStream(g.stream_ptr())
    with torch.cuda.stream(st):
        for _ in range(4):
            g.step_resident(opt, MAX_NORM)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            g.step_resident(opt, MAX_NORM)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        loss = g.read_loss()
        torch.cuda._sleep(20_000_000)
        lib.profile_begin()
        g.step_resident(opt, MAX_NORM)
        prof = lib.profile_end(g.stream_ptr())
        torch.cuda.synchronize()
    g.destroy()
    gemm = {"launches": 0, "ms": 0.0, "flops": 0.0}
    for name, v in prof.items():
        if name.startswith("gemm_tf32"):
            for k in gemm:
                gemm[k] += v[k]
    achieved = gemm["flops"] / (gemm["ms"] * 1e-3) / 1e12 if gemm["ms"] > 0 else None
    peak = pk["burst"] / 2
    return {"dtype": "tf32", "ms_per_step": round(ms, 3), "tokens_per_s": round(B * T / ms * 1e3), "steps": steps,
            "loss_after": loss,
            "workload": "the headline training step with TB_PREC_TF32: float32 operands as tf32 in every linear-layer "
                        "GEMM (forward, dX, dW, LM head); attention core bf16",
            "roofline": {"bound": "tensor", "kernel": "gemm_bf16_kernel<BN, TF32>", "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak if achieved else None,
                         "peak_source": "half of the %s burst bf16 peak (no TF32 peak measured on this pool)" % pk["src"],
                         "launches_per_step": gemm["launches"], "ms_per_step": gemm["ms"],
                         "algorithmic_gflop_per_step": gemm["flops"] / 1e9}}


def cpu_baseline_port():
    """The CPU oracle (a plain-C port of the reference's algorithm) on the host cores, bounded sample: one full
    training step (forward, backward, gradient norm, Adam) at the reference's own CPU sequence length of 128
    (training/train_lm.c:34), one sequence per host core."""
    from oracle.pyoracle import Oracle
    o = Oracle()
    cores = min(os.cpu_count() or 1, 256)
    o.set_threads(cores)
    V, D, H, L, F = (MODEL[k] for k in "VDHLF")
    B, T = max(4, min(cores, 32)), 128
    cfg = (V, D, H, L, F, T, B, 1e-5)
    total = o.model_total_scalars(cfg)
    p = (np.random.default_rng(0).standard_normal(total) * 0.02).astype(np.float32)
    m, v = np.zeros_like(p), np.zeros_like(p)
    ids = zipf_ids(B * T + 1, V, 1)
    t0 = time.time()
    _, grads, _ = o.model_forward_backward(cfg, p, ids[:-1], ids[1:])
    norm = o.grad_norm(grads)
    o.adam(p, grads, m, v, LR, BETA1, BETA2, ADAM_EPS, 1 - BETA1, 1 - BETA2, min(1.0, MAX_NORM / max(norm, 1e-30)))
    dt = time.time() - t0
    return {"value": B * T / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "one training step (forward, backward, gradient norm, Adam) of the full 12-layer model on "
                      "%d sequences x %d tokens, %.1f s" % (B, T, dt)}


# ------------------------------------------------------------------------------------- reference arm

def run_reference(args):
    """The reference's own CPU training step on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import pyoracle
    V, D, H, L, F = (MODEL[k] for k in "VDHLF")
    cores = os.cpu_count() or 1
    budget_s = 200.0
    if os.path.exists(pyoracle.REF_SO):
        kind = "reference"
        ref = pyoracle.Ref()
        workers = max(1, min(cores, 64))          # DATA_PARALLEL_MAX_WORKERS
        T = 128                                   # SEQ_LEN of the reference's CPU training main (training/train_lm.c:34)
        lm = pyoracle.RefLM(ref, V, D, H, L, F, 1e-5, 1337, 1, arena=8 << 30)
        tokens = zipf_ids(400000, V, 1)

        def one(step):
            lm.dp_step(tokens, T, workers, 2026 + step, step_arena=3 << 30)
            lm.adam_step(LR)
        sample = ("data_parallel_step + adam_step of the reference's unmodified C sources: %d worker threads x "
                  "%d tokens per step (one sequence per thread, the reference's own SEQ_LEN)" % (workers, T))
        tokens_per_step = workers * T
    else:
        kind = "port"
        o = pyoracle.Oracle()
        workers = min(cores, 256)
        o.set_threads(workers)
        B, T = 4, 128
        cfg = (V, D, H, L, F, T, B, 1e-5)
        p = (np.random.default_rng(0).standard_normal(o.model_total_scalars(cfg)) * 0.02).astype(np.float32)
        ids = zipf_ids(B * T + 1, V, 1)

        def one(step):
            o.model_forward_backward(cfg, p, ids[:-1], ids[1:])
        sample = "forward+backward of the CPU port on %d x %d tokens per step" % (B, T)
        tokens_per_step = B * T
    t0 = time.time()
    one(0)
    t_first = time.time() - t0
    warm = 1
    while warm < args.warmup and (warm + 1) * t_first < 0.2 * budget_s:
        one(warm)
        warm += 1
    steps = max(1, min(args.steps, int((budget_s - warm * t_first) / max(t_first, 1e-3))))
    t0 = time.time()
    for s in range(steps):
        one(warm + s)
    dt = time.time() - t0
    value = tokens_per_step * steps / dt
    if steps < args.steps or warm < args.warmup:
        sample += ("; %d of the %d requested steps timed after %d warm-up step(s), to keep the run within a few minutes"
                   % (steps, args.steps, warm))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "CPU training step of the same 33,490,176-parameter decoder (bounded sample)",
                   "tokens_per_step": tokens_per_step, "context": T, "host_cores": cores, "cpu_model": cpu_model()},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": workers, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ------------------------------------------------------------------------------------- single-kernel programs

def run_only(args):
    """Small single-kernel programs (also the commands of the ncu captures): python bench.py --only <what> <numbers>
         gemm M N K kind [iters] [out=f32|bf16] [tile_n] [splits]      kind: 0 = NN, 1 = NT, 2 = TN
         timeline M N K kind [out=f32|bf16] [tile_n]     (a library built with TB_NVCC_FLAGS=-DTB_GEMM_STAMPS)
         attention B H T hd [iters]
         decode S prompt_len new_tokens
         lmhead S [V] [K] [iters] [copies]"""
    import torch
    from turkce_llm_b200 import lib
    lib.init(0)
    a = args.numbers
    if args.only == "gemm":
        M, N, K, kind = (int(x) for x in a[:4])
        iters = int(a[4]) if len(a) > 4 else 20
        out = a[5] if len(a) > 5 else "f32"
        tile_n = int(a[6]) if len(a) > 6 else 0
        splits = int(a[7]) if len(a) > 7 else 1
        a_shape = (K, M) if kind == 2 else (M, K)
        b_shape = (N, K) if kind == 1 else (K, N)
        A = torch.randn(a_shape, device="cuda").to(torch.bfloat16)
        B = (torch.randn(b_shape, device="cuda") * 0.02).to(torch.bfloat16)
        C32 = torch.empty(M, N, device="cuda") if out == "f32" else None
        C16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16) if out == "bf16" else None

        def run(i=0):
            lib.gemm_bf16(kind, A, B, M, N, K, a_shape[1], b_shape[1], C32=C32, ldc32=N, C16=C16, ldc16=N,
                          splits=splits, tile_n=tile_n)
        for _ in range(iters):
            run()
        lib.sync_check()
        us = graph_time_us(run, iters)
        print("gemm kind=%d %dx%dx%d out=%s tile_n=%d splits=%d: %.2f us per call in a CUDA graph = %.1f TFLOP/s"
              % (kind, M, N, K, out, tile_n, splits, us, 2.0 * M * N * K / us / 1e6), flush=True)
    elif args.only == "timeline":
        # where one GEMM launch spends its time: needs a library built with TB_NVCC_FLAGS=-DTB_GEMM_STAMPS
        import ctypes as C
        L = lib.load()
        if not hasattr(L, "tb_debug_gemm_stamps"):
            print("timeline: the library was built without -DTB_GEMM_STAMPS", flush=True)
            return 1
        M, N, K, kind = (int(x) for x in a[:4])
        out = a[4] if len(a) > 4 else "f32"
        tile_n = int(a[5]) if len(a) > 5 else 0
        a_shape = (K, M) if kind == 2 else (M, K)
        b_shape = (N, K) if kind == 1 else (K, N)
        sets = []
        for _ in range(4):          # 4 operand sets in turn: the last launch does not find its operands in L2 by luck
            A = torch.randn(a_shape, device="cuda").to(torch.bfloat16)
            B = (torch.randn(b_shape, device="cuda") * 0.02).to(torch.bfloat16)
            C32 = torch.empty(M, N, device="cuda") if out == "f32" else None
            C16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16) if out == "bf16" else None
            sets.append((A, B, C32, C16))
        buf = np.zeros((160, 16), dtype=np.uint64)
        for i in range(6):
            A, B, C32, C16 = sets[i % 4]
            if i == 5:
                lib.sync_check()
                L.tb_debug_gemm_stamps(buf.ctypes.data_as(C.c_void_p))        # clears what the earlier launches left
            lib.gemm_bf16(kind, A, B, M, N, K, a_shape[1], b_shape[1], C32=C32, ldc32=N, C16=C16, ldc16=N, splits=1,
                          tile_n=tile_n)
        lib.sync_check()
        L.tb_debug_gemm_stamps(buf.ctypes.data_as(C.c_void_p))
        ts = buf.astype(np.int64)
        t0 = ts[:, 0][ts[:, 0] > 0].min()
        names = ["entry", "set-up done", "first loads issued", "all loads issued", "first operands arrived",
                 "first tile's products done", "last tile's products done", "epilogue: first accumulator seen",
                 "epilogue: first tile stored", "epilogue: last tile stored", "stores have left shared memory"]
        print("gemm kind=%d %dx%dx%d out=%s tile_n=%d: %d CTAs; us after the first CTA's entry (min / median / max over CTAs)"
              % (kind, M, N, K, out, tile_n, int((ts[:, 0] > 0).sum())), flush=True)
        for i, n in enumerate(names):
            col = (ts[:, i][ts[:, i] > 0] - t0) / 1e3
            if len(col):
                print("  %-34s %6.2f %6.2f %6.2f" % (n, col.min(), float(np.median(col)), col.max()), flush=True)
    elif args.only == "attention":
        B, H, T, hd = (int(x) for x in a[:4])
        iters = int(a[4]) if len(a) > 4 else 10
        g = torch.Generator(device="cuda").manual_seed(0)
        Q, K, V = (torch.randn(B * H, T, hd, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
        att = torch.zeros(B * T, H * hd, device="cuda", dtype=torch.bfloat16)
        datt = torch.randn(B * T, H * hd, device="cuda", generator=g).to(torch.bfloat16)
        lse = torch.zeros(B * H, T, device="cuda")
        delta = torch.zeros(B * H, T, device="cuda")
        dQ, dK, dV = (torch.zeros(B * H, T, hd, device="cuda") for _ in range(3))
        scale = float(hd) ** -0.5
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        for _ in range(2):
            lib.attention_fwd(Q, K, V, att, lse, B, H, T, hd, scale)
            lib.attention_bwd(Q, K, V, att, datt, lse, delta, dQ, dK, dV, B, H, T, hd, scale)
        lib.sync_check()
        e[0].record()
        for _ in range(iters):
            lib.attention_fwd(Q, K, V, att, lse, B, H, T, hd, scale)
        e[1].record()
        for _ in range(iters):
            lib.attention_bwd(Q, K, V, att, datt, lse, delta, dQ, dK, dV, B, H, T, hd, scale)
        e[2].record()
        torch.cuda.synchronize()
        tri = B * H * T * T * hd
        f_us, b_us = e[0].elapsed_time(e[1]) * 1e3 / iters, e[1].elapsed_time(e[2]) * 1e3 / iters
        print("attention B=%d H=%d T=%d hd=%d: fwd %.1f us (%.1f TFLOP/s causal-useful)  bwd %.1f us (%.1f TFLOP/s)"
              % (B, H, T, hd, f_us, 2 * tri / f_us / 1e6, b_us, 5 * tri / b_us / 1e6), flush=True)
    elif args.only == "decode":
        nums = [int(x) for x in a[:3]]
        print(json.dumps(bench_c4(*nums, with_lm_head=False)), flush=True)
    elif args.only == "lmhead":
        print(json.dumps(bench_lmhead(*(int(x) for x in a[:5]))), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--global-batch", type=int, default=0,
                    help="fixed global batch in sequences (strong scaling, e.g. 128); default: 8 sequences per GPU")
    ap.add_argument("--no-extras", action="store_true", help="headline record only (no c1/c3/c4/c5 sub-records)")
    ap.add_argument("--only", choices=["gemm", "timeline", "attention", "decode", "lmhead"], default=None, help=run_only.__doc__)
    ap.add_argument("numbers", nargs="*")
    args = ap.parse_args()
    if args.only:
        return run_only(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
