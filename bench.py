#!/usr/bin/env python3
"""Benchmark of the quantized-weight hot path: one MoE expert block, batch 1, Qwen3-235B shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload moe_block|matvec|gemm|prefill|decode30b|decode235b] [--no-fused | --fused-mode 1|2]
                    [--no-pdl] [--collective push|nccl] [--no-extras] [--decode-tokens T] [--decode-layers L]

Workload (the MoE-block configuration of the benchmark spec): router fp32 128x4096 -> top-8 of 128 experts; per routed expert a
fused gate+up Q4_K matvec (2 x 1536x4096) with SwiGLU and a Q6_K down matvec (4096x1536), weighted
sum + residual. Weights are seeded synthetic GGUF blocks with the benchmark's distributions
(mnemocuda_b200/synth.py); no dataset or checkpoint is involved. A "step" is one block on one
layer; steps rotate over `layers` resident layers (>= 18 GB), so every pass is cold in L2.
By default a block is ONE launch of this library (mb200_moe_block: routing, gate/up, down in one
cooperative kernel); --no-fused times the three-launch form.

`value` is algorithmic GB/s (router + the 8 routed expert blobs = 100 007 936 B per step) with all
inputs resident in HBM, timed with CUDA events around a CUDA graph of the K steps, replayed 20 times
(median; the minimum is reported beside it). `e2e` is the same metric through the host-buffer call
(mb200_moe_block_host: pinned host x/residual in, result out, every step).
The same JSON line also carries, at N = 1: `parity` (the GPU result of one block against the oracle,
outside the timed region; the run fails if it is off), `matvec` (the single Q4_K 8192x4096 matvec of the
benchmark spec and the vocabulary-sized Q4_K / Q6_K matvecs) and `decode` (whole-token decode of the
30B and 235B shapes: tokens/s and the fraction of the HBM roofline).
`roofline` is for the dominant kernel (the expert phases of the fused kernel, timed alone; with
--no-fused the routed gate/up stream kernel). `cpu_baseline` and `--impl reference` time the C
oracle (the CPU restatement of the reference's algorithm -- the reference has no CPU implementation
of this path) on the box's host cores on a bounded sample (the reference arm runs numpy host logic and
the oracle only: no GPU library is loaded). N > 1 shards the experts of the block over the GPUs (router
replicated, the partial hidden vectors summed by the library's push all-reduce over NVLink peer memory;
--collective nccl times NCCL's instead): strong scaling, and the line's `sharded` key adds the NCCL
baseline, a row-sharded matvec and the sharded whole-token decode.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "Q4K/Q6K matvec HBM GB/s"
UNIT = "GB/s"
WORKLOAD = ("configs[1]: MoE expert block, batch 1, Qwen3-235B shape -- router fp32 128x4096 + top-8 of 128 "
            "experts, Q4_K gate/up 2x(1536x4096)+SwiGLU, Q6_K down 4096x1536, weighted sum + residual")

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the kernel at
# this workload's shape; it cannot be measured inside a timed run, so it is recorded here):
GATE_UP_TRAFFIC_BYTES = 56726784 + 569088    # routed gate/up stream kernel, 8 experts (56 623 104 algorithmic bytes)
BLOCK_TRAFFIC_BYTES = 100193024 + 3441792    # the whole block in one launch (100 007 936 algorithmic bytes)
FUSED_TRAFFIC_BYTES = 98054912 + 3864064     # the fused routed-expert kernel alone (98 041 856 algorithmic bytes)


def _launches_per_token(cfg, world: int) -> int:
    """Kernels of this library per decoded token: embedding + RoPE table; per layer Q/K/V (one launch), q/k-norm +
    RoPE + KV store, attention, O projection, MoE block (one launch where the one-launch form covers the shape,
    else router + gate/up + down), plus the exchanges of a sharded layer (two all-gathers and, where the block is not
    one launch with its all-reduce inside, the all-reduce); lm_head + sampling."""
    moe = 1 if (cfg.hidden % 2048 == 0 and cfg.moe_inter % 512 == 0) else 3
    per_layer = 4 + moe + ((2 if moe == 1 else 3) if world > 1 else 0)
    return 2 + per_layer * cfg.n_layers + (2 if world == 1 else 4)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": "nvmlClocksEventReasonHwSlowdown", "hw_thermal_slowdown": "nvmlClocksEventReasonHwThermalSlowdown",
                 "sw_thermal_slowdown": "nvmlClocksEventReasonSwThermalSlowdown", "sw_power_cap": "nvmlClocksEventReasonSwPowerCap"}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self.h)
                for key, const in names.items():
                    bit = getattr(nv, const, None) or getattr(nv, const.replace("Event", "Throttle"), 0)
                    if bit and (mask & bit):
                        self.reasons.add(key)
            except Exception:
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nv:
            self.t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.nv:
            self.t.join(timeout=1)

    def summary(self):
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def cpu_block_baseline(shape, experts_host, router_host, seconds=12.0, threads=None):
    """Oracle MoE blocks per second on the host cores -> GB/s of algorithmic bytes."""
    from oracle import oracle
    from mnemocuda_b200 import synth
    if not threads:  # all host cores, whatever OMP_NUM_THREADS says
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.set_num_threads(threads)
    cores = oracle.num_threads()
    s = shape
    n, t0, first = 0, time.perf_counter(), None
    while True:
        x = synth.normal_f32(900 + n, s.H)
        res = synth.normal_f32(1900 + n, s.H)
        r = oracle.moe_block(router_host, experts_host, s.stride, s.gate_sz, s.up_sz, s.down_type, s.NE, s.K, s.H,
                             s.EFF, x, res)
        if first is None:
            first = r  # (out, ids, weights) of the block on x = stream 900, residual = stream 1900: the parity check
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or n >= 4000:
            break
    return s.algorithmic_bytes * n / dt / 1e9, cores, n, dt, first


def host_layer(shape, seed=1, layer=0):
    """One layer's router + experts as host arrays (numpy generator: same streams as the device fill)."""
    from mnemocuda_b200 import synth
    s = shape
    blobs = []
    for e in range(s.NE):
        tid = (seed * 1000 + layer) * 1000 + e
        q4 = synth.q4k_blocks(tid * 2, (s.gate_sz + s.up_sz) // synth.Q4K_BLOCK).reshape(-1)
        dn = synth.q6k_blocks(tid * 2 + 1, s.down_sz // synth.Q6K_BLOCK).reshape(-1)
        blobs.append(np.concatenate([q4, dn]))
    router = synth.normal_f32(seed * 100003 + layer, s.NE * s.H, s.H ** -0.5)
    return np.concatenate(blobs), router


def run_reference(args):
    """The reference arm: the oracle (CPU restatement of the reference's algorithm) on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from types import SimpleNamespace
    from mnemocuda_b200 import synth
    g, u, d = synth.expert_sizes(4096, 1536, 14)
    shape = SimpleNamespace(NE=128, K=8, H=4096, EFF=1536, down_type=14, gate_sz=g, up_sz=u, down_sz=d, stride=g + u + d,
                            algorithmic_bytes=128 * 4096 * 4 + 8 * (g + u + d))
    experts, router = host_layer(shape)  # numpy generator: nothing of the GPU library is loaded in this arm
    from oracle import oracle
    # all host cores, also under torchrun (which sets OMP_NUM_THREADS=1 for its workers)
    oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    cores = oracle.num_threads()
    from mnemocuda_b200 import synth
    s = shape
    per_step = 4  # blocks per "step": a bounded sample of the workload
    def step(i):
        for j in range(per_step):
            x = synth.normal_f32(900 + i * per_step + j, s.H)
            res = synth.normal_f32(1900 + i * per_step + j, s.H)
            oracle.moe_block(router, experts, s.stride, s.gate_sz, s.up_sz, s.down_type, s.NE, s.K, s.H, s.EFF, x, res)
    for i in range(args.warmup):
        step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(i)
    dt = time.perf_counter() - t0
    value = s.algorithmic_bytes * per_step * args.steps / dt / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp32 (C oracle)",
            "data": "synthetic", "config": {"workload": WORKLOAD},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"{per_step} MoE blocks per step on layer 0 (C oracle, OpenMP over rows)"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


class Timer:
    """CUDA-event timing of a CUDA graph that holds `steps` steps: `replays` replays, each bracketed by events
    on the launching stream; returns (median, min) ms per step."""

    def __init__(self, torch, barrier=None):
        self.torch, self.barrier = torch, barrier or (lambda: torch.cuda.synchronize())

    def graph(self, fn, steps, warmup, replays=20):
        torch = self.torch
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(steps):
                fn(warmup + i)
        g.replay()  # untimed: instantiate / upload
        self.barrier()
        return self.replays(g, steps, replays)

    def replays(self, g, steps, replays=20):
        torch = self.torch
        times = []
        for _ in range(replays):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            self.barrier()
            times.append(e0.elapsed_time(e1) / steps)
        return float(np.median(times)), float(min(times))

    def eager(self, fn, steps, warmup):
        torch = self.torch
        for i in range(warmup):
            fn(i)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        self.barrier()
        ms = e0.elapsed_time(e1) / steps
        return ms, ms


def measure_matvec(torch, K, dev, timer, hbm, steps, warmup):
    """The plain matvecs of the path: the single Q4_K 8192 x 4096 matvec of the benchmark spec (64 weight copies in
    rotation = 1.2 GB, so every call is cold in L2; one PDL chain in one CUDA graph) and the vocabulary-sized
    Q4_K / Q6_K matvecs (151936 x 4096: 350 / 510 MB per call)."""
    out = {}
    cols = 4096
    rows1, copies = 8192, 64
    nb1 = rows1 * cols // 256
    w = torch.empty(copies * nb1 * 144, dtype=torch.uint8, device=dev)
    K.mb200_fill_q4k(w, copies * nb1, 5)
    ws = [w[i * nb1 * 144:(i + 1) * nb1 * 144] for i in range(copies)]
    x = torch.randn(cols, device=dev)
    y = torch.empty(rows1, device=dev)
    med, mn = timer.graph(lambda i: K.cuda_matvec_q4k(ws[i % copies], x, y, rows1, cols), max(steps, 2 * copies), warmup)
    by = nb1 * 144 + 4 * (rows1 + cols)
    out["cfg0_q4k_8192x4096"] = {"ms": med, "ms_min": mn, "GBs": by / med / 1e6, "frac_of_measured_hbm": by / med / 1e6 / hbm,
                                 "bytes": by, "weight_copies": copies}
    del w, ws
    rows = 151936
    for name, bb, fill, call in (("q4k_151936x4096", 144, K.mb200_fill_q4k, K.cuda_matvec_q4k),
                                 ("q6k_151936x4096", 210, K.mb200_fill_q6k, K.cuda_matvec_q6k)):
        nb = rows * cols // 256
        w = torch.empty(nb * bb, dtype=torch.uint8, device=dev)
        fill(w, nb, 3)
        y = torch.empty(rows, device=dev)
        med, mn = timer.graph(lambda i: call(w, x, y, rows, cols), min(steps, 50), warmup, replays=5)
        by = nb * bb + 4 * (rows + cols)
        out[name] = {"ms": med, "ms_min": mn, "GBs": by / med / 1e6, "frac_of_measured_hbm": by / med / 1e6 / hbm, "bytes": by}
        del w
    # the other weight types of the reference's matvec switch at the vocabulary size (random bytes with small fp16
    # block scales: the values do not matter for the timing)
    for name, bb, per, call in (("q8_0_151936x4096", 34, 32, K.cuda_matvec_q8_0), ("q5k_151936x4096", 176, 256, K.cuda_matvec_q5k),
                                ("q3k_151936x4096", 110, 256, K.cuda_matvec_q3k)):
        nb = rows * cols // per
        w = torch.randint(0, 60, (nb * bb,), dtype=torch.uint8, device=dev)
        y = torch.empty(rows, device=dev)
        med, mn = timer.graph(lambda i: call(w, x, y, rows, cols), min(steps, 50), warmup, replays=5)
        by = nb * bb + 4 * (rows + cols)
        out[name] = {"ms": med, "ms_min": mn, "GBs": by / med / 1e6, "frac_of_measured_hbm": by / med / 1e6 / hbm, "bytes": by}
        del w
    torch.cuda.empty_cache()
    return out


def measure_decode(torch, K, dev, timer, hbm, which, tokens, n_layers=None, rank=0, world=1, comm=None):
    """Whole-token decode of a model shape resident in HBM: `tokens` tokens in one CUDA graph at the last
    position of the context (KV cache pre-filled up to it), replayed 5 times."""
    from mnemocuda_b200.decode import DecodeConfig, ResidentModel
    cfg = DecodeConfig.qwen3_30b() if which == "30b" else DecodeConfig.qwen3_235b()
    if n_layers:
        cfg.n_layers = n_layers  # a slice of the model (profiling captures): same per-layer work
    t0 = time.perf_counter()
    model = ResidentModel(cfg, dev, seed=1, rank=rank, world=world, comm=comm)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    model.set_state(1, cfg.ctx_len - 1)
    g = model.capture(tokens, advance=False)
    g.replay()
    torch.cuda.synchronize()
    med, mn = timer.replays(g, tokens, replays=5)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([med, mn], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        med, mn = float(t[0].item()), float(t[1].item())
    by = cfg.algorithmic_bytes_per_token()
    res = {"config": (f"{cfg.name} decode, batch 1, context {cfg.ctx_len} (position {cfg.ctx_len - 1}), {cfg.n_layers} layers, "
                      f"{cfg.n_experts} experts top-{cfg.top_k}, Q4_K_M-style types, all experts resident"
                      + (f"; heads, output-projection / lm_head rows and experts sharded {world}-way, push all-gather / "
                         f"all-reduce over NVLink peer memory" if world > 1 else "")),
           "tok_s": 1e3 / med, "ms_per_token": med, "ms_per_token_min": mn, "bytes_per_token": by,
           "GBs": by / med / 1e6, "frac": by / med / 1e6 / (hbm * world), "frac_of": f"{world} x measured copy bandwidth",
           "resident_GB_per_rank": round(cfg.resident_bytes(cfg.n_experts // world) / 1e9, 1),
           "tokens_per_graph": tokens, "launches_per_token": _launches_per_token(cfg, world),
           "build_s": round(build_s, 1), "sampled_token": int(model.token.item())}
    del model, g
    torch.cuda.empty_cache()
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist
    from mnemocuda_b200 import kernels as K
    from mnemocuda_b200.moe import HostMoEBlock, MoEShape, ResidentMoE

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    shape = MoEShape()
    layers = args.layers
    if world > 1:
        # expert-sharded: this rank holds experts [lo, hi) of every layer; the router is replicated
        from mnemocuda_b200.sharded import ShardedMoE, expert_range
        moe = ResidentMoE(shape, layers, dev, seed=1, expert_range=expert_range(shape.NE, world, rank))
        comm = None
        if args.collective == "push":
            from mnemocuda_b200.peer import PeerComm
            comm = PeerComm(rank, world, 8192)  # pieces up to 32 KB
        smoe = ShardedMoE(moe, rank, world, comm=comm)
    else:
        moe = ResidentMoE(shape, layers, dev, seed=1)
    K.mb200_set_pdl(not args.no_pdl)
    K.mb200_set_fused(0 if args.no_fused else args.fused_mode)
    H = shape.H
    n_x = max(layers, 48)  # distinct activation vectors: a layer sees a different x (hence other experts) each pass
    xs = torch.empty(n_x, H, device=dev)
    rs = torch.empty(n_x, H, device=dev)
    outs = torch.empty(n_x, H, device=dev)
    K.mb200_fill_normal_f32(xs, n_x * H, 4242, 1.0)
    K.mb200_fill_normal_f32(rs, n_x * H, 4243, 1.0)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    timer = Timer(torch, barrier)

    # ---- device-resident: the whole block, K steps in one graph ----
    if world > 1:
        block = lambda i: smoe.forward(i % layers, xs[i % n_x], rs[i % n_x], outs[i % n_x])
    else:
        block = lambda i: moe.forward(i % layers, xs[i % n_x], rs[i % n_x], outs[i % n_x])

    timing_how = "CUDA events around a CUDA graph of the timed steps, 20 replays, median"
    with ClockSampler(local) as clk:
        try:
            ms, ms_min = timer.graph(block, args.steps, args.warmup)
        except Exception as exc:  # a collective that cannot be captured: time the eager loop instead
            if world == 1:
                raise
            torch.cuda.synchronize()
            timing_how = f"CUDA events around the eager loop (graph capture failed: {type(exc).__name__})"
            ms, ms_min = timer.eager(block, args.steps, args.warmup)
        # ---- dominant kernel alone (ids already routed by the runs above) ----
        if world == 1:
            gu_ms, _ = timer.graph(lambda i: moe.gate_up(i % layers, xs[i % layers]), args.steps, args.warmup, 5)
            dn_ms, _ = timer.graph(lambda i: moe.down(i % layers, rs[i % layers], outs[i % layers]), args.steps, args.warmup, 5)
            rt_ms, _ = timer.graph(lambda i: moe.route(i % layers, xs[i % layers]), args.steps, args.warmup, 5)
            try:
                fu_ms, _ = timer.graph(lambda i: moe.experts_fused(i % layers, xs[i % layers], rs[i % layers], outs[i % layers]),
                                       args.steps, args.warmup, 5)
            except RuntimeError:
                fu_ms = None  # shape outside the fused kernel
        else:
            gu_ms = dn_ms = rt_ms = fu_ms = None
    if world > 1:
        t = torch.tensor([ms, ms_min], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_min = float(t[0].item()), float(t[1].item())
    # N > 1 shards ONE block over the GPUs (strong scaling): the job's bytes per step stay those of one block
    value = shape.algorithmic_bytes / (ms * 1e-3) / 1e9

    # ---- end to end through host buffers ----
    host_block = HostMoEBlock(moe, smoe if world > 1 else None)
    hxr = torch.randn(n_x, 2, H).pin_memory()
    ho = torch.empty(n_x, H).pin_memory()
    # warm-up over every (layer, buffer) pair the timed steps use: the library keeps the launches of a host call as
    # an instantiated graph per argument set, built on first use
    n_warm = max(args.warmup, n_x)
    for i in range(n_warm):
        host_block(i % layers, hxr[i % n_x], ho[i % n_x])
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        j = n_warm + i
        host_block(j % layers, hxr[j % n_x], ho[j % n_x])
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = shape.algorithmic_bytes / (e2e_ms * 1e-3) / 1e9

    # ---- N > 1: the other collective variant of the block, and the row-sharded matvec + all-gather ----
    sharded_extra = None
    if world > 1:
        from mnemocuda_b200.sharded import RowShardedMatvec, row_range
        sharded_extra = {}
        other = ShardedMoE(moe, rank, world, comm=None)
        if comm is not None:  # the NCCL all-reduce baseline for the same block
            blk2 = lambda i: other.forward(i % layers, xs[i % n_x], rs[i % n_x], outs[i % n_x])
            try:
                m2, _ = timer.graph(blk2, args.steps, args.warmup, replays=5)
            except Exception:
                torch.cuda.synchronize()
                m2, _ = timer.eager(blk2, args.steps, args.warmup)
            t = torch.tensor([m2], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sharded_extra["moe_block_nccl_allreduce_ms"] = float(t.item())
        # the single Q4_K 8192 x 4096 matvec of the benchmark spec, rows split over the ranks, output all-gathered
        rows, cols, copies = 8192, 4096, 32
        rl, rh = row_range(rows, world, rank)
        rb = cols // 256 * 144
        wl = torch.empty(copies * (rh - rl) * rb, dtype=torch.uint8, device=dev)
        K.mb200_fill_q4k(wl, copies * (rh - rl) * cols // 256, 50 + rank)
        yv = torch.empty(rows, device=dev)
        for name, cm in (("push_allgather", comm), ("nccl_allgather", None)):
            if name == "push_allgather" and comm is None:
                continue
            mvs = [RowShardedMatvec(wl[i * (rh - rl) * rb:(i + 1) * (rh - rl) * rb], rows, cols, rank, world, "q4k", cm)
                   for i in range(copies)]
            f = lambda i: mvs[i % copies].forward(xs[i % n_x], yv)
            try:
                m3, _ = timer.graph(f, max(args.steps, 2 * copies), args.warmup, replays=5)
            except Exception:
                torch.cuda.synchronize()
                m3, _ = timer.eager(f, max(args.steps, 2 * copies), args.warmup)
            t = torch.tensor([m3], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            by = rows * rb + 4 * (rows + cols)
            sharded_extra["row_sharded_q4k_8192x4096_" + name] = {"ms": float(t.item()), "GBs": by / float(t.item()) / 1e6}
        del wl, mvs
        # whole-token decode with the model sharded over the ranks (needs the push collectives)
        if comm is not None and not args.no_extras:
            del moe, smoe, other
            torch.cuda.empty_cache()
            sharded_extra["decode"] = {}
            for which_model in ("30b", "235b"):
                sharded_extra["decode"][which_model] = measure_decode(torch, K, dev, timer, measured_peaks()[0], which_model,
                                                                      args.decode_tokens, rank=rank, world=world, comm=comm)
            moe = None

    err = K.mb200_device_error()
    if err != 0:
        raise RuntimeError(f"a kernel reported device error {err}")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, which = measured_peaks()
    fused = bool(fu_ms) and not args.no_fused
    one_launch = fused and args.fused_mode == 2 and world == 1
    # Dominant kernel. One-launch form: the block IS one kernel (routing + gate/up + down), so its average
    # duration is the step time of the timed graph (launch-to-launch, i.e. including the gap between two
    # launches) and its algorithmic bytes are the block's. Otherwise: the fused expert kernel, or with
    # --no-fused the routed gate/up stream kernel, timed alone.
    gu_bytes = shape.K * (shape.gate_sz + shape.up_sz) + shape.H * 4 + shape.K * shape.EFF * 4
    dn_bytes = shape.K * shape.down_sz + shape.K * shape.EFF * 4 + 2 * shape.H * 4
    if one_launch:
        dom_name = "moe_fused_kernel (routing + gate/up + SwiGLU + down + weighted sum: the whole block in one launch)"
        dom_bytes, dom_ms, dom_traffic = shape.algorithmic_bytes, ms, BLOCK_TRAFFIC_BYTES
    elif fused:
        dom_name = "moe_fused_kernel (routed gate/up + SwiGLU + down + weighted sum, 8 experts, one launch)"
        dom_bytes, dom_ms, dom_traffic = gu_bytes + dn_bytes, fu_ms, FUSED_TRAFFIC_BYTES
    else:
        dom_name = "stream_kernel<Q4,*> (routed gate/up + SwiGLU, 8 experts per launch)"
        dom_bytes, dom_ms, dom_traffic = gu_bytes, gu_ms, GATE_UP_TRAFFIC_BYTES
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9 if dom_ms else None
    per_rank_gb = (shape.NE // world) * layers * shape.stride / 1e9
    launches_per_step = ((1 if args.fused_mode == 2 else 2) if fused or (world > 1 and not args.no_fused) else 3)
    if world > 1 and args.collective == "push":
        launches_per_step += 1  # the push all-reduce kernel
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "ms_per_step_min": ms_min, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 dot (u8 x s8 dp4a), fp32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers_resident": layers, "resident_GB_per_rank": round(per_rank_gb, 2),
                   "l2": (f"inputs larger than L2: steps rotate over {layers} resident layers and {n_x} activation vectors; "
                          f"{per_rank_gb:.1f} GB of expert weights per rank, any of which a step may route to"),
                   "timing": timing_how, "pdl": not args.no_pdl,
                   "parallelism": (f"experts sharded {world}-way (router replicated), "
                                   + ("push all-reduce of the 16 KB partial hidden vector over NVLink peer memory (one kernel per rank)"
                                      if args.collective == "push" else "NCCL all-reduce of the 16 KB partial hidden vector")
                                   if world > 1 else "single GPU")},
        "clocks": clk.summary(),
        "gpu_launches": launches_per_step * args.steps,
        "kernels_ms": {"router_topk": rt_ms, "moe_experts_fused": fu_ms, "moe_gate_up": gu_ms, "moe_down": dn_ms},
    }
    if world == 1:
        line["roofline"] = {"bound": "hbm", "kernel": dom_name,
                            "achieved": achieved, "peak": peak, "peak_source": which + " copy bandwidth (MEASURED_PEAKS.json)",
                            "unit": "GB/s", "frac": achieved / peak, "frac_of_8TBs_nominal": achieved / 8000.0,
                            "algorithmic_bytes_per_launch": dom_bytes, "traffic": dom_traffic}
        if fu_ms:  # the expert phases of the same kernel, timed alone (ids already routed)
            line["roofline"]["expert_phases_alone"] = {
                "ms": fu_ms, "achieved": (gu_bytes + dn_bytes) / (fu_ms * 1e-3) / 1e9,
                "frac": (gu_bytes + dn_bytes) / (fu_ms * 1e-3) / 1e9 / peak, "algorithmic_bytes_per_launch": gu_bytes + dn_bytes}
    if sharded_extra:
        line["sharded"] = sharded_extra
    line["e2e"] = {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": host_block.h2d_bytes,
                   "d2h_bytes_per_step": host_block.d2h_bytes}
    if world == 1 and not args.no_cpu_baseline:
        from mnemocuda_b200 import synth
        experts_host = moe.experts[0].reshape(-1).cpu().numpy()
        router_host = moe.router[0].reshape(-1).cpu().numpy()
        v, cores, n, dt, first = cpu_block_baseline(shape, experts_host, router_host, seconds=args.cpu_seconds)
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"{n} MoE blocks on layer 0 in {dt:.1f} s (C oracle, OpenMP over rows)"}
        # parity, outside any timed region: the same block (layer 0, x = stream 900, residual = stream 1900) on the GPU
        want, i_ref, w_ref = first
        dx = torch.from_numpy(synth.normal_f32(900, H)).to(dev)
        dr = torch.from_numpy(synth.normal_f32(1900, H)).to(dev)
        do = torch.empty(H, device=dev)
        moe.forward(0, dx, dr, do)
        torch.cuda.synchronize()
        got = do.cpu().numpy().astype(np.float64)
        rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        ids_equal = bool(np.array_equal(moe.ids[0].cpu().numpy(), i_ref))
        line["parity"] = {"rel_l2": rel, "ids_equal": ids_equal, "tolerance": 1e-3,
                          "against": "C oracle (CPU restatement of the reference), same layer and inputs"}
        if rel > 1e-3 or not ids_equal:
            print(json.dumps(line), flush=True)
            raise RuntimeError(f"parity check failed: rel L2 {rel:.3e}, ids equal {ids_equal}")
    if world == 1 and not args.no_extras:
        del moe, host_block
        torch.cuda.empty_cache()
        with ClockSampler(local) as clk2:
            line["matvec"] = measure_matvec(torch, K, dev, timer, peak, args.steps, args.warmup)
            line["decode"] = {}
            for which_model in ("30b", "235b"):
                try:
                    line["decode"][which_model] = measure_decode(torch, K, dev, timer, peak, which_model, args.decode_tokens)
                except torch.OutOfMemoryError as exc:
                    line["decode"][which_model] = {"unavailable": f"out of device memory: {exc}"[:200]}
                    torch.cuda.empty_cache()
        line["clocks_extras"] = clk2.summary()
        err = K.mb200_device_error()
        if err != 0:
            raise RuntimeError(f"a kernel reported device error {err}")
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_secondary(args):
    """Other workloads of the same path, one JSON line each (not the headline; used for profiles)."""
    import torch
    from mnemocuda_b200 import kernels as K
    from mnemocuda_b200.moe import MoEShape, ResidentMoE
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the kernels have no CPU fallback")
    K.mb200_init()
    K.mb200_set_pdl(not args.no_pdl)
    dev = torch.device("cuda", 0)
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    tf = float(peaks.get("bf16_tflops", 1590.0))
    timer = Timer(torch)
    timed = lambda fn, steps, warmup: timer.graph(fn, steps, warmup, replays=5)[0]

    steps, warmup = args.steps, args.warmup
    with ClockSampler(0) as clk:
        if args.workload == "matvec":
            line = {"workload": "single Q4_K matvec 8192x4096 (64 weight copies, PDL chain) and 151936x4096 matvecs",
                    "results": measure_matvec(torch, K, dev, timer, hbm, steps, warmup)}
        elif args.workload in ("decode30b", "decode235b"):
            which_model = args.workload[6:]
            line = {"workload": f"whole-token decode, {which_model} shape",
                    "results": measure_decode(torch, K, dev, timer, hbm, which_model, args.decode_tokens,
                                              n_layers=args.decode_layers)}
        elif args.workload == "gemm":
            # prefill configuration, dense part: GEMM 512 tokens x (8192 x 4096), weights rotate over 8 copies
            M, N, Kd, copies = 512, 8192, 4096, 8
            out = {}
            for name, bb, fill, call in (("q4k", 144, K.mb200_fill_q4k, K.mb200_gemm_q4k_f16), ("q6k", 210, K.mb200_fill_q6k, K.mb200_gemm_q6k_f16)):
                nb = N * Kd // 256
                w = torch.empty(copies * nb * bb, dtype=torch.uint8, device=dev)
                fill(w, copies * nb, 3)
                x = torch.randn(M, Kd, device=dev).half()
                y = torch.empty(M, N, device=dev)
                ws = [w[i * nb * bb:(i + 1) * nb * bb] for i in range(copies)]
                ms = timed(lambda i: call(ws[i % copies], x, y, M, N, Kd), steps, warmup)
                fl = 2.0 * M * N * Kd
                out[name] = {"ms": ms, "TFLOPs": fl / ms / 1e9, "frac_of_measured_bf16_burst": fl / ms / 1e9 / tf}
                del w
            line = {"workload": "prefill GEMM 512 x 8192 x 4096, fp16 tcgen05 with in-kernel dequant", "results": out}
        else:
            # prefill configuration, grouped part: 512 tokens, top-8 of 128 experts
            shape = MoEShape()
            s = shape
            moe = ResidentMoE(shape, 1, dev, seed=1)
            M, k = 512, s.K
            x = torch.randn(M, s.H, device=dev).half()
            top = torch.topk(x.float() @ moe.router[0].T, k, dim=1)
            ids = top.indices.int().contiguous()
            wts = torch.softmax(top.values, dim=1).contiguous()
            cnt = torch.bincount(ids.flatten().long(), minlength=s.NE)
            cap = 64 if int(cnt.max()) <= 64 else 0
            nbytes = K.mb200_moe_prefill_workspace_bytes(M, k, s.H, s.EFF, s.NE) + 256
            ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            ws = ws[(256 - ws.data_ptr() % 256) % 256:]
            y = torch.empty(M, s.H, device=dev)
            res = torch.randn(M, s.H, device=dev)
            ms = timed(lambda i: K.mb200_moe_prefill(moe.experts[0], s.stride, s.gate_sz, s.up_sz, s.down_type, s.NE, k, s.H,
                                                     s.EFF, x, ids, wts, res, y, M, cap, ws), steps, warmup)
            fl = 2.0 * M * k * 3 * s.EFF * s.H
            wb = s.NE * s.stride
            line = {"workload": "grouped per-expert prefill MoE block, 512 tokens, top-8 of 128 experts",
                    "results": {"ms": ms, "TFLOPs": fl / ms / 1e9, "weights_GBs": wb / ms / 1e6,
                                "hbm_floor_ms": wb / hbm / 1e6, "tokens_per_expert_max": int(cnt.max()), "cap": cap}}
    err = K.mb200_device_error()
    if err != 0:
        raise RuntimeError(f"a kernel reported device error {err}")
    line.update({"secondary": True, "steps": steps, "warmup": warmup, "clocks": clk.summary(), "data": "synthetic"})
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=12, help="resident MoE layers the steps rotate over")
    ap.add_argument("--no-pdl", action="store_true", help="plain launches instead of programmatic dependent launch")
    ap.add_argument("--no-fused", action="store_true", help="routed experts as two launches (gate/up, down) instead of the fused kernel")
    ap.add_argument("--fused-mode", type=int, default=2, choices=[1, 2],
                    help="2: one launch per block (routing inside the fused kernel); 1: router kernel + fused expert kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--workload", default="moe_block",
                    choices=["moe_block", "matvec", "gemm", "prefill", "decode30b", "decode235b"],
                    help="moe_block is the headline; the others print a secondary line for the same path")
    ap.add_argument("--collective", default="push", choices=["push", "nccl"],
                    help="N > 1: how the partial hidden vectors are summed (push: this library's peer-memory kernel)")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline only: skip the matvec and whole-token decode sections of the JSON line")
    ap.add_argument("--decode-tokens", type=int, default=8, help="tokens per timed CUDA graph of the decode section")
    ap.add_argument("--decode-layers", type=int, default=0,
                    help="--workload decode30b|decode235b only: build this many layers instead of the full model")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        if args.steps > 20:
            args.steps = 20  # each step is 4 CPU blocks: keep the run within a few minutes
        run_reference(args)
    elif args.workload != "moe_block":
        run_secondary(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
