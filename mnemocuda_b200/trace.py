"""In-kernel phase tracing of the streaming kernels (a developer aid; the reference's counterpart is its
MNEMO_PROFILE wall-clock phase timers, src/forward.c:798-802, 1080-1084, src/engine.c:1215).

Built with -DMB200_TRACE the kernels record %globaltimer stamps per CTA at phase boundaries
(MB200_STAMP(slot) in csrc/stream_matvec.cuh and csrc/moe_fused.cu). The product library is built
without it. This module builds the instrumented copy next to the product library and reads the stamps:

    python -m mnemocuda_b200.trace moe_block      # one-launch MoE block, 235B shape: phase timeline
    python -m mnemocuda_b200.trace moe_experts    # the fused expert kernel alone (ids given)
    python -m mnemocuda_b200.trace moe_block_after_matvec   # the block alternating with a 4096 x 8192 Q4_K matvec

Slots of the fused kernel (ns after the earliest CTA entry; median over CTAs):
  0 entry | 3 logits stored, routing barrier arrived | 1 x split done | 4 routing barrier complete |
  44-46 top-k: candidates listed / accept flags counted / accepted compacted | 6 top-k done | 47 tile list ready, first copy requested | 15 first gate/up tile landed |
  7-10 arrival at batch barrier 0-3 | 11-14 batch barrier 0-3 complete, activations being fetched |
  2 gate/up phase done (consumer warp 0) | 32,34,36,38 / 33,35,37,39 down phase needs / has batch 0-3 |
  24-31 down tile k landed | 16-23 down tile k finished by all consumers | 40-43 down tile k requested |
  5 consumer warp 0 done
"""
from __future__ import annotations

import ctypes as C
import glob
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
TRACE_LIB = os.path.join(HERE, "libmnemo_b200_trace.so")

FUSED_SLOTS = {0: "entry", 3: "logits stored + arrived", 1: "x split done", 4: "routing barrier complete",
               44: "top-k: candidates listed", 45: "top-k: accept flags counted", 46: "top-k: accepted compacted",
               6: "top-k done", 47: "first copy requested", 15: "first gate/up tile landed",
               7: "arrive batch 0", 8: "arrive batch 1", 9: "arrive batch 2", 10: "arrive batch 3",
               11: "batch 0 complete", 12: "batch 1 complete", 13: "batch 2 complete", 14: "batch 3 complete",
               2: "gate/up done", 32: "down needs batch 0", 33: "down has batch 0", 34: "down needs batch 1",
               35: "down has batch 1", 36: "down needs batch 2", 37: "down has batch 2", 38: "down needs batch 3",
               39: "down has batch 3", 5: "consumers done"}


def build(force: bool = False) -> str:
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = srcs + glob.glob(os.path.join(CSRC, "*.cuh"))
    if not force and os.path.exists(TRACE_LIB) and all(os.path.getmtime(d) <= os.path.getmtime(TRACE_LIB) for d in deps):
        return TRACE_LIB
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC",
           "-shared", "-DMB200_TRACE", "-o", TRACE_LIB, *srcs, "-lcudart"]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    subprocess.check_call(cmd, env=env)
    return TRACE_LIB


def _run(which: str) -> None:
    import torch
    lib = C.CDLL(build())
    lib.cuda_kernels_init()
    lib.mb200_router_scratch_bytes.restype = C.c_size_t
    H, EFF, K, NE = 4096, 1536, 8, 128
    g = EFF * (H // 256) * 144
    d = H * (EFF // 256) * 210
    stride = 2 * g + d
    ex = torch.randint(0, 255, (NE * stride,), dtype=torch.uint8, device="cuda")
    # plausible block headers: d / dmin small positive halves (random bytes would give NaN / Inf scales)
    router = torch.randn(NE, H, device="cuda") / 64
    # one activation vector per launch of the timed graph: every launch routes to other experts, so the weights
    # come from HBM as in a decode (with one vector the 98 MB of routed experts would stay in the 126 MB L2)
    NX = 20
    xs, res = torch.randn(NX, H, device="cuda"), torch.randn(H, device="cuda")
    x = xs[0]
    y, act = torch.empty(H, device="cuda"), torch.zeros(K, EFF, device="cuda")
    ids = torch.zeros(K, dtype=torch.int32, device="cuda")
    wts = torch.zeros(K, device="cuda")
    nsc = lib.mb200_router_scratch_bytes(C.c_int(NE))
    scratch = torch.zeros(nsc + 64, dtype=torch.uint8, device="cuda")
    sync = torch.zeros(4, dtype=torch.int64, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    sz = C.c_size_t

    wo = torch.randint(0, 255, (H * (2 * H // 256) * 144,), dtype=torch.uint8, device="cuda")  # a 4096 x 8192 Q4_K matrix
    attn = torch.randn(2 * H, device="cuda")
    hid = torch.randn(H, device="cuda")

    def call(stream, i=0):
        x = xs[i % NX]
        if which == "moe_block_after_matvec":  # the block as it runs inside a decode layer: after the O projection
            lib.cuda_matvec_q4k_add(p(wo), p(attn), p(hid), p(hid), C.c_int(H), C.c_int(2 * H), stream)
        if which in ("moe_block", "moe_block_after_matvec"):
            return lib.mb200_moe_block(p(router), p(ex), sz(stride), sz(g), sz(g), C.c_int(14), C.c_int(NE), C.c_int(K),
                                       C.c_int(H), C.c_int(EFF), p(x), p(res), p(y), p(ids), p(wts), p(act), p(scratch), stream)
        return lib.mb200_moe_experts_fused(p(ex), sz(stride), sz(0), sz(g), sz(2 * g), C.c_int(14), p(ids), p(wts), C.c_int(K),
                                           C.c_int(0), C.c_int(1 << 30), p(x), p(act), p(res), p(y), C.c_int(H), C.c_int(EFF),
                                           p(sync), stream)

    lib.mb200_set_pdl(C.c_int(1))
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if which != "moe_block":
        lib.mb200_router_topk(p(router), p(x), p(scratch), p(ids), p(wts), C.c_int(NE), C.c_int(H), C.c_int(K), st)
    for _ in range(3):
        rc = call(st)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        st2 = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        for i in range(20):
            call(st2, i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    print(f"rc {rc}; graph of 20: {e0.elapsed_time(e1) / 20 * 1e3:.2f} us per launch (instrumented build)")
    lt = torch.zeros(64 * 4, dtype=torch.int64, device="cuda")
    lib.mb200_trace_read_launches(p(lt))
    torch.cuda.synchronize()
    rows = sorted((int(r[0]), int(r[1])) for r in lt.cpu().numpy().reshape(64, 4) if r[0] > 0)
    spans = [(b - a) / 1e3 for a, b in rows]
    gaps = [(rows[i + 1][0] - rows[i][1]) / 1e3 for i in range(len(rows) - 1)]
    print(f"CTA 0 entry -> exit: median {np.median(spans):.2f} us; exit -> next entry: median {np.median(gaps):.2f} us")
    buf = torch.zeros(296 * 48, dtype=torch.int64, device="cuda")
    lib.mb200_trace_read_fused(p(buf))
    torch.cuda.synchronize()
    t = buf.cpu().numpy().reshape(296, 48)[:148]
    t0 = t[:, 0].min()
    for slot, name in FUSED_SLOTS.items():
        col = t[:, slot] - t0
        col = col[(col > -10 ** 8) & (col < 10 ** 8)]
        if col.size:
            print(f"  {name:28s} min {col.min() / 1e3:7.2f}  median {np.median(col) / 1e3:7.2f}  max {col.max() / 1e3:7.2f} us")
    for base, name in ((40, "down tile requested"), (24, "down tile landed"), (16, "down tile finished")):
        n = 4 if base == 40 else 8
        for fn, tag in ((np.min, "min"), (np.median, "median"), (np.max, "max")):
            cols = [fn(t[:, base + k] - t0) / 1e3 for k in range(n)]
            print(f"  {name:21s} {tag:6s} " + " ".join(f"{c:7.2f}" for c in cols))


if __name__ == "__main__":
    _run(sys.argv[1] if len(sys.argv) > 1 else "moe_block")
