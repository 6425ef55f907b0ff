"""Worker of tests/test_gpu_multi.py: one process per GPU (torch.distributed.run), NCCL for the baseline.

Checks, on every rank: the push all-reduce and all-gather against NCCL's results; the expert-sharded
MoE block (push and NCCL reduction) against the unsharded block on rank 0's full copy; a row-sharded
Q4_K matvec gathered by push against the unsharded matvec; replay of the sharded block from a CUDA graph.
Prints "RANK r OK" on success."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
sys.path.insert(0, ROOT)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from mnemocuda_b200 import kernels as K
    from mnemocuda_b200 import sharded, synth
    from mnemocuda_b200.moe import MoEShape, ResidentMoE
    from mnemocuda_b200.peer import PeerComm
    K.mb200_init()
    comm = PeerComm(rank, world, 8192)

    # ---- collectives against NCCL ----
    for it, n in enumerate((4096, 8192, 512, 4096, 4096)):
        x = torch.from_numpy(synth.normal_f32(100 * it + rank, n)).to(dev)
        want = x.clone()
        dist.all_reduce(want)
        got = torch.empty_like(x)
        comm.allreduce(x, got)
        torch.cuda.synchronize()
        # NCCL's summation order is its own; the push sums in rank order
        assert torch.allclose(got, want, rtol=1e-6, atol=1e-6), (rank, it, float((got - want).abs().max()))
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        out = torch.empty(world * n if world * n <= 8192 * world else 0, device=dev)
        if n * world <= 8192 * world:
            comm.allgather(x, out)
            torch.cuda.synchronize()
            assert torch.equal(out, torch.cat(parts)), (rank, it)
    # the all-reduce is bit-identical on every rank
    x = torch.from_numpy(synth.normal_f32(777 + rank, 4096)).to(dev)
    got = torch.empty_like(x)
    comm.allreduce(x, got)
    ref = got.clone()
    dist.broadcast(ref, 0)
    assert torch.equal(got, ref)

    # ---- expert-sharded MoE block ----
    shape = MoEShape(n_experts=16)
    s = shape
    full = ResidentMoE(shape, 1, dev, seed=4)            # every rank builds the same full layer ...
    lo, hi = sharded.expert_range(s.NE, world, rank)
    part = ResidentMoE(shape, 1, dev, seed=4, expert_range=(lo, hi))  # ... and its own shard of it
    assert torch.equal(part.experts[0], full.experts[0][lo:hi])
    xh = torch.from_numpy(synth.normal_f32(5, s.H)).to(dev)
    rh = torch.from_numpy(synth.normal_f32(6, s.H)).to(dev)
    want = torch.empty(s.H, device=dev)
    full.forward(0, xh, rh, want)
    for use_comm in (comm, None):
        sm = sharded.ShardedMoE(part, rank, world, comm=use_comm)
        out = torch.full((s.H,), float("nan"), device=dev)
        for _ in range(2):
            sm.forward(0, xh, rh, out)
        torch.cuda.synchronize()
        rel = float((out.double() - want.double()).norm() / want.double().norm())
        assert rel <= 1e-5, (rank, use_comm is not None, rel)
        assert torch.equal(part.ids[0], full.ids[0])
    # replay from a CUDA graph (push reduction)
    sm = sharded.ShardedMoE(part, rank, world, comm=comm)
    out = torch.empty(s.H, device=dev)
    sm.forward(0, xh, rh, out)
    torch.cuda.synchronize()
    first = out.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        sm.forward(0, xh, rh, out)
    for _ in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, first)

    # ---- row-sharded matvec + push all-gather ----
    rows, cols = 8192, 4096
    w = torch.empty(rows * (cols // 256) * 144, dtype=torch.uint8, device=dev)
    K.mb200_fill_q4k(w, rows * cols // 256, 31)
    rl, rh_ = sharded.row_range(rows, world, rank)
    rb = (cols // 256) * 144
    mv = sharded.RowShardedMatvec(w[rl * rb:rh_ * rb], rows, cols, rank, world, "q4k", comm)
    y = torch.empty(rows, device=dev)
    mv.forward(xh, y)
    y_full = torch.empty(rows, device=dev)
    K.cuda_matvec_q4k(w, xh, y_full, rows, cols)
    torch.cuda.synchronize()
    assert torch.equal(y, y_full)  # rows are computed independently: sharding does not change a bit

    assert K.mb200_device_error() == 0
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    print(f"RANK {rank} OK", flush=True)


if __name__ == "__main__":
    main()
