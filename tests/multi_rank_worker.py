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
    # the all-reduce inside the block's kernel (the default with a communicator) against block + push all-reduce:
    # the same bits, on every rank
    outs = []
    for fused_push, pdl in ((True, False), (False, False), (True, True)):
        K.mb200_set_pdl(pdl)
        sm = sharded.ShardedMoE(part, rank, world, comm=comm)
        sm.fused_push = fused_push
        out = torch.full((s.H,), float("nan"), device=dev)
        for _ in range(3):
            sm.forward(0, xh, rh, out)
        torch.cuda.synchronize()
        outs.append(out.clone())
    K.mb200_set_pdl(False)
    assert torch.equal(outs[0], outs[1]), (rank, float((outs[0] - outs[1]).abs().max()))
    assert torch.equal(outs[0], outs[2]), rank
    ref = outs[0].clone()
    dist.broadcast(ref, 0)
    assert torch.equal(outs[0], ref)
    # every routed expert on rank 0 (the other ranks contribute zeros from a launch that serves no slot)
    keep_f, keep_p = full.router[0].clone(), part.router[0].clone()
    n_first = sharded.expert_range(s.NE, world, 0)[1]
    if n_first >= s.K:
        for m_ in (full, part):
            m_.router[0][n_first:] = (-10.0 / float(xh.double().dot(xh.double()))) * xh
        full.forward(0, xh, rh, want)
        assert int(full.ids[0].max()) < n_first
        for fused_push in (True, False):
            sm = sharded.ShardedMoE(part, rank, world, comm=comm)
            sm.fused_push = fused_push
            out = torch.full((s.H,), float("nan"), device=dev)
            for _ in range(2):
                sm.forward(0, xh, rh, out)
            torch.cuda.synchronize()
            rel = float((out.double() - want.double()).norm() / want.double().norm())
            assert rel <= 1e-5, (rank, fused_push, rel)
        full.router[0].copy_(keep_f)
        part.router[0].copy_(keep_p)
        full.forward(0, xh, rh, want)
    assert K.mb200_device_error() == 0
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

    # ---- whole-token decode, model sharded over the ranks, against the unsharded model on every rank ----
    from mnemocuda_b200.decode import DecodeConfig, ResidentModel
    cfg = DecodeConfig(n_layers=2, hidden=1024, n_heads=8, n_kv_heads=4, head_dim=128, n_experts=16, top_k=4, moe_inter=256,
                       vocab=2048, ctx_len=64)
    pos0, tok0, n_tok = 40, 7, 5
    whole = ResidentModel(cfg, dev, seed=17, kv_prefill=pos0, norm_weights="random")
    shard = ResidentModel(cfg, dev, seed=17, kv_prefill=pos0, norm_weights="random", rank=rank, world=world, comm=comm)
    sp = shard.plan
    # the shard holds the bytes it has inside the whole tensors
    rbq = (cfg.hidden // 256) * 144
    assert torch.equal(shard.layers[0]["wq"], whole.layers[0]["wq"][sp["q0"] * 128 * rbq:(sp["q0"] + sp["nq"]) * 128 * rbq])
    assert torch.equal(shard.layers[1]["kv_k"][:pos0], whole.layers[1]["kv_k"][:pos0, sp["kv0"]:sp["kv0"] + sp["nkv"]])
    for pdl in (False, True):
        K.mb200_set_pdl(pdl)
        whole.set_state(tok0, pos0)
        shard.set_state(tok0, pos0)
        want, got = [], []
        for _ in range(n_tok):
            whole.step()
            want.append(int(whole.token.item()))
        for i in range(n_tok):
            shard.step()
            got.append(int(shard.token.item()))
            if i == 0:
                wl = whole.logits  # after n_tok steps: not comparable; only the tokens are compared beyond step 0
        assert got == want, (rank, pdl, got, want)
        assert int(shard.pos.item()) == pos0 + n_tok
    # and replayed from one CUDA graph
    shard.set_state(tok0, pos0)
    g = shard.capture(1)
    shard.set_state(tok0, pos0)
    replay = []
    for _ in range(n_tok):
        g.replay()
        replay.append(int(shard.token.item()))
    assert replay == want, (rank, replay, want)
    K.mb200_set_pdl(False)

    assert K.mb200_device_error() == 0
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    print(f"RANK {rank} OK", flush=True)


if __name__ == "__main__":
    main()
