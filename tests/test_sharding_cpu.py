"""Host logic of the multi-GPU partition on CPU: range arithmetic, and world-size-2 gloo runs in
which each rank computes its shard with the CPU oracle and the collectives assemble the result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mnemocuda_b200 import sharded, synth
from oracle import oracle


def test_split_range_covers_and_balances():
    for n in (0, 1, 7, 128, 151936, 4096):
        for world in (1, 2, 3, 4, 8):
            spans = [sharded.split_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharded.split_range(10, 2, 2)


def test_owner_of_expert():
    for world in (1, 2, 4, 8):
        for e in range(128):
            r = sharded.owner_of_expert(e, 128, world)
            lo, hi = sharded.expert_range(128, world, r)
            assert lo <= e < hi


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # --- expert-sharded MoE block: partial sums + all-reduce == full block ---
        NE, k, H, EFF = 8, 4, 512, 256
        g, u, d = synth.expert_sizes(H, EFF, 14)
        stride = g + u + d
        experts = np.concatenate([synth.expert_blob(40 + e, H, EFF, 14) for e in range(NE)])
        router = synth.normal_f32(1, NE * H, H ** -0.5)
        x, res = synth.normal_f32(2, H), synth.normal_f32(3, H)
        want, ids, wts = oracle.moe_block(router, experts, stride, g, u, 14, NE, k, H, EFF, x, res)
        lo, hi = sharded.expert_range(NE, world, rank)
        part = res.copy() if rank == 0 else np.zeros(H, np.float32)
        for s, e in enumerate(ids):
            if lo <= e < hi:  # the rule the *_local entry points apply on the device
                part = oracle.expert_fwd(experts[e * stride:(e + 1) * stride], g, u, H, EFF, 14, float(wts[s]), x, part)
        t = torch.from_numpy(part)
        sharded.allreduce_partial(t)
        err_moe = float(np.linalg.norm(t.numpy() - want) / np.linalg.norm(want))

        # --- row-sharded matvec: slices + all-gather == full matvec ---
        rows, cols = 301, 512  # uneven split on purpose
        w = synth.q4k_matrix(9, rows, cols)
        xv = synth.normal_f32(10, cols)
        full = oracle.matvec_q4k(w, xv, rows, cols)
        rlo, rhi = sharded.row_range(rows, world, rank)
        rb = synth.q4k_row_bytes(cols)
        mine = oracle.matvec_q4k(w[rlo * rb:rhi * rb], xv, rhi - rlo, cols)
        got = sharded.allgather_rows(torch.from_numpy(mine), rows).numpy()
        q.put((rank, err_moe, bool(np.array_equal(got, full))))
    finally:
        dist.destroy_process_group()


def test_world_size_2_gloo_shards_reassemble():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err_moe, gathered_ok in results:
        assert err_moe < 1e-5, (rank, err_moe)  # fp32 reassociation of the expert sum only
        assert gathered_ok


def _handle_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mnemocuda_b200.peer import exchange_handles
    mine = bytes([rank + 1]) * 64
    got = exchange_handles(mine)
    ok = got == [bytes([r + 1]) * 64 for r in range(world)]
    try:
        exchange_handles(b"short")
        ok = False
    except ValueError:
        pass
    q.put((rank, ok))
    dist.destroy_process_group()


def test_ipc_handle_exchange_over_gloo():
    """The 64-byte buffer handles of the push collectives travel through torch.distributed in rank order."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 2
    procs = [ctx.Process(target=_handle_worker, args=(r, world, 29611, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True), (1, True)]
