"""Sharding of the hot path over the GPUs of one node (one process per GPU, torch.distributed).

This replaces the reference's only form of multi-GPU execution -- contiguous layer ranges with a
peer copy of the hidden vector at each boundary (src/engine.c:761-775, src/forward.c:1555-1581) --
by two partitions of the work itself:

* rows: every matvec is split by output rows; a rank computes rows [lo, hi) and the slices are
  all-gathered (rows of a GGUF tensor are contiguous byte ranges, so a shard is a plain slice);
* experts: a rank holds experts [lo, hi) of every MoE layer; the router is replicated so every rank
  knows the routed ids without communication; each rank adds its local experts and the partial
  hidden vectors are summed with an all-reduce.

The functions here are the host logic (ranges, collectives); the device work is the C ABI
(`mb200_moe_block_local`, `mb200_moe_gate_up_local`, `mb200_moe_down_local`, the plain matvecs on row slices).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def split_range(n: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced-to-one split of range(n): the first n % world ranks get one more."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def expert_range(n_experts: int, world: int, rank: int) -> tuple[int, int]:
    return split_range(n_experts, world, rank)


def row_range(n_rows: int, world: int, rank: int) -> tuple[int, int]:
    return split_range(n_rows, world, rank)


def owner_of_expert(expert: int, n_experts: int, world: int) -> int:
    for r in range(world):
        lo, hi = split_range(n_experts, world, r)
        if lo <= expert < hi:
            return r
    raise ValueError(expert)


def allgather_rows(local: torch.Tensor, n_rows: int, group=None) -> torch.Tensor:
    """Assemble the full output vector from each rank's row slice. Slices may differ by one row;
    all_gather wants equal sizes, so each slice is padded to the longest and trimmed afterwards."""
    world = dist.get_world_size(group)
    sizes = [split_range(n_rows, world, r) for r in range(world)]
    lo, hi = sizes[dist.get_rank(group)]
    if local.numel() != hi - lo:
        raise ValueError(f"rank holds {local.numel()} rows, expected {hi - lo}")
    longest = max(h - l for l, h in sizes)
    padded = torch.zeros(longest, dtype=local.dtype, device=local.device)
    padded[:hi - lo] = local
    parts = [torch.empty(longest, dtype=local.dtype, device=local.device) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:h - l] for p, (l, h) in zip(parts, sizes)])


def allreduce_partial(partial: torch.Tensor, group=None) -> torch.Tensor:
    """Sum the per-rank partial hidden vectors of an expert-sharded MoE block, in place."""
    dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


class ShardedMoE:
    """Expert-sharded MoE block on this rank's GPU. `moe` is a ResidentMoE built with
    expert_range=expert_range(NE, world, rank). The partial hidden vectors are summed either by the push
    all-reduce over peer memory (`comm`, a peer.PeerComm: one kernel per rank, the pieces stored straight
    into the peers' buffers) or, without one, by an NCCL all-reduce (the baseline)."""

    def __init__(self, moe, rank: int, world: int, comm=None):
        from . import kernels as K
        self.K, self.moe, self.rank, self.world, self.comm = K, moe, rank, world, comm
        self.lo, self.cnt = moe.expert_lo, moe.n_local
        self.zero = torch.zeros(moe.shape.H, dtype=torch.float32, device=moe.device)
        self.partial = torch.zeros(moe.shape.H, dtype=torch.float32, device=moe.device)
        self.fused_push = True  # False: block and push all-reduce as two launches (A/B runs, tests)

    def forward(self, layer: int, x: torch.Tensor, residual: torch.Tensor, out: torch.Tensor, reduce=True) -> None:
        """This rank's partial block (one launch where the fused kernel covers the shape), then the all-reduce."""
        s, m, K = self.moe.shape, self.moe, self.K
        push = reduce and self.world > 1 and self.comm is not None
        if push and self.fused_push:
            # the block and its all-reduce in one launch (the kernel's epilogue pushes the rows to the peers)
            if K.mb200_moe_block_push(m.router[layer], m.experts[layer], s.stride, s.gate_sz, s.up_sz, s.down_type, s.NE,
                                      self.lo, self.cnt, s.K, s.H, s.EFF, x, None, 0.0, residual if self.rank == 0 else None,
                                      out, m.ids[layer], m.wts[layer], m.act, m.scratch, self.comm._comm):
                return
        res = residual if self.rank == 0 else self.zero
        dst = self.partial if push else out
        K.mb200_moe_block_local(m.router[layer], m.experts[layer], s.stride, s.gate_sz, s.up_sz, s.down_type, s.NE,
                                self.lo, self.cnt, s.K, s.H, s.EFF, x, res, dst, m.ids[layer], m.wts[layer], m.act,
                                m.scratch)
        if push:
            self.comm.allreduce(self.partial, out)
        elif reduce and self.world > 1:
            allreduce_partial(out)


class RowShardedMatvec:
    """A Q4_K / Q6_K matvec split by output rows over the ranks: this rank holds rows [lo, hi) of the tensor
    (a contiguous byte range of the GGUF tensor) and computes that slice of y; the slices are all-gathered
    by the push collective (`comm`) or by NCCL. n_rows must divide evenly for the push path."""

    def __init__(self, weights_local: torch.Tensor, n_rows: int, n_cols: int, rank: int, world: int, kind: str = "q4k",
                 comm=None):
        from . import kernels as K
        self.K, self.w, self.n_rows, self.n_cols, self.rank, self.world, self.comm = K, weights_local, n_rows, n_cols, rank, world, comm
        self.lo, self.hi = row_range(n_rows, world, rank)
        self.call = K.cuda_matvec_q4k if kind == "q4k" else K.cuda_matvec_q6k
        self.y_local = torch.empty(self.hi - self.lo, dtype=torch.float32, device=weights_local.device)
        self.even = n_rows % world == 0

    def forward(self, x: torch.Tensor, y: torch.Tensor) -> None:
        self.call(self.w, x, self.y_local, self.hi - self.lo, self.n_cols)
        if self.world == 1:
            y.copy_(self.y_local)
        elif self.comm is not None and self.even:
            self.comm.allgather(self.y_local, y)
        else:
            y.copy_(allgather_rows(self.y_local, self.n_rows))
