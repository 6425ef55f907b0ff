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
    expert_range=expert_range(NE, world, rank)."""

    def __init__(self, moe, rank: int, world: int):
        from . import kernels as K
        self.K, self.moe, self.rank, self.world = K, moe, rank, world
        self.lo, self.cnt = moe.expert_lo, moe.n_local
        self.zero = torch.zeros(moe.shape.H, dtype=torch.float32, device=moe.device)

    def forward(self, layer: int, x: torch.Tensor, residual: torch.Tensor, out: torch.Tensor, reduce=True) -> None:
        """This rank's partial block (one launch where the fused kernel covers the shape), then the all-reduce."""
        s, m, K = self.moe.shape, self.moe, self.K
        res = residual if self.rank == 0 else self.zero
        K.mb200_moe_block_local(m.router[layer], m.experts[layer], s.stride, s.gate_sz, s.up_sz, s.down_type, s.NE,
                                self.lo, self.cnt, s.K, s.H, s.EFF, x, res, out, m.ids[layer], m.wts[layer], m.act,
                                m.scratch)
        if reduce and self.world > 1:
            allreduce_partial(out)
