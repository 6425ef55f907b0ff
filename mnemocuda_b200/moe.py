"""Host side of the decode-time MoE block: resident expert weights + the device path
(mb200_moe_block: one launch where the fused kernel covers the shape, else router + expert kernels).

Mirrors what the reference's forward_layer does between ffn_norm and the residual add
(src/forward.c:810-823, 875, 1122-1142, 1114) with every expert resident in HBM, so there
is no cache walk and no host round trip for the routed ids.
"""
from __future__ import annotations

import torch

from . import kernels as K
from . import synth


class MoEShape:
    def __init__(self, n_experts=128, top_k=8, hidden=4096, eff=1536, down_type=14):
        self.NE, self.K, self.H, self.EFF, self.down_type = n_experts, top_k, hidden, eff, down_type
        self.gate_sz, self.up_sz, self.down_sz = synth.expert_sizes(hidden, eff, down_type)
        self.stride = self.gate_sz + self.up_sz + self.down_sz

    @property
    def router_bytes(self) -> int:
        return self.NE * self.H * 4

    @property
    def algorithmic_bytes(self) -> int:
        """Bytes one block must read: the router matrix and the K routed expert blobs."""
        return self.router_bytes + self.K * self.stride


class ResidentMoE:
    """`n_layers` MoE layers' routers and experts resident on one device, seeded synthetic values."""

    def __init__(self, shape: MoEShape, n_layers: int, device="cuda", seed: int = 1, expert_range=None):
        self.shape, self.n_layers, self.device = shape, n_layers, torch.device(device)
        s = shape
        lo, hi = expert_range if expert_range is not None else (0, s.NE)
        self.expert_lo, self.n_local = lo, hi - lo
        self.router = torch.empty(n_layers, s.NE, s.H, dtype=torch.float32, device=self.device)
        self.experts = torch.empty(n_layers, self.n_local, s.stride, dtype=torch.uint8, device=self.device)
        K.mb200_init()
        q4_blocks = (s.gate_sz + s.up_sz) // synth.Q4K_BLOCK
        for layer in range(n_layers):
            K.mb200_fill_normal_f32(self.router[layer], s.NE * s.H, seed * 100003 + layer, s.H ** -0.5)
            for e in range(self.n_local):
                tid = (seed * 1000 + layer) * 1000 + lo + e  # one seed per tensor
                blob = self.experts[layer, e]
                K.mb200_fill_q4k(blob, q4_blocks, tid * 2 + 0)
                if s.down_type == 14:
                    K.mb200_fill_q6k(blob[s.gate_sz + s.up_sz:], s.down_sz // synth.Q6K_BLOCK, tid * 2 + 1)
                else:
                    K.mb200_fill_q4k(blob[s.gate_sz + s.up_sz:], s.down_sz // synth.Q4K_BLOCK, tid * 2 + 1)
        self.ids = torch.zeros(n_layers, s.K, dtype=torch.int32, device=self.device)
        self.wts = torch.zeros(n_layers, s.K, dtype=torch.float32, device=self.device)
        self.act = torch.zeros(s.K, s.EFF, dtype=torch.float32, device=self.device)
        n = K.mb200_router_scratch_bytes(s.NE)
        self.scratch = torch.zeros((n + 15) // 16 * 16, dtype=torch.uint8, device=self.device)
        self.fused_sync = torch.zeros(4, dtype=torch.int64, device=self.device)  # barrier counters of experts_fused()
        torch.cuda.synchronize(self.device)

    def forward(self, layer: int, x: torch.Tensor, residual: torch.Tensor, out: torch.Tensor, stream=None) -> None:
        """out = residual + MoE(x) for one layer; all tensors on the device."""
        s = self.shape
        K.mb200_moe_block(self.router[layer], self.experts[layer], s.stride, s.gate_sz, s.up_sz, s.down_type,
                          s.NE, s.K, s.H, s.EFF, x, residual, out, self.ids[layer], self.wts[layer], self.act,
                          self.scratch, stream)

    def route(self, layer: int, x: torch.Tensor, stream=None) -> None:
        s = self.shape
        K.mb200_router_topk(self.router[layer], x, self.scratch, self.ids[layer], self.wts[layer], s.NE, s.H, s.K,
                            stream)

    def gate_up(self, layer: int, x: torch.Tensor, stream=None) -> None:
        s = self.shape
        K.mb200_moe_gate_up(self.experts[layer], s.stride, 0, s.gate_sz, self.ids[layer], s.K, x, self.act, s.EFF,
                            s.H, stream)

    def experts_fused(self, layer: int, x: torch.Tensor, residual, out: torch.Tensor, stream=None) -> None:
        """Routed experts of the ids route() left, in one launch (raises if the shape is outside the fused kernel)."""
        s = self.shape
        K.mb200_moe_experts_fused(self.experts[layer], s.stride, 0, s.gate_sz, s.gate_sz + s.up_sz, s.down_type,
                                  self.ids[layer], self.wts[layer], s.K, self.expert_lo, self.n_local, x, self.act,
                                  residual, out, s.H, s.EFF, self.fused_sync, stream)

    def down(self, layer: int, residual, out: torch.Tensor, stream=None) -> None:
        s = self.shape
        K.mb200_moe_down(self.experts[layer], s.stride, s.gate_sz + s.up_sz, s.down_type, self.ids[layer],
                         self.wts[layer], s.K, self.act, residual, out, s.H, s.EFF, stream)


class HostMoEBlock:
    """The call a user of host buffers makes: hidden state in, hidden state out (mb200_moe_block_host).

    [x | residual] come from pinned host memory and the result goes back to pinned host memory inside the call: the
    device reads and writes the mapped buffers itself (a staging kernel in, the block's own stores out), then the
    call waits for the stream (the reference's engine does the same per token for the logits). With experts sharded
    over several GPUs the partial results are all-reduced on the device before the copy back."""

    def __init__(self, moe: ResidentMoE, sharded=None):
        self.moe = moe
        self.sharded = sharded  # a sharded.ShardedMoE when the experts are split over several GPUs
        H = moe.shape.H
        self.io = torch.empty(3, H, dtype=torch.float32, device=moe.device)  # x, residual, result
        self.h2d_bytes = 2 * H * 4
        self.d2h_bytes = H * 4
        self._fixed = {}  # per layer: the arguments that do not change from call to call
        # a stream of its own: the library replays an instantiated graph per argument set, and the legacy default
        # stream cannot be captured (there it falls back to plain launches)
        self.stream = torch.cuda.Stream(device=moe.device)

    def __call__(self, layer: int, x_res_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """x_res_host: pinned [2][H] (x, residual); out_host: pinned [H]."""
        m, s = self.moe, self.moe.shape
        if self.sharded is not None:
            self.io[:2].copy_(x_res_host, non_blocking=True)
            self.sharded.forward(layer, self.io[0], self.io[1], self.io[2])
            out_host.copy_(self.io[2], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return
        if not (x_res_host.is_pinned() and out_host.is_pinned()):
            raise ValueError("pinned host tensors expected")
        fx = self._fixed.get(layer)
        if fx is None:
            fx = self._fixed[layer] = (
                (m.router[layer].data_ptr(), m.experts[layer].data_ptr(), s.stride, s.gate_sz, s.up_sz, s.down_type, s.NE,
                 m.expert_lo, m.n_local, s.K, s.H, s.EFF),
                (self.io.data_ptr(), m.ids[layer].data_ptr(), m.wts[layer].data_ptr(), m.act.data_ptr(), m.scratch.data_ptr()))
        K._check(K._lib.lib().mb200_moe_block_host(*fx[0], x_res_host.data_ptr(), out_host.data_ptr(), *fx[1],
                                                   self.stream.cuda_stream), "mb200_moe_block_host")
