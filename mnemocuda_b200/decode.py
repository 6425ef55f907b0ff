"""Host side of the whole-token decode path (mb200_decode_* in include/mnemo_b200.h).

Builds a model of a given shape resident in HBM from seeded synthetic tensors (written on the
device by the library's fill kernels: no dataset, no checkpoint), hands the library a descriptor
of raw device pointers, and drives it: one call decodes one token in the reference's op order
(src/forward.c:1635-1707, 604-1117). The token id and the position live in device memory, so a
CUDA graph captured around one step decodes another token on every replay.

torch supplies device memory, streams and graph capture here, nothing else.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from . import kernels as K
from . import synth


@dataclass
class DecodeConfig:
    n_layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    n_experts: int
    top_k: int
    moe_inter: int
    vocab: int
    ctx_len: int
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    wq_type: int = 12     # GGUF type ids: 12 = Q4_K, 14 = Q6_K (Q4_K_M: V and down in Q6_K)
    wk_type: int = 12
    wv_type: int = 14
    wo_type: int = 12
    down_type: int = 14
    lm_head_type: int = 14
    name: str = "custom"

    @staticmethod
    def qwen3_30b(ctx_len: int = 4096, n_layers: int = 48) -> "DecodeConfig":
        return DecodeConfig(n_layers, 2048, 32, 4, 128, 128, 8, 768, 151936, ctx_len, name="Qwen3-30B-A3B shape")

    @staticmethod
    def qwen3_235b(ctx_len: int = 8192, n_layers: int = 94) -> "DecodeConfig":
        return DecodeConfig(n_layers, 4096, 64, 4, 128, 128, 8, 1536, 151936, ctx_len, name="Qwen3-235B-A22B shape")

    # ---- sizes ----
    @staticmethod
    def _bytes(rows: int, cols: int, type_id: int) -> int:
        per = {12: synth.Q4K_BLOCK, 14: synth.Q6K_BLOCK}[type_id]
        return rows * ((cols + 255) // 256) * per

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def expert_sizes(self):
        return synth.expert_sizes(self.hidden, self.moe_inter, self.down_type)

    @property
    def expert_stride(self) -> int:
        return sum(self.expert_sizes())

    def layer_tensor_bytes(self) -> dict:
        return {
            "wq": self._bytes(self.q_dim, self.hidden, self.wq_type),
            "wk": self._bytes(self.kv_dim, self.hidden, self.wk_type),
            "wv": self._bytes(self.kv_dim, self.hidden, self.wv_type),
            "wo": self._bytes(self.hidden, self.q_dim, self.wo_type),
            "router": self.n_experts * self.hidden * 4,
        }

    def kv_bytes_per_layer(self, seq_len: int | None = None) -> int:
        return 2 * (seq_len if seq_len is not None else self.ctx_len) * self.kv_dim * 2

    def algorithmic_bytes_per_token(self, seq_len: int | None = None) -> int:
        """Bytes one decoded token must read: per layer the four projections, the router, the top_k routed
        expert blobs and the K/V rows of the attended positions; plus the lm_head matrix."""
        t = self.layer_tensor_bytes()
        layer = sum(t.values()) + self.top_k * self.expert_stride + self.kv_bytes_per_layer(seq_len)
        return layer * self.n_layers + self._bytes(self.vocab, self.hidden, self.lm_head_type)

    def resident_bytes(self, n_local_experts: int | None = None) -> int:
        ne = self.n_experts if n_local_experts is None else n_local_experts
        t = self.layer_tensor_bytes()
        layer = sum(t.values()) + ne * self.expert_stride + self.kv_bytes_per_layer()
        return layer * self.n_layers + self._bytes(self.vocab, self.hidden, 12) + self._bytes(self.vocab, self.hidden,
                                                                                              self.lm_head_type)


class LayerWeights(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("wq", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p),
                ("wo", C.c_void_p), ("wq_type", C.c_int), ("wk_type", C.c_int), ("wv_type", C.c_int),
                ("wo_type", C.c_int), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p), ("ffn_norm", C.c_void_p),
                ("router", C.c_void_p), ("experts", C.c_void_p), ("kv_k", C.c_void_p), ("kv_v", C.c_void_p),
                ("expert_stride", C.c_size_t), ("gate_sz", C.c_size_t), ("up_sz", C.c_size_t), ("down_type", C.c_int)]


class DecodeModel(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("hidden", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("head_dim", C.c_int), ("n_experts", C.c_int), ("top_k", C.c_int), ("moe_inter", C.c_int),
                ("vocab", C.c_int), ("ctx_len", C.c_int), ("rms_eps", C.c_float), ("rope_theta", C.c_float),
                ("down_type", C.c_int), ("embd_type", C.c_int), ("lm_head_type", C.c_int),
                ("expert_stride", C.c_size_t), ("gate_sz", C.c_size_t), ("up_sz", C.c_size_t),
                ("expert_lo", C.c_int), ("expert_cnt", C.c_int), ("layers", C.POINTER(LayerWeights)),
                ("token_embd", C.c_void_p), ("output_norm", C.c_void_p), ("lm_head", C.c_void_p),
                ("n_heads_total", C.c_int), ("o_row0", C.c_int), ("o_rows", C.c_int), ("lm_row0", C.c_int),
                ("lm_rows", C.c_int)]


def _tensor_seed(seed: int, layer: int, which: int) -> int:
    return (seed * 1000 + layer) * 64 + which


def shard_plan(cfg: DecodeConfig, rank: int, world: int) -> dict:
    """Which part of the model rank `rank` of `world` holds: query heads [q0, q0 + nq), KV heads [kv0, kv0 + nkv)
    (a KV head is replicated when there are more ranks than KV heads), rows of the output projection and of the
    lm_head, experts. Everything divides evenly for the supported world sizes (1, 2, 4, 8)."""
    c = cfg
    if c.n_heads % world or c.hidden % world or c.vocab % world or c.n_experts % world:
        raise ValueError(f"the model does not split evenly over {world} ranks")
    nq = c.n_heads // world
    if world <= c.n_kv_heads:
        if c.n_kv_heads % world:
            raise ValueError("KV heads do not split evenly")
        nkv = c.n_kv_heads // world
        kv0 = rank * nkv
    else:
        if world % c.n_kv_heads:
            raise ValueError("ranks per KV head must be whole")
        nkv, kv0 = 1, rank // (world // c.n_kv_heads)
    ne = c.n_experts // world
    return dict(q0=rank * nq, nq=nq, kv0=kv0, nkv=nkv, o_row0=rank * (c.hidden // world), o_rows=c.hidden // world,
                lm_row0=rank * (c.vocab // world), lm_rows=c.vocab // world, e0=rank * ne, ne=ne)


class ResidentModel:
    """A model of shape `cfg` resident on one device, or one rank's shard of it (rank / world / comm).

    Tensor values are seeded synthetic GGUF blocks with the benchmark's distributions (see synth.py), written on
    the device; a shard gets exactly the bytes it has inside the whole tensors, so a sharded model computes the
    same network. RMSNorm weights are 1.0; the KV cache is pre-filled with N(0,1) for positions [0, kv_prefill).
    Sharding (this replaces the reference's layer-range split, src/engine.c:761-775): query / KV heads, rows of the
    output projection and of the lm_head, and experts are split over the ranks; per layer the attention outputs and
    the projected rows are all-gathered and the experts' partial sums all-reduced through `comm` (peer.PeerComm)."""

    def __init__(self, cfg: DecodeConfig, device="cuda", seed: int = 1, kv_prefill: int | None = None,
                 norm_weights: str = "ones", rank: int = 0, world: int = 1, comm=None):
        self.cfg, self.device = cfg, torch.device(device)
        self.rank, self.world, self.comm = rank, world, comm
        if world > 1 and comm is None:
            raise ValueError("a sharded model needs a PeerComm")
        K.mb200_init()
        c = cfg
        sp = self.plan = shard_plan(cfg, rank, world)
        self.expert_lo, self.n_local = sp["e0"], sp["ne"]
        g, u, d = c.expert_sizes()
        HD, QDT = c.head_dim, c.n_heads * c.head_dim
        u8 = lambda n: torch.empty(n, dtype=torch.uint8, device=self.device)
        self.layers = []
        blk = {12: synth.Q4K_BLOCK, 14: synth.Q6K_BLOCK}
        fill_at = {12: _lib.lib().mb200_fill_q4k_at, 14: _lib.lib().mb200_fill_q6k_at}
        st = lambda: torch.cuda.current_stream().cuda_stream

        def rows_of(type_id, row0, rows, cols, sd):
            """Rows [row0, row0 + rows) of a [* x cols] tensor of the stream `sd`."""
            bpr = (cols + 255) // 256
            t = u8(rows * bpr * blk[type_id])
            K._check(fill_at[type_id](t.data_ptr(), row0 * bpr, rows * bpr, sd, st()), "mb200_fill_*_at")
            return t

        def norm_vec(n, sd):
            if norm_weights == "ones":
                return torch.ones(n, dtype=torch.float32, device=self.device)
            t = torch.empty(n, dtype=torch.float32, device=self.device)  # 1 + 0.1 N(0,1): parity tests only
            K.mb200_fill_normal_f32(t, n, sd, 0.1)
            return t + 1.0

        kv_prefill = c.ctx_len - 1 if kv_prefill is None else kv_prefill
        kv_tmp = torch.zeros(c.ctx_len, c.n_kv_heads, HD, dtype=torch.float16, device=self.device) if world > 1 else None
        for l in range(c.n_layers):
            T = {}
            T["wq"] = rows_of(c.wq_type, sp["q0"] * HD, sp["nq"] * HD, c.hidden, _tensor_seed(seed, l, 0))
            T["wk"] = rows_of(c.wk_type, sp["kv0"] * HD, sp["nkv"] * HD, c.hidden, _tensor_seed(seed, l, 1))
            T["wv"] = rows_of(c.wv_type, sp["kv0"] * HD, sp["nkv"] * HD, c.hidden, _tensor_seed(seed, l, 2))
            T["wo"] = rows_of(c.wo_type, sp["o_row0"], sp["o_rows"], QDT, _tensor_seed(seed, l, 3))
            T["router"] = torch.empty(c.n_experts, c.hidden, dtype=torch.float32, device=self.device)
            K.mb200_fill_normal_f32(T["router"], c.n_experts * c.hidden, _tensor_seed(seed, l, 4), c.hidden ** -0.5)
            T["attn_norm"], T["ffn_norm"] = norm_vec(c.hidden, _tensor_seed(seed, l, 5)), norm_vec(c.hidden, _tensor_seed(seed, l, 6))
            T["q_norm"], T["k_norm"] = norm_vec(HD, _tensor_seed(seed, l, 7)), norm_vec(HD, _tensor_seed(seed, l, 8))
            T["experts"] = torch.empty(self.n_local, c.expert_stride, dtype=torch.uint8, device=self.device)
            for e in range(self.n_local):
                tid = ((seed * 1000 + l) * 1000 + self.expert_lo + e) * 2 + (1 << 40)
                blob = T["experts"][e]
                K.mb200_fill_q4k(blob, (g + u) // synth.Q4K_BLOCK, tid)
                (K.mb200_fill_q6k if c.down_type == 14 else K.mb200_fill_q4k)(blob[g + u:], d // blk[c.down_type], tid + 1)
            T["kv_k"] = torch.zeros(c.ctx_len, sp["nkv"], HD, dtype=torch.float16, device=self.device)
            T["kv_v"] = torch.zeros(c.ctx_len, sp["nkv"], HD, dtype=torch.float16, device=self.device)
            if kv_prefill > 0:
                for name, which in (("kv_k", 9), ("kv_v", 10)):
                    if world == 1:
                        K.mb200_fill_normal_f16(T[name], kv_prefill * c.n_kv_heads * HD, _tensor_seed(seed, l, which), 1.0)
                    else:  # the whole cache's stream, then this rank's heads of it
                        K.mb200_fill_normal_f16(kv_tmp, kv_prefill * c.n_kv_heads * HD, _tensor_seed(seed, l, which), 1.0)
                        T[name][:kv_prefill].copy_(kv_tmp[:kv_prefill, sp["kv0"]:sp["kv0"] + sp["nkv"]])
            self.layers.append(T)
        del kv_tmp
        self.token_embd = rows_of(12, 0, c.vocab, c.hidden, _tensor_seed(seed, 9999, 0))
        self.lm_head = rows_of(c.lm_head_type, sp["lm_row0"], sp["lm_rows"], c.hidden, _tensor_seed(seed, 9999, 1))
        self.output_norm = norm_vec(c.hidden, _tensor_seed(seed, 9999, 2))
        self._finalize()

    @classmethod
    def from_host(cls, cfg: DecodeConfig, layers: list, token_embd, lm_head, output_norm, embd_type: int = 12,
                  device="cuda", rank: int = 0, world: int = 1, comm=None) -> "ResidentModel":
        """A model from host tensors (numpy arrays or memory maps, as a loader of the reference's split-model
        directory hands them over: split_model.py). `layers[l]` maps the names of the descriptor (attn_norm, wq, wk,
        wv, wo, q_norm, k_norm, ffn_norm, router, experts) to whole tensors, plus "types" = (wq, wk, wv, wo) type ids
        and optionally "expert_layout" = (stride, gate bytes, up bytes, down type). Each rank uploads its part:
        the rows of its heads, of its slice of the output projection and of the lm_head, and its experts."""
        import numpy as np
        self = cls.__new__(cls)
        self.cfg, self.device = cfg, torch.device(device)
        self.rank, self.world, self.comm = rank, world, comm
        if world > 1 and comm is None:
            raise ValueError("a sharded model needs a PeerComm")
        K.mb200_init()
        c = cfg
        sp = self.plan = shard_plan(cfg, rank, world)
        self.expert_lo, self.n_local = sp["e0"], sp["ne"]
        HD, QDT = c.head_dim, c.n_heads * c.head_dim

        def up(a):
            return torch.from_numpy(np.ascontiguousarray(a)).to(self.device)

        def rows(a, type_id, row0, n, cols):
            per, bb = synth.TYPE_BLOCK[type_id]
            rb = (cols + per - 1) // per * bb
            flat = np.asarray(a).reshape(-1).view(np.uint8)
            return up(flat[row0 * rb:(row0 + n) * rb])

        self.layers = []
        for l, src in enumerate(layers):
            tq, tk, tv, to = src["types"]
            T = {"types": (tq, tk, tv, to)}
            T["wq"] = rows(src["wq"], tq, sp["q0"] * HD, sp["nq"] * HD, c.hidden)
            T["wk"] = rows(src["wk"], tk, sp["kv0"] * HD, sp["nkv"] * HD, c.hidden)
            T["wv"] = rows(src["wv"], tv, sp["kv0"] * HD, sp["nkv"] * HD, c.hidden)
            T["wo"] = rows(src["wo"], to, sp["o_row0"], sp["o_rows"], QDT)
            for name in ("attn_norm", "ffn_norm", "q_norm", "k_norm", "router"):
                T[name] = up(np.asarray(src[name], dtype=np.float32)) if src.get(name) is not None else None
            stride = src.get("expert_layout", (c.expert_stride,))[0]
            blob = np.asarray(src["experts"]).reshape(-1).view(np.uint8)
            T["experts"] = up(blob[self.expert_lo * stride:(self.expert_lo + self.n_local) * stride]).reshape(self.n_local, stride)
            if "expert_layout" in src:
                T["expert_layout"] = tuple(src["expert_layout"])
            T["kv_k"] = torch.zeros(c.ctx_len, sp["nkv"], HD, dtype=torch.float16, device=self.device)
            T["kv_v"] = torch.zeros(c.ctx_len, sp["nkv"], HD, dtype=torch.float16, device=self.device)
            self.layers.append(T)
        self.token_embd = rows(token_embd, embd_type, 0, c.vocab, c.hidden)
        self.lm_head = rows(lm_head, c.lm_head_type, sp["lm_row0"], sp["lm_rows"], c.hidden)
        self.output_norm = up(np.asarray(output_norm, dtype=np.float32))
        self._finalize(embd_type)
        return self

    def _finalize(self, embd_type: int = 12) -> None:
        """Descriptor of raw pointers (a rank describes its shard), workspace, token / position / logits."""
        c, sp = self.cfg, self.plan
        world = self.world
        g, u, d = c.expert_sizes()
        HD, QDT = c.head_dim, c.n_heads * c.head_dim
        self._layer_array = (LayerWeights * c.n_layers)()
        for l, T in enumerate(self.layers):
            lw = self._layer_array[l]
            for name in ("attn_norm", "wq", "wk", "wv", "wo", "q_norm", "k_norm", "ffn_norm", "router", "experts",
                         "kv_k", "kv_v"):
                setattr(lw, name, T[name].data_ptr() if T.get(name) is not None else None)
            types = T.get("types", (c.wq_type, c.wk_type, c.wv_type, c.wo_type))
            lw.wq_type, lw.wk_type, lw.wv_type, lw.wo_type = types
            if "expert_layout" in T:  # (stride, gate bytes, up bytes, down type) of this layer's blobs
                lw.expert_stride, lw.gate_sz, lw.up_sz, lw.down_type = T["expert_layout"]
        m = DecodeModel()
        (m.n_layers, m.hidden, m.n_heads, m.n_kv_heads, m.head_dim, m.n_experts, m.top_k, m.moe_inter, m.vocab,
         m.ctx_len) = (c.n_layers, c.hidden, sp["nq"], sp["nkv"], HD, c.n_experts, c.top_k, c.moe_inter, c.vocab, c.ctx_len)
        m.rms_eps, m.rope_theta = c.rms_eps, c.rope_theta
        m.down_type, m.embd_type, m.lm_head_type = c.down_type, embd_type, c.lm_head_type
        m.expert_stride, m.gate_sz, m.up_sz = c.expert_stride, g, u
        m.expert_lo, m.expert_cnt = self.expert_lo, self.n_local
        m.layers = C.cast(self._layer_array, C.POINTER(LayerWeights))
        m.token_embd, m.output_norm, m.lm_head = self.token_embd.data_ptr(), self.output_norm.data_ptr(), self.lm_head.data_ptr()
        if world > 1:
            m.n_heads_total, m.o_row0, m.o_rows, m.lm_row0, m.lm_rows = c.n_heads, sp["o_row0"], sp["o_rows"], sp["lm_row0"], sp["lm_rows"]
        self.desc = m
        lib = _lib.lib()
        n = lib.mb200_decode_workspace_bytes(C.byref(m))
        if n == 0:
            raise ValueError("the library rejects this model shape")
        self.workspace = torch.zeros(n + 256, dtype=torch.uint8, device=self.device)
        off = (-self.workspace.data_ptr()) % 256
        self.workspace = self.workspace[off:off + n]
        self.token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.pos = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.logits = torch.empty(sp["lm_rows"], dtype=torch.float32, device=self.device)  # a shard: its rows only
        hp = lib.mb200_decode_hidden(C.byref(m), self.workspace.data_ptr())
        self._hidden_off = hp - self.workspace.data_ptr()
        if world > 1:
            f32 = lambda n_: torch.zeros(n_, dtype=torch.float32, device=self.device)
            self.attn_local, self.attn_full = f32(sp["nq"] * HD), f32(QDT)
            self.hidden_rows, self.partial = f32(sp["o_rows"]), f32(c.hidden)
            self.pair, self.pairs = f32(2), f32(2 * world)
            self.fused_push = True  # the MoE block's all-reduce inside its kernel (False: block, then push all-reduce)
        torch.cuda.synchronize(self.device)

    # ---- state ----
    def set_state(self, token: int, pos: int) -> None:
        self.token.fill_(token)
        self.pos.fill_(pos)

    @property
    def hidden(self) -> torch.Tensor:
        """The hidden state inside the workspace (fp32 [hidden])."""
        return self.workspace[self._hidden_off:self._hidden_off + 4 * self.cfg.hidden].view(torch.float32)

    # ---- launches ----
    def _st(self, stream):
        return K._stream(stream)

    def begin(self, stream=None):
        K._check(_lib.lib().mb200_decode_begin(C.byref(self.desc), self.workspace.data_ptr(), self.token.data_ptr(),
                                               self.pos.data_ptr(), self._st(stream)), "mb200_decode_begin")

    def layer(self, l: int, stream=None):
        lib, d, ws, st = _lib.lib(), C.byref(self.desc), self.workspace.data_ptr(), self._st(stream)
        if self.world == 1:
            K._check(lib.mb200_decode_layer(d, l, ws, self.pos.data_ptr(), st), "mb200_decode_layer")
            return
        K._check(lib.mb200_decode_layer_attn(d, l, ws, self.pos.data_ptr(), self.attn_local.data_ptr(), st), "mb200_decode_layer_attn")
        self.comm.allgather(self.attn_local, self.attn_full, stream)
        K._check(lib.mb200_decode_layer_oproj(d, l, ws, self.attn_full.data_ptr(), self.hidden_rows.data_ptr(), st),
                 "mb200_decode_layer_oproj")
        self.comm.allgather(self.hidden_rows, self.hidden, stream)
        if self.fused_push:  # the block and its all-reduce in one launch where that form applies
            K._check(lib.mb200_decode_layer_moe_reduce(d, l, ws, 1 if self.rank == 0 else 0, self.partial.data_ptr(),
                                                       self.hidden.data_ptr(), self.comm._comm, st),
                     "mb200_decode_layer_moe_reduce")
            return
        K._check(lib.mb200_decode_layer_moe(d, l, ws, 1 if self.rank == 0 else 0, self.partial.data_ptr(), st),
                 "mb200_decode_layer_moe")
        self.comm.allreduce(self.partial, self.hidden, stream)

    def finish(self, advance: bool = True, stream=None):
        lib, d, ws, st = _lib.lib(), C.byref(self.desc), self.workspace.data_ptr(), self._st(stream)
        pos = self.pos.data_ptr() if advance else None
        if self.world == 1:
            K._check(lib.mb200_decode_finish(d, ws, self.logits.data_ptr(), self.token.data_ptr(), pos, st), "mb200_decode_finish")
            return
        K._check(lib.mb200_decode_logits_local(d, ws, self.logits.data_ptr(), self.pair.data_ptr(), st), "mb200_decode_logits_local")
        self.comm.allgather(self.pair, self.pairs, stream)
        K._check(lib.mb200_decode_pick(self.pairs.data_ptr(), self.world, self.token.data_ptr(), pos, st), "mb200_decode_pick")

    def step(self, advance: bool = True, stream=None):
        """Enqueue one token: embedding, all layers, lm_head, greedy sample. With advance=False the
        position stays (benchmarks that time the same position repeatedly)."""
        if advance and self.world == 1:
            K._check(_lib.lib().mb200_decode_step(C.byref(self.desc), self.workspace.data_ptr(), self.token.data_ptr(),
                                                  self.pos.data_ptr(), self.logits.data_ptr(), self._st(stream)),
                     "mb200_decode_step")
            return
        self.begin(stream)
        for l in range(self.cfg.n_layers):
            self.layer(l, stream)
        self.finish(advance, stream)

    def capture(self, steps: int = 1, advance: bool = True) -> torch.cuda.CUDAGraph:
        """A CUDA graph of `steps` tokens (after one eager token, so that nothing is set up during capture)."""
        tok, pos = int(self.token.item()), int(self.pos.item())
        self.step(advance)
        torch.cuda.synchronize(self.device)
        self.set_state(tok, pos)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(steps):
                self.step(advance)
        return g
