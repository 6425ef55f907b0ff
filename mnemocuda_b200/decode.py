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
                ("router", C.c_void_p), ("experts", C.c_void_p), ("kv_k", C.c_void_p), ("kv_v", C.c_void_p)]


class DecodeModel(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("hidden", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("head_dim", C.c_int), ("n_experts", C.c_int), ("top_k", C.c_int), ("moe_inter", C.c_int),
                ("vocab", C.c_int), ("ctx_len", C.c_int), ("rms_eps", C.c_float), ("rope_theta", C.c_float),
                ("down_type", C.c_int), ("embd_type", C.c_int), ("lm_head_type", C.c_int),
                ("expert_stride", C.c_size_t), ("gate_sz", C.c_size_t), ("up_sz", C.c_size_t),
                ("expert_lo", C.c_int), ("expert_cnt", C.c_int), ("layers", C.POINTER(LayerWeights)),
                ("token_embd", C.c_void_p), ("output_norm", C.c_void_p), ("lm_head", C.c_void_p)]


def _tensor_seed(seed: int, layer: int, which: int) -> int:
    return (seed * 1000 + layer) * 64 + which


class ResidentModel:
    """A model of shape `cfg` resident on one device. Tensor values are seeded synthetic GGUF blocks with
    the benchmark's distributions (see synth.py); RMSNorm weights are 1.0; the KV cache is pre-filled
    with N(0,1) for positions [0, kv_prefill). `expert_range` keeps only experts [lo, hi) of every layer
    (expert-sharded engines)."""

    def __init__(self, cfg: DecodeConfig, device="cuda", seed: int = 1, kv_prefill: int | None = None,
                 expert_range=None, norm_weights: str = "ones"):
        self.cfg, self.device = cfg, torch.device(device)
        K.mb200_init()
        c = cfg
        lo, hi = expert_range if expert_range is not None else (0, c.n_experts)
        self.expert_lo, self.n_local = lo, hi - lo
        g, u, d = c.expert_sizes()
        tb = c.layer_tensor_bytes()
        u8 = lambda n: torch.empty(n, dtype=torch.uint8, device=self.device)
        self.layers = []
        self._keep = []
        fills = {12: (K.mb200_fill_q4k, synth.Q4K_BLOCK), 14: (K.mb200_fill_q6k, synth.Q6K_BLOCK)}

        def fill(t, type_id, sd):
            fn, bb = fills[type_id]
            fn(t, t.numel() // bb, sd)

        def norm_vec(n, sd):
            if norm_weights == "ones":
                return torch.ones(n, dtype=torch.float32, device=self.device)
            t = torch.empty(n, dtype=torch.float32, device=self.device)  # 1 + 0.1 N(0,1): parity tests only
            K.mb200_fill_normal_f32(t, n, sd, 0.1)
            return t + 1.0

        kv_prefill = c.ctx_len - 1 if kv_prefill is None else kv_prefill
        for l in range(c.n_layers):
            T = {}
            for i, (name, ty) in enumerate((("wq", c.wq_type), ("wk", c.wk_type), ("wv", c.wv_type), ("wo", c.wo_type))):
                T[name] = u8(tb[name])
                fill(T[name], ty, _tensor_seed(seed, l, i))
            T["router"] = torch.empty(c.n_experts, c.hidden, dtype=torch.float32, device=self.device)
            K.mb200_fill_normal_f32(T["router"], c.n_experts * c.hidden, _tensor_seed(seed, l, 4), c.hidden ** -0.5)
            T["attn_norm"], T["ffn_norm"] = norm_vec(c.hidden, _tensor_seed(seed, l, 5)), norm_vec(c.hidden, _tensor_seed(seed, l, 6))
            T["q_norm"], T["k_norm"] = norm_vec(c.head_dim, _tensor_seed(seed, l, 7)), norm_vec(c.head_dim, _tensor_seed(seed, l, 8))
            T["experts"] = torch.empty(self.n_local, c.expert_stride, dtype=torch.uint8, device=self.device)
            for e in range(self.n_local):
                tid = ((seed * 1000 + l) * 1000 + lo + e) * 2 + (1 << 40)
                blob = T["experts"][e]
                K.mb200_fill_q4k(blob, (g + u) // synth.Q4K_BLOCK, tid)
                fill(blob[g + u:], c.down_type, tid + 1)
            T["kv_k"] = torch.zeros(c.ctx_len, c.n_kv_heads, c.head_dim, dtype=torch.float16, device=self.device)
            T["kv_v"] = torch.zeros(c.ctx_len, c.n_kv_heads, c.head_dim, dtype=torch.float16, device=self.device)
            if kv_prefill > 0:
                K.mb200_fill_normal_f16(T["kv_k"], kv_prefill * c.kv_dim, _tensor_seed(seed, l, 9), 1.0)
                K.mb200_fill_normal_f16(T["kv_v"], kv_prefill * c.kv_dim, _tensor_seed(seed, l, 10), 1.0)
            self.layers.append(T)
        self.token_embd = u8(c._bytes(c.vocab, c.hidden, 12))
        fill(self.token_embd, 12, _tensor_seed(seed, 9999, 0))
        self.lm_head = u8(c._bytes(c.vocab, c.hidden, c.lm_head_type))
        fill(self.lm_head, c.lm_head_type, _tensor_seed(seed, 9999, 1))
        self.output_norm = norm_vec(c.hidden, _tensor_seed(seed, 9999, 2))

        # ---- descriptor of raw pointers ----
        self._layer_array = (LayerWeights * c.n_layers)()
        for l, T in enumerate(self.layers):
            lw = self._layer_array[l]
            for name in ("attn_norm", "wq", "wk", "wv", "wo", "q_norm", "k_norm", "ffn_norm", "router", "experts",
                         "kv_k", "kv_v"):
                setattr(lw, name, T[name].data_ptr())
            lw.wq_type, lw.wk_type, lw.wv_type, lw.wo_type = c.wq_type, c.wk_type, c.wv_type, c.wo_type
        m = DecodeModel()
        (m.n_layers, m.hidden, m.n_heads, m.n_kv_heads, m.head_dim, m.n_experts, m.top_k, m.moe_inter, m.vocab,
         m.ctx_len) = (c.n_layers, c.hidden, c.n_heads, c.n_kv_heads, c.head_dim, c.n_experts, c.top_k, c.moe_inter,
                       c.vocab, c.ctx_len)
        m.rms_eps, m.rope_theta = c.rms_eps, c.rope_theta
        m.down_type, m.embd_type, m.lm_head_type = c.down_type, 12, c.lm_head_type
        m.expert_stride, m.gate_sz, m.up_sz = c.expert_stride, g, u
        m.expert_lo, m.expert_cnt = lo, self.n_local
        m.layers = C.cast(self._layer_array, C.POINTER(LayerWeights))
        m.token_embd, m.output_norm, m.lm_head = self.token_embd.data_ptr(), self.output_norm.data_ptr(), self.lm_head.data_ptr()
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
        self.logits = torch.empty(c.vocab, dtype=torch.float32, device=self.device)
        hp = lib.mb200_decode_hidden(C.byref(m), self.workspace.data_ptr())
        self._hidden_off = hp - self.workspace.data_ptr()
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
        K._check(_lib.lib().mb200_decode_layer(C.byref(self.desc), l, self.workspace.data_ptr(), self.pos.data_ptr(),
                                               self._st(stream)), "mb200_decode_layer")

    def finish(self, advance: bool = True, stream=None):
        K._check(_lib.lib().mb200_decode_finish(C.byref(self.desc), self.workspace.data_ptr(), self.logits.data_ptr(),
                                                self.token.data_ptr(), self.pos.data_ptr() if advance else None,
                                                self._st(stream)), "mb200_decode_finish")

    def step(self, advance: bool = True, stream=None):
        """Enqueue one token: embedding, all layers, lm_head, greedy sample. With advance=False the
        position stays (benchmarks that time the same position repeatedly)."""
        if advance:
            K._check(_lib.lib().mb200_decode_step(C.byref(self.desc), self.workspace.data_ptr(), self.token.data_ptr(),
                                                  self.pos.data_ptr(), self.logits.data_ptr(), self._st(stream)),
                     "mb200_decode_step")
            return
        self.begin(stream)
        for l in range(self.cfg.n_layers):
            self.layer(l, stream)
        self.finish(False, stream)

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
