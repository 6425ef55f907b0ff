"""Reader and writer of the reference's split-model directory, and the hand-over to the decode path.

The reference engine loads a directory of files made by its prepare step (docs/model-format.md:1-128;
loader: src/engine.c:362-460 config, :524-612 resident manifest, :668-736 expert files):

    config.json               GGUF-style metadata under an architecture prefix
    resident_manifest.json    {"tensors": [{name, offset, size, type_id, dims}, ...]}
    resident_weights.bin      the non-expert tensors at those offsets
    expert_manifest.json      optional {"<layer>": {expert_size, gate_size, up_size, down_size}}
    experts/layer_NN.bin      all experts of layer NN, [gate][up][down] each

The reference streams experts from these files into a VRAM cache at decode time. Here everything is
uploaded once (a B200 holds 180 GB; with several ranks each one uploads its experts, head rows and
lm_head rows only) and the decode path never touches the host again. This module reads the files as
memory maps, applies the checks the reference loader applies (required keys, tensor extents inside
the weights file, expert file size = n_experts x expert size) plus the ones its kernels silently rely
on (row sizes that match dims and type), derives each layer's expert blob layout as
src/forward.c:865-872 does, and builds a decode.ResidentModel. The tokenizer, the heat map and the
hybrid (SSM) layers of the format are outside the decode path and are not read.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

import numpy as np

from . import synth
from .decode import DecodeConfig

PREFIXES = ("qwen35moe", "glm4moe", "qwen3next", "llama", "qwen2", "qwen3moe")  # detection order of src/engine.c:385-391
REQUIRED = ("embedding_length", "block_count", "attention.head_count", "attention.head_count_kv")
LAYER_TENSORS = {"attn_norm": "attn_norm.weight", "wq": "attn_q.weight", "wk": "attn_k.weight", "wv": "attn_v.weight",
                 "q_norm": "attn_q_norm.weight", "k_norm": "attn_k_norm.weight", "wo": "attn_output.weight",
                 "ffn_norm": "ffn_norm.weight", "router": "ffn_gate_inp.weight"}
OPTIONAL = ("q_norm", "k_norm")


class SplitModelError(ValueError):
    """The directory does not describe a model the decode path can run."""


@dataclass
class TensorEntry:
    name: str
    offset: int
    size: int
    type_id: int
    dims: tuple


@dataclass
class ExpertLayer:
    data: np.ndarray            # uint8 memory map of experts/layer_NN.bin
    expert_size: int
    gate_size: int
    up_size: int
    down_size: int
    down_type: int


@dataclass
class SplitModel:
    """Host view of a split-model directory: shape, tensor index and memory maps. Nothing is copied."""
    path: str
    prefix: str
    cfg: DecodeConfig
    tensors: dict = field(default_factory=dict)
    resident: np.ndarray | None = None
    experts: list = field(default_factory=list)

    def entry(self, name: str) -> TensorEntry:
        if name not in self.tensors:
            raise SplitModelError(f"tensor {name} is not in resident_manifest.json")
        return self.tensors[name]

    def has(self, name: str) -> bool:
        return name in self.tensors

    def tensor(self, name: str) -> np.ndarray:
        """The tensor's bytes (uint8), or its values for an fp32 tensor."""
        e = self.entry(name)
        raw = self.resident[e.offset:e.offset + e.size]
        return raw.view(np.float32) if e.type_id == 0 else raw

    def host_layer(self, l: int) -> dict:
        """Layer l in the form decode.ResidentModel.from_host takes."""
        out = {}
        for key, suffix in LAYER_TENSORS.items():
            name = f"blk.{l}.{suffix}"
            if key in OPTIONAL and not self.has(name):
                out[key] = None
                continue
            out[key] = self.tensor(name)
        out["types"] = tuple(self.entry(f"blk.{l}.{LAYER_TENSORS[k]}").type_id for k in ("wq", "wk", "wv", "wo"))
        ex = self.experts[l]
        out["experts"] = ex.data
        out["expert_layout"] = (ex.expert_size, ex.gate_size, ex.up_size, ex.down_type)
        return out

    def to_device(self, device="cuda", rank: int = 0, world: int = 1, comm=None):
        """Upload (this rank's part of) the model and return a decode.ResidentModel."""
        from .decode import ResidentModel
        layers = [self.host_layer(l) for l in range(self.cfg.n_layers)]
        lm = "output.weight" if self.has("output.weight") else "token_embd.weight"  # tied embeddings
        return ResidentModel.from_host(self.cfg, layers, self.tensor("token_embd.weight"), self.tensor(lm),
                                       self.tensor("output_norm.weight"), self.entry("token_embd.weight").type_id, device,
                                       rank, world, comm)


def _row_bytes(type_id: int, cols: int) -> int:
    if type_id not in synth.TYPE_BLOCK:
        raise SplitModelError(f"tensor type {type_id} is not supported")
    per, bb = synth.TYPE_BLOCK[type_id]
    return (cols + per - 1) // per * bb


def _expect(e: TensorEntry, rows: int, cols: int, types) -> None:
    if e.type_id not in types:
        raise SplitModelError(f"{e.name}: type {e.type_id} not supported here (expected one of {sorted(types)})")
    want = rows * _row_bytes(e.type_id, cols)
    if e.size != want:
        raise SplitModelError(f"{e.name}: {e.size} bytes, but [{rows} x {cols}] of type {e.type_id} is {want}")
    if e.dims and tuple(e.dims) not in ((cols, rows), (cols,)) and not (rows == 1 and tuple(e.dims) == (cols,)):
        raise SplitModelError(f"{e.name}: dims {list(e.dims)} do not match [{cols}, {rows}]")


def read_config(path: str, context_length: int | None = None):
    """config.json -> (prefix, DecodeConfig without tensor types). Keys, defaults and the clamp of the
    context length follow src/engine.c:362-460 and :497-508."""
    try:
        with open(os.path.join(path, "config.json")) as f:
            meta = json.load(f)
    except (OSError, json.JSONDecodeError) as e:
        raise SplitModelError(f"cannot read config.json: {e}") from None
    prefix = "qwen3moe"
    for p in PREFIXES:
        if any(k.startswith(p + ".") for k in meta):
            prefix = p
            break
    missing = [k for k in REQUIRED if f"{prefix}.{k}" not in meta]
    if missing:
        raise SplitModelError("config.json lacks required keys: " + ", ".join(f"{prefix}.{k}" for k in missing))
    g = lambda k, d: meta.get(f"{prefix}.{k}", d)
    hidden, n_layers = int(g("embedding_length", 0)), int(g("block_count", 0))
    if not 0 < hidden <= 65536:
        raise SplitModelError(f"invalid hidden size {hidden}")
    if not 0 < n_layers <= 1024:
        raise SplitModelError(f"invalid layer count {n_layers}")
    if int(g("full_attention_interval", 0)) > 0:
        raise SplitModelError("hybrid attention / SSM models are outside the decode path")
    vocab = int(meta.get("tokenizer.ggml.tokens_count", 0)) or int(meta.get("vocab_size", 0)) or 151936
    ctx = int(context_length if context_length is not None else g("context_length", 40960))
    ctx = min(max(ctx, 128), 131072)
    cfg = DecodeConfig(n_layers, hidden, int(g("attention.head_count", 0)), int(g("attention.head_count_kv", 0)),
                       int(g("attention.key_length", 128)), int(g("expert_count", 128)), int(g("expert_used_count", 8)),
                       int(g("expert_feed_forward_length", 1536)), vocab, ctx, float(g("attention.layer_norm_rms_epsilon", 1e-6)),
                       float(g("rope.freq_base", 1e6)), name=f"{prefix} split model")
    return prefix, cfg


def read_split_dir(path: str, context_length: int | None = None) -> SplitModel:
    prefix, cfg = read_config(path, context_length)
    m = SplitModel(path, prefix, cfg)
    # ---- resident tensors ----
    try:
        with open(os.path.join(path, "resident_manifest.json")) as f:
            man = json.load(f)
        m.resident = np.memmap(os.path.join(path, "resident_weights.bin"), dtype=np.uint8, mode="r")
    except (OSError, json.JSONDecodeError, ValueError) as e:
        raise SplitModelError(f"cannot read the resident tensors: {e}") from None
    total = m.resident.size
    for t in man.get("tensors", []):
        e = TensorEntry(str(t["name"]), int(t["offset"]), int(t["size"]), int(t.get("type_id", 0)), tuple(t.get("dims", ())))
        if e.offset < 0 or e.size < 0 or e.offset + e.size > total:
            raise SplitModelError(f"{e.name}: bytes [{e.offset}, {e.offset + e.size}) lie outside resident_weights.bin ({total})")
        m.tensors[e.name] = e
    c = cfg
    quant = {8, 11, 12, 13, 14}
    _expect(m.entry("token_embd.weight"), c.vocab, c.hidden, {11, 12})
    _expect(m.entry("output_norm.weight"), 1, c.hidden, {0})
    lm = m.entry("output.weight") if m.has("output.weight") else m.entry("token_embd.weight")
    _expect(lm, c.vocab, c.hidden, quant)
    c.lm_head_type = lm.type_id
    for l in range(c.n_layers):
        ent = lambda k: m.entry(f"blk.{l}.{LAYER_TENSORS[k]}")
        _expect(ent("attn_norm"), 1, c.hidden, {0})
        _expect(ent("ffn_norm"), 1, c.hidden, {0})
        _expect(ent("wq"), c.q_dim, c.hidden, quant | {0})
        _expect(ent("wk"), c.kv_dim, c.hidden, quant | {0})
        _expect(ent("wv"), c.kv_dim, c.hidden, quant | {0})
        _expect(ent("wo"), c.hidden, c.q_dim, quant | {0})
        _expect(ent("router"), c.n_experts, c.hidden, {0})
        for k in OPTIONAL:
            if m.has(f"blk.{l}.{LAYER_TENSORS[k]}"):
                _expect(ent(k), 1, c.head_dim, {0})
    e0 = lambda k: m.entry(f"blk.0.{LAYER_TENSORS[k]}").type_id
    c.wq_type, c.wk_type, c.wv_type, c.wo_type = e0("wq"), e0("wk"), e0("wv"), e0("wo")
    # ---- expert files ----
    try:
        with open(os.path.join(path, "expert_manifest.json")) as f:
            eman = json.load(f)
    except OSError:
        eman = {}
    except json.JSONDecodeError as e:
        raise SplitModelError(f"expert_manifest.json: {e}") from None
    q4 = lambda rows, cols: rows * _row_bytes(12, cols)
    for l in range(c.n_layers):
        fn = os.path.join(path, "experts", f"layer_{l:02d}.bin")
        try:
            data = np.memmap(fn, dtype=np.uint8, mode="r")
        except (OSError, ValueError) as e:
            raise SplitModelError(f"layer {l}: cannot map {fn}: {e}") from None
        info = eman.get(str(l), {})
        size = int(info.get("expert_size", data.size // c.n_experts))
        if size * c.n_experts != data.size:
            raise SplitModelError(f"layer {l}: {data.size} bytes is not {c.n_experts} experts of {size}")
        gate = int(info.get("gate_size", 0)) or size // 3           # src/forward.c:867-869
        up = int(info.get("up_size", 0)) or size // 3
        down = int(info.get("down_size", 0)) or size - gate - up
        down_type = 14 if down > q4(c.hidden, c.moe_inter) * 1.2 else 12   # src/forward.c:870-872
        if gate != q4(c.moe_inter, c.hidden) or up != gate:
            raise SplitModelError(f"layer {l}: gate / up of {gate} / {up} bytes are not Q4_K [{c.moe_inter} x {c.hidden}]")
        if down != c.hidden * _row_bytes(down_type, c.moe_inter) or gate + up + down != size:
            raise SplitModelError(f"layer {l}: down projection of {down} bytes does not match type {down_type}")
        m.experts.append(ExpertLayer(data, size, gate, up, down, down_type))
    c.down_type = m.experts[0].down_type
    return m


def write_split_dir(path: str, cfg: DecodeConfig, layers: list, token_embd, lm_head, output_norm, embd_type: int = 12,
                    prefix: str = "qwen3moe", with_expert_manifest: bool = True) -> None:
    """Write a model in the reference's split layout (what its prepare step produces from a GGUF file;
    used here for synthetic models and round-trip tests). `layers[l]` as for ResidentModel.from_host;
    lm_head None = tied to the embedding (no output.weight entry)."""
    os.makedirs(os.path.join(path, "experts"), exist_ok=True)
    c = cfg
    meta = {"general.architecture": prefix, f"{prefix}.embedding_length": c.hidden, f"{prefix}.block_count": c.n_layers,
            f"{prefix}.attention.head_count": c.n_heads, f"{prefix}.attention.head_count_kv": c.n_kv_heads,
            f"{prefix}.attention.key_length": c.head_dim, f"{prefix}.expert_count": c.n_experts,
            f"{prefix}.expert_used_count": c.top_k, f"{prefix}.expert_feed_forward_length": c.moe_inter,
            f"{prefix}.rope.freq_base": c.rope_theta, f"{prefix}.attention.layer_norm_rms_epsilon": c.rms_eps,
            f"{prefix}.context_length": c.ctx_len, "vocab_size": c.vocab}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(meta, f, indent=1)
    entries, off = [], 0
    with open(os.path.join(path, "resident_weights.bin"), "wb") as wf:
        def put(name, arr, type_id, dims):
            nonlocal off
            raw = np.ascontiguousarray(arr).reshape(-1).view(np.uint8)
            pad = (-off) % 32  # GGUF's default tensor alignment
            wf.write(b"\0" * pad)
            off += pad
            wf.write(raw.tobytes())
            entries.append({"name": name, "offset": off, "size": int(raw.size), "type_id": type_id, "dims": list(dims)})
            off += raw.size
        put("token_embd.weight", token_embd, embd_type, (c.hidden, c.vocab))
        put("output_norm.weight", np.asarray(output_norm, np.float32), 0, (c.hidden,))
        if lm_head is not None:
            put("output.weight", lm_head, c.lm_head_type, (c.hidden, c.vocab))
        for l, L in enumerate(layers):
            tq, tk, tv, to = L["types"]
            for key, t, dims in (("wq", tq, (c.hidden, c.q_dim)), ("wk", tk, (c.hidden, c.kv_dim)),
                                 ("wv", tv, (c.hidden, c.kv_dim)), ("wo", to, (c.q_dim, c.hidden))):
                put(f"blk.{l}.{LAYER_TENSORS[key]}", L[key], t, dims)
            for key, n in (("attn_norm", c.hidden), ("ffn_norm", c.hidden), ("q_norm", c.head_dim), ("k_norm", c.head_dim)):
                if L.get(key) is not None:
                    put(f"blk.{l}.{LAYER_TENSORS[key]}", np.asarray(L[key], np.float32), 0, (n,))
            put(f"blk.{l}.{LAYER_TENSORS['router']}", np.asarray(L["router"], np.float32), 0, (c.hidden, c.n_experts))
    with open(os.path.join(path, "resident_manifest.json"), "w") as f:
        json.dump({"tensors": entries}, f, indent=1)
    eman = {}
    for l, L in enumerate(layers):
        blob = np.ascontiguousarray(L["experts"]).reshape(-1).view(np.uint8)
        with open(os.path.join(path, "experts", f"layer_{l:02d}.bin"), "wb") as f:
            f.write(blob.tobytes())
        stride, gate, up, _ = L.get("expert_layout", (c.expert_stride, *c.expert_sizes()[:2], c.down_type))
        eman[str(l)] = {"expert_size": int(stride), "gate_size": int(gate), "up_size": int(up),
                        "down_size": int(stride - gate - up)}
    if with_expert_manifest:
        with open(os.path.join(path, "expert_manifest.json"), "w") as f:
            json.dump(eman, f, indent=1)


def synthetic_host_model(cfg: DecodeConfig, seed: int = 1, types=None, down_types=None, embd_type: int = 12):
    """Seeded host tensors of shape `cfg` for write_split_dir: (layers, token_embd, lm_head, output_norm).
    types: per-layer (wq, wk, wv, wo) type ids (default: cfg's); down_types: per-layer expert down type."""
    c = cfg
    layers = []
    for l in range(c.n_layers):
        tq, tk, tv, to = types[l] if types else (c.wq_type, c.wk_type, c.wv_type, c.wo_type)
        dt = down_types[l] if down_types else c.down_type
        sd = seed * 100 + l
        g, u, d = synth.expert_sizes(c.hidden, c.moe_inter, dt)
        L = {"types": (tq, tk, tv, to),
             "wq": synth.typed_matrix(tq, sd * 16 + 0, c.q_dim, c.hidden), "wk": synth.typed_matrix(tk, sd * 16 + 1, c.kv_dim, c.hidden),
             "wv": synth.typed_matrix(tv, sd * 16 + 2, c.kv_dim, c.hidden), "wo": synth.typed_matrix(to, sd * 16 + 3, c.hidden, c.q_dim),
             "router": synth.normal_f32(sd * 16 + 4, c.n_experts * c.hidden, c.hidden ** -0.5)}
        for i, (key, n) in enumerate((("attn_norm", c.hidden), ("ffn_norm", c.hidden), ("q_norm", c.head_dim), ("k_norm", c.head_dim))):
            L[key] = (1.0 + 0.1 * synth.normal_f32(sd * 16 + 5 + i, n)).astype(np.float32)
        L["experts"] = np.concatenate([synth.expert_blob(sd * 1000 + e, c.hidden, c.moe_inter, dt) for e in range(c.n_experts)])
        L["expert_layout"] = (g + u + d, g, u, dt)
        layers.append(L)
    token_embd = synth.typed_matrix(embd_type, seed * 7 + 1, c.vocab, c.hidden)
    lm_head = synth.typed_matrix(c.lm_head_type, seed * 7 + 2, c.vocab, c.hidden)
    output_norm = (1.0 + 0.1 * synth.normal_f32(seed * 7 + 3, c.hidden)).astype(np.float32)
    return layers, token_embd, lm_head, output_norm
