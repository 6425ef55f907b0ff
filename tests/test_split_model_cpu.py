"""Reader / writer of the reference's split-model directory (docs/model-format.md), on the host:
round trip of every tensor, the per-layer expert layouts derived as src/forward.c:865-872 does, and the
loader's refusals (the reference's own checks, src/engine.c:362-460, 524-612, 668-736)."""
import json
import os

import numpy as np
import pytest

from mnemocuda_b200 import split_model as sm
from mnemocuda_b200.decode import DecodeConfig

CFG = dict(n_layers=2, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, n_experts=4, top_k=2, moe_inter=256,
           vocab=300, ctx_len=256)


def _write(tmp_path, **kw):
    cfg = DecodeConfig(**CFG)
    types = kw.pop("types", [(12, 12, 14, 12), (13, 8, 11, 12)])
    down = kw.pop("down_types", [14, 12])
    parts = sm.synthetic_host_model(cfg, seed=3, types=types, down_types=down, embd_type=kw.pop("embd_type", 12))
    sm.write_split_dir(str(tmp_path), cfg, *parts, **kw)
    return cfg, parts


def test_round_trip(tmp_path):
    cfg, (layers, embd, lm, onorm) = _write(tmp_path)
    m = sm.read_split_dir(str(tmp_path))
    c = m.cfg
    assert (c.n_layers, c.hidden, c.n_heads, c.n_kv_heads, c.head_dim, c.n_experts, c.top_k, c.moe_inter, c.vocab) == \
        (2, 512, 4, 2, 128, 4, 2, 256, 300)
    assert c.ctx_len == 256 and c.rms_eps == pytest.approx(1e-6) and c.rope_theta == 1e6
    assert np.array_equal(m.tensor("token_embd.weight"), embd)
    assert np.array_equal(m.tensor("output.weight"), lm)
    assert np.array_equal(m.tensor("output_norm.weight"), onorm)
    for l in range(2):
        H = m.host_layer(l)
        for k in ("wq", "wk", "wv", "wo", "attn_norm", "ffn_norm", "q_norm", "k_norm", "router", "experts"):
            assert np.array_equal(np.asarray(H[k]).reshape(-1), np.asarray(layers[l][k]).reshape(-1)), (l, k)
        assert H["types"] == layers[l]["types"]
        assert H["expert_layout"] == layers[l]["expert_layout"]
    assert [e.down_type for e in m.experts] == [14, 12]
    assert all(e.offset % 32 == 0 for e in m.tensors.values())


def test_expert_layout_without_manifest_follows_the_size_rule(tmp_path):
    """No expert_manifest.json: expert size = file size / n_experts, gate = up = size / 3 -- which only matches
    the tensors when all three have the same byte count (an all-Q4_K expert)."""
    _write(tmp_path, with_expert_manifest=False, down_types=[12, 12])
    m = sm.read_split_dir(str(tmp_path))
    assert [e.down_type for e in m.experts] == [12, 12]
    assert m.experts[0].gate_size == m.experts[0].expert_size // 3


def test_mixed_down_type_needs_the_manifest(tmp_path):
    _write(tmp_path, with_expert_manifest=False, down_types=[14, 12])
    with pytest.raises(sm.SplitModelError, match="gate / up"):
        sm.read_split_dir(str(tmp_path))


def test_context_length_is_clamped_like_the_reference(tmp_path):
    _write(tmp_path)
    assert sm.read_split_dir(str(tmp_path), context_length=5).cfg.ctx_len == 128
    assert sm.read_split_dir(str(tmp_path), context_length=10 ** 7).cfg.ctx_len == 131072


def test_other_prefix_and_tied_embedding(tmp_path):
    cfg = DecodeConfig(**CFG)
    cfg.lm_head_type = 12
    layers, embd, _, onorm = sm.synthetic_host_model(cfg, seed=4)
    sm.write_split_dir(str(tmp_path), cfg, layers, embd, None, onorm, prefix="qwen2")
    m = sm.read_split_dir(str(tmp_path))
    assert m.prefix == "qwen2" and not m.has("output.weight") and m.cfg.lm_head_type == 12


def _edit_json(path, fn):
    with open(path) as f:
        d = json.load(f)
    fn(d)
    with open(path, "w") as f:
        json.dump(d, f)


def test_missing_required_key(tmp_path):
    _write(tmp_path)
    _edit_json(tmp_path / "config.json", lambda d: d.pop("qwen3moe.block_count"))
    with pytest.raises(sm.SplitModelError, match="block_count"):
        sm.read_split_dir(str(tmp_path))


def test_tensor_outside_the_weights_file(tmp_path):
    _write(tmp_path)
    def grow(d):
        d["tensors"][-1]["offset"] += 10 ** 9
    _edit_json(tmp_path / "resident_manifest.json", grow)
    with pytest.raises(sm.SplitModelError, match="outside resident_weights.bin"):
        sm.read_split_dir(str(tmp_path))


def test_tensor_size_must_match_shape_and_type(tmp_path):
    _write(tmp_path)
    def retype(d):
        for t in d["tensors"]:
            if t["name"] == "blk.0.attn_q.weight":
                t["type_id"] = 14
    _edit_json(tmp_path / "resident_manifest.json", retype)
    with pytest.raises(sm.SplitModelError, match="attn_q"):
        sm.read_split_dir(str(tmp_path))


def test_missing_tensor(tmp_path):
    _write(tmp_path)
    _edit_json(tmp_path / "resident_manifest.json",
               lambda d: d.__setitem__("tensors", [t for t in d["tensors"] if t["name"] != "blk.1.ffn_gate_inp.weight"]))
    with pytest.raises(sm.SplitModelError, match="ffn_gate_inp"):
        sm.read_split_dir(str(tmp_path))


def test_expert_file_size_must_be_a_whole_number_of_experts(tmp_path):
    _write(tmp_path)
    with open(tmp_path / "experts" / "layer_01.bin", "ab") as f:
        f.write(b"\0" * 7)
    with pytest.raises(sm.SplitModelError, match="layer 1"):
        sm.read_split_dir(str(tmp_path))


def test_missing_expert_file(tmp_path):
    _write(tmp_path)
    os.remove(tmp_path / "experts" / "layer_00.bin")
    with pytest.raises(sm.SplitModelError, match="layer 0"):
        sm.read_split_dir(str(tmp_path))


def test_hybrid_model_is_refused(tmp_path):
    _write(tmp_path)
    _edit_json(tmp_path / "config.json", lambda d: d.__setitem__("qwen3moe.full_attention_interval", 4))
    with pytest.raises(sm.SplitModelError, match="hybrid"):
        sm.read_split_dir(str(tmp_path))


def test_optional_qk_norm_may_be_absent(tmp_path):
    cfg = DecodeConfig(**CFG)
    layers, embd, lm, onorm = sm.synthetic_host_model(cfg, seed=5)
    for L in layers:
        L["q_norm"] = L["k_norm"] = None
    sm.write_split_dir(str(tmp_path), cfg, layers, embd, lm, onorm, prefix="llama")
    m = sm.read_split_dir(str(tmp_path))
    assert m.prefix == "llama"
    assert m.host_layer(0)["q_norm"] is None and m.host_layer(1)["k_norm"] is None
