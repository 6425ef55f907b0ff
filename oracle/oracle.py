"""ctypes binding of liboracle.so (the CPU restatement in mnemo_oracle.c).

TEST INFRASTRUCTURE ONLY. Imported by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark; never by the product package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def reference_dir() -> str | None:
    """Root of the reference checkout: $MNEMO_REFERENCE_DIR, else a `reference` directory beside this
    repository. None when neither exists (the GPU box: only prebuilt files travel there)."""
    for cand in (os.environ.get("MNEMO_REFERENCE_DIR"), os.path.join(_HERE, "..", "..", "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src")):
            return os.path.abspath(cand)
    return None


def build(force: bool = False) -> str:
    """Compile liboracle.so (and the reference's own kernels, if its tree is here)."""
    src = os.path.join(_HERE, "mnemo_oracle.c")
    hdr = os.path.join(_HERE, "mnemo_oracle.h")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(src),
                                                                                  os.path.getmtime(hdr)):
        subprocess.check_call(["make", "-C", _HERE, "all"], stdout=subprocess.DEVNULL)
    ref = reference_dir()
    if ref and not os.path.exists(os.path.join(_HERE, "_ref", "libmnemo_ref_kernels.so")):
        subprocess.call(["make", "-C", _HERE, "ref", "REFERENCE=" + ref], stdout=subprocess.DEVNULL,
                        stderr=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.mo_f16_to_f32.restype = C.c_float
        _lib.mo_f16_to_f32.argtypes = [C.c_uint16]
        _lib.mo_f32_to_f16.restype = C.c_uint16
        _lib.mo_f32_to_f16.argtypes = [C.c_float]
        _lib.mo_num_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint8))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def num_threads() -> int:
    return lib().mo_num_threads()


def set_num_threads(n: int) -> None:
    lib().mo_set_num_threads(C.c_int(n))


def f16_to_f32(h: int) -> float:
    return float(lib().mo_f16_to_f32(C.c_uint16(h)))


def f32_to_f16(f: float) -> int:
    return int(lib().mo_f32_to_f16(C.c_float(f)))


def get_scale_min_k4(j: int, scales12) -> tuple[int, int]:
    q = _u8(scales12)
    sc, m = C.c_uint8(), C.c_uint8()
    lib().mo_get_scale_min_k4(C.c_int(j), _p(q), C.byref(sc), C.byref(m))
    return sc.value, m.value


def unpack_q4k_block(blk):
    blk = _u8(blk)
    assert blk.size == 144
    d, dm = C.c_uint16(), C.c_uint16()
    sc, m, q = np.zeros(8, np.uint8), np.zeros(8, np.uint8), np.zeros(256, np.uint8)
    lib().mo_unpack_q4k_block(_p(blk), C.byref(d), C.byref(dm), _p(sc), _p(m), _p(q))
    return d.value, dm.value, sc, m, q


def unpack_q6k_block(blk):
    blk = _u8(blk)
    assert blk.size == 210
    d = C.c_uint16()
    sc, q = np.zeros(16, np.int8), np.zeros(256, np.int8)
    lib().mo_unpack_q6k_block(_p(blk), C.byref(d), _p(sc), _p(q))
    return d.value, sc, q


def dequant_q4k(w, n_rows: int, n_cols: int) -> np.ndarray:
    w = _u8(w)
    out = np.zeros((n_rows, n_cols), np.float32)
    lib().mo_dequant_q4k(_p(w), C.c_int(n_rows), C.c_int(n_cols), _p(out))
    return out


def dequant_q6k(w, n_rows: int, n_cols: int) -> np.ndarray:
    w = _u8(w)
    out = np.zeros((n_rows, n_cols), np.float32)
    lib().mo_dequant_q6k(_p(w), C.c_int(n_rows), C.c_int(n_cols), _p(out))
    return out


def matvec_q4k(w, x, n_rows: int, n_cols: int, full: bool = False):
    """fp32 result; with full=True also the fp64 result and sum|w*x| per row."""
    w, x = _u8(w), _f32(x)
    y = np.zeros(n_rows, np.float32)
    y64 = np.zeros(n_rows, np.float64) if full else None
    ad = np.zeros(n_rows, np.float64) if full else None
    lib().mo_matvec_q4k(_p(w), _p(x), _p(y), _p(y64), _p(ad), C.c_int(n_rows), C.c_int(n_cols))
    return (y, y64, ad) if full else y


def matvec_q4k_add(w, x, residual, n_rows: int, n_cols: int) -> np.ndarray:
    w, x, residual = _u8(w), _f32(x), _f32(residual)
    y = np.zeros(n_rows, np.float32)
    lib().mo_matvec_q4k_add(_p(w), _p(x), _p(residual), _p(y), None, C.c_int(n_rows), C.c_int(n_cols))
    return y


def matvec_q4k_qkv(wq, wk, wv, x, q_rows: int, kv_rows: int, n_cols: int):
    wq, wk, wv, x = _u8(wq), _u8(wk), _u8(wv), _f32(x)
    q, k, v = np.zeros(q_rows, np.float32), np.zeros(kv_rows, np.float32), np.zeros(kv_rows, np.float32)
    lib().mo_matvec_q4k_qkv(_p(wq), _p(wk), _p(wv), _p(x), _p(q), _p(k), _p(v),
                            C.c_int(q_rows), C.c_int(kv_rows), C.c_int(n_cols))
    return q, k, v


def matvec_q4k_dual(wa, wb, x, n_rows: int, n_cols: int):
    wa, wb, x = _u8(wa), _u8(wb), _f32(x)
    ya, yb = np.zeros(n_rows, np.float32), np.zeros(n_rows, np.float32)
    lib().mo_matvec_q4k_dual(_p(wa), _p(wb), _p(x), _p(ya), _p(yb), C.c_int(n_rows), C.c_int(n_cols))
    return ya, yb


def matvec_q4k_scaled_add(w, x, y_in, n_rows: int, n_cols: int, scale: float) -> np.ndarray:
    w, x = _u8(w), _f32(x)
    y = _f32(y_in).copy()
    lib().mo_matvec_q4k_scaled_add(_p(w), _p(x), _p(y), C.c_int(n_rows), C.c_int(n_cols), C.c_float(scale))
    return y


def matvec_q6k(w, x, n_rows: int, n_cols: int, full: bool = False):
    w, x = _u8(w), _f32(x)
    y = np.zeros(n_rows, np.float32)
    y64 = np.zeros(n_rows, np.float64) if full else None
    ad = np.zeros(n_rows, np.float64) if full else None
    lib().mo_matvec_q6k(_p(w), _p(x), _p(y), _p(y64), _p(ad), C.c_int(n_rows), C.c_int(n_cols))
    return (y, y64, ad) if full else y


def matvec_f32(w, x, n_rows: int, n_cols: int) -> np.ndarray:
    w, x = _f32(w), _f32(x)
    y = np.zeros(n_rows, np.float32)
    lib().mo_matvec_f32(_p(w), _p(x), _p(y), C.c_int(n_rows), C.c_int(n_cols))
    return y


def matvec_f32_f64(w, x, n_rows: int, n_cols: int) -> np.ndarray:
    w, x = _f32(w), _f32(x)
    y = np.zeros(n_rows, np.float64)
    lib().mo_matvec_f32_f64(_p(w), _p(x), _p(y), C.c_int(n_rows), C.c_int(n_cols))
    return y


def swiglu(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.zeros_like(gate)
    lib().mo_swiglu(_p(gate), _p(up), _p(out), C.c_int(gate.size))
    return out


def scaled_add(out_in, x, scale: float) -> np.ndarray:
    out, x = _f32(out_in).copy(), _f32(x)
    lib().mo_scaled_add(_p(out), _p(x), C.c_float(scale), C.c_int(x.size))
    return out


def topk_softmax(scores, k: int):
    scores = _f32(scores)
    idx, wts = np.zeros(k, np.int32), np.zeros(k, np.float32)
    lib().mo_topk_softmax(_p(scores), _p(idx), _p(wts), C.c_int(scores.size), C.c_int(k))
    return idx, wts


def expert_fwd(expert, gate_sz: int, up_sz: int, H: int, EFF: int, down_type: int, weight: float,
               x, moe_out_in) -> np.ndarray:
    expert, x = _u8(expert), _f32(x)
    out = _f32(moe_out_in).copy()
    lib().mo_expert_fwd(_p(expert), C.c_size_t(gate_sz), C.c_size_t(up_sz), C.c_int(H), C.c_int(EFF),
                        C.c_int(down_type), C.c_float(weight), _p(x), _p(out))
    return out


def moe_block(router_w, experts, expert_stride: int, gate_sz: int, up_sz: int, down_type: int,
              NE: int, K: int, H: int, EFF: int, x, residual):
    router_w, experts, x, residual = _f32(router_w), _u8(experts), _f32(x), _f32(residual)
    out = np.zeros(H, np.float32)
    idx, wts = np.zeros(K, np.int32), np.zeros(K, np.float32)
    lib().mo_moe_block(_p(router_w), _p(experts), C.c_size_t(expert_stride), C.c_size_t(gate_sz),
                       C.c_size_t(up_sz), C.c_int(down_type), C.c_int(NE), C.c_int(K), C.c_int(H),
                       C.c_int(EFF), _p(x), _p(residual), _p(out), _p(idx), _p(wts))
    return out, idx, wts


def gemm_q4k_f16(w, x_f16, M: int, N: int, K: int) -> np.ndarray:
    w = _u8(w)
    x = np.ascontiguousarray(np.asarray(x_f16, dtype=np.float16)).view(np.uint16)
    out = np.zeros((M, N), np.float32)
    lib().mo_gemm_q4k_f16(_p(w), _p(x), _p(out), C.c_int(M), C.c_int(N), C.c_int(K))
    return out


def gemm_q6k_f16(w, x_f16, M: int, N: int, K: int) -> np.ndarray:
    w = _u8(w)
    x = np.ascontiguousarray(np.asarray(x_f16, dtype=np.float16)).view(np.uint16)
    out = np.zeros((M, N), np.float32)
    lib().mo_gemm_q6k_f16(_p(w), _p(x), _p(out), C.c_int(M), C.c_int(N), C.c_int(K))
    return out


# ---- support operators of a decode step --------------------------------------

def rms_norm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.zeros_like(x)
    lib().mo_rms_norm(_p(x), _p(w), _p(out), C.c_int(x.size), C.c_float(eps))
    return out


def rms_norm_heads(x, w, head_dim: int, n_heads: int, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.zeros_like(x)
    lib().mo_rms_norm_heads(_p(x), _p(w), _p(out), C.c_int(head_dim), C.c_int(n_heads), C.c_float(eps))
    return out


def rope(vec, n_heads: int, head_dim: int, pos: int, theta: float) -> np.ndarray:
    out = _f32(vec).copy()
    lib().mo_rope(_p(out), C.c_int(n_heads), C.c_int(head_dim), C.c_int(pos), C.c_float(theta))
    return out


def f32_to_f16_bits(x) -> np.ndarray:
    x = _f32(x)
    out = np.zeros(x.size, np.uint16)
    lib().mo_f32_to_f16_array(_p(x), _p(out), C.c_int(x.size))
    return out


def attention_f16kv(q, kv_k_bits, kv_v_bits, n_heads_q: int, head_dim: int, n_kv_heads: int, seq_len: int,
                    gqa_ratio: int, scale: float) -> np.ndarray:
    """kv_*_bits: uint16 views of the fp16 cache, [position][kv head][head_dim]."""
    q = _f32(q)
    k = np.ascontiguousarray(np.asarray(kv_k_bits)).view(np.uint16)
    v = np.ascontiguousarray(np.asarray(kv_v_bits)).view(np.uint16)
    out = np.zeros(n_heads_q * head_dim, np.float32)
    lib().mo_attention_f16kv(_p(q), _p(k), _p(v), _p(out), C.c_int(n_heads_q), C.c_int(head_dim), C.c_int(n_kv_heads),
                             C.c_int(seq_len), C.c_int(gqa_ratio), C.c_float(scale))
    return out


def embedding_q4k(table, token: int, hidden: int) -> np.ndarray:
    table = _u8(table)
    out = np.zeros(hidden, np.float32)
    lib().mo_embedding_q4k(_p(table), C.c_int(token), C.c_int(hidden), _p(out))
    return out


def argmax(logits) -> int:
    logits = _f32(logits)
    lib().mo_argmax.restype = C.c_int
    return int(lib().mo_argmax(_p(logits), C.c_int(logits.size)))


def sample_top_p(logits, temperature: float, top_p: float, seed: int) -> int:
    logits = _f32(logits)
    lib().mo_sample_top_p.restype = C.c_int
    return int(lib().mo_sample_top_p(_p(logits), C.c_int(logits.size), C.c_float(temperature), C.c_float(top_p),
                                     C.c_ulonglong(seed)))


TYPE_BLOCK = {8: (32, 34), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210)}  # weights, bytes per block


def dequant_type(type_id: int, w, n_rows: int, n_cols: int) -> np.ndarray:
    w = _u8(w)
    out = np.zeros((n_rows, n_cols), np.float32)
    lib().mo_dequant_type.restype = C.c_int
    assert lib().mo_dequant_type(C.c_int(type_id), _p(w), C.c_int(n_rows), C.c_int(n_cols), _p(out)) == 0
    return out


def matvec_type(type_id: int, w, x, n_rows: int, n_cols: int, full: bool = False):
    w, x = _u8(w), _f32(x)
    y = np.zeros(n_rows, np.float32)
    y64 = np.zeros(n_rows, np.float64) if full else None
    ad = np.zeros(n_rows, np.float64) if full else None
    lib().mo_matvec_type.restype = C.c_int
    assert lib().mo_matvec_type(C.c_int(type_id), _p(w), _p(x), _p(y), _p(y64), _p(ad), C.c_int(n_rows), C.c_int(n_cols)) == 0
    return (y, y64, ad) if full else y


def f32_to_int8_kv(x, head_dim: int, n_kv_heads: int):
    x = _f32(x)
    out = np.zeros(n_kv_heads * head_dim, np.int8)
    scales = np.zeros(n_kv_heads, np.float32)
    lib().mo_f32_to_int8_kv(_p(x), _p(out), _p(scales), C.c_int(head_dim), C.c_int(n_kv_heads))
    return out, scales


def attention_int8kv(q, kv_k, kv_v, k_scales, v_scales, n_heads_q: int, head_dim: int, n_kv_heads: int, seq_len: int,
                     gqa_ratio: int, scale: float) -> np.ndarray:
    q = _f32(q)
    k = np.ascontiguousarray(np.asarray(kv_k, dtype=np.int8))
    v = np.ascontiguousarray(np.asarray(kv_v, dtype=np.int8))
    ks, vs = _f32(k_scales), _f32(v_scales)
    out = np.zeros(n_heads_q * head_dim, np.float32)
    lib().mo_attention_int8kv(_p(q), _p(k), _p(v), _p(ks), _p(vs), _p(out), C.c_int(n_heads_q), C.c_int(head_dim),
                              C.c_int(n_kv_heads), C.c_int(seq_len), C.c_int(gqa_ratio), C.c_float(scale))
    return out


def decode_layer(hidden, L: dict, cfg: dict, pos: int, kv_k_bits: np.ndarray, kv_v_bits: np.ndarray):
    """One transformer layer in the reference's op order (src/forward.c:670-823, 1114) on host arrays.
    L: the layer's tensors (attn_norm, wq, wk, wv, wo, q_norm, k_norm, ffn_norm, router, experts; types in
    cfg). The KV cache (uint16 fp16 bits, [ctx][n_kv][hd]) is updated in place at `pos`.
    Returns (new hidden, routed ids)."""
    H, NH, NKV, HD = cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    eps, theta = cfg["rms_eps"], cfg["rope_theta"]
    mv = {12: matvec_q4k, 14: matvec_q6k}
    for tid in (8, 11, 13):  # the other cases of the reference's matvec() switch (src/forward.c:160-173)
        mv[tid] = (lambda t: lambda w, x, r, c: matvec_type(t, w, x, r, c))(tid)
    normed = rms_norm(hidden, L["attn_norm"], eps)
    q = mv[cfg["wq_type"]](L["wq"], normed, NH * HD, H)
    k = mv[cfg["wk_type"]](L["wk"], normed, NKV * HD, H)
    v = mv[cfg["wv_type"]](L["wv"], normed, NKV * HD, H)
    if L.get("q_norm") is not None:
        q = rms_norm_heads(q, L["q_norm"], HD, NH, eps)
        k = rms_norm_heads(k, L["k_norm"], HD, NKV, eps)
    q = rope(q, NH, HD, pos, theta)
    k = rope(k, NKV, HD, pos, theta)
    kv_k_bits.reshape(-1, NKV * HD)[pos] = f32_to_f16_bits(k)
    kv_v_bits.reshape(-1, NKV * HD)[pos] = f32_to_f16_bits(v)
    attn = attention_f16kv(q, kv_k_bits, kv_v_bits, NH, HD, NKV, pos + 1, NH // NKV, 1.0 / np.sqrt(HD))
    hidden2 = mv[cfg["wo_type"]](L["wo"], attn, H, NH * HD) + _f32(hidden)
    normed2 = rms_norm(hidden2, L["ffn_norm"], eps)
    out, ids, _ = moe_block(L["router"], L["experts"], cfg["expert_stride"], cfg["gate_sz"], cfg["up_sz"],
                            cfg["down_type"], cfg["n_experts"], cfg["top_k"], H, cfg["moe_inter"], normed2, hidden2)
    return out, ids
