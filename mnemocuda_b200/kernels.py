"""Host-side mirror of the reference's kernel ABI (src/forward.c:24-152) over torch tensors.

Same names, argument order and meaning as the `extern "C"` functions; tensors
stand in for the raw device pointers, and `stream` defaults to torch's current
stream. torch only supplies device memory and streams here: every function
goes straight into libmnemo_b200.so.
"""
from __future__ import annotations

import torch

from . import _lib

MB200_OK = 0
MB200_ERR_UNSUPPORTED = 4  # include/mnemo_b200.h


def _ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("device tensor expected (the kernels take device pointers)")
    if not t.is_contiguous():
        raise ValueError("contiguous tensor expected")
    return t.data_ptr()


def _f32(t: torch.Tensor) -> int:
    if t.dtype != torch.float32:
        raise TypeError(f"float32 expected, got {t.dtype}")
    return _ptr(t)


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    return int(stream)


def _check(code: int, what: str) -> None:
    if code != MB200_OK:
        where = _lib.lib().mb200_last_status_where()
        raise RuntimeError(f"{what} failed with status {code} ({where.decode() if where else ''})")


def _raise_if_failed(what: str) -> None:
    code = _lib.lib().mb200_last_status()
    if code != MB200_OK:
        where = _lib.lib().mb200_last_status_where()
        _lib.lib().mb200_clear_status()
        raise RuntimeError(f"{what} failed with status {code} ({where.decode() if where else ''})")


def cuda_kernels_init() -> None:
    _lib.lib().cuda_kernels_init()
    _raise_if_failed("cuda_kernels_init")


def cuda_matvec_q4k(weights, x, y, n_rows, n_cols, stream=None):
    _lib.lib().cuda_matvec_q4k(_ptr(weights), _f32(x), _f32(y), n_rows, n_cols, _stream(stream))
    _raise_if_failed("cuda_matvec_q4k")


def cuda_matvec_q4k_add(weights, x, residual, y, n_rows, n_cols, stream=None):
    _lib.lib().cuda_matvec_q4k_add(_ptr(weights), _f32(x), _f32(residual), _f32(y), n_rows, n_cols,
                                   _stream(stream))
    _raise_if_failed("cuda_matvec_q4k_add")


def cuda_matvec_q4k_qkv(w_q, w_k, w_v, x, out_q, out_k, out_v, q_rows, kv_rows, n_cols, stream=None):
    _lib.lib().cuda_matvec_q4k_qkv(_ptr(w_q), _ptr(w_k), _ptr(w_v), _f32(x), _f32(out_q), _f32(out_k),
                                   _f32(out_v), q_rows, kv_rows, n_cols, _stream(stream))
    _raise_if_failed("cuda_matvec_q4k_qkv")


def cuda_matvec_q4k_dual(wa, wb, x, ya, yb, n_rows, n_cols, stream=None):
    _lib.lib().cuda_matvec_q4k_dual(_ptr(wa), _ptr(wb), _f32(x), _f32(ya), _f32(yb), n_rows, n_cols,
                                    _stream(stream))
    _raise_if_failed("cuda_matvec_q4k_dual")


def cuda_matvec_q4k_scaled_add(weights, x, y, n_rows, n_cols, scale, stream=None):
    _lib.lib().cuda_matvec_q4k_scaled_add(_ptr(weights), _f32(x), _f32(y), n_rows, n_cols, float(scale),
                                          _stream(stream))
    _raise_if_failed("cuda_matvec_q4k_scaled_add")


def cuda_matvec_q6k(weights, x, y, n_rows, n_cols, stream=None):
    _lib.lib().cuda_matvec_q6k(_ptr(weights), _f32(x), _f32(y), n_rows, n_cols, _stream(stream))
    _raise_if_failed("cuda_matvec_q6k")


def cuda_matvec_f32(weights, x, y, n_rows, n_cols, stream=None):
    _lib.lib().cuda_matvec_f32(_f32(weights), _f32(x), _f32(y), n_rows, n_cols, _stream(stream))
    _raise_if_failed("cuda_matvec_f32")


def cuda_topk_softmax(scores, indices, weights, n_experts, k, stream=None):
    if indices.dtype != torch.int32:
        raise TypeError("indices must be int32")
    _lib.lib().cuda_topk_softmax(_f32(scores), _ptr(indices), _f32(weights), n_experts, k, _stream(stream))
    _raise_if_failed("cuda_topk_softmax")


def cuda_swiglu(gate, up, out, n, stream=None):
    _lib.lib().cuda_swiglu(_f32(gate), _f32(up), _f32(out), n, _stream(stream))
    _raise_if_failed("cuda_swiglu")


def cuda_scaled_add(out, x, scale, n, stream=None):
    _lib.lib().cuda_scaled_add(_f32(out), _f32(x), float(scale), n, _stream(stream))
    _raise_if_failed("cuda_scaled_add")


# ---- support operators of a decode step (reference names) -------------------

def cuda_rms_norm(x, weight, out, n, eps, stream=None):
    _lib.lib().cuda_rms_norm(_f32(x), _f32(weight), _f32(out), n, float(eps), _stream(stream))
    _raise_if_failed("cuda_rms_norm")


def cuda_rms_norm_residual(x, weight, normed, residual, n, eps, stream=None):
    _lib.lib().cuda_rms_norm_residual(_f32(x), _f32(weight), _f32(normed), _f32(residual), n, float(eps),
                                      _stream(stream))
    _raise_if_failed("cuda_rms_norm_residual")


def cuda_rms_norm_batched(x, weight, out, head_dim, n_heads, eps, stream=None):
    _lib.lib().cuda_rms_norm_batched(_f32(x), _f32(weight), _f32(out), head_dim, n_heads, float(eps), _stream(stream))
    _raise_if_failed("cuda_rms_norm_batched")


def cuda_rms_norm_qk(q, k, q_weight, k_weight, head_dim, n_q, n_k, eps, stream=None):
    _lib.lib().cuda_rms_norm_qk(_f32(q), _f32(k), _f32(q_weight), _f32(k_weight), head_dim, n_q, n_k, float(eps),
                                _stream(stream))
    _raise_if_failed("cuda_rms_norm_qk")


def cuda_rope(q, k, head_dim, pos, theta, n_heads_q, n_heads_k, stream=None):
    _lib.lib().cuda_rope(_f32(q), _f32(k), head_dim, pos, float(theta), n_heads_q, n_heads_k, _stream(stream))
    _raise_if_failed("cuda_rope")


def cuda_f32_to_f16(x, out, n, stream=None):
    _lib.lib().cuda_f32_to_f16(_f32(x), _ptr(out), n, _stream(stream))
    _raise_if_failed("cuda_f32_to_f16")


def cuda_f32_to_f16_dual(a, b, oa, ob, n, stream=None):
    _lib.lib().cuda_f32_to_f16_dual(_f32(a), _f32(b), _ptr(oa), _ptr(ob), n, _stream(stream))
    _raise_if_failed("cuda_f32_to_f16_dual")


def cuda_attention_f16kv(q, kv_k, kv_v, out, n_heads_q, head_dim, n_kv_heads, seq_len, gqa_ratio, scale, stream=None):
    if kv_k.dtype != torch.float16 or kv_v.dtype != torch.float16:
        raise TypeError("the KV cache must be float16")
    _lib.lib().cuda_attention_f16kv(_f32(q), _ptr(kv_k), _ptr(kv_v), _f32(out), n_heads_q, head_dim, n_kv_heads,
                                    seq_len, gqa_ratio, float(scale), _stream(stream))
    _raise_if_failed("cuda_attention_f16kv")


def cuda_residual_add(a, b, out, n, stream=None):
    _lib.lib().cuda_residual_add(_f32(a), _f32(b), _f32(out), n, _stream(stream))
    _raise_if_failed("cuda_residual_add")


def _typed_matvec(name):
    def call(weights, x, y, n_rows, n_cols, stream=None):
        getattr(_lib.lib(), name)(_ptr(weights), _f32(x), _f32(y), n_rows, n_cols, _stream(stream))
        _raise_if_failed(name)
    call.__name__ = name
    return call


cuda_matvec_q8_0 = _typed_matvec("cuda_matvec_q8_0")
cuda_matvec_q5k = _typed_matvec("cuda_matvec_q5k")
cuda_matvec_q3k = _typed_matvec("cuda_matvec_q3k")


def cuda_embedding_lookup_q3k(table, out, token_id, hidden, row_bytes, stream=None):
    _lib.lib().cuda_embedding_lookup_q3k(_ptr(table), _f32(out), token_id, hidden, row_bytes, _stream(stream))
    _raise_if_failed("cuda_embedding_lookup_q3k")


def cuda_f32_to_int8_kv(x, out, scales, head_dim, n_kv_heads, stream=None):
    _lib.lib().cuda_f32_to_int8_kv(_f32(x), _ptr(out), _f32(scales), head_dim, n_kv_heads, _stream(stream))
    _raise_if_failed("cuda_f32_to_int8_kv")


def cuda_f32_to_int8_kv_dual(k, v, out_k, out_v, k_scales, v_scales, head_dim, n_kv_heads, stream=None):
    _lib.lib().cuda_f32_to_int8_kv_dual(_f32(k), _f32(v), _ptr(out_k), _ptr(out_v), _f32(k_scales), _f32(v_scales),
                                        head_dim, n_kv_heads, _stream(stream))
    _raise_if_failed("cuda_f32_to_int8_kv_dual")


def cuda_attention_int8kv(q, kv_k, kv_v, k_scales, v_scales, out, n_heads_q, head_dim, n_kv_heads, seq_len, gqa_ratio,
                          scale, stream=None):
    _lib.lib().cuda_attention_int8kv(_f32(q), _ptr(kv_k), _ptr(kv_v), _f32(k_scales), _f32(v_scales), _f32(out),
                                     n_heads_q, head_dim, n_kv_heads, seq_len, gqa_ratio, float(scale), _stream(stream))
    _raise_if_failed("cuda_attention_int8kv")


def cuda_embedding_lookup_q4k(table, out, token_id, hidden, row_bytes, stream=None):
    _lib.lib().cuda_embedding_lookup_q4k(_ptr(table), _f32(out), token_id, hidden, row_bytes, _stream(stream))
    _raise_if_failed("cuda_embedding_lookup_q4k")


def cuda_sample_token(logits, vocab, temperature, top_p, rng_state, result, stream=None):
    if result.dtype != torch.int32:
        raise TypeError("result must be int32")
    _lib.lib().cuda_sample_token(_f32(logits), vocab, float(temperature), float(top_p), int(rng_state), _ptr(result),
                                 _stream(stream))
    _raise_if_failed("cuda_sample_token")


# ---- additions --------------------------------------------------------------

def mb200_init() -> None:
    _check(_lib.lib().mb200_init(), "mb200_init")


def mb200_device_error() -> int:
    return _lib.lib().mb200_device_error()


def mb200_clear_device_error(stream=None) -> None:
    _check(_lib.lib().mb200_clear_device_error(_stream(stream)), "mb200_clear_device_error")


def mb200_set_pdl(enabled: bool) -> bool:
    """Programmatic dependent launch for the streaming matvecs (see include/mnemo_b200.h)."""
    return bool(_lib.lib().mb200_set_pdl(1 if enabled else 0))


def mb200_matvec_q4k_dual_swiglu(w_gate, w_up, x, act, n_rows, n_cols, stream=None):
    _check(_lib.lib().mb200_matvec_q4k_dual_swiglu(_ptr(w_gate), _ptr(w_up), _f32(x), _f32(act), n_rows,
                                                   n_cols, _stream(stream)), "mb200_matvec_q4k_dual_swiglu")


def mb200_matvec_q6k_scaled_add(weights, x, y, n_rows, n_cols, scale, stream=None):
    _check(_lib.lib().mb200_matvec_q6k_scaled_add(_ptr(weights), _f32(x), _f32(y), n_rows, n_cols,
                                                  float(scale), _stream(stream)), "mb200_matvec_q6k_scaled_add")


def mb200_norm_matvec_q4k(weights, x, norm_w, eps, y, n_rows, n_cols, stream=None):
    """y = W RMSNorm(x), the norm folded into the matvec (include/mnemo_b200.h)."""
    _check(_lib.lib().mb200_norm_matvec_q4k(_ptr(weights), _f32(x), _f32(norm_w), float(eps), _f32(y), n_rows, n_cols,
                                            _stream(stream)), "mb200_norm_matvec_q4k")


def mb200_norm_matvec_q6k(weights, x, norm_w, eps, y, n_rows, n_cols, stream=None):
    _check(_lib.lib().mb200_norm_matvec_q6k(_ptr(weights), _f32(x), _f32(norm_w), float(eps), _f32(y), n_rows, n_cols,
                                            _stream(stream)), "mb200_norm_matvec_q6k")


def mb200_norm_matvec2_q4k(wa, ya, rows_a, wb, yb, rows_b, x, norm_w, eps, n_cols, stream=None):
    _check(_lib.lib().mb200_norm_matvec2_q4k(_ptr(wa), _f32(ya), rows_a, _ptr(wb), _f32(yb), rows_b, _f32(x), _f32(norm_w),
                                             float(eps), n_cols, _stream(stream)), "mb200_norm_matvec2_q4k")


def mb200_norm_matvec_qkv(wq, q, q_rows, wk, k, wv, v, kv_rows, x, norm_w, eps, n_cols, stream=None):
    """Q, K (Q4_K) and V (Q6_K) projections of RMSNorm(x) (norm_w None: of x) in one launch."""
    _check(_lib.lib().mb200_norm_matvec_qkv(_ptr(wq), _f32(q), q_rows, _ptr(wk), _f32(k), _ptr(wv), _f32(v), kv_rows,
                                            _f32(x), _ptr(norm_w) if norm_w is not None else None, float(eps), n_cols,
                                            _stream(stream)), "mb200_norm_matvec_qkv")


def mb200_moe_block_norm(router_w, experts, expert_stride, gate_sz, up_sz, down_type, n_experts, expert_lo, expert_cnt, k,
                         H, EFF, x, norm_w, eps, normed_scratch, residual, out, ids, wts, act, scratch, stream=None):
    """mb200_moe_block_local on RMSNorm(x), the norm folded into the one-launch form."""
    _check(_lib.lib().mb200_moe_block_norm(_f32(router_w), _ptr(experts), expert_stride, gate_sz, up_sz, down_type,
                                           n_experts, expert_lo, expert_cnt, k, H, EFF, _f32(x), _ptr(norm_w), float(eps),
                                           _ptr(normed_scratch), _ptr(residual), _f32(out), _ptr(ids), _f32(wts),
                                           _f32(act), _ptr(scratch), _stream(stream)), "mb200_moe_block_norm")


def mb200_router_scratch_bytes(n_experts: int) -> int:
    return int(_lib.lib().mb200_router_scratch_bytes(n_experts))


def mb200_router_topk(router_w, x, scratch, indices, weights, n_experts, n_cols, k, stream=None):
    _check(_lib.lib().mb200_router_topk(_f32(router_w), _f32(x), _ptr(scratch), _ptr(indices), _f32(weights),
                                        n_experts, n_cols, k, _stream(stream)), "mb200_router_topk")


def mb200_router_topk_static(router_w, x, indices, weights, n_experts, n_cols, k, stream=None):
    """Router + top-k with the library's built-in scratch (no caller scratch, nothing allocated)."""
    _check(_lib.lib().mb200_router_topk_static(_f32(router_w), _f32(x), _ptr(indices), _f32(weights), n_experts,
                                               n_cols, k, _stream(stream)), "mb200_router_topk_static")


def mb200_moe_gate_up(experts, expert_stride, gate_off, up_off, ids, n_slots, x, act, EFF, H, stream=None):
    _check(_lib.lib().mb200_moe_gate_up(_ptr(experts), expert_stride, gate_off, up_off, _ptr(ids), n_slots,
                                        _f32(x), _f32(act), EFF, H, _stream(stream)), "mb200_moe_gate_up")


def mb200_moe_down(experts, expert_stride, down_off, down_type, ids, wts, n_slots, act, residual, y, H, EFF,
                   stream=None):
    _check(_lib.lib().mb200_moe_down(_ptr(experts), expert_stride, down_off, down_type, _ptr(ids), _f32(wts),
                                     n_slots, _f32(act), _ptr(residual), _f32(y), H, EFF, _stream(stream)),
           "mb200_moe_down")


def mb200_moe_gate_up_local(experts, expert_stride, gate_off, up_off, ids, n_slots, expert_lo, expert_cnt, x, act,
                            EFF, H, stream=None):
    _check(_lib.lib().mb200_moe_gate_up_local(_ptr(experts), expert_stride, gate_off, up_off, _ptr(ids), n_slots,
                                              expert_lo, expert_cnt, _f32(x), _f32(act), EFF, H, _stream(stream)),
           "mb200_moe_gate_up_local")


def mb200_moe_down_local(experts, expert_stride, down_off, down_type, ids, wts, n_slots, expert_lo, expert_cnt, act,
                         residual, y, H, EFF, stream=None):
    _check(_lib.lib().mb200_moe_down_local(_ptr(experts), expert_stride, down_off, down_type, _ptr(ids), _f32(wts),
                                           n_slots, expert_lo, expert_cnt, _f32(act), _ptr(residual), _f32(y), H, EFF,
                                           _stream(stream)), "mb200_moe_down_local")


def mb200_moe_block(router_w, experts, expert_stride, gate_sz, up_sz, down_type, n_experts, k, H, EFF, x, residual,
                    out, ids, wts, act, scratch, stream=None):
    _check(_lib.lib().mb200_moe_block(_f32(router_w), _ptr(experts), expert_stride, gate_sz, up_sz, down_type,
                                      n_experts, k, H, EFF, _f32(x), _ptr(residual), _f32(out), _ptr(ids),
                                      _f32(wts), _f32(act), _ptr(scratch), _stream(stream)), "mb200_moe_block")


def mb200_moe_block_local(router_w, experts, expert_stride, gate_sz, up_sz, down_type, n_experts, expert_lo, expert_cnt, k,
                          H, EFF, x, residual, out, ids, wts, act, scratch, stream=None):
    """mb200_moe_block on a device that holds experts [expert_lo, expert_lo + expert_cnt) only."""
    _check(_lib.lib().mb200_moe_block_local(_f32(router_w), _ptr(experts), expert_stride, gate_sz, up_sz, down_type,
                                            n_experts, expert_lo, expert_cnt, k, H, EFF, _f32(x), _ptr(residual),
                                            _f32(out), _ptr(ids), _f32(wts), _f32(act), _ptr(scratch), _stream(stream)),
           "mb200_moe_block_local")


def mb200_moe_block_push(router_w, experts, expert_stride, gate_sz, up_sz, down_type, n_experts, expert_lo, expert_cnt, k,
                         H, EFF, x, norm_w, norm_eps, residual, out, ids, wts, act, scratch, comm, stream=None) -> bool:
    """The expert-sharded block with its all-reduce over `comm` (a communicator handle) in the same launch.
    Returns False, with nothing launched, where the one-launch form does not apply (the caller then uses
    mb200_moe_block_local + a push all-reduce)."""
    rc = _lib.lib().mb200_moe_block_push(_f32(router_w), _ptr(experts), expert_stride, gate_sz, up_sz, down_type,
                                         n_experts, expert_lo, expert_cnt, k, H, EFF, _f32(x), _ptr(norm_w),
                                         float(norm_eps), _ptr(residual), _f32(out), _ptr(ids), _f32(wts), _f32(act),
                                         _ptr(scratch), comm, _stream(stream))
    if rc == MB200_ERR_UNSUPPORTED:
        return False
    _check(rc, "mb200_moe_block_push")
    return True


def mb200_moe_experts_fused(experts, expert_stride, gate_off, up_off, down_off, down_type, ids, wts, n_slots, expert_lo,
                            expert_cnt, x, act, residual, y, H, EFF, sync, stream=None):
    """Gate/up + SwiGLU + down + weighted sum + residual in one cooperative launch (include/mnemo_b200.h)."""
    _check(_lib.lib().mb200_moe_experts_fused(_ptr(experts), expert_stride, gate_off, up_off, down_off, down_type,
                                              _ptr(ids), _f32(wts), n_slots, expert_lo, expert_cnt, _f32(x), _f32(act),
                                              _ptr(residual), _f32(y), H, EFF, _ptr(sync), _stream(stream)),
           "mb200_moe_experts_fused")


def mb200_set_fused(mode) -> None:
    """0 / False: separate expert kernels; 1 / True: router kernel + fused expert kernel; 2: one launch per block."""
    _lib.lib().mb200_set_fused(int(mode))


def mb200_gemm_q4k_f16(w, x_f16, out, M, N, K_, stream=None):
    if x_f16.dtype != torch.float16:
        raise TypeError("x must be float16")
    _check(_lib.lib().mb200_gemm_q4k_f16(_ptr(w), _ptr(x_f16), _f32(out), M, N, K_, _stream(stream)),
           "mb200_gemm_q4k_f16")


def mb200_gemm_q6k_f16(w, x_f16, out, M, N, K_, stream=None):
    if x_f16.dtype != torch.float16:
        raise TypeError("x must be float16")
    _check(_lib.lib().mb200_gemm_q6k_f16(_ptr(w), _ptr(x_f16), _f32(out), M, N, K_, _stream(stream)),
           "mb200_gemm_q6k_f16")


def mb200_moe_prefill_workspace_bytes(M, k, H, EFF, n_experts) -> int:
    return int(_lib.lib().mb200_moe_prefill_workspace_bytes(M, k, H, EFF, n_experts))


def mb200_moe_prefill(experts, expert_stride, gate_sz, up_sz, down_type, n_experts, k, H, EFF, x_f16, ids, wts,
                      residual, y, M, max_tokens_per_expert, workspace, stream=None):
    if x_f16.dtype != torch.float16:
        raise TypeError("x must be float16")
    _check(_lib.lib().mb200_moe_prefill(_ptr(experts), expert_stride, gate_sz, up_sz, down_type, n_experts, k, H, EFF,
                                        _ptr(x_f16), _ptr(ids), _f32(wts), _ptr(residual), _f32(y), M,
                                        max_tokens_per_expert, _ptr(workspace), _stream(stream)), "mb200_moe_prefill")


def mb200_fill_q4k(dst, n_blocks, seed, stream=None):
    _check(_lib.lib().mb200_fill_q4k(_ptr(dst), n_blocks, seed, _stream(stream)), "mb200_fill_q4k")


def mb200_fill_q6k(dst, n_blocks, seed, stream=None):
    _check(_lib.lib().mb200_fill_q6k(_ptr(dst), n_blocks, seed, _stream(stream)), "mb200_fill_q6k")


def mb200_fill_normal_f32(dst, n, seed, scale=1.0, stream=None):
    _check(_lib.lib().mb200_fill_normal_f32(_f32(dst), n, seed, float(scale), _stream(stream)),
           "mb200_fill_normal_f32")


def mb200_fill_normal_f16(dst, n, seed, scale=1.0, stream=None):
    _check(_lib.lib().mb200_fill_normal_f16(_ptr(dst), n, seed, float(scale), _stream(stream)),
           "mb200_fill_normal_f16")
