"""Loader of libmnemo_b200.so (the C ABI declared in include/mnemo_b200.h).

There is no fallback: if the shared library is missing or a symbol is absent,
import fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmnemo_b200.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "mnemo_b200.h")

_vp, _i, _f, _sz, _u64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_uint64

# name -> (restype, argtypes); must list every function the header declares
SIGNATURES = {
    "cuda_kernels_init": (None, []),
    "cuda_matvec_q4k": (None, [_vp, _vp, _vp, _i, _i, _vp]),
    "cuda_matvec_q4k_add": (None, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "cuda_matvec_q4k_qkv": (None, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "cuda_matvec_q4k_dual": (None, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "cuda_matvec_q4k_scaled_add": (None, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "cuda_matvec_q6k": (None, [_vp, _vp, _vp, _i, _i, _vp]),
    "cuda_matvec_f32": (None, [_vp, _vp, _vp, _i, _i, _vp]),
    "cuda_topk_softmax": (None, [_vp, _vp, _vp, _i, _i, _vp]),
    "cuda_swiglu": (None, [_vp, _vp, _vp, _i, _vp]),
    "cuda_scaled_add": (None, [_vp, _vp, _f, _i, _vp]),
    "cuda_rms_norm": (None, [_vp, _vp, _vp, _i, _f, _vp]),
    "cuda_rms_norm_residual": (None, [_vp, _vp, _vp, _vp, _i, _f, _vp]),
    "cuda_rms_norm_batched": (None, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "cuda_rms_norm_qk": (None, [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp]),
    "cuda_rope": (None, [_vp, _vp, _i, _i, _f, _i, _i, _vp]),
    "cuda_f32_to_f16": (None, [_vp, _vp, _i, _vp]),
    "cuda_f32_to_f16_dual": (None, [_vp, _vp, _vp, _vp, _i, _vp]),
    "cuda_attention_f16kv": (None, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp]),
    "cuda_residual_add": (None, [_vp, _vp, _vp, _i, _vp]),
    "cuda_embedding_lookup_q4k": (None, [_vp, _vp, _i, _i, _i, _vp]),
    "cuda_matvec_q8_0": (None, [_vp, _vp, _vp, _i, _i, _vp]),
    "cuda_matvec_q5k": (None, [_vp, _vp, _vp, _i, _i, _vp]),
    "cuda_matvec_q3k": (None, [_vp, _vp, _vp, _i, _i, _vp]),
    "cuda_embedding_lookup_q3k": (None, [_vp, _vp, _i, _i, _i, _vp]),
    "cuda_f32_to_int8_kv": (None, [_vp, _vp, _vp, _i, _i, _vp]),
    "cuda_f32_to_int8_kv_dual": (None, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "cuda_attention_int8kv": (None, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp]),
    "cuda_sample_token": (None, [_vp, _i, _f, _f, C.c_ulonglong, _vp, _vp]),
    "cuda_get_rope_kernel_ptr": (_vp, []),
    "cuda_get_f16dual_kernel_ptr": (_vp, []),
    "cuda_get_attn_f16kv_kernel_ptr": (_vp, []),
    "mb200_init": (_i, []),
    "mb200_last_status": (_i, []),
    "mb200_last_status_where": (C.c_char_p, []),
    "mb200_clear_status": (None, []),
    "mb200_device_error": (_i, []),
    "mb200_clear_device_error": (_i, [_vp]),
    "mb200_set_pdl": (_i, [_i]),
    "mb200_matvec_q4k_dual_swiglu": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "mb200_matvec_q6k_scaled_add": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "mb200_norm_matvec_q4k": (_i, [_vp, _vp, _vp, _f, _vp, _i, _i, _vp]),
    "mb200_norm_matvec_q6k": (_i, [_vp, _vp, _vp, _f, _vp, _i, _i, _vp]),
    "mb200_norm_matvec2_q4k": (_i, [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _f, _i, _vp]),
    "mb200_norm_matvec_qkv": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _f, _i, _vp]),
    "mb200_moe_block_norm": (_i, [_vp, _vp, _sz, _sz, _sz, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mb200_router_scratch_bytes": (_sz, [_i]),
    "mb200_router_topk": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "mb200_router_topk_static": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "mb200_moe_gate_up": (_i, [_vp, _sz, _sz, _sz, _vp, _i, _vp, _vp, _i, _i, _vp]),
    "mb200_moe_down": (_i, [_vp, _sz, _sz, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "mb200_moe_gate_up_local": (_i, [_vp, _sz, _sz, _sz, _vp, _i, _i, _i, _vp, _vp, _i, _i, _vp]),
    "mb200_moe_down_local": (_i, [_vp, _sz, _sz, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "mb200_moe_block": (_i, [_vp, _vp, _sz, _sz, _sz, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mb200_moe_experts_fused": (_i, [_vp, _sz, _sz, _sz, _sz, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "mb200_set_fused": (None, [_i]),
    "mb200_moe_block_local": (_i, [_vp, _vp, _sz, _sz, _sz, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mb200_moe_block_host": (_i, [_vp, _vp, _sz, _sz, _sz, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mb200_gemm_q4k_f16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "mb200_gemm_q6k_f16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "mb200_moe_prefill_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "mb200_moe_prefill": (_i, [_vp, _sz, _sz, _sz, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "mb200_decode_workspace_bytes": (_sz, [_vp]),
    "mb200_decode_hidden": (_vp, [_vp, _vp]),
    "mb200_decode_step": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "mb200_decode_begin": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "mb200_decode_layer": (_i, [_vp, _i, _vp, _vp, _vp]),
    "mb200_decode_finish": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "mb200_comm_buffer_bytes": (_sz, [_i, _sz]),
    "mb200_comm_alloc": (_i, [_i, _sz, _vp, _vp]),
    "mb200_comm_create": (_i, [_i, _i, _sz, _vp, _vp, _vp]),
    "mb200_comm_create_ptrs": (_i, [_i, _i, _sz, _vp, _vp]),
    "mb200_comm_destroy": (None, [_vp, _i]),
    "mb200_push_allreduce": (_i, [_vp, _vp, _vp, _i, _vp]),
    "mb200_moe_block_push": (_i, [_vp, _vp, _sz, _sz, _sz, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mb200_decode_layer_moe_reduce": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _vp]),
    "mb200_push_allgather": (_i, [_vp, _vp, _vp, _i, _vp]),
    "mb200_decode_layer_attn": (_i, [_vp, _i, _vp, _vp, _vp, _vp]),
    "mb200_decode_layer_oproj": (_i, [_vp, _i, _vp, _vp, _vp, _vp]),
    "mb200_decode_layer_moe": (_i, [_vp, _i, _vp, _i, _vp, _vp]),
    "mb200_decode_logits_local": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "mb200_decode_pick": (_i, [_vp, _i, _vp, _vp, _vp]),
    "mb200_fill_q4k_at": (_i, [_vp, _sz, _sz, _u64, _vp]),
    "mb200_fill_q6k_at": (_i, [_vp, _sz, _sz, _u64, _vp]),
    "mb200_fill_q4k": (_i, [_vp, _sz, _u64, _vp]),
    "mb200_fill_q6k": (_i, [_vp, _sz, _u64, _vp]),
    "mb200_fill_normal_f32": (_i, [_vp, _sz, _u64, _f, _vp]),
    "mb200_fill_normal_f16": (_i, [_vp, _sz, _u64, _f, _vp]),
}


def declared_symbols() -> list[str]:
    """Function names declared in include/mnemo_b200.h."""
    text = open(HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:cuda|mb200)_[a-z0-9_]+)\s*\(", text)))


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m mnemocuda_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these kernels.")
    handle = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = handle
    return _lib
