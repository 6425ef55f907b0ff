"""Our kernels against the reference's own CUDA kernels on the same device buffers.

oracle/_ref/libmnemo_ref_kernels.so is the reference's src/kernels.cu +
src/gemm_q4k.cu compiled unmodified by oracle/Makefile (`make ref`); it is a
checker, not part of the product. Skipped when that build is absent.
Shapes are limited to ones the reference kernels handle by reading
(row counts that are multiples of 4 for the fused QKV kernel, whose early
return sits before a block-wide barrier: src/kernels.cu:220).
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from mnemocuda_b200 import synth
from tests.gpu_util import dev, host

pytestmark = pytest.mark.gpu

REF = os.path.join(os.path.dirname(__file__), "..", "oracle", "_ref", "libmnemo_ref_kernels.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF):
        pytest.skip("reference kernels not built (oracle/_ref)")
    lib = C.CDLL(os.path.abspath(REF))
    lib.cuda_kernels_init()
    return lib


@pytest.fixture(scope="module")
def K():
    from mnemocuda_b200 import kernels
    kernels.mb200_init()
    return kernels


def _s():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr())


def _rel(a, b):
    a, b = host(a).astype(np.float64), host(b).astype(np.float64)
    return np.linalg.norm(a - b) / np.linalg.norm(b)


@pytest.mark.parametrize("rows,cols", [(8192, 4096), (4096, 8192), (1536, 4096), (64, 512)])
def test_q4k_matches_reference_kernel(ref, K, rows, cols):
    w, x = dev(synth.q4k_matrix(1, rows, cols)), dev(synth.normal_f32(2, cols))
    y_ref, y = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    ref.cuda_matvec_q4k(_p(w), _p(x), _p(y_ref), C.c_int(rows), C.c_int(cols), _s())
    K.cuda_matvec_q4k(w, x, y, rows, cols)
    torch.cuda.synchronize()
    assert _rel(y, y_ref) <= 1e-3


@pytest.mark.parametrize("rows,cols", [(4096, 1536), (512, 4096), (2048, 768)])
def test_q6k_matches_reference_kernel(ref, K, rows, cols):
    w, x = dev(synth.q6k_matrix(3, rows, cols)), dev(synth.normal_f32(4, cols))
    y_ref, y = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    ref.cuda_matvec_q6k(_p(w), _p(x), _p(y_ref), C.c_int(rows), C.c_int(cols), _s())
    K.cuda_matvec_q6k(w, x, y, rows, cols)
    torch.cuda.synchronize()
    assert _rel(y, y_ref) <= 1e-3


def test_expert_sequence_matches_reference_kernels(ref, K):
    """dual -> swiglu -> q6k -> scaled_add as the reference issues them (src/forward.c:1122-1142)
    against our fused forms."""
    H, EFF = 4096, 1536
    blob = dev(synth.expert_blob(5, H, EFF))
    g_sz, u_sz, _ = synth.expert_sizes(H, EFF)
    x = dev(synth.normal_f32(6, H))
    gate, up, act, out = (torch.empty(n, device="cuda") for n in (EFF, EFF, EFF, H))
    moe_ref = torch.zeros(H, device="cuda")
    ref.cuda_matvec_q4k_dual(_p(blob), _p(blob[g_sz:]), _p(x), _p(gate), _p(up), C.c_int(EFF), C.c_int(H), _s())
    ref.cuda_swiglu(_p(gate), _p(up), _p(act), C.c_int(EFF), _s())
    ref.cuda_matvec_q6k(_p(blob[g_sz + u_sz:]), _p(act), _p(out), C.c_int(H), C.c_int(EFF), _s())
    ref.cuda_scaled_add(_p(moe_ref), _p(out), C.c_float(0.125), C.c_int(H), _s())

    act2 = torch.empty(EFF, device="cuda")
    moe = torch.zeros(H, device="cuda")
    K.mb200_matvec_q4k_dual_swiglu(blob, blob[g_sz:], x, act2, EFF, H)
    K.mb200_matvec_q6k_scaled_add(blob[g_sz + u_sz:], act2, moe, H, EFF, 0.125)
    torch.cuda.synchronize()
    assert _rel(act2, act) <= 1e-3
    assert _rel(moe, moe_ref) <= 1e-3


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_topk_matches_reference_kernel_bit_exact(ref, K, seed):
    s = dev(synth.normal_f32(10 + seed, 128, 2.0))
    i_ref = torch.empty(8, dtype=torch.int32, device="cuda"); w_ref = torch.empty(8, device="cuda")
    i_got = torch.empty(8, dtype=torch.int32, device="cuda"); w_got = torch.empty(8, device="cuda")
    ref.cuda_topk_softmax(_p(s), _p(i_ref), _p(w_ref), C.c_int(128), C.c_int(8), _s())
    K.cuda_topk_softmax(s, i_got, w_got, 128, 8)
    torch.cuda.synchronize()
    assert torch.equal(i_got, i_ref)
    np.testing.assert_allclose(host(w_got), host(w_ref), rtol=1e-4, atol=1e-6)
