"""GPU parity of the tcgen05 prefill GEMM against the oracle: out = f16(X) . dequant(W)^T with the
weights held in fp32 by the oracle (tolerance 1e-3 relative L2 per token row; the fp16 rounding of
the weights inside the kernel costs about 3e-4)."""
import numpy as np
import pytest
import torch

from mnemocuda_b200 import synth
from oracle import oracle
from tests.gpu_util import dev, host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from mnemocuda_b200 import kernels
    kernels.mb200_init()
    yield kernels
    torch.cuda.synchronize()
    assert kernels.mb200_device_error() == 0


def _check_rows(got, want):
    got = got.astype(np.float64); want = want.astype(np.float64)
    assert np.all(np.isfinite(got))
    num = np.linalg.norm(got - want, axis=1)
    den = np.linalg.norm(want, axis=1)
    worst = float((num / den).max())
    assert worst <= 1e-3, worst
    return worst


@pytest.mark.parametrize("M,N,Kd", [(256, 128, 256), (512, 256, 1024), (300, 200, 512), (16, 128, 256), (1, 128, 256),
                                     (512, 1024, 4096)])
def test_gemm_q4k(K, M, N, Kd):
    w = synth.q4k_matrix(700 + N, N, Kd)
    x = synth.normal_f16(701 + M, M * Kd).reshape(M, Kd)
    want = oracle.gemm_q4k_f16(w, x, M, N, Kd)
    out = torch.full((M, N), float("nan"), device="cuda")
    K.mb200_gemm_q4k_f16(dev(w), dev(x), out, M, N, Kd)
    _check_rows(host(out), want)


@pytest.mark.parametrize("M,N,Kd", [(256, 128, 256), (128, 256, 1536), (40, 130, 512)])
def test_gemm_q6k(K, M, N, Kd):
    w = synth.q6k_matrix(710 + N, N, Kd)
    x = synth.normal_f16(711 + M, M * Kd).reshape(M, Kd)
    want = oracle.gemm_q6k_f16(w, x, M, N, Kd)
    out = torch.full((M, N), float("nan"), device="cuda")
    K.mb200_gemm_q6k_f16(dev(w), dev(x), out, M, N, Kd)
    _check_rows(host(out), want)


def test_gemm_matches_matvec_per_token(K):
    """Token t of the GEMM equals the decode matvec on x_t (both within tolerance of the oracle)."""
    M, N, Kd = 8, 256, 1024
    w = synth.q4k_matrix(720, N, Kd)
    x = synth.normal_f16(721, M * Kd).reshape(M, Kd)
    out = torch.empty(M, N, device="cuda")
    K.mb200_gemm_q4k_f16(dev(w), dev(x), out, M, N, Kd)
    y = torch.empty(N, device="cuda")
    for t in range(M):
        K.cuda_matvec_q4k(dev(w), dev(x[t].astype(np.float32)), y, N, Kd)
        a, b = host(out[t]).astype(np.float64), host(y).astype(np.float64)
        assert np.linalg.norm(a - b) / np.linalg.norm(b) <= 1e-3


def test_gemm_rejects_bad_k(K):
    with pytest.raises(RuntimeError):
        K.mb200_gemm_q4k_f16(torch.zeros(144 * 128, dtype=torch.uint8, device="cuda"),
                             torch.zeros(16, 128, dtype=torch.float16, device="cuda"),
                             torch.zeros(16, 128, device="cuda"), 16, 128, 128)
