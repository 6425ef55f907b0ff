"""GPU parity for the fp32 operators of the ABI: router matvec, top-k softmax
(indices bit-exact, in the reference's slot order), SwiGLU, scaled add, and the
device-side synthetic fills."""
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
    return kernels


@pytest.mark.parametrize("rows,cols", [(128, 4096), (128, 2048), (7, 33), (1, 1), (300, 1000), (16, 40000)])
def test_matvec_f32(K, rows, cols):
    w = synth.normal_f32(101, rows * cols, 1.0 / np.sqrt(cols))
    x = synth.normal_f32(102, cols)
    want = oracle.matvec_f32_f64(w, x, rows, cols)
    y = torch.empty(rows, device="cuda")
    K.cuda_matvec_f32(dev(w), dev(x), y, rows, cols)
    scale = np.abs(w.reshape(rows, cols).astype(np.float64) * x).sum(1)
    assert np.all(np.abs(host(y) - want) <= 1e-5 * scale + 1e-30)
    # and against the reference-ordered fp32 restatement, within fp32 reassociation noise
    np.testing.assert_allclose(host(y), oracle.matvec_f32(w, x, rows, cols), rtol=0, atol=2e-5 * scale.max())


def _topk(K, scores, k):
    n = scores.size
    idx = torch.full((k,), -7, dtype=torch.int32, device="cuda")
    wts = torch.full((k,), float("nan"), device="cuda")
    K.cuda_topk_softmax(dev(scores), idx, wts, n, k)
    return host(idx), host(wts)


@pytest.mark.parametrize("n,k,seed", [(128, 8, 1), (128, 8, 2), (128, 8, 3), (512, 8, 4), (64, 16, 5), (256, 1, 6),
                                      (100, 7, 7), (8, 8, 8), (33, 16, 9)])
def test_topk_softmax_indices_bit_exact(K, n, k, seed):
    scores = synth.normal_f32(200 + seed, n, 3.0)
    i_ref, w_ref = oracle.topk_softmax(scores, k)
    i_got, w_got = _topk(K, scores, k)
    assert np.array_equal(i_got, i_ref)
    np.testing.assert_allclose(w_got, w_ref, rtol=1e-5, atol=1e-7)
    assert abs(w_got.sum() - 1.0) < 1e-5


def test_topk_ties_and_duplicates(K):
    cases = [np.zeros(128, np.float32),
             np.tile(np.array([1.0, 2.0, 3.0, 2.0], np.float32), 32),
             np.concatenate([np.full(100, -5.0, np.float32), np.arange(28, dtype=np.float32) % 3]),
             np.array([0.5] * 7 + [0.25] * 121, np.float32)]
    for s in cases:
        i_ref, w_ref = oracle.topk_softmax(s, 8)
        i_got, w_got = _topk(K, s, 8)
        assert np.array_equal(i_got, i_ref)
        np.testing.assert_allclose(w_got, w_ref, rtol=1e-5, atol=1e-7)


def test_topk_fewer_experts_than_k(K):
    s = synth.normal_f32(210, 5)
    i_ref, _ = oracle.topk_softmax(s, 8)
    i_got, _ = _topk(K, s, 8)
    assert np.array_equal(i_got, i_ref)
    assert (i_got == -1).sum() == 3


def test_topk_rejects_bad_k(K):
    s = torch.zeros(128, device="cuda")
    with pytest.raises(RuntimeError):
        K.cuda_topk_softmax(s, torch.zeros(17, dtype=torch.int32, device="cuda"), torch.zeros(17, device="cuda"), 128, 17)


@pytest.mark.parametrize("n", [1, 768, 1536, 5000])
def test_swiglu_and_scaled_add(K, n):
    g, u = synth.normal_f32(301, n, 4.0), synth.normal_f32(302, n, 2.0)
    out = torch.empty(n, device="cuda")
    K.cuda_swiglu(dev(g), dev(u), out, n)
    np.testing.assert_allclose(host(out), oracle.swiglu(g, u), rtol=1e-5, atol=1e-6)
    acc0 = synth.normal_f32(303, n)
    acc = dev(acc0.copy())
    K.cuda_scaled_add(acc, out, 0.3, n)
    np.testing.assert_allclose(host(acc), oracle.scaled_add(acc0, host(out), 0.3), rtol=1e-6, atol=1e-6)


def test_device_fill_matches_host_generator(K):
    nb = 1000
    d4 = torch.empty(nb * 144, dtype=torch.uint8, device="cuda")
    K.mb200_fill_q4k(d4, nb, 77)
    h4 = synth.q4k_blocks(77, nb)
    g4 = host(d4).reshape(nb, 144)
    assert np.array_equal(g4[:, 4:], h4[:, 4:])          # scales + nibbles: bit-identical streams
    dd = g4[:, :4].copy().view(np.float16).astype(np.float32)
    hh = h4[:, :4].copy().view(np.float16).astype(np.float32)
    np.testing.assert_allclose(dd, hh, rtol=2e-3, atol=1e-7)  # fp32 vs fp64 Box-Muller: last fp16 bit

    d6 = torch.empty(nb * 210, dtype=torch.uint8, device="cuda")
    K.mb200_fill_q6k(d6, nb, 78)
    h6 = synth.q6k_blocks(78, nb)
    g6 = host(d6).reshape(nb, 210)
    assert np.array_equal(g6[:, :208], h6[:, :208])
    np.testing.assert_allclose(g6[:, 208:].copy().view(np.float16).astype(np.float32),
                               h6[:, 208:].copy().view(np.float16).astype(np.float32), rtol=2e-3, atol=1e-7)

    x = torch.empty(4096, device="cuda")
    K.mb200_fill_normal_f32(x, 4096, 79, 1.0)
    np.testing.assert_allclose(host(x), synth.normal_f32(79, 4096), rtol=1e-4, atol=1e-5)
    assert abs(float(x.mean())) < 0.1 and abs(float(x.std()) - 1.0) < 0.1
