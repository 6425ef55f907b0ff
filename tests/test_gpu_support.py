"""GPU parity of the support operators of a decode step (RMSNorm family, RoPE, fp16 KV store,
decode attention, residual add, Q4_K embedding row, greedy sampling) against the CPU oracle, whose
RMSNorm / RoPE are pinned to the reference's tools/validate_rope_norm.py replicas. Called through
the C ABI under the reference's names (src/kernels.cu:1178-1333, 1662-1671, 2192-2215)."""
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


@pytest.mark.parametrize("n", [4096, 2048, 128, 1000, 5])
def test_rms_norm_and_residual_save(K, n):
    x = synth.normal_f32(1, n, 3.0)
    w = (1 + 0.1 * synth.normal_f32(2, n)).astype(np.float32)
    want = oracle.rms_norm(x, w, 1e-6)
    out = torch.empty(n, device="cuda")
    K.cuda_rms_norm(dev(x), dev(w), out, n, 1e-6)
    np.testing.assert_allclose(host(out), want, rtol=2e-6, atol=0)
    out2, res = torch.empty(n, device="cuda"), torch.empty(n, device="cuda")
    K.cuda_rms_norm_residual(dev(x), dev(w), out2, res, n, 1e-6)
    assert torch.equal(out2, out) and np.array_equal(host(res), x)
    xin = dev(x)  # in place
    K.cuda_rms_norm(xin, dev(w), xin, n, 1e-6)
    assert torch.equal(xin, out)


@pytest.mark.parametrize("hd,nq,nk", [(128, 64, 4), (128, 32, 4), (64, 3, 1), (256, 2, 2)])
def test_rms_norm_qk_and_batched(K, hd, nq, nk):
    q, k = synth.normal_f32(3, nq * hd, 5.0), synth.normal_f32(4, nk * hd, 0.2)
    wq, wk = (1 + 0.1 * synth.normal_f32(5, hd)).astype(np.float32), (1 + 0.1 * synth.normal_f32(6, hd)).astype(np.float32)
    dq, dk = dev(q), dev(k)
    K.cuda_rms_norm_qk(dq, dk, dev(wq), dev(wk), hd, nq, nk, 1e-6)
    np.testing.assert_allclose(host(dq), oracle.rms_norm_heads(q, wq, hd, nq, 1e-6), rtol=2e-6)
    np.testing.assert_allclose(host(dk), oracle.rms_norm_heads(k, wk, hd, nk, 1e-6), rtol=2e-6)
    out = torch.empty(nq * hd, device="cuda")
    K.cuda_rms_norm_batched(dev(q), dev(wq), out, hd, nq, 1e-6)
    assert torch.equal(out, dq)


@pytest.mark.parametrize("pos", [0, 1, 17, 4095, 8191, 100000])
def test_rope(K, pos):
    nq, nk, hd, theta = 64, 4, 128, 1e6
    q, k = synth.normal_f32(7, nq * hd), synth.normal_f32(8, nk * hd)
    dq, dk = dev(q), dev(k)
    K.cuda_rope(dq, dk, hd, pos, theta, nq, nk)
    for got, src, n in ((dq, q, nq), (dk, k, nk)):
        want = oracle.rope(src, n, hd, pos, theta)
        assert np.max(np.abs(host(got) - want)) <= 4e-7 * np.max(np.abs(want))
    if pos == 0:
        assert np.array_equal(host(dq), q)


def test_f32_to_f16_bit_exact(K):
    a = np.concatenate([synth.normal_f32(9, 512) * s for s in (1e-7, 1e-3, 1.0, 1e4)])
    b = synth.normal_f32(10, a.size, 40.0)
    oa = torch.empty(a.size, dtype=torch.float16, device="cuda")
    ob = torch.empty(a.size, dtype=torch.float16, device="cuda")
    K.cuda_f32_to_f16_dual(dev(a), dev(b), oa, ob, a.size)
    assert np.array_equal(host(oa).view(np.uint16), oracle.f32_to_f16_bits(a))
    assert np.array_equal(host(ob).view(np.uint16), oracle.f32_to_f16_bits(b))
    oc = torch.empty(a.size, dtype=torch.float16, device="cuda")
    K.cuda_f32_to_f16(dev(a), oc, a.size)
    assert torch.equal(oc, oa)


def attention_case(K, NH, NKV, HD, S, seed, q_scale=1.0, ctx=None):
    ctx = ctx or S
    q = synth.normal_f32(seed, NH * HD, q_scale)
    k = synth.normal_f16(seed + 1, ctx * NKV * HD).reshape(ctx, NKV, HD)
    v = synth.normal_f16(seed + 2, ctx * NKV * HD).reshape(ctx, NKV, HD)
    want = oracle.attention_f16kv(q, k.view(np.uint16), v.view(np.uint16), NH, HD, NKV, S, NH // NKV, HD ** -0.5)
    out = torch.full((NH * HD,), float("nan"), device="cuda")
    dk, dv = dev(k), dev(v)
    for _ in range(2):  # the tickets must be back at zero after a call
        K.cuda_attention_f16kv(dev(q), dk, dv, out, NH, HD, NKV, S, NH // NKV, HD ** -0.5)
    got = host(out).reshape(NH, HD).astype(np.float64)
    want = want.reshape(NH, HD).astype(np.float64)
    rel = np.linalg.norm(got - want, axis=1) / np.linalg.norm(want, axis=1)
    assert np.all(np.isfinite(got)) and rel.max() <= 1e-3, (NH, NKV, HD, S, rel.max())
    return rel.max()


@pytest.mark.parametrize("NH,NKV,S", [
    (64, 4, 8192),   # Qwen3-235B heads, full context
    (32, 4, 4096),   # Qwen3-30B heads
    (64, 4, 1), (64, 4, 2), (64, 4, 15), (64, 4, 16), (64, 4, 17), (64, 4, 4097), (64, 4, 600),
    (8, 8, 333),     # no grouping
    (40, 2, 1000),   # 20 query heads per KV head: two query blocks per KV head, the second partly empty
    (3, 1, 77),
])
def test_attention_tensor_core_kernel(K, NH, NKV, S):
    attention_case(K, NH, NKV, 128, S, 30 + S % 7)


def test_attention_peaked_scores(K):
    # large |q|: the softmax is dominated by a few positions (scores of +-40)
    attention_case(K, 64, 4, 128, 2048, 50, q_scale=8.0)


def test_attention_reads_only_seq_len_rows(K):
    # cache longer than seq_len and the rows beyond it poisoned with NaN
    NH, NKV, HD, S, ctx = 16, 2, 128, 100, 128
    q = synth.normal_f32(60, NH * HD)
    k = synth.normal_f16(61, ctx * NKV * HD).reshape(ctx, NKV, HD).copy()
    v = synth.normal_f16(62, ctx * NKV * HD).reshape(ctx, NKV, HD).copy()
    k[S:] = np.nan
    v[S:] = np.nan
    want = oracle.attention_f16kv(q, k.view(np.uint16), v.view(np.uint16), NH, HD, NKV, S, NH // NKV, HD ** -0.5)
    out = torch.empty(NH * HD, device="cuda")
    K.cuda_attention_f16kv(dev(q), dev(k), dev(v), out, NH, HD, NKV, S, NH // NKV, HD ** -0.5)
    np.testing.assert_allclose(host(out), want, rtol=2e-3, atol=2e-4)


@pytest.mark.parametrize("HD,NH,NKV,S", [(64, 8, 2, 300), (256, 4, 1, 129), (96, 6, 3, 50)])
def test_attention_other_head_sizes(K, HD, NH, NKV, S):
    attention_case(K, NH, NKV, HD, S, 70)


def test_residual_add(K):
    a, b = synth.normal_f32(80, 4097), synth.normal_f32(81, 4097)
    out = torch.empty(4097, device="cuda")
    K.cuda_residual_add(dev(a), dev(b), out, 4097)
    assert np.array_equal(host(out), a + b)


@pytest.mark.parametrize("hidden", [4096, 2048, 300])
def test_embedding_row_bit_exact(K, hidden):
    rows = 37
    table = synth.q4k_matrix(90, rows, hidden)
    row_bytes = synth.q4k_row_bytes(hidden)
    for t in (0, 5, rows - 1):
        out = torch.full((hidden,), float("nan"), device="cuda")
        K.cuda_embedding_lookup_q4k(dev(table), out, t, hidden, row_bytes)
        assert np.array_equal(host(out), oracle.embedding_q4k(table, t, hidden))


def test_embedding_known_blocks_bit_exact(K, golden):
    w = golden["q4k_known_w"]  # hand-built blocks: zero, all-ones, one-hot nibbles, subnormal / negative d
    for t in range(w.shape[0]):
        out = torch.empty(256, device="cuda")
        K.cuda_embedding_lookup_q4k(dev(w.reshape(-1)), out, t, 256, 144)
        got, want = host(out), golden["q4k_known_ref"][t]
        assert np.array_equal(got, want, equal_nan=True)


def test_sample_token_greedy_and_ties(K):
    V = 151936
    x = synth.normal_f32(95, V)
    res = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    K.cuda_sample_token(dev(x), V, 0.0, 0.9, 1234, res)
    assert int(res.item()) == oracle.argmax(x) == int(np.argmax(x))
    x[:] = -1.0
    x[[700, 300, 4396, 150000]] = 5.0
    K.cuda_sample_token(dev(x), V, 0.0, 0.9, 1234, res)
    # thread = index % 256: 188, 44, 44, 240; the tree prefers the smaller bit-reversed thread id: 240 (0b11110000)
    assert int(res.item()) == oracle.argmax(x) == 150000


@pytest.mark.parametrize("V,scale,temp,top_p", [(151936, 3.0, 0.7, 0.9), (151936, 1.0, 1.0, 0.5), (32000, 6.0, 0.3, 0.95),
                                                (1000, 2.0, 1.5, 1.0), (300, 1.0, 0.8, 0.8), (151936, 0.5, 1.0, 0.99)])
def test_sample_token_top_p_matches_the_oracle(K, V, scale, temp, top_p):
    """Temperature + top-p sampling: the same token as the oracle's serial restatement of the reference for a set
    of random 64-bit generator states (a draw within float rounding of a boundary may legitimately differ: at most
    one of the states may disagree, and then only by a neighbour in the nucleus)."""
    logits = (synth.normal_f32(96 + V, V) * scale).astype(np.float32)
    d_l = dev(logits)
    res = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    rng = np.random.default_rng(97)
    seeds = [int(s) for s in rng.integers(1, 2 ** 63, 40)]
    miss = 0
    for seed in seeds:
        K.cuda_sample_token(d_l, V, temp, top_p, seed, res)
        got, want = int(res.item()), oracle.sample_top_p(logits, temp, top_p, seed)
        assert 0 <= got < V
        miss += got != want
    assert miss <= 1, miss
    if V == 151936 and scale == 3.0:
        assert len({oracle.sample_top_p(logits, temp, top_p, s) for s in seeds}) > 5  # the draw does vary


def test_sample_token_top_p_degenerate_and_repeat(K):
    V = 50000
    logits = np.full(V, -5.0, np.float32)
    logits[4321] = 30.0
    res = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    for seed in (1, 2 ** 40 + 7, 2 ** 62 + 1):
        K.cuda_sample_token(dev(logits), V, 0.8, 0.9, seed, res)
        assert int(res.item()) == 4321
    # equal logits everywhere: every class keeps its eight smallest ids; the result is one of those and repeats
    logits[:] = 0.0
    picks = set()
    for rep in range(3):
        K.cuda_sample_token(dev(logits), V, 1.0, 0.9, 123456789123, res)
        picks.add(int(res.item()))
    assert len(picks) == 1 and next(iter(picks)) < 256 * 8
    # greedy still works after the sampling kernels have used the library's scratch
    logits[777] = 1.0
    K.cuda_sample_token(dev(logits), V, 0.0, 0.9, 5, res)
    assert int(res.item()) == 777


def test_kernel_pointer_exports(K):
    from mnemocuda_b200 import _lib
    lib = _lib.lib()
    ptrs = [lib.cuda_get_rope_kernel_ptr(), lib.cuda_get_f16dual_kernel_ptr(), lib.cuda_get_attn_f16kv_kernel_ptr()]
    assert all(ptrs) and len(set(ptrs)) == 3
