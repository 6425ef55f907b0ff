"""The oracle's support operators (RMSNorm, RoPE, attention, embedding row, argmax) against the
golden vectors made from the reference's own numpy replicas of its kernels
(tools/validate_rope_norm.py; fixtures: tests/golden/make_golden.py) and against plain numpy."""
import os

import numpy as np
import pytest

from mnemocuda_b200 import synth
from oracle import oracle

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


@pytest.fixture(scope="module")
def sup():
    return np.load(os.path.join(ROOT, "tests", "golden", "support_golden.npz"))


@pytest.mark.parametrize("tag", ["h2048", "h4096", "head128"])
def test_rms_norm_matches_reference_replica(sup, tag):
    got = oracle.rms_norm(sup[f"rms_{tag}_x"], sup[f"rms_{tag}_w"], 1e-6)
    want = sup[f"rms_{tag}_ref"]  # float64 replica; the oracle rounds the same double arithmetic to fp32 once
    assert np.array_equal(got, want.astype(np.float32)) or np.max(np.abs(got - want) / np.abs(want)) <= 2.0 ** -23


def test_rms_norm_heads_is_the_same_norm_per_head():
    x, w = synth.normal_f32(1, 6 * 128, 2.0), (1 + 0.1 * synth.normal_f32(2, 128)).astype(np.float32)
    got = oracle.rms_norm_heads(x, w, 128, 6, 1e-6)
    for h in range(6):
        assert np.array_equal(got[h * 128:(h + 1) * 128], oracle.rms_norm(x[h * 128:(h + 1) * 128], w, 1e-6))


def test_rope_matches_reference_replica(sup):
    nh, hd, theta = int(sup["rope_meta"][0]), int(sup["rope_meta"][1]), float(sup["rope_meta"][2])
    for p, want in zip(sup["rope_pos"], sup["rope_ref"]):
        got = oracle.rope(sup["rope_in"], nh, hd, int(p), theta)
        # same double arithmetic, rounded to fp32 once: half an ulp of the result, and the libm's last bit
        assert np.max(np.abs(got - want)) <= 2.0 ** -22 * np.max(np.abs(want)), int(p)
    assert np.array_equal(oracle.rope(sup["rope_in"], nh, hd, 0, theta), sup["rope_in"])  # position 0: identity


def test_attention_against_numpy():
    rng = np.random.default_rng(3)
    NH, NKV, HD, S = 8, 2, 128, 37
    q = rng.standard_normal(NH * HD).astype(np.float32)
    k = rng.standard_normal((S, NKV, HD)).astype(np.float16)
    v = rng.standard_normal((S, NKV, HD)).astype(np.float16)
    got = oracle.attention_f16kv(q, k.view(np.uint16), v.view(np.uint16), NH, HD, NKV, S, NH // NKV, HD ** -0.5)
    for h in range(NH):
        kk, vv = k[:, h // 4].astype(np.float64), v[:, h // 4].astype(np.float64)
        s = kk @ q[h * HD:(h + 1) * HD].astype(np.float64) * HD ** -0.5
        p = np.exp(s - s.max())
        want = (p / p.sum()) @ vv
        np.testing.assert_allclose(got[h * HD:(h + 1) * HD], want, rtol=1e-6, atol=1e-7)


def test_attention_single_position_returns_v():
    q = synth.normal_f32(5, 4 * 128)
    k = synth.normal_f16(6, 2 * 128).reshape(1, 2, 128)
    v = synth.normal_f16(7, 2 * 128).reshape(1, 2, 128)
    got = oracle.attention_f16kv(q, k.view(np.uint16), v.view(np.uint16), 4, 128, 2, 1, 2, 0.1)
    assert np.array_equal(got.reshape(4, 128), v.astype(np.float32)[0][[0, 0, 1, 1]])


def test_embedding_row_is_the_dequantised_row(golden):
    table = synth.q4k_matrix(21, 5, 1024)
    full = oracle.dequant_q4k(table, 5, 1024)
    for t in range(5):
        assert np.array_equal(oracle.embedding_q4k(table, t, 1024), full[t])
    # and, through the golden file, the reference validator's values
    assert np.array_equal(oracle.embedding_q4k(golden["q4k_seeded_w"], 2, 1024), golden["q4k_seeded_ref"][2])


def test_argmax_follows_the_reference_scan_order():
    x = synth.normal_f32(9, 5000)
    assert oracle.argmax(x) == int(np.argmax(x))
    x[:] = 0.0
    # ties: thread = index % 256 keeps its first maximum; between threads the shared-memory tree keeps the one
    # whose lowest differing bit is 0 (44 = 0b00101100 beats 188 = 0b10111100; 4396 % 256 = 44 comes after 300)
    x[[700, 300, 4396]] = 5.0
    assert oracle.argmax(x) == 300
    x[44] = 5.0
    assert oracle.argmax(x) == 44
    x[4848] = 5.0  # thread 240 = 0b11110000: differs from 44 first in bit 2, where it has the 0
    assert oracle.argmax(x) == 4848
    assert oracle.argmax(np.full(10, -np.inf, np.float32)) == 0


def test_f32_to_f16_array_matches_numpy():
    x = np.concatenate([synth.normal_f32(11, 4096) * s for s in (1e-6, 1.0, 3e4)])
    with np.errstate(over="ignore"):  # values beyond 65504 round to infinity in both
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(oracle.f32_to_f16_bits(x), want)


def _sample_bruteforce(logits, temperature, top_p, seed):
    """An independent reading of the reference's sampler (src/kernels.cu:2073-2174) in numpy."""
    l = logits.astype(np.float32)
    p = np.exp(((l - l.max()) / np.float32(temperature)).astype(np.float32)).astype(np.float32)
    total = float(p.astype(np.float64).sum())
    cand = []
    for c in range(256):
        idx = np.arange(c, l.size, 256)
        order = sorted(idx, key=lambda i: (-p[i], i))[:8]
        cand += order
    cand = sorted(cand, key=lambda i: (-p[i], i))
    M = (1 << 64) - 1
    rs0, rs1 = seed & M, (seed ^ 0xDEADBEEFCAFEBABE) & M
    for _ in range(4):
        t = (rs0 ^ (rs0 << 23)) & M
        rs0 = rs1
        rs1 = (t ^ rs1 ^ (t >> 17) ^ (rs1 >> 26)) & M
    r = float(np.float32(((rs0 + rs1) & M) >> 11) * np.float32(1.0 / 9007199254740992.0))
    cumul, nucleus = 0.0, []
    for i in cand:
        if p[i] <= 0:
            break
        cumul += float(p[i])
        nucleus.append(i)
        if cumul >= top_p * total:
            break
    target, acc = r * sum(float(p[i]) for i in nucleus), 0.0
    for i in nucleus:
        acc += float(p[i])
        if acc >= target:
            return int(i)
    return int(nucleus[0])


def test_top_p_sampler_matches_an_independent_reading():
    rng = np.random.default_rng(5)
    for n, scale, temp, top_p in ((5000, 3.0, 0.7, 0.9), (5000, 1.0, 1.0, 0.5), (1000, 6.0, 0.3, 0.95), (300, 2.0, 1.5, 1.0)):
        logits = (rng.standard_normal(n) * scale).astype(np.float32)
        for seed in rng.integers(1, 2 ** 63, 12):
            assert oracle.sample_top_p(logits, temp, top_p, int(seed)) == _sample_bruteforce(logits, temp, top_p, int(seed))


def test_top_p_sampler_degenerate_cases():
    logits = np.full(1000, -5.0, np.float32)
    logits[123] = 30.0  # one token holds all the mass
    for seed in (1, 2 ** 40 + 7, 2 ** 62 + 1):
        assert oracle.sample_top_p(logits, 0.8, 0.9, seed) == 123
    # top_p -> 0 keeps only the most probable token
    rng = np.random.default_rng(6)
    l = rng.standard_normal(4000).astype(np.float32)
    assert oracle.sample_top_p(l, 1.0, 1e-6, 99) == int(l.argmax())
