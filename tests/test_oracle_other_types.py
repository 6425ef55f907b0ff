"""The oracle's Q8_0 / Q5_K / Q3_K dequantisers and INT8 KV-cache functions.

Q5_K and Q8_0 are held with == against the reference validator's restatements of its kernels
(fixtures from tests/golden/make_golden.py). The validator has no Q3_K function; for that type this
file checks the restatement against a second, independent reading of the reference kernel written
here element by element (src/kernels.cu:497-575), and the GPU suite checks it against the
reference's compiled kernel."""
import numpy as np
import pytest

from mnemocuda_b200 import synth
from oracle import oracle


@pytest.mark.parametrize("tag,tid", [("q5k", 13), ("q8_0", 8)])
def test_seeded_and_ragged_match_the_validator(golden, tag, tid):
    for name, rows, cols in (("seeded", 3, 1024), ("ragged", 2, 300)):
        got = oracle.dequant_type(tid, golden[f"{tag}_{name}_w"], rows, cols)
        assert np.array_equal(got, golden[f"{tag}_{name}_ref"]), (tag, name)


def _q3k_by_element(blk: np.ndarray) -> np.ndarray:
    """Weight j of one 110-byte block, each field looked up from j alone (the form of the reference's
    embedding kernel, src/kernels.cu:1955-2030)."""
    hm, qs, sc = blk[0:32], blk[32:96], blk[96:108]
    d = np.float32(blk[108:110].view(np.float16)[0])
    out = np.zeros(256, np.float32)
    for j in range(256):
        i = j // 16
        ii, hi = i % 8, i // 8
        lo4 = (int(sc[ii]) >> 4) if hi else (int(sc[ii]) & 0xF)
        hi2 = (int(sc[8 + ii // 4]) >> (2 * (ii % 4) + 4 * hi)) & 3
        s = (lo4 | (hi2 << 4)) - 32
        chunk, grp, l = j // 128, (j % 128) // 32, j % 32
        q2 = (int(qs[chunk * 32 + l]) >> (2 * grp)) & 3
        hbit = (int(hm[l]) >> (chunk * 4 + grp)) & 1
        out[j] = np.float32(d * np.float32(s)) * np.float32(q2 - (0 if hbit else 4))
    return out


def test_q3k_matches_an_element_wise_reading():
    w = synth.typed_matrix(11, 23, 2, 512).reshape(4, 110)
    got = oracle.dequant_type(11, w.reshape(-1), 2, 512).reshape(4, 256)
    for b in range(4):
        assert np.array_equal(got[b], _q3k_by_element(w[b]))


def test_q3k_known_block():
    """hmask set and q = 3 everywhere gives +3 * d * (scale - 32); hmask clear and q = 0 gives -4 * ..."""
    b = np.zeros(110, np.uint8)
    b[0:32] = 0xFF
    b[32:96] = 0xFF
    b[96:104] = 0x11   # low nibbles 1: scales 0..7 = 1 - 32, scales 8..15 = 1 - 32
    b[108:110] = np.array([1.0], np.float16).view(np.uint8)
    got = oracle.dequant_type(11, b, 1, 256)[0]
    assert np.all(got == 3.0 * -31.0)
    b[0:96] = 0
    got = oracle.dequant_type(11, b, 1, 256)[0]
    assert np.all(got == -4.0 * -31.0)


@pytest.mark.parametrize("tid", [8, 11, 13])
def test_matvec_equals_dequant_times_x(tid):
    rows, cols = 5, 800 if tid != 8 else 810
    w = synth.typed_matrix(tid, 31, rows, cols)
    x = synth.normal_f32(32, cols)
    y, y64, ad = oracle.matvec_type(tid, w, x, rows, cols, full=True)
    want = oracle.dequant_type(tid, w, rows, cols).astype(np.float64) @ x.astype(np.float64)
    np.testing.assert_allclose(y64, want, rtol=1e-12, atol=1e-12)
    assert np.all(np.abs(y - want) <= 1e-5 * ad + 1e-30)


def test_unknown_type_is_refused():
    lib = oracle.lib()
    import ctypes as C
    lib.mo_dequant_type.restype = C.c_int
    assert lib.mo_dequant_type(C.c_int(99), None, 0, 0, None) == -1


def test_int8_kv_quantise():
    hd, nkv = 128, 4
    x = synth.normal_f32(40, hd * nkv, 2.0)
    x[hd:2 * hd] = 0.0  # an all-zero head: scale 0, all zeros
    q, s = oracle.f32_to_int8_kv(x, hd, nkv)
    xr = x.reshape(nkv, hd)
    am = np.abs(xr).max(1)
    assert np.array_equal(s, np.where(am > 0, am / np.float32(127.0), 0).astype(np.float32))
    assert s[1] == 0.0 and not q.reshape(nkv, hd)[1].any()
    assert np.abs(q).max() == 127
    back = q.reshape(nkv, hd).astype(np.float32) * s[:, None]
    assert np.abs(back - xr).max() <= 0.5 * s.max() * 1.0001


def test_int8_attention_against_numpy():
    nh, nkv, hd, S = 8, 2, 128, 37
    gqa = nh // nkv
    q = synth.normal_f32(41, nh * hd)
    rng = np.random.default_rng(42)
    k8 = rng.integers(-127, 128, (S, nkv, hd), dtype=np.int8)
    v8 = rng.integers(-127, 128, (S, nkv, hd), dtype=np.int8)
    ks = (rng.random((S, nkv)) * 0.02).astype(np.float32)
    vs = (rng.random((S, nkv)) * 0.02).astype(np.float32)
    scale = hd ** -0.5
    got = oracle.attention_int8kv(q, k8, v8, ks, vs, nh, hd, nkv, S, gqa, scale).reshape(nh, hd)
    kf = k8.astype(np.float64) * ks[:, :, None]
    vf = v8.astype(np.float64) * vs[:, :, None]
    for h in range(nh):
        sc = kf[:, h // gqa] @ q.reshape(nh, hd)[h].astype(np.float64) * scale
        p = np.exp(sc - sc.max())
        p /= p.sum()
        np.testing.assert_allclose(got[h], p @ vf[:, h // gqa], rtol=1e-5, atol=1e-7)
