"""The C oracle against the golden vectors made from the reference's own
Python restatement (tools/validate_dequant.py) and gguf.quants -- equality,
not tolerance. Fixtures: tests/golden/make_golden.py."""
import numpy as np

from oracle import oracle


def test_f16_to_f32_all_patterns():
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(v)) for v in h], np.float32)
    nan = np.isnan(want)  # NaN payloads do not survive the ctypes float->double hop; compare NaN-ness
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])


def test_f16_probe_matches_reference_validator(golden):
    got = np.array([oracle.f16_to_f32(int(h)) for h in golden["f16_probe"]], np.float32)
    assert np.array_equal(got, golden["f16_probe_ref"])


def test_f32_to_f16_round_trip_and_rounding():
    rng = np.random.default_rng(0)
    f = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 3e4, 1e6)])
    want = f.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f32_to_f16(float(v)) for v in f], np.uint16)
    assert np.array_equal(got, want)


def test_get_scale_min_k4(golden):
    for r in range(golden["scale_min_in"].shape[0]):
        for j in range(8):
            sc, m = oracle.get_scale_min_k4(j, golden["scale_min_in"][r])
            assert (sc, m) == tuple(int(v) for v in golden["scale_min_out"][r, j])


def test_q4k_seeded(golden):
    got = oracle.dequant_q4k(golden["q4k_seeded_w"], 3, 1024)
    assert np.array_equal(got, golden["q4k_seeded_ref"])


def test_q6k_seeded(golden):
    got = oracle.dequant_q6k(golden["q6k_seeded_w"], 3, 1024)
    assert np.array_equal(got, golden["q6k_seeded_ref"])


def test_q4k_known_blocks(golden):
    w = golden["q4k_known_w"]
    got = oracle.dequant_q4k(w.reshape(-1), w.shape[0], 256)
    assert np.array_equal(got, golden["q4k_known_ref"], equal_nan=True)


def test_q6k_known_blocks(golden):
    w = golden["q6k_known_w"]
    got = oracle.dequant_q6k(w.reshape(-1), w.shape[0], 256)
    assert np.array_equal(got, golden["q6k_known_ref"], equal_nan=True)


def test_ragged(golden):
    assert np.array_equal(oracle.dequant_q4k(golden["q4k_ragged_w"], 2, 300), golden["q4k_ragged_ref"])
    assert np.array_equal(oracle.dequant_q6k(golden["q6k_ragged_w"], 2, 300), golden["q6k_ragged_ref"])


def test_unpack_is_consistent_with_dequant(golden):
    """Integer fields: recombining them with the fp32 formula reproduces the golden floats."""
    w = golden["q4k_seeded_w"].reshape(-1, 144)
    ref = golden["q4k_seeded_ref"].reshape(-1, 256)
    for b in range(w.shape[0]):
        d, dm, sc, m, q = oracle.unpack_q4k_block(w[b])
        assert q.max() <= 15 and sc.max() <= 63 and m.max() <= 63
        df = np.float32(oracle.f16_to_f32(d)); mf = np.float32(oracle.f16_to_f32(dm))
        ds = (df * sc.astype(np.float32)).repeat(32)
        ms = (mf * m.astype(np.float32)).repeat(32)
        assert np.array_equal(ds * q.astype(np.float32) - ms, ref[b])
    w = golden["q6k_seeded_w"].reshape(-1, 210)
    ref = golden["q6k_seeded_ref"].reshape(-1, 256)
    for b in range(w.shape[0]):
        d, sc, q = oracle.unpack_q6k_block(w[b])
        assert q.min() >= -32 and q.max() <= 31
        s = (np.float32(oracle.f16_to_f32(d)) * sc.astype(np.float32)).repeat(16)
        assert np.array_equal(s * q.astype(np.float32), ref[b])
