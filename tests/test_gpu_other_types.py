"""GPU parity of the Q8_0 / Q5_K / Q3_K matvecs, the Q3_K embedding row and the INT8 KV-cache kernels
against the oracle (matvec: 1e-3 relative L2 plus the per-row bound; INT8 store and embedding row:
bit-exact; attention: 1e-3 relative L2 per head)."""
import numpy as np
import pytest
import torch

from mnemocuda_b200 import synth
from oracle import oracle
from tests.gpu_util import assert_close_matvec, dev, host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from mnemocuda_b200 import kernels
    kernels.mb200_init()
    yield kernels
    torch.cuda.synchronize()
    assert kernels.mb200_device_error() == 0


SHAPES = [(8192, 4096), (4096, 1536), (1, 256), (3, 32), (5, 300), (33, 1000), (130, 768), (1000, 512), (7, 8192),
          (2, 16384)]


@pytest.mark.parametrize("tid,name", [(8, "cuda_matvec_q8_0"), (13, "cuda_matvec_q5k"), (11, "cuda_matvec_q3k")])
@pytest.mark.parametrize("rows,cols", SHAPES)
def test_typed_matvec(K, tid, name, rows, cols):
    w = synth.typed_matrix(tid, 3000 + rows + cols, rows, cols)
    x = synth.normal_f32(3100 + cols, cols)
    _, y64, ad = oracle.matvec_type(tid, w, x, rows, cols, full=True)
    y = torch.full((rows,), float("nan"), device="cuda")
    getattr(K, name)(dev(w), dev(x), y, rows, cols)
    assert_close_matvec(host(y), y64, ad, f"{name} {rows}x{cols}")


@pytest.mark.parametrize("tid,name", [(8, "cuda_matvec_q8_0"), (13, "cuda_matvec_q5k"), (11, "cuda_matvec_q3k")])
def test_typed_matvec_at_an_odd_address(K, tid, name):
    """A tensor that starts 2 bytes past a 16-byte boundary (tensors inside a GGUF blob are only
    guaranteed their type's alignment), so rows begin at every residue the staging copy handles."""
    rows, cols = 37, 1280
    w = synth.typed_matrix(tid, 3200, rows, cols)
    buf = torch.zeros(w.size + 32, dtype=torch.uint8, device="cuda")
    off = (16 - buf.data_ptr() % 16) % 16 + 2
    buf[off:off + w.size] = dev(w)
    x = synth.normal_f32(3201, cols)
    _, y64, ad = oracle.matvec_type(tid, w, x, rows, cols, full=True)
    y = torch.full((rows,), float("nan"), device="cuda")
    getattr(K, name)(buf[off:], dev(x), y, rows, cols)
    assert_close_matvec(host(y), y64, ad, name)


@pytest.mark.parametrize("cols", [512, 300])
def test_typed_matvec_one_hot_x_reads_single_weights(K, cols):
    """x = e_c picks weight c of every row: a direct check of the unpacking of each bit field, in the streaming
    kernels (whole 256-column blocks) and in the row-per-warp kernels (ragged width)."""
    rows = 16
    for tid, name in ((8, "cuda_matvec_q8_0"), (13, "cuda_matvec_q5k"), (11, "cuda_matvec_q3k")):
        w = synth.typed_matrix(tid, 3300 + tid, rows, cols)
        full = oracle.dequant_type(tid, w, rows, cols)
        d_w = dev(w)
        y = torch.empty(rows, device="cuda")
        for c in list(range(0, 256)) + [c for c in (299, 300, 511) if c < cols]:
            x = np.zeros(cols, np.float32)
            x[c] = 1.0
            getattr(K, name)(d_w, dev(x), y, rows, cols)
            got = host(y)
            # a weight is evaluated as a difference of scaled partial sums (d*sc*q - dmin*m, or (q + 4h) - 4):
            # a few ulps of the larger term, 2^-20 of the largest weight magnitude
            tol = 2.0 ** -20 * np.abs(full).max()
            assert np.all(np.abs(got - full[:, c]) <= tol), (name, c, float(np.abs(got - full[:, c]).max()), tol)


def test_embedding_lookup_q3k_is_bit_exact(K):
    vocab, hidden = 50, 1024
    w = synth.typed_matrix(11, 3400, vocab, hidden)
    full = oracle.dequant_type(11, w, vocab, hidden)
    out = torch.empty(hidden, device="cuda")
    d_w = dev(w)
    for tok in (0, 17, 49):
        K.cuda_embedding_lookup_q3k(d_w, out, tok, hidden, hidden // 256 * 110)
        assert np.array_equal(host(out), full[tok])


@pytest.mark.parametrize("hd,nkv", [(128, 4), (128, 8), (64, 3), (256, 2)])
def test_int8_kv_store_is_bit_exact(K, hd, nkv):
    k = synth.normal_f32(3500, hd * nkv, 3.0)
    v = synth.normal_f32(3501, hd * nkv, 0.5)
    v[:hd] = 0.0  # an all-zero head
    want_k, want_ks = oracle.f32_to_int8_kv(k, hd, nkv)
    want_v, want_vs = oracle.f32_to_int8_kv(v, hd, nkv)
    ok = torch.full((hd * nkv,), 99, dtype=torch.int8, device="cuda")
    ov = torch.full((hd * nkv,), 99, dtype=torch.int8, device="cuda")
    sk, sv = torch.empty(nkv, device="cuda"), torch.empty(nkv, device="cuda")
    K.cuda_f32_to_int8_kv_dual(dev(k), dev(v), ok, ov, sk, sv, hd, nkv)
    assert np.array_equal(host(ok), want_k) and np.array_equal(host(ov), want_v)
    assert np.array_equal(host(sk), want_ks) and np.array_equal(host(sv), want_vs)
    ok.fill_(99)
    K.cuda_f32_to_int8_kv(dev(k), ok, sk, hd, nkv)
    assert np.array_equal(host(ok), want_k) and np.array_equal(host(sk), want_ks)


def _int8_cache(seed, S, nkv, hd):
    rng = np.random.default_rng(seed)
    k8 = rng.integers(-127, 128, (S, nkv, hd), dtype=np.int8)
    v8 = rng.integers(-127, 128, (S, nkv, hd), dtype=np.int8)
    ks = (0.5 + rng.random((S, nkv))).astype(np.float32) * np.float32(1.0 / 127)
    vs = (0.5 + rng.random((S, nkv))).astype(np.float32) * np.float32(1.0 / 127)
    return k8, v8, ks, vs


@pytest.mark.parametrize("nh,nkv,hd,S", [(32, 4, 128, 4096), (64, 4, 128, 1000), (16, 4, 128, 257), (8, 8, 128, 65),
                                          (32, 4, 128, 1), (32, 4, 128, 5), (12, 4, 64, 300), (6, 2, 256, 77),
                                          (20, 4, 128, 129)])
def test_int8_attention(K, nh, nkv, hd, S):
    gqa = nh // nkv
    q = synth.normal_f32(3600 + S, nh * hd)
    k8, v8, ks, vs = _int8_cache(3601 + S, S, nkv, hd)
    scale = hd ** -0.5
    want = oracle.attention_int8kv(q, k8, v8, ks, vs, nh, hd, nkv, S, gqa, scale).reshape(nh, hd).astype(np.float64)
    out = torch.full((nh * hd,), float("nan"), device="cuda")
    for rep in range(2):  # twice: the tickets of the split kernel must be back at zero
        out.fill_(float("nan"))
        K.cuda_attention_int8kv(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, nh, hd, nkv, S, gqa, scale)
        got = host(out).reshape(nh, hd).astype(np.float64)
        assert np.all(np.isfinite(got))
        rel = np.linalg.norm(got - want, axis=1) / np.linalg.norm(want, axis=1)
        assert rel.max() <= 1e-3, (rep, rel.max())


def test_int8_store_then_attend_matches_fp16_cache_within_quantisation(K):
    """Round trip: quantise real K / V vectors position by position, attend, compare with attention over
    the unquantised vectors (the INT8 cache is lossy: 2 % relative L2 is its expected scale)."""
    nh, nkv, hd, S = 32, 4, 128, 200
    gqa = nh // nkv
    kf = synth.normal_f32(3700, S * nkv * hd).reshape(S, nkv * hd)
    vf = synth.normal_f32(3701, S * nkv * hd).reshape(S, nkv * hd)
    q = synth.normal_f32(3702, nh * hd)
    k8 = torch.empty(S, nkv * hd, dtype=torch.int8, device="cuda")
    v8 = torch.empty(S, nkv * hd, dtype=torch.int8, device="cuda")
    ks, vs = torch.empty(S, nkv, device="cuda"), torch.empty(S, nkv, device="cuda")
    d_k, d_v = dev(kf), dev(vf)
    for p in range(S):
        K.cuda_f32_to_int8_kv_dual(d_k[p], d_v[p], k8[p], v8[p], ks[p], vs[p], hd, nkv)
    out = torch.empty(nh * hd, device="cuda")
    scale = hd ** -0.5
    K.cuda_attention_int8kv(dev(q), k8, v8, ks, vs, out, nh, hd, nkv, S, gqa, scale)
    want = oracle.attention_f16kv(q, kf.astype(np.float16).view(np.uint16), vf.astype(np.float16).view(np.uint16), nh, hd,
                                  nkv, S, gqa, scale)
    got = host(out).astype(np.float64)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-2
