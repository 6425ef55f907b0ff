"""GPU parity: every matvec entry point of the C ABI against the CPU oracle on
seeded synthetic blocks (tolerance: 1e-3 relative L2, fp64-accumulated oracle)."""
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


Q4_SHAPES = [
    (8192, 4096),   # Q projection, 235B shape (benchmark config 1)
    (4096, 8192),   # O projection
    (1536, 4096),   # expert gate / up
    (4096, 1536),   # expert down when stored as Q4_K (6 blocks per row)
    (4096, 2048),   # 30B-shape Q projection
    (1, 256), (3, 256), (64, 256), (5, 300), (33, 1000), (7, 2048), (130, 768), (3, 16384),
    (149, 1280), (1000, 512),
]


@pytest.mark.parametrize("rows,cols", Q4_SHAPES)
def test_matvec_q4k(K, rows, cols):
    w = synth.q4k_matrix(1000 + rows + cols, rows, cols)
    x = synth.normal_f32(2000 + cols, cols)
    y_ref, y64, ad = oracle.matvec_q4k(w, x, rows, cols, full=True)
    y = torch.full((rows,), float("nan"), device="cuda")
    K.cuda_matvec_q4k(dev(w), dev(x), y, rows, cols)
    assert_close_matvec(host(y), y64, ad, f"q4k {rows}x{cols}")


def test_matvec_q4k_outlier_activations(K):
    """Groups with one huge activation: the two-level split must still hold the tolerance."""
    rows, cols = 256, 4096
    w = synth.q4k_matrix(31, rows, cols)
    x = synth.normal_f32(32, cols)
    x[::97] *= 1000.0
    x[5] = 0.0
    x[1024:1056] = 0.0  # an all-zero group
    _, y64, ad = oracle.matvec_q4k(w, x, rows, cols, full=True)
    y = torch.empty(rows, device="cuda")
    K.cuda_matvec_q4k(dev(w), dev(x), y, rows, cols)
    assert_close_matvec(host(y), y64, ad, "q4k outliers")


def test_matvec_q4k_known_blocks(K, golden):
    """Hand-built blocks (subnormal / negative d, extreme scales) as a 1-block-per-row matrix."""
    w = golden["q4k_known_w"][[0, 2, 3, 4, 5, 6]]  # block 1 holds NaN-free but 0xFF data too; keep finite ones
    rows = w.shape[0]
    x = synth.normal_f32(33, 256)
    _, y64, ad = oracle.matvec_q4k(w.reshape(-1), x, rows, 256, full=True)
    y = torch.empty(rows, device="cuda")
    K.cuda_matvec_q4k(dev(w.reshape(-1)), dev(x), y, rows, 256)
    assert_close_matvec(host(y), y64, ad, "q4k known blocks")


def test_matvec_q4k_add(K):
    rows, cols = 4096, 8192
    w = synth.q4k_matrix(41, rows, cols)
    x = synth.normal_f32(42, cols)
    res = synth.normal_f32(43, rows, 50.0)
    _, y64, ad = oracle.matvec_q4k(w, x, rows, cols, full=True)
    y = torch.empty(rows, device="cuda")
    K.cuda_matvec_q4k_add(dev(w), dev(x), dev(res), y, rows, cols)
    assert_close_matvec(host(y), y64 + res, ad + np.abs(res), "q4k_add")
    np.testing.assert_allclose(host(y), oracle.matvec_q4k_add(w, x, res, rows, cols), rtol=0, atol=1e-3 * np.abs(y64).max())


@pytest.mark.parametrize("q_rows,kv_rows,cols", [(8192, 512, 4096), (64, 8, 512), (10, 3, 300), (4096, 512, 2048)])
def test_matvec_q4k_qkv(K, q_rows, kv_rows, cols):
    wq = synth.q4k_matrix(51, q_rows, cols)
    wk = synth.q4k_matrix(52, kv_rows, cols)
    wv = synth.q4k_matrix(53, kv_rows, cols)
    x = synth.normal_f32(54, cols)
    q, k, v = (torch.empty(n, device="cuda") for n in (q_rows, kv_rows, kv_rows))
    K.cuda_matvec_q4k_qkv(dev(wq), dev(wk), dev(wv), dev(x), q, k, v, q_rows, kv_rows, cols)
    for got, w, n, name in ((q, wq, q_rows, "q"), (k, wk, kv_rows, "k"), (v, wv, kv_rows, "v")):
        _, y64, ad = oracle.matvec_q4k(w, x, n, cols, full=True)
        assert_close_matvec(host(got), y64, ad, f"qkv.{name}")


@pytest.mark.parametrize("rows,cols", [(1536, 4096), (768, 2048), (9, 300)])
def test_matvec_q4k_dual(K, rows, cols):
    wa = synth.q4k_matrix(61, rows, cols)
    wb = synth.q4k_matrix(62, rows, cols)
    x = synth.normal_f32(63, cols)
    ya, yb = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    K.cuda_matvec_q4k_dual(dev(wa), dev(wb), dev(x), ya, yb, rows, cols)
    for got, w in ((ya, wa), (yb, wb)):
        _, y64, ad = oracle.matvec_q4k(w, x, rows, cols, full=True)
        assert_close_matvec(host(got), y64, ad, "dual")


def test_matvec_q4k_scaled_add_accumulates(K):
    rows, cols = 4096, 1536
    w = synth.q4k_matrix(71, rows, cols)
    x = synth.normal_f32(72, cols)
    y0 = synth.normal_f32(73, rows, 10.0)
    _, y64, ad = oracle.matvec_q4k(w, x, rows, cols, full=True)
    y = dev(y0.copy())
    K.cuda_matvec_q4k_scaled_add(dev(w), dev(x), y, rows, cols, 0.37)
    K.cuda_matvec_q4k_scaled_add(dev(w), dev(x), y, rows, cols, -1.5)
    want = y0.astype(np.float64) + (0.37 - 1.5) * y64
    assert_close_matvec(host(y), want, 1.87 * ad + np.abs(y0), "q4k_scaled_add x2")


@pytest.mark.parametrize("rows,cols", [(1536, 4096), (768, 2048), (9, 300), (1, 256)])
def test_dual_swiglu(K, rows, cols):
    wg = synth.q4k_matrix(81, rows, cols)
    wu = synth.q4k_matrix(82, rows, cols)
    x = synth.normal_f32(83, cols)
    g, u = oracle.matvec_q4k_dual(wg, wu, x, rows, cols)
    _, g64, gad = oracle.matvec_q4k(wg, x, rows, cols, full=True)
    _, u64, uad = oracle.matvec_q4k(wu, x, rows, cols, full=True)
    want = g64 / (1.0 + np.exp(-g64)) * u64
    act = torch.empty(rows, device="cuda")
    K.mb200_matvec_q4k_dual_swiglu(dev(wg), dev(wu), dev(x), act, rows, cols)
    # error scale of a product: |silu(g)| * err(u) + |u| * err(g)
    scale = np.abs(g64 / (1 + np.exp(-g64))) * uad + np.abs(u64) * 1.1 * gad
    assert_close_matvec(host(act), want, scale, "dual_swiglu")
    np.testing.assert_allclose(host(act), oracle.swiglu(g, u), rtol=2e-3, atol=1e-3 * np.abs(want).max())


Q6_SHAPES = [
    (4096, 1536),   # expert down (benchmark config 2)
    (512, 4096),    # V projection
    (2048, 768),    # 30B expert down: 3 blocks per row, rows only 2-byte aligned
    (1000, 2048),
    (1, 256), (5, 256), (17, 300), (33, 1000), (7, 1280), (3, 12288), (3, 16384), (149, 512),
]


@pytest.mark.parametrize("rows,cols", Q6_SHAPES)
def test_matvec_q6k(K, rows, cols):
    w = synth.q6k_matrix(3000 + rows + cols, rows, cols)
    x = synth.normal_f32(4000 + cols, cols)
    _, y64, ad = oracle.matvec_q6k(w, x, rows, cols, full=True)
    y = torch.full((rows,), float("nan"), device="cuda")
    K.cuda_matvec_q6k(dev(w), dev(x), y, rows, cols)
    assert_close_matvec(host(y), y64, ad, f"q6k {rows}x{cols}")


@pytest.mark.parametrize("offset", [2, 6, 14, 210])
def test_matvec_q6k_unaligned_base(K, offset):
    """Q6_K tensors only promise 2-byte alignment (expert blobs place them after two Q4_K parts)."""
    rows, cols = 96, 1536
    w = synth.q6k_matrix(91, rows, cols)
    x = synth.normal_f32(92, cols)
    _, y64, ad = oracle.matvec_q6k(w, x, rows, cols, full=True)
    buf = torch.zeros(w.size + 512, dtype=torch.uint8, device="cuda")
    buf[offset:offset + w.size] = dev(w)
    y = torch.empty(rows, device="cuda")
    K.cuda_matvec_q6k(buf[offset:], dev(x), y, rows, cols)
    assert_close_matvec(host(y), y64, ad, f"q6k base+{offset}")


def test_matvec_q6k_known_blocks(K, golden):
    w = golden["q6k_known_w"]
    rows = w.shape[0]
    x = synth.normal_f32(93, 256)
    _, y64, ad = oracle.matvec_q6k(w.reshape(-1), x, rows, 256, full=True)
    y = torch.empty(rows, device="cuda")
    K.cuda_matvec_q6k(dev(w.reshape(-1)), dev(x), y, rows, 256)
    assert_close_matvec(host(y), y64, ad, "q6k known blocks")


def test_matvec_q6k_scaled_add(K):
    rows, cols = 4096, 1536
    w = synth.q6k_matrix(94, rows, cols)
    x = synth.normal_f32(95, cols)
    y0 = synth.normal_f32(96, rows)
    _, y64, ad = oracle.matvec_q6k(w, x, rows, cols, full=True)
    y = dev(y0.copy())
    K.mb200_matvec_q6k_scaled_add(dev(w), dev(x), y, rows, cols, 0.25)
    K.mb200_matvec_q6k_scaled_add(dev(w), dev(x), y, rows, cols, 0.5)
    assert_close_matvec(host(y), y0 + 0.75 * y64, 0.75 * ad + np.abs(y0), "q6k_scaled_add x2")


def test_repeat_calls_are_bitwise_stable(K):
    """Fixed tile schedule and ordered partial sums: the same call gives the same bits."""
    rows, cols = 8192, 4096
    w, x = dev(synth.q4k_matrix(97, rows, cols)), dev(synth.normal_f32(98, cols))
    a, b = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    K.cuda_matvec_q4k(w, x, a, rows, cols)
    K.cuda_matvec_q4k(w, x, b, rows, cols)
    assert torch.equal(a, b)


def test_bad_alignment_is_reported_not_run(K):
    rows, cols = 4, 256
    buf = torch.zeros(rows * 144 + 64, dtype=torch.uint8, device="cuda")
    y = torch.zeros(rows, device="cuda")
    with pytest.raises(RuntimeError):
        K.cuda_matvec_q4k(buf[4:], torch.zeros(cols, device="cuda"), y, rows, cols)
    with pytest.raises(RuntimeError):
        K.cuda_matvec_q4k(buf, torch.zeros(20000, device="cuda"), y, rows, 20000)


def _one_hot_rows(K, call, w_dev, rows, cols, positions):
    """y for x = e_c, for each c in positions: column c of the dequantised matrix as the kernel sees it."""
    y = torch.empty(rows, device="cuda")
    x = torch.zeros(cols, device="cuda")
    out = np.zeros((len(positions), rows), np.float32)
    for i, c in enumerate(positions):
        x.zero_()
        x[c] = 1.0
        call(w_dev, x, y, rows, cols)
        out[i] = host(y)
    return out


def _q4k_term_scale(w_blocks):
    """|d*sc*q| + |dmin*m| per weight, [rows][256]: the magnitude the kernel's fp32 arithmetic works at."""
    out = np.zeros((w_blocks.shape[0], 256), np.float64)
    for r, blk in enumerate(w_blocks):
        d, dm, sc, m, q = oracle.unpack_q4k_block(blk)
        df, dmf = abs(oracle.f16_to_f32(d)), abs(oracle.f16_to_f32(dm))
        out[r] = df * np.repeat(sc.astype(np.float64), 32) * q + dmf * np.repeat(m.astype(np.float64), 32)
    return out


def _q6k_term_scale(w_blocks):
    """|d*sc|*(q + 32 + 32) per weight: the kernel forms d*sc*(q_raw*x - 32*x)."""
    out = np.zeros((w_blocks.shape[0], 256), np.float64)
    for r, blk in enumerate(w_blocks):
        d, sc, q = oracle.unpack_q6k_block(blk)
        out[r] = abs(oracle.f16_to_f32(d)) * np.abs(np.repeat(sc.astype(np.float64), 16)) * (q.astype(np.float64) + 64)
    return out


ONE_HOT_TOL = 2.0 ** -20  # a few fp32 roundings at the magnitude of the terms; a wrong integer field is off by >= 1 step


def test_one_hot_sweep_q4k_known_blocks(K, golden):
    """Bit-exact integer unpack on the GPU side: with x a one-hot vector (exactly representable in the
    kernel's two-level int8 split up to one rounding of 1/127) output row r is the dequantised weight
    W[r][c] itself. Every one of the 256 positions of the hand-built blocks and of seeded blocks must
    reproduce the reference validator's value to a few fp32 roundings of its terms -- a wrong scale, min
    or nibble would be off by whole quantisation steps."""
    w = np.concatenate([golden["q4k_known_w"][:6], synth.q4k_blocks(91, 26)])  # 32 rows of one block each
    ref = oracle.dequant_q4k(w.reshape(-1), w.shape[0], 256)
    assert np.array_equal(ref[:6], golden["q4k_known_ref"][:6], equal_nan=True)
    got = _one_hot_rows(K, K.cuda_matvec_q4k, dev(w.reshape(-1)), w.shape[0], 256, range(256)).T  # [row][col]
    scale = _q4k_term_scale(w)
    finite = np.isfinite(ref)
    assert np.all(np.isfinite(got[finite]))
    err = np.abs(got.astype(np.float64) - ref)[finite]
    assert np.all(err <= ONE_HOT_TOL * scale[finite] + 1e-45), float((err / (scale[finite] + 1e-300)).max())
    # the distinct values of a sub-block are d*sc apart: an error of one integer step would be >= 2^-4 of the scale
    assert ONE_HOT_TOL < 2.0 ** -10


def test_one_hot_sweep_q6k_known_blocks(K, golden):
    w = np.concatenate([golden["q6k_known_w"], synth.q6k_blocks(92, 26)])
    ref = oracle.dequant_q6k(w.reshape(-1), w.shape[0], 256)
    n_known = golden["q6k_known_w"].shape[0]
    assert np.array_equal(ref[:n_known], golden["q6k_known_ref"], equal_nan=True)
    got = _one_hot_rows(K, K.cuda_matvec_q6k, dev(w.reshape(-1)), w.shape[0], 256, range(256)).T
    scale = _q6k_term_scale(w)
    finite = np.isfinite(ref)
    err = np.abs(got.astype(np.float64) - ref)[finite]
    assert np.all(err <= ONE_HOT_TOL * scale[finite] + 1e-45), float((err / (scale[finite] + 1e-300)).max())


def test_one_hot_multi_block_rows(K):
    """Same check on rows of several blocks (the column-group split of the kernel): 4096 and 1536 columns."""
    for call, gen, deq, cols in ((K.cuda_matvec_q4k, synth.q4k_matrix, oracle.dequant_q4k, 4096),
                                 (K.cuda_matvec_q6k, synth.q6k_matrix, oracle.dequant_q6k, 1536)):
        rows = 40
        w = gen(93, rows, cols)
        ref = deq(w, rows, cols)
        pos = list(range(0, cols, 37)) + [cols - 1]
        got = _one_hot_rows(K, call, dev(w), rows, cols, pos)
        bb = 144 if cols == 4096 else 210
        blocks = w.reshape(rows * (cols // 256), bb)
        scale = (_q4k_term_scale if cols == 4096 else _q6k_term_scale)(blocks).reshape(rows, cols)
        err = np.abs(got.astype(np.float64) - ref.T[pos])
        assert np.all(err <= ONE_HOT_TOL * scale.T[pos] + 1e-45), (cols, float((err / (scale.T[pos] + 1e-300)).max()))


@pytest.mark.parametrize("kind,rows,cols", [("q4k", 8192, 4096), ("q4k", 4096, 2048), ("q4k", 100, 300), ("q4k", 40, 256),
                                            ("q6k", 512, 4096), ("q6k", 512, 2048), ("q6k", 33, 1536), ("q6k", 7, 300)])
def test_rmsnorm_folded_into_the_matvec(K, kind, rows, cols):
    """mb200_norm_matvec_*: y = W RMSNorm(x) with the norm done inside the matvec's staging of x, against the
    oracle's RMSNorm followed by its matvec (and against the two separate kernels)."""
    gen = synth.q4k_matrix if kind == "q4k" else synth.q6k_matrix
    mv = oracle.matvec_q4k if kind == "q4k" else oracle.matvec_q6k
    call = K.mb200_norm_matvec_q4k if kind == "q4k" else K.mb200_norm_matvec_q6k
    plain = K.cuda_matvec_q4k if kind == "q4k" else K.cuda_matvec_q6k
    w = gen(300 + rows, rows, cols)
    x = synth.normal_f32(301, cols, 3.0)
    nw = (1 + 0.1 * synth.normal_f32(302, cols)).astype(np.float32)
    xn = oracle.rms_norm(x, nw, 1e-6)
    _, want, ad = mv(w, xn, rows, cols, full=True)
    y = torch.full((rows,), float("nan"), device="cuda")
    call(dev(w), dev(x), dev(nw), 1e-6, y, rows, cols)
    assert_close_matvec(host(y), want, ad, f"norm+matvec {kind} {rows}x{cols}")
    # the two-kernel path gives the same up to the rounding of the norm's sum of squares
    xn_d = torch.empty(cols, device="cuda")
    K.cuda_rms_norm(dev(x), dev(nw), xn_d, cols, 1e-6)
    y2 = torch.empty(rows, device="cuda")
    plain(dev(w), xn_d, y2, rows, cols)
    a, b = host(y).astype(np.float64), host(y2).astype(np.float64)
    assert np.linalg.norm(a - b) <= 2e-5 * np.linalg.norm(b)


def test_rmsnorm_folded_two_tensors_and_width_limit(K):
    rows_a, rows_b, cols = 4096, 512, 2048
    wa, wb = synth.q4k_matrix(310, rows_a, cols), synth.q4k_matrix(311, rows_b, cols)
    x = synth.normal_f32(312, cols, 0.5)
    nw = (1 + 0.1 * synth.normal_f32(313, cols)).astype(np.float32)
    xn = oracle.rms_norm(x, nw, 1e-6)
    ya, yb = torch.empty(rows_a, device="cuda"), torch.empty(rows_b, device="cuda")
    K.mb200_norm_matvec2_q4k(dev(wa), ya, rows_a, dev(wb), yb, rows_b, dev(x), dev(nw), 1e-6, cols)
    for y, w, r in ((ya, wa, rows_a), (yb, wb, rows_b)):
        _, want, ad = oracle.matvec_q4k(w, xn, r, cols, full=True)
        assert_close_matvec(host(y), want, ad, "norm + two tensors")
    # wider than one round of loads per CTA: refused, nothing launched
    wide = 8192
    yw = torch.full((4,), 5.0, device="cuda")
    with pytest.raises(RuntimeError, match="status 4"):
        K.mb200_norm_matvec_q4k(dev(synth.q4k_matrix(314, 4, wide)), dev(synth.normal_f32(315, wide)),
                                dev(np.ones(wide, np.float32)), 1e-6, yw, 4, wide)
    assert float(yw.min()) == 5.0


@pytest.mark.parametrize("q_rows,kv_rows,cols,with_norm", [(8192, 512, 4096, True), (4096, 512, 2048, True),
                                                           (2048, 256, 4096, False), (512, 256, 512, True),
                                                           (130, 7, 768, True), (64, 8, 256, False)])
def test_qkv_in_one_launch(K, q_rows, kv_rows, cols, with_norm):
    """Q, K (Q4_K) and V (Q6_K) projections of RMSNorm(x) in one launch of the pair kernel, against the oracle's
    three matvecs (shapes: the 235B and 30B projections, a KV shard of one head pair, ragged ones)."""
    wq, wk = synth.q4k_matrix(5000, q_rows, cols), synth.q4k_matrix(5001, kv_rows, cols)
    wv = synth.q6k_matrix(5002, kv_rows, cols)
    x = synth.normal_f32(5003, cols, 3.0)
    nw = (1.0 + 0.1 * synth.normal_f32(5004, cols)).astype(np.float32)
    xn = oracle.rms_norm(x, nw, 1e-6) if with_norm else x
    q, k, v = (torch.full((n,), float("nan"), device="cuda") for n in (q_rows, kv_rows, kv_rows))
    for rep in range(2):
        K.mb200_norm_matvec_qkv(dev(wq), q, q_rows, dev(wk), k, dev(wv), v, kv_rows, dev(x), dev(nw) if with_norm else None,
                                1e-6, cols)
        for got, (w, fn, rows) in ((q, (wq, oracle.matvec_q4k, q_rows)), (k, (wk, oracle.matvec_q4k, kv_rows)),
                                   (v, (wv, oracle.matvec_q6k, kv_rows))):
            _, y64, ad = fn(w, xn, rows, cols, full=True)
            assert_close_matvec(host(got), y64, ad, f"qkv {rows}x{cols} rep {rep}")
