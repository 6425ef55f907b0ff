"""GPU parity of the device-resident MoE block (router + top-k, routed gate/up + SwiGLU,
routed down + weighted sum + residual) against the CPU oracle's restatement of the
reference sequence (src/forward.c:810-823, 875, 1122-1142, 1114)."""
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


def make_block(seed, NE, H, EFF, down_type):
    g, u, d = synth.expert_sizes(H, EFF, down_type)
    stride = g + u + d
    experts = np.concatenate([synth.expert_blob(seed * 1000 + e, H, EFF, down_type) for e in range(NE)])
    router = synth.normal_f32(seed * 7 + 1, NE * H, 1.0 / np.sqrt(H))
    x = synth.normal_f32(seed * 7 + 2, H)
    res = synth.normal_f32(seed * 7 + 3, H)
    return experts, stride, g, u, router, x, res


def scratch_for(K, NE):
    n = K.mb200_router_scratch_bytes(NE)
    return torch.zeros((n + 15) // 16 * 16, dtype=torch.uint8, device="cuda")


@pytest.mark.parametrize("NE,k,H", [(128, 8, 4096), (128, 8, 2048), (16, 4, 512), (512, 8, 1024), (5, 8, 256)])
def test_router_topk(K, NE, k, H):
    router = synth.normal_f32(11, NE * H, 1.0 / np.sqrt(H))
    x = synth.normal_f32(12, H)
    scratch = scratch_for(K, NE)
    ids = torch.full((k,), -9, dtype=torch.int32, device="cuda")
    wts = torch.zeros(k, device="cuda")
    for _ in range(2):  # the ticket must be back at zero after a call
        K.mb200_router_topk(dev(router), dev(x), scratch, ids, wts, NE, H, k)
    logits = host(scratch[32:32 + 4 * NE].view(torch.float32))
    want = oracle.matvec_f32_f64(router, x, NE, H)
    scale = np.abs(router.reshape(NE, H).astype(np.float64) * x).sum(1)
    assert np.all(np.abs(logits - want) <= 1e-5 * scale)
    # selection: bit-exact against the oracle's restatement applied to the same logits
    i_ref, w_ref = oracle.topk_softmax(logits, k)
    assert np.array_equal(host(ids), i_ref)
    np.testing.assert_allclose(host(wts), w_ref, rtol=1e-5, atol=1e-7)
    assert int(host(scratch[:4].view(torch.int32))[0]) == 0
    # and, for these seeds (no near-ties), against the oracle's own logits too
    i_full, _ = oracle.topk_softmax(oracle.matvec_f32(router, x, NE, H), k)
    assert np.array_equal(host(ids), i_full)


@pytest.mark.parametrize("NE,k,H,EFF,down_type", [
    (16, 8, 4096, 1536, 14),   # Qwen3-235B expert shape, Q6_K down (benchmark config 2, fewer experts)
    (16, 8, 2048, 768, 14),    # Qwen3-30B expert shape
    (8, 2, 512, 256, 12),      # Q4_K down
    (6, 4, 768, 512, 14),
    (4, 8, 256, 256, 14),      # fewer experts than k: empty slots
])
def test_moe_block_matches_oracle(K, NE, k, H, EFF, down_type):
    experts, stride, g, u, router, x, res = make_block(3, NE, H, EFF, down_type)
    want, i_ref, w_ref = oracle.moe_block(router, experts, stride, g, u, down_type, NE, k, H, EFF, x, res)
    d_exp = dev(experts)
    ids = torch.empty(k, dtype=torch.int32, device="cuda")
    wts = torch.empty(k, device="cuda")
    act = torch.full((k, EFF), float("nan"), device="cuda")
    out = torch.full((H,), float("nan"), device="cuda")
    K.mb200_moe_block(dev(router), d_exp, stride, g, u, down_type, NE, k, H, EFF, dev(x), dev(res), out, ids, wts,
                      act, scratch_for(K, NE))
    assert np.array_equal(host(ids), i_ref)
    np.testing.assert_allclose(host(wts), w_ref, rtol=1e-5, atol=1e-7)
    # per-expert activations against the oracle
    for s, e in enumerate(i_ref):
        if e < 0:
            continue  # empty slot: skipped, its activation row is not written
        blob = experts[e * stride:(e + 1) * stride]
        gg, uu = oracle.matvec_q4k_dual(blob, blob[g:], x, EFF, H)
        np.testing.assert_allclose(host(act[s]), oracle.swiglu(gg, uu), rtol=3e-3, atol=1e-3 * np.abs(gg).max() * np.abs(uu).max())
    got = host(out).astype(np.float64)
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel <= 1e-3, rel
    # the MoE contribution alone (residual removed) also within tolerance
    moe_ref = want.astype(np.float64) - res
    rel_moe = np.linalg.norm((got - res) - moe_ref) / np.linalg.norm(moe_ref)
    assert rel_moe <= 2e-3, rel_moe


def test_moe_down_accumulates_without_residual(K):
    NE, k, H, EFF = 4, 3, 512, 256
    experts, stride, g, u, router, x, res = make_block(5, NE, H, EFF, 14)
    ids = dev(np.array([2, 0, 3], np.int32))
    wts = dev(np.array([0.5, 0.25, 0.125], np.float32))
    act_h = synth.normal_f32(9, k * EFF).reshape(k, EFF)
    y0 = synth.normal_f32(10, H)
    y = dev(y0.copy())
    K.mb200_moe_down(dev(experts), stride, g + u, 14, ids, wts, k, dev(act_h), None, y, H, EFF)
    want = y0.astype(np.float64)
    for s, e in enumerate([2, 0, 3]):
        blob = experts[e * stride + g + u:(e + 1) * stride]
        _, y64, _ = oracle.matvec_q6k(blob, act_h[s], H, EFF, full=True)
        want += float(host(wts)[s]) * y64
    assert_close_matvec(host(y), want, None, "moe_down accumulate")


def test_moe_block_is_capturable_and_repeatable(K):
    """The three launches are legal under stream capture and give the same bits on replay."""
    NE, k, H, EFF = 16, 8, 2048, 768
    experts, stride, g, u, router, x, res = make_block(6, NE, H, EFF, 14)
    d = [dev(a) for a in (router, experts, x, res)]
    ids = torch.empty(k, dtype=torch.int32, device="cuda"); wts = torch.empty(k, device="cuda")
    act = torch.empty(k, EFF, device="cuda"); out = torch.empty(H, device="cuda"); scratch = scratch_for(K, NE)
    run = lambda: K.mb200_moe_block(d[0], d[1], stride, g, u, 14, NE, k, H, EFF, d[2], d[3], out, ids, wts, act, scratch)
    run(); torch.cuda.synchronize()
    first = out.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    out.zero_()
    graph.replay(); graph.replay(); torch.cuda.synchronize()
    assert torch.equal(out, first)


def test_moe_block_with_programmatic_dependent_launch(K):
    NE, k, H, EFF = 16, 8, 2048, 768
    experts, stride, g, u, router, x, res = make_block(7, NE, H, EFF, 14)
    want, i_ref, _ = oracle.moe_block(router, experts, stride, g, u, 14, NE, k, H, EFF, x, res)
    d = [dev(a) for a in (router, experts, x, res)]
    ids = torch.empty(k, dtype=torch.int32, device="cuda"); wts = torch.empty(k, device="cuda")
    act = torch.empty(k, EFF, device="cuda"); out = torch.empty(H, device="cuda"); scratch = scratch_for(K, NE)
    prev = K.mb200_set_pdl(True)
    try:
        for _ in range(3):
            K.mb200_moe_block(d[0], d[1], stride, g, u, 14, NE, k, H, EFF, d[2], d[3], out, ids, wts, act, scratch)
        torch.cuda.synchronize()
    finally:
        K.mb200_set_pdl(prev)
    assert np.array_equal(host(ids), i_ref)
    got = host(out).astype(np.float64)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_sharded_partials_sum_to_the_full_block(K, world):
    """The *_local entry points, run for every rank of an expert partition one after the other on
    one GPU: the partial hidden vectors must sum to the unsharded block (and match the oracle)."""
    from mnemocuda_b200 import sharded
    NE, k, H, EFF = 16, 8, 2048, 768
    experts, stride, g, u, router, x, res = make_block(8, NE, H, EFF, 14)
    want, i_ref, _ = oracle.moe_block(router, experts, stride, g, u, 14, NE, k, H, EFF, x, res)
    d_exp, d_x, d_res = dev(experts), dev(x), dev(res)
    ids = torch.empty(k, dtype=torch.int32, device="cuda"); wts = torch.empty(k, device="cuda")
    K.mb200_router_topk(dev(router), d_x, scratch_for(K, NE), ids, wts, NE, H, k)
    zero = torch.zeros(H, device="cuda")
    total = torch.zeros(H, device="cuda", dtype=torch.float64)
    served = 0
    for rank in range(world):
        lo, hi = sharded.expert_range(NE, world, rank)
        act = torch.full((k, EFF), float("nan"), device="cuda")  # slots of other ranks stay untouched
        part = torch.full((H,), float("nan"), device="cuda")
        shard = d_exp[lo * stride:]
        K.mb200_moe_gate_up_local(shard, stride, 0, g, ids, k, lo, hi - lo, d_x, act, EFF, H)
        K.mb200_moe_down_local(shard, stride, g + u, 14, ids, wts, k, lo, hi - lo, act, d_res if rank == 0 else zero,
                               part, H, EFF)
        assert torch.isfinite(part).all()
        total += part.double()
        served += int(((ids >= lo) & (ids < hi)).sum())
    assert served == k
    got = host(total)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3
