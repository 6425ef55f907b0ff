"""The one-launch routed-expert kernel (mb200_moe_experts_fused) against the two-launch path
(mb200_moe_gate_up_local + mb200_moe_down_local, itself checked against the oracle in
test_gpu_moe.py) and against the CPU oracle's expert sequence (src/forward.c:1122-1142)."""
import numpy as np
import pytest
import torch

from mnemocuda_b200 import synth
from oracle import oracle
from tests.gpu_util import dev, host

pytestmark = pytest.mark.gpu

INT_MAX = 0x7FFFFFFF


@pytest.fixture(scope="module")
def K():
    from mnemocuda_b200 import kernels
    kernels.mb200_init()
    yield kernels
    torch.cuda.synchronize()
    assert kernels.mb200_device_error() == 0


def make_experts(seed, NE, H, EFF, down_type):
    g, u, d = synth.expert_sizes(H, EFF, down_type)
    blob = np.concatenate([synth.expert_blob(seed * 1000 + e, H, EFF, down_type) for e in range(NE)])
    return blob, g + u + d, g, u


def two_launch(K, d_exp, stride, g, u, down_type, ids, wts, k, lo, cnt, x, res, y, H, EFF):
    act = torch.full((k, EFF), float("nan"), device="cuda")
    K.mb200_moe_gate_up_local(d_exp, stride, 0, g, ids, k, lo, cnt, x, act, EFF, H)
    K.mb200_moe_down_local(d_exp, stride, g + u, down_type, ids, wts, k, lo, cnt, act, res, y, H, EFF)
    return act


def fused(K, d_exp, stride, g, u, down_type, ids, wts, k, lo, cnt, x, res, y, H, EFF, sync):
    act = torch.full((k, EFF), float("nan"), device="cuda")
    K.mb200_moe_experts_fused(d_exp, stride, 0, g, g + u, down_type, ids, wts, k, lo, cnt, x, act, res, y, H, EFF, sync)
    return act


@pytest.mark.parametrize("H,EFF,down_type,slots", [
    (4096, 1536, 14, [3, 7, 1, 5, 0, 6, 2, 4]),   # Qwen3-235B expert shape (benchmark config 2)
    (4096, 1536, 12, [3, 7, 1, 5, 0, 6, 2, 4]),   # Q4_K down
    (4096, 1536, 14, [5, 2, 6]),                  # three slots: an odd batch
    (4096, 1536, 14, [4]),                        # one slot: a single batch
    (4096, 1536, 14, [1, -1, 3, -1, 0, 2, -1, 7]),  # empty slots in between
    (2048, 512, 14, [0, 3, 2, 1, 5, 4]),          # one gate/up column group, 24-row tiles; narrow down rows
    (2048, 1024, 12, [2, 0, 1, 3]),
    (6144, 1024, 14, [1, 0, 2, 3]),               # three gate/up column groups; two row chunks per CTA in the down phase
])
def test_fused_matches_two_launch_path_and_oracle(K, H, EFF, down_type, slots):
    NE = 8
    k = len(slots)
    experts, stride, g, u = make_experts(21, NE, H, EFF, down_type)
    x = synth.normal_f32(31, H)
    res = synth.normal_f32(32, H)
    w = np.abs(synth.normal_f32(33, k)) + 0.05
    w[np.array(slots) < 0] = 0.0
    w = (w / w.sum()).astype(np.float32)
    d_exp, d_x, d_res = dev(experts), dev(x), dev(res)
    ids, wts = dev(np.array(slots, np.int32)), dev(w)
    sync = torch.zeros(4, dtype=torch.int64, device="cuda")
    y_ref = torch.full((H,), float("nan"), device="cuda")
    act_ref = two_launch(K, d_exp, stride, g, u, down_type, ids, wts, k, 0, INT_MAX, d_x, d_res, y_ref, H, EFF)
    for rep in range(3):  # the barrier counters carry over from launch to launch
        y = torch.full((H,), float("nan"), device="cuda")
        act = fused(K, d_exp, stride, g, u, down_type, ids, wts, k, 0, INT_MAX, d_x, d_res, y, H, EFF, sync)
        torch.cuda.synchronize()
        assert K.mb200_device_error() == 0
        for s, e in enumerate(slots):
            if e >= 0:
                np.testing.assert_allclose(host(act[s]), host(act_ref[s]), rtol=1e-5, atol=1e-6 * float(act_ref[s].abs().max()))
            else:
                assert torch.isnan(act[s]).all()  # skipped slots are never written
        a, b = host(y).astype(np.float64), host(y_ref).astype(np.float64)
        assert np.linalg.norm(a - b) <= 1e-5 * np.linalg.norm(b)
    n_served = sum(e >= 0 for e in slots)
    assert host(sync).tolist()[: (n_served + 1) // 2] == [3 * 148] * ((n_served + 1) // 2)
    # the oracle's expert sequence on the same routing
    moe = np.zeros(H, np.float32)
    for s, e in enumerate(slots):
        if e >= 0:
            moe = oracle.expert_fwd(experts[e * stride:(e + 1) * stride], g, u, H, EFF, down_type, float(w[s]), x, moe)
    want = res.astype(np.float64) + moe
    assert np.linalg.norm(a - want) / np.linalg.norm(want) <= 1e-3


def test_fused_without_served_experts_copies_the_residual(K):
    H, EFF, NE = 4096, 1536, 4
    experts, stride, g, u = make_experts(22, NE, H, EFF, 14)
    d_exp = dev(experts)
    ids, wts = dev(np.array([-1, -1, -1, -1], np.int32)), dev(np.zeros(4, np.float32))
    x, res = dev(synth.normal_f32(1, H)), dev(synth.normal_f32(2, H))
    sync = torch.zeros(4, dtype=torch.int64, device="cuda")
    y = torch.full((H,), float("nan"), device="cuda")
    fused(K, d_exp, stride, g, u, 14, ids, wts, 4, 0, INT_MAX, x, res, y, H, EFF, sync)
    assert torch.equal(y, res)
    assert host(sync).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("world", [2, 4])
def test_fused_expert_shards_sum_to_the_full_block(K, world):
    """Every rank of an expert partition in turn on one GPU: partial hidden vectors, no residual on ranks > 0."""
    from mnemocuda_b200 import sharded
    H, EFF, NE, k = 4096, 1536, 8, 8
    experts, stride, g, u = make_experts(23, NE, H, EFF, 14)
    d_exp = dev(experts)
    slots = [6, 1, 3, 7, 0, 2, 5, 4]
    w = np.full(k, 0.125, np.float32)
    ids, wts = dev(np.array(slots, np.int32)), dev(w)
    x, res = dev(synth.normal_f32(3, H)), dev(synth.normal_f32(4, H))
    y_full = torch.empty(H, device="cuda")
    two_launch(K, d_exp, stride, g, u, 14, ids, wts, k, 0, INT_MAX, x, res, y_full, H, EFF)
    total = torch.zeros(H, dtype=torch.float64, device="cuda")
    zero = torch.zeros(H, device="cuda")
    sync = torch.zeros(4, dtype=torch.int64, device="cuda")
    for rank in range(world):
        lo, hi = sharded.expert_range(NE, world, rank)
        part = torch.full((H,), float("nan"), device="cuda")
        fused(K, d_exp[lo * stride:], stride, g, u, 14, ids, wts, k, lo, hi - lo, x, res if rank == 0 else zero, part, H,
              EFF, sync)
        assert torch.isfinite(part).all()
        total += part.double()
    a, b = host(total), host(y_full).astype(np.float64)
    assert np.linalg.norm(a - b) <= 2e-6 * np.linalg.norm(b)


def test_fused_accumulates_into_y_without_residual(K):
    H, EFF, NE, k = 4096, 1536, 4, 2
    experts, stride, g, u = make_experts(24, NE, H, EFF, 14)
    d_exp = dev(experts)
    ids, wts = dev(np.array([2, 1], np.int32)), dev(np.array([0.75, 0.25], np.float32))
    x = dev(synth.normal_f32(5, H))
    y0 = synth.normal_f32(6, H)
    y_a, y_b = dev(y0.copy()), dev(y0.copy())
    sync = torch.zeros(4, dtype=torch.int64, device="cuda")
    two_launch(K, d_exp, stride, g, u, 14, ids, wts, k, 0, INT_MAX, x, None, y_a, H, EFF)
    fused(K, d_exp, stride, g, u, 14, ids, wts, k, 0, INT_MAX, x, None, y_b, H, EFF, sync)
    a, b = host(y_b).astype(np.float64), host(y_a).astype(np.float64)
    assert np.linalg.norm(a - b) <= 1e-5 * np.linalg.norm(b)


def test_fused_reports_unsupported_shapes_and_launches_nothing(K):
    H, EFF, NE, k = 512, 256, 2, 2   # H / 256 is not a multiple of 8: outside the fused kernel's geometry
    experts, stride, g, u = make_experts(25, NE, H, EFF, 14)
    ids, wts = dev(np.array([0, 1], np.int32)), dev(np.array([0.5, 0.5], np.float32))
    x, res = dev(synth.normal_f32(7, H)), dev(synth.normal_f32(8, H))
    y = torch.full((H,), 7.0, device="cuda")
    act = torch.zeros(k, EFF, device="cuda")
    sync = torch.zeros(4, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="status 4"):
        K.mb200_moe_experts_fused(dev(experts), stride, 0, g, g + u, 14, ids, wts, k, 0, INT_MAX, x, act, res, y, H, EFF, sync)
    assert float(y.min()) == 7.0 and float(y.max()) == 7.0


def test_block_gives_the_same_result_in_all_three_forms(K):
    """mb200_set_fused: 0 = three kernels, 1 = router kernel + fused expert kernel, 2 = one launch."""
    NE, k, H, EFF = 16, 8, 4096, 1536
    g, u, d = synth.expert_sizes(H, EFF, 14)
    experts, stride, g, u = make_experts(26, NE, H, EFF, 14)
    router = synth.normal_f32(41, NE * H, 1.0 / np.sqrt(H))
    x, res = synth.normal_f32(42, H), synth.normal_f32(43, H)
    d_r, d_e, d_x, d_res = dev(router), dev(experts), dev(x), dev(res)
    n = K.mb200_router_scratch_bytes(NE)
    outs = []
    try:
        for mode in (0, 1, 2):
            K.mb200_set_fused(mode)
            scratch = torch.zeros((n + 15) // 16 * 16, dtype=torch.uint8, device="cuda")
            ids = torch.empty(k, dtype=torch.int32, device="cuda"); wts = torch.empty(k, device="cuda")
            act = torch.empty(k, EFF, device="cuda"); out = torch.empty(H, device="cuda")
            for _ in range(2):
                K.mb200_moe_block(d_r, d_e, stride, g, u, 14, NE, k, H, EFF, d_x, d_res, out, ids, wts, act, scratch)
            torch.cuda.synchronize()
            outs.append((host(out).astype(np.float64), host(ids).copy(), host(wts).copy()))
    finally:
        K.mb200_set_fused(2)
    for o, i, w in outs[1:]:
        assert np.array_equal(i, outs[0][1])
        np.testing.assert_allclose(w, outs[0][2], rtol=1e-5)
        assert np.linalg.norm(o - outs[0][0]) <= 1e-5 * np.linalg.norm(outs[0][0])


@pytest.mark.parametrize("world", [2, 4])
def test_block_local_shards_sum_to_the_full_block(K, world):
    """mb200_moe_block_local for every rank of an expert partition in turn (routing replicated on each)."""
    from mnemocuda_b200 import sharded
    NE, k, H, EFF = 16, 8, 4096, 1536
    experts, stride, g, u = make_experts(27, NE, H, EFF, 14)
    router = synth.normal_f32(51, NE * H, 1.0 / np.sqrt(H))
    x, res = synth.normal_f32(52, H), synth.normal_f32(53, H)
    want, i_ref, w_ref = oracle.moe_block(router, experts, stride, g, u, 14, NE, k, H, EFF, x, res)
    d_r, d_e, d_x, d_res = dev(router), dev(experts), dev(x), dev(res)
    zero = torch.zeros(H, device="cuda")
    n = K.mb200_router_scratch_bytes(NE)
    total = torch.zeros(H, dtype=torch.float64, device="cuda")
    for rank in range(world):
        lo, hi = sharded.expert_range(NE, world, rank)
        scratch = torch.zeros((n + 15) // 16 * 16, dtype=torch.uint8, device="cuda")
        ids = torch.empty(k, dtype=torch.int32, device="cuda"); wts = torch.empty(k, device="cuda")
        act = torch.empty(k, EFF, device="cuda"); part = torch.full((H,), float("nan"), device="cuda")
        for _ in range(2):
            K.mb200_moe_block_local(d_r, d_e[lo * stride:], stride, g, u, 14, NE, lo, hi - lo, k, H, EFF, d_x,
                                    d_res if rank == 0 else zero, part, ids, wts, act, scratch)
        assert np.array_equal(host(ids), i_ref)
        assert torch.isfinite(part).all()
        total += part.double()
    got = host(total)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3


def test_host_buffer_block_matches_device_block(K):
    """HostMoEBlock (pinned host buffers in and out, every call: the device reads and writes them in place) against
    ResidentMoE.forward, in every form of the block; the same buffer reused with new contents (nothing may be served
    from a cache); and the C entry point with pageable buffers (copy-engine path)."""
    import ctypes as C
    from mnemocuda_b200 import _lib
    from mnemocuda_b200.moe import HostMoEBlock, MoEShape, ResidentMoE
    shape = MoEShape(n_experts=16)
    moe = ResidentMoE(shape, 2, "cuda", seed=3)
    hb = HostMoEBlock(moe)
    H = shape.H
    xr = torch.empty(2, H).pin_memory()
    o = torch.empty(H).pin_memory()
    for mode in (2, 1, 0):
        K.mb200_set_fused(mode)
        for it in range(4):
            layer = it % 2
            xr.copy_(torch.from_numpy(np.stack([synth.normal_f32(100 + it, H), synth.normal_f32(200 + it, H)])))
            o.fill_(float("nan"))
            hb(layer, xr, o)
            want = torch.empty(H, device="cuda")
            moe.forward(layer, xr[0].cuda(), xr[1].cuda(), want)
            torch.cuda.synchronize()
            assert torch.equal(o, want.cpu()), (mode, it)
    K.mb200_set_fused(2)
    # pageable host memory through the C ABI
    s = shape
    x_np = np.stack([synth.normal_f32(300, H), synth.normal_f32(301, H)]).astype(np.float32)
    out_np = np.full(H, np.nan, np.float32)
    rc = _lib.lib().mb200_moe_block_host(
        moe.router[0].data_ptr(), moe.experts[0].data_ptr(), s.stride, s.gate_sz, s.up_sz, s.down_type, s.NE, 0, 0, s.K,
        s.H, s.EFF, x_np.ctypes.data_as(C.c_void_p), out_np.ctypes.data_as(C.c_void_p), hb.io.data_ptr(),
        moe.ids[0].data_ptr(), moe.wts[0].data_ptr(), moe.act.data_ptr(), moe.scratch.data_ptr(),
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    want = torch.empty(H, device="cuda")
    moe.forward(0, torch.from_numpy(x_np[0]).cuda(), torch.from_numpy(x_np[1]).cuda(), want)
    torch.cuda.synchronize()
    assert np.array_equal(out_np, want.cpu().numpy())
    assert K.mb200_device_error() == 0


@pytest.mark.parametrize("pdl", [False, True])
def test_block_at_the_benchmark_shape_all_forms(K, pdl):
    """The timed configuration itself: 128 experts, top-8, hidden 4096, intermediate 1536, Q6_K down, in
    all three forms of mb200_moe_block, with and without programmatic dependent launch, two calls in a
    row each, against the oracle. The layer is written on the device (as the benchmark does) and copied
    to the host for the oracle."""
    from mnemocuda_b200.moe import MoEShape, ResidentMoE
    shape = MoEShape()  # 128 experts, top-8, 4096, 1536, Q6_K down
    s = shape
    moe = ResidentMoE(shape, 1, "cuda", seed=5)
    experts = moe.experts[0].reshape(-1).cpu().numpy()
    router = moe.router[0].reshape(-1).cpu().numpy()
    prev = K.mb200_set_pdl(pdl)
    try:
        for trial, (sx, sr) in enumerate(((61, 62), (63, 64))):
            x, res = synth.normal_f32(sx, s.H), synth.normal_f32(sr, s.H)
            want, i_ref, w_ref = oracle.moe_block(router, experts, s.stride, s.gate_sz, s.up_sz, s.down_type, s.NE, s.K,
                                                  s.H, s.EFF, x, res)
            d_x, d_res = dev(x), dev(res)
            for mode in (2, 1, 0):
                K.mb200_set_fused(mode)
                out = torch.full((s.H,), float("nan"), device="cuda")
                for _ in range(2):
                    moe.forward(0, d_x, d_res, out)
                torch.cuda.synchronize()
                assert np.array_equal(host(moe.ids[0]), i_ref), (mode, trial)
                np.testing.assert_allclose(host(moe.wts[0]), w_ref, rtol=1e-5, atol=1e-7)
                got = host(out).astype(np.float64)
                rel = np.linalg.norm(got - want) / np.linalg.norm(want)
                assert rel <= 1e-3, (mode, trial, rel)
                rel_moe = np.linalg.norm((got - res) - (want.astype(np.float64) - res)) / np.linalg.norm(want.astype(np.float64) - res)
                assert rel_moe <= 1e-3, (mode, trial, rel_moe)
    finally:
        K.mb200_set_fused(2)
        K.mb200_set_pdl(prev)
    assert K.mb200_device_error() == 0


@pytest.mark.parametrize("NE,k,H,EFF", [(128, 8, 4096, 1536), (16, 8, 2048, 768)])
def test_block_with_the_rmsnorm_folded_in(K, NE, k, H, EFF):
    """mb200_moe_block_norm (the pre-FFN norm inside the block) against the oracle's norm followed by its block,
    in every form (the one-launch form normalises on the fly, the others run the norm kernel first)."""
    from mnemocuda_b200.moe import MoEShape, ResidentMoE
    s = MoEShape(n_experts=NE, top_k=k, hidden=H, eff=EFF)
    moe = ResidentMoE(s, 1, "cuda", seed=9)
    experts = moe.experts[0].reshape(-1).cpu().numpy()
    router = moe.router[0].reshape(-1).cpu().numpy()
    x, res = synth.normal_f32(71, H, 4.0), synth.normal_f32(72, H)
    nw = (1 + 0.1 * synth.normal_f32(73, H)).astype(np.float32)
    xn = oracle.rms_norm(x, nw, 1e-6)
    want, i_ref, w_ref = oracle.moe_block(router, experts, s.stride, s.gate_sz, s.up_sz, s.down_type, NE, k, H, EFF, xn, res)
    d_x, d_res, d_nw = dev(x), dev(res), dev(nw)
    tmp = torch.empty(H, device="cuda")
    try:
        for mode in (2, 1, 0):
            K.mb200_set_fused(mode)
            out = torch.full((H,), float("nan"), device="cuda")
            for _ in range(2):
                K.mb200_moe_block_norm(moe.router[0], moe.experts[0], s.stride, s.gate_sz, s.up_sz, s.down_type, NE, 0, NE, k, H,
                                       EFF, d_x, d_nw, 1e-6, tmp, d_res, out, moe.ids[0], moe.wts[0], moe.act, moe.scratch)
            torch.cuda.synchronize()
            assert np.array_equal(host(moe.ids[0]), i_ref), mode
            got = host(out).astype(np.float64)
            assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3, mode
    finally:
        K.mb200_set_fused(2)
    assert K.mb200_device_error() == 0


def test_block_with_its_allreduce_inside_on_a_world_of_one(K):
    """mb200_moe_block_push with a communicator of one rank (the rows are pushed into this GPU's own receive
    cells and collected from there): the same bits as mb200_moe_block, eagerly, twice in a row (the two
    buffer halves) and replayed from a CUDA graph; the aliasing a decode layer uses (out = x = residual) works;
    shapes the one-launch form does not cover are refused with nothing launched."""
    from mnemocuda_b200.moe import MoEShape, ResidentMoE
    from mnemocuda_b200.peer import PeerComm
    s = MoEShape(n_experts=32)
    moe = ResidentMoE(s, 1, "cuda", seed=9)
    comm = PeerComm(0, 1, 8192)
    try:
        x, res = dev(synth.normal_f32(61, s.H)), dev(synth.normal_f32(62, s.H))
        want = torch.empty(s.H, device="cuda")
        moe.forward(0, x, res, want)
        ids_want = moe.ids[0].clone()
        call = lambda xx, rr, oo: K.mb200_moe_block_push(moe.router[0], moe.experts[0], s.stride, s.gate_sz, s.up_sz,
                                                        s.down_type, s.NE, 0, s.NE, s.K, s.H, s.EFF, xx, None, 0.0, rr, oo,
                                                        moe.ids[0], moe.wts[0], moe.act, moe.scratch, comm._comm)
        for _ in range(3):
            got = torch.full((s.H,), float("nan"), device="cuda")
            assert call(x, res, got)
            torch.cuda.synchronize()
            assert torch.equal(got, want)
            assert torch.equal(moe.ids[0], ids_want)
        h = x.clone()  # in place, as the hidden state of a decode layer
        assert call(h, h, h)
        torch.cuda.synchronize()
        want2 = torch.empty(s.H, device="cuda")
        moe.forward(0, x, x, want2)
        torch.cuda.synchronize()
        assert torch.equal(h, want2)
        got = torch.empty(s.H, device="cuda")
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            call(x, res, got)
        for _ in range(3):
            got.zero_()
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(got, want)
        # a shape outside the one-launch form (hidden 1024): refused, nothing launched
        s2 = MoEShape(n_experts=8, top_k=2, hidden=1024, eff=256)
        moe2 = ResidentMoE(s2, 1, "cuda", seed=10)
        x2 = dev(synth.normal_f32(63, s2.H))
        out2 = torch.full((s2.H,), 7.0, device="cuda")
        assert not K.mb200_moe_block_push(moe2.router[0], moe2.experts[0], s2.stride, s2.gate_sz, s2.up_sz, s2.down_type,
                                          s2.NE, 0, s2.NE, s2.K, s2.H, s2.EFF, x2, None, 0.0, x2, out2, moe2.ids[0],
                                          moe2.wts[0], moe2.act, moe2.scratch, comm._comm)
        torch.cuda.synchronize()
        assert torch.all(out2 == 7.0)
    finally:
        comm.close()
    assert K.mb200_device_error() == 0
