"""The allocation-free router entry point (mb200_router_topk_static) against the regular one.

Some callers have no device memory left to lend and may not allocate: an engine that sized its
caches from all free memory at load, or a decode loop that must not allocate once it is serving.
For them the router's ticket + logits scratch lives inside the library. This test calls that entry
point through the C ABI twice in a row (the built-in array keeps the previous call's contents, so
the second call checks that stale state is harmless) and compares with mb200_router_topk, which
uses scratch the caller provides. It is collected last on purpose.
"""
import numpy as np
import pytest
import torch

from mnemocuda_b200 import synth
from tests.gpu_util import dev, host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from mnemocuda_b200 import kernels
    kernels.mb200_init()
    return kernels


def _reference_call(K, router, x, NE, H, k):
    n = K.mb200_router_scratch_bytes(NE)
    scratch = torch.zeros((n + 15) // 16 * 16, dtype=torch.uint8, device="cuda")
    ids = torch.empty(k, dtype=torch.int32, device="cuda")
    wts = torch.empty(k, device="cuda")
    K.mb200_router_topk(router, x, scratch, ids, wts, NE, H, k)
    return host(ids), host(wts)


def test_static_scratch_router_matches_regular_entry_point_twice(K):
    NE, H, k = 128, 4096, 8
    router = dev(synth.normal_f32(501, NE * H, H ** -0.5))
    for call, seed in enumerate((502, 503)):  # two calls in a row, different inputs
        x = dev(synth.normal_f32(seed, H))
        ids = torch.full((k,), -5, dtype=torch.int32, device="cuda")
        wts = torch.full((k,), float("nan"), device="cuda")
        K.mb200_router_topk_static(router, x, ids, wts, NE, H, k)
        want_ids, want_wts = _reference_call(K, router, x, NE, H, k)
        assert np.array_equal(host(ids), want_ids), f"call {call}"
        np.testing.assert_allclose(host(wts), want_wts, rtol=1e-5, atol=1e-7)


def test_static_scratch_router_after_a_different_shape(K):
    """A smaller problem right after a larger one: leftovers in the shared array must not leak in."""
    for NE, H, k, seed in ((512, 1024, 8, 511), (16, 512, 4, 512)):
        router = dev(synth.normal_f32(seed, NE * H, H ** -0.5))
        x = dev(synth.normal_f32(seed + 100, H))
        ids = torch.empty(k, dtype=torch.int32, device="cuda")
        wts = torch.empty(k, device="cuda")
        K.mb200_router_topk_static(router, x, ids, wts, NE, H, k)
        want_ids, want_wts = _reference_call(K, router, x, NE, H, k)
        assert np.array_equal(host(ids), want_ids)
        np.testing.assert_allclose(host(wts), want_wts, rtol=1e-5, atol=1e-7)


def test_static_scratch_router_refuses_oversize(K):
    NE, H, k = 1025, 64, 8
    router = torch.zeros(NE * H, device="cuda")
    x = torch.zeros(H, device="cuda")
    ids = torch.empty(k, dtype=torch.int32, device="cuda")
    wts = torch.empty(k, device="cuda")
    with pytest.raises(RuntimeError):
        K.mb200_router_topk_static(router, x, ids, wts, NE, H, k)


def test_static_scratch_router_allocates_nothing(K):
    """Free device memory is the same before and after the calls (outputs and inputs exist beforehand; the
    kernel's code is already loaded because the regular entry point, which launches the same kernel, ran)."""
    NE, H, k = 128, 4096, 8
    router = dev(synth.normal_f32(521, NE * H, H ** -0.5))
    x = dev(synth.normal_f32(522, H))
    ids = torch.empty(k, dtype=torch.int32, device="cuda")
    wts = torch.empty(k, device="cuda")
    want_ids, _ = _reference_call(K, router, x, NE, H, k)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        K.mb200_router_topk_static(router, x, ids, wts, NE, H, k)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    assert np.array_equal(host(ids), want_ids)


@pytest.mark.parametrize("pdl", [False, True])
def test_static_scratch_router_in_a_captured_graph(K, pdl):
    """Two calls captured in one CUDA graph (after an eager call, which is where the array's address is
    looked up), with and without programmatic dependent launch, replayed twice."""
    NE, H, k = 128, 2048, 8
    router = dev(synth.normal_f32(531, NE * H, H ** -0.5))
    xs = [dev(synth.normal_f32(532 + i, H)) for i in range(2)]
    ids = [torch.empty(k, dtype=torch.int32, device="cuda") for _ in range(2)]
    wts = [torch.empty(k, device="cuda") for _ in range(2)]
    want = [_reference_call(K, router, x, NE, H, k) for x in xs]
    prev = K.mb200_set_pdl(pdl)
    try:
        K.mb200_router_topk_static(router, xs[0], ids[0], wts[0], NE, H, k)  # eager first
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(2):
                K.mb200_router_topk_static(router, xs[i], ids[i], wts[i], NE, H, k)
        for _ in range(2):
            for t in ids:
                t.fill_(-1)
            g.replay()
            torch.cuda.synchronize()
            for i in range(2):
                assert np.array_equal(host(ids[i]), want[i][0])
                np.testing.assert_allclose(host(wts[i]), want[i][1], rtol=1e-5, atol=1e-7)
    finally:
        K.mb200_set_pdl(prev)
