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
