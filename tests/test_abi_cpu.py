"""No-GPU checks of the boundary: the shared library builds/loads and exports
every symbol include/mnemo_b200.h declares; the host mirror validates arguments."""
import ctypes

import numpy as np
import pytest

from mnemocuda_b200 import _lib, build, synth


def test_library_builds_and_loads():
    path = build.build()
    assert path.endswith("libmnemo_b200.so")
    _lib.lib()


def test_every_declared_symbol_is_exported_and_bound():
    declared = _lib.declared_symbols()
    assert len(declared) >= 22
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    for name in _lib.SIGNATURES:
        assert name in declared, f"{name} bound but not declared in include/mnemo_b200.h"


def test_reference_abi_names_present():
    """The hot-path entry points the reference's forward.c imports (src/forward.c:24-152)."""
    hot = ["cuda_kernels_init", "cuda_matvec_q4k", "cuda_matvec_q4k_add", "cuda_matvec_q4k_qkv",
           "cuda_matvec_q4k_dual", "cuda_matvec_q4k_scaled_add", "cuda_matvec_q6k", "cuda_matvec_f32",
           "cuda_topk_softmax", "cuda_swiglu", "cuda_scaled_add"]
    declared = set(_lib.declared_symbols())
    assert set(hot) <= declared


def test_host_mirror_rejects_cpu_tensors():
    import torch
    from mnemocuda_b200 import kernels
    with pytest.raises(ValueError):
        kernels.cuda_matvec_q4k(torch.zeros(144, dtype=torch.uint8), torch.zeros(256), torch.zeros(1), 1, 256, stream=0)


def test_synth_distributions_and_sizes():
    b = synth.q4k_blocks(1, 4000)
    assert b.shape == (4000, 144)
    d = b[:, :4].copy().view(np.float16).astype(np.float64)
    assert (d >= 0).all() and abs(d.mean() - 2e-3 * np.sqrt(2 / np.pi)) < 1e-4
    nib = np.concatenate([b[:, 16:] & 15, b[:, 16:] >> 4]).ravel()
    assert abs(nib.mean() - 7.5) < 0.05
    q = synth.q6k_blocks(2, 4000)
    assert q.shape == (4000, 210)
    sc = q[:, 192:208].view(np.int8)
    assert sc.min() == -32 and sc.max() == 31
    assert synth.expert_sizes(4096, 1536) == (3538944, 3538944, 5160960)
    # slices of a stream are independent of where generation starts
    assert np.array_equal(synth.q4k_blocks(3, 10, first_block=5), synth.q4k_blocks(3, 15)[5:])
    assert np.array_equal(synth.q6k_blocks(3, 10, first_block=5), synth.q6k_blocks(3, 15)[5:])
