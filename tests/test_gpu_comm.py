"""Push collectives (mb200_push_allreduce / mb200_push_allgather) on one GPU: the single-rank case, replay
from a CUDA graph, argument checks, and the bounded wait -- a two-rank comm whose second rank never runs,
so the counter this rank waits for is never raised: the kernel must give up after its time budget, raise
the device error word and return, leaving the context usable. (Nothing here hangs or faults a GPU; the
real multi-rank runs are in tests/test_gpu_multi.py, one process per GPU.)"""
import ctypes as C

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


def test_single_rank_allreduce_and_allgather(K):
    from mnemocuda_b200.peer import PeerComm
    comm = PeerComm(0, 1, 8192)
    for n in (4096, 8192, 4, 100):
        x = dev(synth.normal_f32(n, n))
        out = torch.zeros(n, device="cuda")
        for _ in range(3):  # sequence numbers 1, 2, 3: both parities of the receive slots
            comm.allreduce(x, out)
        assert torch.equal(out, x)
        out.zero_()
        comm.allgather(x, out)
        assert torch.equal(out, x)
    assert K.mb200_device_error() == 0
    comm.close()


def test_collectives_replay_from_a_graph(K):
    from mnemocuda_b200.peer import PeerComm
    comm = PeerComm(0, 1, 4096)
    x = dev(synth.normal_f32(5, 4096))
    out = torch.zeros(4096, device="cuda")
    comm.allreduce(x, out)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        comm.allreduce(x, out)
        comm.allreduce(out, out)
    for i in range(3):
        x.fill_(float(i + 1))
        g.replay()
        torch.cuda.synchronize()
        assert float(out.min()) == float(out.max()) == float(i + 1)
    assert K.mb200_device_error() == 0
    comm.close()


def test_argument_checks(K):
    from mnemocuda_b200.peer import PeerComm
    comm = PeerComm(0, 1, 64)
    x = torch.zeros(128, device="cuda")
    with pytest.raises(RuntimeError):
        comm.allreduce(x, x)        # larger than the buffers
    y = torch.arange(6, dtype=torch.float32, device="cuda")
    out = torch.zeros(6, device="cuda")
    comm.allreduce(y, out)            # any length up to the buffer size
    assert torch.equal(out, y)
    comm.close()


def test_wait_for_a_rank_that_never_arrives_times_out(K):
    """World of two built from raw pointers in this one process; only rank 0 ever launches."""
    from mnemocuda_b200 import _lib
    lib = _lib.lib()
    world, n = 2, 1024
    nbytes = lib.mb200_comm_buffer_bytes(world, n)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    bases = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
    comm = C.c_void_p()
    assert lib.mb200_comm_create_ptrs(0, world, n, bases, C.byref(comm)) == 0
    x = dev(synth.normal_f32(9, n))
    out = torch.full((n,), 7.0, device="cuda")
    assert K.mb200_device_error() == 0
    rc = lib.mb200_push_allreduce(comm, x.data_ptr(), out.data_ptr(), n, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert K.mb200_device_error() == 3  # MB200_ERR_TIMEOUT, after about two seconds
    assert float(out.min()) == 7.0  # nothing was written
    # rank 0's piece did reach "rank 1"'s buffer: cells (value, sequence number 1) of parity 1, source 0
    cells = bufs[1][: 2 * world * n * 8].view(torch.int32).reshape(2, world, n, 2)[1, 0]
    assert torch.equal(cells[:, 0].view(torch.float32), x) and bool((cells[:, 1] == 1).all())
    K.mb200_clear_device_error()
    assert K.mb200_device_error() == 0
    lib.mb200_comm_destroy(comm, 0)
    # the context is still usable
    y = torch.empty(8, device="cuda")
    K.cuda_matvec_f32(torch.ones(8, 4, device="cuda"), torch.ones(4, device="cuda"), y, 8, 4)
    assert float(y.sum()) == 32.0


def test_block_with_allreduce_inside_times_out_on_a_missing_rank(K):
    """The in-kernel all-reduce of mb200_moe_block_push with a world of two of which only rank 0 ever launches: the
    collecting warps give up after the bounded wait, the device error word reports it, nothing is written to `out`,
    rank 0's rows did reach the other buffer, and the context stays usable."""
    from mnemocuda_b200 import _lib
    from mnemocuda_b200.moe import MoEShape, ResidentMoE
    lib = _lib.lib()
    s = MoEShape(n_experts=16)
    moe = ResidentMoE(s, 1, "cuda", seed=12)
    world, n = 2, s.H
    nbytes = lib.mb200_comm_buffer_bytes(world, n)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    bases = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
    comm = C.c_void_p()
    assert lib.mb200_comm_create_ptrs(0, world, n, bases, C.byref(comm)) == 0
    x, res = dev(synth.normal_f32(19, s.H)), dev(synth.normal_f32(20, s.H))
    want = torch.empty(s.H, device="cuda")
    moe.forward(0, x, res, want)
    out = torch.full((s.H,), 7.0, device="cuda")
    assert K.mb200_device_error() == 0
    assert K.mb200_moe_block_push(moe.router[0], moe.experts[0], s.stride, s.gate_sz, s.up_sz, s.down_type, s.NE, 0, s.NE,
                                  s.K, s.H, s.EFF, x, None, 0.0, res, out, moe.ids[0], moe.wts[0], moe.act, moe.scratch,
                                  comm.value)
    assert K.mb200_device_error() == 3  # MB200_ERR_TIMEOUT, after about two seconds
    assert float(out.min()) == 7.0 and float(out.max()) == 7.0  # nothing was written
    cells = bufs[1][: 2 * world * n * 8].view(torch.int32).reshape(2, world, n, 2)[1, 0]
    assert bool((cells[:, 1] == 1).all()) and torch.equal(cells[:, 0].view(torch.float32), want)
    K.mb200_clear_device_error()
    assert K.mb200_device_error() == 0
    lib.mb200_comm_destroy(comm, 0)
    moe.scratch.zero_()  # the block's barrier counters are to be zeroed after a timeout
    got = torch.empty(s.H, device="cuda")
    moe.forward(0, x, res, got)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
