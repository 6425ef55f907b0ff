"""Multi-GPU runs of the sharded path, one process per GPU over NCCL + the push collectives
(tests/multi_rank_worker.py). Skipped on a box with a single GPU; CPU ranks (gloo) cover the host logic
in tests/test_sharding_cpu.py."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_path_on_real_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29500 + world), os.path.join(ROOT, "tests", "multi_rank_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    for r in range(world):
        assert f"RANK {r} OK" in res.stdout


def test_one_process_drives_two_devices():
    """The reference engine is ONE process that switches devices per layer range (src/forward.c:606). Attributes,
    SM counts and scratch addresses of this library are per device: after initialising on device 0, the streaming
    matvecs, the one-launch MoE block and the static-scratch router run on device 1 (initialised lazily for the
    matvecs, explicitly for the rest) and match the oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import numpy as np
    from mnemocuda_b200 import kernels as K, synth
    from mnemocuda_b200.moe import MoEShape, ResidentMoE
    from oracle import oracle
    from tests.gpu_util import assert_close_matvec, host
    torch.cuda.set_device(0)
    K.mb200_init()
    try:
        torch.cuda.set_device(1)
        rows, cols = 1024, 4096
        w4, w6 = synth.q4k_matrix(61, rows, cols), synth.q6k_matrix(62, rows, cols)
        x = synth.normal_f32(63, cols)
        d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to("cuda:1")
        y = torch.full((rows,), float("nan"), device="cuda:1")
        K.cuda_matvec_q4k(d(w4), d(x), y, rows, cols)  # no init on this device yet: attributes are set on first use
        _, y64, ad = oracle.matvec_q4k(w4, x, rows, cols, full=True)
        assert_close_matvec(host(y), y64, ad, "q4k on device 1")
        K.mb200_init()  # what an engine does once per device it drives
        K.cuda_matvec_q6k(d(w6), d(x), y, rows, cols)
        _, y64, ad = oracle.matvec_q6k(w6, x, rows, cols, full=True)
        assert_close_matvec(host(y), y64, ad, "q6k on device 1")
        shape = MoEShape(n_experts=16)
        moe = ResidentMoE(shape, 1, "cuda:1", seed=5)
        xs, res = d(synth.normal_f32(64, shape.H)), d(synth.normal_f32(65, shape.H))
        out = torch.empty(shape.H, device="cuda:1")
        moe.forward(0, xs, res, out)
        torch.cuda.synchronize()
        want, ids, _ = oracle.moe_block(host(moe.router[0]).reshape(-1), host(moe.experts[0]).reshape(-1), shape.stride,
                                        shape.gate_sz, shape.up_sz, shape.down_type, shape.NE, shape.K, shape.H, shape.EFF,
                                        host(xs), host(res))
        assert np.array_equal(host(moe.ids[0]), ids)
        got = host(out).astype(np.float64)
        assert np.linalg.norm(got - want) <= 1e-3 * np.linalg.norm(want)
        assert K.mb200_device_error() == 0
        # and device 0 still works afterwards
        torch.cuda.set_device(0)
        d0 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to("cuda:0")
        y0 = torch.full((rows,), float("nan"), device="cuda:0")
        K.cuda_matvec_q4k(d0(w4), d0(x), y0, rows, cols)
        _, y64, ad = oracle.matvec_q4k(w4, x, rows, cols, full=True)
        assert_close_matvec(host(y0), y64, ad, "q4k back on device 0")
    finally:
        torch.cuda.set_device(0)
