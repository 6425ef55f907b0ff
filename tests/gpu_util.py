"""Helpers shared by the GPU parity tests (which call the kernels through the C ABI)."""
import numpy as np
import torch


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


# north_star tolerance: each output within 1e-3 relative L2 of the fp32 reference.
REL_L2_TOL = 1e-3


def assert_close_matvec(got: np.ndarray, want64: np.ndarray, abs_dot: np.ndarray | None = None, what=""):
    """Vector-level relative L2 <= 1e-3 against the fp64-accumulated oracle, plus a
    per-row bound |y - y_ref| <= 1e-3 * sum_c |w_rc x_c| when that scale is given."""
    got = got.astype(np.float64)
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    denom = np.linalg.norm(want64)
    err = np.linalg.norm(got - want64)
    if denom > 0:
        assert err / denom <= REL_L2_TOL, f"{what}: rel L2 {err / denom:.3e} > {REL_L2_TOL}"
    else:
        assert err == 0
    if abs_dot is not None:
        bound = REL_L2_TOL * abs_dot + 1e-30
        worst = np.max(np.abs(got - want64) / bound)
        assert worst <= 1.0, f"{what}: per-row error {worst:.3e} x the 1e-3*sum|w x| bound"
    return err / denom if denom > 0 else 0.0
