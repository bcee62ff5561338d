"""Helpers of the GPU parity tests: one shared context, numpy <-> device."""
import numpy as np
import torch

import ovk_b200

_CTX = None


def ctx() -> ovk_b200.Context:
    global _CTX
    if _CTX is None:
        _CTX = ovk_b200.Context(0)
    return _CTX


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    ctx().flush()
    return t.cpu().numpy()


def assert_close(got, want, atol, rtol, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    err = np.abs(got - want)
    bound = atol + rtol * np.abs(want)
    bad = err > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.size} outside atol={atol} rtol={rtol}; "
                           f"worst err {err.max():.3e} at {np.unravel_index(err.argmax(), err.shape)}")
