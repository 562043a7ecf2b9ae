"""Shared helpers for the GPU parity tests."""
import numpy as np
import pytest

RTOL, ATOL = 1e-3, 1e-4  # the path's stated f32 bar: 1e-3 relative / 1e-4 absolute


def need_gpu():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import cera_b200  # noqa: F401  raises if libcera_cuda.so is missing: no silent fallback
    return torch


def assert_close(got, want, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    assert np.abs(want).max() > 0, f"{what}: reference is all zeros"
    err = np.abs(got - want)
    bad = err > ATOL + RTOL * np.abs(want)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance, max err {err.max():.3e}"


def assert_bits(got, want, what=""):
    got = np.ascontiguousarray(got)
    want = np.ascontiguousarray(want)
    assert got.shape == want.shape and got.dtype == want.dtype, (got.shape, want.shape, got.dtype, want.dtype)
    if not np.array_equal(got.view(np.uint8), want.view(np.uint8)):
        idx = np.flatnonzero(got.reshape(-1) != want.reshape(-1))
        raise AssertionError(f"{what}: {idx.size} of {got.size} elements differ, first at {idx[:5]}: "
                             f"{got.reshape(-1)[idx[:5]]} vs {want.reshape(-1)[idx[:5]]}")
