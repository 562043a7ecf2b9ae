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


# ---- model-level bars, the reference's own (cera/tests/llama_batched_prefill_parity.rs:74-147,
# cera/tests/gpu_transformer_parity.rs:168-238): a whole forward pass re-quantizes activations to
# int8 seven times per layer, so a last-ulp difference can flip one quant and move a logit by more
# than the per-operator tolerance.  The reference therefore holds whole-model outputs to a cosine
# floor and a top-1 decision that may differ only inside a tie window anchored on the reference.
COSINE_FLOOR = 0.9999        # FLOOR_TIGHT
TIE_TOP_K = 8
TIE_FRACTION_TIGHT = 2e-2
TIE_FRACTION_LOOSE = 6e-2  # paths whose reduction is tiled differently (cera/tests/llama_batched_prefill_parity.rs:130-141)
MIN_MATCH_PREFIX = 4


def cosine(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def top_k_spread(ref):
    top = np.sort(np.asarray(ref, dtype=np.float64))[-TIE_TOP_K:]
    return float(top[-1] - top[0])


def is_near_tie(ref_logits, pick_a, pick_b):
    """Both picks sit within the tie window of the reference's own logits."""
    ref = np.asarray(ref_logits, dtype=np.float64)
    return abs(ref[pick_a] - ref[pick_b]) <= TIE_FRACTION_TIGHT * top_k_spread(ref)


def assert_model_logits(got, want, what=""):
    got = np.asarray(got)
    want = np.asarray(want)
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    c = cosine(got, want)
    assert c >= COSINE_FLOOR, f"{what}: cosine {c:.6f} below {COSINE_FLOOR}"
    ga, wa = int(np.argmax(got)), int(np.argmax(want))
    assert ga == wa or is_near_tie(want, ga, wa), f"{what}: argmax {ga} vs {wa} is not a near-tie"


def compare_greedy_streams(gpu_stream, ref_stream, ref_logits_at):
    """Identical, or forked at a reference near-tie after at least MIN_MATCH_PREFIX tokens.
    Returns the number of matching leading tokens."""
    n = 0
    for g, r in zip(gpu_stream, ref_stream):
        if g != r:
            break
        n += 1
    if n == len(ref_stream):
        return n
    assert n >= MIN_MATCH_PREFIX, f"streams fork after {n} tokens: {gpu_stream[:n + 1]} vs {ref_stream[:n + 1]}"
    assert is_near_tie(ref_logits_at(n), gpu_stream[n], ref_stream[n]), (
        f"streams fork at {n} and the two picks are not a near-tie in the reference logits")
    return n
