"""The K-quant GEMV / GEMM sweep at its real shapes: 4096x4096, 14336x4096 (gate / up), 4096x14336 (down)
for Q4_K, Q5_K and Q6_K, and the 128256x4096 Q6_K output head, at 1, 8, 64 and 512 activation columns,
CUDA path against the oracle (1e-3 relative / 1e-4 absolute on every output element).

Weights ~ N(0, 0.02) and activations ~ N(0, 1) come from the shared counter-based generator and the
reference's quantizer rules.  The oracle side runs the AVX2 build of the restated x86 kernels on all host
threads (bit-identical to the scalar restatement, see test_oracle_kernels.py); Q5_K has no such build, so
its scalar oracle is evaluated on a spread of rows.
"""
import os

import numpy as np
import pytest

import oracle_lib as O
from gpu_util import assert_close, need_gpu

pytestmark = pytest.mark.gpu

SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336)]
THREADS = os.cpu_count() or 4
_cache = {}


def _weights(cb, t, m, k):
    key = (t, m, k)
    if key not in _cache:
        _cache.clear()  # one matrix at a time: the head alone is 431 MB
        raw = cb.quantize_weights(t, cb.synth_normal(m * k, seed=7000 + 13 * t + m % 997 + k, sigma=0.02))
        _cache[key] = (cb.QuantWeight(t, m, k, raw), raw.cpu().numpy())
    return _cache[key]


def _check(cb, torch, t, m, k, n):
    w, raw = _weights(cb, t, m, k)
    X = cb.synth_normal(n * k, seed=n + k + t, sigma=1.0)
    acts = cb.quantize_q8_0(X, k=k, n=n)
    out = torch.full((m, n), float("nan"), device="cuda")
    if n == 1:
        got = cb.gemv(w, X).cpu().numpy().reshape(m, 1)  # the decode entry point: quantizes x itself
    else:
        got = cb.gemm_preq(w, acts, out).cpu().numpy()
    bs, bq = acts.scales.cpu().numpy(), acts.quants.cpu().numpy()
    if t == O.Q5_K:
        rows = np.unique(np.concatenate([np.arange(0, m, max(1, m // 24)), [m - 1]]))[:32 if n > 64 else 64]
        rb = O.row_bytes(t, k)
        sub = np.concatenate([raw[r * rb:(r + 1) * rb] for r in rows])
        want = O.gemm_preq(t, sub, bs, bq, len(rows), n, k)
        got = got[rows]
    else:
        want = O.gemm_preq(t, raw, bs, bq, m, n, k, avx2=True, threads=THREADS)
        rows = None
    assert_close(got, want, f"{O.NAMES[t]} {m}x{k} n={n}")
    if n == 512 and w.prepare_gemm():  # once more through the resident f16 operand image of the tcgen05 kernel
        got = cb.gemm_preq(w, acts, torch.full((m, n), float("nan"), device="cuda")).cpu().numpy()
        assert_close(got if rows is None else got[rows], want, f"{O.NAMES[t]} {m}x{k} n={n} (weight image)")


@pytest.mark.parametrize("n", [1, 8, 64, 512])
@pytest.mark.parametrize("m,k", SHAPES)
@pytest.mark.parametrize("t", [O.Q4_K, O.Q5_K, O.Q6_K])
def test_k_quant_sweep_full_shapes(t, m, k, n):
    torch = need_gpu()
    import cera_b200 as cb
    if not O.has_avx2():
        pytest.skip("the full-shape oracle needs the AVX2 build to finish in seconds")
    _check(cb, torch, t, m, k, n)


@pytest.mark.parametrize("n", [1, 8, 64, 512])
def test_output_head_q6k_128256x4096(n):
    torch = need_gpu()
    import cera_b200 as cb
    if not O.has_avx2():
        pytest.skip("the full-shape oracle needs the AVX2 build to finish in seconds")
    _check(cb, torch, O.Q6_K, 128256, 4096, n)
    if n == 512:
        _cache.clear()
