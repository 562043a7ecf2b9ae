"""CUDA quantizer / GEMV / GEMM against the oracle.

Bit-exact: Q8_0 activation bytes and scales, per-half-block int32 sums.
Toleranced (1e-3 rel / 1e-4 abs): every f32 output.
"""
import numpy as np
import pytest

import oracle_lib as O
import ref_fixtures as R
from gpu_util import assert_bits, assert_close, need_gpu
from test_oracle_formats import _rand_block_bytes

pytestmark = pytest.mark.gpu


def _cuda(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_quantizer_bit_exact_incl_corner_blocks():
    torch = need_gpu()
    import cera_b200 as cb
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(4096) * 3).astype(np.float32)
    # corner blocks from cera/src/backend/simd.rs:7872-7946
    x[0:32] = 0.0
    for b, amax in enumerate((1e-30, 1e-38, 1e-40, 1e-44), start=1):
        x[32 * b:32 * b + 32] = 0.0
        x[32 * b], x[32 * b + 1], x[32 * b + 2] = amax, -amax, np.float32(amax) / np.float32(2)
    x[160:192] = 0.25
    x[160], x[161] = np.nan, -1.0
    x[192:224] = 0.25
    x[192], x[193] = np.inf, -1.0
    a = cb.quantize_q8_0(_cuda(torch, x))
    ws, wq = O.quantize_q8_0(x)
    assert_bits(a.quants.cpu().numpy(), wq, "quants")
    assert_bits(a.scales.cpu().numpy(), ws, "scales")
    sums = wq.astype(np.int32).reshape(-1, 16).sum(axis=1).astype(np.int16)
    assert_bits(a.sums.cpu().numpy(), sums, "sums")


def test_quantize_columns_matches_oracle():
    torch = need_gpu()
    import cera_b200 as cb
    rng = np.random.default_rng(1)
    dim, n = 256, 9
    mat = rng.standard_normal((dim, n)).astype(np.float32)
    a = cb.quantize_columns(_cuda(torch, mat), dim, n)
    ws, wq = O.quantize_columns(mat, dim, n)
    assert_bits(a.quants.cpu().numpy(), wq)
    assert_bits(a.scales.cpu().numpy(), ws)


@pytest.mark.parametrize("t", O.QUANT_TYPES)
def test_block_sums_bit_exact(t):
    torch = need_gpu()
    import cera_b200 as cb
    rng = np.random.default_rng(40 + t)
    m, k = 3, 1024
    raw = _rand_block_bytes(t, m, k, rng)
    if t == O.Q8_0:  # force the -128 weight extreme of the reference's fixtures
        raw.reshape(-1, 34)[:, 2:4] = 0x80
    aq = rng.integers(-127, 128, size=k, dtype=np.int8)
    aq[0:4] = (127, 127, -127, -127)
    w = cb.QuantWeight(t, m, k, raw)
    rb = O.row_bytes(t, k)
    for row in range(m):
        u, a = cb.block_sums(w, row, _cuda(torch, aq))
        wu, wa = O.block_sums(t, raw[row * rb:(row + 1) * rb], k, aq)
        assert_bits(u.cpu().numpy(), wu, f"{O.NAMES[t]} u row {row}")
        assert_bits(a.cpu().numpy(), wa, f"{O.NAMES[t]} a row {row}")


@pytest.mark.parametrize("t", O.QUANT_TYPES)
@pytest.mark.parametrize("m,k", [(7, 512), (1, 256), (33, 4096), (130, 1024)])
def test_gemv_matches_oracle(t, m, k):
    torch = need_gpu()
    import cera_b200 as cb
    rng = np.random.default_rng(1000 * t + m)
    w32 = O.synth_normal(m * k, seed=t * 7 + m, sigma=0.02)
    raw = O.quantize_weights(t, w32)
    x = rng.standard_normal(k).astype(np.float32)
    w = cb.QuantWeight(t, m, k, raw)
    got = cb.gemv(w, _cuda(torch, x)).cpu().numpy()
    if t == O.Q5_K:
        # the Q8_0-activation Q5_K kernel is an extension: oracle = restated integer form
        xs, xq = O.quantize_q8_0(x)
        want = O.gemm_preq(t, raw, xs, xq, m, 1, k).ravel()
    else:
        want = O.gemv(t, raw, x, m, k)
    assert_close(got, want, f"{O.NAMES[t]} {m}x{k}")


@pytest.mark.parametrize("t", O.QUANT_TYPES)
@pytest.mark.parametrize("m,k", [(64, 4096), (24, 14336), (128, 1024), (8, 2048), (5, 384), (37, 4096), (40, 11008 // 256 * 256)])
def test_gemv_rows_kernel_shapes(t, m, k):
    """Shapes that take the register-resident-activation kernel (k a multiple of 128), ragged m included,
    and rows shared by several warps (k = 14336)."""
    torch = need_gpu()
    import cera_b200 as cb
    if k % O.BLOCK[t][0]:
        pytest.skip("k is not a whole number of super-blocks for this format")
    w32 = cb.synth_normal(m * k, seed=31 * t + m, sigma=0.02)
    raw = cb.quantize_weights(t, w32).cpu().numpy()
    x = cb.synth_normal(k, seed=m + k, sigma=1.0)
    w = cb.QuantWeight(t, m, k, raw)
    got = cb.gemv(w, x).cpu().numpy()
    xh = x.cpu().numpy()
    if t == O.Q5_K:
        xs, xq = O.quantize_q8_0(xh)
        want = O.gemm_preq(t, raw, xs, xq, m, 1, k).ravel()
    else:
        want = O.gemv(t, raw, xh, m, k, avx2=O.has_avx2(), threads=4)
    assert_close(got, want, f"{O.NAMES[t]} {m}x{k}")


def test_gemv_q5k_f32_matches_reference_semantics():
    torch = need_gpu()
    import cera_b200 as cb
    m, k = 19, 1024
    raw = O.quantize_weights(O.Q5_K, O.synth_normal(m * k, seed=5, sigma=0.02))
    x = np.random.default_rng(5).standard_normal(k).astype(np.float32)
    w = cb.QuantWeight(O.Q5_K, m, k, raw)
    got = cb.gemv_q5k_f32(w, _cuda(torch, x)).cpu().numpy()
    assert_close(got, O.gemv(O.Q5_K, raw, x, m, k), "q5_k f32 activations")
    # and the Q8_0 extension agrees with it up to activation-quantisation noise
    ext = cb.gemv(w, _cuda(torch, x)).cpu().numpy()
    assert np.abs(ext - got).max() < 0.02 * np.abs(got).max()


def test_config1_q4_0_gemv_4096():
    """The reference's CPU-runnable benchmark case: W 4096x4096 N(0,0.02) seed 0 -> Q4_0, x N(0,1) seed 1."""
    torch = need_gpu()
    import cera_b200 as cb
    m = k = 4096
    w32 = cb.synth_normal(m * k, seed=0, sigma=0.02)
    raw = cb.quantize_weights(O.Q4_0, w32)
    x = cb.synth_normal(k, seed=1, sigma=1.0)
    w = cb.QuantWeight(O.Q4_0, m, k, raw)
    got = cb.gemv(w, x).cpu().numpy()
    want = O.gemv(O.Q4_0, raw.cpu().numpy(), x.cpu().numpy(), m, k, avx2=O.has_avx2(), threads=4)
    assert_close(got, want, "config 1")


@pytest.mark.parametrize("t", O.QUANT_TYPES)
@pytest.mark.parametrize("n", [1, 2, 3, 5, 8, 9, 17])
def test_gemm_preq_matches_oracle(t, n):
    torch = need_gpu()
    import cera_b200 as cb
    m, k = 21, 512
    raw = O.quantize_weights(t, O.synth_normal(m * k, seed=t + 100 * n, sigma=0.02))
    X = np.random.default_rng(n).standard_normal((n, k)).astype(np.float32)
    acts = cb.quantize_q8_0(_cuda(torch, X), k=k, n=n)
    w = cb.QuantWeight(t, m, k, raw)
    out = torch.full((m, n), float("nan"), device="cuda")  # poison: unwritten cells must show
    got = cb.gemm_preq(w, acts, out).cpu().numpy()
    bs, bq = O.quantize_columns(X.T.copy(), k, n)
    want = O.gemm_preq(t, raw, bs, bq, m, n, k)
    assert_close(got, want, f"{O.NAMES[t]} n={n}")


@pytest.mark.parametrize("t", [O.Q4_K, O.Q6_K, O.Q5_K, O.Q4_0])
@pytest.mark.parametrize("m,n,k", [(70, 130, 1024), (64, 128, 512), (200, 16, 768), (3, 64, 4096), (130, 5, 2048),
                                   (96, 8, 4096), (65, 33, 3072), (256, 100, 1024), (40, 17, 14336), (300, 390, 2048)])
def test_gemm_tensor_core_shapes(t, m, n, k):
    """n >= 5 and k a multiple of 256: the K-quants and Q4_0 take the mma.sync int8 kernel (every column-tile width, ragged tiles, and the k range
    split over clusters of 2, 4 and 8 CTAs)."""
    torch = need_gpu()
    import cera_b200 as cb
    raw = cb.quantize_weights(t, cb.synth_normal(m * k, seed=9 * t + m + n, sigma=0.02)).cpu().numpy()
    X = cb.synth_normal(n * k, seed=n + k, sigma=1.0)
    acts = cb.quantize_q8_0(X, k=k, n=n)
    w = cb.QuantWeight(t, m, k, raw)
    out = torch.full((m, n), float("nan"), device="cuda")
    got = cb.gemm_preq(w, acts, out).cpu().numpy()
    want = O.gemm_preq(t, raw, acts.scales.cpu().numpy(), acts.quants.cpu().numpy(), m, n, k, avx2=t != O.Q5_K, threads=4)
    assert_close(got, want, f"{O.NAMES[t]} {m}x{n}x{k}")
    # the same through the resident f16 operand image of the tcgen05 kernels (the K-quants, k a multiple of 256; Q6_K
    # reaches the tensor-core kernel only through its image)
    has = w.prepare_gemm()
    assert has == (t in (O.Q4_K, O.Q5_K, O.Q6_K) and k % 256 == 0)
    if has:
        out2 = torch.full((m, n), float("nan"), device="cuda")
        assert_close(cb.gemm_preq(w, acts, out2).cpu().numpy(), want, f"{O.NAMES[t]} {m}x{n}x{k} (weight image)")


def test_gemm_on_reference_fixtures():
    """The reference's own extreme fixtures (-128 weights, +/-127 activations)."""
    torch = need_gpu()
    import cera_b200 as cb
    k = 128
    for m, n in [(9, 7), (8, 8), (3, 2), (16, 5)]:
        rng = R.Lcg(0x77AA33CC)
        q4 = R.q4_0_rows(m, k, rng)
        q8 = R.q8_0_rows_with_extremes(m, k, rng)
        bs, bq = R.activations(n, k, rng)
        acts = cb.Q8Activations(k, n)
        acts.scales.copy_(_cuda(torch, bs))
        acts.quants.copy_(_cuda(torch, bq))
        acts.sums.copy_(_cuda(torch, bq.astype(np.int32).reshape(-1, 16).sum(axis=1).astype(np.int16)))
        for t, raw, is4 in ((O.Q4_0, q4, True), (O.Q8_0, q8, False)):
            got = cb.gemm_preq(cb.QuantWeight(t, m, k, raw), acts).cpu().numpy()
            want = R.ref_gemm(raw, bs, bq, m, n, k, is4)
            assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 1.0)), (t, m, n)


def test_operand_image_is_built_once_and_accounted():
    """cera_cuda_weight_prepare_gemm: about 2.3 bytes per weight for Q4_K / Q5_K, 4 for Q6_K, reported by weight_info;
    a second call changes nothing; types and shapes outside the tensor-core kernels get none."""
    need_gpu()
    import cera_b200 as cb
    m, k = 256, 2048
    for t, per_weight in ((O.Q4_K, 2.0), (O.Q5_K, 2.0), (O.Q6_K, 4.0)):
        w = cb.QuantWeight(t, m, k, cb.quantize_weights(t, cb.synth_normal(m * k, seed=3, sigma=0.02)))
        before = w.device_bytes()
        assert w.prepare_gemm()
        grown = w.device_bytes() - before
        assert per_weight * m * k <= grown <= (per_weight + 0.35) * m * k, (t, grown)
        assert w.prepare_gemm() and w.device_bytes() - before == grown
        w.close()
    for t, kk in ((O.Q4_0, 2048), (O.Q8_0, 2048), (O.Q4_1, 1024)):
        w = cb.QuantWeight(t, 64, kk, cb.quantize_weights(t, cb.synth_normal(64 * kk, seed=4, sigma=0.02)))
        before = w.device_bytes()
        assert not w.prepare_gemm() and w.device_bytes() == before
        w.close()


def test_gemm_preq_declines_loudly():
    torch = need_gpu()
    import cera_b200 as cb
    raw = O.quantize_weights(O.Q4_0, O.synth_normal(4 * 64, seed=1, sigma=0.02))
    w = cb.QuantWeight(O.Q4_0, 4, 64, raw)
    acts = cb.quantize_q8_0(torch.zeros(128, device="cuda"), k=128, n=1)
    with pytest.raises(cb.CeraCudaError):
        cb.gemm_preq(w, acts)


def test_tma_staged_gemv_in_its_own_process():
    """The opt-in TMA-staged GEMV (CERA_CUDA_GEMV=tma is read once per process) against the oracle,
    and its bounded waits must not have run out."""
    need_gpu()
    import os
    import subprocess
    import sys
    code = r"""
import sys, numpy as np
sys.path.insert(0, 'tests')
import oracle_lib as O, cera_b200 as cb
from cera_b200 import _lib
for t, m, k in ((O.Q4_K, 64, 4096), (O.Q6_K, 24, 14336), (O.Q4_0, 128, 1024), (O.Q8_0, 32, 2048), (O.Q5_K, 48, 4096), (O.Q4_1, 16, 4096)):
    raw = cb.quantize_weights(t, cb.synth_normal(m * k, 3 * t + m, 0.02)).cpu().numpy()
    x = cb.synth_normal(k, m + k, 1.0)
    got = cb.gemv(cb.QuantWeight(t, m, k, raw), x).cpu().numpy()
    xs, xq = O.quantize_q8_0(x.cpu().numpy())
    want = O.gemm_preq(t, raw, xs, xq, m, 1, k).ravel()
    assert np.all(np.abs(got - want) <= 1e-4 + 1e-3 * np.abs(want)), (t, m, k, np.abs(got - want).max())
assert _lib.kernel_status() == 0
print('tma ok')
"""
    env = dict(os.environ, CERA_CUDA_GEMV="tma")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "tma ok" in r.stdout, r.stdout + r.stderr
