"""Pins the oracle's int8 kernels, quantizer and glue with the reference's tests.

Restates cera/src/backend/simd.rs:6584-6743 (integer reference, GEMV and GEMM),
7017-7103 (GEMV == GEMM at n=1), 7113-7213 (K-quant and Q4_1 against a
dequantize-then-dot f64 reference), 7872-7946 (quantizer corner blocks),
cera/src/backend/cpu.rs:6074-6189 (rmsnorm / softmax / expf), and
cera/src/model/lfm2.rs:3619-3720 (routing).
"""
import math

import numpy as np
import pytest

import oracle_lib as O
import ref_fixtures as R

SHAPES = [(9, 7), (8, 8), (3, 2), (16, 5)]


@pytest.mark.parametrize("avx2", [False, True])
def test_gemm_matches_integer_reference(avx2):
    if avx2 and not O.has_avx2():
        pytest.skip("host has no AVX2")
    k = 128
    for m, n in SHAPES:
        rng = R.Lcg(0x77AA33CC)
        q4 = R.q4_0_rows(m, k, rng)
        q8 = R.q8_0_rows_with_extremes(m, k, rng)
        bs, bq = R.activations(n, k, rng)
        for t, w, is4 in ((O.Q4_0, q4, True), (O.Q8_0, q8, False)):
            got = O.gemm_preq(t, w, bs, bq, m, n, k, avx2=avx2)
            want = R.ref_gemm(w, bs, bq, m, n, k, is4)
            assert np.abs(got).max() > 0
            assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 1.0)), (m, n, t)


@pytest.mark.parametrize("avx2", [False, True])
def test_gemv_matches_integer_reference(avx2):
    if avx2 and not O.has_avx2():
        pytest.skip("host has no AVX2")
    k = 128
    for m in (1, 3, 8, 9, 16):
        rng = R.Lcg(0x22446688)
        q4 = R.q4_0_rows(m, k, rng)
        q8 = R.q8_0_rows_with_extremes(m, k, rng)
        xs, xq = R.activations(1, k, rng)
        for t, w, is4 in ((O.Q4_0, q4, True), (O.Q8_0, q8, False)):
            got = O.gemm_preq(t, w, xs, xq, m, 1, k, avx2=avx2)
            want = R.ref_gemm(w, xs, xq, m, 1, k, is4)
            assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 1.0))


def _dequant_reference(t, w, bs, bq, m, n, k):
    rb = O.row_bytes(t, k)
    out = np.zeros((m, n), dtype=np.float64)
    for i in range(m):
        wf = O.dequantize(t, w[i * rb:(i + 1) * rb], k)
        for j in range(n):
            xa = np.repeat(bs[j * (k // 32):(j + 1) * (k // 32)], 32) * bq[j * k:(j + 1) * k].astype(np.float32)
            out[i, j] = (wf * xa.astype(np.float32)).astype(np.float64).sum()
    return out


@pytest.mark.parametrize("avx2", [False, True])
def test_k_quant_gemm_matches_dequant_reference(avx2):
    if avx2 and not O.has_avx2():
        pytest.skip("host has no AVX2")
    m, k = 3, 512
    rng = R.Lcg(0x9F1E2D3C)
    q4k, q6k = R.k_quant_rows(m, k // 256, rng)
    for n in (5, 1):
        bs, bq = R.activations(n, k, rng)
        for t, w in ((O.Q4_K, q4k), (O.Q6_K, q6k)):
            got = O.gemm_preq(t, w, bs, bq, m, n, k, avx2=avx2).astype(np.float64)
            want = _dequant_reference(t, w, bs, bq, m, n, k)
            assert np.all(np.abs(got - want) <= 1e-5 * (1.0 + np.abs(want))), (t, n)


@pytest.mark.parametrize("avx2", [False, True])
def test_gemm_q4_1_matches_dequant_reference(avx2):
    if avx2 and not O.has_avx2():
        pytest.skip("host has no AVX2")
    m, n, k = 3, 11, 512
    rng = R.Lcg(0x04517B3D)
    w = R.q4_1_rows(m, k, rng)
    bs, bq = R.activations(n, k, rng)
    got = O.gemm_preq(O.Q4_1, w, bs, bq, m, n, k, avx2=avx2).astype(np.float64)
    want = _dequant_reference(O.Q4_1, w, bs, bq, m, n, k)
    assert np.all(np.abs(got - want) <= 1e-5 * (1.0 + np.abs(want)))


def test_q5_k_extension_matches_dequant_reference():
    # No reference kernel exists for Q5_K x Q8_0: this is the only pin it has.
    import test_oracle_formats as F
    m, n, k = 3, 5, 512
    rng = np.random.default_rng(5)
    w = F._rand_block_bytes(O.Q5_K, m, k, rng)
    lcg = R.Lcg(0x5555)
    bs, bq = R.activations(n, k, lcg)
    got = O.gemm_preq(O.Q5_K, w, bs, bq, m, n, k).astype(np.float64)
    want = _dequant_reference(O.Q5_K, w, bs, bq, m, n, k)
    assert np.all(np.abs(got - want) <= 1e-5 * (1.0 + np.abs(want)))


def test_avx2_build_is_bit_identical_to_scalar_restatement():
    if not O.has_avx2():
        pytest.skip("host has no AVX2")
    import test_oracle_formats as F
    rng = np.random.default_rng(11)
    for t in (O.Q4_0, O.Q8_0, O.Q4_1, O.Q4_K, O.Q6_K):
        for (m, n) in ((9, 7), (3, 1), (70, 5), (130, 1)):
            k = 512
            w = F._rand_block_bytes(t, m, k, rng)
            lcg = R.Lcg(0xABCDEF + t)
            bs, bq = R.activations(n, k, lcg)
            a = O.gemm_preq(t, w, bs, bq, m, n, k, avx2=False)
            b = O.gemm_preq(t, w, bs, bq, m, n, k, avx2=True, threads=4)
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), (t, m, n)


def test_vnni_build_is_bit_identical_to_avx2_and_scalar():
    """cera/src/backend/simd.rs:7216-7286 holds the AVX-512 VNNI tier bit-identical to the AVX2 one; so does this
    restatement (vpdpbusd against maddubs + madd on the reference's fixtures, extreme bytes included)."""
    if not O.has_vnni():
        pytest.skip("host has no AVX-512 VNNI + VL")
    import test_oracle_formats as F
    rng = np.random.default_rng(12)
    for t in (O.Q4_0, O.Q8_0, O.Q4_1, O.Q4_K, O.Q6_K):
        for (m, n) in ((9, 7), (3, 1), (70, 5), (130, 1)):
            k = 512
            w = F._rand_block_bytes(t, m, k, rng)
            if t == O.Q8_0:
                w.reshape(-1, 34)[:, 2:4] = 0x80  # the -128 weight extreme
            lcg = R.Lcg(0x13579B + t)
            bs, bq = R.activations(n, k, lcg)
            a = O.gemm_preq(t, w, bs, bq, m, n, k, avx2=False)
            b = O.gemm_preq(t, w, bs, bq, m, n, k, avx2=True, threads=2)
            c = O.gemm_preq(t, w, bs, bq, m, n, k, avx2="vnni", threads=2)
            assert np.array_equal(a.view(np.uint32), c.view(np.uint32)), (t, m, n)
            assert np.array_equal(b.view(np.uint32), c.view(np.uint32)), (t, m, n)


# simd.rs:7017-7103: the GEMV entry is the GEMM at n == 1, bit for bit.
def test_gemv_is_gemm_at_n1():
    import test_oracle_formats as F
    rng = np.random.default_rng(3)
    k, m = 512, 7
    x = rng.standard_normal(k).astype(np.float32)
    xs, xq = O.quantize_q8_0(x)
    for t in (O.Q4_0, O.Q8_0, O.Q4_1, O.Q4_K, O.Q6_K):
        w = F._rand_block_bytes(t, m, k, rng)
        a = O.gemv(t, w, x, m, k)
        b = O.gemm_preq(t, w, xs, xq, m, 1, k).ravel()
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        assert np.abs(a).max() > 0


# ---- Q8_0 activation quantizer -------------------------------------------

def test_quantizer_zero_block():
    s, q = O.quantize_q8_0(np.zeros(64, dtype=np.float32))
    assert np.all(s == 0) and np.all(q == 0)


def test_quantizer_corner_blocks():
    for amax in (1e-30, 1e-38, 1e-40, 1e-44, float("nan")):
        x = np.zeros(32, dtype=np.float32)
        x[0], x[1], x[2] = amax, -amax, np.float32(amax) / np.float32(2)
        s, q = O.quantize_q8_0(x)
        assert np.all(q != -128) or s[0] == 0.0
        assert not np.isnan(s[0])
    x = np.full(32, 0.25, dtype=np.float32)
    x[0], x[1] = np.nan, -1.0
    s, q = O.quantize_q8_0(x)
    assert q[0] == 0 and q[1] == -127 and q[2] == 32
    x[0] = np.inf
    s, q = O.quantize_q8_0(x)
    assert np.isinf(s[0]) and np.all(q == 0)


def test_quantizer_matches_formula():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(4096) * 3).astype(np.float32)
    s, q = O.quantize_q8_0(x)
    xb = x.reshape(-1, 32)
    amax = np.abs(xb).max(axis=1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    assert np.array_equal(s, d.astype(np.float16).astype(np.float32))
    idv = (np.float32(1.0) / d).astype(np.float32)
    want = np.clip(np.rint(xb * idv[:, None]), -128, 127).astype(np.int8)
    assert np.array_equal(q.reshape(-1, 32), want)


def test_quantize_columns_is_per_column_quantize():
    rng = np.random.default_rng(1)
    dim, n = 128, 5
    mat = rng.standard_normal((dim, n)).astype(np.float32)
    s, q = O.quantize_columns(mat, dim, n)
    for j in range(n):
        sj, qj = O.quantize_q8_0(mat[:, j].copy())
        assert np.array_equal(s[j * (dim // 32):(j + 1) * (dim // 32)], sj)
        assert np.array_equal(q[j * dim:(j + 1) * dim], qj)


# ---- weight quantizers: round trip error bounds ---------------------------

@pytest.mark.parametrize("t,tol", [(O.Q8_0, 0.006), (O.Q4_0, 0.13), (O.Q4_1, 0.07), (O.Q4_K, 0.09),
                                   (O.Q5_K, 0.05), (O.Q6_K, 0.05)])
def test_weight_quantizer_round_trip(t, tol):
    w = O.synth_normal(8 * 1024, seed=42, sigma=0.02)
    raw = O.quantize_weights(t, w)
    back = O.dequantize(t, raw, w.size)
    err = np.abs(back - w).max()
    assert err <= tol * np.abs(w).max(), err
    assert np.isfinite(back).all()


def test_synth_normal_moments():
    x = O.synth_normal(1 << 18, seed=1, sigma=1.0)
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1.0) < 0.01
    y = O.synth_normal(1000, seed=1, sigma=1.0, offset=1000)
    assert np.array_equal(x[1000:2000], y)


# ---- glue -----------------------------------------------------------------

def test_expf_tracks_libm():
    for v in np.linspace(-80, 80, 4001):
        got = O.expf(float(np.float32(v)))
        want = math.exp(float(np.float32(v)))
        assert abs(got - want) <= 3e-7 * want + 1e-38
    assert O.expf(-200.0) == 0.0 and math.isinf(O.expf(200.0))


def test_rmsnorm_and_softmax():
    rng = np.random.default_rng(2)
    x = rng.standard_normal(256).astype(np.float32)
    w = rng.standard_normal(256).astype(np.float32)
    got = O.rmsnorm(x, w, 1e-5)
    inv = np.float32(1.0 / math.sqrt(float((x.astype(np.float64) ** 2).mean()) + float(np.float32(1e-5))))
    assert np.array_equal(got, (x * inv) * w)
    p = O.softmax(x)
    assert abs(float(p.sum()) - 1.0) < 1e-5 and p.argmax() == x.argmax()


def test_rope_norm_rotates_adjacent_pairs():
    hd = 8
    q = np.arange(hd, dtype=np.float32) + 1
    k = q.copy()
    q0, _ = O.rope(q, k, 0, 1, 1, hd, 10000.0)
    assert np.array_equal(q0, q)  # pos 0 is the identity
    q1, k1 = O.rope(q, k, 3, 1, 1, hd, 10000.0)
    ts = np.float32(10000.0) ** np.float32(-2.0 / hd)
    theta = np.float32(3.0)
    for i in range(hd // 2):
        c, s = math.cos(float(theta)), math.sin(float(theta))
        assert abs(q1[2 * i] - (q[2 * i] * c - q[2 * i + 1] * s)) < 1e-5
        assert abs(q1[2 * i + 1] - (q[2 * i] * s + q[2 * i + 1] * c)) < 1e-5
        theta = np.float32(theta * ts)
    assert np.array_equal(q1, k1)
    qn, _ = O.rope(q, k, 3, 1, 1, hd, 10000.0, rope_type=1)
    assert abs(qn[0] - (q[0] * math.cos(3.0) - q[hd // 2] * math.sin(3.0))) < 1e-5


def test_flash_prefill_matches_naive_decode_attention():
    rng = np.random.default_rng(4)
    nh, nkv, hd, n, start = 4, 2, 16, 37, 5
    total = start + n
    kc = rng.standard_normal((total, nkv * hd)).astype(np.float32)
    vc = rng.standard_normal((total, nkv * hd)).astype(np.float32)
    qm = rng.standard_normal((nh * hd, n)).astype(np.float32)
    out = O.flash_attention_gqa(qm, kc, vc, nh, nkv, hd, n, start, 0.25)
    for j in (0, 17, n - 1):
        ref = O.decode_attention(qm[:, j].copy(), kc, vc, nh, nkv, hd, start + j + 1, 0.25).reshape(nh, hd)
        assert np.allclose(out[:, j, :], ref, rtol=1e-4, atol=1e-5)


def test_argmax_first_strict_max():
    assert O.argmax(np.array([1.0, 5.0, 5.0, 2.0], dtype=np.float32)) == 1
    assert O.argmax(np.array([np.nan, np.nan], dtype=np.float32)) == 0


# ---- routing (lfm2.rs:3619-3720) -------------------------------------------

def test_bias_ranks_experts_but_does_not_weight_them():
    ids, w = O.select_experts([0.40, 0.30, 0.05, 0.01], [0.0, 0.5, 0.0, 0.0], 2)
    assert list(ids) == [1, 0]
    assert abs(w[0] - 0.30 / 0.70) < 1e-6 and abs(w[1] - 0.40 / 0.70) < 1e-6 and w[0] < w[1]


def test_matches_llama_cpp_non_monotonic_token():
    probs = np.zeros(32, dtype=np.float32)
    bias = np.zeros(32, dtype=np.float32)
    probs[21], probs[17], probs[6], probs[12] = 0.3474, 0.3556, 0.1866, 0.1103
    bias[21] = 0.10
    ids, w = O.select_experts(probs, bias, 4)
    assert list(ids) == [21, 17, 6, 12]
    assert np.all(np.abs(w - np.array([0.3474, 0.3556, 0.1866, 0.1103])) < 1e-3)


def test_routing_ties_zero_gate_and_saturation():
    ids, _ = O.select_experts([0.25] * 4, [0.0] * 4, 2)
    assert list(ids) == [0, 1]
    _, w = O.select_experts([0.0] * 4, [0.0] * 4, 2)
    assert np.isfinite(w).all()
    ids, w = O.select_experts([0.5, 0.3], [0.0, 0.0], 8)
    assert list(ids) == [0, 1] and len(w) == 2


def _cpu_llama(cfg, seed, kv_f16=0, max_seq_len=32):
    """A small random-init llama on the oracle alone (CPU synthetic generator and weight quantizers)."""
    m = O.OracleModel(**cfg, max_seq_len=max_seq_len, kv_f16=kv_f16, n_threads=1)
    hs, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qd, kvd = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"]
    ones = np.ones(hs, dtype=np.float32)

    def mat(role, layer, rows, cols, t=O.Q8_0):
        raw = O.quantize_weights(t, O.synth_normal(rows * cols, seed * 131 + role * 17 + layer, 0.05))
        m.set_tensor(role, layer, t, rows, cols, raw)

    mat(0, 0, cfg["vocab_size"], hs)
    mat(2, 0, cfg["vocab_size"], hs)
    m.set_tensor(1, 0, O.F32, 1, hs, ones)
    for l in range(cfg["n_layers"]):
        m.set_tensor(3, l, O.F32, 1, hs, ones)
        m.set_tensor(8, l, O.F32, 1, hs, ones)
        mat(4, l, qd, hs)
        mat(5, l, kvd, hs)
        mat(6, l, kvd, hs)
        mat(7, l, hs, qd)
        mat(9, l, ff, hs)
        mat(10, l, ff, hs)
        mat(11, l, hs, ff)
    return m


@pytest.mark.parametrize("rope_type", [0, 1])
@pytest.mark.parametrize("kv_f16", [0, 1])
def test_kv_shift_of_a_one_layer_model_equals_the_shorter_sequence(rope_type, kv_f16):
    """cera/src/kv_cache.rs:1091-1320.  In a one-layer model a cached K / V row depends only on (token, position),
    so dropping positions [n_keep, n_keep+shift) and re-rotating the keys that moved must leave the cache of the
    sequence that never had those tokens: R(-shift) R(p) k = R(p - shift) k up to f32 (f16) rounding."""
    cfg = dict(n_layers=1, hidden_size=64, intermediate_size=128, n_heads=4, n_kv_heads=2, head_dim=32, vocab_size=96,
               rope_theta=10000.0, rms_norm_eps=1e-5, rope_type=rope_type)
    toks = [5, 17, 80, 3, 44, 9, 61, 23, 70]
    a = _cpu_llama(cfg, 3, kv_f16)
    for pos, t in enumerate(toks):
        a.forward(t, pos)
    a.shift_kv(2, 3)
    assert a.seq_len == len(toks) - 3
    b = _cpu_llama(cfg, 3, kv_f16)
    short = toks[:2] + toks[5:]
    for pos, t in enumerate(short):
        b.forward(t, pos)
    la, lb = a.forward(11, a.seq_len), b.forward(11, b.seq_len)
    tol = 2e-2 if kv_f16 else 2e-4
    assert np.abs(la - lb).max() <= tol * np.abs(lb).max()
    # the reference's assertion cases
    assert O._lib.cera_oracle_model_shift_kv(a.h, 1, 0) == -1
    assert O._lib.cera_oracle_model_shift_kv(a.h, a.seq_len, 1) == -1


def test_lora_apply_known_answers():
    """cera/src/lora.rs:1198-1215: B = 0 is a no-op whatever the scale; with A = B = 1 every output moves by
    rank * scale * sum(x); a zero scale leaves y untouched bit for bit (no -0.0 -> +0.0 flip)."""
    rank, k, d = 4, 16, 6
    x = (np.arange(k, dtype=np.float32) - 3.0) * 0.25
    y0 = np.array([0.5, -0.0, 1.0, -2.0, 3.5, 0.0], dtype=np.float32)
    ones_a, ones_b = np.ones((rank, k), np.float32), np.ones((d, rank), np.float32)
    assert np.array_equal(O.lora_apply(ones_a, np.zeros((d, rank), np.float32), 2.0, x, y0), y0)
    got = O.lora_apply(ones_a, ones_b, 2.0, x, y0)
    assert np.allclose(got, y0 + rank * 2.0 * x.sum(), rtol=1e-6)
    assert np.array_equal(O.lora_apply(ones_a, ones_b, 0.0, x, y0).view(np.uint32), y0.view(np.uint32))
    # against the plain formula on random factors
    rng = np.random.default_rng(5)
    a, b = rng.standard_normal((rank, k)).astype(np.float32), rng.standard_normal((d, rank)).astype(np.float32)
    want = y0 + b.astype(np.float64) @ (0.5 * (a.astype(np.float64) @ x))
    assert np.allclose(O.lora_apply(a, b, 0.5, x, y0), want, rtol=1e-5, atol=1e-6)


def test_lora_changes_the_model_only_where_attached():
    cfg = dict(n_layers=2, hidden_size=64, intermediate_size=128, n_heads=4, n_kv_heads=2, head_dim=32, vocab_size=96,
               rope_theta=10000.0, rms_norm_eps=1e-5, rope_type=0)
    base, tuned, zero = _cpu_llama(cfg, 4), _cpu_llama(cfg, 4), _cpu_llama(cfg, 4)
    rng = np.random.default_rng(1)
    a = rng.standard_normal((4, 64)).astype(np.float32) * 0.1
    b = rng.standard_normal((64, 4)).astype(np.float32) * 0.1
    tuned.set_lora(3, 1, a, b, 2.0)                                   # o-proj of layer 1: 64 -> 64
    zero.set_lora(3, 1, a, np.zeros_like(b), 2.0)
    for pos, t in enumerate([7, 50, 3]):
        lb, lt, lz = base.forward(t, pos), tuned.forward(t, pos), zero.forward(t, pos)
    assert np.array_equal(lb, lz)
    assert np.abs(lb - lt).max() > 1e-4


@pytest.mark.parametrize("hd,kv_f16", [(128, 0), (64, 1), (72, 0), (12, 0)])
def test_decode_attention_vector_order_against_a_float64_reference(hd, kv_f16):
    """Decode attention restates the reference's x86 dispatch (cera/src/backend/cpu.rs:3264-3290): for head sizes
    that are a multiple of 8 (up to 256) the AVX2+FMA lane order, the scalar loops otherwise (hd = 12).  Both are
    held to a float64 evaluation of the same softmax(q.K) V, like the reference's own SIMD-against-scalar tests
    (cpu.rs:6750-7250), and the lane order is checked by hand on one score."""
    rng = np.random.default_rng(hd)
    nh, nkv, seq = 4, 2, 37
    kv_dim = nkv * hd
    q = rng.standard_normal(nh * hd).astype(np.float32)
    kc = rng.standard_normal((seq, kv_dim)).astype(np.float32)
    vc = rng.standard_normal((seq, kv_dim)).astype(np.float32)
    if kv_f16:
        kc, vc = kc.astype(np.float16), vc.astype(np.float16)
    scale = np.float32(1.0 / np.sqrt(hd))
    got = O.decode_attention(q, kc.view(np.uint16) if kv_f16 else kc, vc.view(np.uint16) if kv_f16 else vc, nh, nkv, hd, seq,
                             float(scale)).reshape(nh, hd)
    k64, v64, q64 = kc.astype(np.float64), vc.astype(np.float64), q.astype(np.float64).reshape(nh, hd)
    for h in range(nh):
        off = (h // (nh // nkv)) * hd
        s = (k64[:, off:off + hd] @ q64[h]) * float(scale)
        p = np.exp(s - s.max())
        want = (p / p.sum()) @ v64[:, off:off + hd]
        assert np.abs(got[h] - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    if hd % 8 == 0 and not kv_f16:
        # one score by hand in the AVX2 order: two 8-lane FMA chains over alternating slices, added, hsum256
        def fma(a, b, c):
            return np.float32(np.float64(a) * np.float64(b) + np.float64(c))
        s0, s1 = np.zeros(8, np.float32), np.zeros(8, np.float32)
        nv, i = hd // 8, 0
        while i + 2 <= nv:
            for L in range(8):
                s0[L] = fma(q[8 * i + L], kc[0, 8 * i + L], s0[L])
                s1[L] = fma(q[8 * (i + 1) + L], kc[0, 8 * (i + 1) + L], s1[L])
            i += 2
        if i < nv:
            for L in range(8):
                s0[L] = fma(q[8 * i + L], kc[0, 8 * i + L], s0[L])
        s = s0 + s1
        lo = np.array([s[0] + s[4], s[1] + s[5], s[2] + s[6], s[3] + s[7]], np.float32)
        score = np.float32(np.float32(np.float32(lo[0] + lo[2]) + np.float32(lo[1] + lo[3])) * scale)
        one = O.decode_attention(q, kc[:1].copy(), vc[:1].copy(), nh, nkv, hd, 1, float(scale)).reshape(nh, hd)
        # a single position: softmax weight is exactly 1, so the output is the value row; the score itself is
        # observable through a two-position softmax below
        assert np.array_equal(one[0], vc[0, :hd])
        two = O.decode_attention(q, kc[:2].copy(), vc[:2].copy(), nh, nkv, hd, 2, float(scale)).reshape(nh, hd)
        assert np.isfinite(two).all() and np.isfinite(score)


def test_host_synthetic_model_matches_the_device_generator_spec():
    """tests/oracle_lib.py and cera_b200/synth.py name the same seeds, roles, tensor mix and prompt hash."""
    from cera_b200 import synth
    from cera_b200.model import Role
    assert synth.LLAMA3_8B == O.LLAMA3_8B
    for name, idx in O.ROLE.items():
        assert int(getattr(Role, name)) == idx
    for role, t in synth.DEFAULT_TYPES.items():
        assert O.DEFAULT_TYPES[role.name] == int(t)
    for seed, role, layer in ((0, 4, 0), (3, 11, 31), (12345, 2, 7)):
        assert synth.tensor_seed(seed, role, layer) == O.tensor_seed(seed, role, layer)
    assert np.array_equal(synth.prompt_tokens(50, 128256, 7), O.prompt_tokens(50, 128256, 7))
