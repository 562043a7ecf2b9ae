"""CUDA glue kernels and flash-decode attention against the oracle."""
import math

import numpy as np
import pytest

import oracle_lib as O
from gpu_util import assert_bits, assert_close, need_gpu

pytestmark = pytest.mark.gpu


def _cuda(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_rmsnorm_and_silu_mul():
    torch = need_gpu()
    import cera_b200 as cb
    rng = np.random.default_rng(0)
    for n in (32, 4096, 14336):
        x = rng.standard_normal(n).astype(np.float32) * 3
        w = rng.standard_normal(n).astype(np.float32)
        got = cb.rmsnorm(_cuda(torch, x), _cuda(torch, w), 1e-5).cpu().numpy()
        want = O.rmsnorm(x, w, 1e-5)
        # f64 partial sums are combined in a different order: equal or one ulp of `inv` apart
        assert np.allclose(got, want, rtol=2e-7, atol=0)
        g = rng.standard_normal(n).astype(np.float32) * 4
        u = rng.standard_normal(n).astype(np.float32)
        assert_bits(cb.silu_mul(_cuda(torch, g), _cuda(torch, u)).cpu().numpy(), O.silu_mul(g, u), "silu_mul")


@pytest.mark.parametrize("n", [32, 1024, 4096, 8192, 14336])
def test_rmsnorm_with_fused_quantizer(n):
    """The normed vector and its Q8_0 form from one launch: the quantizer bytes are those of the
    stand-alone quantizer applied to the same f32 values."""
    torch = need_gpu()
    import cera_b200 as cb
    x = O.synth_normal(n, 31, 2.0)
    w = O.synth_normal(n, 32, 1.0)
    out, acts = cb.rmsnorm_q8_0(_cuda(torch, x), _cuda(torch, w), 1e-5)
    want = O.rmsnorm(x, w, 1e-5)
    assert np.allclose(out.cpu().numpy(), want, rtol=2e-7, atol=0)
    s, q = O.quantize_q8_0(out.cpu().numpy())
    assert_bits(acts.scales.cpu().numpy(), s, "scales")
    assert np.array_equal(acts.quants.cpu().numpy(), q)
    assert np.array_equal(acts.sums.cpu().numpy().astype(np.int32), q.astype(np.int32).reshape(-1, 16).sum(axis=1))


@pytest.mark.parametrize("rope_type", [0, 1])
@pytest.mark.parametrize("pos", [0, 1, 511, 32767])
def test_rope(rope_type, pos):
    torch = need_gpu()
    import cera_b200 as cb
    rng = np.random.default_rng(pos)
    nh, nkv, hd = 32, 8, 128
    q = rng.standard_normal(nh * hd).astype(np.float32)
    k = rng.standard_normal(nkv * hd).astype(np.float32)
    gq, gk = cb.rope(_cuda(torch, q), _cuda(torch, k), pos, nh, nkv, hd, 500000.0, rope_type=rope_type)
    wq, wk = O.rope(q, k, pos, nh, nkv, hd, 500000.0, rope_type=rope_type)
    assert_close(gq.cpu().numpy(), wq, "q")
    assert_close(gk.cpu().numpy(), wk, "k")


def test_rope_freq_factors():
    torch = need_gpu()
    import cera_b200 as cb
    rng = np.random.default_rng(3)
    nh, nkv, hd = 4, 2, 64
    q = rng.standard_normal(nh * hd).astype(np.float32)
    k = rng.standard_normal(nkv * hd).astype(np.float32)
    ff = (1.0 + rng.random(hd // 2) * 7).astype(np.float32)
    gq, gk = cb.rope(_cuda(torch, q), _cuda(torch, k), 77, nh, nkv, hd, 10000.0, _cuda(torch, ff))
    wq, wk = O.rope(q, k, 77, nh, nkv, hd, 10000.0, ff)
    assert_close(gq.cpu().numpy(), wq)
    assert_close(gk.cpu().numpy(), wk)


def _attn_case(torch, cb, nh, nkv, hd, seq, f16, seed):
    kv_dim = nkv * hd
    kc = cb.synth_normal(seq * kv_dim, seed=seed, sigma=1.0).reshape(seq, kv_dim)
    vc = cb.synth_normal(seq * kv_dim, seed=seed + 1, sigma=1.0).reshape(seq, kv_dim)
    q = cb.synth_normal(nh * hd, seed=seed + 2, sigma=1.0)
    scale = 1.0 / math.sqrt(hd)
    if f16:
        kc, vc = kc.half(), vc.half()
        kh, vh = kc.cpu().numpy().view(np.uint16), vc.cpu().numpy().view(np.uint16)
    else:
        kh, vh = kc.cpu().numpy(), vc.cpu().numpy()
    got = cb.decode_attention(q, kc, vc, nh, nkv, hd, seq, scale).cpu().numpy()
    want = O.decode_attention(q.cpu().numpy(), kh, vh, nh, nkv, hd, seq, scale)
    assert_close(got, want, f"seq={seq} f16={f16}")


@pytest.mark.parametrize("f16", [False, True])
@pytest.mark.parametrize("seq", [1, 7, 8, 63, 65, 512, 1000, 4096])
def test_decode_attention_llama_shape(seq, f16):
    torch = need_gpu()
    import cera_b200 as cb
    _attn_case(torch, cb, 32, 8, 128, seq, f16, seed=100 + seq)


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 64), (16, 2, 128), (8, 1, 64)])
def test_decode_attention_other_groupings(nh, nkv, hd):
    torch = need_gpu()
    import cera_b200 as cb
    _attn_case(torch, cb, nh, nkv, hd, 300, False, seed=7)


@pytest.mark.parametrize("seq,f16", [(16384, False), (32768, False), (32768, True)])
def test_decode_attention_long_context(seq, f16):
    torch = need_gpu()
    import cera_b200 as cb
    _attn_case(torch, cb, 32, 8, 128, seq, f16, seed=5)


@pytest.mark.parametrize("f16", [False, True])
@pytest.mark.parametrize("nh,nkv,hd,seq", [(32, 8, 128, 4097), (32, 8, 128, 5000), (32, 8, 128, 8191), (16, 2, 128, 4500),
                                           (8, 2, 64, 6000), (16, 2, 64, 4200)])
def test_decode_attention_streamed_kernel(nh, nkv, hd, seq, f16):
    """The online-softmax split kernel that stages K/V through shared memory with cp.async (the path long
    contexts take when the reference-order kernels are switched off): ragged last tiles, splits with no whole
    tile, both KV widths, head_dim 64 / 128 and groups of 4 / 8; the kernel status word must stay clear."""
    torch = need_gpu()
    import cera_b200 as cb
    from cera_b200._lib import kernel_status
    _attn_case(torch, cb, nh, nkv, hd, seq, f16, seed=40 + seq % 7)
    torch.cuda.synchronize()
    assert kernel_status() == 0


def test_decode_attention_rejects_unsupported_shapes():
    torch = need_gpu()
    import cera_b200 as cb
    # 18 query heads on 2 KV heads (a group of 9) with head_dim 48: no decode kernel covers it, and the call says so
    q = torch.zeros(18 * 48, device="cuda")
    kc = torch.zeros(4, 2 * 48, device="cuda")
    with pytest.raises(cb.CeraCudaError) as e:
        cb.decode_attention(q, kc, kc, 18, 2, 48, 4, 0.125)
    assert e.value.code == 2
    # a group of 3 is served (by the reference-order kernels): finite output of the right size
    q = torch.ones(6 * 64, device="cuda")
    kc = torch.ones(4, 2 * 64, device="cuda")
    out = cb.decode_attention(q, kc, kc, 6, 2, 64, 4, 0.125)
    assert out.shape[0] == 6 * 64 and bool(torch.isfinite(out).all())


@pytest.mark.parametrize("nh,nkv,n,start", [(32, 8, 256, 256), (32, 8, 256, 0), (8, 8, 33, 5), (8, 4, 9, 0), (16, 2, 41, 90),
                                             (4, 1, 1, 0), (4, 1, 1, 63)])
@pytest.mark.parametrize("f16", [False, True])
def test_prefill_attention_tiled_shapes(nh, nkv, n, start, f16):
    """The shared-memory-tiled kernel (f32 and f16 caches, head_dim 128, groups of 1 / 2 / 4 / 8): the 256-token chunk of the
    Llama-3-8B shape at both chunk positions, ragged query blocks, a single query, limits on and off tile boundaries."""
    torch = need_gpu()
    import cera_b200 as cb
    hd = 128
    total = start + n
    kc = cb.synth_normal(total * nkv * hd, seed=11, sigma=1.0).reshape(total, nkv * hd)
    vc = cb.synth_normal(total * nkv * hd, seed=12, sigma=1.0).reshape(total, nkv * hd)
    q = cb.synth_normal(n * nh * hd, seed=13, sigma=1.0).reshape(n, nh * hd)
    scale = 1.0 / math.sqrt(hd)
    kk, vv = (kc.half(), vc.half()) if f16 else (kc, vc)
    got = cb.prefill_attention(q, kk, vv, nh, nkv, hd, n, start, scale).cpu().numpy()
    qm = np.ascontiguousarray(q.cpu().numpy().T)
    want = O.flash_attention_gqa(qm, kk.float().cpu().numpy(), vv.float().cpu().numpy(), nh, nkv, hd, n, start, scale)
    want = np.ascontiguousarray(want.transpose(1, 0, 2)).reshape(n, nh * hd)
    assert_close(got, want, f"tiled prefill attention {nh}/{nkv} n={n} start={start} f16={f16}")


@pytest.mark.parametrize("f16", [False, True])
def test_prefill_attention_matches_flash_oracle(f16):
    torch = need_gpu()
    import cera_b200 as cb
    nh, nkv, hd, n, start = 8, 2, 128, 70, 37   # the reference's own flash test uses n=70, start_pos 37
    total = start + n
    kc = cb.synth_normal(total * nkv * hd, seed=1, sigma=1.0).reshape(total, nkv * hd)
    vc = cb.synth_normal(total * nkv * hd, seed=2, sigma=1.0).reshape(total, nkv * hd)
    q = cb.synth_normal(n * nh * hd, seed=3, sigma=1.0).reshape(n, nh * hd)
    scale = 1.0 / math.sqrt(hd)
    kk, vv = (kc.half(), vc.half()) if f16 else (kc, vc)
    got = cb.prefill_attention(q, kk, vv, nh, nkv, hd, n, start, scale).cpu().numpy()  # [n][nh*hd]
    kf, vf = kk.float().cpu().numpy(), vv.float().cpu().numpy()
    qm = np.ascontiguousarray(q.cpu().numpy().T)  # oracle layout: [q_dim x n]
    want = O.flash_attention_gqa(qm, kf, vf, nh, nkv, hd, n, start, scale)  # [nh][n][hd]
    want = np.ascontiguousarray(want.transpose(1, 0, 2)).reshape(n, nh * hd)
    assert_close(got, want, f"prefill attention f16={f16}")
