"""Decode kernels that reproduce the reference's f32 ARITHMETIC ORDER: their outputs must equal the oracle's
bit for bit, not merely within the path's tolerance.

Covered: the K-quant GEMV at one activation column (four round-robin 8-lane FMA accumulators, sequential min
term, hsum256 - cera/src/backend/simd.rs:5693-5878, 5988-6195), RMSNorm (cpu.rs:2479-2496), decode attention
in the x86 lane order (cpu.rs:3522-3625, 2617-2633), and a whole model wired from them whose logits must be
bit-identical to the oracle's at every position.
"""
import math

import numpy as np
import pytest

import oracle_lib as O
from gpu_util import assert_bits, need_gpu

pytestmark = pytest.mark.gpu


def _cuda(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("t", [O.Q4_K, O.Q5_K, O.Q6_K])
@pytest.mark.parametrize("m,k", [(64, 4096), (40, 14336), (33, 1024), (1, 2048), (300, 3072), (72, 512), (96, 3584), (16, 18944)])
def test_k_quant_gemv_bits(t, m, k):
    torch = need_gpu()
    import cera_b200 as cb
    raw = cb.quantize_weights(t, cb.synth_normal(m * k, seed=77 * t + m, sigma=0.02)).cpu().numpy()
    x = cb.synth_normal(k, seed=m + k, sigma=1.0)
    got = cb.gemv(cb.QuantWeight(t, m, k, raw), x).cpu().numpy()
    xh = x.cpu().numpy()
    if t == O.Q5_K:  # the Q8_0-activation Q5_K product is this build's extension of the Q4_K kernel: oracle = its restated form
        xs, xq = O.quantize_q8_0(xh)
        want = O.gemm_preq(t, raw, xs, xq, m, 1, k).ravel()
    else:
        want = O.gemv(t, raw, xh, m, k)
    assert np.abs(want).max() > 0
    assert_bits(got, want, f"{O.NAMES[t]} {m}x{k}")


@pytest.mark.parametrize("t,m,k", [(O.Q4_K, 4096, 4096), (O.Q4_K, 14336, 4096), (O.Q6_K, 4096, 14336)])
def test_layer_shape_gemv_bits(t, m, k):
    """The decode step's own shapes, all rows, against the AVX2 build of the oracle on every host thread."""
    torch = need_gpu()
    import os
    import cera_b200 as cb
    if not O.has_avx2():
        pytest.skip("needs the AVX2 build of the oracle")
    raw = cb.quantize_weights(t, cb.synth_normal(m * k, seed=5 + t, sigma=0.02))
    x = cb.synth_normal(k, seed=9, sigma=1.0)
    got = cb.gemv(cb.QuantWeight(t, m, k, raw), x).cpu().numpy()
    want = O.gemv(t, raw.cpu().numpy(), x.cpu().numpy(), m, k, avx2=True, threads=os.cpu_count() or 4)
    assert_bits(got, want, f"{O.NAMES[t]} {m}x{k}")


@pytest.mark.parametrize("n", [32, 256, 4096, 14336])
def test_rmsnorm_bits(n):
    torch = need_gpu()
    import cera_b200 as cb
    x = O.synth_normal(n, 31 + n, 2.0)
    w = O.synth_normal(n, 32, 1.0)
    assert_bits(cb.rmsnorm(_cuda(torch, x), _cuda(torch, w), 1e-5).cpu().numpy(), O.rmsnorm(x, w, 1e-5), "rmsnorm")
    out, _ = cb.rmsnorm_q8_0(_cuda(torch, x), _cuda(torch, w), 1e-5)
    assert_bits(out.cpu().numpy(), O.rmsnorm(x, w, 1e-5), "rmsnorm + q8")


@pytest.mark.parametrize("kv_f16", [0, 1])
@pytest.mark.parametrize("nh,nkv,hd,seq", [(32, 8, 128, 1), (32, 8, 128, 37), (32, 8, 128, 640), (32, 8, 128, 4096),
                                           (32, 8, 128, 5000), (16, 2, 64, 300), (8, 8, 128, 129), (8, 4, 96, 77)])
def test_decode_attention_bits(nh, nkv, hd, seq, kv_f16):
    torch = need_gpu()
    import cera_b200 as cb
    kv_dim = nkv * hd
    kc = cb.synth_normal(seq * kv_dim, seed=seq, sigma=1.0).reshape(seq, kv_dim)
    vc = cb.synth_normal(seq * kv_dim, seed=seq + 1, sigma=1.0).reshape(seq, kv_dim)
    q = cb.synth_normal(nh * hd, seed=seq + 2, sigma=1.0)
    if kv_f16:
        kc, vc = kc.half(), vc.half()
    scale = 1.0 / math.sqrt(hd)
    got = cb.decode_attention(q, kc, vc, nh, nkv, hd, seq, scale).cpu().numpy()
    kh = kc.cpu().numpy().view(np.uint16) if kv_f16 else kc.cpu().numpy()
    vh = vc.cpu().numpy().view(np.uint16) if kv_f16 else vc.cpu().numpy()
    want = O.decode_attention(q.cpu().numpy(), kh, vh, nh, nkv, hd, seq, scale)
    assert_bits(got, want, f"attention {nh}/{nkv} x {hd}, {seq} positions, f16={kv_f16}")


@pytest.mark.parametrize("kv_f16", [0, 1])
def test_model_logits_bit_identical_to_the_oracle(kv_f16):
    """A llama-architecture model whose matrices are K-quants with row lengths that are multiples of 512 runs every
    projection, norm, rotation and attention on reference-order kernels: logits equal the oracle's bits at every
    position, so the greedy stream cannot differ."""
    need_gpu()
    from cera_b200 import synth
    cfg = dict(n_layers=3, hidden_size=1024, intermediate_size=2048, n_heads=8, n_kv_heads=2, head_dim=128, vocab_size=2048,
               rope_theta=500000.0, rms_norm_eps=1e-5, rope_type=0)
    oracle = O.OracleModel(**cfg, max_seq_len=48, kv_f16=kv_f16, n_threads=4)
    gpu = synth.build_llama(cfg, seed=17, max_seq_len=48, kv_f16=kv_f16,
                            sink=lambda r, l, t, rows, cols, d: oracle.set_tensor(int(r), l, t, rows, cols, d))
    tok = 5
    for pos in range(40):
        lg, lo = gpu.forward(tok, pos), oracle.forward(tok, pos)
        assert_bits(lg, lo, f"logits at position {pos}")
        tok = int(O.argmax(lo))
    # the per-layer snapshot is the reference's StateSnapshot content: the oracle's key / value cache bytes
    snap = gpu.state_snapshot()
    assert snap["seq_len"] == 40 and len(snap["layers"]) == cfg["n_layers"]
    for l, (kd, vd) in enumerate(snap["layers"]):
        assert np.array_equal(kd, oracle.kv(l, 0)), f"k_data of layer {l}"
        assert np.array_equal(vd, oracle.kv(l, 1)), f"v_data of layer {l}"
    # restoring it into a truncated cache brings the next token's logits back, bit for bit
    want = gpu.forward(tok, 40)
    gpu.truncate_kv(0)
    gpu.restore_state(snap)
    assert_bits(gpu.forward(tok, 40), want, "logits after restore_state")
    with pytest.raises(Exception):  # half the bytes: a snapshot of the other element width
        bad = {"seq_len": snap["seq_len"], "layers": [(k[: k.size // 2], v[: v.size // 2]) for k, v in snap["layers"]]}
        gpu.restore_state(bad)
    gpu.close()


@pytest.mark.gpu
def test_granite_scalar_multipliers_bit_identical_to_the_oracle():
    """Granite's four scalars (cera/src/model/mod.rs:49-112: embedding, residual, attention, logit) are applied where
    cera/src/model/llama.rs applies them: decode logits equal the oracle's bits, the batched prompt path agrees within
    the GEMM tolerance, and the per-layer KV snapshot holds the oracle's K/V bytes."""
    need_gpu()
    from cera_b200 import synth
    cfg = dict(n_layers=2, hidden_size=1024, intermediate_size=2048, n_heads=8, n_kv_heads=2, head_dim=128, vocab_size=2048,
               rope_theta=10000.0, rms_norm_eps=1e-5, rope_type=0,
               embedding_scale=12.0, residual_scale=0.22, attention_scale=0.0078125, logit_scale=8.0)
    oracle = O.OracleModel(**cfg, max_seq_len=48, kv_f16=0, n_threads=4)
    gpu = synth.build_llama(cfg, seed=23, max_seq_len=48, kv_f16=0,
                            sink=lambda r, l, t, rows, cols, d: oracle.set_tensor(int(r), l, t, rows, cols, d))
    toks, tok = [], 9
    for pos in range(12):
        toks.append(tok)
        lg, lo = gpu.forward(tok, pos), oracle.forward(tok, pos)
        assert_bits(lg, lo, f"logits at position {pos}")
        tok = int(O.argmax(lo))
    # the same prompt through the batched kernels: same logits within the GEMM tolerance (1e-3 relative, 1e-4 absolute)
    gpu.truncate_kv(0)
    lb = gpu.forward_prefill(np.asarray(toks, dtype=np.uint32), 0)
    scale = float(np.abs(lo).max())
    assert float(np.abs(lb - lo).max()) <= 1e-3 * scale + 1e-4
    # identity scalars are a no-op: a model created with 1.0 everywhere equals one created with the fields left at 0
    gpu.close()
    cfg1 = dict(cfg, embedding_scale=1.0, residual_scale=1.0, attention_scale=0.0, logit_scale=1.0)
    cfg0 = {k: v for k, v in cfg.items() if not k.endswith("_scale")}
    a, b = synth.build_llama(cfg1, seed=23, max_seq_len=8), synth.build_llama(cfg0, seed=23, max_seq_len=8)
    assert_bits(a.forward(3, 0), b.forward(3, 0), "identity scalars")
    a.close()
    b.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name,cfg_over,types", [
    ("neox rope (qwen layout)", dict(rope_type=1), None),
    ("one query head per KV head", dict(n_heads=8, n_kv_heads=8), None),
    ("eight query heads per KV head, head size 64", dict(n_heads=16, n_kv_heads=2, head_dim=64), None),
    ("three query heads per KV head, rows of 1536", dict(n_heads=12, n_kv_heads=4), None),
    ("every matrix Q6_K", dict(), "q6_k"),
    ("mixed Q4_K / Q6_K attention, Q6_K feed-forward", dict(), "mixed"),
])
def test_model_variants_bit_identical_to_the_oracle(name, cfg_over, types):
    """The whole-model bit identity of the test above across the shapes and tensor-type mixes a llama-architecture GGUF
    brings: NEOX rotation (stand-alone rope kernel instead of the GEMV epilogue), group sizes 1 / 3 / 8, head size 64,
    and K-quant mixes (different types for q/k/v go through separate GEMVs)."""
    need_gpu()
    import cera_b200 as cb
    from cera_b200 import synth
    from cera_b200.model import Role
    cfg = dict(n_layers=2, hidden_size=1024, intermediate_size=2048, n_heads=8, n_kv_heads=2, head_dim=128, vocab_size=2048,
               rope_theta=10000.0, rms_norm_eps=1e-6, rope_type=0)
    cfg.update(cfg_over)
    tmap = None
    if types == "q6_k":
        tmap = {r: cb.Q6_K for r in (Role.TOKEN_EMBD, Role.OUTPUT, Role.ATTN_Q, Role.ATTN_K, Role.ATTN_V, Role.ATTN_OUTPUT,
                                     Role.FFN_GATE, Role.FFN_UP, Role.FFN_DOWN)}
    elif types == "mixed":
        tmap = {Role.ATTN_Q: cb.Q4_K, Role.ATTN_K: cb.Q6_K, Role.ATTN_V: cb.Q6_K, Role.FFN_GATE: cb.Q6_K, Role.FFN_UP: cb.Q6_K}
    oracle = O.OracleModel(**cfg, max_seq_len=32, kv_f16=0, n_threads=4)
    gpu = synth.build_llama(cfg, seed=31, max_seq_len=32, types=tmap,
                            sink=lambda r, l, t, rows, cols, d: oracle.set_tensor(int(r), l, t, rows, cols, d))
    tok = 11
    for pos in range(20):
        lg, lo = gpu.forward(tok, pos), oracle.forward(tok, pos)
        assert_bits(lg, lo, f"{name}: logits at position {pos}")
        tok = int(O.argmax(lo))
    gpu.close()
