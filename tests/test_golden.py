"""The committed golden vectors (tests/golden/quant_path.npz, written by tests/golden/make_golden.py) against the
oracle on CPU and against the CUDA path on a GPU."""
import os

import numpy as np
import pytest

import oracle_lib as O

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quant_path.npz"))
TYPES = {"q4_0": O.Q4_0, "q4_1": O.Q4_1, "q8_0": O.Q8_0, "q4_k": O.Q4_K, "q5_k": O.Q5_K, "q6_k": O.Q6_K}
M, K, N = 6, 512, 3


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32) if a.dtype == np.float32 else a


def test_oracle_reproduces_the_golden_file():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fresh = mod.build()
    assert set(fresh) == set(GOLD.files)
    for k in GOLD.files:
        assert np.array_equal(_bits(fresh[k]), _bits(GOLD[k])), k


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(TYPES))
def test_cuda_path_against_golden_matmul(name):
    from gpu_util import assert_bits, assert_close, need_gpu
    torch = need_gpu()
    import cera_b200 as cb
    t = TYPES[name]
    raw = GOLD[f"{name}_raw"]
    w = cb.QuantWeight(t, M, K, raw)
    assert_bits(cb.dequantize_rows(w).cpu().numpy().reshape(M, K), GOLD[f"{name}_dequant"], "dequantized rows")
    acts = cb.quantize_q8_0(torch.from_numpy(GOLD["x"]).cuda(), k=K, n=N)
    assert_bits(acts.scales.cpu().numpy(), GOLD["x_scales"], "Q8_0 scales")
    assert np.array_equal(acts.quants.cpu().numpy(), GOLD["x_quants"])
    u, a = cb.block_sums(w, 0, acts.quants[:K])
    assert np.array_equal(u.cpu().numpy(), GOLD[f"{name}_sums_u"]) and np.array_equal(a.cpu().numpy(), GOLD[f"{name}_sums_a"])
    out = torch.empty(M, N, device="cuda")
    assert_close(cb.gemm_preq(w, acts, out).cpu().numpy(), GOLD[f"{name}_gemm"], "gemm_preq")
    if name != "q5_k":  # the oracle's Q5_K GEMV is the reference's f32-activation form (its own entry point below)
        assert_close(cb.gemv(w, torch.from_numpy(GOLD["x"][:K]).cuda()).cpu().numpy().ravel(), GOLD[f"{name}_gemv"], "gemv")
    else:
        assert_close(cb.gemv_q5k_f32(w, torch.from_numpy(GOLD["x"][:K]).cuda()).cpu().numpy().ravel(), GOLD[f"{name}_gemv"], "gemv")


@pytest.mark.gpu
def test_cuda_path_against_golden_attention_and_glue():
    from gpu_util import assert_bits, assert_close, need_gpu
    torch = need_gpu()
    import cera_b200 as cb
    q = torch.from_numpy(GOLD["attn_q"]).cuda()
    for tag, kk, vv in (("f32", GOLD["attn_k"], GOLD["attn_v"]),
                        ("f16", GOLD["attn_k_f16"].view(np.float16), GOLD["attn_v_f16"].view(np.float16))):
        got = cb.decode_attention(q, torch.from_numpy(kk).cuda(), torch.from_numpy(vv).cuda(), 8, 2, 64, 37, 0.125)
        assert_close(got.cpu().numpy(), GOLD[f"attn_out_{tag}"], f"decode attention {tag}")
    g, u = torch.from_numpy(GOLD["glue_g"]).cuda(), torch.from_numpy(GOLD["glue_u"]).cuda()
    assert_bits(cb.silu_mul(g, u).cpu().numpy(), GOLD["glue_silu_mul"], "silu_mul")
    got = cb.rmsnorm(g, torch.from_numpy(GOLD["glue_norm_w"]).cuda(), 1e-5).cpu().numpy()
    assert np.allclose(got, GOLD["glue_rmsnorm"], rtol=2e-7, atol=0)
