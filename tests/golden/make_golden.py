"""Writes tests/golden/quant_path.npz: small seeded inputs of the quantized-matmul path with the outputs of the CPU
oracle (itself pinned by the reference's own test vectors, see tests/test_oracle_*.py).  The file anchors both sides:
the CPU suite checks that the oracle still reproduces it, the GPU suite checks the CUDA path against it.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as O  # noqa: E402

TYPES = {"q4_0": O.Q4_0, "q4_1": O.Q4_1, "q8_0": O.Q8_0, "q4_k": O.Q4_K, "q5_k": O.Q5_K, "q6_k": O.Q6_K}
M, K, N = 6, 512, 3


def build():
    out = {}
    x = O.synth_normal(N * K, 1, 1.0)
    scales, quants = O.quantize_q8_0(x)
    out["x"], out["x_scales"], out["x_quants"] = x, scales, quants
    for name, t in TYPES.items():
        w = O.synth_normal(M * K, 100 + t, 0.02)
        raw = O.quantize_weights(t, w)
        out[f"{name}_raw"] = raw
        out[f"{name}_dequant"] = O.dequantize(t, raw, K, rows=M)
        rb = O.row_bytes(t, K)
        u, a = O.block_sums(t, raw[:rb], K, quants[:K])
        out[f"{name}_sums_u"], out[f"{name}_sums_a"] = u, a
        out[f"{name}_gemm"] = O.gemm_preq(t, raw, scales, quants, M, N, K)
        out[f"{name}_gemv"] = O.gemv(t, raw, x[:K], M, K)
    # decode attention: 8 query / 2 KV heads of 64 over 37 positions, f32 and f16 caches
    nh, nkv, hd, seq = 8, 2, 64, 37
    kc = O.synth_normal(seq * nkv * hd, 7, 1.0).reshape(seq, nkv * hd)
    vc = O.synth_normal(seq * nkv * hd, 8, 1.0).reshape(seq, nkv * hd)
    q = O.synth_normal(nh * hd, 9, 1.0)
    out["attn_k"], out["attn_v"], out["attn_q"] = kc, vc, q
    out["attn_out_f32"] = O.decode_attention(q, kc, vc, nh, nkv, hd, seq, 0.125)
    kh = np.array([O.f32_to_f16(v) for v in kc.ravel()], dtype=np.uint16).reshape(kc.shape)
    vh = np.array([O.f32_to_f16(v) for v in vc.ravel()], dtype=np.uint16).reshape(vc.shape)
    out["attn_k_f16"], out["attn_v_f16"] = kh, vh
    out["attn_out_f16"] = O.decode_attention(q, kh, vh, nh, nkv, hd, seq, 0.125)
    # glue
    g, u = O.synth_normal(96, 11, 2.0), O.synth_normal(96, 12, 1.0)
    out["glue_g"], out["glue_u"], out["glue_silu_mul"] = g, u, O.silu_mul(g, u)
    wn = O.synth_normal(96, 13, 1.0)
    out["glue_norm_w"], out["glue_rmsnorm"] = wn, O.rmsnorm(g, wn, 1e-5)
    return out


if __name__ == "__main__":
    np.savez_compressed(os.path.join(HERE, "quant_path.npz"), **build())
    print("wrote", os.path.join(HERE, "quant_path.npz"))
