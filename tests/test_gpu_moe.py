"""Routed (mixture-of-experts) feed-forward on the CUDA device against the per-token composition the
reference runs (cera/src/model/lfm2.rs:735-901): oracle routing rule + oracle int8 GEMVs + SiLU*mul."""
import numpy as np
import pytest

import oracle_lib as O
from gpu_util import ATOL, RTOL, assert_close, cosine, need_gpu

pytestmark = pytest.mark.gpu


def _layer(t, n_expert, hidden, ff, seed):
    gate = O.quantize_weights(t, O.synth_normal(n_expert * ff * hidden, seed, 0.02))
    up = O.quantize_weights(t, O.synth_normal(n_expert * ff * hidden, seed + 1, 0.02))
    down = O.quantize_weights(t, O.synth_normal(n_expert * hidden * ff, seed + 2, 0.02))
    router = O.synth_normal(n_expert * hidden, seed + 3, 0.05).reshape(n_expert, hidden)
    return gate, up, down, router


def _reference(t, layer, n_used, hidden, ff, x, bias, softmax_gate):
    """Per token: route, then for each pick gate/up GEMV, SiLU*mul, down GEMV, weighted sum in pick order."""
    gate, up, down, router = layer
    n_expert = router.shape[0]
    gb, db = len(gate) // n_expert, len(down) // n_expert
    out = np.zeros_like(x)
    ids, wts, margins = [], [], []
    for j, xj in enumerate(x):
        logits = (router.astype(np.float32) @ xj.astype(np.float32)).astype(np.float32)
        if softmax_gate:
            e = np.exp(logits - logits.max(), dtype=np.float32)
            probs = (e / e.sum(dtype=np.float32)).astype(np.float32)
        else:
            probs = (np.float32(1.0) / (np.float32(1.0) + np.exp(-logits, dtype=np.float32))).astype(np.float32)
        sel, w = O.select_experts(probs, bias, n_used)
        biased = np.sort(probs + bias)[::-1]
        margins.append(float(np.min(np.abs(np.diff(biased[:n_used + 1])))))
        acc = np.zeros(hidden, dtype=np.float32)
        for e, we in zip(sel, w):
            fast = O.has_avx2() and t != O.Q5_K  # bit-identical to the scalar restatement (tested), only faster
            g = O.gemv(t, gate[e * gb:(e + 1) * gb], xj, ff, hidden, avx2=fast, threads=4)
            u = O.gemv(t, up[e * gb:(e + 1) * gb], xj, ff, hidden, avx2=fast, threads=4)
            h = O.silu_mul(g, u)
            y = O.gemv(t, down[e * db:(e + 1) * db], h, hidden, ff, avx2=fast, threads=4)
            acc = (acc + (np.float32(we) * y).astype(np.float32)).astype(np.float32)
        out[j] = acc
        ids.append(list(sel))
        wts.append(list(w))
    return out, np.array(ids), np.array(wts, dtype=np.float32), np.array(margins)


def _run(t, n_expert, n_used, hidden, ff, n, seed, bias_sigma=0.0, softmax_gate=False):
    import torch
    import cera_b200 as cb
    layer = _layer(t, n_expert, hidden, ff, seed)
    bias = (O.synth_normal(n_expert, seed + 9, bias_sigma) if bias_sigma else np.zeros(n_expert, dtype=np.float32))
    x = O.synth_normal(n * hidden, seed + 5, 1.0).reshape(n, hidden)
    want, ids_w, wts_w, margins = _reference(t, layer, n_used, hidden, ff, x, bias, softmax_gate)
    moe = cb.MoeFfn(n_expert, n_used, hidden, ff, t, layer[0], layer[1], layer[2], layer[3],
                    exp_probs_b=bias if bias_sigma else None, max_tokens=max(n, 1))
    for _ in range(2):  # the second call reuses the counters the first one must have reset
        out, ids, wts = moe(torch.from_numpy(x).cuda(), softmax_gate=softmax_gate, want_routing=True)
    torch.cuda.synchronize()
    out, ids, wts = out.cpu().numpy(), ids.cpu().numpy(), wts.cpu().numpy()
    clear = margins > 1e-5  # a router near-tie may legitimately resolve either way in f32
    assert clear.mean() > 0.9
    assert np.array_equal(ids[clear], ids_w[clear])
    assert_close(wts[clear], wts_w[clear], "routing weights")
    # The SiLU*mul product is re-quantized to int8 before the down projection, so a last-bit difference in a
    # gate/up output can flip one quant and move an output by more than the per-operator tolerance (the
    # whole-model tests meet the same effect).  Per-operator tolerance for nearly all elements, a bound
    # relative to the output scale for the rest, and the reference's cosine bar.
    g, w = out[clear].astype(np.float64), want[clear].astype(np.float64)
    err = np.abs(g - w)
    assert (err <= ATOL + RTOL * np.abs(w)).mean() >= 0.99
    assert err.max() <= 2e-3 * np.abs(w).max()
    assert cosine(g.ravel(), w.ravel()) >= 0.99999
    moe.close()


@pytest.mark.parametrize("n", [1, 5, 37])
@pytest.mark.parametrize("t_name", ["Q4_0", "Q8_0", "Q4_1"])
def test_routed_ffn_small(t_name, n):
    need_gpu()
    import cera_b200 as cb
    _run(getattr(cb, t_name), n_expert=8, n_used=2, hidden=256, ff=128, n=n, seed=21)


@pytest.mark.parametrize("t_name", ["Q4_K", "Q6_K"])
def test_routed_ffn_k_quants(t_name):
    need_gpu()
    import cera_b200 as cb
    _run(getattr(cb, t_name), n_expert=6, n_used=3, hidden=512, ff=256, n=19, seed=33)


@pytest.mark.parametrize("t_name,n", [("Q4_0", 96), ("Q4_K", 150), ("Q6_K", 70), ("Q4_0", 17)])
def test_routed_ffn_batches_on_the_tensor_core_path(t_name, n):
    """16 tokens and more with 256-aligned widths: 64-column work items through the expert-grouped tensor-core GEMM,
    ragged per-expert counts included.  (Q5_K is left out: the oracle's GEMV for it is the reference's
    f32-activation form, which differs from the Q8_0-activation product by the activation quantization.)"""
    need_gpu()
    import cera_b200 as cb
    _run(getattr(cb, t_name), n_expert=8, n_used=2, hidden=512, ff=256, n=n, seed=61)


def test_selection_bias_steers_rank_not_weight():
    """exp_probs_b changes which experts are picked; the combine weights stay the unbiased probabilities."""
    need_gpu()
    import cera_b200 as cb
    _run(cb.Q4_0, n_expert=16, n_used=4, hidden=256, ff=128, n=23, seed=41, bias_sigma=0.3)


def test_softmax_gate_variant():
    need_gpu()
    import cera_b200 as cb
    _run(cb.Q4_0, n_expert=8, n_used=2, hidden=256, ff=128, n=9, seed=45, softmax_gate=True)


def test_lfm2moe_layer_shape():
    """32 experts x (1792 x 2048), top-4, Q4_0: the shape of the expert-parallel configuration, 24 tokens."""
    need_gpu()
    import cera_b200 as cb
    _run(cb.Q4_0, n_expert=32, n_used=4, hidden=2048, ff=1792, n=24, seed=51)


def test_lfm2moe_config5_512_tokens():
    """The routed-FFN configuration at its full size: 512 tokens of N(0, 1) hidden states through 32 Q4_0
    experts of 1792 x 2048, top-4 (the expert-grouped tensor-core path with ragged per-expert counts),
    against the per-token composition of the reference."""
    need_gpu()
    import cera_b200 as cb
    _run(cb.Q4_0, n_expert=32, n_used=4, hidden=2048, ff=1792, n=512, seed=71)


def test_contract_errors():
    need_gpu()
    import torch
    import cera_b200 as cb
    layer = _layer(cb.Q4_0, 4, 64, 32, 3)
    with pytest.raises(cb.CeraCudaError, match="experts"):
        cb.MoeFfn(4, 5, 64, 32, cb.Q4_0, *layer)
    moe = cb.MoeFfn(4, 2, 64, 32, cb.Q4_0, *layer, max_tokens=4)
    with pytest.raises(cb.CeraCudaError, match="at most"):
        moe(torch.zeros(5, 64, device="cuda"))
    moe.close()
