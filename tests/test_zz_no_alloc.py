"""The allocation-free attention entry point against the ordinary one.

cera_cuda_decode_attention_noalloc serves callers that are not allowed to allocate device memory
(they run inside an engine that owns the device heap, or on a thread where an allocation's implicit
synchronisation is forbidden): its split-KV workspace is an array built into the library.  It must
give what cera_cuda_decode_attention gives with a caller-provided workspace, also on the second call,
when the array still holds the first call's records.  This file sorts last so that a run stopping at
the first failure has already run every other test.
"""
import math

import numpy as np
import pytest

from gpu_util import assert_close, need_gpu

pytestmark = pytest.mark.gpu


def _case(cb, torch, nh, nkv, hd, seq, seed, f16=False):
    kv_dim = nkv * hd
    kc = cb.synth_normal(seq * kv_dim, seed=seed, sigma=1.0).reshape(seq, kv_dim)
    vc = cb.synth_normal(seq * kv_dim, seed=seed + 1, sigma=1.0).reshape(seq, kv_dim)
    q = cb.synth_normal(nh * hd, seed=seed + 2, sigma=1.0)
    if f16:
        kc, vc = kc.half(), vc.half()
    return q, kc, vc, 1.0 / math.sqrt(hd)


def test_noalloc_attention_matches_workspace_attention_twice_in_a_row():
    torch = need_gpu()
    import cera_b200 as cb
    nh, nkv, hd = 32, 8, 128
    out = torch.empty(nh * hd, dtype=torch.float32, device="cuda")
    # Two different problems back to back, both long enough (> 4096 positions) to take the two-kernel path whose
    # split pass writes its partial results into the built-in array and whose merge pass reads them back; the
    # second, shorter problem finds the first call's records still sitting there.  The third case is short
    # enough for the single-launch kernel, which must leave the array alone and still agree.
    for seq, seed, f16 in ((8192, 11, False), (5000, 23, True), (777, 31, False)):
        q, kc, vc, scale = _case(cb, torch, nh, nkv, hd, seq, seed, f16)
        want = cb.decode_attention(q, kc, vc, nh, nkv, hd, seq, scale).cpu().numpy()
        got = cb.decode_attention_noalloc(q, kc, vc, nh, nkv, hd, seq, scale, out=out).cpu().numpy()
        assert_close(got, want, f"seq={seq}")
        assert np.array_equal(got, want), "same kernels, same inputs: the outputs should be identical"


def test_noalloc_attention_rejects_shapes_beyond_the_built_in_scratch():
    torch = need_gpu()
    import cera_b200 as cb
    q = torch.zeros(128 * 128, device="cuda")
    kc = torch.zeros(4, 16 * 128, device="cuda")
    with pytest.raises(cb.CeraCudaError) as e:
        cb.decode_attention_noalloc(q, kc, kc, 128, 16, 128, 4, 0.1)
    assert e.value.code == 1 and "built-in scratch" in str(e.value)
