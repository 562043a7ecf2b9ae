"""CUDA weight upload / dequantize / quantizers against the oracle: bit-exact."""
import numpy as np
import pytest

import oracle_lib as O
from gpu_util import assert_bits, need_gpu
from test_oracle_formats import _rand_block_bytes

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t", O.QUANT_TYPES)
def test_dequantize_rows_bit_exact(t):
    torch = need_gpu()
    import cera_b200 as cb
    rng = np.random.default_rng(t)
    m, k = 37, 1024
    raw = _rand_block_bytes(t, m, k, rng)
    w = cb.QuantWeight(t, m, k, raw)
    got = cb.dequantize_rows(w).cpu().numpy()
    want = O.dequantize(t, raw, k, rows=m)
    assert_bits(got, want, O.NAMES[t])
    part = cb.dequantize_rows(w, 5, 3).cpu().numpy()
    assert_bits(part, want[5:8], "row window")


@pytest.mark.parametrize("t", O.QUANT_TYPES)
def test_weight_quantizer_bytes_match_oracle(t):
    torch = need_gpu()
    import cera_b200 as cb
    n = 64 * 1024
    w = cb.synth_normal(n, seed=1234 + t, sigma=0.02)
    host = w.cpu().numpy()
    assert_bits(host, O.synth_normal(n, 1234 + t, 0.02), "synth_normal")
    got = cb.quantize_weights(t, w).cpu().numpy()
    assert_bits(got, O.quantize_weights(t, host), O.NAMES[t])


def test_synth_normal_offset_and_scale():
    torch = need_gpu()
    import cera_b200 as cb
    a = cb.synth_normal(5000, seed=9, sigma=1.0, offset=123).cpu().numpy()
    assert_bits(a, O.synth_normal(5000, 9, 1.0, offset=123))


def test_weight_create_rejects_bad_arguments():
    need_gpu()
    import cera_b200 as cb
    with pytest.raises(cb.CeraCudaError) as e:
        cb.QuantWeight(O.Q4_K, 4, 300, np.zeros(10, dtype=np.uint8))
    assert e.value.code == 1
    with pytest.raises(cb.CeraCudaError) as e:
        cb.QuantWeight(O.F32, 4, 32, np.zeros(4 * 32 * 4, dtype=np.uint8))
    assert e.value.code == 2
    with pytest.raises(cb.CeraCudaError):
        cb.QuantWeight(O.Q4_0, 4, 64, np.zeros(7, dtype=np.uint8))
