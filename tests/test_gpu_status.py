"""After the GPU tests above have driven every kernel: no bounded device-side wait may have run out."""
import pytest

from gpu_util import need_gpu

pytestmark = pytest.mark.gpu


def test_no_device_wait_ran_out():
    torch = need_gpu()
    import cera_b200 as cb
    from cera_b200 import _lib
    # drive the TMA-staged GEMV once more in this process, then read the health word
    w = cb.QuantWeight(cb.Q4_K, 64, 4096, cb.quantize_weights(cb.Q4_K, cb.synth_normal(64 * 4096, 1, 0.02)))
    cb.gemv(w, cb.synth_normal(4096, 2, 1.0))
    torch.cuda.synchronize()
    assert _lib.kernel_status() == 0
