"""Tensor-parallel decode: the bounded wait on one GPU, and (with two or more GPUs) rank-count
invariance of logits and greedy streams against the single-GPU model."""
import json
import os
import subprocess
import sys

import pytest

from gpu_util import need_gpu

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_exchange_wait_runs_out_and_reports():
    """A peer that never signals: the kernel gives up after its budget and leaves (slot, peer) behind."""
    need_gpu()
    import ctypes as C
    from cera_b200._lib import check, lib
    status, ms = C.c_uint32(), C.c_float()
    check(lib.cera_cuda_tp_wait_selftest(60, C.byref(status), C.byref(ms)))
    assert status.value == 0x80000000 | (1 << 24) | 4
    assert 55.0 <= ms.value < 1500.0
    # the device stays usable
    import cera_b200 as cb
    assert cb.synth_normal(64, seed=1, sigma=1.0).shape[0] == 64


def test_set_tp_contract():
    need_gpu()
    import cera_b200 as cb
    from cera_b200.model import CudaModel
    cfg = dict(n_layers=1, hidden_size=256, intermediate_size=512, n_heads=4, n_kv_heads=2, head_dim=64, vocab_size=512,
               rope_theta=500000.0, rms_norm_eps=1e-5, max_seq_len=8)
    with pytest.raises(cb.CeraCudaError, match="KV heads"):
        CudaModel(tp=(0, 4), **cfg)
    with pytest.raises(cb.CeraCudaError, match="rank"):
        CudaModel(tp=(2, 2), **cfg)
    with pytest.raises(cb.CeraCudaError, match="intermediate"):
        CudaModel(tp=(0, 2), **dict(cfg, intermediate_size=96))
    m = CudaModel(tp=(1, 2), **cfg)
    m.close()


def test_unconnected_model_refuses_to_run():
    need_gpu()
    import cera_b200 as cb
    from cera_b200 import synth
    cfg = dict(n_layers=1, hidden_size=256, intermediate_size=512, n_heads=4, n_kv_heads=2, head_dim=64, vocab_size=512,
               rope_theta=500000.0, rms_norm_eps=1e-5, rope_type=0)
    m = synth.build_llama(cfg, seed=1, max_seq_len=8, tp=(0, 2))
    assert len(m.tp_handle()) == 64
    with pytest.raises(cb.CeraCudaError, match="not connected"):
        m.forward_greedy(1, 0)
    m.close()


def test_ranks_reproduce_single_gpu():
    need_gpu()
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 4 if n >= 4 else 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "tp_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    report = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert report["world"] == world and len(report["cases"]) == 4
    for case in report["cases"]:
        assert case["stream_equal"], case
        assert case["bit_identical"], case  # a row's dot product is the same arithmetic on any number of ranks


def test_expert_parallel_ffn_reproduces_single_gpu():
    need_gpu()
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 4 if n >= 4 else 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "ep_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    report = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert report["world"] == world and len(report["cases"]) == 3
    for case in report["cases"]:
        assert case["bit_identical"] and case["repeatable"], case
    assert report["overflow_refused_on_every_rank"]
