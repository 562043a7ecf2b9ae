"""Host side of the tensor-parallel path on CPU: the row plan, its agreement with the oracle's
arithmetic, and the handle exchange between two gloo ranks."""
import os

import numpy as np
import pytest

import oracle_lib as O
from cera_b200 import tp
from cera_b200._lib import Config
from cera_b200.model import Role
from cera_b200.types import Q4_K, Q6_K, Q8_0


def _cfg(**kw):
    base = dict(n_layers=2, hidden_size=4096, intermediate_size=14336, n_heads=32, n_kv_heads=8, head_dim=128,
                vocab_size=128256, max_seq_len=8, rope_theta=5e5, rms_norm_eps=1e-5, rope_type=0, kv_f16=0, device=0)
    base.update(kw)
    return Config(**base)


def test_llama3_8b_splits_over_1_2_4_8():
    for size in (1, 2, 4, 8):
        tp.check_divisible(_cfg(), size)
    with pytest.raises(ValueError, match="KV heads"):
        tp.check_divisible(_cfg(n_kv_heads=6), 4)
    with pytest.raises(ValueError, match="intermediate"):
        tp.check_divisible(_cfg(intermediate_size=14336 + 32), 8)
    with pytest.raises(ValueError, match="outside"):
        tp.check_divisible(_cfg(), 16)


def test_row_ranges_partition_every_split_tensor():
    rows = {Role.FFN_GATE: 14336, Role.FFN_UP: 14336, Role.FFN_DOWN: 4096, Role.OUTPUT: 128256}
    for size in (1, 2, 4, 8):
        for role, m in rows.items():
            spans = [tp.row_range(role, m, r, size) for r in range(size)]
            assert spans[0][0] == 0 and spans[-1][1] == m
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert len({b - a for a, b in spans}) == 1
    assert tp.row_range(Role.TOKEN_EMBD, 128256, 3, 8) == (0, 128256)
    assert tp.row_range(Role.ATTN_NORM, 1, 1, 2) == (0, 1)
    for role, m in ((Role.ATTN_Q, 4096), (Role.ATTN_K, 1024), (Role.ATTN_V, 1024), (Role.ATTN_OUTPUT, 4096)):
        assert tp.row_range(role, m, 1, 2) == (0, m)  # the attention block is whole on every rank
    with pytest.raises(ValueError):
        tp.row_range(Role.FFN_GATE, 100, 0, 8)
    assert tp.exchange_slots(32) == 129


@pytest.mark.parametrize("t", [Q4_K, Q6_K, Q8_0])
def test_row_split_gemv_is_the_full_gemv(t):
    """The reason the split is along rows: rank slices of the oracle's GEMV, concatenated, are the
    full product bit for bit."""
    m, k, size = 64, 512, 4
    w = O.synth_normal(m * k, 7, 0.02)
    raw = O.quantize_weights(t, w)
    x = O.synth_normal(k, 9, 1.0)
    full = O.gemv(t, raw, x, m, k)
    row_bytes = len(raw) // m
    parts = []
    for r in range(size):
        a, b = tp.row_range(Role.FFN_GATE, m, r, size)
        parts.append(O.gemv(t, raw[a * row_bytes:b * row_bytes], x, b - a, k))
    assert np.array_equal(np.concatenate(parts).view(np.uint32), full.view(np.uint32))


class _FakeModel:
    def __init__(self, rank, size):
        self.tp = (rank, size)
        self.connected = None

    def tp_handle(self):
        return bytes([self.tp[0] + 1]) * 64

    def tp_connect(self, handles):
        self.connected = handles


def _rank_main(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m = _FakeModel(rank, world)
        tp.connect(m)
        ok = m.connected == [bytes([r + 1]) * 64 for r in range(world)]
        wrong = _FakeModel((rank + 1) % world, world)
        try:
            tp.connect(wrong)
            ok = False
        except RuntimeError as e:
            ok = ok and "process group says" in str(e)
        single = _FakeModel(0, 1)
        tp.connect(single)  # no-op, no collective
        ok = ok and single.connected is None
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_handles_travel_in_rank_order_between_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    import socket
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert results == [(0, True), (1, True)]
