"""Whole-model decode on the CUDA device against the oracle's llama forward."""
import numpy as np
import pytest

import oracle_lib as O
from gpu_util import assert_close, assert_model_logits, compare_greedy_streams, cosine, need_gpu

pytestmark = pytest.mark.gpu

SMALL = dict(n_layers=2, hidden_size=256, intermediate_size=512, n_heads=4, n_kv_heads=1, head_dim=64, vocab_size=512,
             rope_theta=500000.0, rms_norm_eps=1e-5, rope_type=0)


# wide enough (k >= 1024) for every projection to take the lane-task GEMV kernel, fused segments included
WIDE = dict(n_layers=2, hidden_size=1024, intermediate_size=2048, n_heads=8, n_kv_heads=2, head_dim=128,
            vocab_size=1024, rope_theta=500000.0, rms_norm_eps=1e-5, rope_type=0)


def _pair(cfg, seed, kv_f16=0, max_seq_len=64, types=None, threads=2):
    from cera_b200 import synth
    oracle = O.OracleModel(**{k: cfg[k] for k in ("n_layers", "hidden_size", "intermediate_size", "n_heads",
                                                   "n_kv_heads", "head_dim", "vocab_size", "rope_theta",
                                                   "rms_norm_eps", "rope_type")},
                           max_seq_len=max_seq_len, kv_f16=kv_f16, n_threads=threads)

    def sink(role, layer, t, rows, cols, data):
        oracle.set_tensor(int(role), layer, t, rows, cols, data)

    gpu = synth.build_llama(cfg, seed=seed, sink=sink, types=types, max_seq_len=max_seq_len, kv_f16=kv_f16)
    return gpu, oracle


@pytest.mark.parametrize("kv_f16", [0, 1])
def test_small_llama_logits_and_greedy_stream(kv_f16):
    need_gpu()
    from cera_b200 import synth
    gpu, oracle = _pair(SMALL, seed=3, kv_f16=kv_f16)
    prompt = synth.prompt_tokens(8, SMALL["vocab_size"], seed=1)
    tok_g = tok_o = None
    for pos, t in enumerate(prompt):
        lg = gpu.forward(int(t), pos)
        lo = oracle.forward(int(t), pos)
        assert_model_logits(lg, lo, f"logits at pos {pos}")
        assert cosine(gpu.last_hidden(), oracle.last_hidden()) >= 0.9999
        if pos == 0:
            # first token: one pass of the kernels on identical inputs, no KV history yet
            assert np.abs(lg - lo).max() <= 5e-3 * np.abs(lo).max()
    first = int(O.argmax(lo))
    assert int(O.argmax(lg)) == first
    # the reference stream, teacher-forced on its own picks, with its logits kept for the tie rule
    pos0 = len(prompt)
    stream_o, logits_o, tok = [], [], first
    for i in range(24):
        lo = oracle.forward(tok, pos0 + i)
        logits_o.append(lo)
        tok = int(O.argmax(lo))
        stream_o.append(tok)
    stream_g, tok = [], first
    for i in range(24):
        tok = gpu.forward_greedy(tok, pos0 + i)
        stream_g.append(tok)
    matched = compare_greedy_streams(stream_g, stream_o, lambda i: logits_o[i])
    assert matched >= 4
    pos = pos0 + 24
    assert gpu.seq_len == oracle.seq_len == pos
    assert gpu.launch_count() > 0 and gpu.gpu_memory_bytes() > 0


def test_prefill_equals_per_token_forward_and_truncate():
    need_gpu()
    from cera_b200 import synth
    gpu, oracle = _pair(SMALL, seed=5)
    prompt = synth.prompt_tokens(12, SMALL["vocab_size"], seed=2)
    lp = gpu.forward_prefill(prompt, 0)
    for pos, t in enumerate(prompt):
        lo = oracle.forward(int(t), pos)
    assert_model_logits(lp, lo, "prefill last logits")
    # rewind and replay: same logits again (truncate_kv moves the device counter)
    gpu.truncate_kv(6)
    assert gpu.seq_len == 6
    again = gpu.forward_prefill(prompt[6:], 6)
    assert np.array_equal(again, lp)


@pytest.mark.parametrize("kv_f16", [0, 1])
def test_wide_llama_matches_oracle(kv_f16):
    """Takes the fused launches: norm + quantize prologue, RoPE + KV-append and SiLU*mul + quantize epilogues."""
    need_gpu()
    from cera_b200 import synth
    gpu, oracle = _pair(WIDE, seed=21, threads=4, kv_f16=kv_f16)
    prompt = synth.prompt_tokens(6, WIDE["vocab_size"], seed=3)
    for pos, t in enumerate(prompt):
        lg, lo = gpu.forward(int(t), pos), oracle.forward(int(t), pos)
        assert_model_logits(lg, lo, f"pos {pos}")
        if pos == 0:
            assert np.abs(lg - lo).max() <= 5e-3 * np.abs(lo).max()
    tok = int(O.argmax(lo))
    stream_o, logits_o, stream_g = [], [], []
    t_o = t_g = tok
    for i in range(12):
        lo = oracle.forward(t_o, len(prompt) + i)
        logits_o.append(lo)
        t_o = int(O.argmax(lo))
        stream_o.append(t_o)
    for i in range(12):
        t_g = gpu.forward_greedy(t_g, len(prompt) + i)
        stream_g.append(t_g)
    assert compare_greedy_streams(stream_g, stream_o, lambda i: logits_o[i]) >= 4


def test_batched_prefill_matches_oracle_and_crosses_a_chunk_boundary():
    """600 prompt tokens = one full 512-token chunk + a ragged one, through the batched kernels; the last-token logits
    against the oracle's per-token forward, then decode continues from the batched KV cache."""
    need_gpu()
    from cera_b200 import synth
    gpu, oracle = _pair(SMALL, seed=13, max_seq_len=620, threads=4)
    prompt = synth.prompt_tokens(600, SMALL["vocab_size"], seed=6)
    lp = gpu.forward_prefill(prompt, 0)
    for pos, t in enumerate(prompt):
        lo = oracle.forward(int(t), pos)
    assert_model_logits(lp, lo, "batched prefill, 600 tokens")
    tok = int(O.argmax(lo))
    assert_model_logits(gpu.forward(tok, 600), oracle.forward(tok, 600), "decode after batched prefill")


def test_batched_prefill_wide_model_and_f16_kv():
    need_gpu()
    from cera_b200 import synth
    for kv_f16 in (0, 1):
        gpu, oracle = _pair(WIDE, seed=17, threads=4, kv_f16=kv_f16)
        prompt = synth.prompt_tokens(21, WIDE["vocab_size"], seed=8)
        lp = gpu.forward_prefill(prompt, 0)
        for pos, t in enumerate(prompt):
            lo = oracle.forward(int(t), pos)
        assert_model_logits(lp, lo, f"batched prefill kv_f16={kv_f16}")


def test_generate_greedy_equals_stepwise_greedy():
    need_gpu()
    gpu, _ = _pair(SMALL, seed=9)
    gpu.forward_prefill(np.array([3, 1, 4, 1, 5], dtype=np.uint32), 0, want_logits=False)
    step, tok = [], 9
    for i in range(10):
        tok = gpu.forward_greedy(tok, 5 + i)
        step.append(tok)
    gpu.truncate_kv(5)
    chained, ms = gpu.generate_greedy(9, 5, 10)
    assert list(chained) == step and ms > 0
    assert gpu.seq_len == 15


def test_model_contract_errors():
    need_gpu()
    import cera_b200 as cb
    from cera_b200 import synth
    gpu, _ = _pair(SMALL, seed=7, max_seq_len=4)
    with pytest.raises(cb.CeraCudaError) as e:
        gpu.forward(1, 3)  # pos != seq_len
    assert e.value.code == 7
    with pytest.raises(cb.CeraCudaError):
        gpu.forward(SMALL["vocab_size"], 0)
    for p in range(4):
        gpu.forward(1, p)
    with pytest.raises(cb.CeraCudaError):
        gpu.forward(1, 4)  # beyond max_seq_len
    m = cb.CudaModel(**SMALL, max_seq_len=8)
    with pytest.raises(cb.CeraCudaError):
        m.finalize()  # tensors missing
    with pytest.raises(cb.CeraCudaError) as e:
        m.add_tensor(cb.Role.ATTN_NORM, 0, cb.Q4_0, 1, 256, np.zeros(144, dtype=np.uint8))
    assert e.value.code == 2


def test_mixed_type_layers():
    """Q4_0 / Q8_0 / Q4_1 / Q5_K tensors in one model take the unfused launch paths."""
    need_gpu()
    import cera_b200 as cb
    from cera_b200 import synth
    types = {cb.Role.ATTN_Q: cb.Q4_0, cb.Role.ATTN_K: cb.Q8_0, cb.Role.ATTN_V: cb.Q6_K, cb.Role.ATTN_OUTPUT: cb.Q4_1,
             cb.Role.FFN_GATE: cb.Q4_K, cb.Role.FFN_UP: cb.Q4_0, cb.Role.FFN_DOWN: cb.Q8_0, cb.Role.TOKEN_EMBD: cb.Q8_0,
             cb.Role.OUTPUT: cb.Q4_K}
    gpu, oracle = _pair(SMALL, seed=11, types=types)
    prompt = synth.prompt_tokens(5, SMALL["vocab_size"], seed=4)
    for pos, t in enumerate(prompt):
        assert_model_logits(gpu.forward(int(t), pos), oracle.forward(int(t), pos), f"pos {pos}")


@pytest.mark.parametrize("kv_f16", [0, 1])
@pytest.mark.parametrize("rope_type", [0, 1])
def test_kv_shift_matches_reference(kv_f16, rope_type):
    """n_keep context shift (cera/src/kv_cache.rs:1091-1320): after dropping a middle range and re-rotating the keys
    that moved, the next tokens' logits follow the oracle, which performs the same shift on its own cache."""
    need_gpu()
    import cera_b200 as cb
    from cera_b200 import synth
    cfg = dict(SMALL, rope_type=rope_type)
    gpu, oracle = _pair(cfg, seed=13, kv_f16=kv_f16)
    prompt = synth.prompt_tokens(26, cfg["vocab_size"], seed=2)
    for pos, t in enumerate(prompt[:20]):
        gpu.forward(int(t), pos)
        oracle.forward(int(t), pos)
    gpu.shift_kv(4, 6)
    oracle.shift_kv(4, 6)
    assert gpu.seq_len == oracle.seq_len == 14
    for i, t in enumerate(prompt[20:]):
        lg = gpu.forward(int(t), 14 + i)
        lo = oracle.forward(int(t), 14 + i)
        assert_model_logits(lg, lo, f"logits {i} tokens after the shift")
    # shifting everything after n_keep away is a truncation
    gpu.shift_kv(3, gpu.seq_len - 3)
    oracle.shift_kv(3, oracle.seq_len - 3)
    assert gpu.seq_len == 3
    assert_model_logits(gpu.forward(5, 3), oracle.forward(5, 3), "after shifting the whole tail away")
    with pytest.raises(cb.CeraCudaError, match="shift must be"):
        gpu.shift_kv(1, 0)
    with pytest.raises(cb.CeraCudaError, match="exceed seq_len"):
        gpu.shift_kv(3, 2)


def test_snapshot_restore_replays_the_same_tokens():
    need_gpu()
    import cera_b200 as cb
    from cera_b200 import synth
    gpu = synth.build_llama(WIDE, seed=21, max_seq_len=64)
    prompt = synth.prompt_tokens(10, WIDE["vocab_size"], seed=4)
    logits = gpu.forward_prefill(prompt, 0)
    first = int(np.argmax(logits))
    snap = gpu.snapshot()
    assert snap.size == 32 + 2 * WIDE["n_layers"] * 10 * WIDE["n_kv_heads"] * WIDE["head_dim"] * 4
    a, _ = gpu.generate_greedy(first, 10, 12)
    gpu.restore(snap)
    assert gpu.seq_len == 10
    b, _ = gpu.generate_greedy(first, 10, 12)
    assert list(a) == list(b)
    # into a second model with the same weights
    twin = synth.build_llama(WIDE, seed=21, max_seq_len=64)
    twin.restore(snap)
    c, _ = twin.generate_greedy(first, 10, 12)
    assert list(a) == list(c)
    other = synth.build_llama(SMALL, seed=21, max_seq_len=64)
    with pytest.raises(cb.CeraCudaError, match="does not fit"):
        other.restore(snap)
    with pytest.raises(cb.CeraCudaError, match="truncated"):
        twin.restore(snap[:-8])
    with pytest.raises(cb.CeraCudaError, match="not a KV snapshot"):
        twin.restore(np.zeros(64, dtype=np.uint8))


def test_prefill_logits_for_every_position():
    """forward_prefill_logits_all: row j is what forward() returns at position j (batched kernels vs the decode
    step: the reference's model-level bars), across a chunk boundary; the cache ends up the same."""
    need_gpu()
    from cera_b200 import synth
    cfg = dict(SMALL, n_layers=1)
    a = synth.build_llama(cfg, seed=17, max_seq_len=560)
    b = synth.build_llama(cfg, seed=17, max_seq_len=560)
    prompt = synth.prompt_tokens(530, cfg["vocab_size"], seed=8)
    rows = a.forward_prefill_logits_all(prompt, 0)
    assert rows.shape == (530, cfg["vocab_size"]) and a.seq_len == 530
    want = [b.forward(int(t), pos) for pos, t in enumerate(prompt)]
    for pos in (0, 1, 100, 255, 256, 511, 512, 529):
        assert_model_logits(rows[pos], want[pos], f"position {pos}")
    nxt = int(np.argmax(rows[-1]))
    assert_model_logits(a.forward(nxt, 530), b.forward(nxt, 530), "next token after the two prefills")


def test_lora_adapters_match_reference_and_detach_cleanly():
    """Dense LoRA on every projection kind (cera/src/lora.rs:794-821, wired as in transformer.rs): logits follow the
    oracle with the same pairs attached; a prompt gives the same logits as token-by-token decoding; B = 0 and a
    detach both give back the base model bit for bit."""
    need_gpu()
    import cera_b200 as cb
    from cera_b200 import synth
    cfg = WIDE
    gpu, oracle = _pair(cfg, seed=29)
    hs, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qd, kvd = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"]
    shapes = {"attn_q": (hs, qd), "attn_k": (hs, kvd), "attn_v": (hs, kvd), "attn_output": (qd, hs), "ffn_gate": (hs, ff),
              "ffn_up": (hs, ff), "ffn_down": (ff, hs)}
    prompt = synth.prompt_tokens(6, cfg["vocab_size"], seed=3)
    base = [gpu.forward(int(t), pos) for pos, t in enumerate(prompt)]
    gpu.truncate_kv(0)
    rng = np.random.default_rng(7)
    pairs = []
    for layer, targets in ((0, ("attn_q", "attn_v", "ffn_gate", "ffn_down")), (1, ("attn_k", "attn_output", "ffn_up"))):
        for name in targets:
            k, d = shapes[name]
            rank = 8 if name != "ffn_down" else 5
            a = (rng.standard_normal((rank, k)) * 0.05).astype(np.float32)
            b = (rng.standard_normal((d, rank)) * 0.05).astype(np.float32)
            pairs.append((name, layer, a, b))
    # B = 0: attached but inert
    for name, layer, a, b in pairs:
        gpu.attach_lora(name, layer, a, np.zeros_like(b), 2.0)
    inert = [gpu.forward(int(t), pos) for pos, t in enumerate(prompt)]
    for x, y in zip(base, inert):
        assert np.array_equal(x, y)
    gpu.truncate_kv(0)
    for name, layer, a, b in pairs:
        gpu.attach_lora(name, layer, a, b, 2.0)
        oracle.set_lora(cb.CudaModel.LORA_TARGETS.index(name), layer, a, b, 2.0)
    moved = 0.0
    for pos, t in enumerate(prompt):
        lg, lo = gpu.forward(int(t), pos), oracle.forward(int(t), pos)
        assert_model_logits(lg, lo, f"adapted logits at pos {pos}")
        moved = max(moved, float(np.abs(lg - base[pos]).max()))
    assert moved > 1e-3  # the adapters do change the model
    last_step = lg
    gpu.truncate_kv(0)
    assert np.array_equal(gpu.forward_prefill(prompt, 0), last_step)  # prompts take the per-token path while adapted
    gpu.detach_lora()
    gpu.truncate_kv(0)
    for pos, t in enumerate(prompt):
        assert np.array_equal(gpu.forward(int(t), pos), base[pos])
    with pytest.raises(cb.CeraCudaError, match="expects"):
        gpu.attach_lora("attn_q", 0, np.zeros((4, hs + 1), np.float32), np.zeros((qd, 4), np.float32), 1.0)
    with pytest.raises(cb.CeraCudaError, match="target"):
        gpu.attach_lora(9, 0, np.zeros((4, hs), np.float32), np.zeros((qd, 4), np.float32), 1.0)
