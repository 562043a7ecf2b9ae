"""GGUF reader (cera_b200/gguf.py) against files the tests write themselves: header, metadata values, tensor table,
alignment, rank-3 expert slicing and the error cases of cera/src/gguf.rs; and, on a GPU, a llama model loaded from a
GGUF file against the same tensors handed over directly and against the oracle."""
import os
import struct

import numpy as np
import pytest

import oracle_lib as O
from gguf_writer import write_gguf


def _meta(cfg, arch="llama", extra=()):
    return [("general.architecture", "str", arch), (f"{arch}.block_count", "u32", cfg["n_layers"]),
            (f"{arch}.embedding_length", "u32", cfg["hidden_size"]), (f"{arch}.feed_forward_length", "u32", cfg["intermediate_size"]),
            (f"{arch}.attention.head_count", "u32", cfg["n_heads"]), (f"{arch}.attention.head_count_kv", "u32", cfg["n_kv_heads"]),
            (f"{arch}.attention.key_length", "u32", cfg["head_dim"]), (f"{arch}.rope.freq_base", "f32", cfg["rope_theta"]),
            (f"{arch}.attention.layer_norm_rms_epsilon", "f32", cfg["rms_norm_eps"]), (f"{arch}.context_length", "u32", 64),
            ("tokenizer.ggml.tokens", "arr", ("str", ["<s>", "a", "b"])), ("tokenizer.ggml.scores", "arr", ("f32", [0.0, -1.0, -2.0]))] + list(extra)


def test_reader_parses_header_metadata_tensors_and_experts(tmp_path):
    import importlib.util
    spec = importlib.util.spec_from_file_location("gguf_only", os.path.join(O.ROOT, "cera_b200", "gguf.py"))
    # the reader itself needs no device: import it by path only if the package (which loads the CUDA library) cannot be imported
    try:
        from cera_b200 import gguf
    except Exception:
        pytest.skip("cera_b200 cannot be imported here")
    rng = np.random.default_rng(0)
    w = O.quantize_weights(O.Q4_K, O.synth_normal(6 * 256, 1, 0.02))          # [6 x 256] Q4_K
    experts = O.quantize_weights(O.Q4_0, O.synth_normal(3 * 4 * 64, 2, 0.02))  # 3 experts of [4 x 64] Q4_0
    norm = rng.standard_normal(256).astype(np.float32)
    path = str(tmp_path / "t.gguf")
    write_gguf(path, [("general.architecture", "str", "llama"), ("general.alignment", "u32", 64), ("x.flag", "bool", True),
                      ("x.big", "u64", 1 << 40), ("x.list", "arr", ("i32", [1, -2, 3]))],
               [("a.weight", [256, 6], O.Q4_K, w), ("n.weight", [256], O.F32, norm), ("e.weight", [64, 4, 3], O.Q4_0, experts)], alignment=64)
    with gguf.GgufFile(path) as g:
        assert g.metadata["general.architecture"] == "llama" and g.metadata["x.flag"] is True and g.metadata["x.big"] == 1 << 40
        assert list(g.metadata["x.list"]) == [1, -2, 3]
        assert g.data_offset % 64 == 0
        assert g.tensor_meta("a.weight") == (6, 256, O.Q4_K) and g.tensor_meta("n.weight") == (1, 256, O.F32)
        assert np.array_equal(g.tensor_bytes("a.weight"), w)
        assert np.array_equal(g.tensor_bytes("a.weight", 2, 3), w[2 * 144:5 * 144])
        assert np.array_equal(g.tensor_bytes("n.weight").view(np.float32), norm)
        per = experts.size // 3
        for e in range(3):
            off, n, rows, cols, t = g.expert_meta("e.weight", e)
            assert (n, rows, cols, t) == (per, 4, 64, O.Q4_0)
            assert np.array_equal(g.expert_bytes("e.weight", e), experts[e * per:(e + 1) * per])
        with pytest.raises(gguf.GgufError):
            g.expert_meta("e.weight", 3)
        with pytest.raises(gguf.GgufError):
            g.expert_meta("a.weight", 0)
    # error cases of the header (cera/src/gguf.rs:433-446, 497-499)
    bad = str(tmp_path / "bad.gguf")
    open(bad, "wb").write(struct.pack("<IIQQ", 0x12345678, 3, 0, 0))
    with pytest.raises(gguf.GgufError, match="not a GGUF"):
        gguf.GgufFile(bad)
    open(bad, "wb").write(struct.pack("<IIQQ", 0x46554747, 2, 0, 0))
    with pytest.raises(gguf.GgufError, match="version"):
        gguf.GgufFile(bad)
    write_gguf(bad, [], [("a.weight", [256, 6], O.Q4_K, w)])
    with open(bad, "r+b") as f:
        f.truncate(os.path.getsize(bad) - 100)
    with pytest.raises(gguf.GgufError, match="past the end"):
        gguf.GgufFile(bad)


@pytest.mark.gpu
def test_llama_loaded_from_gguf_matches_direct_tensors_and_oracle(tmp_path):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cera_b200 import gguf, synth
    from cera_b200.model import Role
    cfg = dict(n_layers=2, hidden_size=1024, intermediate_size=2048, n_heads=8, n_kv_heads=2, head_dim=128, vocab_size=1024,
               rope_theta=500000.0, rms_norm_eps=1e-5, rope_type=0)
    names = {Role.TOKEN_EMBD: "token_embd.weight", Role.OUTPUT_NORM: "output_norm.weight", Role.OUTPUT: "output.weight"}
    stems = {Role.ATTN_NORM: "attn_norm", Role.ATTN_Q: "attn_q", Role.ATTN_K: "attn_k", Role.ATTN_V: "attn_v", Role.ATTN_OUTPUT: "attn_output",
             Role.FFN_NORM: "ffn_norm", Role.FFN_GATE: "ffn_gate", Role.FFN_UP: "ffn_up", Role.FFN_DOWN: "ffn_down"}
    tensors = []
    oracle = O.OracleModel(**cfg, max_seq_len=32, kv_f16=0, n_threads=2)

    def sink(role, layer, t, rows, cols, data):
        oracle.set_tensor(int(role), layer, t, rows, cols, data)
        name = names.get(role) or f"blk.{layer}.{stems[role]}.weight"
        tensors.append((name, [cols] if rows == 1 and t == O.F32 else [cols, rows], t, np.array(data, copy=True)))

    direct = synth.build_llama(cfg, seed=23, max_seq_len=32, sink=sink)
    path = str(tmp_path / "m.gguf")
    write_gguf(path, _meta(cfg), tensors)
    loaded = gguf.load_llama(path, max_seq_len=32)
    tok = 3
    for pos in range(8):
        a, b, c = loaded.forward(tok, pos), direct.forward(tok, pos), oracle.forward(tok, pos)
        assert np.array_equal(a, b), "the same bytes through the file must give the same logits"
        assert np.array_equal(a.view(np.uint32), c.view(np.uint32)), "K-quant model on the reference-order kernels: oracle bits"
        tok = int(np.argmax(c))
    loaded.close()
    direct.close()
