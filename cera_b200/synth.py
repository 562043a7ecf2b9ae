"""Seeded synthetic llama-architecture models, generated and quantized on the device.

Stands in for real GGUF checkpoints: every tensor is N(0, sigma) from the
counter-based generator behind `synth_normal`, quantized with the reference's
own quantizer rules, so any implementation that knows (seed, role, layer)
regenerates identical bytes.
"""
import numpy as np
import torch

from . import ops
from .model import CudaModel, Role
from .types import F32, Q4_K, Q6_K

# The benchmark model's tensor mix (a Q4_K_M-style GGUF): Q4_K attention / gate / up / token_embd, Q6_K ffn_down and output.
LLAMA3_8B = dict(n_layers=32, hidden_size=4096, intermediate_size=14336, n_heads=32, n_kv_heads=8, head_dim=128,
                 vocab_size=128256, rope_theta=500000.0, rms_norm_eps=1e-5, rope_type=0)
DEFAULT_TYPES = {Role.TOKEN_EMBD: Q4_K, Role.OUTPUT: Q6_K, Role.ATTN_Q: Q4_K, Role.ATTN_K: Q4_K, Role.ATTN_V: Q4_K,
                 Role.ATTN_OUTPUT: Q4_K, Role.FFN_GATE: Q4_K, Role.FFN_UP: Q4_K, Role.FFN_DOWN: Q6_K}


def tensor_seed(seed, role, layer):
    return (seed * 1000003 + int(role) * 4099 + layer + 1) & 0xFFFFFFFFFFFFFFFF


def build_llama(cfg, seed=0, sigma=0.02, types=None, sink=None, **model_kw):
    """Create, fill and finalize a CudaModel.  sink(role, layer, ggml_type, rows, cols, host_bytes)
    receives a host copy of every tensor (tests hand these to the CPU oracle)."""
    types = {**DEFAULT_TYPES, **(types or {})}
    m = CudaModel(**cfg, **model_kw)
    hs, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qd, kvd = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"]

    def matrix(role, layer, rows, cols):
        t = types[role]
        w = ops.synth_normal(rows * cols, tensor_seed(seed, role, layer), sigma)
        raw = ops.quantize_weights(t, w)
        del w
        m.add_tensor(role, layer, t, rows, cols, raw)
        if sink:
            sink(role, layer, t, rows, cols, raw.cpu().numpy())
        del raw

    def ones(role, layer, n):
        v = np.ones(n, dtype=np.float32)
        m.add_tensor(role, layer, F32, 1, n, v)
        if sink:
            sink(role, layer, F32, 1, n, v)

    matrix(Role.TOKEN_EMBD, 0, cfg["vocab_size"], hs)
    matrix(Role.OUTPUT, 0, cfg["vocab_size"], hs)
    ones(Role.OUTPUT_NORM, 0, hs)
    for l in range(cfg["n_layers"]):
        ones(Role.ATTN_NORM, l, hs)
        ones(Role.FFN_NORM, l, hs)
        matrix(Role.ATTN_Q, l, qd, hs)
        matrix(Role.ATTN_K, l, kvd, hs)
        matrix(Role.ATTN_V, l, kvd, hs)
        matrix(Role.ATTN_OUTPUT, l, hs, qd)
        matrix(Role.FFN_GATE, l, ff, hs)
        matrix(Role.FFN_UP, l, ff, hs)
        matrix(Role.FFN_DOWN, l, hs, ff)
    torch.cuda.synchronize()
    m.finalize()
    return m


def prompt_tokens(n, vocab, seed):
    """Uniform-random token ids, reproducible without numpy's generator state."""
    mask = (1 << 64) - 1
    out = np.empty(n, dtype=np.uint32)
    for i in range(n):
        x = (i + seed * 0x9E3779B97F4A7C15 + 0x9E3779B97F4A7C15) & mask
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & mask
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & mask
        x ^= x >> 31
        out[i] = x % vocab
    return out
