"""ctypes view of the CPU oracle (oracle/libcera_oracle.so) for the test-suite.

Test infrastructure only: the shipped package never imports this module.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import build as _build  # noqa: E402

F32, F16, Q4_0, Q4_1, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 2, 3, 8, 12, 13, 14, 30
QUANT_TYPES = [Q4_0, Q4_1, Q8_0, Q4_K, Q5_K, Q6_K]
NAMES = {Q4_0: "q4_0", Q4_1: "q4_1", Q8_0: "q8_0", Q4_K: "q4_k", Q5_K: "q5_k", Q6_K: "q6_k", F32: "f32",
         F16: "f16", BF16: "bf16"}
BLOCK = {Q4_0: (32, 18), Q4_1: (32, 20), Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176),
         Q6_K: (256, 210), F32: (1, 4), F16: (1, 2), BF16: (1, 2)}

_lib = C.CDLL(_build.build())

_p = C.c_void_p
_sz = C.c_size_t


def _sig(name, res, *args):
    f = getattr(_lib, name)
    f.restype = res
    f.argtypes = list(args)
    return f


_sig("cera_oracle_f16_to_f32", C.c_float, C.c_uint16)
_sig("cera_oracle_f32_to_f16", C.c_uint16, C.c_float)
_sig("cera_oracle_bf16_to_f32", C.c_float, C.c_uint16)
_sig("cera_oracle_row_bytes", _sz, C.c_int, _sz)
_sig("cera_oracle_dequantize_row", C.c_int, C.c_int, _p, _sz, _p)
_sig("cera_oracle_quantize_weights", C.c_int, C.c_int, _p, _sz, _p)
_sig("cera_oracle_quantize_q8_0", None, _p, _sz, _p, _p)
_sig("cera_oracle_quantize_columns", None, _p, _sz, _sz, _p, _p)
_sig("cera_oracle_block_sums", C.c_int, C.c_int, _p, _sz, _p, _p, _p)
_sig("cera_oracle_gemm_preq", C.c_int, C.c_int, _p, _p, _p, _p, _sz, _sz, _sz)
_sig("cera_oracle_gemv", C.c_int, C.c_int, _p, _p, _p, _sz, _sz)
_sig("cera_oracle_rmsnorm", None, _p, _p, _sz, C.c_float)
_sig("cera_oracle_expf", C.c_float, C.c_float)
_sig("cera_oracle_silu_mul", None, _p, _p, _sz)
_sig("cera_oracle_softmax", None, _p, _sz)
_sig("cera_oracle_rope", None, _p, _p, _sz, _sz, _sz, _sz, C.c_float, _p, C.c_int)
_sig("cera_oracle_decode_attention", None, _p, _p, _p, C.c_int, _sz, _sz, _sz, _sz, C.c_float, _p, _p)
_sig("cera_oracle_flash_attention_gqa", None, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, C.c_float, _p)
_sig("cera_oracle_argmax", C.c_uint32, _p, _sz)
_sig("cera_oracle_select_experts", None, _p, _p, _sz, _sz, _p, _p)
_sig("cera_oracle_synth_normal", None, _p, _sz, C.c_uint64, C.c_uint64, C.c_float)
_sig("cera_cpu_has_avx2", C.c_int)
_sig("cera_cpu_gemm_preq", C.c_int, C.c_int, _p, _p, _p, _p, _sz, _sz, _sz, C.c_int)
_sig("cera_cpu_gemv", C.c_int, C.c_int, _p, _p, _p, _sz, _sz, C.c_int)
_sig("cera_cpu_has_avx2_vnni", C.c_int)
_sig("cera_oracle_set_cpu_tier", None, C.c_int)
_sig("cera_cpu_gemm_preq_vnni", C.c_int, C.c_int, _p, _p, _p, _p, _sz, _sz, _sz, C.c_int)
_sig("cera_cpu_gemv_vnni", C.c_int, C.c_int, _p, _p, _p, _sz, _sz, C.c_int)


class OracleConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_layers", "hidden_size", "intermediate_size", "n_heads",
                                          "n_kv_heads", "head_dim", "vocab_size", "max_seq_len")] + [
        ("rope_theta", C.c_float), ("rms_norm_eps", C.c_float), ("rope_type", C.c_int32),
        ("kv_f16", C.c_int32), ("n_threads", C.c_int32), ("embedding_scale", C.c_float), ("residual_scale", C.c_float),
        ("attention_scale", C.c_float), ("logit_scale", C.c_float)]


_sig("cera_oracle_model_create", _p, C.POINTER(OracleConfig))
_sig("cera_oracle_model_set_tensor", C.c_int, _p, C.c_int, C.c_int, C.c_int, _sz, _sz, _p)
_sig("cera_oracle_model_forward", C.c_int, _p, C.c_uint32, _sz, _p)
_sig("cera_oracle_model_truncate_kv", None, _p, _sz)
_sig("cera_oracle_model_kv", _sz, _p, _sz, C.c_int, _p, _sz)
_sig("cera_oracle_model_shift_kv", C.c_int, _p, _sz, _sz)
_sig("cera_oracle_lora_apply", None, _sz, _sz, _sz, C.c_float, _p, _p, _p, _p)
_sig("cera_oracle_model_set_lora", C.c_int, _p, C.c_int, C.c_int, _sz, _sz, _sz, C.c_float, _p, _p)
_sig("cera_oracle_model_seq_len", _sz, _p)
_sig("cera_oracle_model_set_threads", None, _p, C.c_int)
_sig("cera_oracle_model_last_hidden", C.c_int, _p, _p)
_sig("cera_oracle_model_free", None, _p)


def _ptr(a):
    return a.ctypes.data_as(_p) if a is not None else None


def c32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def f16_to_f32(bits):
    return _lib.cera_oracle_f16_to_f32(int(bits))


def f32_to_f16(v):
    return _lib.cera_oracle_f32_to_f16(C.c_float(v))


def bf16_to_f32(bits):
    return _lib.cera_oracle_bf16_to_f32(int(bits))


def row_bytes(t, k):
    return _lib.cera_oracle_row_bytes(t, k)


def dequantize(t, raw, k, rows=1):
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.empty(rows * k, dtype=np.float32)
    assert raw.size == rows * row_bytes(t, k)
    rc = _lib.cera_oracle_dequantize_row(t, _ptr(raw), rows * k, _ptr(out))
    assert rc == 0
    return out.reshape(rows, k) if rows > 1 else out


def quantize_weights(t, w):
    w = c32(w).ravel()
    e, b = BLOCK[t]
    out = np.empty(w.size // e * b, dtype=np.uint8)
    rc = _lib.cera_oracle_quantize_weights(t, _ptr(w), w.size, _ptr(out))
    assert rc == 0
    return out


def quantize_q8_0(x):
    x = c32(x).ravel()
    s = np.empty(x.size // 32, dtype=np.float32)
    q = np.empty(x.size, dtype=np.int8)
    _lib.cera_oracle_quantize_q8_0(_ptr(x), x.size, _ptr(s), _ptr(q))
    return s, q


def quantize_columns(mat, dim, n):
    mat = c32(mat)
    s = np.empty(n * (dim // 32), dtype=np.float32)
    q = np.empty(n * dim, dtype=np.int8)
    _lib.cera_oracle_quantize_columns(_ptr(mat), dim, n, _ptr(s), _ptr(q))
    return s, q


def block_sums(t, row, k, aq):
    row = np.ascontiguousarray(row, dtype=np.uint8)
    aq = np.ascontiguousarray(aq, dtype=np.int8)
    u = np.empty(k // 16, dtype=np.int32)
    a = np.empty(k // 16, dtype=np.int32)
    rc = _lib.cera_oracle_block_sums(t, _ptr(row), k, _ptr(aq), _ptr(u), _ptr(a))
    assert rc == 0
    return u, a


def gemm_preq(t, w, bs, bq, m, n, k, avx2=False, threads=1):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    bs = c32(bs)
    bq = np.ascontiguousarray(bq, dtype=np.int8)
    out = np.full(m * n, np.nan, dtype=np.float32)
    if avx2 == "vnni":
        rc = _lib.cera_cpu_gemm_preq_vnni(t, _ptr(w), _ptr(bs), _ptr(bq), _ptr(out), m, n, k, threads)
    elif avx2:
        rc = _lib.cera_cpu_gemm_preq(t, _ptr(w), _ptr(bs), _ptr(bq), _ptr(out), m, n, k, threads)
    else:
        rc = _lib.cera_oracle_gemm_preq(t, _ptr(w), _ptr(bs), _ptr(bq), _ptr(out), m, n, k)
    assert rc == 0
    return out.reshape(m, n)


def gemv(t, w, x, m, k, avx2=False, threads=1):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = c32(x)
    y = np.full(m, np.nan, dtype=np.float32)
    if avx2 == "vnni":
        rc = _lib.cera_cpu_gemv_vnni(t, _ptr(w), _ptr(x), _ptr(y), m, k, threads)
    elif avx2:
        rc = _lib.cera_cpu_gemv(t, _ptr(w), _ptr(x), _ptr(y), m, k, threads)
    else:
        rc = _lib.cera_oracle_gemv(t, _ptr(w), _ptr(x), _ptr(y), m, k)
    assert rc == 0
    return y


def has_avx2():
    return bool(_lib.cera_cpu_has_avx2())


def has_vnni():
    return bool(_lib.cera_cpu_has_avx2_vnni())


def set_cpu_tier(tier):
    """Which build of the x86 int8 kernels OracleModel.forward runs: "scalar", "avx2" (default) or "vnni"."""
    _lib.cera_oracle_set_cpu_tier({"scalar": 0, "avx2": 1, "vnni": 2}[tier])


def rmsnorm(x, w, eps):
    x = c32(x).copy()
    w = c32(w)
    _lib.cera_oracle_rmsnorm(_ptr(x), _ptr(w), x.size, C.c_float(eps))
    return x


def expf(x):
    return _lib.cera_oracle_expf(C.c_float(x))


def silu_mul(g, u):
    g = c32(g).copy()
    u = c32(u)
    _lib.cera_oracle_silu_mul(_ptr(g), _ptr(u), g.size)
    return g


def softmax(x):
    x = c32(x).copy()
    _lib.cera_oracle_softmax(_ptr(x), x.size)
    return x


def rope(q, k, pos, n_heads, n_kv_heads, head_dim, base, freq_factors=None, rope_type=0):
    q = c32(q).copy()
    k = c32(k).copy()
    ff = c32(freq_factors) if freq_factors is not None else None
    _lib.cera_oracle_rope(_ptr(q), _ptr(k), pos, n_heads, n_kv_heads, head_dim, C.c_float(base), _ptr(ff),
                          rope_type)
    return q, k


def decode_attention(q, kc, vc, n_heads, n_kv_heads, head_dim, seq_len, scale):
    q = c32(q)
    f16 = kc.dtype == np.uint16
    kc = np.ascontiguousarray(kc)
    vc = np.ascontiguousarray(vc)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    scr = np.empty(max(seq_len, 1), dtype=np.float32)
    _lib.cera_oracle_decode_attention(_ptr(q), _ptr(kc), _ptr(vc), int(f16), n_heads, n_kv_heads, head_dim,
                                      seq_len, C.c_float(scale), _ptr(out), _ptr(scr))
    return out


def flash_attention_gqa(q, kc, vc, n_heads, n_kv_heads, head_dim, n, start_pos, scale):
    q = c32(q)
    kc = c32(kc)
    vc = c32(vc)
    out = np.empty(n_heads * n * head_dim, dtype=np.float32)
    _lib.cera_oracle_flash_attention_gqa(_ptr(q), _ptr(kc), _ptr(vc), n_heads, n_kv_heads, head_dim, n,
                                         start_pos, C.c_float(scale), _ptr(out))
    return out.reshape(n_heads, n, head_dim)


def argmax(x):
    x = c32(x)
    return _lib.cera_oracle_argmax(_ptr(x), x.size)


def select_experts(probs, bias, n_used):
    probs = c32(probs)
    bias = c32(bias) if bias is not None else None
    cnt = min(n_used, probs.size)
    ids = np.zeros(cnt, dtype=np.uint32)
    w = np.zeros(cnt, dtype=np.float32)
    _lib.cera_oracle_select_experts(_ptr(probs), _ptr(bias), probs.size, n_used, _ptr(ids), _ptr(w))
    return ids, w


def lora_apply(a, b, scale, x, y):
    """y + B (scale * (A x)) with the reference's summation order; a [rank, k], b [d, rank]."""
    a, b, x = c32(a), c32(b), c32(x)
    y = c32(y).copy()
    _lib.cera_oracle_lora_apply(a.shape[0], a.shape[1], b.shape[0], C.c_float(scale), _ptr(a), _ptr(b), _ptr(x), _ptr(y))
    return y


def synth_normal(n, seed, sigma, offset=0):
    out = np.empty(n, dtype=np.float32)
    _lib.cera_oracle_synth_normal(_ptr(out), n, seed, offset, C.c_float(sigma))
    return out


class OracleModel:
    """Dense llama-architecture decode on the CPU oracle."""

    def __init__(self, **cfg):
        self.cfg = OracleConfig(**cfg)
        self.h = _lib.cera_oracle_model_create(C.byref(self.cfg))
        self._keep = []

    def set_tensor(self, role, layer, t, rows, cols, data):
        data = np.ascontiguousarray(data)
        self._keep.append(data)
        rc = _lib.cera_oracle_model_set_tensor(self.h, role, layer, t, rows, cols, _ptr(data))
        assert rc == 0

    def forward(self, token, pos, want_logits=True):
        logits = np.empty(self.cfg.vocab_size, dtype=np.float32) if want_logits else None
        rc = _lib.cera_oracle_model_forward(self.h, token, pos, _ptr(logits))
        assert rc == 0, "oracle forward rejected its arguments"
        return logits

    def last_hidden(self):
        out = np.empty(self.cfg.hidden_size, dtype=np.float32)
        assert _lib.cera_oracle_model_last_hidden(self.h, _ptr(out)) == 0
        return out

    def truncate_kv(self, n):
        _lib.cera_oracle_model_truncate_kv(self.h, n)

    def kv(self, layer, which):
        """Bytes of the layer's key (0) / value (1) cache rows [0, seq_len)."""
        n = _lib.cera_oracle_model_kv(self.h, layer, which, None, 0)
        out = np.empty(n, dtype=np.uint8)
        _lib.cera_oracle_model_kv(self.h, layer, which, _ptr(out), n)
        return out

    def set_threads(self, n):
        _lib.cera_oracle_model_set_threads(self.h, n)

    def set_lora(self, target, layer, a, b, scale):
        """a: [rank, k], b: [d, rank] float32."""
        a, b = c32(a), c32(b)
        assert _lib.cera_oracle_model_set_lora(self.h, target, layer, a.shape[0], a.shape[1], b.shape[0], C.c_float(scale),
                                               _ptr(a), _ptr(b)) == 0

    def shift_kv(self, n_keep, shift):
        assert _lib.cera_oracle_model_shift_kv(self.h, n_keep, shift) == 0

    @property
    def seq_len(self):
        return _lib.cera_oracle_model_seq_len(self.h)

    def close(self):
        if self.h:
            _lib.cera_oracle_model_free(self.h)
            self.h = None

    def __del__(self):
        self.close()


# ---- seeded synthetic llama models, generated on the host --------------------------------------
# The same tensors cera_b200.synth.build_llama generates on the device (same seeds, generator and
# quantizer rules; a CPU test holds the two definitions together), built without touching the
# CUDA library so that CPU-only legs can use them.
LLAMA3_8B = dict(n_layers=32, hidden_size=4096, intermediate_size=14336, n_heads=32, n_kv_heads=8, head_dim=128,
                 vocab_size=128256, rope_theta=500000.0, rms_norm_eps=1e-5, rope_type=0)
ROLE = dict(TOKEN_EMBD=0, OUTPUT_NORM=1, OUTPUT=2, ATTN_NORM=3, ATTN_Q=4, ATTN_K=5, ATTN_V=6, ATTN_OUTPUT=7,
            FFN_NORM=8, FFN_GATE=9, FFN_UP=10, FFN_DOWN=11, ROPE_FREQS=12)
DEFAULT_TYPES = {"TOKEN_EMBD": Q4_K, "OUTPUT": Q6_K, "ATTN_Q": Q4_K, "ATTN_K": Q4_K, "ATTN_V": Q4_K,
                 "ATTN_OUTPUT": Q4_K, "FFN_GATE": Q4_K, "FFN_UP": Q4_K, "FFN_DOWN": Q6_K}


def tensor_seed(seed, role, layer):
    return (seed * 1000003 + int(role) * 4099 + layer + 1) & 0xFFFFFFFFFFFFFFFF


def prompt_tokens(n, vocab, seed):
    mask = (1 << 64) - 1
    out = np.empty(n, dtype=np.uint32)
    for i in range(n):
        x = (i + seed * 0x9E3779B97F4A7C15 + 0x9E3779B97F4A7C15) & mask
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & mask
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & mask
        x ^= x >> 31
        out[i] = x % vocab
    return out


def synth_quantized(t, rows, cols, seed, sigma=0.02, threads=1):
    """rows x cols of sigma * IH12(seed, i), quantized to block type t; row ranges in parallel threads."""
    e, b = BLOCK[t]
    rb = cols // e * b
    out = np.empty(rows * rb, dtype=np.uint8)

    def part(lo, hi):
        w = np.empty((hi - lo) * cols, dtype=np.float32)
        _lib.cera_oracle_synth_normal(_ptr(w), w.size, seed, lo * cols, C.c_float(sigma))
        dst = out[lo * rb:hi * rb]
        assert _lib.cera_oracle_quantize_weights(t, _ptr(w), w.size, _ptr(dst)) == 0

    if threads <= 1 or rows < 4 * threads:
        part(0, rows)
    else:
        from concurrent.futures import ThreadPoolExecutor
        per = -(-rows // (4 * threads))
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(lambda lo: part(lo, min(rows, lo + per)), range(0, rows, per)))
    return out


def build_oracle_llama(cfg, seed=0, sigma=0.02, types=None, max_seq_len=64, kv_f16=0, threads=1):
    """OracleModel of cfg with the tensors of cera_b200.synth.build_llama(cfg, seed, sigma, types)."""
    types = {**DEFAULT_TYPES, **(types or {})}
    m = OracleModel(**cfg, max_seq_len=max_seq_len, kv_f16=kv_f16, n_threads=threads)
    hs, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qd, kvd = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"]

    def matrix(role, layer, rows, cols):
        t = types[role]
        raw = synth_quantized(t, rows, cols, tensor_seed(seed, ROLE[role], layer), sigma, threads)
        m.set_tensor(ROLE[role], layer, t, rows, cols, raw)

    def ones(role, layer, n):
        m.set_tensor(ROLE[role], layer, F32, 1, n, np.ones(n, dtype=np.float32))

    matrix("TOKEN_EMBD", 0, cfg["vocab_size"], hs)
    matrix("OUTPUT", 0, cfg["vocab_size"], hs)
    ones("OUTPUT_NORM", 0, hs)
    for l in range(cfg["n_layers"]):
        ones("ATTN_NORM", l, hs)
        ones("FFN_NORM", l, hs)
        matrix("ATTN_Q", l, qd, hs)
        matrix("ATTN_K", l, kvd, hs)
        matrix("ATTN_V", l, kvd, hs)
        matrix("ATTN_OUTPUT", l, hs, qd)
        matrix("FFN_GATE", l, ff, hs)
        matrix("FFN_UP", l, ff, hs)
        matrix("FFN_DOWN", l, hs, ff)
    return m
