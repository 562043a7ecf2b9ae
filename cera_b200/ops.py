"""Operator-level interface, named after the reference's own functions
(cera/src/model/transformer.rs: gemv 450-453, gemm_preq 710-788,
quantize_columns 865-946, decode_attention 1249-1305).

Tensors are torch CUDA tensors used purely as device memory; every function
hands raw device pointers to the C ABI and launches on torch's current stream.
"""
import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import check, lib
from .types import BLOCK, row_bytes


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _dev(t, dtype):
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise TypeError("expected a CUDA tensor: this path has no CPU fallback")
    if t.dtype != dtype or not t.is_contiguous():
        raise TypeError(f"expected a contiguous {dtype} tensor, got {t.dtype}")
    return t


class QuantWeight:
    """A device-resident quantized [m x k] matrix (the device form of a WeightRef,
    cera/src/model/transformer.rs:127-231).  `raw` holds GGUF block bytes: a
    uint8 torch tensor (CPU or CUDA), a numpy uint8 array or bytes."""

    def __init__(self, ggml_type, m, k, raw):
        import numpy as np
        if isinstance(raw, (bytes, bytearray)):
            raw = np.frombuffer(raw, dtype=np.uint8)
        if isinstance(raw, np.ndarray):
            raw = np.ascontiguousarray(raw, dtype=np.uint8)
            ptr, nbytes, keep = raw.ctypes.data, raw.size, raw
        else:
            raw = raw.contiguous()
            ptr, nbytes, keep = raw.data_ptr(), raw.numel() * raw.element_size(), raw
        h = C.c_void_p()
        check(lib.cera_cuda_weight_create(ggml_type, m, k, C.c_void_p(ptr), nbytes, C.byref(h)))
        del keep
        self.handle, self.type, self.m, self.k = h, ggml_type, m, k

    def prepare_gemm(self):
        """Build the resident f16 operand image for many-column GEMMs (K-quants, k a multiple of 256; about 2.3 extra
        bytes per weight, 4 for Q6_K).  True when the weight now holds one; without it the GEMM converts on the fly
        (Q6_K: runs the warp-level kernel), same results within tolerance."""
        has = C.c_int32(0)
        check(lib.cera_cuda_weight_prepare_gemm(self.handle, C.byref(has)))
        return bool(has.value)

    def device_bytes(self):
        """Device memory the weight holds: its planes, the one-column scratch and, once built, the operand image."""
        n = C.c_size_t(0)
        check(lib.cera_cuda_weight_info(self.handle, None, None, None, C.byref(n)))
        return int(n.value)

    def close(self):
        if getattr(self, "handle", None):
            lib.cera_cuda_weight_free(self.handle)
            self.handle = None

    __del__ = close


class Q8Activations:
    """Q8_0 activation columns in the reference's SoA layout
    (cera/src/model/transformer.rs:857-860) plus the 16-wide quant sums."""

    def __init__(self, k, n, device="cuda"):
        self.k, self.n = k, n
        self.scales = torch.empty(n * (k // 32), dtype=torch.float32, device=device)
        self.quants = torch.empty(n * k, dtype=torch.int8, device=device)
        self.sums = torch.empty(n * (k // 16), dtype=torch.int16, device=device)


def quantize_q8_0(x, k=None, n=1):
    """x: n contiguous columns of length k (f32).  -> Q8Activations."""
    x = _dev(x, torch.float32)
    k = k or x.numel() // n
    a = Q8Activations(k, n, x.device)
    check(lib.cera_cuda_quantize_q8_0(_ptr(x), k, n, _ptr(a.scales), _ptr(a.quants), _ptr(a.sums), _stream()))
    return a


def quantize_columns(mat, dim, n):
    """mat: [dim x n] row stride n (token j = column j)."""
    mat = _dev(mat, torch.float32)
    a = Q8Activations(dim, n, mat.device)
    check(lib.cera_cuda_quantize_columns(_ptr(mat), dim, n, _ptr(a.scales), _ptr(a.quants), _ptr(a.sums), _stream()))
    return a


def gemv(w: QuantWeight, x, y=None):
    x = _dev(x, torch.float32)
    if x.numel() != w.k:
        raise ValueError(f"gemv: x has {x.numel()} elements, weight k is {w.k}")
    y = y if y is not None else torch.empty(w.m, dtype=torch.float32, device=x.device)
    check(lib.cera_cuda_gemv(w.handle, _ptr(x), _ptr(_dev(y, torch.float32)), _stream()))
    return y


def gemv_q5k_f32(w: QuantWeight, x, y=None):
    x = _dev(x, torch.float32)
    y = y if y is not None else torch.empty(w.m, dtype=torch.float32, device=x.device)
    check(lib.cera_cuda_gemv_q5k_f32(w.handle, _ptr(x), _ptr(y), _stream()))
    return y


def gemm_preq(w: QuantWeight, acts: Q8Activations, out=None):
    """out[m x n] = W * X for pre-quantized columns."""
    out = out if out is not None else torch.empty(w.m, acts.n, dtype=torch.float32, device=acts.quants.device)
    check(lib.cera_cuda_gemm_preq(w.handle, _ptr(acts.scales), _ptr(acts.quants), _ptr(acts.sums), _ptr(out), w.m,
                                  acts.n, acts.k, _stream()))
    return out


def block_sums(w: QuantWeight, row, quants):
    quants = _dev(quants, torch.int8)
    u = torch.empty(w.k // 16, dtype=torch.int32, device=quants.device)
    a = torch.empty(w.k // 16, dtype=torch.int32, device=quants.device)
    check(lib.cera_cuda_block_sums(w.handle, row, _ptr(quants), _ptr(u), _ptr(a), _stream()))
    return u, a


def dequantize_rows(w: QuantWeight, row0=0, nrows=None):
    nrows = w.m - row0 if nrows is None else nrows
    out = torch.empty(nrows, w.k, dtype=torch.float32, device="cuda")
    check(lib.cera_cuda_dequantize_rows(w.handle, row0, nrows, _ptr(out), _stream()))
    return out


def rmsnorm(x, weight, eps):
    x = _dev(x, torch.float32)
    out = torch.empty_like(x)
    check(lib.cera_cuda_rmsnorm(_ptr(x), _ptr(_dev(weight, torch.float32)), x.numel(), eps, _ptr(out), _stream()))
    return out


def rmsnorm_q8_0(x, weight, eps):
    """RMSNorm and the Q8_0 quantizer in one launch -> (normed f32, Q8Activations)."""
    x = _dev(x, torch.float32)
    out = torch.empty_like(x)
    acts = Q8Activations(x.numel(), 1, device=x.device)
    check(lib.cera_cuda_rmsnorm_q8_0(_ptr(x), _ptr(_dev(weight, torch.float32)), x.numel(), eps, _ptr(out),
                                     _ptr(acts.scales), _ptr(acts.quants), _ptr(acts.sums), _stream()))
    return out, acts


def silu_mul(gate, up):
    gate = _dev(gate, torch.float32).clone()
    check(lib.cera_cuda_silu_mul(_ptr(gate), _ptr(_dev(up, torch.float32)), gate.numel(), _stream()))
    return gate


def rope(q, k, pos, n_heads, n_kv_heads, head_dim, freq_base, freq_factors=None, rope_type=0):
    q = _dev(q, torch.float32).clone()
    k = _dev(k, torch.float32).clone()
    check(lib.cera_cuda_rope(_ptr(q), _ptr(k), pos, n_heads, n_kv_heads, head_dim, freq_base, _ptr(freq_factors),
                             rope_type, _stream()))
    return q, k


def decode_attention(q, k_cache, v_cache, n_heads, n_kv_heads, head_dim, seq_len, scale, workspace=None):
    """k_cache / v_cache: time-major rows of n_kv_heads*head_dim, float32 or float16."""
    q = _dev(q, torch.float32)
    f16 = k_cache.dtype == torch.float16
    if v_cache.dtype != k_cache.dtype or k_cache.dtype not in (torch.float16, torch.float32):
        raise TypeError("KV caches must both be float32 or both float16")
    need = lib.cera_cuda_decode_attention_workspace_bytes(n_heads, head_dim, seq_len)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    out = torch.empty(n_heads * head_dim, dtype=torch.float32, device=q.device)
    check(lib.cera_cuda_decode_attention(_ptr(q), _ptr(k_cache), _ptr(v_cache), int(f16), n_heads, n_kv_heads,
                                         head_dim, seq_len, scale, _ptr(out), _ptr(workspace), workspace.numel(),
                                         _stream()))
    return out


def prefill_attention(q, k_cache, v_cache, n_heads, n_kv_heads, head_dim, n, start_pos, scale):
    """Causal attention of n prompt tokens; q is token-major [n][n_heads*head_dim]
    (cera/src/backend/cpu.rs:4028-4241 flash_attention_gqa_cpu)."""
    q = _dev(q, torch.float32)
    f16 = k_cache.dtype == torch.float16
    out = torch.empty(n * n_heads * head_dim, dtype=torch.float32, device=q.device)
    check(lib.cera_cuda_prefill_attention(_ptr(q), _ptr(k_cache), _ptr(v_cache), int(f16), n_heads, n_kv_heads, head_dim, n,
                                          start_pos, scale, _ptr(out), _stream()))
    return out.reshape(n, n_heads * head_dim)


def decode_attention_noalloc(q, k_cache, v_cache, n_heads, n_kv_heads, head_dim, seq_len, scale, out=None):
    """decode_attention for callers that may not allocate device memory: the split-KV workspace is the
    library's built-in array (n_heads <= 64, head_dim <= 128).  Pass `out` to make the call allocation-free
    on the Python side too.  Calls on different streams must not overlap: they share the array."""
    q = _dev(q, torch.float32)
    f16 = k_cache.dtype == torch.float16
    if v_cache.dtype != k_cache.dtype or k_cache.dtype not in (torch.float16, torch.float32):
        raise TypeError("KV caches must both be float32 or both float16")
    if out is None:
        out = torch.empty(n_heads * head_dim, dtype=torch.float32, device=q.device)
    check(lib.cera_cuda_decode_attention_noalloc(_ptr(q), _ptr(k_cache), _ptr(v_cache), int(f16), n_heads, n_kv_heads,
                                                 head_dim, seq_len, scale, _ptr(_dev(out, torch.float32)), _stream()))
    return out


def synth_normal(n, seed, sigma, offset=0, device="cuda"):
    out = torch.empty(n, dtype=torch.float32, device=device)
    check(lib.cera_cuda_synth_normal(_ptr(out), n, seed, offset, sigma, _stream()))
    return out


def quantize_weights(ggml_type, w):
    """f32 device tensor -> uint8 device tensor of GGUF blocks."""
    w = _dev(w, torch.float32)
    elems, nbytes = BLOCK[ggml_type]
    out = torch.empty(w.numel() // elems * nbytes, dtype=torch.uint8, device=w.device)
    check(lib.cera_cuda_quantize_weights(ggml_type, _ptr(w), w.numel(), _ptr(out), _stream()))
    return out


__all__ = [n for n in dir() if not n.startswith("_")]
_ = (_lib, row_bytes)


class MoeFfn:
    """Routed feed-forward of one lfm2moe layer (cera/src/model/lfm2.rs:735-901 forward_moe_ffn):
    stacked expert tensors, F32 router, optional selection bias.  Byte tensors are raw GGUF blocks
    (CUDA uint8 tensors or numpy arrays)."""

    def __init__(self, n_expert, n_used, hidden, ff, ggml_type, gate_exps, up_exps, down_exps, router, exp_probs_b=None,
                 max_tokens=512, ep=None, max_total_tokens=None):
        """ep = (rank, size): expert-parallel rank of a group of processes, one GPU each; connect with
        cera_b200.tp.connect(moe) before the first call, then every call is collective."""
        def raw(a):
            if isinstance(a, torch.Tensor):
                a = a.contiguous()
                return a, C.c_void_p(a.data_ptr()), a.numel() * a.element_size()
            a = np.ascontiguousarray(a)
            return a, C.c_void_p(a.ctypes.data), a.nbytes
        keep = [raw(gate_exps), raw(up_exps), raw(down_exps), raw(router)]
        if keep[0][2] != keep[1][2]:
            raise ValueError("gate and up expert tensors differ in size")
        bias = raw(exp_probs_b) if exp_probs_b is not None else (None, None, 0)
        self.handle = C.c_void_p()
        self.n_expert, self.n_used, self.hidden, self.ff = n_expert, n_used, hidden, ff
        self.tp = tuple(ep) if ep else (0, 1)
        if self.tp[1] > 1:
            check(lib.cera_cuda_moe_create_ep(n_expert, n_used, hidden, ff, ggml_type, keep[0][1], keep[1][1], keep[2][1],
                                              keep[0][2], keep[2][2], keep[3][1], bias[1], max_tokens, self.tp[0], self.tp[1],
                                              max_total_tokens or max_tokens * self.tp[1], C.byref(self.handle)))
        else:
            check(lib.cera_cuda_moe_create(n_expert, n_used, hidden, ff, ggml_type, keep[0][1], keep[1][1], keep[2][1],
                                           keep[0][2], keep[2][2], keep[3][1], bias[1], max_tokens, C.byref(self.handle)))

    def tp_handle(self):
        buf = (C.c_uint8 * 64)()
        check(lib.cera_cuda_moe_ep_handle(self.handle, buf, 64))
        return bytes(buf)

    def tp_connect(self, handles):
        check(lib.cera_cuda_moe_ep_connect(self.handle, b"".join(handles), len(handles)))

    def check_status(self):
        """After synchronising: raises if a wait on a peer ran out during an earlier call."""
        st = C.c_uint32()
        check(lib.cera_cuda_moe_ep_status(self.handle, C.byref(st)))

    def __call__(self, x, softmax_gate=False, want_routing=False):
        """x: CUDA f32 [n, hidden] -> out [n, hidden] (and ids [n, n_used], weights [n, n_used])."""
        x = _dev(x, torch.float32).contiguous().view(-1, self.hidden)
        n = x.shape[0]
        out = torch.empty_like(x)
        ids = torch.empty(n, self.n_used, dtype=torch.int32, device=x.device) if want_routing else None
        wts = torch.empty(n, self.n_used, dtype=torch.float32, device=x.device) if want_routing else None
        check(lib.cera_cuda_moe_ffn(self.handle, _ptr(x), n, 1 if softmax_gate else 0, _ptr(out), _ptr(ids), _ptr(wts), _stream()))
        return (out, ids, wts) if want_routing else out

    def memory_bytes(self):
        return lib.cera_cuda_moe_memory_bytes(self.handle)

    def close(self):
        if getattr(self, "handle", None):
            lib.cera_cuda_moe_free(self.handle)
            self.handle = None

    __del__ = close
