"""Host-side mirror of `trait Model` (cera/src/model/mod.rs:200-606) over the
C ABI: forward, forward_greedy, forward_prefill, truncate_kv, gpu_memory_bytes."""
import ctypes as C
import enum

import numpy as np

from ._lib import Config, check, lib


class Role(enum.IntEnum):
    TOKEN_EMBD = 0
    OUTPUT_NORM = 1
    OUTPUT = 2
    ATTN_NORM = 3
    ATTN_Q = 4
    ATTN_K = 5
    ATTN_V = 6
    ATTN_OUTPUT = 7
    FFN_NORM = 8
    FFN_GATE = 9
    FFN_UP = 10
    FFN_DOWN = 11
    ROPE_FREQS = 12


ModelConfig = Config


class CudaModel:
    def __init__(self, tp=None, **cfg):
        """tp = (rank, size): this process holds rank `rank` of a `size`-way row split (see tp.py)."""
        cfg.setdefault("device", 0)
        cfg.setdefault("rope_type", 0)
        cfg.setdefault("kv_f16", 0)
        self.cfg = Config(**cfg)
        self.handle = C.c_void_p()
        check(lib.cera_cuda_model_create(C.byref(self.cfg), C.byref(self.handle)))
        self.tp = tuple(tp) if tp else (0, 1)
        if self.tp[1] > 1:
            check(lib.cera_cuda_model_set_tp(self.handle, self.tp[0], self.tp[1]))

    def tp_handle(self):
        """64-byte handle of this rank's exchange region (after finalize)."""
        buf = (C.c_uint8 * 64)()
        check(lib.cera_cuda_model_tp_handle(self.handle, buf, 64))
        return bytes(buf)

    def tp_connect(self, handles):
        """handles: the tp_handle() of every rank, in rank order."""
        blob = b"".join(handles)
        check(lib.cera_cuda_model_tp_connect(self.handle, blob, len(handles)))

    def config(self):
        return self.cfg

    def add_tensor(self, role, layer, ggml_type, rows, cols, data):
        """data: numpy array / bytes (host) or a torch CUDA tensor (device) of raw GGUF bytes."""
        if isinstance(data, (bytes, bytearray)):
            data = np.frombuffer(data, dtype=np.uint8)
        if isinstance(data, np.ndarray):
            data = np.ascontiguousarray(data)
            ptr, nbytes = data.ctypes.data, data.nbytes
        else:
            data = data.contiguous()
            ptr, nbytes = data.data_ptr(), data.numel() * data.element_size()
        check(lib.cera_cuda_model_add_tensor(self.handle, int(role), layer, ggml_type, rows, cols, C.c_void_p(ptr),
                                             nbytes))

    def finalize(self):
        check(lib.cera_cuda_model_finalize(self.handle))

    def forward(self, token, pos):
        logits = np.empty(self.cfg.vocab_size, dtype=np.float32)
        check(lib.cera_cuda_forward(self.handle, token, pos, logits.ctypes.data_as(C.c_void_p)))
        return logits

    def forward_greedy(self, token, pos):
        out = C.c_uint32()
        check(lib.cera_cuda_forward_greedy(self.handle, token, pos, C.byref(out)))
        return out.value

    def generate_greedy(self, first_token, start_pos, n):
        """n greedy tokens decoded on the device back to back -> (tokens, device milliseconds)."""
        out = np.empty(n, dtype=np.uint32)
        ms = C.c_float()
        check(lib.cera_cuda_generate_greedy(self.handle, first_token, start_pos, n, out.ctypes.data_as(C.c_void_p),
                                            C.byref(ms)))
        return out, ms.value

    def forward_prefill(self, tokens, start_pos, want_logits=True):
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits = np.empty(self.cfg.vocab_size, dtype=np.float32) if want_logits else None
        check(lib.cera_cuda_forward_prefill(self.handle, tokens.ctypes.data_as(C.c_void_p), tokens.size, start_pos,
                                            logits.ctypes.data_as(C.c_void_p) if want_logits else None))
        return logits

    def forward_prefill_logits_all(self, tokens, start_pos):
        """Logits of every prompt position -> float32 [n, vocab]."""
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = np.empty((tokens.size, self.cfg.vocab_size), dtype=np.float32)
        check(lib.cera_cuda_forward_prefill_logits_all(self.handle, tokens.ctypes.data_as(C.c_void_p), tokens.size, start_pos,
                                                       out.ctypes.data_as(C.c_void_p)))
        return out

    def truncate_kv(self, n):
        check(lib.cera_cuda_truncate_kv(self.handle, n))

    LORA_TARGETS = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")

    def attach_lora(self, target, layer, a, b, scale):
        """y = W x + scale * B (A x) for one projection: a [rank, k], b [d, rank] float32 (numpy)."""
        t = self.LORA_TARGETS.index(target) if isinstance(target, str) else int(target)
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        if a.ndim != 2 or b.ndim != 2 or b.shape[1] != a.shape[0]:
            raise ValueError("a must be [rank, k] and b [d, rank]")
        check(lib.cera_cuda_model_attach_lora(self.handle, t, layer, a.shape[0], a.shape[1], b.shape[0],
                                              a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), scale))

    def detach_lora(self):
        check(lib.cera_cuda_model_detach_lora(self.handle))

    def shift_kv(self, n_keep, shift):
        """Model::shift_kv: drop positions [n_keep, n_keep + shift) and re-rotate the keys that move down."""
        check(lib.cera_cuda_kv_shift(self.handle, n_keep, shift))

    def snapshot(self):
        """The KV cache up to seq_len as bytes (restore() puts it back, seq_len included)."""
        n = lib.cera_cuda_kv_snapshot_bytes(self.handle)
        buf = np.empty(n, dtype=np.uint8)
        check(lib.cera_cuda_kv_snapshot(self.handle, buf.ctypes.data_as(C.c_void_p), n))
        return buf

    def restore(self, snap):
        snap = np.ascontiguousarray(snap, dtype=np.uint8)
        check(lib.cera_cuda_kv_restore(self.handle, snap.ctypes.data_as(C.c_void_p), snap.size))

    def state_snapshot(self):
        """The reference's StateSnapshot shape (cera/src/kv_cache.rs:1379-1421): {"seq_len", "layers": [(k_data, v_data)]},
        raw little-endian rows in the cache's element type."""
        n = lib.cera_cuda_kv_layer_bytes(self.handle)
        layers = []
        for l in range(self.cfg.n_layers):
            k, v = np.empty(n, dtype=np.uint8), np.empty(n, dtype=np.uint8)
            check(lib.cera_cuda_kv_snapshot_layer(self.handle, l, k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p), n))
            layers.append((k, v))
        return {"seq_len": self.seq_len, "layers": layers}

    def restore_state(self, snap):
        for l, (k, v) in enumerate(snap["layers"]):
            k, v = np.ascontiguousarray(k, dtype=np.uint8), np.ascontiguousarray(v, dtype=np.uint8)
            check(lib.cera_cuda_kv_restore_layer(self.handle, l, k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p), k.size,
                                                 snap["seq_len"]))

    @property
    def seq_len(self):
        return lib.cera_cuda_seq_len(self.handle)

    def gpu_memory_bytes(self):
        return lib.cera_cuda_memory_bytes(self.handle)

    def launch_count(self):
        return lib.cera_cuda_launch_count(self.handle)

    def last_hidden(self):
        out = np.empty(self.cfg.hidden_size, dtype=np.float32)
        check(lib.cera_cuda_last_hidden(self.handle, out.ctypes.data_as(C.c_void_p)))
        return out

    def close(self):
        if getattr(self, "handle", None):
            lib.cera_cuda_model_free(self.handle)
            self.handle = None

    __del__ = close
