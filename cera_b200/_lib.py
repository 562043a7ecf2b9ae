"""ctypes binding of include/cera_cuda.h."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "libcera_cuda.so")


class CeraCudaError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"cera_cuda error {code}: {text}")
        self.code = code


if not os.path.exists(_PATH):
    raise ImportError(
        f"{_PATH} is missing: build it with `python cera_b200/build.py` (needs nvcc). "
        "cera_b200 has no CPU fallback.")

lib = C.CDLL(_PATH)

_p, _sz, _i32, _u32, _u64, _f = C.c_void_p, C.c_size_t, C.c_int32, C.c_uint32, C.c_uint64, C.c_float


class Config(C.Structure):
    _fields_ = [("n_layers", _u32), ("hidden_size", _u32), ("intermediate_size", _u32), ("n_heads", _u32),
                ("n_kv_heads", _u32), ("head_dim", _u32), ("vocab_size", _u32), ("max_seq_len", _u32),
                ("rope_theta", _f), ("rms_norm_eps", _f), ("rope_type", _i32), ("kv_f16", _i32), ("device", _i32),
                ("reserved", _i32), ("embedding_scale", _f), ("residual_scale", _f), ("attention_scale", _f),
                ("logit_scale", _f)]


# name -> (restype, argtypes); every symbol include/cera_cuda.h declares.
SIGNATURES = {
    "cera_cuda_last_error": (C.c_char_p, []),
    "cera_cuda_kernel_status": (_i32, [C.POINTER(_u32)]),
    "cera_cuda_device_count": (_i32, [C.POINTER(_i32)]),
    "cera_cuda_weight_create": (_i32, [_i32, _sz, _sz, _p, _sz, C.POINTER(_p)]),
    "cera_cuda_weight_free": (None, [_p]),
    "cera_cuda_weight_prepare_gemm": (_i32, [_p, C.POINTER(_i32)]),
    "cera_cuda_weight_info": (_i32, [_p, C.POINTER(_i32), C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz)]),
    "cera_cuda_dequantize_rows": (_i32, [_p, _sz, _sz, _p, _p]),
    "cera_cuda_quantize_q8_0": (_i32, [_p, _sz, _sz, _p, _p, _p, _p]),
    "cera_cuda_quantize_columns": (_i32, [_p, _sz, _sz, _p, _p, _p, _p]),
    "cera_cuda_gemv": (_i32, [_p, _p, _p, _p]),
    "cera_cuda_gemv_q5k_f32": (_i32, [_p, _p, _p, _p]),
    "cera_cuda_gemm_preq": (_i32, [_p, _p, _p, _p, _p, _sz, _sz, _sz, _p]),
    "cera_cuda_block_sums": (_i32, [_p, _sz, _p, _p, _p, _p]),
    "cera_cuda_rmsnorm": (_i32, [_p, _p, _sz, _f, _p, _p]),
    "cera_cuda_rmsnorm_q8_0": (_i32, [_p, _p, _sz, _f, _p, _p, _p, _p, _p]),
    "cera_cuda_silu_mul": (_i32, [_p, _p, _sz, _p]),
    "cera_cuda_rope": (_i32, [_p, _p, _sz, _sz, _sz, _sz, _f, _p, _i32, _p]),
    "cera_cuda_decode_attention_workspace_bytes": (_sz, [_sz, _sz, _sz]),
    "cera_cuda_decode_attention": (_i32, [_p, _p, _p, _i32, _sz, _sz, _sz, _sz, _f, _p, _p, _sz, _p]),
    "cera_cuda_prefill_attention": (_i32, [_p, _p, _p, _i32, _sz, _sz, _sz, _sz, _sz, _f, _p, _p]),
    "cera_cuda_decode_attention_noalloc": (_i32, [_p, _p, _p, _i32, _sz, _sz, _sz, _sz, _f, _p, _p]),
    "cera_cuda_synth_normal": (_i32, [_p, _sz, _u64, _u64, _f, _p]),
    "cera_cuda_quantize_weights": (_i32, [_i32, _p, _sz, _p, _p]),
    "cera_cuda_model_create": (_i32, [C.POINTER(Config), C.POINTER(_p)]),
    "cera_cuda_model_add_tensor": (_i32, [_p, _i32, _i32, _i32, _sz, _sz, _p, _sz]),
    "cera_cuda_model_finalize": (_i32, [_p]),
    "cera_cuda_model_set_tp": (_i32, [_p, _u32, _u32]),
    "cera_cuda_model_tp_handle": (_i32, [_p, _p, _sz]),
    "cera_cuda_model_tp_connect": (_i32, [_p, _p, _sz]),
    "cera_cuda_tp_wait_selftest": (_i32, [_u32, C.POINTER(_u32), C.POINTER(C.c_float)]),
    "cera_cuda_forward": (_i32, [_p, _u32, _sz, _p]),
    "cera_cuda_forward_greedy": (_i32, [_p, _u32, _sz, C.POINTER(_u32)]),
    "cera_cuda_generate_greedy": (_i32, [_p, _u32, _sz, _sz, _p, C.POINTER(_f)]),
    "cera_cuda_forward_prefill": (_i32, [_p, _p, _sz, _sz, _p]),
    "cera_cuda_truncate_kv": (_i32, [_p, _sz]),
    "cera_cuda_seq_len": (_sz, [_p]),
    "cera_cuda_memory_bytes": (_sz, [_p]),
    "cera_cuda_last_hidden": (_i32, [_p, _p]),
    "cera_cuda_launch_count": (_u64, [_p]),
    "cera_cuda_model_free": (None, [_p]),
    "cera_cuda_forward_prefill_logits_all": (_i32, [_p, _p, _sz, _sz, _p]),
    "cera_cuda_model_attach_lora": (_i32, [_p, _i32, _i32, _sz, _sz, _sz, _p, _p, _f]),
    "cera_cuda_model_detach_lora": (_i32, [_p]),
    "cera_cuda_kv_shift": (_i32, [_p, _sz, _sz]),
    "cera_cuda_kv_snapshot_bytes": (_sz, [_p]),
    "cera_cuda_kv_snapshot": (_i32, [_p, _p, _sz]),
    "cera_cuda_kv_restore": (_i32, [_p, _p, _sz]),
    "cera_cuda_kv_layer_bytes": (_sz, [_p]),
    "cera_cuda_kv_snapshot_layer": (_i32, [_p, _u32, _p, _p, _sz]),
    "cera_cuda_kv_restore_layer": (_i32, [_p, _u32, _p, _p, _sz, _sz]),
    "cera_cuda_moe_create": (_i32, [_u32, _u32, _u32, _u32, _i32, _p, _p, _p, _sz, _sz, _p, _p, _sz, C.POINTER(_p)]),
    "cera_cuda_moe_create_ep": (_i32, [_u32, _u32, _u32, _u32, _i32, _p, _p, _p, _sz, _sz, _p, _p, _sz, _u32, _u32, _sz,
                                       C.POINTER(_p)]),
    "cera_cuda_moe_ep_handle": (_i32, [_p, _p, _sz]),
    "cera_cuda_moe_ep_connect": (_i32, [_p, _p, _sz]),
    "cera_cuda_moe_ep_status": (_i32, [_p, C.POINTER(_u32)]),
    "cera_cuda_moe_ffn": (_i32, [_p, _p, _sz, _i32, _p, _p, _p, _p]),
    "cera_cuda_moe_memory_bytes": (_sz, [_p]),
    "cera_cuda_moe_free": (None, [_p]),
}

for _name, (_res, _args) in SIGNATURES.items():
    try:
        _fn = getattr(lib, _name)
    except AttributeError as e:  # the library does not export a declared symbol: stale build
        raise ImportError(f"{_PATH} does not export {_name}: rebuild it with `python cera_b200/build.py`") from e
    _fn.restype = _res
    _fn.argtypes = _args


def lib_path():
    return _PATH


def last_error():
    return lib.cera_cuda_last_error().decode("utf-8", "replace")


def check(code):
    if code != 0:
        raise CeraCudaError(code, last_error())


def kernel_status():
    """0 when no bounded device-side wait has run out on the current device."""
    v = _u32()
    lib.cera_cuda_kernel_status(C.byref(v))
    return v.value
