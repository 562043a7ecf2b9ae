"""cera_b200: the B200 (sm_100a) CUDA device for cera's quantized decode hot path.

Host-side mirror of the reference's operator interface over the C ABI in
include/cera_cuda.h.  Importing the package loads cera_b200/libcera_cuda.so
and fails loudly when it has not been built; there is no CPU fallback.
"""
from . import _lib  # noqa: F401  (loads the shared library or raises)
from ._lib import CeraCudaError, last_error, lib_path  # noqa: F401
from .types import (F16, F32, BF16, Q4_0, Q4_1, Q4_K, Q5_K, Q6_K, Q8_0, BLOCK, QUANT_TYPES, TYPE_NAMES,  # noqa: F401
                    row_bytes)
from .ops import (MoeFfn, QuantWeight, Q8Activations, decode_attention, decode_attention_noalloc, dequantize_rows, gemm_preq, gemv, gemv_q5k_f32, prefill_attention,  # noqa: F401
                  block_sums, quantize_columns, quantize_q8_0, quantize_weights, rmsnorm, rmsnorm_q8_0, rope, silu_mul,
                  synth_normal)
from .model import CudaModel, ModelConfig, Role  # noqa: F401
