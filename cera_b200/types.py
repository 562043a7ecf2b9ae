"""GGML tensor type ids and block geometry (cera/src/tensor.rs:3-62,
cera/src/convert/writer.rs:23-37)."""

F32, F16, Q4_0, Q4_1, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 2, 3, 8, 12, 13, 14, 30
QUANT_TYPES = (Q4_0, Q4_1, Q8_0, Q4_K, Q5_K, Q6_K)
TYPE_NAMES = {F32: "f32", F16: "f16", BF16: "bf16", Q4_0: "q4_0", Q4_1: "q4_1", Q8_0: "q8_0", Q4_K: "q4_k",
              Q5_K: "q5_k", Q6_K: "q6_k"}
# type -> (elements per block, bytes per block)
BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q4_0: (32, 18), Q4_1: (32, 20), Q8_0: (32, 34),
         Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}


def row_bytes(ggml_type: int, k: int) -> int:
    elems, nbytes = BLOCK[ggml_type]
    if k % elems:
        raise ValueError(f"k={k} is not a multiple of the block width {elems}")
    return k // elems * nbytes
