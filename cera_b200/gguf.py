"""GGUF (version 3) reader and the llama-architecture load path onto the CUDA device.

What cera's loader does for a device backend (cera/src/gguf.rs:425-560 header, metadata and tensor
table; 724-813 tensor_data / tensor_meta_expert; cera/src/model/llama.rs:158-450 which metadata keys
and tensor names a dense llama / qwen / granite model reads; cera/src/model/gpu_weight_source.rs:40-118
the surface a device loader walks) restated above the C ABI: the file is mapped, never copied, and every
tensor's raw block bytes go to cera_cuda_model_add_tensor exactly as stored, which copies them to the
device before it returns (a tensor-parallel model keeps only its rank's rows of the split matrices).

Only what the decode path needs is interpreted; tokenizer and chat-template metadata stay as parsed
values in `GgufFile.metadata` for the caller.
"""
import mmap
import struct

import numpy as np

from .model import CudaModel, Role

GGUF_MAGIC = 0x46554747  # "GGUF", little endian
# ggml type id -> (elements per block, bytes per block); ids as in cera/src/convert/writer.rs:23-37
BLOCKS = {0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210), 30: (1, 2)}
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class GgufError(ValueError):
    pass


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GgufError("GGUF header runs past the end of the file")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self):
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GgufError("GGUF string runs past the end of the file")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, type_id):
        if type_id in _SCALARS:
            return self.take(_SCALARS[type_id])
        if type_id == 8:
            return self.string()
        if type_id == 9:
            inner, count = self.take("<I"), self.take("<Q")
            if inner in _SCALARS and inner != 7:  # numeric arrays in one go
                fmt = _SCALARS[inner]
                size = struct.calcsize(fmt)
                if self.pos + size * count > len(self.buf):
                    raise GgufError("GGUF array runs past the end of the file")
                arr = np.frombuffer(self.buf, dtype=np.dtype(fmt), count=count, offset=self.pos).copy()
                self.pos += size * count
                return arr
            return [self.value(inner) for _ in range(count)]
        raise GgufError(f"unknown GGUF value type {type_id}")


def tensor_nbytes(shape, ggml_type):
    """Bytes of a tensor stored as rows of blocks (cera/src/gguf.rs:304-330)."""
    if ggml_type not in BLOCKS:
        raise GgufError(f"ggml type {ggml_type} is not supported")
    elems, bsz = BLOCKS[ggml_type]
    if not shape:
        return 0
    if shape[0] % elems:
        raise GgufError(f"row length {shape[0]} is not a whole number of {elems}-element blocks")
    n = 1
    for d in shape:
        n *= d
    return n // elems * bsz


class GgufFile:
    """A mapped GGUF file: `.metadata` (key -> value) and `.tensors` (name -> (shape, ggml_type, offset, nbytes))."""

    def __init__(self, path):
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        buf = memoryview(self._map)
        r = _Reader(buf)
        magic = r.take("<I")
        if magic != GGUF_MAGIC:
            raise GgufError(f"not a GGUF file (magic 0x{magic:08X})")
        version = r.take("<I")
        if version != 3:
            raise GgufError(f"unsupported GGUF version {version} (expected 3)")
        n_tensors, n_kv = r.take("<Q"), r.take("<Q")
        self.metadata = {}
        for _ in range(n_kv):
            key = r.string()
            self.metadata[key] = r.value(r.take("<I"))
        raw = []
        for _ in range(n_tensors):
            name = r.string()
            n_dims = r.take("<I")
            if n_dims > 8:
                raise GgufError(f"tensor {name} has too many dimensions: {n_dims}")
            shape = [r.take("<Q") for _ in range(n_dims)]
            raw.append((name, shape, r.take("<I"), r.take("<Q")))
        alignment = int(self.metadata.get("general.alignment", 32))
        if not 0 < alignment <= 1024 * 1024:
            raise GgufError(f"invalid GGUF alignment: {alignment}")
        self.data_offset = (r.pos + alignment - 1) // alignment * alignment
        self.tensors = {}
        for name, shape, t, off in raw:
            nbytes = tensor_nbytes(shape, t)
            start = self.data_offset + off
            if start + nbytes > len(buf):
                raise GgufError(f"tensor {name} extends past the end of the file")
            self.tensors[name] = (shape, t, start, nbytes)
        self._buf = buf

    def close(self):
        self._buf.release()
        self._map.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def has(self, name):
        return name in self.tensors

    def tensor_meta(self, name):
        """(rows, cols, ggml_type): GGUF stores ne0 = row length first (cera/src/gguf.rs:740-750)."""
        shape, t, _, _ = self.tensors[name]
        if len(shape) == 1:
            return 1, shape[0], t
        if len(shape) == 2:
            return shape[1], shape[0], t
        raise GgufError(f"tensor {name} has rank {len(shape)}, expected 1 or 2")

    def tensor_bytes(self, name, row0=0, n_rows=None):
        """Raw block bytes of rows [row0, row0 + n_rows) as a numpy view into the mapping."""
        shape, t, start, nbytes = self.tensors[name]
        rows, cols, _ = self.tensor_meta(name)
        row_bytes = nbytes // rows
        n_rows = rows - row0 if n_rows is None else n_rows
        if row0 + n_rows > rows:
            raise GgufError(f"rows [{row0}, {row0 + n_rows}) outside tensor {name} of {rows} rows")
        return np.frombuffer(self._buf, dtype=np.uint8, count=n_rows * row_bytes, offset=start + row0 * row_bytes)

    def expert_meta(self, name, expert):
        """(offset, nbytes, rows, cols, ggml_type) of one expert of a stacked rank-3 tensor (cera/src/gguf.rs:779-813)."""
        shape, t, start, nbytes = self.tensors[name]
        if len(shape) != 3:
            raise GgufError(f"{name} must be rank 3, got rank {len(shape)}")
        ne0, ne1, n_expert = shape
        if not 0 <= expert < n_expert:
            raise GgufError(f"expert {expert} out of range for {name} ({n_expert} experts)")
        slice_bytes = tensor_nbytes([ne0, ne1], t)
        off = start + expert * slice_bytes
        if off + slice_bytes > start + nbytes:
            raise GgufError(f"tensor {name} expert {expert} slice extends past the tensor")
        return off, slice_bytes, ne1, ne0, t

    def expert_bytes(self, name, expert):
        off, n, _, _, _ = self.expert_meta(name, expert)
        return np.frombuffer(self._buf, dtype=np.uint8, count=n, offset=off)


def llama_config(g):
    """ModelConfig fields from the metadata keys LlamaModel::from_gguf reads (cera/src/model/llama.rs:158-260)."""
    arch = g.metadata.get("general.architecture", "llama")

    def need(key):
        full = f"{arch}.{key}"
        if full not in g.metadata:
            raise GgufError(f"missing metadata key {full}")
        return g.metadata[full]

    hidden, n_heads = int(need("embedding_length")), int(need("attention.head_count"))
    head_dim = int(g.metadata.get(f"{arch}.attention.key_length", hidden // n_heads))
    rows, _, _ = g.tensor_meta("token_embd.weight")
    return dict(n_layers=int(need("block_count")), hidden_size=hidden, intermediate_size=int(need("feed_forward_length")),
                n_heads=n_heads, n_kv_heads=int(g.metadata.get(f"{arch}.attention.head_count_kv", n_heads)), head_dim=head_dim,
                vocab_size=int(g.metadata.get(f"{arch}.vocab_size", rows)),
                rope_theta=float(g.metadata.get(f"{arch}.rope.freq_base", 10000.0)),
                rms_norm_eps=float(need("attention.layer_norm_rms_epsilon")),
                rope_type=1 if arch in ("qwen2", "qwen3") else 0,
                # Granite's scalar multipliers (cera/src/model/mod.rs:84-111): absent keys are identity (0 here)
                embedding_scale=float(g.metadata.get(f"{arch}.embedding_scale", 0.0)),
                residual_scale=float(g.metadata.get(f"{arch}.residual_scale", 0.0)),
                attention_scale=float(g.metadata.get(f"{arch}.attention.scale", 0.0)),
                logit_scale=float(g.metadata.get(f"{arch}.logit_scale", 0.0))), int(g.metadata.get(f"{arch}.context_length", 4096))


_LAYER_TENSORS = [("attn_norm", Role.ATTN_NORM), ("attn_q", Role.ATTN_Q), ("attn_k", Role.ATTN_K), ("attn_v", Role.ATTN_V),
                  ("attn_output", Role.ATTN_OUTPUT), ("ffn_norm", Role.FFN_NORM), ("ffn_gate", Role.FFN_GATE),
                  ("ffn_up", Role.FFN_UP), ("ffn_down", Role.FFN_DOWN)]


def load_llama(path, max_seq_len=None, kv_f16=0, device=0, tp=None):
    """A finalized CudaModel holding the tensors of a dense llama-architecture GGUF file.
    tp = (rank, size): this process keeps only its rows of every split matrix (connect the ranks afterwards)."""
    with GgufFile(path) as g:
        cfg, ctx = llama_config(g)
        model = CudaModel(**cfg, max_seq_len=max_seq_len or ctx, kv_f16=kv_f16, device=device, tp=tp)

        def put(name, role, layer):
            # the whole tensor, as the mapping holds it: a tensor-parallel model copies only its rank's rows to the device
            rows, cols, t = g.tensor_meta(name)
            model.add_tensor(role, layer, t, rows, cols, g.tensor_bytes(name))

        put("token_embd.weight", Role.TOKEN_EMBD, 0)
        put("output_norm.weight", Role.OUTPUT_NORM, 0)
        if g.has("output.weight"):
            put("output.weight", Role.OUTPUT, 0)
        if g.has("rope_freqs.weight"):
            put("rope_freqs.weight", Role.ROPE_FREQS, 0)
        for layer in range(cfg["n_layers"]):
            for stem, role in _LAYER_TENSORS:
                put(f"blk.{layer}.{stem}.weight", role, layer)
        model.finalize()
        return model
