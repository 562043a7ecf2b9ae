"""Minimal GGUF (version 3) writer for the tests: metadata of scalar / string / numeric-array values and tensors given as
(name, shape in GGUF order [ne0, ne1, ...], ggml type id, raw bytes)."""
import struct

import numpy as np

_T = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "arr": 9, "u64": 10, "i64": 11, "f64": 12}
_FMT = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


def _s(b):
    e = b.encode("utf-8")
    return struct.pack("<Q", len(e)) + e


def _value(kind, v):
    t = _T[kind]
    if t == 8:
        return struct.pack("<I", t) + _s(v)
    if t == 9:
        inner, items = v
        it = _T[inner]
        body = b"".join(_s(x) if it == 8 else struct.pack(_FMT[it], x) for x in items)
        return struct.pack("<I", t) + struct.pack("<I", it) + struct.pack("<Q", len(items)) + body
    return struct.pack("<I", t) + struct.pack(_FMT[t], v)


def write_gguf(path, metadata, tensors, alignment=32):
    """metadata: list of (key, kind, value); tensors: list of (name, shape, ggml_type, bytes-like)."""
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(metadata))
    for key, kind, v in metadata:
        head += _s(key) + _value(kind, v)
    infos, blobs, off = b"", [], 0
    for name, shape, t, data in tensors:
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        infos += _s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape) + struct.pack("<IQ", t, off)
        blobs.append((off, data))
        off = (off + data.size + alignment - 1) // alignment * alignment
    head += infos
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        base = f.tell()
        for o, data in blobs:
            f.seek(base + o)
            f.write(data.tobytes())
        f.truncate(base + off)
