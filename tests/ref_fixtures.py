"""The reference's deterministic test fixtures, restated.

Generators follow cera/src/backend/simd.rs:6420-6568 (the LCG, the Q8_0 rows
that force -128 weights, the Q4_0 / Q4_1 / K-quant rows with controlled scale
fields, and the activations pinned at +/-127) so the oracle is exercised on the
same inputs the reference's own kernel tests use.
"""
import numpy as np

M64 = (1 << 64) - 1


class Lcg:
    def __init__(self, seed):
        self.st = seed & M64

    def next(self):
        self.st = (self.st * 6364136223846793005 + 1442695040888963407) & M64
        return self.st >> 33


def _h(v):
    return int(np.array([v], dtype=np.float32).astype(np.float16).view(np.uint16)[0])


def _f32(v):
    return float(np.float32(v))


def q8_0_rows_with_extremes(m, k, rng):
    out = bytearray()
    for blk in range(m * (k // 32)):
        h = _h(np.float32(0.01) + np.float32(0.003) * np.float32(blk % 5))
        out += bytes([h & 0xFF, h >> 8])
        for t in range(32):
            if t in (0, 1):
                q = -128
            elif t in (2, 3):
                q = 127
            elif t == 4:
                q = -127
            else:
                q = rng.next() % 256
            out.append(q & 0xFF)
    return np.frombuffer(bytes(out), dtype=np.uint8).copy()


def q4_0_rows(m, k, rng):
    out = bytearray()
    for blk in range(m * (k // 32)):
        h = _h(np.float32(0.01) + np.float32(0.004) * np.float32(blk % 7))
        out += bytes([h & 0xFF, h >> 8])
        for _ in range(16):
            out.append(rng.next() % 256)
    return np.frombuffer(bytes(out), dtype=np.uint8).copy()


def q4_1_rows(m, k, rng):
    out = bytearray()
    for blk in range(m * (k // 32)):
        h = _h(np.float32(0.01) + np.float32(0.004) * np.float32(blk % 7))
        mm = _h(np.float32(-0.05) + np.float32(0.02) * np.float32(blk % 5))
        out += bytes([h & 0xFF, h >> 8, mm & 0xFF, mm >> 8])
        for _ in range(16):
            out.append(rng.next() % 256)
    return np.frombuffer(bytes(out), dtype=np.uint8).copy()


def k_quant_rows(m, sb, rng):
    q4 = bytearray()
    for bi in range(m * sb):
        d = _h(np.float32(0.01) + np.float32(0.005) * np.float32(bi % 7))
        dm = _h(np.float32(0.02) + np.float32(0.003) * np.float32(bi % 5))
        q4 += bytes([d & 0xFF, d >> 8, dm & 0xFF, dm >> 8])
        for _ in range(140):
            q4.append(rng.next() % 256)
    q6 = bytearray()
    for bi in range(m * sb):
        for _ in range(208):
            q6.append(rng.next() % 256)
        d = _h(np.float32(0.01) + np.float32(0.004) * np.float32(bi % 6))
        q6 += bytes([d & 0xFF, d >> 8])
    return (np.frombuffer(bytes(q4), dtype=np.uint8).copy(), np.frombuffer(bytes(q6), dtype=np.uint8).copy())


def activations(n, k, rng):
    nb = k // 32
    scales = np.zeros(n * nb, dtype=np.float32)
    quants = np.zeros(n * k, dtype=np.int8)
    for j in range(n):
        for b in range(nb):
            scales[j * nb + b] = np.float32(0.02) + np.float32(0.001) * np.float32((j + b) % 9)
            for t in range(32):
                if t in (0, 1):
                    q = 127
                elif t in (2, 3):
                    q = -127
                else:
                    q = (rng.next() % 255) - 127
                quants[j * k + b * 32 + t] = q
    return scales, quants


def ref_gemm(weights, bs, bq, m, n, k, q4):
    """Exact integer reference (cera/src/backend/simd.rs:6437-6465)."""
    nb = k // 32
    bsz = 18 if q4 else 34
    out = np.zeros((m, n), dtype=np.float32)
    w = weights.reshape(m, nb, bsz)
    d = (w[:, :, 0].astype(np.uint16) | (w[:, :, 1].astype(np.uint16) << 8)).view(np.float16).astype(np.float32)
    if q4:
        qs = w[:, :, 2:]
        q = np.concatenate([(qs & 15).astype(np.int32) - 8, (qs >> 4).astype(np.int32) - 8], axis=2)
    else:
        q = w[:, :, 2:].view(np.int8).astype(np.int32)
    a = bq.reshape(n, nb, 32).astype(np.int32)
    s = bs.reshape(n, nb)
    for i in range(m):
        for j in range(n):
            acc = (q[i] * a[j]).sum(axis=1)
            total = np.float32(0.0)
            for b in range(nb):
                total = np.float32(total + np.float32(np.float32(d[i, b] * s[j, b]) * np.float32(acc[b])))
            out[i, j] = total
    return out
