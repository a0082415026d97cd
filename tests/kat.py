"""Known-answer inputs restated from the reference's own unit tests for this path.

Every builder cites the reference test it restates (paths relative to the reference
repository root). Encoders here are written independently of any decoder: they place
semantic values (codes, scales) into packed planes, and the expected values are computed
with explicit numpy float32 steps. Both the CPU oracle tests and the GPU parity tests use
them, so the CUDA path is held to the same vectors as the reference's CPU path.
"""
from __future__ import annotations

import struct

import numpy as np

f32 = np.float32

Q8_0, Q4_K, Q5_K, Q6_K = 8, 12, 13, 14


def f16_bits(v: float) -> int:
    """Exact small values only, like the reference's test helper
    (crates/beholdd-kernel/src/kquant.rs:322-329)."""
    return int(np.array([v], dtype=np.float16).view(np.uint16)[0])


def half(bits: int) -> np.float32:
    return np.array([bits], dtype=np.uint16).view(np.float16).astype(np.float32)[0]


# f16 decode cases: crates/beholdd-core/src/quant.rs:505-521 and the bit-level table in
# crates/beholdd-backend/src/hag/kernels/kquant.rs:320-339.
F16_VALUE_CASES = [
    (0x0000, 0.0), (0x3C00, 1.0), (0xBC00, -1.0), (0x3555, 0.33325195), (0x0400, 6.1035156e-5),
    (0x0001, 5.9604645e-8), (0x03FF, 6.097555e-5), (0x7BFF, 65504.0),
]
F16_BIT_CASES = [
    (0x0000, 0x00000000), (0x8000, 0x80000000), (0x0001, 0x33800000), (0x8001, 0xB3800000),
    (0x03FF, 0x387FC000), (0x0400, 0x38800000), (0x3C00, 0x3F800000), (0x7BFF, 0x477FE000),
]


def q8_row(scale: float, vals) -> np.ndarray:
    """crates/beholdd-backend/src/cpu.rs:953-965: blocks of one f16 scale + 32 int8, zero padded."""
    vals = list(vals)
    out = bytearray()
    for c in range(0, len(vals), 32):
        chunk = vals[c:c + 32]
        out += struct.pack("<H", f16_bits(scale))
        for i in range(32):
            out.append((chunk[i] if i < len(chunk) else 0) & 0xFF)
    return np.frombuffer(bytes(out), dtype=np.uint8).copy()


def encode_q6_k(codes, scales, d_bits: int) -> np.ndarray:
    """Plane-traversal encoder, crates/beholdd-kernel/src/kquant.rs:333-358."""
    codes = np.asarray(codes, dtype=np.uint8)
    assert codes.shape == (256,) and codes.max() < 64
    packed = np.zeros(210, dtype=np.uint8)
    for h in range(2):
        c = codes[h * 128:(h + 1) * 128]
        packed[h * 64:(h + 1) * 64] = (c[:64] & 0x0F) | ((c[64:] & 0x0F) << 4)
        for group in range(4):
            packed[128 + h * 32:128 + (h + 1) * 32] |= (c[group * 32:(group + 1) * 32] >> 4) << (2 * group)
    packed[192:208] = np.asarray(scales, dtype=np.int8).view(np.uint8)
    packed[208:210] = np.frombuffer(struct.pack("<H", d_bits), dtype=np.uint8)
    return packed


def q6_block_by_index(d_bits: int, scales, codes) -> np.ndarray:
    """Index-addressed encoder, crates/beholdd-backend/src/hag/kernels/kquant.rs:284-298."""
    raw = np.zeros(210, dtype=np.uint8)
    for index, code in enumerate(codes):
        group = (index % 128) // 32
        lane = index % 32
        raw[(index // 128) * 64 + (group % 2) * 32 + lane] |= (code & 15) << (4 * (group // 2))
        raw[128 + (index // 128) * 32 + lane] |= (code >> 4) << (2 * group)
    raw[192:208] = np.asarray(scales, dtype=np.int8).view(np.uint8)
    raw[208:210] = np.frombuffer(struct.pack("<H", d_bits), dtype=np.uint8)
    return raw


def q4_block_by_index(d_bits: int, dmin_bits: int, scales, minima, codes) -> np.ndarray:
    """crates/beholdd-backend/src/hag/kernels/kquant.rs:258-282."""
    raw = np.zeros(144, dtype=np.uint8)
    raw[0:2] = np.frombuffer(struct.pack("<H", d_bits), dtype=np.uint8)
    raw[2:4] = np.frombuffer(struct.pack("<H", dmin_bits), dtype=np.uint8)
    for i, (s, m) in enumerate(zip(scales, minima)):
        assert s < 64 and m < 64
        if i < 4:
            raw[4 + i] |= s
            raw[8 + i] |= m
        else:
            raw[i] |= (s >> 4) << 6
            raw[4 + i] |= (m >> 4) << 6
            raw[8 + i] = (s & 15) | ((m & 15) << 4)
    for i, code in enumerate(codes):
        assert code < 16
        raw[16 + (i // 64) * 32 + i % 32] |= code << (4 * ((i // 32) % 2))
    return raw


def q6_every_code_case():
    """crates/beholdd-kernel/src/kquant.rs:361-389: 64 blocks visiting all codes at all positions."""
    scales = [-128, -127, -63, -31, -17, -3, -1, 1, 2, 5, 19, 33, 65, 101, 126, 127]
    packed, expected = [], []
    for rotation in range(64):
        idx = np.arange(256)
        codes = ((idx * 29 + (idx // 32) * 7 + (idx // 128) * 11 + rotation) % 64).astype(np.uint8)
        d_bits = [0x3555, 0xBC01, 0x0001, 0x7BFF][rotation % 4]
        packed.append(encode_q6_k(codes, scales, d_bits))
        d = half(d_bits)
        sc = np.array(scales, dtype=np.float32)[idx // 16]
        with np.errstate(over="ignore"):
            expected.append((f32(d) * sc).astype(np.float32) * (codes.astype(np.int32) - 32).astype(np.float32))
    return np.concatenate(packed), np.concatenate(expected).astype(np.float32)


def q6_signed_scale_cases():
    """crates/beholdd-kernel/src/kquant.rs:391-412."""
    codes = np.array([[0, 31, 32, 33, 63][i % 5] for i in range(256)], dtype=np.uint8)
    for d_bits in (0x3555, 0xB555, 0x0000, 0x8000):
        d = half(d_bits)
        for batch in range(16):
            scales = np.array([(batch * 16 + i) & 0xFF for i in range(16)], dtype=np.uint8).view(np.int8)
            packed = encode_q6_k(codes, scales, d_bits)
            sc = scales.astype(np.float32)[np.arange(256) // 16]
            expected = (f32(d) * sc).astype(np.float32) * (codes.astype(np.int32) - 32).astype(np.float32)
            yield packed, expected.astype(np.float32)


def hag_q4_case():
    """crates/beholdd-backend/src/hag/kernels/kquant.rs:343-360."""
    scales = [1, 17, 32, 63, 61, 33, 18, 7]
    minima = [62, 31, 16, 4, 3, 19, 34, 63]
    i = np.arange(256)
    codes = ((i * 7 + i // 32) % 16).astype(np.uint8)
    raw = q4_block_by_index(0x3000, 0x2C00, scales, minima, codes)  # d = 1/8, dmin = 1/16
    sc = np.array(scales, dtype=np.float32)[i // 32]
    mn = np.array(minima, dtype=np.float32)[i // 32]
    expected = (f32(0.125) * sc).astype(np.float32) * codes.astype(np.float32) - (f32(0.0625) * mn).astype(np.float32)
    return raw, expected.astype(np.float32)


def hag_q6_case():
    """crates/beholdd-backend/src/hag/kernels/kquant.rs:362-382."""
    scales = [-128, -97, -63, -32, -1, 0, 1, 17, 31, 63, 95, 127, -2, 3, -4, 5]
    i = np.arange(256)
    codes = ((i * 13 + i // 16) % 64).astype(np.uint8)
    raw = np.concatenate([q6_block_by_index(0x3000, scales, codes), q6_block_by_index(1, scales, codes)])
    expected = []
    for d in (f32(0.125), np.array([0x33800000], dtype=np.uint32).view(np.float32)[0]):
        sc = np.array(scales, dtype=np.float32)[i // 16]
        expected.append((d * sc).astype(np.float32) * (codes.astype(np.int32) - 32).astype(np.float32))
    return raw, np.concatenate(expected).astype(np.float32)


def hag_increasing_f32_case(kind: int):
    """crates/beholdd-backend/src/hag/kernels/kquant.rs:384-405: a 2x512 matrix whose rows
    only give [0.75, 1.5] under strictly increasing-column f32 accumulation."""
    def make(two: bool):
        if kind == Q4_K:
            return q4_block_by_index(0x3C00, 0, [1] * 8, [0] * 8, [2 if two else 1] * 256)
        return q6_block_by_index(0x3C00, [1] * 16, [34 if two else 33] * 256)
    raw = np.concatenate([make(False), make(False), make(True), make(True)])
    x = np.zeros(512, dtype=np.float32)
    x[0], x[1], x[2], x[255], x[256] = 16777216.0, 1.0, -16777216.0, 0.25, 0.5
    return raw, x, np.array([0.75, 1.5], dtype=np.float32)


Q8_SCALE_BITS = [0x3800, 0xB400, 0x0000, 0x3A00, 0x3000, 0xC000]
HAG_Q8_SHAPES = [(1, 32), (3, 64), (5, 96), (7, 224), (63, 256), (64, 256)]


def hag_q8_fixture(rows: int, cols: int):
    """crates/beholdd-backend/src/hag/fixtures.rs:74-115: signed extremes, six exact scales
    (including zero and negatives), dyadic activations."""
    out = bytearray()
    for row in range(rows):
        for block in range(cols // 32):
            out += struct.pack("<H", Q8_SCALE_BITS[(row + block * 3) % 6])
            for element in range(32):
                q = {0: -128, 1: 127, 2: -1, 3: 0, 4: 1}.get(element, None)
                if q is None:
                    q = (row * 19 + block * 11 + element * 7) % 256
                out.append(q & 0xFF)
    x = np.array([{0: 1.0, 1: -1.0, 2: 0.0}.get(c, (((c * 29 + 7) % 97) - 48.0) / 32.0) for c in range(cols)],
                 dtype=np.float32)
    return np.frombuffer(bytes(out), dtype=np.uint8).copy(), x


def fused_q8_case():
    """crates/beholdd-backend/src/cpu.rs:1222-1274: 37x96 with seven scales per row pattern."""
    rows, cols = 37, 96
    out = bytearray()
    for row in range(rows):
        for block in range(cols // 32):
            scale = 0.0078125 * (1 + ((row + block) % 7))
            out += struct.pack("<H", f16_bits(scale))
            for i in range(32):
                out.append((((row * 19 + block * 11 + i * 7) % 241) - 120) & 0xFF)
    i = np.arange(cols)
    x = (np.sin((i.astype(np.float32) * f32(0.137)).astype(np.float32)).astype(np.float32)
         * ((i % 5 + 1).astype(np.float32))).astype(np.float32)
    return np.frombuffer(bytes(out), dtype=np.uint8).copy(), x, rows, cols


def sequential_dot_f32(dequantized: np.ndarray, x: np.ndarray) -> np.ndarray:
    """Independent statement of crates/beholdd-backend/src/cpu.rs:198-218: per row one f32
    accumulator, left to right, product and sum rounded separately."""
    rows = dequantized.shape[0]
    y = np.zeros(rows, dtype=np.float32)
    for r in range(rows):
        acc = f32(0.0)
        prod = (dequantized[r] * x).astype(np.float32)
        for p in prod:
            acc = f32(acc + p)
        y[r] = acc
    return y


def q8_dequant_numpy(raw: np.ndarray) -> np.ndarray:
    """Independent Q8_0 decode: f16 scale times int8 quant, one f32 rounding."""
    blocks = raw.reshape(-1, 34)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)
    q = blocks[:, 2:].copy().view(np.int8).astype(np.float32)
    return (d * q).astype(np.float32).reshape(-1)
