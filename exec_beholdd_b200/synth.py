"""Seeded synthetic inputs for the quantised-matvec / routed-expert path.

One counter-based 64-bit generator (splitmix64 over `seed + index`) produces every byte, so
the CPU oracle and the GPU library always see identical inputs and a value depends only on
(seed, stream, index) -- never on how the work was split. The distributions are the ones
the benchmark configurations name:

* Q8_0 blocks  : 32 int8 quants uniform in [-127, 127] + one f16 scale uniform in [1e-3, 1e-2]
* Q4_K blocks  : uniform nibbles, uniform 6-bit scales and mins, f16 d / dmin uniform in [1e-4, 1e-2]
* Q6_K blocks  : uniform 6-bit codes, int8 sub-scales uniform in [-64, 63], f16 d uniform in [1e-4, 1e-2]
* activations  : f32 N(0, 1), optionally with 1 % of entries scaled x20
* router       : f32 N(0, 0.02)

Block layouts follow the GGUF formats as the reference decodes them
(crates/beholdd-kernel/src/kquant.rs:29-36, 82-104, 187-207).
"""
from __future__ import annotations

import numpy as np

F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 8, 12, 13, 14, 30

#: ggml type code -> (elements per block, bytes per block); crates/beholdd-core/src/quant.rs:79-118
BLOCK_GEOMETRY = {F32: (1, 4), F16: (1, 2), Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210),
                  BF16: (1, 2)}

_GAMMA = np.uint64(0x9E3779B97F4A7C15)


def packed_bytes(kind: int, rows: int, cols: int) -> int:
    elems, nbytes = BLOCK_GEOMETRY[kind]
    assert cols % elems == 0
    return rows * (cols // elems) * nbytes


def _stream_key(seed: int, stream: int) -> np.uint64:
    return np.uint64((seed * 0x2545F4914F6CDD1D + stream * 0xD6E8FEB86659FD93) & 0xFFFFFFFFFFFFFFFF)


def u64(seed: int, stream: int, n: int, start: int = 0) -> np.ndarray:
    """n splitmix64 outputs of the (seed, stream) sequence, beginning at index `start`."""
    with np.errstate(over="ignore"):
        z = _stream_key(seed, stream) + (np.arange(start + 1, start + n + 1, dtype=np.uint64) * _GAMMA)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def random_bytes(seed: int, stream: int, n: int) -> np.ndarray:
    words = u64(seed, stream, (n + 7) // 8)
    return words.view(np.uint8)[:n].copy()


def uniform01(seed: int, stream: int, n: int) -> np.ndarray:
    """float64 uniform in [0, 1) with 53 random bits."""
    return (u64(seed, stream, n) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def normal(seed: int, stream: int, n: int, std: float = 1.0) -> np.ndarray:
    """f32 N(0, std) by Box-Muller on two uniform streams."""
    u1 = 1.0 - uniform01(seed, stream * 2 + 1000003, n)  # (0, 1]
    u2 = uniform01(seed, stream * 2 + 1000004, n)
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2) * std).astype(np.float32)


def activations(seed: int, shape, outliers: bool = False, stream: int = 7) -> np.ndarray:
    n = int(np.prod(shape))
    x = normal(seed, stream, n)
    if outliers:
        mask = uniform01(seed, stream + 500, n) < 0.01
        x = np.where(mask, x * np.float32(20.0), x).astype(np.float32)
    return x.reshape(shape)


def router_weights(seed: int, n_experts: int, dim: int, stream: int = 11) -> np.ndarray:
    return normal(seed, stream, n_experts * dim, std=0.02).reshape(n_experts, dim)


def _f16_uniform(seed: int, stream: int, n: int, lo: float, hi: float) -> np.ndarray:
    return (lo + (hi - lo) * uniform01(seed, stream, n)).astype(np.float16)


def q8_0_matrix(seed: int, rows: int, cols: int, stream: int = 1) -> np.ndarray:
    """Packed Q8_0 [rows x cols] as a flat uint8 array of rows*(cols/32)*34 bytes."""
    assert cols % 32 == 0
    nb = rows * (cols // 32)
    out = np.empty((nb, 34), dtype=np.uint8)
    out[:, :2] = _f16_uniform(seed, stream * 16 + 1, nb, 1e-3, 1e-2).view(np.uint8).reshape(nb, 2)
    q = (u64(seed, stream * 16 + 2, nb * 32) % np.uint64(255)).astype(np.int16) - 127
    out[:, 2:] = q.astype(np.int8).view(np.uint8).reshape(nb, 32)
    return out.reshape(-1)


def q4_k_matrix(seed: int, rows: int, cols: int, stream: int = 2) -> np.ndarray:
    """Packed Q4_K [rows x cols]: per 256 elements d, dmin (f16), 12 scale bytes, 128 quant bytes."""
    assert cols % 256 == 0
    nb = rows * (cols // 256)
    out = np.empty((nb, 144), dtype=np.uint8)
    out[:, 0:2] = _f16_uniform(seed, stream * 16 + 1, nb, 1e-4, 1e-2).view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = _f16_uniform(seed, stream * 16 + 2, nb, 1e-4, 1e-2).view(np.uint8).reshape(nb, 2)
    # Twelve uniform bytes are exactly eight uniform 6-bit scales and eight uniform 6-bit mins.
    out[:, 4:16] = random_bytes(seed, stream * 16 + 3, nb * 12).reshape(nb, 12)
    out[:, 16:144] = random_bytes(seed, stream * 16 + 4, nb * 128).reshape(nb, 128)
    return out.reshape(-1)


def q6_k_matrix(seed: int, rows: int, cols: int, stream: int = 3) -> np.ndarray:
    """Packed Q6_K [rows x cols]: ql[128], qh[64], int8 scales[16], f16 d per 256 elements."""
    assert cols % 256 == 0
    nb = rows * (cols // 256)
    out = np.empty((nb, 210), dtype=np.uint8)
    out[:, 0:192] = random_bytes(seed, stream * 16 + 1, nb * 192).reshape(nb, 192)
    sc = (u64(seed, stream * 16 + 2, nb * 16) % np.uint64(128)).astype(np.int16) - 64
    out[:, 192:208] = sc.astype(np.int8).view(np.uint8).reshape(nb, 16)
    out[:, 208:210] = _f16_uniform(seed, stream * 16 + 3, nb, 1e-4, 1e-2).view(np.uint8).reshape(nb, 2)
    return out.reshape(-1)


def q5_k_matrix(seed: int, rows: int, cols: int, stream: int = 4) -> np.ndarray:
    """Packed Q5_K [rows x cols]: d, dmin, 12 scale bytes, qh[32], qs[128] per 256 elements."""
    assert cols % 256 == 0
    nb = rows * (cols // 256)
    out = np.empty((nb, 176), dtype=np.uint8)
    out[:, 0:2] = _f16_uniform(seed, stream * 16 + 1, nb, 1e-4, 1e-2).view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = _f16_uniform(seed, stream * 16 + 2, nb, 1e-4, 1e-2).view(np.uint8).reshape(nb, 2)
    out[:, 4:176] = random_bytes(seed, stream * 16 + 3, nb * 172).reshape(nb, 172)
    return out.reshape(-1)


def matrix(kind: int, seed: int, rows: int, cols: int, stream: int | None = None) -> np.ndarray:
    gen = {Q8_0: q8_0_matrix, Q4_K: q4_k_matrix, Q5_K: q5_k_matrix, Q6_K: q6_k_matrix}[kind]
    return gen(seed, rows, cols) if stream is None else gen(seed, rows, cols, stream)


def expert_slabs(seed: int, n_experts: int, rows: int, cols: int, stream: int) -> np.ndarray:
    """n_experts contiguous Q8_0 [rows x cols] slabs, the layout of a 3-D GGUF expert tensor
    (crates/beholdd-model/src/qwen3moe/forward.rs:1668-1690)."""
    return q8_0_matrix(seed, n_experts * rows, cols, stream)
