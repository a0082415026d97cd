"""Host-side logic of the qwen3moe mirror that needs no GPU."""
import numpy as np
import pytest

from exec_beholdd_b200 import synth
from exec_beholdd_b200.qwen3moe import qkv_weights, rope_tables


class _Bytes:
    """Stands in for a CUDA uint8 tensor: slicing and numel()."""

    def __init__(self, a):
        self.a = a

    def __getitem__(self, key):
        return _Bytes(self.a[key])

    def numel(self):
        return int(self.a.size)


class _FakeDevice:
    def __init__(self):
        self.wrapped = []

    def wrap_weight(self, packed, kind, rows, cols, slabs=1):
        self.wrapped.append((packed.a, kind, rows, cols))
        return (kind, rows, cols, packed.numel())


def test_qkv_weights_wrap_the_three_parts_and_the_whole_of_one_buffer():
    """[wq; wk; wv] stored back to back is itself a packed matrix: the parts and the whole are wrapped over the same bytes,
    nothing is copied, and a buffer of the wrong size is refused."""
    q_width, kv_width, dim = 64, 16, 256
    wq, wk, wv = (synth.q8_0_matrix(7, q_width, dim, 1), synth.q8_0_matrix(7, kv_width, dim, 2), synth.q8_0_matrix(7, kv_width, dim, 3))
    buf = np.concatenate([wq.reshape(-1), wk.reshape(-1), wv.reshape(-1)])
    dev = _FakeDevice()
    out = qkv_weights(dev, _Bytes(buf), 8, q_width, kv_width, dim)
    assert out["wq"] == (8, q_width, dim, wq.size) and out["wk"] == (8, kv_width, dim, wk.size) and out["wv"] == (8, kv_width, dim, wv.size)
    assert out["wqkv"] == (8, q_width + 2 * kv_width, dim, buf.size)
    assert np.array_equal(dev.wrapped[0][0], wq.reshape(-1)) and np.array_equal(dev.wrapped[1][0], wk.reshape(-1))
    assert np.array_equal(dev.wrapped[2][0], wv.reshape(-1)) and dev.wrapped[3][0] is buf
    assert all(np.shares_memory(a, buf) for a, *_ in dev.wrapped)           # views, not copies
    # the rows of the fused matrix are the rows of the parts, in order: row q_width is wk's first row
    row_bytes = synth.packed_bytes(8, 1, dim)
    assert np.array_equal(buf[q_width * row_bytes:(q_width + 1) * row_bytes], wk.reshape(-1)[:row_bytes])
    with pytest.raises(ValueError):
        qkv_weights(dev, _Bytes(buf[:-1]), 8, q_width, kv_width, dim)
    # K-quant formats: same rule with their own block geometry
    w4 = [synth.q4_k_matrix(9, r, dim, 4) for r in (q_width, kv_width, kv_width)]
    buf4 = np.concatenate([w.reshape(-1) for w in w4])
    out4 = qkv_weights(_FakeDevice(), _Bytes(buf4), 12, q_width, kv_width, dim)
    assert out4["wqkv"] == (12, q_width + 2 * kv_width, dim, buf4.size)


def test_rope_tables_are_f64_angles_rounded_once():
    cos, sin = rope_tables(1.0e6, 8, 5)
    assert cos.shape == (5, 4) and cos.dtype == np.float32
    freqs = 1.0 / np.power(np.float64(1.0e6), 2.0 * np.arange(4, dtype=np.float64) / 8.0)
    a = np.arange(5, dtype=np.float64)[:, None] * freqs[None, :]
    assert np.array_equal(cos, np.cos(a).astype(np.float32)) and np.array_equal(sin, np.sin(a).astype(np.float32))
    assert np.all(cos[0] == 1.0) and np.all(sin[0] == 0.0)


def test_integer_widening_rule_of_the_attention_kernels_matches_the_conversion():
    """The attention kernels widen f32 to f64 with integer operations for normal numbers and zeros (sign kept, exponent
    re-biased by 896, mantissa shifted by 29 bits) and leave subnormals, infinities and NaNs to the conversion instruction.
    The rule, restated on the host, gives the bits of the exact conversion on every normal number and zero."""
    rng = np.random.default_rng(5)
    bits32 = np.concatenate([rng.integers(0, 2**32, 200000, dtype=np.uint64).astype(np.uint32),
                             np.array([0x00000000, 0x80000000, 0x00800000, 0x80800000, 0x7f7fffff, 0xff7fffff, 0x3f800000, 0x00000001,
                                       0x007fffff, 0x7f800000, 0xff800000, 0x7fc00000], dtype=np.uint32)])
    exp = bits32 & np.uint32(0x7f800000)
    special = (exp == 0) | (exp == np.uint32(0x7f800000))
    zero = (bits32 << np.uint32(1)) == 0
    hi = (bits32 & np.uint32(0x80000000)) | (((bits32 & np.uint32(0x7fffffff)) >> np.uint32(3)) + np.uint32(0x38000000))
    lo = bits32 << np.uint32(29)
    widened = (hi.astype(np.uint64) << np.uint64(32)) | lo.astype(np.uint64)
    widened[zero] = bits32[zero].astype(np.uint64) << np.uint64(32)
    with np.errstate(invalid="ignore"):        # signalling NaN patterns among the random bits
        exact = bits32.view(np.float32).astype(np.float64).view(np.uint64)
    fast = ~special | zero
    assert fast.sum() > 190000 and np.array_equal(widened[fast], exact[fast])
    # the cases the kernels hand to the instruction are exactly the ones the rule would get wrong
    slow = special & ~zero
    assert slow.sum() >= 5 and not np.any(widened[slow] == exact[slow])
