"""The CPU oracle against the reference's own known-answer tests for this path.

Each test names the reference test it replays. These pin the oracle: a restatement that
passed none of the reference's vectors would only prove agreement with itself.
"""
import numpy as np
import pytest

import kat
from oracle.binding import OracleError, SHAPE, UNSUPPORTED, INVALID

f32 = np.float32


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_f16_handles_normals_subnormals_and_specials(oracle):
    # crates/beholdd-core/src/quant.rs:505-521
    for b, want in kat.F16_VALUE_CASES:
        assert oracle.f16_to_f32(b) == f32(want), hex(b)
    assert oracle.f16_to_f32(0x7C00) == np.inf
    assert np.isnan(oracle.f16_to_f32(0x7E00))
    # crates/beholdd-backend/src/hag/kernels/kquant.rs:320-339
    for b, want_bits in kat.F16_BIT_CASES:
        assert bits([oracle.f16_to_f32(b)])[0] == want_bits, hex(b)


def test_f16_matches_numpy_for_every_bit_pattern(oracle):
    allbits = np.arange(65536, dtype=np.uint16)
    want = allbits.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(b)) for b in allbits], dtype=np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(bits(got[finite]), bits(want[finite]))
    assert np.all(np.isnan(got[~finite]))


def test_q8_0_dequantises_exactly(oracle):
    # crates/beholdd-kernel/src/kquant.rs:415-427
    src = kat.q8_row(0.5, [i - 16 for i in range(32)])
    out = oracle.dequantize(src, kat.Q8_0, 1, 32)
    assert np.array_equal(out, np.array([0.5 * (i - 16) for i in range(32)], dtype=np.float32))


def test_q6_k_decodes_every_code_at_every_position_across_blocks(oracle):
    # crates/beholdd-kernel/src/kquant.rs:361-389
    packed, expected = kat.q6_every_code_case()
    out = oracle.dequantize(packed, kat.Q6_K, 64, 256)
    assert np.array_equal(bits(out), bits(expected))


def test_q6_k_preserves_all_signed_scales_and_signed_zero(oracle):
    # crates/beholdd-kernel/src/kquant.rs:391-412
    for packed, expected in kat.q6_signed_scale_cases():
        out = oracle.dequantize(packed, kat.Q6_K, 1, 256)
        assert np.array_equal(bits(out), bits(expected))


def _q6_unit():
    src = np.zeros(210, dtype=np.uint8)
    src[192:208] = 1
    src[208:210] = np.frombuffer(np.array([kat.f16_bits(1.0)], dtype="<u2").tobytes(), dtype=np.uint8)
    return src


def test_q6_k_bias_interleave_high_bits_and_sub_block_scales(oracle):
    # crates/beholdd-kernel/src/kquant.rs:433-498
    out = oracle.dequantize(_q6_unit(), kat.Q6_K, 1, 256)
    assert np.all(out == -32.0)
    s = _q6_unit(); s[0] = 0x0F
    out = oracle.dequantize(s, kat.Q6_K, 1, 256)
    assert out[0] == -17.0 and out[1] == -32.0
    s = _q6_unit(); s[0] = 0xF0
    out = oracle.dequantize(s, kat.Q6_K, 1, 256)
    assert out[64] == -17.0 and out[0] == -32.0
    s = _q6_unit(); s[0] = 0x0F; s[128] = 0x03
    assert oracle.dequantize(s, kat.Q6_K, 1, 256)[0] == 31.0
    s = _q6_unit(); s[192:208] = np.arange(1, 17, dtype=np.uint8)
    out = oracle.dequantize(s, kat.Q6_K, 1, 256)
    assert (out[0], out[16], out[32]) == (-32.0, -64.0, -96.0)


def test_packed_6bit_scales_split_correctly_past_sub_block_four(oracle):
    # crates/beholdd-kernel/src/kquant.rs:503-517
    q = np.zeros(12, dtype=np.uint8); q[0] = 37; q[4] = 21
    assert oracle.scale_min_k4(0, q) == (37, 21)
    q = np.zeros(12, dtype=np.uint8); q[8] = 0x9; q[0] = 0b11 << 6
    assert oracle.scale_min_k4(4, q)[0] == (9 | (3 << 4))


def test_q4_k_carries_an_explicit_offset_not_a_bias(oracle):
    # crates/beholdd-kernel/src/kquant.rs:519-538
    src = np.zeros(144, dtype=np.uint8)
    one = np.frombuffer(np.array([kat.f16_bits(1.0)], dtype="<u2").tobytes(), dtype=np.uint8)
    src[0:2] = one; src[2:4] = one; src[4] = 2; src[8] = 5
    assert oracle.dequantize(src, kat.Q4_K, 1, 256)[0] == -5.0
    src[16] = 0x03
    assert oracle.dequantize(src, kat.Q4_K, 1, 256)[0] == 2.0 * 3.0 - 5.0


def test_q5_k_high_bit_plane_advances_per_pass(oracle):
    # crates/beholdd-kernel/src/kquant.rs:543-565
    src = np.zeros(176, dtype=np.uint8)
    src[0:2] = np.frombuffer(np.array([kat.f16_bits(1.0)], dtype="<u2").tobytes(), dtype=np.uint8)
    src[4:8] = 1
    src[16] = 0b0000_0001
    out = oracle.dequantize(src, kat.Q5_K, 1, 256)
    assert out[0] == 16.0 and out[64] == 0.0
    src[16] = 0b0000_0100
    out = oracle.dequantize(src, kat.Q5_K, 1, 256)
    assert out[0] == 0.0 and out[64] == 16.0


def test_k_formats_consume_exactly_their_declared_geometry(oracle):
    # crates/beholdd-kernel/src/kquant.rs:570-598
    import ctypes as C
    for code, geom in [(8, (32, 34)), (14, (256, 210)), (0, (1, 4)), (12, (256, 144)), (13, (256, 176))]:
        e, b = C.c_uint64(), C.c_uint64()
        assert oracle.lib.orc_block_geometry(code, C.byref(e), C.byref(b)) == 0
        assert (e.value, b.value) == geom
    for code in (23, 9999):
        e, b = C.c_uint64(), C.c_uint64()
        assert oracle.lib.orc_block_geometry(code, C.byref(e), C.byref(b)) == UNSUPPORTED
    for code, nbytes in [(12, 144), (13, 176), (14, 210)]:
        assert oracle.dequantize(np.zeros(nbytes * 3, dtype=np.uint8), code, 3, 256).size == 768


def test_hag_q4_six_bit_scales_minima_and_nibble_order(oracle):
    # crates/beholdd-backend/src/hag/kernels/kquant.rs:343-360
    raw, expected = kat.hag_q4_case()
    assert np.array_equal(bits(oracle.dequantize(raw, kat.Q4_K, 1, 256)), bits(expected))
    raw = kat.q4_block_by_index(1, 1, [1] * 8, [2] * 8, [3] * 256)
    assert np.all(bits(oracle.dequantize(raw, kat.Q4_K, 1, 256)) == 0x33800000)


def test_hag_q6_signed_scales_all_high_pairs_and_two_byte_block_starts(oracle):
    # crates/beholdd-backend/src/hag/kernels/kquant.rs:362-382
    raw, expected = kat.hag_q6_case()
    assert np.array_equal(bits(oracle.dequantize(raw, kat.Q6_K, 1, 512)), bits(expected))


@pytest.mark.parametrize("kind", [kat.Q4_K, kat.Q6_K])
def test_hag_accumulation_is_increasing_f32(oracle, kind):
    # crates/beholdd-backend/src/hag/kernels/kquant.rs:384-405
    raw, x, want = kat.hag_increasing_f32_case(kind)
    assert np.array_equal(oracle.serial_matvec(raw, kind, 2, 512, x), want)
    assert np.array_equal(oracle.matvec(raw, kind, 2, 512, x), want)
    with pytest.raises(OracleError):
        oracle.serial_matvec(raw[:-1], kind, 2, 512, x)
    with pytest.raises(OracleError):
        oracle.serial_matvec(raw, kind, 2, 512, x[:511])
    with pytest.raises(OracleError):
        oracle.dequantize(raw[:-1], kind, 2, 512)


@pytest.mark.parametrize("rows,cols", kat.HAG_Q8_SHAPES)
def test_hag_q8_boundary_fixtures_match_serial_no_fma_model(oracle, rows, cols):
    # crates/beholdd-backend/src/hag/fixtures.rs:45-115, 191-266
    raw, x = kat.hag_q8_fixture(rows, cols)
    want = kat.sequential_dot_f32(kat.q8_dequant_numpy(raw).reshape(rows, cols), x)
    assert np.array_equal(bits(oracle.matvec(raw, kat.Q8_0, rows, cols, x)), bits(want))


def test_matvec_overwrites_and_matvec_add_accumulates(oracle):
    # crates/beholdd-backend/src/cpu.rs:974-999
    vals = [i % 5 for i in range(32)]
    w = kat.q8_row(0.5, vals)
    x = np.ones(32, dtype=np.float32)
    expect = f32(0)
    for v in vals:
        expect = f32(expect + f32(0.5 * v))
    y = np.array([99.0], dtype=np.float32)
    oracle.matvec(w, kat.Q8_0, 1, 32, x, y=y)
    assert y[0] == expect
    y2 = np.array([10.0], dtype=np.float32)
    oracle.matvec(w, kat.Q8_0, 1, 32, x, y=y2, scale=2.0, accumulate=True)
    assert y2[0] == f32(10.0) + expect * f32(2.0)


def test_zero_width_reductions(oracle):
    # crates/beholdd-backend/src/cpu.rs:1048-1067
    y = np.full(3, 7.0, dtype=np.float32)
    oracle.matvec(np.zeros(0, dtype=np.uint8), kat.Q8_0, 3, 0, np.zeros(0, dtype=np.float32), y=y)
    assert np.all(y == 0.0)
    y = np.full(3, 0.25, dtype=np.float32)
    oracle.matvec(np.zeros(0, dtype=np.uint8), kat.Q8_0, 3, 0, np.zeros(0, dtype=np.float32), y=y, scale=0.375,
                  accumulate=True)
    assert np.all(y == 0.25)


def test_unsupported_format_and_shape_mismatch_are_refused(oracle):
    # crates/beholdd-backend/src/cpu.rs:1069-1103
    with pytest.raises(OracleError) as e:
        oracle.matvec(np.zeros(18, dtype=np.uint8), 2, 1, 32, np.zeros(32, dtype=np.float32))
    assert e.value.status == UNSUPPORTED
    with pytest.raises(OracleError) as e:
        oracle.matvec(kat.q8_row(0.5, [1] * 32), kat.Q8_0, 1, 32, np.zeros(8, dtype=np.float32))
    assert e.value.status == SHAPE


def test_fused_q8_matvec_is_bit_identical_to_dequantize_then_dot(oracle):
    # crates/beholdd-backend/src/cpu.rs:1222-1274
    raw, x, rows, cols = kat.fused_q8_case()
    deq = oracle.dequantize(raw, kat.Q8_0, rows, cols).reshape(rows, cols)
    assert np.array_equal(bits(deq), bits(kat.q8_dequant_numpy(raw).reshape(rows, cols)))
    expected = kat.sequential_dot_f32(deq, x)
    for threads in (1, 2, 3, 4, 8, 37, 1000):
        got = oracle.matvec(raw, kat.Q8_0, rows, cols, x, threads=threads)
        assert np.array_equal(bits(got), bits(expected)), threads
        acc = np.full(rows, 3.25, dtype=np.float32)
        oracle.matvec(raw, kat.Q8_0, rows, cols, x, y=acc, scale=0.375, accumulate=True, threads=threads)
        want = (f32(3.25) + (expected * f32(0.375)).astype(np.float32)).astype(np.float32)
        assert np.array_equal(bits(acc), bits(want)), threads


def test_fused_q8_refuses_truncated_storage_without_touching_output(oracle):
    # crates/beholdd-backend/src/cpu.rs:1277-1292
    y = np.array([7.0, -3.0], dtype=np.float32)
    with pytest.raises(OracleError) as e:
        oracle.matvec(kat.q8_row(0.5, [1] * 32), kat.Q8_0, 2, 32, np.ones(32, dtype=np.float32), y=y)
    assert e.value.status == SHAPE
    assert np.array_equal(y, [7.0, -3.0])


def test_row_parallel_matvec_is_bit_identical_to_sequential(oracle):
    # crates/beholdd-backend/src/cpu.rs:1193-1220
    vals = [((i * 7) % 61) - 30 for i in range(1024 * 128)]
    w = kat.q8_row(0.03125, vals)
    x = np.sin(np.arange(128, dtype=np.float32) * f32(0.3)).astype(np.float32)
    seq = oracle.matvec(w, kat.Q8_0, 1024, 128, x, threads=1)
    for threads in (2, 3, 4, 5, 7, 8, 13, 16, 1024, 4096):
        assert np.array_equal(bits(oracle.matvec(w, kat.Q8_0, 1024, 128, x, threads=threads)), bits(seq))


def test_worker_count_is_pure_and_respects_the_granularity_threshold(oracle):
    # crates/beholdd-backend/src/cpu.rs:1127-1144
    assert oracle.worker_count(8, 32, 32) == 1
    assert oracle.worker_count(1024, 128, 8) == 8
    assert oracle.worker_count(3, 30_000, 8) == 3
    assert oracle.worker_count(1024, 128, 0) == 1
    assert oracle.worker_count(1024, 128, 32) == 8
    assert oracle.worker_count(151_936, 2048, 32) == 8


def test_softmax_masks_stability_and_refusals(oracle):
    # crates/beholdd-kernel/src/vecops.rs:223-248 and crates/beholdd-backend/src/cpu.rs:572-583
    v = oracle.softmax([1.0, 2.0, 3.0, -np.inf])
    assert v[3] == 0.0 and abs(float(v.sum()) - 1.0) < 1e-6 and v[2] > v[1] > v[0]
    assert np.all(oracle.softmax([-np.inf] * 4) == 0.0)
    v = oracle.softmax([1000.0, 1001.0, 1002.0])
    assert np.all(np.isfinite(v)) and abs(float(v.sum()) - 1.0) < 1e-6
    with pytest.raises(OracleError):
        oracle.softmax([])
    with pytest.raises(OracleError):
        oracle.softmax([0.0, np.nan])


def test_swiglu_clamps_asymmetrically(oracle):
    # crates/beholdd-kernel/src/vecops.rs:250-260
    silu = lambda v: v / (1.0 + np.exp(-v))
    g = oracle.swiglu([100.0, -100.0], [100.0, -100.0], 10.0)
    assert abs(g[0] - silu(10.0) * 10.0) < 1e-4
    assert abs(g[1] - silu(-100.0) * -10.0) < 1e-4
    g = oracle.swiglu([1.5, -2.0], [2.0, 3.0], 0.0)
    assert np.allclose(g, [silu(1.5) * 2.0, silu(-2.0) * 3.0], rtol=1e-6)


def test_rmsnorm(oracle):
    # crates/beholdd-kernel/src/vecops.rs:203-220
    x = (np.sin(np.arange(512, dtype=np.float32) * f32(0.1)) * f32(3.0)).astype(np.float32)
    y = oracle.rmsnorm(x, None, 1e-6)
    assert abs(np.sqrt((y.astype(np.float64) ** 2).mean()) - 1.0) < 1e-4
    w = np.array([2.0, 3.0, 4.0, 5.0], dtype=np.float32)
    assert np.array_equal(oracle.rmsnorm(np.ones(4, dtype=np.float32), w, 0.0), w)


def test_stable_top_k(oracle):
    # crates/beholdd-model/src/qwen3moe/forward.rs:2231-2254
    idx, w, near = oracle.stable_top_k([0.1, 0.4, 0.4, 0.1], 2)
    assert list(idx) == [1, 2] and list(w) == [0.5, 0.5] and list(near) == [0, 3]
    p = np.array([40 - i for i in range(40)], dtype=np.float32)
    idx, _, near = oracle.stable_top_k(p, 3)
    assert list(idx) == [0, 1, 2] and list(near) == list(range(3, 11))
    for bad_k in (0, 5):
        with pytest.raises(OracleError) as e:
            oracle.stable_top_k([0.25] * 4, bad_k)
        assert e.value.status == INVALID
    with pytest.raises(OracleError):
        oracle.stable_top_k([0.5, np.inf], 1)
    with pytest.raises(OracleError):
        oracle.stable_top_k([0.5, -0.5], 1)


# ---- the rest of a layer: rotary embedding and causal attention (the reference's own vectors) ----

def test_rope_layouts_follow_the_reference(oracle):
    # crates/beholdd-backend/src/cpu.rs:1369-1386
    cos, sin = [0.0, 0.0], [1.0, 1.0]
    assert oracle.rope([1.0, 2.0, 3.0, 4.0], cos, sin, split_half=False).tolist() == [-2.0, 1.0, -4.0, 3.0]
    half = oracle.rope([1.0, 2.0, 3.0, 4.0], cos, sin, split_half=True)
    assert half.tolist() == [-3.0, -4.0, 1.0, 2.0]
    assert oracle.rope(half, cos, sin, split_half=True, inverse=True).tolist() == [1.0, 2.0, 3.0, 4.0]


def test_rope_table_is_theta_to_the_minus_two_i_over_dim(oracle):
    # crates/beholdd-kernel/src/vecops.rs:118-161 without YaRN
    cos, sin = oracle.rope_table(1.0e6, 8, 3)
    for i in range(4):
        a = 3.0 / (1.0e6 ** (2 * i / 8))
        assert cos[i] == np.float32(np.cos(a)) and sin[i] == np.float32(np.sin(a))
    cos0, sin0 = oracle.rope_table(1.0e6, 128, 0)
    assert np.all(cos0 == 1.0) and np.all(sin0 == 0.0)


def test_causal_attention_known_softmax_result(oracle):
    # crates/beholdd-backend/src/cpu.rs:1389-1411
    out = oracle.causal_attention([1.0, 0.0, 1.0, 0.0], [0.0, 0.0, np.log(np.float32(3.0)), 0.0], [2.0, 4.0, 6.0, 8.0], 2, 1, 1, 2, 1.0)
    assert np.abs(out.reshape(-1) - np.array([2.0, 4.0, 5.0, 7.0])).max() < 1e-6


def test_causal_attention_masks_the_future_and_maps_gqa_groups(oracle):
    # crates/beholdd-backend/src/cpu.rs:1414-1440
    out = oracle.causal_attention(np.zeros(8), np.zeros(4), [1.0, 10.0, 3.0, 30.0], 2, 4, 2, 1, 1.0)
    assert out.reshape(-1).tolist() == [1.0, 1.0, 10.0, 10.0, 2.0, 2.0, 20.0, 20.0]


def test_incremental_attention_equals_the_full_sequence_chunk_bitwise(oracle):
    # crates/beholdd-backend/src/cpu.rs:1495-1541
    q = np.sin((np.arange(24, dtype=np.float32) + np.float32(1.0)) * np.float32(0.37)).astype(np.float32)
    k = np.cos((np.arange(12, dtype=np.float32) + np.float32(2.0)) * np.float32(0.23)).astype(np.float32)
    v = (np.arange(12, dtype=np.float32) * np.float32(0.5) - np.float32(2.0)).astype(np.float32)
    full = oracle.causal_attention(q, k, v, 3, 4, 2, 2, 0.5).reshape(-1)
    inc = oracle.incremental_attention(q[8:], k, v, 2, 1, 3, 4, 2, 2, 0.5).reshape(-1)
    assert np.array_equal(inc.view(np.uint32), full[8:].view(np.uint32))


def test_incremental_attention_uses_the_absolute_position(oracle):
    # crates/beholdd-backend/src/cpu.rs:1544-1570: the third cache entry is in the query's future
    out = oracle.incremental_attention([1.0], [0.0, np.log(np.float32(3.0)), 100.0], [2.0, 6.0, 10000.0], 1, 1, 3, 1, 1, 1, 1.0)
    assert abs(float(out.reshape(-1)[0]) - 5.0) < 1e-6
    with pytest.raises(Exception):
        oracle.incremental_attention([1.0], [0.0], [0.0], 1, 1, 1, 1, 1, 1, 1.0)  # query range 1..2 exceeds one cached position
