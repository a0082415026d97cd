"""GPU parity: the CUDA path through the C ABI against the CPU oracle, the reference's
known-answer vectors and the NumPy golden vectors.

Bar: integer outputs (expert indices, assignments, counts) bit-exact; floating point within
max relative error 2e-3, measured as max_i |g_i - r_i| / max(|r_i|, rms(r)).
"""
import numpy as np
import pytest

import golden_cases as gc
import kat

pytestmark = pytest.mark.gpu

TOL = 2e-3  # the stated floating-point tolerance of the path (fp32 accumulate)


def max_rel_err(got, want):
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    rms = np.sqrt((want ** 2).mean()) if want.size else 0.0
    den = np.maximum(np.abs(want), max(rms, 1e-30))
    return float((np.abs(got - want) / den).max()) if want.size else 0.0


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.fixture(scope="module")
def dev():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from exec_beholdd_b200 import CudaDevice

    d = CudaDevice(0)
    yield d
    d.close()


@pytest.fixture(scope="module")
def W():
    from exec_beholdd_b200 import Weight

    return Weight


def cuda(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# ---- dequantize: bit-exact on the reference's vectors -----------------------------------

def test_dequantize_known_answers_bit_exact(dev, W, oracle):
    cases = []
    packed, expected = kat.q6_every_code_case()
    cases.append((packed, kat.Q6_K, 64, 256, expected))
    for packed, expected in list(kat.q6_signed_scale_cases())[::7]:
        cases.append((packed, kat.Q6_K, 1, 256, expected))
    raw, expected = kat.hag_q4_case()
    cases.append((raw, kat.Q4_K, 1, 256, expected))
    raw, expected = kat.hag_q6_case()
    cases.append((raw, kat.Q6_K, 1, 512, expected))
    src = kat.q8_row(0.5, [i - 16 for i in range(32)])
    cases.append((src, kat.Q8_0, 1, 32, np.array([0.5 * (i - 16) for i in range(32)], dtype=np.float32)))
    for packed, kind, rows, cols, expected in cases:
        out = np.zeros(rows * cols, dtype=np.float32)
        dev.dequantize(out, W(packed, kind, rows, cols))
        assert np.array_equal(bits(out), bits(expected)), (kind, rows, cols)


@pytest.mark.parametrize("kind", [8, 12, 13, 14])
def test_dequantize_matches_oracle_bit_exact_on_seeded_blocks(dev, W, oracle, kind):
    from exec_beholdd_b200 import synth

    rows, cols = 5, 512
    packed = synth.matrix(kind, 17, rows, cols)
    out = np.zeros(rows * cols, dtype=np.float32)
    dev.dequantize(out, W(packed, kind, rows, cols))
    assert np.array_equal(bits(out), bits(oracle.dequantize(packed, kind, rows, cols)))


# ---- matvec ------------------------------------------------------------------------------

@pytest.mark.parametrize("rows,cols", kat.HAG_Q8_SHAPES)
def test_q8_boundary_fixtures_are_exact(dev, W, oracle, rows, cols):
    # Dyadic inputs make every partial sum exact, so any summation order must give the
    # reference's bits (crates/beholdd-backend/src/hag/fixtures.rs:45-115).
    raw, x = kat.hag_q8_fixture(rows, cols)
    y = np.full(rows, np.float32(np.nan))
    dev.matvec(y, x, W(raw, kat.Q8_0, rows, cols))
    assert np.array_equal(bits(y), bits(oracle.matvec(raw, kat.Q8_0, rows, cols, x)))


def test_matvec_overwrites_and_matvec_add_accumulates(dev, W, oracle):
    # crates/beholdd-backend/src/cpu.rs:974-999
    vals = [i % 5 for i in range(32)]
    w = W(kat.q8_row(0.5, vals), kat.Q8_0, 1, 32)
    x = np.ones(32, dtype=np.float32)
    expect = np.float32(sum(0.5 * v for v in vals))
    y = np.array([99.0], dtype=np.float32)
    dev.matvec(y, x, w)
    assert y[0] == expect
    y2 = np.array([10.0], dtype=np.float32)
    dev.matvec_add(y2, x, w, 2.0)
    assert y2[0] == np.float32(10.0) + expect * np.float32(2.0)


def test_fused_q8_case_and_scaled_add(dev, W, oracle):
    # crates/beholdd-backend/src/cpu.rs:1222-1274 (values within tolerance; add semantics exact in form)
    raw, x, rows, cols = kat.fused_q8_case()
    want = oracle.matvec(raw, kat.Q8_0, rows, cols, x)
    y = np.zeros(rows, dtype=np.float32)
    dev.matvec(y, x, W(raw, kat.Q8_0, rows, cols))
    assert max_rel_err(y, want) <= TOL
    acc = np.full(rows, 3.25, dtype=np.float32)
    dev.matvec_add(acc, x, W(raw, kat.Q8_0, rows, cols), 0.375)
    want_add = oracle.matvec(raw, kat.Q8_0, rows, cols, x, y=np.full(rows, 3.25, dtype=np.float32), scale=0.375,
                             accumulate=True)
    assert max_rel_err(acc, want_add) <= TOL


def test_zero_width_and_refusals_leave_output_untouched(dev, W):
    from exec_beholdd_b200 import ShapeError, UnsupportedFormat

    # crates/beholdd-backend/src/cpu.rs:1048-1067
    y = np.full(3, 7.0, dtype=np.float32)
    dev.matvec(y, np.zeros(0, dtype=np.float32), W(np.zeros(0, dtype=np.uint8), kat.Q8_0, 3, 0))
    assert np.all(y == 0.0)
    y = np.full(3, 0.25, dtype=np.float32)
    dev.matvec_add(y, np.zeros(0, dtype=np.float32), W(np.zeros(0, dtype=np.uint8), kat.Q8_0, 3, 0), 0.375)
    assert np.all(y == 0.25)
    # crates/beholdd-backend/src/cpu.rs:1277-1292
    out = np.array([7.0, -3.0], dtype=np.float32)
    with pytest.raises(ShapeError) as e:
        dev.matvec(out, np.ones(32, dtype=np.float32), W(kat.q8_row(0.5, [1] * 32), kat.Q8_0, 2, 32))
    assert "needs 68 bytes" in str(e.value)
    assert np.array_equal(out, [7.0, -3.0])
    # crates/beholdd-backend/src/cpu.rs:1069-1103
    with pytest.raises(UnsupportedFormat):
        dev.matvec(out[:1], np.zeros(32, dtype=np.float32), W(np.zeros(18, dtype=np.uint8), 2, 1, 32))
    with pytest.raises(ShapeError) as e:
        dev.matvec(out[:1], np.zeros(8, dtype=np.float32), W(kat.q8_row(0.5, [1] * 32), kat.Q8_0, 1, 32))
    assert "1x32" in str(e.value)
    assert not dev.supports(23) and dev.supports(8) and dev.name() == "cuda-b200"


MATVEC_CASES = [
    # (kind, rows, cols, batch): config-0 shapes, reduced config-1 shapes, ragged edges
    (8, 3072, 1024, 1), (8, 1024, 3072, 1), (8, 768, 2048, 3), (8, 2048, 768, 8), (8, 37, 96, 2), (8, 1, 32, 1),
    (8, 100, 32 * 7, 5), (12, 1536, 4096, 1), (12, 512, 12288, 2), (12, 1024, 4096, 4), (12, 768, 4096, 8),
    (12, 19, 256, 1), (12, 130, 768, 7), (14, 1536, 4096, 1), (14, 512, 12288, 2), (14, 1024, 4096, 8),
    (14, 21, 256, 3), (14, 70, 2304, 2), (13, 64, 512, 2), (0, 128, 2048, 4), (1, 33, 100, 2),
    (8, 512, 8192, 1), (12, 100, 5120, 1), (12, 4096, 4096, 1),
]


@pytest.mark.parametrize("kind,rows,cols,batch", MATVEC_CASES)
def test_matvec_matches_oracle_on_seeded_inputs(dev, oracle, kind, rows, cols, batch):
    import torch
    from exec_beholdd_b200 import Weight, synth

    if kind == 0:
        packed = synth.normal(5, 3, rows * cols).view(np.uint8)
    elif kind == 1:
        packed = synth.normal(5, 3, rows * cols).astype(np.float16).view(np.uint8)
    else:
        packed = synth.matrix(kind, 5, rows, cols)
    x = synth.activations(9, (batch, cols))
    want = oracle.matvec_batch(packed, kind, rows, cols, x)
    w = dev.upload_weight(Weight(packed, kind, rows, cols))
    xd = cuda(x)
    yd = torch.full((batch, rows), float("nan"), device="cuda")
    dev.matvec_resident(w, xd, yd)
    got = yd.cpu().numpy()
    assert max_rel_err(got, want) <= TOL
    # scaled accumulate on top of existing values
    base = synth.activations(10, (batch, rows))
    yd = cuda(base)
    dev.matvec_resident(w, xd, yd, scale=-0.75, accumulate=True)
    want_add = base + want * np.float32(-0.75)
    assert max_rel_err(yd.cpu().numpy(), want_add) <= TOL
    # bit-determinism across runs (crates/beholdd-backend/src/lib.rs:159-163)
    y2 = torch.empty((batch, rows), device="cuda")
    dev.matvec_resident(w, xd, y2)
    y3 = torch.empty((batch, rows), device="cuda")
    dev.matvec_resident(w, xd, y3)
    assert torch.equal(y2, y3)
    dev.check_status()
    w.free()


@pytest.mark.parametrize("kind,rows,cols,batch", [(12, 1536, 4096, 1), (8, 768, 2048, 3), (14, 512, 1024, 6)])
def test_matvec_host_gives_the_same_result_for_pageable_and_page_locked_buffers(dev, oracle, kind, rows, cols, batch):
    """bhd_matvec_host stages pageable buffers through device memory and lets the kernels
    address page-locked ones directly; both must produce the bits of the device-resident call."""
    import torch
    from exec_beholdd_b200 import Weight, synth

    packed = synth.matrix(kind, 31, rows, cols)
    x = synth.activations(32, (batch, cols))
    base = synth.activations(33, (batch, rows))
    want = oracle.matvec_batch(packed, kind, rows, cols, x)
    w = dev.upload_weight(Weight(packed, kind, rows, cols))
    yd = torch.empty((batch, rows), device="cuda")
    dev.matvec_resident(w, cuda(x), yd)
    resident = yd.cpu().numpy()
    assert max_rel_err(resident, want) <= TOL
    # pageable numpy arrays
    y_page = np.full((batch, rows), np.nan, dtype=np.float32)
    dev.matvec_host_resident(w, x, y_page)
    assert np.array_equal(bits(y_page), bits(resident))
    # page-locked buffers
    xp = torch.from_numpy(x.copy()).pin_memory()
    yp = torch.full((batch, rows), float("nan")).pin_memory()
    dev.matvec_host_resident(w, xp.numpy(), yp.numpy())
    assert np.array_equal(bits(yp.numpy()), bits(resident))
    # scaled accumulate into page-locked y
    yp.copy_(torch.from_numpy(base))
    dev.matvec_host_resident(w, xp.numpy(), yp.numpy(), scale=0.5, accumulate=True)
    assert max_rel_err(yp.numpy(), base + want * np.float32(0.5)) <= TOL
    dev.check_status()
    w.free()


@pytest.mark.parametrize("kind,batch,bad", [(12, 1, np.nan), (8, 1, np.inf), (14, 1, -np.inf), (12, 3, np.nan), (8, 8, np.inf)])
def test_non_finite_activation_is_reported_through_the_status_word(dev, kind, batch, bad):
    """A NaN or infinite activation cannot be represented in the packed operand formats; the
    kernels flag it (and feed zero) instead of producing silent garbage, and the next
    check_status raises and clears the flag."""
    import torch
    from exec_beholdd_b200 import DeviceError, Weight, synth

    rows, cols = 1536, 4096
    w = dev.upload_weight(Weight(synth.matrix(kind, 41, rows, cols), kind, rows, cols))
    x = synth.activations(42, (batch, cols))
    x[batch - 1, 1234] = bad
    y = torch.empty((batch, rows), device="cuda")
    dev.matvec_resident(w, cuda(x), y)
    with pytest.raises(DeviceError):
        dev.check_status()
    dev.check_status()  # the flag was cleared by the failed check
    w.free()


@pytest.mark.parametrize("kind,rows,cols,batch,world", [(12, 1024, 4096, 1, 2), (8, 768, 2048, 4, 4), (14, 512, 1024, 2, 2)])
def test_row_split_shards_reproduce_the_whole_projection(dev, oracle, kind, rows, cols, batch, world):
    """Every rank's shard (whole packed rows) gives that rank's slice of y; the slices laid
    side by side are the single-GPU result (one process plays all ranks here)."""
    import torch
    from exec_beholdd_b200 import synth
    from exec_beholdd_b200.row_parallel import RowSplitLinear

    packed = synth.matrix(kind, 21, rows, cols)
    x = synth.activations(22, (batch, cols))
    want = oracle.matvec_batch(packed, kind, rows, cols, x)
    xd = cuda(x)
    per = rows // world
    got = np.empty((batch, rows), dtype=np.float32)
    for r in range(world):
        lin = RowSplitLinear.from_host(dev, packed, kind, rows, cols, r, world)
        yl = torch.full((batch, per), float("nan"), device="cuda")
        lin._local(xd, yl)
        got[:, r * per:(r + 1) * per] = yl.cpu().numpy()
        lin.free()
    assert max_rel_err(got, want) <= TOL
    dev.check_status()


@pytest.mark.parametrize("kind,rows,cols", [(12, 12288, 4096), (12, 4096, 12288), (14, 12288, 4096), (8, 12288, 4096)])
def test_full_size_matvec_properties(dev, kind, rows, cols):
    """Full benchmark sizes, where the scalar oracle is too slow: compare with the f64 product
    of the library's own bit-exact decode, and check linearity and batch consistency."""
    import torch
    from exec_beholdd_b200 import Weight, synth

    packed = synth.matrix(kind, 23, rows, cols)
    w = dev.upload_weight(Weight(packed, kind, rows, cols))
    deq = torch.empty(rows * cols, device="cuda")
    dev.dequantize_resident(w, deq)
    x = cuda(synth.activations(31, (8, cols)))
    y = torch.empty((8, rows), device="cuda")
    dev.matvec_resident(w, x, y)
    want = (deq.view(rows, cols).double() @ x.double().T).T
    assert max_rel_err(y.cpu().numpy(), want.cpu().numpy()) <= TOL
    # a batch equals its single-vector calls
    y1 = torch.empty((1, rows), device="cuda")
    dev.matvec_resident(w, x[3:4].contiguous(), y1)
    assert max_rel_err(y1.cpu().numpy(), y[3:4].cpu().numpy()) <= 5e-4  # different kernels: 16-bit block-floating vs 22-bit split activations
    # linearity in x
    ysum = torch.empty((1, rows), device="cuda")
    dev.matvec_resident(w, (x[0:1] + x[1:2]).contiguous(), ysum)
    assert max_rel_err(ysum.cpu().numpy(), (y[0:1] + y[1:2]).cpu().numpy()) <= 1e-3
    dev.check_status()
    w.free()


@pytest.mark.parametrize("m,n,k", [(128, 512, 1024), (70, 96, 256), (512, 256, 4096)])
def test_prefill_matmul_matches_oracle(dev, oracle, m, n, k):
    import torch
    from exec_beholdd_b200 import Weight, synth

    packed = synth.q8_0_matrix(41, n, k)
    x = synth.activations(43, (m, k), outliers=True)
    sample = np.arange(0, m, max(1, m // 16))  # the scalar oracle on a row sample of X
    want = oracle.matvec_batch(packed, 8, n, k, x[sample])
    w = dev.upload_weight(Weight(packed, 8, n, k))
    y = torch.empty((m, n), device="cuda")
    dev.matmul_resident(w, cuda(x), y)
    assert max_rel_err(y.cpu().numpy()[sample], want) <= TOL
    w.free()


# ---- softmax / swiglu ------------------------------------------------------------------------

def test_softmax_and_swiglu_follow_the_reference(dev, oracle):
    from exec_beholdd_b200 import ShapeError, synth

    v = np.array([1.0, 2.0, 3.0, -np.inf], dtype=np.float32)
    dev.softmax(v)
    assert v[3] == 0.0 and abs(float(v.sum()) - 1.0) < 1e-6
    v = np.full(4, -np.inf, dtype=np.float32)
    dev.softmax(v)
    assert np.all(v == 0.0)
    v = synth.normal(3, 5, 128) * np.float32(3.0)
    got = v.copy()
    dev.softmax(got)
    assert np.array_equal(bits(got), bits(oracle.softmax(v)))  # same expf algorithm, same order
    with pytest.raises(ShapeError):
        dev.softmax(np.array([0.0, np.nan], dtype=np.float32))
    with pytest.raises(ShapeError):
        dev.softmax(np.zeros(0, dtype=np.float32))
    g, u = synth.normal(4, 1, 768) * np.float32(4.0), synth.normal(4, 2, 768)
    got = g.copy()
    dev.swiglu(got, u, 0.0)
    assert max_rel_err(got, oracle.swiglu(g, u, 0.0)) <= 1e-5
    got = np.array([100.0, -100.0], dtype=np.float32)
    dev.swiglu(got, np.array([100.0, -100.0], dtype=np.float32), 10.0)
    assert max_rel_err(got, oracle.swiglu([100.0, -100.0], [100.0, -100.0], 10.0)) <= 1e-5


# ---- routed experts ------------------------------------------------------------------------

def moe_inputs(seed, n_experts, dim, ff, T):
    from exec_beholdd_b200 import synth

    router = synth.router_weights(seed, n_experts, dim)
    gate = synth.expert_slabs(seed, n_experts, ff, dim, stream=21)
    up = synth.expert_slabs(seed, n_experts, ff, dim, stream=22)
    down = synth.expert_slabs(seed, n_experts, dim, ff, stream=23)
    x = synth.activations(seed + 1, (T, dim))
    return router, gate, up, down, x


def upload_moe(dev, router, gate, up, down, n_experts, dim, ff):
    from exec_beholdd_b200 import Weight

    return (dev.upload_weight(Weight(router.view(np.uint8).reshape(-1), 0, n_experts, dim)),
            dev.upload_weight(Weight(gate, 8, ff, dim), slabs=n_experts),
            dev.upload_weight(Weight(up, 8, ff, dim), slabs=n_experts),
            dev.upload_weight(Weight(down, 8, dim, ff), slabs=n_experts))


@pytest.mark.parametrize("n_experts,dim,top_k,T", [(128, 2048, 8, 1), (128, 2048, 8, 16), (128, 2048, 8, 200),
                                                  (4, 64, 2, 5), (40, 96, 3, 9), (8, 32, 8, 3)])
def test_routing_is_bit_exact(dev, oracle, n_experts, dim, top_k, T):
    import torch
    from exec_beholdd_b200 import Weight, synth

    router = synth.router_weights(77, n_experts, dim)
    x = synth.activations(78, (T, dim))
    probs, experts, weights, near, counts = oracle.moe_route(router, x, top_k)
    rw = dev.upload_weight(Weight(router.view(np.uint8).reshape(-1), 0, n_experts, dim))
    near_per = min(8, n_experts - top_k)
    e = torch.full((T, top_k), -1, dtype=torch.int32, device="cuda")
    w = torch.zeros((T, top_k), device="cuda")
    c = torch.full((n_experts,), -1, dtype=torch.int32, device="cuda")
    nm = torch.full((T, max(near_per, 1)), -1, dtype=torch.int32, device="cuda")
    p = torch.zeros((T, n_experts), device="cuda")
    dev.moe_route(rw, cuda(x), top_k, e, w, c, nm if near_per else None, p)
    dev.check_status()
    assert np.array_equal(e.cpu().numpy(), experts)                 # indices: exact
    assert np.array_equal(c.cpu().numpy(), counts)                  # per-expert counts: exact
    if near_per:
        assert np.array_equal(nm.cpu().numpy()[:, :near_per], near)
    assert np.array_equal(bits(p.cpu().numpy()), bits(probs))       # same order + same expf: bit-equal
    assert np.array_equal(bits(w.cpu().numpy()), bits(weights))
    rw.free()


def test_routing_ties_break_to_the_lower_index(dev, oracle):
    # crates/beholdd-model/src/qwen3moe/forward.rs:2231-2242: equal probabilities
    import torch
    from exec_beholdd_b200 import Weight

    router = np.zeros((4, 32), dtype=np.float32)
    router[1, 0] = router[2, 0] = 1.0   # experts 1 and 2 tie above 0 and 3
    x = np.zeros((1, 32), dtype=np.float32); x[0, 0] = 1.0
    rw = dev.upload_weight(Weight(router.view(np.uint8).reshape(-1), 0, 4, 32))
    e = torch.zeros((1, 2), dtype=torch.int32, device="cuda")
    w = torch.zeros((1, 2), device="cuda")
    nm = torch.zeros((1, 2), dtype=torch.int32, device="cuda")
    dev.moe_route(rw, cuda(x), 2, e, w, None, nm, None)
    assert e.cpu().numpy().tolist() == [[1, 2]] and w.cpu().numpy().tolist() == [[0.5, 0.5]]
    assert nm.cpu().numpy().tolist() == [[0, 3]]
    rw.free()


@pytest.mark.parametrize("n_experts,dim,ff,top_k,T", [(128, 2048, 768, 8, 1), (128, 2048, 768, 8, 16),
                                                     (128, 2048, 768, 8, 64), (8, 64, 32, 2, 5), (16, 256, 96, 4, 33),
                                                     (8, 512, 256, 2, 40), (4, 512, 256, 2, 150), (4, 256, 512, 4, 3), (4, 320, 96, 2, 70)])
def test_moe_layer_matches_oracle(dev, oracle, n_experts, dim, ff, top_k, T):
    import torch

    router, gate, up, down, x = moe_inputs(300 + T, n_experts, dim, ff, T)
    want, experts, weights, counts = oracle.moe_layer(router, gate, up, down, ff, x, top_k)
    rw, gw, uw, dw = upload_moe(dev, router, gate, up, down, n_experts, dim, ff)
    y = torch.full((T, dim), float("nan"), device="cuda")
    e = torch.zeros((T, top_k), dtype=torch.int32, device="cuda")
    w = torch.zeros((T, top_k), device="cuda")
    c = torch.zeros((n_experts,), dtype=torch.int32, device="cuda")
    dev.moe_layer(rw, gw, uw, dw, cuda(x), y, top_k, e, w, c)
    dev.check_status()
    assert np.array_equal(e.cpu().numpy(), experts)
    assert np.array_equal(c.cpu().numpy(), counts)
    assert np.array_equal(bits(w.cpu().numpy()), bits(weights))
    assert max_rel_err(y.cpu().numpy(), want) <= TOL
    # residual form: hidden += output (forward.rs:1405-1407)
    hidden = x.copy()
    hd = cuda(hidden)
    dev.moe_layer(rw, gw, uw, dw, cuda(x), hd, top_k, e, w, c, accumulate=True)
    assert max_rel_err(hd.cpu().numpy(), hidden + want) <= TOL
    # host-buffer entry point
    yh = np.zeros((T, dim), dtype=np.float32)
    eh = np.zeros((T, top_k), dtype=np.int32)
    dev.moe_layer_host(rw, gw, uw, dw, x, yh, top_k, experts=eh)
    assert np.array_equal(eh, experts) and max_rel_err(yh, want) <= TOL
    for h in (rw, gw, uw, dw):
        h.free()


@pytest.mark.parametrize("T,top_k,pattern", [(100, 2, "two_hot"), (70, 1, "one_expert"), (33, 4, "round_robin"), (0, 2, "empty")])
def test_moe_experts_with_skewed_and_empty_routing(dev, oracle, T, top_k, pattern):
    """Routing given from outside: every position on the same experts (one expert gets more
    than 32 routes and is cut into several groups), experts nobody selects, and no position
    at all. Assignments are explicit, so only the expert arithmetic is under test."""
    import torch
    from exec_beholdd_b200 import DeviceError, Weight

    n_experts, dim, ff = 8, 320, 96
    _, gate, up, down, x = moe_inputs(777, n_experts, dim, ff, max(T, 1))
    x = x[:T]
    if pattern == "two_hot":
        experts = np.tile(np.array([[5, 2]], dtype=np.int32), (T, 1))
    elif pattern == "one_expert":
        experts = np.full((T, 1), 3, dtype=np.int32)
    elif pattern == "round_robin":
        experts = (np.arange(T * top_k, dtype=np.int32).reshape(T, top_k) * 3) % n_experts
    else:
        experts = np.zeros((0, top_k), dtype=np.int32)
    from exec_beholdd_b200 import synth
    weights = np.abs(synth.activations(778, (max(T, 1), top_k)))[:T].astype(np.float32) + np.float32(0.25)
    gw = dev.upload_weight(Weight(gate, 8, ff, dim), slabs=n_experts)
    uw = dev.upload_weight(Weight(up, 8, ff, dim), slabs=n_experts)
    dw = dev.upload_weight(Weight(down, 8, dim, ff), slabs=n_experts)
    y = torch.full((T, dim), float("nan"), device="cuda")
    dev.moe_experts(gw, uw, dw, cuda(x) if T else torch.empty((0, dim), device="cuda"),
                    cuda(experts) if T else torch.empty((0, top_k), dtype=torch.int32, device="cuda"),
                    cuda(weights) if T else torch.empty((0, top_k), device="cuda"), y)
    dev.check_status()
    if T:
        want = oracle.moe_experts(gate, up, down, n_experts, dim, ff, x, experts, weights)
        assert max_rel_err(y.cpu().numpy(), want) <= TOL
        # a negative expert id is reported, not dereferenced (ids beyond the local range belong
        # to other ranks of an expert-parallel group and are skipped)
        bad = experts.copy()
        bad[0, 0] = -2
        dev.moe_experts(gw, uw, dw, cuda(x), cuda(bad), cuda(weights), y)
        with pytest.raises(DeviceError):
            dev.check_status()
    for h in (gw, uw, dw):
        h.free()


def test_grouped_expert_path_reports_an_expert_named_twice_by_a_position(dev, oracle):
    """The grouped kernels are launched only for the group sizes the number of positions allows (an expert has at most
    one route per position, as a top-k of distinct experts guarantees). Assignments that break the rule are reported
    through the status word instead of being computed wrongly."""
    import torch
    from exec_beholdd_b200 import DeviceError, Weight, synth

    n_experts, dim, ff, T, top_k = 8, 512, 256, 6, 2
    _, gate, up, down, x = moe_inputs(779, n_experts, dim, ff, T)
    experts = np.stack([np.arange(T) % n_experts, (np.arange(T) + 3) % n_experts], axis=1).astype(np.int32)
    weights = np.abs(synth.activations(780, (T, top_k))).astype(np.float32) + np.float32(0.25)
    gw = dev.upload_weight(Weight(gate, 8, ff, dim), slabs=n_experts)
    uw = dev.upload_weight(Weight(up, 8, ff, dim), slabs=n_experts)
    dw = dev.upload_weight(Weight(down, 8, dim, ff), slabs=n_experts)
    y = torch.full((T, dim), float("nan"), device="cuda")
    dev.moe_experts(gw, uw, dw, cuda(x), cuda(experts), cuda(weights), y)
    dev.check_status()
    assert max_rel_err(y.cpu().numpy(), oracle.moe_experts(gate, up, down, n_experts, dim, ff, x, experts, weights)) <= TOL
    dup = np.full((T, top_k), 5, dtype=np.int32)     # expert 5 gets 12 routes from 6 positions
    dev.moe_experts(gw, uw, dw, cuda(x), cuda(dup), cuda(weights), y)
    with pytest.raises(DeviceError):
        dev.check_status()
    dev.moe_experts(gw, uw, dw, cuda(x), cuda(experts), cuda(weights), y)   # the next call works
    dev.check_status()
    for h in (gw, uw, dw):
        h.free()


def test_expert_parallel_partition_sums_to_the_whole(dev, oracle):
    """Each rank of an expert-parallel group applies only its experts; the partial outputs
    add up to the full layer."""
    import torch
    from exec_beholdd_b200 import Weight

    n_experts, dim, ff, top_k, T = 16, 256, 96, 4, 12
    router, gate, up, down, x = moe_inputs(555, n_experts, dim, ff, T)
    want, experts, weights, _ = oracle.moe_layer(router, gate, up, down, ff, x, top_k)
    xd, ed, wd = cuda(x), cuda(experts), cuda(weights)
    total = torch.zeros((T, dim), device="cuda")
    parts = 4
    per = n_experts // parts
    gu_slab, d_slab = ff * (dim // 32) * 34, dim * (ff // 32) * 34
    for r in range(parts):
        gw = dev.upload_weight(Weight(gate[r * per * gu_slab:(r + 1) * per * gu_slab], 8, ff, dim), slabs=per)
        uw = dev.upload_weight(Weight(up[r * per * gu_slab:(r + 1) * per * gu_slab], 8, ff, dim), slabs=per)
        dw = dev.upload_weight(Weight(down[r * per * d_slab:(r + 1) * per * d_slab], 8, dim, ff), slabs=per)
        dev.moe_experts(gw, uw, dw, xd, ed, wd, total, first_expert=r * per, n_local=per, accumulate=True)
        for h in (gw, uw, dw):
            h.free()
    dev.check_status()
    assert max_rel_err(total.cpu().numpy(), want) <= TOL


@pytest.mark.parametrize("name", gc.names())
def test_routed_block_matches_reference_numpy_golden(dev, oracle, name):
    """The CUDA path against the outputs of the reference's own f64 NumPy implementation."""
    import torch

    g = gc.load(name)
    dim, ff, k, ne = int(g["dim"]), int(g["expert_ff"]), int(g["top_k"]), int(g["n_experts"])
    x = np.stack([oracle.dequantize(r, 8, 1, dim) for r in g["embedding_rows_q8_0"]])
    h2 = np.stack([oracle.rmsnorm(xi, g["ffn_norm"], float(g["eps"])) for xi in x])
    rw, gw, uw, dw = upload_moe(dev, g["router"], g["gate_exps"], g["up_exps"], g["down_exps"], ne, dim, ff)
    T = x.shape[0]
    hidden = cuda(x)
    e = torch.zeros((T, k), dtype=torch.int32, device="cuda")
    w = torch.zeros((T, k), device="cuda")
    dev.moe_layer(rw, gw, uw, dw, cuda(h2), hidden, k, e, w, None, accumulate=True)
    dev.check_status()
    assert np.array_equal(e.cpu().numpy(), g["ref_experts"])
    assert np.abs(w.cpu().numpy() - g["ref_weights"]).max() <= gc.ROUTING_MAX_ABS
    assert gc.rel_l2(hidden.cpu().numpy(), g["ref_hidden"]) <= 1e-5
    for h in (rw, gw, uw, dw):
        h.free()


def test_full_size_moe_layer_is_deterministic_and_linear_in_route_weights(dev):
    """T = 512 at the benchmark shapes: too slow for the scalar oracle, so check the
    size-independent properties: run-to-run bit identity, counts sum to T*k, and the
    expert half is linear in the route weights."""
    import torch

    n_experts, dim, ff, top_k, T = 128, 2048, 768, 8, 512
    router, gate, up, down, x = moe_inputs(909, n_experts, dim, ff, T)
    rw, gw, uw, dw = upload_moe(dev, router, gate, up, down, n_experts, dim, ff)
    xd = cuda(x)
    outs = []
    for _ in range(2):
        y = torch.empty((T, dim), device="cuda")
        e = torch.zeros((T, top_k), dtype=torch.int32, device="cuda")
        w = torch.zeros((T, top_k), device="cuda")
        c = torch.zeros((n_experts,), dtype=torch.int32, device="cuda")
        dev.moe_layer(rw, gw, uw, dw, xd, y, top_k, e, w, c)
        outs.append((y, e, w, c))
    dev.check_status()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    e, w, c = outs[0][1], outs[0][2], outs[0][3]
    assert int(c.sum()) == T * top_k
    assert np.array_equal(c.cpu().numpy(), np.bincount(e.cpu().numpy().reshape(-1), minlength=n_experts))
    assert torch.all(e.sort(dim=1).values[:, 1:] != e.sort(dim=1).values[:, :-1])  # no expert twice per position
    assert torch.allclose(w.sum(dim=1), torch.ones(T, device="cuda"), atol=1e-6)
    y2 = torch.empty((T, dim), device="cuda")
    dev.moe_experts(gw, uw, dw, xd, e, (w * 2.0).contiguous(), y2)
    assert max_rel_err(y2.cpu().numpy(), (outs[0][0] * 2.0).cpu().numpy()) <= 1e-5
    for h in (rw, gw, uw, dw):
        h.free()
