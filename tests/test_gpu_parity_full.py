"""GPU parity at the full benchmark shapes, against the CPU oracle.

The scalar oracle is slow, so each case compares a sample: a few dozen weight rows of a full
matrix (the oracle runs on exactly those packed rows), a 16-row sample of a prefill batch, or
the whole routed layer at T = 512 (a few seconds of CPU). Inputs are also drawn with heavy
tails: 1 % of the activations scaled by 20, and one scale group holding a 1e4 spike, because
the decode and routed-expert kernels quantise activations per scale group.

Bar: indices and counts bit-exact; floating point within 2e-3, measured as
max_i |g_i - r_i| / max(|r_i|, rms(r)).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 2e-3


def max_rel_err(got, want):
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    rms = np.sqrt((want ** 2).mean()) if want.size else 0.0
    den = np.maximum(np.abs(want), max(rms, 1e-30))
    return float((np.abs(got - want) / den).max()) if want.size else 0.0


@pytest.fixture(scope="module")
def dev():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from exec_beholdd_b200 import CudaDevice

    d = CudaDevice(0)
    yield d
    d.close()


def cuda(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def heavy_tailed(seed, shape, spike=True):
    """N(0,1) with 1 % of entries x20 and, per vector, one 32-column group holding a 1e4 spike."""
    from exec_beholdd_b200 import synth

    x = synth.activations(seed, shape, outliers=True)
    if spike:
        flat = x.reshape(-1, shape[-1])
        for b in range(flat.shape[0]):
            flat[b, (37 * (b + 1)) % shape[-1]] = np.float32(1.0e4 * (-1) ** b)
    return x


def sample_rows(packed, kind, rows, cols, picks):
    """The packed bytes of the picked rows, as their own small matrix."""
    from exec_beholdd_b200 import synth

    rb = synth.packed_bytes(kind, 1, cols)
    m = packed.reshape(rows, rb)
    return np.ascontiguousarray(m[picks]).reshape(-1)


@pytest.mark.parametrize("rows,cols", [(12288, 4096), (4096, 12288)])
@pytest.mark.parametrize("kind", [8, 12, 14])
def test_decode_matvec_full_size_against_oracle_rows(dev, oracle, kind, rows, cols):
    """Batches 1, 2, 4 and 8 (every dispatch class of bhd_matvec) at the decode configuration's
    shapes, N(0,1) and heavy-tailed activations, against the oracle on 48 sampled rows."""
    import torch
    from exec_beholdd_b200 import Weight, synth

    packed = synth.matrix(kind, 101, rows, cols)
    picks = np.unique(np.concatenate([np.arange(0, rows, rows // 40), [1, 15, 16, rows - 17, rows - 1]]))
    sub = sample_rows(packed, kind, rows, cols, picks)
    w = dev.upload_weight(Weight(packed, kind, rows, cols))
    worst = 0.0
    for batch in (1, 2, 4, 8):
        for tails in (False, True):
            x = heavy_tailed(200 + batch, (batch, cols)) if tails else synth.activations(200 + batch, (batch, cols))
            want = oracle.matvec_batch(sub, kind, len(picks), cols, x)
            y = torch.full((batch, rows), float("nan"), device="cuda")
            dev.matvec_resident(w, cuda(x), y)
            got = y.cpu().numpy()
            assert np.isfinite(got).all()
            err = max_rel_err(got[:, picks], want)
            worst = max(worst, err)
            assert err <= TOL, (kind, rows, cols, batch, tails, err)
    dev.check_status()
    print(f"kind {kind} {rows}x{cols}: worst max-rel-err {worst:.2e}")
    w.free()


@pytest.mark.parametrize("m,n,k", [(128, 12288, 4096), (512, 12288, 4096), (2048, 12288, 4096), (128, 4096, 4096),
                                   (512, 4096, 4096), (2048, 4096, 4096), (192, 384, 32 * 129), (100, 130, 32 * 3)])
def test_prefill_matmul_full_size_against_oracle_sample(dev, oracle, m, n, k):
    """The prefill configuration's shapes (and two K = 32 * odd cases, where the last 64-column
    slice is half filled): 16 sampled positions against the oracle, all columns; activations
    N(0,1) with 1 % x20 outliers as the configuration states."""
    import torch
    from exec_beholdd_b200 import Weight, synth

    packed = synth.q8_0_matrix(141, n, k)
    x = synth.activations(143, (m, k), outliers=True)
    sample = np.unique(np.concatenate([np.arange(0, m, max(1, m // 14)), [m - 1]]))
    want = oracle.matvec_batch(packed, 8, n, k, x[sample])
    w = dev.upload_weight(Weight(packed, 8, n, k))
    y = torch.full((m, n), float("nan"), device="cuda")
    dev.matmul_resident(w, cuda(x), y)
    dev.check_status()
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    err = max_rel_err(got[sample], want)
    print(f"prefill M={m} N={n} K={k}: max-rel-err {err:.2e}")
    assert err <= TOL
    w.free()


@pytest.mark.parametrize("m,n,k", [(700, 520, 2048), (256, 130, 1024), (1300, 256, 3072)])
def test_every_prefill_kernel_form_gives_the_same_bits(dev, oracle, m, n, k):
    """The prefill matmul exists as one CTA per tile (weight operand in shared or in tensor memory), persistent CTAs, and
    persistent CTA pairs on 256- and 512-token tiles (the library chooses by shape). Ragged shapes (a last row pair with few rows, a last token tile with few
    tokens): every form against the oracle on a sample; the forms that add a column's products in one chain (all but
    the one-CTA-per-tile form, which keeps even and odd slices in two accumulators) are bit-identical."""
    import torch
    from exec_beholdd_b200 import Weight, synth

    packed = synth.q8_0_matrix(151, n, k)
    x = synth.activations(153, (m, k), outliers=True)
    sample = np.unique(np.minimum(np.concatenate([np.arange(0, m, max(1, m // 12)), [255, 256, m - 1]]), m - 1))
    want = oracle.matvec_batch(packed, 8, n, k, x[sample])
    w = dev.upload_weight(Weight(packed, 8, n, k))
    xd = cuda(x)
    outs = {}
    try:
        for impl in (1, 2, 3, 4, 5, 0):
            assert dev.lib.bhd_debug_option(dev.ctx, 3, impl) == 0
            y = torch.full((m, n), float("nan"), device="cuda")
            dev.matmul_resident(w, xd, y)
            dev.check_status()
            outs[impl] = y.cpu().numpy()
            assert np.isfinite(outs[impl]).all()
            assert max_rel_err(outs[impl][sample], want) <= TOL, impl
    finally:
        dev.lib.bhd_debug_option(dev.ctx, 3, 0)
    for impl in (4, 5, 0):
        assert np.array_equal(outs[impl].view(np.uint32), outs[3].view(np.uint32)), impl
    assert max_rel_err(outs[1], outs[3]) <= 1e-4
    w.free()


@pytest.mark.parametrize("m,n,k", [(512, 4096, 4096), (2048, 12288, 4096), (700, 520, 2048), (256, 130, 1024)])
def test_q4_k_prefill_on_the_tensor_cores_against_oracle_sample(dev, oracle, m, n, k):
    """Q4_K weights take the CTA-pair matmul from 256 tokens on (the converter forms fp16((d * sc) * q - dmin * m) from
    the nibbles): 16 sampled positions against the oracle on all columns, both tile widths bit-identical."""
    import torch
    from exec_beholdd_b200 import Weight, synth

    packed = synth.q4_k_matrix(161, n, k)
    x = synth.activations(163, (m, k), outliers=True)
    sample = np.unique(np.minimum(np.concatenate([np.arange(0, m, max(1, m // 14)), [255, 256, m - 1]]), m - 1))
    want = oracle.matvec_batch(packed, 12, n, k, x[sample])
    w = dev.upload_weight(Weight(packed, 12, n, k))
    xd = cuda(x)
    outs = {}
    try:
        for impl in (0, 3, 5):
            assert dev.lib.bhd_debug_option(dev.ctx, 3, impl) == 0
            launches = dev.launch_count
            y = torch.full((m, n), float("nan"), device="cuda")
            dev.matmul_resident(w, xd, y)
            dev.check_status()
            assert dev.launch_count - launches == 2          # the fp16 conversion of x and one matmul kernel
            outs[impl] = y.cpu().numpy()
            assert np.isfinite(outs[impl]).all()
            err = max_rel_err(outs[impl][sample], want)
            print(f"Q4_K prefill M={m} N={n} K={k} form {impl}: max-rel-err {err:.2e}")
            assert err <= TOL, impl
    finally:
        dev.lib.bhd_debug_option(dev.ctx, 3, 0)
    assert np.array_equal(outs[3].view(np.uint32), outs[5].view(np.uint32))
    w.free()


@pytest.mark.parametrize("m,n,k", [(512, 4096, 4096), (2048, 12288, 4096), (700, 520, 2048), (256, 130, 6144)])
def test_q6_k_prefill_on_the_tensor_cores_against_oracle_sample(dev, oracle, m, n, k):
    """Q6_K weights whose rows are a multiple of 16 bytes (columns a multiple of 2048) take the CTA-pair matmul from 256
    tokens on: the 210-byte superblocks sit at every even offset 0..14 of their 16-byte aligned windows over a row, and the
    converter forms fp16((d * scale) * (code - 32)). 16 sampled positions against the oracle, both tile widths
    bit-identical."""
    import torch
    from exec_beholdd_b200 import Weight, synth

    packed = synth.q6_k_matrix(171, n, k)
    x = synth.activations(173, (m, k), outliers=True)
    sample = np.unique(np.minimum(np.concatenate([np.arange(0, m, max(1, m // 14)), [255, 256, m - 1]]), m - 1))
    want = oracle.matvec_batch(packed, 14, n, k, x[sample])
    w = dev.upload_weight(Weight(packed, 14, n, k))
    xd = cuda(x)
    outs = {}
    try:
        for impl in (0, 3, 5):
            assert dev.lib.bhd_debug_option(dev.ctx, 3, impl) == 0
            launches = dev.launch_count
            y = torch.full((m, n), float("nan"), device="cuda")
            dev.matmul_resident(w, xd, y)
            dev.check_status()
            assert dev.launch_count - launches == 2          # the fp16 conversion of x and one matmul kernel
            outs[impl] = y.cpu().numpy()
            assert np.isfinite(outs[impl]).all()
            err = max_rel_err(outs[impl][sample], want)
            print(f"Q6_K prefill M={m} N={n} K={k} form {impl}: max-rel-err {err:.2e}")
            assert err <= TOL, impl
    finally:
        dev.lib.bhd_debug_option(dev.ctx, 3, 0)
    assert np.array_equal(outs[3].view(np.uint32), outs[5].view(np.uint32))
    w.free()


def test_q6_k_prefill_with_rows_off_the_16_byte_grid_keeps_the_batched_kernels(dev, oracle):
    """Three Q6_K superblocks a row are 630 bytes: no tensor map can stride over such rows, so the matmul stays on the
    integer batched kernels and still agrees with the oracle."""
    from exec_beholdd_b200 import Weight, synth

    m, n, k = 256, 96, 768
    packed = synth.q6_k_matrix(175, n, k)
    x = synth.activations(177, (m, k))
    w = dev.upload_weight(Weight(packed, 14, n, k))
    import torch
    y = torch.full((m, n), float("nan"), device="cuda")
    dev.matmul_resident(w, cuda(x), y)
    dev.check_status()
    got = y.cpu().numpy()
    want = oracle.matvec_batch(packed, 14, n, k, x)
    assert max_rel_err(got, want) <= TOL
    w.free()


def moe_inputs(seed, n_experts, dim, ff, T, tails):
    from exec_beholdd_b200 import synth

    router = synth.router_weights(seed, n_experts, dim)
    gate = synth.expert_slabs(seed, n_experts, ff, dim, stream=21)
    up = synth.expert_slabs(seed, n_experts, ff, dim, stream=22)
    down = synth.expert_slabs(seed, n_experts, dim, ff, stream=23)
    x = heavy_tailed(seed + 1, (T, dim), spike=True) if tails else synth.activations(seed + 1, (T, dim))
    return router, gate, up, down, x


@pytest.mark.parametrize("T,tails", [(512, False), (512, True), (64, True), (16, True), (1, True)])
def test_routed_layer_at_benchmark_shapes_against_oracle(dev, oracle, T, tails):
    """Qwen3-30B-A3B shapes, every token count of the configuration, the whole layer against the
    oracle: indices, counts and route weights exact, outputs within tolerance."""
    import torch
    from exec_beholdd_b200 import Weight

    ne, dim, ff, k = 128, 2048, 768, 8
    router, gate, up, down, x = moe_inputs(400 + T, ne, dim, ff, T, tails)
    want, experts, weights, counts = oracle.moe_layer(router, gate, up, down, ff, x, k)
    rw = dev.upload_weight(Weight(router.view(np.uint8).reshape(-1), 0, ne, dim))
    gw = dev.upload_weight(Weight(gate, 8, ff, dim), slabs=ne)
    uw = dev.upload_weight(Weight(up, 8, ff, dim), slabs=ne)
    dw = dev.upload_weight(Weight(down, 8, dim, ff), slabs=ne)
    y = torch.full((T, dim), float("nan"), device="cuda")
    e = torch.zeros((T, k), dtype=torch.int32, device="cuda")
    w = torch.zeros((T, k), device="cuda")
    c = torch.zeros((ne,), dtype=torch.int32, device="cuda")
    dev.moe_layer(rw, gw, uw, dw, cuda(x), y, k, e, w, c)
    dev.check_status()
    assert np.array_equal(e.cpu().numpy(), experts)
    assert np.array_equal(c.cpu().numpy(), counts)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), weights.view(np.uint32))
    err = max_rel_err(y.cpu().numpy(), want)
    print(f"routed layer T={T} tails={tails}: max-rel-err {err:.2e}, busiest expert {int(counts.max())} routes")
    assert err <= TOL
    for h in (rw, gw, uw, dw):
        h.free()


@pytest.mark.parametrize("min_cls,T", [(3, 512), (2, 512), (4, 2048), (2, 40)])
def test_tensor_core_grouped_expert_kernel_against_oracle(dev, oracle, min_cls, T):
    """The tcgen05 grouped kernel (weights in tensor memory, exact hi + lo operands) is an option of the routed
    layer (groups of 9+ / 17+ / 33+ routes per expert; the default runs every group on the integer kernel). At the
    benchmark shapes against the oracle (T = 2048: against the default path, to keep the CPU time in bounds)."""
    import torch
    from exec_beholdd_b200 import Weight

    ne, dim, ff, k = 128, 2048, 768, 8
    if T == 40:
        ne = 8  # few experts: 40 routes per expert
    router, gate, up, down, x = moe_inputs(900 + T, ne, dim, ff, T, tails=True)
    rw = dev.upload_weight(Weight(router.view(np.uint8).reshape(-1), 0, ne, dim))
    gw = dev.upload_weight(Weight(gate, 8, ff, dim), slabs=ne)
    uw = dev.upload_weight(Weight(up, 8, ff, dim), slabs=ne)
    dw = dev.upload_weight(Weight(down, 8, dim, ff), slabs=ne)
    xd = cuda(x)
    e = torch.zeros((T, k), dtype=torch.int32, device="cuda")
    w = torch.zeros((T, k), device="cuda")
    c = torch.zeros((ne,), dtype=torch.int32, device="cuda")
    if T <= 512:
        want, experts, _, _ = oracle.moe_layer(router, gate, up, down, ff, x, k)
    else:
        yd = torch.empty((T, dim), device="cuda")
        dev.moe_layer(rw, gw, uw, dw, xd, yd, k, e, w, c)
        want, experts = yd.cpu().numpy(), e.cpu().numpy()
    try:
        assert dev.lib.bhd_debug_option(dev.ctx, 1, min_cls) == 0
        y = torch.full((T, dim), float("nan"), device="cuda")
        dev.moe_layer(rw, gw, uw, dw, xd, y, k, e, w, c)
        dev.check_status()
    finally:
        dev.lib.bhd_debug_option(dev.ctx, 1, 0)
    assert np.array_equal(e.cpu().numpy(), experts)
    err = max_rel_err(y.cpu().numpy(), want)
    print(f"tensor-core grouped kernel, groups of class {min_cls}+, T={T}: max-rel-err {err:.2e}, busiest expert {int(c.max())} routes")
    assert err <= TOL
    for h in (rw, gw, uw, dw):
        h.free()


def test_route_margin_is_reported(dev, oracle):
    """The smallest gap between the last selected and the first rejected probability: the
    distance of the selection from a tie that a one-ulp difference in expf could flip
    (the reference's HIP benches export the same figure as "route_margin")."""
    import torch
    from exec_beholdd_b200 import Weight, synth

    ne, dim, k, T = 128, 2048, 8, 512
    router = synth.router_weights(77, ne, dim)
    x = synth.activations(78, (T, dim))
    probs, experts, _, _, _ = oracle.moe_route(router, x, k)
    rw = dev.upload_weight(Weight(router.view(np.uint8).reshape(-1), 0, ne, dim))
    e = torch.zeros((T, k), dtype=torch.int32, device="cuda")
    w = torch.zeros((T, k), device="cuda")
    p = torch.zeros((T, ne), device="cuda")
    dev.moe_route(rw, cuda(x), k, e, w, None, None, p)
    dev.check_status()
    ps = np.sort(p.cpu().numpy(), axis=1)[:, ::-1]
    margin = float((ps[:, k - 1] - ps[:, k]).min())
    ulp = float(np.spacing(ps[:, k - 1]).max())
    print(f"min rank-{k}/rank-{k + 1} probability gap over {T} positions: {margin:.3e} ({margin / ulp:.0f} ulps)")
    assert margin >= 0.0
    assert np.array_equal(e.cpu().numpy(), experts)
    assert np.array_equal(p.cpu().numpy().view(np.uint32), probs.view(np.uint32))
    rw.free()
