"""GPU parity of the operators around the projections and the experts in a transformer layer:
RMSNorm / QK-norm, rotary embedding, causal and incremental attention, embedding rows, BF16
weights; and one whole qwen3moe-style layer composed from the library's operators against the
same layer composed from the oracle's.

The kernels follow the CPU's arithmetic step by step, so most comparisons are exact.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 2e-3


def max_rel_err(got, want):
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    den = np.maximum(np.abs(want), max(np.sqrt((want ** 2).mean()), 1e-30))
    return float((np.abs(got - want) / den).max())


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


def cuda(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_rmsnorm_rows_and_qk_norm(dev, oracle):
    import torch
    from exec_beholdd_b200 import ShapeError, synth

    for rows, n, with_w in ((5, 2048, True), (3, 4096, False), (64, 128, True), (1, 7, True)):
        x = synth.activations(11 + n, (rows, n), outliers=True)
        w = synth.normal(12, 3, n) * np.float32(0.1) + np.float32(1.0) if with_w else None
        want = np.stack([oracle.rmsnorm(x[r], w, 1e-6) for r in range(rows)])
        y = torch.empty((rows, n), device="cuda")
        dev.rmsnorm_resident(y, cuda(x), cuda(w) if with_w else None, 1e-6)
        got = y.cpu().numpy()
        # the f64 sum of squares is added in another order: the f32 factor differs by at most one ulp
        assert max_rel_err(got, want) <= 2e-7, (rows, n)
    with pytest.raises(ShapeError):
        dev.rmsnorm_resident(torch.empty((1, 4), device="cuda"), torch.zeros((1, 4), device="cuda"), None, -1.0)


def test_rope_both_layouts_bit_exact(dev, oracle):
    import torch
    from exec_beholdd_b200 import synth

    # the reference's routing test, crates/beholdd-backend/src/cpu.rs:1369-1386
    cos, sin = cuda(np.array([[0.0, 0.0]], dtype=np.float32)), cuda(np.array([[1.0, 1.0]], dtype=np.float32))
    x = cuda(np.array([[[1.0, 2.0, 3.0, 4.0]]], dtype=np.float32))
    dev.rope_resident(x, cos, sin, split_half=False)
    assert x.cpu().numpy().reshape(-1).tolist() == [-2.0, 1.0, -4.0, 3.0]
    x = cuda(np.array([[[1.0, 2.0, 3.0, 4.0]]], dtype=np.float32))
    dev.rope_resident(x, cos, sin, split_half=True)
    assert x.cpu().numpy().reshape(-1).tolist() == [-3.0, -4.0, 1.0, 2.0]
    dev.rope_resident(x, cos, sin, split_half=True, inverse=True)
    assert x.cpu().numpy().reshape(-1).tolist() == [1.0, 2.0, 3.0, 4.0]
    # seeded: 9 positions x 6 heads x head_dim 128, theta 1e6, positions 40..48
    n_pos, heads, hd = 9, 6, 128
    xs = synth.activations(21, (n_pos, heads, hd))
    tables = [oracle.rope_table(1.0e6, hd, 40 + p) for p in range(n_pos)]
    cos_np, sin_np = np.stack([t[0] for t in tables]), np.stack([t[1] for t in tables])
    for split in (True, False):
        want = np.stack([np.stack([oracle.rope(xs[p, h], cos_np[p], sin_np[p], split_half=split) for h in range(heads)]) for p in range(n_pos)])
        xd = cuda(xs)
        dev.rope_resident(xd, cuda(cos_np), cuda(sin_np), split_half=split)
        assert np.array_equal(bits(xd.cpu().numpy()), bits(want))


def test_attention_reference_vectors_and_seeded_cache_bit_exact(dev, oracle):
    import torch
    from exec_beholdd_b200 import ShapeError, synth

    # crates/beholdd-backend/src/cpu.rs:1389-1411
    out = torch.zeros((2, 1, 2), device="cuda")
    dev.attention_resident(out, cuda(np.array([1.0, 0.0, 1.0, 0.0], np.float32).reshape(2, 1, 2)),
                           cuda(np.array([0.0, 0.0, np.log(np.float32(3.0)), 0.0], np.float32).reshape(2, 1, 2)),
                           cuda(np.array([2.0, 4.0, 6.0, 8.0], np.float32).reshape(2, 1, 2)), 0, 2, 1.0)
    assert np.abs(out.cpu().numpy().reshape(-1) - np.array([2.0, 4.0, 5.0, 7.0])).max() < 1e-6
    # crates/beholdd-backend/src/cpu.rs:1414-1440: the causal mask and contiguous GQA groups
    out = torch.full((2, 4, 1), float("nan"), device="cuda")
    dev.attention_resident(out, torch.zeros((2, 4, 1), device="cuda"), torch.zeros((2, 2, 1), device="cuda"),
                           cuda(np.array([1.0, 10.0, 3.0, 30.0], np.float32).reshape(2, 2, 1)), 0, 2, 1.0)
    assert out.cpu().numpy().reshape(-1).tolist() == [1.0, 1.0, 10.0, 10.0, 2.0, 2.0, 20.0, 20.0]
    # crates/beholdd-backend/src/cpu.rs:1544-1570: a cache entry in the query's future is ignored
    out = torch.full((1, 1, 1), float("nan"), device="cuda")
    dev.attention_resident(out, cuda(np.ones((1, 1, 1), np.float32)), cuda(np.array([0.0, np.log(np.float32(3.0)), 100.0], np.float32).reshape(3, 1, 1)),
                           cuda(np.array([2.0, 6.0, 10000.0], np.float32).reshape(3, 1, 1)), 1, 3, 1.0)
    assert abs(float(out.cpu().numpy().reshape(-1)[0]) - 5.0) < 1e-6
    with pytest.raises(ShapeError):
        dev.attention_resident(out, cuda(np.ones((1, 1, 1), np.float32)), torch.zeros((1, 1, 1), device="cuda"),
                               torch.zeros((1, 1, 1), device="cuda"), 1, 1, 1.0)
    # seeded, the shapes of the full-forward configuration: 32 query heads, 4 kv heads, head_dim 128;
    # a 70-position prefill, then 3 more positions against the cache (absolute positions 70..72)
    n_heads, n_kv, hd, n_pos = 32, 4, 128, 73
    q = synth.activations(31, (n_pos, n_heads, hd))
    k = synth.activations(32, (n_pos, n_kv, hd))
    v = synth.activations(33, (n_pos, n_kv, hd))
    scale = float(1.0 / np.sqrt(np.float32(hd)))
    want = oracle.causal_attention(q, k, v, n_pos, n_heads, n_kv, hd, scale).reshape(n_pos, n_heads, hd)
    kd, vd = cuda(k), cuda(v)
    out = torch.empty((70, n_heads, hd), device="cuda")
    dev.attention_resident(out, cuda(q[:70]), kd, vd, 0, 70, scale)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want[:70]))
    out = torch.empty((3, n_heads, hd), device="cuda")
    dev.attention_resident(out, cuda(q[70:]), kd, vd, 70, 73, scale)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want[70:]))
    # a block-of-queries launch that starts inside the cache (33 queries at positions 40..72), and other group sizes
    # (2 and 1 query heads per kv head: 16 and 32 positions per CTA)
    out = torch.empty((33, n_heads, hd), device="cuda")
    dev.attention_resident(out, cuda(q[40:]), kd, vd, 40, 73, scale)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want[40:]))
    for heads2 in (8, 4):
        q2 = synth.activations(37, (n_pos, heads2, hd))
        want2 = oracle.causal_attention(q2, k, v, n_pos, heads2, n_kv, hd, scale).reshape(n_pos, heads2, hd)
        out = torch.empty((n_pos, heads2, hd), device="cuda")
        dev.attention_resident(out, cuda(q2), kd, vd, 0, n_pos, scale)
        assert np.array_equal(bits(out.cpu().numpy()), bits(want2))
    # a longer cache (several value tiles of the kernel), one decode query: the launch-parameter form and the form that
    # reads the position from device memory, both against the oracle to the bit
    n_pos = 203
    q1 = synth.activations(34, (1, n_heads, hd))
    k = synth.activations(35, (n_pos + 5, n_kv, hd))
    v = synth.activations(36, (n_pos + 5, n_kv, hd))
    want = oracle.incremental_attention(q1, k[:n_pos], v[:n_pos], 1, n_pos - 1, n_pos, n_heads, n_kv, hd, scale).reshape(1, n_heads, hd)
    kd, vd = cuda(k), cuda(v)
    out = torch.empty((1, n_heads, hd), device="cuda")
    dev.attention_resident(out, cuda(q1), kd, vd, n_pos - 1, n_pos, scale)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want))
    out.fill_(float("nan"))
    pos = torch.tensor([n_pos - 1], dtype=torch.int32, device="cuda")
    dev.attention_at_resident(out, cuda(q1), kd, vd, pos, scale)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want))
    dev.check_status()
    # a block-of-queries launch over a cache too long for the scores to sit in shared memory (persistent CTAs, scores in
    # the context workspace): 40 queries at positions 1100..1139
    n_long, n_q = 1140, 40
    ql = synth.activations(44, (n_q, n_heads, hd))
    kl, vl = synth.activations(45, (n_long, n_kv, hd)), synth.activations(46, (n_long, n_kv, hd))
    want_l = oracle.incremental_attention(ql, kl, vl, n_q, n_long - n_q, n_long, n_heads, n_kv, hd, scale).reshape(n_q, n_heads, hd)
    out_l = torch.full((n_q, n_heads, hd), float("nan"), device="cuda")
    dev.attention_resident(out_l, cuda(ql), cuda(kl), cuda(vl), n_long - n_q, n_long, scale)
    assert np.array_equal(bits(out_l.cpu().numpy()), bits(want_l))
    # the four-CTA decode kernel at its edges: fewer keys than CTAs, one key tile, several key and value tiles
    for n_vis in (1, 2, 5, 130, 1100):
        qn = synth.activations(38 + n_vis, (1, n_heads, hd))
        kn, vn = synth.activations(39, (n_vis, n_kv, hd)), synth.activations(40, (n_vis, n_kv, hd))
        want_n = oracle.incremental_attention(qn, kn, vn, 1, n_vis - 1, n_vis, n_heads, n_kv, hd, scale).reshape(1, n_heads, hd)
        out_n = torch.full((1, n_heads, hd), float("nan"), device="cuda")
        dev.attention_resident(out_n, cuda(qn), cuda(kn), cuda(vn), n_vis - 1, n_vis, scale)
        assert np.array_equal(bits(out_n.cpu().numpy()), bits(want_n)), n_vis
    dev.check_status()
    pos.fill_(n_pos + 5)                       # a position outside the cache: reported, nothing written
    out.fill_(7.0)
    dev.attention_at_resident(out, cuda(q1), kd, vd, pos, scale)
    with pytest.raises(Exception):
        dev.check_status()
    assert float(out.min()) == 7.0


def test_fused_decode_step_operator_equals_the_separate_calls(dev):
    """QK-norm, rope and the cache append of one decode position in one launch, with the position read from device
    memory, against the separate operators (which are checked against the oracle above): the same bits."""
    import torch
    from exec_beholdd_b200 import synth
    from exec_beholdd_b200.qwen3moe import rope_tables

    n_heads, n_kv, hd, ctx_len, eps = 32, 4, 128, 40, 1e-6
    cos, sin = rope_tables(1.0e6, hd, ctx_len)
    cos, sin = cuda(cos), cuda(sin)
    qn, kn = cuda(synth.normal(3, 1, hd) * np.float32(0.1) + np.float32(1.0)), cuda(synth.normal(3, 2, hd) * np.float32(0.1) + np.float32(1.0))
    for p in (0, 17, 39):
        q, k, v = cuda(synth.activations(50 + p, (1, n_heads, hd))), cuda(synth.activations(60 + p, (1, n_kv, hd))), cuda(synth.activations(70 + p, (1, n_kv, hd)))
        pos = torch.tensor([p], dtype=torch.int32, device="cuda")
        q1, k1 = q.clone(), k.clone()
        kc1, vc1 = torch.zeros((ctx_len, n_kv, hd), device="cuda"), torch.zeros((ctx_len, n_kv, hd), device="cuda")
        dev.rmsnorm_resident(q1, q1, qn, eps)
        dev.rmsnorm_resident(k1, k1, kn, eps)
        dev.rope_at_resident(q1, cos, sin, pos)
        dev.rope_at_resident(k1, cos, sin, pos)
        dev.store_row_at_resident(kc1.view(ctx_len, -1), k1.view(-1), pos)
        dev.store_row_at_resident(vc1.view(ctx_len, -1), v.view(-1), pos)
        ref = torch.empty_like(q)                      # and rope_at against the launch-parameter form
        ref.copy_(q)
        dev.rmsnorm_resident(ref, ref, qn, eps)
        dev.rope_resident(ref, cos[p:p + 1], sin[p:p + 1])
        assert torch.equal(ref, q1)
        q2, k2 = q.clone(), k.clone()
        kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(vc1)
        dev.qk_norm_rope_store_at_resident(q2, k2, v, qn, kn, cos, sin, kc2, vc2, pos, eps)
        dev.check_status()
        for a, b in ((q1, q2), (k1, k2), (kc1, kc2), (vc1, vc2)):
            assert np.array_equal(bits(a.cpu().numpy()), bits(b.cpu().numpy()))
        assert float(kc2[p].abs().max()) > 0 and float(vc2[p].abs().max()) > 0
    pos = torch.tensor([ctx_len], dtype=torch.int32, device="cuda")   # outside the cache: reported, nothing written
    kc2.zero_()
    dev.qk_norm_rope_store_at_resident(q2, k2, v, qn, kn, cos, sin, kc2, vc2, pos, eps)
    with pytest.raises(Exception):
        dev.check_status()
    assert float(kc2.abs().max()) == 0.0


def test_embedding_rows_and_bf16_weights(dev, oracle):
    import torch
    from exec_beholdd_b200 import DeviceError, Weight, synth

    rows, cols = 300, 2048
    packed = synth.q8_0_matrix(41, rows, cols)
    table = dev.upload_weight(Weight(packed, 8, rows, cols))
    ids = np.array([0, 299, 17, 17, 123], dtype=np.int32)
    out = torch.empty((len(ids), cols), device="cuda")
    dev.embedding_rows_resident(table, cuda(ids), out)
    dev.check_status()
    full = oracle.dequantize(packed, 8, rows, cols).reshape(rows, cols)
    assert np.array_equal(bits(out.cpu().numpy()), bits(full[ids]))
    dev.embedding_rows_resident(table, cuda(np.array([300], dtype=np.int32)), out[:1])
    with pytest.raises(DeviceError):
        dev.check_status()
    table.free()
    # BF16 weights (ggml type 30): the formats Cpu::supports accepts, crates/beholdd-backend/src/cpu.rs:1357-1366
    assert dev.supports(30)
    r, c, b = 96, 1024, 3
    f = synth.normal(42, 5, r * c).astype(np.float32)
    bf = (f.view(np.uint32) >> 16).astype(np.uint16)          # truncation is a valid BF16 encoding of some value
    packed = bf.view(np.uint8)
    deq = np.zeros(r * c, dtype=np.float32)
    dev.dequantize(deq, Weight(packed, 30, r, c))
    assert np.array_equal(bits(deq), (bf.astype(np.uint32) << 16))
    x = synth.activations(43, (b, c))
    w = dev.upload_weight(Weight(packed, 30, r, c))
    y = torch.empty((b, r), device="cuda")
    dev.matvec_resident(w, cuda(x), y)
    want = (deq.reshape(r, c).astype(np.float64) @ x.astype(np.float64).T).T
    assert max_rel_err(y.cpu().numpy(), want) <= 1e-5
    w.free()


def test_one_qwen3moe_layer_composed_from_the_operators(dev, oracle):
    """RMSNorm -> q/k/v projections (Q8_0) -> per-head QK-norm -> split-half rope -> incremental attention over an f32
    cache -> output projection -> residual -> RMSNorm -> routed experts with residual, as
    crates/beholdd-model/src/qwen3moe/forward.rs:1022-1414 orders them; the same layer composed from the oracle's
    operators is the reference. Two calls: a 6-position prefill, then one decode position against the cache."""
    import torch
    from exec_beholdd_b200 import Weight, synth

    dim, n_heads, n_kv, hd, ne, ff, k, eps, theta = 512, 4, 2, 128, 8, 256, 2, 1e-6, 1.0e6
    seed = 77
    wq, wk, wv = synth.q8_0_matrix(seed, n_heads * hd, dim, 31), synth.q8_0_matrix(seed, n_kv * hd, dim, 32), synth.q8_0_matrix(seed, n_kv * hd, dim, 33)
    wo = synth.q8_0_matrix(seed, dim, n_heads * hd, 34)
    attn_norm = synth.normal(seed, 41, dim) * np.float32(0.1) + np.float32(1.0)
    ffn_norm = synth.normal(seed, 42, dim) * np.float32(0.1) + np.float32(1.0)
    q_norm = synth.normal(seed, 43, hd) * np.float32(0.1) + np.float32(1.0)
    k_norm = synth.normal(seed, 44, hd) * np.float32(0.1) + np.float32(1.0)
    router = synth.router_weights(seed, ne, dim)
    gate, up, down = synth.expert_slabs(seed, ne, ff, dim, 21), synth.expert_slabs(seed, ne, ff, dim, 22), synth.expert_slabs(seed, ne, dim, ff, 23)
    scale = float(1.0 / np.sqrt(np.float32(hd)))
    up_w = lambda b, kind, r, c, slabs=1: dev.upload_weight(Weight(b, kind, r, c), slabs=slabs)
    Wq, Wk, Wv, Wo = up_w(wq, 8, n_heads * hd, dim), up_w(wk, 8, n_kv * hd, dim), up_w(wv, 8, n_kv * hd, dim), up_w(wo, 8, dim, n_heads * hd)
    R = up_w(router.view(np.uint8).reshape(-1), 0, ne, dim)
    G, U, D = up_w(gate, 8, ff, dim, ne), up_w(up, 8, ff, dim, ne), up_w(down, 8, dim, ff, ne)
    max_pos = 7
    k_cache_o, v_cache_o = np.zeros((max_pos, n_kv, hd), np.float32), np.zeros((max_pos, n_kv, hd), np.float32)
    k_cache_d, v_cache_d = torch.zeros((max_pos, n_kv, hd), device="cuda"), torch.zeros((max_pos, n_kv, hd), device="cuda")

    def oracle_layer(h, start):
        T = h.shape[0]
        x = np.stack([oracle.rmsnorm(h[t], attn_norm, eps) for t in range(T)])
        q = oracle.matvec_batch(wq, 8, n_heads * hd, dim, x).reshape(T, n_heads, hd)
        kk = oracle.matvec_batch(wk, 8, n_kv * hd, dim, x).reshape(T, n_kv, hd)
        vv = oracle.matvec_batch(wv, 8, n_kv * hd, dim, x).reshape(T, n_kv, hd)
        for t in range(T):
            cos, sin = oracle.rope_table(theta, hd, start + t)
            for hh in range(n_heads):
                q[t, hh] = oracle.rope(oracle.rmsnorm(q[t, hh], q_norm, eps), cos, sin, split_half=True)
            for hh in range(n_kv):
                kk[t, hh] = oracle.rope(oracle.rmsnorm(kk[t, hh], k_norm, eps), cos, sin, split_half=True)
        k_cache_o[start:start + T], v_cache_o[start:start + T] = kk, vv
        att = oracle.incremental_attention(q, k_cache_o[:start + T], v_cache_o[:start + T], T, start, start + T, n_heads, n_kv, hd, scale)
        h = h + oracle.matvec_batch(wo, 8, dim, n_heads * hd, att.reshape(T, n_heads * hd))
        x2 = np.stack([oracle.rmsnorm(h[t], ffn_norm, eps) for t in range(T)])
        y, experts, _, _ = oracle.moe_layer(router, gate, up, down, ff, x2, k)
        return h + y, experts

    def device_layer(h, start):
        T = h.shape[0]
        hd_ = cuda(h)
        x = torch.empty_like(hd_)
        dev.rmsnorm_resident(x, hd_, cuda(attn_norm), eps)
        q = torch.empty((T, n_heads, hd), device="cuda")
        kk = torch.empty((T, n_kv, hd), device="cuda")
        vv = torch.empty((T, n_kv, hd), device="cuda")
        proj = dev.matvec_resident if T <= 8 else dev.matmul_resident
        proj(Wq, x, q.view(T, -1)); proj(Wk, x, kk.view(T, -1)); proj(Wv, x, vv.view(T, -1))
        dev.rmsnorm_resident(q, q, cuda(q_norm), eps)
        dev.rmsnorm_resident(kk, kk, cuda(k_norm), eps)
        tables = [oracle.rope_table(theta, hd, start + t) for t in range(T)]  # the host computes the tables (f64), as in the reference
        cos, sin = cuda(np.stack([t[0] for t in tables])), cuda(np.stack([t[1] for t in tables]))
        dev.rope_resident(q, cos, sin, split_half=True)
        dev.rope_resident(kk, cos, sin, split_half=True)
        k_cache_d[start:start + T].copy_(kk)
        v_cache_d[start:start + T].copy_(vv)
        att = torch.empty((T, n_heads, hd), device="cuda")
        dev.attention_resident(att, q, k_cache_d, v_cache_d, start, start + T, scale)
        o = torch.empty((T, dim), device="cuda")
        proj(Wo, att.view(T, -1), o)
        dev.lib.bhd_add_in_place(dev.ctx, C.c_void_p(hd_.data_ptr()), C.c_void_p(o.data_ptr()), hd_.numel(), dev._stream())
        x2 = torch.empty_like(hd_)
        dev.rmsnorm_resident(x2, hd_, cuda(ffn_norm), eps)
        e = torch.empty((T, k), dtype=torch.int32, device="cuda")
        w = torch.empty((T, k), device="cuda")
        dev.moe_layer(R, G, U, D, x2, hd_, k, e, w, None, accumulate=True)
        dev.check_status()
        return hd_.cpu().numpy(), e.cpu().numpy()

    h0 = synth.activations(seed + 1, (6, dim))
    want, experts_o = oracle_layer(h0.copy(), 0)
    got, experts_d = device_layer(h0.copy(), 0)
    assert np.array_equal(experts_d, experts_o)
    assert max_rel_err(got, want) <= TOL
    h1 = synth.activations(seed + 2, (1, dim))
    want1, experts_o1 = oracle_layer(h1.copy(), 6)
    got1, experts_d1 = device_layer(h1.copy(), 6)
    assert np.array_equal(experts_d1, experts_o1)
    assert max_rel_err(got1, want1) <= TOL
    for hdl in (Wq, Wk, Wv, Wo, R, G, U, D):
        hdl.free()


def test_device_weight_generator_reproduces_the_host_generator(dev):
    """The benchmark's 48-layer model is generated on the device; its Q8_0 blocks must be the host generator's."""
    import torch
    from exec_beholdd_b200 import synth

    rows, cols, slabs, seed = 96, 512, 3, 1234
    t = torch.empty(slabs * rows * (cols // 32) * 34, dtype=torch.uint8, device="cuda")
    st = dev.lib.bhd_debug_fill_q8_0(dev.ctx, t.data_ptr(), rows * (cols // 32), slabs, seed, 21000 + 5, 1, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, dev._message()
    want = np.concatenate([synth.q8_0_matrix(seed, rows, cols, stream=21000 + 5 + s) for s in range(slabs)])
    assert np.array_equal(t.cpu().numpy(), want)
    n = 1 << 20
    f = torch.empty(n, device="cuda")
    assert dev.lib.bhd_debug_fill_normal(dev.ctx, f.data_ptr(), n, seed, 5, 0.02, C.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    fn = f.cpu().numpy()
    assert abs(float(fn.mean())) < 2e-4 and abs(float(fn.std()) - 0.02) < 2e-4


def small_model(synth, Qwen3MoeConfig):
    """A 2-layer qwen3moe-architecture model with seeded host weights."""
    cfg = Qwen3MoeConfig(n_layers=2, dim=512, n_heads=4, n_kv_heads=2, head_dim=128, n_experts=8, top_k=2, expert_ff=256, vocab=300,
                         rope_theta=1.0e6, eps=1e-6, context=16)
    seed, qw, kvw = 99, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    norm = lambda st, n: synth.normal(seed, st, n) * np.float32(0.1) + np.float32(1.0)
    host = {"token_embd": synth.normal(seed, 5, cfg.vocab * cfg.dim, std=0.02).reshape(cfg.vocab, cfg.dim), "out_norm": norm(6, cfg.dim),
            "lm_head": synth.q8_0_matrix(seed, cfg.vocab, cfg.dim, 7), "layers": []}
    for l in range(cfg.n_layers):
        b = 100 * (l + 1)
        host["layers"].append({"attn_norm": norm(b + 1, cfg.dim), "q_norm": norm(b + 2, cfg.head_dim), "k_norm": norm(b + 3, cfg.head_dim),
                               "ffn_norm": norm(b + 4, cfg.dim), "wq": synth.q8_0_matrix(seed, qw, cfg.dim, b + 31),
                               "wk": synth.q8_0_matrix(seed, kvw, cfg.dim, b + 32), "wv": synth.q8_0_matrix(seed, kvw, cfg.dim, b + 33),
                               "wo": synth.q8_0_matrix(seed, cfg.dim, qw, b + 34), "router": synth.router_weights(seed + l, cfg.n_experts, cfg.dim),
                               "gate": synth.expert_slabs(seed + l, cfg.n_experts, cfg.expert_ff, cfg.dim, 21),
                               "up": synth.expert_slabs(seed + l, cfg.n_experts, cfg.expert_ff, cfg.dim, 22),
                               "down": synth.expert_slabs(seed + l, cfg.n_experts, cfg.dim, cfg.expert_ff, 23)})
    return cfg, host


def test_small_model_forward_matches_the_oracle_composition(dev, oracle):
    """A 2-layer qwen3moe-architecture model, teacher-forced: a 5-token prefill and two decode steps against the same
    model composed from the oracle's operators (crates/beholdd-model/src/qwen3moe/forward.rs:954-972, 1022-1455).
    Expert indices of every layer exact, logits within tolerance."""
    import torch
    from exec_beholdd_b200 import synth
    from exec_beholdd_b200.qwen3moe import Qwen3MoeConfig, Qwen3MoeModel

    cfg, host = small_model(synth, Qwen3MoeConfig)
    qw, kvw = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    model = Qwen3MoeModel.from_host(dev, cfg, host)
    scale = float(1.0 / np.sqrt(np.float32(cfg.head_dim)))
    kc = [np.zeros((cfg.context, cfg.n_kv_heads, cfg.head_dim), np.float32) for _ in range(cfg.n_layers)]
    vc = [np.zeros((cfg.context, cfg.n_kv_heads, cfg.head_dim), np.float32) for _ in range(cfg.n_layers)]

    def oracle_forward(ids, start):
        T = len(ids)
        h = host["token_embd"][ids].astype(np.float32).copy()
        picked = []
        for l, L in enumerate(host["layers"]):
            x = np.stack([oracle.rmsnorm(h[t], L["attn_norm"], cfg.eps) for t in range(T)])
            q = oracle.matvec_batch(L["wq"], 8, qw, cfg.dim, x).reshape(T, cfg.n_heads, cfg.head_dim)
            k = oracle.matvec_batch(L["wk"], 8, kvw, cfg.dim, x).reshape(T, cfg.n_kv_heads, cfg.head_dim)
            v = oracle.matvec_batch(L["wv"], 8, kvw, cfg.dim, x).reshape(T, cfg.n_kv_heads, cfg.head_dim)
            for t in range(T):
                cos, sin = oracle.rope_table(cfg.rope_theta, cfg.head_dim, start + t)
                for hh in range(cfg.n_heads):
                    q[t, hh] = oracle.rope(oracle.rmsnorm(q[t, hh], L["q_norm"], cfg.eps), cos, sin, split_half=True)
                for hh in range(cfg.n_kv_heads):
                    k[t, hh] = oracle.rope(oracle.rmsnorm(k[t, hh], L["k_norm"], cfg.eps), cos, sin, split_half=True)
            kc[l][start:start + T], vc[l][start:start + T] = k, v
            att = oracle.incremental_attention(q, kc[l][:start + T], vc[l][:start + T], T, start, start + T, cfg.n_heads, cfg.n_kv_heads,
                                               cfg.head_dim, scale)
            h = h + oracle.matvec_batch(L["wo"], 8, cfg.dim, qw, att.reshape(T, qw))
            x2 = np.stack([oracle.rmsnorm(h[t], L["ffn_norm"], cfg.eps) for t in range(T)])
            y, experts, _, _ = oracle.moe_layer(L["router"], L["gate"], L["up"], L["down"], cfg.expert_ff, x2, cfg.top_k)
            picked.append(experts)
            h = h + y
        xn = np.stack([oracle.rmsnorm(h[t], host["out_norm"], cfg.eps) for t in range(T)])
        return oracle.matvec_batch(host["lm_head"], 8, cfg.vocab, cfg.dim, xn), picked

    ids = np.array([3, 250, 17, 299, 42, 7, 123], dtype=np.int32)
    for lo, hi in ((0, 5), (5, 6), (6, 7)):                      # teacher-forced: prefill, then two single positions
        want, picked = oracle_forward(ids[lo:hi], lo)
        h = torch.empty((hi - lo, cfg.dim), device="cuda")
        dev.embedding_rows_resident(model.w["token_embd"], cuda(ids[lo:hi]), h)
        for l in range(cfg.n_layers):
            experts, _ = model.layer_forward(l, h, lo)
            assert np.array_equal(experts.cpu().numpy(), picked[l]), (lo, l)
        model.n_cached = lo
        got = model.forward(cuda(ids[lo:hi]), start=lo, all_logits=True)
        dev.check_status()
        assert max_rel_err(got.cpu().numpy(), want) <= TOL, (lo, hi)
        assert int(torch.argmax(got[-1])) == int(np.argmax(want[-1]))
    # Greedy decoding: the decode step replayed as one CUDA graph (position and token read from device memory)
    # gives the tokens and the last logits of the step-by-step loop, to the bit; a second call reuses the graph.
    eager = model.generate_greedy(cuda(ids[:5]), 6, use_graph=False)
    eager_logits = model.forward(eager[5:6]).clone()
    graph = model.generate_greedy(cuda(ids[:5]), 6, use_graph=True)
    graph_logits = model.forward(graph[5:6]).clone()
    dev.check_status()
    assert graph.shape[0] == 6 and int(graph.min()) >= 0 and int(graph.max()) < cfg.vocab
    assert np.array_equal(graph.cpu().numpy(), eager.cpu().numpy())
    assert np.array_equal(bits(graph_logits.cpu().numpy()), bits(eager_logits.cpu().numpy()))
    again = model.generate_greedy(cuda(ids[:5]), 4, use_graph=True)
    assert np.array_equal(again.cpu().numpy(), eager.cpu().numpy()[:4])
    # A larger workspace replaces the one the captured kernels point into: the step must be captured again, not replayed.
    captured = model._dec["graph"]
    assert dev.lib.bhd_workspace_reserve(dev.ctx, dev.workspace_bytes() + (64 << 20)) == 0
    regrown = model.generate_greedy(cuda(ids[:5]), 6, use_graph=True)
    dev.check_status()
    assert model._dec["graph"] is not captured
    assert np.array_equal(regrown.cpu().numpy(), eager.cpu().numpy())
    model.free()


def test_model_read_from_a_gguf_file_equals_the_model_given_as_arrays(dev, tmp_path):
    """GGUF ingestion end to end: the small model written as a GGUF checkpoint (llama.cpp's qwen3moe tensor names,
    3-D expert tensors), read back through the memory-mapped reader into HBM, gives the bits of the model uploaded
    from the arrays themselves."""
    import os
    import sys

    import torch
    from exec_beholdd_b200 import synth
    from exec_beholdd_b200.gguf import GgufFile
    from exec_beholdd_b200.qwen3moe import Qwen3MoeConfig, Qwen3MoeModel

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    import make_moe_block_golden as g

    cfg, host = small_model(synth, Qwen3MoeConfig)
    A = "qwen3moe"
    meta = [("general.architecture", 8, A), (f"{A}.block_count", 4, cfg.n_layers), (f"{A}.embedding_length", 4, cfg.dim),
            (f"{A}.attention.head_count", 4, cfg.n_heads), (f"{A}.attention.head_count_kv", 4, cfg.n_kv_heads),
            (f"{A}.attention.key_length", 4, cfg.head_dim), (f"{A}.expert_count", 4, cfg.n_experts), (f"{A}.expert_used_count", 4, cfg.top_k),
            (f"{A}.expert_feed_forward_length", 4, cfg.expert_ff), (f"{A}.attention.layer_norm_rms_epsilon", 6, cfg.eps),
            (f"{A}.rope.freq_base", 6, cfg.rope_theta)]
    f32b = lambda a: np.ascontiguousarray(a, dtype="<f4").tobytes()
    qw, kvw = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    tensors = [("token_embd.weight", 0, [cfg.dim, cfg.vocab], f32b(host["token_embd"])), ("output_norm.weight", 0, [cfg.dim], f32b(host["out_norm"])),
               ("output.weight", 8, [cfg.dim, cfg.vocab], host["lm_head"].tobytes())]
    for i, L in enumerate(host["layers"]):
        P = f"blk.{i}."
        tensors += [(P + "attn_norm.weight", 0, [cfg.dim], f32b(L["attn_norm"])), (P + "attn_q_norm.weight", 0, [cfg.head_dim], f32b(L["q_norm"])),
                    (P + "attn_k_norm.weight", 0, [cfg.head_dim], f32b(L["k_norm"])), (P + "ffn_norm.weight", 0, [cfg.dim], f32b(L["ffn_norm"])),
                    (P + "attn_q.weight", 8, [cfg.dim, qw], L["wq"].tobytes()), (P + "attn_k.weight", 8, [cfg.dim, kvw], L["wk"].tobytes()),
                    (P + "attn_v.weight", 8, [cfg.dim, kvw], L["wv"].tobytes()), (P + "attn_output.weight", 8, [qw, cfg.dim], L["wo"].tobytes()),
                    (P + "ffn_gate_inp.weight", 0, [cfg.dim, cfg.n_experts], f32b(L["router"])),
                    (P + "ffn_gate_exps.weight", 8, [cfg.dim, cfg.expert_ff, cfg.n_experts], L["gate"].tobytes()),
                    (P + "ffn_up_exps.weight", 8, [cfg.dim, cfg.expert_ff, cfg.n_experts], L["up"].tobytes()),
                    (P + "ffn_down_exps.weight", 8, [cfg.expert_ff, cfg.dim, cfg.n_experts], L["down"].tobytes())]
    path = str(tmp_path / "small.gguf")
    g.write_gguf(path, meta, tensors)
    ids = cuda(np.array([3, 250, 17, 299, 42], dtype=np.int32))
    a = Qwen3MoeModel.from_host(dev, cfg, host)
    want = a.forward(ids, start=0, all_logits=True).clone()
    a.free()
    with GgufFile(path) as f:
        b = Qwen3MoeModel.from_gguf(dev, f, context=cfg.context)
        import dataclasses

        assert dataclasses.replace(b.cfg, eps=cfg.eps) == cfg and abs(b.cfg.eps - cfg.eps) < 1e-12   # eps travels as an f32
        got = b.forward(ids, start=0, all_logits=True)
        dev.check_status()
        assert torch.equal(got, want)
        b.free()
