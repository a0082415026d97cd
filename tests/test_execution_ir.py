"""The recorded-execution mirror: command lists validate shapes and ownership on the host
(crates/beholdd-backend/src/execution.rs:547-880, tests :1177-1507 for the rules checked here);
on a GPU, a recorded decode layer equals the oracle's composition and replays identically."""
import numpy as np
import pytest


def fake_weight(ex, owner, kind, rows, cols, slabs=1):
    from exec_beholdd_b200.device import ResidentWeight

    return ex.PreparedWeight(owner, ResidentWeight(None, 0, kind, rows, cols, slabs, 0))


def host_tensor(ex, owner, n):
    import torch

    return ex.F32Tensor(owner, torch.zeros(n))


def test_command_list_checks_shapes_as_commands_are_added():
    from exec_beholdd_b200 import execution as ex

    w = fake_weight(ex, 1, 8, 6, 32)
    x, y = host_tensor(ex, 1, 32), host_tensor(ex, 1, 6)
    cl = ex.CommandList()
    cl.linear(y.full_view(), x.full_view(), w)
    cl.linear(y.full_view(), x.full_view(), w, ex.LinearMode.scaled_add(0.5))
    assert len(cl) == 2
    with pytest.raises(ex.ShapeMismatch):
        cl.linear(y.view(0, 5), x.full_view(), w)
    with pytest.raises(ex.ShapeMismatch):
        cl.linear(y.full_view(), x.full_view(), w, ex.LinearMode.scaled_add(float("nan")))
    with pytest.raises(ex.ShapeMismatch):
        cl.embedding_row(x.full_view(), w, 6)
    cl.embedding_row(x.full_view(), w, 5)
    with pytest.raises(ex.ShapeMismatch):
        cl.swiglu(x.view(0, 4), x.view(4, 5))
    with pytest.raises(ex.ShapeMismatch):
        cl.swiglu(x.view(0, 4), x.view(4, 4), limit=-1.0)
    with pytest.raises(ex.ShapeMismatch):
        cl.rmsnorm(x.view(0, 8), x.view(8, 8), x.view(16, 4), 1e-6)
    with pytest.raises(ex.ShapeMismatch):
        cl.rmsnorm(x.view(0, 8), x.view(8, 8), None, -1.0)
    with pytest.raises(ex.ShapeMismatch):
        cl.rope(x.view(0, 8), x.view(8, 4), x.view(12, 3), True)
    cl.rope(x.view(0, 8), x.view(8, 4), x.view(12, 4), True)
    with pytest.raises(ex.ShapeMismatch):
        cl.sigmoid_gate(x.view(0, 8), x.view(8, 8), x.view(16, 7))
    cfg = ex.IncrementalAttentionConfig(1, 0, 2, 2, 1, 4, 0.5)
    with pytest.raises(ex.ShapeMismatch):
        cl.incremental_causal_attention(x.view(0, 8), x.view(8, 8), x.view(16, 8), x.view(24, 4), cfg)
    with pytest.raises(ex.ShapeMismatch):
        x.view(30, 3)
    with pytest.raises(ex.ShapeMismatch):
        x.view(0, 8).view(4, 5)
    assert len(cl) == 4


def test_command_list_holds_one_owner():
    from exec_beholdd_b200 import execution as ex

    w1, w2 = fake_weight(ex, 1, 8, 6, 32), fake_weight(ex, 2, 8, 6, 32)
    x1, y1, y2 = host_tensor(ex, 1, 32), host_tensor(ex, 1, 6), host_tensor(ex, 2, 6)
    cl = ex.CommandList()
    cl.linear(y1.full_view(), x1.full_view(), w1)
    with pytest.raises(ex.ForeignResource):
        cl.linear(y1.full_view(), x1.full_view(), w2)
    with pytest.raises(ex.ForeignResource):
        cl.linear(y2.full_view(), x1.full_view(), w1)
    assert len(cl) == 1 and cl.owner == 1


def test_views_know_when_they_overlap():
    from exec_beholdd_b200 import execution as ex

    t, u = host_tensor(ex, 1, 16), host_tensor(ex, 1, 16)
    assert t.view(0, 8).overlaps(t.view(7, 4)) and not t.view(0, 8).overlaps(t.view(8, 8))
    assert not t.view(0, 8).overlaps(u.view(0, 8)) and not t.view(4, 0).overlaps(t.view(0, 8))
    assert t.view(2, 4).same(t.view(0, 8).view(2, 4))


@pytest.mark.gpu
def test_recorded_decode_layer_matches_the_oracle_and_replays(oracle):
    """One qwen3moe decode layer as a command list (embedding row, RMSNorm, q/k/v projections, per-head QK-norm, rope,
    attention over the cache, output projection as ScaledAdd, RMSNorm, routed experts accumulated onto the residual),
    recorded once per position and submitted; the oracle's composition of the same operators is the reference."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from exec_beholdd_b200 import Weight, synth
    from exec_beholdd_b200 import execution as ex

    dim, n_heads, n_kv, hd, ne, ff, k, eps, theta, vocab = 512, 4, 2, 128, 8, 256, 2, 1e-6, 1.0e6, 40
    seed, qw, kvw = 55, 4 * 128, 2 * 128
    emb = synth.normal(seed, 5, vocab * dim, std=0.5).reshape(vocab, dim)
    wq, wk, wv, wo = (synth.q8_0_matrix(seed, qw, dim, 31), synth.q8_0_matrix(seed, kvw, dim, 32), synth.q8_0_matrix(seed, kvw, dim, 33),
                      synth.q8_0_matrix(seed, dim, qw, 34))
    norms = {n: synth.normal(seed, 41 + i, m) * np.float32(0.1) + np.float32(1.0) for i, (n, m) in
             enumerate([("attn", dim), ("ffn", dim), ("q", hd), ("k", hd)])}
    router = synth.router_weights(seed, ne, dim)
    gate, up, down = synth.expert_slabs(seed, ne, ff, dim, 21), synth.expert_slabs(seed, ne, ff, dim, 22), synth.expert_slabs(seed, ne, dim, ff, 23)
    scale = float(1.0 / np.sqrt(np.float32(hd)))

    d = ex.CudaExecutionDevice(0)
    prep = lambda b, kind, r, c, slabs=1: d.prepare_weight(d.upload_weight(Weight(b, kind, r, c), slabs))
    E = prep(emb.view(np.uint8).reshape(-1), 0, vocab, dim)
    Wq, Wk, Wv, Wo = prep(wq, 8, qw, dim), prep(wk, 8, kvw, dim), prep(wv, 8, kvw, dim), prep(wo, 8, dim, qw)
    R = prep(router.view(np.uint8).reshape(-1), 0, ne, dim)
    G, U, D = prep(gate, 8, ff, dim, ne), prep(up, 8, ff, dim, ne), prep(down, 8, dim, ff, ne)
    N = {n: d.upload_f32(v) for n, v in norms.items()}
    max_pos = 4
    h, x, q, kk, att = d.allocate_f32(dim), d.allocate_f32(dim), d.allocate_f32(qw), d.allocate_f32(kvw), d.allocate_f32(qw)
    kc, vc = d.allocate_f32(max_pos * kvw), d.allocate_f32(max_pos * kvw)
    tables = d.allocate_f32(hd)
    kc_o, vc_o = np.zeros((max_pos, n_kv, hd), np.float32), np.zeros((max_pos, n_kv, hd), np.float32)

    def oracle_step(tok, pos):
        hh = emb[tok].copy()
        xx = oracle.rmsnorm(hh, norms["attn"], eps)
        qq = oracle.matvec(wq, 8, qw, dim, xx).reshape(n_heads, hd)
        k1 = oracle.matvec(wk, 8, kvw, dim, xx).reshape(n_kv, hd)
        v1 = oracle.matvec(wv, 8, kvw, dim, xx).reshape(n_kv, hd)
        cos, sin = oracle.rope_table(theta, hd, pos)
        for i in range(n_heads):
            qq[i] = oracle.rope(oracle.rmsnorm(qq[i], norms["q"], eps), cos, sin, split_half=True)
        for i in range(n_kv):
            k1[i] = oracle.rope(oracle.rmsnorm(k1[i], norms["k"], eps), cos, sin, split_half=True)
        kc_o[pos], vc_o[pos] = k1, v1
        a = oracle.incremental_attention(qq[None], kc_o[:pos + 1], vc_o[:pos + 1], 1, pos, pos + 1, n_heads, n_kv, hd, scale)
        hh = hh + np.float32(0.5) * oracle.matvec(wo, 8, dim, qw, a.reshape(-1))
        x2 = oracle.rmsnorm(hh, norms["ffn"], eps)
        y, experts, _, _ = oracle.moe_layer(router, gate, up, down, ff, x2[None], k)
        return hh + y[0]

    def record_step(tok, pos):
        cl = ex.CommandList()
        cl.embedding_row(h.full_view(), E, tok)
        cl.rmsnorm(x.full_view(), h.full_view(), N["attn"].full_view(), eps)
        cl.linear(q.full_view(), x.full_view(), Wq)
        cl.linear(kc.view(pos * kvw, kvw), x.full_view(), Wk)
        cl.linear(vc.view(pos * kvw, kvw), x.full_view(), Wv)
        cos, sin = tables.view(0, hd // 2), tables.view(hd // 2, hd // 2)
        for i in range(n_heads):
            cl.rmsnorm(q.view(i * hd, hd), q.view(i * hd, hd), N["q"].full_view(), eps)
            cl.rope(q.view(i * hd, hd), cos, sin, True)
        for i in range(n_kv):
            cl.rmsnorm(kc.view(pos * kvw + i * hd, hd), kc.view(pos * kvw + i * hd, hd), N["k"].full_view(), eps)
            cl.rope(kc.view(pos * kvw + i * hd, hd), cos, sin, True)
        cl.incremental_causal_attention(att.full_view(), q.full_view(), kc.view(0, (pos + 1) * kvw), vc.view(0, (pos + 1) * kvw),
                                        ex.IncrementalAttentionConfig(1, pos, pos + 1, n_heads, n_kv, hd, scale))
        cl.linear(h.full_view(), att.full_view(), Wo, ex.LinearMode.scaled_add(0.5))
        cl.rmsnorm(x.full_view(), h.full_view(), N["ffn"].full_view(), eps)
        cl.routed_moe(h.full_view(), x.full_view(), R, G, U, D, k, accumulate=True)
        return d.record(cl)

    got = np.empty(dim, np.float32)
    for pos, tok in enumerate([7, 31, 2]):
        cos, sin = oracle.rope_table(theta, hd, pos)
        d.write_f32(tables.full_view(), np.concatenate([cos, sin]))
        batch = record_step(tok, pos)
        assert len(batch) == 21
        d.wait(d.submit(batch))
        d.read_f32(h.full_view(), got)
        want = oracle_step(tok, pos)
        rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
        err = float((np.abs(got - want) / np.maximum(np.abs(want), rms)).max())
        assert err <= 2e-3, (pos, err)
        first = got.copy()
        d.wait(d.submit(batch))                       # every command overwrites or starts from the embedding row: a replay repeats it
        d.read_f32(h.full_view(), got)
        assert np.array_equal(got.view(np.uint32), first.view(np.uint32))

    # Aliasing the backend cannot honour is refused at record, and foreign resources before anything is interpreted.
    cl = ex.CommandList()
    cl.rmsnorm(h.view(0, 64), h.view(32, 64), None, eps)
    with pytest.raises(ex.IncompatibleResource):
        d.record(cl)
    cl = ex.CommandList()
    cl.linear(h.full_view(), h.full_view(), Wo)
    with pytest.raises(ex.IncompatibleResource):
        d.record(cl)
    # A batch recorded before the device's workspace was replaced by a larger one points into freed memory: refused.
    assert d.dev.lib.bhd_workspace_reserve(d.dev.ctx, d.dev.workspace_bytes() + (64 << 20)) == 0
    with pytest.raises(ex.IncompatibleResource):
        d.submit(batch)
    d.wait(d.submit(record_step(2, 2)))
    other = ex.CudaExecutionDevice(0)
    with pytest.raises(ex.ForeignResource):
        other.record(_list_of(ex, h, x, N, eps))
    with pytest.raises(ex.ForeignResource):
        other.submit(batch)
    with pytest.raises(ex.ForeignResource):
        other.prepare_weight(d.upload_weight(Weight(wq, 8, qw, dim)))
    with pytest.raises(ex.ShapeMismatch):
        d.write_f32(h.view(0, 8), np.zeros(9, np.float32))
    other.close()
    d.close()


def _list_of(ex, h, x, N, eps):
    cl = ex.CommandList()
    cl.rmsnorm(x.full_view(), h.full_view(), N["attn"].full_view(), eps)
    return cl
