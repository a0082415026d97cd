"""GGUF ingestion on the CPU side: header, metadata, tensor table, slabs, refusals. The writer is the one that
produced the golden fixtures (tests/golden/make_moe_block_golden.py); reading what it wrote back byte for byte,
and reading the hyper-parameters the forward pass needs, pins the reader to the same format the reference's own
NumPy implementation parsed when the fixtures were made."""
import os
import struct
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))


def _write_case(tmp_path):
    import make_moe_block_golden as g
    from exec_beholdd_b200 import synth

    dim, ne, ff, vocab = 64, 4, 32, 96
    A = "qwen3moe"
    meta = [("general.architecture", 8, A), (f"{A}.embedding_length", 4, dim), (f"{A}.attention.head_count", 4, 4),
            (f"{A}.attention.head_count_kv", 4, 2), (f"{A}.attention.key_length", 4, 16), (f"{A}.expert_count", 4, ne),
            (f"{A}.expert_used_count", 4, 2), (f"{A}.attention.layer_norm_rms_epsilon", 6, 1e-6), (f"{A}.rope.freq_base", 6, 1.0e6)]
    gate = synth.expert_slabs(3, ne, ff, dim, stream=21)
    router = synth.router_weights(3, ne, dim)
    embd = synth.q8_0_matrix(3, vocab, dim, stream=24)
    norm = np.linspace(0.5, 1.5, dim, dtype=np.float32)
    tensors = [("token_embd.weight", 8, [dim, vocab], embd.tobytes()), ("blk.0.attn_norm.weight", 0, [dim], norm.tobytes()),
               ("blk.0.ffn_gate_inp.weight", 0, [dim, ne], router.astype("<f4").tobytes()),
               ("blk.0.ffn_gate_exps.weight", 8, [dim, ff, ne], gate.tobytes()),
               ("blk.0.odd.weight", 2, [32, 2], bytes(2 * 18))]  # a kind the library does not decode (Q4_0)
    path = str(tmp_path / "case.gguf")
    g.write_gguf(path, meta, tensors)
    return path, dict(dim=dim, ne=ne, ff=ff, vocab=vocab, gate=gate, router=router, embd=embd, norm=norm)


def test_reader_returns_what_the_writer_wrote(tmp_path):
    from exec_beholdd_b200.gguf import GgufError, GgufFile

    path, c = _write_case(tmp_path)
    with GgufFile(path) as f:
        assert f.meta["general.architecture"] == "qwen3moe" and f.meta["qwen3moe.expert_count"] == c["ne"]
        assert abs(f.meta["qwen3moe.rope.freq_base"] - 1.0e6) < 1.0
        t = f.tensors["blk.0.ffn_gate_exps.weight"]
        assert t.kind == 8 and t.dims == (c["dim"], c["ff"], c["ne"]) and t.offset % 32 == 0
        assert np.array_equal(f.tensor_bytes("blk.0.ffn_gate_exps.weight"), c["gate"])
        per = c["gate"].size // c["ne"]
        assert np.array_equal(f.tensor_bytes("blk.0.ffn_gate_exps.weight", 1, 2), c["gate"][per:3 * per])   # one rank's experts
        assert np.array_equal(f.tensor_bytes("token_embd.weight"), c["embd"])
        assert np.array_equal(f.f32("blk.0.ffn_gate_inp.weight"), c["router"]) and f.f32("blk.0.ffn_gate_inp.weight").shape == (c["ne"], c["dim"])
        assert np.array_equal(f.f32("blk.0.attn_norm.weight"), c["norm"])
        cfg = f.qwen3moe_config(context=128)
        assert (cfg.n_layers, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.n_experts, cfg.top_k, cfg.expert_ff, cfg.vocab) == \
               (1, c["dim"], 4, 2, 16, c["ne"], 2, c["ff"], c["vocab"])
        with pytest.raises(GgufError):
            f.tensor_bytes("blk.0.odd.weight")          # listed, but of a kind without a decoder
        with pytest.raises(GgufError):
            f.tensor_bytes("no.such.tensor")
        with pytest.raises(GgufError):
            f.tensor_bytes("blk.0.ffn_gate_exps.weight", 3, 2)


def test_reader_refuses_damaged_files(tmp_path):
    from exec_beholdd_b200.gguf import GgufError, GgufFile

    path, _ = _write_case(tmp_path)
    raw = open(path, "rb").read()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUX" + raw[4:])
    with pytest.raises(GgufError):
        GgufFile(str(bad))
    bad.write_bytes(raw[:4] + struct.pack("<I", 1) + raw[8:])
    with pytest.raises(GgufError):
        GgufFile(str(bad))
    bad.write_bytes(raw[:len(raw) - 4000])              # tensor data cut off
    with pytest.raises(GgufError):
        GgufFile(str(bad))
    bad.write_bytes(raw[:40])                           # header cut off
    with pytest.raises(GgufError):
        GgufFile(str(bad))
