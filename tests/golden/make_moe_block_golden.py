#!/usr/bin/env python3
"""Generate golden vectors for the routed-expert block from the reference's own f64 NumPy
implementation (tools/qwen3moe_ref.py in the reference repository).

The reference script is imported unmodified and run on a synthetic qwen3moe GGUF written
here. The checkpoint's attention output projection is all zeros, so the attention branch
adds exactly nothing and the block output is `x + moe(rmsnorm(x))`: the routed path alone,
computed by the reference's independent implementation (own GGUF reader, own Q8_0 decoder,
softmax -> stable argsort -> renormalise, f64 arithmetic).

Usage:  make_moe_block_golden.py --reference-root <checkout of the reference> [--out-dir DIR]

Writes one .npz per case next to this script. The tests read only the .npz files; the
reference checkout is needed only to regenerate them.
"""
from __future__ import annotations

import argparse
import io
import os
import struct
import sys
import tempfile
from contextlib import redirect_stdout

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from exec_beholdd_b200 import synth  # noqa: E402

CASES = {
    # name: dim, heads, kv heads, head_dim, experts, top_k, expert_ff, positions
    "moe_block_d64_e8_k4": dict(dim=64, n_heads=4, n_kv=2, hd=32, n_exp=8, topk=4, ff=64, npos=4, seed=101),
    "moe_block_d128_e16_k8": dict(dim=128, n_heads=4, n_kv=2, hd=32, n_exp=16, topk=8, ff=32, npos=6, seed=202),
}

EPS = 1e-6
ROPE_BASE = 1_000_000.0


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path: str, meta: list, tensors: list) -> None:
    """Minimal GGUF v3 writer: (key, type, value) metadata and (name, kind, dims, bytes) tensors."""
    align = 32
    head = io.BytesIO()
    head.write(b"GGUF" + struct.pack("<I", 3) + struct.pack("<Q", len(tensors)) + struct.pack("<Q", len(meta)))
    for key, typ, val in meta:
        head.write(_s(key) + struct.pack("<I", typ))
        if typ == 8:
            head.write(_s(val))
        elif typ == 4:
            head.write(struct.pack("<I", val))
        elif typ == 6:
            head.write(struct.pack("<f", val))
        else:
            raise ValueError(typ)
    offset = 0
    blobs = []
    for name, kind, dims, data in tensors:
        head.write(_s(name) + struct.pack("<I", len(dims)))
        for d in dims:
            head.write(struct.pack("<Q", d))
        head.write(struct.pack("<I", kind) + struct.pack("<Q", offset))
        pad = (-len(data)) % align
        blobs.append(bytes(data) + b"\0" * pad)
        offset += len(data) + pad
    raw = head.getvalue()
    raw += b"\0" * ((-len(raw)) % align)
    with open(path, "wb") as fh:
        fh.write(raw)
        for b in blobs:
            fh.write(b)


def build_case(cfg: dict, ref, out_path: str) -> None:
    dim, nh, nkv, hd = cfg["dim"], cfg["n_heads"], cfg["n_kv"], cfg["hd"]
    ne, k, ff, npos, seed = cfg["n_exp"], cfg["topk"], cfg["ff"], cfg["npos"], cfg["seed"]
    toks = [(i * 7919 + 13) % 100000 for i in range(npos)]  # the reference's own token choice
    vocab = (max(toks) + 32) // 32 * 32

    f32b = lambda a: np.ascontiguousarray(a, dtype="<f4").tobytes()
    ones = lambda n: f32b(np.ones(n))
    zero_q8 = lambda rows, cols: bytes(rows * (cols // 32) * 34)
    ffn_norm = (0.5 + synth.uniform01(seed, 90, dim)).astype(np.float32)
    router = (synth.router_weights(seed, ne, dim) * np.float32(40.0)).astype(np.float32)  # spread the logits
    gate = synth.expert_slabs(seed, ne, ff, dim, stream=21)
    up = synth.expert_slabs(seed, ne, ff, dim, stream=22)
    down = synth.expert_slabs(seed, ne, dim, ff, stream=23)
    embd = synth.q8_0_matrix(seed, vocab, dim, stream=24)

    A = "qwen3moe"
    meta = [
        ("general.architecture", 8, A), (f"{A}.embedding_length", 4, dim), (f"{A}.attention.head_count", 4, nh),
        (f"{A}.attention.head_count_kv", 4, nkv), (f"{A}.attention.key_length", 4, hd),
        (f"{A}.attention.value_length", 4, hd), (f"{A}.expert_count", 4, ne), (f"{A}.expert_used_count", 4, k),
        (f"{A}.expert_shared_feed_forward_length", 4, 0), (f"{A}.attention.layer_norm_rms_epsilon", 6, EPS),
        (f"{A}.rope.freq_base", 6, ROPE_BASE),
    ]
    P = "blk.0."
    tensors = [
        ("token_embd.weight", 8, [dim, vocab], embd.tobytes()),
        (P + "attn_norm.weight", 0, [dim], ones(dim)),
        (P + "attn_q.weight", 8, [dim, nh * hd], synth.q8_0_matrix(seed, nh * hd, dim, stream=31).tobytes()),
        (P + "attn_k.weight", 8, [dim, nkv * hd], synth.q8_0_matrix(seed, nkv * hd, dim, stream=32).tobytes()),
        (P + "attn_v.weight", 8, [dim, nkv * hd], synth.q8_0_matrix(seed, nkv * hd, dim, stream=33).tobytes()),
        (P + "attn_q_norm.weight", 0, [hd], ones(hd)),
        (P + "attn_k_norm.weight", 0, [hd], ones(hd)),
        # All-zero output projection: the attention branch contributes exactly 0.
        (P + "attn_output.weight", 8, [nh * hd, dim], zero_q8(dim, nh * hd)),
        (P + "ffn_norm.weight", 0, [dim], f32b(ffn_norm)),
        (P + "ffn_gate_inp.weight", 0, [dim, ne], f32b(router)),
        (P + "ffn_gate_exps.weight", 8, [dim, ff, ne], gate.tobytes()),
        (P + "ffn_up_exps.weight", 8, [dim, ff, ne], up.tobytes()),
        (P + "ffn_down_exps.weight", 8, [ff, dim, ne], down.tobytes()),
    ]
    with tempfile.TemporaryDirectory() as tmp:
        gguf, out_bin = os.path.join(tmp, "synthetic.gguf"), os.path.join(tmp, "ref.bin")
        write_gguf(gguf, meta, tensors)
        argv = sys.argv
        sys.argv = ["qwen3moe_ref.py", gguf, out_bin, str(npos)]
        try:
            with redirect_stdout(io.StringIO()):
                ref.main()
        finally:
            sys.argv = argv
        raw = open(out_bin, "rb").read()
    n, d, kk = struct.unpack("<3i", raw[:12])
    assert (n, d, kk) == (npos, dim, k)
    pos = 12
    r_toks = np.frombuffer(raw, "<i4", npos, pos); pos += 4 * npos
    r_sel = np.frombuffer(raw, "<i4", npos * k, pos).reshape(npos, k); pos += 4 * npos * k
    r_w = np.frombuffer(raw, "<f4", npos * k, pos).reshape(npos, k); pos += 4 * npos * k
    r_hidden = np.frombuffer(raw, "<f4", npos * dim, pos).reshape(npos, dim)
    assert list(r_toks) == toks
    row_bytes = dim // 32 * 34
    embd_rows = np.stack([embd[t * row_bytes:(t + 1) * row_bytes] for t in toks])
    np.savez(out_path, dim=dim, n_experts=ne, top_k=k, expert_ff=ff, eps=np.float32(EPS), tokens=np.array(toks),
             embedding_rows_q8_0=embd_rows, ffn_norm=ffn_norm, router=router, gate_exps=gate, up_exps=up,
             down_exps=down, ref_experts=r_sel, ref_weights=r_w, ref_hidden=r_hidden)
    print(f"wrote {out_path}: experts[0]={list(r_sel[0])}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", required=True, help="checkout of the reference repository")
    ap.add_argument("--out-dir", default=HERE)
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference_root, "tools"))
    sys.dont_write_bytecode = True
    import qwen3moe_ref as ref

    for name, cfg in CASES.items():
        build_case(cfg, ref, os.path.join(args.out_dir, name + ".npz"))


if __name__ == "__main__":
    main()
