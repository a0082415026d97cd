"""GGUF checkpoint ingestion: packed tensors go from the file to HBM unchanged.

Reads what the reference's loader reads (crates/beholdd-format/src/gguf.rs:191-431: GGUF v2 / v3 header,
typed key-value metadata, tensor table, data section aligned to `general.alignment`, default 32) and
hands tensors to the device in checkpoint layout: a 2-D tensor [ne0 = columns, ne1 = rows] becomes a
`ResidentWeight` of rows x cols, and a 3-D expert tensor [columns, rows, experts] becomes one weight
with `experts` slabs (crates/beholdd-model/src/qwen3moe.rs:879-910); with expert parallelism a rank
uploads only the slabs of its own experts. The file is memory-mapped, so a tensor's bytes are copied
once, from the page cache to the device.

Only what the hot path consumes is interpreted: tensor kinds this library decodes (F32, F16, BF16,
Q8_0, Q4_K, Q5_K, Q6_K) and the qwen3moe hyper-parameters. Split checkpoints (several shards) are
opened one file at a time by the caller.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass

import numpy as np

from . import synth

#: metadata value types of the GGUF specification: code -> (struct format, size)
_SCALARS = {0: ("<B", 1), 1: ("<b", 1), 2: ("<H", 2), 3: ("<h", 2), 4: ("<I", 4), 5: ("<i", 4), 6: ("<f", 4), 7: ("<?", 1),
            10: ("<Q", 8), 11: ("<q", 8), 12: ("<d", 8)}
_STRING, _ARRAY = 8, 9


class GgufError(ValueError):
    pass


@dataclass(frozen=True)
class GgufTensor:
    name: str
    kind: int          # ggml type code
    dims: tuple        # ne0 (innermost, columns) first, as stored
    offset: int        # from the start of the file
    n_bytes: int


class GgufFile:
    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        self.meta: dict = {}
        self.tensors: dict[str, GgufTensor] = {}
        self._parse()

    def close(self):
        self._map.close()
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- parsing -------------------------------------------------------------------------
    def _need(self, pos: int, n: int):
        if pos + n > len(self._map):
            raise GgufError(f"{self.path}: truncated (needs {pos + n} bytes, file has {len(self._map)})")

    def _u32(self, pos):
        self._need(pos, 4)
        return struct.unpack_from("<I", self._map, pos)[0], pos + 4

    def _u64(self, pos):
        self._need(pos, 8)
        return struct.unpack_from("<Q", self._map, pos)[0], pos + 8

    def _string(self, pos):
        n, pos = self._u64(pos)
        self._need(pos, n)
        return bytes(self._map[pos:pos + n]).decode("utf-8", errors="replace"), pos + n

    def _value(self, typ, pos):
        if typ in _SCALARS:
            fmt, size = _SCALARS[typ]
            self._need(pos, size)
            return struct.unpack_from(fmt, self._map, pos)[0], pos + size
        if typ == _STRING:
            return self._string(pos)
        if typ == _ARRAY:
            inner, pos = self._u32(pos)
            n, pos = self._u64(pos)
            if inner in _SCALARS:
                fmt, size = _SCALARS[inner]
                self._need(pos, n * size)
                arr = np.frombuffer(self._map, dtype=np.dtype(fmt[1:]).newbyteorder("<"), count=n, offset=pos)
                return arr, pos + n * size
            out = []
            for _ in range(n):
                v, pos = self._value(inner, pos)
                out.append(v)
            return out, pos
        raise GgufError(f"{self.path}: unknown metadata value type {typ}")

    def _parse(self):
        self._need(0, 24)
        if bytes(self._map[:4]) != b"GGUF":
            raise GgufError(f"{self.path}: not a GGUF file")
        version, pos = self._u32(4)
        if version not in (2, 3):
            raise GgufError(f"{self.path}: GGUF version {version} is not supported (2 or 3)")
        n_tensors, pos = self._u64(pos)
        n_meta, pos = self._u64(pos)
        for _ in range(n_meta):
            key, pos = self._string(pos)
            typ, pos = self._u32(pos)
            self.meta[key], pos = self._value(typ, pos)
        infos = []
        for _ in range(n_tensors):
            name, pos = self._string(pos)
            n_dims, pos = self._u32(pos)
            if n_dims > 4:
                raise GgufError(f"{self.path}: tensor {name} has {n_dims} dimensions")
            dims = []
            for _ in range(n_dims):
                d, pos = self._u64(pos)
                dims.append(d)
            kind, pos = self._u32(pos)
            rel, pos = self._u64(pos)
            infos.append((name, kind, tuple(dims), rel))
        align = int(self.meta.get("general.alignment", 32))
        if align <= 0 or align & (align - 1):
            raise GgufError(f"{self.path}: alignment {align} is not a power of two")
        data0 = (pos + align - 1) // align * align
        for name, kind, dims, rel in infos:
            n_elems = int(np.prod(dims, dtype=np.uint64)) if dims else 1
            geo = synth.BLOCK_GEOMETRY.get(kind)
            if geo is None:
                n_bytes = -1            # a kind this library does not decode: listed, not loadable
            else:
                elems, nbytes = geo
                if dims and dims[0] % elems:
                    raise GgufError(f"{self.path}: tensor {name} has {dims[0]} columns, not a whole number of {elems}-element blocks")
                n_bytes = n_elems // elems * nbytes
                if rel % align or data0 + rel + n_bytes > len(self._map):
                    raise GgufError(f"{self.path}: tensor {name} lies outside the file or off the alignment grid")
            if name in self.tensors:
                raise GgufError(f"{self.path}: tensor {name} appears twice")
            self.tensors[name] = GgufTensor(name, kind, dims, data0 + rel, n_bytes)

    # ---- access --------------------------------------------------------------------------
    def tensor_bytes(self, name: str, first_slab: int = 0, n_slabs: int | None = None) -> np.ndarray:
        """The packed bytes of a tensor (a view of the mapped file), or of slabs [first_slab, +n_slabs) of a 3-D one."""
        t = self._get(name)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=t.n_bytes, offset=t.offset)
        if len(t.dims) < 3:
            if first_slab or n_slabs not in (None, 1):
                raise GgufError(f"tensor {name} has no slabs")
            return raw
        slabs = int(np.prod(t.dims[2:]))
        n_slabs = slabs - first_slab if n_slabs is None else n_slabs
        if first_slab < 0 or first_slab + n_slabs > slabs:
            raise GgufError(f"tensor {name} has {slabs} slabs, asked for {first_slab}..{first_slab + n_slabs}")
        per = t.n_bytes // slabs
        return raw[first_slab * per:(first_slab + n_slabs) * per]

    def _get(self, name: str) -> GgufTensor:
        t = self.tensors.get(name)
        if t is None:
            raise GgufError(f"{self.path}: no tensor named {name}")
        if t.n_bytes < 0:
            raise GgufError(f"{self.path}: tensor {name} has ggml type {t.kind}, which this library does not decode")
        return t

    def f32(self, name: str) -> np.ndarray:
        """A small F32 tensor (norm weights, router) as a float array of shape dims reversed (rows first)."""
        t = self._get(name)
        if t.kind != synth.F32:
            raise GgufError(f"tensor {name} is not F32")
        return np.frombuffer(self._map, dtype="<f4", count=t.n_bytes // 4, offset=t.offset).reshape(tuple(reversed(t.dims)))

    def upload(self, dev, name: str, first_slab: int = 0, n_slabs: int | None = None):
        """The tensor as a resident weight: rows = ne1, cols = ne0, slabs = the product of the remaining dimensions
        (or the requested range of them, for one rank of an expert-parallel group)."""
        from .device import Weight

        t = self._get(name)
        if not 1 <= len(t.dims) <= 4:
            raise GgufError(f"tensor {name} has no matrix shape")
        cols, rows = t.dims[0], (t.dims[1] if len(t.dims) > 1 else 1)
        total = int(np.prod(t.dims[2:])) if len(t.dims) > 2 else 1
        n = (total - first_slab) if n_slabs is None else n_slabs
        return dev.upload_weight(Weight(self.tensor_bytes(name, first_slab, n) if len(t.dims) > 2 else self.tensor_bytes(name),
                                        t.kind, rows, cols), slabs=n)

    def qwen3moe_config(self, context: int = 4096):
        """The qwen3moe hyper-parameters a forward pass needs (crates/beholdd-model/src/qwen3moe.rs:879-955)."""
        from .qwen3moe import Qwen3MoeConfig

        a = self.meta.get("general.architecture")
        if a != "qwen3moe":
            raise GgufError(f"{self.path}: architecture {a!r}, expected 'qwen3moe'")
        m = lambda key, default=None: self.meta.get(f"{a}.{key}", default)
        n_layers = m("block_count")
        if n_layers is None:
            n_layers = 1 + max((int(n.split(".")[1]) for n in self.tensors if n.startswith("blk.")), default=-1)
        gate = self.tensors.get("blk.0.ffn_gate_exps.weight")
        vocab = self.tensors["token_embd.weight"].dims[1]
        return Qwen3MoeConfig(n_layers=int(n_layers), dim=int(m("embedding_length")), n_heads=int(m("attention.head_count")),
                              n_kv_heads=int(m("attention.head_count_kv")), head_dim=int(m("attention.key_length")),
                              n_experts=int(m("expert_count")), top_k=int(m("expert_used_count")),
                              expert_ff=int(m("expert_feed_forward_length", gate.dims[1] if gate else 0)), vocab=int(vocab),
                              rope_theta=float(m("rope.freq_base", 1.0e6)), eps=float(m("attention.layer_norm_rms_epsilon", 1.0e-6)),
                              context=context)
