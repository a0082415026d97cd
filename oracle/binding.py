"""ctypes binding of the CPU oracle (test infrastructure only).

The oracle restates the reference's CPU arithmetic (see beholdd_oracle.cpp); this module
builds it with `make` when the shared object is missing and wraps it with numpy-typed
helpers whose names follow the reference's operator interface
(crates/beholdd-backend/src/lib.rs:164-272).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

OK, UNSUPPORTED, SHAPE, INVALID = 0, -1, -2, -3

F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 8, 12, 13, 14, 30


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile; returns the path of the shared object."""
    src = os.path.join(_HERE, "beholdd_oracle.cpp")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


def _u8(a):
    a = np.ascontiguousarray(a, dtype=np.uint8)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint8))


def _f32(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _i32(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


class OracleError(Exception):
    def __init__(self, status):
        super().__init__({UNSUPPORTED: "unsupported format", SHAPE: "shape", INVALID: "invalid"}.get(status, str(status)))
        self.status = status


class Oracle:
    def __init__(self, path: str | None = None):
        self.lib = C.CDLL(path or build())
        L = self.lib
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_q8_0_dot.restype = C.c_float
        L.orc_q8_0_dot.argtypes = [C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.c_uint64]
        L.orc_worker_count.restype = C.c_uint64
        L.orc_worker_count.argtypes = [C.c_uint64] * 3
        L.orc_available_parallelism.restype = C.c_uint64
        L.orc_dequantize.argtypes = [C.POINTER(C.c_uint8), C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint64,
                                     C.POINTER(C.c_float), C.c_uint64]
        L.orc_matvec.argtypes = [C.POINTER(C.c_float), C.c_uint64, C.POINTER(C.c_float), C.c_uint64,
                                 C.POINTER(C.c_uint8), C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint64, C.c_float,
                                 C.c_int32, C.c_uint64]
        L.orc_serial_matvec.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_uint8), C.c_uint64,
                                        C.c_uint32, C.c_uint64, C.c_uint64]
        L.orc_softmax.argtypes = [C.POINTER(C.c_float), C.c_uint64]
        L.orc_expf_array.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_uint64]
        L.orc_expf_array.restype = None
        L.orc_rope_table.argtypes = [C.c_double, C.c_uint64, C.c_uint64, C.c_double, C.c_double, C.c_double, C.c_uint64,
                                     C.POINTER(C.c_float), C.POINTER(C.c_float)]
        L.orc_rope.argtypes = [C.POINTER(C.c_float), C.c_uint64, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_uint64, C.c_int32,
                               C.c_int32]
        L.orc_incremental_attention.argtypes = [C.POINTER(C.c_float)] * 4 + [C.c_uint64] * 6 + [C.c_float]
        L.orc_swiglu.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_uint64, C.c_float]
        L.orc_rmsnorm.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_uint64, C.c_float]
        L.orc_stable_top_k.argtypes = [C.POINTER(C.c_float), C.c_uint64, C.c_uint64, C.POINTER(C.c_int32),
                                       C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_uint64)]
        L.orc_scale_min_k4.argtypes = [C.c_int32, C.POINTER(C.c_uint8), C.POINTER(C.c_uint8), C.POINTER(C.c_uint8)]
        L.orc_scale_min_k4.restype = None
        L.orc_moe_route.argtypes = [C.POINTER(C.c_float), C.c_uint64, C.c_uint64, C.POINTER(C.c_float), C.c_uint64,
                                    C.c_uint64, C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_float),
                                    C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
        L.orc_moe_experts.argtypes = [C.POINTER(C.c_uint8)] * 3 + [C.c_uint64] * 3 + [C.POINTER(C.c_float), C.c_uint64,
                                      C.c_uint64, C.POINTER(C.c_int32), C.POINTER(C.c_float), C.POINTER(C.c_float),
                                      C.c_uint64]
        L.orc_moe_layer.argtypes = [C.POINTER(C.c_float)] + [C.POINTER(C.c_uint8)] * 3 + [C.c_uint64] * 3 + [
            C.POINTER(C.c_float), C.c_uint64, C.c_uint64, C.POINTER(C.c_float), C.c_int32, C.POINTER(C.c_int32),
            C.POINTER(C.c_float), C.POINTER(C.c_int32), C.c_uint64]

    # ---- scalar helpers -------------------------------------------------------------
    def f16_to_f32(self, bits: int) -> np.float32:
        return np.float32(self.lib.orc_f16_to_f32(bits))

    def scale_min_k4(self, j: int, q12) -> tuple[int, int]:
        q, qp = _u8(q12)
        sc, m = C.c_uint8(), C.c_uint8()
        self.lib.orc_scale_min_k4(j, qp, C.byref(sc), C.byref(m))
        return sc.value, m.value

    def worker_count(self, rows, cols, available) -> int:
        return int(self.lib.orc_worker_count(rows, cols, available))

    def available_parallelism(self) -> int:
        return int(self.lib.orc_available_parallelism())

    # ---- Device operators -----------------------------------------------------------
    def dequantize(self, bytes_, kind, rows, cols, out_len=None) -> np.ndarray:
        b, bp = _u8(bytes_)
        n = rows * cols if out_len is None else out_len
        out = np.zeros(n, dtype=np.float32)
        st = self.lib.orc_dequantize(bp, b.size, kind, rows, cols, _f32(out), n)
        if st != OK:
            raise OracleError(st)
        return out

    def q8_0_dot(self, row_bytes, x) -> np.float32:
        b, bp = _u8(row_bytes)
        x = np.ascontiguousarray(x, dtype=np.float32)
        return np.float32(self.lib.orc_q8_0_dot(bp, _f32(x), x.size))

    def matvec(self, bytes_, kind, rows, cols, x, y=None, scale=1.0, accumulate=False, threads=0) -> np.ndarray:
        """Device::matvec (y=None / accumulate False) or Device::matvec_add. A refused call
        raises and leaves `y` untouched, like the reference."""
        b, bp = _u8(bytes_)
        x = np.ascontiguousarray(x, dtype=np.float32)
        if y is None:
            y = np.zeros(rows, dtype=np.float32)
        assert y.dtype == np.float32 and y.flags.c_contiguous
        st = self.lib.orc_matvec(_f32(y), y.size, _f32(x), x.size, bp, b.size, kind, rows, cols, scale,
                                 1 if accumulate else 0, threads)
        if st != OK:
            raise OracleError(st)
        return y

    def matvec_batch(self, bytes_, kind, rows, cols, xs, threads=0) -> np.ndarray:
        """The reference has no batched matvec; it loops matvec per position
        (crates/beholdd-model/src/qwen3moe/forward.rs:1091-1100)."""
        xs = np.ascontiguousarray(xs, dtype=np.float32).reshape(-1, cols)
        return np.stack([self.matvec(bytes_, kind, rows, cols, x, threads=threads) for x in xs])

    def serial_matvec(self, bytes_, kind, rows, cols, x) -> np.ndarray:
        b, bp = _u8(bytes_)
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.size != cols:
            raise OracleError(SHAPE)
        y = np.zeros(rows, dtype=np.float32)
        st = self.lib.orc_serial_matvec(_f32(y), _f32(x), bp, b.size, kind, rows, cols)
        if st != OK:
            raise OracleError(st)
        return y

    def softmax(self, v) -> np.ndarray:
        v = np.array(v, dtype=np.float32)
        st = self.lib.orc_softmax(_f32(v), v.size)
        if st != OK:
            raise OracleError(st)
        return v

    def expf(self, v) -> np.ndarray:
        """The host libm's expf, element by element."""
        v = np.ascontiguousarray(v, dtype=np.float32)
        out = np.empty_like(v)
        self.lib.orc_expf_array(_f32(v), _f32(out), v.size)
        return out

    def rope_table(self, theta, dim, pos, orig_seq_len=0, factor=1.0, beta_fast=32.0, beta_slow=1.0):
        """cos / sin of one position (vecops::rope_freqs + rope_at)."""
        cos, sin = np.zeros(dim // 2, dtype=np.float32), np.zeros(dim // 2, dtype=np.float32)
        st = self.lib.orc_rope_table(theta, dim, orig_seq_len, factor, beta_fast, beta_slow, pos, _f32(cos), _f32(sin))
        if st != OK:
            raise OracleError(st)
        return cos, sin

    def rope(self, x, cos, sin, split_half: bool, inverse: bool = False) -> np.ndarray:
        """Device::rope on one vector; returns the rotated copy."""
        x = np.array(x, dtype=np.float32)
        cos, sin = np.ascontiguousarray(cos, dtype=np.float32), np.ascontiguousarray(sin, dtype=np.float32)
        if sin.size != cos.size:
            raise OracleError(SHAPE)
        st = self.lib.orc_rope(_f32(x), x.size, _f32(cos), _f32(sin), cos.size, 1 if split_half else 0, 1 if inverse else 0)
        if st != OK:
            raise OracleError(st)
        return x

    def incremental_attention(self, q, k_cache, v_cache, n_query, query_start, n_kv, n_heads, n_kv_heads, head_dim, scale):
        """Device::incremental_causal_attention; q [n_query][n_heads][head_dim], caches [n_kv][n_kv_heads][head_dim]."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k_cache, dtype=np.float32)
        v = np.ascontiguousarray(v_cache, dtype=np.float32)
        if q.size != n_query * n_heads * head_dim or k.size != n_kv * n_kv_heads * head_dim or v.size != k.size:
            raise OracleError(SHAPE)
        out = np.zeros(q.size, dtype=np.float32)
        st = self.lib.orc_incremental_attention(_f32(out), _f32(q), _f32(k), _f32(v), n_query, query_start, n_kv, n_heads, n_kv_heads,
                                                head_dim, scale)
        if st != OK:
            raise OracleError(st)
        return out.reshape(q.shape)

    def causal_attention(self, q, k, v, n_positions, n_heads, n_kv_heads, head_dim, scale):
        """Device::causal_attention: every position attends to itself and the positions before it."""
        return self.incremental_attention(q, k, v, n_positions, 0, n_positions, n_heads, n_kv_heads, head_dim, scale)

    def swiglu(self, gate, up, limit=0.0) -> np.ndarray:
        g = np.array(gate, dtype=np.float32)
        u = np.ascontiguousarray(up, dtype=np.float32)
        self.lib.orc_swiglu(_f32(g), _f32(u), g.size, limit)
        return g

    def rmsnorm(self, x, w=None, eps=1e-6) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.zeros_like(x)
        wp = None if w is None else _f32(np.ascontiguousarray(w, dtype=np.float32))
        st = self.lib.orc_rmsnorm(_f32(y), _f32(x), wp, x.size, eps)
        if st != OK:
            raise OracleError(st)
        return y

    def stable_top_k(self, probs, k):
        p = np.ascontiguousarray(probs, dtype=np.float32)
        idx = np.zeros(max(k, 1), dtype=np.int32)
        w = np.zeros(max(k, 1), dtype=np.float32)
        near = np.zeros(8, dtype=np.int32)
        nlen = C.c_uint64(0)
        st = self.lib.orc_stable_top_k(_f32(p), p.size, k, _i32(idx), _f32(w), _i32(near), C.byref(nlen))
        if st != OK:
            raise OracleError(st)
        return idx[:k], w[:k], near[: nlen.value]

    # ---- routed-expert block --------------------------------------------------------
    def moe_route(self, router, x, top_k):
        router = np.ascontiguousarray(router, dtype=np.float32)
        n_experts, dim = router.shape
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, dim)
        T = x.shape[0]
        near_per = min(8, max(n_experts - top_k, 0))
        probs = np.zeros((T, n_experts), dtype=np.float32)
        experts = np.zeros((T, top_k), dtype=np.int32)
        weights = np.zeros((T, top_k), dtype=np.float32)
        near = np.zeros((T, max(near_per, 1)), dtype=np.int32)
        counts = np.zeros(n_experts, dtype=np.int32)
        st = self.lib.orc_moe_route(_f32(router), n_experts, dim, _f32(x), T, top_k, _f32(probs), _i32(experts),
                                    _f32(weights), _i32(near), _i32(counts))
        if st != OK:
            raise OracleError(st)
        return probs, experts, weights, near[:, :near_per], counts

    def moe_experts(self, gate_exps, up_exps, down_exps, n_experts, dim, expert_ff, x, experts, weights, threads=0):
        g, gp = _u8(gate_exps)
        u, up_ = _u8(up_exps)
        d, dp = _u8(down_exps)
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, dim)
        experts = np.ascontiguousarray(experts, dtype=np.int32)
        weights = np.ascontiguousarray(weights, dtype=np.float32)
        T, k = experts.shape
        out = np.zeros((T, dim), dtype=np.float32)
        st = self.lib.orc_moe_experts(gp, up_, dp, n_experts, dim, expert_ff, _f32(x), T, k, _i32(experts),
                                      _f32(weights), _f32(out), threads)
        if st != OK:
            raise OracleError(st)
        return out

    def moe_layer(self, router, gate_exps, up_exps, down_exps, expert_ff, x, top_k, y=None, threads=0):
        router = np.ascontiguousarray(router, dtype=np.float32)
        n_experts, dim = router.shape
        g, gp = _u8(gate_exps)
        u, up_ = _u8(up_exps)
        d, dp = _u8(down_exps)
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, dim)
        T = x.shape[0]
        accumulate = y is not None
        if y is None:
            y = np.zeros((T, dim), dtype=np.float32)
        experts = np.zeros((T, top_k), dtype=np.int32)
        weights = np.zeros((T, top_k), dtype=np.float32)
        counts = np.zeros(n_experts, dtype=np.int32)
        st = self.lib.orc_moe_layer(_f32(router), gp, up_, dp, n_experts, dim, expert_ff, _f32(x), T, top_k, _f32(y),
                                    1 if accumulate else 0, _i32(experts), _f32(weights), _i32(counts), threads)
        if st != OK:
            raise OracleError(st)
        return y, experts, weights, counts


_singleton: Oracle | None = None


def load() -> Oracle:
    global _singleton
    if _singleton is None:
        _singleton = Oracle()
    return _singleton
