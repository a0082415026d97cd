"""Host side of the drop-in boundary: the reference's operator interface over the C ABI.

`CudaDevice` mirrors `beholdd_backend::Device` (crates/beholdd-backend/src/lib.rs:164-272)
for the operators on the quantised-matvec / routed-expert path, with the same names,
argument meaning and refusal behaviour, and the resident half of `ExecutionDevice`
(crates/beholdd-backend/src/execution.rs:1066-1114: upload_weight, then operators on
device-resident tensors). Everything runs in `libbeholdd_b200.so`; there is no CPU
fallback, and importing the library fails loudly when the shared object is missing.

torch is used only to own device memory and streams.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libbeholdd_b200.so")

OK = 0
ERR_UNSUPPORTED_FORMAT, ERR_SHAPE, ERR_ALLOCATION, ERR_BACKEND, ERR_INVALID_ARGUMENT, ERR_DEVICE_STATUS = -1, -2, -3, -4, -5, -6

#: every symbol include/beholdd_b200.h declares
EXPORTS = [
    "bhd_error_text", "bhd_last_error_message", "bhd_device_name", "bhd_ctx_create", "bhd_ctx_destroy", "bhd_supports",
    "bhd_weight_upload", "bhd_weight_wrap_device", "bhd_weight_free", "bhd_dequantize", "bhd_matvec", "bhd_matvec_noalloc", "bhd_matvec_host", "bhd_matvec_host_async", "bhd_sync",
    "bhd_matmul", "bhd_softmax", "bhd_swiglu", "bhd_add_in_place", "bhd_moe_route", "bhd_moe_experts", "bhd_moe_combine", "bhd_moe_layer",
    "bhd_moe_layer_host", "bhd_check_status", "bhd_launch_count", "bhd_debug_wait_test", "bhd_debug_expf", "bhd_debug_option", "bhd_peer_alloc", "bhd_peer_open", "bhd_peer_close", "bhd_peer_free",
    "bhd_ep_create", "bhd_ep_connect", "bhd_ep_layer", "bhd_ep_destroy", "bhd_rowsplit_create", "bhd_rowsplit_connect",
    "bhd_rowsplit_matvec", "bhd_rowsplit_destroy", "bhd_rmsnorm", "bhd_rope", "bhd_incremental_attention", "bhd_embedding_rows", "bhd_debug_fill_q8_0", "bhd_debug_fill_normal", "bhd_sigmoid_gate", "bhd_workspace_reserve", "bhd_rope_at", "bhd_store_row_at", "bhd_incremental_attention_at", "bhd_workspace_bytes", "bhd_qk_norm_rope_store_at",
]


class DeviceError(Exception):
    """crates/beholdd-backend/src/lib.rs:60-101"""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class UnsupportedFormat(DeviceError):
    pass


class ShapeError(DeviceError):
    pass


class AllocationError(DeviceError):
    pass


class BackendError(DeviceError):
    pass


_ERRORS = {ERR_UNSUPPORTED_FORMAT: UnsupportedFormat, ERR_SHAPE: ShapeError, ERR_ALLOCATION: AllocationError}


def load_library(path: str | None = None) -> C.CDLL:
    path = path or LIB_PATH
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: build it with `python -m exec_beholdd_b200.build` "
                          "(there is no fallback implementation)")
    lib = C.CDLL(path)
    vp, u64, u32, i32, f32 = C.c_void_p, C.c_uint64, C.c_uint32, C.c_int32, C.c_float
    lib.bhd_error_text.restype = C.c_char_p
    lib.bhd_error_text.argtypes = [i32]
    lib.bhd_device_name.restype = C.c_char_p
    lib.bhd_last_error_message.argtypes = [vp, C.c_char_p, i32]
    lib.bhd_ctx_create.argtypes = [i32, C.POINTER(vp)]
    lib.bhd_ctx_destroy.argtypes = [vp]
    lib.bhd_supports.argtypes = [u32]
    lib.bhd_weight_upload.argtypes = [vp, vp, u64, u32, u64, u64, u64, C.POINTER(vp)]
    lib.bhd_weight_wrap_device.argtypes = [vp, vp, u64, u32, u64, u64, u64, C.POINTER(vp)]
    lib.bhd_weight_free.argtypes = [vp]
    lib.bhd_dequantize.argtypes = [vp, vp, u64, vp, u64, vp]
    lib.bhd_matvec.argtypes = [vp, vp, u64, vp, vp, u32, f32, i32, vp]
    lib.bhd_matvec_noalloc.argtypes = [vp, vp, u64, vp, vp, u32, f32, i32, vp]
    lib.bhd_matvec_host.argtypes = [vp, vp, u64, vp, vp, u32, f32, i32]
    lib.bhd_matvec_host_async.argtypes = [vp, vp, u64, vp, vp, u32, f32, i32]
    lib.bhd_sync.argtypes = [vp]
    lib.bhd_matmul.argtypes = [vp, vp, u64, vp, vp, u64, vp]
    lib.bhd_softmax.argtypes = [vp, vp, u64, u64, vp]
    lib.bhd_swiglu.argtypes = [vp, vp, vp, u64, f32, vp]
    lib.bhd_add_in_place.argtypes = [vp, vp, vp, u64, vp]
    lib.bhd_moe_route.argtypes = [vp, vp, vp, u64, u32, vp, vp, vp, vp, vp, vp]
    lib.bhd_moe_experts.argtypes = [vp, vp, vp, vp, vp, u64, u32, vp, vp, u32, u32, u32, vp, i32, vp]
    lib.bhd_moe_combine.argtypes = [vp, vp, vp, u64, u32, u64, i32, vp]
    lib.bhd_moe_layer.argtypes = [vp, vp, vp, vp, vp, vp, vp, u64, u32, vp, vp, vp, i32, vp]
    lib.bhd_moe_layer_host.argtypes = [vp, vp, vp, vp, vp, vp, vp, u64, u32, vp, vp, vp, i32]
    lib.bhd_check_status.argtypes = [vp, vp]
    lib.bhd_debug_wait_test.argtypes = [vp, u32, u32]
    lib.bhd_debug_expf.argtypes = [vp, vp, vp, u64, vp]
    lib.bhd_debug_option.argtypes = [vp, u32, u32]
    lib.bhd_peer_alloc.argtypes = [vp, u64, C.POINTER(vp), vp]
    lib.bhd_peer_open.argtypes = [vp, vp, C.POINTER(vp)]
    lib.bhd_peer_close.argtypes = [vp, vp]
    lib.bhd_peer_free.argtypes = [vp, vp]
    lib.bhd_ep_create.argtypes = [vp, u32, u32, u32, u32, u32, u32, C.POINTER(vp), vp]
    lib.bhd_ep_connect.argtypes = [vp, vp]
    lib.bhd_ep_layer.argtypes = [vp, vp, vp, vp, vp, vp, vp, u64, vp, vp, vp, i32, vp]
    lib.bhd_ep_destroy.argtypes = [vp]
    lib.bhd_rowsplit_create.argtypes = [vp, u32, u32, u32, u32, C.POINTER(vp), vp]
    lib.bhd_rowsplit_connect.argtypes = [vp, vp]
    lib.bhd_rowsplit_matvec.argtypes = [vp, vp, u64, vp, vp, u32, f32, vp]
    lib.bhd_rowsplit_destroy.argtypes = [vp]
    lib.bhd_rmsnorm.argtypes = [vp, vp, vp, vp, u64, u64, f32, vp]
    lib.bhd_rope.argtypes = [vp, vp, vp, vp, u64, u32, u32, i32, i32, vp]
    lib.bhd_incremental_attention.argtypes = [vp, vp, vp, vp, vp, u64, u64, u64, u32, u32, u32, f32, vp]
    lib.bhd_embedding_rows.argtypes = [vp, vp, vp, u64, vp, vp]
    lib.bhd_debug_fill_q8_0.argtypes = [vp, vp, u64, u64, u64, u64, u64, vp]
    lib.bhd_debug_fill_normal.argtypes = [vp, vp, u64, u64, u64, f32, vp]
    lib.bhd_sigmoid_gate.argtypes = [vp, vp, vp, vp, u64, vp]
    lib.bhd_workspace_reserve.argtypes = [vp, u64]
    lib.bhd_qk_norm_rope_store_at.argtypes = [vp] * 11 + [u64, u32, u32, u32, f32, i32, vp]
    lib.bhd_workspace_bytes.restype = u64
    lib.bhd_workspace_bytes.argtypes = [vp]
    lib.bhd_rope_at.argtypes = [vp, vp, vp, vp, vp, u32, u32, i32, i32, vp]
    lib.bhd_store_row_at.argtypes = [vp, vp, vp, vp, u64, u64, vp]
    lib.bhd_incremental_attention_at.argtypes = [vp, vp, vp, vp, vp, vp, u64, u32, u32, u32, C.c_float, vp]
    lib.bhd_launch_count.restype = u64
    lib.bhd_launch_count.argtypes = [vp]
    return lib


@dataclass(frozen=True)
class Weight:
    """A weight as it sits in host memory: packed bytes plus their meaning
    (crates/beholdd-backend/src/lib.rs:47-57)."""
    bytes: np.ndarray
    kind: int
    rows: int
    cols: int


class ResidentWeight:
    """A packed weight in HBM (EncodedWeight/PreparedWeight, execution.rs:1066-1070).
    `slabs` > 1 holds a 3-D expert tensor; `rows` is per slab."""

    def __init__(self, device: "CudaDevice", handle: int, kind: int, rows: int, cols: int, slabs: int, n_bytes: int,
                 keepalive=None):
        self.device, self.handle, self.kind, self.rows, self.cols, self.slabs = device, handle, kind, rows, cols, slabs
        self.n_bytes = n_bytes
        self._keepalive = keepalive

    def free(self) -> None:
        if self.handle:
            self.device.lib.bhd_weight_free(self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _ptr(t):
    """Device pointer of a torch tensor (or None)."""
    return None if t is None else C.c_void_p(t.data_ptr())


class CudaDevice:
    """`Device` for one B200. Host-array methods follow the immediate trait; `*_resident`
    methods take torch CUDA tensors and run asynchronously on torch's current stream."""

    def __init__(self, index: int = 0, lib_path: str | None = None):
        self.lib = load_library(lib_path)
        self.index = index
        h = C.c_void_p()
        st = self.lib.bhd_ctx_create(index, C.byref(h))
        if st != OK:
            raise BackendError(st, f"cuda-b200 backend error: cannot create a context on device {index}: "
                                   f"{self.lib.bhd_error_text(st).decode()}")
        self.ctx = h

    # ---- plumbing -------------------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "ctx", None):
            self.lib.bhd_ctx_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _message(self) -> str:
        buf = C.create_string_buffer(600)
        self.lib.bhd_last_error_message(self.ctx, buf, 600)
        return buf.value.decode(errors="replace")

    def _check(self, st: int) -> None:
        if st != OK:
            raise _ERRORS.get(st, BackendError if st == ERR_BACKEND else DeviceError)(st, self._message() or
                                                                                        self.lib.bhd_error_text(st).decode())

    @staticmethod
    def _stream():
        import torch

        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def check_status(self) -> None:
        """Synchronise the current stream and raise if a kernel flagged a problem."""
        self._check(self.lib.bhd_check_status(self.ctx, self._stream()))

    @property
    def launch_count(self) -> int:
        return int(self.lib.bhd_launch_count(self.ctx))

    # ---- Device ---------------------------------------------------------------------
    def name(self) -> str:
        return self.lib.bhd_device_name().decode()

    def supports(self, kind: int) -> bool:
        return bool(self.lib.bhd_supports(kind))

    def upload_weight(self, weight: Weight, slabs: int = 1) -> ResidentWeight:
        b = np.ascontiguousarray(weight.bytes, dtype=np.uint8)
        h = C.c_void_p()
        self._check(self.lib.bhd_weight_upload(self.ctx, b.ctypes.data_as(C.c_void_p), b.size, weight.kind, weight.rows,
                                               weight.cols, slabs, C.byref(h)))
        return ResidentWeight(self, h.value, weight.kind, weight.rows, weight.cols, slabs, b.size)

    def wrap_weight(self, packed, kind: int, rows: int, cols: int, slabs: int = 1) -> ResidentWeight:
        """Wrap packed bytes that already live in a torch uint8 CUDA tensor (no copy)."""
        h = C.c_void_p()
        self._check(self.lib.bhd_weight_wrap_device(self.ctx, _ptr(packed), packed.numel(), kind, rows, cols, slabs,
                                                    C.byref(h)))
        return ResidentWeight(self, h.value, kind, rows, cols, slabs, packed.numel(), keepalive=packed)

    def dequantize(self, out: np.ndarray, weight: Weight) -> None:
        import torch

        w = self.upload_weight(weight)
        try:
            if out.size != weight.rows * weight.cols:
                self._check(self.lib.bhd_dequantize(self.ctx, w.handle, 0, None, out.size, None))
            o = torch.empty(max(out.size, 1), dtype=torch.float32, device=f"cuda:{self.index}")
            self._check(self.lib.bhd_dequantize(self.ctx, w.handle, 0, _ptr(o), out.size, self._stream()))
            out[...] = o[: out.size].cpu().numpy().reshape(out.shape)
        finally:
            w.free()

    def _matvec_host(self, y: np.ndarray, x: np.ndarray, weight: Weight, scale: float, accumulate: bool) -> None:
        assert y.dtype == np.float32 and y.flags.c_contiguous
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.size != weight.cols or y.size != weight.rows:
            raise ShapeError(ERR_SHAPE, f"shape mismatch: weight is {weight.rows}x{weight.cols}, got x={x.size} y={y.size}")
        w = self.upload_weight(weight)  # the immediate trait borrows host bytes on every call
        try:
            self._check(self.lib.bhd_matvec_host(self.ctx, w.handle, 0, x.ctypes.data_as(C.c_void_p),
                                                 y.ctypes.data_as(C.c_void_p), 1, scale, 1 if accumulate else 0))
        finally:
            w.free()

    def matvec(self, y: np.ndarray, x: np.ndarray, w: Weight) -> None:
        """y[r] = sum_i W[r][i] * x[i], overwriting y (lib.rs:182-183)."""
        self._matvec_host(y, x, w, 1.0, False)

    def matvec_add(self, y: np.ndarray, x: np.ndarray, w: Weight, scale: float) -> None:
        """y[r] += (sum_i W[r][i] * x[i]) * scale (lib.rs:189-198)."""
        self._matvec_host(y, x, w, scale, True)

    def softmax(self, v: np.ndarray) -> None:
        import torch

        if v.size == 0:
            raise ShapeError(ERR_SHAPE, "shape mismatch: softmax input cannot be empty")
        t = torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32)).to(f"cuda:{self.index}")
        self._check(self.lib.bhd_softmax(self.ctx, _ptr(t), 1, v.size, self._stream()))
        try:
            self.check_status()
        except DeviceError as e:
            raise ShapeError(ERR_SHAPE, "shape mismatch: " + str(e)) from None
        v[...] = t.cpu().numpy().reshape(v.shape)

    def swiglu(self, gate: np.ndarray, up: np.ndarray, limit: float) -> None:
        import torch

        if gate.size != up.size:
            raise ShapeError(ERR_SHAPE, f"shape mismatch: swiglu gate={gate.size} up={up.size}")
        g = torch.from_numpy(np.ascontiguousarray(gate, dtype=np.float32)).to(f"cuda:{self.index}")
        u = torch.from_numpy(np.ascontiguousarray(up, dtype=np.float32)).to(f"cuda:{self.index}")
        self._check(self.lib.bhd_swiglu(self.ctx, _ptr(g), _ptr(u), gate.size, limit, self._stream()))
        gate[...] = g.cpu().numpy().reshape(gate.shape)

    def add_in_place(self, output: np.ndarray, residual: np.ndarray) -> None:
        import torch

        if output.size != residual.size:
            raise ShapeError(ERR_SHAPE, f"shape mismatch: add_in_place output={output.size} residual={residual.size}")
        o = torch.from_numpy(np.ascontiguousarray(output, dtype=np.float32)).to(f"cuda:{self.index}")
        r = torch.from_numpy(np.ascontiguousarray(residual, dtype=np.float32)).to(f"cuda:{self.index}")
        self._check(self.lib.bhd_add_in_place(self.ctx, _ptr(o), _ptr(r), output.size, self._stream()))
        output[...] = o.cpu().numpy().reshape(output.shape)

    # ---- resident operators (torch CUDA tensors, asynchronous) ------------------------
    def dequantize_resident(self, w: ResidentWeight, out, slab: int = 0) -> None:
        self._check(self.lib.bhd_dequantize(self.ctx, w.handle, slab, _ptr(out), out.numel(), self._stream()))

    def matvec_resident(self, w: ResidentWeight, x, y, scale: float = 1.0, accumulate: bool = False, slab: int = 0) -> None:
        """x [batch x cols] (or [cols]), y [batch x rows]: Command::Linear with
        LinearMode::Overwrite or ScaledAdd (execution.rs:404-425)."""
        batch = 1 if x.dim() == 1 else x.shape[0]
        if x.numel() != batch * w.cols or y.numel() != batch * w.rows:
            raise ShapeError(ERR_SHAPE, f"shape mismatch: weight is {w.rows}x{w.cols}, got x={tuple(x.shape)} y={tuple(y.shape)}")
        self._check(self.lib.bhd_matvec(self.ctx, w.handle, slab, _ptr(x), _ptr(y), batch, scale, 1 if accumulate else 0,
                                        self._stream()))

    def matvec_host_resident(self, w: ResidentWeight, x: np.ndarray, y: np.ndarray, scale: float = 1.0,
                             accumulate: bool = False, slab: int = 0) -> None:
        """Resident weight, host activations: x in, y back, synchronous."""
        batch = 1 if x.ndim == 1 else x.shape[0]
        if x.size != batch * w.cols or y.size != batch * w.rows:
            raise ShapeError(ERR_SHAPE, f"shape mismatch: weight is {w.rows}x{w.cols}, got x={x.shape} y={y.shape}")
        self._check(self.lib.bhd_matvec_host(self.ctx, w.handle, slab, x.ctypes.data_as(C.c_void_p),
                                             y.ctypes.data_as(C.c_void_p), batch, scale, 1 if accumulate else 0))

    def matvec_host_async(self, w: ResidentWeight, x: np.ndarray, y: np.ndarray, scale: float = 1.0,
                          accumulate: bool = False, slab: int = 0) -> None:
        """matvec_host_resident without the wait: queued on the context's own stream; `sync()` waits
        (ExecutionDevice::submit / wait, execution.rs:1101-1114). A page-locked x must stay unchanged
        until then."""
        batch = 1 if x.ndim == 1 else x.shape[0]
        if x.size != batch * w.cols or y.size != batch * w.rows:
            raise ShapeError(ERR_SHAPE, f"shape mismatch: weight is {w.rows}x{w.cols}, got x={x.shape} y={y.shape}")
        self._check(self.lib.bhd_matvec_host_async(self.ctx, w.handle, slab, x.ctypes.data_as(C.c_void_p),
                                                   y.ctypes.data_as(C.c_void_p), batch, scale, 1 if accumulate else 0))

    def sync(self) -> None:
        """Wait for the queued host-buffer calls; raises if a kernel flagged a problem."""
        self._check(self.lib.bhd_sync(self.ctx))

    def matmul_resident(self, w: ResidentWeight, x, y, slab: int = 0) -> None:
        """Prefill: y[m][n] = sum_k x[m][k] * W[n][k]."""
        m = x.shape[0]
        if x.numel() != m * w.cols or y.numel() != m * w.rows:
            raise ShapeError(ERR_SHAPE, f"shape mismatch: weight is {w.rows}x{w.cols}, got x={tuple(x.shape)} y={tuple(y.shape)}")
        self._check(self.lib.bhd_matmul(self.ctx, w.handle, slab, _ptr(x), _ptr(y), m, self._stream()))

    def rmsnorm_resident(self, y, x, weight=None, eps: float = 1e-6) -> None:
        """Rows of x [n_rows x n] (or one vector) normalised into y (Command::RmsNorm, execution.rs:415-457)."""
        n = x.shape[-1]
        self._check(self.lib.bhd_rmsnorm(self.ctx, _ptr(y), _ptr(x), _ptr(weight), x.numel() // n, n, eps, self._stream()))

    def rope_resident(self, x, cos, sin, split_half: bool = True, inverse: bool = False) -> None:
        """x [n_positions x heads x head_dim] rotated in place with cos/sin [n_positions x head_dim / 2] (Command::Rope)."""
        n_pos, heads, hd = x.shape
        self._check(self.lib.bhd_rope(self.ctx, _ptr(x), _ptr(cos), _ptr(sin), n_pos, heads, hd // 2, 1 if split_half else 0,
                                      1 if inverse else 0, self._stream()))

    def attention_resident(self, out, q, k_cache, v_cache, query_start: int, n_kv_positions: int, scale: float) -> None:
        """q [n_query x n_heads x head_dim] against caches [>= n_kv_positions x n_kv_heads x head_dim]
        (Command::IncrementalCausalAttention)."""
        n_q, n_heads, hd = q.shape
        self._check(self.lib.bhd_incremental_attention(self.ctx, _ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), n_q, query_start,
                                                       n_kv_positions, n_heads, k_cache.shape[1], hd, scale, self._stream()))

    def workspace_bytes(self) -> int:
        """Size of the context's workspace; it changes exactly when the workspace is replaced (CUDA graphs captured before
        then point into freed memory)."""
        return int(self.lib.bhd_workspace_bytes(self.ctx))

    def rope_at_resident(self, x, cos_table, sin_table, pos_dev, split_half: bool = True, inverse: bool = False) -> None:
        """x [heads x head_dim] of the one position *pos_dev, rotated with row *pos_dev of the tables."""
        heads, hd = x.shape[-2], x.shape[-1]
        self._check(self.lib.bhd_rope_at(self.ctx, _ptr(x), _ptr(cos_table), _ptr(sin_table), _ptr(pos_dev), heads, hd // 2,
                                         1 if split_half else 0, 1 if inverse else 0, self._stream()))

    def qk_norm_rope_store_at_resident(self, q, k, v, q_norm, k_norm, cos_table, sin_table, k_cache, v_cache, pos_dev, eps: float,
                                       split_half: bool = True) -> None:
        """q [n_heads x head_dim], k / v [n_kv_heads x head_dim] of the position *pos_dev: QK-norm and rope in place, k and v
        appended to the caches [max_positions x n_kv_heads x head_dim]."""
        n_heads, hd = q.shape[-2], q.shape[-1]
        self._check(self.lib.bhd_qk_norm_rope_store_at(self.ctx, _ptr(q), _ptr(k), _ptr(v), _ptr(q_norm), _ptr(k_norm), _ptr(cos_table),
                                                       _ptr(sin_table), _ptr(k_cache), _ptr(v_cache), _ptr(pos_dev), k_cache.shape[0], n_heads,
                                                       k_cache.shape[1], hd, eps, 1 if split_half else 0, self._stream()))

    def store_row_at_resident(self, dst, src, pos_dev) -> None:
        """dst[*pos_dev] = src; dst [max_rows x row]."""
        self._check(self.lib.bhd_store_row_at(self.ctx, _ptr(dst), _ptr(src), _ptr(pos_dev), src.numel(), dst.shape[0], self._stream()))

    def attention_at_resident(self, out, q, k_cache, v_cache, pos_dev, scale: float) -> None:
        """One query [n_heads x head_dim] at position *pos_dev against the caches [max_positions x n_kv_heads x head_dim]."""
        n_heads, hd = q.shape[-2], q.shape[-1]
        self._check(self.lib.bhd_incremental_attention_at(self.ctx, _ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(pos_dev),
                                                          k_cache.shape[0], n_heads, k_cache.shape[1], hd, scale, self._stream()))

    def embedding_rows_resident(self, table: ResidentWeight, ids, out) -> None:
        """out[i] = decoded row ids[i] of the table (Command::EmbeddingRow)."""
        self._check(self.lib.bhd_embedding_rows(self.ctx, table.handle, _ptr(ids), ids.numel(), _ptr(out), self._stream()))

    def moe_route(self, router: ResidentWeight, x, top_k: int, experts, weights, counts=None, near=None, probs=None) -> None:
        T = x.shape[0]
        self._check(self.lib.bhd_moe_route(self.ctx, router.handle, _ptr(x), T, top_k, _ptr(experts), _ptr(weights),
                                           _ptr(counts), _ptr(near), _ptr(probs), self._stream()))

    def moe_experts(self, gate: ResidentWeight, up: ResidentWeight, down: ResidentWeight, x, experts, weights, y,
                    first_expert: int = 0, n_local: int | None = None, accumulate: bool = False, n_experts: int = 0) -> None:
        """`n_experts`: the layer's expert count over all ranks (0 = not known to the caller)."""
        T, k = experts.shape
        n_local = gate.slabs if n_local is None else n_local
        self._check(self.lib.bhd_moe_experts(self.ctx, gate.handle, up.handle, down.handle, _ptr(x), T, k, _ptr(experts),
                                             _ptr(weights), first_expert, n_local, n_experts, _ptr(y),
                                             1 if accumulate else 0, self._stream()))

    def moe_combine(self, per_route, y, accumulate: bool = False) -> None:
        """per_route [k, T, dim] (rows pre-scaled by their route weights) summed in route order into y."""
        k, T, dim = per_route.shape
        self._check(self.lib.bhd_moe_combine(self.ctx, _ptr(per_route), _ptr(y), T, k, dim, 1 if accumulate else 0,
                                             self._stream()))

    def moe_layer(self, router: ResidentWeight, gate: ResidentWeight, up: ResidentWeight, down: ResidentWeight, x, y,
                  top_k: int, experts, weights, counts=None, accumulate: bool = False) -> None:
        T = x.shape[0]
        self._check(self.lib.bhd_moe_layer(self.ctx, router.handle, gate.handle, up.handle, down.handle, _ptr(x), _ptr(y),
                                           T, top_k, _ptr(experts), _ptr(weights), _ptr(counts), 1 if accumulate else 0,
                                           self._stream()))

    def moe_layer_host(self, router: ResidentWeight, gate: ResidentWeight, up: ResidentWeight, down: ResidentWeight,
                       x: np.ndarray, y: np.ndarray, top_k: int, experts: np.ndarray | None = None,
                       weights: np.ndarray | None = None, counts: np.ndarray | None = None, accumulate: bool = False) -> None:
        T = x.shape[0]
        p = lambda a: None if a is None else a.ctypes.data_as(C.c_void_p)
        self._check(self.lib.bhd_moe_layer_host(self.ctx, router.handle, gate.handle, up.handle, down.handle, p(x), p(y), T,
                                                top_k, p(experts), p(weights), p(counts), 1 if accumulate else 0))
