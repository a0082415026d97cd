"""The recorded-execution interface of the reference (`ExecutionDevice`) over the CUDA library.

Mirrors crates/beholdd-backend/src/execution.rs: resident weights and f32 tensors are opaque handles
that carry the id of the device object that made them (:9-12, 67-92: a foreign handle is refused before
it is interpreted); a `CommandList` (:547-880) collects commands in order -- EmbeddingRow, Linear
(Overwrite or ScaledAdd), SwiGlu, SigmoidGate, RmsNorm, Rope, IncrementalCausalAttention (:415-457) --
and validates shapes as they are added; `record` (:1093-1099) turns the list into a `RecordedBatch`,
`submit` (:1101-1109) runs it, `wait` (:1111-1114) blocks until it is done. One more command exists
here, `routed_moe`, for the routed-expert block the reference still runs outside its IR.

The B200 form of "record" is a CUDA graph: the list is captured once on a private stream (no kernel
runs during capture) and every submission is one graph launch, so a decode step of dozens of small
kernels costs the host one call. Commands execute in list order and see earlier commands' writes.
The reference lets a backend refuse aliasing it cannot honour at `record`: partially overlapping views
within one command are refused here, in-place forms whose kernels read all inputs before writing
(RmsNorm, Rope, SwiGlu, SigmoidGate on identical views) are accepted.

Batches and submissions keep their tensors and weights alive; concurrent submissions are serialised on
the device object's stream.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass

import numpy as np

from .device import CudaDevice, DeviceError, ResidentWeight, Weight

_owner_ids = itertools.count(1)


class ExecutionError(Exception):
    """crates/beholdd-backend/src/execution.rs:34-65"""


class ForeignResource(ExecutionError):
    pass


class ShapeMismatch(ExecutionError):
    pass


class IncompatibleResource(ExecutionError):
    pass


class SynchronizationError(ExecutionError):
    pass


class BackendFailure(ExecutionError):
    """ExecutionError::Device: the wrapped DeviceError is `__cause__`."""


@dataclass(frozen=True)
class EncodedWeight:
    """Packed bytes resident on the device, not yet bound to a kernel layout (execution.rs:99-150)."""
    owner: int
    resident: ResidentWeight

    kind = property(lambda self: self.resident.kind)
    rows = property(lambda self: self.resident.rows)
    cols = property(lambda self: self.resident.cols)
    byte_len = property(lambda self: self.resident.n_bytes)


@dataclass(frozen=True)
class PreparedWeight:
    """A weight ready for Linear / EmbeddingRow (execution.rs:172-243). The library's kernels read the checkpoint
    layout directly, so preparing shares the encoded storage (clones alias storage, :240-243)."""
    owner: int
    resident: ResidentWeight

    kind = property(lambda self: self.resident.kind)
    rows = property(lambda self: self.resident.rows)
    cols = property(lambda self: self.resident.cols)
    byte_len = property(lambda self: self.resident.n_bytes)


class F32Tensor:
    """execution.rs:245-319"""

    def __init__(self, owner: int, storage):
        self.owner, self.storage = owner, storage

    def __len__(self):
        return self.storage.numel()

    def full_view(self) -> "F32TensorView":
        return F32TensorView(self, 0, len(self))

    def view(self, offset: int, length: int) -> "F32TensorView":
        if offset < 0 or length < 0 or offset + length > len(self):
            raise ShapeMismatch(f"view {offset}..{offset + length} exceeds a tensor of {len(self)} floats")
        return F32TensorView(self, offset, length)


@dataclass(frozen=True)
class F32TensorView:
    """execution.rs:321-393"""
    tensor: F32Tensor
    offset: int
    len: int

    owner = property(lambda self: self.tensor.owner)

    def view(self, offset: int, length: int) -> "F32TensorView":
        if offset < 0 or length < 0 or offset + length > self.len:
            raise ShapeMismatch(f"view {offset}..{offset + length} exceeds a view of {self.len} floats")
        return F32TensorView(self.tensor, self.offset + offset, length)

    def overlaps(self, other: "F32TensorView") -> bool:
        return (self.tensor is other.tensor and self.len > 0 and other.len > 0 and self.offset < other.offset + other.len
                and other.offset < self.offset + self.len)

    def same(self, other: "F32TensorView") -> bool:
        return self.tensor is other.tensor and self.offset == other.offset and self.len == other.len

    def torch(self):
        return self.tensor.storage[self.offset:self.offset + self.len]


@dataclass(frozen=True)
class LinearMode:
    """execution.rs:401-412: Overwrite (scale None) or ScaledAdd {scale}."""
    scale: float | None = None

    @classmethod
    def overwrite(cls):
        return cls(None)

    @classmethod
    def scaled_add(cls, scale: float):
        return cls(float(scale))


@dataclass(frozen=True)
class IncrementalAttentionConfig:
    """crates/beholdd-backend/src/lib.rs:228-253"""
    n_query_positions: int
    query_start: int
    n_kv_positions: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float


class CommandList:
    """Commands in insertion order, shape-checked as they are added (execution.rs:547-880)."""

    def __init__(self):
        self.owner: int | None = None
        self.commands: list[tuple] = []

    def __len__(self):
        return len(self.commands)

    def _accept(self, *resources):
        for r in resources:
            if r is None:
                continue
            if self.owner is None:
                self.owner = r.owner
            elif r.owner != self.owner:
                raise ForeignResource("a command list may hold resources of one execution device only")

    def embedding_row(self, output: F32TensorView, weight: PreparedWeight, row: int):
        if output.len != weight.cols or not 0 <= row < weight.rows * weight.resident.slabs:
            raise ShapeMismatch(f"embedding table is {weight.rows}x{weight.cols}, got row={row} output={output.len}")
        self._accept(output, weight)
        self.commands.append(("embedding_row", output, weight, int(row)))

    def linear(self, output: F32TensorView, input: F32TensorView, weight: PreparedWeight, mode: LinearMode = LinearMode()):
        if input.len != weight.cols or output.len != weight.rows:
            raise ShapeMismatch(f"linear weight is {weight.rows}x{weight.cols}, got input={input.len} output={output.len}")
        if mode.scale is not None and not np.isfinite(mode.scale):
            raise ShapeMismatch(f"linear scaled-add multiplier must be finite, got {mode.scale}")
        self._accept(output, input, weight)
        self.commands.append(("linear", output, input, weight, mode))

    def swiglu(self, gate: F32TensorView, up: F32TensorView, limit: float = 0.0):
        if gate.len != up.len:
            raise ShapeMismatch(f"SwiGLU expected gate={gate.len} to match up={up.len}")
        if not np.isfinite(limit) or limit < 0:
            raise ShapeMismatch(f"SwiGLU limit must be finite and non-negative, got {limit}")
        self._accept(gate, up)
        self.commands.append(("swiglu", gate, up, float(limit)))

    def sigmoid_gate(self, output: F32TensorView, input: F32TensorView, gate: F32TensorView):
        if not (output.len == input.len == gate.len):
            raise ShapeMismatch(f"sigmoid gate expected equal lengths, got output={output.len} input={input.len} gate={gate.len}")
        self._accept(output, input, gate)
        self.commands.append(("sigmoid_gate", output, input, gate))

    def rmsnorm(self, output: F32TensorView, input: F32TensorView, weight: F32TensorView | None, eps: float):
        if output.len != input.len or input.len == 0 or (weight is not None and weight.len != input.len):
            raise ShapeMismatch(f"RMSNorm expected output={input.len} and {input.len} weights, got output={output.len} "
                                f"weights={None if weight is None else weight.len}")
        if not np.isfinite(eps) or eps < 0:
            raise ShapeMismatch(f"RMSNorm epsilon must be finite and non-negative, got {eps}")
        self._accept(output, input, weight)
        self.commands.append(("rmsnorm", output, input, weight, float(eps)))

    def rope(self, x: F32TensorView, cos: F32TensorView, sin: F32TensorView, split_half: bool, inverse: bool = False):
        if sin.len != cos.len or x.len != 2 * cos.len:
            raise ShapeMismatch(f"RoPE expected x={2 * cos.len}, cos={cos.len} and sin={cos.len}, got x={x.len} cos={cos.len} sin={sin.len}")
        self._accept(x, cos, sin)
        self.commands.append(("rope", x, cos, sin, bool(split_half), bool(inverse)))

    def incremental_causal_attention(self, output: F32TensorView, q: F32TensorView, k_cache: F32TensorView, v_cache: F32TensorView,
                                     config: IncrementalAttentionConfig):
        c = config
        q_len, kv_len = c.n_query_positions * c.n_heads * c.head_dim, c.n_kv_positions * c.n_kv_heads * c.head_dim
        if output.len != q_len or q.len != q_len or k_cache.len != kv_len or v_cache.len != kv_len:
            raise ShapeMismatch(f"incremental causal attention expected out={q_len} q={q_len} k_cache={kv_len} v_cache={kv_len}, got "
                                f"out={output.len} q={q.len} k_cache={k_cache.len} v_cache={v_cache.len}")
        self._accept(output, q, k_cache, v_cache)
        self.commands.append(("attention", output, q, k_cache, v_cache, c))

    def routed_moe(self, output: F32TensorView, input: F32TensorView, router: PreparedWeight, gate: PreparedWeight, up: PreparedWeight,
                   down: PreparedWeight, top_k: int, accumulate: bool = False):
        """The routed-expert block (crates/beholdd-model/src/qwen3moe/forward.rs:1299-1407) as one command; the reference has
        no such command yet (its Vulkan precedent is VulkanDevice::routed_moe_bf16, vulkan.rs:1792-1799). input / output hold
        whole positions of router.cols floats."""
        dim = router.cols
        if dim == 0 or input.len % dim or output.len != input.len or gate.cols != dim or down.rows != dim:
            raise ShapeMismatch(f"routed experts of width {dim} got input={input.len} output={output.len}")
        if not 1 <= top_k <= router.rows:
            raise ShapeMismatch(f"top-k must be between 1 and {router.rows}, got {top_k}")
        self._accept(output, input, router, gate, up, down)
        self.commands.append(("routed_moe", output, input, router, gate, up, down, int(top_k), bool(accumulate)))


class RecordedBatch:
    """A command list bound to kernels: one CUDA graph (execution.rs:917-970). Holds its resources."""

    def __init__(self, owner, graph, commands):
        self.owner, self.graph, self.commands = owner, graph, commands

    def __len__(self):
        return len(self.commands)


class Submission:
    """execution.rs:972-996"""

    def __init__(self, owner, event, batch):
        self.owner, self.event, self.batch = owner, event, batch


class CudaExecutionDevice:
    """`ExecutionDevice` (execution.rs:1020-1115) for one B200."""

    def __init__(self, index: int = 0):
        import torch

        self.dev = CudaDevice(index)
        self.index = index
        self.owner = next(_owner_ids)
        self.stream = torch.cuda.Stream(device=index)

    def close(self):
        self.dev.close()

    def name(self) -> str:
        return self.dev.name()

    def supports(self, kind: int) -> bool:
        return self.dev.supports(kind)

    # ---- resources --------------------------------------------------------------------------
    def _wrap(self, fn):
        try:
            return fn()
        except DeviceError as e:
            raise BackendFailure(str(e)) from e

    def upload_weight(self, weight: Weight, slabs: int = 1) -> EncodedWeight:
        return EncodedWeight(self.owner, self._wrap(lambda: self.dev.upload_weight(weight, slabs)))

    def prepare_weight(self, weight: EncodedWeight) -> PreparedWeight:
        self._own(weight)
        return PreparedWeight(self.owner, weight.resident)

    def allocate_f32(self, length: int) -> F32Tensor:
        import torch

        return F32Tensor(self.owner, torch.zeros(int(length), dtype=torch.float32, device=f"cuda:{self.index}"))

    def upload_f32(self, values) -> F32Tensor:
        t = self.allocate_f32(len(values))
        self.write_f32(t.full_view(), values)
        return t

    def write_f32(self, destination: F32TensorView, values) -> None:
        import torch

        self._own(destination)
        v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        if v.size != destination.len:
            raise ShapeMismatch(f"write of {v.size} floats into a view of {destination.len}")
        with torch.cuda.stream(self.stream):
            destination.torch().copy_(torch.from_numpy(v), non_blocking=False)

    def read_f32(self, source: F32TensorView, values: np.ndarray) -> None:
        import torch

        self._own(source)
        if values.size != source.len:
            raise ShapeMismatch(f"read of a view of {source.len} floats into {values.size}")
        with torch.cuda.stream(self.stream):
            values.reshape(-1)[...] = source.torch().cpu().numpy()

    def _own(self, resource):
        if resource is not None and resource.owner != self.owner:
            raise ForeignResource("the resource belongs to another execution device")

    # ---- record / submit / wait -----------------------------------------------------------------
    @staticmethod
    def _refuse_partial_overlap(what, dest, *sources):
        for s in sources:
            if s is not None and dest.overlaps(s) and not dest.same(s):
                raise IncompatibleResource(f"{what}: the destination partially overlaps an input (only identical views may alias)")

    def _prepare(self, cmd):
        """Device-side operands a command needs besides its views, made before the capture starts (nothing may be
        allocated or copied from pageable memory while a graph is being captured)."""
        import torch

        if cmd[0] == "embedding_row":
            return torch.tensor([cmd[3]], dtype=torch.int32, device=f"cuda:{self.index}")
        if cmd[0] == "routed_moe":
            T, top_k = cmd[2].len // cmd[3].cols, cmd[7]
            return (torch.empty((T, top_k), dtype=torch.int32, device=f"cuda:{self.index}"),
                    torch.empty((T, top_k), dtype=torch.float32, device=f"cuda:{self.index}"))
        return None

    def _issue(self, cmd, aux):
        from .device import _ptr

        d, p = self.dev, lambda v: None if v is None else v.torch()
        kind = cmd[0]
        if kind == "embedding_row":
            _, out, w, row = cmd
            d.embedding_rows_resident(w.resident, aux, out.torch())
        elif kind == "linear":
            _, out, x, w, mode = cmd
            d.matvec_resident(w.resident, p(x), p(out), scale=1.0 if mode.scale is None else mode.scale, accumulate=mode.scale is not None)
        elif kind == "swiglu":
            _, gate, up, limit = cmd
            d._check(d.lib.bhd_swiglu(d.ctx, _ptr(p(gate)), _ptr(p(up)), gate.len, limit, d._stream()))
        elif kind == "sigmoid_gate":
            _, out, x, gate = cmd
            d._check(d.lib.bhd_sigmoid_gate(d.ctx, _ptr(p(out)), _ptr(p(x)), _ptr(p(gate)), out.len, d._stream()))
        elif kind == "rmsnorm":
            _, out, x, w, eps = cmd
            d.rmsnorm_resident(p(out), p(x), p(w), eps)
        elif kind == "rope":
            _, x, cos, sin, split, inverse = cmd
            d.rope_resident(p(x).view(1, 1, -1), p(cos).view(1, -1), p(sin).view(1, -1), split_half=split, inverse=inverse)
        elif kind == "attention":
            _, out, q, k, v, c = cmd
            d.attention_resident(p(out).view(c.n_query_positions, c.n_heads, c.head_dim), p(q).view(c.n_query_positions, c.n_heads, c.head_dim),
                                 p(k).view(c.n_kv_positions, c.n_kv_heads, c.head_dim), p(v).view(c.n_kv_positions, c.n_kv_heads, c.head_dim),
                                 c.query_start, c.n_kv_positions, c.scale)
        elif kind == "routed_moe":
            _, out, x, router, gate, up, down, top_k, accumulate = cmd
            T = x.len // router.cols
            d.moe_layer(router.resident, gate.resident, up.resident, down.resident, p(x).view(T, -1), p(out).view(T, -1), top_k, aux[0], aux[1],
                        None, accumulate=accumulate)
        else:
            raise IncompatibleResource(f"unknown command {kind}")

    def _workspace_bound(self, commands) -> int:
        need = 8 << 20
        for cmd in commands:
            if cmd[0] == "routed_moe":
                _, out, x, router, gate, up, down, top_k, _ = cmd
                routes = (x.len // router.cols) * top_k
                need = max(need, (16 << 20) + routes * (gate.rows + router.cols) * 16)
        return need

    def record(self, commands: CommandList) -> RecordedBatch:
        import torch

        if commands.owner is not None and commands.owner != self.owner:
            raise ForeignResource("the command list belongs to another execution device")
        for cmd in commands.commands:
            kind = cmd[0]
            if kind == "linear":
                self._refuse_partial_overlap("linear", cmd[1], cmd[2])
                if cmd[1].overlaps(cmd[2]):
                    raise IncompatibleResource("linear: the output may not alias the input")
            elif kind in ("swiglu",):
                self._refuse_partial_overlap("SwiGLU", cmd[1], cmd[2])
            elif kind == "sigmoid_gate":
                self._refuse_partial_overlap("sigmoid gate", cmd[1], cmd[2], cmd[3])
            elif kind == "rmsnorm":
                self._refuse_partial_overlap("RMSNorm", cmd[1], cmd[2], cmd[3])
            elif kind == "rope":
                if cmd[1].overlaps(cmd[2]) or cmd[1].overlaps(cmd[3]):
                    raise IncompatibleResource("RoPE: x may not alias its tables")
            elif kind == "attention":
                if any(cmd[1].overlaps(s) for s in cmd[2:5]):
                    raise IncompatibleResource("attention: the output may not alias q or the caches")
            elif kind == "routed_moe":
                if cmd[1].overlaps(cmd[2]):
                    raise IncompatibleResource("routed experts: the output may not alias the input")
        self._wrap(lambda: self.dev._check(self.dev.lib.bhd_workspace_reserve(self.dev.ctx, self._workspace_bound(commands.commands))))
        with torch.cuda.device(self.index):
            aux = [self._prepare(cmd) for cmd in commands.commands]
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize(self.index)
            try:
                with torch.cuda.graph(graph, stream=self.stream, capture_error_mode="thread_local"):
                    for cmd, a in zip(commands.commands, aux):
                        self._issue(cmd, a)
            except DeviceError as e:
                raise BackendFailure(str(e)) from e
        batch = RecordedBatch(self.owner, graph, list(commands.commands))
        batch._keep = aux
        batch._ws_bytes = self.dev.workspace_bytes()
        return batch

    def submit(self, batch: RecordedBatch) -> Submission:
        import torch

        if batch.owner != self.owner:
            raise ForeignResource("the recorded batch belongs to another execution device")
        if batch._ws_bytes != self.dev.workspace_bytes():
            raise IncompatibleResource("the device's workspace was replaced by a larger one after this batch was recorded; record it again")
        with torch.cuda.stream(self.stream):
            batch.graph.replay()
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return Submission(self.owner, ev, batch)

    def wait(self, submission: Submission) -> None:
        if submission.owner != self.owner:
            raise ForeignResource("the submission belongs to another execution device")
        try:
            submission.event.synchronize()
        except RuntimeError as e:
            raise SynchronizationError(str(e)) from e
        import torch

        with torch.cuda.stream(self.stream):
            try:
                self.dev.check_status()
            except DeviceError as e:
                raise BackendFailure(str(e)) from e
