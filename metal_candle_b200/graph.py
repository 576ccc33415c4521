"""Lazy computation graph: the host-side mirror of the reference's `src/graph`.

`LazyTensor` records operations as nodes of a `ComputationGraph`; `eval()` schedules them in DFS post-order
and `AsyncExecutor.execute_operation` dispatches each one to a CUDA kernel through the C ABI
(src/graph/lazy_tensor.rs:342-424, src/graph/node.rs:183-345, src/graph/operation.rs, src/graph/executor.rs).
Names, arities and error messages follow the reference.  Differences: every operation runs its CUDA kernel
(there is no "fused on Metal, otherwise candle ops" split: the fused kernel is the only path), work is enqueued
on the current stream and `synchronize()` really synchronises, and `Operation.LoRA.output_shape` returns
`[..., out_features]` (the reference returns the input shape, which is wrong when out != in,
src/graph/operation.rs:152).
"""
from __future__ import annotations

import threading
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib, backend
from .backend import TrainingError


@dataclass(frozen=True)
class NodeId:
    """src/graph/node.rs:9."""
    index: int

    def __repr__(self) -> str:
        return f"NodeId({self.index})"


class Operation:
    """src/graph/operation.rs:7-50.  Build with the class methods; `kind` is the variant name."""

    def __init__(self, kind: str, **params):
        self.kind, self.params = kind, params

    @staticmethod
    def Input():
        return Operation("Input")

    @staticmethod
    def Matmul():
        return Operation("Matmul")

    @staticmethod
    def Add():
        return Operation("Add")

    @staticmethod
    def Mul():
        return Operation("Mul")

    @staticmethod
    def MulScalar(value: float):
        return Operation("MulScalar", value=float(value))

    @staticmethod
    def LoRA(a: NodeId, b: NodeId, scale: float):
        return Operation("LoRA", a=a, b=b, scale=float(scale))

    @staticmethod
    def Softmax(dim: int):
        return Operation("Softmax", dim=int(dim))

    @staticmethod
    def RMSNorm(eps: float):
        return Operation("RMSNorm", eps=float(eps))

    _NAMES = {"Input": "input", "Matmul": "matmul", "Add": "add", "Mul": "mul", "MulScalar": "mul_scalar",
              "LoRA": "lora", "Softmax": "softmax", "RMSNorm": "rms_norm"}

    def name(self) -> str:
        return self._NAMES[self.kind]

    def output_shape(self, input_shapes: Sequence[Tuple[int, ...]]) -> Tuple[int, ...]:
        """src/graph/operation.rs:74-166; raises ValueError with the reference's messages."""
        k, n = self.kind, len(input_shapes)
        if k == "Input":
            if n == 0:
                raise ValueError("Input operation requires shape")
            return tuple(input_shapes[0])
        if k == "Matmul":
            if n != 2:
                raise ValueError(f"Matmul requires 2 inputs, got {n}")
            a, b = input_shapes
            if len(a) < 2 or len(b) < 2:
                raise ValueError("Matmul requires at least 2D tensors")
            if a[-1] != b[-2]:
                raise ValueError(f"Matmul dimension mismatch: {a[-2]}×{a[-1]} @ {b[-2]}×{b[-1]}")
            return tuple(a[:-2]) + (a[-2], b[-1])
        if k in ("Add", "Mul"):
            if n != 2:
                raise ValueError(f"{self.name()} requires 2 inputs, got {n}")
            if tuple(input_shapes[0]) != tuple(input_shapes[1]):
                raise ValueError(f"Shape mismatch: {list(input_shapes[0])} vs {list(input_shapes[1])}")
            return tuple(input_shapes[0])
        if k == "MulScalar":
            if n != 1:
                raise ValueError(f"MulScalar requires 1 input, got {n}")
            return tuple(input_shapes[0])
        if k == "LoRA":
            if n != 3:
                raise ValueError(f"LoRA requires 3 inputs (input, a, b), got {n}")
            return tuple(input_shapes[0][:-1]) + (input_shapes[2][-1],)
        if n != 1:
            raise ValueError(f"{self.name()} requires 1 input, got {n}")
        return tuple(input_shapes[0])

    def output_dtype(self, input_dtypes: Sequence[torch.dtype]) -> torch.dtype:
        return input_dtypes[0]


@dataclass
class GraphNode:
    """src/graph/node.rs:58-116.  `data` is None while pending (NodeData::Pending)."""
    id: NodeId
    operation: Operation
    inputs: List[NodeId]
    output_shape: Tuple[int, ...]
    output_dtype: torch.dtype
    data: Optional[torch.Tensor] = None

    def is_available(self) -> bool:
        return self.data is not None


class ComputationGraph:
    """src/graph/node.rs:119-345: dense node ids, shape/dtype inference at record time."""

    def __init__(self, device):
        self._device = torch.device(device)
        self.nodes: List[GraphNode] = []
        self.lock = threading.RLock()

    def device(self):
        return self._device

    def __len__(self) -> int:
        return len(self.nodes)

    def is_empty(self) -> bool:
        return not self.nodes

    def get_node(self, nid: NodeId) -> GraphNode:
        if nid.index >= len(self.nodes):
            raise KeyError(f"Node {nid!r} not found")
        return self.nodes[nid.index]

    def add_input(self, tensor: torch.Tensor) -> NodeId:
        nid = NodeId(len(self.nodes))
        self.nodes.append(GraphNode(nid, Operation.Input(), [], tuple(tensor.shape), tensor.dtype, tensor))
        return nid

    def add_node(self, operation: Operation, inputs: List[NodeId]) -> NodeId:
        for i in inputs:
            if i.index >= len(self.nodes):
                raise ValueError(f"Input node {i!r} not found")
        shape = operation.output_shape([self.nodes[i.index].output_shape for i in inputs])
        dtype = operation.output_dtype([self.nodes[i.index].output_dtype for i in inputs])
        nid = NodeId(len(self.nodes))
        self.nodes.append(GraphNode(nid, operation, list(inputs), shape, dtype))
        return nid

    def topological_order(self, output_node: NodeId) -> List[NodeId]:
        """DFS post-order with a cycle check (src/graph/node.rs:229-268); iterative, so deep chains are fine."""
        visited, visiting, order = set(), set(), []
        stack = [(output_node, False)]
        while stack:
            nid, expanded = stack.pop()
            if expanded:
                visiting.discard(nid)
                if nid not in visited:
                    visited.add(nid)
                    order.append(nid)
                continue
            if nid in visited:
                continue
            if nid in visiting:
                raise ValueError(f"Circular dependency detected at node {nid!r}")
            visiting.add(nid)
            stack.append((nid, True))
            for i in reversed(self.get_node(nid).inputs):
                if i not in visited:
                    if i in visiting:
                        raise ValueError(f"Circular dependency detected at node {i!r}")
                    stack.append((i, False))
        return order

    def merge_from(self, other: "ComputationGraph", target: NodeId) -> NodeId:
        """Deep-copies the sub-graph of `target` from `other` with id remapping (src/graph/node.rs:292-345)."""
        id_map: Dict[NodeId, NodeId] = {}
        for nid in other.topological_order(target):
            src = other.get_node(nid)
            new = NodeId(len(self.nodes))
            self.nodes.append(GraphNode(new, src.operation, [id_map[i] for i in src.inputs], src.output_shape,
                                        src.output_dtype, src.data))
            id_map[nid] = new
        return id_map[target]


class AsyncExecutor:
    """src/graph/executor.rs:25-227: one operation at a time, each a kernel launch on the current stream."""

    def __init__(self, device):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise TrainingError("AsyncExecutor needs a CUDA device (this library has no CPU path)")
        self.lib = _lib.init(self.device.index or 0)

    def execute_operation(self, operation: Operation, inputs: Sequence[torch.Tensor]) -> torch.Tensor:
        k, n = operation.kind, len(inputs)
        if k == "Input":
            raise TrainingError("Cannot execute Input operation")
        if k == "Matmul":
            if n != 2:
                raise TrainingError(f"Matmul requires 2 inputs, got {n}")
            return self._matmul(inputs[0], inputs[1])
        if k in ("Add", "Mul"):
            if n != 2:
                raise TrainingError(f"{k} requires 2 inputs, got {n}")
            return self._binary(k, inputs[0], inputs[1])
        if k == "MulScalar":
            if n != 1:
                raise TrainingError(f"MulScalar requires 1 input, got {n}")
            x = inputs[0].contiguous()
            backend._require_cuda(x)
            out = torch.empty_like(x)
            self._check("MulScalar", self.lib.mcb_mul_scalar(x.data_ptr(), out.data_ptr(), x.numel(),
                                                             operation.params["value"], backend._dtype_code(x),
                                                             backend._stream()))
            return out
        if k == "LoRA":
            if n != 3:
                raise TrainingError(f"LoRA requires 3 inputs (input, a, b), got {n}")
            return backend.lora_forward_fused(inputs[0].contiguous(), inputs[1].float().contiguous(),
                                              inputs[2].float().contiguous(), operation.params["scale"])
        if k == "Softmax":
            if n != 1:
                raise TrainingError(f"Softmax requires 1 input, got {n}")
            x, dim = inputs[0], operation.params["dim"]
            if dim >= x.dim():
                raise TrainingError(f"Softmax failed: dimension {dim} out of range for shape {list(x.shape)}")
            if dim == x.dim() - 1:
                return backend.softmax_fused(x.contiguous())
            # the kernel reduces the last dimension: bring `dim` there and back (data movement only)
            xt = x.transpose(dim, -1).contiguous()
            return backend.softmax_fused(xt).transpose(dim, -1).contiguous()
        if k == "RMSNorm":
            if n != 1:
                raise TrainingError(f"RMSNorm requires 1 input, got {n}")
            return backend.rms_norm_fused(inputs[0].contiguous(), operation.params["eps"])
        raise TrainingError(f"unknown operation {k}")

    def _check(self, what: str, rc: int) -> None:
        try:
            _lib.check(rc)
        except _lib.McbError as e:
            raise TrainingError(f"{what} failed: {e}") from e

    def _matmul(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        """Tensor::broadcast_matmul (src/graph/executor.rs:71-82): `a` [..., m, k] times `b` [k, n] or a batch of
        matrices with a's leading dims."""
        backend._require_cuda(a.contiguous(), b.contiguous())
        if a.dim() < 2 or b.dim() < 2 or a.shape[-1] != b.shape[-2]:
            raise TrainingError(f"Matmul failed: shape mismatch {list(a.shape)} @ {list(b.shape)}")
        if a.dtype != b.dtype:
            raise TrainingError("Matmul failed: dtype mismatch")
        a, b = a.contiguous(), b.contiguous()
        K, N = b.shape[-2], b.shape[-1]
        dt = backend._dtype_code(a)
        out = torch.empty(*a.shape[:-1], N, dtype=a.dtype, device=a.device)
        ws = backend.workspace(a.device, self.lib.mcb_matmul_workspace_bytes(K, N, dt))
        if b.dim() == 2:
            M = a.numel() // K
            self._check("Matmul", self.lib.mcb_matmul(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, K, N, dt,
                                                      ws.data_ptr(), ws.numel(), backend._stream()))
            return out
        if tuple(b.shape[:-2]) != tuple(a.shape[:-2]):
            raise TrainingError(f"Matmul failed: batch dims {list(a.shape[:-2])} vs {list(b.shape[:-2])}")
        m = a.shape[-2]
        a3, b3, o3 = a.reshape(-1, m, K), b.reshape(-1, K, N), out.view(-1, m, N)
        for i in range(a3.shape[0]):
            self._check("Matmul", self.lib.mcb_matmul(a3[i].data_ptr(), b3[i].data_ptr(), o3[i].data_ptr(), m, K, N, dt,
                                                      ws.data_ptr(), ws.numel(), backend._stream()))
        return out

    def _binary(self, kind: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        a, b = a.contiguous(), b.contiguous()
        backend._require_cuda(a, b)
        if a.shape != b.shape or a.dtype != b.dtype:
            raise TrainingError(f"{kind} failed: shape mismatch {list(a.shape)} vs {list(b.shape)}")
        out = torch.empty_like(a)
        fn = self.lib.mcb_add if kind == "Add" else self.lib.mcb_mul
        self._check(kind, fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), backend._dtype_code(a), backend._stream()))
        return out

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.device)


class LazyTensor:
    """src/graph/lazy_tensor.rs:36-468."""

    def __init__(self, node_id: NodeId, graph: ComputationGraph, shape, dtype, device):
        self._node_id, self._graph = node_id, graph
        self._shape, self._dtype, self._device = tuple(shape), dtype, torch.device(device)

    # -- constructors --
    @staticmethod
    def from_tensor(tensor: torch.Tensor) -> "LazyTensor":
        graph = ComputationGraph(tensor.device)
        nid = graph.add_input(tensor)
        return LazyTensor(nid, graph, tensor.shape, tensor.dtype, tensor.device)

    @staticmethod
    def from_slice(data, shape, device) -> "LazyTensor":
        t = torch.tensor(list(data), dtype=torch.float32)
        if t.numel() != int(torch.tensor(shape).prod()):
            raise TrainingError(f"shape {list(shape)} does not match {t.numel()} elements")
        return LazyTensor.from_tensor(t.reshape(tuple(shape)).to(device))

    @staticmethod
    def zeros(shape, dtype, device) -> "LazyTensor":
        return LazyTensor.from_tensor(torch.zeros(tuple(shape), dtype=dtype, device=device))

    @staticmethod
    def ones(shape, dtype, device) -> "LazyTensor":
        return LazyTensor.from_tensor(torch.ones(tuple(shape), dtype=dtype, device=device))

    def add_tensor_to_graph(self, tensor: torch.Tensor) -> "LazyTensor":
        with self._graph.lock:
            nid = self._graph.add_input(tensor)
        return LazyTensor(nid, self._graph, tensor.shape, tensor.dtype, tensor.device)

    # -- accessors --
    def shape(self):
        return self._shape

    def dtype(self):
        return self._dtype

    def device(self):
        return self._device

    def node_id(self) -> NodeId:
        return self._node_id

    def graph_size(self) -> int:
        return len(self._graph)

    def is_evaluated(self) -> bool:
        return self._graph.get_node(self._node_id).is_available()

    # -- recording --
    def _merge_graph_from(self, other: "LazyTensor") -> NodeId:
        if other._graph is self._graph:
            return other._node_id
        with self._graph.lock, other._graph.lock:
            return self._graph.merge_from(other._graph, other._node_id)

    def _add_operation(self, operation: Operation, inputs: List[NodeId]) -> "LazyTensor":
        with self._graph.lock:
            try:
                nid = self._graph.add_node(operation, inputs)
            except ValueError as e:
                raise TrainingError(str(e)) from e
            node = self._graph.get_node(nid)
        return LazyTensor(nid, self._graph, node.output_shape, node.output_dtype, self._device)

    def matmul(self, other: "LazyTensor") -> "LazyTensor":
        return self._add_operation(Operation.Matmul(), [self._node_id, self._merge_graph_from(other)])

    def add(self, other: "LazyTensor") -> "LazyTensor":
        return self._add_operation(Operation.Add(), [self._node_id, self._merge_graph_from(other)])

    def mul(self, other: "LazyTensor") -> "LazyTensor":
        return self._add_operation(Operation.Mul(), [self._node_id, self._merge_graph_from(other)])

    def mul_scalar(self, value: float) -> "LazyTensor":
        return self._add_operation(Operation.MulScalar(value), [self._node_id])

    def softmax(self, dim: int) -> "LazyTensor":
        return self._add_operation(Operation.Softmax(dim), [self._node_id])

    def rms_norm(self, eps: float) -> "LazyTensor":
        return self._add_operation(Operation.RMSNorm(eps), [self._node_id])

    def lora_fused(self, lora_a: "LazyTensor", lora_b: "LazyTensor", scale: float) -> "LazyTensor":
        a_id, b_id = self._merge_graph_from(lora_a), self._merge_graph_from(lora_b)
        return self._add_operation(Operation.LoRA(a_id, b_id, scale), [self._node_id, a_id, b_id])

    # -- evaluation --
    def eval(self) -> torch.Tensor:
        """Runs every pending node this tensor depends on, in topological order, and returns the result.
        Kernels are enqueued on the current stream; the call ends with a device synchronisation."""
        g = self._graph
        with g.lock:
            try:
                order = g.topological_order(self._node_id)
            except ValueError as e:
                raise TrainingError(f"Failed to compute execution order: {e}") from e
            executor = AsyncExecutor(self._device)
            for nid in order:
                node = g.get_node(nid)
                if node.is_available():
                    continue
                inputs = []
                for i in node.inputs:
                    src = g.get_node(i)
                    if not src.is_available():
                        raise TrainingError(f"Input not available: node {i!r}")
                    inputs.append(src.data)
                node.data = executor.execute_operation(node.operation, inputs)
            executor.synchronize()
            return g.get_node(self._node_id).data

    def __repr__(self) -> str:
        return f"LazyTensor(node_id={self._node_id!r}, shape={list(self._shape)}, dtype={self._dtype})"


class AsyncGraphExecutor:
    """src/graph/async_executor.rs:32-148: `execute_tensor` evaluates off the calling thread
    (`spawn_blocking` in the reference; a worker thread here) and hands back a future."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._pool = ThreadPoolExecutor(max_workers=1)

    def execute_tensor(self, tensor: LazyTensor) -> Future:
        dev = self.device

        def run():
            if dev.type == "cuda":
                torch.cuda.set_device(dev)
            return tensor.eval()

        return self._pool.submit(run)

    def shutdown(self) -> None:
        self._pool.shutdown(wait=True)
