"""Custom-op entry points: the host-side mirror of the reference's `src/backend` for this path.

Names follow the reference: the `CustomMetalOps` trait's three methods become the functions
`lora_forward_fused`, `softmax_fused`, `rms_norm_fused` (src/backend/metal_ops.rs:33-171), and the op
structs `FusedLoRAOp`, `FusedRMSNormOp`, `FusedSoftmaxOp` keep their constructors and validation
(src/backend/custom_ops.rs:73-148,443-470,644-660).  Each call allocates its output through torch
(the reference's ops allocate theirs through the device allocator, custom_ops.rs:395-397), enqueues
the CUDA kernel on torch's current stream through the C ABI, and does not synchronise.

torch is used for device memory and streams only; no arithmetic here runs in torch and nothing falls
back to it: a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import MCB_BF16, MCB_F32, MCB_W_IN_OUT, MCB_W_OUT_IN, McbError


class TrainingError(RuntimeError):
    """Counterpart of `TrainingError::Failed { reason }` (src/error.rs:95-131)."""


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return MCB_F32
    if t.dtype == torch.bfloat16:
        return MCB_BF16
    raise TrainingError(f"unsupported dtype {t.dtype}: the kernels take float32 or bfloat16")


def _require_cuda(*tensors):
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise TrainingError("tensor is not on a CUDA device (this library has no CPU path)")
        if not t.is_contiguous():
            raise TrainingError("tensor must be contiguous")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _lib_for(t: torch.Tensor):
    return _lib.init(t.device.index if t.device.index is not None else torch.cuda.current_device())


_ws_cache = {}


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A per-device scratch buffer that only grows.  The returned view starts on a 1024-byte boundary (the
    bf16 GEMM requires it; torch's allocator only promises 512)."""
    key = (device.type, device.index)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        raw = torch.empty(max(nbytes, 1 << 20) + 1024, dtype=torch.uint8, device=device)
        off = (-raw.data_ptr()) % 1024
        buf = raw[off:off + max(nbytes, 1 << 20)]
        _ws_cache[key] = buf
    return buf


def workspace_refs(device: torch.device):
    """The scratch buffer currently cached for `device` (a list of zero or one tensors).  Whoever bakes its address
    into something replayable (a CUDA graph) keeps these references for as long as that thing lives."""
    buf = _ws_cache.get((device.type, device.index))
    return [] if buf is None else [buf]


# ---------------------------------------------------------------------------------------------
# LoRA
# ---------------------------------------------------------------------------------------------

def _lora_shapes(x, lora_a, lora_b):
    a_dims, b_dims = tuple(lora_a.shape), tuple(lora_b.shape)
    if len(a_dims) != 2 or len(b_dims) != 2:
        raise TrainingError(f"LoRA matrices must be 2D, got shapes {list(a_dims)} and {list(b_dims)}")
    if a_dims[1] != b_dims[0]:
        raise TrainingError(
            f"Incompatible LoRA matrix dimensions: {a_dims[0]}×{a_dims[1]} and {b_dims[0]}×{b_dims[1]}")
    if x.dim() == 0:
        raise TrainingError("Input must have at least 1 dimension")
    if x.shape[-1] != a_dims[0]:
        raise TrainingError(f"Input feature dimension mismatch: expected {a_dims[0]}, got {x.shape[-1]}")
    if lora_a.dtype != torch.float32 or lora_b.dtype != torch.float32:
        raise TrainingError(
            f"LoRA matrices are float32 master copies (got {lora_a.dtype} and {lora_b.dtype}); the bf16 path rounds them itself")
    K, r = a_dims
    N = b_dims[1]
    M = x.numel() // K
    return M, K, N, r


class FusedLoRAOp:
    """`out = scaling * (x @ A) @ B` in one kernel launch sequence; FusedLoRAOp::new's checks
    (src/backend/custom_ops.rs:118-148)."""

    def __init__(self, lora_a: torch.Tensor, lora_b: torch.Tensor, scaling: float):
        a_dims, b_dims = tuple(lora_a.shape), tuple(lora_b.shape)
        if len(a_dims) != 2 or len(b_dims) != 2:
            raise TrainingError(f"LoRA matrices must be 2D, got shapes {list(a_dims)} and {list(b_dims)}")
        if a_dims[1] != b_dims[0]:
            raise TrainingError(
                f"Incompatible LoRA matrix dimensions: {a_dims[0]}×{a_dims[1]} and {b_dims[0]}×{b_dims[1]}")
        self.lora_a, self.lora_b, self.scaling = lora_a, lora_b, float(scaling)

    def name(self) -> str:
        return "fused-lora"

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return lora_forward_fused(x, self.lora_a, self.lora_b, self.scaling)


def lora_forward_fused(x: torch.Tensor, lora_a: torch.Tensor, lora_b: torch.Tensor, scaling: float) -> torch.Tensor:
    """CustomMetalOps::lora_forward_fused (src/backend/metal_ops.rs:126-144).  A, B are float32."""
    M, K, N, r = _lora_shapes(x, lora_a, lora_b)
    _require_cuda(x, lora_a, lora_b)
    lib = _lib_for(x)
    dt = _dtype_code(x)
    out = torch.empty(*x.shape[:-1], N, dtype=x.dtype, device=x.device)
    nws = lib.mcb_lora_workspace_bytes(M, K, N, r, dt)
    ws = workspace(x.device, nws)
    try:
        _lib.check(lib.mcb_lora_delta_fwd(_ptr(x), _ptr(lora_a), _ptr(lora_b), _ptr(out), M, K, N, r, float(scaling),
                                          dt, _ptr(ws), ws.numel(), _stream()))
    except McbError as e:
        raise TrainingError(f"Failed to apply fused LoRA op: {e}") from e
    return out


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """`a` [..., k] times `b` [k, n] (Tensor::broadcast_matmul with a 2-D right operand)."""
    _require_cuda(a, b)
    if b.dim() != 2 or a.shape[-1] != b.shape[0] or a.dtype != b.dtype:
        raise TrainingError(f"matmul: {list(a.shape)} @ {list(b.shape)} ({a.dtype}, {b.dtype})")
    a, b = a.contiguous(), b.contiguous()
    K, N = b.shape
    lib, dt = _lib_for(a), _dtype_code(a)
    out = torch.empty(*a.shape[:-1], N, dtype=a.dtype, device=a.device)
    ws = workspace(a.device, lib.mcb_matmul_workspace_bytes(K, N, dt))
    _lib.check(lib.mcb_matmul(_ptr(a), _ptr(b), _ptr(out), a.numel() // K, K, N, dt, _ptr(ws), ws.numel(), _stream()))
    return out


def dropout(x: torch.Tensor, p: float, seed: int, offset: int = 0) -> torch.Tensor:
    """Inverted dropout with the library's counter-based mask over (seed, offset + element index); applied to the
    upstream gradient with the same arguments it is its own backward."""
    _require_cuda(x)
    x = x.contiguous()
    out = torch.empty_like(x)
    _lib.check(_lib_for(x).mcb_dropout(_ptr(x), _ptr(out), x.numel(), float(p), int(seed) & 0xFFFFFFFFFFFFFFFF,
                                       int(offset) & 0xFFFFFFFFFFFFFFFF, _dtype_code(x), _stream()))
    return out


def scale(x: torch.Tensor, value: float) -> torch.Tensor:
    _require_cuda(x)
    x = x.contiguous()
    out = torch.empty_like(x)
    _lib.check(_lib_for(x).mcb_mul_scalar(_ptr(x), _ptr(out), x.numel(), float(value), _dtype_code(x), _stream()))
    return out


def lora_linear_forward(x, weight, bias, lora_a, lora_b, scaling, save_hidden=True, residual=None):
    """`y = x W^T (+b) + scaling (x A) B` with W [out, in].  Returns (y, h_save or None); h_save is
    `scaling * (x A)` transposed, [rank padded to 16, tokens padded to 64]."""
    K = x.shape[-1]
    N = weight.shape[0]
    if weight.dim() != 2 or weight.shape[1] != K:
        raise TrainingError(f"weight must be [out, in={K}], got {list(weight.shape)}")
    r = 0 if lora_a is None else lora_a.shape[1]
    if r:
        _lora_shapes(x, lora_a, lora_b)
        if lora_b.shape[1] != N:
            raise TrainingError(f"LoRA B must be [r, out={N}], got {list(lora_b.shape)}")
    _require_cuda(x, weight, bias, lora_a, lora_b, residual)
    M = x.numel() // K
    lib = _lib_for(x)
    dt = _dtype_code(x)
    y = torch.empty(*x.shape[:-1], N, dtype=x.dtype, device=x.device)
    h = None
    if r and save_hidden:
        h = torch.empty(lib.mcb_lora_rank_padded(r), lib.mcb_lora_h_pitch(M), dtype=x.dtype, device=x.device)
    nws = lib.mcb_lora_workspace_bytes(M, K, N, r, dt)
    ws = workspace(x.device, nws)
    _lib.check(lib.mcb_lora_linear_fwd_ex(_ptr(x), _ptr(weight), _ptr(bias), _ptr(lora_a), _ptr(lora_b), _ptr(residual),
                                          _ptr(y), _ptr(h), M, K, N, r, float(scaling), dt, MCB_W_OUT_IN, _ptr(ws),
                                          ws.numel(), _stream()))
    return y, h


def lora_linear_backward(x, weight_t, lora_a, lora_b, scaling, dy, h_save=None, need_dx=True, grad_a=None,
                         grad_b=None, accumulate=False, weight_layout=MCB_W_IN_OUT, dx_residual=None, dx_out=None):
    """Reverse of `lora_linear_forward`.  `weight_t` is the [in, out] copy of the frozen weight (for
    float32 either layout works, say which with `weight_layout`).  Returns (dx, dA, dB)."""
    N = dy.shape[-1]
    K = weight_t.shape[0] if weight_layout == MCB_W_IN_OUT else weight_t.shape[1]
    r = 0 if lora_a is None else lora_a.shape[1]
    if r and x is None:
        raise TrainingError("lora_linear_backward: the layer input x is needed for the LoRA gradients")
    _require_cuda(x, weight_t, lora_a, lora_b, dy, h_save, grad_a, grad_b, dx_residual)
    M = dy.numel() // N
    lib = _lib_for(dy)
    dt = _dtype_code(dy)
    dx = None
    if need_dx:
        if dx_out is not None:
            if tuple(dx_out.shape) != (*dy.shape[:-1], K) or dx_out.dtype != dy.dtype or not dx_out.is_contiguous():
                raise TrainingError(f"lora_linear_backward: dx_out must be a contiguous {list((*dy.shape[:-1], K))} {dy.dtype} tensor")
            dx = dx_out
        else:
            dx = torch.empty(*dy.shape[:-1], K, dtype=dy.dtype, device=dy.device)
    if r and grad_a is None:
        grad_a = torch.empty(K, r, dtype=torch.float32, device=dy.device)
        grad_b = torch.empty(r, N, dtype=torch.float32, device=dy.device)
        accumulate = False
    nws = lib.mcb_lora_workspace_bytes(M, K, N, r, dt)
    ws = workspace(dy.device, nws)
    _lib.check(lib.mcb_lora_linear_bwd_ex(_ptr(x), _ptr(weight_t), _ptr(lora_a), _ptr(lora_b), _ptr(dy), _ptr(h_save),
                                       _ptr(dx_residual), _ptr(dx), _ptr(grad_a), _ptr(grad_b), int(bool(accumulate)), M, K, N, r,
                                       float(scaling), dt, weight_layout, _ptr(ws), ws.numel(), _stream()))
    return dx, grad_a, grad_b


def lora_linear_backward_swiglu_supported(M: int, K: int, N: int, r: int, dtype=torch.bfloat16) -> bool:
    """Whether `lora_linear_backward_swiglu` takes a down projection of K inputs, N outputs and rank r over M tokens."""
    if dtype != torch.bfloat16:
        return False
    return bool(_lib.load().mcb_lora_linear_bwd_swiglu_supported(int(M), int(K), int(N), int(r), MCB_BF16))


def lora_linear_backward_swiglu(x, weight_t, lora_a, lora_b, scaling, dy, gate, up, h_save=None, grad_a=None, grad_b=None,
                                accumulate=False):
    """Backward of the down projection of a SwiGLU MLP with the SwiGLU backward in the GEMM's epilogue: `gate` and
    `up` [.., K] (the saved pre-activations) are overwritten with their gradients; the gradient of the activation
    itself is never stored.  `weight_t` is the [in, out] copy of the frozen weight.  Returns (dA, dB)."""
    N = dy.shape[-1]
    K = weight_t.shape[0]
    r = 0 if lora_a is None else lora_a.shape[1]
    if r and x is None:
        raise TrainingError("lora_linear_backward_swiglu: the layer input x is needed for the LoRA gradients")
    _require_cuda(x, weight_t, lora_a, lora_b, dy, h_save, grad_a, grad_b, gate, up)
    M = dy.numel() // N
    for name, t in (("gate", gate), ("up", up)):
        if t.numel() != M * K or t.dtype != dy.dtype or not t.is_contiguous():
            raise TrainingError(f"lora_linear_backward_swiglu: {name} must be a contiguous [{M}, {K}] {dy.dtype} tensor")
    lib = _lib_for(dy)
    dt = _dtype_code(dy)
    if r and grad_a is None:
        grad_a = torch.empty(K, r, dtype=torch.float32, device=dy.device)
        grad_b = torch.empty(r, N, dtype=torch.float32, device=dy.device)
        accumulate = False
    nws = lib.mcb_lora_workspace_bytes(M, K, N, r, dt)
    ws = workspace(dy.device, nws)
    _lib.check(lib.mcb_lora_linear_bwd_swiglu(_ptr(x), _ptr(weight_t), _ptr(lora_a), _ptr(lora_b), _ptr(dy), _ptr(h_save),
                                           _ptr(gate), _ptr(up), _ptr(grad_a), _ptr(grad_b), int(bool(accumulate)), M, K, N, r,
                                           float(scaling), dt, MCB_W_IN_OUT, _ptr(ws), ws.numel(), _stream()))
    return grad_a, grad_b


def _segment_table(segments, with_grads: bool):
    arr = (_lib.LoraSegment * len(segments))()
    for i, sg in enumerate(segments):
        a, b = sg["A"], sg["B"]
        arr[i] = _lib.LoraSegment(a.data_ptr(), b.data_ptr(), sg["dA"].data_ptr() if with_grads else None,
                                  sg["dB"].data_ptr() if with_grads else None, int(sg["offset"]), int(b.shape[1]))
    return arr


def _check_segments(segments, K: int):
    if not segments:
        raise TrainingError("fused LoRA linear: no segments")
    r = segments[0]["A"].shape[1]
    for sg in segments:
        a, b = sg["A"], sg["B"]
        if a.dim() != 2 or b.dim() != 2 or a.shape != (K, r) or b.shape[0] != r:
            raise TrainingError(f"fused LoRA linear: every segment needs A [{K}, {r}] and B [{r}, n] "
                                f"(got {list(a.shape)} and {list(b.shape)})")
        if a.dtype != torch.float32 or b.dtype != torch.float32:
            raise TrainingError("fused LoRA linear: LoRA matrices are float32 master copies")
        _require_cuda(a, b, sg.get("dA"), sg.get("dB"))
    return r


def lora_linear_fused_forward(x, weight_cat, bias_cat, segments, scaling, save_hidden=True):
    """Several projections of the same input as one linear: `weight_cat` [N, K] stacks their weights, segment i =
    dict(A=[K,r], B=[r,n_i], offset=first output column) is the adapter of columns [offset, offset + n_i).  Returns
    (y [.., N], h_save): the rank paths run as one block-diagonal update.  bfloat16 only."""
    K, N = x.shape[-1], weight_cat.shape[0]
    if weight_cat.dim() != 2 or weight_cat.shape[1] != K:
        raise TrainingError(f"weight must be [out, in={K}], got {list(weight_cat.shape)}")
    r = _check_segments(segments, K)
    _require_cuda(x, weight_cat, bias_cat)
    M = x.numel() // K
    lib = _lib_for(x)
    dt = _dtype_code(x)
    y = torch.empty(*x.shape[:-1], N, dtype=x.dtype, device=x.device)
    h = torch.empty(lib.mcb_lora_rank_padded(r * len(segments)), lib.mcb_lora_h_pitch(M), dtype=x.dtype, device=x.device)
    ws = workspace(x.device, lib.mcb_lora_fused_workspace_bytes(M, K, N, r, len(segments), dt))
    _lib.check(lib.mcb_lora_linear_fused_fwd(_ptr(x), _ptr(weight_cat), _ptr(bias_cat), _segment_table(segments, False),
                                             len(segments), _ptr(y), _ptr(h), M, K, N, r, float(scaling), dt, _ptr(ws),
                                             ws.numel(), _stream()))
    return y, (h if save_hidden else None)


def lora_linear_fused_backward(x, weight_cat_t, segments, scaling, dy, h_save, accumulate=False, dx_residual=None):
    """Reverse of `lora_linear_fused_forward`: dx, and every segment's gradients written (accumulate: added) into
    its `dA` [K,r] / `dB` [r,n] tensors.  `weight_cat_t` is the [in, out] copy of the stacked weight."""
    N = dy.shape[-1]
    K = weight_cat_t.shape[0]
    r = _check_segments(segments, K)
    _require_cuda(x, weight_cat_t, dy, h_save, dx_residual)
    M = dy.numel() // N
    lib = _lib_for(dy)
    dt = _dtype_code(dy)
    dx = torch.empty(*dy.shape[:-1], K, dtype=dy.dtype, device=dy.device)
    ws = workspace(dy.device, lib.mcb_lora_fused_workspace_bytes(M, K, N, r, len(segments), dt))
    _lib.check(lib.mcb_lora_linear_fused_bwd(_ptr(x), _ptr(weight_cat_t), _segment_table(segments, True), len(segments),
                                             _ptr(dy), _ptr(h_save), _ptr(dx_residual), _ptr(dx), int(bool(accumulate)), M, K, N,
                                             r, float(scaling), dt, _ptr(ws), ws.numel(), _stream()))
    return dx


def transpose_2d(src: torch.Tensor) -> torch.Tensor:
    _require_cuda(src)
    if src.dim() != 2:
        raise TrainingError("transpose_2d takes a matrix")
    lib = _lib_for(src)
    dst = torch.empty(src.shape[1], src.shape[0], dtype=src.dtype, device=src.device)
    _lib.check(lib.mcb_transpose_2d(_ptr(src), _ptr(dst), src.shape[0], src.shape[1], _dtype_code(src), _stream()))
    return dst


# ---------------------------------------------------------------------------------------------
# gate / up projections + SwiGLU in one kernel
# ---------------------------------------------------------------------------------------------

def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[2F, K] weight for `linear_swiglu_forward`: blocks of 128 gate rows alternate with the same 128 up rows."""
    F, K = w_gate.shape
    if w_up.shape != w_gate.shape or F % 128 != 0:
        raise TrainingError(f"gate/up weights {list(w_gate.shape)} / {list(w_up.shape)}: equal shapes with a multiple of 128 rows")
    return torch.stack([w_gate.view(F // 128, 128, K), w_up.view(F // 128, 128, K)], dim=1).reshape(2 * F, K).contiguous()


def linear_swiglu_forward(x: torch.Tensor, w_gate_up: torch.Tensor):
    """MLP::forward's first half (src/models/transformer.rs:389-395): returns (gate, up, silu(gate) * up)."""
    _require_cuda(x, w_gate_up)
    K = x.shape[-1]
    F = w_gate_up.shape[0] // 2
    if w_gate_up.shape[1] != K:
        raise TrainingError(f"interleaved gate/up weight must be [2F, {K}], got {list(w_gate_up.shape)}")
    M = x.numel() // K
    lib = _lib_for(x)
    gate, up, act = (torch.empty(*x.shape[:-1], F, dtype=x.dtype, device=x.device) for _ in range(3))
    _lib.check(lib.mcb_linear_swiglu_fwd(_ptr(x), _ptr(w_gate_up), _ptr(gate), _ptr(up), _ptr(act), M, K, F, _dtype_code(x),
                                         _stream()))
    return gate, up, act


# ---------------------------------------------------------------------------------------------
# fused causal attention
# ---------------------------------------------------------------------------------------------

def attention_supported(q: torch.Tensor, seq: int) -> bool:
    """Shapes the fused attention kernels are built for (others use the unfused sequence)."""
    return q.dtype == torch.bfloat16 and q.shape[-1] == 64 and seq % 128 == 0


def attention_causal_forward(q, k, v, groups: int, scale: float, kv_heads: int = 0):
    """Attention::forward's core (src/models/transformer.rs:257-285) in one kernel.  q [nb, groups*S, d]
    (row g*S + s), k and v [nb, S, d].  Returns (o, lse [nb, groups*S] float32); o is laid out like q, or, with
    kv_heads > 0 (nb = batch*kv_heads), token-major [batch*S, kv_heads*groups*d] - the o_proj input as it is."""
    _require_cuda(q, k, v)
    nb, S, d = k.shape
    if q.shape != (nb, groups * S, d) or v.shape != k.shape:
        raise TrainingError(f"attention: q {list(q.shape)}, k {list(k.shape)}, v {list(v.shape)} do not fit groups={groups}")
    if kv_heads and nb % kv_heads != 0:
        raise TrainingError(f"attention: nb={nb} is not a multiple of kv_heads={kv_heads}")
    lib = _lib_for(q)
    o = (torch.empty((nb // kv_heads) * S, kv_heads * groups * d, dtype=q.dtype, device=q.device) if kv_heads
         else torch.empty_like(q))
    lse = torch.empty(nb, groups * S, dtype=torch.float32, device=q.device)
    ws = workspace(q.device, lib.mcb_attention_workspace_bytes(nb, groups, S, d))
    _lib.check(lib.mcb_attention_causal_fwd_ex(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), nb, groups, S, d, float(scale),
                                               _dtype_code(q), int(kv_heads), int(bool(kv_heads)), _ptr(ws), ws.numel(),
                                               _stream()))
    return o, lse


def attention_causal_backward(q, k, v, o, lse, dout, groups: int, scale: float, kv_heads: int = 0):
    """Gradients of `attention_causal_forward`: (dq like q, dk and dv like k, summed over the group).  With
    kv_heads > 0, o and dout are token-major as returned by the forward."""
    _require_cuda(q, k, v, o, lse, dout)
    nb, S, d = k.shape
    want = ((nb // kv_heads) * S, kv_heads * groups * d) if kv_heads else tuple(q.shape)
    if tuple(o.shape) != want or tuple(dout.shape) != want:
        raise TrainingError(f"attention backward: o {list(o.shape)} / dout {list(dout.shape)}, expected {list(want)}")
    lib = _lib_for(q)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws = workspace(q.device, lib.mcb_attention_workspace_bytes(nb, groups, S, d))
    _lib.check(lib.mcb_attention_causal_bwd_ex(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(dout), _ptr(lse), _ptr(dq), _ptr(dk),
                                               _ptr(dv), nb, groups, S, d, float(scale), _dtype_code(q), int(kv_heads),
                                               int(bool(kv_heads)), _ptr(ws), ws.numel(), _stream()))
    return dq, dk, dv


# ---------------------------------------------------------------------------------------------
# RMSNorm
# ---------------------------------------------------------------------------------------------

class FusedRMSNormOp:
    """FusedRMSNormOp::new (src/backend/custom_ops.rs:443-470): `x / sqrt(mean(x^2) + eps)`."""

    def __init__(self, eps: float):
        self.eps = float(eps)

    def name(self) -> str:
        return "fused-rms-norm"

    def __call__(self, x):
        return rms_norm_fused(x, self.eps)


def _rows(x: torch.Tensor, what: str):
    if x.dim() == 0:
        raise TrainingError(f"Input tensor for {what} must have at least 1 dimension, got []")
    D = x.shape[-1]
    if D == 0 or x.numel() == 0:
        raise TrainingError(f"{what}: empty tensor")
    return x.numel() // D, D


def rms_norm_fused(x: torch.Tensor, eps: float, weight: torch.Tensor | None = None, return_rstd: bool = False):
    """CustomMetalOps::rms_norm_fused (src/backend/metal_ops.rs:160-170).  The reference's op accepts
    1-3-D input (src/backend/custom_ops.rs:550-558); any rank is accepted here, rows = product of the
    leading dims.  `weight` folds in the model layer's multiply (src/models/qwen.rs:314-325)."""
    rows, D = _rows(x, "FusedRMSNormOp")
    _require_cuda(x, weight)
    if weight is not None and (weight.shape != (D,) or weight.dtype != x.dtype):
        raise TrainingError(f"RMSNorm weight must be [{D}] of {x.dtype}")
    lib = _lib_for(x)
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if return_rstd else None
    try:
        _lib.check(lib.mcb_rmsnorm_fwd(_ptr(x), _ptr(weight), _ptr(y), _ptr(rstd), rows, D, float(eps), _dtype_code(x),
                                       _stream()))
    except McbError as e:
        raise TrainingError(f"Fused RMS Norm kernel execution failed: {e}") from e
    return (y, rstd) if return_rstd else y


def rms_norm_backward(x, weight, dy, eps, need_dw=True, grad_w=None, accumulate=False, dx_residual=None):
    """dx (and dw) of rms_norm_fused.  `dx_residual`, if given, is added to dx inside the kernel (the gradient that
    reaches the same tensor along the residual connection)."""
    rows, D = _rows(x, "rms_norm_backward")
    _require_cuda(x, weight, dy, grad_w, dx_residual)
    lib = _lib_for(x)
    if dx_residual is not None:
        if dx_residual.shape != x.shape or dx_residual.dtype != x.dtype or not dx_residual.is_contiguous():
            raise ValueError("rms_norm_backward: dx_residual must match x in shape, dtype and be contiguous")
        dx = torch.empty_like(x)   # (the kernel could write over dx_residual; shapes it declines could not)
    else:
        dx = torch.empty_like(x)
    if need_dw and grad_w is None:
        grad_w = torch.empty(D, dtype=torch.float32, device=x.device)
        accumulate = False
    nws = lib.mcb_rmsnorm_bwd_workspace_bytes(rows, D) if need_dw else 0
    ws = workspace(x.device, nws)
    if dx_residual is not None:
        _lib.check(lib.mcb_rmsnorm_bwd_ex(_ptr(x), _ptr(weight), _ptr(dy), _ptr(dx_residual), _ptr(dx),
                                          _ptr(grad_w) if need_dw else None, int(bool(accumulate)), rows, D, float(eps),
                                          _dtype_code(x), _ptr(ws), ws.numel(), _stream()))
    else:
        _lib.check(lib.mcb_rmsnorm_bwd(_ptr(x), _ptr(weight), _ptr(dy), _ptr(dx), _ptr(grad_w) if need_dw else None,
                                       int(bool(accumulate)), rows, D, float(eps), _dtype_code(x), _ptr(ws), ws.numel(),
                                       _stream()))
    return dx, (grad_w if need_dw else None)


# ---------------------------------------------------------------------------------------------
# softmax
# ---------------------------------------------------------------------------------------------

class FusedSoftmaxOp:
    """FusedSoftmaxOp::new (src/backend/custom_ops.rs:644-660): softmax over the last dimension."""

    def name(self) -> str:
        return "fused-softmax"

    def __call__(self, x):
        return softmax_fused(x)


def softmax_fused(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """CustomMetalOps::softmax_fused (src/backend/metal_ops.rs:146-158).  Any rank (the reference's op
    stops at 3-D, src/backend/custom_ops.rs:743-751, which makes the model's 4-D scores fall back)."""
    rows, D = _rows(x, "FusedSoftmaxOp")
    _require_cuda(x, out)
    lib = _lib_for(x)
    y = torch.empty_like(x) if out is None else out
    try:
        _lib.check(lib.mcb_softmax_fwd(_ptr(x), _ptr(y), rows, D, _dtype_code(x), _stream()))
    except McbError as e:
        raise TrainingError(f"Fused Softmax kernel execution failed: {e}") from e
    return y


def softmax_backward(y: torch.Tensor, dy: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    rows, D = _rows(y, "softmax_backward")
    _require_cuda(y, dy, out)
    lib = _lib_for(y)
    dx = torch.empty_like(y) if out is None else out
    _lib.check(lib.mcb_softmax_bwd(_ptr(y), _ptr(dy), _ptr(dx), rows, D, _dtype_code(y), _stream()))
    return dx
