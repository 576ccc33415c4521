"""CPU oracle: a numpy restatement of the reference's CPU arithmetic for the LoRA hot path.

TEST INFRASTRUCTURE ONLY.  Only tests/, `__graft_entry__.smoke()` and bench.py's CPU-baseline
legs may import this package; the product (metal_candle_b200) never does and fails loudly when
its CUDA library is missing.

What "the reference's CPU implementation" means here.  The reference (GarthDB/metal-candle,
v1.3.0) is Rust on candle-core/candle-nn "0.9" (Cargo.toml:29-31; resolved to 0.9.1 in the
authors' logs, benchmark_results/20251217_125054/fused_lora_bench_run1.txt:2).  Neither a Rust
toolchain nor candle's source is available where this oracle is built, and the Metal shader
cannot run, so the oracle restates (a) the reference's own op *sequences* at its call sites and
(b) the bodies of its Metal kernels as serial loops.  Its fused custom ops have no CPU body
(`cpu_fwd` bails, src/backend/custom_ops.rs:235-245,526-532,719-725): the CPU path is the
unfused candle-op fallback, which is what is followed below.  Backward passes are not in the
reference tree at all (candle autograd is invoked at src/training/trainer.rs:388); the analytic
gradients here are pinned by finite differences and torch-CPU autograd in tests/.

PARITY PINNING: forward ops are pinned against every known-answer value the reference's tests
hold for this path (tests/test_oracle_golden.py lists them with file:line).  Backward, AdamW
values and training curves are UNPINNED by the reference (its tests assert only shape /
non-zero / "changed"), so for those the oracle is anchored by independent derivations only.

Every function takes `dtype` (np.float32 = what candle's CPU device computes in; np.float64 =
the high-precision arbiter used for tolerances).
"""
from __future__ import annotations

import math

import numpy as np

# ------------------------------------------------------------------------------------------
# LoRA
# ------------------------------------------------------------------------------------------


def lora_forward(x, A, B, scaling, dtype=np.float64):
    """LoRA delta `scaling * ((x @ A) @ B)`.

    Follows LoRALayer::forward's fallback, src/training/lora.rs:323 (`input.broadcast_matmul(A)`),
    :336 (`hidden.broadcast_matmul(B)`), :339 (`affine(scaling, 0)`), and equally
    AsyncExecutor::execute_lora's fallback, src/graph/executor.rs:141-158.
    A is [in, r], B is [r, out] (src/training/lora.rs:236-247).  Returns (delta, hidden).
    """
    x = np.asarray(x, dtype=dtype)
    h = x @ np.asarray(A, dtype=dtype)
    o = h @ np.asarray(B, dtype=dtype)
    return (o * dtype(scaling)).astype(dtype), h


def lora_forward_msl(x, A, B, scaling):
    """Serial restatement of the Metal kernel `fused_lora_forward_tiled`
    (src/backend/kernels.metal:108-159): one output element at a time, the rank loop outside the
    in_features loop, float32 accumulators, scale applied last.  Small cases only."""
    x = np.asarray(x, dtype=np.float32)
    A = np.asarray(A, dtype=np.float32)
    B = np.asarray(B, dtype=np.float32)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    M, K = x2.shape
    r, N = B.shape
    out = np.zeros((M, N), dtype=np.float32)
    for m in range(M):
        for o in range(N):
            result = np.float32(0.0)
            for j in range(r):
                hidden = np.float32(0.0)
                for i in range(K):
                    hidden = np.float32(hidden + x2[m, i] * A[i, j])
                result = np.float32(result + hidden * B[j, o])
            out[m, o] = np.float32(result * np.float32(scaling))
    return out.reshape(*lead, N)


def linear(x, W, bias=None, dtype=np.float64):
    """candle_nn::Linear: `x @ W^T (+ b)` with W stored [out, in]
    (created at src/models/transformer.rs:189-192, applied at :241-243,285)."""
    y = np.asarray(x, dtype=dtype) @ np.asarray(W, dtype=dtype).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=dtype)
    return y


def lora_linear_forward(x, W, bias, A, B, scaling, dtype=np.float64):
    """Frozen linear plus LoRA delta, `y = x W^T (+b) + s (x A) B`: the base projection followed by
    the separate add of the adapter output as in src/models/qwen.rs:114-118.  Returns (y, h)."""
    base = linear(x, W, bias, dtype)
    delta, h = lora_forward(x, A, B, scaling, dtype)
    return base + delta, h


def lora_linear_backward(x, W, A, B, scaling, dy, dtype=np.float64):
    """Analytic reverse pass of `lora_linear_forward` with W (and bias) frozen.

    The reference gets these from candle autograd at src/training/trainer.rs:388 over the op
    sequence of src/training/lora.rs:323-339; the chain rule over that sequence gives, with
    g = s*dy and h = x A:   dB = h^T g,  dh = g B^T,  dA = x^T dh,  dx = dy W + dh A^T.
    Returns (dx, dA, dB)."""
    x = np.asarray(x, dtype=dtype)
    W = np.asarray(W, dtype=dtype)
    A = np.asarray(A, dtype=dtype)
    B = np.asarray(B, dtype=dtype)
    dy = np.asarray(dy, dtype=dtype)
    x2 = x.reshape(-1, x.shape[-1])
    dy2 = dy.reshape(-1, dy.shape[-1])
    g = dy2 * dtype(scaling)
    h = x2 @ A
    dB = h.T @ g
    dh = g @ B.T
    dA = x2.T @ dh
    dx = dy2 @ W + dh @ A.T
    return dx.reshape(x.shape), dA, dB


def lora_merge_weights(W, A, B, scaling, dtype=np.float64):
    """LoRAAdapter::merge_weights, src/training/adapter.rs:315-354: `W + s (A B)^T` for W [out, in]."""
    return np.asarray(W, dtype=dtype) + dtype(scaling) * (np.asarray(A, dtype=dtype) @ np.asarray(B, dtype=dtype)).T


# ------------------------------------------------------------------------------------------
# RMSNorm
# ------------------------------------------------------------------------------------------


def rms_norm(x, eps, dtype=np.float64):
    """TensorExt::rms_norm, src/backend/tensor.rs:111-117: sqr -> mean_keepdim(-1) -> +eps -> sqrt ->
    broadcast_div.  No weight (the Metal kernel has none either, kernels.metal:281-330)."""
    x = np.asarray(x, dtype=dtype)
    ms = np.mean(x * x, axis=-1, keepdims=True, dtype=dtype)
    rms = np.sqrt(ms + dtype(eps))
    return x / rms


def rms_norm_msl(x, eps):
    """Serial restatement of the Metal kernel `fused_rms_norm` (kernels.metal:281-330): float32 sum of
    squares, `sqrt(sum/dim + eps)`, then a divide per element."""
    x = np.asarray(x, dtype=np.float32)
    x2 = x.reshape(-1, x.shape[-1])
    out = np.empty_like(x2)
    for i in range(x2.shape[0]):
        acc = np.float32(0.0)
        for v in x2[i]:
            acc = np.float32(acc + v * v)
        rms = np.float32(math.sqrt(np.float32(acc / np.float32(x2.shape[1]) + np.float32(eps))))
        out[i] = x2[i] / rms
    return out.reshape(x.shape)


def rms_norm_weighted(x, w, eps, dtype=np.float64):
    """The model's RMSNorm layer, src/models/qwen.rs:314-325: rms_norm(eps) then broadcast_mul(weight)."""
    return rms_norm(x, eps, dtype) * np.asarray(w, dtype=dtype)


def rms_norm_backward(x, w, eps, dy, dtype=np.float64):
    """Reverse pass of `rms_norm_weighted` (w=None: of `rms_norm`).  With rinv = 1/sqrt(mean(x^2)+eps),
    xh = x*rinv, g = dy*w:   dx = rinv * (g - xh * mean(g*xh)),   dw = sum_rows dy*xh.
    Not in the reference tree (candle autograd).  Returns (dx, dw)."""
    x = np.asarray(x, dtype=dtype)
    dy = np.asarray(dy, dtype=dtype)
    D = x.shape[-1]
    rinv = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True, dtype=dtype) + dtype(eps))
    xh = x * rinv
    g = dy if w is None else dy * np.asarray(w, dtype=dtype)
    dx = rinv * (g - xh * (np.sum(g * xh, axis=-1, keepdims=True, dtype=dtype) / dtype(D)))
    dw = None if w is None else np.sum((dy * xh).reshape(-1, D), axis=0, dtype=dtype)
    return dx, dw


# ------------------------------------------------------------------------------------------
# Softmax
# ------------------------------------------------------------------------------------------


def softmax_stable(x, dtype=np.float64):
    """TensorExt::softmax_stable, src/backend/tensor.rs:91-98: max_keepdim -> broadcast_sub -> exp ->
    sum_keepdim -> broadcast_div over the last dim.  An additive mask is applied by the caller
    beforehand (src/models/transformer.rs:269-273), so -inf arrives in x; exp(-inf - max) = 0."""
    x = np.asarray(x, dtype=dtype)
    m = np.max(x, axis=-1, keepdims=True)
    with np.errstate(invalid="ignore"):
        e = np.exp(x - m)
    s = np.sum(e, axis=-1, keepdims=True, dtype=dtype)
    return e / s


def softmax_msl(x):
    """Serial restatement of the Metal kernel `fused_softmax` (kernels.metal:187-261): max sweep,
    `exp(x-max)` stored to the output while summing in float32, then a divide sweep."""
    x = np.asarray(x, dtype=np.float32)
    x2 = x.reshape(-1, x.shape[-1])
    out = np.empty_like(x2)
    for i in range(x2.shape[0]):
        mx = np.float32(-np.inf)
        for v in x2[i]:
            mx = max(mx, v)
        tot = np.float32(0.0)
        for j, v in enumerate(x2[i]):
            e = np.float32(math.exp(np.float32(v - mx))) if np.isfinite(v) or v > 0 else np.float32(0.0)
            out[i, j] = e
            tot = np.float32(tot + e)
        out[i] = out[i] / tot
    return out.reshape(x.shape)


def softmax_backward(y, dy, dtype=np.float64):
    """Reverse pass of softmax over the last dim: dx = y * (dy - sum_j dy_j y_j).  Not in the
    reference tree (candle autograd)."""
    y = np.asarray(y, dtype=dtype)
    dy = np.asarray(dy, dtype=dtype)
    return y * (dy - np.sum(dy * y, axis=-1, keepdims=True, dtype=dtype))


# ------------------------------------------------------------------------------------------
# AdamW and learning-rate schedules
# ------------------------------------------------------------------------------------------

ADAMW_DEFAULTS = dict(learning_rate=1e-4, beta1=0.9, beta2=0.999, epsilon=1e-8, weight_decay=0.01)
"""AdamWConfig::default, src/training/optimizer.rs:51-61."""


def powi_f32(base: float, n: int) -> np.float32:
    """f32::powi as used at src/training/optimizer.rs:252-255, evaluated by repeated squaring in
    float32 (the exact rounding of Rust's powi is unspecified; float32 square-and-multiply is within
    an ulp or two of it, far inside every tolerance used here)."""
    result = np.float32(1.0)
    b = np.float32(base)
    while n > 0:
        if n & 1:
            result = np.float32(result * b)
        b = np.float32(b * b)
        n >>= 1
    return result


def adamw_step(p, g, m, v, t, lr, beta1, beta2, eps, weight_decay, dtype=np.float32):
    """One AdamW::step for one tensor, src/training/optimizer.rs:236-279, in that order:
    m' = b1 m + (1-b1) g;  v' = b2 v + (1-b2) g^2;  mh = m'/(1-b1^t);  vh = v'/(1-b2^t);
    p' = p - lr * mh/(sqrt(vh)+eps) - (wd*lr) * p.   `t` is the optimizer's counter *after* its
    increment for this call (:236-238).  (1-b), b^t and wd*lr are formed in float32 as the Rust code
    does before widening to f64 scalars.  Returns (p', m', v')."""
    p = np.asarray(p, dtype=dtype)
    g = np.asarray(g, dtype=dtype)
    m = np.asarray(m, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    b1 = np.float32(beta1)
    b2 = np.float32(beta2)
    one_m_b1 = dtype(np.float32(1.0) - b1)
    one_m_b2 = dtype(np.float32(1.0) - b2)
    m_new = m * dtype(b1) + g * one_m_b1
    v_new = v * dtype(b2) + (g * g) * one_m_b2
    # candle evaluates `tensor / f64` as an affine by the reciprocal (third-party candle-core 0.9,
    # not in the reference tree), so the bias corrections are multiplications by 1/(1-b^t).
    inv_bc1 = dtype(1.0 / np.float64(np.float32(1.0) - powi_f32(b1, t)))
    inv_bc2 = dtype(1.0 / np.float64(np.float32(1.0) - powi_f32(b2, t)))
    m_hat = m_new * inv_bc1
    v_hat = v_new * inv_bc2
    update = m_hat / (np.sqrt(v_hat) + dtype(np.float32(eps)))
    lr_update = update * dtype(np.float32(lr))
    wd_update = p * dtype(np.float32(weight_decay) * np.float32(lr))
    p_new = (p - lr_update) - wd_update
    return p_new.astype(dtype), m_new.astype(dtype), v_new.astype(dtype)


class AdamWOracle:
    """AdamW with the reference's state handling: ONE step counter shared by all tensors and bumped
    once per tensor update (src/training/optimizer.rs:172-176,236-238), state created lazily as zeros
    (:298-316).  The reference visits tensors in HashMap order (src/training/trainer.rs:398-402); the
    caller here fixes the order (sorted `layers.{i}.{module}`, A before B)."""

    def __init__(self, dtype=np.float32, **cfg):
        self.cfg = dict(ADAMW_DEFAULTS)
        self.cfg.update(cfg)
        self.state = {}
        self.step_count = 0
        self.dtype = dtype

    def set_lr(self, lr):
        self.cfg["learning_rate"] = lr

    def step(self, name, p, g):
        if name not in self.state:
            self.state[name] = (np.zeros_like(p, dtype=self.dtype), np.zeros_like(p, dtype=self.dtype))
        self.step_count += 1
        m, v = self.state[name]
        c = self.cfg
        p2, m2, v2 = adamw_step(p, g, m, v, self.step_count, c["learning_rate"], c["beta1"], c["beta2"],
                                c["epsilon"], c["weight_decay"], self.dtype)
        self.state[name] = (m2, v2)
        return p2


def lr_constant(step, lr):
    """LRScheduler::Constant, src/training/scheduler.rs:150."""
    return np.float32(lr)


def lr_linear(step, warmup_steps, max_lr):
    """LRScheduler::Linear, src/training/scheduler.rs:152-162 (float32 arithmetic)."""
    if step < warmup_steps:
        return np.float32(np.float32(max_lr) * (np.float32(step) / np.float32(warmup_steps)))
    return np.float32(max_lr)


def lr_cosine(step, total_steps, max_lr, min_lr):
    """LRScheduler::Cosine, src/training/scheduler.rs:164-172."""
    progress = min(np.float32(step) / np.float32(total_steps), np.float32(1.0))
    c = np.float32(math.cos(np.float32(np.float32(math.pi) * progress)))
    return np.float32(np.float32(min_lr) + np.float32(0.5) * (np.float32(max_lr) - np.float32(min_lr)) * (np.float32(1.0) + c))


def lr_warmup_cosine(step, warmup_steps, total_steps, max_lr, min_lr):
    """LRScheduler::WarmupCosine, src/training/scheduler.rs:174-193."""
    if step < warmup_steps:
        return np.float32(np.float32(max_lr) * (np.float32(step) / np.float32(warmup_steps)))
    decay_steps = total_steps - warmup_steps
    progress = min(np.float32(step - warmup_steps) / np.float32(decay_steps), np.float32(1.0))
    c = np.float32(math.cos(np.float32(np.float32(math.pi) * progress)))
    return np.float32(np.float32(min_lr) + np.float32(0.5) * (np.float32(max_lr) - np.float32(min_lr)) * (np.float32(1.0) + c))


# ------------------------------------------------------------------------------------------
# Cross-entropy
# ------------------------------------------------------------------------------------------

IGNORE_INDEX = 0xFFFFFFFF
"""TrainingStep::execute passes Some(u32::MAX), src/training/trainer.rs:385."""


def cross_entropy_loss(logits, targets, ignore_index=IGNORE_INDEX, dtype=np.float64):
    """cross_entropy_loss, src/training/loss.rs:97-146: log_softmax over vocab, gather the target
    log-probability, zero ignored positions, mean over the non-ignored count, negate.
    Returns (loss, dlogits) where dlogits = (softmax - onehot) / count on non-ignored rows."""
    lg = np.asarray(logits, dtype=dtype).reshape(-1, np.asarray(logits).shape[-1])
    tg = np.asarray(targets).reshape(-1).astype(np.int64)
    valid = np.ones_like(tg, dtype=bool) if ignore_index is None else tg != ignore_index
    count = int(valid.sum())
    if count == 0:
        raise ValueError("all tokens are ignored, cannot compute loss")
    mx = lg.max(axis=-1, keepdims=True)
    lse = mx + np.log(np.sum(np.exp(lg - mx), axis=-1, keepdims=True, dtype=dtype))
    logp = lg - lse
    safe_t = np.where(valid, tg, 0)
    picked = logp[np.arange(lg.shape[0]), safe_t] * valid
    loss = -(picked.sum(dtype=dtype) / dtype(count))
    d = np.exp(logp)
    d[np.arange(lg.shape[0]), safe_t] -= 1.0
    d = d * valid[:, None] / dtype(count)
    return dtype(loss), d.reshape(np.asarray(logits).shape)


# ------------------------------------------------------------------------------------------
# Lazy-graph primitives (src/graph/executor.rs:71-120)
# ------------------------------------------------------------------------------------------


def causal_gqa_attention(q, k, v, scale, dtype=np.float64):
    """Attention::forward's core (src/models/transformer.rs:257-285): scores = q k^T * scale, an additive
    causal mask (-inf above the diagonal, as the callers pass it), softmax over keys, times v; grouped-query
    heads share a kv head (the reference repeats k and v, src/models/transformer.rs:260-261,295-310).
    q [nb, G, S, d], k and v [nb, S, d] -> (o [nb, G, S, d], lse [nb, G, S], p [nb, G, S, S])."""
    q, k, v = (np.asarray(t, dtype=dtype) for t in (q, k, v))
    nb, G, S, d = q.shape
    scores = np.einsum("ngsd,ntd->ngst", q, k) * dtype(scale)
    mask = np.triu(np.ones((S, S), dtype=bool), 1)
    scores = np.where(mask, -np.inf, scores)
    m = scores.max(axis=-1, keepdims=True)
    e = np.exp(scores - m)
    l = e.sum(axis=-1, keepdims=True)
    p = e / l
    o = np.einsum("ngst,ntd->ngsd", p, v)
    lse = (m + np.log(l))[..., 0]
    return o, lse, p


def causal_gqa_attention_backward(q, k, v, scale, do, dtype=np.float64):
    """Gradients of `causal_gqa_attention` (the reference gets them from candle's autograd,
    src/training/trainer.rs:388): dv = p^T do, dp = do v^T, ds = p * (dp - rowsum(dp * p)) * scale,
    dq = ds k, dk = ds^T q, with dk and dv summed over the query heads of a group."""
    q, k, v, do = (np.asarray(t, dtype=dtype) for t in (q, k, v, do))
    _, _, p = causal_gqa_attention(q, k, v, scale, dtype)
    dv = np.einsum("ngst,ngsd->ntd", p, do)
    dp = np.einsum("ngsd,ntd->ngst", do, v)
    ds = p * (dp - (dp * p).sum(axis=-1, keepdims=True)) * dtype(scale)
    dq = np.einsum("ngst,ntd->ngsd", ds, k)
    dk = np.einsum("ngst,ngsd->ntd", ds, q)
    return dq, dk, dv


def dropout_mask(n, p, seed, offset=0):
    """The keep mask of the library's dropout (include/mcb200.h, mcb_dropout): element i is kept when the 24 high bits
    of splitmix64(seed ^ (offset + i) * 0x9E3779B97F4A7C15), as a fraction of one, are >= p.  candle_nn::ops::dropout
    (used by src/training/lora.rs:325-330) draws from candle's own generator; only the distribution is shared."""
    with np.errstate(over="ignore"):
        idx = np.uint64(offset) + np.arange(n, dtype=np.uint64)
        z = np.uint64(seed) ^ (idx * np.uint64(0x9E3779B97F4A7C15))
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    u = (z >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    return u >= np.float32(p)


def lora_forward_dropout(x, A, B, scaling, p, seed, offset=0, dtype=np.float64):
    """LoRALayer::forward in training mode with dropout (src/training/lora.rs:312-339): hidden = x A, inverted dropout
    on hidden, hidden B, scaling."""
    h = x.astype(dtype) @ A.astype(dtype)
    keep = dropout_mask(h.size, p, seed, offset).reshape(h.shape)
    h = np.where(keep, h / (1.0 - np.float32(p)).astype(dtype), 0.0)
    return (h @ B.astype(dtype)) * dtype(scaling)


def matmul(a, b, dtype=np.float64):
    """Operation::Matmul -> broadcast_matmul, src/graph/executor.rs:71-82."""
    return np.asarray(a, dtype=dtype) @ np.asarray(b, dtype=dtype)


# ------------------------------------------------------------------------------------------
# Error metric used by every parity test
# ------------------------------------------------------------------------------------------


def max_abs_normalised(got, want) -> float:
    """max|got - want| / max|want| (1 when `want` is all zero and `got` is not)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    den = float(np.max(np.abs(want))) if want.size else 0.0
    num = float(np.max(np.abs(got - want))) if want.size else 0.0
    if den == 0.0:
        return 0.0 if num == 0.0 else 1.0
    return num / den
