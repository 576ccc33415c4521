"""CPU oracle of the Qwen-shaped LoRA training step: a torch-CPU restatement of the reference's op
sequence with autograd standing in for candle's.

TEST INFRASTRUCTURE ONLY (tests/, smoke(), and bench.py's CPU-baseline legs).  PARITY UNPINNED by the
reference: no reference test ever trains a model end to end (its trainer tests feed random logits,
tests/training/trainer_test.rs:11-26), so there are no values to pin this against; it is anchored by
following the reference's op order line by line and by torch autograd.

Sequence followed (metal-candle source tree):
  Qwen::forward                    src/models/qwen.rs:236-251   embed -> layers -> norm -> lm_head
  QwenDecoderLayer::forward        src/models/qwen.rs:95-143    pre-norm residual blocks
  RMSNorm::forward                 src/models/qwen.rs:314-325   rms_norm(eps) then * weight
  TensorExt::rms_norm              src/backend/tensor.rs:111-117
  Attention::forward               src/models/transformer.rs:233-286  q/k/v (+bias), RoPE, repeat_kv,
                                   QK^T / sqrt(d), + mask, softmax_stable, PV, o_proj
  RotaryEmbedding                  src/models/transformer.rs:47-120   half-split, f32 tables
  MLP::forward                     src/models/transformer.rs:389-395  silu(gate) * up -> down
  LoRALayer::forward               src/training/lora.rs:323-339       (x A) B * scaling
  cross_entropy_loss               src/training/loss.rs:97-146        ignore index u32::MAX
  AdamW::step / TrainingStep       src/training/optimizer.rs:236-279, src/training/trainer.rs:380-413
Differences from the reference, shared with the CUDA implementation being checked: LoRA deltas are added
to the projections they name, computed from those projections' true inputs (the reference only wires
o_proj/down_proj and feeds them the normed layer input), and a causal mask is always applied (the
reference leaves the mask to its caller).
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import reference_ops as R


def _rms_norm(x, w, eps):
    ms = (x * x).mean(-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * w


def _rope_tables(head_dim, seq_len, theta, dtype):
    inv_freq = torch.tensor([1.0 / np.float32(theta) ** (np.float32(i) / np.float32(head_dim))
                             for i in range(0, head_dim, 2)], dtype=torch.float32)
    pos = torch.arange(seq_len, dtype=torch.float32)
    freqs = pos[:, None] * inv_freq[None, :]
    emb = torch.cat([freqs, freqs], 1)
    return emb.sin().to(dtype), emb.cos().to(dtype)


def _apply_rope(x, sin, cos):
    # x [B, S, H, d]
    d = x.shape[-1]
    s, c = sin[None, :, None, :], cos[None, :, None, :]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    r1 = x1 * c[..., : d // 2] - x2 * s[..., : d // 2]
    r2 = x1 * s[..., d // 2:] + x2 * c[..., d // 2:]
    return torch.cat([r1, r2], -1)


def _repeat_kv(x, n_rep):
    if n_rep == 1:
        return x
    B, Hk, S, d = x.shape
    return x[:, :, None].expand(B, Hk, n_rep, S, d).reshape(B, Hk * n_rep, S, d)


class QwenOracle:
    """weights: dict of numpy/torch arrays named like the checkpoint keys: `embed_tokens`, `norm`, `lm_head`,
    `layers.{i}.{input_layernorm,post_attention_layernorm}`, `layers.{i}.{q,k,v,o,gate,up,down}_proj.weight`
    and `.bias` (q,k,v).  lora: dict `layers.{i}.{module}` -> (A [in,r], B [r,out]); scaling = alpha/rank."""

    def __init__(self, cfg, weights, lora, scaling, dtype=torch.float64):
        self.cfg, self.dtype, self.scaling = cfg, dtype, float(scaling)
        self.w = {k: torch.as_tensor(np.asarray(v, dtype=np.float64) if not torch.is_tensor(v) else v).to(dtype)
                  for k, v in weights.items()}
        self.lora = {k: (torch.as_tensor(a).to(dtype).clone().requires_grad_(True),
                         torch.as_tensor(b).to(dtype).clone().requires_grad_(True)) for k, (a, b) in lora.items()}

    def lora_params(self):
        out = []
        for k in self.lora:
            out += list(self.lora[k])
        return out

    def _proj(self, x, i, name):
        w = self.w[f"layers.{i}.{name}.weight"]
        y = x @ w.T
        b = self.w.get(f"layers.{i}.{name}.bias")
        if b is not None:
            y = y + b
        key = f"layers.{i}.{name}"
        if key in self.lora:
            A, B = self.lora[key]
            y = y + ((x @ A) @ B) * self.scaling
        return y

    def forward(self, ids):
        c = self.cfg
        ids = torch.as_tensor(np.asarray(ids)).long()
        B, S = ids.shape
        Hq, Hk, d = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        h = self.w["embed_tokens"][ids]
        sin, cos = _rope_tables(d, S, c.rope_theta, self.dtype)
        mask = torch.full((S, S), float("-inf"), dtype=self.dtype).triu(1)
        for i in range(c.num_hidden_layers):
            x = _rms_norm(h, self.w[f"layers.{i}.input_layernorm"], c.rms_norm_eps)
            q = self._proj(x, i, "q_proj").reshape(B, S, Hq, d)
            k = self._proj(x, i, "k_proj").reshape(B, S, Hk, d)
            v = self._proj(x, i, "v_proj").reshape(B, S, Hk, d)
            q, k = _apply_rope(q, sin, cos), _apply_rope(k, sin, cos)
            q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
            k, v = _repeat_kv(k, Hq // Hk), _repeat_kv(v, Hq // Hk)
            att = q @ k.transpose(2, 3) / math.sqrt(d)
            att = att + mask
            att = R_softmax(att)
            o = (att @ v).transpose(1, 2).reshape(B, S, Hq * d)
            h = h + self._proj(o, i, "o_proj")
            x = _rms_norm(h, self.w[f"layers.{i}.post_attention_layernorm"], c.rms_norm_eps)
            g = torch.nn.functional.silu(self._proj(x, i, "gate_proj"))
            u = self._proj(x, i, "up_proj")
            h = h + self._proj(g * u, i, "down_proj")
        h = _rms_norm(h, self.w["norm"], c.rms_norm_eps)
        return h @ self.w["lm_head"].T

    def loss(self, ids, targets):
        logits = self.forward(ids)
        V = logits.shape[-1]
        tg = torch.as_tensor(np.asarray(targets).astype(np.int64)).reshape(-1)
        valid = tg != R.IGNORE_INDEX
        logp = torch.log_softmax(logits.reshape(-1, V), 1)
        picked = logp[torch.arange(tg.numel()), torch.where(valid, tg, torch.zeros_like(tg))] * valid
        return -(picked.sum() / valid.sum())

    def loss_and_grads(self, ids, targets):
        for p in self.lora_params():
            p.grad = None
        l = self.loss(ids, targets)
        l.backward()
        return float(l), [p.grad.detach().numpy().copy() for p in self.lora_params()]


def R_softmax(x):
    """softmax_stable (src/backend/tensor.rs:91-98) in torch so autograd can follow it."""
    m = x.max(-1, keepdim=True).values
    e = torch.exp(x - m)
    return e / e.sum(-1, keepdim=True)


def train(oracle: QwenOracle, batches, lr_fn, adamw_cfg=None):
    """The loop of src/training/trainer.rs:368-414 with the shared per-tensor AdamW counter; returns the
    loss per step.  `batches` yields (ids, targets); tensors are visited in adapter order, A before B."""
    opt = R.AdamWOracle(dtype=np.float64 if oracle.dtype == torch.float64 else np.float32, **(adamw_cfg or {}))
    losses = []
    for step, (ids, tg) in enumerate(batches):
        l, grads = oracle.loss_and_grads(ids, tg)
        opt.set_lr(float(lr_fn(step)))
        for i, (p, g) in enumerate(zip(oracle.lora_params(), grads)):
            new = opt.step(f"t{i}", p.detach().numpy(), g)
            with torch.no_grad():
                p.copy_(torch.as_tensor(new))
        losses.append(l)
    return losses
