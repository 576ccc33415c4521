"""Qwen2.5-shaped decoder with LoRA adapters and an explicit training step (forward, loss, backward).

Mirrors the reference's model frame for this path -- `ModelConfig` (src/models/config.rs:25-76),
`Qwen` / `QwenDecoderLayer` (src/models/qwen.rs:20-273), `Attention` / `MLP` / `RotaryEmbedding`
(src/models/transformer.rs:27-396) -- with two deliberate differences: adapters are applied to the
projections they name, on those projections' true inputs (the reference only consults o_proj and
down_proj and feeds them the layer-norm output, src/models/qwen.rs:106-138), and K/V adapters are sized
by the grouped-query width.  There is no autograd: the backward pass is written out and runs the
library's own kernels; the frozen weights get no gradients.

Everything with arithmetic in it is a kernel of libmetal_candle_b200 except the six batched attention
contractions (Q K^T, P V and their reverses): the fused attention kernels of csrc/flash_attn.cu where they apply
(bf16, head_dim 64, sequence a multiple of 128), otherwise plain library GEMMs (torch.bmm -> cuBLAS).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import _lib, backend
from .backend import TrainingError, _ptr, _stream
from .training import LoRAAdapter, LoRALayer, TargetModule


@dataclass
class ModelConfig:
    """The fields of src/models/config.rs:25-64 that the training path reads."""
    vocab_size: int = 151936
    hidden_size: int = 896
    intermediate_size: int = 4864
    num_hidden_layers: int = 24
    num_attention_heads: int = 14
    num_key_value_heads: int = 2
    max_position_embeddings: int = 32768
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0

    @staticmethod
    def qwen25_05b() -> "ModelConfig":
        return ModelConfig()

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def validate(self) -> None:
        if self.hidden_size % self.num_attention_heads != 0:
            raise TrainingError("hidden_size must be divisible by num_attention_heads")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise TrainingError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2 != 0:
            raise TrainingError("head_dim must be even")


class _Linear:
    """A frozen projection: W [out, in] (candle_nn::Linear's layout) plus its [in, out] copy for the
    backward contraction, an optional bias, and an optional LoRA layer."""

    def __init__(self, out_f: int, in_f: int, bias: bool, dtype, device, gen, std=0.02):
        self.weight = (torch.randn(out_f, in_f, device=device, generator=gen) * std).to(dtype).contiguous()
        self.weight_t = backend.transpose_2d(self.weight)
        self.bias = torch.zeros(out_f, dtype=dtype, device=device) if bias else None
        self.lora: Optional[LoRALayer] = None
        self.in_f, self.out_f = in_f, out_f

    def ab(self):
        if self.lora is None:
            return None, None, 1.0
        return self.lora.lora_a, self.lora.lora_b, self.lora.config.scaling()


class CapturedStep:
    """forward_backward of a fixed shape as a CUDA graph (Qwen.capture_forward_backward)."""

    def __init__(self, graph, ids, targets, loss, grads, keepalive=(), count=None):
        self.graph, self.ids, self.targets, self.loss, self.grads = graph, ids, targets, loss, grads
        self.count = count   # int32 [1]: targets of the last replayed batch that were not ignored
        # The graph's kernels carry the ADDRESSES of the scratch buffers that were current at capture time (GEMM
        # operand packs, partial sums, attention and RMSNorm scratch).  The per-device scratch buffer is replaced
        # when a later call needs a larger one; holding the captured ones here keeps their memory from being handed
        # to another tensor while this graph can still be replayed.
        self._keepalive = list(keepalive)

    def __call__(self, input_ids: torch.Tensor, target_ids: torch.Tensor):
        """Copies the batch into the graph's input buffers (device to device, or from pinned host memory) and
        replays; returns (loss, grads) like Qwen.forward_backward - the same tensors on every call."""
        self.ids.copy_(input_ids, non_blocking=True)
        self.targets.copy_(target_ids, non_blocking=True)
        self.graph.replay()
        return self.loss, self.grads


class Qwen:
    """Random-init weights N(0, 0.02^2) for embedding and projections, norm weights 1, biases 0."""

    MODULES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")

    def __init__(self, config: ModelConfig, device, dtype=torch.bfloat16, seed: int = 0):
        config.validate()
        self.config = config
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise TrainingError("Qwen needs a CUDA device (this library has no CPU path)")
        self.dtype = dtype
        self.lib = _lib.init(self.device.index or 0)
        self.dt = backend._dtype_code(torch.empty(0, dtype=dtype))
        c = config
        g = torch.Generator(device=self.device).manual_seed(seed)
        H, I, kv = c.hidden_size, c.intermediate_size, c.kv_size
        self.embed_tokens = (torch.randn(c.vocab_size, H, device=self.device, generator=g) * 0.02).to(dtype)
        self.layers: List[Dict[str, object]] = []
        for _ in range(c.num_hidden_layers):
            L = dict(
                input_layernorm=torch.ones(H, dtype=dtype, device=self.device),
                post_attention_layernorm=torch.ones(H, dtype=dtype, device=self.device),
                q_proj=_Linear(H, H, True, dtype, self.device, g), k_proj=_Linear(kv, H, True, dtype, self.device, g),
                v_proj=_Linear(kv, H, True, dtype, self.device, g), o_proj=_Linear(H, H, False, dtype, self.device, g),
                gate_proj=_Linear(I, H, False, dtype, self.device, g), up_proj=_Linear(I, H, False, dtype, self.device, g),
                down_proj=_Linear(H, I, False, dtype, self.device, g))
            self.layers.append(L)
        self.norm = torch.ones(H, dtype=dtype, device=self.device)
        self.lm_head = _Linear(c.vocab_size, H, False, dtype, self.device, g)
        self.lora_adapter: Optional[LoRAAdapter] = None
        self._grad_flat: Optional[torch.Tensor] = None
        self._grad_views: List[torch.Tensor] = []
        self._grad_slices: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}
        # Tokens per chunk of the lm_head + cross-entropy stage of forward_backward (None: one chunk).  The logits of a
        # chunk are produced, turned into their gradient in place and consumed by the lm_head backward before the
        # next chunk starts, so only [chunk, vocabulary] is ever resident (2.5 GB at 8192 tokens instead of 10 GB for
        # 32768; measured on the 16 x 2048 step: peak 35.7 -> 28.3 GB and 107.9 -> 106.1 ms, 4096 tokens: 27.0 GB, 107.3 ms).
        self.ce_chunk_tokens: Optional[int] = 0    # 0: the library picks it (mcb_ce_chunk_tokens), None: one chunk
        # q, k and v projections of a layer as one fused linear with a block-diagonal rank path (bf16, adapters of
        # equal rank): the normed input is read once and the three input gradients are summed in one pass
        self.fuse_qkv = True
        # SwiGLU backward inside the epilogue of the down projection's input-gradient GEMM (where the library takes it)
        self.fuse_swiglu_bwd = True
        self.layer_done_hook = None  # called as hook(layer_idx) when a layer's LoRA gradients are final
        self.backward_done_hook = None  # called once at the end of forward_backward (joins side-stream work)

    # -- adapter management (Qwen::apply_adapter / remove_adapter, src/models/qwen.rs:150-175) --
    def apply_adapter(self, adapter: LoRAAdapter) -> None:
        c = self.config
        for key, layer in adapter.layers():
            _, idx, module = key.split(".")
            lin: _Linear = self.layers[int(idx)][module]
            if (layer.in_features, layer.out_features) != (lin.in_f, lin.out_f):
                raise TrainingError(f"adapter {key} is {layer.in_features}x{layer.out_features} but the projection is "
                                    f"{lin.in_f}x{lin.out_f} (size K/V adapters with kv_size={c.kv_size})")
            if layer.config.dropout > 0.0:
                raise TrainingError(f"adapter {key} has dropout {layer.config.dropout}: the fused training step applies none "
                                    "(LoRALayer.forward has the reference's unfused dropout branch); use dropout = 0 here")
            lin.lora = layer
        self.lora_adapter = adapter
        n = sum(l.lora_a.numel() + l.lora_b.numel() for _, l in adapter.layers())
        self._grad_flat = torch.zeros(n, dtype=torch.float32, device=self.device)
        self._grad_views, self._grad_slices, off = [], {}, 0
        self._layer_ranges: Dict[int, Tuple[int, int]] = {}
        for key, l in adapter.layers():
            idx = int(key.split(".")[1])
            start = off
            ga = self._grad_flat[off:off + l.lora_a.numel()].view_as(l.lora_a)
            off += l.lora_a.numel()
            gb = self._grad_flat[off:off + l.lora_b.numel()].view_as(l.lora_b)
            off += l.lora_b.numel()
            self._grad_views += [ga, gb]
            self._grad_slices[key] = (ga, gb)
            lo, hi = self._layer_ranges.get(idx, (start, start))
            self._layer_ranges[idx] = (min(lo, start), off)

    def remove_adapter(self) -> None:
        for L in self.layers:
            for m in self.MODULES:
                L[m].lora = None
        self.lora_adapter = None

    def has_adapter(self) -> bool:
        return self.lora_adapter is not None

    def num_layers(self) -> int:
        return self.config.num_hidden_layers

    def grad_flat(self) -> torch.Tensor:
        """All LoRA gradients as one float32 buffer (adapter order: layer, module, A then B)."""
        return self._grad_flat

    def grad_layer_range(self, layer_idx: int) -> Tuple[int, int]:
        return self._layer_ranges[layer_idx]

    # -- thin kernel wrappers --
    def _norm(self, x, w):
        return backend.rms_norm_fused(x, self.config.rms_norm_eps, weight=w)

    def _lin(self, x, lin: _Linear, save: bool, residual=None):
        A, B, s = lin.ab()
        return backend.lora_linear_forward(x, lin.weight, lin.bias, A, B, s, save_hidden=save and A is not None,
                                           residual=residual)

    def _lin_bwd(self, x, lin: _Linear, dy, h_save, key: Optional[str], accumulate: bool, dx_residual=None):
        A, B, s = lin.ab()
        ga = gb = None
        if A is not None:
            ga, gb = self._grad_slices[key]
        dx, _, _ = backend.lora_linear_backward(x, lin.weight_t, A, B, s, dy, h_save=h_save, grad_a=ga, grad_b=gb,
                                                accumulate=accumulate, dx_residual=dx_residual)
        return dx

    def _rope(self, x, heads: int, B: int, S: int, rotate: bool, inverse: bool, pitch: int = 0, offset: int = 0, out=None):
        """Rotary embedding + head relayout.  `pitch` / `offset` place the token-major side inside wider rows (a
        column block of the fused q/k/v buffer); for the inverse direction `out` is that buffer."""
        d = self.config.head_dim
        if out is None:
            out = torch.empty((B, heads, S, d) if not inverse else (B * S, heads * d), dtype=x.dtype, device=x.device)
        _lib.check(self.lib.mcb_rope_relayout_ex(_ptr(x), _ptr(out), B, S, heads, d, float(self.config.rope_theta),
                                                 int(rotate), int(inverse), int(pitch), int(offset), self.dt, _stream()))
        return out

    def _rope_qkv(self, fused, heads_major, B: int, S: int, pitch: int):
        """Rotary embedding + head relayout of the q, k and v column blocks of a fused buffer in one launch.
        `heads_major` None: fused -> (Q, K rotated, V) as [B, heads, S, d]; a (dQ, dK, dV) triple: the reverse
        pass into `fused`."""
        c = self.config
        d, Hq, Hk = c.head_dim, c.num_attention_heads, c.num_key_value_heads
        inverse = heads_major is not None
        if not inverse:
            heads_major = tuple(torch.empty((B, h, S, d), dtype=fused.dtype, device=fused.device) for h in (Hq, Hk, Hk))
        q, k, v = heads_major
        _lib.check(self.lib.mcb_rope_relayout_qkv(_ptr(fused), _ptr(q), _ptr(k), _ptr(v), B, S, Hq, Hk, d, float(c.rope_theta),
                                                  int(inverse), int(pitch), self.dt, _stream()))
        return heads_major

    def _qkv_fused(self, L):
        """The q, k and v projections as one linear (they read the same normed input): the stacked weight [q;k;v]
        in both majors, the stacked bias, and one segment per adapted projection; or None when this does not
        apply (float32, no adapter on any of the three, adapters of different rank or scaling).  Cached per layer
        and rebuilt when a weight or bias tensor has been written to."""
        if self.dtype != torch.bfloat16 or not self.fuse_qkv:
            return None
        lins = [L["q_proj"], L["k_proj"], L["v_proj"]]
        loras = [l.lora for l in lins if l.lora is not None]
        if not loras:
            return None
        r, sc = loras[0].config.rank, loras[0].config.scaling()
        if any(l.config.rank != r or l.config.scaling() != sc for l in loras) or r * len(loras) > 64:
            return None
        ver = tuple((l.weight._version, l.weight.data_ptr(), l.bias._version) for l in lins)
        cached = L.get("_qkv")
        if cached is None or cached[0] != ver:
            w = torch.cat([l.weight for l in lins], 0).contiguous()
            cached = (ver, w, backend.transpose_2d(w), torch.cat([l.bias for l in lins], 0).contiguous())
            L["_qkv"] = cached
        offs, off = [], 0
        for l in lins:
            offs.append(off)
            off += l.out_f
        return dict(w=cached[1], wt=cached[2], bias=cached[3], scale=sc, offsets=offs, width=off, lins=lins)

    def _embed(self, ids32: torch.Tensor) -> torch.Tensor:
        M = ids32.numel()
        out = torch.empty(M, self.config.hidden_size, dtype=self.dtype, device=self.device)
        _lib.check(self.lib.mcb_embedding_fwd(_ptr(ids32), _ptr(self.embed_tokens), _ptr(out), M, self.config.hidden_size,
                                              self.config.vocab_size, self.dt, _stream()))
        return out

    def _gate_up_weight(self, L):
        """The gate and up weights interleaved for `linear_swiglu_forward`, or None when that kernel does not
        apply (an adapter on either projection, float32, or a width that is not a multiple of 128).  Cached per
        layer and rebuilt when either weight tensor has been written to."""
        g, u = L["gate_proj"], L["up_proj"]
        if g.lora is not None or u.lora is not None or self.dtype != torch.bfloat16 or g.out_f % 128 != 0:
            return None
        ver = (g.weight._version, u.weight._version, g.weight.data_ptr(), u.weight.data_ptr())
        cached = L.get("_gate_up")
        if cached is None or cached[0] != ver:
            cached = (ver, backend.interleave_gate_up(g.weight, u.weight))
            L["_gate_up"] = cached
        return cached[1]

    # -- attention core on [B,H,S,d] tensors; grouped-query heads are folded into the row dimension --
    def _attention_fwd(self, Qr, Kr, Vr, B, S):
        """Returns (P, O, lse): the fused kernel (bf16, head_dim 64, S a multiple of 128) keeps only the
        log-sum-exp of each row; other shapes materialise the probabilities P as the reference does."""
        c = self.config
        Hk, G, d = c.num_key_value_heads, c.num_attention_heads // c.num_key_value_heads, c.head_dim
        if backend.attention_supported(Qr, S):
            # the fused kernel writes its output token-major, [B*S, hidden]: the o_proj input as it is
            O, lse = backend.attention_causal_forward(Qr.view(B * Hk, G * S, d), Kr.view(B * Hk, S, d),
                                                      Vr.view(B * Hk, S, d), G, 1.0 / math.sqrt(d), kv_heads=Hk)
            return None, O, lse
        scores = torch.bmm(Qr.view(B * Hk, G * S, d), Kr.view(B * Hk, S, d).transpose(1, 2))  # [B*Hk, G*S, S]
        rows = scores.numel() // S
        _lib.check(self.lib.mcb_softmax_causal_fwd(_ptr(scores), _ptr(scores), rows, S, S, 1.0 / math.sqrt(d), self.dt,
                                                   _stream()))
        O = torch.bmm(scores, Vr.view(B * Hk, S, d))  # [B*Hk, G*S, d] == [B, Hq, S, d]
        return scores, O, None

    def _attention_bwd(self, Qr, Kr, Vr, P, O, lse, dO, B, S):
        c = self.config
        Hk, G, d = c.num_key_value_heads, c.num_attention_heads // c.num_key_value_heads, c.head_dim
        if P is None:
            # fused: O and dO are token-major [B*S, hidden] (o_proj's input and its gradient as they are)
            return backend.attention_causal_backward(Qr.view(B * Hk, G * S, d), Kr.view(B * Hk, S, d),
                                                     Vr.view(B * Hk, S, d), O, lse, dO, G, 1.0 / math.sqrt(d),
                                                     kv_heads=Hk)
        dO3 = dO.view(B * Hk, G * S, d)
        dV = torch.bmm(P.transpose(1, 2), dO3)                       # [B*Hk, S, d], summed over the group
        dP = torch.bmm(dO3, Vr.view(B * Hk, S, d).transpose(1, 2))   # [B*Hk, G*S, S]
        rows = dP.numel() // S
        _lib.check(self.lib.mcb_softmax_causal_bwd(_ptr(P), _ptr(dP), _ptr(dP), rows, S, S, 1.0 / math.sqrt(d), self.dt,
                                                   _stream()))
        dQ = torch.bmm(dP, Kr.view(B * Hk, S, d))                    # [B*Hk, G*S, d]
        dK = torch.bmm(dP.transpose(1, 2), Qr.view(B * Hk, G * S, d))  # [B*Hk, S, d]
        return dQ, dK, dV

    # -- forward --
    def _layer_fwd(self, h, L, B, S, save: bool):
        c = self.config
        n1 = self._norm(h, L["input_layernorm"])
        fq = self._qkv_fused(L)
        hqkv = None
        if fq is not None:
            segs = [dict(A=l.lora.lora_a, B=l.lora.lora_b, offset=o) for l, o in zip(fq["lins"], fq["offsets"]) if l.lora is not None]
            qkv, hqkv = backend.lora_linear_fused_forward(n1, fq["w"], fq["bias"], segs, fq["scale"], save_hidden=save)
            W3, o = fq["width"], fq["offsets"]
            Qr, Kr, Vr = self._rope_qkv(qkv, None, B, S, W3)
            del qkv
            hq = hk = hv = None
        else:
            q, hq = self._lin(n1, L["q_proj"], save)
            k, hk = self._lin(n1, L["k_proj"], save)
            v, hv = self._lin(n1, L["v_proj"], save)
            Qr = self._rope(q, c.num_attention_heads, B, S, True, False)
            Kr = self._rope(k, c.num_key_value_heads, B, S, True, False)
            Vr = self._rope(v, c.num_key_value_heads, B, S, False, False)
            del q, k, v
        P, O, lse = self._attention_fwd(Qr, Kr, Vr, B, S)
        # [M, hidden] for o_proj: the fused kernel's output already is; the unfused one goes through a relayout
        o = O if P is None else self._rope(O, c.num_attention_heads, B, S, False, True)
        O = None   # the fused backward takes the saved o_proj input as the attention output
        h2, ho = self._lin(o, L["o_proj"], save, residual=h)   # residual connection fused into the epilogue
        n2 = self._norm(h2, L["post_attention_layernorm"])
        w_gu = self._gate_up_weight(L)
        if w_gu is not None:
            # gate and up projections and silu(gate) * up from one kernel (no adapters on either)
            gt, up, act = backend.linear_swiglu_forward(n2, w_gu)
            hg = hu = None
        else:
            gt, hg = self._lin(n2, L["gate_proj"], save)
            up, hu = self._lin(n2, L["up_proj"], save)
            act = torch.empty_like(gt)
            _lib.check(self.lib.mcb_swiglu_fwd(_ptr(gt), _ptr(up), _ptr(act), gt.numel(), self.dt, _stream()))
        h3, hd = self._lin(act, L["down_proj"], save, residual=h2)
        if not save:
            return h3, None
        keep_n2 = L["gate_proj"].lora is not None or L["up_proj"].lora is not None
        keep_act = L["down_proj"].lora is not None
        saved = dict(h=h, n1=n1, Qr=Qr, Kr=Kr, Vr=Vr, P=P, O=O, lse=lse, o=o, h2=h2, n2=n2 if keep_n2 else None, gate=gt, up=up,
                     act=act if keep_act else None, hq=hq, hk=hk, hv=hv, ho=ho, hg=hg, hu=hu, hd=hd, hqkv=hqkv)
        return h3, saved

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Qwen::forward (src/models/qwen.rs:236-251) with a causal mask: logits [B, S, vocab]."""
        B, S = input_ids.shape
        h = self._embed(input_ids.to(torch.int32).contiguous().view(-1))
        for L in self.layers:
            h, _ = self._layer_fwd(h, L, B, S, save=False)
        nf = self._norm(h, self.norm)
        logits, _ = self._lin(nf, self.lm_head, False)
        return logits.view(B, S, -1)

    # -- forward + loss + backward --
    def forward_backward(self, input_ids: torch.Tensor, target_ids: torch.Tensor, accumulate: bool = False):
        """One pass of the training step's first three stages (src/training/trainer.rs:380-388): returns
        (loss, grads) with loss a 1-element float32 CUDA tensor (mean next-token cross-entropy over
        targets != u32::MAX) and grads the LoRA gradients in `TrainingStep.collect_trainable_vars` order.
        With accumulate=True the gradients are added to what the buffers hold (micro-batching)."""
        if self.lora_adapter is None:
            raise TrainingError("forward_backward needs an adapter (apply_adapter)")
        c = self.config
        B, S = input_ids.shape
        M = B * S
        ids32 = input_ids.to(torch.int32).contiguous().view(-1)
        tgt32 = target_ids.to(torch.int32).contiguous().view(-1)  # u32::MAX wraps to -1 = ignored
        h = self._embed(ids32)
        saved = []
        for L in self.layers:
            h, sv = self._layer_fwd(h, L, B, S, save=True)
            saved.append(sv)
        nf = self._norm(h, self.norm)
        nll = torch.empty(M, dtype=torch.float32, device=self.device)
        count = torch.empty(1, dtype=torch.int32, device=self.device)
        loss = torch.empty(2, dtype=torch.float32, device=self.device)
        chunk = self.ce_chunk_tokens
        if chunk == 0:
            chunk = int(self.lib.mcb_ce_chunk_tokens(M, c.hidden_size))
        if chunk is None or chunk >= M:
            logits, _ = self._lin(nf, self.lm_head, False)
            _lib.check(self.lib.mcb_cross_entropy(_ptr(logits), _ptr(tgt32), _ptr(nll), _ptr(count), _ptr(loss), M,
                                                  c.vocab_size, 1, self.dt, _stream()))
            dnf = self._lin_bwd(nf, self.lm_head, logits, None, None, False)
            del logits
        else:
            # lm_head, loss and lm_head backward one chunk of tokens at a time (cross_entropy_loss,
            # src/training/loss.rs:58-147, over logits that never exist for the whole batch)
            _lib.check(self.lib.mcb_cross_entropy_count(_ptr(tgt32), _ptr(count), M, c.vocab_size, _stream()))
            dnf = torch.empty_like(nf)
            for c0 in range(0, M, chunk):
                c1 = min(M, c0 + chunk)
                logits, _ = self._lin(nf[c0:c1], self.lm_head, False)
                _lib.check(self.lib.mcb_cross_entropy_chunk(_ptr(logits), _ptr(tgt32[c0:c1]), _ptr(nll[c0:c1]), _ptr(count),
                                                            c1 - c0, c.vocab_size, 1, self.dt, _stream()))
                backend.lora_linear_backward(None, self.lm_head.weight_t, None, None, 1.0, logits, dx_out=dnf[c0:c1])
                del logits
            _lib.check(self.lib.mcb_cross_entropy_finish(_ptr(nll), _ptr(count), _ptr(loss), M, _stream()))
        self.last_count = count
        # backward
        dh, _ = backend.rms_norm_backward(h, self.norm, dnf, c.rms_norm_eps, need_dw=False)
        del dnf
        for idx in range(len(self.layers) - 1, -1, -1):
            dh = self._layer_bwd(dh, self.layers[idx], saved[idx], idx, B, S, accumulate)
            saved[idx] = None
            if self.layer_done_hook is not None:
                self.layer_done_hook(idx)
        if self.backward_done_hook is not None:
            self.backward_done_hook()
        return loss[:1], self._grad_views

    def capture_forward_backward(self, batch: int, seq: int, keep_hooks: bool = False, pool=None) -> "CapturedStep":
        """Records forward_backward for one (batch, seq) shape into a CUDA graph.  The step is some thousand
        short launches; replayed from a graph they run back to back without the host in the loop.  Call it
        after at least one eager forward_backward of the same shape (kernel attributes and cached workspaces
        are set up on first use, which must not happen during capture).  The adapter's tensors are read in
        place, so optimizer updates between replays are seen; inputs go into the returned object's `ids` and
        `targets` buffers.  `keep_hooks` leaves `layer_done_hook` / `backward_done_hook` installed during the
        capture: only for hooks that enqueue stream work which a graph can record (the C-ABI communicator's
        all-reduce on a side stream that forks from and joins the capturing stream), never host-side work.
        `pool` (another capture's `graph.pool()`) lets graphs that are never replayed concurrently share memory."""
        if self.lora_adapter is None:
            raise TrainingError("capture_forward_backward needs an adapter (apply_adapter)")
        ids = torch.zeros(batch, seq, dtype=torch.int32, device=self.device)
        targets = torch.full((batch, seq), -1, dtype=torch.int32, device=self.device)
        hook, done_hook = self.layer_done_hook, self.backward_done_hook
        if not keep_hooks:
            self.layer_done_hook = self.backward_done_hook = None   # no host callbacks inside a graph
        was_profiling = _lib.profile_enabled()
        _lib.profile_enable(False)                                # per-launch events cannot be recorded either
        graph = torch.cuda.CUDAGraph()
        keep = backend.workspace_refs(self.device)   # the scratch buffer the first captured kernels will point at
        try:
            torch.cuda.synchronize(self.device)
            with torch.cuda.graph(graph, pool=pool, capture_error_mode="thread_local"):
                loss, grads = self.forward_backward(ids, targets)
        finally:
            self.layer_done_hook, self.backward_done_hook = hook, done_hook
            _lib.profile_enable(was_profiling)
        return CapturedStep(graph, ids, targets, loss, grads, keepalive=keep + backend.workspace_refs(self.device),
                            count=self.last_count)

    def _layer_bwd(self, dh3, L, sv, idx, B, S, accumulate):
        c = self.config
        key = lambda m: f"layers.{idx}.{m}"
        # MLP
        gt, up = sv["gate"], sv["up"]
        down = L["down_proj"]
        A, Bm, s = down.ab()
        r = 0 if A is None else A.shape[1]
        if self.fuse_swiglu_bwd and backend.lora_linear_backward_swiglu_supported(B * S, c.intermediate_size, c.hidden_size, r,
                                                                                   self.dtype):
            # the SwiGLU backward runs in the epilogue of the down projection's input-gradient GEMM
            ga, gb = self._grad_slices[key("down_proj")] if A is not None else (None, None)
            backend.lora_linear_backward_swiglu(sv["act"], down.weight_t, A, Bm, s, dh3, gt, up, h_save=sv["hd"], grad_a=ga,
                                                grad_b=gb, accumulate=accumulate)
        else:
            dact = self._lin_bwd(sv["act"], down, dh3, sv["hd"], key("down_proj"), accumulate)
            _lib.check(self.lib.mcb_swiglu_bwd(_ptr(gt), _ptr(up), _ptr(dact), _ptr(gt), _ptr(up), gt.numel(), self.dt,
                                               _stream()))  # in place: gate <- d gate, up <- d up
            del dact
        dn2 = self._lin_bwd(sv["n2"], L["gate_proj"], gt, sv["hg"], key("gate_proj"), accumulate)
        dn2 = self._lin_bwd(sv["n2"], L["up_proj"], up, sv["hu"], key("up_proj"), accumulate, dx_residual=dn2)
        # gradient through the norm plus the one along the residual connection, added inside the norm's kernel
        dh2, _ = backend.rms_norm_backward(sv["h2"], L["post_attention_layernorm"], dn2, c.rms_norm_eps, need_dw=False,
                                           dx_residual=dh3)
        # attention
        do = self._lin_bwd(sv["o"], L["o_proj"], dh2, sv["ho"], key("o_proj"), accumulate)
        fused = sv["P"] is None
        dO = do if fused else self._rope(do, c.num_attention_heads, B, S, False, False)
        del do
        dQ, dK, dV = self._attention_bwd(sv["Qr"], sv["Kr"], sv["Vr"], sv["P"], sv["o"] if fused else None, sv["lse"], dO, B, S)
        n1 = sv["n1"]
        fq = self._qkv_fused(L) if sv["hqkv"] is not None else None
        if fq is not None:
            W3, o = fq["width"], fq["offsets"]
            dqkv = torch.empty(B * S, W3, dtype=self.dtype, device=self.device)
            self._rope_qkv(dqkv, (dQ, dK, dV), B, S, W3)
            del dQ, dK, dV, dO
            segs = []
            for l, off, m in zip(fq["lins"], fq["offsets"], ("q_proj", "k_proj", "v_proj")):
                if l.lora is not None:
                    ga, gb = self._grad_slices[key(m)]
                    segs.append(dict(A=l.lora.lora_a, B=l.lora.lora_b, dA=ga, dB=gb, offset=off))
            dn1 = backend.lora_linear_fused_backward(n1, fq["wt"], segs, fq["scale"], dqkv, sv["hqkv"], accumulate=accumulate)
            del dqkv
        else:
            dq = self._rope(dQ, c.num_attention_heads, B, S, True, True)
            dk = self._rope(dK, c.num_key_value_heads, B, S, True, True)
            dv = self._rope(dV, c.num_key_value_heads, B, S, False, True)
            del dQ, dK, dV, dO
            dn1 = self._lin_bwd(n1, L["q_proj"], dq, sv["hq"], key("q_proj"), accumulate)
            dn1 = self._lin_bwd(n1, L["k_proj"], dk, sv["hk"], key("k_proj"), accumulate, dx_residual=dn1)
            dn1 = self._lin_bwd(n1, L["v_proj"], dv, sv["hv"], key("v_proj"), accumulate, dx_residual=dn1)
        dh, _ = backend.rms_norm_backward(sv["h"], L["input_layernorm"], dn1, c.rms_norm_eps, need_dw=False,
                                          dx_residual=dh2)
        return dh
