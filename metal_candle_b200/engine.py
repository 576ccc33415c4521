"""The training step through the C-ABI engine (`mcb_qwen_*`, include/mcb200.h): what a non-Python host calls.

`QwenEngine` wraps an existing `Qwen` model: it hands the engine the model's weight tensors and the adapter's
parameter and gradient tensors (nothing is copied except what the engine derives once: transposed weights, the
stacked q/k/v weight, the interleaved gate/up weight), allocates the one arena the engine works in, and exposes
`forward_backward` / `adamw_step` / `train_step` with the signatures of `Qwen.forward_backward` and `AdamW`.  The
engine issues the same kernels in the same order as the Python step, so the two agree bit for bit.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from . import _lib
from .backend import TrainingError
from .qwen import Qwen

MODULE_INDEX = {"q_proj": 0, "k_proj": 1, "v_proj": 2, "o_proj": 3, "gate_proj": 4, "up_proj": 5, "down_proj": 6}


class QwenEngine:
    def __init__(self, model: Qwen, batch: int, seq: int):
        if model.lora_adapter is None:
            raise TrainingError("QwenEngine needs a model with an adapter (apply_adapter)")
        if model.dtype != torch.bfloat16:
            raise TrainingError("QwenEngine runs the bfloat16 production path only")
        self.model, self.batch, self.seq = model, batch, seq
        self.lib = _lib.init(model.device.index or 0)
        c = model.config
        self._cfg = _lib.QwenConfig(c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers,
                                    c.num_attention_heads, c.num_key_value_heads, c.rms_norm_eps, c.rope_theta)
        n_layers = c.num_hidden_layers
        self._layers = (_lib.QwenLayer * n_layers)()
        for i, L in enumerate(model.layers):
            ly = self._layers[i]
            ly.input_layernorm = L["input_layernorm"].data_ptr()
            ly.post_attention_layernorm = L["post_attention_layernorm"].data_ptr()
            for name, m in MODULE_INDEX.items():
                ly.weight[m] = L[name].weight.data_ptr()
            for j, name in enumerate(("q_proj", "k_proj", "v_proj")):
                ly.bias[j] = L[name].bias.data_ptr() if L[name].bias is not None else None
        self._weights = _lib.QwenWeights(model.embed_tokens.data_ptr(), model.norm.data_ptr(), model.lm_head.weight.data_ptr(),
                                         self._layers)
        entries = list(model.lora_adapter.layers())
        ranks = {l.config.rank for _, l in entries}
        scales = {l.config.scaling() for _, l in entries}
        if len(ranks) != 1 or len(scales) != 1:
            raise TrainingError("QwenEngine needs one rank and one scaling for all adapters")
        self.rank, self.scale = ranks.pop(), scales.pop()
        self._entries = (_lib.QwenAdapterEntry * len(entries))()
        for i, (key, layer) in enumerate(entries):
            _, idx, module = key.split(".")
            ga, gb = model._grad_slices[key]
            self._entries[i] = _lib.QwenAdapterEntry(int(idx), MODULE_INDEX[module], layer.lora_a.data_ptr(), layer.lora_b.data_ptr(),
                                                     ga.data_ptr(), gb.data_ptr())
        nbytes = self.lib.mcb_qwen_arena_bytes(C.byref(self._cfg), self._entries, len(entries), self.rank, batch, seq)
        if nbytes == 0:
            raise TrainingError(f"mcb_qwen_arena_bytes: {self.lib.mcb_last_error().decode()}")
        raw = torch.empty(nbytes + 1024, dtype=torch.uint8, device=model.device)
        off = (-raw.data_ptr()) % 1024
        self._arena = raw[off:off + nbytes]
        self._h = C.c_void_p(None)
        _lib.check(self.lib.mcb_qwen_create(C.byref(self._h), C.byref(self._cfg), C.byref(self._weights), self._entries, len(entries),
                                            self.rank, float(self.scale), self._arena.data_ptr(), nbytes,
                                            torch.cuda.current_stream().cuda_stream))
        self._loss = torch.zeros(2, dtype=torch.float32, device=model.device)
        self._keep = []   # tensors handed to set_exchange

    @property
    def arena_bytes(self) -> int:
        return self._arena.numel()

    def set_ce_chunk(self, tokens: int) -> None:
        _lib.check(self.lib.mcb_qwen_set_ce_chunk(self._h, int(tokens)))

    def set_exchange(self, comm, side_stream: Optional[torch.cuda.Stream], buckets) -> None:
        """`buckets`: list of (first_layer, lo, hi) element ranges of the model's flat gradient buffer; `comm` a
        `metal_candle_b200.comm.Communicator` (None switches the exchange off)."""
        if comm is None:
            _lib.check(self.lib.mcb_qwen_set_exchange(self._h, None, None, None, None, None, None, 0))
            return
        n = len(buckets)
        lo = (C.c_int64 * n)(*[b[1] for b in buckets])
        hi = (C.c_int64 * n)(*[b[2] for b in buckets])
        first = (C.c_int * n)(*[b[0] for b in buckets])
        self._keep = [comm, side_stream]
        _lib.check(self.lib.mcb_qwen_set_exchange(self._h, comm._h, side_stream.cuda_stream, self.model.grad_flat().data_ptr(), lo, hi,
                                                  first, n))

    def _check_batch(self, ids, targets):
        if ids.dtype != torch.int32 or targets.dtype != torch.int32 or not ids.is_cuda or not targets.is_cuda:
            raise TrainingError("QwenEngine takes int32 CUDA tensors of token ids and targets (ignored positions: -1)")
        if ids.shape != targets.shape or ids.dim() != 2 or not ids.is_contiguous() or not targets.is_contiguous():
            raise TrainingError("QwenEngine: ids and targets must be contiguous [batch, seq] tensors of one shape")
        B, S = ids.shape
        if B * S > self.batch * self.seq:
            raise TrainingError(f"QwenEngine was sized for {self.batch} x {self.seq} tokens, got {B} x {S}")
        return B, S

    def forward_backward(self, ids: torch.Tensor, targets: torch.Tensor, accumulate: bool = False):
        """Like `Qwen.forward_backward`: (loss [1] float32 on the device, the LoRA gradients in adapter order)."""
        B, S = self._check_batch(ids, targets)
        _lib.check(self.lib.mcb_qwen_forward_backward(self._h, ids.data_ptr(), targets.data_ptr(), B, S, int(bool(accumulate)),
                                                      self._loss.data_ptr(), torch.cuda.current_stream().cuda_stream))
        return self._loss[:1], self.model._grad_views

    def adamw_step(self, lr: float, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, grad_scale=1.0) -> None:
        _lib.check(self.lib.mcb_qwen_adamw_step(self._h, float(lr), beta1, beta2, eps, weight_decay, float(grad_scale),
                                                torch.cuda.current_stream().cuda_stream))

    def train_step(self, ids, targets, lr: float, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, grad_scale=1.0):
        B, S = self._check_batch(ids, targets)
        _lib.check(self.lib.mcb_qwen_train_step(self._h, ids.data_ptr(), targets.data_ptr(), B, S, float(lr), beta1, beta2, eps,
                                                weight_decay, float(grad_scale), self._loss.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream))
        return self._loss[:1]

    def info(self) -> dict:
        steps, pers, cnt = C.c_int64(0), C.c_int64(0), C.c_void_p(None)
        _lib.check(self.lib.mcb_qwen_info(self._h, C.byref(steps), C.byref(pers), C.byref(cnt)))
        return {"adamw_steps": steps.value, "persistent_bytes": pers.value}

    def destroy(self) -> None:
        if self._h:
            h, self._h = self._h, C.c_void_p(None)
            self.lib.mcb_qwen_destroy(h)

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass
