"""Host-side mirror of the reference's `src/training` for the LoRA hot path: `LoRAConfig`, `LoRALayer`,
`TargetModule`, `LoRAAdapterConfig`, `LoRAAdapter`, `AdamWConfig`, `AdamW`, `LRScheduler`,
`TrainingConfig`, `StepMetrics`, `TrainingStep`.  Same names, argument meaning, defaults, validation
messages and step/counter semantics; all arithmetic runs in the CUDA kernels behind the C ABI.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

from . import _lib, backend
from .backend import TrainingError


class InvalidConfig(TrainingError):
    """`TrainingError::InvalidConfig { reason }`."""


# ---------------------------------------------------------------------------------------------
# LoRA layer (src/training/lora.rs)
# ---------------------------------------------------------------------------------------------

@dataclass
class LoRAConfig:
    """src/training/lora.rs:50-121; defaults rank 8, alpha 16, dropout 0."""
    rank: int = 8
    alpha: float = 16.0
    dropout: float = 0.0

    def scaling(self) -> float:
        return float(np.float32(self.alpha) / np.float32(self.rank))

    def validate(self) -> None:
        if self.rank == 0:
            raise InvalidConfig("LoRA rank must be greater than 0")
        if self.alpha <= 0.0:
            raise InvalidConfig("LoRA alpha must be positive")
        if not (0.0 <= self.dropout < 1.0):
            raise InvalidConfig("LoRA dropout must be in [0, 1)")


class LoRALayer:
    """A [in, r] ~ N(0, 1/r) and B [r, out] = 0, both float32 and trainable
    (LoRALayer::new, src/training/lora.rs:212-257).  `forward` returns the delta
    `scaling * (x @ A) @ B` (src/training/lora.rs:292-342)."""

    def __init__(self, in_features: int, out_features: int, config: LoRAConfig, device,
                 generator: Optional[torch.Generator] = None):
        config.validate()
        max_rank = min(in_features, out_features)
        if config.rank > max_rank:
            raise InvalidConfig(
                f"LoRA rank {config.rank} exceeds maximum rank {max_rank} "
                f"(min of in_features={in_features}, out_features={out_features})")
        device = torch.device(device)
        if device.type != "cuda":
            raise TrainingError("LoRALayer needs a CUDA device (this library has no CPU path)")
        std = 1.0 / math.sqrt(config.rank)
        self.lora_a = (torch.randn(in_features, config.rank, dtype=torch.float32, device=device, generator=generator)
                       * std).contiguous()
        self.lora_b = torch.zeros(config.rank, out_features, dtype=torch.float32, device=device)
        self.config = LoRAConfig(config.rank, config.alpha, config.dropout)
        self.in_features, self.out_features = in_features, out_features
        self.training = True
        # dropout stream of this layer: mask element i of a call is drawn from (dropout_seed, dropout_offset + i)
        self.dropout_seed, self.dropout_offset, self.last_dropout = 0, 0, None

    # -- accessors (src/training/lora.rs:441-574) --
    def lora_a_tensor(self) -> torch.Tensor:
        return self.lora_a

    def lora_b_tensor(self) -> torch.Tensor:
        return self.lora_b

    def trainable_variables(self) -> List[torch.Tensor]:
        return [self.lora_a, self.lora_b]

    def num_parameters(self) -> int:
        return self.config.rank * (self.in_features + self.out_features)

    def rank(self) -> int:
        return self.config.rank

    def set_training(self, training: bool) -> None:
        self.training = bool(training)

    def eval(self) -> None:
        self.training = False

    def is_training(self) -> bool:
        return self.training

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.training and self.config.dropout > 0.0:
            # LoRALayer::forward's unfused branch (src/training/lora.rs:312-339): hidden = x A, dropout on hidden,
            # hidden B, then the scaling.  float32 throughout (the rank may be any size); the mask of this call covers
            # the elements [dropout_offset, dropout_offset + hidden.numel()) of the layer's stream.
            h = backend.matmul(x.float().contiguous(), self.lora_a)
            self.last_dropout = (self.dropout_seed, self.dropout_offset)
            h = backend.dropout(h, self.config.dropout, self.dropout_seed, self.dropout_offset)
            self.dropout_offset += h.numel()
            return backend.scale(backend.matmul(h, self.lora_b), self.config.scaling()).to(x.dtype)
        return backend.lora_forward_fused(x, self.lora_a, self.lora_b, self.config.scaling())

    def forward_lazy(self, x_lazy):
        """LoRALayer::forward_lazy (src/training/lora.rs:373-397): records one fused LoRA node."""
        graph_a = x_lazy.add_tensor_to_graph(self.lora_a)
        graph_b = x_lazy.add_tensor_to_graph(self.lora_b)
        return x_lazy.lora_fused(graph_a, graph_b, self.config.scaling())


# ---------------------------------------------------------------------------------------------
# Adapter (src/training/adapter.rs)
# ---------------------------------------------------------------------------------------------

class TargetModule(Enum):
    QProj = "q_proj"
    KProj = "k_proj"
    VProj = "v_proj"
    OProj = "o_proj"
    GateProj = "gate_proj"
    UpProj = "up_proj"
    DownProj = "down_proj"

    def name_(self) -> str:
        return self.value

    @staticmethod
    def from_name(name: str) -> Optional["TargetModule"]:
        for m in TargetModule:
            if m.value == name:
                return m
        return None


@dataclass
class LoRAAdapterConfig:
    """src/training/adapter.rs:82-124; default targets are q_proj and v_proj."""
    rank: int = 8
    alpha: float = 16.0
    dropout: float = 0.0
    target_modules: List[TargetModule] = field(default_factory=lambda: [TargetModule.QProj, TargetModule.VProj])

    def to_lora_config(self) -> LoRAConfig:
        return LoRAConfig(self.rank, self.alpha, self.dropout)

    def is_target(self, module: TargetModule) -> bool:
        return module in self.target_modules


class LoRAAdapter:
    """Per-(layer, module) LoRA layers keyed `layers.{i}.{module}` (src/training/adapter.rs:159-300).

    The reference sizes every attention projection hidden x hidden (src/training/adapter.rs:197-201),
    which is wrong for grouped-query K/V; pass `kv_size` (num_kv_heads * head_dim) to size k_proj /
    v_proj by their real output width.  Left at None it reproduces the reference."""

    def __init__(self, hidden_size: int, intermediate_size: int, num_layers: int, config: LoRAAdapterConfig, device,
                 kv_size: Optional[int] = None, generator: Optional[torch.Generator] = None):
        lora_config = config.to_lora_config()
        self._layers: Dict[str, LoRALayer] = {}
        for layer_idx in range(num_layers):
            for target in config.target_modules:
                if target in (TargetModule.QProj, TargetModule.OProj):
                    dims = (hidden_size, hidden_size)
                elif target in (TargetModule.KProj, TargetModule.VProj):
                    dims = (hidden_size, hidden_size if kv_size is None else kv_size)
                elif target in (TargetModule.GateProj, TargetModule.UpProj):
                    dims = (hidden_size, intermediate_size)
                else:
                    dims = (intermediate_size, hidden_size)
                self._layers[f"layers.{layer_idx}.{target.value}"] = LoRALayer(dims[0], dims[1], lora_config, device,
                                                                               generator=generator)
        self._config = config
        self._num_layers = num_layers

    def forward(self, layer_idx: int, module: TargetModule, x: torch.Tensor) -> Optional[torch.Tensor]:
        layer = self._layers.get(f"layers.{layer_idx}.{module.value}")
        return None if layer is None else layer.forward(x)

    def num_trainable_parameters(self) -> int:
        return sum(l.num_parameters() for l in self._layers.values())

    def num_frozen_parameters(self, total_model_params: int) -> int:
        return max(0, total_model_params - self.num_trainable_parameters())

    def config(self) -> LoRAAdapterConfig:
        return self._config

    def num_layers(self) -> int:
        return self._num_layers

    def layers(self) -> Iterable[Tuple[str, LoRALayer]]:
        """Fixed order (layer index, then the config's module order).  The reference iterates a HashMap
        whose order is random per process (src/training/adapter.rs:284-286)."""
        return list(self._layers.items())

    def get_layer(self, layer_idx: int, module: TargetModule) -> Optional[LoRALayer]:
        return self._layers.get(f"layers.{layer_idx}.{module.value}")

    def set_training(self, training: bool) -> None:
        for l in self._layers.values():
            l.set_training(training)

    def eval(self) -> None:
        self.set_training(False)

    def merge_weights(self, base_weight: torch.Tensor, layer_idx: int, module: TargetModule) -> torch.Tensor:
        """`W + scaling * (A @ B)^T` for W [out, in] (src/training/adapter.rs:315-354): a rank-r update of the
        base weight, K * N * r multiply-adds in one element-wise kernel."""
        layer = self.get_layer(layer_idx, module)
        if layer is None:
            return base_weight
        if tuple(base_weight.shape) != (layer.out_features, layer.in_features):
            raise TrainingError(f"merge_weights: base weight {list(base_weight.shape)} does not match the adapter "
                                f"[{layer.out_features}, {layer.in_features}]")
        w = base_weight.contiguous()
        backend._require_cuda(w)
        out = torch.empty_like(w)
        lib = backend._lib_for(w)
        _lib.check(lib.mcb_lora_merge_weights(w.data_ptr(), layer.lora_a.data_ptr(), layer.lora_b.data_ptr(), out.data_ptr(),
                                              layer.in_features, layer.out_features, layer.config.rank,
                                              layer.config.scaling(), backend._dtype_code(w), backend._stream()))
        return out


# ---------------------------------------------------------------------------------------------
# AdamW (src/training/optimizer.rs)
# ---------------------------------------------------------------------------------------------

@dataclass
class AdamWConfig:
    """src/training/optimizer.rs:34-107."""
    learning_rate: float = 1e-4
    beta1: float = 0.9
    beta2: float = 0.999
    epsilon: float = 1e-8
    weight_decay: float = 0.01

    def validate(self) -> None:
        if self.learning_rate <= 0.0:
            raise InvalidConfig("learning rate must be positive")
        if not (0.0 <= self.beta1 < 1.0):
            raise InvalidConfig(f"beta1 must be in [0, 1), got {self.beta1}")
        if not (0.0 <= self.beta2 < 1.0):
            raise InvalidConfig(f"beta2 must be in [0, 1), got {self.beta2}")
        if self.epsilon <= 0.0:
            raise InvalidConfig("epsilon must be positive")
        if self.weight_decay < 0.0:
            raise InvalidConfig("weight decay must be non-negative")


class StateError(TrainingError):
    """`TrainingError::StateError { reason }`."""


class AdamW:
    """AdamW with decoupled weight decay.  ONE step counter is shared by all parameters and advances
    once per tensor update, as in the reference (src/training/optimizer.rs:172-176,236-238).  Parameters
    are float32 CUDA tensors updated in place (`Var::set`, optimizer.rs:313)."""

    def __init__(self, config: Optional[AdamWConfig] = None):
        self.config = AdamWConfig() if config is None else AdamWConfig(**config.__dict__)
        self.config.validate()
        self.state: Dict[object, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.step_count = 0

    def add_parameter(self, name, param: torch.Tensor) -> None:
        self.state[name] = (torch.zeros_like(param, dtype=torch.float32), torch.zeros_like(param, dtype=torch.float32))

    def _key(self, var: torch.Tensor):
        return ("var", var.data_ptr())

    def state_of(self, var: torch.Tensor):
        return self.state[self._key(var)]

    def _launch(self, items, grad_scale: float = 1.0) -> None:
        arr = (_lib.AdamWTensor * len(items))()
        dev = None
        for i, (p, g, m, v, t) in enumerate(items):
            if p.dtype != torch.float32 or g.dtype != torch.float32:
                raise TrainingError("AdamW parameters and gradients must be float32")
            if g.shape != p.shape:
                raise TrainingError(f"gradient shape {list(g.shape)} does not match parameter {list(p.shape)}")
            backend._require_cuda(p, g)
            dev = p.device
            arr[i] = _lib.AdamWTensor(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), t, 0)
        lib = backend._lib_for(items[0][0])
        c = self.config
        _lib.check(lib.mcb_adamw_multi(arr, len(items), c.learning_rate, c.beta1, c.beta2, c.epsilon, c.weight_decay,
                                       float(grad_scale), backend._stream()))

    def step(self, name, param: torch.Tensor, grad: torch.Tensor) -> torch.Tensor:
        """AdamW::step (src/training/optimizer.rs:227-279).  Updates `param` in place and returns it."""
        if name not in self.state:
            raise StateError(f"parameter '{name}' not found in optimizer")
        self.step_count += 1
        m, v = self.state[name]
        self._launch([(param, grad.contiguous(), m, v, self.step_count)])
        return param

    def step_var(self, var: torch.Tensor, grad: torch.Tensor) -> None:
        """AdamW::step_var (src/training/optimizer.rs:298-316): state is created lazily as zeros."""
        key = self._key(var)
        if key not in self.state:
            self.add_parameter(key, var)
        self.step(key, var, grad)

    def step_vars(self, variables: List[torch.Tensor], grads: List[torch.Tensor], grad_scale: float = 1.0) -> None:
        """The loop `for var in vars { step_var(var, grad) }` of src/training/trainer.rs:398-402 as one
        multi-tensor launch: tensor j of this call gets step number step_count + j + 1."""
        items = []
        for var, g in zip(variables, grads):
            key = self._key(var)
            if key not in self.state:
                self.add_parameter(key, var)
            self.step_count += 1
            m, v = self.state[key]
            items.append((var, g.contiguous(), m, v, self.step_count))
        if items:
            self._launch(items, grad_scale)

    def set_lr(self, lr: float) -> None:
        self.config.learning_rate = float(lr)

    def learning_rate(self) -> float:
        return self.config.learning_rate

    def zero_state(self) -> None:
        self.state.clear()
        self.step_count = 0


# ---------------------------------------------------------------------------------------------
# LR schedules (src/training/scheduler.rs)
# ---------------------------------------------------------------------------------------------

class LRScheduler:
    """Constant / Linear / Cosine / WarmupCosine in float32, step 0-indexed
    (src/training/scheduler.rs:29-93,148-195)."""

    def __init__(self, kind: str, **kw):
        self.kind, self.kw = kind, kw

    @staticmethod
    def constant(lr):
        return LRScheduler("constant", lr=lr)

    @staticmethod
    def linear(warmup_steps, max_lr):
        return LRScheduler("linear", warmup_steps=warmup_steps, max_lr=max_lr)

    @staticmethod
    def cosine(total_steps, max_lr, min_lr):
        return LRScheduler("cosine", total_steps=total_steps, max_lr=max_lr, min_lr=min_lr)

    @staticmethod
    def warmup_cosine(warmup_steps, total_steps, max_lr, min_lr):
        return LRScheduler("warmup_cosine", warmup_steps=warmup_steps, total_steps=total_steps, max_lr=max_lr,
                           min_lr=min_lr)

    def get_lr(self, step: int) -> float:
        f = np.float32
        k = self.kw
        if self.kind == "constant":
            return float(f(k["lr"]))
        if self.kind == "linear":
            if step < k["warmup_steps"]:
                return float(f(k["max_lr"]) * (f(step) / f(k["warmup_steps"])))
            return float(f(k["max_lr"]))
        if self.kind == "cosine":
            progress = min(f(step) / f(k["total_steps"]), f(1.0))
            c = f(math.cos(f(f(math.pi) * progress)))
            return float(f(k["min_lr"]) + f(0.5) * (f(k["max_lr"]) - f(k["min_lr"])) * (f(1.0) + c))
        if self.kind == "warmup_cosine":
            if step < k["warmup_steps"]:
                return float(f(k["max_lr"]) * (f(step) / f(k["warmup_steps"])))
            decay_steps = k["total_steps"] - k["warmup_steps"]
            progress = min(f(step - k["warmup_steps"]) / f(decay_steps), f(1.0))
            c = f(math.cos(f(f(math.pi) * progress)))
            return float(f(k["min_lr"]) + f(0.5) * (f(k["max_lr"]) - f(k["min_lr"])) * (f(1.0) + c))
        raise InvalidConfig(f"unknown scheduler {self.kind}")

    def validate(self) -> None:
        """src/training/scheduler.rs:197-290."""
        k = self.kw
        if self.kind == "constant":
            if k["lr"] <= 0:
                raise InvalidConfig("learning rate must be positive")
            return
        if k["max_lr"] <= 0:
            raise InvalidConfig("max_lr must be positive")
        if self.kind in ("linear", "warmup_cosine") and k["warmup_steps"] == 0:
            raise InvalidConfig("warmup_steps must be greater than 0")
        if self.kind in ("cosine", "warmup_cosine"):
            if k["total_steps"] == 0:
                raise InvalidConfig("total_steps must be greater than 0")
            if k["min_lr"] < 0:
                raise InvalidConfig("min_lr must be non-negative")
            if k["min_lr"] >= k["max_lr"]:
                raise InvalidConfig("min_lr must be less than max_lr")
        if self.kind == "warmup_cosine" and k["warmup_steps"] >= k["total_steps"]:
            raise InvalidConfig("warmup_steps must be less than total_steps")


# ---------------------------------------------------------------------------------------------
# Step orchestration (src/training/trainer.rs)
# ---------------------------------------------------------------------------------------------

@dataclass
class TrainingConfig:
    """src/training/trainer.rs:16-39.  `max_grad_norm` is carried but, as in the reference, nothing reads it."""
    num_epochs: int = 3
    lr_scheduler: LRScheduler = field(default_factory=lambda: LRScheduler.constant(1e-4))
    optimizer_config: AdamWConfig = field(default_factory=AdamWConfig)
    max_grad_norm: Optional[float] = 1.0


@dataclass
class StepMetrics:
    """src/training/trainer.rs:264-274."""
    loss: float
    step: int
    learning_rate: float


IGNORE_INDEX = 0xFFFFFFFF  # u32::MAX, what TrainingStep passes (src/training/trainer.rs:385)


def cross_entropy_loss(logits: torch.Tensor, targets: torch.Tensor, ignore_index: Optional[int] = None,
                       return_grad: bool = False):
    """cross_entropy_loss (src/training/loss.rs:58-147): mean over non-ignored tokens of
    -log_softmax(logits)[target].  logits [batch, seq, vocab], targets [batch, seq] integer.  Returns a
    1-element float32 CUDA tensor; with return_grad also d loss / d logits (the logits are left untouched)."""
    ls, ts = tuple(logits.shape), tuple(targets.shape)
    if len(ls) != 3:
        raise InvalidConfig(f"logits must be 3D (batch, seq_len, vocab_size), got shape {list(ls)}")
    if len(ts) != 2:
        raise InvalidConfig(f"targets must be 2D (batch, seq_len), got shape {list(ts)}")
    if ls[0] != ts[0] or ls[1] != ts[1]:
        raise InvalidConfig(f"logits and targets batch/seq_len mismatch: logits {list(ls[:2])} vs targets {list(ts)}")
    backend._require_cuda(logits.contiguous(), targets.contiguous())
    M, V = ls[0] * ls[1], ls[2]
    t = targets.contiguous().view(-1).to(torch.int64)
    if ignore_index is not None:
        t = torch.where(t == ignore_index, torch.full_like(t, -1), t)
    if bool(((t >= V) | ((t < 0) & (t != -1))).any()):
        raise TrainingError(f"target index out of range for vocab size {V}")
    t32 = t.to(torch.int32)
    work = logits.contiguous().clone() if return_grad else logits.contiguous()
    lib = backend._lib_for(work)
    nll = torch.empty(M, dtype=torch.float32, device=work.device)
    count = torch.empty(1, dtype=torch.int32, device=work.device)
    loss = torch.empty(2, dtype=torch.float32, device=work.device)
    _lib.check(lib.mcb_cross_entropy(work.data_ptr(), t32.data_ptr(), nll.data_ptr(), count.data_ptr(), loss.data_ptr(),
                                     M, V, int(return_grad), backend._dtype_code(work), backend._stream()))
    if int(count.item()) == 0:
        raise InvalidConfig("all tokens are ignored, cannot compute loss")
    return (loss[:1], work) if return_grad else loss[:1]


class TrainingStep:
    """One optimisation step: forward, loss, backward, AdamW (src/training/trainer.rs:297-442).

    The reference's `forward_fn` returns logits and candle's autograd walks back through them.  There is
    no autograd here: `forward_backward_fn(input_ids, target_ids)` runs the model's explicit forward and
    backward kernels and returns `(loss, grads)` with `grads[i]` the gradient of variable i of
    `collect_trainable_vars(adapter)`; the loss is the reference's cross-entropy with ignore index
    u32::MAX (trainer.rs:385)."""

    def __init__(self):
        self._step = 0

    @staticmethod
    def collect_trainable_vars(lora_adapter: LoRAAdapter) -> List[torch.Tensor]:
        out: List[torch.Tensor] = []
        for _key, layer in lora_adapter.layers():
            out.extend(layer.trainable_variables())
        return out

    def execute(self, input_ids, target_ids, lora_adapter: LoRAAdapter, optimizer: AdamW, learning_rate: float,
                forward_backward_fn: Callable) -> StepMetrics:
        loss, grads = forward_backward_fn(input_ids, target_ids)
        variables = self.collect_trainable_vars(lora_adapter)
        optimizer.set_lr(learning_rate)
        optimizer.step_vars(variables, grads)
        loss_value = float(loss) if not torch.is_tensor(loss) else float(loss.item())  # host sync, trainer.rs:405
        self._step += 1
        return StepMetrics(loss=loss_value, step=self._step, learning_rate=learning_rate)

    def step(self) -> int:
        return self._step

    def reset(self) -> None:
        self._step = 0


class Trainer:
    """Trainer (src/training/trainer.rs:60-259): owns the adapter, the optimiser and the step counter; `train`
    runs epochs x batches with the configured LR schedule and prints the reference's progress lines.
    `forward_backward_fn` has the contract described at TrainingStep."""

    def __init__(self, hidden_size: int, intermediate_size: int, num_layers: int, lora_config: LoRAAdapterConfig,
                 training_config: TrainingConfig, device, kv_size: Optional[int] = None,
                 generator: Optional[torch.Generator] = None):
        self._lora_adapter = LoRAAdapter(hidden_size, intermediate_size, num_layers, lora_config, device,
                                         kv_size=kv_size, generator=generator)
        self.optimizer = AdamW(training_config.optimizer_config)
        self.config = training_config
        self.training_step = TrainingStep()
        self._global_step = 0

    def train(self, dataset, forward_backward_fn: Callable, verbose: bool = True) -> List[StepMetrics]:
        import time

        say = print if verbose else (lambda *a, **k: None)
        all_metrics: List[StepMetrics] = []
        say("\nStarting LoRA Training")
        say(f"Epochs: {self.config.num_epochs}")
        say(f"Batches per epoch: {len(dataset)}")
        say(f"Total steps: {self.config.num_epochs * len(dataset)}")
        say(f"LoRA trainable params: {self._lora_adapter.num_trainable_parameters()}")
        t_start = time.perf_counter()
        for epoch in range(self.config.num_epochs):
            t_epoch, epoch_loss = time.perf_counter(), 0.0
            say(f"Epoch {epoch + 1}/{self.config.num_epochs}")
            for batch_idx, (input_ids, target_ids) in enumerate(dataset):
                lr = self.config.lr_scheduler.get_lr(self._global_step)
                m = self.training_step.execute(input_ids, target_ids, self._lora_adapter, self.optimizer, lr,
                                               forward_backward_fn)
                epoch_loss += m.loss
                all_metrics.append(m)
                self._global_step += 1
                if (batch_idx + 1) % 10 == 0 or batch_idx + 1 == len(dataset):
                    say(f"  Step {batch_idx + 1}/{len(dataset)} | Loss: {m.loss:.4f} | LR: {m.learning_rate:.6f}")
            say(f"  Epoch {epoch + 1} complete | Avg Loss: {epoch_loss / max(1, len(dataset)):.4f} | "
                f"Time: {time.perf_counter() - t_epoch:.2f}s")
        say(f"Training Complete! Total time: {time.perf_counter() - t_start:.2f}s")
        say(f"Final loss: {all_metrics[-1].loss if all_metrics else 0.0:.4f}")
        return all_metrics

    def lora_adapter(self) -> LoRAAdapter:
        return self._lora_adapter

    def global_step(self) -> int:
        return self._global_step
