"""GPU parity of the Qwen-shaped LoRA training step against the torch-CPU oracle (oracle/qwen_oracle.py).

float32 validation path: loss and LoRA gradients within 1e-4 (max-abs normalised) of the float64 oracle;
bfloat16 production path: within 2e-2 of the float64 oracle run on the bf16-rounded weights.  Loss curves
over 50 optimiser steps with the WarmupCosine schedule agree step by step within the same tolerances.
"""
import numpy as np
import pytest
import torch

from oracle import qwen_oracle as QO
from oracle import reference_ops as R
from oracle import seeded as S

pytestmark = pytest.mark.gpu


def tiny_config():
    from metal_candle_b200.qwen import ModelConfig

    return ModelConfig(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                       rms_norm_eps=1e-6, rope_theta=1.0e6)


def fused_attention_config():
    """head_dim 64 and a sequence of 128: the shapes the fused attention kernels take; an MLP width that is a
    multiple of 128, so that steps without gate/up adapters also take the fused gate/up/SwiGLU kernel."""
    from metal_candle_b200.qwen import ModelConfig

    return ModelConfig(vocab_size=320, hidden_size=256, intermediate_size=384, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                       rms_norm_eps=1e-6, rope_theta=1.0e6)


def build(dev, dtype, targets, rank=4, seed=3, b_std=0.05, cfg=None):
    from metal_candle_b200.qwen import Qwen
    from metal_candle_b200.training import LoRAAdapter, LoRAAdapterConfig, TargetModule

    cfg = tiny_config() if cfg is None else cfg
    model = Qwen(cfg, dev, dtype=dtype, seed=seed)
    g = torch.Generator(device=dev).manual_seed(seed + 1)
    # non-trivial norm weights and biases so those code paths are exercised
    for L in model.layers:
        for k in ("input_layernorm", "post_attention_layernorm"):
            L[k].copy_((1 + 0.1 * torch.randn(cfg.hidden_size, device=dev, generator=g)).to(dtype))
        for m in ("q_proj", "k_proj", "v_proj"):
            L[m].bias.copy_((0.05 * torch.randn(L[m].out_f, device=dev, generator=g)).to(dtype))
        for m in model.MODULES:  # larger weights than 0.02 so that gradients are well above rounding noise
            L[m].weight.copy_((torch.randn(L[m].out_f, L[m].in_f, device=dev, generator=g) / L[m].in_f ** 0.5).to(dtype))
            L[m].weight_t.copy_(L[m].weight.t())
    model.norm.copy_((1 + 0.1 * torch.randn(cfg.hidden_size, device=dev, generator=g)).to(dtype))
    acfg = LoRAAdapterConfig(rank=rank, alpha=2.0 * rank, target_modules=targets)
    adapter = LoRAAdapter(cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers, acfg, dev,
                          kv_size=cfg.kv_size, generator=g)
    for _, l in adapter.layers():
        l.lora_a.mul_(0.3)
        l.lora_b.normal_(0, b_std, generator=g)
    model.apply_adapter(adapter)
    return cfg, model, adapter


def oracle_of(cfg, model, adapter, round_lora_bf16):
    w = {"embed_tokens": model.embed_tokens.float().cpu().numpy(), "norm": model.norm.float().cpu().numpy(),
         "lm_head": model.lm_head.weight.float().cpu().numpy()}
    for i, L in enumerate(model.layers):
        w[f"layers.{i}.input_layernorm"] = L["input_layernorm"].float().cpu().numpy()
        w[f"layers.{i}.post_attention_layernorm"] = L["post_attention_layernorm"].float().cpu().numpy()
        for m in model.MODULES:
            w[f"layers.{i}.{m}.weight"] = L[m].weight.float().cpu().numpy()
            if L[m].bias is not None:
                w[f"layers.{i}.{m}.bias"] = L[m].bias.float().cpu().numpy()
    rnd = (lambda a: S.bf16_round(a)) if round_lora_bf16 else (lambda a: a)
    lora = {k: (rnd(l.lora_a.cpu().numpy()), rnd(l.lora_b.cpu().numpy())) for k, l in adapter.layers()}
    return QO.QwenOracle(cfg, w, lora, adapter.config().to_lora_config().scaling())


def batch(seed, B, Sq, vocab):
    ids = S.token_ids(seed, "ids", (B, Sq), vocab)
    tg = np.concatenate([ids[:, 1:], np.full((B, 1), R.IGNORE_INDEX, dtype=np.int64)], 1)  # next token; last ignored
    return ids, tg


ALL = None


def all_targets():
    from metal_candle_b200.training import TargetModule

    return [TargetModule.QProj, TargetModule.KProj, TargetModule.VProj, TargetModule.OProj, TargetModule.GateProj,
            TargetModule.UpProj, TargetModule.DownProj]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_step_loss_and_gradients(cuda_device, dtype, tol):
    cfg, model, adapter = build(cuda_device, dtype, all_targets())
    ids, tg = batch(5, 2, 64, cfg.vocab_size)
    loss, grads = model.forward_backward(torch.from_numpy(ids).to(cuda_device), torch.from_numpy(tg).to(cuda_device))
    orc = oracle_of(cfg, model, adapter, dtype == torch.bfloat16)
    want_loss, want_grads = orc.loss_and_grads(ids, tg)
    assert abs(float(loss) - want_loss) <= tol * abs(want_loss)
    assert len(grads) == len(want_grads) == 2 * 7 * cfg.num_hidden_layers
    errs = [R.max_abs_normalised(g.cpu().numpy(), w) for g, w in zip(grads, want_grads)]
    names = [f"{k}.{ab}" for k, _ in adapter.layers() for ab in "AB"]
    worst = sorted(zip(errs, names), reverse=True)[:6]
    # Every kernel holds 2e-2 on its own (tests/test_gpu_lora.py, test_gpu_row_ops.py).  Through the whole
    # two-layer chain the attention scores are rounded to bf16 before the softmax (as a bf16 matmul output
    # is in the reference too), which moves the q/k gradients by up to ~3%: the chain bound is 4e-2.
    assert worst[0][0] <= (tol if dtype == torch.float32 else 4e-2), worst
    # logits of the inference path agree with the oracle's forward
    logits = model.forward(torch.from_numpy(ids).to(cuda_device)).float().cpu().numpy()
    assert R.max_abs_normalised(logits, orc.forward(ids).detach().numpy()) <= tol
    from metal_candle_b200 import _lib
    assert _lib.device_status() == 0


@pytest.mark.parametrize("seq", [128, 256])
def test_step_with_fused_attention(cuda_device, seq):
    """bf16, head_dim 64, sequence a multiple of 128: the step runs the fused attention kernels (forward keeps
    only the log-sum-exp, backward recomputes the probabilities).  Loss, logits and LoRA gradients against the
    oracle, same bounds as the unfused chain."""
    cfg, model, adapter = build(cuda_device, torch.bfloat16, all_targets(), cfg=fused_attention_config())
    from metal_candle_b200 import backend as B
    assert B.attention_supported(torch.empty(1, 1, cfg.head_dim, dtype=torch.bfloat16), seq)
    ids, tg = batch(6, 2, seq, cfg.vocab_size)
    loss, grads = model.forward_backward(torch.from_numpy(ids).to(cuda_device), torch.from_numpy(tg).to(cuda_device))
    orc = oracle_of(cfg, model, adapter, True)
    want_loss, want_grads = orc.loss_and_grads(ids, tg)
    assert abs(float(loss) - want_loss) <= 2e-2 * abs(want_loss)
    errs = [R.max_abs_normalised(g.cpu().numpy(), w) for g, w in zip(grads, want_grads)]
    names = [f"{k}.{ab}" for k, _ in adapter.layers() for ab in "AB"]
    worst = sorted(zip(errs, names), reverse=True)[:6]
    assert worst[0][0] <= 4e-2, worst
    logits = model.forward(torch.from_numpy(ids).to(cuda_device)).float().cpu().numpy()
    assert R.max_abs_normalised(logits, orc.forward(ids).detach().numpy()) <= 2e-2
    from metal_candle_b200 import _lib
    assert _lib.device_status() == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_fifty_step_loss_curve(cuda_device, dtype, tol):
    """q_proj/v_proj adapters, rank 4, B = 0 at step 0 as in the reference (src/training/lora.rs:244),
    AdamW lr 1e-3 peak with WarmupCosine(5, 50), 50 steps: identical loss curves within tolerance."""
    from metal_candle_b200.training import AdamW, AdamWConfig, LRScheduler, TargetModule, TrainingStep

    cfg, model, adapter = build(cuda_device, dtype, [TargetModule.QProj, TargetModule.VProj], b_std=0.0)
    orc = oracle_of(cfg, model, adapter, False)
    sched = LRScheduler.warmup_cosine(5, 50, 1e-3, 1e-5)
    batches = [batch(100 + s, 2, 32, cfg.vocab_size) for s in range(50)]
    want = QO.train(orc, batches, sched.get_lr)
    opt, stepper, got = AdamW(AdamWConfig()), TrainingStep(), []
    for s, (ids, tg) in enumerate(batches):
        m = stepper.execute(torch.from_numpy(ids).to(cuda_device), torch.from_numpy(tg).to(cuda_device), adapter, opt,
                            sched.get_lr(s), model.forward_backward)
        got.append(m.loss)
    got, want = np.array(got), np.array(want)
    assert stepper.step() == 50 and opt.step_count == 50 * 2 * 2 * cfg.num_hidden_layers
    assert np.abs(got - want).max() / np.abs(want).max() <= tol, (got[:5], want[:5])
    assert want[-1] < want[0]  # it trains


def test_loss_curve_with_fused_attention(cuda_device):
    """The 50-step curve once more on the shapes that take the fused attention kernels (bf16, head_dim 64,
    128 positions): q_proj/v_proj adapters, B = 0 at step 0, AdamW with WarmupCosine(5, 50)."""
    from metal_candle_b200.training import AdamW, AdamWConfig, LRScheduler, TargetModule, TrainingStep

    cfg, model, adapter = build(cuda_device, torch.bfloat16, [TargetModule.QProj, TargetModule.VProj], b_std=0.0,
                                cfg=fused_attention_config())
    orc = oracle_of(cfg, model, adapter, False)
    sched = LRScheduler.warmup_cosine(5, 50, 1e-3, 1e-5)
    batches = [batch(200 + s, 2, 128, cfg.vocab_size) for s in range(50)]
    want = QO.train(orc, batches, sched.get_lr)
    opt, stepper, got = AdamW(AdamWConfig()), TrainingStep(), []
    for s, (ids, tg) in enumerate(batches):
        m = stepper.execute(torch.from_numpy(ids).to(cuda_device), torch.from_numpy(tg).to(cuda_device), adapter, opt,
                            sched.get_lr(s), model.forward_backward)
        got.append(m.loss)
    got, want = np.array(got), np.array(want)
    assert np.abs(got - want).max() / np.abs(want).max() <= 2e-2, (got[:5], want[:5])
    assert stepper.step() == 50


def test_gradient_accumulation_matches_one_big_batch(cuda_device):
    """Two micro-batches accumulated == one batch of both (how the N-GPU step is checked on one GPU)."""
    from metal_candle_b200.training import TargetModule

    cfg, model, adapter = build(cuda_device, torch.float32, [TargetModule.QProj, TargetModule.VProj])
    ids, tg = batch(9, 4, 32, cfg.vocab_size)
    dev = cuda_device
    _, g_all = model.forward_backward(torch.from_numpy(ids).to(dev), torch.from_numpy(tg).to(dev))
    g_all = [g.clone() for g in g_all]
    model.forward_backward(torch.from_numpy(ids[:2]).to(dev), torch.from_numpy(tg[:2]).to(dev))
    _, g_acc = model.forward_backward(torch.from_numpy(ids[2:]).to(dev), torch.from_numpy(tg[2:]).to(dev), accumulate=True)
    for a, b in zip(g_all, g_acc):
        assert torch.allclose(a, 0.5 * b, rtol=1e-4, atol=1e-7)


def test_captured_step_matches_eager(cuda_device):
    """forward_backward replayed from a CUDA graph gives bit-for-bit the loss and gradients of the eager call
    (the kernels are deterministic), for the capture batch and for a different batch copied in afterwards, and
    sees optimizer updates made between replays."""
    from metal_candle_b200 import _lib
    from metal_candle_b200.training import AdamW, AdamWConfig, TrainingStep

    cfg, model, adapter = build(cuda_device, torch.bfloat16, all_targets(), cfg=fused_attention_config())
    seq = 128
    batches = []
    for seed in (11, 12):
        ids, tg = batch(seed, 2, seq, cfg.vocab_size)
        tg = np.where(tg == R.IGNORE_INDEX, -1, tg)
        batches.append((torch.from_numpy(ids).to(cuda_device).to(torch.int32),
                        torch.from_numpy(tg).to(cuda_device).to(torch.int32)))
    eager = []
    for ids, tg in batches:
        loss, grads = model.forward_backward(ids, tg)
        eager.append((loss.clone(), [g.clone() for g in grads]))
    step = model.capture_forward_backward(2, seq)
    for (ids, tg), (want_loss, want_grads) in zip(batches, eager):
        loss, grads = step(ids, tg)
        torch.cuda.synchronize()
        assert torch.equal(loss, want_loss)
        for g, w in zip(grads, want_grads):
            assert torch.equal(g, w)
    # an optimizer step changes the adapter in place; the next replay must use the new values
    opt = AdamW(AdamWConfig(learning_rate=1e-2))
    opt.step_vars(TrainingStep.collect_trainable_vars(adapter), step.grads)
    want_loss, want_grads = model.forward_backward(*batches[0])
    want_loss, want_grads = want_loss.clone(), [g.clone() for g in want_grads]
    loss, grads = step(*batches[0])
    torch.cuda.synchronize()
    assert torch.equal(loss, want_loss) and not torch.equal(loss, eager[0][0])
    for g, w in zip(grads, want_grads):
        assert torch.equal(g, w)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_chunked_lm_head_and_loss_equal_the_unchunked_step(cuda_device, dtype):
    """forward_backward with the lm_head + cross-entropy stage cut into chunks of tokens (logits of one chunk at a
    time, never the whole [tokens, vocabulary] matrix) gives bit for bit the loss and gradients of the unchunked
    step: every row's logits, loss term and gradient are computed by the same arithmetic either way.  Chunk sizes
    that do not divide the token count, and a chunk of one tile, included; ignored targets fall into several chunks."""
    from metal_candle_b200 import _lib

    cfg, model, adapter = build(cuda_device, dtype, all_targets(), cfg=fused_attention_config())
    ids, tg = batch(21, 3, 128, cfg.vocab_size)
    tg[1, 5:40] = R.IGNORE_INDEX
    ids_d, tg_d = torch.from_numpy(ids).to(cuda_device), torch.from_numpy(tg).to(cuda_device)
    model.ce_chunk_tokens = None
    loss0, g0 = model.forward_backward(ids_d, tg_d)
    loss0, g0 = loss0.clone(), [g.clone() for g in g0]
    for chunk in (128, 100, 383):
        model.ce_chunk_tokens = chunk
        loss1, g1 = model.forward_backward(ids_d, tg_d)
        torch.cuda.synchronize()
        assert torch.equal(loss1, loss0), (chunk, float(loss1), float(loss0))
        for a, b in zip(g1, g0):
            assert torch.equal(a, b), chunk
    # and the oracle agrees (the chunked path is the default for large batches)
    orc = oracle_of(cfg, model, adapter, dtype == torch.bfloat16)
    want_loss, _ = orc.loss_and_grads(ids, tg)
    assert abs(float(loss0) - want_loss) <= (1e-4 if dtype == torch.float32 else 2e-2) * abs(want_loss)
    assert _lib.device_status() == 0


def test_fused_qkv_step_equals_the_separate_projections(cuda_device):
    """The layer's q, k and v projections as one fused linear (the default in bf16) against three separate fused
    LoRA linears: same loss and logits bit for bit (zero blocks of the block-diagonal rank path add nothing), LoRA
    gradients within the bf16 bound of each other (the fused input gradient is summed in one pass, unrounded)."""
    cfg, model, adapter = build(cuda_device, torch.bfloat16, all_targets(), cfg=fused_attention_config())
    ids, tg = batch(31, 2, 128, cfg.vocab_size)
    ids_d, tg_d = torch.from_numpy(ids).to(cuda_device), torch.from_numpy(tg).to(cuda_device)
    assert model.fuse_qkv and model._qkv_fused(model.layers[0]) is not None
    loss1, g1 = model.forward_backward(ids_d, tg_d)
    loss1, g1 = loss1.clone(), [g.clone() for g in g1]
    model.fuse_qkv = False
    loss0, g0 = model.forward_backward(ids_d, tg_d)
    assert torch.equal(loss0, loss1)
    for a, b in zip(g1, g0):
        assert R.max_abs_normalised(a.cpu().numpy(), b.cpu().numpy().astype(np.float64)) <= 2e-2
    model.fuse_qkv = True
