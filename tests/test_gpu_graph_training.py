"""GPU tests of the lazy graph, the executor, cross-entropy, the adapter and the trainer, modelled on the
reference's tests/lora_lazy.rs, softmax_lazy.rs, rmsnorm_lazy.rs, lazy_execution.rs, executor_direct.rs,
async_execution.rs, training/trainer_test.rs and the inline tests of src/training/{adapter,loss}.rs."""
import numpy as np
import pytest
import torch

from oracle import reference_ops as R
from oracle import seeded as S

pytestmark = pytest.mark.gpu


def back(t):
    return t.detach().float().cpu().numpy()


def test_lazy_known_answers(cuda_device):
    from metal_candle_b200.graph import LazyTensor

    dev = cuda_device
    # tests/lazy_execution.rs:54-74
    a = LazyTensor.from_slice([1, 2, 3, 4, 5, 6], (2, 3), dev)
    b = LazyTensor.from_slice([1, 2, 3, 4, 5, 6], (3, 2), dev)
    assert np.array_equal(back(a.matmul(b).eval()), [[22, 28], [49, 64]])
    # tests/lazy_execution.rs:33-51: (a + b) * 2
    x = LazyTensor.from_slice([1, 2, 3], (3,), dev)
    y = LazyTensor.from_slice([4, 5, 6], (3,), dev)
    z = x.add(y).mul_scalar(2.0)
    assert not z.is_evaluated()
    assert np.array_equal(back(z.eval()), [10, 14, 18]) and z.is_evaluated()
    assert np.array_equal(back(x.mul(y).eval()), [4, 10, 18])
    # tests/executor_direct.rs:480-496 and tests/softmax_lazy.rs:137-169 through the graph
    assert np.allclose(back(LazyTensor.from_slice([3, 4], (1, 2), dev).rms_norm(0.0).eval()), [[0.8485, 1.1314]], atol=1e-3)
    sm = back(LazyTensor.from_slice([100, 200, 300, 400], (1, 4), dev).softmax(1).eval())
    assert np.isfinite(sm).all() and abs(sm.sum() - 1) < 1e-5 and sm[0, 3] > 0.99


@pytest.mark.parametrize("rank", [2, 4, 8, 16])
def test_lora_lazy_equals_eager(cuda_device, rank):
    """tests/lora_lazy.rs:16-110: lazy == eager within 1e-4, shape known before eval, chains."""
    from metal_candle_b200.graph import LazyTensor
    from metal_candle_b200.training import LoRAConfig, LoRALayer

    g = torch.Generator(device=cuda_device).manual_seed(rank)
    layer = LoRALayer(64, 48, LoRAConfig(rank=rank, alpha=2.0 * rank), cuda_device, generator=g)
    layer.lora_b.normal_(0, 0.05, generator=g)
    x = torch.randn(2, 16, 64, device=cuda_device, generator=g)
    lazy = layer.forward_lazy(LazyTensor.from_tensor(x))
    assert lazy.shape() == (2, 16, 48)
    eager = layer.forward(x)
    assert np.abs(back(lazy.eval()) - back(eager)).max() < 1e-4
    want, _ = R.lora_forward(back(x), back(layer.lora_a), back(layer.lora_b), 2.0)
    assert np.abs(back(eager) - want).max() < 1e-4
    # chained: two layers then a scale
    l2 = LoRALayer(48, 32, LoRAConfig(rank=rank, alpha=2.0 * rank), cuda_device, generator=g)
    l2.lora_b.normal_(0, 0.05, generator=g)
    chain = l2.forward_lazy(layer.forward_lazy(LazyTensor.from_tensor(x))).mul_scalar(0.5)
    w2, _ = R.lora_forward(want, back(l2.lora_a), back(l2.lora_b), 2.0)
    assert np.abs(back(chain.eval()) - 0.5 * w2).max() < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lazy_softmax_rmsnorm_matmul(cuda_device, dtype):
    from metal_candle_b200.graph import LazyTensor

    tol = 1e-4 if dtype == torch.float32 else 2e-2
    x = S.normal(4, "x", (3, 8, 64))
    w = S.normal(4, "w", (64, 32)) / 8
    if dtype == torch.bfloat16:
        x, w = S.bf16_round(x), S.bf16_round(w)
    xt = torch.from_numpy(x).to(cuda_device).to(dtype)
    wt = torch.from_numpy(w).to(cuda_device).to(dtype)
    lx = LazyTensor.from_tensor(xt)
    assert R.max_abs_normalised(back(lx.softmax(2).eval()), R.softmax_stable(x)) <= tol
    # a non-last dimension is moved to the end and back
    want1 = np.moveaxis(R.softmax_stable(np.moveaxis(x, 1, -1)), -1, 1)
    assert R.max_abs_normalised(back(lx.softmax(1).eval()), want1) <= tol
    assert R.max_abs_normalised(back(lx.rms_norm(1e-5).eval()), R.rms_norm(x, 1e-5)) <= tol
    y = lx.matmul(lx.add_tensor_to_graph(wt))
    assert y.shape() == (3, 8, 32)
    assert R.max_abs_normalised(back(y.eval()), x.astype(np.float64) @ w.astype(np.float64)) <= tol
    # batched right operand (same leading dims)
    wb = torch.from_numpy(np.stack([w, 2 * w, 3 * w])).to(cuda_device).to(dtype)
    yb = lx.matmul(lx.add_tensor_to_graph(wb)).eval()
    wantb = np.stack([x[i].astype(np.float64) @ (w * (i + 1)).astype(np.float64) for i in range(3)])
    assert R.max_abs_normalised(back(yb), wantb) <= tol


def test_executor_direct_errors_and_async(cuda_device):
    """tests/executor_direct.rs (arity errors with the reference's message substrings),
    tests/async_execution.rs."""
    from metal_candle_b200.backend import TrainingError
    from metal_candle_b200.graph import AsyncExecutor, AsyncGraphExecutor, LazyTensor, NodeId, Operation

    ex = AsyncExecutor(cuda_device)
    t = torch.ones(2, 2, device=cuda_device)
    for op, ins, msg in ((Operation.Input(), [], "Cannot execute Input operation"),
                         (Operation.Matmul(), [t], "Matmul requires 2 inputs, got 1"),
                         (Operation.Add(), [t, t, t], "Add requires 2 inputs, got 3"),
                         (Operation.Mul(), [t], "Mul requires 2 inputs, got 1"),
                         (Operation.MulScalar(2.0), [], "MulScalar requires 1 input, got 0"),
                         (Operation.LoRA(NodeId(0), NodeId(1), 1.0), [t, t], r"LoRA requires 3 inputs \(input, a, b\), got 2"),
                         (Operation.Softmax(1), [t, t], "Softmax requires 1 input, got 2"),
                         (Operation.RMSNorm(1e-5), [], "RMSNorm requires 1 input, got 0")):
        with pytest.raises(TrainingError, match=msg):
            ex.execute_operation(op, ins)
    assert np.array_equal(back(ex.execute_operation(Operation.MulScalar(3.0), [t])), np.full((2, 2), 3.0))
    # the fixed LoRA inputs of tests/executor_direct.rs:339-376
    x = torch.tensor([[1.0, 2, 3, 4], [5, 6, 7, 8]], device=cuda_device)
    A = torch.tensor([[0.1, 0.2], [0.3, 0.4], [0.5, 0.6], [0.7, 0.8]], device=cuda_device)
    Bm = torch.tensor([[1.0, 2, 3, 4], [5, 6, 7, 8]], device=cuda_device)
    out = back(ex.execute_operation(Operation.LoRA(NodeId(1), NodeId(2), 0.5), [x, A, Bm]))
    assert out.shape == (2, 4) and np.allclose(out[0], 0.5 * np.array([35.0, 46.0, 57.0, 68.0]), rtol=1e-5)
    ex.synchronize()
    with pytest.raises(TrainingError):
        AsyncExecutor("cpu")
    agx = AsyncGraphExecutor(cuda_device)
    futs = [agx.execute_tensor(LazyTensor.from_tensor(t).mul_scalar(float(k))) for k in range(1, 4)]
    assert [float(f.result(timeout=60)[0, 0]) for f in futs] == [1.0, 2.0, 3.0]
    agx.shutdown()


def test_cross_entropy_loss(cuda_device):
    """src/training/loss.rs:246-380."""
    from metal_candle_b200.training import IGNORE_INDEX, InvalidConfig, cross_entropy_loss

    dev = cuda_device
    lg = torch.tensor([[[10.0, 0.0, 0.0]]], device=dev)
    assert float(cross_entropy_loss(lg, torch.tensor([[0]], device=dev))) < 0.1
    assert float(cross_entropy_loss(lg, torch.tensor([[2]], device=dev))) > 5.0
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        x = S.normal(8, "lg", (3, 5, 1000)) * 2
        if dtype == torch.bfloat16:
            x = S.bf16_round(x)
        tg = S.token_ids(8, "tg", (3, 5), 1000)
        tg[0, 1] = tg[2, 4] = IGNORE_INDEX
        want_l, want_d = R.cross_entropy_loss(x, tg)
        loss, d = cross_entropy_loss(torch.from_numpy(x).to(dev).to(dtype), torch.from_numpy(tg).to(dev), IGNORE_INDEX,
                                     return_grad=True)
        assert abs(float(loss) - want_l) <= tol * abs(want_l)
        assert R.max_abs_normalised(back(d), want_d) <= max(tol, 1e-4)
        assert float(back(d)[0, 1].max()) == 0.0  # ignored rows get no gradient
    with pytest.raises(InvalidConfig, match="logits must be 3D"):
        cross_entropy_loss(torch.zeros(4, 3, device=dev), torch.zeros(4, device=dev, dtype=torch.long))
    with pytest.raises(InvalidConfig, match="targets must be 2D"):
        cross_entropy_loss(torch.zeros(1, 4, 3, device=dev), torch.zeros(4, device=dev, dtype=torch.long))
    with pytest.raises(InvalidConfig, match="batch/seq_len mismatch"):
        cross_entropy_loss(torch.zeros(1, 4, 3, device=dev), torch.zeros(1, 5, device=dev, dtype=torch.long))
    with pytest.raises(InvalidConfig, match="all tokens are ignored"):
        cross_entropy_loss(torch.zeros(1, 2, 3, device=dev), torch.full((1, 2), IGNORE_INDEX, device=dev), IGNORE_INDEX)


def test_adapter_parameters_forward_and_merge(cuda_device):
    """src/training/adapter.rs:357-477: 2 modules x 4 layers of 768x768 r8 = 98,304 parameters."""
    from metal_candle_b200.backend import TrainingError
    from metal_candle_b200.training import InvalidConfig, LoRAAdapter, LoRAAdapterConfig, LoRAConfig, LoRALayer, TargetModule

    dev = cuda_device
    ad = LoRAAdapter(768, 2048, 4, LoRAAdapterConfig(rank=8), dev)
    assert ad.num_layers() == 4 and len(ad.layers()) == 8 and ad.num_trainable_parameters() == 98_304
    assert ad.num_frozen_parameters(1_000_000) == 1_000_000 - 98_304
    assert ad.get_layer(0, TargetModule.QProj).num_parameters() == 12_288
    assert ad.get_layer(0, TargetModule.OProj) is None and ad.forward(0, TargetModule.OProj, torch.zeros(1, 768, device=dev)) is None
    x = torch.randn(2, 5, 768, device=dev)
    d = ad.forward(1, TargetModule.VProj, x)
    assert d.shape == (2, 5, 768) and float(d.abs().max()) == 0.0  # B starts at zero (src/training/lora.rs:244)
    layer = ad.get_layer(1, TargetModule.VProj)
    assert tuple(layer.lora_a_tensor().shape) == (768, 8) and tuple(layer.lora_b_tensor().shape) == (8, 768)
    assert float(layer.lora_b_tensor().abs().sum()) == 0.0 and len(layer.trainable_variables()) == 2
    # grouped-query sizing of K/V adapters
    assert LoRAAdapter(896, 4864, 1, LoRAAdapterConfig(target_modules=[TargetModule.KProj]), dev, kv_size=128) \
        .get_layer(0, TargetModule.KProj).out_features == 128
    with pytest.raises(InvalidConfig, match="LoRA rank 16 exceeds maximum rank 8"):
        LoRALayer(8, 64, LoRAConfig(rank=16), dev)
    # merge_weights: W + s (A B)^T (src/training/adapter.rs:315-354)
    layer.lora_b.normal_(0, 0.05)
    W = torch.randn(768, 768, device=dev) * 0.02
    merged = back(ad.merge_weights(W, 1, TargetModule.VProj))
    want = R.lora_merge_weights(back(W), back(layer.lora_a), back(layer.lora_b), 2.0)
    assert R.max_abs_normalised(merged, want) <= 1e-4
    assert ad.merge_weights(W, 1, TargetModule.OProj) is W
    # dropout (tests/lora_dropout.rs): training-mode calls draw different masks, eval mode is deterministic
    dl = LoRALayer(64, 64, LoRAConfig(rank=4, alpha=8.0, dropout=0.5), dev)
    dl.lora_b.normal_(0, 0.5)
    xs = torch.randn(4, 64, device=dev)
    outs = [dl.forward(xs) for _ in range(5)]
    assert any(float((a - b).abs().mean()) > 0.01 for i, a in enumerate(outs) for b in outs[i + 1:])
    dl.eval()
    assert not dl.is_training() and torch.equal(dl.forward(xs), dl.forward(xs))
    dl.set_training(True)
    assert dl.is_training()


def test_trainer_counts_steps_and_follows_schedule(cuda_device):
    """tests/training/trainer_test.rs: step counting, LR sequence, loss >= 0."""
    from metal_candle_b200.qwen import ModelConfig, Qwen
    from metal_candle_b200.training import LoRAAdapterConfig, LRScheduler, TargetModule, Trainer, TrainingConfig

    cfg = ModelConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2)
    model = Qwen(cfg, cuda_device, dtype=torch.float32, seed=1)
    tc = TrainingConfig(num_epochs=2, lr_scheduler=LRScheduler.linear(4, 1e-3))
    tr = Trainer(cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers,
                 LoRAAdapterConfig(rank=4, alpha=8.0, target_modules=[TargetModule.QProj, TargetModule.VProj]), tc,
                 cuda_device, kv_size=cfg.kv_size)
    model.apply_adapter(tr.lora_adapter())
    data = []
    for i in range(3):
        ids = torch.from_numpy(S.token_ids(i, "ids", (2, 16), cfg.vocab_size)).to(cuda_device)
        data.append((ids, torch.roll(ids, -1, 1)))
    metrics = tr.train(data, model.forward_backward, verbose=False)
    assert len(metrics) == 6 and tr.global_step() == 6 and [m.step for m in metrics] == [1, 2, 3, 4, 5, 6]
    assert [m.learning_rate for m in metrics] == [tc.lr_scheduler.get_lr(s) for s in range(6)]
    assert all(m.loss >= 0 and np.isfinite(m.loss) for m in metrics)
    assert metrics[0].learning_rate == 0.0 and metrics[-1].learning_rate == float(np.float32(1e-3))
