"""The C-ABI training-step engine (mcb_qwen_*) against the Python step it mirrors and against the CPU oracle.

The engine issues the same kernels in the same order as `Qwen.forward_backward`, so loss and LoRA gradients must
agree bit for bit; AdamW through the engine must move the parameters exactly as `AdamW.step_vars` does (same
shared per-tensor counter).  The oracle comparison anchors both."""
import numpy as np
import pytest
import torch

from oracle import reference_ops as R

from tests.test_gpu_qwen_step import all_targets, batch, build, fused_attention_config, oracle_of

pytestmark = pytest.mark.gpu


def _i32(a, dev):
    return torch.from_numpy(np.where(a == R.IGNORE_INDEX, -1, a)).to(dev).to(torch.int32).contiguous()


@pytest.mark.parametrize("which,nb", [("all", 3), ("qv", 3), ("qv", 8)])
def test_engine_matches_python_step_and_oracle(cuda_device, which, nb):
    """nb = 8 gives 1024 tokens: from there the MLP's plain linears run on CTA pairs and the SwiGLU backward moves
    into the epilogue of the down projection's input-gradient GEMM."""
    from metal_candle_b200 import _lib, backend
    from metal_candle_b200.engine import QwenEngine
    from metal_candle_b200.training import TargetModule

    targets = all_targets() if which == "all" else [TargetModule.QProj, TargetModule.VProj]
    cfg, model, adapter = build(cuda_device, torch.bfloat16, targets, cfg=fused_attention_config())
    ids, tg = batch(41, nb, 128, cfg.vocab_size)
    tg[2, 10:30] = R.IGNORE_INDEX
    ids_d, tg_d = _i32(ids, cuda_device), _i32(tg, cuda_device)
    assert backend.lora_linear_backward_swiglu_supported(nb * 128, cfg.intermediate_size, cfg.hidden_size, 0) == (nb == 8)
    loss_p, g_p = model.forward_backward(ids_d, tg_d)
    loss_p, g_p = loss_p.clone(), [g.clone() for g in g_p]
    eng = QwenEngine(model, nb, 128)
    for chunk in (8192, 100):            # one chunk, and several ragged ones
        eng.set_ce_chunk(chunk)
        for g in model._grad_views:
            g.fill_(7.0)
        loss_e, g_e = eng.forward_backward(ids_d, tg_d)
        torch.cuda.synchronize()
        assert torch.equal(loss_e, loss_p), (float(loss_e), float(loss_p))
        for a, b in zip(g_e, g_p):
            assert torch.equal(a, b)
    # accumulate adds
    eng.forward_backward(ids_d, tg_d, accumulate=True)
    for a, b in zip(model._grad_views, g_p):
        assert torch.allclose(a, 2 * b, rtol=1e-5, atol=1e-7)
    # the oracle
    orc = oracle_of(cfg, model, adapter, True)
    want_loss, want_grads = orc.loss_and_grads(ids, tg)
    assert abs(float(loss_p) - want_loss) <= 2e-2 * abs(want_loss)
    errs = [R.max_abs_normalised(g.cpu().numpy(), w) for g, w in zip(g_p, want_grads)]
    assert max(errs) <= 4e-2, sorted(errs)[-4:]
    # a smaller batch in the same arena; a larger one is refused
    loss_s, _ = eng.forward_backward(ids_d[:1].contiguous(), tg_d[:1].contiguous())
    want_s, _ = model.forward_backward(ids_d[:1].contiguous(), tg_d[:1].contiguous())
    assert torch.equal(loss_s.clone(), want_s)
    with pytest.raises(Exception):
        eng.forward_backward(torch.cat([ids_d, ids_d]), torch.cat([tg_d, tg_d]))
    with pytest.raises(_lib.McbError, match="multiples of 128"):
        eng.forward_backward(ids_d[:, :100].contiguous(), tg_d[:, :100].contiguous())
    assert _lib.device_status() == 0
    eng.destroy()


def test_engine_train_steps_match_python_training(cuda_device):
    """Five optimizer steps through mcb_qwen_train_step against TrainingStep.execute with the Python model: the same
    losses and, at the end, the same parameters, bit for bit (AdamW's shared counter advances once per tensor)."""
    from metal_candle_b200.engine import QwenEngine
    from metal_candle_b200.training import AdamW, AdamWConfig, LRScheduler, TargetModule, TrainingStep

    tm = [TargetModule.QProj, TargetModule.KProj, TargetModule.VProj, TargetModule.OProj]
    sched = LRScheduler.warmup_cosine(2, 10, 1e-3, 1e-5)
    batches = [batch(500 + s, 2, 128, 320) for s in range(5)]

    def run(engine: bool):
        cfg, model, adapter = build(cuda_device, torch.bfloat16, tm, cfg=fused_attention_config(), b_std=0.0)
        losses = []
        if engine:
            eng = QwenEngine(model, 2, 128)
            for s, (ids, tg) in enumerate(batches):
                loss = eng.train_step(_i32(ids, cuda_device), _i32(tg, cuda_device), sched.get_lr(s))
                losses.append(float(loss))
            assert eng.info()["adamw_steps"] == 5 * 2 * len(tm) * cfg.num_hidden_layers
            eng.destroy()
        else:
            opt, stepper = AdamW(AdamWConfig()), TrainingStep()
            for s, (ids, tg) in enumerate(batches):
                m = stepper.execute(_i32(ids, cuda_device), _i32(tg, cuda_device), adapter, opt, sched.get_lr(s), model.forward_backward)
                losses.append(m.loss)
        return losses, [v.clone() for v in TrainingStep.collect_trainable_vars(adapter)]

    l_py, p_py = run(False)
    l_en, p_en = run(True)
    assert l_py == l_en, (l_py, l_en)
    for a, b in zip(p_py, p_en):
        assert torch.equal(a, b)
    assert l_py[-1] != l_py[0]


def test_engine_step_in_a_cuda_graph(cuda_device):
    """The engine allocates nothing inside a step and issues only stream work: a captured step replays to the same
    result."""
    from metal_candle_b200.engine import QwenEngine

    cfg, model, adapter = build(cuda_device, torch.bfloat16, all_targets(), cfg=fused_attention_config())
    ids, tg = batch(61, 2, 128, cfg.vocab_size)
    ids_d, tg_d = _i32(ids, cuda_device), _i32(tg, cuda_device)
    eng = QwenEngine(model, 2, 128)
    loss0, g0 = eng.forward_backward(ids_d, tg_d)
    loss0, g0 = loss0.clone(), [g.clone() for g in g0]
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        eng.forward_backward(ids_d, tg_d)
    for g in model._grad_views:
        g.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(eng._loss[:1], loss0)
    for a, b in zip(model._grad_views, g0):
        assert torch.equal(a, b)
    del graph
    eng.destroy()
