"""GPU parity at the benchmark configurations' own shapes (the other GPU test files use small stand-ins):

* the real Qwen2.5-0.5B architecture (24 layers, hidden 896, 14 query / 2 kv heads, MLP 4864, vocabulary 151 936) on a
  bounded number of tokens, with configuration 4's adapter set (q/v, r = 8, alpha 16) and configuration 5's
  (q/k/v/o, r = 16, alpha 32): loss, logits and every LoRA gradient against the float64 torch-CPU oracle;
* a 50-step loss curve on that architecture with configuration 4's optimizer and schedule;
* the fused LoRA linear at configuration 3's wide shapes;
* the causal, scaled softmax entry points called directly; cross-entropy at the real vocabulary width.

Tolerances as everywhere: float32 path 1e-4, bf16 path 2e-2 (max-abs normalised) against the float64 oracle on the
same (bf16-rounded) inputs.  Through the whole 24-layer bf16 chain the LoRA gradients carry the rounding noise of every
activation in between: the measured errors are printed (run with -s), see the note at `test_real_architecture_step`.
"""
import math

import numpy as np
import pytest
import torch

from oracle import qwen_oracle as QO
from oracle import reference_ops as R
from oracle import seeded as S

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------------------------------------------------------
# the real architecture
# ---------------------------------------------------------------------------------------------------------------

ADAPTER_SETS = {
    "c4": dict(rank=8, alpha=16.0, targets=("q_proj", "v_proj")),
    "c5": dict(rank=16, alpha=32.0, targets=("q_proj", "k_proj", "v_proj", "o_proj")),
}


class _Real:
    """One model per dtype for the whole module (2 GB of weights in bf16), and its weights once as float64 torch
    tensors for the oracle (4 GB on the host)."""

    def __init__(self):
        self.models = {}

    def get(self, dev, dtype):
        if dtype not in self.models:
            from metal_candle_b200.qwen import ModelConfig, Qwen

            cfg = ModelConfig.qwen25_05b()
            model = Qwen(cfg, dev, dtype=dtype, seed=21)
            g = torch.Generator(device=dev).manual_seed(22)
            # non-trivial norm weights and q/k/v biases (the checkpointed model has both; random init has 1 and 0)
            for L in model.layers:
                for k in ("input_layernorm", "post_attention_layernorm"):
                    L[k].copy_((1 + 0.1 * torch.randn(cfg.hidden_size, device=dev, generator=g)).to(dtype))
                for m in ("q_proj", "k_proj", "v_proj"):
                    L[m].bias.copy_((0.05 * torch.randn(L[m].out_f, device=dev, generator=g)).to(dtype))
            model.norm.copy_((1 + 0.1 * torch.randn(cfg.hidden_size, device=dev, generator=g)).to(dtype))
            w = {"embed_tokens": model.embed_tokens, "norm": model.norm, "lm_head": model.lm_head.weight}
            for i, L in enumerate(model.layers):
                w[f"layers.{i}.input_layernorm"] = L["input_layernorm"]
                w[f"layers.{i}.post_attention_layernorm"] = L["post_attention_layernorm"]
                for m in model.MODULES:
                    w[f"layers.{i}.{m}.weight"] = L[m].weight
                    if L[m].bias is not None:
                        w[f"layers.{i}.{m}.bias"] = L[m].bias
            w64 = {k: v.detach().to("cpu", torch.float64) for k, v in w.items()}
            self.models[dtype] = (cfg, model, w64)
        return self.models[dtype]


@pytest.fixture(scope="module")
def real():
    r = _Real()
    yield r
    r.models.clear()
    torch.cuda.empty_cache()


def _attach(cfg, model, dev, which, seed, b_std):
    from metal_candle_b200.training import LoRAAdapter, LoRAAdapterConfig, TargetModule

    a = ADAPTER_SETS[which]
    acfg = LoRAAdapterConfig(rank=a["rank"], alpha=a["alpha"], target_modules=[TargetModule.from_name(t) for t in a["targets"]])
    g = torch.Generator(device=dev).manual_seed(seed)
    adapter = LoRAAdapter(cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers, acfg, dev, kv_size=cfg.kv_size,
                          generator=g)
    for _, l in adapter.layers():
        s = 1.0 / math.sqrt(l.in_features)     # A ~ U(+-1/sqrt(in)), the benchmark configurations' rule
        l.lora_a.copy_((torch.rand(l.lora_a.shape, device=dev, generator=g) * 2 - 1) * s)
        if b_std > 0:
            l.lora_b.normal_(0, b_std, generator=g)   # non-zero so that dA is not trivially zero
    model.remove_adapter()
    model.apply_adapter(adapter)
    return adapter


def _oracle(cfg, w64, adapter, round_bf16, dtype=torch.float64):
    rnd = (lambda a: S.bf16_round(a)) if round_bf16 else (lambda a: a)
    lora = {k: (rnd(l.lora_a.cpu().numpy()), rnd(l.lora_b.cpu().numpy())) for k, l in adapter.layers()}
    w = w64 if dtype == torch.float64 else {k: v.to(dtype) for k, v in w64.items()}
    return QO.QwenOracle(cfg, w, lora, adapter.config().to_lora_config().scaling(), dtype=dtype)


def _batch(seed, B, Sq, vocab):
    ids = S.token_ids(seed, "ids", (B, Sq), vocab)
    tg = np.concatenate([ids[:, 1:], np.full((B, 1), R.IGNORE_INDEX, dtype=np.int64)], 1)
    return ids, tg


@pytest.mark.parametrize("dtype,which,B,Sq", [
    (torch.bfloat16, "c5", 1, 256),     # fused attention kernels (head_dim 64, sequence a multiple of 128)
    (torch.bfloat16, "c4", 2, 128),
    (torch.float32, "c5", 2, 96),       # validation path: materialised scores, CUDA-core GEMMs
    (torch.float32, "c4", 1, 160),
])
def test_real_architecture_step(cuda_device, real, dtype, which, B, Sq):
    """Loss, logits and all LoRA gradients of one forward+backward of the 24-layer model.

    bf16 bound on the gradients: each kernel alone holds 2e-2 (tests/test_gpu_lora.py, test_gpu_row_ops.py,
    test_gpu_attention.py), and the float32 path of the same model holds 1e-4 here, so the arithmetic is the
    oracle's.  Along the 24-layer bf16 chain every activation and the residual stream are rounded to bf16 between
    kernels (as a bf16 candle graph rounds them too) while the oracle rounds nothing; a LoRA gradient depends on all
    layers (forward through the ones below, backward through the ones above), so the rounding noise it carries
    does not depend on its depth: measured 2.2-3.3 % relative Frobenius error per layer at every depth (0 to 23), the
    worst single tensor of 192 at 4.8 % max-abs, while the loss agrees to 2e-5 and the logits to 1.6e-2.  (The
    logits' own 1.6 % is what drives it: d loss / d logits = softmax - onehot moves by as much.)  Held to 6e-2
    max-abs and 4e-2 relative Frobenius; the measured values are printed."""
    from metal_candle_b200 import _lib

    cfg, model, w64 = real.get(cuda_device, dtype)
    adapter = _attach(cfg, model, cuda_device, which, seed=31, b_std=0.02)
    ids, tg = _batch(41, B, Sq, cfg.vocab_size)
    loss, grads = model.forward_backward(torch.from_numpy(ids).to(cuda_device), torch.from_numpy(tg).to(cuda_device))
    bf = dtype == torch.bfloat16
    orc = _oracle(cfg, w64, adapter, bf)
    want_loss, want_grads = orc.loss_and_grads(ids, tg)
    tol = 2e-2 if bf else 1e-4
    assert abs(float(loss) - want_loss) <= tol * abs(want_loss), (float(loss), want_loss)
    n_mod = len(ADAPTER_SETS[which]["targets"])
    assert len(grads) == len(want_grads) == 2 * n_mod * cfg.num_hidden_layers
    got_grads = [g.cpu().numpy().astype(np.float64) for g in grads]
    errs = [R.max_abs_normalised(g, w) for g, w in zip(got_grads, want_grads)]
    fro = [float(np.linalg.norm(g - w) / np.linalg.norm(w)) for g, w in zip(got_grads, want_grads)]
    names = [f"{k}.{ab}" for k, _ in adapter.layers() for ab in "AB"]
    worst = sorted(zip(errs, names), reverse=True)[:5]
    by_layer, fro_layer = {}, {}
    for e, f, n in zip(errs, fro, names):
        i = int(n.split(".")[1])
        by_layer[i] = max(by_layer.get(i, 0.0), e)
        fro_layer[i] = max(fro_layer.get(i, 0.0), f)
    print(f"\n[{which} {dtype} {B}x{Sq}] loss {float(loss):.6f} vs {want_loss:.6f}; worst max-abs gradient errors {worst}; "
          f"max-abs per layer (0, 4, 8, 12, 16, 20, 23): {[round(by_layer[i], 4) for i in (0, 4, 8, 12, 16, 20, 23)]}; "
          f"relative Frobenius per layer: {[round(fro_layer[i], 4) for i in (0, 4, 8, 12, 16, 20, 23)]}; worst {max(fro):.4f}")
    if bf:
        # max-abs normalised: the largest of ~14 000 noisy elements per tensor, over 96-192 tensors; the relative
        # Frobenius error is the steadier measure of the same rounding noise
        assert worst[0][0] <= 6e-2, worst
        assert max(fro) <= 4e-2, sorted(zip(fro, names), reverse=True)[:5]
    else:
        assert worst[0][0] <= tol, worst
    assert all(float(np.abs(w).max()) > 0 for w in want_grads)          # no gradient is trivially zero
    logits = model.forward(torch.from_numpy(ids).to(cuda_device)).float().cpu().numpy()
    err_logits = R.max_abs_normalised(logits, orc.forward(ids).detach().numpy())
    print(f"    logits error {err_logits:.3e}")
    assert err_logits <= tol
    assert _lib.device_status() == 0


def test_real_architecture_fifty_step_curve(cuda_device, real):
    """Benchmark configuration 4's training recipe on the real architecture at a bounded batch (1 x 128 tokens):
    q/v adapters r = 8, alpha 16, B = 0 at step 0 (src/training/lora.rs:244), AdamW lr 1e-4 with
    WarmupCosine(5, 50, 1e-4, 1e-6), 50 steps; the bf16 loss curve against the oracle's, step by step.  The oracle
    runs in float32 here (the reference's own precision; ~0.3 s per step instead of seconds in float64)."""
    from metal_candle_b200.training import AdamW, AdamWConfig, LRScheduler, TrainingStep

    cfg, model, w64 = real.get(cuda_device, torch.bfloat16)
    adapter = _attach(cfg, model, cuda_device, "c4", seed=51, b_std=0.0)
    orc = _oracle(cfg, w64, adapter, False, dtype=torch.float32)
    sched = LRScheduler.warmup_cosine(5, 50, 1e-4, 1e-6)
    batches = [_batch(300 + s, 1, 128, cfg.vocab_size) for s in range(50)]
    want = QO.train(orc, batches, sched.get_lr)
    opt, stepper, got = AdamW(AdamWConfig(learning_rate=1e-4)), TrainingStep(), []
    for s, (ids, tg) in enumerate(batches):
        m = stepper.execute(torch.from_numpy(ids).to(cuda_device), torch.from_numpy(tg).to(cuda_device), adapter, opt,
                            sched.get_lr(s), model.forward_backward)
        got.append(m.loss)
    got, want = np.array(got), np.array(want)
    rel = np.abs(got - want) / np.abs(want)
    print(f"\n50-step curve: first {got[:3]} vs {want[:3]}, last {got[-3:]} vs {want[-3:]}, max rel diff {rel.max():.3e}")
    assert rel.max() <= 2e-2
    assert stepper.step() == 50 and opt.step_count == 50 * 2 * 2 * cfg.num_hidden_layers
    # B = 0 at the start: the first step's loss is the base model's, and the adapters have moved by the end
    assert any(float(l.lora_b.abs().max()) > 0 for _, l in adapter.layers())


def test_real_architecture_captured_step_survives_workspace_growth(cuda_device, real):
    """A step captured into a CUDA graph keeps the scratch buffers it points at: an eager call that needs a larger
    scratch buffer afterwards (which replaces the cached one) must not disturb later replays."""
    from metal_candle_b200 import backend as B

    cfg, model, _ = real.get(cuda_device, torch.bfloat16)
    adapter = _attach(cfg, model, cuda_device, "c5", seed=61, b_std=0.02)
    ids, tg = _batch(71, 1, 128, cfg.vocab_size)
    ids_d = torch.from_numpy(ids).to(cuda_device).to(torch.int32)
    tg_d = torch.from_numpy(np.where(tg == R.IGNORE_INDEX, -1, tg)).to(cuda_device).to(torch.int32)
    loss0, g0 = model.forward_backward(ids_d, tg_d)
    loss0, g0 = loss0.clone(), [g.clone() for g in g0]
    step = model.capture_forward_backward(1, 128)
    before = B.workspace_refs(cuda_device)[0]
    # a far larger LoRA problem: the cached scratch buffer is replaced
    big = torch.randn(65536, 2048, device=cuda_device).to(torch.bfloat16)
    A = torch.randn(2048, 64, device=cuda_device) * 0.01
    Bm = torch.randn(64, 2048, device=cuda_device) * 0.01
    B.lora_forward_fused(big, A, Bm, 2.0)
    after = B.workspace_refs(cuda_device)[0]
    assert after.data_ptr() != before.data_ptr() or after.numel() != before.numel()
    junk = [torch.full((1 << 22,), 7.0, device=cuda_device) for _ in range(8)]   # would land in freed scratch memory
    loss1, g1 = step(ids_d, tg_d)
    torch.cuda.synchronize()
    assert torch.equal(loss1, loss0)
    for a, b in zip(g1, g0):
        assert torch.equal(a, b)
    del junk


# ---------------------------------------------------------------------------------------------------------------
# fused LoRA linear at benchmark configuration 3's wide shapes
# ---------------------------------------------------------------------------------------------------------------

def _lora_case(dev, dtype, M, K, N, r, seed=17):
    from metal_candle_b200 import _lib
    from metal_candle_b200 import backend as B

    scale = 2.0            # alpha = 2r
    c = S.lora_linear_case(seed, M, K, N, r)
    o = {k: S.bf16_round(v) for k, v in c.items()} if dtype == torch.bfloat16 else dict(c)
    t = lambda a, dt=dtype: torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(dt).contiguous()
    x, W, dy = t(o["x"]), t(o["W"]), t(o["dy"])
    A, Bm = t(c["A"], torch.float32), t(c["B"], torch.float32)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    y, h = B.lora_linear_forward(x, W, None, A, Bm, scale)
    want_y, _ = R.lora_linear_forward(o["x"], o["W"], None, o["A"], o["B"], scale)
    assert R.max_abs_normalised(y.float().cpu().numpy(), want_y) <= tol, "y"
    del want_y
    dx, dA, dB = B.lora_linear_backward(x, B.transpose_2d(W), A, Bm, scale, dy, h_save=h)
    wdx, wdA, wdB = R.lora_linear_backward(o["x"], o["W"], o["A"], o["B"], scale, o["dy"])
    assert R.max_abs_normalised(dx.float().cpu().numpy(), wdx) <= tol, "dx"
    assert R.max_abs_normalised(dA.cpu().numpy(), wdA) <= tol, "dA"
    assert R.max_abs_normalised(dB.cpu().numpy(), wdB) <= tol, "dB"
    assert _lib.device_status() == 0


WIDE = [(2048, 2048), (4096, 4096), (4096, 14336)]


@pytest.mark.parametrize("K,N", WIDE)
@pytest.mark.parametrize("r", [8, 16, 64])
def test_lora_linear_wide_shapes_bf16_m512(cuda_device, K, N, r):
    _lora_case(cuda_device, torch.bfloat16, 512, K, N, r)


@pytest.mark.parametrize("K,N,r", [(2048, 2048, 64), (4096, 4096, 16), (4096, 14336, 8)])
def test_lora_linear_wide_shapes_bf16_m4096(cuda_device, K, N, r):
    _lora_case(cuda_device, torch.bfloat16, 4096, K, N, r)


@pytest.mark.parametrize("K,N,r", [(2048, 2048, 8), (4096, 4096, 64), (4096, 14336, 16)])
def test_lora_linear_wide_shapes_f32_m512(cuda_device, K, N, r):
    _lora_case(cuda_device, torch.float32, 512, K, N, r)


# ---------------------------------------------------------------------------------------------------------------
# causal, scaled softmax entry points called directly; cross-entropy at the real vocabulary width
# ---------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("blocks,seq,scale", [(3, 128, 0.125), (2, 1024, 0.25), (2, 200, 1.7), (1, 2048, 0.125)])
def test_softmax_causal_entry_points(cuda_device, dtype, blocks, seq, scale):
    """mcb_softmax_causal_fwd / _bwd: scale and mask inside the kernel (Attention::forward's divide, mask add and
    softmax_stable, src/models/transformer.rs:264-275).  The input carries NO mask: finite values everywhere, the
    kernel must ignore the columns behind the diagonal and write zeros there."""
    from metal_candle_b200 import _lib

    lib = _lib.init(0)
    rows = blocks * seq
    x = S.normal(5, "x", (rows, seq), 0.0, 3.0)
    dy = S.normal(5, "dy", (rows, seq))
    if dtype == torch.bfloat16:
        x, dy = S.bf16_round(x), S.bf16_round(dy)
    mask = np.triu(np.ones((seq, seq), dtype=bool), 1)
    xm = (scale * x.astype(np.float64)).reshape(blocks, seq, seq)
    xm[:, mask] = -np.inf
    want_y = R.softmax_stable(xm.reshape(rows, seq))
    code = _lib.MCB_BF16 if dtype == torch.bfloat16 else _lib.MCB_F32
    st = torch.cuda.current_stream().cuda_stream
    xd = torch.from_numpy(x).to(cuda_device).to(dtype)
    yd = torch.full_like(xd, 7.0)
    _lib.check(lib.mcb_softmax_causal_fwd(xd.data_ptr(), yd.data_ptr(), rows, seq, seq, scale, code, st))
    got = yd.float().cpu().numpy()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert R.max_abs_normalised(got, want_y) <= tol
    assert (got.reshape(blocks, seq, seq)[:, mask] == 0).all()
    # backward on the oracle's y (rounded to the storage type) and dy values that would pollute a kernel that read
    # the masked columns
    y_in = want_y.astype(np.float32)
    if dtype == torch.bfloat16:
        y_in = S.bf16_round(y_in)
    want_dx = scale * R.softmax_backward(y_in, dy)
    want_dx = want_dx.reshape(blocks, seq, seq)
    want_dx[:, mask] = 0.0
    ydev = torch.from_numpy(y_in).to(cuda_device).to(dtype)
    dyd = torch.from_numpy(dy).to(cuda_device).to(dtype)
    dxd = torch.full_like(ydev, 7.0)
    _lib.check(lib.mcb_softmax_causal_bwd(ydev.data_ptr(), dyd.data_ptr(), dxd.data_ptr(), rows, seq, seq, scale, code, st))
    gdx = dxd.float().cpu().numpy()
    assert R.max_abs_normalised(gdx, want_dx.reshape(rows, seq)) <= tol
    assert (gdx.reshape(blocks, seq, seq)[:, mask] == 0).all()
    # seq = 0: no mask, scale only
    _lib.check(lib.mcb_softmax_causal_bwd(ydev.data_ptr(), dyd.data_ptr(), dxd.data_ptr(), rows, seq, 0, scale, code, st))
    assert R.max_abs_normalised(dxd.float().cpu().numpy(), scale * R.softmax_backward(y_in, dy)) <= tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_cross_entropy_at_the_real_vocabulary(cuda_device, dtype, tol):
    """cross_entropy_loss (src/training/loss.rs:58-147) over rows of 151 936 logits, ignored rows included."""
    from metal_candle_b200.training import IGNORE_INDEX, cross_entropy_loss

    V, Bq, Sq = 151936, 2, 24
    x = S.normal(9, "lg", (Bq, Sq, V)) * 2
    if dtype == torch.bfloat16:
        x = S.bf16_round(x)
    tg = S.token_ids(9, "tg", (Bq, Sq), V)
    tg[0, 3] = tg[1, 23] = tg[1, 0] = IGNORE_INDEX
    tg[0, 0], tg[0, 1] = 0, V - 1              # first and last column as targets
    want_l, want_d = R.cross_entropy_loss(x, tg)
    loss, d = cross_entropy_loss(torch.from_numpy(x).to(cuda_device).to(dtype), torch.from_numpy(tg).to(cuda_device),
                                 IGNORE_INDEX, return_grad=True)
    assert abs(float(loss) - want_l) <= tol * abs(want_l)
    got = d.float().cpu().numpy()
    assert R.max_abs_normalised(got, want_d) <= max(tol, 1e-4)
    assert float(np.abs(got[0, 3]).max()) == 0.0 and float(np.abs(got[1, 23]).max()) == 0.0


@pytest.mark.parametrize("V", [1024, 1000])
def test_cross_entropy_with_masked_logits(cuda_device, V):
    """-inf logits (a masked or padded vocabulary) in whole 16-byte vectors, also at the start of a row, must not
    produce NaN: they contribute exp(-inf) = 0 (V = 1024 takes the vector sweep, V = 1000 the scalar one)."""
    from metal_candle_b200.training import cross_entropy_loss

    x = S.normal(10, "lg", (1, 6, V)).astype(np.float32)
    x[0, :, :64] = -np.inf
    x[0, 2, 512:640] = -np.inf
    x[0, 3, V - 32:] = -np.inf
    tg = S.token_ids(10, "tg", (1, 6), V - 200) + 100
    tg[0, 2], tg[0, 3] = 700, 300          # targets sit on finite logits
    want_l, want_d = R.cross_entropy_loss(x, tg)
    assert np.isfinite(want_l)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        xin = x if dtype == torch.float32 else S.bf16_round(x)
        wl, wd = R.cross_entropy_loss(xin, tg)
        loss, d = cross_entropy_loss(torch.from_numpy(xin).to(cuda_device).to(dtype), torch.from_numpy(tg).to(cuda_device),
                                     None, return_grad=True)
        got = d.float().cpu().numpy()
        assert np.isfinite(float(loss)) and np.isfinite(got).all()
        assert abs(float(loss) - wl) <= tol * abs(wl)
        assert R.max_abs_normalised(got, wd) <= max(tol, 1e-4)
        assert (got[0, :, :64] == 0).all()


# ---------------------------------------------------------------------------------------------------------------
# a bounded device-side wait that runs out; checkpoints with a real adapter
# ---------------------------------------------------------------------------------------------------------------

def test_bounded_wait_runs_out_and_the_device_stays_usable(cuda_device):
    """The failure path of every mbarrier / flag wait in the tensor-core kernels, made to happen: a warp waits on a
    barrier nothing arrives at, with a limit of about a millisecond of SM cycles.  The kernel must return by itself,
    the status word must carry the wait's code, mcb_check_device must map it to MCB_ERR_DEVICE_TIMEOUT once, and the
    kernels launched right after must work."""
    import ctypes

    from metal_candle_b200 import _lib
    from metal_candle_b200 import backend as B

    lib = _lib.init(0)
    assert _lib.device_status() == 0
    waited = ctypes.c_int64(0)
    limit = 2_000_000            # ~1 ms at 2 GHz
    _lib.check(lib.mcb_selftest_wait_timeout(limit, ctypes.byref(waited), torch.cuda.current_stream().cuda_stream))
    assert limit < waited.value < 100 * limit, waited.value
    rc = lib.mcb_check_device()
    assert rc == _lib.MCB_ERR_DEVICE_TIMEOUT and b"code 90" in lib.mcb_last_error()
    assert lib.mcb_check_device() == 0                   # reported once, then cleared
    # status word read the other way round
    _lib.check(lib.mcb_selftest_wait_timeout(limit, None, torch.cuda.current_stream().cuda_stream))
    assert _lib.device_status() == _lib.MCB_WAIT_CODE_SELFTEST
    assert _lib.device_status() == 0
    # the context is intact: a tensor-core kernel with real waits runs and is right
    x = torch.randn(256, 256, device=cuda_device).to(torch.bfloat16)
    W = torch.randn(128, 256, device=cuda_device).to(torch.bfloat16)
    y, _ = B.lora_linear_forward(x, W, None, None, None, 1.0)
    want = x.float().cpu().numpy().astype(np.float64) @ W.float().cpu().numpy().astype(np.float64).T
    assert R.max_abs_normalised(y.float().cpu().numpy(), want) <= 2e-2
    assert lib.mcb_check_device() == 0
    assert lib.mcb_selftest_wait_timeout(0, None, None) == -2


def test_checkpoint_round_trip_with_a_real_adapter(cuda_device, tmp_path):
    """save_checkpoint / load_checkpoint (src/training/checkpoint.rs:65-178) on CUDA tensors, optimizer state
    included; a reloaded run continues exactly where the saved one stood."""
    from metal_candle_b200 import checkpoint as CK
    from metal_candle_b200.training import AdamW, AdamWConfig, LoRAAdapter, LoRAAdapterConfig, TargetModule, TrainingStep

    def make(seed):
        g = torch.Generator(device=cuda_device).manual_seed(seed)
        return LoRAAdapter(64, 160, 2, LoRAAdapterConfig(rank=4, alpha=8.0, target_modules=[TargetModule.QProj, TargetModule.VProj]),
                           cuda_device, kv_size=32, generator=g)

    a, b = make(1), make(2)
    va, vb = TrainingStep.collect_trainable_vars(a), TrainingStep.collect_trainable_vars(b)
    g = torch.Generator(device=cuda_device).manual_seed(3)
    grads = [[torch.randn(v.shape, device=cuda_device, generator=g) for v in va] for _ in range(3)]
    opt = AdamW(AdamWConfig(learning_rate=1e-2))
    opt.step_vars(va, grads[0])
    opt.step_vars(va, grads[1])
    p = tmp_path / "ck.safetensors"
    CK.save_checkpoint(a, p, CK.CheckpointMetadata(2, 1.25, 1e-2, 99), optimizer=opt)
    opt2 = AdamW(AdamWConfig(learning_rate=1e-2))
    meta = CK.load_checkpoint(b, p, optimizer=opt2)
    assert meta == CK.CheckpointMetadata(2, 1.25, 1e-2, 99) and opt2.step_count == opt.step_count == 2 * len(va)
    for x, y in zip(va, vb):
        assert torch.equal(x, y)
    opt.step_vars(va, grads[2])
    opt2.step_vars(vb, grads[2])
    for x, y in zip(va, vb):
        assert torch.equal(x, y)
    # the file is the reference's layout
    tensors, _ = CK.load_file(p)
    assert {"layers.0.q_proj.lora_a", "layers.1.v_proj.lora_b"} <= set(tensors)
    assert tensors["layers.0.v_proj.lora_b"].shape == (4, 32)


# ---------------------------------------------------------------------------------------------------------------
# rotary embedding + head relayout, called directly
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("B,Sq,Hq,Hk,d,pad", [(2, 256, 14, 2, 64, 0), (1, 100, 4, 2, 64, 16), (2, 33, 3, 1, 6, 0)])
def test_rope_relayout_entry_points(cuda_device, dtype, tol, B, Sq, Hq, Hk, d, pad):
    """mcb_rope_relayout_ex per projection and mcb_rope_relayout_qkv for the three at once, on the q / k / v column
    blocks of a fused row (the 0.5B model's 14 + 2 + 2 heads of 64; a padded row; a head size the vector kernel does
    not take): against the oracle's rotary tables (src/models/transformer.rs:47-120) and [B,S,H,d] -> [B,H,S,d]
    transpose, forward and reverse; the merged call must equal the three single calls bit for bit."""
    from metal_candle_b200 import _lib

    lib, dev, theta = _lib.init(0), cuda_device, 1.0e6
    code = _lib.MCB_F32 if dtype == torch.float32 else _lib.MCB_BF16
    st = torch.cuda.current_stream().cuda_stream
    width = (Hq + 2 * Hk) * d
    pitch = width + pad
    x = S.normal(9, "qkv", (B * Sq, pitch))
    if dtype == torch.bfloat16:
        x = S.bf16_round(x)
    xd = torch.from_numpy(x).to(dev).to(dtype).contiguous()
    sin, cos = QO._rope_tables(d, Sq, theta, torch.float64)
    heads, offs, rot = (Hq, Hk, Hk), (0, Hq * d, (Hq + Hk) * d), (1, 1, 0)
    want = []
    for H, off, r in zip(heads, offs, rot):
        blk = torch.from_numpy(x[:, off:off + H * d]).double().reshape(B, Sq, H, d)
        if r:
            blk = QO._apply_rope(blk, sin, cos)
        want.append(blk.permute(0, 2, 1, 3).contiguous().numpy())
    single = [torch.empty(B, H, Sq, d, device=dev, dtype=dtype) for H in heads]
    for out, H, off, r in zip(single, heads, offs, rot):
        _lib.check(lib.mcb_rope_relayout_ex(xd.data_ptr(), out.data_ptr(), B, Sq, H, d, theta, r, 0, pitch, off, code, st))
    merged = [torch.empty_like(t) for t in single]
    _lib.check(lib.mcb_rope_relayout_qkv(xd.data_ptr(), *(t.data_ptr() for t in merged), B, Sq, Hq, Hk, d, theta, 0, pitch, code, st))
    for got, one, w in zip(merged, single, want):
        assert torch.equal(got, one)
        assert R.max_abs_normalised(got.float().cpu().numpy().astype(np.float64), w) <= tol
    # the reverse pass: gradients in [B,H,S,d] back into the fused row with the transposed rotation
    g = [S.normal(10 + i, "g", (B, H, Sq, d)) for i, H in enumerate(heads)]
    if dtype == torch.bfloat16:
        g = [S.bf16_round(a) for a in g]
    gd = [torch.from_numpy(a).to(dev).to(dtype).contiguous() for a in g]
    back_single = torch.zeros(B * Sq, pitch, device=dev, dtype=dtype)
    for t, H, off, r in zip(gd, heads, offs, rot):
        _lib.check(lib.mcb_rope_relayout_ex(t.data_ptr(), back_single.data_ptr(), B, Sq, H, d, theta, r, 1, pitch, off, code, st))
    back_merged = torch.zeros_like(back_single)
    _lib.check(lib.mcb_rope_relayout_qkv(back_merged.data_ptr(), *(t.data_ptr() for t in gd), B, Sq, Hq, Hk, d, theta, 1, pitch, code, st))
    assert torch.equal(back_merged, back_single)
    got = back_merged.float().cpu().numpy().astype(np.float64)
    for a, H, off, r in zip(g, heads, offs, rot):
        blk = torch.from_numpy(a).double().permute(0, 2, 1, 3)           # [B,S,H,d]
        if r:
            blk = QO._apply_rope(blk, -sin, cos)                          # the transpose of a rotation is the rotation by -angle
        assert R.max_abs_normalised(got[:, off:off + H * d], blk.reshape(B * Sq, H * d).numpy()) <= tol
    if pad:
        assert float(back_merged[:, width:].abs().max()) == 0.0           # the padding columns are not touched
    assert _lib.device_status() == 0
