"""Pins the CPU oracle (oracle/reference_ops.py) before anything is compared with it.

(1) Every known-answer value the reference's own tests hold for this path, cited file:line in the
    metal-candle tree.  The reference holds no golden files and seeds nothing, so these few values are
    all the forward pinning there is.
(2) The reference's "fused == unfused within 1e-4" criterion (tests/custom_ops_correctness.rs:81-85,
    tests/rmsnorm_correctness.rs:71-74, tests/softmax_correctness.rs:61-64), applied to the serial
    restatements of the Metal kernel bodies against the unfused op sequences.
(3) Backward formulas -- which the reference does not pin -- against central finite differences in
    float64 and torch-CPU autograd over the same op sequence.
(4) The committed fixtures under tests/golden/ (regression pin; see tests/golden/make_golden.py).
"""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import reference_ops as R
from oracle import seeded as S

GOLDEN = Path(__file__).parent / "golden"


# ---- (1) known answers ------------------------------------------------------------------------
def test_rmsnorm_known_answers():
    # tests/executor_direct.rs:480-496: [3,4], eps 0 -> [0.8485, 1.1314] +-1e-3
    assert np.allclose(R.rms_norm(np.array([[3.0, 4.0]]), 0.0), [[0.8485, 1.1314]], atol=1e-3)
    assert np.allclose(R.rms_norm_msl(np.array([[3.0, 4.0]]), 0.0), [[0.8485, 1.1314]], atol=1e-3)
    # src/backend/tensor.rs:321-336: ones -> ones +-1e-5 (eps 1e-5)
    assert np.allclose(R.rms_norm(np.ones((1, 4)), 1e-5, np.float32), 1.0, atol=1e-5)
    # src/backend/tensor.rs:382-397: ratios 2:4:6 preserved
    y = R.rms_norm(np.array([[2.0, 4.0, 6.0]]), 1e-5)[0]
    assert abs(y[1] / y[0] - 2) < 1e-4 and abs(y[2] / y[0] - 3) < 1e-4
    # tests/rmsnorm_correctness.rs:133-140: RMS of the output is 1 +- 1%
    y = R.rms_norm(S.normal(1, "x", (8, 512)), 1e-5)
    assert np.allclose(np.sqrt((y ** 2).mean(-1)), 1.0, atol=1e-2)


def test_softmax_known_answers():
    # src/backend/tensor.rs:262-275
    assert np.allclose(R.softmax_stable(np.zeros((1, 3))), 1 / 3, atol=1e-5)
    # tests/softmax_lazy.rs:137-169
    y = R.softmax_stable(np.array([[100.0, 200.0, 300.0, 400.0]]), np.float32)
    assert np.isfinite(y).all() and abs(y.sum() - 1) < 1e-5 and y[0, 3] > 0.99
    # src/backend/tensor.rs:400-419
    assert np.allclose(R.softmax_stable(np.array([[7.0]])), 1.0)
    # tests/softmax_correctness.rs:107-141: constant rows, row sums 1 +- 1e-5
    for c in (100.0, -100.0):
        y = R.softmax_stable(np.full((4, 256), c), np.float32)
        assert np.allclose(y, 1 / 256) and np.abs(y.sum(-1) - 1).max() < 1e-5
    # -inf from an additive causal mask (src/models/transformer.rs:269-273)
    y = R.softmax_stable(np.array([[0.0, -np.inf, 0.0, -np.inf]]))
    assert np.allclose(y, [[0.5, 0, 0.5, 0]])


def test_lora_known_answers():
    # tests/executor_direct.rs:339-376: fixed inputs, scale 0.5 -> shape [2,4], non-zero
    x = np.array([[1.0, 2, 3, 4], [5, 6, 7, 8]])
    A = np.array([[0.1, 0.2], [0.3, 0.4], [0.5, 0.6], [0.7, 0.8]])
    B = np.array([[1.0, 2, 3, 4], [5, 6, 7, 8]])
    out, h = R.lora_forward(x, A, B, 0.5)
    assert out.shape == (2, 4) and (out != 0).all()
    assert np.allclose(h, [[5.0, 6.0], [11.4, 14.0]])          # by hand
    assert np.allclose(out[0], 0.5 * np.array([35.0, 46.0, 57.0, 68.0]))
    assert np.allclose(R.lora_forward_msl(x, A, B, 0.5), out, rtol=1e-6)
    # tests/lazy_execution.rs:54-74
    assert np.array_equal(R.matmul([[1, 2, 3], [4, 5, 6]], [[1, 2], [3, 4], [5, 6]]), [[22, 28], [49, 64]])
    # src/training/lora.rs:695-707: 768/768/r8 -> 12288 parameters; B = 0 -> zero delta (:645-660)
    assert 8 * (768 + 768) == 12_288
    out, _ = R.lora_forward(S.normal(0, "x", (4, 16)), S.normal(0, "a", (16, 2)), np.zeros((2, 16)), 2.0)
    assert (out == 0).all()


def test_scheduler_known_answers():
    # src/training/scheduler.rs:312-373,401-419
    assert abs(R.lr_constant(100, 1e-4) - 1e-4) < 1e-9
    assert abs(R.lr_linear(0, 1000, 1e-3)) < 1e-9
    assert abs(R.lr_linear(500, 1000, 1e-3) - 5e-4) < 1e-7
    assert abs(R.lr_linear(1000, 1000, 1e-3) - 1e-3) < 1e-9
    assert abs(R.lr_linear(2000, 1000, 1e-3) - 1e-3) < 1e-9
    assert abs(R.lr_cosine(0, 10_000, 1e-3, 1e-5) - 1e-3) < 1e-7
    assert 1e-5 < R.lr_cosine(5000, 10_000, 1e-3, 1e-5) < 1e-3
    assert abs(R.lr_cosine(10_000, 10_000, 1e-3, 1e-5) - 1e-5) < 1e-4
    assert abs(R.lr_warmup_cosine(0, 1000, 10_000, 1e-3, 1e-5)) < 1e-9
    assert abs(R.lr_warmup_cosine(500, 1000, 10_000, 1e-3, 1e-5) - 5e-4) < 1e-7
    assert abs(R.lr_warmup_cosine(1000, 1000, 10_000, 1e-3, 1e-5) - 1e-3) < 1e-7
    lrs = [R.lr_warmup_cosine(s, 1000, 10_000, 1e-3, 1e-5) for s in (1000, 5000, 9000, 10_000, 20_000)]
    assert all(a > b for a, b in zip(lrs[:3], lrs[1:4])) and abs(lrs[3] - 1e-5) < 1e-7 and lrs[4] == lrs[3]


def test_cross_entropy_known_answers():
    # src/training/loss.rs:252-284
    lg = np.array([[[10.0, 0.0, 0.0]]])
    assert R.cross_entropy_loss(lg, np.array([[0]]), None)[0] < 0.1
    assert R.cross_entropy_loss(lg, np.array([[2]]), None)[0] > 5.0
    # ignore index: only the kept positions contribute (loss.rs:286-320)
    lg = S.normal(3, "lg", (2, 2, 3))
    tg = np.array([[0, R.IGNORE_INDEX], [2, R.IGNORE_INDEX]])
    full, _ = R.cross_entropy_loss(lg, tg)
    kept, _ = R.cross_entropy_loss(lg[:, :1], tg[:, :1])
    assert abs(full - kept) < 1e-12
    with pytest.raises(ValueError, match="all tokens are ignored"):
        R.cross_entropy_loss(lg, np.full((2, 2), R.IGNORE_INDEX))


def test_adamw_defaults_and_first_step():
    # src/training/optimizer.rs:51-61
    assert R.ADAMW_DEFAULTS == dict(learning_rate=1e-4, beta1=0.9, beta2=0.999, epsilon=1e-8, weight_decay=0.01)
    # with zero state and t = 1, m_hat = g and v_hat = g^2: p' = p - lr*g/(|g|+eps) - wd*lr*p
    p = np.array([1.0, -2.0, 0.5], dtype=np.float32)
    g = np.array([0.3, -0.1, 0.0], dtype=np.float32)
    p2, m2, v2 = R.adamw_step(p, g, 0 * p, 0 * p, 1, 1e-3, 0.9, 0.999, 1e-8, 0.01)
    want = p - 1e-3 * g / (np.abs(g) + 1e-8) - 0.01 * 1e-3 * p
    assert np.allclose(p2, want, rtol=1e-5) and np.allclose(m2, 0.1 * g, rtol=1e-5)
    # the shared counter advances once per tensor (optimizer.rs:236-238)
    o = R.AdamWOracle()
    o.step("a", p, g)
    o.step("b", p, g)
    assert o.step_count == 2


# ---- (2) Metal kernel bodies vs. unfused op sequences --------------------------------------------
def test_msl_restatements_match_unfused():
    c = S.lora_linear_case(2, 6, 32, 24, 4)
    want, _ = R.lora_forward(c["x"], c["A"], c["B"], 2.0, np.float32)
    assert np.abs(R.lora_forward_msl(c["x"], c["A"], c["B"], 2.0) - want).max() < 1e-4
    x = S.normal(2, "r", (5, 64))
    assert np.abs(R.rms_norm_msl(x, 1e-5) - R.rms_norm(x, 1e-5, np.float32)).max() < 1e-4
    assert np.abs(R.softmax_msl(x) - R.softmax_stable(x, np.float32)).max() < 1e-4


# ---- (3) backward formulas -------------------------------------------------------------------------
def _fd(f, x, eps=1e-6):
    g = np.zeros_like(x)
    it = np.nditer(x, flags=["multi_index"])
    for _ in it:
        i = it.multi_index
        old = x[i]
        x[i] = old + eps
        fp = f()
        x[i] = old - eps
        fm = f()
        x[i] = old
        g[i] = (fp - fm) / (2 * eps)
    return g


def test_lora_backward_finite_differences_and_autograd():
    c = {k: v.astype(np.float64) for k, v in S.lora_linear_case(4, 5, 12, 10, 3).items()}
    x, W, A, B, dy = c["x"], c["W"], c["A"], c["B"], c["dy"]
    s = 2.0
    dx, dA, dB = R.lora_linear_backward(x, W, A, B, s, dy)
    loss = lambda: float((R.lora_linear_forward(x, W, None, A, B, s)[0] * dy).sum())
    assert np.allclose(dx, _fd(loss, x), atol=1e-6)
    assert np.allclose(dA, _fd(loss, A), atol=1e-6)
    assert np.allclose(dB, _fd(loss, B), atol=1e-6)
    tx, tA, tB = (torch.tensor(v, requires_grad=True) for v in (x, A, B))
    y = tx @ torch.tensor(W).T + (tx @ tA @ tB) * s
    (y * torch.tensor(dy)).sum().backward()
    assert np.allclose(dx, tx.grad.numpy()) and np.allclose(dA, tA.grad.numpy()) and np.allclose(dB, tB.grad.numpy())


def test_rmsnorm_softmax_ce_backward():
    c = {k: v.astype(np.float64) for k, v in S.rmsnorm_case(6, 4, 16).items()}
    x, w, dy = c["x"], c["w"], c["dy"]
    dx, dw = R.rms_norm_backward(x, w, 1e-6, dy)
    loss = lambda: float((R.rms_norm_weighted(x, w, 1e-6) * dy).sum())
    assert np.allclose(dx, _fd(loss, x), atol=1e-6) and np.allclose(dw, _fd(loss, w), atol=1e-6)
    sm = S.softmax_case(6, 1, 8)
    xs, dys = sm["x"].astype(np.float64), sm["dy"].astype(np.float64)
    t = torch.tensor(xs, requires_grad=True)
    (torch.softmax(t, -1) * torch.tensor(dys)).sum().backward()
    assert np.allclose(R.softmax_backward(R.softmax_stable(xs), dys), t.grad.numpy(), atol=1e-12)
    lg = S.normal(6, "lg", (2, 3, 7)).astype(np.float64)
    tg = np.array([[1, 2, R.IGNORE_INDEX], [0, 6, 3]])
    l, d = R.cross_entropy_loss(lg, tg)
    t = torch.tensor(lg, requires_grad=True)
    tt = torch.tensor(np.where(tg == R.IGNORE_INDEX, -100, tg))
    lt = torch.nn.functional.cross_entropy(t.reshape(-1, 7), tt.reshape(-1), ignore_index=-100)
    lt.backward()
    assert abs(l - float(lt)) < 1e-12 and np.allclose(d, t.grad.numpy(), atol=1e-12)


def test_adamw_matches_torch_adamw_up_to_bias_correction_form():
    """torch.optim.AdamW uses the same update when eps is negligible against sqrt(v_hat)."""
    p0 = S.normal(8, "p", (32,)).astype(np.float32)
    gs = [S.normal(8, f"g{i}", (32,)).astype(np.float32) for i in range(5)]
    tp = torch.tensor(p0.copy(), requires_grad=True)
    opt = torch.optim.AdamW([tp], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    p, m, v = p0.copy(), np.zeros_like(p0), np.zeros_like(p0)
    for t, g in enumerate(gs, 1):
        tp.grad = torch.tensor(g)
        opt.step()
        p, m, v = R.adamw_step(p, g, m, v, t, 1e-3, 0.9, 0.999, 1e-8, 0.01)
    assert np.allclose(p, tp.detach().numpy(), rtol=1e-5, atol=1e-6)


# ---- (4) committed fixtures ----------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["lora_c1_small", "rmsnorm_small", "softmax_small", "adamw_small"])
def test_oracle_reproduces_fixtures(name):
    from tests.golden import make_golden

    stored = np.load(GOLDEN / f"{name}.npz")
    fresh = make_golden.CASES[name]()
    assert set(stored.files) == set(fresh)
    for k in stored.files:
        assert np.allclose(stored[k], fresh[k], rtol=1e-6, atol=1e-7, equal_nan=True), (name, k)


def test_seeded_generator_is_stable():
    """First values of the documented splitmix64 streams (a change here invalidates every fixture)."""
    stored = np.load(GOLDEN / "generator.npz")
    assert np.array_equal(stored["u64"], S.raw_u64(S.DEFAULT_SEED, "pin", 8))
    assert np.array_equal(stored["normal"], S.normal(S.DEFAULT_SEED, "pin", (8,)))
    assert np.array_equal(stored["bf16"], S.bf16_bits(S.normal(S.DEFAULT_SEED, "pin", (8,))))
    # bf16 rounding agrees with torch's round-to-nearest-even
    x = S.normal(1, "b", (4096,)) * 100
    assert np.array_equal(S.bf16_round(x), torch.from_numpy(x).bfloat16().float().numpy())


def test_oracle_attention_matches_torch_autograd():
    """The attention restatement (forward and gradients) against torch-CPU autograd of the same op sequence
    as Attention::forward (src/models/transformer.rs:257-285): matmul, scale, additive mask, softmax, matmul."""
    import math

    import torch

    from oracle import reference_ops as R
    from oracle import seeded as S

    nb, G, seq, d = 2, 3, 16, 8
    q = S.normal(3, "q", (nb, G, seq, d)).astype(np.float64)
    k = S.normal(3, "k", (nb, seq, d)).astype(np.float64)
    v = S.normal(3, "v", (nb, seq, d)).astype(np.float64)
    do = S.normal(3, "do", (nb, G, seq, d)).astype(np.float64)
    scale = 1.0 / math.sqrt(d)
    tq, tk, tv = (torch.tensor(t, requires_grad=True) for t in (q, k, v))
    scores = torch.matmul(tq, tk[:, None].transpose(-1, -2)) * scale
    mask = torch.full((seq, seq), float("-inf"), dtype=torch.float64).triu(1)
    p = torch.softmax(scores + mask, dim=-1)
    o = torch.matmul(p, tv[:, None])
    o.backward(torch.tensor(do))
    wo, wlse, _ = R.causal_gqa_attention(q, k, v, scale)
    assert np.allclose(wo, o.detach().numpy(), atol=1e-12)
    assert np.allclose(wlse, torch.logsumexp(scores + mask, dim=-1).detach().numpy(), atol=1e-12)
    dq, dk, dv = R.causal_gqa_attention_backward(q, k, v, scale, do)
    assert np.allclose(dq, tq.grad.numpy(), atol=1e-12)
    assert np.allclose(dk, tk.grad.numpy(), atol=1e-12)
    assert np.allclose(dv, tv.grad.numpy(), atol=1e-12)
