"""GPU parity of the RMSNorm / softmax / AdamW kernels against the CPU oracle, through the C ABI.

Tolerances (max|gpu - oracle| / max|oracle|): float32 <= 1e-4, bfloat16 <= 2e-2, the oracle being the
float64 evaluation on the same (for bf16: bf16-rounded) inputs.
"""
import numpy as np
import pytest
import torch

from oracle import reference_ops as R
from oracle import seeded as S

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def to_dev(a, dtype, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(dtype).contiguous()


def as_input(a, dtype):
    """What the oracle should consume: the value the device actually holds."""
    return S.bf16_round(a) if dtype == torch.bfloat16 else a


def back(t):
    return t.detach().float().cpu().numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,D", [(64, 896), (33, 2048), (16, 4096), (7, 256), (5, 1024), (3, 8192),
                                      (9, 24), (4, 50), (2, 40000)])
@pytest.mark.parametrize("weighted", [False, True])
def test_rmsnorm_fwd_bwd(cuda_device, dtype, rows, D, weighted):
    from metal_candle_b200 import backend as B

    c = S.rmsnorm_case(1234, rows, D)
    x, w, dy = (as_input(c[k], dtype) for k in ("x", "w", "dy"))
    eps = 1e-6
    xd, wd, dyd = to_dev(x, dtype, cuda_device), to_dev(w, dtype, cuda_device), to_dev(dy, dtype, cuda_device)
    y, rstd = B.rms_norm_fused(xd, eps, weight=wd if weighted else None, return_rstd=True)
    want = R.rms_norm_weighted(x, w, eps) if weighted else R.rms_norm(x, eps)
    assert R.max_abs_normalised(back(y), want) <= TOL[dtype]
    want_rstd = 1.0 / np.sqrt(np.mean(x.astype(np.float64) ** 2, axis=-1) + eps)
    assert R.max_abs_normalised(back(rstd), want_rstd) <= 1e-5
    dx, dw = B.rms_norm_backward(xd, wd if weighted else None, dyd, eps, need_dw=True)
    wdx, wdw = R.rms_norm_backward(x, w if weighted else None, eps, dy)
    assert R.max_abs_normalised(back(dx), wdx) <= TOL[dtype]
    if weighted:
        assert R.max_abs_normalised(back(dw), wdw) <= 1e-4  # dw is accumulated and returned in float32
    else:
        # without a weight dw is sum(dy * xhat) all the same
        xh = R.rms_norm(x, eps)
        assert R.max_abs_normalised(back(dw), (dy.astype(np.float64) * xh).sum(0)) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,D", [(300, 896), (33, 2048), (16, 4096), (5, 1024), (3, 8192), (9, 24), (4, 50)])
@pytest.mark.parametrize("need_dw", [False, True])
def test_rmsnorm_bwd_with_residual(cuda_device, dtype, rows, D, need_dw):
    """dx = (gradient through the norm) + dx_residual in one kernel (rows that are not whole 16-byte vectors take
    the plain kernels plus an add): against the oracle's dx plus the residual; dw is unaffected."""
    from metal_candle_b200 import backend as B

    c = S.rmsnorm_case(4321, rows, D)
    x, w, dy = (as_input(c[k], dtype) for k in ("x", "w", "dy"))
    res = as_input(S.rmsnorm_case(99, rows, D)["dy"], dtype)
    eps = 1e-6
    xd, wd, dyd = to_dev(x, dtype, cuda_device), to_dev(w, dtype, cuda_device), to_dev(dy, dtype, cuda_device)
    resd = to_dev(res, dtype, cuda_device)
    dx, dw = B.rms_norm_backward(xd, wd, dyd, eps, need_dw=need_dw, dx_residual=resd)
    wdx, wdw = R.rms_norm_backward(x, w, eps, dy)
    assert R.max_abs_normalised(back(dx), wdx + res) <= TOL[dtype]
    if need_dw:
        assert R.max_abs_normalised(back(dw), wdw) <= 1e-4
    else:
        assert dw is None


def test_rmsnorm_known_answers(cuda_device):
    """The reference's own known-answer values (tests/executor_direct.rs:480-496,
    src/backend/tensor.rs:321-336,382-397)."""
    from metal_candle_b200 import backend as B

    y = back(B.rms_norm_fused(torch.tensor([[3.0, 4.0]], device=cuda_device), 0.0))
    assert np.allclose(y, [[0.8485, 1.1314]], atol=1e-3)
    y = back(B.rms_norm_fused(torch.ones(1, 4, device=cuda_device), 1e-5))
    assert np.allclose(y, 1.0, atol=1e-5)
    y = back(B.rms_norm_fused(torch.tensor([[2.0, 4.0, 6.0]], device=cuda_device), 1e-5))[0]
    assert abs(y[1] / y[0] - 2.0) < 1e-4 and abs(y[2] / y[0] - 3.0) < 1e-4
    # extreme magnitudes as in tests/rmsnorm_correctness.rs (large and tiny rows stay finite)
    big = torch.full((2, 512), 1.0e4, device=cuda_device)
    assert torch.isfinite(B.rms_norm_fused(big, 1e-5)).all()


def test_rmsnorm_accumulate_dw(cuda_device):
    from metal_candle_b200 import backend as B

    c = S.rmsnorm_case(5, 40, 896)
    xd, wd, dyd = (torch.from_numpy(c[k]).to(cuda_device) for k in ("x", "w", "dy"))
    _, dw1 = B.rms_norm_backward(xd, wd, dyd, 1e-6)
    acc = dw1.clone()
    B.rms_norm_backward(xd, wd, dyd, 1e-6, grad_w=acc, accumulate=True)
    assert torch.allclose(acc, 2 * dw1, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("blocks,Sq", [(3, 128), (2, 1024), (1, 200), (1, 24), (1, 4096), (1, 6000)])
def test_softmax_causal_fwd_bwd(cuda_device, dtype, blocks, Sq):
    from metal_candle_b200 import backend as B

    c = S.softmax_case(77, blocks, Sq, causal=True)
    x, dy = as_input(c["x"], dtype), as_input(c["dy"], dtype)
    xd, dyd = to_dev(x, dtype, cuda_device), to_dev(dy, dtype, cuda_device)
    y = B.softmax_fused(xd)
    want = R.softmax_stable(x)
    got = back(y)
    assert np.isfinite(got).all()
    assert R.max_abs_normalised(got, want) <= TOL[dtype]
    # row sums are 1 (tests/softmax_correctness.rs:132-136 uses 1e-5 for float32)
    assert np.abs(got.sum(-1) - 1.0).max() <= (1e-5 if dtype == torch.float32 else 2e-2)
    # masked entries are exactly zero
    assert (got[np.isneginf(x)] == 0).all()
    y_in = as_input(want.astype(np.float32), dtype)
    dx = B.softmax_backward(to_dev(y_in, dtype, cuda_device), dyd)
    assert R.max_abs_normalised(back(dx), R.softmax_backward(y_in, dy)) <= TOL[dtype]


def test_softmax_known_answers_and_edges(cuda_device):
    """src/backend/tensor.rs:262-275,400-419; tests/softmax_lazy.rs:137-169;
    tests/softmax_correctness.rs:107-141 (constant +-100 rows)."""
    from metal_candle_b200 import backend as B

    dev = cuda_device
    assert np.allclose(back(B.softmax_fused(torch.zeros(1, 3, device=dev))), 1 / 3, atol=1e-5)
    y = back(B.softmax_fused(torch.tensor([[100.0, 200.0, 300.0, 400.0]], device=dev)))
    assert np.isfinite(y).all() and abs(y.sum() - 1) < 1e-5 and y[0, 3] > 0.99
    assert np.allclose(back(B.softmax_fused(torch.tensor([[5.0]], device=dev))), 1.0)
    for c in (100.0, -100.0):
        y = back(B.softmax_fused(torch.full((4, 256), c, device=dev)))
        assert np.allclose(y, 1 / 256, atol=1e-6)
    # a fully masked row yields zeros, not NaN
    x = torch.full((2, 64), float("-inf"), device=dev)
    x[1, :3] = 0.0
    y = back(B.softmax_fused(x))
    assert (y[0] == 0).all() and np.allclose(y[1, :3], 1 / 3, atol=1e-6)
    # in place
    x = torch.randn(8, 1024, device=dev)
    ref = back(B.softmax_fused(x))
    B.softmax_fused(x, out=x)
    assert np.array_equal(back(x), ref)
    # 4-D scores (the model's [B,H,S,S]) are flattened, not rejected
    x4 = torch.randn(2, 3, 16, 16, device=dev)
    assert np.allclose(back(B.softmax_fused(x4)), R.softmax_stable(back(x4)), atol=1e-6)


def test_row_ops_reject_bad_arguments(cuda_device):
    from metal_candle_b200 import backend as B

    with pytest.raises(B.TrainingError):
        B.softmax_fused(torch.zeros(4, 4))  # CPU tensor: no fallback
    with pytest.raises(B.TrainingError):
        B.rms_norm_fused(torch.zeros((), device=cuda_device), 1e-5)
    with pytest.raises(B.TrainingError):
        B.rms_norm_fused(torch.zeros(2, 8, device=cuda_device, dtype=torch.float16), 1e-5)


def _adamw_case(seed, shapes):
    ps = [S.normal(seed, f"p{i}", s) for i, s in enumerate(shapes)]
    gs = [S.normal(seed, f"g{i}", s, 0.0, 0.1) for i, s in enumerate(shapes)]
    return ps, gs


@pytest.mark.parametrize("n_steps", [3])
def test_adamw_multi_matches_oracle(cuda_device, n_steps):
    """Shared per-tensor step counter as in the reference (src/training/optimizer.rs:236-238)."""
    from metal_candle_b200.training import AdamW, AdamWConfig

    shapes = [(896, 8), (8, 896), (896, 8), (8, 128), (5, 7), (1,)] + [(64, 4)] * 70
    ps, gs = _adamw_case(3, shapes)
    oracle = R.AdamWOracle(dtype=np.float32)
    opt = AdamW(AdamWConfig())
    dps = [torch.from_numpy(p.copy()).to(cuda_device) for p in ps]
    cur = [p.copy() for p in ps]
    for step in range(n_steps):
        lr = 1e-4 * (step + 1)
        oracle.set_lr(lr)
        opt.set_lr(lr)
        grads = [g * (1 + 0.1 * step) for g in gs]
        for i in range(len(shapes)):
            cur[i] = oracle.step(f"t{i}", cur[i], grads[i])
        opt.step_vars(dps, [torch.from_numpy(g).to(cuda_device) for g in grads])
    for i in range(len(shapes)):
        got = dps[i].cpu().numpy()
        assert np.allclose(got, cur[i], rtol=2e-6, atol=1e-9), i
        m, v = oracle.state[f"t{i}"]
        assert np.allclose(opt.state_of(dps[i])[0].cpu().numpy(), m, rtol=2e-6, atol=1e-12)
        assert np.allclose(opt.state_of(dps[i])[1].cpu().numpy(), v, rtol=2e-6, atol=1e-15)
    assert opt.step_count == oracle.step_count == n_steps * len(shapes)
