"""GPU parity of the fused LoRA linear (forward, backward) against the CPU oracle, through the C ABI.

float32 validation path: max|gpu - oracle| / max|oracle| <= 1e-4 against the float64 oracle.
bfloat16 production path: <= 2e-2 against the float64 oracle evaluated on the bf16-rounded inputs.
"""
import numpy as np
import pytest
import torch

from oracle import reference_ops as R
from oracle import seeded as S

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def dev_t(a, dtype, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(dtype).contiguous()


def back(t):
    return t.detach().float().cpu().numpy()


def rounded(c, dtype):
    """Activations and the frozen weight live in `dtype`; A and B stay float32 masters, but the bf16 path
    rounds them to bf16 when packing its operands, so the oracle sees the same values."""
    if dtype == torch.float32:
        return dict(c)
    return {k: S.bf16_round(v) for k, v in c.items()}


def run_case(dev, dtype, M, K, N, r, seed=11, with_bias=True, save_h=True):
    from metal_candle_b200 import backend as B

    scale = 2.0
    c = S.lora_linear_case(seed, M, K, N, r)
    c["bias"] = S.normal(seed, "bias", (N,), 0.0, 0.1)
    o = rounded(c, dtype)
    x, W, dy = dev_t(o["x"], dtype, dev), dev_t(o["W"], dtype, dev), dev_t(o["dy"], dtype, dev)
    bias = dev_t(o["bias"], dtype, dev) if with_bias else None
    A, Bm = dev_t(c["A"], torch.float32, dev), dev_t(c["B"], torch.float32, dev)
    tol = TOL[dtype]

    # forward
    y, h = B.lora_linear_forward(x, W, bias, A, Bm, scale, save_hidden=save_h)
    want_y, want_h = R.lora_linear_forward(o["x"], o["W"], o["bias"] if with_bias else None, o["A"], o["B"], scale)
    assert R.max_abs_normalised(back(y), want_y) <= tol, "y"
    if save_h:
        assert R.max_abs_normalised(back(h)[:r, :M].T, scale * want_h) <= tol, "h_save"

    # delta only (the reference's FusedLoRAOp)
    d = B.lora_forward_fused(x, A, Bm, scale)
    want_d, _ = R.lora_forward(o["x"], o["A"], o["B"], scale)
    assert R.max_abs_normalised(back(d), want_d) <= tol, "delta"

    # backward
    Wt = B.transpose_2d(W)
    dx, dA, dB = B.lora_linear_backward(x, Wt, A, Bm, scale, dy, h_save=h)
    wdx, wdA, wdB = R.lora_linear_backward(o["x"], o["W"], o["A"], o["B"], scale, o["dy"])
    assert R.max_abs_normalised(back(dx), wdx) <= tol, "dx"
    assert R.max_abs_normalised(back(dA), wdA) <= tol, "dA"
    assert R.max_abs_normalised(back(dB), wdB) <= tol, "dB"
    from metal_candle_b200 import _lib
    assert _lib.device_status() == 0


# The reference benchmark shape (M = 4*128, 768 -> 768, r = 8) first, then Qwen2.5-0.5B projection shapes, ragged
# sizes (M, N, K not multiples of the tiles), and the rank range of tests/custom_ops_correctness.rs.
CASES = [
    (512, 768, 768, 8),
    (256, 896, 896, 8),
    (256, 896, 128, 8),
    (384, 896, 896, 16),
    (128, 512, 512, 4),
    (200, 264, 200, 8),
    (130, 64, 72, 16),
    (1000, 1024, 2048, 32),
    (300, 896, 4864, 8),
    (257, 2048, 896, 64),
    # large enough for the CTA-pair kernel: rank path in both directions (reduction >= 1536 forward and
    # backward), ragged tile edges; then the pair kernel without and the one-CTA kernel with the rank path
    (1280, 1536, 1600, 16),
    (1100, 1792, 1544, 64),
    (1024, 896, 1024, 8),
    # many CTAs in the backward kernel, whose tail phase (dA, dB) reads rank-intermediate rows written by other
    # CTAs of the same launch; ragged token count; the narrow k/v projection shape
    (4224, 896, 896, 16),
    (5000, 896, 128, 16),
    (20000, 1024, 512, 32),
    # the backward kernel is a single CTA: the gradients take their own launch
    (100, 128, 64, 4),
]


@pytest.mark.parametrize("M,K,N,r", CASES)
def test_lora_linear_f32(cuda_device, M, K, N, r):
    run_case(cuda_device, torch.float32, M, K, N, r)


@pytest.mark.parametrize("M,K,N,r", CASES)
def test_lora_linear_bf16(cuda_device, M, K, N, r):
    run_case(cuda_device, torch.bfloat16, M, K, N, r)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lora_variants(cuda_device, dtype):
    run_case(cuda_device, dtype, 256, 512, 512, 8, with_bias=False, save_h=False)


@pytest.mark.parametrize("M", [300, 1300])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_plain_linear_rank0(cuda_device, dtype, M):
    """r = 0: the frozen projection alone (k_proj, o_proj, MLP, lm_head in the training step); 1300 rows
    reach the CTA-pair kernel."""
    from metal_candle_b200 import backend as B

    K, N = 896, 1000 if dtype == torch.float32 else 1024
    c = rounded(S.lora_linear_case(5, M, K, N, 1), dtype)
    x, W, dy = (dev_t(c[k], dtype, cuda_device) for k in ("x", "W", "dy"))
    y, h = B.lora_linear_forward(x, W, None, None, None, 1.0)
    assert h is None
    assert R.max_abs_normalised(back(y), R.linear(c["x"], c["W"])) <= TOL[dtype]
    dx, dA, dB = B.lora_linear_backward(x, B.transpose_2d(W), None, None, 1.0, dy)
    assert dA is None and dB is None
    assert R.max_abs_normalised(back(dx), c["dy"].astype(np.float64) @ c["W"].astype(np.float64)) <= TOL[dtype]


@pytest.mark.parametrize("M,K,N,r", [(300, 896, 512, 8), (1100, 1792, 1600, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lora_linear_fused_residuals(cuda_device, dtype, M, K, N, r):
    """y = x W^T + s (x A) B + residual and dx = dy W + ... + dx_residual, the epilogue-fused adds that carry the
    model's residual connections (src/models/qwen.rs:121,140) and the sum of input gradients."""
    from metal_candle_b200 import backend as B

    scale = 2.0
    c = S.lora_linear_case(21, M, K, N, r)
    c["res"] = S.normal(21, "res", (M, N))
    c["dres"] = S.normal(21, "dres", (M, K))
    o = rounded(c, dtype)
    x, W, dy, res, dres = (dev_t(o[k], dtype, cuda_device) for k in ("x", "W", "dy", "res", "dres"))
    A, Bm = dev_t(c["A"], torch.float32, cuda_device), dev_t(c["B"], torch.float32, cuda_device)
    y, h = B.lora_linear_forward(x, W, None, A, Bm, scale, residual=res)
    want_y, _ = R.lora_linear_forward(o["x"], o["W"], None, o["A"], o["B"], scale)
    assert R.max_abs_normalised(back(y), want_y + o["res"]) <= TOL[dtype]
    dx, dA, dB = B.lora_linear_backward(x, B.transpose_2d(W), A, Bm, scale, dy, h_save=h, dx_residual=dres)
    wdx, wdA, wdB = R.lora_linear_backward(o["x"], o["W"], o["A"], o["B"], scale, o["dy"])
    assert R.max_abs_normalised(back(dx), wdx + o["dres"]) <= TOL[dtype]
    assert R.max_abs_normalised(back(dA), wdA) <= TOL[dtype] and R.max_abs_normalised(back(dB), wdB) <= TOL[dtype]


def test_lora_reference_fixed_inputs(cuda_device):
    """The fixed inputs of tests/executor_direct.rs:339-376: x [[1..4],[5..8]], A 4x2, B 2x4, scale 0.5."""
    from metal_candle_b200 import backend as B

    x = torch.tensor([[1.0, 2, 3, 4], [5, 6, 7, 8]], device=cuda_device)
    A = torch.tensor([[0.1, 0.2], [0.3, 0.4], [0.5, 0.6], [0.7, 0.8]], device=cuda_device)
    Bm = torch.tensor([[1.0, 2, 3, 4], [5, 6, 7, 8]], device=cuda_device)
    out = back(B.lora_forward_fused(x, A, Bm, 0.5))
    want = 0.5 * (back(x) @ back(A)) @ back(Bm)
    assert out.shape == (2, 4) and np.abs(out).min() > 0
    assert np.allclose(out, want, rtol=1e-5)
    assert np.allclose(out, R.lora_forward_msl(back(x), back(A), back(Bm), 0.5), rtol=1e-5)


def test_lora_batched_shapes_and_zero_b(cuda_device):
    """[2,64,512] r=8 as in tests/custom_ops_correctness.rs:16-85 (max-abs < 1e-4), 1-D and 2-D inputs
    (custom_ops.rs:254-270), and B = 0 (the initial state, src/training/lora.rs:244) gives exactly 0."""
    from metal_candle_b200 import backend as B
    from metal_candle_b200.training import LoRAConfig, LoRALayer

    g = torch.Generator(device=cuda_device).manual_seed(1)
    layer = LoRALayer(512, 512, LoRAConfig(), cuda_device, generator=g)
    x = torch.randn(2, 64, 512, device=cuda_device, generator=g)
    assert layer.forward(x).shape == (2, 64, 512)
    assert float(layer.forward(x).abs().max()) == 0.0
    layer.lora_b.normal_(0, 0.02, generator=g)
    got = back(layer.forward(x))
    want, _ = R.lora_forward(back(x), back(layer.lora_a), back(layer.lora_b), 2.0)
    assert np.abs(got - want).max() < 1e-4
    assert layer.forward(x[0]).shape == (64, 512)
    assert layer.forward(x[0, 0]).shape == (512,)
    assert np.abs(back(layer.forward(x[0, 0])) - want[0, 0]).max() < 1e-4


def test_lora_gradient_accumulation(cuda_device):
    from metal_candle_b200 import backend as B

    c = S.lora_linear_case(9, 256, 512, 384, 8)
    for dtype in (torch.float32, torch.bfloat16):
        x, W, dy = (dev_t(c[k], dtype, cuda_device) for k in ("x", "W", "dy"))
        A, Bm = dev_t(c["A"], torch.float32, cuda_device), dev_t(c["B"], torch.float32, cuda_device)
        Wt = B.transpose_2d(W)
        _, dA, dB = B.lora_linear_backward(x, Wt, A, Bm, 2.0, dy)
        ga, gb = dA.clone(), dB.clone()
        B.lora_linear_backward(x, Wt, A, Bm, 2.0, dy, grad_a=ga, grad_b=gb, accumulate=True)
        assert torch.allclose(ga, 2 * dA, rtol=1e-5, atol=1e-6) and torch.allclose(gb, 2 * dB, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("M,K,N,r", [(1024, 64, 128, 16), (1500, 1024, 1000, 16), (2048, 1536, 896, 16),
                                     (1100, 4864, 896, 32), (1024, 1600, 448, 64), (512, 64, 128, 16)])
def test_bf16_kernels_exact_on_small_integers(cuda_device, M, K, N, r):
    """Small-integer operands make every partial sum exact in fp32 and the rank intermediate exact in bf16,
    so the tensor-core kernels (one CTA and CTA pair, with bias and fused residual) must match an fp32
    matmul bit for bit after the final rounding, and the saved intermediate must be exact."""
    from metal_candle_b200 import _lib, backend as B

    g = torch.Generator(device="cpu").manual_seed(1000 * M + K + N + r)

    def ints(shape, lo=-2, hi=3):
        return torch.randint(lo, hi, shape, generator=g).float()

    x, W, res, bias = ints((M, K)), ints((N, K)), ints((M, N)), ints((N,))
    A = (torch.rand((K, r), generator=g) < 0.05).float() * ints((K, r), -1, 2)
    Bm = ints((r, N), -1, 2)
    dev = cuda_device
    y, h = B.lora_linear_forward(x.to(dev).bfloat16(), W.to(dev).bfloat16(), bias.to(dev).bfloat16(), A.to(dev),
                                 Bm.to(dev), 0.5, residual=res.to(dev).bfloat16())
    hb = (0.5 * (x @ A)).bfloat16().float()
    assert torch.equal(hb, 0.5 * (x @ A)), "test data: the intermediate must be exact in bf16"
    want = x @ W.T + bias + res + hb @ Bm
    assert torch.equal(h[:r, :M].float().T.cpu(), hb)
    assert torch.equal(y.float().cpu(), want.bfloat16().float())
    assert _lib.device_status() == 0


@pytest.mark.parametrize("M,K,F", [(300, 896, 256), (1300, 896, 4864), (2048, 256, 128)])
def test_linear_swiglu_forward(cuda_device, M, K, F):
    """gate = x Wg^T, up = x Wu^T, act = silu(gate) * up from one kernel, against the unfused restatement."""
    from metal_candle_b200 import _lib, backend as B

    x = S.bf16_round(S.normal(31, "x", (M, K)))
    wg = S.bf16_round(S.normal(31, "wg", (F, K)) / np.sqrt(K))
    wu = S.bf16_round(S.normal(31, "wu", (F, K)) / np.sqrt(K))
    xd, wgd, wud = (dev_t(a, torch.bfloat16, cuda_device) for a in (x, wg, wu))
    gate, up, act = B.linear_swiglu_forward(xd, B.interleave_gate_up(wgd, wud))
    want_g, want_u = R.linear(x, wg), R.linear(x, wu)
    want_a = want_g / (1.0 + np.exp(-want_g)) * want_u
    assert R.max_abs_normalised(back(gate), want_g) <= 2e-2
    assert R.max_abs_normalised(back(up), want_u) <= 2e-2
    assert R.max_abs_normalised(back(act), want_a) <= 2e-2
    assert _lib.device_status() == 0


@pytest.mark.parametrize("M,I,H,r", [(1300, 4864, 896, 0), (2048, 512, 1536, 16), (1100, 360, 896, 0), (4096, 1000, 2048, 8)])
def test_down_projection_backward_with_swiglu_epilogue(cuda_device, M, I, H, r):
    """mcb_lora_linear_bwd_swiglu: the input gradient of the MLP's down projection (I -> H, with and without an
    adapter) goes through the SwiGLU backward inside the GEMM's epilogue and replaces gate and up; against the CPU
    oracle's linear backward followed by the SwiGLU derivative.  Ragged rows and a width that is not a multiple of
    the 32-column store chunk included."""
    from metal_candle_b200 import _lib, backend as B

    dev, scale = cuda_device, 2.0
    c = S.lora_linear_case(77, M, I, H, max(r, 1))
    act64, W, dy = S.bf16_round(c["x"]), S.bf16_round(c["W"]), S.bf16_round(c["dy"])
    gate64 = S.bf16_round(S.normal(78, "gate", (M, I), 0.0, 1.5))
    up64 = S.bf16_round(S.normal(78, "up", (M, I)))
    A = S.bf16_round(c["A"]) if r else np.zeros((I, 1))
    Bm = S.bf16_round(c["B"]) if r else np.zeros((1, H))
    want_dact, want_dA, want_dB = R.lora_linear_backward(act64, W, A, Bm, scale if r else 0.0, dy)
    sg = 1.0 / (1.0 + np.exp(-gate64))
    want_dgate = want_dact * up64 * sg * (1.0 + gate64 * (1.0 - sg))
    want_dup = want_dact * gate64 * sg
    assert B.lora_linear_backward_swiglu_supported(M, I, H, r)
    gate, up = dev_t(gate64, torch.bfloat16, dev), dev_t(up64, torch.bfloat16, dev)
    wt = B.transpose_2d(dev_t(W, torch.bfloat16, dev))
    dyd = dev_t(dy, torch.bfloat16, dev)
    if r:
        actd = dev_t(act64, torch.bfloat16, dev)
        Ad, Bd = dev_t(c["A"], torch.float32, dev), dev_t(c["B"], torch.float32, dev)
        _, h = B.lora_linear_forward(actd, dev_t(W, torch.bfloat16, dev), None, Ad, Bd, scale)
        dA, dB = B.lora_linear_backward_swiglu(actd, wt, Ad, Bd, scale, dyd, gate, up, h_save=h)
        assert R.max_abs_normalised(back(dA), want_dA) <= 2e-2
        assert R.max_abs_normalised(back(dB), want_dB) <= 2e-2
    else:
        B.lora_linear_backward_swiglu(None, wt, None, None, 1.0, dyd, gate, up)
    assert R.max_abs_normalised(back(gate), want_dgate) <= 2e-2, "d gate"
    assert R.max_abs_normalised(back(up), want_dup) <= 2e-2, "d up"
    # the unfused pair of calls gives the same result up to the bf16 rounding of the stored activation gradient
    g2, u2 = dev_t(gate64, torch.bfloat16, dev), dev_t(up64, torch.bfloat16, dev)
    dact, _, _ = B.lora_linear_backward(actd if r else None, wt, Ad if r else None, Bd if r else None, scale if r else 1.0, dyd,
                                        h_save=h if r else None)
    _lib.check(_lib.load().mcb_swiglu_bwd(g2.data_ptr(), u2.data_ptr(), dact.data_ptr(), g2.data_ptr(), u2.data_ptr(), g2.numel(),
                                          _lib.MCB_BF16, torch.cuda.current_stream().cuda_stream))
    assert R.max_abs_normalised(back(gate), back(g2)) <= 1e-2 and R.max_abs_normalised(back(up), back(u2)) <= 1e-2
    assert _lib.device_status() == 0


def test_swiglu_epilogue_refuses_what_the_pair_kernel_does_not_take(cuda_device):
    from metal_candle_b200 import _lib, backend as B

    dev = cuda_device
    assert not B.lora_linear_backward_swiglu_supported(300, 4864, 896, 0)        # too few rows for CTA pairs
    assert not B.lora_linear_backward_swiglu_supported(4096, 4864, 896, 16)      # rank path with a short reduction
    assert not B.lora_linear_backward_swiglu_supported(4096, 4864, 896, 0, torch.float32)
    g = torch.zeros(300, 256, device=dev, dtype=torch.bfloat16)
    with pytest.raises(_lib.McbError, match="does not run on CTA pairs"):
        B.lora_linear_backward_swiglu(None, torch.zeros(256, 128, device=dev, dtype=torch.bfloat16), None, None, 1.0,
                                      torch.zeros(300, 128, device=dev, dtype=torch.bfloat16), g, torch.zeros_like(g))


def test_lora_rejects_bad_arguments(cuda_device):
    from metal_candle_b200 import backend as B

    dev = cuda_device
    x = torch.zeros(4, 16, device=dev)
    with pytest.raises(B.TrainingError, match="LoRA matrices must be 2D"):
        B.lora_forward_fused(x, torch.zeros(16, device=dev), torch.zeros(2, 8, device=dev), 1.0)
    with pytest.raises(B.TrainingError, match="Incompatible LoRA matrix dimensions"):
        B.lora_forward_fused(x, torch.zeros(16, 2, device=dev), torch.zeros(3, 8, device=dev), 1.0)
    with pytest.raises(B.TrainingError, match="Input feature dimension mismatch: expected 8, got 16"):
        B.lora_forward_fused(x, torch.zeros(8, 2, device=dev), torch.zeros(2, 8, device=dev), 1.0)
    with pytest.raises(B.TrainingError):
        B.lora_forward_fused(x.cpu(), torch.zeros(16, 2), torch.zeros(2, 8), 1.0)
    with pytest.raises(B.TrainingError, match="float32 master copies"):
        B.lora_forward_fused(x.bfloat16(), torch.zeros(16, 2, device=dev, dtype=torch.bfloat16),
                             torch.zeros(2, 8, device=dev, dtype=torch.bfloat16), 1.0)
    # bf16 path: feature counts must be multiples of 8 (TMA row pitch)
    xb = torch.zeros(4, 20, device=dev, dtype=torch.bfloat16)
    with pytest.raises(B.TrainingError):
        B.lora_forward_fused(xb, torch.zeros(20, 2, device=dev), torch.zeros(2, 8, device=dev), 1.0)


@pytest.mark.parametrize("M,r,which", [(300, 16, (0, 1, 2)), (1300, 8, (0, 2)), (4224, 16, (0, 1, 2)), (256, 4, (1,))])
def test_fused_projections_with_block_diagonal_rank_path(cuda_device, M, r, which):
    """mcb_lora_linear_fused_fwd / _bwd: the q, k and v projections of the 0.5B model (896 -> 896, 128, 128) as one
    linear with one adapter per listed projection.  Every projection's output, the summed input gradient and every
    adapter's dA / dB against the CPU oracle applied projection by projection; then once more accumulating."""
    from metal_candle_b200 import _lib
    from metal_candle_b200 import backend as B

    dev, K, widths, scale = cuda_device, 896, (896, 128, 128), 2.0
    offs = (0, 896, 1024)
    cases = [S.lora_linear_case(30 + i, M, K, n, r) for i, n in enumerate(widths)]
    x64 = S.bf16_round(cases[0]["x"])
    xd = dev_t(x64, torch.bfloat16, dev)
    Ws = [S.bf16_round(c["W"]) for c in cases]
    biases = [S.bf16_round(S.normal(40 + i, "bias", (n,), 0.0, 0.1)) for i, n in enumerate(widths)]
    dys = [S.bf16_round(c["dy"]) for c in cases]
    Wcat = dev_t(np.concatenate(Ws, 0), torch.bfloat16, dev)
    bcat = dev_t(np.concatenate(biases, 0), torch.bfloat16, dev)
    dycat = dev_t(np.concatenate(dys, 1), torch.bfloat16, dev)
    segs = []
    for i in which:
        segs.append(dict(A=dev_t(cases[i]["A"], torch.float32, dev), B=dev_t(cases[i]["B"], torch.float32, dev), offset=offs[i],
                         dA=torch.full((K, r), 7.0, device=dev), dB=torch.full((r, widths[i]), 7.0, device=dev)))
    y, h = B.lora_linear_fused_forward(xd, Wcat, bcat, segs, scale)
    dx = B.lora_linear_fused_backward(xd, B.transpose_2d(Wcat), segs, scale, dycat, h)
    want_dx = 0.0
    for i, n in enumerate(widths):
        A = S.bf16_round(cases[i]["A"]) if i in which else np.zeros((K, r))
        Bm = S.bf16_round(cases[i]["B"]) if i in which else np.zeros((r, n))
        wy, _ = R.lora_linear_forward(x64, Ws[i], biases[i], A, Bm, scale)
        assert R.max_abs_normalised(back(y)[:, offs[i]:offs[i] + n], wy) <= 2e-2, f"y of projection {i}"
        wdx, wdA, wdB = R.lora_linear_backward(x64, Ws[i], A, Bm, scale, dys[i])
        want_dx = want_dx + wdx
        if i in which:
            sg = segs[which.index(i)]
            assert R.max_abs_normalised(back(sg["dA"]), wdA) <= 2e-2, f"dA of projection {i}"
            assert R.max_abs_normalised(back(sg["dB"]), wdB) <= 2e-2, f"dB of projection {i}"
    assert R.max_abs_normalised(back(dx), want_dx) <= 2e-2, "dx"
    # accumulate: a second backward adds the same gradients once more
    once = [(sg["dA"].clone(), sg["dB"].clone()) for sg in segs]
    B.lora_linear_fused_backward(xd, B.transpose_2d(Wcat), segs, scale, dycat, h, accumulate=True)
    for sg, (a1, b1) in zip(segs, once):
        assert torch.allclose(sg["dA"], 2 * a1, rtol=1e-6, atol=1e-6) and torch.allclose(sg["dB"], 2 * b1, rtol=1e-6, atol=1e-6)
    assert _lib.device_status() == 0


def test_fused_projections_reject_bad_segments(cuda_device):
    from metal_candle_b200 import _lib
    from metal_candle_b200 import backend as B

    dev = cuda_device
    x = torch.zeros(64, 128, device=dev, dtype=torch.bfloat16)
    W = torch.zeros(256, 128, device=dev, dtype=torch.bfloat16)
    mk = lambda n, off: dict(A=torch.zeros(128, 8, device=dev), B=torch.zeros(8, n, device=dev), offset=off)
    with pytest.raises(_lib.McbError, match="ascending and disjoint"):
        B.lora_linear_fused_forward(x, W, None, [mk(128, 0), mk(128, 64)], 1.0)
    with pytest.raises(_lib.McbError, match="ascending and disjoint"):
        B.lora_linear_fused_forward(x, W, None, [mk(128, 192)], 1.0)
    with pytest.raises(_lib.McbError, match="bfloat16 only"):
        B.lora_linear_fused_forward(x.float(), W.float(), None, [mk(128, 0)], 1.0)
    with pytest.raises(_lib.McbError, match="64 rank columns"):
        big = lambda off: dict(A=torch.zeros(128, 32, device=dev), B=torch.zeros(32, 64, device=dev), offset=off)
        B.lora_linear_fused_forward(x, W, None, [big(0), big(64), big(128)], 1.0)


def test_dropout_mask_and_lora_layer_training_forward(cuda_device):
    """mcb_dropout against the oracle's restatement of its counter-based mask (bit for bit), and LoRALayer.forward in
    training mode with dropout > 0 (the reference's unfused branch, src/training/lora.rs:312-339) against the oracle
    with the same mask; eval mode stays on the fused kernel."""
    from metal_candle_b200 import _lib, backend as B
    from metal_candle_b200.training import LoRAConfig, LoRALayer

    dev = cuda_device
    x = S.normal(3, "x", (1000, 37)).astype(np.float32)
    for dtype, p, seed, off in ((torch.float32, 0.25, 99, 0), (torch.bfloat16, 0.1, 2**40 + 5, 123457), (torch.float32, 0.0, 1, 0)):
        xd = torch.from_numpy(x).to(dev).to(dtype)
        got = B.dropout(xd, p, seed, off).float().cpu().numpy()
        keep = R.dropout_mask(x.size, p, seed, off).reshape(x.shape)
        ref = xd.float().cpu().numpy()
        assert np.array_equal(got != 0, keep & (ref != 0))
        want = np.where(keep, ref / np.float32(1.0 - p), 0.0)
        assert R.max_abs_normalised(got, want) <= (1e-6 if dtype == torch.float32 else 4e-3)
        assert abs(keep.mean() - (1.0 - p)) < 5e-3
    with pytest.raises(_lib.McbError, match="not in"):
        B.dropout(torch.zeros(8, device=dev), 1.0, 0, 0)
    # the layer
    layer = LoRALayer(64, 48, LoRAConfig(rank=8, alpha=16.0, dropout=0.2), dev, generator=torch.Generator(device=dev).manual_seed(5))
    layer.lora_b.copy_(torch.from_numpy(S.normal(4, "B", (8, 48), 0.0, 0.05)).float())
    layer.dropout_seed = 4242
    xin = S.normal(6, "xin", (3, 50, 64)).astype(np.float32)
    xd = torch.from_numpy(xin).to(dev)
    A, Bm = layer.lora_a.cpu().numpy(), layer.lora_b.cpu().numpy()
    y1 = layer.forward(xd).cpu().numpy()
    assert layer.last_dropout == (4242, 0) and layer.dropout_offset == 3 * 50 * 8
    want1 = R.lora_forward_dropout(xin.reshape(-1, 64), A, Bm, layer.config.scaling(), 0.2, 4242, 0).reshape(3, 50, 48)
    assert R.max_abs_normalised(y1, want1) <= 1e-4
    y2 = layer.forward(xd).cpu().numpy()                     # the next call draws the next part of the stream
    want2 = R.lora_forward_dropout(xin.reshape(-1, 64), A, Bm, layer.config.scaling(), 0.2, 4242, 3 * 50 * 8).reshape(3, 50, 48)
    assert R.max_abs_normalised(y2, want2) <= 1e-4 and not np.allclose(y1, y2)
    layer.eval()
    y3 = layer.forward(xd).cpu().numpy()
    assert R.max_abs_normalised(y3, R.lora_forward(xin.reshape(-1, 64), A, Bm, layer.config.scaling())[0].reshape(3, 50, 48)) <= 1e-4
    assert _lib.device_status() == 0
