"""mcb_rmsnorm_bwd_noalloc: the RMSNorm reverse pass for callers that cannot allocate device memory.

Some embedders of this library own no allocator they may call at this point -- a runtime whose pool has
already taken the whole GPU, or a thread that must not trigger the device-wide synchronisation an
allocation brings -- so they cannot hand mcb_rmsnorm_bwd a workspace.  This variant keeps the dw partial
sums in an array built into the library.  The test calls it through the C ABI twice in a row (the array
keeps the first call's contents, which the second call must not be confused by) and compares with the
workspace-taking entry point and with the CPU oracle's RMSNorm reverse pass; it also checks that sizes past the
built-in limit are refused.

Collected last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_pair(lib, dev, rows, D, dtype, seed, weighted=True):
    from metal_candle_b200 import _lib, backend

    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(rows, D, device=dev, generator=g).to(dtype)
    dy = torch.randn(rows, D, device=dev, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(D, device=dev, generator=g)).to(dtype) if weighted else None
    code = _lib.MCB_BF16 if dtype == torch.bfloat16 else _lib.MCB_F32
    st = torch.cuda.current_stream().cuda_stream
    # existing entry point, caller-owned workspace
    ws = torch.empty(lib.mcb_rmsnorm_bwd_workspace_bytes(rows, D), dtype=torch.uint8, device=dev)
    dx_ref, dw_ref = torch.empty_like(x), torch.empty(D, device=dev)
    _lib.check(lib.mcb_rmsnorm_bwd(x.data_ptr(), w.data_ptr() if weighted else None, dy.data_ptr(), dx_ref.data_ptr(),
                                   dw_ref.data_ptr(), 0, rows, D, 1e-6, code, ws.data_ptr(), ws.numel(), st))
    # new entry point: inputs and outputs only
    dx, dw = torch.empty_like(x), torch.empty(D, device=dev)
    _lib.check(lib.mcb_rmsnorm_bwd_noalloc(x.data_ptr(), w.data_ptr() if weighted else None, dy.data_ptr(),
                                           dx.data_ptr(), dw.data_ptr(), 0, rows, D, 1e-6, code, st))
    torch.cuda.synchronize()
    # the CPU oracle on the same (already rounded) inputs: both entry points share kernels, so agreeing with each
    # other is not enough
    from oracle import reference_ops as R

    xw = x.float().cpu().numpy()
    ww = w.float().cpu().numpy() if weighted else np.ones(D, dtype=np.float32)
    odx, odw = R.rms_norm_backward(xw, ww, 1e-6, dy.float().cpu().numpy())
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert _close(dx.float().cpu().numpy(), odx, tol), "dx against the oracle"
    assert _close(dw.cpu().numpy(), odw, tol if dtype == torch.float32 else 1e-3), "dw against the oracle"
    return dx.float().cpu().numpy(), dw.cpu().numpy(), dx_ref.float().cpu().numpy(), dw_ref.cpu().numpy()


def _close(got, want, tol):
    den = max(np.abs(want).max(), 1e-30)
    return np.abs(got - want).max() / den <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_matches_workspace_entry_point_twice(cuda_device, dtype):
    from metal_candle_b200 import _lib

    lib = _lib.init(0)
    # first call: many rows so that the block count is capped differently in the two entry points;
    # second call: another shape, right after, reading a scratch array that still holds the first result
    for seed, (rows, D) in enumerate([(5000, 896), (333, 4096)]):
        dx, dw, dx_ref, dw_ref = _call_pair(lib, cuda_device, rows, D, dtype, seed)
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        assert _close(dx, dx_ref, tol)             # the two entry points may run different kernels
        assert _close(dw, dw_ref, 1e-4)            # dw is summed over a different number of partial rows
    # and once more with the first shape: no residue from the wider second call
    dx, dw, dx_ref, dw_ref = _call_pair(lib, cuda_device, 5000, 896, dtype, 0)
    assert _close(dx, dx_ref, 1e-4 if dtype == torch.float32 else 2e-2) and _close(dw, dw_ref, 1e-4)


def test_noalloc_accumulate_and_no_weight(cuda_device):
    from metal_candle_b200 import _lib

    lib = _lib.init(0)
    dx, dw, dx_ref, dw_ref = _call_pair(lib, cuda_device, 257, 2048, torch.float32, 7, weighted=False)
    assert _close(dx, dx_ref, 1e-4) and _close(dw, dw_ref, 1e-4)
    dx, dw, dx_ref, dw_ref = _call_pair(lib, cuda_device, 700, 896, torch.bfloat16, 8, weighted=False)
    assert _close(dx, dx_ref, 2e-2) and _close(dw, dw_ref, 1e-4)
    # dw not wanted: dx alone, against the oracle
    from oracle import reference_ops as R

    g = torch.Generator(device=cuda_device).manual_seed(9)
    x = torch.randn(300, 1024, device=cuda_device, generator=g)
    dy = torch.randn(300, 1024, device=cuda_device, generator=g)
    w = 1 + 0.1 * torch.randn(1024, device=cuda_device, generator=g)
    dx_only = torch.empty_like(x)
    _lib.check(lib.mcb_rmsnorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), dy.data_ptr(), dx_only.data_ptr(), None, 0, 300, 1024,
                                           1e-6, _lib.MCB_F32, torch.cuda.current_stream().cuda_stream))
    odx, _ = R.rms_norm_backward(x.cpu().numpy(), w.cpu().numpy(), 1e-6, dy.cpu().numpy())
    assert _close(dx_only.cpu().numpy(), odx, 1e-4)
    dev = cuda_device
    x = torch.randn(64, 256, device=dev)
    dy = torch.randn(64, 256, device=dev)
    dxb, dw = torch.empty_like(x), torch.zeros(256, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        _lib.check(lib.mcb_rmsnorm_bwd_noalloc(x.data_ptr(), None, dy.data_ptr(), dxb.data_ptr(), dw.data_ptr(), 1,
                                               64, 256, 1e-6, _lib.MCB_F32, st))
    once = torch.zeros(256, device=dev)
    _lib.check(lib.mcb_rmsnorm_bwd_noalloc(x.data_ptr(), None, dy.data_ptr(), dxb.data_ptr(), once.data_ptr(), 0,
                                           64, 256, 1e-6, _lib.MCB_F32, st))
    assert torch.allclose(dw, 2 * once, rtol=1e-6, atol=1e-6)


def test_noalloc_refuses_sizes_past_the_built_in_scratch(cuda_device):
    from metal_candle_b200 import _lib

    lib = _lib.init(0)
    dev = cuda_device
    x = torch.zeros(4, 8192, device=dev)
    out = torch.empty_like(x)
    dw = torch.empty(8192, device=dev)
    rc = lib.mcb_rmsnorm_bwd_noalloc(x.data_ptr(), None, x.data_ptr(), out.data_ptr(), dw.data_ptr(), 0, 4, 8192, 1e-6,
                                     _lib.MCB_F32, torch.cuda.current_stream().cuda_stream)
    assert rc == -2 and b"exceeds the built-in scratch limit" in lib.mcb_last_error()
    # a row width the vector kernels cannot take is refused too, not silently routed elsewhere
    y = torch.zeros(4, 30, device=dev)
    rc = lib.mcb_rmsnorm_bwd_noalloc(y.data_ptr(), None, y.data_ptr(), torch.empty_like(y).data_ptr(),
                                     torch.empty(30, device=dev).data_ptr(), 0, 4, 30, 1e-6, _lib.MCB_F32,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == -3
