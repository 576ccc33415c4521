"""GPU parity of the fused causal attention kernels against the CPU oracle, through the C ABI.

Tolerance: max|gpu - oracle| / max|oracle| <= 2e-2 (bf16 path; the oracle is the float64 evaluation on the
bf16-rounded inputs); the log-sum-exp, kept in float32, within 2e-2 absolute (scores are rounded products of bf16).
"""
import math

import numpy as np
import pytest
import torch

from oracle import reference_ops as R
from oracle import seeded as S

pytestmark = pytest.mark.gpu


def _case(seed, nb, G, seq, d=64):
    q = S.bf16_round(S.normal(seed, "q", (nb, G, seq, d)))
    k = S.bf16_round(S.normal(seed, "k", (nb, seq, d)))
    v = S.bf16_round(S.normal(seed, "v", (nb, seq, d)))
    do = S.bf16_round(S.normal(seed, "do", (nb, G, seq, d)))
    return q, k, v, do


def _dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(torch.bfloat16).contiguous()


@pytest.mark.parametrize("nb,G,seq", [(1, 1, 128), (2, 2, 256), (3, 7, 384), (1, 3, 1024)])
def test_attention_forward(cuda_device, nb, G, seq):
    from metal_candle_b200 import _lib, backend as B

    q, k, v, _ = _case(77, nb, G, seq)
    scale = 1.0 / math.sqrt(64)
    want_o, want_lse, _ = R.causal_gqa_attention(q, k, v, scale)
    o, lse = B.attention_causal_forward(_dev(q.reshape(nb, G * seq, 64), cuda_device), _dev(k, cuda_device),
                                        _dev(v, cuda_device), G, scale)
    got = o.float().cpu().numpy().reshape(nb, G, seq, 64)
    assert R.max_abs_normalised(got, want_o) <= 2e-2
    assert np.abs(lse.cpu().numpy().reshape(nb, G, seq) - want_lse).max() <= 2e-2
    assert _lib.device_status() == 0


@pytest.mark.parametrize("nb,G,seq", [(1, 1, 128), (2, 2, 256), (3, 7, 384), (1, 3, 1024)])
def test_attention_backward(cuda_device, nb, G, seq):
    from metal_candle_b200 import _lib, backend as B

    q, k, v, do = _case(78, nb, G, seq)
    scale = 1.0 / math.sqrt(64)
    wdq, wdk, wdv = R.causal_gqa_attention_backward(q, k, v, scale, do)
    qd, kd, vd = _dev(q.reshape(nb, G * seq, 64), cuda_device), _dev(k, cuda_device), _dev(v, cuda_device)
    o, lse = B.attention_causal_forward(qd, kd, vd, G, scale)
    dq, dk, dv = B.attention_causal_backward(qd, kd, vd, o, lse, _dev(do.reshape(nb, G * seq, 64), cuda_device), G, scale)
    assert R.max_abs_normalised(dq.float().cpu().numpy().reshape(nb, G, seq, 64), wdq) <= 2e-2, "dq"
    assert R.max_abs_normalised(dk.float().cpu().numpy(), wdk) <= 2e-2, "dk"
    assert R.max_abs_normalised(dv.float().cpu().numpy(), wdv) <= 2e-2, "dv"
    assert _lib.device_status() == 0


def _token_major(a, batch, hkv, G, seq):
    """[batch*hkv, G, seq, d] (kv head fastest in the first index) -> [batch*seq, hkv*G*d], head kvh*G + g."""
    d = a.shape[-1]
    return np.ascontiguousarray(a.reshape(batch, hkv, G, seq, d).transpose(0, 3, 1, 2, 4).reshape(batch * seq, hkv * G * d))


@pytest.mark.parametrize("batch,hkv,G,seq", [(1, 1, 1, 128), (2, 2, 2, 256), (2, 2, 7, 384), (3, 1, 3, 256)])
def test_attention_token_major_output(cuda_device, batch, hkv, G, seq):
    """O written, and O / dO read, in the o_proj layout [batch*seq, heads*d]: forward against the oracle's output
    permuted into that layout; backward (with O and dO token-major) against the oracle's gradients."""
    from metal_candle_b200 import _lib, backend as B

    nb = batch * hkv
    q, k, v, do = _case(79, nb, G, seq)
    scale = 1.0 / math.sqrt(64)
    want_o, want_lse, _ = R.causal_gqa_attention(q, k, v, scale)
    wdq, wdk, wdv = R.causal_gqa_attention_backward(q, k, v, scale, do)
    qd, kd, vd = _dev(q.reshape(nb, G * seq, 64), cuda_device), _dev(k, cuda_device), _dev(v, cuda_device)
    o, lse = B.attention_causal_forward(qd, kd, vd, G, scale, kv_heads=hkv)
    assert tuple(o.shape) == (batch * seq, hkv * G * 64)
    assert R.max_abs_normalised(o.float().cpu().numpy(), _token_major(want_o, batch, hkv, G, seq)) <= 2e-2
    assert np.abs(lse.cpu().numpy().reshape(nb, G, seq) - want_lse).max() <= 2e-2
    dod = _dev(_token_major(do, batch, hkv, G, seq), cuda_device)
    dq, dk, dv = B.attention_causal_backward(qd, kd, vd, o, lse, dod, G, scale, kv_heads=hkv)
    assert R.max_abs_normalised(dq.float().cpu().numpy().reshape(nb, G, seq, 64), wdq) <= 2e-2, "dq"
    assert R.max_abs_normalised(dk.float().cpu().numpy(), wdk) <= 2e-2, "dk"
    assert R.max_abs_normalised(dv.float().cpu().numpy(), wdv) <= 2e-2, "dv"
    assert _lib.device_status() == 0


def test_attention_rejects_unsupported_shapes(cuda_device):
    from metal_candle_b200 import backend as B
    from metal_candle_b200._lib import McbError

    q = torch.zeros(1, 100, 64, device=cuda_device, dtype=torch.bfloat16)
    k = torch.zeros(1, 100, 64, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(McbError):
        B.attention_causal_forward(q, k, k.clone(), 1, 0.125)   # sequence not a multiple of 128
    assert not B.attention_supported(q, 100)
