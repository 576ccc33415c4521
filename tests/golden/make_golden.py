"""Generates the committed fixtures under tests/golden/ from the CPU oracle.

    python -m tests.golden.make_golden

The reference (Rust + candle, Metal shaders) cannot be built or run where these fixtures are made, and
it ships no golden files for this path, so the fixtures are outputs of oracle/reference_ops.py in
float64 on seeded inputs (oracle/seeded.py), stored as float32.  They pin the oracle against silent
change and give the GPU tests a second, file-based target.  Inputs are regenerated from the seed, so
only the expected outputs (and the shapes) are stored.
"""
from pathlib import Path

import numpy as np

from oracle import reference_ops as R
from oracle import seeded as S

HERE = Path(__file__).parent
SEED = S.DEFAULT_SEED


def lora_c1_small():
    """Benchmark configuration 1 at reduced token count: M=64 of [4,128] tokens, 768 -> 768, r=8, alpha=16."""
    c = S.lora_linear_case(SEED, 64, 768, 768, 8, tag="c1")
    y, h = R.lora_linear_forward(c["x"], c["W"], None, c["A"], c["B"], 2.0)
    dx, dA, dB = R.lora_linear_backward(c["x"], c["W"], c["A"], c["B"], 2.0, c["dy"])
    f = np.float32
    return dict(y=y.astype(f), h=h.astype(f), dx=dx.astype(f), dA=dA.astype(f), dB=dB.astype(f))


def rmsnorm_small():
    c = S.rmsnorm_case(SEED, 16, 896, tag="g.rms")
    y = R.rms_norm_weighted(c["x"], c["w"], 1e-6)
    dx, dw = R.rms_norm_backward(c["x"], c["w"], 1e-6, c["dy"])
    f = np.float32
    return dict(y=y.astype(f), dx=dx.astype(f), dw=dw.astype(f))


def softmax_small():
    c = S.softmax_case(SEED, 2, 64, causal=True, tag="g.sm")
    y = R.softmax_stable(c["x"])
    dx = R.softmax_backward(y, c["dy"])
    return dict(y=y.astype(np.float32), dx=dx.astype(np.float32))


def adamw_small():
    """Three tensors, four steps, shared step counter, WarmupCosine(2, 10, 1e-3, 1e-5) learning rates."""
    shapes = [(16, 4), (4, 24), (7,)]
    ps = [S.normal(SEED, f"g.p{i}", s) for i, s in enumerate(shapes)]
    o = R.AdamWOracle(dtype=np.float32)
    for step in range(4):
        o.set_lr(float(R.lr_warmup_cosine(step + 1, 2, 10, 1e-3, 1e-5)))
        for i, s in enumerate(shapes):
            ps[i] = o.step(f"t{i}", ps[i], S.normal(SEED, f"g.g{i}.{step}", s, 0.0, 0.1))
    out = {f"p{i}": ps[i] for i in range(3)}
    out.update({f"m{i}": o.state[f"t{i}"][0] for i in range(3)})
    out.update({f"v{i}": o.state[f"t{i}"][1] for i in range(3)})
    return out


CASES = dict(lora_c1_small=lora_c1_small, rmsnorm_small=rmsnorm_small, softmax_small=softmax_small,
             adamw_small=adamw_small)

if __name__ == "__main__":
    for name, fn in CASES.items():
        np.savez_compressed(HERE / f"{name}.npz", **fn())
    np.savez_compressed(HERE / "generator.npz", u64=S.raw_u64(SEED, "pin", 8), normal=S.normal(SEED, "pin", (8,)),
                        bf16=S.bf16_bits(S.normal(SEED, "pin", (8,))))
    for p in sorted(HERE.glob("*.npz")):
        print(p.name, p.stat().st_size)
