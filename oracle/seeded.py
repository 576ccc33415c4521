"""Seeded synthetic-input generator shared by the oracle, the parity tests and the bench.

TEST INFRASTRUCTURE ONLY: nothing on the product path imports this package.

The reference (GarthDB/metal-candle) never seeds its test data (its hot-path tests draw
unseeded `Tensor::randn`, e.g. tests/custom_ops_correctness.rs:28-40), so the generator here
is this build's own definition.  One u64 seed per run; every tensor gets an independent
counter-based stream keyed by its name:

    key    = splitmix64(seed XOR fnv1a64(name))
    u64[i] = splitmix64(key + (i + 1) * 0x9E3779B97F4A7C15)
    uniform[i] = (u64[i] >> 40) * 2**-24                      in [0, 1)
    normal[i]  = sqrt(-2 ln u1) * cos(2 pi u2)                Box-Muller, one value per pair,
                 u1 = ((u64[2i] >> 40) + 1) * 2**-24  in (0, 1],   u2 = (u64[2i+1] >> 40) * 2**-24

The transcendental part is evaluated in float64 and rounded once to float32.
"""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
DEFAULT_SEED = 0x5EED


def _mix(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h ^= b
        h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def stream_key(seed: int, name: str) -> np.uint64:
    z = np.array([(seed ^ fnv1a64(name)) & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64)
    with np.errstate(over="ignore"):
        return _mix(z + _GOLDEN)[0]


def raw_u64(seed: int, name: str, n: int, offset: int = 0) -> np.ndarray:
    key = stream_key(seed, name)
    idx = np.arange(offset + 1, offset + n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        return _mix(key + idx * _GOLDEN)


def uniform01(seed: int, name: str, shape) -> np.ndarray:
    n = int(np.prod(shape)) if len(tuple(shape)) else 1
    u = (raw_u64(seed, name, n) >> np.uint64(40)).astype(np.float64) * 2.0 ** -24
    return u.astype(np.float32).reshape(shape)


def uniform(seed: int, name: str, shape, lo: float, hi: float) -> np.ndarray:
    n = int(np.prod(shape)) if len(tuple(shape)) else 1
    u = (raw_u64(seed, name, n) >> np.uint64(40)).astype(np.float64) * 2.0 ** -24
    return (lo + (hi - lo) * u).astype(np.float32).reshape(shape)


def normal(seed: int, name: str, shape, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape)) if len(tuple(shape)) else 1
    r = raw_u64(seed, name, 2 * n)
    u1 = ((r[0::2] >> np.uint64(40)).astype(np.float64) + 1.0) * 2.0 ** -24
    u2 = (r[1::2] >> np.uint64(40)).astype(np.float64) * 2.0 ** -24
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (mean + std * z).astype(np.float32).reshape(shape)


def token_ids(seed: int, name: str, shape, vocab: int) -> np.ndarray:
    n = int(np.prod(shape))
    r = raw_u64(seed, name, n) >> np.uint64(11)
    return (r % np.uint64(vocab)).astype(np.int64).reshape(shape)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16, returned as float32 holding the rounded value."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    lsb = (u >> np.uint64(16)) & np.uint64(1)
    r = (u + np.uint64(0x7FFF) + lsb) & np.uint64(0xFFFF0000)
    out = r.astype(np.uint32).view(np.float32).reshape(a.shape).copy()
    nan = np.isnan(a)
    out[nan] = np.nan
    inf = np.isinf(a)
    out[inf] = a[inf]
    return out


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> uint16 bfloat16 bit patterns (RNE)."""
    return (bf16_round(x).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


# ---------------------------------------------------------------------------------------------
# The synthetic workloads (shapes and value distributions of the benchmark configurations).
# ---------------------------------------------------------------------------------------------

def lora_linear_case(seed: int, M: int, K: int, N: int, r: int, tag: str = "lora"):
    """x~N(0,1), W[N,K]~N(0,1/K) (variance), A[K,r]~U(+-1/sqrt(K)), B[r,N]~N(0,0.02^2) (non-zero
    so that dA is non-trivial), dy~N(0,1).  W follows candle's Linear layout [out, in]."""
    s = 1.0 / np.sqrt(K)
    return dict(
        x=normal(seed, f"{tag}.x", (M, K)),
        W=normal(seed, f"{tag}.W", (N, K), 0.0, s),
        A=uniform(seed, f"{tag}.A", (K, r), -s, s),
        B=normal(seed, f"{tag}.B", (r, N), 0.0, 0.02),
        dy=normal(seed, f"{tag}.dy", (M, N)),
    )


def rmsnorm_case(seed: int, rows: int, D: int, tag: str = "rms"):
    return dict(
        x=normal(seed, f"{tag}.x", (rows, D)),
        w=normal(seed, f"{tag}.w", (D,), 1.0, 0.1),
        dy=normal(seed, f"{tag}.dy", (rows, D)),
    )


def softmax_case(seed: int, blocks: int, S: int, causal: bool = True, tag: str = "sm"):
    """Attention-score rows [blocks, S, S] ~ N(0, 3^2) with -inf strictly above each diagonal."""
    x = normal(seed, f"{tag}.x", (blocks, S, S), 0.0, 3.0)
    if causal:
        iu = np.triu_indices(S, k=1)
        x[:, iu[0], iu[1]] = -np.inf
    return dict(x=x.reshape(blocks * S, S), dy=normal(seed, f"{tag}.dy", (blocks * S, S)))
