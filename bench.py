#!/usr/bin/env python
"""Benchmarks of the B200 LoRA hot path.

Headline (the line the driver reads):
    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
        one LoRA training step (forward + backward + AdamW) on the Qwen2.5-0.5B-shaped decoder,
        batch-data-parallel over N GPUs; prints ONE JSON line (tokens/s).

Kernel micro-benchmarks (one JSON line per case; used for the roofline sweeps and for ncu captures):
    python bench.py --micro lora    --M 32768 --K 896 --N 896 --r 16 [--dtype bf16|f32] [--pass fwd|bwd|both]
    python bench.py --micro lora_qkv --M 32768 --r 16 [--pass fwd|bwd|both]     (q, k, v projections as one fused linear)
    python bench.py --micro attention --nb 32 --G 7 --S 2048 [--pass fwd|bwd|both]
    python bench.py --micro rmsnorm --rows 114688 --D 896  [--dtype bf16|f32]
    python bench.py --micro softmax --rows 114688 --D 1024 [--dtype bf16|f32]
    python bench.py --micro adamw   --n 67108864
    python bench.py --sweep c2 | c3          the row-kernel / LoRA-GEMM sweeps of the benchmark configurations

All inputs are synthetic (seeded torch generators on the device; shapes and value distributions of the
benchmark configurations).  Kernel timings use CUDA events on the launching stream and rotate through
enough input copies that the working set exceeds twice the 126 MB L2.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
NO_GRAPH = False  # --no-graph: time launch by launch (what profiler captures use)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # under load = samples in the upper half of what was seen
        busy = [s for s in sm if s >= 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _time_kernel(torch, fn, n_variants, iters, warmup):
    """fn(i) launches the kernel(s) on input set i % n_variants.  The `iters` launches are captured into one
    CUDA graph and the graph is replayed, so that what is timed (CUDA events on the replay stream) is the
    device time of the kernels back to back and not the Python launch path.  Returns (median_ms, min_ms)
    per iteration over five replays."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    try:
        if NO_GRAPH:
            raise RuntimeError("--no-graph")
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(iters):
                    fn(warmup + i)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / iters)
        return statistics.median(ts), min(ts)
    except Exception as e:  # capture refused: time launch by launch
        if not NO_GRAPH:
            sys.stderr.write(f"graph capture failed ({e!r}); timing individual launches\n")
        torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for i, (a, b) in enumerate(evs):
        a.record()
        fn(warmup + i)
        b.record()
    torch.cuda.synchronize()
    ts = [a.elapsed_time(b) for a, b in evs]
    return statistics.median(ts), min(ts)


def _variants(bytes_per_set: int) -> int:
    return max(2, min(64, math.ceil(2.2 * L2_BYTES / max(1, bytes_per_set))))


def micro_lora(torch, M, K, N, r, dtype, which, iters=20, warmup=5):
    from metal_candle_b200 import backend as B

    dev = torch.device("cuda", 0)
    dt = torch.bfloat16 if dtype == "bf16" else torch.float32
    e = 2 if dtype == "bf16" else 4
    g = torch.Generator(device=dev).manual_seed(0x5EED)
    nv = _variants((M * K + M * N) * e)
    nv = min(nv, max(2, int(40e9 // max(1, (2 * M * K + 2 * M * N) * e))))
    xs = [torch.randn(M, K, device=dev, generator=g).to(dt) for _ in range(nv)]
    dys = [torch.randn(M, N, device=dev, generator=g).to(dt) for _ in range(nv)]
    W = (torch.randn(N, K, device=dev, generator=g) / math.sqrt(K)).to(dt)
    Wt = B.transpose_2d(W)
    s = 1.0 / math.sqrt(K)
    A = ((torch.rand(K, max(r, 1), device=dev, generator=g) * 2 - 1) * s) if r else None
    Bm = (torch.randn(max(r, 1), N, device=dev, generator=g) * 0.02) if r else None
    scale = 2.0
    hs = [None] * nv
    for i in range(nv):
        _, hs[i] = B.lora_linear_forward(xs[i], W, None, A, Bm, scale)
    dA = torch.zeros(K, r, device=dev) if r else None
    dB = torch.zeros(r, N, device=dev) if r else None

    def fwd(i):
        B.lora_linear_forward(xs[i % nv], W, None, A, Bm, scale)

    def bwd(i):
        B.lora_linear_backward(xs[i % nv], Wt, A, Bm, scale, dys[i % nv], h_save=hs[i % nv], grad_a=dA, grad_b=dB)

    def both(i):
        fwd(i)
        bwd(i)

    lib = B._lib_for(xs[0])
    dxbuf = torch.empty(M, K, device=dev, dtype=dt)
    ws = B.workspace(dev, lib.mcb_lora_workspace_bytes(M, K, N, r, B._dtype_code(xs[0])))

    def bwd_dx(i):   # dx alone (no dA / dB): what the rank path costs the backward GEMM by itself
        from metal_candle_b200 import _lib as L
        L.check(lib.mcb_lora_linear_bwd(xs[i % nv].data_ptr(), Wt.data_ptr(), A.data_ptr() if r else None,
                                        Bm.data_ptr() if r else None, dys[i % nv].data_ptr(), None, dxbuf.data_ptr(), None, None,
                                        0, M, K, N, r, scale, B._dtype_code(xs[0]), L.MCB_W_IN_OUT, ws.data_ptr(), ws.numel(),
                                        torch.cuda.current_stream().cuda_stream))

    fl_f = 2 * M * K * N + 2 * M * r * (K + N)
    fl_b = 2 * M * K * N + 4 * M * r * (K + N)
    by_f = e * (M * K + K * N + M * N) + e * r * (K + N)
    by_b = e * (M * N + K * N + 2 * M * K) + 6 * r * (K + N)
    fn, fl, by = {"fwd": (fwd, fl_f, by_f), "bwd": (bwd, fl_b, by_b), "both": (both, fl_f + fl_b, by_f + by_b),
                  "bwd_dx": (bwd_dx, fl_f, by_f)}[which]
    med, mn = _time_kernel(torch, fn, nv, iters, warmup)
    pk = measured_peaks()
    tf = fl / med / 1e9
    gbs = by / med / 1e6
    ridge = pk["bf16_tflops"] * 1e3 / pk["hbm_gbs"]
    bound = "tensor" if (dtype == "bf16" and fl / by >= ridge) else "hbm"
    roof = ({"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
             "frac": tf / pk["bf16_tflops"]} if bound == "tensor" else
            {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"]})
    roof["traffic"] = None
    roof["peak_source"] = pk["source"]
    return {"metric": f"fused LoRA linear {which}", "value": tf, "unit": "TFLOP/s", "ms": med, "ms_min": mn,
            "dtype": dtype, "config": {"workload": "lora_linear", "M": M, "K": K, "N": N, "r": r, "pass": which,
                                       "input_sets": nv, "l2": "inputs rotated through >2x L2"},
            "flop_per_byte": fl / by, "roofline": roof}


def micro_lora_qkv(torch, M, r, which, iters=20, warmup=5):
    """The 0.5B model's q, k and v projections (896 -> 896 + 128 + 128) as one fused linear with three adapters of
    rank r (mcb_lora_linear_fused_*).  Algorithmic FLOP = the three projections' own 2MKN + 2Mr(K+N) forward and
    2MKN + 4Mr(K+N) backward (the zero blocks of the block-diagonal rank path are not counted)."""
    from metal_candle_b200 import backend as B

    dev = torch.device("cuda", 0)
    K, widths = 896, (896, 128, 128)
    N = sum(widths)
    g = torch.Generator(device=dev).manual_seed(0x5EED)
    nv = max(2, min(8, _variants((M * K + M * N) * 2)))
    xs = [torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16) for _ in range(nv)]
    dys = [torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16) for _ in range(nv)]
    W = (torch.randn(N, K, device=dev, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    Wt = B.transpose_2d(W)
    bias = torch.zeros(N, device=dev, dtype=torch.bfloat16)
    segs, off = [], 0
    for n in widths:
        segs.append(dict(A=(torch.rand(K, r, device=dev, generator=g) * 2 - 1) / math.sqrt(K), B=torch.randn(r, n, device=dev, generator=g) * 0.02,
                         dA=torch.zeros(K, r, device=dev), dB=torch.zeros(r, n, device=dev), offset=off))
        off += n
    hs = [B.lora_linear_fused_forward(xs[i], W, bias, segs, 2.0)[1] for i in range(nv)]

    def fwd(i):
        B.lora_linear_fused_forward(xs[i % nv], W, bias, segs, 2.0)

    def bwd(i):
        B.lora_linear_fused_backward(xs[i % nv], Wt, segs, 2.0, dys[i % nv], hs[i % nv])

    def both(i):
        fwd(i)
        bwd(i)

    fl_f = sum(2 * M * K * n + 2 * M * r * (K + n) for n in widths)
    fl_b = sum(2 * M * K * n + 4 * M * r * (K + n) for n in widths)
    by_f = 2 * (M * K + K * N + M * N) + sum(2 * r * (K + n) for n in widths)
    by_b = 2 * (M * N + K * N + 2 * M * K) + sum(6 * r * (K + n) for n in widths)
    fn, fl, by = {"fwd": (fwd, fl_f, by_f), "bwd": (bwd, fl_b, by_b), "both": (both, fl_f + fl_b, by_f + by_b)}[which]
    med, mn = _time_kernel(torch, fn, nv, iters, warmup)
    pk = measured_peaks()
    tf = fl / med / 1e9
    return {"metric": f"fused q/k/v LoRA linear {which}", "value": tf, "unit": "TFLOP/s", "ms": med, "ms_min": mn, "dtype": "bf16",
            "config": {"workload": "lora_linear_qkv", "M": M, "K": K, "N": list(widths), "r": r, "pass": which, "input_sets": nv,
                       "l2": "inputs rotated through >2x L2"},
            "flop_per_byte": fl / by,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / pk["bf16_tflops"],
                         "traffic": None, "peak_source": pk["source"]}}


def micro_mlp_down_bwd(torch, M, I, H, which, iters=20, warmup=5):
    """Backward of the MLP's down projection (I -> H, no adapter) up to d gate / d up: `fused` = the SwiGLU backward in
    the GEMM's epilogue (mcb_lora_linear_bwd_swiglu), `unfused` = mcb_lora_linear_bwd_ex + mcb_swiglu_bwd, `gemm` = the
    input-gradient GEMM alone.  gate and up are updated in place, so later launches work on earlier results (the
    timing does not depend on the values).  Algorithmic bytes: dy + W + gate, up read and written once each."""
    from metal_candle_b200 import _lib, backend as B

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0x5EED)
    nv = max(1, min(4, _variants(4 * M * I * 2)))
    dys = [torch.randn(M, H, device=dev, generator=g).to(torch.bfloat16) for _ in range(nv)]
    gates = [torch.randn(M, I, device=dev, generator=g).to(torch.bfloat16) for _ in range(nv)]
    ups = [torch.randn(M, I, device=dev, generator=g).to(torch.bfloat16) for _ in range(nv)]
    wt = (torch.randn(I, H, device=dev, generator=g) / math.sqrt(I)).to(torch.bfloat16)
    dact = torch.empty(M, I, device=dev, dtype=torch.bfloat16)
    lib = _lib.load()

    def gemm(i):
        B.lora_linear_backward(None, wt, None, None, 1.0, dys[i % nv], dx_out=dact)

    def unfused(i):
        gemm(i)
        gt, up = gates[i % nv], ups[i % nv]
        _lib.check(lib.mcb_swiglu_bwd(gt.data_ptr(), up.data_ptr(), dact.data_ptr(), gt.data_ptr(), up.data_ptr(), gt.numel(),
                                      _lib.MCB_BF16, torch.cuda.current_stream().cuda_stream))

    def fused(i):
        B.lora_linear_backward_swiglu(None, wt, None, None, 1.0, dys[i % nv], gates[i % nv], ups[i % nv])

    fn = {"gemm": gemm, "unfused": unfused, "fused": fused}[which]
    med, mn = _time_kernel(torch, fn, nv, iters, warmup)
    pk = measured_peaks()
    fl = 2.0 * M * I * H
    by = 2.0 * (M * H + I * H + (1 if which == "gemm" else 4) * M * I)
    tf, gbs = fl / med / 1e9, by / med / 1e6
    return {"metric": f"MLP down projection backward ({which})", "value": med * 1e3, "unit": "us", "ms": med, "ms_min": mn, "dtype": "bf16",
            "higher_is_better": False, "tflops": tf, "algorithmic_GBps": gbs,
            "config": {"workload": "mlp_down_bwd", "M": M, "I": I, "H": H, "pass": which, "input_sets": nv,
                       "l2": "operands larger than L2"},
            "roofline": {"bound": "hbm" if which != "gemm" else "tensor", "achieved": gbs if which != "gemm" else tf,
                         "peak": pk["hbm_gbs"] if which != "gemm" else pk["bf16_tflops"], "unit": "GB/s" if which != "gemm" else "TFLOP/s",
                         "frac": (gbs / pk["hbm_gbs"]) if which != "gemm" else tf / pk["bf16_tflops"], "traffic": None,
                         "peak_source": pk["source"]}}


def micro_cross_entropy(torch, rows, V, iters=10, warmup=3):
    """One chunk of the loss stage: mcb_cross_entropy_chunk over [rows, V] bf16 logits, the gradient written in place
    (so later launches read earlier gradients: the timing does not depend on the values).  Algorithmic bytes: the
    logits read once and the gradient written once."""
    from metal_candle_b200 import _lib

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0x5EED)
    nv = max(1, min(3, _variants(rows * V * 2)))
    logits = [torch.randn(rows, V, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16) for _ in range(nv)]
    targets = torch.randint(0, V, (rows,), device=dev, generator=g, dtype=torch.int32)
    nll = torch.empty(rows, device=dev, dtype=torch.float32)
    count = torch.full((1,), rows, device=dev, dtype=torch.int32)
    lib = _lib.load()

    def fn(i):
        _lib.check(lib.mcb_cross_entropy_chunk(logits[i % nv].data_ptr(), targets.data_ptr(), nll.data_ptr(), count.data_ptr(),
                                               rows, V, 1, _lib.MCB_BF16, torch.cuda.current_stream().cuda_stream))

    med, mn = _time_kernel(torch, fn, nv, iters, warmup)
    pk = measured_peaks()
    by = 4.0 * rows * V
    gbs = by / med / 1e6
    return {"metric": "cross-entropy forward+backward, one chunk", "value": gbs, "unit": "GB/s", "ms": med, "ms_min": mn, "dtype": "bf16",
            "config": {"workload": "cross_entropy_chunk", "rows": rows, "V": V, "input_sets": nv, "l2": "logits larger than L2"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                         "traffic": None, "peak_source": pk["source"]}}


def micro_attention(torch, nb, G, S, which, iters=20, warmup=5):
    """Fused causal grouped-query attention at one layer's shape (nb = batch * kv heads, G query heads per kv head,
    head_dim 64, bf16).  FLOP counted over the causal half only: forward 4*nb*G*S*S*64/2, backward 2.5x that."""
    from metal_candle_b200 import backend as B

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0x5EED)
    d = 64
    nv = _variants(4 * nb * G * S * d * 2)
    nv = min(nv, 6)
    mk = lambda *shape: torch.randn(*shape, device=dev, generator=g).to(torch.bfloat16)
    qs = [mk(nb, G * S, d) for _ in range(nv)]
    ks = [mk(nb, S, d) for _ in range(nv)]
    vs = [mk(nb, S, d) for _ in range(nv)]
    dos = [mk(nb, G * S, d) for _ in range(nv)]
    scale = 1.0 / math.sqrt(d)
    saved = [B.attention_causal_forward(qs[i], ks[i], vs[i], G, scale) for i in range(nv)]

    def fwd(i):
        B.attention_causal_forward(qs[i % nv], ks[i % nv], vs[i % nv], G, scale)

    def bwd(i):
        j = i % nv
        B.attention_causal_backward(qs[j], ks[j], vs[j], saved[j][0], saved[j][1], dos[j], G, scale)

    def both(i):
        fwd(i)
        bwd(i)

    fl_f = 4.0 * nb * G * S * S * d / 2
    fn, fl = {"fwd": (fwd, fl_f), "bwd": (bwd, 2.5 * fl_f), "both": (both, 3.5 * fl_f)}[which]
    med, mn = _time_kernel(torch, fn, nv, iters, warmup)
    pk = measured_peaks()
    tf = fl / med / 1e9
    return {"metric": f"fused causal attention {which}", "value": tf, "unit": "TFLOP/s", "ms": med, "ms_min": mn,
            "dtype": "bf16", "config": {"workload": "causal_gqa_attention", "nb": nb, "G": G, "S": S, "head_dim": d,
                                        "pass": which, "input_sets": nv},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf / pk["bf16_tflops"], "traffic": None, "peak_source": pk["source"]}}


def micro_rows(torch, op, rows, D, dtype, iters=20, warmup=5):
    from metal_candle_b200 import backend as B

    dev = torch.device("cuda", 0)
    dt = torch.bfloat16 if dtype == "bf16" else torch.float32
    e = 2 if dtype == "bf16" else 4
    g = torch.Generator(device=dev).manual_seed(0x5EED)
    nv = _variants(3 * rows * D * e)
    nv = min(nv, max(2, int(30e9 // (4 * rows * D * e))))
    out = []
    if op == "rmsnorm":
        xs = [torch.randn(rows, D, device=dev, generator=g).to(dt) for _ in range(nv)]
        dys = [torch.randn(rows, D, device=dev, generator=g).to(dt) for _ in range(nv)]
        w = (1 + 0.1 * torch.randn(D, device=dev, generator=g)).to(dt)
        ybuf = torch.empty_like(xs[0])
        dw = torch.empty(D, device=dev)
        lib = B._lib_for(xs[0])
        ws = B.workspace(dev, lib.mcb_rmsnorm_bwd_workspace_bytes(rows, D))
        code = B._dtype_code(xs[0])
        cur = lambda: torch.cuda.current_stream().cuda_stream  # the capture stream while a graph is recorded

        def fwd(i):
            lib.mcb_rmsnorm_fwd(xs[i % nv].data_ptr(), w.data_ptr(), ybuf.data_ptr(), None, rows, D, 1e-6, code, cur())

        def bwd(i):
            lib.mcb_rmsnorm_bwd(xs[i % nv].data_ptr(), w.data_ptr(), dys[i % nv].data_ptr(), ybuf.data_ptr(),
                                dw.data_ptr(), 0, rows, D, 1e-6, code, ws.data_ptr(), ws.numel(), cur())

        cases = [("rmsnorm fwd", fwd, 2 * rows * D * e + D * e), ("rmsnorm bwd", bwd, 3 * rows * D * e + D * e + 4 * D)]
    else:
        S = D
        xs = []
        for _ in range(nv):
            x = (3.0 * torch.randn(rows, D, device=dev, generator=g))
            if rows % S == 0:  # attention-score blocks: causal mask, -inf strictly above each diagonal
                mask = torch.triu(torch.ones(S, S, device=dev, dtype=torch.bool), 1)
                x.view(-1, S, S).masked_fill_(mask, float("-inf"))
            xs.append(x.to(dt))
        dys = [torch.randn(rows, D, device=dev, generator=g).to(dt) for _ in range(nv)]
        ys = [B.softmax_fused(x) for x in xs]
        buf = torch.empty_like(xs[0])

        def fwd(i):
            B.softmax_fused(xs[i % nv], out=buf)

        def bwd(i):
            B.softmax_backward(ys[i % nv], dys[i % nv], out=buf)

        cases = [("softmax fwd", fwd, 2 * rows * D * e), ("softmax bwd", bwd, 3 * rows * D * e)]
        if rows % S == 0:
            # the attention form: scale + causal mask inside the kernel, masked columns never read.  Reported
            # against the same dense byte count (masked elements count as traffic in the contract).
            lib = B._lib_for(xs[0])
            code = B._dtype_code(xs[0])
            cur = lambda: torch.cuda.current_stream().cuda_stream

            def cfwd(i):
                lib.mcb_softmax_causal_fwd(xs[i % nv].data_ptr(), buf.data_ptr(), rows, D, S, 0.125, code, cur())

            def cbwd(i):
                lib.mcb_softmax_causal_bwd(ys[i % nv].data_ptr(), dys[i % nv].data_ptr(), buf.data_ptr(), rows, D, S,
                                           0.125, code, cur())

            cases += [("softmax causal fwd (dense-equivalent bytes)", cfwd, 2 * rows * D * e),
                      ("softmax causal bwd (dense-equivalent bytes)", cbwd, 3 * rows * D * e)]
    pk = measured_peaks()
    for name, fn, by in cases:
        med, mn = _time_kernel(torch, fn, nv, iters, warmup)
        gbs = by / med / 1e6
        out.append({"metric": name, "value": gbs, "unit": "GB/s", "ms": med, "ms_min": mn, "dtype": dtype,
                    "config": {"workload": op, "rows": rows, "D": D, "input_sets": nv,
                               "l2": "inputs rotated through >2x L2"},
                    "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                                 "frac": gbs / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"]}})
    return out


def micro_adamw(torch, n, n_tensors=1, iters=20, warmup=5):
    from metal_candle_b200.training import AdamW, AdamWConfig

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0x5EED)
    per = n // n_tensors
    ps = [torch.randn(per, device=dev, generator=g) for _ in range(n_tensors)]
    gs = [0.1 * torch.randn(per, device=dev, generator=g) for _ in range(n_tensors)]
    opt = AdamW(AdamWConfig())

    def step(i):
        opt.step_vars(ps, gs)

    med, mn = _time_kernel(torch, step, 1, iters, warmup)
    by = 28 * per * n_tensors
    gbs = by / med / 1e6
    pk = measured_peaks()
    return {"metric": "AdamW multi-tensor", "value": gbs, "unit": "GB/s", "ms": med, "ms_min": mn, "dtype": "f32",
            "config": {"workload": "adamw", "elements": per * n_tensors, "tensors": n_tensors,
                       "l2": "working set 16 B/element" + (" > L2" if 16 * n > L2_BYTES else " (fits L2: latency regime)")},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"]}}


# ---- CPU legs: the only code outside tests/ and smoke() that touches oracle/ ------------------------------
def cpu_baseline(wl: dict, steps: int, warmup: int):
    """The torch-CPU restatement of the reference's step (oracle/qwen_oracle.py, float32) timed on the host
    cores on a bounded sample of the workload: ONE sequence of 512 tokens through the full 24-layer model."""
    import numpy as np
    import torch

    from oracle import qwen_oracle as QO
    from oracle import reference_ops as R

    from metal_candle_b200.qwen import ModelConfig

    torch.set_num_threads(_host_threads())
    cfg = ModelConfig.qwen25_05b()
    S = 512
    g = torch.Generator().manual_seed(0)
    H, I, kv, V = cfg.hidden_size, cfg.intermediate_size, cfg.kv_size, cfg.vocab_size
    w = {"embed_tokens": torch.randn(V, H, generator=g) * 0.02, "norm": torch.ones(H),
         "lm_head": torch.randn(V, H, generator=g) * 0.02}
    shapes = dict(q_proj=(H, H), k_proj=(kv, H), v_proj=(kv, H), o_proj=(H, H), gate_proj=(I, H), up_proj=(I, H),
                  down_proj=(H, I))
    lora = {}
    for i in range(cfg.num_hidden_layers):
        w[f"layers.{i}.input_layernorm"] = torch.ones(H)
        w[f"layers.{i}.post_attention_layernorm"] = torch.ones(H)
        for m, (o, n) in shapes.items():
            w[f"layers.{i}.{m}.weight"] = torch.randn(o, n, generator=g) * 0.02
            if m in ("q_proj", "k_proj", "v_proj"):
                w[f"layers.{i}.{m}.bias"] = torch.zeros(o)
            if m in wl["targets"]:
                lora[f"layers.{i}.{m}"] = (torch.randn(n, wl["rank"], generator=g) * 0.03,
                                           torch.zeros(wl["rank"], o))
    orc = QO.QwenOracle(cfg, w, lora, wl["alpha"] / wl["rank"], dtype=torch.float32)
    ids = torch.randint(0, V, (1, S), generator=g).numpy()
    tg = np.concatenate([ids[:, 1:], np.full((1, 1), R.IGNORE_INDEX, dtype=np.int64)], 1)
    opt = R.AdamWOracle(dtype=np.float32)

    def step():
        _, grads = orc.loss_and_grads(ids, tg)
        for i, (p, gr) in enumerate(zip(orc.lora_params(), grads)):
            new = opt.step(f"t{i}", p.detach().numpy(), gr)
            with torch.no_grad():
                p.copy_(torch.as_tensor(new))

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return {"value": S * steps / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{steps} step(s) of 1 sequence x {S} tokens, full 24-layer model, float32, torch-CPU "
                      "restatement of the reference's op sequence (the Rust reference cannot be built here)",
            "ms_per_step": dt / steps * 1e3}


def _host_threads() -> int:
    """Host threads this process may use: all the cores it is allowed on, divided among the ranks a launcher
    started on this node (torchrun exports OMP_NUM_THREADS=1 to every rank, which would otherwise leave the CPU
    arm on one core)."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    return max(1, cores)


def run_reference(args):
    """`--impl reference`: the reference's CPU path (its torch-CPU restatement) on the host cores.  Under a
    multi-rank launch only rank 0 works, so it takes every core of the box."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from metal_candle_b200.step_bench import WORKLOADS

    torch.set_num_threads(_host_threads())
    wl = WORKLOADS[args.workload]
    steps, warmup = max(1, min(args.steps, 3)), max(1, min(args.warmup, 1))
    cb = cpu_baseline(wl, steps=steps, warmup=warmup)
    line = {"impl": "reference", "metric": "LoRA fwd+bwd tokens/s, Qwen2.5-0.5B shape", "value": cb["value"],
            "unit": "tokens/s", "n_gpus": max(1, args.gpus), "steps": steps, "warmup": warmup,
            "ms_per_step": cb["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["name"], "sample": cb["sample"]},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def kernel_numbers(torch):
    """Driver-run numbers for the kernels the targets name, measured in the same process as the headline: the row
    kernels of benchmark configuration 2 at 114 688 rows (bf16) and the fused LoRA linear forward+backward of
    configuration 3 at M = 32768 for the 0.5B model's 896-wide projection and a 4096-wide one (r = 16)."""
    out = {"note": "graph replay, inputs rotated through > 2x L2, CUDA events; fractions of the measured peaks "
                   "(copy bandwidth for the row kernels, cuBLAS bf16 burst for the GEMM)"}
    rows = {}
    for op, D in (("rmsnorm", 896), ("rmsnorm", 4096), ("softmax", 1024)):
        for r in micro_rows(torch, op, 114688, D, "bf16", 20, 5):
            rows[f"{r['metric']} D={D}"] = {"GBps": round(r["value"], 1), "frac": round(r["roofline"]["frac"], 3),
                                            "ms": round(r["ms"], 4)}
    out["rows_bf16_114688"] = rows
    lora = {}
    for K, N in ((896, 896), (4096, 4096)):
        r = micro_lora(torch, 32768, K, N, 16, "bf16", "both", 20, 5)
        lora[f"{K}x{N} r16 M=32768 fwd+bwd"] = {"TFLOPs": round(r["value"], 1), "frac": round(r["roofline"]["frac"], 3),
                                                 "ms": round(r["ms"], 4), "bound": r["roofline"]["bound"]}
    r = micro_lora_qkv(torch, 32768, 16, "both", 20, 5)
    lora["q/k/v fused (896 -> 896+128+128) r16 M=32768 fwd+bwd"] = {"TFLOPs": round(r["value"], 1), "frac": round(r["roofline"]["frac"], 3),
                                                                    "ms": round(r["ms"], 4), "bound": "tensor"}
    out["lora_linear"] = lora
    frame = {}
    for which in ("fused", "unfused", "gemm"):
        r = micro_mlp_down_bwd(torch, 32768, 4864, 896, which, 10, 3)
        frame[f"MLP down projection backward to d gate / d up, {which} (M=32768, 4864 -> 896)"] = {
            "us": round(r["value"], 1), "algorithmic_GBps": round(r["algorithmic_GBps"]), "TFLOPs": round(r["tflops"])}
    r = micro_cross_entropy(torch, 8192, 151936, 10, 3)
    frame["cross-entropy forward+backward, 8192 x 151936"] = {"ms": round(r["ms"], 3), "GBps": round(r["value"]),
                                                            "frac": round(r["roofline"]["frac"], 3)}
    out["frame"] = frame
    return out


C3_SHAPES = [(896, 896), (896, 128), (2048, 2048), (4096, 4096), (4096, 14336)]


def run_micro(args):
    import torch

    from metal_candle_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    lib = _lib.init(0)
    for kv in args.opt:
        k, v = kv.split("=")
        _lib.check(lib.mcb_set_option(int(k), int(v)))
    if args.sweep == "c2":
        for dtype in ("bf16", "f32"):
            for D in (896, 2048, 4096):
                for rows in (4096, 16384, 114688, 262144, 1048576):
                    if rows * D * (2 if dtype == "bf16" else 4) > 6e9:
                        continue
                    for r in micro_rows(torch, "rmsnorm", rows, D, dtype, args.iters, args.warmup_iters):
                        print(json.dumps(r), flush=True)
            for r in micro_rows(torch, "softmax", 8 * 14 * 1024, 1024, dtype, args.iters, args.warmup_iters):
                print(json.dumps(r), flush=True)
        return
    if args.sweep == "c3":
        for (K, N) in C3_SHAPES:
            for M in (512, 4096, 32768, 131072):
                for r in (8, 16, 64):
                    if M * max(K, N) * 2 > 5e9:
                        continue
                    print(json.dumps(micro_lora(torch, M, K, N, r, "bf16", "both", args.iters, args.warmup_iters)),
                          flush=True)
        return
    if args.micro == "lora":
        print(json.dumps(micro_lora(torch, args.M, args.K, args.N, args.r, args.dtype, args.which, args.iters,
                                    args.warmup_iters)), flush=True)
    elif args.micro == "lora_qkv":
        print(json.dumps(micro_lora_qkv(torch, args.M, args.r, args.which, args.iters, args.warmup_iters)), flush=True)
    elif args.micro == "mlp_down_bwd":
        which = args.which if args.which in ("fused", "unfused", "gemm") else "fused"
        print(json.dumps(micro_mlp_down_bwd(torch, args.M, args.I, args.H, which, args.iters, args.warmup_iters)), flush=True)
    elif args.micro == "cross_entropy":
        print(json.dumps(micro_cross_entropy(torch, min(args.rows, 8192), args.V, args.iters, args.warmup_iters)), flush=True)
    elif args.micro == "attention":
        print(json.dumps(micro_attention(torch, args.nb, args.G, args.S, args.which, args.iters, args.warmup_iters)),
              flush=True)
    elif args.micro in ("rmsnorm", "softmax"):
        for r in micro_rows(torch, args.micro, args.rows, args.D, args.dtype, args.iters, args.warmup_iters):
            print(json.dumps(r), flush=True)
    elif args.micro == "adamw":
        print(json.dumps(micro_adamw(torch, args.n, args.tensors, args.iters, args.warmup_iters)), flush=True)
    else:
        raise SystemExit(f"unknown --micro {args.micro}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c5", choices=["c4", "c5"])
    ap.add_argument("--micro", default=None)
    ap.add_argument("--sweep", default=None, choices=[None, "c2", "c3"])
    ap.add_argument("--M", type=int, default=32768)
    ap.add_argument("--K", type=int, default=896)
    ap.add_argument("--N", type=int, default=896)
    ap.add_argument("--r", type=int, default=16)
    ap.add_argument("--nb", type=int, default=32)
    ap.add_argument("--G", type=int, default=7)
    ap.add_argument("--S", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=114688)
    ap.add_argument("--D", type=int, default=1024)
    ap.add_argument("--n", type=int, default=1 << 26)
    ap.add_argument("--tensors", type=int, default=1)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--pass", dest="which", default="both", choices=["fwd", "bwd", "both", "bwd_dx", "fused", "unfused", "gemm"])
    ap.add_argument("--V", type=int, default=151936)
    ap.add_argument("--I", type=int, default=4864)
    ap.add_argument("--H", type=int, default=896)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup-iters", type=int, default=5)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--comm", default="mcb", choices=["mcb", "mcb-blocking", "torch"],
                    help="gradient exchange: the library's communicator (default), the same with a blocking NCCL "
                         "communicator, or torch.distributed")
    ap.add_argument("--step-impl", default="engine", choices=["engine", "python"],
                    help="run the step through the C-ABI engine (mcb_qwen_*) or through the Python mirror of the reference API")
    ap.add_argument("--grad-tail", default="auto", choices=["auto", "on", "off"],
                    help="dA/dB in the tail phase of the dx launch (auto: on with one GPU, off beside a collective)")
    ap.add_argument("--opt", action="append", default=[], metavar="ID=VALUE",
                    help="library switch for this run (mcb_set_option), e.g. --opt 1=512")
    ap.add_argument("--buckets", type=int, default=1,
                    help="gradient buckets of the data-parallel exchange (N > 1).  1 (default): one all-reduce of the 8.65 MB "
                         "gradient buffer when the backward pass has finished; k > 1: k layer groups, each all-reduced on a side "
                         "stream as soon as its lowest layer is done, overlapped with the rest of the backward pass - measured "
                         "slower on 4 GPUs (101.6-102.0 against 100.3 ms per step): NCCL's kernels take SMs from the persistent "
                         "GEMM grids for longer than the 0.18 ms the single all-reduce costs")
    ap.add_argument("--no-dp-check", action="store_true", help="skip the data-parallel arithmetic check at N > 1")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel numbers at N = 1")
    args = ap.parse_args()
    global NO_GRAPH
    NO_GRAPH = args.no_graph
    if args.micro or args.sweep:
        return run_micro(args)
    if args.impl == "reference":
        return run_reference(args)
    from metal_candle_b200 import step_bench  # the Qwen-shaped training-step benchmark

    return step_bench.run_b200(args, ClockSampler, measured_peaks, cpu_baseline, kernel_numbers)


if __name__ == "__main__":
    main()
