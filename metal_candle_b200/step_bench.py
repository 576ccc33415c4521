"""The headline benchmark: one LoRA training step (forward, loss, backward, LoRA-gradient all-reduce,
AdamW) of the Qwen2.5-0.5B-shaped decoder, batch-data-parallel with one process per GPU.

Workloads (synthetic token ids uniform in [0, vocab), next-token targets, random-init bf16 weights):
  c5 (default)  per-GPU batch 16 x seq 2048, LoRA rank 16 (alpha 32) on q/k/v/o_proj    -- weak scaling
  c4            batch 8 x seq 1024, LoRA rank 8 (alpha 16) on q_proj and v_proj

Data parallelism: weights and LoRA parameters are replicated (same seed on every rank); each rank takes
its own rows of the global batch; the only exchange is a float32 sum all-reduce (NCCL) of the LoRA
gradients, issued per group of layers from the backward pass as soon as the group is final so that it
overlaps the rest of the backward; AdamW then runs identically everywhere with gradients scaled by
1/world.
"""
from __future__ import annotations

import json
import math
import os
import sys
import time

WORKLOADS = {
    "c5": dict(batch=16, seq=2048, rank=16, alpha=32.0, targets=("q_proj", "k_proj", "v_proj", "o_proj"),
               name="Qwen2.5-0.5B-shaped LoRA step, per-GPU batch 16 x seq 2048, r=16 on q/k/v/o_proj"),
    "c4": dict(batch=8, seq=1024, rank=8, alpha=16.0, targets=("q_proj", "v_proj"),
               name="Qwen2.5-0.5B-shaped LoRA step, batch 8 x seq 1024, r=8 on q/v_proj"),
}
N_BUCKETS = 4


class DataParallelLoRA:
    """Bucketed, overlapped all-reduce of the flat LoRA-gradient buffer."""

    def __init__(self, model, world: int):
        import torch.distributed as dist

        self.model, self.world, self.dist = model, world, dist
        L = model.num_layers()
        per = math.ceil(L / N_BUCKETS)
        self.buckets = {}  # lowest layer of the bucket -> (lo, hi) element range
        for b in range(0, L, per):
            lo = model.grad_layer_range(b)[0]
            hi = model.grad_layer_range(min(L, b + per) - 1)[1]
            self.buckets[b] = (lo, hi)
        self.pending = []
        model.layer_done_hook = self.on_layer_done if world > 1 else None

    def on_layer_done(self, idx: int) -> None:
        rng = self.buckets.get(idx)
        if rng is not None:
            flat = self.model.grad_flat()
            self.pending.append(self.dist.all_reduce(flat[rng[0]:rng[1]], op=self.dist.ReduceOp.SUM, async_op=True))

    def finish(self) -> None:
        for w in self.pending:
            w.wait()
        self.pending = []

    def reduce_all(self) -> None:
        """The whole flat buffer in one all-reduce: what follows a step replayed from a CUDA graph, which
        cannot call back per layer (the buffer is a few MB; there is nothing worth overlapping)."""
        if self.world > 1:
            self.dist.all_reduce(self.model.grad_flat(), op=self.dist.ReduceOp.SUM)


def _build(torch, wl, device, seed=0):
    from .qwen import ModelConfig, Qwen
    from .training import AdamW, AdamWConfig, LoRAAdapter, LoRAAdapterConfig, LRScheduler, TargetModule

    cfg = ModelConfig.qwen25_05b()
    model = Qwen(cfg, device, dtype=torch.bfloat16, seed=seed)
    acfg = LoRAAdapterConfig(rank=wl["rank"], alpha=wl["alpha"],
                             target_modules=[TargetModule.from_name(t) for t in wl["targets"]])
    gen = torch.Generator(device=device).manual_seed(seed + 1)
    adapter = LoRAAdapter(cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers, acfg, device,
                          kv_size=cfg.kv_size, generator=gen)
    # A ~ U(+-1/sqrt(in)) as the benchmark configurations state; B = 0 at step 0 as in the reference
    for _, l in adapter.layers():
        s = 1.0 / math.sqrt(l.in_features)
        l.lora_a.copy_((torch.rand(l.lora_a.shape, device=device, generator=gen) * 2 - 1) * s)
    model.apply_adapter(adapter)
    opt = AdamW(AdamWConfig(learning_rate=1e-4))
    sched = LRScheduler.warmup_cosine(5, 50, 1e-4, 1e-6)
    return cfg, model, adapter, opt, sched


def _host_batches(torch, n, B, S, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, vocab, (B, S), generator=g, dtype=torch.int32)
        tg = torch.cat([ids[:, 1:], torch.full((B, 1), -1, dtype=torch.int32)], 1)  # last position ignored
        out.append((ids.pin_memory(), tg.pin_memory()))
    return out


def run_b200(args, ClockSampler, measured_peaks, cpu_baseline):
    """`ClockSampler`, `measured_peaks` and `cpu_baseline` are supplied by the repo-root bench.py (the CPU
    baseline is the one leg that may touch the oracle, so it lives outside this package)."""
    import torch

    from . import _lib
    from .training import TrainingStep

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != max(1, args.gpus) and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    wl = WORKLOADS[args.workload]
    B, S = wl["batch"], wl["seq"]
    cfg, model, adapter, opt, sched = _build(torch, wl, device)
    dp = DataParallelLoRA(model, world)
    variables = TrainingStep.collect_trainable_vars(adapter)
    n_steps = args.warmup + 2 * args.steps
    host = _host_batches(torch, min(n_steps, 8), B, S, cfg.vocab_size, seed=1234 + rank)
    dev_batches = [(i.to(device), t.to(device)) for i, t in host]
    ids_dev = torch.empty(B, S, dtype=torch.int32, device=device)
    tg_dev = torch.empty(B, S, dtype=torch.int32, device=device)
    state = {"step": 0}

    captured = {"fb": None}

    def one_step(ids, tg):
        if captured["fb"] is not None:
            loss, grads = captured["fb"](ids, tg)   # forward + loss + backward replayed from a CUDA graph
            dp.reduce_all()
        else:
            loss, grads = model.forward_backward(ids, tg)
            dp.finish()
        opt.set_lr(sched.get_lr(state["step"]))
        opt.step_vars(variables, grads, grad_scale=1.0 / world)
        state["step"] += 1
        return loss

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # Warm-up: eager steps first (kernel attributes, workspaces), the last of them with per-launch CUDA events on
    # the GEMM launches for the roofline object; then the step is captured into a CUDA graph and warmed up again.
    n_eager = max(2, args.warmup)
    for i in range(n_eager):
        if i == n_eager - 1:
            torch.cuda.synchronize()
            _lib.profile_enable(True)
        one_step(*dev_batches[i % len(dev_batches)])
    torch.cuda.synchronize()
    _lib.profile_enable(False)
    gemm = _lib.profile_summary(0)
    grad = _lib.profile_summary(1)
    prof_steps = 1
    capture_note = None
    if not getattr(args, "no_graph", False):
        hook = model.layer_done_hook
        try:
            model.layer_done_hook = None
            captured["fb"] = model.capture_forward_backward(B, S)
        except Exception as e:  # the eager path stays valid; say why the graph is not used
            captured["fb"] = None
            model.layer_done_hook = hook
            capture_note = f"{type(e).__name__}: {e}"[:200]
            print(f"bench: CUDA-graph capture failed, timing eager launches instead ({capture_note})", file=sys.stderr)
            torch.cuda.synchronize()
        if dist is not None:
            # every rank must exchange gradients the same way: the graph is used only if all of them captured it
            okf = torch.tensor([1 if captured["fb"] is not None else 0], device=device, dtype=torch.int32)
            dist.all_reduce(okf, op=dist.ReduceOp.MIN)
            if int(okf.item()) == 0 and captured["fb"] is not None:
                captured["fb"] = None
                model.layer_done_hook = hook
                capture_note = "another rank could not capture"
        for i in range(args.warmup):
            one_step(*dev_batches[i % len(dev_batches)])
    barrier()
    # ---- device-resident timing: exactly K steps between barriers, CUDA events, max over ranks ----
    sampler = ClockSampler(local).start() if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    loss = None
    for i in range(args.steps):
        loss = one_step(*dev_batches[(args.warmup + i) % len(dev_batches)])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler is not None else None
    # ---- end to end: pinned host ids -> device, step, loss back to the host, every step ----
    barrier()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        hi, ht = host[i % len(host)]
        if captured["fb"] is not None:
            last = float(one_step(hi, ht).item())     # pinned host ids straight into the graph's input buffers
        else:
            ids_dev.copy_(hi, non_blocking=True)
            tg_dev.copy_(ht, non_blocking=True)
            last = float(one_step(ids_dev, tg_dev).item())
    barrier()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([ms, e2e_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    status = _lib.device_status()
    if rank == 0:
        tokens = B * S * world * args.steps
        pk = measured_peaks()
        n_l, g_ms, g_fl, g_by = gemm
        achieved = g_fl / g_ms / 1e9 if g_ms > 0 else 0.0
        peak = pk["bf16_tflops_sustained"]
        per_step_launches = _count_launches(cfg, wl)
        line = {
            "metric": "LoRA fwd+bwd tokens/s, Qwen2.5-0.5B shape", "value": tokens / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl["name"], "per_gpu_batch": B, "seq_len": S, "global_batch": B * world,
                       "lora_rank": wl["rank"], "lora_targets": list(wl["targets"]), "parallelism": f"dp{world}",
                       "optimizer": "AdamW lr 1e-4 warmup-cosine",
                       "execution": ("forward+loss+backward replayed from a CUDA graph, then gradient all-reduce and AdamW"
                                     if captured["fb"] is not None else
                                     "eager launches" + (f" (graph capture failed: {capture_note})" if capture_note else "")),
                       "l2": "inputs larger than L2 (activations of one "
                       "step are tens of GB)", "loss_last": last},
            "e2e": {"value": tokens / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * S * 4,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": per_step_launches * args.steps,
            "roofline": {"bound": "tensor", "kernel": "lora_gemm2_kernel + lora_gemm_kernel (all projections of the step; the dx launches of the LoRA "
                                   "projections include their dA/dB tail phase)",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": pk["source"] + " (sustained cuBLAS bf16)",
                         "measured_in": "per-launch CUDA events in the last eager warm-up step of this run"
                                        + (" (the timed steps replay a CUDA graph)" if captured["fb"] is not None else ""),
                         "launches": n_l, "kernel_ms_per_step": g_ms / prof_steps,
                         "share_of_step": (g_ms / prof_steps) / (ms / args.steps) if ms > 0 else None,
                         "lora_grad_kernel": {"launches": grad[0], "ms_per_step": grad[1] / prof_steps,
                                              "achieved_GBps": grad[3] / grad[1] / 1e6 if grad[1] > 0 else None,
                                              "hbm_peak_GBps": pk["hbm_gbs"]}},
            "clocks": clocks, "device_status": status,
        }
        if world == 1:
            line["cpu_baseline"] = cpu_baseline(WORKLOADS[args.workload], steps=1, warmup=0)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def _count_launches(cfg, wl) -> int:
    """Kernels of this library launched per training step (counted from the step's structure)."""
    L = cfg.num_hidden_layers
    n_lora = len(wl["targets"])
    fused_attn = cfg.head_dim == 64 and wl["seq"] % 128 == 0   # else the scores are materialised (cuBLAS + row softmax)
    fused_mlp = (cfg.intermediate_size % 128 == 0 and "gate_proj" not in wl["targets"] and "up_proj" not in wl["targets"])
    # forward: 2 norms, 7 GEMMs, operand packs, 3 rope/relayout (+ 1 inverse relayout unless the fused attention
    # writes the o_proj layout itself), attention (or softmax), swiglu
    # (gate, up and swiglu are one kernel when neither projection has an adapter)
    per_layer_fwd = 2 + (5 if fused_mlp else 8) + n_lora + (3 if fused_attn else 4) + 1
    # backward: 7 GEMMs, packs, dA/dB, swiglu, 2 norms (each adds the residual-path gradient as it writes dx),
    # 4 rope/relayout, attention (dq + dkv kernels, or one softmax).  dA and dB of an adapter are accumulated in the tail phase of its dx
    # GEMM launch and cost one partial-sum launch more; adapters whose dx runs on CTA pairs (out features >= 1536)
    # or that are wider than 1024 features take a gradient launch of their own as well.
    out_f = {"q_proj": cfg.hidden_size, "k_proj": cfg.kv_size, "v_proj": cfg.kv_size, "o_proj": cfg.hidden_size,
             "gate_proj": cfg.intermediate_size, "up_proj": cfg.intermediate_size, "down_proj": cfg.hidden_size}
    in_f = {"down_proj": cfg.intermediate_size}
    grad_launches = 0
    for t in wl["targets"]:
        o, i = out_f[t], in_f.get(t, cfg.hidden_size)
        tail = o < 1536 and max(o, i) <= 1024 and o % 64 == 0 and i % 64 == 0
        grad_launches += 1 if tail else 2
    per_layer_bwd = 7 + n_lora + grad_launches + 1 + 2 + (3 if fused_attn else 4) + (2 if fused_attn else 1)
    tail = 1 + 1 + 1 + 3 + 1 + 1  # embed, norm, lm_head, CE x3, lm_head bwd, norm bwd
    adamw = math.ceil(2 * n_lora * L / 64)
    return L * (per_layer_fwd + per_layer_bwd) + tail + adamw
