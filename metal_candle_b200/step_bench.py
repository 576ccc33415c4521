"""The headline benchmark: one LoRA training step (forward, loss, backward, LoRA-gradient all-reduce,
AdamW) of the Qwen2.5-0.5B-shaped decoder, batch-data-parallel with one process per GPU.

Workloads (synthetic token ids uniform in [0, vocab), next-token targets, random-init bf16 weights):
  c5 (default)  per-GPU batch 16 x seq 2048, LoRA rank 16 (alpha 32) on q/k/v/o_proj    -- weak scaling
  c4            batch 8 x seq 1024, LoRA rank 8 (alpha 16) on q_proj and v_proj

Data parallelism: weights and LoRA parameters are replicated (same seed on every rank); each rank takes
its own rows of the global batch; the only exchange is a float32 sum all-reduce of the LoRA gradients, issued
per group of layers from the backward pass as soon as the group is final, on a side stream, so that it overlaps
the rest of the backward; AdamW then runs identically everywhere with gradients scaled by 1/world.  The
all-reduce goes through the library's own communicator (mcb_comm_*, NCCL bound at run time); because it is plain
stream work it is recorded into the CUDA graph of the step together with the kernels it overlaps.
"""
from __future__ import annotations

import json
import math
import os
import statistics
import sys
import time

WORKLOADS = {
    "c5": dict(batch=16, seq=2048, rank=16, alpha=32.0, targets=("q_proj", "k_proj", "v_proj", "o_proj"),
               name="Qwen2.5-0.5B-shaped LoRA step, per-GPU batch 16 x seq 2048, r=16 on q/k/v/o_proj"),
    "c4": dict(batch=8, seq=1024, rank=8, alpha=16.0, targets=("q_proj", "v_proj"),
               name="Qwen2.5-0.5B-shaped LoRA step, batch 8 x seq 1024, r=8 on q/v_proj"),
}
N_BUCKETS = 4


class DataParallelError(RuntimeError):
    """The gradient exchange failed (a peer left, a deadline passed); the step's gradients are not valid."""


class DataParallelLoRA:
    """Bucketed, overlapped all-reduce of the flat LoRA-gradient buffer.

    With `comm` (a `metal_candle_b200.comm.Communicator`) every bucket is enqueued on a side stream that waits for
    the backward pass up to that point; `finish` makes the current stream wait for the side stream.  Nothing in
    it is host-synchronous, so it can be recorded into a CUDA graph.  Without `comm` the exchange goes through
    torch.distributed (any backend; what the CPU tests use with gloo)."""

    def __init__(self, model, world: int, comm=None, n_buckets: int = N_BUCKETS):
        self.model, self.world, self.comm = model, world, comm
        self.dist = None
        self.side = None
        self.inflight = False
        if comm is None and world > 1:
            import torch.distributed as dist

            self.dist = dist
        if comm is not None and world > 1:
            import torch

            self.torch = torch
            self.side = torch.cuda.Stream(priority=-1)
        L = model.num_layers()
        per = math.ceil(L / max(1, min(L, n_buckets)))
        self.buckets = {}  # lowest layer of the bucket -> (lo, hi) element range
        for b in range(0, L, per):
            lo = model.grad_layer_range(b)[0]
            hi = model.grad_layer_range(min(L, b + per) - 1)[1]
            self.buckets[b] = (lo, hi)
        self.pending = []
        model.layer_done_hook = self.on_layer_done if world > 1 else None
        model.backward_done_hook = self.finish if (world > 1 and comm is not None) else None

    def _issue(self, lo: int, hi: int, async_op: bool):
        flat = self.model.grad_flat()
        if self.comm is not None:
            cur = self.torch.cuda.current_stream()
            self.side.wait_stream(cur)     # the bucket's gradients are final on the current stream
            self.comm.allreduce_bucket(flat.data_ptr() + 4 * lo, hi - lo, self.side.cuda_stream)
            self.inflight = True
            return None
        try:
            return self.dist.all_reduce(flat[lo:hi], op=self.dist.ReduceOp.SUM, async_op=async_op)
        except RuntimeError as e:
            raise DataParallelError(f"gradient all-reduce failed: {e}") from e

    def on_layer_done(self, idx: int) -> None:
        rng = self.buckets.get(idx)
        if rng is not None:
            w = self._issue(rng[0], rng[1], async_op=True)
            if w is not None:
                self.pending.append(w)

    def finish(self) -> None:
        if self.comm is not None:
            if self.inflight:
                self.torch.cuda.current_stream().wait_stream(self.side)
                self.inflight = False
            return
        try:
            for w in self.pending:
                w.wait()
        except RuntimeError as e:
            raise DataParallelError(f"gradient all-reduce failed: {e}") from e
        finally:
            self.pending = []

    def reduce_all(self) -> None:
        """The whole flat buffer in one all-reduce on the current stream (no overlap)."""
        if self.world > 1:
            n = self.model.grad_flat().numel()
            if self.comm is not None:
                self.comm.allreduce_bucket(self.model.grad_flat().data_ptr(), n, self.torch.cuda.current_stream().cuda_stream)
            else:
                self._issue(0, n, async_op=False)


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


class _CapturedEngineStep:
    """QwenEngine.forward_backward of a fixed shape as a CUDA graph; called like `CapturedStep`."""

    def __init__(self, torch, eng, batch, seq):
        self.ids = torch.zeros(batch, seq, dtype=torch.int32, device=eng.model.device)
        self.targets = torch.full((batch, seq), -1, dtype=torch.int32, device=eng.model.device)
        self.graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize(eng.model.device)
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            self.loss, self.grads = eng.forward_backward(self.ids, self.targets)

    def __call__(self, input_ids, target_ids):
        self.ids.copy_(input_ids, non_blocking=True)
        self.targets.copy_(target_ids, non_blocking=True)
        self.graph.replay()
        return self.loss, self.grads


class _Step:
    """The two implementations of the step behind one face: the C-ABI engine (mcb_qwen_*) or the Python mirror
    (Qwen.forward_backward + AdamW.step_vars).  Both issue the same kernels."""

    def __init__(self, torch, model, adapter, dp, world, comm, use_engine, B, S):
        from .training import AdamW, AdamWConfig, TrainingStep

        self.torch, self.model, self.dp, self.world, self.comm = torch, model, dp, world, comm
        self.variables = TrainingStep.collect_trainable_vars(adapter)
        self.eng = None
        self.opt = AdamW(AdamWConfig(learning_rate=1e-4))
        self.B, self.S = B, S
        if use_engine:
            from .engine import QwenEngine

            self.eng = QwenEngine(model, B, S)
            model.layer_done_hook = model.backward_done_hook = None    # the engine issues the exchange itself
            self.exchange(True)

    def exchange(self, on: bool) -> None:
        """Engine only: the bucketed all-reduce inside forward_backward on / off."""
        if self.eng is None:
            return
        if on and self.comm is not None and self.world > 1:
            self.eng.set_exchange(self.comm, self.dp.side, [(layer, lo, hi) for layer, (lo, hi) in self.dp.buckets.items()])
        else:
            self.eng.set_exchange(None, None, None)

    def fb(self, ids, tg, accumulate=False, exchange=True):
        """forward + loss + backward (+ the exchange, finished on the current stream); returns (loss, grads)."""
        if self.eng is not None:
            return self.eng.forward_backward(ids, tg, accumulate=accumulate)
        loss, grads = self.model.forward_backward(ids, tg, accumulate=accumulate)
        if exchange:
            self.dp.finish()
        return loss, grads

    def capture(self, with_exchange: bool, pool=None):
        if self.eng is not None:
            self.exchange(with_exchange)
            try:
                return _CapturedEngineStep(self.torch, self.eng, self.B, self.S)
            finally:
                self.exchange(True)
        return self.model.capture_forward_backward(self.B, self.S, keep_hooks=with_exchange, pool=pool)

    def adamw(self, lr, grads, opt=None):
        if self.eng is not None and opt is None:
            self.eng.adamw_step(lr, grad_scale=1.0 / self.world)
            return
        o = self.opt if opt is None else opt
        o.set_lr(lr)
        o.step_vars(self.variables, grads, grad_scale=1.0 / self.world)


def dp_check(torch, step, adapter, world, rank, B, S, vocab, device, steps=3):
    """The data-parallel arithmetic checked on the GPUs themselves.  For `steps` optimizer steps, from the SAME
    parameters and optimizer state each time: (a) the data-parallel form (this rank's micro-batch, bucketed
    all-reduce, AdamW on gradients / world) and (b) one rank's arithmetic (the `world` micro-batches accumulated
    into the gradient buffer, then the same AdamW).  Compared are the mean loss, the summed gradients (they may
    differ only by the order of the fp32 additions: sequential accumulation against the all-reduce's ring or tree)
    and the parameter update each gives.  The trajectory then continues from (a).

    The comparison is made step by step rather than between two free-running trajectories on purpose: with four
    ranks the gradients of the first steps differ by 1.5e-7 (addition order), but B is then a few 1e-5 after
    AdamW's sign-like first update, its bf16 rounding inside the LoRA GEMM flips for a few elements, and by the
    third step the two free-running gradients differ by 1 % and AdamW's normalisation turns that into a 10 %
    difference of single updates -- the sensitivity of this bf16 training step to one ulp, not of the exchange.

    Every rank computes (b) redundantly from the same seeds.  Leaves the adapter as it found it."""
    import torch.distributed as dist

    from .training import AdamW, AdamWConfig, LRScheduler

    variables = step.variables
    snapshot = [v.clone() for v in variables]
    sched = LRScheduler.warmup_cosine(5, 50, 1e-4, 1e-6)
    micro = {r: _host_batches(torch, steps, B, S, vocab, seed=777 + r) for r in range(world)}
    model = step.model
    hook, done = model.layer_done_hook, model.backward_done_hook
    opt = AdamW(AdamWConfig(learning_rate=1e-4))

    def rel(xs, ys):
        """largest |x - y| over the tensors, relative to the largest |y|"""
        num = max(float((x - y).abs().max()) for x, y in zip(xs, ys))
        return num / max(max(float(y.abs().max()) for y in ys), 1e-30)

    def set_values(dst, src):
        with torch.no_grad():
            for d, s0 in zip(dst, src):
                d.copy_(s0)

    dp_losses, acc_losses, grad_diff, update_diff = [], [], [], []
    try:
        for s in range(steps):
            lr = sched.get_lr(s)
            # (a) data parallel
            ids, tg = micro[rank][s]
            loss, grads = step.fb(ids.to(device), tg.to(device))
            g_dp = [g.clone() for g in grads]
            l = loss.detach().clone().double()
            dist.all_reduce(l, op=dist.ReduceOp.SUM)       # every micro-batch keeps the same number of tokens
            dp_losses.append(float(l) / world)
            # (b) one rank, the micro-batches of all ranks accumulated
            model.layer_done_hook = model.backward_done_hook = None
            step.exchange(False)
            tot = 0.0
            for r in range(world):
                ids, tg = micro[r][s]
                loss, grads = step.fb(ids.to(device), tg.to(device), accumulate=(r > 0), exchange=False)
                tot += float(loss)
            acc_losses.append(tot / world)
            model.layer_done_hook, model.backward_done_hook = hook, done
            step.exchange(True)
            grad_diff.append(rel(g_dp, grads))
            # AdamW from the same parameters and moments with either gradient
            before = [v.clone() for v in variables]
            moments = {k: (m.clone(), v.clone()) for k, (m, v) in opt.state.items()}
            count = opt.step_count
            step.adamw(lr, grads, opt=opt)
            upd_acc = [v - b0 for v, b0 in zip(variables, before)]
            set_values(variables, before)
            for k, (m, v) in list(opt.state.items()):
                if k in moments:
                    m.copy_(moments[k][0]), v.copy_(moments[k][1])
                else:
                    m.zero_(), v.zero_()
            opt.step_count = count
            step.adamw(lr, g_dp, opt=opt)
            upd_dp = [v - b0 for v, b0 in zip(variables, before)]
            update_diff.append(rel(upd_dp, upd_acc) if max(float(u.abs().max()) for u in upd_acc) > 0 else 0.0)
    finally:
        model.layer_done_hook, model.backward_done_hook = hook, done
        step.exchange(True)
        set_values(variables, snapshot)
        torch.cuda.synchronize()
    rel_loss = max(abs(a - b) / max(abs(b), 1e-30) for a, b in zip(dp_losses, acc_losses))
    tol = {"loss": 1e-5, "grad": 1e-5, "update": 2e-4}
    out = {"steps": steps, "max_rel_loss_diff": rel_loss, "max_rel_grad_diff": max(grad_diff),
           "max_rel_update_diff": max(update_diff), "rel_grad_diff_by_step": grad_diff,
           "rel_update_diff_by_step": update_diff, "loss_dp": dp_losses, "loss_accumulated": acc_losses,
           "compared": "each step from the same parameters and optimizer state", "tolerance": tol}
    out["ok"] = bool(rel_loss <= tol["loss"] and out["max_rel_grad_diff"] <= tol["grad"]
                     and out["max_rel_update_diff"] <= tol["update"])
    return out


def _median_ms(torch, fn, reps):
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def run_b200(args, ClockSampler, measured_peaks, cpu_baseline, kernel_numbers=None):
    """`ClockSampler`, `measured_peaks`, `cpu_baseline` and `kernel_numbers` are supplied by the repo-root bench.py
    (the CPU baseline is the one leg that may touch the oracle, so it lives outside this package)."""
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
    lib = _lib.init(local)
    dist = None
    comm = None
    comm_mode = getattr(args, "comm", "mcb")
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
        if comm_mode != "torch":
            from . import comm as C

            comm = C.Communicator(world, rank, C.broadcast_id(rank), timeout_ms=30_000,
                                  blocking=(comm_mode == "mcb-blocking"))
    # the backward's tail phase needs its whole grid resident: off where a collective runs beside the backward pass
    # (more than one exchange bucket); with one bucket the all-reduce starts when the backward pass has finished
    tail = getattr(args, "grad_tail", "auto")
    tail_on = (tail == "on") or (tail == "auto" and (world == 1 or getattr(args, "buckets", N_BUCKETS) <= 1))
    _lib.check(lib.mcb_set_option(_lib.MCB_OPT_GRAD_TAIL, int(tail_on)))
    wl = WORKLOADS[args.workload]
    B, S = wl["batch"], wl["seq"]
    cfg, model, adapter, opt, sched = _build(torch, wl, device)
    dp = DataParallelLoRA(model, world, comm=comm, n_buckets=getattr(args, "buckets", N_BUCKETS))
    use_engine = getattr(args, "step_impl", "engine") == "engine" and (world == 1 or comm is not None)
    step = _Step(torch, model, adapter, dp, world, comm, use_engine, B, S)
    check = None
    if world > 1 and not getattr(args, "no_dp_check", False):
        check = dp_check(torch, step, adapter, world, rank, B, S, cfg.vocab_size, device)
    n_steps = args.warmup + 2 * args.steps
    host = _host_batches(torch, min(n_steps, 8), B, S, cfg.vocab_size, seed=1234 + rank)
    dev_batches = [(i.to(device), t.to(device)) for i, t in host]
    ids_dev = torch.empty(B, S, dtype=torch.int32, device=device)
    tg_dev = torch.empty(B, S, dtype=torch.int32, device=device)
    state = {"step": 0}
    captured = {"fb": None, "fb_nocomm": None}
    graph_has_comm = comm is not None

    def one_step(ids, tg):
        if captured["fb"] is not None:
            loss, grads = captured["fb"](ids, tg)   # forward + loss + backward (+ the exchange) replayed from a CUDA graph
            if not graph_has_comm:
                dp.reduce_all()
        else:
            if step.eng is not None and not ids.is_cuda:
                ids_dev.copy_(ids, non_blocking=True)
                tg_dev.copy_(tg, non_blocking=True)
                ids, tg = ids_dev, tg_dev
            loss, grads = step.fb(ids, tg)
        step.adamw(sched.get_lr(state["step"]), grads)
        state["step"] += 1
        return loss

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # Warm-up: eager steps first (kernel attributes, workspaces, NCCL connections), the last of them with per-launch
    # CUDA events on the GEMM launches for the roofline object; then the step is captured into a CUDA graph and
    # warmed up again.
    n_eager = max(2, args.warmup)
    launches_before = 0
    for i in range(n_eager):
        if i == n_eager - 1:
            torch.cuda.synchronize()
            _lib.profile_enable(True)
            launches_before = lib.mcb_launch_count()
        one_step(*dev_batches[i % len(dev_batches)])
    per_step_launches = lib.mcb_launch_count() - launches_before   # this library's kernels in one step (AdamW included)
    torch.cuda.synchronize()
    _lib.profile_enable(False)
    plain = _lib.profile_summary(0)
    grad = _lib.profile_summary(1)
    lora = _lib.profile_summary(2)
    swig = _lib.profile_summary(3)
    capture_note = None
    if not getattr(args, "no_graph", False):
        hooks = (model.layer_done_hook, model.backward_done_hook)
        try:
            if not graph_has_comm:
                model.layer_done_hook = model.backward_done_hook = None
            captured["fb"] = step.capture(graph_has_comm)
            if graph_has_comm:   # the same step without the exchange, sharing the first graph's memory: for comm.exposed_ms
                captured["fb_nocomm"] = step.capture(False, pool=captured["fb"].graph.pool())
        except Exception as e:  # the eager path stays valid; say why the graph is not used
            captured["fb"] = captured["fb_nocomm"] = None
            model.layer_done_hook, model.backward_done_hook = hooks
            capture_note = f"{type(e).__name__}: {e}"[:200]
            print(f"bench: CUDA-graph capture failed, timing eager launches instead ({capture_note})", file=sys.stderr)
            torch.cuda.synchronize()
        if dist is not None:
            # every rank must exchange gradients the same way: the graph is used only if all of them captured it
            okf = torch.tensor([1 if captured["fb"] is not None else 0], device=device, dtype=torch.int32)
            dist.all_reduce(okf, op=dist.ReduceOp.MIN)
            if int(okf.item()) == 0 and captured["fb"] is not None:
                captured["fb"] = captured["fb_nocomm"] = None
                model.layer_done_hook, model.backward_done_hook = hooks
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
    if captured["fb"] is not None and getattr(captured["fb"], "count", None) is not None and int(captured["fb"].count.item()) == 0:
        raise SystemExit("bench: every target of the last batch was ignored; the loss is undefined")
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
    own_ms = ms
    comm_info = None
    if dist is not None:
        t = torch.tensor([ms, e2e_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
        per_rank = [torch.zeros(1, device=device, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(per_rank, torch.tensor([own_ms], device=device, dtype=torch.float64))
        per_rank = [float(x) / args.steps for x in per_rank]
        # ---- the exchange on its own, and how much of it the step does not hide ----
        nbytes = model.grad_flat().numel() * 4
        scratch = torch.zeros_like(model.grad_flat())

        def exchange_alone():
            for lo, hi in dp.buckets.values():
                if comm is not None:
                    comm.allreduce_bucket(scratch.data_ptr() + 4 * lo, hi - lo, torch.cuda.current_stream().cuda_stream)
                else:
                    dist.all_reduce(scratch[lo:hi])

        barrier()
        exchange_alone()
        alone_ms = _median_ms(torch, exchange_alone, 5)
        exposed = rank_spread = None
        with_ms = without_ms = -1e9
        if captured["fb_nocomm"] is not None:
            ids0, tg0 = dev_batches[0]
            barrier()
            with_ms = _median_ms(torch, lambda: captured["fb"](ids0, tg0), 5)
            barrier()
            without_ms = _median_ms(torch, lambda: captured["fb_nocomm"](ids0, tg0), 5)
        # the exchange couples the ranks (every step ends with the slowest one), so compare the SLOWEST rank's step
        # with and without it; a per-rank difference would read the spread between the GPUs as communication
        t = torch.tensor([alone_ms, with_ms, without_ms, -without_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        alone_ms = float(t[0])
        if captured["fb_nocomm"] is not None:
            exposed = float(t[1]) - float(t[2])
            rank_spread = {"fastest_ms": -float(t[3]), "slowest_ms": float(t[2])}
        comm_info = {"backend": ("mcb_comm (NCCL through the C ABI, " + ("blocking" if comm_mode == "mcb-blocking" else "non-blocking") + ")")
                     if comm is not None else "torch.distributed nccl",
                     "nccl_version": comm.info()["nccl_version"] if comm is not None else None,
                     "bytes_per_step": nbytes, "buckets": len(dp.buckets),
                     "overlapped": bool((comm is not None or captured["fb"] is None) and len(dp.buckets) > 1),
                     "in_graph": bool(graph_has_comm and captured["fb"] is not None),
                     "exposed_ms": exposed,
                     "exposed_how": "slowest rank's step graph with the exchange minus the slowest rank's same graph without it "
                                    "(median of 5 replays each)" if exposed is not None else None,
                     "step_without_exchange": rank_spread,
                     "allreduce_alone_ms": alone_ms,
                     "bus_GBps": 2.0 * (world - 1) / world * nbytes / (alone_ms * 1e-3) / 1e9 if alone_ms > 0 else None,
                     "rank_ms_per_step": {"min": min(per_rank), "max": max(per_rank)}}
    used_graph = captured["fb"] is not None
    status = _lib.device_status()
    if dist is not None:
        t = torch.tensor([status], device=device, dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        status = int(t.item())
    if status != 0:
        print(f"bench: a bounded device-side wait ran out (code {status}); the run's results are invalid", file=sys.stderr)
        if dist is not None:
            dist.destroy_process_group()
        raise SystemExit(3)
    if comm is not None:
        # NCCL keeps a communicator alive for as long as a CUDA graph that recorded its collectives exists, and
        # finalizing it waits for those graphs: let go of them first
        captured["fb"] = captured["fb_nocomm"] = None
        torch.cuda.synchronize()
        try:
            comm.destroy()
        except Exception as e:   # a communicator that will not shut down must not cost the run its result
            print(f"bench: communicator shutdown: {e}", file=sys.stderr)
    if dist is not None:
        dist.destroy_process_group()
    if rank == 0:
        tokens = B * S * world * args.steps
        pk = measured_peaks()
        peak = pk["bf16_tflops_sustained"]

        def klass(rec):
            n_l, g_ms, g_fl, g_by = rec
            ach = g_fl / g_ms / 1e9 if g_ms > 0 else 0.0
            return {"launches": n_l, "ms_per_step": g_ms, "flop_per_step": g_fl, "achieved": ach, "frac": ach / peak}

        both_ms, both_fl = plain[1] + lora[1] + swig[1], plain[2] + lora[2] + swig[2]
        achieved = both_fl / both_ms / 1e9 if both_ms > 0 else 0.0
        line = {
            "metric": "LoRA fwd+bwd tokens/s, Qwen2.5-0.5B shape", "value": tokens / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl["name"], "per_gpu_batch": B, "seq_len": S, "global_batch": B * world,
                       "lora_rank": wl["rank"], "lora_targets": list(wl["targets"]), "parallelism": f"dp{world}",
                       "optimizer": "AdamW lr 1e-4 warmup-cosine",
                       "step_through": "the C-ABI engine (mcb_qwen_forward_backward, mcb_qwen_adamw_step)" if use_engine
                       else "the Python mirror (Qwen.forward_backward, AdamW.step_vars)",
                       "execution": (("forward+loss+backward" + ((" with the bucketed gradient all-reduce overlapped on a side stream" if len(dp.buckets) > 1
                                                                  else " and the gradient all-reduce") if graph_has_comm and world > 1 else "")
                                      + " replayed from a CUDA graph, then " + ("" if graph_has_comm or world == 1 else "gradient all-reduce and ") + "AdamW")
                                     if used_graph else
                                     "eager launches" + (f" (graph capture failed: {capture_note})" if capture_note else "")),
                       "l2": "inputs larger than L2 (activations of one "
                       "step are tens of GB)", "loss_last": last},
            "e2e": {"value": tokens / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * S * 4,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": per_step_launches * args.steps,
            "roofline": {"bound": "tensor", "kernel": "lora_gemm2_kernel + lora_gemm_kernel (all projections of the step; the dx launches of the LoRA "
                                   "projections include their dA/dB tail phase when it is on)",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": 79.3e6,
                         "traffic_source": "ncu, one launch: fused LoRA forward 32768x896x896 r16 (dram read 60.5 MB + write 18.8 MB; "
                                           "algorithmic 119.1 MB, the rest of the output was still in L2) - profiles/lora_gemm_kernel.md; "
                                           "the step as a whole is too large to capture",
                         "peak_source": pk["source"] + " (sustained cuBLAS bf16)",
                         "measured_in": "per-launch CUDA events in the last eager warm-up step of this run"
                                        + (" (the timed steps replay a CUDA graph)" if used_graph else ""),
                         "launches": plain[0] + lora[0] + swig[0], "kernel_ms_per_step": both_ms,
                         "share_of_step": both_ms / (ms / args.steps) if ms > 0 else None,
                         "classes": {"lora": dict(klass(lora), what="launches with a rank path: the fused LoRA linear forward and "
                                                  "backward of the adapted projections (dA/dB tail phase included when on)"),
                                     "plain": dict(klass(plain), what="frozen projections without an adapter (MLP, lm_head, ...)"),
                                     "plain_swiglu_bwd": dict(klass(swig), achieved_GBps=swig[3] / swig[1] / 1e6 if swig[1] > 0 else None,
                                                              hbm_peak_GBps=pk["hbm_gbs"],
                                                              what="input-gradient GEMM of the MLP down projection with the SwiGLU "
                                                              "backward in its epilogue (reads and rewrites gate and up: bound by "
                                                              "that traffic, not by the tensor pipe; replaces a GEMM launch and an "
                                                              "element-wise kernel)")},
                         "lora_grad_kernel": {"launches": grad[0], "ms_per_step": grad[1],
                                              "achieved_GBps": grad[3] / grad[1] / 1e6 if grad[1] > 0 else None,
                                              "hbm_peak_GBps": pk["hbm_gbs"]}},
            "clocks": clocks, "device_status": status,
        }
        if comm_info is not None:
            line["comm"] = comm_info
        if check is not None:
            line["dp_check"] = check
        if world == 1:
            if kernel_numbers is not None and not getattr(args, "no_kernels", False):
                step.eng = None
                del model, adapter, opt, dp, captured, dev_batches, step
                torch.cuda.empty_cache()
                line["kernels"] = kernel_numbers(torch)
            line["cpu_baseline"] = cpu_baseline(WORKLOADS[args.workload], steps=2, warmup=1)
        print(json.dumps(line), flush=True)
