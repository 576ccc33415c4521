"""The data-parallel exchange step on CPU: world_size 2, gloo backend, 127.0.0.1.

Checks the host logic of DataParallelLoRA (metal_candle_b200/step_bench.py) with a stand-in model whose
gradient buffer lives on the CPU: the layer-group buckets tile the flat gradient buffer exactly once, each
is all-reduced when its lowest layer finishes the backward pass, and after finish() every rank holds the
sum over ranks -- the same result as accumulating both micro-batches on one rank.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


class FakeModel:
    def __init__(self, n_layers=24, per_layer=37):
        self.n_layers, self.per_layer = n_layers, per_layer
        self.flat = torch.zeros(n_layers * per_layer, dtype=torch.float32)
        self.layer_done_hook = None

    def num_layers(self):
        return self.n_layers

    def grad_layer_range(self, idx):
        return idx * self.per_layer, (idx + 1) * self.per_layer

    def grad_flat(self):
        return self.flat

    def backward(self, rank):
        # layers finish from the last to the first, as in the real backward pass
        for idx in range(self.n_layers - 1, -1, -1):
            lo, hi = self.grad_layer_range(idx)
            self.flat[lo:hi] = torch.arange(lo, hi, dtype=torch.float32) * (rank + 1)
            if self.layer_done_hook is not None:
                self.layer_done_hook(idx)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from metal_candle_b200.step_bench import DataParallelLoRA

        model = FakeModel()
        dp = DataParallelLoRA(model, world)
        # buckets tile the buffer exactly once
        cover = torch.zeros_like(model.flat)
        for lo, hi in dp.buckets.values():
            cover[lo:hi] += 1
        assert bool((cover == 1).all())
        assert model.layer_done_hook is not None
        for _ in range(2):  # two steps: pending work is drained each time
            model.backward(rank)
            dp.finish()
            want = torch.arange(model.flat.numel(), dtype=torch.float32) * sum(r + 1 for r in range(world))
            assert torch.equal(model.flat, want)
            assert dp.pending == []
        # the graph-replay path: no per-layer callbacks, one all-reduce of the whole buffer afterwards
        model.layer_done_hook = None
        model.backward(rank)
        dp.reduce_all()
        assert torch.equal(model.flat, want)
        out.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the parent
        out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.timeout(120)
def test_bucketed_allreduce_world2_gloo():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=100) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert results == {0: "ok", 1: "ok"}, results


def test_single_process_installs_no_hook():
    from metal_candle_b200.step_bench import DataParallelLoRA

    model = FakeModel(n_layers=5)
    dp = DataParallelLoRA(model, 1)
    assert model.layer_done_hook is None
    model.backward(0)
    dp.finish()
    assert sorted(dp.buckets) == [0, 2, 4]


# ---- failure detection on the host: a rank that leaves between steps, a rank that never joins --------------------

def _leaver_worker(rank, world, port, out):
    """Rank 1 completes step 0 and then exits (between steps, with nothing in flight).  Rank 0 goes on to step 1:
    its exchange must end with an error within the process group's timeout instead of blocking."""
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from metal_candle_b200.step_bench import DataParallelError, DataParallelLoRA

    model = FakeModel(n_layers=8)
    dp = DataParallelLoRA(model, world)
    model.backward(rank)
    dp.finish()
    ok0 = bool(torch.equal(model.flat, torch.arange(model.flat.numel(), dtype=torch.float32) * 3))
    if rank == 1:
        out.put((rank, "left" if ok0 else "bad step 0"))
        out.close()
        out.join_thread()      # the message is on its way before the process disappears
        os._exit(0)            # gone: no further collective, no clean shutdown
    t0 = time.perf_counter()
    try:
        model.backward(rank)
        dp.finish()
        out.put((rank, "no error"))
    except DataParallelError as e:
        out.put((rank, ("error", ok0, time.perf_counter() - t0, str(e)[:80])))
    out.close()
    out.join_thread()
    os._exit(0)


@pytest.mark.timeout(120)
def test_rank_that_leaves_between_steps_gives_the_survivor_an_error():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaver_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=100) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert results[1] == "left"
    kind, ok0, waited, msg = results[0]
    assert kind == "error" and ok0, results
    assert waited < 60.0, f"the survivor waited {waited:.1f} s"


def _lonely_worker(port, out):
    """World size 2, but the second rank is never started: the rendezvous must time out on the host."""
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK="0", WORLD_SIZE="2")
    t0 = time.perf_counter()
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        out.put("joined")
    except Exception as e:
        out.put(("error", time.perf_counter() - t0, type(e).__name__))
    out.close()
    out.join_thread()
    os._exit(0)


@pytest.mark.timeout(120)
def test_rank_that_never_joins_times_out_on_the_host():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    p = ctx.Process(target=_lonely_worker, args=(_free_port(), out))
    p.start()
    res = out.get(timeout=100)
    p.join(timeout=30)
    assert res[0] == "error" and res[1] < 60.0, res
