"""The data-parallel exchange step through the C ABI (`mcb_comm_*`, include/mcb200.h): a float32 sum all-reduce of
LoRA gradient buckets over NCCL, with host deadlines and abort instead of hangs.

The reference trains on one device and has nothing like it.  One `Communicator` per process and GPU; the 128-byte
id that rank 0 creates travels to the other ranks by any host channel (`broadcast_id` uses a torch.distributed
process group when one exists).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

from . import _lib


class CommError(_lib.McbError):
    """A failed or timed-out collective / rendezvous; `.code` is the C-ABI status."""


def _check(rc: int) -> None:
    if rc != 0:
        raise CommError(rc, _lib.load().mcb_last_error().decode("utf-8", "replace"))


def unique_id() -> bytes:
    buf = C.create_string_buffer(_lib.MCB_COMM_ID_BYTES)
    _check(_lib.load().mcb_comm_unique_id(buf))
    return buf.raw


def broadcast_id(rank: int, src: int = 0) -> bytes:
    """The id made on rank `src`, handed to every rank of the default torch.distributed group."""
    import torch.distributed as dist

    box = [unique_id() if rank == src else None]
    dist.broadcast_object_list(box, src=src)
    return box[0]


class Communicator:
    """`timeout_ms` bounds the rendezvous, every enqueue and (by default) `wait`; 0 means no deadline.  `blocking`
    asks NCCL for a blocking communicator (its work then runs in the calling thread; the rendezvous has no deadline)."""

    def __init__(self, nranks: int, rank: int, id_bytes: bytes, timeout_ms: int = 60_000, blocking: bool = False):
        if len(id_bytes) != _lib.MCB_COMM_ID_BYTES:
            raise ValueError(f"communicator id must be {_lib.MCB_COMM_ID_BYTES} bytes")
        self._lib = _lib.load()
        self._h = C.c_void_p(None)
        self.nranks, self.rank, self.timeout_ms = nranks, rank, timeout_ms
        _check(self._lib.mcb_comm_init_rank(C.byref(self._h), nranks, rank, id_bytes, int(timeout_ms),
                                            _lib.MCB_COMM_BLOCKING if blocking else 0))

    def allreduce_bucket(self, ptr: int, count: int, stream: int) -> None:
        """In-place float32 sum over ranks of `count` elements at device address `ptr`, enqueued on `stream`."""
        _check(self._lib.mcb_comm_allreduce_bucket(self._h, ptr, count, stream))

    def allreduce_tensor(self, t, stream: Optional[int] = None) -> None:
        import torch

        if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
            raise ValueError("allreduce_tensor takes a contiguous float32 CUDA tensor")
        s = torch.cuda.current_stream().cuda_stream if stream is None else stream
        self.allreduce_bucket(t.data_ptr(), t.numel(), s)

    def wait(self, stream: Optional[int] = None, timeout_ms: Optional[int] = None) -> None:
        """Host wait until the communicator's work (and `stream`, if given) is done, or the deadline aborts it."""
        s = _lib.MCB_COMM_NO_STREAM if stream is None else stream
        _check(self._lib.mcb_comm_wait(self._h, s, int(self.timeout_ms if timeout_ms is None else timeout_ms)))

    def info(self) -> dict:
        n, r, d, v = C.c_int(0), C.c_int(0), C.c_int(0), C.c_int(0)
        _check(self._lib.mcb_comm_info(self._h, C.byref(n), C.byref(r), C.byref(d), C.byref(v)))
        return {"nranks": n.value, "rank": r.value, "dead": bool(d.value), "nccl_version": v.value}

    def abort(self) -> None:
        _check(self._lib.mcb_comm_abort(self._h))

    def destroy(self) -> None:
        if self._h:
            h, self._h = self._h, C.c_void_p(None)
            _check(self._lib.mcb_comm_destroy(h))

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass
