"""Adapter checkpoints in the reference's safetensors layout (src/training/checkpoint.rs:65-100,147-178).

`save_checkpoint` writes one F32 tensor per LoRA matrix under the keys `layers.{i}.{module}.lora_a` and
`layers.{i}.{module}.lora_b` (checkpoint.rs:75-85) and, when metadata is given, the string entry
`checkpoint_metadata` = JSON of `CheckpointMetadata` in the file's `__metadata__` map (checkpoint.rs:87-96).
`load_checkpoint` copies every key that the adapter has into the adapter's tensors and ignores the rest
(checkpoint.rs:164-175), so files written by either side load on the other.

Two extensions, both optional and invisible to the reference's loader: the AdamW state (`m`, `v` per tensor
and the shared step counter, which the reference does not save) goes under `optimizer.*` keys, and
`load_checkpoint` returns the metadata that the reference's loader drops (it returns `None`,
checkpoint.rs:158-160).

The container is written and parsed here (8-byte little-endian header length, JSON header with
`dtype` / `shape` / `data_offsets` per tensor, raw little-endian data), byte-compatible with the `safetensors`
crate's `serialize_to_file`: tensors ordered by descending dtype alignment and then by name, header padded with
spaces to a multiple of 8 bytes.
"""
from __future__ import annotations

import json
import struct
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Dict, Optional, Tuple

import numpy as np

from .backend import TrainingError

_DTYPES = {"F32": np.dtype("<f4"), "F64": np.dtype("<f8"), "I64": np.dtype("<i8"), "I32": np.dtype("<i4"),
           "U8": np.dtype("u1"), "F16": np.dtype("<f2")}
_NAMES = {v: k for k, v in _DTYPES.items()}


class CheckpointError(TrainingError):
    """I/O or format error while reading or writing a checkpoint (`Error::Io`, src/error.rs)."""


@dataclass
class CheckpointMetadata:
    """src/training/checkpoint.rs:11-25."""
    global_step: int
    loss: float
    learning_rate: float
    timestamp: int = 0

    def to_json(self) -> str:
        return json.dumps(asdict(self), separators=(",", ":"))

    @staticmethod
    def from_json(s: str) -> "CheckpointMetadata":
        d = json.loads(s)
        return CheckpointMetadata(int(d["global_step"]), float(d["loss"]), float(d["learning_rate"]),
                                  int(d.get("timestamp", 0)))

    @staticmethod
    def now(global_step: int, loss: float, learning_rate: float) -> "CheckpointMetadata":
        return CheckpointMetadata(global_step, loss, learning_rate, int(time.time()))


# ---------------------------------------------------------------------------------------------
# safetensors container
# ---------------------------------------------------------------------------------------------

def serialize(tensors: Dict[str, np.ndarray], metadata: Optional[Dict[str, str]] = None) -> bytes:
    """The file image for `tensors` (name -> array) and a string-to-string metadata map."""
    items = []
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        dt = a.dtype.newbyteorder("<") if a.dtype.byteorder == ">" else a.dtype
        if np.dtype(dt) not in _NAMES:
            raise CheckpointError(f"tensor '{name}': dtype {a.dtype} cannot be stored")
        items.append((name, a.astype(dt, copy=False)))
    # the crate sorts by dtype alignment (descending), then by name
    items.sort(key=lambda kv: (-kv[1].dtype.itemsize, kv[0]))
    header: Dict[str, object] = {}
    if metadata is not None:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, a in items:
        header[name] = {"dtype": _NAMES[np.dtype(a.dtype)], "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        off += a.nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((-len(hj)) % 8)
    return struct.pack("<Q", len(hj)) + hj + b"".join(a.tobytes() for _, a in items)


def deserialize(blob: bytes) -> Tuple[Dict[str, np.ndarray], Dict[str, str]]:
    """(tensors, metadata) of a file image; validates offsets like the crate does."""
    if len(blob) < 8:
        raise CheckpointError("safetensors: file shorter than its 8-byte header length")
    (n,) = struct.unpack("<Q", blob[:8])
    if n > len(blob) - 8 or n > 100_000_000:
        raise CheckpointError(f"safetensors: header length {n} exceeds the file")
    try:
        header = json.loads(blob[8:8 + n].decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise CheckpointError(f"safetensors: header is not valid JSON ({e})") from e
    if not isinstance(header, dict):
        raise CheckpointError("safetensors: header is not a JSON object")
    meta = header.pop("__metadata__", None) or {}
    data = memoryview(blob)[8 + n:]
    out: Dict[str, np.ndarray] = {}
    for name, info in header.items():
        try:
            dt = _DTYPES[info["dtype"]]
            shape = tuple(int(s) for s in info["shape"])
            lo, hi = (int(x) for x in info["data_offsets"])
        except (KeyError, TypeError, ValueError) as e:
            raise CheckpointError(f"safetensors: bad entry for '{name}' ({e!r})") from e
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if lo < 0 or hi < lo or hi > len(data) or hi - lo != count * dt.itemsize:
            raise CheckpointError(f"safetensors: '{name}' has offsets [{lo},{hi}) for shape {list(shape)} {info['dtype']}")
        out[name] = np.frombuffer(data[lo:hi], dtype=dt).reshape(shape).copy()
    return out, {str(k): str(v) for k, v in meta.items()}


def save_file(path, tensors: Dict[str, np.ndarray], metadata: Optional[Dict[str, str]] = None) -> None:
    try:
        Path(path).write_bytes(serialize(tensors, metadata))
    except OSError as e:
        raise CheckpointError(f"cannot write {path}: {e}") from e


def load_file(path) -> Tuple[Dict[str, np.ndarray], Dict[str, str]]:
    try:
        blob = Path(path).read_bytes()
    except OSError as e:
        raise CheckpointError(f"cannot read {path}: {e}") from e
    return deserialize(blob)


# ---------------------------------------------------------------------------------------------
# adapter <-> file
# ---------------------------------------------------------------------------------------------

def _host(t) -> np.ndarray:
    return t.detach().to("cpu").contiguous().numpy() if hasattr(t, "detach") else np.asarray(t)


def save_checkpoint(adapter, path, metadata: Optional[CheckpointMetadata] = None, optimizer=None) -> None:
    """save_checkpoint (src/training/checkpoint.rs:65-100).  With `optimizer` (an `AdamW` whose state was
    created by `step_var` / `step_vars` on this adapter's tensors) the moments and the shared step counter are
    stored too, under `optimizer.{key}.lora_{a,b}.{m,v}` and `optimizer.step_count`."""
    tensors: Dict[str, np.ndarray] = {}
    for layer_key, layer in adapter.layers():
        tensors[f"{layer_key}.lora_a"] = _host(layer.lora_a_tensor()).astype(np.float32)
        tensors[f"{layer_key}.lora_b"] = _host(layer.lora_b_tensor()).astype(np.float32)
    if optimizer is not None:
        for layer_key, layer in adapter.layers():
            for which, var in (("lora_a", layer.lora_a_tensor()), ("lora_b", layer.lora_b_tensor())):
                st = optimizer.state.get(optimizer._key(var))
                if st is not None:
                    tensors[f"optimizer.{layer_key}.{which}.m"] = _host(st[0]).astype(np.float32)
                    tensors[f"optimizer.{layer_key}.{which}.v"] = _host(st[1]).astype(np.float32)
        tensors["optimizer.step_count"] = np.array([optimizer.step_count], dtype=np.int64)
    meta = None if metadata is None else {"checkpoint_metadata": metadata.to_json()}
    save_file(path, tensors, meta)


def load_checkpoint(adapter, path, optimizer=None) -> Optional[CheckpointMetadata]:
    """load_checkpoint (src/training/checkpoint.rs:147-178): keys the adapter has are copied in, anything else in
    the file is ignored, a key the file lacks leaves that tensor as it is.  A stored tensor whose shape differs
    from the adapter's is an error (candle's `Var::set` refuses it).  Returns the stored metadata, or None."""
    import torch

    tensors, meta = load_file(path)

    def put(dst, name):
        src = tensors.get(name)
        if src is None:
            return False
        if tuple(src.shape) != tuple(dst.shape):
            raise CheckpointError(f"checkpoint tensor '{name}' has shape {list(src.shape)}, the adapter expects "
                                  f"{list(dst.shape)}")
        with torch.no_grad():
            dst.copy_(torch.from_numpy(np.ascontiguousarray(src, dtype=np.float32)).to(dst.device))
        return True

    for layer_key, layer in adapter.layers():
        put(layer.lora_a_tensor(), f"{layer_key}.lora_a")
        put(layer.lora_b_tensor(), f"{layer_key}.lora_b")
    if optimizer is not None and "optimizer.step_count" in tensors:
        optimizer.step_count = int(tensors["optimizer.step_count"].reshape(-1)[0])
        for layer_key, layer in adapter.layers():
            for which, var in (("lora_a", layer.lora_a_tensor()), ("lora_b", layer.lora_b_tensor())):
                if f"optimizer.{layer_key}.{which}.m" not in tensors:
                    continue
                key = optimizer._key(var)
                if key not in optimizer.state:
                    optimizer.add_parameter(key, var)
                m, v = optimizer.state[key]
                put(m, f"optimizer.{layer_key}.{which}.m")
                put(v, f"optimizer.{layer_key}.{which}.v")
    s = meta.get("checkpoint_metadata")
    return CheckpointMetadata.from_json(s) if s else None
