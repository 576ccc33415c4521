"""Adapter checkpoints in the reference's safetensors layout (src/training/checkpoint.rs:65-178): byte-level
agreement with the `safetensors` crate (through its Python binding), round trips, and a hand-built file in the
reference's key layout loading into an adapter.  Host-only."""
import json
import struct

import numpy as np
import pytest
import torch

from metal_candle_b200 import checkpoint as CK


class _Layer:
    def __init__(self, in_f, out_f, r, gen):
        self.lora_a = torch.randn(in_f, r, generator=gen)
        self.lora_b = torch.randn(r, out_f, generator=gen)

    def lora_a_tensor(self):
        return self.lora_a

    def lora_b_tensor(self):
        return self.lora_b


class _Adapter:
    """The two accessors save/load use, over CPU tensors (LoRAAdapter itself needs a CUDA device)."""

    def __init__(self, seed, n_layers=2, modules=("q_proj", "v_proj"), in_f=32, out_f=(32, 16), r=4):
        g = torch.Generator().manual_seed(seed)
        self._layers = {f"layers.{i}.{m}": _Layer(in_f, out_f[j], r, g) for i in range(n_layers)
                        for j, m in enumerate(modules)}

    def layers(self):
        return list(self._layers.items())


def test_container_matches_the_safetensors_crate_byte_for_byte(tmp_path):
    st = pytest.importorskip("safetensors.numpy")
    rng = np.random.default_rng(0)
    tensors = {"layers.1.q_proj.lora_b": rng.standard_normal((4, 32)).astype(np.float32),
               "layers.0.q_proj.lora_a": rng.standard_normal((32, 4)).astype(np.float32),
               "layers.10.v_proj.lora_a": rng.standard_normal((32, 4)).astype(np.float32),
               "optimizer.step_count": np.array([7], dtype=np.int64)}
    meta = {"checkpoint_metadata": CK.CheckpointMetadata(100, 1.5, 1e-4, 1234567890).to_json()}
    mine = CK.serialize(tensors, meta)
    assert mine == st.save(tensors, metadata=meta)
    assert CK.serialize(tensors, None) == st.save(tensors)
    back, m2 = CK.deserialize(mine)
    assert m2 == meta and set(back) == set(tensors)
    for k in tensors:
        assert back[k].dtype == tensors[k].dtype and np.array_equal(back[k], tensors[k])
    # and the crate reads what this module writes
    p = tmp_path / "a.safetensors"
    CK.save_file(p, tensors, meta)
    theirs = st.load_file(str(p))
    for k in tensors:
        assert np.array_equal(theirs[k], tensors[k])


def test_save_load_round_trip_with_metadata(tmp_path):
    """checkpoint.rs:185-222 (save with metadata, load into a fresh adapter) and :252-296 (weights preserved)."""
    a, b = _Adapter(1), _Adapter(2)
    p = tmp_path / "ck.safetensors"
    CK.save_checkpoint(a, p, CK.CheckpointMetadata(global_step=100, loss=1.5, learning_rate=1e-4, timestamp=1_234_567_890))
    got = CK.load_checkpoint(b, p)
    assert got == CK.CheckpointMetadata(100, 1.5, 1e-4, 1_234_567_890)   # the reference's loader returns None here
    for (ka, la), (kb, lb) in zip(a.layers(), b.layers()):
        assert ka == kb
        assert torch.equal(la.lora_a, lb.lora_a) and torch.equal(la.lora_b, lb.lora_b)
    # the file's key set and dtypes are the reference's
    tensors, meta = CK.load_file(p)
    assert set(tensors) == {f"layers.{i}.{m}.lora_{ab}" for i in range(2) for m in ("q_proj", "v_proj") for ab in "ab"}
    assert all(t.dtype == np.float32 for t in tensors.values())
    assert json.loads(meta["checkpoint_metadata"]) == {"global_step": 100, "loss": 1.5, "learning_rate": 1e-4,
                                                        "timestamp": 1234567890}


def test_save_without_metadata(tmp_path):
    """checkpoint.rs:224-249."""
    a, b = _Adapter(3, n_layers=1, modules=("q_proj",)), _Adapter(4, n_layers=1, modules=("q_proj",))
    p = tmp_path / "ck.safetensors"
    CK.save_checkpoint(a, p, None)
    assert CK.load_checkpoint(b, p) is None
    assert torch.equal(a.layers()[0][1].lora_a, b.layers()[0][1].lora_a)
    n = struct.unpack("<Q", p.read_bytes()[:8])[0]
    assert "__metadata__" not in json.loads(p.read_bytes()[8:8 + n])


def test_hand_built_reference_file_loads(tmp_path):
    """A file assembled by hand in the reference's key layout (extra and missing keys included) loads the way
    load_checkpoint (checkpoint.rs:164-175) does: present keys are set, absent ones stay, unknown ones are ignored."""
    a = _Adapter(5, n_layers=2, modules=("q_proj",))
    keep = a.layers()[1][1].lora_b.clone()
    want_a0 = np.arange(32 * 4, dtype=np.float32).reshape(32, 4)
    want_b0 = -np.arange(4 * 32, dtype=np.float32).reshape(4, 32)
    want_a1 = np.full((32, 4), 0.25, dtype=np.float32)
    payload = want_a0.tobytes() + want_b0.tobytes() + want_a1.tobytes() + np.zeros(3, np.float32).tobytes()
    header = {"__metadata__": {"checkpoint_metadata": '{"global_step":7,"loss":0.5,"learning_rate":0.001,"timestamp":9}'},
              "layers.0.q_proj.lora_a": {"dtype": "F32", "shape": [32, 4], "data_offsets": [0, 512]},
              "layers.0.q_proj.lora_b": {"dtype": "F32", "shape": [4, 32], "data_offsets": [512, 1024]},
              "layers.1.q_proj.lora_a": {"dtype": "F32", "shape": [32, 4], "data_offsets": [1024, 1536]},
              "something.else": {"dtype": "F32", "shape": [3], "data_offsets": [1536, 1548]}}
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    p = tmp_path / "ref.safetensors"
    p.write_bytes(struct.pack("<Q", len(hj)) + hj + payload)
    meta = CK.load_checkpoint(a, p)
    assert meta.global_step == 7 and meta.loss == 0.5 and meta.timestamp == 9
    l0, l1 = a.layers()[0][1], a.layers()[1][1]
    assert np.array_equal(l0.lora_a.numpy(), want_a0) and np.array_equal(l0.lora_b.numpy(), want_b0)
    assert np.array_equal(l1.lora_a.numpy(), want_a1) and torch.equal(l1.lora_b, keep)


def test_optimizer_state_round_trip(tmp_path):
    from metal_candle_b200.training import AdamW, AdamWConfig

    a, b = _Adapter(6), _Adapter(7)
    opt = AdamW(AdamWConfig())
    g = torch.Generator().manual_seed(0)
    for _, l in a.layers():
        for var in (l.lora_a, l.lora_b):
            key = opt._key(var)
            opt.add_parameter(key, var)
            opt.state[key][0].normal_(generator=g)
            opt.state[key][1].uniform_(generator=g)
    opt.step_count = 4 * 8
    p = tmp_path / "ck.safetensors"
    CK.save_checkpoint(a, p, CK.CheckpointMetadata.now(8, 2.0, 5e-5), optimizer=opt)
    opt2 = AdamW(AdamWConfig())
    meta = CK.load_checkpoint(b, p, optimizer=opt2)
    assert meta.global_step == 8 and opt2.step_count == 32
    for (_, la), (_, lb) in zip(a.layers(), b.layers()):
        for va, vb in ((la.lora_a, lb.lora_a), (la.lora_b, lb.lora_b)):
            ma, va_ = opt.state_of(va)
            mb, vb_ = opt2.state_of(vb)
            assert torch.equal(ma, mb) and torch.equal(va_, vb_)
    # a loader that knows nothing of the optimizer keys (the reference's) still gets the adapter
    c = _Adapter(8)
    CK.load_checkpoint(c, p)
    assert torch.equal(c.layers()[0][1].lora_a, a.layers()[0][1].lora_a)


def test_errors(tmp_path):
    a = _Adapter(9)
    with pytest.raises(CK.CheckpointError):
        CK.load_checkpoint(a, tmp_path / "missing.safetensors")
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\x05\x00\x00")
    with pytest.raises(CK.CheckpointError):
        CK.load_checkpoint(a, bad)
    bad.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(CK.CheckpointError):
        CK.load_checkpoint(a, bad)
    # offsets that do not match the shape
    hj = json.dumps({"layers.0.q_proj.lora_a": {"dtype": "F32", "shape": [32, 4], "data_offsets": [0, 8]}}).encode()
    bad.write_bytes(struct.pack("<Q", len(hj)) + hj + b"\0" * 8)
    with pytest.raises(CK.CheckpointError):
        CK.load_checkpoint(a, bad)
    # a stored tensor of the wrong shape is refused, like Var::set
    CK.save_file(bad, {"layers.0.q_proj.lora_a": np.zeros((8, 4), np.float32)})
    with pytest.raises(CK.CheckpointError, match="shape"):
        CK.load_checkpoint(a, bad)
