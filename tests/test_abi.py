"""CPU checks of the C-ABI boundary: the library loads without a GPU, exports every symbol that
include/mcb200.h declares, and refuses to run without a CUDA device (no CPU fallback)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "mcb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mcb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from metal_candle_b200 import _lib

    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in mcb200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes prototype"
    assert set(_lib.SIGNATURES) == set(names)
    assert lib.mcb_version() >= 100


def test_no_cpu_fallback():
    import torch

    from metal_candle_b200 import _lib, backend

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = _lib.load()
    assert lib.mcb_init(0) != 0
    assert b"no CPU path" in lib.mcb_last_error() or b"CUDA" in lib.mcb_last_error()
    # the ops reject host tensors instead of computing on the CPU
    with pytest.raises(backend.TrainingError):
        backend.softmax_fused(torch.zeros(2, 4))
    with pytest.raises(backend.TrainingError):
        backend.rms_norm_fused(torch.zeros(2, 4), 1e-5)
    with pytest.raises(backend.TrainingError):
        backend.lora_forward_fused(torch.zeros(2, 4), torch.zeros(4, 2), torch.zeros(2, 4), 1.0)


def test_pure_host_helpers():
    from metal_candle_b200 import _lib

    lib = _lib.load()
    assert [lib.mcb_lora_rank_padded(r) for r in (0, 1, 8, 16, 17, 64)] == [0, 16, 16, 16, 32, 64]
    assert lib.mcb_lora_workspace_bytes(512, 768, 768, 8, _lib.MCB_F32) == 2 * 512 * 16 * 4
    assert [lib.mcb_lora_h_pitch(m) for m in (1, 64, 65, 8192)] == [64, 64, 128, 8192]
    assert lib.mcb_lora_workspace_bytes(512, 768, 768, 8, _lib.MCB_BF16) % 1024 == 0
    assert lib.mcb_lora_workspace_bytes(512, 768, 768, 0, _lib.MCB_BF16) == 0
    assert lib.mcb_rmsnorm_bwd_workspace_bytes(1000, 896) >= 296 * 896 * 4


def test_product_never_imports_oracle():
    for py in (ROOT / "metal_candle_b200").rglob("*.py"):
        src = py.read_text()
        assert "import oracle" not in src and "from oracle" not in src, py


def test_rust_sys_crate_source_matches_the_header():
    """The `-sys` crate a maintainer of the reference would add (metal_candle_b200/sys_crate) is generated from
    include/mcb200.h: it must be up to date and declare every exported entry point exactly once."""
    import subprocess
    import sys

    gen = ROOT / "metal_candle_b200" / "sys_crate" / "generate.py"
    r = subprocess.run([sys.executable, str(gen), "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    src = (ROOT / "metal_candle_b200" / "sys_crate" / "src" / "lib.rs").read_text()
    declared = re.findall(r"pub fn (mcb_[a-z0-9_]+)\(", src)
    assert sorted(declared) == declared_symbols()
    assert "#[repr(C)]" in src and "pub struct mcb_adamw_tensor" in src


def test_host_only_entry_points_work_without_a_gpu():
    """Switches, the launch counter and the engine's arena sizing are pure host code."""
    import ctypes as C

    from metal_candle_b200 import _lib

    lib = _lib.load()
    v = C.c_int(-1)
    assert lib.mcb_get_option(_lib.MCB_OPT_GRAD_TAIL, C.byref(v)) == 0 and v.value == 1
    assert lib.mcb_set_option(_lib.MCB_OPT_GRAD_TAIL, 0) == 0
    assert lib.mcb_get_option(_lib.MCB_OPT_GRAD_TAIL, C.byref(v)) == 0 and v.value == 0
    assert lib.mcb_set_option(_lib.MCB_OPT_GRAD_TAIL, 1) == 0
    assert lib.mcb_get_option(_lib.MCB_OPT_PAIR_MIN_K, C.byref(v)) == 0 and v.value == 1536
    assert lib.mcb_set_option(99, 1) == -2 and lib.mcb_get_option(0, None) == -1
    assert lib.mcb_launch_count() >= 0
    # the 0.5B model, rank 16 on q/k/v/o, 16 x 2048 tokens: derived weights + 24 layers of saved activations + scratch
    cfg = _lib.QwenConfig(151936, 896, 4864, 24, 14, 2, 1e-6, 1e6)
    entries = (_lib.QwenAdapterEntry * 96)()
    for i in range(24):
        for j, m in enumerate((0, 1, 2, 3)):
            entries[4 * i + j] = _lib.QwenAdapterEntry(i, m, None, None, None, None)
    big = lib.mcb_qwen_arena_bytes(C.byref(cfg), entries, 96, 16, 16, 2048)
    small = lib.mcb_qwen_arena_bytes(C.byref(cfg), entries, 96, 16, 1, 128)
    assert 20e9 < big < 40e9 and 1e9 < small < 3e9 and small < big
    assert lib.mcb_qwen_arena_bytes(C.byref(cfg), entries, 96, 32, 16, 2048) == 0      # 3 x 32 rank columns > 64
    # the loss chunk: whole waves of the lm_head backward's 256-token tiles over 74 CTA pairs (37 x 4 = 148 tiles)
    assert lib.mcb_ce_chunk_tokens(32768, 896) == 9472 and lib.mcb_ce_chunk_tokens(384, 256) == 384
    assert 4096 <= lib.mcb_ce_chunk_tokens(100000, 4096) <= 12288 and lib.mcb_ce_chunk_tokens(0, 896) == 0
    bad = _lib.QwenConfig(151936, 896, 4864, 24, 7, 1, 1e-6, 1e6)                      # head_dim 128
    assert lib.mcb_qwen_arena_bytes(C.byref(bad), entries, 96, 16, 1, 128) == 0
    assert b"head_dim" in lib.mcb_last_error()
