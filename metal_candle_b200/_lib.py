"""ctypes binding of libmetal_candle_b200.so (the C ABI declared in include/mcb200.h).

There is no fallback: if the library is missing, or it cannot bind a Blackwell GPU, every op raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmetal_candle_b200.so"

MCB_F32, MCB_BF16 = 0, 1
MCB_W_OUT_IN, MCB_W_IN_OUT = 0, 1
MCB_ERR_DEVICE_TIMEOUT, MCB_ERR_COMM_TIMEOUT, MCB_ERR_COMM_DEAD, MCB_ERR_COMM_UNAVAILABLE = 100001, 100002, 100003, 100004
MCB_ERR_COMM_BASE = 200000
MCB_OPT_GRAD_TAIL = 0
MCB_OPT_PAIR_MIN_K = 1
MCB_OPT_PDL = 2
MCB_WAIT_CODE_SELFTEST = 90
MCB_COMM_ID_BYTES = 128
MCB_COMM_BLOCKING = 1
MCB_COMM_NO_STREAM = C.c_void_p(-1 & 0xFFFFFFFFFFFFFFFF)


class McbError(RuntimeError):
    """A non-zero status from the C ABI; `.code` is the status, the message is mcb_last_error()."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"[mcb status {code}] {msg}")
        self.code = code


class LoraSegment(C.Structure):
    _fields_ = [("A", C.c_void_p), ("B", C.c_void_p), ("dA", C.c_void_p), ("dB", C.c_void_p),
                ("n_offset", C.c_int64), ("n", C.c_int64)]


class QwenConfig(C.Structure):
    _fields_ = [("vocab_size", C.c_int64), ("hidden_size", C.c_int64), ("intermediate_size", C.c_int64),
                ("num_layers", C.c_int64), ("num_heads", C.c_int64), ("num_kv_heads", C.c_int64),
                ("rms_norm_eps", C.c_float), ("rope_theta", C.c_float)]


class QwenLayer(C.Structure):
    _fields_ = [("input_layernorm", C.c_void_p), ("post_attention_layernorm", C.c_void_p),
                ("weight", C.c_void_p * 7), ("bias", C.c_void_p * 3)]


class QwenWeights(C.Structure):
    _fields_ = [("embed_tokens", C.c_void_p), ("final_norm", C.c_void_p), ("lm_head", C.c_void_p),
                ("layers", C.POINTER(QwenLayer))]


class QwenAdapterEntry(C.Structure):
    _fields_ = [("layer", C.c_int32), ("module", C.c_int32), ("A", C.c_void_p), ("B", C.c_void_p),
                ("dA", C.c_void_p), ("dB", C.c_void_p)]


class AdamWTensor(C.Structure):
    _fields_ = [("p", C.c_void_p), ("g", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
                ("n", C.c_int64), ("t", C.c_int32), ("pad_", C.c_int32)]


_vp, _i64, _i32, _f32, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t

# name -> (restype, argtypes); every symbol include/mcb200.h declares
SIGNATURES = {
    "mcb_init": (_i32, [_i32]),
    "mcb_last_error": (C.c_char_p, []),
    "mcb_version": (_i32, []),
    "mcb_device_status": (_i32, [C.POINTER(C.c_int)]),
    "mcb_check_device": (_i32, []),
    "mcb_selftest_wait_timeout": (_i32, [_i64, C.POINTER(C.c_int64), _vp]),
    "mcb_set_option": (_i32, [_i32, _i32]),
    "mcb_get_option": (_i32, [_i32, C.POINTER(C.c_int)]),
    "mcb_comm_unique_id": (_i32, [_vp]),
    "mcb_comm_init_rank": (_i32, [C.POINTER(_vp), _i32, _i32, _vp, _i32, _i32]),
    "mcb_comm_allreduce_bucket": (_i32, [_vp, _vp, _i64, _vp]),
    "mcb_comm_wait": (_i32, [_vp, _vp, _i32]),
    "mcb_comm_abort": (_i32, [_vp]),
    "mcb_comm_info": (_i32, [_vp, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "mcb_comm_destroy": (_i32, [_vp]),
    "mcb_launch_count": (_i64, []),
    "mcb_profile_enable": (_i32, [_i32]),
    "mcb_profile_summary": (_i32, [_i32, C.POINTER(C.c_int64), C.POINTER(C.c_double), C.POINTER(C.c_double),
                                   C.POINTER(C.c_double)]),
    "mcb_lora_delta_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32, _vp, _sz, _vp]),
    "mcb_lora_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _i32]),
    "mcb_lora_linear_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32, _i32,
                                   _vp, _sz, _vp]),
    "mcb_lora_linear_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _f32,
                                   _i32, _i32, _vp, _sz, _vp]),
    "mcb_lora_linear_fwd_ex": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32, _i32,
                                      _vp, _sz, _vp]),
    "mcb_lora_linear_bwd_ex": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64,
                                      _f32, _i32, _i32, _vp, _sz, _vp]),
    "mcb_lora_linear_bwd_swiglu_supported": (_i32, [_i64, _i64, _i64, _i64, _i32]),
    "mcb_lora_linear_bwd_swiglu": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64,
                                          _f32, _i32, _i32, _vp, _sz, _vp]),
    "mcb_lora_merge_weights": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _i32, _vp]),
    "mcb_lora_fused_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _i32, _i32]),
    "mcb_lora_linear_fused_fwd": (_i32, [_vp, _vp, _vp, C.POINTER(LoraSegment), _i32, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32,
                                         _vp, _sz, _vp]),
    "mcb_lora_linear_fused_bwd": (_i32, [_vp, _vp, C.POINTER(LoraSegment), _i32, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64,
                                         _f32, _i32, _vp, _sz, _vp]),
    "mcb_lora_rank_padded": (_i64, [_i64]),
    "mcb_lora_h_pitch": (_i64, [_i64]),
    "mcb_transpose_2d": (_i32, [_vp, _vp, _i64, _i64, _i32, _vp]),
    "mcb_matmul_workspace_bytes": (_sz, [_i64, _i64, _i32]),
    "mcb_matmul": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "mcb_mul": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "mcb_dropout": (_i32, [_vp, _vp, _i64, _f32, C.c_uint64, C.c_uint64, _i32, _vp]),
    "mcb_mul_scalar": (_i32, [_vp, _vp, _i64, _f32, _i32, _vp]),
    "mcb_rmsnorm_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _f32, _i32, _vp]),
    "mcb_rmsnorm_bwd_workspace_bytes": (_sz, [_i64, _i64]),
    "mcb_rmsnorm_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _f32, _i32, _vp, _sz, _vp]),
    "mcb_rmsnorm_bwd_ex": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _f32, _i32, _vp, _sz, _vp]),
    "mcb_rmsnorm_bwd_noalloc": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _f32, _i32, _vp]),
    "mcb_softmax_fwd": (_i32, [_vp, _vp, _i64, _i64, _i32, _vp]),
    "mcb_softmax_bwd": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _vp]),
    "mcb_softmax_causal_fwd": (_i32, [_vp, _vp, _i64, _i64, _i64, _f32, _i32, _vp]),
    "mcb_softmax_causal_bwd": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _f32, _i32, _vp]),
    "mcb_linear_swiglu_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "mcb_attention_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64]),
    "mcb_attention_causal_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32, _vp, _sz, _vp]),
    "mcb_attention_causal_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32,
                                        _vp, _sz, _vp]),
    "mcb_attention_causal_fwd_ex": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32, _i64, _i32, _vp, _sz,
                                           _vp]),
    "mcb_attention_causal_bwd_ex": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32,
                                           _i64, _i32, _vp, _sz, _vp]),
    "mcb_embedding_fwd": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "mcb_rope_relayout": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32, _i32, _i32, _vp]),
    "mcb_rope_relayout_qkv": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _f32, _i32, _i64, _i32, _vp]),
    "mcb_rope_relayout_ex": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32, _i32, _i64, _i64, _i32, _vp]),
    "mcb_swiglu_fwd": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "mcb_swiglu_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _vp]),
    "mcb_add": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "mcb_cross_entropy": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "mcb_cross_entropy_count": (_i32, [_vp, _vp, _i64, _i64, _vp]),
    "mcb_cross_entropy_chunk": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "mcb_cross_entropy_finish": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "mcb_qwen_arena_bytes": (_sz, [C.POINTER(QwenConfig), C.POINTER(QwenAdapterEntry), _i32, _i32, _i64, _i64]),
    "mcb_qwen_create": (_i32, [C.POINTER(_vp), C.POINTER(QwenConfig), C.POINTER(QwenWeights), C.POINTER(QwenAdapterEntry), _i32, _i32,
                               _f32, _vp, _sz, _vp]),
    "mcb_qwen_set_exchange": (_i32, [_vp, _vp, _vp, _vp, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int), _i32]),
    "mcb_ce_chunk_tokens": (_i64, [_i64, _i64]),
    "mcb_qwen_set_ce_chunk": (_i32, [_vp, _i64]),
    "mcb_qwen_forward_backward": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _vp, _vp]),
    "mcb_qwen_adamw_step": (_i32, [_vp, _f32, _f32, _f32, _f32, _f32, _f32, _vp]),
    "mcb_qwen_train_step": (_i32, [_vp, _vp, _vp, _i64, _i64, _f32, _f32, _f32, _f32, _f32, _f32, _vp, _vp]),
    "mcb_qwen_info": (_i32, [_vp, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(_vp)]),
    "mcb_qwen_destroy": (_i32, [_vp]),
    "mcb_adamw_multi": (_i32, [C.POINTER(AdamWTensor), _i32, _f32, _f32, _f32, _f32, _f32, _f32, _vp]),
}

_lib = None
_inited = set()


def load() -> C.CDLL:
    """Loads the shared library and declares the prototypes.  Needs no GPU."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise McbError(-100, f"{LIB_PATH} is not built; run `python -m metal_candle_b200.build` "
                                 "(there is no CPU or PyTorch fallback)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise McbError(rc, load().mcb_last_error().decode("utf-8", "replace"))


def init(device: int = 0) -> C.CDLL:
    """Binds the library to a CUDA device (idempotent) and returns it."""
    lib = load()
    if device not in _inited:
        check(lib.mcb_init(device))
        _inited.add(device)
    return lib


def device_status() -> int:
    out = C.c_int(0)
    check(load().mcb_device_status(C.byref(out)))
    return out.value


_profiling = False


def profile_enable(on: bool) -> None:
    global _profiling
    check(load().mcb_profile_enable(int(on)))
    _profiling = bool(on)


def profile_enabled() -> bool:
    return _profiling


def profile_summary(kind: int):
    """(launches, total_ms, total_flops, total_bytes) of the finished records of `kind`; clears them."""
    n, ms, fl, by = C.c_int64(0), C.c_double(0), C.c_double(0), C.c_double(0)
    check(load().mcb_profile_summary(kind, C.byref(n), C.byref(ms), C.byref(fl), C.byref(by)))
    return n.value, ms.value, fl.value, by.value
