//! Raw bindings to libmetal_candle_b200.so, the B200 (sm_100a) kernels behind metal-candle's custom-op hot path.
//!
//! GENERATED from include/mcb200.h by metal_candle_b200/sys_crate/generate.py - do not edit.  The header
//! documents every entry point (which reference interface it replaces, argument layouts, error codes).
//! All pointers are CUDA device pointers owned by the caller unless the header says otherwise; every call
//! returns a status (`MCB_OK` = 0) and enqueues its work on the given `cudaStream_t` (passed as `*mut c_void`).
//!
//! This crate has never been compiled: the machines the library is built on carry no Rust toolchain.
#![allow(non_camel_case_types, non_snake_case)]

use core::ffi::{c_char, c_int, c_void};

pub const MCB_OK: c_int = 0;
pub const MCB_ERR_NULL: c_int = -1;
pub const MCB_ERR_SHAPE: c_int = -2;
pub const MCB_ERR_ALIGN: c_int = -3;
pub const MCB_ERR_UNSUPPORTED: c_int = -4;
pub const MCB_ERR_WORKSPACE: c_int = -5;
pub const MCB_ERR_NOT_INIT: c_int = -6;
pub const MCB_ERR_DEVICE_TIMEOUT: c_int = 100001;
pub const MCB_ERR_COMM_TIMEOUT: c_int = 100002;
pub const MCB_ERR_COMM_DEAD: c_int = 100003;
pub const MCB_ERR_COMM_UNAVAILABLE: c_int = 100004;
pub const MCB_ERR_COMM_BASE: c_int = 200000;
pub const MCB_F32: c_int = 0;
pub const MCB_BF16: c_int = 1;
pub const MCB_W_OUT_IN: c_int = 0;
pub const MCB_W_IN_OUT: c_int = 1;
pub const MCB_WAIT_CODE_SELFTEST: c_int = 90;
pub const MCB_OPT_GRAD_TAIL: c_int = 0;
pub const MCB_OPT_PAIR_MIN_K: c_int = 1;
pub const MCB_OPT_PDL: c_int = 2;
pub const MCB_COMM_ID_BYTES: c_int = 128;
pub const MCB_COMM_BLOCKING: c_int = 1;

/// `MCB_COMM_NO_STREAM`: wait on the communicator's own state only.
pub const MCB_COMM_NO_STREAM: *mut c_void = usize::MAX as *mut c_void;

/// One tensor of an `mcb_adamw_multi` call (a HOST array of these is passed).
#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct mcb_adamw_tensor {
    pub p: *mut f32,
    pub g: *const f32,
    pub m: *mut f32,
    pub v: *mut f32,
    pub n: i64,
    pub t: i32,
    pub pad_: i32,
}

/// One projection of a fused linear (`mcb_lora_linear_fused_*`; a HOST array of these is passed).
#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct mcb_lora_segment {
    pub A: *const f32,
    pub B: *const f32,
    pub dA: *mut f32,
    pub dB: *mut f32,
    pub n_offset: i64,
    pub n: i64,
}

/// The model's shape (`mcb_qwen_*`).
#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct mcb_qwen_config {
    pub vocab_size: i64,
    pub hidden_size: i64,
    pub intermediate_size: i64,
    pub num_layers: i64,
    pub num_heads: i64,
    pub num_kv_heads: i64,
    pub rms_norm_eps: f32,
    pub rope_theta: f32,
}

/// One decoder layer's bf16 device tensors, weights in [out, in] layout, by module q k v o gate up down.
#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct mcb_qwen_layer {
    pub input_layernorm: *const c_void,
    pub post_attention_layernorm: *const c_void,
    pub weight: [*const c_void; 7],
    pub bias: [*const c_void; 3],
}

#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct mcb_qwen_weights {
    pub embed_tokens: *const c_void,
    pub final_norm: *const c_void,
    pub lm_head: *const c_void,
    pub layers: *const mcb_qwen_layer,
}

#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct mcb_qwen_adapter_entry {
    pub layer: i32,
    pub module: i32,
    pub A: *const f32,
    pub B: *const f32,
    pub dA: *mut f32,
    pub dB: *mut f32,
}

/// Opaque training-step engine (`mcb_qwen_*`).
#[repr(C)]
pub struct mcb_qwen {
    _private: [u8; 0],
}

/// Opaque communicator handle (`mcb_comm_*`).
#[repr(C)]
pub struct mcb_comm {
    _private: [u8; 0],
}

#[link(name = "metal_candle_b200")]
extern "C" {
    pub fn mcb_init(device: c_int) -> c_int;
    pub fn mcb_last_error() -> *const c_char;
    pub fn mcb_version() -> c_int;
    pub fn mcb_device_status(status_out: *mut c_int) -> c_int;
    pub fn mcb_check_device() -> c_int;
    pub fn mcb_selftest_wait_timeout(limit_cycles: i64, waited_cycles_out: *mut i64, stream: *mut c_void) -> c_int;
    pub fn mcb_set_option(option_id: c_int, value: c_int) -> c_int;
    pub fn mcb_get_option(option_id: c_int, value_out: *mut c_int) -> c_int;
    pub fn mcb_launch_count() -> i64;
    pub fn mcb_profile_enable(on: c_int) -> c_int;
    pub fn mcb_profile_summary(kind: c_int, launches: *mut i64, total_ms: *mut f64, total_flops: *mut f64, total_bytes: *mut f64) -> c_int;
    pub fn mcb_lora_delta_fwd(x: *const c_void, A: *const f32, B: *const f32, out: *mut c_void, M: i64, K: i64, N: i64, r: i64, scale: f32, dtype: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_lora_workspace_bytes(M: i64, K: i64, N: i64, r: i64, dtype: c_int) -> usize;
    pub fn mcb_lora_linear_fwd(x: *const c_void, W: *const c_void, bias: *const c_void, A: *const f32, B: *const f32, y: *mut c_void, h_save: *mut c_void, M: i64, K: i64, N: i64, r: i64, scale: f32, dtype: c_int, w_layout: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_lora_linear_bwd(x: *const c_void, W: *const c_void, A: *const f32, B: *const f32, dy: *const c_void, h_save: *const c_void, dx: *mut c_void, dA: *mut f32, dB: *mut f32, accumulate: c_int, M: i64, K: i64, N: i64, r: i64, scale: f32, dtype: c_int, w_layout: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_lora_linear_fwd_ex(x: *const c_void, W: *const c_void, bias: *const c_void, A: *const f32, B: *const f32, residual: *const c_void, y: *mut c_void, h_save: *mut c_void, M: i64, K: i64, N: i64, r: i64, scale: f32, dtype: c_int, w_layout: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_lora_linear_bwd_ex(x: *const c_void, W: *const c_void, A: *const f32, B: *const f32, dy: *const c_void, h_save: *const c_void, dx_residual: *const c_void, dx: *mut c_void, dA: *mut f32, dB: *mut f32, accumulate: c_int, M: i64, K: i64, N: i64, r: i64, scale: f32, dtype: c_int, w_layout: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_lora_linear_bwd_swiglu_supported(M: i64, K: i64, N: i64, r: i64, dtype: c_int) -> c_int;
    pub fn mcb_lora_linear_bwd_swiglu(x: *const c_void, W: *const c_void, A: *const f32, B: *const f32, dy: *const c_void, h_save: *const c_void, gate: *mut c_void, up: *mut c_void, dA: *mut f32, dB: *mut f32, accumulate: c_int, M: i64, K: i64, N: i64, r: i64, scale: f32, dtype: c_int, w_layout: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_lora_merge_weights(W: *const c_void, A: *const f32, B: *const f32, out: *mut c_void, K: i64, N: i64, r: i64, scale: f32, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_lora_fused_workspace_bytes(M: i64, K: i64, N: i64, r: i64, n_segments: c_int, dtype: c_int) -> usize;
    pub fn mcb_lora_linear_fused_fwd(x: *const c_void, W: *const c_void, bias: *const c_void, segments: *const mcb_lora_segment, n_segments: c_int, y: *mut c_void, h_save: *mut c_void, M: i64, K: i64, N: i64, r: i64, scale: f32, dtype: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_lora_linear_fused_bwd(x: *const c_void, Wt: *const c_void, segments: *const mcb_lora_segment, n_segments: c_int, dy: *const c_void, h_save: *const c_void, dx_residual: *const c_void, dx: *mut c_void, accumulate: c_int, M: i64, K: i64, N: i64, r: i64, scale: f32, dtype: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_lora_rank_padded(r: i64) -> i64;
    pub fn mcb_lora_h_pitch(M: i64) -> i64;
    pub fn mcb_transpose_2d(src: *const c_void, dst: *mut c_void, rows: i64, cols: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_linear_swiglu_fwd(x: *const c_void, w_gate_up: *const c_void, gate: *mut c_void, up: *mut c_void, act: *mut c_void, M: i64, K: i64, F: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_matmul_workspace_bytes(K: i64, N: i64, dtype: c_int) -> usize;
    pub fn mcb_matmul(a: *const c_void, b: *const c_void, out: *mut c_void, M: i64, K: i64, N: i64, dtype: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_mul(a: *const c_void, b: *const c_void, out: *mut c_void, n: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_mul_scalar(a: *const c_void, out: *mut c_void, n: i64, value: f32, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_dropout(x: *const c_void, out: *mut c_void, n: i64, p: f32, seed: u64, offset: u64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_rmsnorm_fwd(x: *const c_void, w: *const c_void, y: *mut c_void, rstd: *mut f32, rows: i64, D: i64, eps: f32, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_rmsnorm_bwd_workspace_bytes(rows: i64, D: i64) -> usize;
    pub fn mcb_rmsnorm_bwd(x: *const c_void, w: *const c_void, dy: *const c_void, dx: *mut c_void, dw: *mut f32, accumulate: c_int, rows: i64, D: i64, eps: f32, dtype: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_rmsnorm_bwd_ex(x: *const c_void, w: *const c_void, dy: *const c_void, dx_residual: *const c_void, dx: *mut c_void, dw: *mut f32, accumulate: c_int, rows: i64, D: i64, eps: f32, dtype: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_rmsnorm_bwd_noalloc(x: *const c_void, w: *const c_void, dy: *const c_void, dx: *mut c_void, dw: *mut f32, accumulate: c_int, rows: i64, D: i64, eps: f32, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_softmax_fwd(x: *const c_void, y: *mut c_void, rows: i64, D: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_softmax_bwd(y: *const c_void, dy: *const c_void, dx: *mut c_void, rows: i64, D: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_softmax_causal_fwd(x: *const c_void, y: *mut c_void, rows: i64, D: i64, seq: i64, scale: f32, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_softmax_causal_bwd(y: *const c_void, dy: *const c_void, dx: *mut c_void, rows: i64, D: i64, seq: i64, scale: f32, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_attention_workspace_bytes(nb: i64, groups: i64, seq: i64, head_dim: i64) -> usize;
    pub fn mcb_attention_causal_fwd(q: *const c_void, k: *const c_void, v: *const c_void, o: *mut c_void, lse: *mut f32, nb: i64, groups: i64, seq: i64, head_dim: i64, scale: f32, dtype: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_attention_causal_bwd(q: *const c_void, k: *const c_void, v: *const c_void, o: *const c_void, dout: *const c_void, lse: *const f32, dq: *mut c_void, dk: *mut c_void, dv: *mut c_void, nb: i64, groups: i64, seq: i64, head_dim: i64, scale: f32, dtype: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_attention_causal_fwd_ex(q: *const c_void, k: *const c_void, v: *const c_void, o: *mut c_void, lse: *mut f32, nb: i64, groups: i64, seq: i64, head_dim: i64, scale: f32, dtype: c_int, kv_heads: i64, o_token_major: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_attention_causal_bwd_ex(q: *const c_void, k: *const c_void, v: *const c_void, o: *const c_void, dout: *const c_void, lse: *const f32, dq: *mut c_void, dk: *mut c_void, dv: *mut c_void, nb: i64, groups: i64, seq: i64, head_dim: i64, scale: f32, dtype: c_int, kv_heads: i64, o_token_major: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_comm_unique_id(id_out: *mut c_void) -> c_int;
    pub fn mcb_comm_init_rank(comm_out: *mut *mut mcb_comm, nranks: c_int, rank: c_int, id: *const c_void, timeout_ms: c_int, flags: c_int) -> c_int;
    pub fn mcb_comm_allreduce_bucket(comm: *mut mcb_comm, buf: *mut f32, count: i64, stream: *mut c_void) -> c_int;
    pub fn mcb_comm_wait(comm: *mut mcb_comm, stream: *mut c_void, timeout_ms: c_int) -> c_int;
    pub fn mcb_comm_abort(comm: *mut mcb_comm) -> c_int;
    pub fn mcb_comm_info(comm: *const mcb_comm, nranks: *mut c_int, rank: *mut c_int, dead: *mut c_int, nccl_version: *mut c_int) -> c_int;
    pub fn mcb_comm_destroy(comm: *mut mcb_comm) -> c_int;
    pub fn mcb_adamw_multi(tensors: *const mcb_adamw_tensor, n_tensors: c_int, lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32, grad_scale: f32, stream: *mut c_void) -> c_int;
    pub fn mcb_embedding_fwd(ids: *const i32, table: *const c_void, out: *mut c_void, M: i64, H: i64, vocab: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_rope_relayout(src: *const c_void, dst: *mut c_void, B: i64, S: i64, H: i64, d: i64, theta: f32, rotate: c_int, inverse: c_int, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_rope_relayout_ex(src: *const c_void, dst: *mut c_void, B: i64, S: i64, H: i64, d: i64, theta: f32, rotate: c_int, inverse: c_int, token_pitch: i64, col_offset: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_rope_relayout_qkv(fused: *mut c_void, q: *mut c_void, k: *mut c_void, v: *mut c_void, B: i64, S: i64, Hq: i64, Hk: i64, d: i64, theta: f32, inverse: c_int, token_pitch: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_swiglu_fwd(gate: *const c_void, up: *const c_void, out: *mut c_void, n: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_swiglu_bwd(gate: *const c_void, up: *const c_void, dout: *const c_void, dgate: *mut c_void, dup: *mut c_void, n: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_add(a: *const c_void, b: *const c_void, out: *mut c_void, n: i64, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_cross_entropy(logits: *mut c_void, targets: *const i32, nll: *mut f32, count: *mut i32, loss: *mut f32, M: i64, V: i64, write_grad: c_int, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_cross_entropy_count(targets: *const i32, count: *mut i32, M: i64, V: i64, stream: *mut c_void) -> c_int;
    pub fn mcb_cross_entropy_chunk(logits: *mut c_void, targets: *const i32, nll: *mut f32, count: *const i32, rows: i64, V: i64, write_grad: c_int, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn mcb_cross_entropy_finish(nll: *const f32, count: *const i32, loss: *mut f32, M: i64, stream: *mut c_void) -> c_int;
    pub fn mcb_qwen_arena_bytes(cfg: *const mcb_qwen_config, adapters: *const mcb_qwen_adapter_entry, n_adapters: c_int, rank: c_int, batch: i64, seq: i64) -> usize;
    pub fn mcb_qwen_create(out: *mut *mut mcb_qwen, cfg: *const mcb_qwen_config, weights: *const mcb_qwen_weights, adapters: *const mcb_qwen_adapter_entry, n_adapters: c_int, rank: c_int, scale: f32, arena: *mut c_void, arena_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn mcb_qwen_set_exchange(q: *mut mcb_qwen, comm: *mut mcb_comm, side_stream: *mut c_void, grad_flat: *mut f32, bucket_lo: *const i64, bucket_hi: *const i64, bucket_first_layer: *const c_int, n_buckets: c_int) -> c_int;
    pub fn mcb_qwen_set_ce_chunk(q: *mut mcb_qwen, tokens: i64) -> c_int;
    pub fn mcb_ce_chunk_tokens(tokens: i64, hidden: i64) -> i64;
    pub fn mcb_qwen_forward_backward(q: *mut mcb_qwen, ids: *const i32, targets: *const i32, batch: i64, seq: i64, accumulate: c_int, loss_out: *mut f32, stream: *mut c_void) -> c_int;
    pub fn mcb_qwen_adamw_step(q: *mut mcb_qwen, lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32, grad_scale: f32, stream: *mut c_void) -> c_int;
    pub fn mcb_qwen_train_step(q: *mut mcb_qwen, ids: *const i32, targets: *const i32, batch: i64, seq: i64, lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32, grad_scale: f32, loss_out: *mut f32, stream: *mut c_void) -> c_int;
    pub fn mcb_qwen_info(q: *const mcb_qwen, adamw_steps: *mut i64, persistent_bytes: *mut i64, kept_targets_dev: *mut *mut i32) -> c_int;
    pub fn mcb_qwen_destroy(q: *mut mcb_qwen) -> c_int;
}
