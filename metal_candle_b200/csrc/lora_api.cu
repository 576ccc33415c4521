// extern "C" entry points of the fused LoRA linear: argument validation (the checks FusedLoRAOp::new
// and its forward do, src/backend/custom_ops.rs:118-168,283-313) and dispatch to the float32 or the
// bfloat16 implementation.
#include "lora_internal.cuh"

using namespace mcb;

namespace {

int check_dims(const char* op, int64_t M, int64_t K, int64_t N, int64_t r, int dtype, bool rank_required) {
  if (M <= 0 || K <= 0 || N <= 0)
    return fail(MCB_ERR_SHAPE, "%s: M=%lld K=%lld N=%lld must be positive", op, (long long)M, (long long)K, (long long)N);
  // The reference range-checks every dimension into u32 (src/backend/custom_ops.rs:283-313).
  if (M > 0xffffffffll || K > 0xffffffffll || N > 0xffffffffll)
    return fail(MCB_ERR_SHAPE, "%s: dimension exceeds u32", op);
  if (r < 0 || (rank_required && r == 0))
    return fail(MCB_ERR_SHAPE, "%s: LoRA rank must be greater than 0", op);
  // LoRALayer::new rejects rank > min(in, out) (src/training/lora.rs:222-231).
  if (r > (K < N ? K : N))
    return fail(MCB_ERR_SHAPE, "%s: LoRA rank %lld exceeds maximum rank %lld (min of in_features=%lld, out_features=%lld)", op,
                (long long)r, (long long)(K < N ? K : N), (long long)K, (long long)N);
  if (dtype != MCB_F32 && dtype != MCB_BF16) return fail(MCB_ERR_UNSUPPORTED, "%s: dtype %d", op, dtype);
  return MCB_OK;
}

}  // namespace

extern "C" int64_t mcb_lora_rank_padded(int64_t r) { return rank_padded(r); }

extern "C" int64_t mcb_lora_h_pitch(int64_t M) { return M <= 0 ? 0 : h_pitch(M); }

extern "C" size_t mcb_lora_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t r, int dtype) {
  if (M <= 0 || K <= 0 || N <= 0 || r <= 0) return 0;
  return dtype == MCB_F32 ? f32path::workspace_bytes(M, K, N, r) : bf16path::workspace_bytes(M, K, N, r);
}

extern "C" int mcb_lora_delta_fwd(const void* x, const float* A, const float* B, void* out, int64_t M, int64_t K,
                                  int64_t N, int64_t r, float scale, int dtype, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  MCB_NVTX_RANGE("mcb_lora_delta_fwd");
  if (!x || !A || !B || !out) return fail(MCB_ERR_NULL, "lora_delta_fwd: null pointer");
  if (int rc = check_dims("lora_delta_fwd", M, K, N, r, dtype, true)) return rc;
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  LoraArgs a;
  a.x = x; a.A = A; a.B = B; a.y = out;
  a.M = M; a.K = K; a.N = N; a.r = r; a.scale = scale;
  a.ws = workspace; a.ws_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return dtype == MCB_F32 ? f32path::delta_fwd(a) : bf16path::delta_fwd(a, ds);
}

extern "C" int mcb_lora_linear_fwd_ex(const void* x, const void* W, const void* bias, const float* A, const float* B,
                                      const void* residual, void* y, void* h_save, int64_t M, int64_t K, int64_t N, int64_t r, float scale, int dtype,
                                   int w_layout, void* workspace, size_t workspace_bytes, void* stream) {
  MCB_NVTX_RANGE("mcb_lora_linear_fwd_ex");
  if (!x || !W || !y) return fail(MCB_ERR_NULL, "lora_linear_fwd: x, W or y is null");
  if (r > 0 && (!A || !B)) return fail(MCB_ERR_NULL, "lora_linear_fwd: rank %lld but A or B is null", (long long)r);
  if (int rc = check_dims("lora_linear_fwd", M, K, N, r, dtype, false)) return rc;
  if (w_layout != MCB_W_OUT_IN && w_layout != MCB_W_IN_OUT) return fail(MCB_ERR_UNSUPPORTED, "lora_linear_fwd: w_layout %d", w_layout);
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  LoraArgs a;
  a.x = x; a.W = W; a.bias = bias; a.A = A; a.B = B; a.y = y; a.h_save = h_save; a.residual = residual;
  a.M = M; a.K = K; a.N = N; a.r = r; a.scale = scale; a.w_layout = w_layout;
  a.ws = workspace; a.ws_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return dtype == MCB_F32 ? f32path::linear_fwd(a) : bf16path::linear_fwd(a, ds);
}

extern "C" int mcb_lora_linear_bwd_ex(const void* x, const void* W, const float* A, const float* B, const void* dy,
                                      const void* h_save, const void* dx_residual, void* dx, float* dA, float* dB, int accumulate, int64_t M,
                                   int64_t K, int64_t N, int64_t r, float scale, int dtype, int w_layout, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  MCB_NVTX_RANGE("mcb_lora_linear_bwd_ex");
  if (!dy) return fail(MCB_ERR_NULL, "lora_linear_bwd: dy is null");
  if (dx && !W) return fail(MCB_ERR_NULL, "lora_linear_bwd: dx wanted but W is null");
  if (r > 0 && (!A || !B)) return fail(MCB_ERR_NULL, "lora_linear_bwd: rank %lld but A or B is null", (long long)r);
  if (r > 0 && (dA || dB) && !x) return fail(MCB_ERR_NULL, "lora_linear_bwd: dA/dB wanted but x is null");
  if ((dA == nullptr) != (dB == nullptr)) return fail(MCB_ERR_NULL, "lora_linear_bwd: pass both dA and dB, or neither");
  if (int rc = check_dims("lora_linear_bwd", M, K, N, r, dtype, false)) return rc;
  if (w_layout != MCB_W_OUT_IN && w_layout != MCB_W_IN_OUT) return fail(MCB_ERR_UNSUPPORTED, "lora_linear_bwd: w_layout %d", w_layout);
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  LoraArgs a;
  a.x = x; a.W = W; a.A = A; a.B = B; a.dy = dy; a.h_save = const_cast<void*>(h_save);
  a.dx = dx; a.dA = dA; a.dB = dB; a.accumulate = accumulate; a.residual = dx_residual;
  a.M = M; a.K = K; a.N = N; a.r = r; a.scale = scale; a.w_layout = w_layout;
  a.ws = workspace; a.ws_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return dtype == MCB_F32 ? f32path::linear_bwd(a) : bf16path::linear_bwd(a, ds);
}

extern "C" int mcb_lora_linear_bwd_swiglu_supported(int64_t M, int64_t K, int64_t N, int64_t r, int dtype) {
  return dtype == MCB_BF16 && bf16path::swiglu_bwd_supported(M, K, N, r) ? 1 : 0;
}

extern "C" int mcb_lora_linear_bwd_swiglu(const void* x, const void* W, const float* A, const float* B, const void* dy,
                                          const void* h_save, void* gate, void* up, float* dA, float* dB, int accumulate,
                                          int64_t M, int64_t K, int64_t N, int64_t r, float scale, int dtype, int w_layout,
                                          void* workspace, size_t workspace_bytes, void* stream) {
  MCB_NVTX_RANGE("mcb_lora_linear_bwd_swiglu");
  if (!dy || !W || !gate || !up) return fail(MCB_ERR_NULL, "lora_linear_bwd_swiglu: dy, W, gate or up is null");
  if (gate == up) return fail(MCB_ERR_SHAPE, "lora_linear_bwd_swiglu: gate and up are the same buffer");
  if (r > 0 && (!A || !B)) return fail(MCB_ERR_NULL, "lora_linear_bwd_swiglu: rank %lld but A or B is null", (long long)r);
  if (r > 0 && (dA || dB) && !x) return fail(MCB_ERR_NULL, "lora_linear_bwd_swiglu: dA/dB wanted but x is null");
  if ((dA == nullptr) != (dB == nullptr)) return fail(MCB_ERR_NULL, "lora_linear_bwd_swiglu: pass both dA and dB, or neither");
  if (int rc = check_dims("lora_linear_bwd_swiglu", M, K, N, r, dtype, false)) return rc;
  if (dtype != MCB_BF16) return fail(MCB_ERR_UNSUPPORTED, "lora_linear_bwd_swiglu: bfloat16 only (use mcb_lora_linear_bwd_ex and mcb_swiglu_bwd)");
  if (w_layout != MCB_W_IN_OUT) return fail(MCB_ERR_UNSUPPORTED, "lora_linear_bwd_swiglu: W must be [in,out] (MCB_W_IN_OUT)");
  if (!aligned16(gate) || !aligned16(up)) return fail(MCB_ERR_ALIGN, "lora_linear_bwd_swiglu: 16-byte alignment");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  LoraArgs a;
  a.x = x; a.W = W; a.A = A; a.B = B; a.dy = dy; a.h_save = const_cast<void*>(h_save);
  a.dx = gate; a.swiglu_up = up; a.dA = dA; a.dB = dB; a.accumulate = accumulate;
  a.M = M; a.K = K; a.N = N; a.r = r; a.scale = scale; a.w_layout = w_layout;
  a.ws = workspace; a.ws_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return bf16path::linear_bwd(a, ds);
}

extern "C" size_t mcb_matmul_workspace_bytes(int64_t K, int64_t N, int dtype) {
  if (K <= 0 || N <= 0 || dtype != MCB_BF16) return 0;
  return static_cast<size_t>(K) * static_cast<size_t>(N) * 2;
}

extern "C" int mcb_matmul(const void* a, const void* b, void* out, int64_t M, int64_t K, int64_t N, int dtype,
                          void* workspace, size_t workspace_bytes, void* stream) {
  MCB_NVTX_RANGE("mcb_matmul");
  if (!a || !b || !out) return fail(MCB_ERR_NULL, "matmul: null pointer");
  if (M <= 0 || K <= 0 || N <= 0) return fail(MCB_ERR_SHAPE, "matmul: M=%lld K=%lld N=%lld must be positive", (long long)M, (long long)K, (long long)N);
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MCB_F32)
    return f32path::matmul(static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(out), M, K, N, st);
  if (dtype != MCB_BF16) return fail(MCB_ERR_UNSUPPORTED, "matmul: dtype %d", dtype);
  // tensor cores want both operands with the reduction index contiguous: transpose b into the workspace
  if (!workspace || workspace_bytes < mcb_matmul_workspace_bytes(K, N, dtype))
    return fail(MCB_ERR_WORKSPACE, "matmul(bf16): workspace %zu < %zu bytes", workspace_bytes, mcb_matmul_workspace_bytes(K, N, dtype));
  if (int rc = mcb_transpose_2d(b, workspace, K, N, dtype, stream)) return rc;
  return bf16path::matmul_nt(a, workspace, out, M, K, N, ds, st);
}

extern "C" int mcb_linear_swiglu_fwd(const void* x, const void* w_gate_up, void* gate, void* up, void* act, int64_t M,
                                     int64_t K, int64_t F, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_linear_swiglu_fwd");
  if (!x || !w_gate_up || !gate || !up || !act) return fail(MCB_ERR_NULL, "linear_swiglu_fwd: null pointer");
  if (M <= 0 || K <= 0 || F <= 0) return fail(MCB_ERR_SHAPE, "linear_swiglu_fwd: M=%lld K=%lld F=%lld must be positive", (long long)M, (long long)K, (long long)F);
  if (dtype != MCB_BF16) return fail(MCB_ERR_UNSUPPORTED, "linear_swiglu_fwd: bfloat16 only (use two mcb_lora_linear_fwd calls and mcb_swiglu_fwd)");
  if (!aligned16(x) || !aligned16(w_gate_up) || !aligned16(gate) || !aligned16(up) || !aligned16(act))
    return fail(MCB_ERR_ALIGN, "linear_swiglu_fwd: 16-byte alignment");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  return bf16path::launch_gemm2_swiglu(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w_gate_up),
                                       static_cast<__nv_bfloat16*>(gate), static_cast<__nv_bfloat16*>(up),
                                       static_cast<__nv_bfloat16*>(act), M, K, F, ds, static_cast<cudaStream_t>(stream));
}

extern "C" int mcb_lora_linear_fwd(const void* x, const void* W, const void* bias, const float* A, const float* B, void* y,
                                   void* h_save, int64_t M, int64_t K, int64_t N, int64_t r, float scale, int dtype,
                                   int w_layout, void* workspace, size_t workspace_bytes, void* stream) {
  return mcb_lora_linear_fwd_ex(x, W, bias, A, B, nullptr, y, h_save, M, K, N, r, scale, dtype, w_layout, workspace,
                                workspace_bytes, stream);
}

extern "C" int mcb_lora_linear_bwd(const void* x, const void* W, const float* A, const float* B, const void* dy,
                                   const void* h_save, void* dx, float* dA, float* dB, int accumulate, int64_t M,
                                   int64_t K, int64_t N, int64_t r, float scale, int dtype, int w_layout, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  return mcb_lora_linear_bwd_ex(x, W, A, B, dy, h_save, nullptr, dx, dA, dB, accumulate, M, K, N, r, scale, dtype, w_layout,
                                workspace, workspace_bytes, stream);
}

// ---- several projections of one input as one linear (block-diagonal rank path) ---------------------------------
namespace {
int to_segments(const char* op, const mcb_lora_segment* segs, int n_segments, int64_t N, int64_t r, bool backward, LoraSegments* out) {
  if (!segs) return fail(MCB_ERR_NULL, "%s: null segment table", op);
  if (n_segments < 1 || n_segments > kMaxSegments) return fail(MCB_ERR_SHAPE, "%s: %d segments (1..%d)", op, n_segments, kMaxSegments);
  out->count = n_segments;
  for (int i = 0; i < n_segments; ++i) {
    out->A[i] = segs[i].A; out->B[i] = segs[i].B;
    out->dA[i] = backward ? segs[i].dA : nullptr; out->dB[i] = backward ? segs[i].dB : nullptr;
    out->n_off[i] = segs[i].n_offset; out->n[i] = segs[i].n;
    if (r > segs[i].n) return fail(MCB_ERR_SHAPE, "%s: LoRA rank %lld exceeds the width %lld of segment %d", op, (long long)r, (long long)segs[i].n, i);
  }
  (void)N;
  return MCB_OK;
}
}  // namespace

extern "C" size_t mcb_lora_fused_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t r, int n_segments, int dtype) {
  if (M <= 0 || K <= 0 || N <= 0 || r <= 0 || n_segments <= 0 || dtype != MCB_BF16) return 0;
  return bf16path::fused_workspace_bytes(M, K, N, r, n_segments);
}

extern "C" int mcb_lora_linear_fused_fwd(const void* x, const void* W, const void* bias, const mcb_lora_segment* segments,
                                         int n_segments, void* y, void* h_save, int64_t M, int64_t K, int64_t N, int64_t r,
                                         float scale, int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  MCB_NVTX_RANGE("mcb_lora_linear_fused_fwd");
  if (!x || !W || !y) return fail(MCB_ERR_NULL, "lora_linear_fused_fwd: x, W or y is null");
  if (int rc = check_dims("lora_linear_fused_fwd", M, K, N, r, dtype, true)) return rc;
  if (dtype != MCB_BF16) return fail(MCB_ERR_UNSUPPORTED, "lora_linear_fused_fwd: bfloat16 only (call mcb_lora_linear_fwd per projection for float32)");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  LoraSegments sg;
  if (int rc = to_segments("lora_linear_fused_fwd", segments, n_segments, N, r, false, &sg)) return rc;
  LoraArgs a;
  a.x = x; a.W = W; a.bias = bias; a.y = y; a.h_save = h_save;
  a.M = M; a.K = K; a.N = N; a.r = r; a.scale = scale; a.w_layout = MCB_W_OUT_IN;
  a.ws = workspace; a.ws_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return bf16path::linear_fused_fwd(a, sg, ds);
}

extern "C" int mcb_lora_linear_fused_bwd(const void* x, const void* Wt, const mcb_lora_segment* segments, int n_segments,
                                         const void* dy, const void* h_save, const void* dx_residual, void* dx, int accumulate,
                                         int64_t M, int64_t K, int64_t N, int64_t r, float scale, int dtype, void* workspace,
                                         size_t workspace_bytes, void* stream) {
  MCB_NVTX_RANGE("mcb_lora_linear_fused_bwd");
  if (!x || !dy || !h_save) return fail(MCB_ERR_NULL, "lora_linear_fused_bwd: x, dy or h_save is null");
  if (dx && !Wt) return fail(MCB_ERR_NULL, "lora_linear_fused_bwd: dx wanted but the weight is null");
  if (int rc = check_dims("lora_linear_fused_bwd", M, K, N, r, dtype, true)) return rc;
  if (dtype != MCB_BF16) return fail(MCB_ERR_UNSUPPORTED, "lora_linear_fused_bwd: bfloat16 only (call mcb_lora_linear_bwd per projection for float32)");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  LoraSegments sg;
  if (int rc = to_segments("lora_linear_fused_bwd", segments, n_segments, N, r, true, &sg)) return rc;
  LoraArgs a;
  a.x = x; a.W = Wt; a.dy = dy; a.h_save = const_cast<void*>(h_save); a.dx = dx; a.residual = dx_residual; a.accumulate = accumulate;
  a.M = M; a.K = K; a.N = N; a.r = r; a.scale = scale; a.w_layout = MCB_W_IN_OUT;
  a.ws = workspace; a.ws_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return bf16path::linear_fused_bwd(a, sg, ds);
}
