// Internal interface between the C-ABI LoRA entry points (lora_api.cu) and the two implementations:
// the float32 validation path on CUDA cores (sgemm_f32.cu) and the bfloat16 production path on
// tcgen05 tensor cores (umma_gemm.cu).
#pragma once
#include "common.cuh"

namespace mcb {

struct LoraArgs {
  const void* x = nullptr;     // [M,K]
  const void* W = nullptr;     // [N,K] or [K,N] per w_layout
  const void* bias = nullptr;  // [N] or null
  const void* residual = nullptr;  // added to y (forward, [M,N]) or to dx (backward, [M,K]); may alias the output
  const float* A = nullptr;    // [K,r] float32
  const float* B = nullptr;    // [r,N] float32
  void* y = nullptr;           // [M,N]
  void* h_save = nullptr;      // [rp, h_pitch(M)] scale*(x A) transposed, optional
  const void* dy = nullptr;    // [M,N]
  void* dx = nullptr;          // [M,K]
  void* swiglu_up = nullptr;   // backward, with dx: dx holds gate and this holds up [M,K]; both are replaced by the
                               // SwiGLU backward of the input gradient, which itself is not stored
  float* dA = nullptr;         // [K,r]
  float* dB = nullptr;         // [r,N]
  int accumulate = 0;
  int64_t M = 0, K = 0, N = 0, r = 0;
  float scale = 1.0f;
  int w_layout = MCB_W_OUT_IN;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  cudaStream_t stream = nullptr;
};

// Several projections that share one input, computed as ONE linear with a block-diagonal rank path: segment i owns
// output columns [n_off, n_off + n) of the fused output and has its own adapter (A_i [K,r], B_i [r,n]).
constexpr int kMaxSegments = 4;
struct LoraSegments {
  int count = 0;
  const float* A[kMaxSegments] = {nullptr, nullptr, nullptr, nullptr};
  const float* B[kMaxSegments] = {nullptr, nullptr, nullptr, nullptr};
  float* dA[kMaxSegments] = {nullptr, nullptr, nullptr, nullptr};
  float* dB[kMaxSegments] = {nullptr, nullptr, nullptr, nullptr};
  int64_t n_off[kMaxSegments] = {0, 0, 0, 0};
  int64_t n[kMaxSegments] = {0, 0, 0, 0};
};

inline int64_t rank_padded(int64_t r) { return r <= 0 ? 0 : ((r + 15) / 16) * 16; }
// Row pitch (in elements) of the saved rank intermediate [rp, pitch]: tokens rounded up to 64.
inline int64_t h_pitch(int64_t M) { return ((M + 63) / 64) * 64; }

namespace f32path {
size_t workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t r);
int delta_fwd(const LoraArgs& a);
int linear_fwd(const LoraArgs& a);
int linear_bwd(const LoraArgs& a);
// out[M,N] = a[M,K] b[K,N]
int matmul(const float* a, const float* b, float* out, int64_t M, int64_t K, int64_t N, cudaStream_t st);
}  // namespace f32path

namespace bf16path {
struct GradRequest;
// One call of the fused GEMM  Y = X W^T (+bias) (+R) + (scale X P^T) Q^T ; all operands bf16, K-major.
struct GemmCall {
  const __nv_bfloat16* X = nullptr;   // [M,K]
  const __nv_bfloat16* W = nullptr;   // [N,K] or null
  const __nv_bfloat16* P = nullptr;   // [rp,K] or null
  const __nv_bfloat16* Q = nullptr;   // [N,rp] or null
  const __nv_bfloat16* bias = nullptr;
  const __nv_bfloat16* R = nullptr;   // [M,N] or null
  __nv_bfloat16* Y = nullptr;         // [M,N] or null
  __nv_bfloat16* H = nullptr;         // [rp,h_pitch] or null
  int64_t h_pitch = 0;
  int64_t M = 0, N = 0, K = 0;
  int rp = 0;
  int r_true = 0;  // unpadded rank, for the algorithmic flop count
  float scale = 1.0f;
  // Weight-gradient problems to run as a tail phase of the same launch (one-CTA kernel only), or null.  Problem 0
  // reads the H this call writes.
  const GradRequest* grads = nullptr;
  // The launch directly before this call's GEMM on the same stream is the operand-pack kernel of this call (the
  // GEMM may then be launched as its programmatic dependent).
  bool after_pack = false;
  // Y is the gate buffer of a SwiGLU and this its up buffer: the product is d act, and the epilogue replaces gate and
  // up by d gate and d up instead of storing it (pair kernel only).
  __nv_bfloat16* swiglu_up = nullptr;
};
size_t workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t r);
int delta_fwd(const LoraArgs& a, const DeviceState* ds);
int linear_fwd(const LoraArgs& a, const DeviceState* ds);
int linear_bwd(const LoraArgs& a, const DeviceState* ds);
// Whether linear_bwd can run the SwiGLU backward in the epilogue of its input-gradient product (a.swiglu_up).
bool swiglu_bwd_supported(int64_t M, int64_t K, int64_t N, int64_t r);
// The same two passes for a fused projection with one adapter of rank a.r per segment (a.A / a.B / a.dA / a.dB unused).
size_t fused_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t r, int segments);
int linear_fused_fwd(const LoraArgs& a, const LoraSegments& sg, const DeviceState* ds);
int linear_fused_bwd(const LoraArgs& a, const LoraSegments& sg, const DeviceState* ds);
// out[M,N] = a[M,K] bt[N,K]^T (bt is b transposed, both operands K-major)
int matmul_nt(const void* a, const void* bt, void* out, int64_t M, int64_t K, int64_t N, const DeviceState* ds,
              cudaStream_t st);
// gate, up [M,F] = x w_gu^T (w_gu: gate and up rows interleaved in blocks of 128), act = silu(gate) * up
int launch_gemm2_swiglu(const __nv_bfloat16* X, const __nv_bfloat16* Wgu, __nv_bfloat16* G, __nv_bfloat16* U,
                        __nv_bfloat16* Act, int64_t M, int64_t K, int64_t F, const DeviceState* ds, cudaStream_t st);
}  // namespace bf16path

}  // namespace mcb
