/*
 * mcb200.h -- C ABI of libmetal_candle_b200.so: the B200 (sm_100a) kernels behind the
 * custom-op hot path of GarthDB/metal-candle (fused LoRA linear, RMSNorm, row softmax, AdamW).
 *
 * Conventions (all entry points):
 *   - return 0 on success; a negative value for an invalid argument (null pointer, bad shape,
 *     misalignment, unsupported layout); a positive value for a CUDA runtime error (its
 *     cudaError_t) or MCB_ERR_DEVICE_TIMEOUT.  Nothing aborts or throws across the boundary.
 *   - mcb_last_error() returns a thread-local message for the last non-zero status.
 *   - every pointer named x/W/A/B/y/... is a DEVICE pointer owned by the caller, outputs and
 *     workspaces included.  The library allocates no device memory in these calls (the one small
 *     per-device status word is created by mcb_init).  There is no CPU fallback.
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, never synchronised.
 *   - matrices are dense row-major.  M = product of the leading dims (batch*seq tokens),
 *     K = in_features, N = out_features, r = LoRA rank.
 *
 * Reference paths are given as file:line within the metal-candle source tree.
 */
#ifndef MCB200_H_
#define MCB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MCB_OK 0
#define MCB_ERR_NULL (-1)          /* a required pointer is null */
#define MCB_ERR_SHAPE (-2)         /* a dimension is zero/negative/out of range, or shapes disagree */
#define MCB_ERR_ALIGN (-3)         /* pointer or row pitch not aligned as the kernel needs */
#define MCB_ERR_UNSUPPORTED (-4)   /* dtype / layout / rank combination the kernel does not implement */
#define MCB_ERR_WORKSPACE (-5)     /* workspace missing or too small */
#define MCB_ERR_NOT_INIT (-6)      /* mcb_init was not called for the current device */
#define MCB_ERR_DEVICE_TIMEOUT 100001 /* a bounded device-side wait ran out (mcb_check_device, mcb_device_status) */
#define MCB_ERR_COMM_TIMEOUT 100002   /* a collective or the rendezvous passed its host deadline; communicator aborted */
#define MCB_ERR_COMM_DEAD 100003      /* the communicator was aborted earlier and takes no more work */
#define MCB_ERR_COMM_UNAVAILABLE 100004 /* no NCCL library could be bound at run time */
#define MCB_ERR_COMM_BASE 200000      /* + ncclResult_t: an error reported by NCCL */

/* Element types.  MCB_F32 is the validation path (CUDA-core FMA, matches the reference's f32 CPU
 * arithmetic to <=1e-4); MCB_BF16 is the production path (tcgen05 tensor cores, fp32 accumulate). */
#define MCB_F32 0
#define MCB_BF16 1

/* Layout of the frozen weight.  candle_nn::Linear stores [out, in] (src/models/transformer.rs:189-192). */
#define MCB_W_OUT_IN 0 /* W is [N, K]: what the forward consumes  */
#define MCB_W_IN_OUT 1 /* W is [K, N]: what the backward consumes */

/* ---- library / device ------------------------------------------------------------------ */

/* Replaces Device::new_metal / MetalKernelCompiler::new (src/backend/device.rs:58-87,
 * src/backend/metal_kernels.rs:70-81): binds the library to CUDA device `device`, checks that it is
 * compute capability 10.x, resolves the driver's tensor-map encoder, raises the kernels' dynamic
 * shared-memory limits and allocates the per-device status word.  Idempotent. */
int mcb_init(int device);
const char* mcb_last_error(void);
int mcb_version(void);
/* Reads (and clears) the device-side status word of the current device: 0, or a code naming the
 * bounded wait that gave up.  Synchronises the device. */
int mcb_device_status(int* status_out);

/* mcb_device_status as a status: synchronises the device, returns MCB_OK when no bounded wait has run out since the
 * last check and MCB_ERR_DEVICE_TIMEOUT (message naming the wait's code) otherwise; clears the word.  This is the
 * library's failure detection for its own kernels: a wait on an mbarrier or a flag that runs out does not trap or
 * hang, the kernel records a code and returns, and the results of that launch are invalid.  No counterpart in the
 * reference (its kernels have no waits). */
int mcb_check_device(void);
/* Makes a bounded wait run out on purpose: one warp waits on a barrier that nothing arrives at, for at most
 * `limit_cycles` SM cycles (1 .. 2e9), records MCB_WAIT_CODE_SELFTEST in the status word and returns normally.
 * Synchronises `stream`.  Returns MCB_OK when the wait gave up as designed (the next mcb_check_device then reports
 * MCB_ERR_DEVICE_TIMEOUT once); waited_cycles_out, if not null, receives the cycles spent.  Test support. */
#define MCB_WAIT_CODE_SELFTEST 90
int mcb_selftest_wait_timeout(int64_t limit_cycles, int64_t* waited_cycles_out, void* stream);

/* Library switches.  MCB_OPT_GRAD_TAIL (default 1): mcb_lora_linear_bwd may accumulate dA and dB in the tail phase
 * of the dx launch.  That phase makes CTAs wait for rows other CTAs of the same launch write, so it needs the whole
 * grid (one CTA per SM) resident at once; the library checks the device's occupancy itself, but a caller that runs
 * other kernels beside the backward pass (a collective on a second stream), or a context limited to a share of the
 * SMs, should set it to 0: the gradients then take their own launch, which waits for nothing. */
#define MCB_OPT_GRAD_TAIL 0
/* Smallest reduction length (in features) from which a linear WITH a rank path runs on CTA pairs instead of the
 * one-CTA kernel (default 1536; linears without a rank path always take the pair kernel when large enough). */
#define MCB_OPT_PAIR_MIN_K 1
/* 1 (default): the small operand-pack and partial-sum kernels around the fused LoRA GEMM are chained to it by
 * programmatic dependent launch, so that each kernel's launch and set-up run under its predecessor's tail; 0: plain
 * stream order. */
#define MCB_OPT_PDL 2
#define MCB_OPT_COUNT_ 3
int mcb_set_option(int option_id, int value);
int mcb_get_option(int option_id, int* value_out);

/* Kernels this library has launched (or recorded into a graph being captured) since it was loaded, all devices and
 * threads together: the difference across a step is the step's launch count. */
int64_t mcb_launch_count(void);

/* Per-kernel timing for roofline reports.  While enabled, every launch of the tensor-core kernels is
 * bracketed by CUDA events on its own stream and tagged with its algorithmic work; mcb_profile_summary
 * synchronises the device, sums the finished records of one kind (0 = GEMM launches without a rank path: the frozen
 * projections; 1 = the stand-alone LoRA weight-gradient kernel; 2 = GEMM launches with a rank path: the fused LoRA
 * linear forward and backward, the backward including its dA/dB tail phase; 3 = GEMM launches whose epilogue runs the
 * SwiGLU backward, mcb_lora_linear_bwd_swiglu: bound by the gate / up traffic, not by the tensor pipe) and forgets them.
 * No counterpart in the reference. */
int mcb_profile_enable(int on);
int mcb_profile_summary(int kind, int64_t* launches, double* total_ms, double* total_flops, double* total_bytes);

/* ---- fused LoRA -------------------------------------------------------------------------- */

/* Replaces FusedLoRAOp / CustomMetalOps::lora_forward_fused (src/backend/custom_ops.rs:73-431,
 * src/backend/metal_ops.rs:126-144) and the kernel fused_lora_forward_tiled
 * (src/backend/kernels.metal:108-159):   out[M,N] = scale * (x[M,K] @ A[K,r]) @ B[r,N].
 * A and B are float32 (the reference keeps them F32, src/training/lora.rs:238,244); x/out are `dtype`. */
int mcb_lora_delta_fwd(const void* x, const float* A, const float* B, void* out,
                       int64_t M, int64_t K, int64_t N, int64_t r, float scale, int dtype,
                       void* workspace, size_t workspace_bytes, void* stream);

/* Workspace needed by the three mcb_lora_* calls for these sizes. */
size_t mcb_lora_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t r, int dtype);

/* Frozen linear + LoRA in one pass:  y = x W^T (+ bias) + scale * (x A) B.
 * Replaces the sequence candle_nn::Linear (src/models/transformer.rs:241-243) + LoRALayer::forward
 * (src/training/lora.rs:292-342) + the add at src/models/qwen.rs:114-118.
 *   W      [N,K] (w_layout MCB_W_OUT_IN; the bf16 path accepts only this), dtype
 *   bias   [N] dtype, or null
 *   A,B    float32 [K,r], [r,N]; r may be 0 with A=B=null (plain frozen linear)
 *   y      [M,N] dtype
 *   h_save [mcb_lora_rank_padded(r), mcb_lora_h_pitch(M)] dtype, or null: receives scale*(x A),
 *          transposed (rank-major, token index contiguous), for the backward. */
int mcb_lora_linear_fwd(const void* x, const void* W, const void* bias, const float* A, const float* B,
                        void* y, void* h_save, int64_t M, int64_t K, int64_t N, int64_t r, float scale,
                        int dtype, int w_layout, void* workspace, size_t workspace_bytes, void* stream);

/* Reverse pass of mcb_lora_linear_fwd with W and bias frozen (candle autograd at
 * src/training/trainer.rs:388 over src/training/lora.rs:323-339):
 *   dx = dy W + scale (dy B^T) A^T ;  dA = x^T (scale dy B^T) ;  dB = (scale x A)^T dy
 *   W      [K,N] (w_layout MCB_W_IN_OUT) for bf16; either layout for f32
 *   h_save from the forward; null makes the call recompute it
 *   dx     [M,K] dtype, or null to skip;  dA [K,r], dB [r,N] float32, or both null to skip
 *   accumulate != 0 adds into dA/dB instead of overwriting (gradient accumulation).
 * bf16: with h_save given, both gradients asked for and K, N multiples of 64 up to 1024 (and N < 1536), the token
 * reductions for dA and dB run in the same kernel launch as dx, as its tail phase; a small kernel then sums
 * the per-CTA partials in a fixed order (results do not depend on which form ran beyond float32 summation order). */
int mcb_lora_linear_bwd(const void* x, const void* W, const float* A, const float* B, const void* dy,
                        const void* h_save, void* dx, float* dA, float* dB, int accumulate,
                        int64_t M, int64_t K, int64_t N, int64_t r, float scale, int dtype, int w_layout,
                        void* workspace, size_t workspace_bytes, void* stream);

/* The two calls above with one more operand fused into the epilogue: `residual` [M,N] is added to y (the
 * residual connections around attention and MLP, src/models/qwen.rs:121,140), `dx_residual` [M,K] is added
 * to dx (summing the input gradients of projections that share an input).  Null means none.  On the bf16
 * path the operand may be the output buffer itself. */
int mcb_lora_linear_fwd_ex(const void* x, const void* W, const void* bias, const float* A, const float* B,
                           const void* residual, void* y, void* h_save, int64_t M, int64_t K, int64_t N, int64_t r,
                           float scale, int dtype, int w_layout, void* workspace, size_t workspace_bytes, void* stream);
int mcb_lora_linear_bwd_ex(const void* x, const void* W, const float* A, const float* B, const void* dy,
                           const void* h_save, const void* dx_residual, void* dx, float* dA, float* dB, int accumulate,
                           int64_t M, int64_t K, int64_t N, int64_t r, float scale, int dtype, int w_layout,
                           void* workspace, size_t workspace_bytes, void* stream);

/* mcb_lora_linear_bwd_ex for the down projection of a SwiGLU MLP (down(silu(gate) * up),
 * src/models/transformer.rs:389-395), with the SwiGLU backward in the epilogue of the input-gradient product.  The input
 * gradient d act [M,K] is never stored: gate and up [M,K] (the pre-activations the forward saved) are overwritten
 * with  d gate = d act * up * silu'(gate)  and  d up = d act * silu(gate),  d act taken from the float32 accumulator.
 * Saves one write and one read of [M,K] against mcb_lora_linear_bwd_ex followed by mcb_swiglu_bwd.  bf16, W as
 * [in,out].  Runs where mcb_lora_linear_bwd_swiglu_supported returns 1 (host-only query: the product must run on CTA
 * pairs); elsewhere MCB_ERR_UNSUPPORTED, and the caller uses the two calls. */
int mcb_lora_linear_bwd_swiglu_supported(int64_t M, int64_t K, int64_t N, int64_t r, int dtype);
int mcb_lora_linear_bwd_swiglu(const void* x, const void* W, const float* A, const float* B, const void* dy,
                               const void* h_save, void* gate, void* up, float* dA, float* dB, int accumulate,
                               int64_t M, int64_t K, int64_t N, int64_t r, float scale, int dtype, int w_layout,
                               void* workspace, size_t workspace_bytes, void* stream);

/* out[N,K] = W[N,K] + scale * (A B)^T: the adapter folded into a base weight stored [out, in]
 * (LoRAAdapter::merge_weights, src/training/adapter.rs:315-354).  A [K,r], B [r,N] float32; W, out `dtype`; out may be W. */
int mcb_lora_merge_weights(const void* W, const float* A, const float* B, void* out, int64_t K, int64_t N, int64_t r,
                           float scale, int dtype, void* stream);

/* Several projections of the SAME input as one linear (the q, k and v projections of an attention block,
 * src/models/transformer.rs:241-243, each with its own adapter): W is the projections' weights stacked [N, K] (N = sum
 * of their widths), y / dy hold their outputs / gradients side by side [M, N], and segment i names the adapter of
 * output columns [n_offset, n_offset + n).  The rank paths run as one block-diagonal update with n_segments * r rank
 * columns (at most 64), so x is read once for all projections and their input gradients are summed in one pass.
 * bf16 only.  h_save: [mcb_lora_rank_padded(n_segments * r), mcb_lora_h_pitch(M)], required by the backward.
 * The backward writes (accumulate: adds to) every segment's dA [K,r] and dB [r,n] (all null: dx only). */
typedef struct {
  const float* A;     /* [K, r]  */
  const float* B;     /* [r, n]  */
  float* dA;          /* [K, r]  (backward) */
  float* dB;          /* [r, n]  (backward) */
  int64_t n_offset;   /* first output column of this projection */
  int64_t n;          /* its width */
} mcb_lora_segment;
size_t mcb_lora_fused_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t r, int n_segments, int dtype);
int mcb_lora_linear_fused_fwd(const void* x, const void* W, const void* bias, const mcb_lora_segment* segments, int n_segments,
                              void* y, void* h_save, int64_t M, int64_t K, int64_t N, int64_t r, float scale, int dtype,
                              void* workspace, size_t workspace_bytes, void* stream);
int mcb_lora_linear_fused_bwd(const void* x, const void* Wt, const mcb_lora_segment* segments, int n_segments, const void* dy,
                              const void* h_save, const void* dx_residual, void* dx, int accumulate, int64_t M, int64_t K,
                              int64_t N, int64_t r, float scale, int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* Rank rounded up to the tensor-core K granule (16): the row count of h_save. */
int64_t mcb_lora_rank_padded(int64_t r);
/* Row pitch of h_save in elements: the token count rounded up to 64. */
int64_t mcb_lora_h_pitch(int64_t M);

/* dst[cols,rows] = src[rows,cols]^T; makes the [K,N] copy of a frozen weight for the backward. */
int mcb_transpose_2d(const void* src, void* dst, int64_t rows, int64_t cols, int dtype, void* stream);

/* The MLP's first half in one kernel: gate = x Wg^T, up = x Wu^T, act = silu(gate) * up  (MLP::forward,
 * src/models/transformer.rs:389-395: two candle_nn::Linear calls, silu, mul).  w_gate_up is [2F, K]: the gate and up
 * weights (each [F, K]) interleaved in blocks of 128 rows - gate rows 0..127, up rows 0..127, gate rows 128..255,
 * ... - so that one output tile holds both projections of the same 128 features.  gate, up, act are [M, F]; gate
 * and up are written too because the backward needs them.  bf16 only, F a multiple of 128, K of 8. */
int mcb_linear_swiglu_fwd(const void* x, const void* w_gate_up, void* gate, void* up, void* act, int64_t M, int64_t K,
                          int64_t F, int dtype, void* stream);

/* ---- lazy-graph primitives (Operation::{Matmul, Add, Mul, MulScalar}, src/graph/executor.rs:71-120) ---- */

/* out[M,N] = a[M,K] b[K,N] (Tensor::broadcast_matmul with a 2-D right operand).  The bf16 path transposes b
 * into `workspace` (mcb_matmul_workspace_bytes) and runs the tensor-core kernel. */
size_t mcb_matmul_workspace_bytes(int64_t K, int64_t N, int dtype);
int mcb_matmul(const void* a, const void* b, void* out, int64_t M, int64_t K, int64_t N, int dtype,
               void* workspace, size_t workspace_bytes, void* stream);
/* out = a * b element-wise; out = a * value. */
int mcb_mul(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream);
int mcb_mul_scalar(const void* a, void* out, int64_t n, float value, int dtype, void* stream);

/* candle_nn::ops::dropout as LoRALayer::forward applies it to x A in training mode (src/training/lora.rs:325-330):
 * out[i] = x[i] / (1 - p) where element i is kept, 0 where it is dropped; kept with probability 1 - p.  The mask comes
 * from a counter-based generator over (seed, offset + i) - element i is kept when the 24 high bits of
 * splitmix64(seed ^ (offset + i) * 0x9E3779B97F4A7C15), as a fraction of one, are >= p - so the same call on the
 * upstream gradient is the backward pass.  Not candle's generator: draw by draw the masks differ from the reference's,
 * their distribution and the inverted scaling are the same.  out may be x. */
int mcb_dropout(const void* x, void* out, int64_t n, float p, uint64_t seed, uint64_t offset, int dtype, void* stream);

/* ---- RMSNorm ------------------------------------------------------------------------------ */

/* Replaces FusedRMSNormOp / rms_norm_fused (src/backend/custom_ops.rs:443-632, kernels.metal:281-330)
 * and, with w != null, the model layer's extra broadcast_mul (src/models/qwen.rs:314-325):
 *   y = x / sqrt(mean(x^2) + eps) (* w).   x,y [rows,D] dtype; w [D] dtype or null;
 *   rstd [rows] float32 or null (saved 1/sqrt(..) for the backward). */
int mcb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int64_t rows, int64_t D,
                    float eps, int dtype, void* stream);
size_t mcb_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t D);
/* Reverse pass (candle autograd in the reference):  dx [rows,D] dtype; dw [D] float32 or null
 * (overwritten unless accumulate).  `workspace` holds the per-block partial sums of dw. */
int mcb_rmsnorm_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, int accumulate,
                    int64_t rows, int64_t D, float eps, int dtype,
                    void* workspace, size_t workspace_bytes, void* stream);

/* The same with one more operand fused into the store: dx = (gradient through the norm) + dx_residual, where
 * dx_residual [rows,D] dtype is the gradient that reaches the same tensor along the residual connection
 * (src/models/qwen.rs:121,140: the block input feeds both the norm and the skip path).  Null means none.
 * dx may be the dx_residual buffer itself when rows are whole, 16-byte aligned vectors. */
int mcb_rmsnorm_bwd_ex(const void* x, const void* w, const void* dy, const void* dx_residual, void* dx,
                       float* dw, int accumulate, int64_t rows, int64_t D, float eps, int dtype,
                       void* workspace, size_t workspace_bytes, void* stream);

/* The same reverse pass for callers that cannot allocate device memory at all -- for example a host
 * runtime that has already handed every byte of the GPU to its own memory pool, or a service thread that
 * must never hit the device-wide synchronisation an allocation implies -- and so can neither cudaMalloc a
 * workspace nor size one in advance.  It has no counterpart in the reference.  The partial sums of dw go
 * into a 2 MiB array compiled into the library (128 blocks x 4096 columns of float32), which every GPU
 * that loads the library keeps until the process exits; the call itself runs no cudaMalloc/cudaFree and
 * no allocating library routine.  Limits: D <= 4096, rows 16-byte aligned with D a multiple of 8 (bf16)
 * or 4 (f32); anything larger is refused with MCB_ERR_SHAPE / MCB_ERR_ALIGN -- use mcb_rmsnorm_bwd then.
 * The first call on each device looks up the array's device address (with that device current); make
 * that first call before starting any stream capture.  All calls on a device share the one array, which
 * keeps whatever the previous call left in it (each call overwrites the part it reads, nothing has to
 * be cleared): two calls whose kernels overlap on the GPU -- different streams, or different host threads
 * -- race on it, so serialise them.  The first call per device also writes the library's host-side cache of the
 * array's address; make that first call from one host thread. */
int mcb_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, void* dx, float* dw, int accumulate,
                            int64_t rows, int64_t D, float eps, int dtype, void* stream);

/* ---- softmax ------------------------------------------------------------------------------ */

/* Replaces FusedSoftmaxOp / softmax_fused (src/backend/custom_ops.rs:644-824, kernels.metal:187-261)
 * and TensorExt::softmax_stable (src/backend/tensor.rs:91-98): softmax over the last dim of [rows,D].
 * -inf entries (an additive causal mask, src/models/transformer.rs:269-273) give 0; a row that is
 * all -inf gives zeros.  In-place (y == x) is allowed. */
int mcb_softmax_fwd(const void* x, void* y, int64_t rows, int64_t D, int dtype, void* stream);
/* dx = y * (dy - sum_j dy_j y_j).  In-place on dy is allowed. */
int mcb_softmax_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t D, int dtype,
                    void* stream);

/* Scaled scores with a causal mask, then softmax: row i belongs to query position i % seq and keeps
 * columns c <= i % seq; y = softmax(scale * x) over the kept columns, 0 elsewhere.  Replaces the
 * sequence divide-by-sqrt(d), broadcast_add(mask), softmax_stable in Attention::forward
 * (src/models/transformer.rs:264-275); the reference builds no mask itself (its callers pass one). */
int mcb_softmax_causal_fwd(const void* x, void* y, int64_t rows, int64_t D, int64_t seq, float scale, int dtype,
                           void* stream);
/* Reverse of the call above: dx = scale * y * (dy - sum_j dy_j y_j), with the masked columns (where y
 * is 0) neither read nor computed: they get 0.  seq = 0 means "no mask, scale only". */
int mcb_softmax_causal_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t D, int64_t seq,
                           float scale, int dtype, void* stream);

/* ---- fused causal attention ----------------------------------------------------------------- */

/* O = softmax(scale * Q K^T + causal mask) V for grouped-query attention without materialising the scores:
 * Attention::forward computes matmul(q, k^T) / sqrt(d), adds the mask, applies softmax and multiplies by v as
 * separate ops over a [B, H, S, S] tensor (src/models/transformer.rs:257-285).  nb = batch * kv_heads;
 * q, o [nb, groups*seq, head_dim] (row g*seq + s = query head g of the group, position s); k, v [nb, seq,
 * head_dim]; lse [nb, groups*seq] float32 (log-sum-exp of each row's scaled scores, which the backward needs;
 * may be null for inference).  Built for bf16, head_dim 64, seq a multiple of 128; other shapes return
 * MCB_ERR_UNSUPPORTED (callers then use the unfused sequence above).  The workspace (1024-byte aligned,
 * mcb_attention_workspace_bytes) holds two float32 values per query row during the backward; the forward
 * ignores it. */
size_t mcb_attention_workspace_bytes(int64_t nb, int64_t groups, int64_t seq, int64_t head_dim);
int mcb_attention_causal_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int64_t nb,
                             int64_t groups, int64_t seq, int64_t head_dim, float scale, int dtype,
                             void* workspace, size_t workspace_bytes, void* stream);
/* Gradients of the call above (candle's autograd in the reference, src/training/trainer.rs:388): given o, lse
 * from the forward and dout = dL/do, writes dq [like q], dk and dv [like k] (summed over the query heads of a
 * group).  The probabilities are recomputed from q, k and lse; nothing of size seq x seq is stored. */
int mcb_attention_causal_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                             const float* lse, void* dq, void* dk, void* dv, int64_t nb, int64_t groups,
                             int64_t seq, int64_t head_dim, float scale, int dtype, void* workspace,
                             size_t workspace_bytes, void* stream);

/* The same two calls with O (forward output) and dO (backward input) optionally token-major,
 * [batch*seq, kv_heads*groups*head_dim] with head kvh*groups + g at column offset (kvh*groups + g)*head_dim: the layout
 * of the o_proj input (src/models/transformer.rs:283-285 transposes and reshapes the per-head output into it), so
 * that no relayout pass stands between the attention kernels and the projection.  nb = batch*kv_heads with the kv
 * head varying fastest.  o_token_major == 0 gives the calls above. */
int mcb_attention_causal_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse, int64_t nb,
                                int64_t groups, int64_t seq, int64_t head_dim, float scale, int dtype,
                                int64_t kv_heads, int o_token_major, void* workspace, size_t workspace_bytes,
                                void* stream);
int mcb_attention_causal_bwd_ex(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                const float* lse, void* dq, void* dk, void* dv, int64_t nb, int64_t groups,
                                int64_t seq, int64_t head_dim, float scale, int dtype, int64_t kv_heads,
                                int o_token_major, void* workspace, size_t workspace_bytes, void* stream);

/* ---- data-parallel exchange ------------------------------------------------------------------- */

/* The reference trains on one device and has no communication layer; these calls are the one exchange step of the
 * batch-data-parallel training step: a float32 sum all-reduce of the LoRA gradient buckets (NCCL over NVLink), one
 * communicator rank per GPU and process.  NCCL is bound at run time: the copy the process already carries
 * (PyTorch's), else libnccl.so.2 from the loader path, else the file MCB_NCCL_LIBRARY names.
 * Failure handling: communicators are non-blocking; the rendezvous, every enqueue and mcb_comm_wait poll
 * ncclCommGetAsyncError against a host deadline (timeout_ms; 0 = none).  On a deadline or an asynchronous NCCL
 * error the communicator is aborted (ncclCommAbort) and marked dead; the call returns MCB_ERR_COMM_TIMEOUT or
 * MCB_ERR_COMM_BASE + the NCCL result, and later calls return MCB_ERR_COMM_DEAD instead of hanging. */
#define MCB_COMM_ID_BYTES 128
typedef struct mcb_comm mcb_comm;
/* Rank 0 creates the id and hands its 128 bytes to every rank by any host channel. */
int mcb_comm_unique_id(void* id_out);
/* Joins the communicator as `rank` of `nranks` on the CURRENT device.  flags: 0, or MCB_COMM_BLOCKING for a
 * blocking communicator (NCCL then works inside the calling thread and the rendezvous has no deadline; the
 * deadline of mcb_comm_wait and the asynchronous-error checks stay). */
#define MCB_COMM_BLOCKING 1
int mcb_comm_init_rank(mcb_comm** comm_out, int nranks, int rank, const void* id, int timeout_ms, int flags);
/* In-place sum over ranks of buf[0..count) float32, enqueued on `stream` (may be captured into a CUDA graph). */
int mcb_comm_allreduce_bucket(mcb_comm* comm, float* buf, int64_t count, void* stream);
/* Waits, on the host and at most timeout_ms, until the communicator's enqueued work and `stream` have finished
 * (MCB_COMM_NO_STREAM: the communicator's own state only).  A peer that never joined a collective shows up here. */
#define MCB_COMM_NO_STREAM ((void*)(intptr_t)-1)
int mcb_comm_wait(mcb_comm* comm, void* stream, int timeout_ms);
int mcb_comm_abort(mcb_comm* comm);
int mcb_comm_info(const mcb_comm* comm, int* nranks, int* rank, int* dead, int* nccl_version);
/* Finalizes (within the communicator's deadline) and frees; also frees a dead communicator.  CUDA graphs that
 * recorded this communicator's collectives must be destroyed first: NCCL waits for them. */
int mcb_comm_destroy(mcb_comm* comm);

/* ---- AdamW -------------------------------------------------------------------------------- */

typedef struct {
  float* p;        /* parameter, updated in place   */
  const float* g;  /* gradient                      */
  float* m;        /* first moment, updated         */
  float* v;        /* second moment, updated        */
  int64_t n;       /* element count                 */
  int32_t t;       /* bias-correction step for THIS tensor (the reference's shared counter advances
                      once per tensor, src/training/optimizer.rs:236-238) */
  int32_t pad_;
} mcb_adamw_tensor;

/* Replaces AdamW::step / step_var (src/training/optimizer.rs:227-316) for a list of float32 tensors
 * in a few launches:  m=b1 m+(1-b1)g; v=b2 v+(1-b2)g^2; p -= lr*(m/(1-b1^t))/(sqrt(v/(1-b2^t))+eps)
 * + (wd*lr)*p.  `tensors` is a HOST array.  g is multiplied by grad_scale first (1/world size in the
 * data-parallel step; 1 otherwise). */
int mcb_adamw_multi(const mcb_adamw_tensor* tensors, int n_tensors, float lr, float beta1, float beta2,
                    float eps, float weight_decay, float grad_scale, void* stream);

/* ---- element-wise frame of the Qwen-shaped training step ------------------------------------- */

/* out[m,:] = table[ids[m],:]  (candle_nn::embedding, src/models/qwen.rs:189).  ids are int32. */
int mcb_embedding_fwd(const int32_t* ids, const void* table, void* out, int64_t M, int64_t H, int64_t vocab,
                      int dtype, void* stream);
/* Rotary embedding (half-split, angle = position * theta^(-2i/d); src/models/transformer.rs:47-120)
 * fused with the [B,S,H,d] -> [B,H,S,d] transpose of Attention::forward (transformer.rs:255-257).
 * rotate = 0 only re-lays out (V).  inverse = 1 is the reverse pass: [B,H,S,d] -> [B,S,H,d] with the
 * transposed rotation. */
int mcb_rope_relayout(const void* src, void* dst, int64_t B, int64_t S, int64_t H, int64_t d, float theta,
                      int rotate, int inverse, int dtype, void* stream);
/* The same where the [B,S,H,d] side is a column block of wider token rows: rows `token_pitch` elements apart (0 =
 * H*d), the heads starting at column `col_offset` - the q, k or v part of a fused q/k/v projection's output (forward:
 * the source) or of the fused gradient buffer (inverse: the destination). */
int mcb_rope_relayout_ex(const void* src, void* dst, int64_t B, int64_t S, int64_t H, int64_t d, float theta, int rotate,
                         int inverse, int64_t token_pitch, int64_t col_offset, int dtype, void* stream);
/* The three mcb_rope_relayout_ex calls that split a fused q/k/v projection's output (inverse = 0) or assemble the fused
 * gradient buffer (inverse = 1), as one launch: the sines and cosines of a position are computed once for the query
 * and the key heads, and the value heads are only re-laid out (Attention::forward, src/models/transformer.rs:241-257).
 * fused: token rows `token_pitch` elements apart (0 = (Hq + 2 Hk) * d) holding Hq query heads, then Hk key heads, then
 * Hk value heads; q [B,Hq,S,d], k and v [B,Hk,S,d].  Results equal those of the three calls bit for bit. */
int mcb_rope_relayout_qkv(void* fused, void* q, void* k, void* v, int64_t B, int64_t S, int64_t Hq, int64_t Hk, int64_t d,
                          float theta, int inverse, int64_t token_pitch, int dtype, void* stream);
/* out = silu(gate) * up and its reverse (MLP::forward, src/models/transformer.rs:389-395). */
int mcb_swiglu_fwd(const void* gate, const void* up, void* out, int64_t n, int dtype, void* stream);
int mcb_swiglu_bwd(const void* gate, const void* up, const void* dout, void* dgate, void* dup, int64_t n,
                   int dtype, void* stream);
/* out = a + b (the residual connections, src/models/qwen.rs:121,140). */
int mcb_add(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream);
/* Cross-entropy over logits [M,V] with targets int32 [M]; a target outside [0,V) (u32::MAX, the
 * reference's ignore index, src/training/trainer.rs:385) is ignored.  Replaces cross_entropy_loss
 * (src/training/loss.rs:58-147) and its autograd reverse: loss[0] = mean nll over kept rows,
 * loss[1] = sum, count[0] = kept rows, nll [M] scratch; with write_grad the logits are overwritten by
 * d loss / d logits. */
int mcb_cross_entropy(void* logits, const int32_t* targets, float* nll, int32_t* count, float* loss,
                      int64_t M, int64_t V, int write_grad, int dtype, void* stream);
/* The same loss a chunk of tokens at a time, for a caller that produces the logits chunk by chunk (lm_head on a
 * slice of the tokens), turns each chunk into its gradient in place and feeds that straight to the lm_head backward,
 * so that the [tokens, vocabulary] matrix of the whole batch never exists (the reference materialises it, and walks
 * it with a host loop: src/training/loss.rs:109-186).  _count: count[0] = targets inside [0, V) over ALL M tokens
 * (the mean's denominator, needed by every chunk's gradient).  _chunk: rows of one chunk -> nll[rows] and, with
 * write_grad, d loss / d logits in place.  _finish: loss[0] = sum(nll) / count, loss[1] = sum(nll) over all M. */
int mcb_cross_entropy_count(const int32_t* targets, int32_t* count, int64_t M, int64_t V, void* stream);
int mcb_cross_entropy_chunk(void* logits, const int32_t* targets, float* nll, const int32_t* count, int64_t rows,
                            int64_t V, int write_grad, int dtype, void* stream);
int mcb_cross_entropy_finish(const float* nll, const int32_t* count, float* loss, int64_t M, void* stream);

/* ---- the training step as one engine ------------------------------------------------------------ */

/* TrainingStep::execute (src/training/trainer.rs:368-414) over Qwen::forward (src/models/qwen.rs:95-143,236-251) for
 * a host that is not Python: forward, next-token cross-entropy (ignore index = any target outside [0, vocab)),
 * the written-out backward pass for the LoRA parameters, the optional bucketed gradient all-reduce, and AdamW - all
 * enqueued on the caller's stream, nothing allocated inside a step, recordable into a CUDA graph.  Adapters sit on
 * the projections they name and see those projections' true inputs (the reference wires only o_proj / down_proj,
 * src/models/qwen.rs:106-138).  Production configuration only: bfloat16, head_dim 64, sequence a multiple of 128;
 * anything else returns MCB_ERR_UNSUPPORTED.
 * Modules are numbered q 0, k 1, v 2, o 3, gate 4, up 5, down 6 (TargetModule, src/training/adapter.rs:15-62).
 * All weights are bf16 device tensors in candle's [out, in] layout; the engine keeps the pointers (the caller keeps
 * the memory) and derives what its kernels want ([in, out] copies, the stacked q/k/v weight, the interleaved
 * gate/up weight) into the head of `arena`, next to the AdamW moments.  The rest of the arena is re-cut for every
 * step; mcb_qwen_arena_bytes says how much a (batch, seq) needs. */
typedef struct {
  int64_t vocab_size, hidden_size, intermediate_size, num_layers, num_heads, num_kv_heads;
  float rms_norm_eps, rope_theta;
} mcb_qwen_config;
typedef struct {
  const void* input_layernorm;           /* [hidden] */
  const void* post_attention_layernorm;  /* [hidden] */
  const void* weight[7];                 /* by module: [out, in] */
  const void* bias[3];                   /* q, k, v: [out] or null */
} mcb_qwen_layer;
typedef struct {
  const void* embed_tokens;              /* [vocab, hidden] */
  const void* final_norm;                /* [hidden] */
  const void* lm_head;                   /* [vocab, hidden] */
  const mcb_qwen_layer* layers;          /* HOST array, num_layers entries */
} mcb_qwen_weights;
typedef struct {
  int32_t layer, module;
  const float* A;   /* [in, r]  float32, trained in place */
  const float* B;   /* [r, out] */
  float* dA;        /* gradients, written by every forward_backward (added to with accumulate) */
  float* dB;
} mcb_qwen_adapter_entry;
typedef struct mcb_qwen mcb_qwen;

size_t mcb_qwen_arena_bytes(const mcb_qwen_config* cfg, const mcb_qwen_adapter_entry* adapters, int n_adapters, int rank,
                            int64_t batch, int64_t seq);
/* `adapters` (a HOST array) fixes the order in which AdamW visits the tensors: entry order, A before B.  `arena` is
 * 1024-byte aligned device memory.  The derived weights are written on `stream`. */
int mcb_qwen_create(mcb_qwen** out, const mcb_qwen_config* cfg, const mcb_qwen_weights* weights,
                    const mcb_qwen_adapter_entry* adapters, int n_adapters, int rank, float scale, void* arena,
                    size_t arena_bytes, void* stream);
/* Data-parallel exchange: with a communicator, forward_backward all-reduces bucket i (elements [lo, hi) of grad_flat,
 * which must be the buffer the adapters' dA / dB live in) on `side_stream` as soon as layer bucket_first_layer[i] has
 * finished its backward, and joins the side stream before it returns.  comm = null switches it off. */
int mcb_qwen_set_exchange(mcb_qwen* q, mcb_comm* comm, void* side_stream, float* grad_flat, const int64_t* bucket_lo,
                          const int64_t* bucket_hi, const int* bucket_first_layer, int n_buckets);
/* Tokens per chunk of the lm_head + cross-entropy stage (see mcb_cross_entropy_chunk); 0 (the default) lets
 * mcb_ce_chunk_tokens choose.  The results do not depend on it. */
int mcb_qwen_set_ce_chunk(mcb_qwen* q, int64_t tokens);
/* The chunk size (4096 .. 12288 tokens) for which the lm_head backward GEMM of `tokens` rows and `hidden` columns fills
 * whole waves of CTA pairs best; host-only (assumes 148 SMs before mcb_init). */
int64_t mcb_ce_chunk_tokens(int64_t tokens, int64_t hidden);
/* ids, targets: int32 [batch, seq] on the device.  loss_out: device float[2] = {mean, sum} of the token losses. */
int mcb_qwen_forward_backward(mcb_qwen* q, const int32_t* ids, const int32_t* targets, int64_t batch, int64_t seq,
                              int accumulate, float* loss_out, void* stream);
/* AdamW::step_var over all adapter tensors (src/training/trainer.rs:398-402) with the reference's shared counter. */
int mcb_qwen_adamw_step(mcb_qwen* q, float lr, float beta1, float beta2, float eps, float weight_decay, float grad_scale,
                        void* stream);
/* forward_backward + adamw_step. */
int mcb_qwen_train_step(mcb_qwen* q, const int32_t* ids, const int32_t* targets, int64_t batch, int64_t seq, float lr,
                        float beta1, float beta2, float eps, float weight_decay, float grad_scale, float* loss_out, void* stream);
int mcb_qwen_info(const mcb_qwen* q, int64_t* adamw_steps, int64_t* persistent_bytes, int32_t** kept_targets_dev);
int mcb_qwen_destroy(mcb_qwen* q);

#ifdef __cplusplus
}
#endif
#endif /* MCB200_H_ */
