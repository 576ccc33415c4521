// Fused multi-tensor AdamW for the float32 LoRA parameters.
//
// One launch updates up to kMaxTensors tensors (their descriptors travel in the kernel parameters,
// so no device-side table has to be kept in step with the host); grid.y selects the tensor, grid.x
// strides over its elements four at a time.  HBM-bound: 28 bytes per element (read p,g,m,v; write
// p,m,v).  The arithmetic keeps the reference's operation order and roundings -- each candle op in
// src/training/optimizer.rs:243-272 is one float32 rounding, so products and sums are NOT contracted
// into FMAs, and "tensor / scalar" is a multiplication by the float32 reciprocal of the scalar, as
// candle's scalar division is an affine by 1/rhs.
#include "common.cuh"

namespace mcb {
namespace {

constexpr int kMaxTensors = 64;

struct AdamWTensorDev {
  float* p;
  const float* g;
  float* m;
  float* v;
  int64_t n;
  float inv_bc1;  // 1 / (1 - beta1^t)
  float inv_bc2;  // 1 / (1 - beta2^t)
};
struct AdamWBatch {
  AdamWTensorDev t[kMaxTensors];
};

struct AdamWScalars {
  float b1, b2, one_m_b1, one_m_b2, eps, lr, wd_lr, grad_scale;
};

__device__ __forceinline__ void adamw_one(float& p, float g, float& m, float& v, const AdamWScalars& s,
                                          float inv_bc1, float inv_bc2) {
  g = __fmul_rn(g, s.grad_scale);
  const float m_new = __fadd_rn(__fmul_rn(m, s.b1), __fmul_rn(g, s.one_m_b1));
  const float v_new = __fadd_rn(__fmul_rn(v, s.b2), __fmul_rn(__fmul_rn(g, g), s.one_m_b2));
  const float m_hat = __fmul_rn(m_new, inv_bc1);
  const float v_hat = __fmul_rn(v_new, inv_bc2);
  const float denom = __fadd_rn(__fsqrt_rn(v_hat), s.eps);
  const float update = __fdiv_rn(m_hat, denom);
  const float lr_update = __fmul_rn(update, s.lr);
  const float wd_update = __fmul_rn(p, s.wd_lr);
  p = __fsub_rn(__fsub_rn(p, lr_update), wd_update);
  m = m_new;
  v = v_new;
}

__global__ void __launch_bounds__(256) adamw_multi_kernel(const __grid_constant__ AdamWBatch batch,
                                                          const AdamWScalars s) {
  const AdamWTensorDev& t = batch.t[blockIdx.y];
  const int64_t n = t.n;
  const bool vec = ((reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.g) |
                     reinterpret_cast<uintptr_t>(t.m) | reinterpret_cast<uintptr_t>(t.v)) & 15u) == 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    for (int64_t i = tid; i < n4; i += stride) {
      float4 p = reinterpret_cast<float4*>(t.p)[i];
      const float4 g = reinterpret_cast<const float4*>(t.g)[i];
      float4 m = reinterpret_cast<float4*>(t.m)[i];
      float4 v = reinterpret_cast<float4*>(t.v)[i];
      adamw_one(p.x, g.x, m.x, v.x, s, t.inv_bc1, t.inv_bc2);
      adamw_one(p.y, g.y, m.y, v.y, s, t.inv_bc1, t.inv_bc2);
      adamw_one(p.z, g.z, m.z, v.z, s, t.inv_bc1, t.inv_bc2);
      adamw_one(p.w, g.w, m.w, v.w, s, t.inv_bc1, t.inv_bc2);
      reinterpret_cast<float4*>(t.p)[i] = p;
      reinterpret_cast<float4*>(t.m)[i] = m;
      reinterpret_cast<float4*>(t.v)[i] = v;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) {
      float p = t.p[i], m = t.m[i], v = t.v[i];
      adamw_one(p, t.g[i], m, v, s, t.inv_bc1, t.inv_bc2);
      t.p[i] = p; t.m[i] = m; t.v[i] = v;
    }
  } else {
    for (int64_t i = tid; i < n; i += stride) {
      float p = t.p[i], m = t.m[i], v = t.v[i];
      adamw_one(p, t.g[i], m, v, s, t.inv_bc1, t.inv_bc2);
      t.p[i] = p; t.m[i] = m; t.v[i] = v;
    }
  }
}

// f32::powi by repeated squaring in float32 (src/training/optimizer.rs:252-255).
float powi_f32(float base, int n) {
  float result = 1.0f, b = base;
  while (n > 0) {
    if (n & 1) result = result * b;
    b = b * b;
    n >>= 1;
  }
  return result;
}

}  // namespace
}  // namespace mcb

using namespace mcb;

extern "C" int mcb_adamw_multi(const mcb_adamw_tensor* tensors, int n_tensors, float lr, float beta1, float beta2,
                               float eps, float weight_decay, float grad_scale, void* stream) {
  MCB_NVTX_RANGE("mcb_adamw_multi");
  if (n_tensors < 0) return fail(MCB_ERR_SHAPE, "adamw_multi: n_tensors=%d", n_tensors);
  if (n_tensors == 0) return MCB_OK;
  if (!tensors) return fail(MCB_ERR_NULL, "adamw_multi: tensors is null");
  // The same ranges AdamWConfig::validate enforces (src/training/optimizer.rs:69-107).
  // AdamWConfig::validate wants lr > 0 at construction, but set_lr does not re-validate and a warm-up
  // schedule starts at exactly 0 (src/training/scheduler.rs:152-160), so 0 is accepted here.
  if (!(lr >= 0.0f)) return fail(MCB_ERR_SHAPE, "learning rate must be non-negative");
  if (!(beta1 >= 0.0f && beta1 < 1.0f)) return fail(MCB_ERR_SHAPE, "beta1 must be in [0, 1), got %g", beta1);
  if (!(beta2 >= 0.0f && beta2 < 1.0f)) return fail(MCB_ERR_SHAPE, "beta2 must be in [0, 1), got %g", beta2);
  if (!(eps > 0.0f)) return fail(MCB_ERR_SHAPE, "epsilon must be positive");
  if (!(weight_decay >= 0.0f)) return fail(MCB_ERR_SHAPE, "weight decay must be non-negative");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  for (int i = 0; i < n_tensors; ++i) {
    const mcb_adamw_tensor& t = tensors[i];
    if (!t.p || !t.g || !t.m || !t.v) return fail(MCB_ERR_NULL, "adamw_multi: tensor %d has a null pointer", i);
    if (t.n <= 0) return fail(MCB_ERR_SHAPE, "adamw_multi: tensor %d has n=%lld", i, (long long)t.n);
    if (t.t <= 0) return fail(MCB_ERR_SHAPE, "adamw_multi: tensor %d has step t=%d (must be >= 1)", i, t.t);
  }
  AdamWScalars s;
  s.b1 = beta1; s.b2 = beta2;
  s.one_m_b1 = 1.0f - beta1; s.one_m_b2 = 1.0f - beta2;
  s.eps = eps; s.lr = lr; s.wd_lr = weight_decay * lr; s.grad_scale = grad_scale;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int base = 0; base < n_tensors; base += kMaxTensors) {
    const int cnt = n_tensors - base < kMaxTensors ? n_tensors - base : kMaxTensors;
    AdamWBatch batch;
    memset(&batch, 0, sizeof(batch));
    int64_t max_n = 0;
    for (int i = 0; i < cnt; ++i) {
      const mcb_adamw_tensor& t = tensors[base + i];
      AdamWTensorDev& d = batch.t[i];
      d.p = t.p; d.g = t.g; d.m = t.m; d.v = t.v; d.n = t.n;
      const float bc1 = 1.0f - powi_f32(beta1, t.t);
      const float bc2 = 1.0f - powi_f32(beta2, t.t);
      d.inv_bc1 = static_cast<float>(1.0 / static_cast<double>(bc1));
      d.inv_bc2 = static_cast<float>(1.0 / static_cast<double>(bc2));
      if (t.n > max_n) max_n = t.n;
    }
    int64_t gx = (max_n / 4 + 255) / 256;
    if (gx < 1) gx = 1;
    const int64_t cap = static_cast<int64_t>(ds->sm_count) * 8;
    if (gx * cnt > cap) gx = (cap + cnt - 1) / cnt;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(cnt));
    adamw_multi_kernel<<<grid, 256, 0, st>>>(batch, s);
    MCB_CHECK_LAUNCH("adamw_multi");
  }
  return MCB_OK;
}
