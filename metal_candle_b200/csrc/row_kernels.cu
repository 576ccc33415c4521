// RMSNorm and row-softmax, forward and backward, for [rows, D] matrices in float32 or bfloat16.
//
// Design (HBM-bound kernels): a row is owned by a group of TPR threads that keep it in registers
// as float (VPT 16-byte vectors per thread), so every element is read from HBM once and written
// once.  Groups are packed into 256-thread blocks and walk the rows grid-stride, which keeps a
// thread on the same columns for its whole life: the RMSNorm weight is loaded once per thread and
// the dw partial sums of the backward live in registers until the block is done.  Reductions are
// warp shuffles, plus one shared-memory hop when a group spans several warps.
//
// Algorithmic traffic per row of D elements of e bytes: rmsnorm fwd 2De, bwd 3De; softmax fwd 2De,
// bwd 3De (plus the [D] weight / dw vectors once per block).
//
// Rows wider than 4096 vectors, or rows that are not 16-byte aligned, take the scalar "wide"
// kernels at the end of the file (one block per row, data re-read from L2).
#include "common.cuh"

namespace mcb {
namespace rowpipe {
enum Op { kRmsFwd = 0, kRmsBwd = 1, kSmFwd = 2, kSmBwd = 3 };
template <typename T>
int try_launch(int op, const void* in0, const void* in1, const void* w, void* out, float* rstd, float* dw_part,
               int* dw_blocks, int64_t rows, int64_t D, float eps, int causal_seq, float scale, const DeviceState* ds,
               cudaStream_t st, const void* res = nullptr);
}  // namespace rowpipe
namespace {

constexpr float kLog2e = 1.4426950408889634f;

// ---- group reductions ---------------------------------------------------------------------
// A group of TPR threads owns a row.  Up to a warp: shuffles only.  Wider groups add one shared-memory
// hop synchronised with a named barrier of their own (bar.sync id, TPR), so groups in a block do not
// wait for each other; the two halves of `red_smem` alternate between consecutive reductions, which is
// what makes a single barrier per reduction enough.
template <int TPR, int NV, bool IS_MAX>
__device__ __forceinline__ void group_reduce(float (&v)[NV], float* red_smem, int& parity) {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float other = __shfl_xor_sync(0xffffffffu, v[i], o);
      v[i] = IS_MAX ? fmaxf(v[i], other) : v[i] + other;
    }
  }
  if constexpr (TPR > 32) {
    constexpr int WPG = TPR / 32;  // warps per group
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = warp / WPG, group_first_warp = group * WPG;
    float* buf = red_smem + parity * (32 * NV);
    parity ^= 1;
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i) buf[warp * NV + i] = v[i];
    }
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(TPR) : "memory");
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float acc = buf[group_first_warp * NV + i];
#pragma unroll
      for (int w = 1; w < WPG; ++w) {
        float other = buf[(group_first_warp + w) * NV + i];
        acc = IS_MAX ? fmaxf(acc, other) : acc + other;
      }
      v[i] = acc;
    }
  }
}

template <int TPR>
struct RowGeom {
  static constexpr int THREADS = TPR < 256 ? 256 : TPR;
  static constexpr int RPB = THREADS / TPR;  // rows per block per iteration
};

template <typename V>
__device__ __forceinline__ V load_stream(const void* base, int64_t vec_index) {
  V t;
  t.raw = __ldcs(reinterpret_cast<const decltype(t.raw)*>(base) + vec_index);
  return t;
}
template <typename V>
__device__ __forceinline__ void store_stream(void* base, int64_t vec_index, const V& t) {
  __stcs(reinterpret_cast<decltype(t.raw)*>(base) + vec_index, t.raw);
}

// ---- RMSNorm forward ------------------------------------------------------------------------
template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__(RowGeom<TPR>::THREADS)
rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                   float* __restrict__ rstd, int64_t rows, int D, float eps) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  constexpr int RPB = RowGeom<TPR>::RPB;
  __shared__ float red[64];
  int parity = 0;
  const int tg = threadIdx.x % TPR, g = threadIdx.x / TPR;
  const int nvec = D / N;
  float wv[VPT][N];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = tg + i * TPR;
    if (w != nullptr && vi < nvec) {
      V t; t.raw = reinterpret_cast<const decltype(t.raw)*>(w)[vi];
      t.to_float(wv[i]);
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j) wv[i][j] = 1.0f;
    }
  }
  const float inv_d = 1.0f / static_cast<float>(D);
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * RPB; row0 < rows;
       row0 += static_cast<int64_t>(gridDim.x) * RPB) {
    const int64_t row = row0 + g;
    const bool live = row < rows;
    float xv[VPT][N];
    float ss[1] = {0.0f};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tg + i * TPR;
      if (live && vi < nvec) {
        load_stream<V>(x + row * D, vi).to_float(xv[i]);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) xv[i][j] = 0.0f;
      }
#pragma unroll
      for (int j = 0; j < N; ++j) ss[0] = fmaf(xv[i][j], xv[i][j], ss[0]);
    }
    group_reduce<TPR, 1, false>(ss, red, parity);
    const float rinv = 1.0f / sqrtf(ss[0] * inv_d + eps);
    if (live) {
      if (rstd != nullptr && tg == 0) rstd[row] = rinv;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = tg + i * TPR;
        if (vi < nvec) {
          float o[N];
#pragma unroll
          for (int j = 0; j < N; ++j) o[j] = xv[i][j] * rinv * wv[i][j];
          V t; t.from_float(o);
          store_stream<V>(y + row * D, vi, t);
        }
      }
    }
  }
}

// ---- RMSNorm backward -----------------------------------------------------------------------
// dx = rinv * (g - xh * mean(g*xh)), g = dy*w, xh = x*rinv;  dw_partial[block][c] = sum dy*xh (NEED_DW).
template <typename T, int TPR, int VPT, bool NEED_DW>
__global__ void __launch_bounds__(RowGeom<TPR>::THREADS)
rmsnorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ dy,
                   T* __restrict__ dx, float* __restrict__ dw_partial, int64_t rows, int D, float eps) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  constexpr int RPB = RowGeom<TPR>::RPB;
  __shared__ float red[128];
  extern __shared__ float dw_smem[];  // [RPB][D] when RPB > 1 and dw is wanted
  int parity = 0;
  const int tg = threadIdx.x % TPR, g = threadIdx.x / TPR;
  const int nvec = D / N;
  float wv[VPT][N], dwa[NEED_DW ? VPT : 1][N];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = tg + i * TPR;
    if (w != nullptr && vi < nvec) {
      V t; t.raw = reinterpret_cast<const decltype(t.raw)*>(w)[vi];
      t.to_float(wv[i]);
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j) wv[i][j] = 1.0f;
    }
    if constexpr (NEED_DW) {
#pragma unroll
      for (int j = 0; j < N; ++j) dwa[i][j] = 0.0f;
    }
  }
  const float inv_d = 1.0f / static_cast<float>(D);
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * RPB; row0 < rows;
       row0 += static_cast<int64_t>(gridDim.x) * RPB) {
    const int64_t row = row0 + g;
    const bool live = row < rows;
    float xv[VPT][N], gv[VPT][N];
    float acc[2] = {0.0f, 0.0f};  // sum x^2, sum (dy*w)*x
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tg + i * TPR;
      if (live && vi < nvec) {
        load_stream<V>(x + row * D, vi).to_float(xv[i]);
        load_stream<V>(dy + row * D, vi).to_float(gv[i]);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) { xv[i][j] = 0.0f; gv[i][j] = 0.0f; }
      }
#pragma unroll
      for (int j = 0; j < N; ++j) {
        acc[0] = fmaf(xv[i][j], xv[i][j], acc[0]);
        acc[1] = fmaf(gv[i][j] * wv[i][j], xv[i][j], acc[1]);
      }
    }
    group_reduce<TPR, 2, false>(acc, red, parity);
    const float rinv = 1.0f / sqrtf(acc[0] * inv_d + eps);
    const float c = acc[1] * rinv * inv_d;  // mean(g * xh)
    if (live) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = tg + i * TPR;
        if (vi < nvec) {
          float o[N];
#pragma unroll
          for (int j = 0; j < N; ++j) {
            const float xh = xv[i][j] * rinv;
            if constexpr (NEED_DW) dwa[i][j] = fmaf(gv[i][j], xh, dwa[i][j]);
            o[j] = rinv * (gv[i][j] * wv[i][j] - xh * c);
          }
          V t; t.from_float(o);
          store_stream<V>(dx + row * D, vi, t);
        }
      }
    }
  }
  if constexpr (NEED_DW) {
    float* out = dw_partial + static_cast<int64_t>(blockIdx.x) * D;
    if constexpr (RPB == 1) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = tg + i * TPR;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < N; ++j) out[vi * N + j] = dwa[i][j];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = tg + i * TPR;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < N; ++j) dw_smem[g * D + vi * N + j] = dwa[i][j];
        }
      }
      __syncthreads();
      for (int cc = threadIdx.x; cc < D; cc += blockDim.x) {
        float s = 0.0f;
#pragma unroll
        for (int gg = 0; gg < RPB; ++gg) s += dw_smem[gg * D + cc];  // fixed order: deterministic
        out[cc] = s;
      }
    }
  }
}

// dw[c] (+)= sum over blocks of dw_partial[b][c] (deterministic: fixed order).  A CTA owns 32 columns; its 8
// warps each sum every 8th partial row (independent loads, unrolled), then warp 0 adds the 8 sums in warp order.
__global__ void __launch_bounds__(256)
colsum_partials_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nblocks, int D, int accumulate) {
  __shared__ float red[8][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.0f;
  if (c < D) {
#pragma unroll 8
    for (int b = warp; b < nblocks; b += 8) s += partial[static_cast<int64_t>(b) * D + c];
  }
  red[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < D) {
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][lane];
    dw[c] = accumulate ? dw[c] + t : t;
  }
}

// ---- softmax forward --------------------------------------------------------------------------
// causal_seq > 0: row i is query position i % causal_seq; columns beyond it are masked and are not even
// read (their output is 0), and the kept scores are multiplied by `scale` first.
template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__(RowGeom<TPR>::THREADS)
softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int D, int causal_seq, float scale) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  constexpr int RPB = RowGeom<TPR>::RPB;
  __shared__ float red[64];
  int parity = 0;
  const int tg = threadIdx.x % TPR, g = threadIdx.x / TPR;
  const int nvec = D / N;
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * RPB; row0 < rows;
       row0 += static_cast<int64_t>(gridDim.x) * RPB) {
    const int64_t row = row0 + g;
    const bool live = row < rows;
    const int q = causal_seq > 0 ? static_cast<int>(row % causal_seq) : D;  // last kept column
    float xv[VPT][N];
    float mx[1] = {-INFINITY};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tg + i * TPR;
      if (live && vi < nvec && vi * N <= q) {
        load_stream<V>(x + row * D, vi).to_float(xv[i]);
        if (causal_seq > 0) {
#pragma unroll
          for (int j = 0; j < N; ++j) xv[i][j] = (vi * N + j <= q) ? xv[i][j] * scale : -INFINITY;
        } else if (scale != 1.0f) {
#pragma unroll
          for (int j = 0; j < N; ++j) xv[i][j] *= scale;
        }
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) xv[i][j] = -INFINITY;
      }
#pragma unroll
      for (int j = 0; j < N; ++j) mx[0] = fmaxf(mx[0], xv[i][j]);
    }
    group_reduce<TPR, 1, true>(mx, red, parity);
    // A fully masked row has max = -inf; use 0 so that exp2(-inf) = 0 instead of NaN.
    const float m = (mx[0] == -INFINITY) ? 0.0f : mx[0];
    float sum[1] = {0.0f};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
#pragma unroll
      for (int j = 0; j < N; ++j) {
        xv[i][j] = exp2f((xv[i][j] - m) * kLog2e);
        sum[0] += xv[i][j];
      }
    }
    group_reduce<TPR, 1, false>(sum, red, parity);
    const float inv = sum[0] > 0.0f ? 1.0f / sum[0] : 0.0f;
    if (live) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = tg + i * TPR;
        if (vi < nvec) {
          float o[N];
#pragma unroll
          for (int j = 0; j < N; ++j) o[j] = xv[i][j] * inv;
          V t; t.from_float(o);
          store_stream<V>(y + row * D, vi, t);
        }
      }
    }
  }
}

// ---- softmax backward -------------------------------------------------------------------------
// dx = scale * y * (dy - sum_j dy_j y_j).  causal_seq > 0: y is known to be 0 beyond the query position,
// so those vectors of y and dy are not read and dx gets zeros there.
template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__(RowGeom<TPR>::THREADS)
softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                   int64_t rows, int D, int causal_seq, float scale) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  constexpr int RPB = RowGeom<TPR>::RPB;
  __shared__ float red[64];
  int parity = 0;
  const int tg = threadIdx.x % TPR, g = threadIdx.x / TPR;
  const int nvec = D / N;
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * RPB; row0 < rows;
       row0 += static_cast<int64_t>(gridDim.x) * RPB) {
    const int64_t row = row0 + g;
    const bool live = row < rows;
    const int q = causal_seq > 0 ? static_cast<int>(row % causal_seq) : D;
    float yv[VPT][N], gv[VPT][N];
    float dot[1] = {0.0f};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tg + i * TPR;
      if (live && vi < nvec && vi * N <= q) {
        load_stream<V>(y + row * D, vi).to_float(yv[i]);
        load_stream<V>(dy + row * D, vi).to_float(gv[i]);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) { yv[i][j] = 0.0f; gv[i][j] = 0.0f; }
      }
#pragma unroll
      for (int j = 0; j < N; ++j) dot[0] = fmaf(yv[i][j], gv[i][j], dot[0]);
    }
    group_reduce<TPR, 1, false>(dot, red, parity);
    if (live) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = tg + i * TPR;
        if (vi < nvec) {
          float o[N];
#pragma unroll
          for (int j = 0; j < N; ++j) o[j] = yv[i][j] * (gv[i][j] - dot[0]) * scale;
          V t; t.from_float(o);
          store_stream<V>(dx + row * D, vi, t);
        }
      }
    }
  }
}

// ---- wide / unaligned rows: one block per row, scalar, data re-read from L2 --------------------
__device__ __forceinline__ float block_reduce(float v, bool is_max, float* smem) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = smem[0];
  for (int i = 1; i < nw; ++i) r = is_max ? fmaxf(r, smem[i]) : r + smem[i];
  return r;
}

template <typename T>
__global__ void rmsnorm_fwd_wide_kernel(const T* x, const T* w, T* y, float* rstd, int64_t rows, int64_t D,
                                        float eps) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * D;
    float ss = 0.0f;
    for (int64_t c = threadIdx.x; c < D; c += blockDim.x) { float v = to_f32(xr[c]); ss = fmaf(v, v, ss); }
    ss = block_reduce(ss, false, red);
    const float rinv = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
    if (rstd != nullptr && threadIdx.x == 0) rstd[row] = rinv;
    for (int64_t c = threadIdx.x; c < D; c += blockDim.x)
      y[row * D + c] = from_f32<T>(to_f32(xr[c]) * rinv * (w ? to_f32(w[c]) : 1.0f));
  }
}

// Writes dx and the per-row rinv (into `rinv_out`, [rows]) for the column pass below.
template <typename T>
__global__ void rmsnorm_bwd_wide_kernel(const T* x, const T* w, const T* dy, T* dx, float* rinv_out,
                                        int64_t rows, int64_t D, float eps) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * D;
    const T* gr = dy + row * D;
    float ss = 0.0f, gx = 0.0f;
    for (int64_t c = threadIdx.x; c < D; c += blockDim.x) {
      float v = to_f32(xr[c]);
      float gg = to_f32(gr[c]) * (w ? to_f32(w[c]) : 1.0f);
      ss = fmaf(v, v, ss);
      gx = fmaf(gg, v, gx);
    }
    ss = block_reduce(ss, false, red);
    gx = block_reduce(gx, false, red);
    const float rinv = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
    const float c0 = gx * rinv / static_cast<float>(D);
    if (rinv_out != nullptr && threadIdx.x == 0) rinv_out[row] = rinv;
    for (int64_t c = threadIdx.x; c < D; c += blockDim.x) {
      float xh = to_f32(xr[c]) * rinv;
      float gg = to_f32(gr[c]) * (w ? to_f32(w[c]) : 1.0f);
      dx[row * D + c] = from_f32<T>(rinv * (gg - xh * c0));
    }
  }
}

template <typename T>
__global__ void rmsnorm_dw_wide_kernel(const T* x, const T* dy, const float* rinv, float* dw, int64_t rows,
                                       int64_t D, int accumulate) {
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.0f;
  for (int64_t r = 0; r < rows; ++r) s = fmaf(to_f32(dy[r * D + c]), to_f32(x[r * D + c]) * rinv[r], s);
  dw[c] = accumulate ? dw[c] + s : s;
}

template <typename T>
__global__ void softmax_fwd_wide_kernel(const T* x, T* y, int64_t rows, int64_t D, int causal_seq, float scale) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * D;
    const int64_t q = causal_seq > 0 ? row % causal_seq : D;
    auto val = [&](int64_t c) { return c <= q ? to_f32(xr[c]) * scale : -INFINITY; };
    float mx = -INFINITY;
    for (int64_t c = threadIdx.x; c < D; c += blockDim.x) mx = fmaxf(mx, val(c));
    mx = block_reduce(mx, true, red);
    const float m = (mx == -INFINITY) ? 0.0f : mx;
    float sum = 0.0f;
    for (int64_t c = threadIdx.x; c < D; c += blockDim.x) sum += exp2f((val(c) - m) * kLog2e);
    sum = block_reduce(sum, false, red);
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    for (int64_t c = threadIdx.x; c < D; c += blockDim.x)
      y[row * D + c] = from_f32<T>(exp2f((val(c) - m) * kLog2e) * inv);
  }
}

template <typename T>
__global__ void softmax_bwd_wide_kernel(const T* y, const T* dy, T* dx, int64_t rows, int64_t D, float scale) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float dot = 0.0f;
    for (int64_t c = threadIdx.x; c < D; c += blockDim.x)
      dot = fmaf(to_f32(y[row * D + c]), to_f32(dy[row * D + c]), dot);
    dot = block_reduce(dot, false, red);
    for (int64_t c = threadIdx.x; c < D; c += blockDim.x)
      dx[row * D + c] = from_f32<T>(to_f32(y[row * D + c]) * (to_f32(dy[row * D + c]) - dot) * scale);
  }
}

// ---- dispatch ---------------------------------------------------------------------------------
struct RowPlan {
  int tpr = 0, vpt = 0;  // 0 = wide kernel
};
template <typename T>
RowPlan plan_rows(int64_t D, bool all_aligned, bool /*light*/) {
  constexpr int N = Vec16<T>::N;
  RowPlan p;
  if (!all_aligned || D % N != 0 || D > 4096 * N) return p;
  const int64_t nvec = D / N;
  if (nvec <= 32) { p.tpr = 32; p.vpt = 1; }
  else if (nvec <= 64) { p.tpr = 32; p.vpt = 2; }
  else if (nvec <= 128) { p.tpr = 64; p.vpt = 2; }
  else if (nvec <= 256) { p.tpr = 128; p.vpt = 2; }
  else if (nvec <= 512) { p.tpr = 256; p.vpt = 2; }
  else if (nvec <= 1024) { p.tpr = 256; p.vpt = 4; }
  else if (nvec <= 2048) { p.tpr = 512; p.vpt = 4; }
  else { p.tpr = 1024; p.vpt = 4; }
  return p;
}

#define MCB_ROW_DISPATCH(plan, CALL)                    \
  switch ((plan).tpr * 16 + (plan).vpt) {               \
    case 32 * 16 + 1: { CALL(32, 1); } break;           \
    case 32 * 16 + 2: { CALL(32, 2); } break;           \
    case 64 * 16 + 2: { CALL(64, 2); } break;           \
    case 128 * 16 + 2: { CALL(128, 2); } break;         \
    case 256 * 16 + 2: { CALL(256, 2); } break;         \
    case 256 * 16 + 4: { CALL(256, 4); } break;         \
    case 512 * 16 + 4: { CALL(512, 4); } break;         \
    case 1024 * 16 + 4: { CALL(1024, 4); } break;       \
    default: return fail(MCB_ERR_UNSUPPORTED, "row plan"); \
  }

int row_grid(int64_t rows, int tpr, int sm_count, int blocks_per_sm) {
  const int threads = tpr < 256 ? 256 : tpr;
  const int rpb = threads / tpr;
  int64_t need = (rows + rpb - 1) / rpb;
  int64_t cap = static_cast<int64_t>(sm_count) * blocks_per_sm;
  return static_cast<int>(need < cap ? (need > 0 ? need : 1) : cap);
}

template <typename T>
int rmsnorm_fwd_t(const void* x, const void* w, void* y, float* rstd, int64_t rows, int64_t D, float eps,
                  cudaStream_t st, const DeviceState* ds) {
  {
    const int rc = rowpipe::try_launch<T>(rowpipe::kRmsFwd, x, nullptr, w, y, rstd, nullptr, nullptr, rows, D, eps, 0, 1.0f, ds, st);
    if (rc != 1) return rc;
  }
  const bool al = aligned16(x) && aligned16(y) && (w == nullptr || aligned16(w));
  RowPlan p = plan_rows<T>(D, al, false);
  if (p.tpr == 0) {
    int grid = static_cast<int>(rows < ds->sm_count * 8 ? rows : ds->sm_count * 8);
    rmsnorm_fwd_wide_kernel<T><<<grid, 256, 0, st>>>((const T*)x, (const T*)w, (T*)y, rstd, rows, D, eps);
  } else {
#define CALL(TPR, VPT)                                                                               \
  rmsnorm_fwd_kernel<T, TPR, VPT><<<row_grid(rows, TPR, ds->sm_count, 8), RowGeom<TPR>::THREADS, 0, st>>>( \
      (const T*)x, (const T*)w, (T*)y, rstd, rows, (int)D, eps)
    MCB_ROW_DISPATCH(p, CALL)
#undef CALL
  }
  MCB_CHECK_LAUNCH("rmsnorm_fwd");
  return MCB_OK;
}

// Blocks of the RMSNorm backward.  Without dw: as many as keep the SMs full.  With dw every block also writes
// and later re-reads one float32 row of partial sums, so the count is capped to keep that below a few
// per cent of the main traffic (and within the workspace, kMaxDwBlocks rows).
constexpr int kMaxDwBlocks = 2048;
int bwd_blocks(int64_t rows, int tpr, int sm_count, bool need_dw, int elem_bytes) {
  int n = row_grid(rows, tpr, sm_count, 8);
  if (need_dw) {
    int64_t cap = rows * elem_bytes / 96;
    if (cap < 2 * static_cast<int64_t>(sm_count)) cap = 2 * static_cast<int64_t>(sm_count);
    if (n > cap) n = static_cast<int>(cap);
    if (n > kMaxDwBlocks) n = kMaxDwBlocks;
  }
  return n < 1 ? 1 : n;
}

template <typename T>
int rmsnorm_bwd_t(const void* x, const void* w, const void* dy, void* dx, float* dw, int accumulate,
                  int64_t rows, int64_t D, float eps, void* ws, size_t ws_bytes, cudaStream_t st,
                  const DeviceState* ds, const void* res = nullptr) {
  if (dw != nullptr && ws_bytes < mcb_rmsnorm_bwd_workspace_bytes(rows, D))
    return fail(MCB_ERR_WORKSPACE, "rmsnorm_bwd: workspace %zu < %zu bytes", ws_bytes,
                mcb_rmsnorm_bwd_workspace_bytes(rows, D));
  if (dw != nullptr && ws == nullptr) return fail(MCB_ERR_WORKSPACE, "rmsnorm_bwd: workspace is null");
  {
    int blocks = 0;
    const int rc = rowpipe::try_launch<T>(rowpipe::kRmsBwd, x, dy, w, dx, nullptr, dw ? (float*)ws : nullptr, &blocks, rows, D,
                                          eps, 0, 1.0f, ds, st, res);
    if (rc == MCB_OK && dw != nullptr) {
      colsum_partials_kernel<<<(unsigned)((D + 31) / 32), 256, 0, st>>>((const float*)ws, dw, blocks, (int)D, accumulate);
      MCB_CHECK_LAUNCH("rmsnorm_dw_reduce");
    }
    if (rc != 1) return rc;
  }
  const bool al = aligned16(x) && aligned16(dy) && aligned16(dx) && (w == nullptr || aligned16(w));
  RowPlan p = plan_rows<T>(D, al, false);
  if (dw != nullptr && ws_bytes < mcb_rmsnorm_bwd_workspace_bytes(rows, D))
    return fail(MCB_ERR_WORKSPACE, "rmsnorm_bwd: workspace %zu < %zu bytes", ws_bytes,
                mcb_rmsnorm_bwd_workspace_bytes(rows, D));
  if (dw != nullptr && ws == nullptr) return fail(MCB_ERR_WORKSPACE, "rmsnorm_bwd: workspace is null");
  if (p.tpr == 0) {
    int grid = static_cast<int>(rows < ds->sm_count * 8 ? rows : ds->sm_count * 8);
    rmsnorm_bwd_wide_kernel<T><<<grid, 256, 0, st>>>((const T*)x, (const T*)w, (const T*)dy, (T*)dx,
                                                     dw ? (float*)ws : nullptr, rows, D, eps);
    MCB_CHECK_LAUNCH("rmsnorm_bwd_wide");
    if (dw != nullptr) {
      rmsnorm_dw_wide_kernel<T><<<(unsigned)((D + 255) / 256), 256, 0, st>>>((const T*)x, (const T*)dy,
                                                                             (const float*)ws, dw, rows, D,
                                                                             accumulate);
      MCB_CHECK_LAUNCH("rmsnorm_dw_wide");
    }
    return MCB_OK;
  }
  const int nblocks = bwd_blocks(rows, p.tpr, ds->sm_count, dw != nullptr, (int)sizeof(T));
  const int rpb = (p.tpr < 256 ? 256 : p.tpr) / p.tpr;
  const size_t smem = (dw != nullptr && rpb > 1) ? static_cast<size_t>(rpb) * D * sizeof(float) : 0;
  if (dw != nullptr) {
#define CALL(TPR, VPT)                                                                           \
  rmsnorm_bwd_kernel<T, TPR, VPT, true><<<nblocks, RowGeom<TPR>::THREADS, smem, st>>>(           \
      (const T*)x, (const T*)w, (const T*)dy, (T*)dx, (float*)ws, rows, (int)D, eps)
    MCB_ROW_DISPATCH(p, CALL)
#undef CALL
  } else {
#define CALL(TPR, VPT)                                                                           \
  rmsnorm_bwd_kernel<T, TPR, VPT, false><<<nblocks, RowGeom<TPR>::THREADS, 0, st>>>(             \
      (const T*)x, (const T*)w, (const T*)dy, (T*)dx, nullptr, rows, (int)D, eps)
    MCB_ROW_DISPATCH(p, CALL)
#undef CALL
  }
  MCB_CHECK_LAUNCH("rmsnorm_bwd");
  if (dw != nullptr) {
    colsum_partials_kernel<<<(unsigned)((D + 31) / 32), 256, 0, st>>>((const float*)ws, dw, nblocks, (int)D,
                                                                        accumulate);
    MCB_CHECK_LAUNCH("rmsnorm_dw_reduce");
  }
  return MCB_OK;
}

template <typename T>
int softmax_fwd_t(const void* x, void* y, int64_t rows, int64_t D, int causal_seq, float scale, cudaStream_t st,
                  const DeviceState* ds) {
  {
    const int rc = rowpipe::try_launch<T>(rowpipe::kSmFwd, x, nullptr, nullptr, y, nullptr, nullptr, nullptr, rows, D, 0.0f,
                                          causal_seq, scale, ds, st);
    if (rc != 1) return rc;
  }
  RowPlan p = plan_rows<T>(D, aligned16(x) && aligned16(y), true);
  if (p.tpr == 0) {
    int grid = static_cast<int>(rows < ds->sm_count * 8 ? rows : ds->sm_count * 8);
    softmax_fwd_wide_kernel<T><<<grid, 256, 0, st>>>((const T*)x, (T*)y, rows, D, causal_seq, scale);
  } else {
#define CALL(TPR, VPT)                                                                                \
  softmax_fwd_kernel<T, TPR, VPT><<<row_grid(rows, TPR, ds->sm_count, 8), RowGeom<TPR>::THREADS, 0, st>>>( \
      (const T*)x, (T*)y, rows, (int)D, causal_seq, scale)
    MCB_ROW_DISPATCH(p, CALL)
#undef CALL
  }
  MCB_CHECK_LAUNCH("softmax_fwd");
  return MCB_OK;
}

template <typename T>
int softmax_bwd_t(const void* y, const void* dy, void* dx, int64_t rows, int64_t D, int causal_seq, float scale, cudaStream_t st,
                  const DeviceState* ds) {
  {
    const int rc = rowpipe::try_launch<T>(rowpipe::kSmBwd, y, dy, nullptr, dx, nullptr, nullptr, nullptr, rows, D, 0.0f,
                                          causal_seq, scale, ds, st);
    if (rc != 1) return rc;
  }
  RowPlan p = plan_rows<T>(D, aligned16(y) && aligned16(dy) && aligned16(dx), true);
  if (p.tpr == 0) {
    int grid = static_cast<int>(rows < ds->sm_count * 8 ? rows : ds->sm_count * 8);
    softmax_bwd_wide_kernel<T><<<grid, 256, 0, st>>>((const T*)y, (const T*)dy, (T*)dx, rows, D, scale);
  } else {
#define CALL(TPR, VPT)                                                                                \
  softmax_bwd_kernel<T, TPR, VPT><<<row_grid(rows, TPR, ds->sm_count, 8), RowGeom<TPR>::THREADS, 0, st>>>( \
      (const T*)y, (const T*)dy, (T*)dx, rows, (int)D, causal_seq, scale)
    MCB_ROW_DISPATCH(p, CALL)
#undef CALL
  }
  MCB_CHECK_LAUNCH("softmax_bwd");
  return MCB_OK;
}

int check_rows(const char* op, int64_t rows, int64_t D, int dtype) {
  if (rows <= 0 || D <= 0) return fail(MCB_ERR_SHAPE, "%s: rows=%lld D=%lld must be positive", op, (long long)rows, (long long)D);
  if (rows > (1ll << 40) || D > (1ll << 30)) return fail(MCB_ERR_SHAPE, "%s: dimension too large", op);
  if (dtype != MCB_F32 && dtype != MCB_BF16) return fail(MCB_ERR_UNSUPPORTED, "%s: dtype %d", op, dtype);
  return MCB_OK;
}

}  // namespace
}  // namespace mcb

using namespace mcb;

extern "C" int mcb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int64_t rows, int64_t D,
                               float eps, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_rmsnorm_fwd");
  if (!x || !y) return fail(MCB_ERR_NULL, "rmsnorm_fwd: x or y is null");
  if (int rc = check_rows("rmsnorm_fwd", rows, D, dtype)) return rc;
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MCB_F32 ? rmsnorm_fwd_t<float>(x, w, y, rstd, rows, D, eps, st, ds)
                          : rmsnorm_fwd_t<__nv_bfloat16>(x, w, y, rstd, rows, D, eps, st, ds);
}

extern "C" size_t mcb_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t D) {
  if (rows <= 0 || D <= 0) return 0;
  // Either per-block partial sums of dw (at most kMaxDwBlocks rows) or, for the wide kernel, one float per row.
  size_t partials = static_cast<size_t>(kMaxDwBlocks) * static_cast<size_t>(D) * sizeof(float);
  size_t per_row = static_cast<size_t>(rows) * sizeof(float);
  return partials > per_row ? partials : per_row;
}

extern "C" int mcb_add(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream);

extern "C" int mcb_rmsnorm_bwd_ex(const void* x, const void* w, const void* dy, const void* dx_residual, void* dx,
                                  float* dw, int accumulate, int64_t rows, int64_t D, float eps, int dtype,
                                  void* workspace, size_t workspace_bytes, void* stream) {
  MCB_NVTX_RANGE("mcb_add");
  if (dx_residual == nullptr)
    return mcb_rmsnorm_bwd(x, w, dy, dx, dw, accumulate, rows, D, eps, dtype, workspace, workspace_bytes, stream);
  if (!x || !dy || !dx) return fail(MCB_ERR_NULL, "rmsnorm_bwd_ex: x, dy or dx is null");
  if (int rc = check_rows("rmsnorm_bwd_ex", rows, D, dtype)) return rc;
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  if (ds->sm_count > 256) return fail(MCB_ERR_UNSUPPORTED, "rmsnorm_bwd_ex: more than 256 SMs");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The bulk-copy pipeline adds the residual as it writes dx.  Shapes it declines (rows that are not whole
  // 16-byte vectors, unaligned operands) take the plain kernels and one more element-wise pass.
  {
    int blocks = 0;
    const bool has_ws = dw == nullptr || (workspace != nullptr && workspace_bytes >= mcb_rmsnorm_bwd_workspace_bytes(rows, D));
    if (!has_ws) return fail(MCB_ERR_WORKSPACE, "rmsnorm_bwd_ex: workspace %zu < %zu bytes", workspace_bytes,
                             mcb_rmsnorm_bwd_workspace_bytes(rows, D));
    const int rc = dtype == MCB_F32
        ? rowpipe::try_launch<float>(rowpipe::kRmsBwd, x, dy, w, dx, nullptr, dw ? (float*)workspace : nullptr, &blocks,
                                     rows, D, eps, 0, 1.0f, ds, st, dx_residual)
        : rowpipe::try_launch<__nv_bfloat16>(rowpipe::kRmsBwd, x, dy, w, dx, nullptr, dw ? (float*)workspace : nullptr,
                                             &blocks, rows, D, eps, 0, 1.0f, ds, st, dx_residual);
    if (rc == MCB_OK && dw != nullptr) {
      colsum_partials_kernel<<<(unsigned)((D + 31) / 32), 256, 0, st>>>((const float*)workspace, dw, blocks, (int)D, accumulate);
      MCB_CHECK_LAUNCH("rmsnorm_dw_reduce");
    }
    if (rc != 1) return rc;
  }
  if (dx == dx_residual) return fail(MCB_ERR_UNSUPPORTED, "rmsnorm_bwd_ex: dx may alias dx_residual only for rows of whole, aligned 16-byte vectors");
  if (int rc = mcb_rmsnorm_bwd(x, w, dy, dx, dw, accumulate, rows, D, eps, dtype, workspace, workspace_bytes, stream)) return rc;
  return mcb_add(dx, dx_residual, dx, rows * D, dtype, stream);
}

extern "C" int mcb_rmsnorm_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, int accumulate,
                               int64_t rows, int64_t D, float eps, int dtype, void* workspace,
                               size_t workspace_bytes, void* stream) {
  if (!x || !dy || !dx) return fail(MCB_ERR_NULL, "rmsnorm_bwd: x, dy or dx is null");
  if (int rc = check_rows("rmsnorm_bwd", rows, D, dtype)) return rc;
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  if (ds->sm_count > 256) return fail(MCB_ERR_UNSUPPORTED, "rmsnorm_bwd: more than 256 SMs");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MCB_F32
             ? rmsnorm_bwd_t<float>(x, w, dy, dx, dw, accumulate, rows, D, eps, workspace, workspace_bytes, st, ds)
             : rmsnorm_bwd_t<__nv_bfloat16>(x, w, dy, dx, dw, accumulate, rows, D, eps, workspace,
                                            workspace_bytes, st, ds);
}

extern "C" int mcb_softmax_fwd(const void* x, void* y, int64_t rows, int64_t D, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_softmax_fwd");
  if (!x || !y) return fail(MCB_ERR_NULL, "softmax_fwd: x or y is null");
  if (int rc = check_rows("softmax_fwd", rows, D, dtype)) return rc;
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MCB_F32 ? softmax_fwd_t<float>(x, y, rows, D, 0, 1.0f, st, ds)
                          : softmax_fwd_t<__nv_bfloat16>(x, y, rows, D, 0, 1.0f, st, ds);
}

extern "C" int mcb_softmax_causal_fwd(const void* x, void* y, int64_t rows, int64_t D, int64_t seq, float scale, int dtype,
                                      void* stream) {
  MCB_NVTX_RANGE("mcb_softmax_causal_fwd");
  if (!x || !y) return fail(MCB_ERR_NULL, "softmax_causal_fwd: x or y is null");
  if (int rc = check_rows("softmax_causal_fwd", rows, D, dtype)) return rc;
  if (seq <= 0 || seq > 0x7fffffff || rows % seq != 0)
    return fail(MCB_ERR_SHAPE, "softmax_causal_fwd: rows=%lld must be a multiple of seq=%lld", (long long)rows, (long long)seq);
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MCB_F32 ? softmax_fwd_t<float>(x, y, rows, D, (int)seq, scale, st, ds)
                          : softmax_fwd_t<__nv_bfloat16>(x, y, rows, D, (int)seq, scale, st, ds);
}

extern "C" int mcb_softmax_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t D, int dtype,
                               void* stream) {
  MCB_NVTX_RANGE("mcb_softmax_bwd");
  if (!y || !dy || !dx) return fail(MCB_ERR_NULL, "softmax_bwd: y, dy or dx is null");
  if (int rc = check_rows("softmax_bwd", rows, D, dtype)) return rc;
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MCB_F32 ? softmax_bwd_t<float>(y, dy, dx, rows, D, 0, 1.0f, st, ds)
                          : softmax_bwd_t<__nv_bfloat16>(y, dy, dx, rows, D, 0, 1.0f, st, ds);
}

extern "C" int mcb_softmax_causal_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t D, int64_t seq,
                                      float scale, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_softmax_causal_bwd");
  if (!y || !dy || !dx) return fail(MCB_ERR_NULL, "softmax_causal_bwd: y, dy or dx is null");
  if (int rc = check_rows("softmax_causal_bwd", rows, D, dtype)) return rc;
  if (seq < 0 || seq > 0x7fffffff || (seq > 0 && rows % seq != 0))
    return fail(MCB_ERR_SHAPE, "softmax_causal_bwd: rows=%lld must be a multiple of seq=%lld", (long long)rows, (long long)seq);
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MCB_F32 ? softmax_bwd_t<float>(y, dy, dx, rows, D, (int)seq, scale, st, ds)
                          : softmax_bwd_t<__nv_bfloat16>(y, dy, dx, rows, D, (int)seq, scale, st, ds);
}

// ---- RMSNorm backward for callers that cannot allocate ------------------------------------------------
// The per-block partial sums of dw live in this fixed device array instead of a caller workspace.  Every
// GPU that loads the library holds these 2 MiB until the process exits.
constexpr int kNoAllocMaxBlocks = 128;
constexpr int kNoAllocMaxD = 4096;
static __device__ __align__(256) float g_rmsnorm_dw_scratch[kNoAllocMaxBlocks * kNoAllocMaxD];

namespace {
// Device address of the array above, per device; filled on the first call on that device.
float* g_noalloc_scratch_ptr[64] = {};

template <typename T>
int rmsnorm_bwd_noalloc_t(const void* x, const void* w, const void* dy, void* dx, float* dw, int accumulate,
                          int64_t rows, int64_t D, float eps, float* scratch, cudaStream_t st, const mcb::DeviceState* ds) {
  using namespace mcb;
  const bool al = aligned16(x) && aligned16(dy) && aligned16(dx) && (w == nullptr || aligned16(w));
  RowPlan p = plan_rows<T>(D, al, false);
  if (p.tpr == 0)
    return fail(MCB_ERR_ALIGN, "rmsnorm_bwd_noalloc: rows must be 16-byte aligned and D a multiple of %d", Vec16<T>::N);
  int nblocks = bwd_blocks(rows, p.tpr, ds->sm_count, dw != nullptr, (int)sizeof(T));
  if (dw != nullptr && nblocks > kNoAllocMaxBlocks) nblocks = kNoAllocMaxBlocks;
  const int rpb = (p.tpr < 256 ? 256 : p.tpr) / p.tpr;
  const size_t smem = (dw != nullptr && rpb > 1) ? static_cast<size_t>(rpb) * D * sizeof(float) : 0;
  if (dw != nullptr) {
#define CALL(TPR, VPT)                                                                           \
  rmsnorm_bwd_kernel<T, TPR, VPT, true><<<nblocks, RowGeom<TPR>::THREADS, smem, st>>>(           \
      (const T*)x, (const T*)w, (const T*)dy, (T*)dx, scratch, rows, (int)D, eps)
    MCB_ROW_DISPATCH(p, CALL)
#undef CALL
  } else {
#define CALL(TPR, VPT)                                                                           \
  rmsnorm_bwd_kernel<T, TPR, VPT, false><<<nblocks, RowGeom<TPR>::THREADS, 0, st>>>(             \
      (const T*)x, (const T*)w, (const T*)dy, (T*)dx, nullptr, rows, (int)D, eps)
    MCB_ROW_DISPATCH(p, CALL)
#undef CALL
  }
  MCB_CHECK_LAUNCH("rmsnorm_bwd_noalloc");
  if (dw != nullptr) {
    // every block wrote its whole row of partials above, so nothing stale from an earlier call is read
    colsum_partials_kernel<<<(unsigned)((D + 31) / 32), 256, 0, st>>>(scratch, dw, nblocks, (int)D, accumulate);
    MCB_CHECK_LAUNCH("rmsnorm_dw_reduce_noalloc");
  }
  return MCB_OK;
}
}  // namespace

extern "C" int mcb_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, void* dx, float* dw, int accumulate,
                                       int64_t rows, int64_t D, float eps, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_rmsnorm_bwd_noalloc");
  using namespace mcb;
  if (!x || !dy || !dx) return fail(MCB_ERR_NULL, "rmsnorm_bwd_noalloc: x, dy or dx is null");
  if (int rc = check_rows("rmsnorm_bwd_noalloc", rows, D, dtype)) return rc;
  if (D > kNoAllocMaxD)
    return fail(MCB_ERR_SHAPE, "rmsnorm_bwd_noalloc: D=%lld exceeds the built-in scratch limit of %d columns; "
                "use mcb_rmsnorm_bwd with a caller workspace", (long long)D, kNoAllocMaxD);
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  int dev = 0;
  MCB_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MCB_ERR_SHAPE, "rmsnorm_bwd_noalloc: device %d out of range", dev);
  if (g_noalloc_scratch_ptr[dev] == nullptr) {
    // First call on this device: ask the runtime where the array lives on the CURRENT device.  (The symbol's
    // name in host code is only a handle; passing it to a kernel directly would not be a device address.)
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_rmsnorm_dw_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_rmsnorm_dw_scratch)");
    if (ptr == nullptr) return fail(MCB_ERR_UNSUPPORTED, "rmsnorm_bwd_noalloc: scratch symbol has no device address");
    g_noalloc_scratch_ptr[dev] = ptr;
  }
  float* scratch = g_noalloc_scratch_ptr[dev];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MCB_F32
             ? rmsnorm_bwd_noalloc_t<float>(x, w, dy, dx, dw, accumulate, rows, D, eps, scratch, st, ds)
             : rmsnorm_bwd_noalloc_t<__nv_bfloat16>(x, w, dy, dx, dw, accumulate, rows, D, eps, scratch, st, ds);
}
