// The element-wise "frame" of the Qwen-shaped training step around the LoRA hot path: embedding
// gather, rotary embedding with the head-major re-layout attention wants, SwiGLU, residual add, and a
// fused cross-entropy forward+backward.  All are HBM-bound streaming kernels; float32 or bfloat16
// storage, float32 arithmetic.
#include "common.cuh"

namespace mcb {
namespace {

// ---- embedding (candle_nn::embedding, src/models/qwen.rs:189; gather of table rows) -----------------
template <typename T>
__global__ void embedding_fwd_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                     int64_t M, int H, int vocab) {
  const int64_t row = blockIdx.x;
  if (row >= M) return;
  int32_t id = ids[row];
  if (id < 0 || id >= vocab) id = 0;  // ids are validated on the host; never read out of range
  const T* src = table + static_cast<int64_t>(id) * H;
  T* dst = out + row * H;
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0 && (H * sizeof(T)) % 16 == 0) {
    const int nv = H * sizeof(T) / 16;
    for (int i = threadIdx.x; i < nv; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
  }
}

// ---- rotary embedding + [B,S,H,d] -> [B,H,S,d] (src/models/transformer.rs:47-120,255-257) ----------------
// Half-split rotation: (x1, x2) -> (x1 cos - x2 sin, x1 sin + x2 cos), angle = pos * theta^(-2i/d).
// inverse != 0 applies the transposed rotation and the inverse layout change (the backward pass).
// rotate == 0 only changes the layout (used for V).
template <typename T>
__global__ void rope_relayout_kernel(const T* __restrict__ src, T* __restrict__ dst, int B, int S, int H, int d,
                                     float theta, int rotate, int inverse, int64_t pitch, int64_t offset) {
  // One thread owns a 16-byte chunk of the first half of a head (and the matching chunk of the second
  // half) at one (batch, position), computes its sines and cosines once, and walks over the heads.
  using V = Vec16<T>;
  constexpr int N = V::N;
  const int half = d / 2;
  const int chunks = half / N;  // host guarantees half % N == 0
  const int64_t total = static_cast<int64_t>(B) * S * chunks;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % chunks);
    const int64_t bs = idx / chunks;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    float cs[N], sn[N];
#pragma unroll
    for (int j = 0; j < N; ++j) {
      if (rotate) {
        // 1 / theta^(2i/d) as in the reference's table (float32 powf), angle = position * inv_freq
        const int i = c * N + j;
        const float inv_freq = 1.0f / powf(theta, static_cast<float>(2 * i) / static_cast<float>(d));
        sincosf(static_cast<float>(s) * inv_freq, &sn[j], &cs[j]);
        if (inverse) sn[j] = -sn[j];
      } else {
        cs[j] = 1.0f; sn[j] = 0.0f;
      }
    }
    for (int h = 0; h < H; ++h) {
      // [B,S,H,d] side: token rows `pitch` elements apart, the heads starting `offset` elements into a row
      const int64_t bshd = (static_cast<int64_t>(b) * S + s) * pitch + offset + static_cast<int64_t>(h) * d;
      const int64_t bhsd = ((static_cast<int64_t>(b) * H + h) * S + s) * d;   // [B,H,S,d]
      const int64_t in = inverse ? bhsd : bshd, out = inverse ? bshd : bhsd;
      V a, bb;
      a.raw = *reinterpret_cast<const decltype(a.raw)*>(src + in + c * N);
      bb.raw = *reinterpret_cast<const decltype(bb.raw)*>(src + in + half + c * N);
      float x1[N], x2[N], o1[N], o2[N];
      a.to_float(x1); bb.to_float(x2);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        o1[j] = x1[j] * cs[j] - x2[j] * sn[j];
        o2[j] = x1[j] * sn[j] + x2[j] * cs[j];
      }
      a.from_float(o1); bb.from_float(o2);
      *reinterpret_cast<decltype(a.raw)*>(dst + out + c * N) = a.raw;
      *reinterpret_cast<decltype(bb.raw)*>(dst + out + half + c * N) = bb.raw;
    }
  }
}

// Scalar variant for head sizes whose half is not a multiple of the vector width.
// The same for the query, key and value heads of a fused q/k/v row in one launch: the sines and cosines of a
// (position, chunk) are computed once and used for the rotated segments (q and k); v is only re-laid out.
template <typename T>
struct RopeSegment {
  T* head_major;    // [B, H, S, d]
  int H;
  int64_t offset;   // first column of the segment's heads in a token row
  int rotate;
};
template <typename T>
__global__ void rope_relayout_qkv_kernel(T* __restrict__ fused, RopeSegment<T> s0, RopeSegment<T> s1, RopeSegment<T> s2, int B, int S,
                                         int d, float theta, int inverse, int64_t pitch) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  const int half = d / 2;
  const int chunks = half / N;
  const int64_t total = static_cast<int64_t>(B) * S * chunks;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % chunks);
    const int64_t bs = idx / chunks;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    float cs[N], sn[N];
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const int i = c * N + j;
      const float inv_freq = 1.0f / powf(theta, static_cast<float>(2 * i) / static_cast<float>(d));
      sincosf(static_cast<float>(s) * inv_freq, &sn[j], &cs[j]);
      if (inverse) sn[j] = -sn[j];
    }
#pragma unroll
    for (int g = 0; g < 3; ++g) {
      const RopeSegment<T>& sg = g == 0 ? s0 : g == 1 ? s1 : s2;
      for (int h = 0; h < sg.H; ++h) {
        const int64_t tok = (static_cast<int64_t>(b) * S + s) * pitch + sg.offset + static_cast<int64_t>(h) * d;
        const int64_t hm = ((static_cast<int64_t>(b) * sg.H + h) * S + s) * d;
        const T* in = inverse ? sg.head_major + hm : fused + tok;
        T* out = inverse ? fused + tok : sg.head_major + hm;
        V a, bb;
        a.raw = *reinterpret_cast<const decltype(a.raw)*>(in + c * N);
        bb.raw = *reinterpret_cast<const decltype(bb.raw)*>(in + half + c * N);
        if (sg.rotate) {
          float x1[N], x2[N], o1[N], o2[N];
          a.to_float(x1); bb.to_float(x2);
#pragma unroll
          for (int j = 0; j < N; ++j) {
            o1[j] = x1[j] * cs[j] - x2[j] * sn[j];
            o2[j] = x1[j] * sn[j] + x2[j] * cs[j];
          }
          a.from_float(o1); bb.from_float(o2);
        }
        *reinterpret_cast<decltype(a.raw)*>(out + c * N) = a.raw;
        *reinterpret_cast<decltype(bb.raw)*>(out + half + c * N) = bb.raw;
      }
    }
  }
}

template <typename T>
__global__ void rope_relayout_scalar_kernel(const T* __restrict__ src, T* __restrict__ dst, int B, int S, int H, int d,
                                            float theta, int rotate, int inverse, int64_t pitch, int64_t offset) {
  const int half = d / 2;
  const int64_t total = static_cast<int64_t>(B) * S * H * half;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % half);
    int64_t t = idx / half;
    const int h = static_cast<int>(t % H); t /= H;
    const int s = static_cast<int>(t % S);
    const int b = static_cast<int>(t / S);
    const int64_t bshd = (static_cast<int64_t>(b) * S + s) * pitch + offset + static_cast<int64_t>(h) * d;
    const int64_t bhsd = ((static_cast<int64_t>(b) * H + h) * S + s) * d;
    const int64_t in = inverse ? bhsd : bshd, out = inverse ? bshd : bhsd;
    const float x1 = to_f32(src[in + i]), x2 = to_f32(src[in + half + i]);
    float o1 = x1, o2 = x2;
    if (rotate) {
      const float inv_freq = 1.0f / powf(theta, static_cast<float>(2 * i) / static_cast<float>(d));
      float sn, cs;
      sincosf(static_cast<float>(s) * inv_freq, &sn, &cs);
      if (inverse) sn = -sn;
      o1 = x1 * cs - x2 * sn;
      o2 = x1 * sn + x2 * cs;
    }
    dst[out + i] = from_f32<T>(o1);
    dst[out + half + i] = from_f32<T>(o2);
  }
}

// ---- SwiGLU (src/models/transformer.rs:389-395) ---------------------------------------------------------
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out, int64_t n) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  const int64_t nv = n / N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    V g, u, o;
    g.raw = reinterpret_cast<const decltype(g.raw)*>(gate)[i];
    u.raw = reinterpret_cast<const decltype(u.raw)*>(up)[i];
    float gf[N], uf[N], of[N];
    g.to_float(gf); u.to_float(uf);
#pragma unroll
    for (int j = 0; j < N; ++j) of[j] = gf[j] / (1.0f + __expf(-gf[j])) * uf[j];
    o.from_float(of);
    reinterpret_cast<decltype(o.raw)*>(out)[i] = o.raw;
  }
}

// d_gate = d_out * up * sig(g) * (1 + g (1 - sig(g))),  d_up = d_out * silu(g).  In place on gate/up allowed.
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gate, const T* __restrict__ up, const T* __restrict__ dout,
                                  T* __restrict__ dgate, T* __restrict__ dup, int64_t n) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  const int64_t nv = n / N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    V g, u, d, og, ou;
    g.raw = reinterpret_cast<const decltype(g.raw)*>(gate)[i];
    u.raw = reinterpret_cast<const decltype(u.raw)*>(up)[i];
    d.raw = reinterpret_cast<const decltype(d.raw)*>(dout)[i];
    float gf[N], uf[N], df[N], a[N], b[N];
    g.to_float(gf); u.to_float(uf); d.to_float(df);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const float sg = 1.0f / (1.0f + __expf(-gf[j]));
      a[j] = df[j] * uf[j] * sg * (1.0f + gf[j] * (1.0f - sg));
      b[j] = df[j] * gf[j] * sg;
    }
    og.from_float(a); ou.from_float(b);
    reinterpret_cast<decltype(og.raw)*>(dgate)[i] = og.raw;
    reinterpret_cast<decltype(ou.raw)*>(dup)[i] = ou.raw;
  }
}

template <typename T>
__global__ void add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  const int64_t nv = n / N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    V x, y, o;
    x.raw = reinterpret_cast<const decltype(x.raw)*>(a)[i];
    y.raw = reinterpret_cast<const decltype(y.raw)*>(b)[i];
    float xf[N], yf[N];
    x.to_float(xf); y.to_float(yf);
#pragma unroll
    for (int j = 0; j < N; ++j) xf[j] += yf[j];
    o.from_float(xf);
    reinterpret_cast<decltype(o.raw)*>(out)[i] = o.raw;
  }
}

template <typename T>
__global__ void add_scalar_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    out[i] = from_f32<T>(to_f32(a[i]) + to_f32(b[i]));
}

// out = a * b (mode 0) or out = a * scalar (mode 1): Operation::Mul / Operation::MulScalar of the lazy graph
// (src/graph/executor.rs:97-120).
template <typename T>
__global__ void mul_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n, float scalar,
                           int mode) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    out[i] = from_f32<T>(to_f32(a[i]) * (mode == 0 ? to_f32(b[i]) : scalar));
}

// ---- cross-entropy forward + backward (src/training/loss.rs:97-146) ----------------------------------------
// One block per row of logits [M,V].  Sweep 1: online max / sum-exp (HBM read).  Sweep 2 (the row is in
// L2 by now): overwrite the row with d loss / d logits = (softmax - onehot) * inv_count; ignored rows get
// zeros.  nll[row] = logsumexp - logit[target] (0 for ignored rows); a second tiny kernel sums nll in
// row order, so the loss is deterministic.
constexpr float kLog2e = 1.4426950408889634f;
// 2^x with denormal results flushed to zero: one instruction, where __expf's denormal handling takes several
// (relative error about 2^-22; the long-row loops below are bound by their instruction count)
__device__ __forceinline__ float ex2_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void online_combine(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  if (mm == -INFINITY) { m = mm; s = 0.0f; return; }
  s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
  m = mm;
}

// Persistent: block b takes rows b, b + gridDim.x, ...  Measured on [8192, 151936] bf16: how many rows are in flight
// (148 blocks of 1024 threads = 45 MB, inside the L2, up to 1184 blocks of 256 threads = 360 MB) moves the time by
// 10 % at most, smaller blocks ahead: the loops are bound by their instructions (two exponentials per element over
// the two sweeps), not by where sweep 2 finds the row.
template <typename T>
__global__ void __launch_bounds__(1024)
cross_entropy_kernel(T* __restrict__ logits, const int32_t* __restrict__ targets, float* __restrict__ nll,
                     const int32_t* __restrict__ count_ptr, int64_t M, int V, int write_grad) {
  __shared__ float sm[32], ss[32];
  const float inv_count = 1.0f / static_cast<float>(max(1, *count_ptr));
  using VT = Vec16<T>;
  constexpr int NV = VT::N;
  const int bd = blockDim.x;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    T* lr = logits + row * V;
    const int32_t tgt = targets[row];
    const bool ignored = tgt < 0 || tgt >= V;  // u32::MAX (src/training/trainer.rs:385) reads as -1
    if (ignored) {   // the same for every thread of the block
      if (threadIdx.x == 0) nll[row] = 0.0f;
      if (write_grad)
        for (int c = threadIdx.x; c < V; c += bd) lr[c] = from_f32<T>(0.0f);
      continue;
    }
    const bool vec = (V % NV == 0) && ((reinterpret_cast<uintptr_t>(lr) & 15u) == 0);
    float m = -INFINITY, s = 0.0f;
    if (vec) {
      const int nvec = V / NV;
      const auto* src = reinterpret_cast<const decltype(VT::raw)*>(lr);
      auto absorb = [&](const VT& t) {
        float f[NV];
        t.to_float(f);
        float vm = f[0];
#pragma unroll
        for (int j = 1; j < NV; ++j) vm = fmaxf(vm, f[j]);
        if (vm == -INFINITY) return;  // a wholly masked vector adds nothing (and exp(-inf - -inf) would be NaN)
        if (vm > m) { s *= __expf(m - vm); m = vm; }
        const float m2 = -m * kLog2e;   // exp(f - m) = 2^(f log2e - m log2e): one fused multiply-add and one special function
#pragma unroll
        for (int j = 0; j < NV; ++j) s += ex2_ftz(fmaf(f[j], kLog2e, m2));
      };
      int c = threadIdx.x;
      for (; c + 3 * bd < nvec; c += 4 * bd) {   // four loads in flight per thread
        VT t0, t1, t2, t3;
        t0.raw = src[c]; t1.raw = src[c + bd]; t2.raw = src[c + 2 * bd]; t3.raw = src[c + 3 * bd];
        absorb(t0); absorb(t1); absorb(t2); absorb(t3);
      }
      for (; c < nvec; c += bd) {
        VT t; t.raw = src[c];
        absorb(t);
      }
    } else {
      for (int c = threadIdx.x; c < V; c += bd) {
        const float v = to_f32(lr[c]);
        if (v > m) { s = s * __expf(m - v) + 1.0f; m = v; } else if (v != -INFINITY) { s += __expf(v - m); }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_combine(m, s, m2, s2);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = bd >> 5;
    if (lane == 0) { sm[warp] = m; ss[warp] = s; }
    __syncthreads();
    m = sm[0]; s = ss[0];
    for (int w = 1; w < nw; ++w) online_combine(m, s, sm[w], ss[w]);
    const float lse = m + logf(s);
    if (threadIdx.x == 0) nll[row] = lse - to_f32(lr[tgt]);
    __syncthreads();  // thread 0 has read lr[tgt] before anyone overwrites it; sm / ss are free for the next row
    if (write_grad) {
      if (vec) {
        const int nvec = V / NV;
        auto* dst = reinterpret_cast<decltype(VT::raw)*>(lr);
        const float lse2 = -lse * kLog2e;
        auto grad = [&](VT& t, int c) {
          float f[NV];
          t.to_float(f);
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            float p = ex2_ftz(fmaf(f[j], kLog2e, lse2));
            if (c * NV + j == tgt) p -= 1.0f;
            f[j] = p * inv_count;
          }
          t.from_float(f);
          dst[c] = t.raw;
        };
        int c = threadIdx.x;
        for (; c + 3 * bd < nvec; c += 4 * bd) {
          VT t0, t1, t2, t3;
          t0.raw = dst[c]; t1.raw = dst[c + bd]; t2.raw = dst[c + 2 * bd]; t3.raw = dst[c + 3 * bd];
          grad(t0, c); grad(t1, c + bd); grad(t2, c + 2 * bd); grad(t3, c + 3 * bd);
        }
        for (; c < nvec; c += bd) {
          VT t; t.raw = dst[c];
          grad(t, c);
        }
      } else {
        for (int c = threadIdx.x; c < V; c += bd) {
          float p = __expf(to_f32(lr[c]) - lse);
          if (c == tgt) p -= 1.0f;
          lr[c] = from_f32<T>(p * inv_count);
        }
      }
    }
  }
}

// Launch shape of cross_entropy_kernel: eight blocks of 256 threads per SM, fewer when there are fewer rows.
static void cross_entropy_launch_shape(int64_t rows, int64_t V, unsigned* grid, unsigned* block) {
  const DeviceState* ds = current_device_state();
  const int sms = ds ? ds->sm_count : 148;
  const int threads = 256, per_sm = 8;
  const int64_t blocks = static_cast<int64_t>(sms) * per_sm;
  *block = static_cast<unsigned>(threads);
  *grid = static_cast<unsigned>(rows < blocks ? rows : blocks);
}

// out[n,k] = W[n,k] + scale * sum_j A[k,j] B[j,n]   (LoRAAdapter::merge_weights, src/training/adapter.rs:315-354:
// base + scaling * (A B)^T for a base weight stored [out, in]).  One thread per 4 consecutive k of one n; A rows
// and the B column are read through the read-only cache, the product is accumulated in float32.
template <typename T>
__global__ void merge_weights_kernel(const T* __restrict__ W, const float* __restrict__ A, const float* __restrict__ B,
                                     T* __restrict__ out, int K, int N, int r, float scale) {
  const int64_t total = static_cast<int64_t>(N) * ((K + 3) / 4);
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int kq = static_cast<int>(idx % ((K + 3) / 4));
    const int n = static_cast<int>(idx / ((K + 3) / 4));
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int j = 0; j < r; ++j) {
      const float b = __ldg(B + static_cast<int64_t>(j) * N + n);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int k = kq * 4 + e;
        if (k < K) acc[e] = fmaf(__ldg(A + static_cast<int64_t>(k) * r + j), b, acc[e]);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = kq * 4 + e;
      if (k < K) {
        const int64_t o = static_cast<int64_t>(n) * K + k;
        out[o] = from_f32<T>(to_f32(W[o]) + scale * acc[e]);
      }
    }
  }
}

__global__ void count_valid_kernel(const int32_t* __restrict__ targets, int64_t M, int V, int32_t* __restrict__ count) {
  __shared__ int red[32];
  int c = 0;
  for (int64_t i = threadIdx.x; i < M; i += blockDim.x) c += (targets[i] >= 0 && targets[i] < V) ? 1 : 0;
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    *count = t;
  }
}

// loss[0] = sum(nll) / count, loss[1] = sum(nll); serial tree in fixed order (one block).
__global__ void reduce_nll_kernel(const float* __restrict__ nll, int64_t M, const int32_t* __restrict__ count,
                                  float* __restrict__ loss) {
  __shared__ double red[1024];
  double acc = 0.0;
  for (int64_t i = threadIdx.x; i < M; i += blockDim.x) acc += static_cast<double>(nll[i]);
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int o = blockDim.x / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    loss[1] = static_cast<float>(red[0]);
    loss[0] = static_cast<float>(red[0] / static_cast<double>(max(1, *count)));
  }
}

int grid_for(int64_t work_items, int threads, int sm_count) {
  int64_t g = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sm_count) * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace
}  // namespace mcb

using namespace mcb;

#define MCB_DTYPE_SWITCH(dtype, CALL)                                    \
  if ((dtype) == MCB_F32) { using T = float; CALL; }                     \
  else if ((dtype) == MCB_BF16) { using T = __nv_bfloat16; CALL; }       \
  else return fail(MCB_ERR_UNSUPPORTED, "dtype %d", (dtype));

extern "C" int mcb_embedding_fwd(const int32_t* ids, const void* table, void* out, int64_t M, int64_t H, int64_t vocab,
                                 int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_embedding_fwd");
  if (!ids || !table || !out) return fail(MCB_ERR_NULL, "embedding_fwd: null pointer");
  if (M <= 0 || H <= 0 || vocab <= 0 || M > 0x7fffffff) return fail(MCB_ERR_SHAPE, "embedding_fwd: bad shape");
  if (!current_device_state()) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MCB_DTYPE_SWITCH(dtype, (embedding_fwd_kernel<T><<<(unsigned)M, 128, 0, st>>>(ids, (const T*)table, (T*)out, M, (int)H, (int)vocab)));
  MCB_CHECK_LAUNCH("embedding_fwd");
  return MCB_OK;
}

extern "C" int mcb_rope_relayout_qkv(void* fused, void* q, void* k, void* v, int64_t B, int64_t S, int64_t Hq, int64_t Hk, int64_t d,
                                     float theta, int inverse, int64_t token_pitch, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_rope_relayout_qkv");
  if (!fused || !q || !k || !v) return fail(MCB_ERR_NULL, "rope_relayout_qkv: null pointer");
  if (B <= 0 || S <= 0 || Hq <= 0 || Hk <= 0 || d <= 0 || d % 2 != 0)
    return fail(MCB_ERR_SHAPE, "rope_relayout_qkv: bad shape (head_dim must be even)");
  const int64_t width = (Hq + 2 * Hk) * d;
  if (token_pitch == 0) token_pitch = width;
  if (token_pitch < width)
    return fail(MCB_ERR_SHAPE, "rope_relayout_qkv: %lld + 2 x %lld heads of %lld do not fit a row of %lld", (long long)Hq, (long long)Hk,
                (long long)d, (long long)token_pitch);
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  const int64_t half = d / 2;
  const int vec_n = dtype == MCB_F32 ? 4 : 8;
  if (dtype != MCB_F32 && dtype != MCB_BF16) return fail(MCB_ERR_UNSUPPORTED, "rope_relayout_qkv: dtype %d", dtype);
  if (!(half % vec_n == 0 && aligned16(fused) && aligned16(q) && aligned16(k) && aligned16(v) && token_pitch % vec_n == 0)) {
    // shapes the vector kernel does not take: the three single calls (same arithmetic)
    const void* src[3] = {inverse ? q : fused, inverse ? k : fused, inverse ? v : fused};
    void* dst[3] = {inverse ? fused : q, inverse ? fused : k, inverse ? fused : v};
    const int64_t H[3] = {Hq, Hk, Hk}, off[3] = {0, Hq * d, (Hq + Hk) * d};
    for (int g = 0; g < 3; ++g)
      if (int rc = mcb_rope_relayout_ex(src[g], dst[g], B, S, H[g], d, theta, g < 2 ? 1 : 0, inverse, token_pitch, off[g], dtype, stream))
        return rc;
    return MCB_OK;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(B * S * (half / vec_n), 128, ds->sm_count);
  MCB_DTYPE_SWITCH(dtype, ({
    RopeSegment<T> s0{static_cast<T*>(q), static_cast<int>(Hq), 0, 1};
    RopeSegment<T> s1{static_cast<T*>(k), static_cast<int>(Hk), Hq * d, 1};
    RopeSegment<T> s2{static_cast<T*>(v), static_cast<int>(Hk), (Hq + Hk) * d, 0};
    rope_relayout_qkv_kernel<T><<<grid, 128, 0, st>>>(static_cast<T*>(fused), s0, s1, s2, (int)B, (int)S, (int)d, theta, inverse, token_pitch);
  }));
  MCB_CHECK_LAUNCH("rope_relayout_qkv");
  return MCB_OK;
}

extern "C" int mcb_rope_relayout_ex(const void* src, void* dst, int64_t B, int64_t S, int64_t H, int64_t d, float theta,
                                    int rotate, int inverse, int64_t token_pitch, int64_t col_offset, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_rope_relayout");
  if (!src || !dst) return fail(MCB_ERR_NULL, "rope_relayout: null pointer");
  if (B <= 0 || S <= 0 || H <= 0 || d <= 0 || d % 2 != 0) return fail(MCB_ERR_SHAPE, "rope_relayout: bad shape (head_dim must be even)");
  if (token_pitch == 0) token_pitch = H * d;
  if (col_offset < 0 || col_offset + H * d > token_pitch)
    return fail(MCB_ERR_SHAPE, "rope_relayout: %lld heads x %lld at column %lld do not fit a row of %lld", (long long)H, (long long)d,
                (long long)col_offset, (long long)token_pitch);
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t half = d / 2;
  const int vec_n = dtype == MCB_F32 ? 4 : 8;
  if (half % vec_n == 0 && aligned16(src) && aligned16(dst) && token_pitch % vec_n == 0 && col_offset % vec_n == 0) {
    const int grid = grid_for(B * S * (half / vec_n), 128, ds->sm_count);
    MCB_DTYPE_SWITCH(dtype, (rope_relayout_kernel<T><<<grid, 128, 0, st>>>((const T*)src, (T*)dst, (int)B, (int)S, (int)H, (int)d, theta, rotate, inverse, token_pitch, col_offset)));
  } else {
    const int grid = grid_for(B * S * H * half, 256, ds->sm_count);
    MCB_DTYPE_SWITCH(dtype, (rope_relayout_scalar_kernel<T><<<grid, 256, 0, st>>>((const T*)src, (T*)dst, (int)B, (int)S, (int)H, (int)d, theta, rotate, inverse, token_pitch, col_offset)));
  }
  MCB_CHECK_LAUNCH("rope_relayout");
  return MCB_OK;
}

extern "C" int mcb_rope_relayout(const void* src, void* dst, int64_t B, int64_t S, int64_t H, int64_t d, float theta,
                                 int rotate, int inverse, int dtype, void* stream) {
  return mcb_rope_relayout_ex(src, dst, B, S, H, d, theta, rotate, inverse, 0, 0, dtype, stream);
}

extern "C" int mcb_swiglu_fwd(const void* gate, const void* up, void* out, int64_t n, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_swiglu_fwd");
  if (!gate || !up || !out) return fail(MCB_ERR_NULL, "swiglu_fwd: null pointer");
  if (n <= 0 || n % 8 != 0) return fail(MCB_ERR_SHAPE, "swiglu_fwd: element count must be a positive multiple of 8");
  if (!aligned16(gate) || !aligned16(up) || !aligned16(out)) return fail(MCB_ERR_ALIGN, "swiglu_fwd: 16-byte alignment");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n / 4, 256, ds->sm_count);
  MCB_DTYPE_SWITCH(dtype, (swiglu_fwd_kernel<T><<<grid, 256, 0, st>>>((const T*)gate, (const T*)up, (T*)out, n)));
  MCB_CHECK_LAUNCH("swiglu_fwd");
  return MCB_OK;
}

extern "C" int mcb_swiglu_bwd(const void* gate, const void* up, const void* dout, void* dgate, void* dup, int64_t n,
                              int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_swiglu_bwd");
  if (!gate || !up || !dout || !dgate || !dup) return fail(MCB_ERR_NULL, "swiglu_bwd: null pointer");
  if (n <= 0 || n % 8 != 0) return fail(MCB_ERR_SHAPE, "swiglu_bwd: element count must be a positive multiple of 8");
  if (!aligned16(gate) || !aligned16(up) || !aligned16(dout) || !aligned16(dgate) || !aligned16(dup))
    return fail(MCB_ERR_ALIGN, "swiglu_bwd: 16-byte alignment");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n / 4, 256, ds->sm_count);
  MCB_DTYPE_SWITCH(dtype, (swiglu_bwd_kernel<T><<<grid, 256, 0, st>>>((const T*)gate, (const T*)up, (const T*)dout, (T*)dgate, (T*)dup, n)));
  MCB_CHECK_LAUNCH("swiglu_bwd");
  return MCB_OK;
}

extern "C" int mcb_add(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_add");
  if (!a || !b || !out) return fail(MCB_ERR_NULL, "add: null pointer");
  if (n <= 0) return fail(MCB_ERR_SHAPE, "add: element count must be positive");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n / 4 + 1, 256, ds->sm_count);
  if (n % 8 != 0 || !aligned16(a) || !aligned16(b) || !aligned16(out)) {
    MCB_DTYPE_SWITCH(dtype, (add_scalar_kernel<T><<<grid, 256, 0, st>>>((const T*)a, (const T*)b, (T*)out, n)));
  } else {
    MCB_DTYPE_SWITCH(dtype, (add_kernel<T><<<grid, 256, 0, st>>>((const T*)a, (const T*)b, (T*)out, n)));
  }
  MCB_CHECK_LAUNCH("add");
  return MCB_OK;
}

extern "C" int mcb_mul(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_mul");
  if (!a || !b || !out) return fail(MCB_ERR_NULL, "mul: null pointer");
  if (n <= 0) return fail(MCB_ERR_SHAPE, "mul: element count must be positive");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n, 256, ds->sm_count);
  MCB_DTYPE_SWITCH(dtype, (mul_kernel<T><<<grid, 256, 0, st>>>((const T*)a, (const T*)b, (T*)out, n, 0.0f, 0)));
  MCB_CHECK_LAUNCH("mul");
  return MCB_OK;
}

// Inverted dropout with a counter-based generator: element i of the call is kept when the 24 high bits of
// splitmix64(seed, offset + i), read as a fraction of one, are >= p.  The mask depends on (seed, offset + i) only,
// so the same call on the upstream gradient is the backward pass, whatever the launch shape.
__device__ __forceinline__ bool dropout_keep(uint64_t seed, uint64_t index, float p) {
  uint64_t z = seed ^ (index * 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return static_cast<float>(z >> 40) * (1.0f / 16777216.0f) >= p;
}
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n, float p, float keep_scale, uint64_t seed,
                               uint64_t offset) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    out[i] = dropout_keep(seed, offset + static_cast<uint64_t>(i), p) ? from_f32<T>(to_f32(x[i]) * keep_scale) : from_f32<T>(0.0f);
}

extern "C" int mcb_dropout(const void* x, void* out, int64_t n, float p, uint64_t seed, uint64_t offset, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_dropout");
  if (!x || !out) return fail(MCB_ERR_NULL, "dropout: null pointer");
  if (n <= 0) return fail(MCB_ERR_SHAPE, "dropout: element count must be positive");
  if (!(p >= 0.0f && p < 1.0f)) return fail(MCB_ERR_SHAPE, "dropout: probability %g is not in [0, 1)", static_cast<double>(p));
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n, 256, ds->sm_count);
  const float keep_scale = 1.0f / (1.0f - p);
  MCB_DTYPE_SWITCH(dtype, (dropout_kernel<T><<<grid, 256, 0, st>>>((const T*)x, (T*)out, n, p, keep_scale, seed, offset)));
  MCB_CHECK_LAUNCH("dropout");
  return MCB_OK;
}

extern "C" int mcb_mul_scalar(const void* a, void* out, int64_t n, float value, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_mul_scalar");
  if (!a || !out) return fail(MCB_ERR_NULL, "mul_scalar: null pointer");
  if (n <= 0) return fail(MCB_ERR_SHAPE, "mul_scalar: element count must be positive");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n, 256, ds->sm_count);
  MCB_DTYPE_SWITCH(dtype, (mul_kernel<T><<<grid, 256, 0, st>>>((const T*)a, (const T*)a, (T*)out, n, value, 1)));
  MCB_CHECK_LAUNCH("mul_scalar");
  return MCB_OK;
}

extern "C" int mcb_cross_entropy(void* logits, const int32_t* targets, float* nll, int32_t* count, float* loss,
                                 int64_t M, int64_t V, int write_grad, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_cross_entropy");
  if (!logits || !targets || !nll || !count || !loss) return fail(MCB_ERR_NULL, "cross_entropy: null pointer");
  if (M <= 0 || V <= 0 || M > 0x7fffffff || V > 0x7fffffff) return fail(MCB_ERR_SHAPE, "cross_entropy: bad shape");
  if (!current_device_state()) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  count_valid_kernel<<<1, 1024, 0, st>>>(targets, M, (int)V, count);
  MCB_CHECK_LAUNCH("count_valid");
  unsigned grid = 0, block = 0;
  cross_entropy_launch_shape(M, V, &grid, &block);
  MCB_DTYPE_SWITCH(dtype, (cross_entropy_kernel<T><<<grid, block, 0, st>>>((T*)logits, targets, nll, count, M, (int)V, write_grad)));
  MCB_CHECK_LAUNCH("cross_entropy");
  reduce_nll_kernel<<<1, 1024, 0, st>>>(nll, M, count, loss);
  MCB_CHECK_LAUNCH("reduce_nll");
  return MCB_OK;
}

// The three stages of mcb_cross_entropy as separate calls, so that the logits can be produced, consumed and
// discarded a chunk of tokens at a time (the [tokens, vocabulary] matrix of the whole batch never exists).
extern "C" int mcb_cross_entropy_count(const int32_t* targets, int32_t* count, int64_t M, int64_t V, void* stream) {
  MCB_NVTX_RANGE("mcb_cross_entropy_count");
  if (!targets || !count) return fail(MCB_ERR_NULL, "cross_entropy_count: null pointer");
  if (M <= 0 || V <= 0 || M > 0x7fffffff || V > 0x7fffffff) return fail(MCB_ERR_SHAPE, "cross_entropy_count: bad shape");
  if (!current_device_state()) return MCB_ERR_NOT_INIT;
  count_valid_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(targets, M, (int)V, count);
  MCB_CHECK_LAUNCH("count_valid");
  return MCB_OK;
}

extern "C" int mcb_cross_entropy_chunk(void* logits, const int32_t* targets, float* nll, const int32_t* count, int64_t rows,
                                       int64_t V, int write_grad, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_cross_entropy_chunk");
  if (!logits || !targets || !nll || !count) return fail(MCB_ERR_NULL, "cross_entropy_chunk: null pointer");
  if (rows <= 0 || V <= 0 || rows > 0x7fffffff || V > 0x7fffffff) return fail(MCB_ERR_SHAPE, "cross_entropy_chunk: bad shape");
  if (!current_device_state()) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned grid = 0, block = 0;
  cross_entropy_launch_shape(rows, V, &grid, &block);
  MCB_DTYPE_SWITCH(dtype, (cross_entropy_kernel<T><<<grid, block, 0, st>>>((T*)logits, targets, nll, count, rows, (int)V, write_grad)));
  MCB_CHECK_LAUNCH("cross_entropy");
  return MCB_OK;
}

extern "C" int mcb_cross_entropy_finish(const float* nll, const int32_t* count, float* loss, int64_t M, void* stream) {
  MCB_NVTX_RANGE("mcb_cross_entropy_finish");
  if (!nll || !count || !loss) return fail(MCB_ERR_NULL, "cross_entropy_finish: null pointer");
  if (M <= 0 || M > 0x7fffffff) return fail(MCB_ERR_SHAPE, "cross_entropy_finish: bad shape");
  if (!current_device_state()) return MCB_ERR_NOT_INIT;
  reduce_nll_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(nll, M, count, loss);
  MCB_CHECK_LAUNCH("reduce_nll");
  return MCB_OK;
}

extern "C" int mcb_lora_merge_weights(const void* W, const float* A, const float* B, void* out, int64_t K, int64_t N,
                                      int64_t r, float scale, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_lora_merge_weights");
  if (!W || !A || !B || !out) return fail(MCB_ERR_NULL, "lora_merge_weights: null pointer");
  if (K <= 0 || N <= 0 || r <= 0 || K > 0x7fffffff || N > 0x7fffffff || r > 0x7fffffff)
    return fail(MCB_ERR_SHAPE, "lora_merge_weights: K=%lld N=%lld r=%lld", (long long)K, (long long)N, (long long)r);
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(N * ((K + 3) / 4), 256, ds->sm_count);
  MCB_DTYPE_SWITCH(dtype, (merge_weights_kernel<T><<<grid, 256, 0, st>>>((const T*)W, A, B, (T*)out, (int)K, (int)N, (int)r, scale)));
  MCB_CHECK_LAUNCH("merge_weights");
  return MCB_OK;
}
