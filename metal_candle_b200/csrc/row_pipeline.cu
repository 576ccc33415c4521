// RMSNorm / softmax row kernels fed by bulk asynchronous copies (cp.async.bulk + mbarrier).
//
// The register kernels of row_kernels.cu can only keep as many bytes in flight as their registers hold,
// which on B200 is not enough to cover HBM latency at 6.5 TB/s.  Here the bytes in flight live in shared
// memory instead: a producer thread streams tiles of W consecutive rows (one row per consumer warp) of
// every input into a ring of stages with cp.async.bulk.shared.global (completion counted on an mbarrier),
// W consumer warps each take one row of the tile out of shared memory, reduce with warp shuffles only, and
// store the result straight to global memory with 16-byte stores.  The consumers are bound by instruction
// issue, not by memory, so the forward kernels read a row from shared memory ONCE into registers (rows of up
// to 256 vectors), do their arithmetic two lanes at a time (fma/mul/add .f32x2) and, for RMSNorm, take the
// weight as float32 from a shared-memory copy made once per CTA; wider rows stream from shared memory twice.
// Two CTAs per SM with up to ~100 KB of stages each keep ~100-200 KB in flight per SM.
//
// Causal softmax rows are copied only up to the query position (rounded up to 16 bytes), so the masked
// part of the scores is never read from HBM.
//
// Every mbarrier wait is bounded; on expiry the CTA records a code in the device status word and leaves.
#include "common.cuh"
#include "umma_ptx.cuh"

namespace mcb {
namespace rowpipe {
using namespace umma;

enum Op { kRmsFwd = 0, kRmsBwd = 1, kSmFwd = 2, kSmBwd = 3 };

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 100 * 1024;

struct Params {
  const void* in0;   // x (rms), x (softmax fwd), y (softmax bwd)
  const void* in1;   // dy (backward ops) or null
  const void* w;     // rmsnorm weight or null
  void* out;         // y / dx
  const void* res;   // rms bwd: [rows, D] added to dx (a second gradient of the same tensor), or null
  float* rstd;       // rms fwd, optional
  float* dw_part;    // rms bwd with dw: [gridDim.x][D] partial sums
  int64_t rows;
  int D, nvec, row_bytes;
  int stages, n_streams;
  int wpr;           // consumer warps per row (1; 2 or 4 for the rmsnorm backward of wide rows)
  int causal_seq;
  float eps, scale;
  int* status;
  uint32_t stage_bytes, bar_off;
  uint32_t w_off;    // float32 copy of the rmsnorm weight in shared memory, 0 = none (no weight, or streamed forward)
};

// 2^x by the special-function unit (ex2.approx.ftz): x <= 0 here, -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}


// ---- two-lane float32 arithmetic (fma.rn.f32x2 and friends) ----
__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// This lane's vectors lane, lane+32, ... of a row in shared memory, kept as they are (16 bytes each); vectors
// at or beyond nv read as `fill`.
template <typename T, int KMAX>
__device__ __forceinline__ void load_row(const uint8_t* s0, int lane, int nv, Vec16<T> (&v)[KMAX], float fill) {
  using V = Vec16<T>;
  float ff[V::N];
#pragma unroll
  for (int j = 0; j < V::N; ++j) ff[j] = fill;
  V fv;
  fv.from_float(ff);
#pragma unroll
  for (int k = 0; k < KMAX; ++k) {
    const int vi = lane + 32 * k;
    if (vi < nv) v[k].raw = reinterpret_cast<const decltype(fv.raw)*>(s0)[vi];
    else v[k].raw = fv.raw;
  }
}

// bytes of a causal row that are needed: columns 0..q, rounded up to 16 bytes
__device__ __forceinline__ uint32_t causal_bytes(int q, int elem_bytes, int row_bytes) {
  uint32_t b = (static_cast<uint32_t>(q + 1) * elem_bytes + 15u) & ~15u;
  return b < static_cast<uint32_t>(row_bytes) ? b : static_cast<uint32_t>(row_bytes);
}

// Two CTAs per SM wherever the registers allow it without heavy spilling (a 9-warp CTA pair needs <= 96
// registers per thread, a 17-warp pair <= 56); the wide register-resident forms run one CTA per SM.
__host__ __device__ constexpr int rowpipe_min_blocks(int op, int w, int elems_per_lane) {
  if (op == kRmsFwd) return elems_per_lane > 0 ? 2 : 1;
  if (op == kSmFwd) return (elems_per_lane > 0 && (elems_per_lane <= 32 || w <= 8)) ? 2 : 1;
  if (op == kRmsBwd) return (w <= 8 && elems_per_lane <= 32) ? 2 : 1;
  return w <= 8 ? 2 : 1;
}

// KMAX > 0: a lane owns vectors lane, lane+32, ... (KMAX of them) of every row and keeps them in registers —
// the row itself (forward ops) or the dw sums (rmsnorm backward with dw).  KMAX == 0: rows of any width,
// streamed from shared memory twice.
template <typename T, int OP, int W, int KMAX>
__global__ void __launch_bounds__((W + 1) * 32, rowpipe_min_blocks(OP, W, KMAX * Vec16<T>::N))
rowpipe_kernel(const Params p) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  constexpr bool kTwoIn = (OP == kRmsBwd || OP == kSmBwd);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = base + p.bar_off, empty0 = full0 + 8 * kMaxStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + p.bar_off + 16 * kMaxStages);
  __shared__ float2 xch[16][4];   // per row of a tile: the partial sums of the warps that share it

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, W); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  const float* wsm = nullptr;
  if constexpr ((OP == kRmsFwd && KMAX > 0) || OP == kRmsBwd) {
    if (p.w_off != 0) {
      float* wd = reinterpret_cast<float*>(gen_base + p.w_off);
      for (int c = threadIdx.x; c < p.D; c += blockDim.x) wd[c] = to_f32(static_cast<const T*>(p.w)[c]);
      wsm = wd;
    }
  }
  __syncthreads();

  const int R = W / p.wpr;   // rows per tile
  const int64_t n_tiles = (p.rows + R - 1) / R;
  const uint32_t stream_bytes = static_cast<uint32_t>(R) * p.row_bytes;

  constexpr bool kDw = (OP == kRmsBwd && KMAX > 0);  // per-lane dw sums kept in registers
  float dwa[kDw ? KMAX : 1][N];
  if constexpr (kDw) {
#pragma unroll
    for (int k = 0; k < KMAX; ++k)
#pragma unroll
      for (int j = 0; j < N; ++j) dwa[k][j] = 0.0f;
  }

  if (warp == W) {
    // ---------------- producer (one warp; lane 0 alone unless rows are copied one by one) ----------------
    int stage = 0;
    uint32_t phase = 0;
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
      bool ok = true;
      if (lane == 0) ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, 51, p.status);
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      const int64_t row0 = t * R;
      const int nrows = static_cast<int>(p.rows - row0 < R ? p.rows - row0 : R);
      const uint32_t fb = full0 + 8 * stage, sb = base + stage * p.stage_bytes;
      const char* g0 = static_cast<const char*>(p.in0) + row0 * p.row_bytes;
      const char* g1 = kTwoIn ? static_cast<const char*>(p.in1) + row0 * p.row_bytes : nullptr;
      if (p.causal_seq > 0) {
        // lane r copies row r of the tile, only up to its query position
        const int q0 = static_cast<int>(row0 % p.causal_seq);  // one division per tile
        int q = q0 + lane;
        if (q >= p.causal_seq) q -= p.causal_seq;              // W <= causal_seq is checked on the host
        const uint32_t b = lane < nrows ? causal_bytes(q, sizeof(T), p.row_bytes) : 0u;
        uint32_t total = b;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (lane == 0) mbar_expect_tx(fb, total * (kTwoIn ? 2u : 1u));
        __syncwarp();
        if (lane < nrows) {
          bulk_load(sb + lane * p.row_bytes, g0 + static_cast<int64_t>(lane) * p.row_bytes, b, fb);
          if (kTwoIn) bulk_load(sb + stream_bytes + lane * p.row_bytes, g1 + static_cast<int64_t>(lane) * p.row_bytes, b, fb);
        }
      } else if (lane == 0) {
        const uint32_t b = static_cast<uint32_t>(nrows) * p.row_bytes;
        mbar_expect_tx(fb, b * (kTwoIn ? 2u : 1u));
        bulk_load(sb, g0, b, fb);
        if (kTwoIn) bulk_load(sb + stream_bytes, g1, b, fb);
      }
      if (++stage == p.stages) { stage = 0; phase ^= 1; }
    }
  } else {
    // ---------------- consumers: warp `warp` owns row `warp` of every tile ----------------
    int stage = 0;
    uint32_t phase = 0;
    const float inv_d = 1.0f / static_cast<float>(p.D);
    const int nvec = p.nvec;
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
      if (!__all_sync(0xffffffffu, mbar_wait(full0 + 8 * stage, phase, abort_flag, 52, p.status))) break;
      const int rit = warp / p.wpr, seg = warp - rit * p.wpr;   // row of the tile, segment of the row
      const int64_t row = t * R + rit;
      if (row < p.rows) {
        const uint8_t* s0 = gen_base + stage * p.stage_bytes + rit * p.row_bytes;
        const uint8_t* s1 = s0 + stream_bytes;
        T* orow = static_cast<T*>(p.out) + row * p.D;
        if constexpr (OP == kRmsFwd && KMAX > 0) {
          V v[KMAX];
          load_row<T, KMAX>(s0, lane, nvec, v, 0.0f);
          float2 acc = f2(0.0f, 0.0f);
#pragma unroll
          for (int k = 0; k < KMAX; ++k) {
            float f[N];
            v[k].to_float(f);
#pragma unroll
            for (int j = 0; j < N; j += 2) acc = __ffma2_rn(f2(f[j], f[j + 1]), f2(f[j], f[j + 1]), acc);
          }
          const float ss = warp_sum(acc.x + acc.y);
          const float rinv = 1.0f / sqrtf(ss * inv_d + p.eps);
          if (p.rstd != nullptr && lane == 0) p.rstd[row] = rinv;
          const float2 r2 = f2(rinv, rinv);
#pragma unroll
          for (int k = 0; k < KMAX; ++k) {
            const int vi = lane + 32 * k;
            if (vi < nvec) {
              float f[N], o[N];
              v[k].to_float(f);
#pragma unroll
              for (int j = 0; j < N; j += 4) {
                float2 a = __fmul2_rn(f2(f[j], f[j + 1]), r2), b = __fmul2_rn(f2(f[j + 2], f[j + 3]), r2);
                if (wsm != nullptr) {
                  const float4 g = *reinterpret_cast<const float4*>(wsm + vi * N + j);
                  a = __fmul2_rn(a, f2(g.x, g.y));
                  b = __fmul2_rn(b, f2(g.z, g.w));
                }
                o[j] = a.x; o[j + 1] = a.y; o[j + 2] = b.x; o[j + 3] = b.y;
              }
              V a;
              a.from_float(o);
              __stcs(reinterpret_cast<decltype(a.raw)*>(orow) + vi, a.raw);
            }
          }
        } else if constexpr (OP == kRmsFwd) {
          float ss = 0.0f;
#pragma unroll 4
          for (int vi = lane; vi < nvec; vi += 32) {
            V a; a.raw = reinterpret_cast<const decltype(a.raw)*>(s0)[vi];
            float f[N]; a.to_float(f);
#pragma unroll
            for (int j = 0; j < N; ++j) ss = fmaf(f[j], f[j], ss);
          }
          ss = warp_sum(ss);
          const float rinv = 1.0f / sqrtf(ss * inv_d + p.eps);
          if (p.rstd != nullptr && lane == 0) p.rstd[row] = rinv;
#pragma unroll 4
          for (int vi = lane; vi < nvec; vi += 32) {
            V a; a.raw = reinterpret_cast<const decltype(a.raw)*>(s0)[vi];
            float f[N]; a.to_float(f);
            if (p.w != nullptr) {
              V wv; wv.raw = __ldg(reinterpret_cast<const decltype(wv.raw)*>(p.w) + vi);
              float g[N]; wv.to_float(g);
#pragma unroll
              for (int j = 0; j < N; ++j) f[j] = f[j] * rinv * g[j];
            } else {
#pragma unroll
              for (int j = 0; j < N; ++j) f[j] *= rinv;
            }
            a.from_float(f);
            __stcs(reinterpret_cast<decltype(a.raw)*>(orow) + vi, a.raw);
          }
        } else if constexpr (OP == kRmsBwd) {
          // pass 1: sum x^2 and sum (dy*w)*x, two lanes of float32 at a time
          // (a row may be shared by p.wpr warps, each with a contiguous segment of its vectors)
          const int vseg = nvec / p.wpr, v_begin = seg * vseg, v_end = v_begin + vseg;
          float2 ss2 = f2(0.0f, 0.0f), gx2 = f2(0.0f, 0.0f);
#pragma unroll 4
          for (int vi = v_begin + lane; vi < v_end; vi += 32) {
            V a, b; a.raw = reinterpret_cast<const decltype(a.raw)*>(s0)[vi];
            b.raw = reinterpret_cast<const decltype(b.raw)*>(s1)[vi];
            float x[N], g[N]; a.to_float(x); b.to_float(g);
#pragma unroll
            for (int j = 0; j < N; j += 4) {
              float2 g0 = f2(g[j], g[j + 1]), g1 = f2(g[j + 2], g[j + 3]);
              if (wsm != nullptr) {
                const float4 ww = *reinterpret_cast<const float4*>(wsm + vi * N + j);
                g0 = __fmul2_rn(g0, f2(ww.x, ww.y));
                g1 = __fmul2_rn(g1, f2(ww.z, ww.w));
              }
              const float2 x0 = f2(x[j], x[j + 1]), x1 = f2(x[j + 2], x[j + 3]);
              ss2 = __ffma2_rn(x0, x0, ss2);
              ss2 = __ffma2_rn(x1, x1, ss2);
              gx2 = __ffma2_rn(g0, x0, gx2);
              gx2 = __ffma2_rn(g1, x1, gx2);
            }
          }
          float ss = warp_sum(ss2.x + ss2.y);
          float gx = warp_sum(gx2.x + gx2.y);
          if (p.wpr > 1) {
            // the row's warps exchange their sums through shared memory and add them in segment order
            if (lane == 0) xch[rit][seg] = f2(ss, gx);
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rit), "r"(p.wpr * 32) : "memory");
            ss = 0.0f; gx = 0.0f;
            for (int q2 = 0; q2 < p.wpr; ++q2) { ss += xch[rit][q2].x; gx += xch[rit][q2].y; }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rit), "r"(p.wpr * 32) : "memory");
          }
          const float rinv = 1.0f / sqrtf(ss * inv_d + p.eps);
          const float c = gx * rinv * inv_d;
          const float2 r2 = f2(rinv, rinv), nc2 = f2(-c, -c);
          // pass 2: dx = rinv * (dy*w - xhat*c), dw += dy*xhat
          const T* rrow = p.res != nullptr ? static_cast<const T*>(p.res) + row * p.D : nullptr;
          auto body = [&](int vi, float* dw_slot) {
            V a, b, rr; a.raw = reinterpret_cast<const decltype(a.raw)*>(s0)[vi];
            b.raw = reinterpret_cast<const decltype(b.raw)*>(s1)[vi];
            // the residual comes straight from global memory (read once, streaming), issued ahead of the arithmetic
            if (rrow != nullptr) rr.raw = __ldcs(reinterpret_cast<const decltype(rr.raw)*>(rrow) + vi);
            float x[N], g[N], o[N]; a.to_float(x); b.to_float(g);
#pragma unroll
            for (int j = 0; j < N; j += 2) {
              const float2 gg = f2(g[j], g[j + 1]);
              const float2 xh = __fmul2_rn(f2(x[j], x[j + 1]), r2);
              if (dw_slot != nullptr) {
                const float2 d = __ffma2_rn(gg, xh, f2(dw_slot[j], dw_slot[j + 1]));
                dw_slot[j] = d.x; dw_slot[j + 1] = d.y;
              }
              float2 gw = gg;
              if (wsm != nullptr) gw = __fmul2_rn(gg, *reinterpret_cast<const float2*>(wsm + vi * N + j));
              const float2 u = __fmul2_rn(__ffma2_rn(xh, nc2, gw), r2);
              o[j] = u.x; o[j + 1] = u.y;
            }
            if (rrow != nullptr) {
              float rf[N];
              rr.to_float(rf);
#pragma unroll
              for (int j = 0; j < N; ++j) o[j] += rf[j];
            }
            a.from_float(o);
            __stcs(reinterpret_cast<decltype(a.raw)*>(orow) + vi, a.raw);
          };
          auto body_res = [&](int vi, const V& rr) {
            V a, b; a.raw = reinterpret_cast<const decltype(a.raw)*>(s0)[vi];
            b.raw = reinterpret_cast<const decltype(b.raw)*>(s1)[vi];
            float x[N], g[N], o[N], rf[N]; a.to_float(x); b.to_float(g); rr.to_float(rf);
#pragma unroll
            for (int j = 0; j < N; j += 2) {
              const float2 xh = __fmul2_rn(f2(x[j], x[j + 1]), r2);
              float2 gw = f2(g[j], g[j + 1]);
              if (wsm != nullptr) gw = __fmul2_rn(gw, *reinterpret_cast<const float2*>(wsm + vi * N + j));
              const float2 u = __ffma2_rn(__ffma2_rn(xh, nc2, gw), r2, f2(rf[j], rf[j + 1]));
              o[j] = u.x; o[j + 1] = u.y;
            }
            a.from_float(o);
            __stcs(reinterpret_cast<decltype(a.raw)*>(orow) + vi, a.raw);
          };
          if constexpr (kDw) {
#pragma unroll
            for (int k = 0; k < KMAX; ++k) {
              const int vi = v_begin + lane + 32 * k;
              if (vi < v_end) body(vi, dwa[k]);
            }
          } else if (rrow != nullptr) {
            // the residual vectors of the whole row segment are requested before pass 2 touches the first one,
            // so that their global-memory latency is paid once per row, not once per vector
            constexpr int kRes = 2;
            for (int v0 = v_begin + lane; v0 < v_end; v0 += 32 * kRes) {
              V rr[kRes];
#pragma unroll
              for (int k = 0; k < kRes; ++k)
                if (v0 + 32 * k < v_end) rr[k].raw = __ldcs(reinterpret_cast<const decltype(rr[k].raw)*>(rrow) + v0 + 32 * k);
#pragma unroll
              for (int k = 0; k < kRes; ++k)
                if (v0 + 32 * k < v_end) body_res(v0 + 32 * k, rr[k]);
            }
          } else {
            for (int vi = v_begin + lane; vi < v_end; vi += 32) body(vi, nullptr);
          }
        } else if constexpr (OP == kSmFwd && KMAX > 0) {
          const bool causal = p.causal_seq > 0;
          const int q = causal ? static_cast<int>(row % p.causal_seq) : p.D;  // last kept column
          const int nv_keep = causal ? min(nvec, q / N + 1) : nvec;
          const int vq = causal ? q / N : -1;  // only the vector that holds column q has masked elements behind it
          const float sc = p.scale * kLog2e;   // work in base-2 logits
          V v[KMAX];
          load_row<T, KMAX>(s0, lane, nv_keep, v, -INFINITY);
          float m = -INFINITY;
#pragma unroll
          for (int k = 0; k < KMAX; ++k) {
            float f[N];
            v[k].to_float(f);
            if (lane + 32 * k == vq) {
#pragma unroll
              for (int j = 0; j < N; ++j)
                if (vq * N + j > q) f[j] = -INFINITY;
            }
#pragma unroll
            for (int j = 0; j < N; ++j) m = fmaxf(m, f[j]);
          }
          m = warp_max(m) * sc;  // sc > 0: max commutes with the scaling
          // Up to 32 elements per lane keep their exponentials in registers; wider rows compute them twice
          // (once for the sum, once for the output) rather than spill.
          constexpr bool kKeep = KMAX * N <= 32;
          float e[kKeep ? KMAX : 1][N];
          float inv = 0.0f;
          const float2 sc2 = f2(sc, sc), nm2 = f2(-m, -m);
          auto exps = [&](int k, float (&o)[N]) {
            float f[N];
            v[k].to_float(f);
            if (lane + 32 * k == vq) {
#pragma unroll
              for (int j = 0; j < N; ++j)
                if (vq * N + j > q) f[j] = -INFINITY;
            }
#pragma unroll
            for (int j = 0; j < N; j += 2) {
              const float2 a = __ffma2_rn(f2(f[j], f[j + 1]), sc2, nm2);
              o[j] = fast_exp2(a.x);
              o[j + 1] = fast_exp2(a.y);
            }
          };
          if (m != -INFINITY) {
            float2 acc0 = f2(0.0f, 0.0f), acc1 = f2(0.0f, 0.0f);
#pragma unroll
            for (int k = 0; k < KMAX; ++k) {
              float t[N];
              exps(k, t);
#pragma unroll
              for (int j = 0; j < N; j += 4) {
                acc0 = __fadd2_rn(acc0, f2(t[j], t[j + 1]));
                acc1 = __fadd2_rn(acc1, f2(t[j + 2], t[j + 3]));
              }
              if constexpr (kKeep) {
#pragma unroll
                for (int j = 0; j < N; ++j) e[k][j] = t[j];
              }
            }
            const float ssum = warp_sum((acc0.x + acc0.y) + (acc1.x + acc1.y));
            inv = ssum > 0.0f ? 1.0f / ssum : 0.0f;
          }
          const float2 i2 = f2(inv, inv);
#pragma unroll
          for (int k = 0; k < KMAX; ++k) {
            const int vi = lane + 32 * k;
            if (vi < nvec) {
              float t[N], o[N];
              if (m == -INFINITY) {
#pragma unroll
                for (int j = 0; j < N; ++j) t[j] = 0.0f;
              } else if constexpr (kKeep) {
#pragma unroll
                for (int j = 0; j < N; ++j) t[j] = e[k][j];
              } else {
                exps(k, t);
              }
#pragma unroll
              for (int j = 0; j < N; j += 2) {
                const float2 a = __fmul2_rn(f2(t[j], t[j + 1]), i2);
                o[j] = a.x; o[j + 1] = a.y;
              }
              V a;
              a.from_float(o);
              __stcs(reinterpret_cast<decltype(a.raw)*>(orow) + vi, a.raw);
            }
          }
        } else if constexpr (OP == kSmFwd) {
          const int q = p.causal_seq > 0 ? static_cast<int>(row % p.causal_seq) : p.D;  // last kept column (one division per row per warp)
          const int nv_keep = p.causal_seq > 0 ? min(nvec, q / N + 1) : nvec;
          const float sc = p.scale * kLog2e;  // work in base-2 logits
          // pass 1: row maximum (cheap), pass 2: sum of 2^(x - max) with independent partial sums
          float m = -INFINITY;
#pragma unroll 4
          for (int vi = lane; vi < nv_keep; vi += 32) {
            V a; a.raw = reinterpret_cast<const decltype(a.raw)*>(s0)[vi];
            float f[N]; a.to_float(f);
#pragma unroll
            for (int j = 0; j < N; ++j) m = fmaxf(m, (vi * N + j <= q) ? f[j] : -INFINITY);
          }
          m = warp_max(m) * sc;  // sc > 0: max commutes with the scaling
          float s = 0.0f;
          if (m != -INFINITY) {
            float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
            for (int vi = lane; vi < nv_keep; vi += 32) {
              V a; a.raw = reinterpret_cast<const decltype(a.raw)*>(s0)[vi];
              float f[N]; a.to_float(f);
#pragma unroll
              for (int j = 0; j < N; ++j)
                part[j & 3] += (vi * N + j <= q) ? fast_exp2(fmaf(f[j], sc, -m)) : 0.0f;
            }
            s = (part[0] + part[1]) + (part[2] + part[3]);
          }
          s = warp_sum(s);
          const float inv = s > 0.0f ? 1.0f / s : 0.0f;
          const float mref = (m == -INFINITY) ? 0.0f : m;
#pragma unroll 4
          for (int vi = lane; vi < nvec; vi += 32) {
            float f[N];
            if (vi < nv_keep) {
              V a; a.raw = reinterpret_cast<const decltype(a.raw)*>(s0)[vi];
              a.to_float(f);
#pragma unroll
              for (int j = 0; j < N; ++j) f[j] = (vi * N + j <= q) ? fast_exp2(fmaf(f[j], sc, -mref)) * inv : 0.0f;
            } else {
#pragma unroll
              for (int j = 0; j < N; ++j) f[j] = 0.0f;
            }
            V a; a.from_float(f);
            __stcs(reinterpret_cast<decltype(a.raw)*>(orow) + vi, a.raw);
          }
        } else {  // kSmBwd
          const int q = p.causal_seq > 0 ? static_cast<int>(row % p.causal_seq) : p.D;
          const int nv_keep = p.causal_seq > 0 ? min(nvec, q / N + 1) : nvec;
          float dot = 0.0f;
#pragma unroll 4
          for (int vi = lane; vi < nv_keep; vi += 32) {
            V a, b; a.raw = reinterpret_cast<const decltype(a.raw)*>(s0)[vi];
            b.raw = reinterpret_cast<const decltype(b.raw)*>(s1)[vi];
            float y[N], g[N]; a.to_float(y); b.to_float(g);
#pragma unroll
            for (int j = 0; j < N; ++j) dot = fmaf((vi * N + j <= q) ? y[j] : 0.0f, g[j], dot);
          }
          dot = warp_sum(dot);
#pragma unroll 4
          for (int vi = lane; vi < nvec; vi += 32) {
            float o[N];
            if (vi < nv_keep) {
              V a, b; a.raw = reinterpret_cast<const decltype(a.raw)*>(s0)[vi];
              b.raw = reinterpret_cast<const decltype(b.raw)*>(s1)[vi];
              float y[N], g[N]; a.to_float(y); b.to_float(g);
#pragma unroll
              for (int j = 0; j < N; ++j) o[j] = (vi * N + j <= q) ? y[j] * (g[j] - dot) * p.scale : 0.0f;
            } else {
#pragma unroll
              for (int j = 0; j < N; ++j) o[j] = 0.0f;
            }
            V a; a.from_float(o);
            __stcs(reinterpret_cast<decltype(a.raw)*>(orow) + vi, a.raw);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * stage);
      if (++stage == p.stages) { stage = 0; phase ^= 1; }
    }
  }

  if constexpr (kDw) {
    // Sum the W warps' dw accumulators in warp order through shared memory (the stage ring is idle now:
    // every load that was issued has been consumed), then write this CTA's partial row.
    __syncthreads();
    float* red = reinterpret_cast<float*>(gen_base);
    if (warp < W) {
      const int rit = warp / p.wpr, seg = warp - rit * p.wpr;
      const int vseg = p.nvec / p.wpr, v_begin = seg * vseg, v_end = v_begin + vseg;
#pragma unroll
      for (int k = 0; k < KMAX; ++k) {
        const int vi = v_begin + lane + 32 * k;
        if (vi < v_end) {
#pragma unroll
          for (int j = 0; j < N; ++j) red[rit * p.D + vi * N + j] = dwa[k][j];
        }
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < p.D; c += blockDim.x) {
      float s = 0.0f;
      for (int w = 0; w < R; ++w) s += red[w * p.D + c];
      p.dw_part[static_cast<int64_t>(blockIdx.x) * p.D + c] = s;
    }
  }
  if (*abort_flag != 0) {
    for (int k = 0; k < 200; ++k) __nanosleep(1000);
  }
}

template <typename T, int OP, int W, int KMAX>
int launch_one(const Params& p, int grid, size_t smem, cudaStream_t st) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(rowpipe_kernel<T, OP, W, KMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (227 * 1024) / 2 - 1024);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(rowpipe_kernel)");
    // ask for the largest shared-memory carve-out so that two CTAs of ~100 KB fit an SM
    e = cudaFuncSetAttribute(rowpipe_kernel<T, OP, W, KMAX>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(rowpipe_kernel carve-out)");
    attr_set[dev] = true;
  }
  rowpipe_kernel<T, OP, W, KMAX><<<grid, (W + 1) * 32, smem, st>>>(p);
  MCB_CHECK_LAUNCH("rowpipe_kernel");
  return MCB_OK;
}

template <typename T, int OP, int KMAX>
int launch_w(int W, const Params& p, int grid, size_t smem, cudaStream_t st) {
  switch (W) {
    case 16: return launch_one<T, OP, 16, KMAX>(p, grid, smem, st);
    case 8: return launch_one<T, OP, 8, KMAX>(p, grid, smem, st);
    case 4: return launch_one<T, OP, 4, KMAX>(p, grid, smem, st);
    case 2: return launch_one<T, OP, 2, KMAX>(p, grid, smem, st);
  }
  return fail(MCB_ERR_UNSUPPORTED, "rowpipe: W=%d", W);
}

// Returns MCB_OK when the pipelined kernel was launched, 1 when the shape does not fit it (the caller
// then uses the register kernels), or an error.
template <typename T>
int try_launch(int op, const void* in0, const void* in1, const void* w, void* out, float* rstd, float* dw_part,
               int* dw_blocks, int64_t rows, int64_t D, float eps, int causal_seq, float scale, const DeviceState* ds,
               cudaStream_t st, const void* res) {
  constexpr int N = Vec16<T>::N;
  if (D % N != 0 || D > (1 << 20)) return 1;
  if (res != nullptr && (op != kRmsBwd || !aligned16(res))) return 1;
  if (!aligned16(in0) || !aligned16(out) || (in1 && !aligned16(in1)) || (w && !aligned16(w))) return 1;
  const int n_streams = (op == kRmsBwd || op == kSmBwd) ? 2 : 1;
  const int64_t row_bytes = D * static_cast<int64_t>(sizeof(T));
  // RMSNorm with a weight keeps a float32 copy of it in shared memory, taken out of the stage budget
  const int64_t w_bytes = (w != nullptr && (op == kRmsFwd || op == kRmsBwd)) ? D * 4 : 0;
  // two CTAs per SM: each may take half of the 227 KB less the 1 KB the system keeps per CTA
  const int64_t per_cta = (227 * 1024) / 2 - 1024 - 1024;
  const int64_t budget = w_bytes + kSmemBudget <= per_cta ? kSmemBudget : per_cta - w_bytes;
  if (budget < kSmemBudget / 2) return 1;
  int W = 0, stages = 0;
  for (int cand : {16, 8, 4, 2}) {
    const int64_t stage_bytes = cand * row_bytes * n_streams;
    const int s = static_cast<int>(budget / stage_bytes);
    if (s >= 3) { W = cand; stages = s > kMaxStages ? kMaxStages : s; break; }
  }
  if (W == 0 && op == kRmsBwd && budget / (2 * row_bytes * n_streams) >= 2) {
    // very wide rows: two rows per stage, two stages, four warps per row (below)
    W = 2;
    stages = 2;
  }
  // One warp per row only pays while enough warps fit: forward ops (one input stream, more arithmetic per
  // byte) want at least 8 rows per tile, backward ops at least 4; wider rows go to the register kernels.
  const int nvec = static_cast<int>(D / N);
  // The RMSNorm backward of very wide rows (only 2 rows fit a stage) gives every row 4 warps, each with a
  // contiguous segment of the row; the warps of a row exchange their two sums through shared memory.
  // (Measured: at 4 rows per stage, 2 warps per row are slower than one.)
  int wpr = 1, R = W;   // warps per row, rows per tile
  if (op == kRmsBwd && W == 2 && nvec % 4 == 0) {
    wpr = 4;
    W = 8;
  }
  if (W < (n_streams == 1 ? 8 : 4) || rows < 4 * R) return 1;
  if (causal_seq > 0 && causal_seq < W) return 1;
  int kmax = 0;
  if (op == kRmsFwd || op == kSmFwd) {
    const int need = (nvec + 31) / 32;  // register-resident rows of up to 8 vectors per lane
    kmax = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : need <= 8 ? 8 : 0;
    if (kmax * N >= 32 && W > 8) {
      // 32 or more elements per lane: eight rows per tile and two CTAs per SM keep the register file from spilling
      W = 8;
      const int sN = static_cast<int>(budget / (W * row_bytes * n_streams));
      stages = sN > kMaxStages ? kMaxStages : sN;
    }
  }
  if (op != kRmsBwd) R = W;
  if (dw_part != nullptr) {
    const int need = (nvec / wpr + 31) / 32;
    kmax = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : need <= 8 ? 8 : need <= 16 ? 16 : 0;
    if (kmax == 0) return 1;
    if (static_cast<int64_t>(R) * D * 4 > static_cast<int64_t>(stages) * R * row_bytes * n_streams) return 1;
  }
  Params p;
  p.in0 = in0; p.in1 = in1; p.w = w; p.out = out; p.res = res; p.rstd = rstd; p.dw_part = dw_part;
  p.rows = rows; p.D = static_cast<int>(D); p.nvec = nvec; p.row_bytes = static_cast<int>(row_bytes);
  p.stages = stages; p.n_streams = n_streams; p.wpr = wpr; p.causal_seq = causal_seq; p.eps = eps; p.scale = scale;
  p.status = ds->status_word;
  p.stage_bytes = static_cast<uint32_t>(R * row_bytes * n_streams);
  p.bar_off = (static_cast<uint32_t>(stages) * p.stage_bytes + 127u) & ~127u;
  size_t smem = p.bar_off + 16 * kMaxStages + 16 + 128;
  p.w_off = 0;
  if (w != nullptr && ((op == kRmsFwd && kmax > 0) || op == kRmsBwd)) {
    p.w_off = static_cast<uint32_t>((smem + 15) & ~static_cast<size_t>(15));
    smem = p.w_off + static_cast<size_t>(D) * 4 + 128;
  }
  const int64_t n_tiles = (rows + R - 1) / R;
  int grid = 2 * ds->sm_count;
  if (grid > n_tiles) grid = static_cast<int>(n_tiles);
  if (dw_blocks) *dw_blocks = grid;
#define MCB_RP(OPC, KM) return launch_w<T, OPC, KM>(W, p, grid, smem, st)
  switch (op) {
    case kRmsFwd:
      switch (kmax) {
        case 0: MCB_RP(kRmsFwd, 0);
        case 1: MCB_RP(kRmsFwd, 1);
        case 2: MCB_RP(kRmsFwd, 2);
        case 4: MCB_RP(kRmsFwd, 4);
        case 8: MCB_RP(kRmsFwd, 8);
      }
      break;
    case kSmFwd:
      switch (kmax) {
        case 0: MCB_RP(kSmFwd, 0);
        case 1: MCB_RP(kSmFwd, 1);
        case 2: MCB_RP(kSmFwd, 2);
        case 4: MCB_RP(kSmFwd, 4);
        case 8: MCB_RP(kSmFwd, 8);
      }
      break;
    case kSmBwd: MCB_RP(kSmBwd, 0);
    case kRmsBwd:
      switch (kmax) {
        case 0: MCB_RP(kRmsBwd, 0);
        case 1: MCB_RP(kRmsBwd, 1);
        case 2: MCB_RP(kRmsBwd, 2);
        case 4: MCB_RP(kRmsBwd, 4);
        case 8: MCB_RP(kRmsBwd, 8);
        case 16: MCB_RP(kRmsBwd, 16);
      }
  }
#undef MCB_RP
  return 1;
}

template int try_launch<float>(int, const void*, const void*, const void*, void*, float*, float*, int*, int64_t, int64_t,
                               float, int, float, const DeviceState*, cudaStream_t, const void*);
template int try_launch<__nv_bfloat16>(int, const void*, const void*, const void*, void*, float*, float*, int*, int64_t,
                                       int64_t, float, int, float, const DeviceState*, cudaStream_t, const void*);

}  // namespace rowpipe
}  // namespace mcb
