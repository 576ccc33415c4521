// Causal grouped-query attention, fused:  O = softmax(scale * Q K^T + causal mask) V  without ever writing
// the [S, S] score matrix (src/models/transformer.rs:257-285 computes scores, adds the mask, applies softmax
// and multiplies by V as four separate tensor ops over a materialised [B, H, S, S] tensor).
//
// Layouts (bf16, head dimension 64, S a multiple of 128); nb = batch * kv_heads, G query heads per kv head:
//   Q  [nb, G*S, 64]   row g*S + s is query head g, position s           O  the same
//   K, V  [nb, S, 64]
//   LSE [nb, G*S] float32: log-sum-exp of the scaled scores of a row (natural log), kept for the backward
//
// Forward: persistent CTAs (two per SM) walk over (128 queries, head) items, heavy ones first; key blocks of 64.
// Warp 0 streams K / V tiles by TMA into a four-stage ring, warp 1 issues the tensor-core MMAs (S = Q K^T into
// one of two tensor-memory buffers, two blocks ahead of the softmax; then O += P V with P read from tensor
// memory), warps 2-5 do the online softmax with one query row per thread: read S from tensor memory (once),
// write P (bf16 pairs) back into tensor memory; O accumulates in tensor memory and is rescaled there
// (tcgen05.ld / tcgen05.st) only when a row maximum has grown by more than 2^8.
//
// Backward: two kernels, each recomputes the probabilities from Q, K and the saved log-sum-exp, so that no
// [S, S] tensor is ever stored and nothing is accumulated with atomics:
//   dq kernel   persistent like the forward, key blocks of 64, one query row per thread:
//               S = Q K^T (double-buffered, ahead) and dP = dO V^T into tensor memory, P = exp(scale*S - lse),
//               dS = P (dP - delta) with delta = rowsum(dO * O), dS (bf16 pairs) written over the half of dP already
//               read, dQ += dS K accumulated in tensor memory with dS as a tensor-memory A operand.
//               It also writes delta and lse*log2(e) for the second kernel.
//   dkv kernel  one CTA per (128 keys, kv head), steps of 64 queries over the heads of the group, one key row
//               per thread pair: S^T = K Q^T, dP^T = V dO^T, P^T and dS^T back into tensor memory (A operands),
//               dV += P^T dO and dK += dS^T Q accumulated in tensor memory over all steps (which also sums over
//               the group).
// Operands whose reduction index is the slow one in memory (V in P V, K in dS K, dO and Q in the dK / dV
// products) are used as they lie, as N-major B operands (instruction-descriptor bit 16); nothing is transposed.
// Every wait is bounded; on expiry the CTA records a code in the device status word and leaves.
#include <cuda.h>
#include <string.h>

#include "lora_internal.cuh"
#include "umma_ptx.cuh"

namespace mcb {
namespace attn {
using namespace umma;
namespace {

constexpr int kD = 64;        // head dimension
constexpr int kBQ = 128;      // queries per CTA
constexpr int kBK = 64;       // keys per block
constexpr int kThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

constexpr uint32_t kQBytes = kBQ * kD * 2;   // 16 KB
constexpr uint32_t kKBytes = kBK * kD * 2;   // 8 KB
constexpr uint32_t kPBytes = kBQ * kBK * 2;  // 16 KB
// shared memory map (from the 1024-aligned base)
constexpr uint32_t kOffQ = 0;
constexpr int kFwdStages = 4;                         // K / V ring: a load has three blocks' time to arrive
constexpr uint32_t kOffK = kOffQ + kQBytes;
constexpr uint32_t kOffV = kOffK + kFwdStages * kKBytes;
constexpr uint32_t kOffBar = kOffV + kFwdStages * kKBytes;
constexpr uint32_t kFwdSmem = kOffBar + 256 + 1024;

struct FwdParams {
  int S, G, NB;
  int HKV, o_tok;   // o_tok != 0: O is token-major [batch*S, HKV*G*64] (nb = batch*HKV + kv head), else like Q
  float sc;  // scale * log2(e)
  __nv_bfloat16* O;
  float* lse;
  int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Work item t (heavy first): query block qb = nqb-1 - t / (G*nb), then head g and batch*kv-head nb.
struct FwdTile {
  int qb, g, nb, nkb;
  int64_t qrow0;
};
__device__ __forceinline__ FwdTile fwd_tile(const FwdParams& p, int t) {
  FwdTile w;
  const int per_qb = p.G * p.NB;
  const int r = t % per_qb;
  w.qb = p.S / kBQ - 1 - t / per_qb;
  w.g = r % p.G;
  w.nb = r / p.G;
  w.nkb = 2 * w.qb + 2;  // key blocks of 64 up to and including the diagonal
  w.qrow0 = (static_cast<int64_t>(w.nb) * p.G + w.g) * p.S + static_cast<int64_t>(w.qb) * kBQ;
  return w;
}

// Where the 64 values of (kv-head index nb, head g of its group, position s) start in O / dO, in elements, and the
// two tile coordinates (column, row) of the same place for a tiled copy.
__device__ __forceinline__ int64_t o_offset(int S, int G, int HKV, int o_tok, int nb, int g, int s) {
  if (!o_tok) return ((static_cast<int64_t>(nb) * G + g) * S + s) * kD;
  const int b = nb / HKV, kvh = nb - b * HKV;
  return ((static_cast<int64_t>(b) * S + s) * (HKV * G) + kvh * G + g) * kD;
}
__device__ __forceinline__ void o_coords(int S, int G, int HKV, int o_tok, int nb, int g, int s, int& col, int& row) {
  if (!o_tok) { col = 0; row = (nb * G + g) * S + s; return; }
  const int b = nb / HKV, kvh = nb - b * HKV;
  col = (kvh * G + g) * kD;
  row = b * S + s;
}

__global__ void __launch_bounds__(kThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmVt, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Persistent: a CTA walks over work items (128 queries of one head) and carries its rings and barrier phases
  // from one to the next, so that the next item's Q / K / V loads and first S products run under this item's
  // last blocks and its write-out.  n below is the running number of a key block over all items of this CTA.
  // S is double-buffered in tensor memory and runs two blocks ahead of the softmax; P is double-buffered in
  // tensor memory as well (this block's exponentials are written under the previous block's P V).
  const uint32_t q_full = base + kOffBar, q_free = q_full + 8, o_free = q_free + 8, kv_full0 = o_free + 8;
  const uint32_t kv_empty0 = kv_full0 + 8 * kFwdStages;
  const uint32_t s_full0 = kv_empty0 + 8 * kFwdStages, p_ready0 = s_full0 + 16, pv_done0 = p_ready0 + 16;
  const uint32_t s_free0 = pv_done0 + 16, tmem_slot = s_free0 + 16, abort_addr = tmem_slot + 4;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_addr - base));

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_free, 1);
    mbar_init(o_free, 4);
    for (int s = 0; s < kFwdStages; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(s_full0 + 8 * s, 1); mbar_init(p_ready0 + 8 * s, 4); mbar_init(pv_done0 + 8 * s, 1); mbar_init(s_free0 + 8 * s, 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // S buffers at columns 0 and 64, O at 128, the two P buffers (bf16 pairs: 32 columns each) at 192 and 224
  const uint32_t tO = tmem_base + 128, tP0 = tmem_base + 192;
  const int n_tiles = (p.S / kBQ) * p.G * p.NB;

  if (warp == 0) {
    if (lane == 0) {
      int st = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x, ++it) {
        const FwdTile w = fwd_tile(p, t);
        // the previous item's last S product has read Q
        if (it > 0) ok = mbar_wait(q_free, (it - 1) & 1, abort_flag, 69, p.status);
        if (!ok) break;
        mbar_expect_tx(q_full, kQBytes);
        tma_load_2d(base + kOffQ, &tmQ, q_full, 0, static_cast<int>(w.qrow0));
        for (int j = 0; j < w.nkb; ++j) {
          ok = mbar_wait(kv_empty0 + 8 * st, ph ^ 1, abort_flag, 71, p.status);
          if (!ok) break;
          mbar_expect_tx(kv_full0 + 8 * st, 2 * kKBytes);
          tma_load_2d(base + kOffK + st * kKBytes, &tmK, kv_full0 + 8 * st, 0, w.nb * p.S + j * kBK);
          tma_load_2d(base + kOffV + st * kKBytes, &tmVt, kv_full0 + 8 * st, 0, w.nb * p.S + j * kBK);
          if (++st == kFwdStages) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kBK);  // M = 128, N = 64 for both products
      bool ok = true;
      int it = 0;
      uint32_t n0 = 0;            // running number of this item's block 0
      int sst = 0;                // ring stage and phase of the next block to get its S product
      uint32_t sph = 0;
      int pst = 0;                // ring stage of the next block to get its P V product
      // S_j = Q K_j^T for block j of the current item (running number n) into tensor-memory buffer n & 1; the
      // buffer is free once the softmax warps have read block n - 2 into registers (s_free)
      auto issue_s = [&](uint32_t n, bool last) -> bool {
        if (n >= 2 && !mbar_wait(s_free0 + 8 * (n & 1), ((n - 2) >> 1) & 1, abort_flag, 70, p.status)) return false;
        if (!mbar_wait(kv_full0 + 8 * sst, sph, abort_flag, 75, p.status)) return false;
        tcgen05_fence_after();
        const uint32_t tS = tmem_base + (n & 1) * 64;
#pragma unroll
        for (int k4 = 0; k4 < kD / 16; ++k4)
          umma_bf16(tS, desc_sw128(base + kOffQ + k4 * 32), desc_sw128(base + kOffK + sst * kKBytes + k4 * 32), idesc,
                    k4 != 0 ? 1u : 0u);
        umma_commit(s_full0 + 8 * (n & 1));
        if (last) umma_commit(q_free);   // Q may be replaced by the next item's
        if (++sst == kFwdStages) { sst = 0; sph ^= 1; }
        return true;
      };
      for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x, ++it) {
        const FwdTile w = fwd_tile(p, t);
        ok = mbar_wait(q_full, it & 1, abort_flag, 72, p.status);
        for (int j = 0; ok && j < 2; ++j) ok = issue_s(n0 + j, j == w.nkb - 1);   // nkb >= 2
        for (int j = 0; ok && j < w.nkb; ++j) {
          const uint32_t n = n0 + j;
          if (j + 2 < w.nkb) {
            ok = issue_s(n + 2, j + 2 == w.nkb - 1);
            if (!ok) break;
          }
          ok = mbar_wait(p_ready0 + 8 * (n & 1), (n >> 1) & 1, abort_flag, 74, p.status);
          // the first product of an item overwrites O: the previous item's write-out must have read it
          if (ok && j == 0 && it > 0) ok = mbar_wait(o_free, (it - 1) & 1, abort_flag, 68, p.status);
          if (!ok) break;
          tcgen05_fence_after();
          // O += P_j V_j   (A = P [128 x 64 keys] in tensor memory, 16 keys = 8 columns; B = the V tile as it lies,
          // [64 keys x 64 d]: N-major, 16 keys further = two 8-row groups of 1024 bytes)
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4)
            umma_bf16_ts(tO, tP0 + (n & 1) * 32 + k4 * 8,
                         desc_sw128_mn(base + kOffV + pst * kKBytes + k4 * 2048, kKBytes, 1024), idesc | (1u << 16),
                         (j | k4) != 0 ? 1u : 0u);
          umma_commit(pv_done0 + 8 * (n & 1));
          umma_commit(kv_empty0 + 8 * pst);
          if (++pst == kFwdStages) pst = 0;
        }
        n0 += static_cast<uint32_t>(w.nkb);
      }
    }
  } else {
    // ---------------- online softmax, one query row per thread ----------------
    // O accumulates in tensor memory (the P V product adds onto it).  The running maximum a row's exponentials
    // are taken against is only raised when the true maximum has grown by more than 2^8 over it; then the
    // warp rescales its 32 rows of O in tensor memory.  Between such events nothing but S is touched.
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    uint32_t n0 = 0;
    for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
      const FwdTile w = fwd_tile(p, t);
      const int qpos = w.qb * kBQ + row;
      float m = -INFINITY, l = 0.0f;   // m: the maximum in use (base-2 logits)
      for (int j = 0; j < w.nkb; ++j) {
        const uint32_t n = n0 + j;
        ok = __all_sync(0xffffffffu, mbar_wait(s_full0 + 8 * (n & 1), (n >> 1) & 1, abort_flag, 76, p.status));
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tS = tmem_base + (n & 1) * 64;
        const int key0 = j * kBK;
        const bool diag = key0 + kBK - 1 > w.qb * kBQ;  // some element of this block may lie above the diagonal
        // the row's 64 scores of this block, read from tensor memory once (four loads in flight, one wait)
        uint32_t sv[4][16];
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) tmem_ld_x16(tS + lane_addr + 16 * c4, sv[c4]);
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free0 + 8 * (n & 1));   // the buffer may take block n + 2
        if (diag) {
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4)
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (key0 + 16 * c4 + e > qpos) sv[c4][e] = 0xff800000u;   // -inf
        }
        // row maximum: four independent chains of three-input maxima (8 instructions each)
        float mxc[4];
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          float tmx = fmaxf(__uint_as_float(sv[c4][0]), __uint_as_float(sv[c4][1]));
#pragma unroll
          for (int e = 2; e < 16; e += 2) tmx = fmax3(tmx, __uint_as_float(sv[c4][e]), __uint_as_float(sv[c4][e + 1]));
          mxc[c4] = tmx;
        }
        const float mx = fmaxf(fmax3(mxc[0], mxc[1], mxc[2]), mxc[3]);
        const float m_true = fmaxf(m, mx * p.sc);  // key 0 is never masked, so this is finite from block 0 on
        const bool raise = m_true > m + 8.0f;       // block 0: m = -inf, always
        if (n >= 2) {
          // the P V product of block n-2 has read the P buffer that this block overwrites
          ok = __all_sync(0xffffffffu, mbar_wait(pv_done0 + 8 * (n & 1), ((n - 2) >> 1) & 1, abort_flag, 77, p.status));
          if (!ok) break;
        }
        if (__any_sync(0xffffffffu, raise)) {
          const float alpha = ex2(m - m_true);   // rows that did not ask get alpha <= 1 as well and move their maximum
          if (j > 0) {
            // every P V product so far must have landed before O is rescaled
            ok = __all_sync(0xffffffffu, mbar_wait(pv_done0 + 8 * ((n - 1) & 1), ((n - 1) >> 1) & 1, abort_flag, 79, p.status));
            if (!ok) break;
            tcgen05_fence_after();
#pragma unroll
            for (int c = 0; c < kD; c += 16) {
              uint32_t v[16];
              tmem_ld_x16(tO + lane_addr + c, v);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
              tmem_st_x16(tO + lane_addr + c, v);
            }
            tmem_st_wait();
          }
          l *= alpha;
          m = m_true;
        }
        // P = 2^(s*sc - m) (masked scores are -inf and give 0), row sum, bf16 pairs into this block's P buffer in
        // tensor memory (the A operand of the P V product: no trip through shared memory)
        // (packed two-wide FMA and add: the special-function unit's 64 exponentials are the only per-element work)
        float2 lsa = f2(0.0f, 0.0f), lsb = f2(0.0f, 0.0f);
        const float2 sc2 = f2(p.sc, p.sc), nm2 = f2(-m, -m);
        const uint32_t tP = tP0 + lane_addr + (n & 1) * 32;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t pw[16];
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const uint32_t* q4 = &sv[2 * c2 + (e >> 4)][e & 15];
            const float2 ta = __ffma2_rn(f2(__uint_as_float(q4[0]), __uint_as_float(q4[1])), sc2, nm2);
            const float2 tb = __ffma2_rn(f2(__uint_as_float(q4[2]), __uint_as_float(q4[3])), sc2, nm2);
            const float2 pa = f2(ex2(ta.x), ex2(ta.y)), pb = f2(ex2(tb.x), ex2(tb.y));
            lsa = __fadd2_rn(lsa, pa);
            lsb = __fadd2_rn(lsb, pb);
            pw[e >> 1] = pack_bf16(pa.x, pa.y);
            pw[(e >> 1) + 1] = pack_bf16(pb.x, pb.y);
          }
          tmem_st_x16(tP + 16 * c2, pw);
        }
        tmem_st_wait();
        l += (lsa.x + lsa.y) + (lsb.x + lsb.y);
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready0 + 8 * (n & 1));
      }
      if (!ok) break;
      // write-out: the item's last P V product has landed
      const uint32_t nl = n0 + static_cast<uint32_t>(w.nkb) - 1;
      ok = __all_sync(0xffffffffu, mbar_wait(pv_done0 + 8 * (nl & 1), (nl >> 1) & 1, abort_flag, 78, p.status));
      if (!ok) break;
      tcgen05_fence_after();
      const float inv = 1.0f / l;
      __nv_bfloat16* orow = p.O + o_offset(p.S, p.G, p.HKV, p.o_tok, w.nb, w.g, w.qb * kBQ + row);
      uint32_t ov[4][16];
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) tmem_ld_x16(tO + lane_addr + 16 * c4, ov[c4]);
      tmem_ld_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);   // the next item's products may overwrite O
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t ow[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2)
          ow[e >> 1] = pack_bf16(__uint_as_float(ov[c4][e]) * inv, __uint_as_float(ov[c4][e + 1]) * inv);
        *reinterpret_cast<uint4*>(orow + 16 * c4) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        *reinterpret_cast<uint4*>(orow + 16 * c4 + 8) = make_uint4(ow[4], ow[5], ow[6], ow[7]);
      }
      if (p.lse != nullptr) p.lse[w.qrow0 + row] = (m + lg2(l)) * kLn2;
      n0 += static_cast<uint32_t>(w.nkb);
    }
  }

  __syncwarp();
  if (*abort_flag != 0) {
    for (int k = 0; k < 200; ++k) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}


// ---------------------------------------------------------------------------------------------------------
// backward, part 1: dQ (and delta, lse2 for part 2)
// ---------------------------------------------------------------------------------------------------------
constexpr uint32_t kDqOffQ = 0;
constexpr uint32_t kDqOffDO = kDqOffQ + kQBytes;
constexpr int kDqStages = 4;
constexpr uint32_t kDqOffStage = kDqOffDO + kQBytes;     // stages of a K and a V tile (8 KB each)
constexpr uint32_t kDqStageBytes = 2 * kKBytes;
constexpr uint32_t kDqOffBar = kDqOffStage + kDqStages * kDqStageBytes;
constexpr uint32_t kDqSmem = kDqOffBar + 256 + 1024;

struct BwdParams {
  int S, G, NB;
  int HKV, o_tok;   // o_tok != 0: O and dO are token-major [batch*S, HKV*G*64], else laid out like Q
  float sc;     // scale * log2(e)
  float scale;
  const __nv_bfloat16* O;
  const __nv_bfloat16* dO;
  const float* lse;
  float* delta;   // [nb, G*S]
  float* lse2;    // [nb, G*S]: lse * log2(e)
  __nv_bfloat16* dQ;
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  int* status;
};

// Persistent like the forward: a CTA walks over (query block, head, batch) items, heavy first, and carries its
// rings and barrier phases along (n = running number of a key block over all items of the CTA).
// Tensor memory (256 columns): S double-buffered at 0 and 64 (the next blocks' Q K^T run under this block's
// arithmetic), dP at 128, dQ at 192.  dS (bf16 pairs, 32 columns) is written over the first half of dP, which has
// been read by then, and is the A operand of dQ += dS K straight from tensor memory.
__global__ void __launch_bounds__(kThreads, 2)
attn_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
               const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t q_full = base + kDqOffBar, q_free = q_full + 8, dq_full = q_free + 8, dq_free = dq_full + 8;
  const uint32_t kv_full0 = dq_free + 8, kv_empty0 = kv_full0 + 8 * kDqStages;
  const uint32_t s_full0 = kv_empty0 + 8 * kDqStages, s_free0 = s_full0 + 16;
  const uint32_t dp_full = s_free0 + 16, ds_ready = dp_full + 8, tmem_slot = ds_ready + 8, abort_addr = tmem_slot + 4;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_addr - base));

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_free, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 4);
    for (int s = 0; s < kDqStages; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(s_full0 + 8 * s, 1); mbar_init(s_free0 + 8 * s, 4); }
    mbar_init(dp_full, 1);
    mbar_init(ds_ready, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t tDP = tmem_base + 128, tDQ = tmem_base + 192;
  FwdParams tp;   // the item order of the forward
  tp.S = p.S; tp.G = p.G; tp.NB = p.NB;
  const int n_tiles = (p.S / kBQ) * p.G * p.NB;

  if (warp == 0) {
    if (lane == 0) {
      int st = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x, ++it) {
        const FwdTile w = fwd_tile(tp, t);
        // the previous item's last S and dP products have read Q and dO
        if (it > 0) ok = mbar_wait(q_free, (it - 1) & 1, abort_flag, 80, p.status);
        if (!ok) break;
        mbar_expect_tx(q_full, 2 * kQBytes);
        tma_load_2d(base + kDqOffQ, &tmQ, q_full, 0, static_cast<int>(w.qrow0));
        int dcol, drow;
        o_coords(p.S, p.G, p.HKV, p.o_tok, w.nb, w.g, w.qb * kBQ, dcol, drow);
        tma_load_2d(base + kDqOffDO, &tmdO, q_full, dcol, drow);
        for (int j = 0; j < w.nkb; ++j) {
          ok = mbar_wait(kv_empty0 + 8 * st, ph ^ 1, abort_flag, 81, p.status);
          if (!ok) break;
          const uint32_t sb = base + kDqOffStage + st * kDqStageBytes;
          mbar_expect_tx(kv_full0 + 8 * st, kDqStageBytes);
          tma_load_2d(sb, &tmK, kv_full0 + 8 * st, 0, w.nb * p.S + j * kBK);
          tma_load_2d(sb + kKBytes, &tmV, kv_full0 + 8 * st, 0, w.nb * p.S + j * kBK);
          if (++st == kDqStages) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kBK);
      bool ok = true;
      int it = 0;
      uint32_t n0 = 0;
      int sst = 0;                // ring stage and phase of the next block to get its S product
      uint32_t sph = 0;
      int dst = 0;                // ring stage of the next block to get its dP and dQ products
      auto issue_s = [&](uint32_t n) -> bool {
        if (n >= 2 && !mbar_wait(s_free0 + 8 * (n & 1), ((n - 2) >> 1) & 1, abort_flag, 82, p.status)) return false;
        if (!mbar_wait(kv_full0 + 8 * sst, sph, abort_flag, 83, p.status)) return false;
        tcgen05_fence_after();
        const uint32_t sb = base + kDqOffStage + sst * kDqStageBytes;
#pragma unroll
        for (int k4 = 0; k4 < kD / 16; ++k4)
          umma_bf16(tmem_base + (n & 1) * 64, desc_sw128(base + kDqOffQ + k4 * 32), desc_sw128(sb + k4 * 32), idesc,
                    k4 != 0 ? 1u : 0u);
        umma_commit(s_full0 + 8 * (n & 1));
        if (++sst == kDqStages) { sst = 0; sph ^= 1; }
        return true;
      };
      for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x, ++it) {
        const FwdTile w = fwd_tile(tp, t);
        ok = mbar_wait(q_full, it & 1, abort_flag, 84, p.status);
        for (int j = 0; ok && j < 2; ++j) ok = issue_s(n0 + j);   // nkb >= 2
        for (int j = 0; ok && j < w.nkb; ++j) {
          const uint32_t n = n0 + j;
          const uint32_t sb = base + kDqOffStage + dst * kDqStageBytes;
          // dP_j = dO V_j^T.  Its buffer (and the dS written over it) was last read by the dQ product of block
          // n - 1, issued before this point (the tensor core runs them in order); the V tile arrived with the K
          // tile that S_j has waited for.
#pragma unroll
          for (int k4 = 0; k4 < kD / 16; ++k4)
            umma_bf16(tDP, desc_sw128(base + kDqOffDO + k4 * 32), desc_sw128(sb + kKBytes + k4 * 32), idesc, k4 != 0 ? 1u : 0u);
          umma_commit(dp_full);
          if (j == w.nkb - 1) umma_commit(q_free);   // Q and dO may be replaced by the next item's
          if (j + 2 < w.nkb) {
            ok = issue_s(n + 2);
            if (!ok) break;
          }
          ok = mbar_wait(ds_ready, n & 1, abort_flag, 86, p.status);
          // the first product of an item overwrites dQ: the previous item's write-out must have read it
          if (ok && j == 0 && it > 0) ok = mbar_wait(dq_free, (it - 1) & 1, abort_flag, 87, p.status);
          if (!ok) break;
          tcgen05_fence_after();
          // dQ += dS_j K_j   (A = dS [128 x 64 keys] in tensor memory; B = the K tile as it lies: N-major)
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4)
            umma_bf16_ts(tDQ, tDP + k4 * 8, desc_sw128_mn(sb + k4 * 2048, kKBytes, 1024), idesc | (1u << 16),
                         (j | k4) != 0 ? 1u : 0u);
          umma_commit(kv_empty0 + 8 * dst);
          if (j == w.nkb - 1) umma_commit(dq_full);
          if (++dst == kDqStages) dst = 0;
        }
        n0 += static_cast<uint32_t>(w.nkb);
      }
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    uint32_t n0 = 0;
    int it = 0;
    for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x, ++it) {
      const FwdTile w = fwd_tile(tp, t);
      const int qpos = w.qb * kBQ + row;
      // delta = sum_d dO * O of this row, straight from global memory (once per item)
      float delta = 0.0f;
      {
        const int64_t ooff = o_offset(p.S, p.G, p.HKV, p.o_tok, w.nb, w.g, w.qb * kBQ + row);
        const uint4* o4 = reinterpret_cast<const uint4*>(p.O + ooff);
        const uint4* d4 = reinterpret_cast<const uint4*>(p.dO + ooff);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 a = o4[c], b = d4[c];
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            delta = fmaf(__uint_as_float(aw[e] << 16), __uint_as_float(bw[e] << 16), delta);
            delta = fmaf(__uint_as_float(aw[e] & 0xffff0000u), __uint_as_float(bw[e] & 0xffff0000u), delta);
          }
        }
      }
      const float lse2 = p.lse[w.qrow0 + row] * kLog2e;
      p.delta[w.qrow0 + row] = delta;
      p.lse2[w.qrow0 + row] = lse2;
      const float2 sc2 = f2(p.sc, p.sc), nl2 = f2(-lse2, -lse2), nd2 = f2(-delta, -delta);
      for (int j = 0; j < w.nkb; ++j) {
        const uint32_t n = n0 + j;
        ok = __all_sync(0xffffffffu, mbar_wait(s_full0 + 8 * (n & 1), (n >> 1) & 1, abort_flag, 88, p.status));
        if (!ok) break;
        tcgen05_fence_after();
        const int key0 = j * kBK;
        const bool diag = key0 + kBK - 1 > w.qb * kBQ;
        // the row's 64 scores, read once; P = 2^(s*sc - lse2) takes their place in the registers
        uint32_t sv[4][16];
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) tmem_ld_x16(tmem_base + (n & 1) * 64 + lane_addr + 16 * c4, sv[c4]);
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free0 + 8 * (n & 1));   // the buffer may take block n + 2
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const float2 tt = __ffma2_rn(f2(__uint_as_float(sv[c4][e]), __uint_as_float(sv[c4][e + 1])), sc2, nl2);
            float p0 = ex2(tt.x), p1 = ex2(tt.y);
            if (diag) {
              if (key0 + 16 * c4 + e > qpos) p0 = 0.0f;
              if (key0 + 16 * c4 + e + 1 > qpos) p1 = 0.0f;
            }
            sv[c4][e] = __float_as_uint(p0);
            sv[c4][e + 1] = __float_as_uint(p1);
          }
        }
        // dS = P (dP - delta), bf16 pairs written over the half of dP already read
        ok = __all_sync(0xffffffffu, mbar_wait(dp_full, n & 1, abort_flag, 89, p.status));
        if (!ok) break;
        tcgen05_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t vd[2][16];
          tmem_ld_x16(tDP + lane_addr + 32 * h, vd[0]);
          tmem_ld_x16(tDP + lane_addr + 32 * h + 16, vd[1]);
          tmem_ld_wait();
          uint32_t dw[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const uint32_t* pv = &sv[2 * h + (e >> 4)][e & 15];
            const uint32_t* dv = &vd[e >> 4][e & 15];
            const float2 d2 = __fadd2_rn(f2(__uint_as_float(dv[0]), __uint_as_float(dv[1])), nd2);
            const float2 r2 = __fmul2_rn(f2(__uint_as_float(pv[0]), __uint_as_float(pv[1])), d2);
            dw[e >> 1] = pack_bf16(r2.x, r2.y);
          }
          tmem_st_x16(tDP + lane_addr + 16 * h, dw);
        }
        tmem_st_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_ready);
      }
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(dq_full, it & 1, abort_flag, 90, p.status));
      if (!ok) break;
      tcgen05_fence_after();
      uint32_t qv[4][16];
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) tmem_ld_x16(tDQ + lane_addr + 16 * c4, qv[c4]);
      tmem_ld_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_free);   // the next item's products may overwrite dQ
      __nv_bfloat16* orow = p.dQ + (w.qrow0 + row) * kD;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t ow[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2)
          ow[e >> 1] = pack_bf16(__uint_as_float(qv[c4][e]) * p.scale, __uint_as_float(qv[c4][e + 1]) * p.scale);
        *reinterpret_cast<uint4*>(orow + 16 * c4) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        *reinterpret_cast<uint4*>(orow + 16 * c4 + 8) = make_uint4(ow[4], ow[5], ow[6], ow[7]);
      }
      n0 += static_cast<uint32_t>(w.nkb);
    }
  }

  __syncwarp();
  if (*abort_flag != 0) {
    for (int k = 0; k < 200; ++k) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------
// backward, part 2: dK, dV
// ---------------------------------------------------------------------------------------------------------
// One CTA per SM: 2 control warps + 8 element-wise warps (two per tensor-memory lane quadrant, 32 of the 64 query
// columns each; no row reductions are needed here because the log-sum-exp is known).  Loads are double-buffered,
// S^T / dP^T are double-buffered in tensor memory and so are P^T / dS^T (bf16 pairs, handed to the dV / dK products
// as tensor-memory A operands), so the tensor core computes the next step's S^T, dP^T while the element-wise
// warps work on the current one.
constexpr int kKvThreads = 320;
constexpr uint32_t kKvOffK = 0;                       // K block [128 keys x 64]
constexpr uint32_t kKvOffV = kKvOffK + kQBytes;
constexpr int kKvStages = 4;
constexpr uint32_t kKvOffStage = kKvOffV + kQBytes;   // per stage: Q and dO tiles (8 KB each), then lse2 and delta (256 B each)
constexpr uint32_t kKvStageBytes = 2 * kKBytes + 512;
constexpr uint32_t kKvStageStride = 2 * kKBytes + 1024;
constexpr uint32_t kKvOffBar = kKvOffStage + kKvStages * kKvStageStride;
constexpr uint32_t kKvSmem = kKvOffBar + 256 + 1024;

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__global__ void __launch_bounds__(kKvThreads, 1)
attn_dkv_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t kv_full = base + kKvOffBar, ld_full0 = kv_full + 8, ld_empty0 = ld_full0 + 8 * kKvStages;
  const uint32_t sdp_full0 = ld_empty0 + 8 * kKvStages;
  // pds_ready has one barrier per buffer: an element-wise warp may run one step ahead of the slowest one
  const uint32_t pds_ready0 = sdp_full0 + 16, out_full = pds_ready0 + 16, tmem_slot = out_full + 8, abort_addr = tmem_slot + 4;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_addr - base));

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < kKvStages; ++s) { mbar_init(ld_full0 + 8 * s, 1); mbar_init(ld_empty0 + 8 * s, 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(sdp_full0 + 8 * s, 1); mbar_init(pds_ready0 + 8 * s, 8); }
    mbar_init(out_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // columns: S^T buffers at 0 and 128, dP^T at 64 and 192, dV at 256, dK at 320, then per buffer P^T (32 columns
  // of bf16 pairs) and dS^T (32): 384 / 416 and 448 / 480
  const uint32_t tDV = tmem_base + 256, tDK = tmem_base + 320, tPT0 = tmem_base + 384;

  const int kb = blockIdx.y, nb = blockIdx.x;   // all kv heads of key block 0 (the most query steps) start first
  const int nq = p.S / kBK;                      // query steps of 64 per head
  const int i0 = 2 * kb;                         // first query step that sees this key block
  const int per_head = nq - i0;
  const int nsteps = p.G * per_head;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * kQBytes);
      tma_load_2d(base + kKvOffK, &tmK, kv_full, 0, nb * p.S + kb * kBQ);
      tma_load_2d(base + kKvOffV, &tmV, kv_full, 0, nb * p.S + kb * kBQ);
      for (int t = 0; t < nsteps; ++t) {
        const int st = t % kKvStages;
        const int g = t / per_head, i = i0 + t % per_head;
        if (!mbar_wait(ld_empty0 + 8 * st, ((t / kKvStages) & 1) ^ 1, abort_flag, 91, p.status)) break;
        const int64_t qrow = (static_cast<int64_t>(nb) * p.G + g) * p.S + static_cast<int64_t>(i) * kBK;
        const uint32_t sb = base + kKvOffStage + st * kKvStageStride, fb = ld_full0 + 8 * st;
        mbar_expect_tx(fb, kKvStageBytes);
        tma_load_2d(sb, &tmQ, fb, 0, static_cast<int>(qrow));
        int dcol, drow;
        o_coords(p.S, p.G, p.HKV, p.o_tok, nb, g, i * kBK, dcol, drow);
        tma_load_2d(sb + kKBytes, &tmdO, fb, dcol, drow);
        bulk_load_1d(sb + 2 * kKBytes, p.lse2 + qrow, 256, fb);
        bulk_load_1d(sb + 2 * kKBytes + 256, p.delta + qrow, 256, fb);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kBK);
      // descriptors of the resident K / V block and of stage 0's Q / dO tiles (K-major for S^T and dP^T, as N-major
      // B operands for dV and dK), built once; a stage or a K slice further is one add
      const uint64_t dK = desc_sw128(base + kKvOffK), dV = desc_sw128(base + kKvOffV);
      const uint64_t dQk = desc_sw128(base + kKvOffStage), dQn = desc_sw128_mn(base + kKvOffStage, kKBytes, 1024);
      // S^T = K Q^T, dP^T = V dO^T of step t into tensor-memory buffer t & 1
      auto issue_sdp = [&](int t) {
        const int st = t & 1;
        const uint32_t so = static_cast<uint32_t>(t % kKvStages) * kKvStageStride;
        const uint32_t tS = tmem_base + st * 128, tDP = tS + 64;
        // the two accumulation chains are independent: interleaved, one product's latency hides the other's
#pragma unroll
        for (int k4 = 0; k4 < kD / 16; ++k4) {
          umma_bf16(tS, desc_advance(dK, k4 * 32), desc_advance(dQk, so + k4 * 32), idesc, k4 != 0 ? 1u : 0u);
          umma_bf16(tDP, desc_advance(dV, k4 * 32), desc_advance(dQk, so + kKBytes + k4 * 32), idesc, k4 != 0 ? 1u : 0u);
        }
        umma_commit(sdp_full0 + 8 * st);
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, 92, p.status);
      if (ok) ok = mbar_wait(ld_full0, 0, abort_flag, 93, p.status);
      if (ok) {
        tcgen05_fence_after();
        issue_sdp(0);
      }
      for (int t = 0; ok && t < nsteps; ++t) {
        const int st = t & 1;
        if (t + 1 < nsteps) {
          // buffer (t+1)&1 of tensor memory was last read by the element-wise warps of step t-1, whose
          // pds_ready this thread has already waited for
          ok = mbar_wait(ld_full0 + 8 * ((t + 1) % kKvStages), ((t + 1) / kKvStages) & 1, abort_flag, 93, p.status);
          if (!ok) break;
          tcgen05_fence_after();
          issue_sdp(t + 1);
        }
        ok = mbar_wait(pds_ready0 + 8 * (t & 1), (t >> 1) & 1, abort_flag, 94, p.status);
        if (!ok) break;
        tcgen05_fence_after();
        const int ls = t % kKvStages;
        const uint32_t so = static_cast<uint32_t>(ls) * kKvStageStride;
        // dV += P^T dO, dK += dS^T Q   (A = P^T / dS^T [128 keys x 64 queries] in tensor memory, 16 queries = 8
        // columns; B = the dO / Q tile as it lies, [64 queries x 64 d]: N-major, 16 queries further = two 8-row
        // groups of 1024 bytes)
        const uint32_t acc = t != 0 ? 1u : 0u;
#pragma unroll
        for (int k4 = 0; k4 < kBK / 16; ++k4) {
          umma_bf16_ts(tDV, tPT0 + st * 64 + k4 * 8, desc_advance(dQn, so + kKBytes + k4 * 2048), idesc | (1u << 16),
                       k4 != 0 ? 1u : acc);
          umma_bf16_ts(tDK, tPT0 + st * 64 + 32 + k4 * 8, desc_advance(dQn, so + k4 * 2048), idesc | (1u << 16),
                       k4 != 0 ? 1u : acc);
        }
        umma_commit(ld_empty0 + 8 * ls);
        if (t + 1 == nsteps) umma_commit(out_full);
      }
    }
  } else {
    const int quad = warp & 3;            // tensor-memory lane quadrant of this warp
    const int half = (warp - 2) >> 2;     // which 32 of the 64 query columns
    const int row = quad * 32 + lane;
    const int key = kb * kBQ + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    for (int t = 0; t < nsteps; ++t) {
      const int st = t & 1;
      const int i = i0 + t % per_head;
      ok = __all_sync(0xffffffffu, mbar_wait(sdp_full0 + 8 * st, (t >> 1) & 1, abort_flag, 95, p.status));
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t tS = tmem_base + st * 128 + lane_addr, tDP = tS + 64;
      // this warp's 32 query columns are 16 packed columns of each of P^T and dS^T
      const uint32_t tPT = tPT0 + st * 64 + lane_addr + half * 16;
      uint32_t wp[16], wd[16];
      const float* st_lse2 = reinterpret_cast<const float*>(gen_base + kKvOffStage + (t % kKvStages) * kKvStageStride + 2 * kKBytes);
      const float* st_delta = st_lse2 + 64;
      const int q0 = i * kBK;
      const bool diag = q0 < (kb + 1) * kBQ;   // some query of this step lies before some key of the block
#pragma unroll
      for (int cb = 0; cb < 32; cb += 16) {
        const int c = half * 32 + cb;
        uint32_t vs[16], vd[16];
        tmem_ld_x16(tS + c, vs);
        tmem_ld_x16(tDP + c, vd);
        float l2[16], dl[16];
#pragma unroll
        for (int e = 0; e < 16; e += 4) {
          const float4 a = *reinterpret_cast<const float4*>(st_lse2 + c + e);
          const float4 b = *reinterpret_cast<const float4*>(st_delta + c + e);
          l2[e] = a.x; l2[e + 1] = a.y; l2[e + 2] = a.z; l2[e + 3] = a.w;
          dl[e] = b.x; dl[e + 1] = b.y; dl[e + 2] = b.z; dl[e + 3] = b.w;
        }
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          float p0 = ex2(fmaf(__uint_as_float(vs[e]), p.sc, -l2[e]));
          float p1 = ex2(fmaf(__uint_as_float(vs[e + 1]), p.sc, -l2[e + 1]));
          if (diag) {
            if (key > q0 + c + e) p0 = 0.0f;
            if (key > q0 + c + e + 1) p1 = 0.0f;
          }
          wp[(cb + e) >> 1] = pack_bf16(p0, p1);
          wd[(cb + e) >> 1] = pack_bf16(p0 * (__uint_as_float(vd[e]) - dl[e]), p1 * (__uint_as_float(vd[e + 1]) - dl[e + 1]));
        }
      }
      tmem_st_x16(tPT, wp);
      tmem_st_x16(tPT + 32, wd);
      tmem_st_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready0 + 8 * (t & 1));
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(out_full, 0, abort_flag, 96, p.status));
    if (ok) {
      tcgen05_fence_after();
      const int64_t krow = static_cast<int64_t>(nb) * p.S + key;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* orow = (which == 0 ? p.dV : p.dK) + krow * kD;
        const float f = which == 0 ? 1.0f : p.scale;
#pragma unroll
        for (int cb = 0; cb < 32; cb += 16) {
          const int c = half * 32 + cb;
          uint32_t v[16];
          tmem_ld_x16((which == 0 ? tDV : tDK) + lane_addr + c, v);
          tmem_ld_wait();
          uint32_t w[8];
#pragma unroll
          for (int e = 0; e < 16; e += 2) w[e >> 1] = pack_bf16(__uint_as_float(v[e]) * f, __uint_as_float(v[e + 1]) * f);
          *reinterpret_cast<uint4*>(orow + c) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(orow + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
    }
  }

  __syncwarp();
  if (*abort_flag != 0) {
    for (int k = 0; k < 200; ++k) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D bf16 tensor [outer, inner], 128-byte swizzle, box [box_outer, 64]
int encode(const DeviceState* ds, CUtensorMap* map, const void* ptr, int64_t inner, int64_t outer, int box_outer,
           const char* what) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(inner) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ds->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MCB_ERR_ALIGN, "attention: tensor map for %s rejected (CUresult %d)", what, static_cast<int>(r));
  return MCB_OK;
}

int check_shape(const char* who, int64_t nb, int64_t groups, int64_t seq, int64_t head_dim, int dtype) {
  if (dtype != MCB_BF16) return fail(MCB_ERR_UNSUPPORTED, "%s: bfloat16 only", who);
  if (head_dim != kD) return fail(MCB_ERR_UNSUPPORTED, "%s: head dimension %lld (only 64 is built)", who, (long long)head_dim);
  if (seq <= 0 || seq % kBQ != 0) return fail(MCB_ERR_UNSUPPORTED, "%s: sequence length %lld is not a multiple of 128", who, (long long)seq);
  if (nb <= 0 || groups <= 0 || nb > 65535 || groups > 65535) return fail(MCB_ERR_SHAPE, "%s: nb=%lld groups=%lld", who, (long long)nb, (long long)groups);
  if (nb * groups * seq > 0x7fffff00ll) return fail(MCB_ERR_SHAPE, "%s: more than 2^31 query rows", who);
  return MCB_OK;
}

}  // namespace
}  // namespace attn
}  // namespace mcb

using namespace mcb;

namespace {
inline size_t up1k(size_t v) { return (v + 1023) & ~static_cast<size_t>(1023); }
int set_attrs_once(const void* fn, uint32_t smem, bool* done) {
  if (*done) return MCB_OK;
  MCB_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  MCB_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  *done = true;
  return MCB_OK;
}
}  // namespace

extern "C" size_t mcb_attention_workspace_bytes(int64_t nb, int64_t groups, int64_t seq, int64_t head_dim) {
  if (nb <= 0 || groups <= 0 || seq <= 0 || head_dim <= 0) return 0;
  (void)head_dim;
  const size_t rows = static_cast<size_t>(nb) * groups * seq * 4;
  // backward: delta = rowsum(dO * O) and lse * log2(e), one float32 per query row each; the forward needs none
  return 2 * up1k(rows) + 1024;
}

extern "C" int mcb_attention_causal_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse, int64_t nb,
                                           int64_t groups, int64_t seq, int64_t head_dim, float scale, int dtype,
                                           int64_t kv_heads, int o_token_major, void* workspace, size_t workspace_bytes,
                                           void* stream) {
  MCB_NVTX_RANGE("mcb_attention_causal_fwd_ex");
  using namespace mcb::attn;
  if (!q || !k || !v || !o) return fail(MCB_ERR_NULL, "attention_causal_fwd: q, k, v or o is null");
  if (int rc = check_shape("attention_causal_fwd", nb, groups, seq, head_dim, dtype)) return rc;
  if (o_token_major && (kv_heads <= 0 || nb % kv_heads != 0))
    return fail(MCB_ERR_SHAPE, "attention_causal_fwd: nb=%lld is not a multiple of kv_heads=%lld", (long long)nb, (long long)kv_heads);
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return fail(MCB_ERR_ALIGN, "attention_causal_fwd: 16-byte alignment");
  (void)workspace; (void)workspace_bytes;  // the forward needs no scratch memory
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  static bool attr_set[64] = {};
  int dev = 0;
  MCB_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MCB_ERR_SHAPE, "attention: device %d out of range", dev);
  if (int rc = set_attrs_once(reinterpret_cast<const void*>(attn_fwd_kernel), kFwdSmem, &attr_set[dev])) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap tmQ, tmK, tmVt;
  if (int rc = encode(ds, &tmQ, q, kD, nb * groups * seq, kBQ, "Q")) return rc;
  if (int rc = encode(ds, &tmK, k, kD, nb * seq, kBK, "K")) return rc;
  if (int rc = encode(ds, &tmVt, v, kD, nb * seq, kBK, "V")) return rc;
  FwdParams p;
  p.S = static_cast<int>(seq); p.G = static_cast<int>(groups); p.NB = static_cast<int>(nb);
  p.HKV = o_token_major ? static_cast<int>(kv_heads) : 1; p.o_tok = o_token_major ? 1 : 0;
  p.sc = scale * kLog2e;
  p.O = static_cast<__nv_bfloat16*>(o); p.lse = lse; p.status = ds->status_word;
  // persistent: two CTAs per SM walk over the (query block, head, batch) items, heavy ones first
  const int64_t n_tiles = (seq / kBQ) * groups * nb;
  const int64_t slots = 2 * static_cast<int64_t>(ds->sm_count);
  const unsigned grid = static_cast<unsigned>(n_tiles < slots ? n_tiles : slots);
  attn_fwd_kernel<<<grid, kThreads, kFwdSmem, st>>>(tmQ, tmK, tmVt, p);
  MCB_CHECK_LAUNCH("attn_fwd_kernel");
  return MCB_OK;
}

extern "C" int mcb_attention_causal_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int64_t nb,
                                        int64_t groups, int64_t seq, int64_t head_dim, float scale, int dtype,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  return mcb_attention_causal_fwd_ex(q, k, v, o, lse, nb, groups, seq, head_dim, scale, dtype, 1, 0, workspace,
                                     workspace_bytes, stream);
}

extern "C" int mcb_attention_causal_bwd_ex(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                           const float* lse, void* dq, void* dk, void* dv, int64_t nb, int64_t groups,
                                           int64_t seq, int64_t head_dim, float scale, int dtype, int64_t kv_heads,
                                           int o_token_major, void* workspace, size_t workspace_bytes, void* stream) {
  MCB_NVTX_RANGE("mcb_attention_causal_bwd_ex");
  using namespace mcb::attn;
  if (o_token_major && (kv_heads <= 0 || nb % kv_heads != 0))
    return fail(MCB_ERR_SHAPE, "attention_causal_bwd: nb=%lld is not a multiple of kv_heads=%lld", (long long)nb, (long long)kv_heads);
  if (!q || !k || !v || !o || !dout || !lse || !dq || !dk || !dv)
    return fail(MCB_ERR_NULL, "attention_causal_bwd: a required pointer is null");
  if (int rc = check_shape("attention_causal_bwd", nb, groups, seq, head_dim, dtype)) return rc;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(dout) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv))
    return fail(MCB_ERR_ALIGN, "attention_causal_bwd: 16-byte alignment");
  if (!workspace || workspace_bytes < mcb_attention_workspace_bytes(nb, groups, seq, head_dim) ||
      (reinterpret_cast<uintptr_t>(workspace) & 1023u) != 0)
    return fail(MCB_ERR_WORKSPACE, "attention_causal_bwd: workspace of %zu bytes, 1024-byte aligned, needed",
                mcb_attention_workspace_bytes(nb, groups, seq, head_dim));
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  static bool attr_dq[64] = {}, attr_kv[64] = {};
  int dev = 0;
  MCB_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MCB_ERR_SHAPE, "attention: device %d out of range", dev);
  if (int rc = set_attrs_once(reinterpret_cast<const void*>(attn_dq_kernel), kDqSmem, &attr_dq[dev])) return rc;
  if (int rc = set_attrs_once(reinterpret_cast<const void*>(attn_dkv_kernel), kKvSmem, &attr_kv[dev])) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t rows = static_cast<size_t>(nb) * groups * seq * 4;
  uint8_t* w = static_cast<uint8_t*>(workspace);
  float* delta = reinterpret_cast<float*>(w); w += up1k(rows);
  float* lse2 = reinterpret_cast<float*>(w);
  CUtensorMap tmQ128, tmdO128, tmK64, tmV64, tmK128, tmV128, tmQ64, tmdO64;
  if (int rc = encode(ds, &tmQ128, q, kD, nb * groups * seq, kBQ, "Q")) return rc;
  // dO either like Q ([rows, 64]) or token-major ([batch*S, heads*64]: a head's tile is a column offset)
  const int64_t do_inner = o_token_major ? kv_heads * groups * kD : kD;
  const int64_t do_outer = o_token_major ? (nb / kv_heads) * seq : nb * groups * seq;
  if (int rc = encode(ds, &tmdO128, dout, do_inner, do_outer, kBQ, "dO")) return rc;
  if (int rc = encode(ds, &tmK64, k, kD, nb * seq, kBK, "K")) return rc;
  if (int rc = encode(ds, &tmV64, v, kD, nb * seq, kBK, "V")) return rc;
  if (int rc = encode(ds, &tmK128, k, kD, nb * seq, kBQ, "K block")) return rc;
  if (int rc = encode(ds, &tmV128, v, kD, nb * seq, kBQ, "V block")) return rc;
  if (int rc = encode(ds, &tmQ64, q, kD, nb * groups * seq, kBK, "Q step")) return rc;
  if (int rc = encode(ds, &tmdO64, dout, do_inner, do_outer, kBK, "dO step")) return rc;
  BwdParams p;
  p.S = static_cast<int>(seq); p.G = static_cast<int>(groups); p.NB = static_cast<int>(nb);
  p.HKV = o_token_major ? static_cast<int>(kv_heads) : 1; p.o_tok = o_token_major ? 1 : 0;
  p.sc = scale * kLog2e; p.scale = scale;
  p.O = static_cast<const __nv_bfloat16*>(o); p.dO = static_cast<const __nv_bfloat16*>(dout); p.lse = lse;
  p.delta = delta; p.lse2 = lse2;
  p.dQ = static_cast<__nv_bfloat16*>(dq); p.dK = static_cast<__nv_bfloat16*>(dk); p.dV = static_cast<__nv_bfloat16*>(dv);
  p.status = ds->status_word;
  // persistent: two CTAs per SM walk over the (query block, head, batch) items, heavy ones first
  const int64_t n_tiles = (seq / kBQ) * groups * nb;
  const int64_t slots = 2 * static_cast<int64_t>(ds->sm_count);
  const unsigned gq = static_cast<unsigned>(n_tiles < slots ? n_tiles : slots);
  attn_dq_kernel<<<gq, kThreads, kDqSmem, st>>>(tmQ128, tmdO128, tmK64, tmV64, p);
  MCB_CHECK_LAUNCH("attn_dq_kernel");
  dim3 gk(static_cast<unsigned>(nb), static_cast<unsigned>(seq / kBQ));
  attn_dkv_kernel<<<gk, kKvThreads, kKvSmem, st>>>(tmK128, tmV128, tmQ64, tmdO64, p);
  MCB_CHECK_LAUNCH("attn_dkv_kernel");
  return MCB_OK;
}

extern "C" int mcb_attention_causal_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                        const float* lse, void* dq, void* dk, void* dv, int64_t nb, int64_t groups,
                                        int64_t seq, int64_t head_dim, float scale, int dtype, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  return mcb_attention_causal_bwd_ex(q, k, v, o, dout, lse, dq, dk, dv, nb, groups, seq, head_dim, scale, dtype, 1, 0,
                                     workspace, workspace_bytes, stream);
}
