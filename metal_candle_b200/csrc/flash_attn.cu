// Causal grouped-query attention, fused:  O = softmax(scale * Q K^T + causal mask) V  without ever writing
// the [S, S] score matrix (src/models/transformer.rs:257-285 computes scores, adds the mask, applies softmax
// and multiplies by V as four separate tensor ops over a materialised [B, H, S, S] tensor).
//
// Layouts (bf16, head dimension 64, S a multiple of 128); nb = batch * kv_heads, G query heads per kv head:
//   Q  [nb, G*S, 64]   row g*S + s is query head g, position s           O  the same
//   K  [nb, S, 64]     Vt [nb, 64, S]  (V transposed, so that both MMA operands are K-major)
//   LSE [nb, G*S] float32: log-sum-exp of the scaled scores of a row (natural log), kept for the backward
//
// Forward: one CTA per (128 queries, head); key blocks of 64.  Warp 0 streams K / Vt tiles by TMA into a
// two-stage ring, warp 1 issues the tensor-core MMAs (S = Q K^T into tensor memory, then O_blk = P V),
// warps 2-5 do the online softmax with one query row per thread: read S from tensor memory, rescale, write
// P (bf16) into shared memory in the 128-byte-swizzled K-major operand layout, and accumulate O in
// registers.  Two CTAs per SM overlap one CTA's softmax with the other's MMAs.
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
constexpr uint32_t kOffK = kOffQ + kQBytes;           // 2 stages
constexpr uint32_t kOffV = kOffK + 2 * kKBytes;       // 2 stages
constexpr uint32_t kOffP = kOffV + 2 * kKBytes;
constexpr uint32_t kOffBar = kOffP + kPBytes;
constexpr uint32_t kFwdSmem = kOffBar + 256 + 1024;

struct FwdParams {
  int S, G;
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
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmVt, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t q_full = base + kOffBar, kv_full0 = q_full + 8, kv_empty0 = kv_full0 + 16, s_full = kv_empty0 + 16;
  const uint32_t p_ready = s_full + 8, o_full = p_ready + 8, tmem_slot = o_full + 8, abort_addr = tmem_slot + 4;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_addr - base));

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(128u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t tS = tmem_base, tO = tmem_base + 64;

  // heavy (late) query blocks first
  const int qb = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int g = blockIdx.y, nb = blockIdx.z;
  const int nkb = 2 * qb + 2;  // key blocks of 64 up to and including the diagonal
  const int64_t qrow0 = (static_cast<int64_t>(nb) * p.G + g) * p.S + static_cast<int64_t>(qb) * kBQ;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, kQBytes);
      tma_load_2d(base + kOffQ, &tmQ, q_full, 0, static_cast<int>(qrow0));
      for (int j = 0; j < nkb; ++j) {
        const int st = j & 1;
        if (!mbar_wait(kv_empty0 + 8 * st, ((j >> 1) & 1) ^ 1, abort_flag, 71, p.status)) break;
        mbar_expect_tx(kv_full0 + 8 * st, 2 * kKBytes);
        tma_load_2d(base + kOffK + st * kKBytes, &tmK, kv_full0 + 8 * st, 0, nb * p.S + j * kBK);
        tma_load_2d(base + kOffV + st * kKBytes, &tmVt, kv_full0 + 8 * st, j * kBK, nb * kD);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kBK);  // M = 128, N = 64 for both products
      bool ok = mbar_wait(q_full, 0, abort_flag, 72, p.status);
      if (ok) ok = mbar_wait(kv_full0, 0, abort_flag, 73, p.status);
      if (ok) {
        tcgen05_fence_after();
#pragma unroll
        for (int k4 = 0; k4 < kD / 16; ++k4)
          umma_bf16(tS, desc_sw128(base + kOffQ + k4 * 32), desc_sw128(base + kOffK + k4 * 32), idesc, k4 != 0 ? 1u : 0u);
        umma_commit(s_full);
      }
      for (int j = 0; ok && j < nkb; ++j) {
        const int st = j & 1;
        ok = mbar_wait(p_ready, j & 1, abort_flag, 74, p.status);
        if (!ok) break;
        tcgen05_fence_after();
        // O_blk = P_j V_j   (A = P [128 x 64 keys], B = Vt tile [64 d x 64 keys], both K-major)
#pragma unroll
        for (int k4 = 0; k4 < kBK / 16; ++k4)
          umma_bf16(tO, desc_sw128(base + kOffP + k4 * 32), desc_sw128(base + kOffV + st * kKBytes + k4 * 32), idesc,
                    k4 != 0 ? 1u : 0u);
        umma_commit(o_full);
        umma_commit(kv_empty0 + 8 * st);
        if (j + 1 < nkb) {
          const int s2 = (j + 1) & 1;
          ok = mbar_wait(kv_full0 + 8 * s2, ((j + 1) >> 1) & 1, abort_flag, 75, p.status);
          if (!ok) break;
          tcgen05_fence_after();
#pragma unroll
          for (int k4 = 0; k4 < kD / 16; ++k4)
            umma_bf16(tS, desc_sw128(base + kOffQ + k4 * 32), desc_sw128(base + kOffK + s2 * kKBytes + k4 * 32), idesc,
                      k4 != 0 ? 1u : 0u);
          umma_commit(s_full);
        }
      }
    }
  } else {
    // ---------------- online softmax, one query row per thread ----------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int qpos = qb * kBQ + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    uint8_t* prow = gen_base + kOffP + row * 128;
    const int sw = row & 7;
    float m = -INFINITY, l = 0.0f;
    float o[kD];
#pragma unroll
    for (int c = 0; c < kD; ++c) o[c] = 0.0f;
    bool ok = true;
    for (int j = 0; j < nkb; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(s_full, j & 1, abort_flag, 76, p.status));
      if (!ok) break;
      tcgen05_fence_after();
      const int key0 = j * kBK;
      const bool diag = key0 + kBK - 1 > qb * kBQ;  // some element of this block may lie above the diagonal
      // pass 1: row maximum of the raw scores
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < kBK; c += 16) {
        uint32_t v[16];
        tmem_ld_x16(tS + lane_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float s = __uint_as_float(v[e]);
          mx = fmaxf(mx, (!diag || key0 + c + e <= qpos) ? s : -INFINITY);
        }
      }
      const float m_new = fmaxf(m, mx * p.sc);  // key 0 is never masked, so m_new is finite from block 0 on
      const float alpha = ex2(m - m_new);       // block 0: 2^(-inf) = 0
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(o_full, (j - 1) & 1, abort_flag, 77, p.status));
        if (!ok) break;
        tcgen05_fence_after();
#pragma unroll
        for (int c = 0; c < kD; c += 16) {
          uint32_t v[16];
          tmem_ld_x16(tO + lane_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) o[c + e] = (o[c + e] + __uint_as_float(v[e])) * alpha;
        }
      }
      l *= alpha;
      // pass 2: P = 2^(s*sc - m_new), row sum, bf16 into the swizzled operand buffer
      float ls = 0.0f;
#pragma unroll
      for (int c = 0; c < kBK; c += 16) {
        uint32_t v[16];
        tmem_ld_x16(tS + lane_addr + c, v);
        tmem_ld_wait();
        uint32_t w[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          float p0 = ex2(fmaf(__uint_as_float(v[e]), p.sc, -m_new));
          float p1 = ex2(fmaf(__uint_as_float(v[e + 1]), p.sc, -m_new));
          if (diag) {
            if (key0 + c + e > qpos) p0 = 0.0f;
            if (key0 + c + e + 1 > qpos) p1 = 0.0f;
          }
          // the sum uses the rounded values, the ones the P V product sees
          const uint32_t pk = pack_bf16(p0, p1);
          ls += __uint_as_float(pk << 16) + __uint_as_float(pk & 0xffff0000u);
          w[e >> 1] = pk;
        }
        const int cc = c >> 3;  // 16-byte chunk index of columns c .. c+7
        *reinterpret_cast<uint4*>(prow + (((cc) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(prow + (((cc + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
      }
      l += ls;
      m = m_new;
      tcgen05_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_full, (nkb - 1) & 1, abort_flag, 78, p.status));
    if (ok) {
      tcgen05_fence_after();
      const float inv = 1.0f / l;
      __nv_bfloat16* orow = p.O + (qrow0 + row) * kD;
#pragma unroll
      for (int c = 0; c < kD; c += 16) {
        uint32_t v[16];
        tmem_ld_x16(tO + lane_addr + c, v);
        tmem_ld_wait();
        uint32_t w[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2)
          w[e >> 1] = pack_bf16((o[c + e] + __uint_as_float(v[e])) * inv, (o[c + e + 1] + __uint_as_float(v[e + 1])) * inv);
        *reinterpret_cast<uint4*>(orow + c) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(orow + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
      }
      if (p.lse != nullptr) p.lse[qrow0 + row] = (m + lg2(l)) * kLn2;
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
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

extern "C" int mcb_attention_causal_fwd(const void* q, const void* k, const void* vt, void* o, float* lse, int64_t nb,
                                        int64_t groups, int64_t seq, int64_t head_dim, float scale, int dtype,
                                        void* stream) {
  using namespace mcb::attn;
  if (!q || !k || !vt || !o) return fail(MCB_ERR_NULL, "attention_causal_fwd: q, k, vt or o is null");
  if (int rc = check_shape("attention_causal_fwd", nb, groups, seq, head_dim, dtype)) return rc;
  if (!aligned16(q) || !aligned16(k) || !aligned16(vt) || !aligned16(o)) return fail(MCB_ERR_ALIGN, "attention_causal_fwd: 16-byte alignment");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  static bool attr_set[64] = {};
  int dev = 0;
  MCB_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    MCB_CHECK_CUDA(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem));
    MCB_CHECK_CUDA(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    attr_set[dev] = true;
  }
  CUtensorMap tmQ, tmK, tmVt;
  if (int rc = encode(ds, &tmQ, q, kD, nb * groups * seq, kBQ, "Q")) return rc;
  if (int rc = encode(ds, &tmK, k, kD, nb * seq, kBK, "K")) return rc;
  if (int rc = encode(ds, &tmVt, vt, seq, nb * kD, kD, "Vt")) return rc;
  FwdParams p;
  p.S = static_cast<int>(seq); p.G = static_cast<int>(groups);
  p.sc = scale * kLog2e;
  p.O = static_cast<__nv_bfloat16*>(o); p.lse = lse; p.status = ds->status_word;
  dim3 grid(static_cast<unsigned>(seq / kBQ), static_cast<unsigned>(groups), static_cast<unsigned>(nb));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  attn_fwd_kernel<<<grid, kThreads, kFwdSmem, st>>>(tmQ, tmK, tmVt, p);
  MCB_CHECK_LAUNCH("attn_fwd_kernel");
  return MCB_OK;
}
