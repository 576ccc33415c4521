// Frozen linear  Y[M,N] = X[M,K] . W[N,K]^T (+ bias) (+ residual)  on CTA pairs (tcgen05 cta_group::2).
//
// The one-CTA kernel of umma_gemm.cu moves 48 KB from L2 per 128x256 tile and k-block and can hold only
// four such stages, which leaves the tensor pipe waiting for loads about a third of the time.  Here two
// CTAs of a cluster (two neighbouring SMs) own one 256 x BN tile: each loads its own 128 rows of X and
// HALF of the W tile (BN/2 rows), the pair's leader issues one tcgen05.mma.cta_group::2 (M = 256) that
// reads both halves from both CTAs' shared memory, and each CTA finds its 128 x BN accumulator rows in
// its own tensor memory.  Per SM and k-block that is 32 KB instead of 48 KB, and six stages fit.
//
// Synchronisation (no load uses cluster multicast):
//   full[s]      in the LEADER: the leader's producer arms it for the bytes of BOTH CTAs; both producers'
//                TMA loads (cp.async.bulk.tensor...cta_group::2) complete on it
//   empty[s]     in each CTA: tcgen05.commit.cta_group::2 ... multicast::cluster from the leader's MMA thread
//   acc_full[a]  in each CTA: same commit, after the last k-block of a tile
//   acc_empty[a] in the LEADER: 8 arrivals, the 4 epilogue warps of each CTA (the peer's arrive remotely)
// Every wait is bounded; both CTAs always meet at the cluster barrier before tensor memory is released.
#include <cuda.h>
#include <string.h>

#include "lora_internal.cuh"
#include "umma_ptx.cuh"

namespace mcb {
namespace bf16path {
using namespace umma;
namespace {

constexpr int BK2 = 64;
constexpr int kThreads2 = 192;
constexpr int kMaxStages2 = 8;
constexpr int kSmem2 = 227 * 1024 - 1024;

struct Gemm2Params {
  int M, N, K;
  int BN, stages;
  int num_m_tiles, num_n_tiles, num_tiles, num_k_blocks, group_m;  // m tiles of 256 rows
  __nv_bfloat16* Y;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* R;
  int* status;
  uint32_t stage_bytes, w_off, bar_off;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `cta` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(cta));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t cta) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
      ::"r"(bar), "r"(cta) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma2_commit_both(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .b16 m;\n\t"
      "mov.b16 m, 3;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
      ::"r"(bar) : "memory");
}
// kind::f16, D=f32, A=B=bf16 K-major, M=256 (the pair), N=n
__host__ __device__ constexpr uint32_t make_idesc2(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
}

__device__ __forceinline__ void tile_coords2(const Gemm2Params& p, int t, int& mt, int& nt) {
  const int per_band = p.group_m * p.num_n_tiles;
  const int band = t / per_band;
  const int in = t - band * per_band;
  const int m_first = band * p.group_m;
  const int gm = min(p.group_m, p.num_m_tiles - m_first);
  nt = in / gm;
  mt = m_first + in % gm;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
lora_gemm2_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  const uint32_t full0 = base + p.bar_off;
  const uint32_t empty0 = full0 + 8 * kMaxStages2;
  const uint32_t acc_full0 = empty0 + 8 * kMaxStages2;
  const uint32_t acc_empty0 = acc_full0 + 16;
  const uint32_t tmem_slot = acc_empty0 + 16;
  const uint32_t abort_addr = tmem_slot + 4;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_addr - base));

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them remotely
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const int nkb = p.num_k_blocks;
  const int half_n = p.BN / 2;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; ok && t < p.num_tiles; t += npairs) {
        int mt, nt;
        tile_coords2(p, t, mt, nt);
        const int m0 = mt * 256 + static_cast<int>(rank) * 128;
        const int n0 = nt * p.BN + static_cast<int>(rank) * half_n;
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, 61, p.status);
          if (!ok) break;
          const uint32_t fb = map_to_cta(full0 + 8 * stage, 0);  // the leader's barrier
          const uint32_t sb = base + stage * p.stage_bytes;
          if (rank == 0) mbar_expect_tx(full0 + 8 * stage, 2 * p.stage_bytes);
          tma_load_2d_pair(sb, &tmX, fb, kb * BK2, m0);
          tma_load_2d_pair(sb + p.w_off, &tmW, fb, kb * BK2, n0);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc2(p.BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int i = 0;
      for (int t = pair; ok && t < p.num_tiles; t += npairs, ++i) {
        const int a = i & 1;
        const uint32_t u = static_cast<uint32_t>(i >> 1);
        ok = mbar_wait(acc_empty0 + 8 * a, (u & 1) ^ 1, abort_flag, 62, p.status);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t d = tmem_base + a * 256;
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, 63, p.status);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t sb = base + stage * p.stage_bytes;
#pragma unroll
          for (int k4 = 0; k4 < BK2 / 16; ++k4)
            umma2_bf16(d, desc_sw128(sb + k4 * 32), desc_sw128(sb + p.w_off + k4 * 32), idesc, (kb | k4) != 0 ? 1u : 0u);
          umma2_commit_both(empty0 + 8 * stage);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma2_commit_both(acc_full0 + 8 * a);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5, both CTAs): own 128 rows of the pair's tile ----------------
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    int i = 0;
    for (int t = pair; ok && t < p.num_tiles; t += npairs, ++i) {
      int mt, nt;
      tile_coords2(p, t, mt, nt);
      const int m0 = mt * 256 + static_cast<int>(rank) * 128, n0 = nt * p.BN;
      const int a = i & 1;
      const uint32_t u = static_cast<uint32_t>(i >> 1);
      const int64_t grow = static_cast<int64_t>(m0) + row_in_tile;
      const uint32_t d = tmem_base + lane_addr + a * 256;
      ok = __all_sync(0xffffffffu, mbar_wait(acc_full0 + 8 * a, u & 1, abort_flag, 64, p.status));
      if (!ok) break;
      tcgen05_fence_after();
      for (int c = 0; c < p.BN; c += 32) {
        uint32_t v0[16], v1[16];
        tmem_ld_x16(d + c, v0);
        tmem_ld_x16(d + c + 16, v1);
        tmem_ld_wait();
        const int gcol = n0 + c;
        if (grow < p.M && gcol < p.N) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 16; ++j) { f[j] = __uint_as_float(v0[j]); f[16 + j] = __uint_as_float(v1[j]); }
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (gcol + j < p.N) f[j] += __bfloat162float(p.bias[gcol + j]);
          }
          uint4* yp = reinterpret_cast<uint4*>(p.Y + grow * p.N + gcol);
          if (p.R != nullptr) {
            const uint4* rp4 = reinterpret_cast<const uint4*>(p.R + grow * p.N + gcol);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              if (gcol + 8 * q4 + 8 <= p.N) {
                const uint4 rv = rp4[q4];
                const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int e2 = 0; e2 < 4; ++e2) {
                  f[8 * q4 + 2 * e2] += __uint_as_float(rw[e2] << 16);
                  f[8 * q4 + 2 * e2 + 1] += __uint_as_float(rw[e2] & 0xffff0000u);
                }
              }
            }
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            if (gcol + 8 * q4 + 8 <= p.N)
              yp[q4] = make_uint4(pack_bf16(f[8 * q4], f[8 * q4 + 1]), pack_bf16(f[8 * q4 + 2], f[8 * q4 + 3]),
                                  pack_bf16(f[8 * q4 + 4], f[8 * q4 + 5]), pack_bf16(f[8 * q4 + 6], f[8 * q4 + 7]));
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(acc_empty0 + 8 * a);
        else mbar_arrive_remote(acc_empty0 + 8 * a, 0);
      }
    }
  }

  // ---------------- common exit: both CTAs meet before either lets go of shared or tensor memory ----------------
  __syncwarp();
  if (*abort_flag != 0) {
    for (int k = 0; k < 200; ++k) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_map2(const DeviceState* ds, CUtensorMap* map, const void* ptr, int64_t inner, int64_t outer, int box_outer,
              const char* what) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(inner) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(BK2), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn2>(ds->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MCB_ERR_ALIGN, "tensor map for %s rejected (CUresult %d)", what, static_cast<int>(r));
  return MCB_OK;
}

}  // namespace

int init_gemm2_kernel() {
  cudaError_t e = cudaFuncSetAttribute(lora_gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2 + 1024);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(lora_gemm2_kernel)");
  return MCB_OK;
}

// Whether the pair kernel takes this plain linear (everything else stays on the one-CTA kernel).
bool gemm2_eligible(int64_t M, int64_t N, int64_t K) { return M >= 1024 && N >= 128 && K >= 64; }

int launch_gemm2(const __nv_bfloat16* X, const __nv_bfloat16* W, const __nv_bfloat16* bias, const __nv_bfloat16* R,
                 __nv_bfloat16* Y, int64_t M, int64_t N, int64_t K, const DeviceState* ds, cudaStream_t st) {
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  // tile width: fewest n-tiles of at most 256 columns, evened out, multiple of 32 (so each half is a multiple of 16)
  const int64_t tiles = (N + 255) / 256;
  int bn = static_cast<int>(((N + tiles - 1) / tiles + 31) / 32 * 32);
  if (bn > 256) bn = 256;
  if (bn < 32) bn = 32;
  p.BN = bn;
  p.num_m_tiles = static_cast<int>((M + 255) / 256);
  p.num_n_tiles = static_cast<int>((N + bn - 1) / bn);
  p.num_tiles = p.num_m_tiles * p.num_n_tiles;
  p.num_k_blocks = static_cast<int>((K + BK2 - 1) / BK2);
  p.group_m = p.num_m_tiles < 8 ? p.num_m_tiles : 8;
  p.Y = Y; p.bias = bias; p.R = R; p.status = ds->status_word;
  const uint32_t x_bytes = 128 * BK2 * 2, w_bytes = static_cast<uint32_t>(bn / 2) * BK2 * 2;
  p.w_off = x_bytes;
  p.stage_bytes = x_bytes + w_bytes;
  int stages = static_cast<int>((kSmem2 - 512) / p.stage_bytes);
  if (stages > kMaxStages2) stages = kMaxStages2;
  p.stages = stages;
  p.bar_off = stages * p.stage_bytes;
  CUtensorMap tmX, tmW;
  if (int rc = make_map2(ds, &tmX, X, K, M, 128, "X (pair)")) return rc;
  if (int rc = make_map2(ds, &tmW, W, K, N, bn / 2, "W (pair)")) return rc;
  int pairs = ds->sm_count / 2;
  if (pairs > p.num_tiles) pairs = p.num_tiles;
  const bool prof = profile_on();
  if (prof) profile_begin(kProfGemm, 2.0 * M * N * K, 2.0 * (static_cast<double>(M) * K + static_cast<double>(N) * K + static_cast<double>(M) * N), st);
  lora_gemm2_kernel<<<2 * pairs, kThreads2, kSmem2 + 1024, st>>>(tmX, tmW, p);
  if (prof) profile_end(st);
  MCB_CHECK_LAUNCH("lora_gemm2_kernel");
  return MCB_OK;
}

}  // namespace bf16path
}  // namespace mcb
