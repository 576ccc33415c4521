// LoRA weight gradients on tensor cores:  out[C, rp] = X[M, C]^T . H[M, rp]  (a reduction over tokens).
//
//   dA [K, r] = x^T  (scale * dy B^T)        X = x  [M,K],  H = the rank intermediate of the backward GEMM
//   dB [r, N] = (scale * x A)^T dy           X = dy [M,N],  H = the rank intermediate saved by the forward
//
// Both operands are token-major in memory, i.e. the reduction index is the SLOW one.  X is handed to tcgen05.mma
// as an MN-major A operand exactly as it lies; H arrives already transposed ([rp, tokens], written that way by
// the GEMM epilogue) as a K-major B operand.  One launch serves both gradients of a LoRA linear.
//
// The kernel is HBM-bound (it reads X once, 2 bytes per element, and issues one 128 x rp x 16 MMA per 4 KB of
// it), so what matters is how DRAM is read: a CTA owns a slice of the tokens and a GROUP of up to 1024 features
// (all of them for the model's 896-wide projections) and streams whole token rows of its group - one
// three-dimensional TMA copy per stage (features within a 64-wide atom, tokens, atoms), 16 or 32 tokens deep.
// Every 128-feature tile of the group has its own [128 x rp] accumulator in tensor memory.  A CTA writes one
// float32 partial; a second small kernel sums the partials in slice order, so the result is deterministic.
//
// Feature counts that are not a multiple of 64 cannot be seen as whole 64-feature atoms; they take the older
// form further down (a CTA owns 128 features, [64 tokens] x [64 features] boxes, one problem per launch), which
// reads 256-byte pieces of each row and reaches about half of the copy bandwidth.
#include <cuda.h>
#include <string.h>

#include "grad_phase.cuh"
#include "lora_internal.cuh"
#include "umma_ptx.cuh"

namespace mcb {
namespace bf16path {
using namespace umma;
namespace {

constexpr int kGradThreads = 192;

__global__ void __launch_bounds__(kGradThreads)
lora_grad_umma_kernel(const __grid_constant__ CUtensorMap tmX0, const __grid_constant__ CUtensorMap tmH0,
                      const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmH1,
                      const GradParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = base + p.bar_off, empty0 = full0 + 8 * kGradMaxStages, done_bar = empty0 + 8 * kGradMaxStages;
  const uint32_t tmem_slot = done_bar + 8, abort_addr = tmem_slot + 4;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_addr - base));

  // tensor-memory columns for this CTA's problem: one [128 x rp] accumulator per 128-feature tile of a group
  const int acc_cols = p.pr[static_cast<int>(blockIdx.x) >= p.n_cta0 ? 1 : 0].tiles * p.rp;
  const uint32_t tmem_cols = acc_cols <= 32 ? 32u : acc_cols <= 64 ? 64u : acc_cols <= 128 ? 128u : acc_cols <= 256 ? 256u : 512u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGradMaxStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (threadIdx.x == 0) grid_launch_dependents();   // the partial-sum kernel may be set up; it waits for this grid
  GradShared sh;
  sh.base = base; sh.full0 = full0; sh.empty0 = empty0; sh.done_bar = done_bar; sh.tmem_base = tmem_base;
  sh.abort_flag = abort_flag;
  grad_roles(p, &tmX0, &tmH0, &tmX1, &tmH1, sh, static_cast<int>(blockIdx.x));
  __syncwarp();
  if (*abort_flag != 0) {
    for (int k = 0; k < 200; ++k) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// out (+)= sum over slices (fixed order: deterministic), for both problems in one launch.  A CTA owns 32
// consecutive (feature, rank column) pairs of one problem; its 8 warps each sum every 8th slice (independent,
// coalesced loads), then warp 0 adds the 8 sums in warp order.  transposed == 0 writes out[c*r + j] (dA [K,r]);
// 1 writes out[j*C + c] (dB [r,N]).
struct ReduceProblem {
  const float* part;
  float* out;
  int slices, C, transposed;
};
__global__ void __launch_bounds__(256)
lora_grad_reduce_kernel(ReduceProblem a, ReduceProblem b, int blocks_a, int r, int rp, int accumulate) {
  __shared__ float red[8][32];
  grid_dependency_wait();   // launched as a programmatic dependent of the kernel that writes the partials
  const bool second = static_cast<int>(blockIdx.x) >= blocks_a;
  const ReduceProblem q = second ? b : a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n = static_cast<int64_t>(q.C) * rp;
  const int64_t e = (static_cast<int64_t>(blockIdx.x) - (second ? blocks_a : 0)) * 32 + lane;   // index into [C][rp]
  float s = 0.0f;
  if (e < n) {
#pragma unroll 4
    for (int sp = warp; sp < q.slices; sp += 8) s += q.part[static_cast<int64_t>(sp) * n + e];
  }
  red[warp][lane] = s;
  __syncthreads();
  if (warp != 0 || e >= n) return;
  float t = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) t += red[w][lane];
  const int c = static_cast<int>(e / rp), j = static_cast<int>(e % rp);
  if (j >= r) return;
  const int64_t o = q.transposed ? static_cast<int64_t>(j) * q.C + c : static_cast<int64_t>(c) * r + j;
  q.out[o] = accumulate ? q.out[o] + t : t;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// X [M, C] (C a multiple of 64) seen as [64 features][M tokens][C/64 atoms]: box = 64 x T x atoms, 128-byte swizzle
int encode_x(const DeviceState* ds, CUtensorMap* map, const void* ptr, int64_t M, int64_t C, int T, int atoms) {
  cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(C / 64)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(C) * 2, 128};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(T), static_cast<cuuint32_t>(atoms)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ds->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MCB_ERR_ALIGN, "tensor map for grad X rejected (CUresult %d)", static_cast<int>(r));
  return MCB_OK;
}
// H^T [rp, h_pitch]: box = 8 tokens x rp rows, no swizzle
int encode_h(const DeviceState* ds, CUtensorMap* map, const void* ptr, int64_t M, int64_t h_pitch, int rp) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(rp)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(h_pitch) * 2};
  cuuint32_t box[2] = {8, static_cast<cuuint32_t>(rp)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ds->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MCB_ERR_ALIGN, "tensor map for grad H rejected (CUresult %d)", static_cast<int>(r));
  return MCB_OK;
}

constexpr int kGradSmem = kGradSmemBudget + 16 * kGradMaxStages + 64 + 1024;

// feature groups of a problem: as few as keep a group within kGradGroup features and its accumulators within the
// 512 tensor-memory columns; all groups equally wide (a multiple of 128), the last may hang over C (zero-filled)
void plan_groups(int64_t C, int rp, GradProblem* q) {
  int max_tiles = 512 / rp;
  if (max_tiles > kGradGroup / 128) max_tiles = kGradGroup / 128;
  const int tiles_total = static_cast<int>((C + 127) / 128);
  q->groups = (tiles_total + max_tiles - 1) / max_tiles;
  q->tiles = (tiles_total + q->groups - 1) / q->groups;
  q->group_feats = q->tiles * 128;
  q->C = static_cast<int>(C);
}

// ---------------------------------------------------------------------------------------------------------
// older form, for feature counts that are not a multiple of 64: one problem per launch, a CTA owns 128 features
// ---------------------------------------------------------------------------------------------------------
constexpr int kTileBK = 64;       // tokens per stage
constexpr int kTileMaxStages = 12;  // enough bytes in flight per SM to cover HBM latency under load
constexpr int kTileSmemBudget = 216 * 1024;
constexpr uint32_t kTileBoxBytes = 64 * 64 * 2;  // one [64 tokens x 64 features] box

struct TileParams {
  int M, C, rp;
  int total_kb, kb_per_split;
  float* part;  // [splits][C][rp]
  int* status;
  uint32_t stage_bytes, bar_off;
  int stages;
};

__global__ void __launch_bounds__(kGradThreads)
lora_grad_tile_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmH,
                      const TileParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = base + p.bar_off, empty0 = full0 + 8 * kTileMaxStages, done_bar = empty0 + 8 * kTileMaxStages;
  const uint32_t tmem_slot = done_bar + 8, abort_addr = tmem_slot + 4;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_addr - base));

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(64u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  const int c0 = blockIdx.x * BM;
  const int kb_begin = blockIdx.y * p.kb_per_split;
  const int kb_end = min(p.total_kb, kb_begin + p.kb_per_split);
  const int nkb = kb_end - kb_begin;  // >= 1 by construction of the grid

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, 41, p.status)) break;
        const uint32_t fb = full0 + 8 * stage, sb = base + stage * p.stage_bytes;
        mbar_expect_tx(fb, p.stage_bytes);
        tma_load_2d(sb, &tmX, fb, c0, kb * kTileBK);
        tma_load_2d(sb + kTileBoxBytes, &tmX, fb, c0 + 64, kb * kTileBK);
        tma_load_2d(sb + 2 * kTileBoxBytes, &tmH, fb, kb * kTileBK, 0);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_a_mn(p.rp);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, 42, p.status);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t sb = base + stage * p.stage_bytes;
#pragma unroll
        for (int k4 = 0; k4 < kTileBK / 16; ++k4) {
          // A: 16 token rows further = 2 K-groups of 8 rows x 128 bytes; the second 64-feature atom is the
          // second box.  B: 16 tokens further along the contiguous dimension = 32 bytes.
          const uint64_t ad = desc_sw128_mn(sb + k4 * 2048, kTileBoxBytes, 1024);
          const uint64_t bd = desc_sw128(sb + 2 * kTileBoxBytes + k4 * 32);
          umma_bf16(tmem_base, ad, bd, idesc, (i | k4) != 0 ? 1u : 0u);
        }
        umma_commit(empty0 + 8 * stage);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(done_bar);
    }
  } else {
    const int quad = warp & 3;
    const int c = c0 + quad * 32 + lane;
    const bool ok = __all_sync(0xffffffffu, mbar_wait(done_bar, 0, abort_flag, 43, p.status));
    if (ok) {
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      for (int j = 0; j < p.rp; j += 16) {
        uint32_t v[16];
        tmem_ld_x16(taddr + j, v);
        tmem_ld_wait();
        if (c < p.C) {
          float4* o = reinterpret_cast<float4*>(p.part + (static_cast<int64_t>(blockIdx.y) * p.C + c) * p.rp + j);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            o[q] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                               __uint_as_float(v[4 * q + 3]));
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(64u) : "memory");
  }
}

// out (+)= sum over splits, in split order.  One thread per (feature c, rank column j < rp); reads are
// contiguous across the block.  transposed == 0 writes out[c*r + j] (dA [K,r]); 1 writes out[j*C + c] (dB [r,N]).
__global__ void lora_grad_tile_reduce_kernel(const float* __restrict__ part, float* __restrict__ out, int splits, int C,
                                        int r, int rp, int transposed, int accumulate) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t n = static_cast<int64_t>(C) * rp;
  if (tid >= n) return;
  const int c = static_cast<int>(tid / rp), j = static_cast<int>(tid % rp);
  if (j >= r) return;
  float s = 0.0f;
#pragma unroll 8
  for (int sp = 0; sp < splits; ++sp) s += part[static_cast<int64_t>(sp) * n + tid];
  const int64_t o = transposed ? static_cast<int64_t>(j) * C + c : static_cast<int64_t>(c) * r + j;
  out[o] = accumulate ? out[o] + s : s;
}

typedef CUresult (*EncodeTiledFnT)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_tile(const DeviceState* ds, CUtensorMap* map, const void* ptr, int64_t inner, int64_t outer, int64_t pitch_elems,
           int box_inner, int box_outer, const char* what) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_elems) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFnT>(ds->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MCB_ERR_ALIGN, "tensor map for %s rejected (CUresult %d)", what, static_cast<int>(r));
  return MCB_OK;
}

constexpr int kTileSmem = kTileSmemBudget + 1024 + 512;


// Token slices per feature tile: at most one CTA per SM, all resident at once (measured: more, shorter CTAs
// lose to their set-up cost, and a second round of CTAs doubles the time).
int tile_splits(int64_t M, int64_t C, int sm_count, int* kb_per_split) {
  const int64_t c_tiles = (C + BM - 1) / BM;
  const int64_t total_kb = (M + kTileBK - 1) / kTileBK;
  int64_t target = static_cast<int64_t>(sm_count) / c_tiles;
  if (target > total_kb) target = total_kb;
  if (target < 1) target = 1;
  const int64_t per = (total_kb + target - 1) / target;
  if (kb_per_split) *kb_per_split = static_cast<int>(per);
  return static_cast<int>((total_kb + per - 1) / per);
}


int launch_grad_tile(const __nv_bfloat16* X, const __nv_bfloat16* Ht, int64_t h_pitch, float* out, float* part, int64_t M,
                int64_t C, int r, int rp, int transposed, int accumulate, const DeviceState* ds, cudaStream_t st) {
  if (C % 8 != 0) return fail(MCB_ERR_ALIGN, "bf16 LoRA gradients need a feature count that is a multiple of 8 (got %lld)", (long long)C);
  if (!aligned16(X) || !aligned16(Ht) || h_pitch % 8 != 0) return fail(MCB_ERR_ALIGN, "bf16 LoRA gradients: operand alignment");
  TileParams p;
  p.M = static_cast<int>(M); p.C = static_cast<int>(C); p.rp = rp;
  p.total_kb = static_cast<int>((M + kTileBK - 1) / kTileBK);
  const int splits = tile_splits(M, C, ds->sm_count, &p.kb_per_split);
  p.part = part;
  p.status = ds->status_word;
  p.stage_bytes = 2 * kTileBoxBytes + static_cast<uint32_t>(rp) * 128;
  p.stages = static_cast<int>(kTileSmemBudget / p.stage_bytes);
  if (p.stages > kTileMaxStages) p.stages = kTileMaxStages;
  p.bar_off = p.stages * p.stage_bytes;
  CUtensorMap tmX, tmH;
  if (int rc = encode_tile(ds, &tmX, X, C, M, C, 64, kTileBK, "grad X")) return rc;
  if (int rc = encode_tile(ds, &tmH, Ht, M, rp, h_pitch, kTileBK, rp, "grad H")) return rc;
  dim3 grid(static_cast<unsigned>((C + BM - 1) / BM), static_cast<unsigned>(splits));
  const bool prof = profile_on();
  if (prof) profile_begin(kProfGrad, 2.0 * M * C * r, 2.0 * M * C + 2.0 * M * rp, st);
  lora_grad_tile_kernel<<<grid, kGradThreads, kTileSmem, st>>>(tmX, tmH, p);
  if (prof) profile_end(st);
  MCB_CHECK_LAUNCH("lora_grad_tile_kernel");
  const int64_t n = C * rp;
  lora_grad_tile_reduce_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(part, out, splits, static_cast<int>(C), r,
                                                                                   rp, transposed, accumulate);
  MCB_CHECK_LAUNCH("lora_grad_reduce");
  return MCB_OK;
}


}  // namespace

int init_grad_kernel() {
  cudaError_t e = cudaFuncSetAttribute(lora_grad_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGradSmem);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(lora_grad_umma_kernel)");
  e = cudaFuncSetAttribute(lora_grad_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileSmem);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(lora_grad_tile_kernel)");
  return MCB_OK;
}

// Partial sums of one launch: the CTAs of both problems together are at most the SM count (<= 256 assumed), each
// writes at most kGradGroup x rp floats; the older form needs at most 256 slices of C x rp.
size_t grad_partial_bytes(int64_t M, int64_t K, int64_t N, int rp) {
  size_t b = static_cast<size_t>(256) * kGradGroup * rp * sizeof(float);
  for (int64_t C : {K, N}) {
    if (C % 64 != 0) {
      const size_t t = static_cast<size_t>(tile_splits(M, C, 256, nullptr)) * C * rp * sizeof(float);
      if (t > b) b = t;
    }
  }
  return b;
}

bool grad_tail_possible(int64_t C0, int64_t C1, int rp) {
  for (int64_t C : {C0, C1}) {
    if (C <= 0 || C % 64 != 0) return false;
    GradProblem q;
    plan_groups(C, rp, &q);
    if (q.groups != 1) return false;
  }
  return true;
}

int plan_grad2(const GradRequest& rq, int64_t M, int rp, int max_ctas, uint32_t smem_budget, const DeviceState* ds,
               GradPlan* plan) {
  const int np = rq.X[1] != nullptr ? 2 : 1;
  plan->np = np;
  plan->rq = rq;
  for (int i = 0; i < np; ++i)
    if (!aligned16(rq.X[i]) || !aligned16(rq.Ht[i]) || rq.C[i] % 64 != 0)
      return fail(MCB_ERR_ALIGN, "bf16 LoRA gradients: operand alignment");
  if (rq.h_pitch % 8 != 0) return fail(MCB_ERR_ALIGN, "bf16 LoRA gradients: operand alignment");
  GradParams& p = plan->p;
  memset(&p, 0, sizeof(p));
  p.M = static_cast<int>(M); p.rp = rp;
  p.status = ds->status_word;
  p.h_flags = rq.h_flags;
  for (int i = 0; i < np; ++i) plan_groups(rq.C[i], rp, &p.pr[i]);
  // tokens per stage, per problem: as many (a multiple of 16, at most 256) as keep a stage near 48 KB, so that
  // narrow problems have as many bytes in flight as wide ones
  for (int i = 0; i < np; ++i) {
    int T = (48 * 1024) / (p.pr[i].group_feats * 2) / 16 * 16;
    if (T < 16) T = 16;
    if (T > 256) T = 256;
    p.T[i] = T;
    p.x_bytes[i] = static_cast<uint32_t>(T) * p.pr[i].group_feats * 2;
    const uint32_t sbytes = p.x_bytes[i] + static_cast<uint32_t>(rp) * T * 2;
    p.stage_stride[i] = (sbytes + 1023u) & ~1023u;
    p.stages[i] = static_cast<int>(smem_budget / p.stage_stride[i]);
    if (p.stages[i] > kGradMaxStages) p.stages[i] = kGradMaxStages;
    if (p.stages[i] < 2) return fail(MCB_ERR_UNSUPPORTED, "bf16 LoRA gradients: stage does not fit shared memory");
  }
  p.bar_off = kGradSmemBudget;
  // CTAs: shared between the problems in proportion to their bytes, whole token slices per feature group
  const double wsum = static_cast<double>(rq.C[0]) + static_cast<double>(np == 2 ? rq.C[1] : 0);
  int used = 0;
  float* pp = rq.part;
  for (int i = 0; i < np; ++i) {
    int share = np == 1 ? max_ctas : static_cast<int>(max_ctas * (static_cast<double>(rq.C[i]) / wsum));
    if (i == 1) share = max_ctas - used;
    int slices = share / p.pr[i].groups;
    if (slices < 1) slices = 1;
    const int total_steps = static_cast<int>((M + p.T[i] - 1) / p.T[i]);
    if (slices > total_steps) slices = total_steps;
    p.pr[i].slices = slices;
    p.pr[i].part = pp;
    pp += static_cast<size_t>(slices) * rq.C[i] * rp;
    const int n = slices * p.pr[i].groups;
    if (i == 0) p.n_cta0 = n;
    used += n;
  }
  p.n_cta = used;
  if (static_cast<size_t>(pp - rq.part) * sizeof(float) > static_cast<size_t>(256) * kGradGroup * rp * sizeof(float))
    return fail(MCB_ERR_WORKSPACE, "bf16 LoRA gradients: partial sums exceed the workspace");
  for (int i = 0; i < np; ++i) {
    if (int rc = encode_x(ds, &plan->tmX[i], rq.X[i], M, rq.C[i], p.T[i], p.pr[i].group_feats / 64)) return rc;
    if (int rc = encode_h(ds, &plan->tmH[i], rq.Ht[i], M, rq.h_pitch, rp)) return rc;
  }
  if (np == 1) { plan->tmX[1] = plan->tmX[0]; plan->tmH[1] = plan->tmH[0]; }
  return MCB_OK;
}

int launch_grad_reduce(const GradPlan& plan, cudaStream_t st) {
  const GradParams& p = plan.p;
  const GradRequest& rq = plan.rq;
  const bool two = plan.np == 2;
  ReduceProblem ra = {p.pr[0].part, rq.out[0], p.pr[0].slices, static_cast<int>(rq.C[0]), rq.transposed[0]};
  ReduceProblem rb = {two ? p.pr[1].part : nullptr, rq.out[1], two ? p.pr[1].slices : 0, two ? static_cast<int>(rq.C[1]) : 0,
                      rq.transposed[1]};
  const int blocks_a = static_cast<int>((rq.C[0] * p.rp + 31) / 32);
  const int blocks_b = two ? static_cast<int>((rq.C[1] * p.rp + 31) / 32) : 0;
  {
    const cudaError_t le = launch_kernel(lora_grad_reduce_kernel, dim3(static_cast<unsigned>(blocks_a + blocks_b)), dim3(256), 0, st,
                                         option(MCB_OPT_PDL) != 0 && !profile_on(), ra, rb, blocks_a, rq.r, p.rp, rq.accumulate);
    if (le != cudaSuccess) return cuda_fail(le, "lora_grad_reduce launch");
  }
  MCB_CHECK_LAUNCH("lora_grad_reduce");
  return MCB_OK;
}

// out_i = X_i^T H_i with H_i given transposed as Ht_i [rp, h_pitch] (token index contiguous), for one or two
// problems over the same M tokens (X1 == nullptr: one problem).
int launch_grad2(const __nv_bfloat16* X0, const __nv_bfloat16* Ht0, int64_t C0, float* out0, int transposed0,
                 const __nv_bfloat16* X1, const __nv_bfloat16* Ht1, int64_t C1, float* out1, int transposed1,
                 int64_t h_pitch, float* part, int64_t M, int r, int rp, int accumulate, const DeviceState* ds,
                 cudaStream_t st) {
  const int np = X1 != nullptr ? 2 : 1;
  GradRequest rq;
  rq.X[0] = X0; rq.X[1] = X1;
  rq.Ht[0] = Ht0; rq.Ht[1] = Ht1;
  rq.C[0] = C0; rq.C[1] = np == 2 ? C1 : 0;
  rq.out[0] = out0; rq.out[1] = out1;
  rq.transposed[0] = transposed0; rq.transposed[1] = transposed1;
  rq.h_pitch = h_pitch; rq.part = part; rq.r = r; rq.accumulate = accumulate;
  bool ragged = false;
  for (int i = 0; i < np; ++i) ragged = ragged || (rq.C[i] % 64 != 0);
  if (ragged) {
    for (int i = 0; i < np; ++i)
      if (int rc = launch_grad_tile(rq.X[i], rq.Ht[i], h_pitch, rq.out[i], part, M, rq.C[i], r, rp, rq.transposed[i], accumulate, ds, st))
        return rc;
    return MCB_OK;
  }
  GradPlan plan;
  if (int rc = plan_grad2(rq, M, rp, ds->sm_count, kGradSmemBudget, ds, &plan)) return rc;
  const bool prof = profile_on();
  if (prof) profile_begin(kProfGrad, 2.0 * M * (rq.C[0] + rq.C[1]) * r, 2.0 * M * (rq.C[0] + rq.C[1]) + 2.0 * np * M * rp, st);
  lora_grad_umma_kernel<<<plan.p.n_cta, kGradThreads, kGradSmem, st>>>(plan.tmX[0], plan.tmH[0], plan.tmX[1], plan.tmH[1], plan.p);
  if (prof) profile_end(st);
  MCB_CHECK_LAUNCH("lora_grad_umma_kernel");
  return launch_grad_reduce(plan, st);
}

}  // namespace bf16path
}  // namespace mcb
