// LoRA weight gradients on tensor cores:  out[C, rp] = X[M, C]^T . H[M, rp]  (a reduction over tokens).
//
//   dA [K, r] = x^T  (scale * dy B^T)        X = x  [M,K],  H = the rank intermediate of the backward GEMM
//   dB [r, N] = (scale * x A)^T dy           X = dy [M,N],  H = the rank intermediate saved by the forward
//
// Both operands are token-major in memory, i.e. the reduction index is the SLOW one.  X tiles are loaded
// by TMA exactly as they lie ([64 tokens] x [64 features], 128-byte swizzle) and handed to tcgen05.mma as
// an MN-major A operand; H arrives already transposed ([rp, tokens], written that way by the GEMM
// epilogue) as a K-major B operand.  A CTA owns 128 features and one slice of the tokens, accumulates
// [128 x rp] in tensor memory and writes one float32 partial; a second small kernel sums the partials
// in slice order, so the result is deterministic.  The kernel is HBM-bound: it reads X once (2 bytes per
// element) and issues one 128 x rp x 16 MMA per 4 KB of it.
#include "lora_internal.cuh"
#include "umma_ptx.cuh"

namespace mcb {
namespace bf16path {
using namespace umma;
namespace {

constexpr int kGradThreads = 192;
constexpr int kGradBK = 64;       // tokens per stage
constexpr int kGradMaxStages = 12;  // enough bytes in flight per SM to cover HBM latency under load
constexpr int kGradSmemBudget = 216 * 1024;
constexpr uint32_t kXBoxBytes = 64 * 64 * 2;  // one [64 tokens x 64 features] box

struct GradParams {
  int M, C, rp;
  int total_kb, kb_per_split;
  float* part;  // [splits][C][rp]
  int* status;
  uint32_t stage_bytes, bar_off;
  int stages;
};

__global__ void __launch_bounds__(kGradThreads)
lora_grad_umma_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmH,
                      const GradParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = base + p.bar_off, empty0 = full0 + 8 * kGradMaxStages, done_bar = empty0 + 8 * kGradMaxStages;
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
        tma_load_2d(sb, &tmX, fb, c0, kb * kGradBK);
        tma_load_2d(sb + kXBoxBytes, &tmX, fb, c0 + 64, kb * kGradBK);
        tma_load_2d(sb + 2 * kXBoxBytes, &tmH, fb, kb * kGradBK, 0);
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
        for (int k4 = 0; k4 < kGradBK / 16; ++k4) {
          // A: 16 token rows further = 2 K-groups of 8 rows x 128 bytes; the second 64-feature atom is the
          // second box.  B: 16 tokens further along the contiguous dimension = 32 bytes.
          const uint64_t ad = desc_sw128_mn(sb + k4 * 2048, kXBoxBytes, 1024);
          const uint64_t bd = desc_sw128(sb + 2 * kXBoxBytes + k4 * 32);
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
__global__ void lora_grad_reduce_kernel(const float* __restrict__ part, float* __restrict__ out, int splits, int C,
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode(const DeviceState* ds, CUtensorMap* map, const void* ptr, int64_t inner, int64_t outer, int64_t pitch_elems,
           int box_inner, int box_outer, const char* what) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_elems) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ds->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MCB_ERR_ALIGN, "tensor map for %s rejected (CUresult %d)", what, static_cast<int>(r));
  return MCB_OK;
}

constexpr int kGradSmem = kGradSmemBudget + 1024 + 512;

}  // namespace

int init_grad_kernel() {
  cudaError_t e = cudaFuncSetAttribute(lora_grad_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGradSmem);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(lora_grad_umma_kernel)");
  return MCB_OK;
}

// Token slices per feature tile: at most one CTA per SM, all resident at once (measured: more, shorter CTAs
// lose to their set-up cost, and a second round of CTAs doubles the time).
int grad_splits(int64_t M, int64_t C, int sm_count, int* kb_per_split) {
  const int64_t c_tiles = (C + BM - 1) / BM;
  const int64_t total_kb = (M + kGradBK - 1) / kGradBK;
  int64_t target = static_cast<int64_t>(sm_count) / c_tiles;
  if (target > total_kb) target = total_kb;
  if (target < 1) target = 1;
  const int64_t per = (total_kb + target - 1) / target;
  if (kb_per_split) *kb_per_split = static_cast<int>(per);
  return static_cast<int>((total_kb + per - 1) / per);
}

size_t grad_partial_bytes(int64_t M, int64_t C, int rp) {
  return static_cast<size_t>(grad_splits(M, C, 256, nullptr)) * C * rp * sizeof(float);
}

// out = X^T H with H given transposed as Ht [rp, h_pitch] (token index contiguous).
int launch_grad(const __nv_bfloat16* X, const __nv_bfloat16* Ht, int64_t h_pitch, float* out, float* part, int64_t M,
                int64_t C, int r, int rp, int transposed, int accumulate, const DeviceState* ds, cudaStream_t st) {
  if (C % 8 != 0) return fail(MCB_ERR_ALIGN, "bf16 LoRA gradients need a feature count that is a multiple of 8 (got %lld)", (long long)C);
  if (!aligned16(X) || !aligned16(Ht) || h_pitch % 8 != 0) return fail(MCB_ERR_ALIGN, "bf16 LoRA gradients: operand alignment");
  GradParams p;
  p.M = static_cast<int>(M); p.C = static_cast<int>(C); p.rp = rp;
  p.total_kb = static_cast<int>((M + kGradBK - 1) / kGradBK);
  const int splits = grad_splits(M, C, ds->sm_count, &p.kb_per_split);
  p.part = part;
  p.status = ds->status_word;
  p.stage_bytes = 2 * kXBoxBytes + static_cast<uint32_t>(rp) * 128;
  p.stages = static_cast<int>(kGradSmemBudget / p.stage_bytes);
  if (p.stages > kGradMaxStages) p.stages = kGradMaxStages;
  p.bar_off = p.stages * p.stage_bytes;
  CUtensorMap tmX, tmH;
  if (int rc = encode(ds, &tmX, X, C, M, C, 64, kGradBK, "grad X")) return rc;
  if (int rc = encode(ds, &tmH, Ht, M, rp, h_pitch, kGradBK, rp, "grad H")) return rc;
  dim3 grid(static_cast<unsigned>((C + BM - 1) / BM), static_cast<unsigned>(splits));
  const bool prof = profile_on();
  if (prof) profile_begin(kProfGrad, 2.0 * M * C * r, 2.0 * M * C + 2.0 * M * rp, st);
  lora_grad_umma_kernel<<<grid, kGradThreads, kGradSmem, st>>>(tmX, tmH, p);
  if (prof) profile_end(st);
  MCB_CHECK_LAUNCH("lora_grad_umma_kernel");
  const int64_t n = C * rp;
  lora_grad_reduce_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(part, out, splits, static_cast<int>(C), r,
                                                                                   rp, transposed, accumulate);
  MCB_CHECK_LAUNCH("lora_grad_reduce");
  return MCB_OK;
}

}  // namespace bf16path
}  // namespace mcb
