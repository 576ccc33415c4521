// The token-reduction phase of the LoRA weight gradients, shared by the stand-alone gradient kernel
// (umma_grad.cu) and the backward GEMM kernel (umma_gemm.cu), which runs it as a tail phase in the same
// launch as dx.
//
//   out[C, rp] = X[M, C]^T . H[M, rp]       (dA: X = x, H = scale dy B^T;   dB: X = dy, H = scale x A)
//
// A CTA owns a slice of the tokens and a group of up to 1024 features of one of (at most) two problems, streams
// whole token rows of its group through a ring of shared-memory stages (one three-dimensional TMA copy per
// stage) and accumulates one [128 x rp] tile per 128 features in tensor memory; it leaves one float32 partial
// that a small second kernel sums in slice order.
#pragma once
#include <cuda.h>

#include "lora_internal.cuh"
#include "umma_ptx.cuh"

namespace mcb {
namespace bf16path {

constexpr int kGradMaxStages = 8;
constexpr int kGradGroup = 1024;               // features per CTA at most (8 tiles of 128)
constexpr int kGradSmemBudget = 208 * 1024;

struct GradProblem {
  int C, groups, slices, tiles;   // features, feature groups, token slices, 128-feature tiles per group
  int group_feats;                // features per group (a multiple of 128)
  float* part;                    // [slices][C][rp]
};
struct GradParams {
  int M, rp;                      // tokens, padded rank
  int T[2];                       // tokens per stage of each problem (a multiple of 16, at most 256)
  int stages[2];                  // stage ring depth of each problem
  int n_cta0, n_cta;              // CTAs of problem 0, CTAs of both problems
  GradProblem pr[2];
  int* status;
  uint32_t x_bytes[2], bar_off;   // X bytes per stage of each problem; H follows at x_bytes
  uint32_t stage_stride[2];
  // Tail-phase use only: problem 0's H is written by other CTAs of the same launch.  h_flags[mt] counts the
  // epilogue warps (4 per tile) that have stored the rows of 128-token tile mt; null when H is already there.
  const int* h_flags;
};

// What a CTA needs of its surroundings: the aligned shared-memory base of the stage ring, the barrier addresses,
// its tensor-memory allocation and the CTA-wide abort flag.
struct GradShared {
  uint32_t base, full0, empty0, done_bar, tmem_base;
  volatile int* abort_flag;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Bounded wait until *flag >= target (written by other CTAs with a release at gpu scope).
__device__ __forceinline__ bool flag_wait(const int* flag, int target, volatile int* abort_flag, int code, int* status) {
  const unsigned long long t0 = umma::globaltimer_ns();
  while (true) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= target) return true;
    if (*abort_flag != 0) return false;
    if (umma::globaltimer_ns() - t0 > umma::kWaitLimitNs) {
      *abort_flag = code;
      atomicCAS(status, 0, code);
      return false;
    }
    __nanosleep(200);
  }
}

// The three roles (warp 0: loads, warp 1: MMA issue, warps 2-5: partial store) for CTA number `cta` of the
// phase.  Contains no CTA-wide synchronisation; the barriers in `sh` must be freshly initialised.
__device__ __forceinline__ void grad_roles(const GradParams& p, const CUtensorMap* tmX0, const CUtensorMap* tmH0,
                                           const CUtensorMap* tmX1, const CUtensorMap* tmH1, const GradShared& sh,
                                           int cta) {
  using namespace umma;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int which = cta >= p.n_cta0 ? 1 : 0;
  const GradProblem& q = p.pr[which];
  const int local = cta - (which ? p.n_cta0 : 0);
  const int group = local % q.groups, slice = local / q.groups;
  const CUtensorMap* tmX = which ? tmX1 : tmX0;
  const CUtensorMap* tmH = which ? tmH1 : tmH0;

  // token steps of T tokens, split evenly over the slices
  const int T = p.T[which];
  const int n_stages = p.stages[which];
  const uint32_t stride = p.stage_stride[which];
  const int total_steps = (p.M + T - 1) / T;
  const int per = (total_steps + q.slices - 1) / q.slices;
  const int step_begin = slice * per;
  const int step_end = min(total_steps, step_begin + per);
  const int nsteps = max(0, step_end - step_begin);
  const uint32_t xb = p.x_bytes[which];
  const uint32_t atom_bytes = static_cast<uint32_t>(T) * 128;   // one 64-feature atom of a stage: T rows of 128 bytes

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const bool flagged = which == 0 && p.h_flags != nullptr;
      int next_mt = (step_begin * T) / BM;    // first 128-token tile not yet known to be written
      for (int s = step_begin; s < step_end; ++s) {
        if (flagged) {
          const int last_tok = min(p.M, (s + 1) * T) - 1;
          bool ok = true;
          for (; ok && next_mt <= last_tok / BM; ++next_mt) ok = flag_wait(p.h_flags + next_mt, 4, sh.abort_flag, 44, p.status);
          if (!ok) break;
          // the rows were written through the generic proxy; the copies below read them through the async proxy
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        if (!mbar_wait(sh.empty0 + 8 * stage, phase ^ 1, sh.abort_flag, 41, p.status)) break;
        const uint32_t fb = sh.full0 + 8 * stage, sb = sh.base + stage * stride;
        mbar_expect_tx(fb, xb + static_cast<uint32_t>(p.rp) * T * 2);
        // X: [64 features][T tokens][atoms of the group]; in shared memory atom-major blocks of T rows x 128 bytes
        tma_load_3d(sb, tmX, fb, 0, s * T, group * (q.group_feats / 64));
        // H^T: K-major B operand, unswizzled 16-byte columns of 8 tokens each
        for (int j = 0; j < T / 8; ++j) tma_load_2d(sb + xb + j * p.rp * 16, tmH, fb, s * T + j * 8, 0);
        if (++stage == n_stages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_a_mn(p.rp);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < nsteps; ++i) {
        ok = mbar_wait(sh.full0 + 8 * stage, phase, sh.abort_flag, 42, p.status);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t sb = sh.base + stage * stride;
        for (int k16 = 0; k16 < T / 16; ++k16) {
          // B: 16 tokens further = two 16-byte columns of rp rows
          const uint64_t bd = desc_noswz(sb + xb + k16 * 2 * (p.rp * 16), p.rp * 16, 128);
          for (int f = 0; f < q.tiles; ++f) {
            // A: tile f = atoms 2f, 2f+1 (LBO = one atom); 16 token rows further = two 8-row groups of 1024 bytes
            const uint64_t ad = desc_sw128_mn(sb + (2 * f) * atom_bytes + k16 * 2048, atom_bytes, 1024);
            umma_bf16(sh.tmem_base + f * p.rp, ad, bd, idesc, (i | k16) != 0 ? 1u : 0u);
          }
        }
        umma_commit(sh.empty0 + 8 * stage);
        if (++stage == n_stages) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(sh.done_bar);   // with no steps at all this completes at once
    }
  } else {
    const int quad = warp & 3;
    const bool ok = __all_sync(0xffffffffu, mbar_wait(sh.done_bar, 0, sh.abort_flag, 43, p.status));
    if (ok) {
      tcgen05_fence_after();
      const uint32_t taddr = sh.tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      for (int f = 0; f < q.tiles; ++f) {
        const int c = group * q.group_feats + f * BM + quad * 32 + lane;
        for (int j = 0; j < p.rp; j += 16) {
          uint32_t v[16];
          tmem_ld_x16(taddr + f * p.rp + j, v);
          tmem_ld_wait();
          if (c < q.C) {
            float4* o = reinterpret_cast<float4*>(q.part + (static_cast<int64_t>(slice) * q.C + c) * p.rp + j);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // a slice without steps has accumulated nothing (its tensor memory is undefined): write zeros
              o[e] = nsteps > 0 ? make_float4(__uint_as_float(v[4 * e]), __uint_as_float(v[4 * e + 1]),
                                              __uint_as_float(v[4 * e + 2]), __uint_as_float(v[4 * e + 3]))
                                : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
          }
        }
      }
    }
  }
}

// ---- host side -------------------------------------------------------------------------------------------
// Two gradient problems over the same M tokens (X1 == nullptr: one).  Ht_i is H_i transposed, [rp, h_pitch].
struct GradRequest {
  const __nv_bfloat16* X[2] = {nullptr, nullptr};
  const __nv_bfloat16* Ht[2] = {nullptr, nullptr};
  int64_t C[2] = {0, 0};
  float* out[2] = {nullptr, nullptr};
  int transposed[2] = {0, 0};   // 0: out[c*r + j] (dA [K,r]); 1: out[j*C + c] (dB [r,N])
  int64_t h_pitch = 0;
  float* part = nullptr;        // workspace for the partial sums (grad_partial_bytes)
  int r = 0, accumulate = 0;
  int* h_flags = nullptr;       // tail phase: per 128-token tile counters for problem 0's H, zeroed before the launch
};
struct GradPlan {
  GradParams p;
  CUtensorMap tmX[2], tmH[2];
  int np = 0;
  GradRequest rq;
};
// Whether the two problems can run as the tail phase of the backward GEMM (one feature group each).
bool grad_tail_possible(int64_t C0, int64_t C1, int rp);
// Lays the problems out over at most max_ctas CTAs with smem_budget bytes of stage ring each.
int plan_grad2(const GradRequest& rq, int64_t M, int rp, int max_ctas, uint32_t smem_budget, const DeviceState* ds,
               GradPlan* plan);
// Sums the partials the planned CTAs have written into out (+)= .
int launch_grad_reduce(const GradPlan& plan, cudaStream_t st);

}  // namespace bf16path
}  // namespace mcb
