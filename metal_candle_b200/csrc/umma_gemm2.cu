// Linear with optional LoRA rank path
//     Y[M,N] = X[M,K] . W[N,K]^T (+ bias) (+ residual) + (scale X P^T) Q^T
// on CTA pairs (tcgen05 cta_group::2).
//
// The one-CTA kernel of umma_gemm.cu moves 48 KB from L2 per 128x256 tile and k-block and can hold only
// four such stages, which leaves the tensor pipe waiting for loads about a third of the time.  Here two
// CTAs of a cluster (two neighbouring SMs) own one 256 x BN tile: each loads its own 128 rows of X and
// HALF of the W tile (BN/2 rows), the pair's leader issues one tcgen05.mma.cta_group::2 (M = 256) that
// reads both halves from both CTAs' shared memory, and each CTA finds its 128 x BN accumulator rows in
// its own tensor memory.  Per SM and k-block that is 32 KB instead of 48 KB, and six stages fit.
//
// Rank path (rp > 0).  Each CTA puts its half of P (rp/2 rows) directly behind its half of W in a stage, so
// the pair's B operand has BN + rp rows and one MMA fills the accumulator columns
//     [ W half 0 : BN/2 | rank half 0 : rp/2 | W half 1 : BN/2 | rank half 1 : rp/2 ].
// The epilogue warps of each CTA scale the rank columns of their own 128 rows, round them to bf16 into an
// unswizzled K-major operand in their own shared memory (and store them transposed to H for the
// weight-gradient kernel), and the leader then adds  H . Q^T  onto the two W halves with two more pair
// MMAs per 16 rank columns, each CTA holding a quarter-tile of Q rows for either half.
//
// Synchronisation (no load uses cluster multicast):
//   full[s]      in the LEADER: the leader's producer arms it for the bytes of BOTH CTAs; both producers'
//                TMA loads (cp.async.bulk.tensor...cta_group::2) complete on it
//   empty[s]     in each CTA: tcgen05.commit.cta_group::2 ... multicast::cluster from the leader's MMA thread
//   d2_full[a]   in each CTA: same commit after the last k-block of a tile (rank columns complete)
//   h_ready[a]   in the LEADER: 8 arrivals (epilogue warps of both CTAs) once the bf16 rank operand is in place
//   q_full[a]    in the LEADER: the Q quarter-tiles of both CTAs have landed
//   d1_full[a]   in each CTA: same commit, after the rank update (or the last k-block when rp == 0)
//   acc_empty[a] in the LEADER: 8 arrivals, the 4 epilogue warps of each CTA (the peer's arrive remotely); 16 in the
//                SwiGLU-backward form, which runs 8 epilogue warps per CTA
//   gu_full[q][s] in each CTA (SwiGLU-backward form): the gate and up boxes of rows 32q.. have landed in buffer pair s
//   hb[q][s]     in each CTA (same form): the helper warp of rows 32q.. has written its half of pair s
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
constexpr int kThreads2Wide = 320;  // SwiGLU-backward form: a second set of four epilogue warps
constexpr int kMaxStages2 = 8;
constexpr int kSmem2 = 227 * 1024 - 1024;
constexpr int kEpiBufs = kEpiBufsMax;

struct Gemm2Params {
  int M, N, K;
  int BN, stages, rp;
  int pdl_wait; // 1: launched as a programmatic dependent of the operand-pack kernel
  int swiglu;   // 1: the tile is [128 gate columns | 128 up columns]; the epilogue also writes silu(gate) * up
                // 2: the product is d act of a SwiGLU; the epilogue turns it into d gate and d up (see U) and stores those
  int epi_bufs; // 2-KB staging buffers per 32 rows of the tile (kEpiBufs; 12 in the SwiGLU-backward form)
  int sw_pairs, sw_ahead;  // SwiGLU backward: buffer pairs per 32 rows, jobs loaded ahead
  int num_m_tiles, num_n_tiles, num_tiles, num_k_blocks, group_m;  // m tiles of 256 rows
  float scale;
  __nv_bfloat16* Y;
  __nv_bfloat16* U;  // swiglu == 2: Y holds gate and U holds up [M,N] on entry, d gate and d up on return
  const __nv_bfloat16* bias;
  const __nv_bfloat16* R;
  __nv_bfloat16* H;  // [rp, h_pitch]: scale * X P^T transposed, or null
  int64_t h_pitch;
  int* status;
  uint32_t stage_bytes, w_off, p_off, bar_off;
  uint32_t epi_off;  // output staging: 4 row groups x epi_bufs buffers of 32 rows x 64 bytes
  uint32_t q_off, q_bytes, hs_off, hs_bytes;  // per CTA and accumulator buffer; q_bytes covers both halves' quarter-tiles
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

// Two neighbouring elements of the SwiGLU backward: d gate = d u s (1 + g (1 - s)), d up = d g s with s = sigmoid(g).
// The epilogue warps are bound by their instruction count, so: the two approximate special functions flush
// denormals (the compiler then adds no range handling around them; relative error about 2^-22), products are shared
// between the two results, and the multiplies and adds run as packed pairs (one instruction for two elements).
// g -> -inf gives s = 0 and both results 0; g -> +inf gives s = 1, d gate = d u, d up = d g.
__device__ __forceinline__ void swiglu_bwd_pair(float2 d, float2 g, float2 u, float2& dgate, float2& dup) {
  const float2 a = __fmul2_rn(g, make_float2(-1.4426950408889634f, -1.4426950408889634f));
  float2 e, s;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(a.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(a.y));
  e = __fadd2_rn(e, make_float2(1.0f, 1.0f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(s.x) : "f"(e.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(s.y) : "f"(e.y));
  const float2 t = __fmul2_rn(d, s);
  dup = __fmul2_rn(t, g);
  const float2 q = __ffma2_rn(make_float2(-g.x, -g.y), s, g);   // g (1 - s)
  const float2 tu = __fmul2_rn(t, u);
  dgate = __ffma2_rn(tu, q, tu);
}

// silu(g) * u with the same two flushing special functions (5 instructions)
__device__ __forceinline__ float silu_mul(float g, float u) {
  float e, s;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(s) : "f"(1.0f + e));
  return g * s * u;
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

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2Wide, 1)
lora_gemm2_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                  const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                  const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmU,
                  const __grid_constant__ CUtensorMap tmAct, const __grid_constant__ CUtensorMap tmY64,
                  const __grid_constant__ CUtensorMap tmU64, const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  const uint32_t full0 = base + p.bar_off;
  const uint32_t empty0 = full0 + 8 * kMaxStages2;
  const uint32_t d1_full0 = empty0 + 8 * kMaxStages2;
  const uint32_t acc_empty0 = d1_full0 + 16;
  const uint32_t d2_full0 = acc_empty0 + 16;
  const uint32_t h_ready0 = d2_full0 + 16;
  const uint32_t q_full0 = h_ready0 + 16;
  const uint32_t tmem_slot = q_full0 + 16;
  const uint32_t abort_addr = tmem_slot + 4;
  const uint32_t gu_full0 = tmem_slot + 8;   // SwiGLU backward: 4 epilogue warps x 4 buffer pairs, "gate and up have landed"
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_addr - base));

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int a = 0; a < 2; ++a) {
      mbar_init(d1_full0 + 8 * a, 1);
      mbar_init(acc_empty0 + 8 * a, 8 * ((blockDim.x >> 5) > 6 ? 2 : 1));   // every epilogue warp of both CTAs
      mbar_init(d2_full0 + 8 * a, 1);
      mbar_init(h_ready0 + 8 * a, 8);
      mbar_init(q_full0 + 8 * a, 1);
    }
    if (p.swiglu == 2)
      for (int b = 0; b < 32; ++b) mbar_init(gu_full0 + 8 * b, 1);
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
  const int half_n = p.BN / 2, half_r = p.rp / 2, quarter_n = p.BN / 4;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int i = 0;
      if (p.pdl_wait) grid_dependency_wait();   // the operand-pack kernel has finished
      for (int t = pair; ok && t < p.num_tiles; t += npairs, ++i) {
        int mt, nt;
        tile_coords2(p, t, mt, nt);
        const int m0 = mt * 256 + static_cast<int>(rank) * 128;
        const int n0 = nt * p.BN + static_cast<int>(rank) * half_n;
        if (p.rp > 0) {
          // Q buffer a is free once the rank update of the tile before last has been read by the tensor pipe
          const int a = i & 1;
          if (i >= 2) ok = mbar_wait(d1_full0 + 8 * a, ((i - 2) >> 1) & 1, abort_flag, 60, p.status);
          if (!ok) break;
          const uint32_t qb = map_to_cta(q_full0 + 8 * a, 0);
          if (rank == 0) mbar_expect_tx(q_full0 + 8 * a, 2 * p.q_bytes);
          const uint32_t qs = base + p.q_off + a * p.q_bytes;
          for (int h = 0; h < 2; ++h) {
            const int rows0 = nt * p.BN + h * half_n + static_cast<int>(rank) * quarter_n;
            for (int j = 0; j < p.rp / 8; ++j)
              tma_load_2d_pair(qs + h * (p.q_bytes / 2) + j * quarter_n * 16, &tmQ, qb, j * 8, rows0);
          }
        }
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, 61, p.status);
          if (!ok) break;
          const uint32_t fb = map_to_cta(full0 + 8 * stage, 0);  // the leader's barrier
          const uint32_t sb = base + stage * p.stage_bytes;
          if (rank == 0) mbar_expect_tx(full0 + 8 * stage, 2 * p.stage_bytes);
          tma_load_2d_pair(sb, &tmX, fb, kb * BK2, m0);
          tma_load_2d_pair(sb + p.w_off, &tmW, fb, kb * BK2, n0);
          if (p.rp > 0) tma_load_2d_pair(sb + p.p_off, &tmP, fb, kb * BK2, static_cast<int>(rank) * half_r);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc2(p.BN + p.rp);
      const uint32_t idesc_half = make_idesc2(half_n);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int i = 0;
      // The rank update of a tile waits for the epilogue warps of both CTAs to turn the rank accumulator into the
      // bf16 operand.  Meanwhile this thread goes on with the next tile's main loop in the other accumulator
      // buffer and polls between k-blocks; the update is issued as soon as its operands are there.
      int pend_a = -1;
      uint32_t pend_u = 0;
      auto finish_pending = [&]() -> bool {
        const int pa = pend_a;
        pend_a = -1;
        if (!mbar_wait(h_ready0 + 8 * pa, pend_u & 1, abort_flag, 65, p.status)) return false;
        if (!mbar_wait(q_full0 + 8 * pa, pend_u & 1, abort_flag, 66, p.status)) return false;
        asm volatile("fence.acq_rel.cluster;" ::: "memory");
        tcgen05_fence_after();
        const uint32_t pd = tmem_base + pa * 256;
        const uint32_t hs = base + p.hs_off + pa * p.hs_bytes;
        const uint32_t qs = base + p.q_off + pa * p.q_bytes;
        for (int kk = 0; kk < p.rp / 16; ++kk) {
          const uint64_t hd = desc_noswz(hs + kk * 2 * (128 * 16), 128 * 16, 128);
          const uint64_t q0 = desc_noswz(qs + kk * 2 * (quarter_n * 16), quarter_n * 16, 128);
          const uint64_t q1 = desc_noswz(qs + p.q_bytes / 2 + kk * 2 * (quarter_n * 16), quarter_n * 16, 128);
          umma2_bf16(pd, hd, q0, idesc_half, 1u);
          umma2_bf16(pd + half_n + half_r, hd, q1, idesc_half, 1u);
        }
        umma2_commit_both(d1_full0 + 8 * pa);
        return true;
      };
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
          if (pend_a >= 0 && mbar_try_wait(h_ready0 + 8 * pend_a, pend_u & 1) &&
              mbar_try_wait(q_full0 + 8 * pend_a, pend_u & 1)) {
            ok = finish_pending();   // both operands are there: does not wait
            if (!ok) break;
          }
        }
        if (!ok) break;
        if (p.rp > 0) {
          umma2_commit_both(d2_full0 + 8 * a);
          if (pend_a >= 0) {         // the previous tile's update has still not been issued: wait for it now
            ok = finish_pending();
            if (!ok) break;
          }
          pend_a = a;
          pend_u = u;
        } else {
          umma2_commit_both(d1_full0 + 8 * a);
        }
      }
      if (ok && pend_a >= 0) ok = finish_pending();
    }
  } else {
    // ---------------- epilogue (warps 2 and up, both CTAs): own 128 rows of the pair's tile ----------------
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t epi_base = base + p.epi_off + static_cast<uint32_t>(quad * p.epi_bufs) * kEpiBufBytes;
    int sbuf = 0;
    // SwiGLU backward (swiglu == 2), launched with four more warps: warps 2..5 lead, warps 6..9 help the leader of the
    // same 32 rows (one warp per scheduler issues an instruction about every fourth cycle on this dependent
    // arithmetic; two per scheduler hide each other's latencies).  The 64-column pieces of a quad's rows over all its
    // tiles form one sequence of jobs.  Job j stages 32 rows x 64 columns of gate and of up (128-byte rows: half as
    // many TMA row requests as 32-column boxes) in the buffer pair j % np by two TMA loads that the leader issues
    // `ahead` jobs early; leader and helper each turn 32 of the 64 columns into d gate and d up in place, the helper
    // reports on an mbarrier, and the leader sends the pair off with two TMA stores.  A piece with only 32 columns
    // left in the tile (or the matrix) uses the 32-column boxes in the same buffers and the leader alone.
    const bool helper = warp >= 6;
    const int jw = 64, pair_bufs = 4;   // columns per job; 2-KB buffers per pair (gate 4 KB + up 4 KB)
    const int cset = (p.BN + jw - 1) / jw;   // jobs per tile
    const int np = p.sw_pairs, ahead = p.sw_ahead;
    const int pending = min(2, np - ahead - 1);   // store groups that may still be reading their pair
    const uint32_t gu_bar0 = gu_full0 + static_cast<uint32_t>(quad * np) * 8;
    const uint32_t hb_bar0 = gu_full0 + static_cast<uint32_t>(16 + quad * np) * 8;   // per pair: "the helper's half is in place"
    uint32_t gu_parity = 0, hb_parity = 0;   // bit s: parity of the next completion of pair s's barrier
    // columns of piece c of a tile at column n0 that exist: 64, 32 (a lone half) or <= 0 (none)
    auto piece_cols = [&](int n0_, int c) { return min(jw, min(p.BN - c, p.N - (n0_ + c))); };
    // the load cursor (lane 0) runs `ahead` jobs in front of the consumer; both step through tiles, pieces and
    // buffer pairs by increments (the tile coordinates, with their divisions, once per tile)
    int pf_t = pair, pf_k = 0, pf_slot = 0, pf_row0 = 0, pf_n0 = 0;
    auto pf_tile = [&]() {
      if (pf_t >= p.num_tiles) return;
      int mt2, nt2;
      tile_coords2(p, pf_t, mt2, nt2);
      pf_row0 = mt2 * 256 + static_cast<int>(rank) * 128 + quad * 32;
      pf_n0 = nt2 * p.BN;
    };
    auto gu_issue_next = [&]() {
      if (pf_t >= p.num_tiles) return;
      const int c = pf_k * jw;
      const int cols = piece_cols(pf_n0, c);
      if (pf_row0 < p.M && cols > 0) {   // the consumer skips the same jobs
        const uint32_t buf = epi_base + static_cast<uint32_t>(pair_bufs * pf_slot) * kEpiBufBytes;
        const uint32_t half = static_cast<uint32_t>(pair_bufs >> 1) * kEpiBufBytes;
        const uint32_t bar = gu_bar0 + 8 * pf_slot;
        if (cols > 32) {
          mbar_expect_tx(bar, 4 * kEpiBufBytes);   // a box clipped at the edges still counts in full
          tma_load_2d(buf, &tmY64, bar, pf_n0 + c, pf_row0);
          tma_load_2d(buf + half, &tmU64, bar, pf_n0 + c, pf_row0);
        } else {
          mbar_expect_tx(bar, 2 * kEpiBufBytes);
          tma_load_2d(buf, &tmY, bar, pf_n0 + c, pf_row0);
          tma_load_2d(buf + half, &tmU, bar, pf_n0 + c, pf_row0);
        }
      }
      if (++pf_slot == np) pf_slot = 0;
      if (++pf_k == cset) { pf_k = 0; pf_t += npairs; pf_tile(); }
    };
    if (p.swiglu == 2 && lane == 0 && !helper) {
      if (p.pdl_wait) grid_dependency_wait();   // gate and up may come from the kernel before the operand pack
      pf_tile();
      for (int j = 0; j < ahead; ++j) gu_issue_next();
    }
    int sl = 0;   // the consumer's buffer pair
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
      if (p.rp > 0 && !helper) {
        ok = __all_sync(0xffffffffu, mbar_wait(d2_full0 + 8 * a, u & 1, abort_flag, 67, p.status));
        if (!ok) break;
        tcgen05_fence_after();
        uint8_t* hs_gen = gen_base + p.hs_off + a * p.hs_bytes;
        for (int h = 0; h < 2; ++h) {
          const uint32_t tcol = d + (h == 0 ? half_n : p.BN + half_r);
          for (int g = 0; g < half_r / 8; ++g) {
            uint32_t v[8];
            tmem_ld_x8(tcol + 8 * g, v);
            tmem_ld_wait();
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              w[j] = pack_bf16(__uint_as_float(v[2 * j]) * p.scale, __uint_as_float(v[2 * j + 1]) * p.scale);
            // unswizzled K-major operand: 16-byte K chunk j of row m lives at j*(128*16) + m*16
            const int chunk = h * (half_r / 8) + g;
            *reinterpret_cast<uint4*>(hs_gen + chunk * (128 * 16) + row_in_tile * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            if (p.H != nullptr && nt == 0 && grow < p.M) {
              __nv_bfloat16* hp = p.H + static_cast<int64_t>(chunk * 8) * p.h_pitch + grow;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                hp[(2 * j) * p.h_pitch] = __ushort_as_bfloat16(static_cast<unsigned short>(w[j] & 0xffffu));
                hp[(2 * j + 1) * p.h_pitch] = __ushort_as_bfloat16(static_cast<unsigned short>(w[j] >> 16));
              }
            }
          }
        }
        fence_proxy_async_smem();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) mbar_arrive(h_ready0 + 8 * a);
          else mbar_arrive_remote(h_ready0 + 8 * a, 0);
        }
      }
      ok = __all_sync(0xffffffffu, mbar_wait(d1_full0 + 8 * a, u & 1, abort_flag, 64, p.status));
      if (!ok) break;
      tcgen05_fence_after();
      if (p.swiglu == 2) {
        // d gate = d act * up * silu'(gate), d up = d act * silu(gate), d act straight from the float32 accumulator
        const bool rows_ok = m0 + quad * 32 < p.M;
        for (int k = 0; k < cset; ++k) {
          const int c = k * jw, gcol = n0 + c;
          if (lane == 0 && !helper) {
            bulk_wait_group_read_n(pending);   // the stores that last used the pair the next load goes into have read it
            gu_issue_next();
          }
          const int cols = piece_cols(n0, c);
          if (rows_ok && cols > 0) {
            const bool wide = cols > 32;
            const uint32_t buf = epi_base + static_cast<uint32_t>(pair_bufs * sl) * kEpiBufBytes;
            const uint32_t half = static_cast<uint32_t>(pair_bufs >> 1) * kEpiBufBytes;
            uint8_t* bg = gen_base + (buf - base);
            uint8_t* bu = bg + half;
            if (wide || !helper) {
              const int h = helper ? 1 : 0, cc = c + 32 * h;
              uint32_t v0[16], v1[16];
              tmem_ld_x16(d + (cc < half_n ? cc : cc + half_r), v0);
              tmem_ld_x16(d + (cc + 16 < half_n ? cc + 16 : cc + 16 + half_r), v1);
              ok = __all_sync(0xffffffffu, mbar_wait(gu_bar0 + 8 * sl, (gu_parity >> sl) & 1u, abort_flag, 68, p.status));
              if (!ok) break;
              uint32_t gw[16], uw[16];
              if (wide) { unstage_half128(bg, lane, h, gw); unstage_half128(bu, lane, h, uw); }
              else { unstage_row(bg, lane, gw); unstage_row(bu, lane, uw); }
              tmem_ld_wait();
              uint32_t wg[16], wu[16];
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const float2 dd = make_float2(__uint_as_float(e < 8 ? v0[2 * e] : v1[2 * e - 16]),
                                              __uint_as_float(e < 8 ? v0[2 * e + 1] : v1[2 * e - 15]));
                float2 dg, du;
                swiglu_bwd_pair(dd, make_float2(__uint_as_float(gw[e] << 16), __uint_as_float(gw[e] & 0xffff0000u)),
                                make_float2(__uint_as_float(uw[e] << 16), __uint_as_float(uw[e] & 0xffff0000u)), dg, du);
                wg[e] = pack_bf16(dg.x, dg.y);
                wu[e] = pack_bf16(du.x, du.y);
              }
              if (wide) { stage_half128(bg, lane, h, wg); stage_half128(bu, lane, h, wu); }
              else { stage_row(bg, lane, wg); stage_row(bu, lane, wu); }
              fence_proxy_async_smem();
              __syncwarp();
              if (helper) {
                if (lane == 0) mbar_arrive(hb_bar0 + 8 * sl);
              } else {
                if (wide) {
                  ok = __all_sync(0xffffffffu, mbar_wait(hb_bar0 + 8 * sl, (hb_parity >> sl) & 1u, abort_flag, 69, p.status));
                  if (!ok) break;
                  hb_parity ^= 1u << sl;
                }
                if (lane == 0) {
                  tma_store_2d(wide ? &tmY64 : &tmY, buf, gcol, m0 + quad * 32);
                  tma_store_2d(wide ? &tmU64 : &tmU, buf + half, gcol, m0 + quad * 32);
                }
              }
            }
            gu_parity ^= 1u << sl;   // the pair's barrier has completed once more, whether or not this warp waited on it
          }
          if (lane == 0 && !helper) bulk_commit_group();   // one group per job, empty or not: the wait above counts groups
          if (++sl == np) sl = 0;
        }
        if (!ok) break;
      } else if (p.swiglu) {
        // SwiGLU tile: accumulator columns [0, 128) are gate features nt*128.., columns [128, 256) the same
        // features of up.  Per 32 features: gate, up and silu(gate)*up go out through three staging buffers.
        const int F = p.N >> 1;
        for (int c = 0; c < 128; c += 32) {
          const int fcol = nt * 128 + c;
          if (fcol >= F) break;
          uint32_t g0[16], g1[16], u0[16], u1[16];
          tmem_ld_x16(d + c, g0);
          tmem_ld_x16(d + c + 16, g1);
          tmem_ld_x16(d + 128 + c, u0);
          tmem_ld_x16(d + 128 + c + 16, u1);
          if (lane == 0) bulk_wait_group_read<0>();  // all three staging buffers have been read
          __syncwarp();
          tmem_ld_wait();
          uint32_t wg[16], wu[16], wa[16];
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const float ga = __uint_as_float(g0[j]), gb = __uint_as_float(g0[j + 1]);
            const float ua = __uint_as_float(u0[j]), ub = __uint_as_float(u0[j + 1]);
            wg[j >> 1] = pack_bf16(ga, gb);
            wu[j >> 1] = pack_bf16(ua, ub);
            wa[j >> 1] = pack_bf16(silu_mul(ga, ua), silu_mul(gb, ub));
            const float gc = __uint_as_float(g1[j]), gd = __uint_as_float(g1[j + 1]);
            const float uc = __uint_as_float(u1[j]), ud = __uint_as_float(u1[j + 1]);
            wg[8 + (j >> 1)] = pack_bf16(gc, gd);
            wu[8 + (j >> 1)] = pack_bf16(uc, ud);
            wa[8 + (j >> 1)] = pack_bf16(silu_mul(gc, uc), silu_mul(gd, ud));
          }
          stage_row(gen_base + (epi_base - base), lane, wg);
          stage_row(gen_base + (epi_base - base) + kEpiBufBytes, lane, wu);
          stage_row(gen_base + (epi_base - base) + 2 * kEpiBufBytes, lane, wa);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && m0 + quad * 32 < p.M) {
            tma_store_2d(&tmY, epi_base, fcol, m0 + quad * 32);
            tma_store_2d(&tmU, epi_base + kEpiBufBytes, fcol, m0 + quad * 32);
            tma_store_2d(&tmAct, epi_base + 2 * kEpiBufBytes, fcol, m0 + quad * 32);
            bulk_commit_group();
          }
        }
      } else
      // The W halves sit at columns [0, BN/2) and [BN/2 + rp/2, BN + rp/2) of the accumulator.  Output leaves in
      // chunks of 32 columns: each thread rounds its row's 64 bytes into this warp's staging buffer (64-byte
      // swizzle, conflict-free) and one tiled store per chunk writes 32 rows x 64 bytes, clipped at the edges.
      {
      for (int c = 0; c < p.BN; c += 32) {
        const int gcol = n0 + c;
        if (gcol >= p.N) break;
        uint32_t v0[16], v1[16];
        tmem_ld_x16(d + (c < half_n ? c : c + half_r), v0);
        tmem_ld_x16(d + (c + 16 < half_n ? c + 16 : c + 16 + half_r), v1);
        if (lane == 0) bulk_wait_group_read<kEpiBufs - 1>();  // the store that last used this buffer has read it
        __syncwarp();
        tmem_ld_wait();
        float f[32];
#pragma unroll
        for (int j = 0; j < 16; ++j) { f[j] = __uint_as_float(v0[j]); f[16 + j] = __uint_as_float(v1[j]); }
        uint32_t w[16];
        finish_cols(f, p.bias, p.R, grow, gcol, p.M, p.N, w);
        const uint32_t buf = epi_base + static_cast<uint32_t>(sbuf) * kEpiBufBytes;
        stage_row(gen_base + (buf - base), lane, w);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && m0 + quad * 32 < p.M) {
          tma_store_2d(&tmY, buf, gcol, m0 + quad * 32);
          bulk_commit_group();
        }
        if (++sbuf == kEpiBufs) sbuf = 0;
      }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(acc_empty0 + 8 * a);
        else mbar_arrive_remote(acc_empty0 + 8 * a, 0);
      }
    }
    if (lane == 0) bulk_wait_group<0>();  // this warp's output stores are complete before the CTA may exit
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

int make_map2(const DeviceState* ds, CUtensorMap* map, const void* ptr, int64_t inner, int64_t outer, int box_inner,
              int box_outer, int swizzle_bytes, const char* what) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(inner) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn2>(ds->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE,
      swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MCB_ERR_ALIGN, "tensor map for %s rejected (CUresult %d)", what, static_cast<int>(r));
  return MCB_OK;
}

}  // namespace

int init_gemm2_kernel() {
  cudaError_t e = cudaFuncSetAttribute(lora_gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2 + 1024);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(lora_gemm2_kernel)");
  return MCB_OK;
}

// Whether the pair kernel takes this call (everything else stays on the one-CTA kernel): a main product
// with an output, large enough to fill CTA pairs; with a rank path, rank padded to a multiple of 16 and at
// most 64 and a long enough reduction.
bool gemm2_eligible(const GemmCall& c) {
  if (c.W == nullptr || c.Y == nullptr || c.M < 1024 || c.N < 128 || c.K < 64) return false;
  if (c.rp == 0) return true;
  // Short reductions stay on the one-CTA kernel.  Alone, the pair is a little ahead even there once the rank
  // update is issued between the next tile's k-blocks (32768x896x896 r16 forward 953 against 922 TFLOP/s), but
  // inside the training step, with its k/v projections of 128 outputs and its backward calls, the one-CTA kernel
  // measured 1-2 % faster per step on the same box (116.1-118.5 against 118.4-119.5 ms).
  return c.rp % 16 == 0 && c.rp <= 64 && c.K >= option(MCB_OPT_PAIR_MIN_K);
}

int launch_gemm2(const GemmCall& c, const DeviceState* ds, cudaStream_t st) {
  const int64_t M = c.M, N = c.N, K = c.K;
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.rp = c.rp;
  p.scale = c.scale;
  // tile width: fewest n-tiles that leave room for the rank columns in a 256-column accumulator, evened
  // out, multiple of 32 (each half a multiple of 16, each quarter a multiple of 8)
  const int cap = ((256 - c.rp) / 32) * 32;
  const int64_t tiles = (N + cap - 1) / cap;
  int bn = static_cast<int>(((N + tiles - 1) / tiles + 31) / 32 * 32);
  if (bn > cap) bn = cap;
  if (bn < 32) bn = 32;
  p.BN = bn;
  p.num_m_tiles = static_cast<int>((M + 255) / 256);
  p.num_n_tiles = static_cast<int>((N + bn - 1) / bn);
  p.num_tiles = p.num_m_tiles * p.num_n_tiles;
  p.num_k_blocks = static_cast<int>((K + BK2 - 1) / BK2);
  p.group_m = p.num_m_tiles < 8 ? p.num_m_tiles : 8;
  p.Y = c.Y; p.bias = c.bias; p.R = c.R; p.H = c.H; p.h_pitch = c.h_pitch; p.status = ds->status_word;
  p.epi_bufs = kEpiBufs;
  bool helpers = false;   // launch the four helper epilogue warps of the SwiGLU-backward form
  if (c.swiglu_up != nullptr) {
    if (c.bias != nullptr || c.R != nullptr)
      return fail(MCB_ERR_UNSUPPORTED, "pair GEMM: the SwiGLU-backward epilogue takes neither bias nor residual");
    p.swiglu = 2;
    p.U = c.swiglu_up;
    p.sw_pairs = 3; p.sw_ahead = 1;
    helpers = true;
    p.epi_bufs = p.sw_pairs * 4;   // per 32 rows: pairs of two buffers of 32 rows x 128 bytes (gate, up)
  }
  const uint32_t x_bytes = 128 * BK2 * 2, w_bytes = static_cast<uint32_t>(bn / 2) * BK2 * 2;
  const uint32_t p_bytes = static_cast<uint32_t>(c.rp / 2) * BK2 * 2;  // 8-row groups: a multiple of 1024
  p.w_off = x_bytes;
  p.p_off = x_bytes + w_bytes;
  p.stage_bytes = x_bytes + w_bytes + p_bytes;
  p.q_bytes = static_cast<uint32_t>(bn / 2) * c.rp * 2;
  p.hs_bytes = 128u * c.rp * 2;
  const uint32_t epi_bytes = 4u * static_cast<uint32_t>(p.epi_bufs) * kEpiBufBytes;
  const uint32_t fixed = 2 * p.q_bytes + 2 * p.hs_bytes + epi_bytes + 512;
  int stages = static_cast<int>((kSmem2 - fixed) / p.stage_bytes);
  if (stages > kMaxStages2) stages = kMaxStages2;
  if (stages < 2) return fail(MCB_ERR_UNSUPPORTED, "pair GEMM: tile does not fit shared memory (BN=%d rp=%d)", bn, c.rp);
  p.stages = stages;
  p.q_off = stages * p.stage_bytes;
  p.hs_off = p.q_off + 2 * p.q_bytes;
  p.epi_off = p.hs_off + 2 * p.hs_bytes;  // a multiple of 1024, as the swizzled staging rows need
  p.bar_off = p.epi_off + epi_bytes;
  CUtensorMap tmX, tmW, tmP, tmQ, tmY, tmU, tmY64, tmU64;
  if (int rc = make_map2(ds, &tmY, c.Y, N, M, 32, 32, 64, "Y (pair)")) return rc;
  if (c.swiglu_up != nullptr) {
    if (int rc = make_map2(ds, &tmU, c.swiglu_up, N, M, 32, 32, 64, "up (pair)")) return rc;
    if (int rc = make_map2(ds, &tmY64, c.Y, N, M, 64, 32, 128, "gate, 64 columns (pair)")) return rc;
    if (int rc = make_map2(ds, &tmU64, c.swiglu_up, N, M, 64, 32, 128, "up, 64 columns (pair)")) return rc;
  } else {
    tmU = tmY; tmY64 = tmY; tmU64 = tmY;
  }
  if (int rc = make_map2(ds, &tmX, c.X, K, M, BK2, 128, 128, "X (pair)")) return rc;
  if (int rc = make_map2(ds, &tmW, c.W, K, N, BK2, bn / 2, 128, "W (pair)")) return rc;
  if (c.rp > 0) {
    if (int rc = make_map2(ds, &tmP, c.P, K, c.rp, BK2, c.rp / 2, 128, "P (pair)")) return rc;
    if (int rc = make_map2(ds, &tmQ, c.Q, c.rp, N, 8, bn / 4, 0, "Q (pair)")) return rc;
  } else { tmP = tmX; tmQ = tmX; }
  int pairs = ds->sm_count / 2;
  if (pairs > p.num_tiles) pairs = p.num_tiles;
  const bool prof = profile_on();
  if (prof) {
    const double m = static_cast<double>(M), n = static_cast<double>(N), k = static_cast<double>(K);
    profile_begin(c.swiglu_up != nullptr ? kProfGemmSwigluBwd : c.rp > 0 ? kProfGemmLora : kProfGemm,
                  2.0 * m * n * k + 2.0 * m * c.r_true * (k + n),
                  2.0 * (m * k + n * k + (c.swiglu_up != nullptr ? 4.0 : 1.0) * m * n) + 2.0 * c.rp * (k + n), st);
  }
  const bool pdl = c.after_pack && c.rp > 0 && !prof && option(MCB_OPT_PDL) != 0;
  p.pdl_wait = pdl ? 1 : 0;
  {
    const cudaError_t le = launch_kernel(lora_gemm2_kernel, dim3(2 * pairs), dim3(helpers ? kThreads2Wide : kThreads2), kSmem2 + 1024, st, pdl, tmX, tmW, tmP,
                                         tmQ, tmY, tmU, tmY, tmY64, tmU64, p);
    if (le != cudaSuccess) return cuda_fail(le, "lora_gemm2_kernel launch");
  }
  if (prof) profile_end(st);
  MCB_CHECK_LAUNCH("lora_gemm2_kernel");
  return MCB_OK;
}

// gate, up, act [M, F] = x [M, K] . w_gu^T with w_gu [2F, K] holding the gate and up weights interleaved in blocks
// of 128 rows (gate rows f0..f0+127, then up rows f0..f0+127), and act = silu(gate) * up.
int launch_gemm2_swiglu(const __nv_bfloat16* X, const __nv_bfloat16* Wgu, __nv_bfloat16* G, __nv_bfloat16* U,
                        __nv_bfloat16* Act, int64_t M, int64_t K, int64_t F, const DeviceState* ds, cudaStream_t st) {
  if (F % 128 != 0 || K % 8 != 0) return fail(MCB_ERR_ALIGN, "linear_swiglu: features %lld must be a multiple of 128, reduction %lld of 8", (long long)F, (long long)K);
  if (M > 0x7fffff00ll || 2 * F > 0x7fffff00ll || K > 0x7fffff00ll) return fail(MCB_ERR_SHAPE, "linear_swiglu: dimension exceeds 2^31");
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.M = static_cast<int>(M); p.N = static_cast<int>(2 * F); p.K = static_cast<int>(K);
  p.swiglu = 1;
  p.epi_bufs = kEpiBufs;
  p.BN = 256;
  p.num_m_tiles = static_cast<int>((M + 255) / 256);
  p.num_n_tiles = static_cast<int>(F / 128);
  p.num_tiles = p.num_m_tiles * p.num_n_tiles;
  p.num_k_blocks = static_cast<int>((K + BK2 - 1) / BK2);
  p.group_m = p.num_m_tiles < 8 ? p.num_m_tiles : 8;
  p.Y = G; p.status = ds->status_word;
  const uint32_t x_bytes = 128 * BK2 * 2, w_bytes = 128u * BK2 * 2;
  p.w_off = x_bytes;
  p.p_off = x_bytes + w_bytes;
  p.stage_bytes = x_bytes + w_bytes;
  const uint32_t epi_bytes = 4 * kEpiBufs * kEpiBufBytes;
  int stages = static_cast<int>((kSmem2 - epi_bytes - 512) / p.stage_bytes);
  if (stages > kMaxStages2) stages = kMaxStages2;
  p.stages = stages;
  p.q_off = stages * p.stage_bytes;
  p.hs_off = p.q_off;
  p.epi_off = p.hs_off;
  p.bar_off = p.epi_off + epi_bytes;
  CUtensorMap tmX, tmW, tmG, tmU, tmA;
  if (int rc = make_map2(ds, &tmG, G, F, M, 32, 32, 64, "gate (pair)")) return rc;
  if (int rc = make_map2(ds, &tmU, U, F, M, 32, 32, 64, "up (pair)")) return rc;
  if (int rc = make_map2(ds, &tmA, Act, F, M, 32, 32, 64, "act (pair)")) return rc;
  if (int rc = make_map2(ds, &tmX, X, K, M, BK2, 128, 128, "X (pair)")) return rc;
  if (int rc = make_map2(ds, &tmW, Wgu, K, 2 * F, BK2, 128, 128, "W gate/up (pair)")) return rc;
  int pairs = ds->sm_count / 2;
  if (pairs > p.num_tiles) pairs = p.num_tiles;
  const bool prof = profile_on();
  if (prof) {
    const double m = static_cast<double>(M), n = static_cast<double>(2 * F), k = static_cast<double>(K);
    profile_begin(kProfGemm, 2.0 * m * n * k, 2.0 * (m * k + n * k + 1.5 * m * n), st);
  }
  lora_gemm2_kernel<<<2 * pairs, kThreads2, kSmem2 + 1024, st>>>(tmX, tmW, tmX, tmX, tmG, tmU, tmA, tmG, tmG, p);
  if (prof) profile_end(st);
  MCB_CHECK_LAUNCH("lora_gemm2_kernel");
  return MCB_OK;
}

}  // namespace bf16path
}  // namespace mcb
