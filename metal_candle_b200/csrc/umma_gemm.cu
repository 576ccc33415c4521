// bfloat16 production path of the fused LoRA linear on Blackwell tensor cores.
//
// One persistent, warp-specialised kernel computes
//
//     Y[M,N] = X[M,K] . W[N,K]^T  (+ bias)  +  (scale * X . P[rp,K]^T) . Q[N,rp]^T
//
// with every operand K-major (the reduction index is the contiguous one).  The forward uses it with
// X = x, W = the frozen weight [out,in], P = A^T, Q = B^T; the backward uses the SAME kernel with
// X = dy, W = the [in,out] copy of the frozen weight, P = B, Q = A, so dx and the rank-r path share one
// pass over dy.  The rank-r intermediate H = scale * X P^T never goes through HBM on its way to the
// output: it is accumulated in tensor memory beside the main accumulator, converted to bf16 by the
// epilogue warps into shared memory, and applied as one more tcgen05.mma onto the main accumulator.
// (The [M,rp] copy that the weight-gradient kernel needs is written out by the n-tile-0 CTAs only.)
//
// Roles per CTA (192 threads, one CTA per SM, grid = min(#tiles, #SMs)):
//   warp 0    TMA producer: cp.async.bulk.tensor loads of the X / W / P tiles (128B swizzle) into a
//             multi-stage ring, and of the Q tile (no swizzle, 16-byte columns) once per output tile
//   warp 1    owns tensor memory (tcgen05.alloc of all 512 columns) and issues tcgen05.mma
//             (M=128, N=BN and N=rp, K=16, bf16 x bf16 -> fp32) from one thread
//   warps 2-5 epilogue: tcgen05.ld the accumulators (32 lanes per warp), convert, store
// Two accumulator buffers (256 columns each: BN main + rp rank columns) let the epilogue of tile i
// overlap the main loop of tile i+1.
//
// In the backward the same launch can go on to the LoRA weight gradients: once a CTA has no tiles left it
// takes a token slice of dA = x^T H or dB = h^T dy (the tail phase, grad_phase.cuh), waiting per 128-token tile
// for the H rows that the n-tile-0 CTAs of this launch publish.
//
// Every wait on an mbarrier is bounded (about two seconds); a wait that runs out records a code in
// the device status word, raises a CTA-wide abort flag, and all roles fall through to the common
// exit where tensor memory is released.  No loads use cluster multicast.
#include <cuda.h>
#include <string.h>

#include "grad_phase.cuh"
#include "lora_internal.cuh"
#include "umma_ptx.cuh"

namespace mcb {
namespace bf16path {
using namespace umma;

int init_grad_kernel();
int init_gemm2_kernel();
bool gemm2_eligible(const GemmCall& c);
int launch_gemm2(const GemmCall& c, const DeviceState* ds, cudaStream_t st);
size_t grad_partial_bytes(int64_t M, int64_t K, int64_t N, int rp);
int launch_grad2(const __nv_bfloat16* X0, const __nv_bfloat16* Ht0, int64_t C0, float* out0, int transposed0,
                 const __nv_bfloat16* X1, const __nv_bfloat16* Ht1, int64_t C1, float* out1, int transposed1,
                 int64_t h_pitch, float* part, int64_t M, int r, int rp, int accumulate, const DeviceState* ds,
                 cudaStream_t st);

namespace {

constexpr int BK = 64;              // 64 bf16 = 128 bytes = one swizzle row
constexpr int kThreads = 192;
constexpr int kMaxStages = 8;
constexpr uint32_t kTmemCols = 512;
constexpr int kSmemBudget = 227 * 1024 - 1024;  // dynamic shared memory we ask for (minus alignment slack)

struct GemmParams {
  int M, N, K;
  int BN, rp, has_w, stages;
  int num_m_tiles, num_n_tiles, num_tiles, num_k_blocks, group_m;
  int pdl_wait;       // 1: launched as a programmatic dependent of the operand-pack kernel: wait for it before loading
  float scale;
  __nv_bfloat16* Y;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* R;   // [M,N] added to the output (residual / gradient accumulation), or null
  __nv_bfloat16* H;   // [rp, h_pitch]: scale * X P^T, transposed (token index contiguous), or null
  int64_t h_pitch;
  int* h_flags;       // per m-tile count of epilogue warps that have stored their H rows (tail phase), or null
  int* status;
  uint32_t stage_bytes, w_off, p_off;        // within a stage
  uint32_t q_off, q_bytes, hs_off, hs_bytes; // from the aligned base
  uint32_t epi_off;  // output staging (epi_bufs buffers per epilogue warp); epi_bufs == 0: direct stores
  int epi_bufs;
  uint32_t bar_off;
};

__device__ __forceinline__ void tile_coords(const GemmParams& p, int t, int& mt, int& nt) {
  const int per_band = p.group_m * p.num_n_tiles;
  const int band = t / per_band;
  const int in = t - band * per_band;
  const int m_first = band * p.group_m;
  const int gm = min(p.group_m, p.num_m_tiles - m_first);
  nt = in / gm;
  mt = m_first + in % gm;
}

// Barrier slots (8 bytes each) after the tile buffers.
struct Bars {
  uint32_t full0, empty0, d2_full0, h_ready0, d1_full0, acc_empty0, q_full0;
};

__global__ void __launch_bounds__(kThreads, 1)
lora_gemm_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                 const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                 const __grid_constant__ CUtensorMap tmY,
                 const __grid_constant__ CUtensorMap tmGX0, const __grid_constant__ CUtensorMap tmGH0,
                 const __grid_constant__ CUtensorMap tmGX1, const __grid_constant__ CUtensorMap tmGH1,
                 const GemmParams p, const GradParams g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  Bars b;
  b.full0 = base + p.bar_off;
  b.empty0 = b.full0 + 8 * kMaxStages;
  b.d2_full0 = b.empty0 + 8 * kMaxStages;
  b.h_ready0 = b.d2_full0 + 16;
  b.d1_full0 = b.h_ready0 + 16;
  b.acc_empty0 = b.d1_full0 + 16;
  b.q_full0 = b.acc_empty0 + 16;
  const uint32_t tmem_slot = b.q_full0 + 16;
  const uint32_t abort_addr = tmem_slot + 4;
  // generic pointers to the two words after the barriers
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_addr - base));

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(b.full0 + 8 * s, 1);
      mbar_init(b.empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(b.d2_full0 + 8 * a, 1);
      mbar_init(b.h_ready0 + 8 * a, 4);
      mbar_init(b.d1_full0 + 8 * a, 1);
      mbar_init(b.acc_empty0 + 8 * a, 4);
      mbar_init(b.q_full0 + 8 * a, 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // a partial-sum kernel chained behind this launch may be set up now; it waits for this grid before it reads
  if (threadIdx.x == 0) grid_launch_dependents();

  const int nkb = p.num_k_blocks;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int i = 0;
      // everything up to here (barriers, tensor memory) ran under the tail of the operand-pack kernel
      if (p.pdl_wait) grid_dependency_wait();
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x, ++i) {
        int mt, nt;
        tile_coords(p, t, mt, nt);
        const int m0 = mt * BM, n0 = nt * p.BN;
        const int a = i & 1;
        if (p.rp > 0) {
          if (i >= 2) ok = mbar_wait(b.d1_full0 + 8 * a, ((i - 2) >> 1) & 1, abort_flag, 11, p.status);
          if (!ok) break;
          const uint32_t qbar = b.q_full0 + 8 * a;
          mbar_expect_tx(qbar, p.q_bytes);
          const uint32_t qs = base + p.q_off + a * p.q_bytes;
          for (int j = 0; j < p.rp / 8; ++j) tma_load_2d(qs + j * p.BN * 16, &tmQ, qbar, j * 8, n0);
        }
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(b.empty0 + 8 * stage, phase ^ 1, abort_flag, 12, p.status);
          if (!ok) break;
          const uint32_t fb = b.full0 + 8 * stage;
          const uint32_t sb = base + stage * p.stage_bytes;
          mbar_expect_tx(fb, p.stage_bytes);
          tma_load_2d(sb, &tmX, fb, kb * BK, m0);
          if (p.has_w) tma_load_2d(sb + p.w_off, &tmW, fb, kb * BK, n0);
          if (p.rp > 0) tma_load_2d(sb + p.p_off, &tmP, fb, kb * BK, 0);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc_main = make_idesc(p.BN);
      const uint32_t idesc_rank = make_idesc(p.rp);
      // The P tile lies directly behind the W tile in a stage (same 128B-swizzled K-major layout), and the rank
      // accumulator directly behind the main one in tensor memory, so one MMA with N = BN + rp produces both
      // and reads the X tile from shared memory once.
      const uint32_t idesc_both = make_idesc(p.BN + p.rp);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int i = 0;
      // The rank update of a tile needs the epilogue warps to turn its rank accumulator into the bf16 operand
      // first (about a microsecond: barrier, tensor-memory load, conversion, barrier).  Instead of waiting, this
      // thread goes on with the next tile's main loop in the other accumulator buffer and polls between
      // k-blocks; the update is issued as soon as its operands are there.  (Deferring it behind the WHOLE next
      // main loop gains nothing: the accumulator then stays occupied for an epilogue longer.)
      int pend_a = -1;
      uint32_t pend_u = 0;
      auto finish_pending = [&]() -> bool {
        const int pa = pend_a;
        pend_a = -1;
        if (!mbar_wait(b.h_ready0 + 8 * pa, pend_u & 1, abort_flag, 23, p.status)) return false;
        if (!mbar_wait(b.q_full0 + 8 * pa, pend_u & 1, abort_flag, 24, p.status)) return false;
        tcgen05_fence_after();
        const uint32_t pd1 = tmem_base + pa * 256;
        const uint32_t hs = base + p.hs_off + pa * p.hs_bytes;
        const uint32_t qs = base + p.q_off + pa * p.q_bytes;
        for (int kk = 0; kk < p.rp / 16; ++kk) {
          const uint64_t hd = desc_noswz(hs + kk * 2 * (BM * 16), BM * 16, 128);
          const uint64_t qd = desc_noswz(qs + kk * 2 * (p.BN * 16), p.BN * 16, 128);
          umma_bf16(pd1, hd, qd, idesc_main, (p.has_w || kk > 0) ? 1u : 0u);
        }
        umma_commit(b.d1_full0 + 8 * pa);
        return true;
      };
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x, ++i) {
        const int a = i & 1;
        const uint32_t u = static_cast<uint32_t>(i >> 1);
        ok = mbar_wait(b.acc_empty0 + 8 * a, (u & 1) ^ 1, abort_flag, 21, p.status);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t d1 = tmem_base + a * 256;
        const uint32_t d2 = d1 + p.BN;
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(b.full0 + 8 * stage, phase, abort_flag, 22, p.status);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t sb = base + stage * p.stage_bytes;
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            const uint64_t ad = desc_sw128(sb + k4 * 32);
            const uint32_t acc = (kb | k4) != 0 ? 1u : 0u;
            if (p.has_w) umma_bf16(d1, ad, desc_sw128(sb + p.w_off + k4 * 32), p.rp > 0 ? idesc_both : idesc_main, acc);
            else umma_bf16(d2, ad, desc_sw128(sb + p.p_off + k4 * 32), idesc_rank, acc);
          }
          umma_commit(b.empty0 + 8 * stage);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
          if (pend_a >= 0 && mbar_try_wait(b.h_ready0 + 8 * pend_a, pend_u & 1) &&
              mbar_try_wait(b.q_full0 + 8 * pend_a, pend_u & 1)) {
            ok = finish_pending();   // both operands are there: does not wait
            if (!ok) break;
          }
        }
        if (!ok) break;
        if (p.rp > 0) {
          umma_commit(b.d2_full0 + 8 * a);
          if (pend_a >= 0) {         // the previous tile's update has still not been issued: wait for it now
            ok = finish_pending();
            if (!ok) break;
          }
          pend_a = a;
          pend_u = u;
        } else {
          umma_commit(b.d1_full0 + 8 * a);
        }
      }
      if (ok && pend_a >= 0) ok = finish_pending();
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quad = warp & 3;            // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t epi_base = base + p.epi_off + static_cast<uint32_t>(quad * p.epi_bufs) * kEpiBufBytes;
    int sbuf = 0;
    bool ok = true;
    int i = 0;
    for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x, ++i) {
      int mt, nt;
      tile_coords(p, t, mt, nt);
      const int m0 = mt * BM, n0 = nt * p.BN;
      const int a = i & 1;
      const uint32_t u = static_cast<uint32_t>(i >> 1);
      const int64_t grow = static_cast<int64_t>(m0) + row_in_tile;
      const uint32_t d1 = tmem_base + lane_addr + a * 256;
      if (p.rp > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(b.d2_full0 + 8 * a, u & 1, abort_flag, 31, p.status));
        if (!ok) break;
        tcgen05_fence_after();
        uint8_t* hs_gen = gen_base + p.hs_off + a * p.hs_bytes;
        for (int c = 0; c < p.rp; c += 16) {
          uint32_t v[16];
          tmem_ld_x16(d1 + p.BN + c, v);
          tmem_ld_wait();
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            w[j] = pack_bf16(__uint_as_float(v[2 * j]) * p.scale, __uint_as_float(v[2 * j + 1]) * p.scale);
          const uint4 lo = make_uint4(w[0], w[1], w[2], w[3]);
          const uint4 hi = make_uint4(w[4], w[5], w[6], w[7]);
          // no-swizzle K-major operand: 16-byte K chunk j of row m lives at j*(128*16) + m*16
          *reinterpret_cast<uint4*>(hs_gen + (c / 8) * (BM * 16) + row_in_tile * 16) = lo;
          *reinterpret_cast<uint4*>(hs_gen + (c / 8 + 1) * (BM * 16) + row_in_tile * 16) = hi;
          if (p.H != nullptr && nt == 0 && grow < p.M) {
            // transposed copy for the weight-gradient kernel: lanes hold consecutive tokens, so each of
            // these 2-byte stores is a contiguous 64-byte run across the warp
            __nv_bfloat16* hp = p.H + static_cast<int64_t>(c) * p.h_pitch + grow;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              hp[(2 * j) * p.h_pitch] = __ushort_as_bfloat16(static_cast<unsigned short>(w[j] & 0xffffu));
              hp[(2 * j + 1) * p.h_pitch] = __ushort_as_bfloat16(static_cast<unsigned short>(w[j] >> 16));
            }
          }
        }
        fence_proxy_async_smem();
        tcgen05_fence_before();
        if (p.h_flags != nullptr && nt == 0) {
          // the tail phase of other CTAs reads these rows of H with TMA copies: publish them
          __threadfence();
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(b.h_ready0 + 8 * a);
          if (p.h_flags != nullptr && nt == 0)
            asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.h_flags + mt) : "memory");
        }
      }
      ok = __all_sync(0xffffffffu, mbar_wait(b.d1_full0 + 8 * a, u & 1, abort_flag, 32, p.status));
      if (!ok) break;
      tcgen05_fence_after();
      if (p.Y != nullptr && p.epi_bufs > 0) {
        // Output leaves in chunks of 32 columns: each thread rounds its row's 64 bytes into this warp's staging
        // buffer (64-byte swizzle, conflict-free) and one tiled store per chunk writes 32 rows x 64 bytes,
        // clipped at the matrix edges.
        for (int c = 0; c < p.BN; c += 32) {
          const int gcol = n0 + c;
          if (gcol >= p.N) break;
          uint32_t v0[16], v1[16];
          tmem_ld_x16(d1 + c, v0);
          tmem_ld_x16(d1 + c + 16, v1);
          if (lane == 0) bulk_wait_group_read_n(p.epi_bufs - 1);  // the store that last used this buffer has read it
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
          if (++sbuf == p.epi_bufs) sbuf = 0;
        }
      } else if (p.Y != nullptr) {
        // no room for staging: 64 contiguous bytes per thread straight to global memory
        for (int c = 0; c < p.BN; c += 32) {
          uint32_t v0[16], v1[16];
          tmem_ld_x16(d1 + c, v0);
          tmem_ld_x16(d1 + c + 16, v1);
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
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(b.acc_empty0 + 8 * a);
    }
    if (lane == 0) bulk_wait_group<0>();  // this warp's output stores are complete before the CTA may exit
  }

  // ---------------- common exit ----------------
  __syncwarp();
  if (*abort_flag != 0) {
    // give loads still in flight time to land before the CTA's shared memory is released
    for (int k = 0; k < 200; ++k) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  // ---------------- tail phase: the LoRA weight gradients of the same linear ----------------
  // Every role is through with the tiles: the stage ring, the staging buffers and tensor memory are free.  The
  // CTA now takes a token slice of dA = x^T H or dB = h^T dy (grad_phase.cuh) with a fresh set of barriers behind
  // the ones used so far.  H rows written by other CTAs of this launch are awaited per 128-token tile.
  if (g.n_cta > 0 && *abort_flag == 0) {
    GradShared sh;
    sh.base = base;
    sh.full0 = base + p.bar_off + 256;
    sh.empty0 = sh.full0 + 8 * kGradMaxStages;
    sh.done_bar = sh.empty0 + 8 * kGradMaxStages;
    sh.tmem_base = tmem_base;
    sh.abort_flag = abort_flag;
    if (threadIdx.x == 0) {
      for (int s = 0; s < kGradMaxStages; ++s) { mbar_init(sh.full0 + 8 * s, 1); mbar_init(sh.empty0 + 8 * s, 1); }
      mbar_init(sh.done_bar, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      fence_proxy_async_smem();
    }
    __syncthreads();
    tcgen05_fence_after();
    if (static_cast<int>(blockIdx.x) < g.n_cta) grad_roles(g, &tmGX0, &tmGH0, &tmGX1, &tmGH1, sh, static_cast<int>(blockIdx.x));
    __syncwarp();
    if (*abort_flag != 0) {
      for (int k = 0; k < 200; ++k) __nanosleep(1000);
    }
    tcgen05_fence_before();
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- operand packing -----------------------------------------------------------------------------
// Turns the float32 LoRA factors into the two K-major bf16 operands of the kernel above, zero-padded
// from r to rp rows/columns.
//   forward  (mode 0): P = A^T [rp,K],  Q = B^T [N,rp]
//   backward (mode 1): P = B   [rp,N],  Q = A   [K,rp]
// and zeroes `n_flags` counters.
__global__ void pack_lora_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                 __nv_bfloat16* __restrict__ P, __nv_bfloat16* __restrict__ Q, int K, int N, int r,
                                 int rp, int mode, int* __restrict__ flags, int n_flags) {
  grid_launch_dependents();   // the GEMM chained behind this kernel may start its set-up; it waits before it loads P / Q
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // the per-tile counters of the backward kernel's tail phase start from zero in every call
  for (int64_t i = tid; i < n_flags; i += static_cast<int64_t>(gridDim.x) * blockDim.x) flags[i] = 0;
  const int64_t nP = static_cast<int64_t>(rp) * (mode == 0 ? K : N);
  const int64_t nQ = static_cast<int64_t>(rp) * (mode == 0 ? N : K);
  if (tid < nP) {
    if (mode == 0) {  // P[j,k] = A[k,j]
      const int j = static_cast<int>(tid / K), k = static_cast<int>(tid % K);
      P[tid] = __float2bfloat16_rn(j < r ? A[static_cast<int64_t>(k) * r + j] : 0.0f);
    } else {  // P[j,n] = B[j,n]
      const int j = static_cast<int>(tid / N);
      P[tid] = __float2bfloat16_rn(j < r ? B[tid] : 0.0f);
    }
  } else if (tid < nP + nQ) {
    const int64_t q = tid - nP;
    const int j = static_cast<int>(q % rp);
    const int64_t row = q / rp;
    if (mode == 0)  // Q[n,j] = B[j,n]
      Q[q] = __float2bfloat16_rn(j < r ? B[static_cast<int64_t>(j) * N + row] : 0.0f);
    else  // Q[k,j] = A[k,j]
      Q[q] = __float2bfloat16_rn(j < r ? A[row * r + j] : 0.0f);
  }
}

// The same packing for a fused projection: the adapters of up to kMaxSegments segments side by side.  Rank column
// jt = segment * r + j.  The A factors are concatenated ([K, r_tot]); the B factors form a block-diagonal
// [r_tot, N] matrix (segment i's B in its own rows and in the output columns it owns, zero elsewhere), so the one
// rank update  (x A_cat) B_bd  adds every segment's delta to its own columns only.
struct SegTable {
  const float* A[kMaxSegments];
  const float* B[kMaxSegments];
  int n_off[kMaxSegments], n[kMaxSegments];
  int count;
};
__global__ void pack_lora_fused_kernel(const SegTable t, __nv_bfloat16* __restrict__ P, __nv_bfloat16* __restrict__ Q, int K,
                                       int N, int r, int rp, int mode, int* __restrict__ flags, int n_flags) {
  grid_launch_dependents();
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (int64_t i = tid; i < n_flags; i += static_cast<int64_t>(gridDim.x) * blockDim.x) flags[i] = 0;
  const int64_t nP = static_cast<int64_t>(rp) * (mode == 0 ? K : N);
  const int64_t nQ = static_cast<int64_t>(rp) * (mode == 0 ? N : K);
  auto a_at = [&](int k, int jt) -> float {     // A_cat[k, jt]
    const int sg = jt / r, j = jt - sg * r;
    return sg < t.count ? t.A[sg][static_cast<int64_t>(k) * r + j] : 0.0f;
  };
  auto b_at = [&](int jt, int n) -> float {     // B_bd[jt, n]
    const int sg = jt / r, j = jt - sg * r;
    if (sg >= t.count || n < t.n_off[sg] || n >= t.n_off[sg] + t.n[sg]) return 0.0f;
    return t.B[sg][static_cast<int64_t>(j) * t.n[sg] + (n - t.n_off[sg])];
  };
  if (tid < nP) {
    if (mode == 0) {  // P[jt,k] = A_cat[k,jt]
      P[tid] = __float2bfloat16_rn(a_at(static_cast<int>(tid % K), static_cast<int>(tid / K)));
    } else {          // P[jt,n] = B_bd[jt,n]
      P[tid] = __float2bfloat16_rn(b_at(static_cast<int>(tid / N), static_cast<int>(tid % N)));
    }
  } else if (tid < nP + nQ) {
    const int64_t q = tid - nP;
    const int jt = static_cast<int>(q % rp);
    const int row = static_cast<int>(q / rp);
    Q[q] = __float2bfloat16_rn(mode == 0 ? b_at(jt, row) : a_at(row, jt));   // Q[n,jt] = B_bd[jt,n]  /  Q[k,jt] = A_cat[k,jt]
  }
}

// The fused gradients dA_cat [K, r_tot] and dB_cat [r_tot, N] hold every segment's dA_i in its own columns and
// dB_i in its own diagonal block; this writes (or adds) them to the segments' own tensors.
struct ScatterTable {
  float* dA[kMaxSegments];
  float* dB[kMaxSegments];
  int n_off[kMaxSegments], n[kMaxSegments];
  int count;
};
__global__ void scatter_fused_grads_kernel(const ScatterTable t, const float* __restrict__ dA_cat, const float* __restrict__ dB_cat,
                                           int K, int N, int r, int accumulate) {
  const int r_tot = t.count * r;
  const int64_t nA = static_cast<int64_t>(K) * r_tot;
  int64_t nB = 0;
  for (int sg = 0; sg < t.count; ++sg) nB += static_cast<int64_t>(r) * t.n[sg];
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nA + nB;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    if (i < nA) {
      const int k = static_cast<int>(i / r_tot), jt = static_cast<int>(i % r_tot);
      const int sg = jt / r, j = jt - sg * r;
      float* o = t.dA[sg] + static_cast<int64_t>(k) * r + j;
      *o = accumulate ? *o + dA_cat[i] : dA_cat[i];
    } else {
      int64_t e = i - nA;
      int sg = 0;
      while (e >= static_cast<int64_t>(r) * t.n[sg]) { e -= static_cast<int64_t>(r) * t.n[sg]; ++sg; }
      const int j = static_cast<int>(e / t.n[sg]), n = static_cast<int>(e % t.n[sg]);
      const float v = dB_cat[static_cast<int64_t>(sg * r + j) * N + t.n_off[sg] + n];
      float* o = t.dB[sg] + e;
      *o = accumulate ? *o + v : v;
    }
  }
}

// ---- host side -----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_map(const DeviceState* ds, CUtensorMap* map, const void* ptr, int64_t inner, int64_t outer, int box_inner,
             int box_outer, int swizzle_bytes, const char* what) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(inner) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ds->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE,
      swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MCB_ERR_ALIGN, "tensor map for %s rejected (CUresult %d): ptr=%p inner=%lld outer=%lld box=%dx%d", what,
                static_cast<int>(r), ptr, (long long)inner, (long long)outer, box_inner, box_outer);
  return MCB_OK;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Tile width: the fewest n-tiles of at most `cap` columns, evened out, in multiples of 32.
int pick_bn(int64_t N, int rp) {
  const int cap = rp > 0 ? ((256 - rp) / 32) * 32 : 256;
  const int64_t tiles = (N + cap - 1) / cap;
  int bn = static_cast<int>(((N + tiles - 1) / tiles + 31) / 32 * 32);
  if (bn > cap) bn = cap;
  if (bn < 32) bn = 32;
  return bn;
}

int launch_gemm(const GemmCall& c, const DeviceState* ds, cudaStream_t st) {
  if (c.M > 0x7fffff00ll || c.N > 0x7fffff00ll || c.K > 0x7fffff00ll)
    return fail(MCB_ERR_SHAPE, "bf16 GEMM: dimension exceeds 2^31");
  if (c.K % 8 != 0 || c.N % 8 != 0)
    return fail(MCB_ERR_ALIGN, "bf16 path needs in/out features that are multiples of 8 (got reduction %lld, output %lld)",
                (long long)c.K, (long long)c.N);
  if (!aligned16(c.X) || (c.W && !aligned16(c.W)) || (c.Y && !aligned16(c.Y)) || (c.H && !aligned16(c.H)) || (c.R && !aligned16(c.R)))
    return fail(MCB_ERR_ALIGN, "bf16 path needs 16-byte aligned matrices");
  // linears of useful size (with or without the rank path) run on CTA pairs (umma_gemm2.cu)
  if (gemm2_eligible(c)) return launch_gemm2(c, ds, st);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = static_cast<int>(c.M); p.N = static_cast<int>(c.N); p.K = static_cast<int>(c.K);
  p.rp = c.rp;
  p.has_w = c.W != nullptr ? 1 : 0;
  p.BN = pick_bn(c.N, c.rp);
  p.num_m_tiles = (p.M + BM - 1) / BM;
  p.num_n_tiles = (p.N + p.BN - 1) / p.BN;
  p.num_tiles = p.num_m_tiles * p.num_n_tiles;
  p.num_k_blocks = (p.K + BK - 1) / BK;
  p.group_m = p.num_m_tiles < 16 ? p.num_m_tiles : 16;
  p.scale = c.scale;
  p.Y = c.Y; p.bias = c.bias; p.R = c.R; p.H = c.H; p.h_pitch = c.h_pitch; p.status = ds->status_word;
  const uint32_t x_bytes = BM * BK * 2;
  const uint32_t w_bytes = p.has_w ? p.BN * BK * 2 : 0;
  const uint32_t p_bytes = p.rp * BK * 2;
  p.w_off = x_bytes;
  p.p_off = x_bytes + w_bytes;
  p.stage_bytes = x_bytes + w_bytes + p_bytes;  // every part is a multiple of 1024
  p.q_bytes = static_cast<uint32_t>(p.BN) * p.rp * 2;
  p.hs_bytes = static_cast<uint32_t>(BM) * p.rp * 2;
  uint32_t fixed = 2 * p.q_bytes + 2 * p.hs_bytes + 512;
  int stages = static_cast<int>((kSmemBudget - fixed) / p.stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  // output staging takes what the stage ring leaves over, never a stage
  p.epi_bufs = 0;
  if (c.Y != nullptr && stages >= 2) {
    const uint32_t spare = kSmemBudget - fixed - static_cast<uint32_t>(stages) * p.stage_bytes;
    p.epi_bufs = static_cast<int>(spare / (4 * kEpiBufBytes));
    if (p.epi_bufs > kEpiBufsMax) p.epi_bufs = kEpiBufsMax;
  }
  const uint32_t epi_bytes = 4 * kEpiBufBytes * p.epi_bufs;
  fixed += epi_bytes;
  if (stages < 2) return fail(MCB_ERR_UNSUPPORTED, "bf16 GEMM: tile does not fit shared memory (BN=%d rp=%d)", p.BN, p.rp);
  p.stages = stages;
  p.q_off = stages * p.stage_bytes;
  p.hs_off = p.q_off + 2 * p.q_bytes;
  p.epi_off = p.hs_off + 2 * p.hs_bytes;  // a multiple of 1024
  p.bar_off = p.epi_off + epi_bytes;

  CUtensorMap tmX, tmW, tmP, tmQ, tmY;
  if (p.epi_bufs > 0) { if (int rc = make_map(ds, &tmY, c.Y, c.N, c.M, 32, 32, 64, "Y")) return rc; }
  else tmY = CUtensorMap{};
  if (int rc = make_map(ds, &tmX, c.X, c.K, c.M, BK, BM, 128, "X")) return rc;
  if (p.has_w) { if (int rc = make_map(ds, &tmW, c.W, c.K, c.N, BK, p.BN, 128, "W")) return rc; }
  else tmW = tmX;
  if (p.rp > 0) {
    if (int rc = make_map(ds, &tmP, c.P, c.K, p.rp, BK, p.rp, 128, "P")) return rc;
    if (int rc = make_map(ds, &tmQ, c.Q, p.rp, c.N, 8, p.BN, 0, "Q")) return rc;
  } else { tmP = tmX; tmQ = tmX; }
  const int grid = p.num_tiles < ds->sm_count ? p.num_tiles : ds->sm_count;
  // the weight gradients as a tail phase: the same CTAs, the stage ring re-cut for token rows
  GradPlan tail;
  memset(&tail.p, 0, sizeof(tail.p));
  // The tail phase makes CTAs wait for rank-intermediate rows that OTHER CTAs of this launch write, which is only
  // safe when the whole grid is resident at once (a CTA that has not started cannot be waited for by CTAs that hold
  // every SM).  One CTA fits an SM, so the grid must not exceed what the occupancy query says the device can hold;
  // a context restricted to fewer SMs than it reports, or a caller that runs other kernels beside this one (a
  // collective overlapping the backward pass), switches the tail off with MCB_OPT_GRAD_TAIL = 0 and gets the
  // separate gradient launch, which waits for nothing.
  bool tail_on = c.grads != nullptr && option(MCB_OPT_GRAD_TAIL) != 0;
  if (tail_on) {
    static int occ_cached = -1;
    if (occ_cached < 0) {
      int occ = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, lora_gemm_kernel, kThreads, kSmemBudget + 1024) != cudaSuccess) occ = 0;
      occ_cached = occ;
    }
    if (static_cast<long long>(occ_cached) * ds->sm_count < grid) tail_on = false;
  }
  if (tail_on) {
    const uint32_t budget = p.bar_off < static_cast<uint32_t>(kGradSmemBudget) ? p.bar_off : static_cast<uint32_t>(kGradSmemBudget);
    if (int rc = plan_grad2(*c.grads, c.M, c.rp, grid, budget, ds, &tail)) return rc;
    // a grid of a single CTA cannot hold both problems: the gradients then take their own launch below
    if (tail.p.n_cta > grid) tail_on = false;
  }
  if (tail_on) {
    p.h_flags = c.grads->h_flags;
  } else {
    memset(&tail.p, 0, sizeof(tail.p));
    tail.tmX[0] = tail.tmX[1] = tail.tmH[0] = tail.tmH[1] = tmX;
  }
  const bool prof = profile_on();
  if (prof) {
    const double m = static_cast<double>(c.M), n = static_cast<double>(c.N), k = static_cast<double>(c.K);
    double flops = (p.has_w ? 2.0 * m * n * k : 0.0) + 2.0 * m * c.r_true * (k + n);
    double bytes = 2.0 * (m * k + (p.has_w ? n * k : 0.0) + (c.Y ? m * n : 0.0)) + 2.0 * p.rp * (k + n);
    if (tail_on) {
      flops += 2.0 * m * (c.grads->C[0] + c.grads->C[1]) * c.r_true;
      bytes += 2.0 * m * (c.grads->C[0] + c.grads->C[1]) + 4.0 * m * c.rp;
    }
    profile_begin(c.rp > 0 ? kProfGemmLora : kProfGemm, flops, bytes, st);
  }
  // with a rank path the launch directly before this one is the operand-pack kernel
  const bool pdl = c.after_pack && !prof && option(MCB_OPT_PDL) != 0;
  p.pdl_wait = pdl ? 1 : 0;
  {
    const cudaError_t le = launch_kernel(lora_gemm_kernel, dim3(grid), dim3(kThreads), kSmemBudget + 1024, st, pdl, tmX, tmW, tmP, tmQ,
                                         tmY, tail.tmX[0], tail.tmH[0], tail.tmX[1], tail.tmH[1], p, tail.p);
    if (le != cudaSuccess) return cuda_fail(le, "lora_gemm_kernel launch");
  }
  if (prof) profile_end(st);
  MCB_CHECK_LAUNCH("lora_gemm_kernel");
  if (tail_on) return launch_grad_reduce(tail, st);
  if (c.grads != nullptr) {
    const GradRequest& q = *c.grads;
    return launch_grad2(q.X[0], q.Ht[0], q.C[0], q.out[0], q.transposed[0], q.X[1], q.Ht[1], q.C[1], q.out[1], q.transposed[1],
                        q.h_pitch, q.part, c.M, q.r, c.rp, q.accumulate, ds, st);
  }
  return MCB_OK;
}

struct Workspace {
  __nv_bfloat16 *P, *Q, *H1, *H2;
  float* part;
  int* flags;   // one counter per 128-token tile
  size_t total;
};
Workspace carve(void* ws, int64_t M, int64_t K, int64_t N, int64_t r) {
  const int64_t rp = rank_padded(r);
  const int64_t big = K > N ? K : N;
  Workspace w;
  size_t off = 0;
  uint8_t* b = static_cast<uint8_t*>(ws);
  auto take = [&](size_t bytes) { uint8_t* q = b ? b + off : nullptr; off += align_up(bytes, 1024); return q; };
  w.P = reinterpret_cast<__nv_bfloat16*>(take(static_cast<size_t>(rp) * big * 2));
  w.Q = reinterpret_cast<__nv_bfloat16*>(take(static_cast<size_t>(rp) * big * 2));
  w.H1 = reinterpret_cast<__nv_bfloat16*>(take(static_cast<size_t>(h_pitch(M)) * rp * 2));
  w.H2 = reinterpret_cast<__nv_bfloat16*>(take(static_cast<size_t>(h_pitch(M)) * rp * 2));
  w.part = reinterpret_cast<float*>(take(grad_partial_bytes(M, K, N, static_cast<int>(rp))));
  w.flags = reinterpret_cast<int*>(take(static_cast<size_t>((M + BM - 1) / BM) * sizeof(int)));
  w.total = off;
  return w;
}

int pack(const LoraArgs& a, const Workspace& w, int mode) {
  const int rp = static_cast<int>(rank_padded(a.r));
  const int64_t n = static_cast<int64_t>(rp) * (a.K + a.N);
  pack_lora_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, a.stream>>>(
      a.A, a.B, w.P, w.Q, static_cast<int>(a.K), static_cast<int>(a.N), static_cast<int>(a.r), rp, mode,
      mode == 1 ? w.flags : nullptr, mode == 1 ? static_cast<int>((a.M + BM - 1) / BM) : 0);
  MCB_CHECK_LAUNCH("pack_lora");
  return MCB_OK;
}

int check_ws(const LoraArgs& a, const char* op) {
  if (a.r == 0) return MCB_OK;
  if (a.r > 64) return fail(MCB_ERR_UNSUPPORTED, "%s(bf16): rank %lld > 64", op, (long long)a.r);
  if (!a.ws || a.ws_bytes < workspace_bytes(a.M, a.K, a.N, a.r))
    return fail(MCB_ERR_WORKSPACE, "%s(bf16): workspace %zu < %zu bytes", op, a.ws_bytes,
                workspace_bytes(a.M, a.K, a.N, a.r));
  if ((reinterpret_cast<uintptr_t>(a.ws) & 1023u) != 0) return fail(MCB_ERR_ALIGN, "%s(bf16): workspace must be 1024-byte aligned", op);
  return MCB_OK;
}

}  // namespace

int init_kernels() {
  cudaError_t e = cudaFuncSetAttribute(lora_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 1024);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(lora_gemm_kernel)");
  if (int rc = init_gemm2_kernel()) return rc;
  return init_grad_kernel();
}

size_t workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t r) {
  if (r <= 0) return 0;
  return carve(nullptr, M, K, N, r).total;
}

int delta_fwd(const LoraArgs& a, const DeviceState* ds) {
  if (int rc = check_ws(a, "lora_delta_fwd")) return rc;
  Workspace w = carve(a.ws, a.M, a.K, a.N, a.r);
  if (int rc = pack(a, w, 0)) return rc;
  GemmCall c;
  c.after_pack = true;
  c.X = static_cast<const __nv_bfloat16*>(a.x);
  c.P = w.P; c.Q = w.Q;
  c.Y = static_cast<__nv_bfloat16*>(a.y);
  c.M = a.M; c.N = a.N; c.K = a.K;
  c.rp = static_cast<int>(rank_padded(a.r));
  c.r_true = static_cast<int>(a.r);
  c.scale = a.scale;
  return launch_gemm(c, ds, a.stream);
}

int linear_fwd(const LoraArgs& a, const DeviceState* ds) {
  if (a.w_layout != MCB_W_OUT_IN)
    return fail(MCB_ERR_UNSUPPORTED, "lora_linear_fwd(bf16) needs W as [out,in] (MCB_W_OUT_IN); transpose it once with mcb_transpose_2d");
  if (int rc = check_ws(a, "lora_linear_fwd")) return rc;
  GemmCall c;
  c.X = static_cast<const __nv_bfloat16*>(a.x);
  c.W = static_cast<const __nv_bfloat16*>(a.W);
  c.bias = static_cast<const __nv_bfloat16*>(a.bias);
  c.R = static_cast<const __nv_bfloat16*>(a.residual);
  c.Y = static_cast<__nv_bfloat16*>(a.y);
  c.M = a.M; c.N = a.N; c.K = a.K;
  if (a.r > 0) {
    Workspace w = carve(a.ws, a.M, a.K, a.N, a.r);
    if (int rc = pack(a, w, 0)) return rc;
    c.after_pack = true;
    c.P = w.P; c.Q = w.Q;
    c.H = static_cast<__nv_bfloat16*>(a.h_save);
    c.h_pitch = h_pitch(a.M);
    c.rp = static_cast<int>(rank_padded(a.r));
  c.r_true = static_cast<int>(a.r);
    c.scale = a.scale;
  }
  return launch_gemm(c, ds, a.stream);
}

bool swiglu_bwd_supported(int64_t M, int64_t K, int64_t N, int64_t r) {
  if (M <= 0 || K <= 0 || N <= 0 || r < 0 || K % 8 != 0 || N % 8 != 0) return false;
  GemmCall c;   // the input-gradient product: [M,N] . [K,N]^T, rank path over N
  c.X = c.W = c.Y = reinterpret_cast<__nv_bfloat16*>(16);   // placeholders: only their presence is looked at
  c.M = M; c.N = K; c.K = N;
  c.rp = static_cast<int>(rank_padded(r));
  return gemm2_eligible(c);
}

int linear_bwd(const LoraArgs& a, const DeviceState* ds) {
  if (a.dx != nullptr && a.w_layout != MCB_W_IN_OUT)
    return fail(MCB_ERR_UNSUPPORTED, "lora_linear_bwd(bf16) needs W as [in,out] (MCB_W_IN_OUT); transpose it once with mcb_transpose_2d");
  if (a.swiglu_up != nullptr && (a.dx == nullptr || a.residual != nullptr || !swiglu_bwd_supported(a.M, a.K, a.N, a.r)))
    return fail(MCB_ERR_UNSUPPORTED, "lora_linear_bwd_swiglu: M=%lld K=%lld N=%lld r=%lld does not run on CTA pairs; use "
                "mcb_lora_linear_bwd_ex and mcb_swiglu_bwd", (long long)a.M, (long long)a.K, (long long)a.N, (long long)a.r);
  if (int rc = check_ws(a, "lora_linear_bwd")) return rc;
  const int rp = static_cast<int>(rank_padded(a.r));
  const bool want_grads = a.r > 0 && (a.dA != nullptr || a.dB != nullptr);
  Workspace w;
  memset(&w, 0, sizeof(w));
  if (a.r > 0) {
    w = carve(a.ws, a.M, a.K, a.N, a.r);
    if (int rc = pack(a, w, 1)) return rc;
  }
  // Both gradients asked for, the forward's rank intermediate at hand and shapes of one feature group each: dA and
  // dB are accumulated by the CTAs of the dx kernel themselves, as its tail phase (one launch instead of two).
  GradRequest rq;
  bool fused_grads = false;
  if (a.dx != nullptr || want_grads) {
    // dx = dy W + (scale dy B^T) A^T ; the rank intermediate scale*dy*B^T lands in w.H1 for dA.
    GemmCall c;
    c.X = static_cast<const __nv_bfloat16*>(a.dy);
    c.W = a.dx != nullptr ? static_cast<const __nv_bfloat16*>(a.W) : nullptr;
    c.Y = static_cast<__nv_bfloat16*>(a.dx);
    c.R = a.dx != nullptr ? static_cast<const __nv_bfloat16*>(a.residual) : nullptr;
    c.swiglu_up = static_cast<__nv_bfloat16*>(a.swiglu_up);
    c.M = a.M; c.N = a.K; c.K = a.N;
    if (a.r > 0) {
      c.after_pack = true;   // pack(a, w, 1) above is the launch directly before the GEMM
      c.P = w.P; c.Q = w.Q;
      c.H = (a.dA != nullptr) ? w.H1 : nullptr;
      c.h_pitch = h_pitch(a.M);
      c.rp = rp;
      c.r_true = static_cast<int>(a.r);
      c.scale = a.scale;
    }
    if (a.dA != nullptr && a.dB != nullptr && a.h_save != nullptr && !gemm2_eligible(c) &&
        grad_tail_possible(a.K, a.N, rp)) {
      rq.X[0] = static_cast<const __nv_bfloat16*>(a.x);  rq.Ht[0] = w.H1; rq.C[0] = a.K; rq.out[0] = a.dA; rq.transposed[0] = 0;
      rq.X[1] = static_cast<const __nv_bfloat16*>(a.dy); rq.Ht[1] = static_cast<const __nv_bfloat16*>(a.h_save);
      rq.C[1] = a.N; rq.out[1] = a.dB; rq.transposed[1] = 1;
      rq.h_pitch = h_pitch(a.M); rq.part = w.part; rq.r = static_cast<int>(a.r); rq.accumulate = a.accumulate;
      rq.h_flags = w.flags;
      c.grads = &rq;
      fused_grads = true;
    }
    if (c.W != nullptr || c.rp > 0) {
      if (int rc = launch_gemm(c, ds, a.stream)) return rc;
    }
  }
  if (!want_grads || fused_grads) return MCB_OK;
  const __nv_bfloat16* hs = nullptr;
  if (a.dB != nullptr) {
    hs = static_cast<const __nv_bfloat16*>(a.h_save);
    if (hs == nullptr) {
      // recompute scale * x A with the forward operands
      LoraArgs f = a;
      Workspace wf = w;
      // P/Q of the backward are still needed by nothing after the GEMM above, so they can be repacked
      if (int rc = pack(f, wf, 0)) return rc;
      GemmCall c;
      c.after_pack = true;
      c.X = static_cast<const __nv_bfloat16*>(a.x);
      c.P = wf.P; c.Q = wf.Q;
      c.H = w.H2;
      c.h_pitch = h_pitch(a.M);
      c.M = a.M; c.N = a.N; c.K = a.K;
      c.rp = rp;
      c.r_true = static_cast<int>(a.r);
      c.scale = a.scale;
      if (int rc = launch_gemm(c, ds, a.stream)) return rc;
      hs = w.H2;
    }
  }
  // dA = x^T (scale dy B^T) and dB = (scale x A)^T dy, both in one launch where both are asked for
  const __nv_bfloat16* xa = static_cast<const __nv_bfloat16*>(a.x);
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(a.dy);
  if (a.dA != nullptr && a.dB != nullptr)
    return launch_grad2(xa, w.H1, a.K, a.dA, 0, xb, hs, a.N, a.dB, 1, h_pitch(a.M), w.part, a.M, static_cast<int>(a.r), rp,
                        a.accumulate, ds, a.stream);
  if (a.dA != nullptr)
    return launch_grad2(xa, w.H1, a.K, a.dA, 0, nullptr, nullptr, 0, nullptr, 0, h_pitch(a.M), w.part, a.M,
                        static_cast<int>(a.r), rp, a.accumulate, ds, a.stream);
  return launch_grad2(xb, hs, a.N, a.dB, 1, nullptr, nullptr, 0, nullptr, 0, h_pitch(a.M), w.part, a.M, static_cast<int>(a.r), rp,
                      a.accumulate, ds, a.stream);
}

// ---- fused projections (several adapters, one GEMM) ----------------------------------------------------------
namespace {
struct FusedWorkspace {
  Workspace w;
  float *dA_cat, *dB_cat;
  size_t total;
};
FusedWorkspace carve_fused(void* ws, int64_t M, int64_t K, int64_t N, int64_t r_tot) {
  FusedWorkspace f;
  f.w = carve(ws, M, K, N, r_tot);
  size_t off = f.w.total;
  uint8_t* b = static_cast<uint8_t*>(ws);
  auto take = [&](size_t bytes) { uint8_t* q = b ? b + off : nullptr; off += align_up(bytes, 1024); return q; };
  f.dA_cat = reinterpret_cast<float*>(take(static_cast<size_t>(K) * r_tot * sizeof(float)));
  f.dB_cat = reinterpret_cast<float*>(take(static_cast<size_t>(N) * r_tot * sizeof(float)));
  f.total = off;
  return f;
}
int pack_fused(const LoraArgs& a, const LoraSegments& sg, const Workspace& w, int rp, int mode) {
  SegTable t;
  memset(&t, 0, sizeof(t));
  t.count = sg.count;
  for (int i = 0; i < sg.count; ++i) {
    t.A[i] = sg.A[i]; t.B[i] = sg.B[i];
    t.n_off[i] = static_cast<int>(sg.n_off[i]); t.n[i] = static_cast<int>(sg.n[i]);
  }
  const int64_t n = static_cast<int64_t>(rp) * (a.K + a.N);
  pack_lora_fused_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, a.stream>>>(
      t, w.P, w.Q, static_cast<int>(a.K), static_cast<int>(a.N), static_cast<int>(a.r), rp, mode,
      mode == 1 ? w.flags : nullptr, mode == 1 ? static_cast<int>((a.M + BM - 1) / BM) : 0);
  MCB_CHECK_LAUNCH("pack_lora_fused");
  return MCB_OK;
}
int check_fused(const LoraArgs& a, const LoraSegments& sg, const char* op) {
  if (sg.count < 1 || sg.count > kMaxSegments) return fail(MCB_ERR_SHAPE, "%s: %d segments (1..%d)", op, sg.count, kMaxSegments);
  if (a.r < 1 || a.r * sg.count > 64) return fail(MCB_ERR_UNSUPPORTED, "%s: rank %lld x %d segments exceeds 64 rank columns", op, (long long)a.r, sg.count);
  int64_t end = 0;
  for (int i = 0; i < sg.count; ++i) {
    if (!sg.A[i] || !sg.B[i]) return fail(MCB_ERR_NULL, "%s: segment %d has no adapter", op, i);
    if (sg.n[i] <= 0 || sg.n_off[i] < end || sg.n_off[i] + sg.n[i] > a.N)
      return fail(MCB_ERR_SHAPE, "%s: segment %d covers columns [%lld, %lld) of %lld (segments must be ascending and disjoint)", op, i,
                  (long long)sg.n_off[i], (long long)(sg.n_off[i] + sg.n[i]), (long long)a.N);
    end = sg.n_off[i] + sg.n[i];
  }
  const size_t need = fused_workspace_bytes(a.M, a.K, a.N, a.r, sg.count);
  if (!a.ws || a.ws_bytes < need) return fail(MCB_ERR_WORKSPACE, "%s: workspace %zu < %zu bytes", op, a.ws_bytes, need);
  if ((reinterpret_cast<uintptr_t>(a.ws) & 1023u) != 0) return fail(MCB_ERR_ALIGN, "%s: workspace must be 1024-byte aligned", op);
  return MCB_OK;
}
}  // namespace

size_t fused_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t r, int segments) {
  if (r <= 0 || segments <= 0) return 0;
  return carve_fused(nullptr, M, K, N, r * segments).total;
}

int linear_fused_fwd(const LoraArgs& a, const LoraSegments& sg, const DeviceState* ds) {
  if (a.w_layout != MCB_W_OUT_IN) return fail(MCB_ERR_UNSUPPORTED, "lora_linear_fused_fwd(bf16) needs W as [out,in]");
  if (int rc = check_fused(a, sg, "lora_linear_fused_fwd")) return rc;
  const int64_t r_tot = a.r * sg.count;
  const int rp = static_cast<int>(rank_padded(r_tot));
  FusedWorkspace f = carve_fused(a.ws, a.M, a.K, a.N, r_tot);
  if (int rc = pack_fused(a, sg, f.w, rp, 0)) return rc;
  GemmCall c;
  c.after_pack = true;
  c.X = static_cast<const __nv_bfloat16*>(a.x);
  c.W = static_cast<const __nv_bfloat16*>(a.W);
  c.bias = static_cast<const __nv_bfloat16*>(a.bias);
  c.R = static_cast<const __nv_bfloat16*>(a.residual);
  c.Y = static_cast<__nv_bfloat16*>(a.y);
  c.M = a.M; c.N = a.N; c.K = a.K;
  c.P = f.w.P; c.Q = f.w.Q;
  c.H = static_cast<__nv_bfloat16*>(a.h_save);
  c.h_pitch = h_pitch(a.M);
  c.rp = rp;
  c.r_true = static_cast<int>(r_tot);
  c.scale = a.scale;
  return launch_gemm(c, ds, a.stream);
}

int linear_fused_bwd(const LoraArgs& a, const LoraSegments& sg, const DeviceState* ds) {
  if (a.dx != nullptr && a.w_layout != MCB_W_IN_OUT) return fail(MCB_ERR_UNSUPPORTED, "lora_linear_fused_bwd(bf16) needs W as [in,out]");
  if (int rc = check_fused(a, sg, "lora_linear_fused_bwd")) return rc;
  if (a.h_save == nullptr) return fail(MCB_ERR_NULL, "lora_linear_fused_bwd: the forward's h_save is required");
  bool want_grads = false;
  for (int i = 0; i < sg.count; ++i) {
    if ((sg.dA[i] == nullptr) != (sg.dB[i] == nullptr) || (i > 0 && (sg.dA[i] == nullptr) != (sg.dA[0] == nullptr)))
      return fail(MCB_ERR_NULL, "lora_linear_fused_bwd: pass dA and dB for every segment, or for none");
    want_grads = want_grads || sg.dA[i] != nullptr;
  }
  const int64_t r_tot = a.r * sg.count;
  const int rp = static_cast<int>(rank_padded(r_tot));
  FusedWorkspace f = carve_fused(a.ws, a.M, a.K, a.N, r_tot);
  if (int rc = pack_fused(a, sg, f.w, rp, 1)) return rc;
  GemmCall c;
  c.after_pack = true;
  c.X = static_cast<const __nv_bfloat16*>(a.dy);
  c.W = a.dx != nullptr ? static_cast<const __nv_bfloat16*>(a.W) : nullptr;
  c.Y = static_cast<__nv_bfloat16*>(a.dx);
  c.R = a.dx != nullptr ? static_cast<const __nv_bfloat16*>(a.residual) : nullptr;
  c.M = a.M; c.N = a.K; c.K = a.N;
  c.P = f.w.P; c.Q = f.w.Q;
  c.H = want_grads ? f.w.H1 : nullptr;
  c.h_pitch = h_pitch(a.M);
  c.rp = rp;
  c.r_true = static_cast<int>(r_tot);
  c.scale = a.scale;
  if (int rc = launch_gemm(c, ds, a.stream)) return rc;
  if (!want_grads) return MCB_OK;
  // dA_cat = x^T (scale dy B_bd^T), dB_cat = (scale x A_cat)^T dy: one launch, then the segments' own blocks go out
  if (int rc = launch_grad2(static_cast<const __nv_bfloat16*>(a.x), f.w.H1, a.K, f.dA_cat, 0,
                            static_cast<const __nv_bfloat16*>(a.dy), static_cast<const __nv_bfloat16*>(a.h_save), a.N, f.dB_cat, 1,
                            h_pitch(a.M), f.w.part, a.M, static_cast<int>(r_tot), rp, 0, ds, a.stream))
    return rc;
  ScatterTable t;
  memset(&t, 0, sizeof(t));
  t.count = sg.count;
  int64_t elems = a.K * r_tot;
  for (int i = 0; i < sg.count; ++i) {
    t.dA[i] = sg.dA[i]; t.dB[i] = sg.dB[i];
    t.n_off[i] = static_cast<int>(sg.n_off[i]); t.n[i] = static_cast<int>(sg.n[i]);
    elems += a.r * sg.n[i];
  }
  scatter_fused_grads_kernel<<<static_cast<unsigned>((elems + 255) / 256), 256, 0, a.stream>>>(
      t, f.dA_cat, f.dB_cat, static_cast<int>(a.K), static_cast<int>(a.N), static_cast<int>(a.r), a.accumulate);
  MCB_CHECK_LAUNCH("scatter_fused_grads");
  return MCB_OK;
}

int matmul_nt(const void* a, const void* bt, void* out, int64_t M, int64_t K, int64_t N, const DeviceState* ds,
              cudaStream_t st) {
  GemmCall c;
  c.X = static_cast<const __nv_bfloat16*>(a);
  c.W = static_cast<const __nv_bfloat16*>(bt);
  c.Y = static_cast<__nv_bfloat16*>(out);
  c.M = M; c.N = N; c.K = K;
  return launch_gemm(c, ds, st);
}

}  // namespace bf16path

int init_gemm_kernels() { return bf16path::init_kernels(); }

}  // namespace mcb
