// Inline-PTX wrappers for the Blackwell (sm_100a) asynchronous machinery used by the tensor-core kernels:
// mbarriers with bounded waits, TMA tile loads (never multicast), tcgen05 MMA / commit / fences / tensor-
// memory loads, and the shared-memory matrix and instruction descriptors.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace mcb {
namespace umma {

constexpr int BM = 128;  // rows of every accumulator tile (tensor-memory lanes)
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // waits on global-memory flags (rare, long)
constexpr long long kWaitLimitCycles = 4000000000ll;          // waits on mbarriers: about two seconds of SM cycles

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait or another one ran out).  The limit is counted
// on the SM's own cycle counter, read (like the abort flag) only every 16th poll: the global nanosecond timer is
// slow to read, and a wait that has to poll at all must not pay for that on the critical path of a handshake.
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                                int* status, long long limit_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = 0;
  for (uint32_t spins = 1;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 15u) != 0) continue;
    if (*abort_flag != 0) return false;
    const long long now = clock64();
    if (t0 == 0) t0 = now;
    if (now - t0 > limit_cycles) {
      *abort_flag = code;
      atomicCAS(status, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                          int* status) {
  return mbar_wait_limit(bar, parity, abort_flag, code, status, kWaitLimitCycles);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute may start while
// its predecessor in the stream is still running; `grid_dependency_wait` blocks until the predecessor grid has
// completed and its writes are visible.  `grid_launch_dependents` lets a dependent grid launched with that attribute
// start early (it has no effect otherwise).  Both are no-ops for kernels launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Tiled store shared -> global (rows and columns beyond the tensor's extent are clipped by the copy engine).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// at most N of this thread's store groups may still be reading their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// at most N of this thread's store groups may still be incomplete
template <int N>
__device__ __forceinline__ void bulk_wait_group() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
// at most n (0..2) store groups may still be reading their source
__device__ __forceinline__ void bulk_wait_group_read_n(int n) {
  if (n >= 2) bulk_wait_group_read<2>();
  else if (n == 1) bulk_wait_group_read<1>();
  else bulk_wait_group_read<0>();
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the A operand in tensor memory: row i of A in lane i, its K elements packed two bf16 per 32-bit
// column from a_tmem on (element 2c in the low half of column c); 16 K elements per instruction = 8 columns.
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Shared-memory matrix descriptors (sm_100 format: version 1 in bits 46-47).
//   K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart (SBO); LBO unused (=1).
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
//   K-major, no swizzle: 8x16-byte core matrices; LBO = byte step between 16-byte K chunks,
//   SBO = byte step between 8-row groups.
__device__ __forceinline__ uint64_t desc_noswz(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo >> 4) << 16) |
         (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 46);
}
// Instruction descriptor for kind::f16: D=f32, A=B=bf16, both K-major, M=128, N=n.
__host__ __device__ constexpr uint32_t make_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(BM >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Output staging of the GEMM epilogues: per epilogue warp, up to kEpiBufsMax buffers of 32 rows x 64 bytes
// (32 bf16 columns), rows swizzled in 16-byte units as CU_TENSOR_MAP_SWIZZLE_64B expects.
constexpr int kEpiBufsMax = 3;
constexpr uint32_t kEpiBufBytes = 32 * 64;

// 32 accumulator columns of output row `grow`: + bias, + residual (both only where the element exists),
// rounded to bf16 and packed two per word.
__device__ __forceinline__ void finish_cols(float (&f)[32], const __nv_bfloat16* bias, const __nv_bfloat16* R, int64_t grow,
                                            int gcol, int M, int N, uint32_t (&w)[16]) {
  if (grow < M) {
    if (bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (gcol + j < N) f[j] += __bfloat162float(bias[gcol + j]);
    }
    if (R != nullptr) {
      const uint4* rp4 = reinterpret_cast<const uint4*>(R + grow * N + gcol);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        if (gcol + 8 * q4 + 8 <= N) {
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
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) w[j] = pack_bf16(f[2 * j], f[2 * j + 1]);
}
// This lane's 64-byte row into a staging buffer (generic address of the buffer's first byte).
__device__ __forceinline__ void stage_row(uint8_t* buf, int lane, const uint32_t (&w)[16]) {
  uint8_t* bg = buf + lane * 64;
  const int sw = (lane >> 1) & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(bg + ((j ^ sw) << 4)) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}
// The reverse: this lane's 64-byte row of a staging buffer that a 64-byte-swizzled TMA load has filled.
__device__ __forceinline__ void unstage_row(const uint8_t* buf, int lane, uint32_t (&w)[16]) {
  const uint8_t* bg = buf + lane * 64;
  const int sw = (lane >> 1) & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 v = *reinterpret_cast<const uint4*>(bg + ((j ^ sw) << 4));
    w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
  }
}// Staging buffers with 128-byte rows (64 bf16 columns, CU_TENSOR_MAP_SWIZZLE_128B): 16-byte piece q of row r sits at
// piece q ^ (r & 7).  This lane's row, half `h` (columns 32h .. 32h + 31).
__device__ __forceinline__ void stage_half128(uint8_t* buf, int lane, int h, const uint32_t (&w)[16]) {
  uint8_t* bg = buf + lane * 128;
  const int sw = lane & 7;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(bg + (((4 * h + j) ^ sw) << 4)) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}
__device__ __forceinline__ void unstage_half128(const uint8_t* buf, int lane, int h, uint32_t (&w)[16]) {
  const uint8_t* bg = buf + lane * 128;
  const int sw = lane & 7;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 v = *reinterpret_cast<const uint4*>(bg + (((4 * h + j) ^ sw) << 4));
    w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
  }
}

//   MN-major, 128-byte swizzle: the M (or N) index is the contiguous one.  An atom is 64 elements of M
//   (128 bytes) by 8 rows of K; LBO = byte step between 64-element M atoms, SBO = byte step between
//   8-row K groups.
__device__ __forceinline__ uint64_t desc_sw128_mn(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo >> 4) << 16) |
         (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// A descriptor moved by `bytes` (a multiple of 16) within shared memory: one 32-bit add on its low word.  Lets the
// issuing thread build the descriptors of a tile once and step through stages and K slices cheaply.
__device__ __forceinline__ uint64_t desc_advance(uint64_t d, uint32_t bytes) {
  const uint32_t lo = static_cast<uint32_t>(d) + (bytes >> 4);
  return (d & 0xFFFFFFFF00000000ull) | lo;
}
// Instruction descriptor with the A operand MN-major (bit 15) and B K-major.
__host__ __device__ constexpr uint32_t make_idesc_a_mn(int n) { return make_idesc(n) | (1u << 15); }

}  // namespace umma
}  // namespace mcb
