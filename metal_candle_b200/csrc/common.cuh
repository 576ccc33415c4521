// Shared helpers for the C-ABI implementation: status/error plumbing, dtype access, reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <nvtx3/nvToolsExt.h>

#include "../../include/mcb200.h"

namespace mcb {

// Thread-local message behind mcb_last_error().
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

// Per-device state created by mcb_init.
struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int* status_word = nullptr;  // device int: 0, or the code of a bounded wait that gave up
  long long* selftest_out = nullptr;  // three device words behind the status word (mcb_selftest_wait_timeout)
  void* encode_tiled = nullptr;  // cuTensorMapEncodeTiled resolved through the runtime
};
DeviceState* current_device_state();  // null (and error set) when mcb_init was not called

// Optional per-kernel timing (mcb_profile_enable): CUDA events recorded on the launching stream right
// around one kernel launch, tagged with the launch's algorithmic work.
enum ProfileKind { kProfGemm = 0, kProfGrad = 1, kProfGemmLora = 2, kProfGemmSwigluBwd = 3, kProfKinds = 4 };
bool profile_on();
void profile_begin(int kind, double flops, double bytes, cudaStream_t st);
void profile_end(cudaStream_t st);

// Library switches (mcb_set_option).
int option(int which);

// An NVTX range around the body of an entry point: shows each call (and the kernels it enqueues) by name on a
// profiler's timeline; costs a pointer test when no tool is attached.
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};
#define MCB_NVTX_RANGE(name) mcb::NvtxRange mcb_nvtx_range_(name)

#define MCB_CHECK_CUDA(expr)                                   \
  do {                                                         \
    cudaError_t e_ = (expr);                                   \
    if (e_ != cudaSuccess) return mcb::cuda_fail(e_, #expr);   \
  } while (0)

// Every kernel launch of the library passes through this check; it also counts them (mcb_launch_count).
void note_launch();
#define MCB_CHECK_LAUNCH(name)                                 \
  do {                                                         \
    cudaError_t e_ = cudaGetLastError();                       \
    if (e_ != cudaSuccess) return mcb::cuda_fail(e_, name);    \
    mcb::note_launch();                                        \
  } while (0)

// Kernel launch with or without the programmatic-serialization attribute (see umma_ptx.cuh).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- device-side helpers -----------------------------------------------------------------

template <typename T>
struct Vec16;  // a 16-byte vector of T, convertible to/from floats
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void to_float(float* f) const {
    f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w;
  }
  __device__ __forceinline__ void from_float(const float* f) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ void to_float(float* f) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ void from_float(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    raw = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace mcb
