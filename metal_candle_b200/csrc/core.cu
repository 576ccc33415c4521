// Library state: mcb_init, error strings, the device status word, and small utility kernels.
#include <cuda.h>
#include <stdarg.h>
#include <string.h>

#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"

namespace mcb {

namespace {
thread_local char g_err[512] = "";
std::mutex g_mu;
DeviceState g_dev[64];
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_err, sizeof(g_err), "CUDA error %d (%s) at %s", static_cast<int>(e), cudaGetErrorString(e), what);
  return static_cast<int>(e) > 0 ? static_cast<int>(e) : 1;
}

DeviceState* current_device_state() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("no current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_dev[dev].ready) {
    set_error("mcb_init(%d) has not been called", dev);
    return nullptr;
  }
  return &g_dev[dev];
}

int init_gemm_kernels();  // umma_gemm.cu: raises dynamic shared-memory limits

// ---- per-kernel timing -----------------------------------------------------------------------------
namespace {
struct ProfRecord {
  cudaEvent_t a, b;
  int kind;
  double flops, bytes;
};
std::mutex g_prof_mu;
bool g_prof_on = false;
std::vector<ProfRecord> g_prof_live;
std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_prof_pool;
}  // namespace

bool profile_on() { return g_prof_on; }

void profile_begin(int kind, double flops, double bytes, cudaStream_t st) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  ProfRecord r;
  if (!g_prof_pool.empty()) {
    r.a = g_prof_pool.back().first;
    r.b = g_prof_pool.back().second;
    g_prof_pool.pop_back();
  } else {
    if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
  }
  r.kind = kind; r.flops = flops; r.bytes = bytes;
  cudaEventRecord(r.a, st);
  g_prof_live.push_back(r);
}

void profile_end(cudaStream_t st) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (!g_prof_live.empty()) cudaEventRecord(g_prof_live.back().b, st);
}

}  // namespace mcb

using namespace mcb;

extern "C" int mcb_version(void) { return 100; }

extern "C" const char* mcb_last_error(void) { return g_err; }

extern "C" int mcb_init(int device) {
  if (device < 0 || device >= 64) return fail(MCB_ERR_SHAPE, "mcb_init: device %d out of range", device);
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount (no CUDA device: this library has no CPU path)");
  if (device >= count) return fail(MCB_ERR_SHAPE, "mcb_init: device %d but only %d visible", device, count);
  MCB_CHECK_CUDA(cudaSetDevice(device));
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_dev[device].ready) return MCB_OK;
  }
  cudaDeviceProp prop;
  MCB_CHECK_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(MCB_ERR_UNSUPPORTED, "mcb_init: device %d is sm_%d%d; this library is built for sm_100a only",
                device, prop.major, prop.minor);
  DeviceState st;
  st.sm_count = prop.multiProcessorCount;
  MCB_CHECK_CUDA(cudaMalloc(&st.status_word, 64));
  MCB_CHECK_CUDA(cudaMemset(st.status_word, 0, 64));
  st.selftest_out = reinterpret_cast<long long*>(reinterpret_cast<char*>(st.status_word) + 16);
  cudaDriverEntryPointQueryResult qres;
  void* fn = nullptr;
  MCB_CHECK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  if (fn == nullptr || qres != cudaDriverEntryPointSuccess)
    return fail(MCB_ERR_UNSUPPORTED, "mcb_init: driver does not export cuTensorMapEncodeTiled");
  st.encode_tiled = fn;
  if (int rc = init_gemm_kernels()) return rc;
  st.ready = true;
  std::lock_guard<std::mutex> lk(g_mu);
  g_dev[device] = st;
  return MCB_OK;
}

extern "C" int mcb_device_status(int* status_out) {
  if (!status_out) return fail(MCB_ERR_NULL, "mcb_device_status: null output");
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  MCB_CHECK_CUDA(cudaDeviceSynchronize());
  MCB_CHECK_CUDA(cudaMemcpy(status_out, ds->status_word, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status_out != 0) MCB_CHECK_CUDA(cudaMemset(ds->status_word, 0, sizeof(int)));
  return MCB_OK;
}

extern "C" int mcb_profile_enable(int on) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  g_prof_on = on != 0;
  return MCB_OK;
}

extern "C" int mcb_profile_summary(int kind, int64_t* launches, double* total_ms, double* total_flops, double* total_bytes) {
  if (!launches || !total_ms || !total_flops || !total_bytes) return fail(MCB_ERR_NULL, "profile_summary: null output");
  if (kind < 0 || kind >= kProfKinds) return fail(MCB_ERR_SHAPE, "profile_summary: kind %d", kind);
  MCB_CHECK_CUDA(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> lk(g_prof_mu);
  *launches = 0; *total_ms = 0; *total_flops = 0; *total_bytes = 0;
  std::vector<ProfRecord> keep;
  for (const ProfRecord& r : g_prof_live) {
    if (r.kind != kind) { keep.push_back(r); continue; }
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
      *launches += 1; *total_ms += ms; *total_flops += r.flops; *total_bytes += r.bytes;
    }
    g_prof_pool.emplace_back(r.a, r.b);
  }
  g_prof_live.swap(keep);
  return MCB_OK;
}

// ---- transpose ---------------------------------------------------------------------------------
namespace mcb_detail {
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ src, T* __restrict__ dst, int64_t rows, int64_t cols) {
  __shared__ T tile[32][33];
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 32, r0 = static_cast<int64_t>(blockIdx.y) * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    int64_t r = r0 + i, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[i][threadIdx.x] = src[r * cols + c];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    int64_t c = c0 + i, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[c * rows + r] = tile[threadIdx.x][i];
  }
}
}  // namespace mcb_detail
using mcb_detail::transpose_kernel;

extern "C" int mcb_transpose_2d(const void* src, void* dst, int64_t rows, int64_t cols, int dtype, void* stream) {
  MCB_NVTX_RANGE("mcb_transpose_2d");
  if (!src || !dst) return fail(MCB_ERR_NULL, "transpose_2d: null pointer");
  if (rows <= 0 || cols <= 0) return fail(MCB_ERR_SHAPE, "transpose_2d: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (!current_device_state()) return MCB_ERR_NOT_INIT;
  int64_t gy = (rows + 31) / 32, gx = (cols + 31) / 32;
  if (gy > 65535) return fail(MCB_ERR_SHAPE, "transpose_2d: too many rows");
  dim3 grid((unsigned)gx, (unsigned)gy), block(32, 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MCB_F32)
    transpose_kernel<float><<<grid, block, 0, st>>>((const float*)src, (float*)dst, rows, cols);
  else if (dtype == MCB_BF16)
    transpose_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, rows, cols);
  else
    return fail(MCB_ERR_UNSUPPORTED, "transpose_2d: dtype %d", dtype);
  MCB_CHECK_LAUNCH("transpose_2d");
  return MCB_OK;
}
