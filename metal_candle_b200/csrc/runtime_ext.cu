// Library switches, the device-status check that maps a run-out wait to MCB_ERR_DEVICE_TIMEOUT, and the
// self-test that makes a bounded wait run out on purpose (without faulting or hanging anything).
#include <atomic>

#include "common.cuh"
#include "umma_ptx.cuh"

namespace mcb {
namespace {
std::atomic<int> g_options[MCB_OPT_COUNT_] = {{1}, {1536}, {1}};   // MCB_OPT_GRAD_TAIL on, MCB_OPT_PAIR_MIN_K 1536, MCB_OPT_PDL on
}

namespace {
std::atomic<long long> g_launches{0};
}
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int option(int which) { return (which >= 0 && which < MCB_OPT_COUNT_) ? g_options[which].load() : 0; }

namespace {

// One warp.  Thread 0 waits on an mbarrier that nothing ever arrives at, with the same bounded wait the GEMM and
// attention kernels use but a caller-chosen limit.  When the limit passes the wait records `code` in the device
// status word and in the CTA's abort flag, every thread falls through, and the kernel returns normally: the
// context stays usable.  out[0] = 1 if the wait gave up, 0 if it (impossibly) succeeded; out[1] = cycles waited.
__global__ void wait_timeout_selftest_kernel(long long limit_cycles, int code, int* status, long long* out) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t bar_addr = umma::smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    umma::mbar_init(bar_addr, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool ok = umma::mbar_wait_limit(bar_addr, 0, &abort_flag, code, status, limit_cycles);
    out[0] = ok ? 0 : 1;
    out[1] = clock64() - t0;
  }
  __syncwarp();
  // the other lanes see the abort flag exactly as the roles of the real kernels do
  if (threadIdx.x == 1) out[2] = abort_flag;
}

}  // namespace
}  // namespace mcb

using namespace mcb;

extern "C" int mcb_set_option(int option_id, int value) {
  if (option_id < 0 || option_id >= MCB_OPT_COUNT_) return fail(MCB_ERR_SHAPE, "mcb_set_option: unknown option %d", option_id);
  g_options[option_id].store(value);
  return MCB_OK;
}

extern "C" int mcb_get_option(int option_id, int* value_out) {
  if (!value_out) return fail(MCB_ERR_NULL, "mcb_get_option: null output");
  if (option_id < 0 || option_id >= MCB_OPT_COUNT_) return fail(MCB_ERR_SHAPE, "mcb_get_option: unknown option %d", option_id);
  *value_out = g_options[option_id].load();
  return MCB_OK;
}

extern "C" int64_t mcb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int mcb_check_device(void) {
  int st = 0;
  if (int rc = mcb_device_status(&st)) return rc;
  if (st != 0)
    return fail(MCB_ERR_DEVICE_TIMEOUT, "a bounded device-side wait ran out (code %d): results of the calls since the last "
                "check are invalid", st);
  return MCB_OK;
}

extern "C" int mcb_selftest_wait_timeout(int64_t limit_cycles, int64_t* waited_cycles_out, void* stream) {
  if (limit_cycles <= 0 || limit_cycles > 2000000000ll)
    return fail(MCB_ERR_SHAPE, "mcb_selftest_wait_timeout: limit of %lld cycles (1 .. 2e9)", (long long)limit_cycles);
  DeviceState* ds = current_device_state();
  if (!ds) return MCB_ERR_NOT_INIT;
  // the three result words live behind the status word's allocation-free neighbour: a pinned host buffer would
  // need an allocation per call, so the kernel writes into a small device buffer owned by the device state
  long long* out = ds->selftest_out;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MCB_CHECK_CUDA(cudaMemsetAsync(out, 0, 3 * sizeof(long long), st));
  wait_timeout_selftest_kernel<<<1, 32, 0, st>>>(static_cast<long long>(limit_cycles), MCB_WAIT_CODE_SELFTEST, ds->status_word, out);
  MCB_CHECK_LAUNCH("wait_timeout_selftest_kernel");
  long long host[3] = {0, 0, 0};
  MCB_CHECK_CUDA(cudaMemcpyAsync(host, out, sizeof(host), cudaMemcpyDeviceToHost, st));
  MCB_CHECK_CUDA(cudaStreamSynchronize(st));
  if (waited_cycles_out) *waited_cycles_out = host[1];
  if (host[0] != 1 || host[2] != MCB_WAIT_CODE_SELFTEST)
    return fail(MCB_ERR_UNSUPPORTED, "mcb_selftest_wait_timeout: the wait did not give up (gave_up=%lld abort_flag=%lld)",
                host[0], host[2]);
  return MCB_OK;
}
