// The data-parallel exchange step behind the C ABI: a float32 sum all-reduce of the LoRA gradient buckets over
// NCCL, with the failure handling a training job needs around it.
//
// The reference has no communication layer at all (single device).  This file is host code only.  NCCL is bound at
// run time (dlopen), not at link time: a process that already carries an NCCL (PyTorch's) shares it, any other
// process loads libnccl.so.2 from the loader path, and MCB_NCCL_LIBRARY names another file (the CPU tests point it
// at a stand-in that fails on demand).
//
// Failure handling: communicators are created NON-BLOCKING, so that neither the rendezvous nor an enqueue can
// block the host for ever.  Every call polls ncclCommGetAsyncError against a host deadline; when the deadline
// passes, or NCCL reports an asynchronous error (a peer process died, a link went down), the communicator is
// aborted (ncclCommAbort), marked dead, and the call returns MCB_ERR_COMM_TIMEOUT / MCB_ERR_COMM.  A dead
// communicator refuses further work instead of hanging.  mcb_comm_wait applies the same deadline to work already
// enqueued on a stream (a peer that never joins the collective leaves the kernel spinning on the device; the abort
// is what ends it).
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <mutex>
#include <thread>

#include "common.cuh"

using namespace mcb;

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetVersion)(int*) = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommFinalize)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

std::mutex g_api_mu;
NcclApi g_api;

template <typename F>
bool bind(void* h, const char* name, F* out) {
  *out = reinterpret_cast<F>(dlsym(h, name));
  return *out != nullptr;
}

// 0, or an error status with the message set
int load_nccl() {
  std::lock_guard<std::mutex> lk(g_api_mu);
  if (g_api.handle != nullptr) return MCB_OK;
  void* h = nullptr;
  const char* env = getenv("MCB_NCCL_LIBRARY");
  if (env != nullptr && env[0] != '\0') {
    h = dlopen(env, RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) return fail(MCB_ERR_COMM_UNAVAILABLE, "mcb_comm: cannot load MCB_NCCL_LIBRARY=%s (%s)", env, dlerror());
  } else {
    h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);   // the copy this process already carries, if any
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) return fail(MCB_ERR_COMM_UNAVAILABLE, "mcb_comm: libnccl.so.2 not found (%s)", dlerror());
  }
  NcclApi a;
  a.handle = h;
  const bool ok = bind(h, "ncclGetVersion", &a.GetVersion) && bind(h, "ncclGetUniqueId", &a.GetUniqueId) &&
                  bind(h, "ncclCommInitRankConfig", &a.CommInitRankConfig) &&
                  bind(h, "ncclCommGetAsyncError", &a.CommGetAsyncError) && bind(h, "ncclCommAbort", &a.CommAbort) &&
                  bind(h, "ncclCommDestroy", &a.CommDestroy) && bind(h, "ncclAllReduce", &a.AllReduce) &&
                  bind(h, "ncclGetErrorString", &a.GetErrorString);
  bind(h, "ncclCommFinalize", &a.CommFinalize);  // optional (2.14+)
  if (!ok) return fail(MCB_ERR_COMM_UNAVAILABLE, "mcb_comm: the NCCL library lacks a required entry point");
  g_api = a;
  return MCB_OK;
}

int nccl_fail(ncclResult_t r, const char* what) {
  return fail(MCB_ERR_COMM_BASE + static_cast<int>(r), "NCCL error %d (%s) at %s", static_cast<int>(r),
              g_api.GetErrorString ? g_api.GetErrorString(r) : "?", what);
}

using Clock = std::chrono::steady_clock;

}  // namespace

struct mcb_comm {
  ncclComm_t comm = nullptr;
  int nranks = 0, rank = 0;
  int timeout_ms = 0;
  bool dead = false;      // aborted: every further call is refused
  int aborts = 0;
};

namespace {

void abort_comm(mcb_comm* c) {
  if (c->comm != nullptr && !c->dead) {
    g_api.CommAbort(c->comm);
    c->aborts += 1;
  }
  c->dead = true;
  c->comm = nullptr;
}

// Polls the communicator's asynchronous state until it leaves ncclInProgress or the deadline passes.
// `pending` is the result of the call being completed (ncclSuccess or ncclInProgress).
int settle(mcb_comm* c, ncclResult_t pending, int timeout_ms, const char* what) {
  if (pending != ncclSuccess && pending != ncclInProgress) {
    const int rc = nccl_fail(pending, what);
    abort_comm(c);
    return rc;
  }
  const Clock::time_point t0 = Clock::now();
  for (;;) {
    ncclResult_t st = ncclSuccess;
    const ncclResult_t q = g_api.CommGetAsyncError(c->comm, &st);
    if (q != ncclSuccess) { const int rc = nccl_fail(q, "ncclCommGetAsyncError"); abort_comm(c); return rc; }
    if (st == ncclSuccess) return MCB_OK;
    if (st != ncclInProgress) { const int rc = nccl_fail(st, what); abort_comm(c); return rc; }
    const long long ms = std::chrono::duration_cast<std::chrono::milliseconds>(Clock::now() - t0).count();
    if (timeout_ms > 0 && ms > timeout_ms) {
      abort_comm(c);
      return fail(MCB_ERR_COMM_TIMEOUT, "%s did not complete within %d ms (rank %d of %d): communicator aborted", what,
                  timeout_ms, c->rank, c->nranks);
    }
    std::this_thread::sleep_for(std::chrono::microseconds(ms < 5 ? 20 : 500));
  }
}

}  // namespace

extern "C" int mcb_comm_unique_id(void* id_out) {
  if (!id_out) return fail(MCB_ERR_NULL, "mcb_comm_unique_id: null output");
  if (int rc = load_nccl()) return rc;
  ncclUniqueId id;
  const ncclResult_t r = g_api.GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
  memcpy(id_out, id.internal, MCB_COMM_ID_BYTES);
  return MCB_OK;
}

extern "C" int mcb_comm_init_rank(mcb_comm** comm_out, int nranks, int rank, const void* id, int timeout_ms, int flags) {
  if (!comm_out || !id) return fail(MCB_ERR_NULL, "mcb_comm_init_rank: null pointer");
  *comm_out = nullptr;
  if (nranks <= 0 || rank < 0 || rank >= nranks)
    return fail(MCB_ERR_SHAPE, "mcb_comm_init_rank: rank %d of %d", rank, nranks);
  if (int rc = load_nccl()) return rc;
  mcb_comm* c = new mcb_comm();
  c->nranks = nranks; c->rank = rank; c->timeout_ms = timeout_ms;
  ncclUniqueId uid;
  memcpy(uid.internal, id, MCB_COMM_ID_BYTES);
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = (flags & MCB_COMM_BLOCKING) ? 1 : 0;
  const ncclResult_t r = g_api.CommInitRankConfig(&c->comm, nranks, uid, rank, &cfg);
  if (c->comm == nullptr && r != ncclSuccess && r != ncclInProgress) {
    const int rc = nccl_fail(r, "ncclCommInitRankConfig");
    delete c;
    return rc;
  }
  if (int rc = settle(c, r, timeout_ms, "communicator rendezvous (ncclCommInitRankConfig)")) {
    delete c;
    return rc;
  }
  *comm_out = c;
  return MCB_OK;
}

extern "C" int mcb_comm_allreduce_bucket(mcb_comm* c, float* buf, int64_t count, void* stream) {
  if (!c || !buf) return fail(MCB_ERR_NULL, "mcb_comm_allreduce_bucket: null pointer");
  if (count <= 0) return fail(MCB_ERR_SHAPE, "mcb_comm_allreduce_bucket: count %lld", (long long)count);
  if (c->dead) return fail(MCB_ERR_COMM_DEAD, "mcb_comm_allreduce_bucket: the communicator was aborted");
  MCB_NVTX_RANGE("mcb_comm_allreduce_bucket");
  const ncclResult_t r = g_api.AllReduce(buf, buf, static_cast<size_t>(count), ncclFloat32, ncclSum, c->comm,
                                         static_cast<cudaStream_t>(stream));
  // a non-blocking communicator may hand the enqueue back unfinished; it must settle before the next call
  return settle(c, r, c->timeout_ms, "ncclAllReduce (enqueue)");
}

extern "C" int mcb_comm_wait(mcb_comm* c, void* stream, int timeout_ms) {
  if (!c) return fail(MCB_ERR_NULL, "mcb_comm_wait: null communicator");
  if (c->dead) return fail(MCB_ERR_COMM_DEAD, "mcb_comm_wait: the communicator was aborted");
  const Clock::time_point t0 = Clock::now();
  for (;;) {
    ncclResult_t st = ncclSuccess;
    const ncclResult_t q = g_api.CommGetAsyncError(c->comm, &st);
    if (q != ncclSuccess) { const int rc = nccl_fail(q, "ncclCommGetAsyncError"); abort_comm(c); return rc; }
    if (st != ncclSuccess && st != ncclInProgress) { const int rc = nccl_fail(st, "collective in flight"); abort_comm(c); return rc; }
    bool done = st == ncclSuccess;
    if (done && stream != MCB_COMM_NO_STREAM) {
      const cudaError_t e = cudaStreamQuery(static_cast<cudaStream_t>(stream));
      if (e == cudaErrorNotReady) done = false;
      else if (e != cudaSuccess) return cuda_fail(e, "cudaStreamQuery (mcb_comm_wait)");
    }
    if (done) return MCB_OK;
    const long long ms = std::chrono::duration_cast<std::chrono::milliseconds>(Clock::now() - t0).count();
    if (timeout_ms > 0 && ms > timeout_ms) {
      abort_comm(c);
      return fail(MCB_ERR_COMM_TIMEOUT, "work on the communicator did not finish within %d ms (rank %d of %d; a peer that "
                  "never joined?): communicator aborted", timeout_ms, c->rank, c->nranks);
    }
    std::this_thread::sleep_for(std::chrono::microseconds(ms < 5 ? 20 : 500));
  }
}

extern "C" int mcb_comm_abort(mcb_comm* c) {
  if (!c) return fail(MCB_ERR_NULL, "mcb_comm_abort: null communicator");
  abort_comm(c);
  return MCB_OK;
}

extern "C" int mcb_comm_info(const mcb_comm* c, int* nranks, int* rank, int* dead, int* nccl_version) {
  if (!c) return fail(MCB_ERR_NULL, "mcb_comm_info: null communicator");
  if (nranks) *nranks = c->nranks;
  if (rank) *rank = c->rank;
  if (dead) *dead = c->dead ? 1 : 0;
  if (nccl_version) {
    int v = 0;
    if (g_api.GetVersion) g_api.GetVersion(&v);
    *nccl_version = v;
  }
  return MCB_OK;
}

extern "C" int mcb_comm_destroy(mcb_comm* c) {
  if (!c) return MCB_OK;
  int rc = MCB_OK;
  if (!c->dead && c->comm != nullptr) {
    // flush what was issued, within the deadline; then free
    if (g_api.CommFinalize) {
      const ncclResult_t r = g_api.CommFinalize(c->comm);
      rc = settle(c, r, c->timeout_ms, "ncclCommFinalize");
    }
    if (!c->dead) {
      const ncclResult_t r = g_api.CommDestroy(c->comm);
      if (r != ncclSuccess && rc == MCB_OK) rc = nccl_fail(r, "ncclCommDestroy");
    }
  }
  delete c;
  return rc;
}
