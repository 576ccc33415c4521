/* A stand-in for libnccl.so.2 used by the CPU tests of the communicator's failure handling (tests/test_comm_failures.py).
 * It moves no data.  FAKE_NCCL_MODE selects how it misbehaves; every call appends a line to the file FAKE_NCCL_LOG
 * names, so a test can see that the abort really happened.
 *   ok            everything succeeds at once
 *   stuck_init    the rendezvous never completes (a rank that never joins)
 *   slow_init     the rendezvous completes after ~100 ms of ncclInProgress
 *   async_error   after the first all-reduce the communicator reports ncclRemoteError (a peer process died)
 *   stuck_wait    after the first all-reduce the communicator stays ncclInProgress for ever (a peer never joined)
 *   enqueue_error the all-reduce call itself fails with ncclInvalidArgument
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

typedef enum { ncclSuccess = 0, ncclUnhandledCudaError = 1, ncclSystemError = 2, ncclInternalError = 3,
               ncclInvalidArgument = 4, ncclInvalidUsage = 5, ncclRemoteError = 6, ncclInProgress = 7 } ncclResult_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef struct fake_comm { int nranks, rank, reduces; double t0; } *ncclComm_t;
typedef struct { size_t size; unsigned magic, version; int blocking; } ncclConfigHead;

static const char* mode(void) { const char* m = getenv("FAKE_NCCL_MODE"); return m ? m : "ok"; }
static int is(const char* m) { return strcmp(mode(), m) == 0; }
static void note(const char* what) {
  const char* p = getenv("FAKE_NCCL_LOG");
  if (!p) return;
  FILE* f = fopen(p, "a");
  if (f) { fprintf(f, "%s\n", what); fclose(f); }
}
static double now(void) { struct timespec ts; clock_gettime(CLOCK_MONOTONIC, &ts); return ts.tv_sec + ts.tv_nsec * 1e-9; }

ncclResult_t ncclGetVersion(int* v) { *v = 22703; return ncclSuccess; }
const char* ncclGetErrorString(ncclResult_t r) { return r == ncclRemoteError ? "remote process exited or there was a network error" : r == ncclInProgress ? "in progress" : r == ncclSuccess ? "no error" : "fake error"; }
ncclResult_t ncclGetUniqueId(ncclUniqueId* id) { memset(id->internal, 0x5a, sizeof(id->internal)); note("unique_id"); return ncclSuccess; }
ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, void* config) {
  (void)id;
  const ncclConfigHead* c = (const ncclConfigHead*)config;
  note(c && c->blocking == 0 ? "init nonblocking" : "init blocking");
  struct fake_comm* f = (struct fake_comm*)calloc(1, sizeof(*f));
  f->nranks = nranks; f->rank = rank; f->t0 = now();
  *comm = f;
  return (is("stuck_init") || is("slow_init")) ? ncclInProgress : ncclSuccess;
}
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* st) {
  if (is("stuck_init")) *st = ncclInProgress;
  else if (is("slow_init")) *st = (now() - comm->t0 < 0.1) ? ncclInProgress : ncclSuccess;
  else if (is("async_error") && comm->reduces > 0) *st = ncclRemoteError;
  else if (is("stuck_wait") && comm->reduces > 0) *st = ncclInProgress;
  else *st = ncclSuccess;
  return ncclSuccess;
}
ncclResult_t ncclAllReduce(const void* s, void* r, size_t count, int dtype, int op, ncclComm_t comm, void* stream) {
  (void)s; (void)r; (void)count; (void)stream;
  if (dtype != 7 /* ncclFloat32 */ || op != 0 /* ncclSum */) { note("allreduce bad-args"); return ncclInvalidArgument; }
  if (is("enqueue_error")) { note("allreduce error"); return ncclInvalidArgument; }
  comm->reduces += 1;
  note("allreduce");
  return is("stuck_wait") ? ncclInProgress : ncclSuccess;
}
ncclResult_t ncclCommAbort(ncclComm_t comm) { note("abort"); free(comm); return ncclSuccess; }
ncclResult_t ncclCommFinalize(ncclComm_t comm) { (void)comm; note("finalize"); return ncclSuccess; }
ncclResult_t ncclCommDestroy(ncclComm_t comm) { note("destroy"); free(comm); return ncclSuccess; }
