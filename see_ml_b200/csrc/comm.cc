// Data-parallel exchange behind the C ABI: NCCL communicators over NVLink for the one
// collective the path has (an all-gather of per-rank partial gradient sets; the fixed-order
// tree over the gathered sets is finished by this library's own kernels, so the result does
// not depend on the GPU count). The reference is single-process and has no counterpart.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, or the library named by
// SEEML_B200_NCCL_LIB): the backend library itself loads on a machine without NCCL, and inside
// a process that already uses NCCL (e.g. through torch) the same copy is shared.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

#include "backend.h"

using namespace seeml_b200;

namespace {

struct NcclApi {
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRank) CommInitRank = nullptr;
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  decltype(&ncclCommAbort) CommAbort = nullptr;
  decltype(&ncclAllGather) AllGather = nullptr;
  decltype(&ncclGetErrorString) GetErrorString = nullptr;
  decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
  bool ok = false;
  std::string why;
};

const NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* name = std::getenv("SEEML_B200_NCCL_LIB");
    void* h = dlopen(name && name[0] ? name : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
      api.why = std::string("cannot load NCCL (") + (dlerror() ? dlerror() : "dlopen failed") + ")";
      return;
    }
    auto sym = [&](const char* s) { return dlsym(h, s); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.CommAbort && api.AllGather &&
             api.GetErrorString && api.CommGetAsyncError;
    if (!api.ok) api.why = "the NCCL library lacks a required entry point";
  });
  return api;
}

int nccl_fail(ncclResult_t r, const char* what) {
  return fail(std::string("UpdateEngine: NCCL error in ") + what + ": " + nccl().GetErrorString(r));
}

}  // namespace

struct seeml_b200_comm {
  ncclComm_t comm = nullptr;
  int device = 0, rank = 0, world = 1;
  bool broken = false;
};

extern "C" {

int seeml_b200_comm_unique_id(void* id_out) {
  if (!id_out) return fail("UpdateEngine: null argument");
  const NcclApi& n = nccl();
  if (!n.ok) return fail("UpdateEngine: " + n.why);
  static_assert(sizeof(ncclUniqueId) == SEEML_B200_COMM_ID_BYTES, "NCCL unique id size");
  ncclUniqueId id;
  if (ncclResult_t r = n.GetUniqueId(&id); r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
  std::memcpy(id_out, &id, sizeof(id));
  return 0;
}

int seeml_b200_comm_init(int device, const void* id, int rank, int world, seeml_b200_comm** out) {
  if (!out || !id) return fail("UpdateEngine: null argument");
  *out = nullptr;
  if (world < 1 || rank < 0 || rank >= world) return fail("UpdateEngine: rank / world size out of range");
  const NcclApi& n = nccl();
  if (!n.ok) return fail("UpdateEngine: " + n.why);
  if (cudaError_t e = cudaSetDevice(device); e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  ncclUniqueId uid;
  std::memcpy(&uid, id, sizeof(uid));
  auto c = new seeml_b200_comm();
  c->device = device;
  c->rank = rank;
  c->world = world;
  if (ncclResult_t r = n.CommInitRank(&c->comm, world, uid, rank); r != ncclSuccess) {
    delete c;
    return nccl_fail(r, "ncclCommInitRank");
  }
  *out = c;
  return 0;
}

void seeml_b200_comm_destroy(seeml_b200_comm* c) {
  if (!c) return;
  if (c->comm) {
    cudaSetDevice(c->device);
    if (c->broken) nccl().CommAbort(c->comm);
    else nccl().CommDestroy(c->comm);
  }
  delete c;
}

int seeml_b200_comm_rank(const seeml_b200_comm* c) { return c ? c->rank : 0; }
int seeml_b200_comm_world(const seeml_b200_comm* c) { return c ? c->world : 1; }

int seeml_b200_comm_allgather(seeml_b200_comm* c, const void* send_device, void* recv_device, uint64_t floats,
                              void* stream) {
  if (!c || !send_device || !recv_device) return fail("UpdateEngine: null argument");
  if (c->broken) return fail("UpdateEngine: the communicator was aborted after an earlier failure");
  if (ncclResult_t r = nccl().AllGather(send_device, recv_device, floats, ncclFloat, c->comm,
                                        static_cast<cudaStream_t>(stream));
      r != ncclSuccess)
    return nccl_fail(r, "ncclAllGather");
  return 0;
}

// Waits for `stream` on the host while watching the communicator: an asynchronous NCCL error, or
// a collective that does not finish within timeout_s (a rank that never posted), aborts the
// communicator and is reported instead of hanging the caller.
int seeml_b200_comm_wait(seeml_b200_comm* c, void* stream, double timeout_s) {
  if (!c) return fail("UpdateEngine: null argument");
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    const cudaError_t q = cudaStreamQuery(static_cast<cudaStream_t>(stream));
    if (q == cudaSuccess) return 0;
    if (q != cudaErrorNotReady) return cuda_fail(q, "stream query");
    ncclResult_t ar = ncclSuccess;
    if (nccl().CommGetAsyncError(c->comm, &ar) != ncclSuccess || (ar != ncclSuccess && ar != ncclInProgress)) {
      c->broken = true;
      nccl().CommAbort(c->comm);
      c->comm = nullptr;
      return fail(std::string("UpdateEngine: NCCL reported an asynchronous error: ") + nccl().GetErrorString(ar));
    }
    const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (timeout_s > 0 && waited > timeout_s) {
      c->broken = true;
      nccl().CommAbort(c->comm);
      c->comm = nullptr;
      return fail("UpdateEngine: gradient exchange did not finish within " + std::to_string(timeout_s) +
                  " s (a rank never posted its collective); communicator aborted");
    }
    std::this_thread::sleep_for(std::chrono::microseconds(waited < 0.01 ? 20 : 200));
  }
}

}  // extern "C"
