// Softmax cross-entropy forward for callers that must not allocate device memory.
//
// Some hosts of this library run with the CUDA allocator off limits: a runtime that
// handed the whole device to its own arena at start-up, or code on a latency path
// where cudaMalloc's implicit device synchronisation is not acceptable. The regular
// path keeps its reduction scratch (one double per row plus 256 chunk partials) in a
// buffer the context allocates when a program is built. This entry point keeps the
// same scratch in a fixed array that is part of the loaded module instead, so a call
// launches kernels and nothing else. The price is a fixed ceiling on the row count
// and about half a MiB of device memory held by every GPU that loads the library.
#include <cuda_runtime.h>

#include <atomic>

#include "backend.h"
#include "kernels.h"

namespace {

constexpr unsigned long long kMaxRows = 65536;
// per-row loss terms, then the ordered chunk partials (see k::xent_fwd)
static __device__ __align__(256) double g_xent_scratch[kMaxRows + 256];

// Device address of the array, per device ordinal. Several host threads may make their first
// call at once: each looks the address up and publishes the same value.
constexpr int kMaxDevices = 64;
std::atomic<double*> g_scratch_addr[kMaxDevices];

}  // namespace

extern "C" int seeml_b200_xent_fwd_noalloc(const float* logits, const int32_t* labels, float* loss,
                                           float* probs, uint64_t rows, uint64_t classes, void* stream) {
  using namespace seeml_b200;
  if (!logits || !labels || !loss || !probs) return fail("UpdateEngine: null operand");
  if (rows == 0 || classes == 0) return fail("UpdateEngine: empty softmax cross-entropy");
  if (rows > kMaxRows)
    return fail("UpdateEngine: seeml_b200_xent_fwd_noalloc handles at most " + std::to_string(kMaxRows) +
                " rows per call (got " + std::to_string(rows) + "); use the context path for larger batches");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return fail("UpdateEngine: no current CUDA device");
  if (dev >= kMaxDevices)
    return fail("UpdateEngine: seeml_b200_xent_fwd_noalloc supports device ordinals below " +
                std::to_string(kMaxDevices) + " (current device " + std::to_string(dev) + ")");
  // The scratch used is the current device's copy of the array, so the operands must live on the
  // current device too (a pointer query; nothing is allocated).
  cudaPointerAttributes pa{};
  if (cudaPointerGetAttributes(&pa, logits) != cudaSuccess) {
    cudaGetLastError();
    return fail("UpdateEngine: logits is not a CUDA pointer");
  }
  if (pa.type != cudaMemoryTypeDevice && pa.type != cudaMemoryTypeManaged)
    return fail("UpdateEngine: logits must be device memory");
  if (pa.type == cudaMemoryTypeDevice && pa.device != dev)
    return fail("UpdateEngine: the operands live on device " + std::to_string(pa.device) + " but device " +
                std::to_string(dev) + " is current; make the operands' device current before the call");
  double* scratch = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (!scratch) {
    // The array's name is only a handle on the host; the kernels need its device address.
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_xent_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(xent scratch)");
    scratch = static_cast<double*>(p);
    g_scratch_addr[dev].store(scratch, std::memory_order_release);
  }
  k::xent_fwd(logits, labels, loss, probs, rows, classes, scratch, static_cast<cudaStream_t>(stream));
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "xent launch");
  return 0;
}
