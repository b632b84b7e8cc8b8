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

#include "backend.h"
#include "kernels.h"

namespace {

constexpr unsigned long long kMaxRows = 65536;
// per-row loss terms, then the ordered chunk partials (see k::xent_fwd)
static __device__ __align__(256) double g_xent_scratch[kMaxRows + 256];

constexpr int kMaxDevices = 64;
double* g_scratch_addr[kMaxDevices] = {};   // device address of the array, per device ordinal

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
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail("UpdateEngine: no current CUDA device");
  if (!g_scratch_addr[dev]) {
    // The array's name is only a handle on the host; the kernels need its device address.
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_xent_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(xent scratch)");
    g_scratch_addr[dev] = static_cast<double*>(p);
  }
  k::xent_fwd(logits, labels, loss, probs, rows, classes, g_scratch_addr[dev], static_cast<cudaStream_t>(stream));
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "xent launch");
  return 0;
}
