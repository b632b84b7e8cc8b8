// placeholder until the tcgen05 kernel lands
#include "backend.h"
namespace seeml_b200 {
int gemm_tensor_core(seeml_b200_ctx*, const Instr&, int*) { return 0; }
int gemm_tensor_core_prepare(seeml_b200_ctx*, const Instr&) { return 0; }
void gemm_tensor_core_release(seeml_b200_ctx*) {}
}
