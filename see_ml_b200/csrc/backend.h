// Device context and program executor behind the C ABI (include/seeml_b200.h).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <tuple>
#include <vector>

#include "kernels.h"
#include "plan_abi.h"
#include "seeml_b200.h"

namespace seeml_b200 {

void set_error(const std::string& msg);
int fail(const std::string& msg);           // sets the message, returns 1
int cuda_fail(cudaError_t e, const char* what);

// Host-side validator (validate.cc): empty string = accepted.
std::string validate_instruction(const Instr& ins, uint64_t arena_size, uint64_t rodata_size,
                                 uint32_t version);
// The same proof, also returning the operand byte ranges it established (reads and writes).
struct OpRange { uint64_t off, bytes; bool write, ro; };
std::string validate_instruction_ranges(const Instr& ins, uint64_t arena_size, uint64_t rodata_size,
                                        uint32_t version, std::vector<OpRange>* ranges_out);
std::string verify_plan(const uint8_t* plan, uint64_t size, PlanHeader* header_out);
uint64_t content_hash64(const uint8_t* p, uint64_t n);
uint64_t plan_self_hash(const uint8_t* p, uint64_t n, uint64_t hash_off);

// Tensor-core GEMM hooks (gemm_tc.cu). gemm_tensor_core returns 1 when it handled
// the instruction (launch count in *launches), 0 when the shape/operands are not
// eligible (the CUDA-core path runs instead), -1 on error.
}  // namespace seeml_b200
struct seeml_b200_ctx;
namespace seeml_b200 {
// Destroys every captured range graph of the context (they are captured again on later runs).
void drop_graphs(seeml_b200_ctx* c);
int gemm_tensor_core(seeml_b200_ctx* c, const Instr& ins, int* launches);
int gemm_tensor_core_prepare(seeml_b200_ctx* c, const Instr& ins);
void gemm_tensor_core_release(seeml_b200_ctx* c);
int gemm_tensor_core_error(seeml_b200_ctx* c);
// C[M,N] = (addend +) A[M,K].Bt[N,K]^T (+ A2[M,K2].B2t[N,K2]^T), then bias / activation.
struct TcGemm {
  const float* A; const float* Bt; float* C;
  uint64_t M, N, K;
  const float* A2; const float* B2t; uint64_t K2;
  const float* addend; const float* bias; int act;
  float alpha;                                  // 0 is read as 1 (zero-initialised descriptors)
};
bool gemm_tc_shape_ok(const seeml_b200_ctx* c, uint64_t M, uint64_t N, uint64_t K);
// Batched per-head product C_z = alpha * A_z . B_z (z = b * H + h); every operand is a window
// of a 2-D row-major f32 matrix whose origin for item z is (x, y) = (b*?x[0] + h*?x[1],
// b*?y[0] + h*?y[1]) in (column, row) coordinates. a_t: A stored [K,M]; b_t: B stored [K,N]
// (otherwise [M,K] and [N,K]). causal as in the CUDA-core GEMM descriptor (0..3).
struct TcBatched {
  const float* A; const float* B; float* C;
  uint64_t a_rows, a_cols, b_rows, b_cols, c_rows, c_cols;
  bool a_t, b_t;
  int ax[2], ay[2], bx[2], by[2], cx[2], cy[2];
  int M, N, K, batch, H, causal;
  float alpha;
};
int gemm_tc_batched(seeml_b200_ctx* c, const TcBatched& g);
// Attention forward scores + causal row softmax in one kernel (head width 64, S <= 512).
int attn_scores_softmax_tc(seeml_b200_ctx* c, const float* Q, const float* K, float* P, uint64_t B, uint64_t S,
                           uint64_t H, uint64_t dh, float alpha);
// Backward: dS = P * (dP - rowsum(dP * P)) with dP = dO V^T kept in TMEM (same shape limits).
bool attn_rows_eligible(const seeml_b200_ctx* c, uint64_t B, uint64_t S, uint64_t H, uint64_t dh);
int attn_ds_tc(seeml_b200_ctx* c, const float* dO, const float* V, const float* P, float* dS, uint64_t B, uint64_t S,
               uint64_t H, uint64_t dh);
// Rank-r (LoRA factor) products on the tensor cores; each returns 1 when launched, 0 when the
// shape is not eligible. rank_n: out[M,n] = alpha A[M,K] Bnk[n,K]^T. rank_tn: per-chunk partial
// sums partial[chunk][big][small] of W[T,big]^T S[T,small] over chunk_rows rows each.
int gemm_tc_rank_n(seeml_b200_ctx* c, const float* A, const float* Bnk, float* out, uint64_t M, uint64_t n,
                   uint64_t K, float alpha);
float* gemm_tc_rank_scratch(seeml_b200_ctx* c, uint64_t floats);
void gemm_tc_transpose(seeml_b200_ctx* c, const float* in, float* out, uint64_t K, uint64_t N);
uint64_t gemm_tc_rank_tn_chunk_rows(uint64_t T, uint64_t big, uint64_t small);
int gemm_tc_rank_tn(seeml_b200_ctx* c, const float* W, const float* S, float* partial, uint64_t T, uint64_t big,
                    uint64_t small, uint64_t chunk_rows);
int gemm_tc_launch(seeml_b200_ctx* c, const TcGemm& g);
const float* gemm_tc_transposed_weight(seeml_b200_ctx* c, uint64_t rodata_off, uint64_t K, uint64_t N, bool create);

// A group of consecutive instructions executed by fewer, fused kernels (FUSED mode).
struct FusedStep {
  enum Kind { kLoraFwd = 1, kLoraBwd = 2, kDgradAdd = 3, kAttnDs = 4, kSwigluFwd = 5, kSwigluBwd = 6,
              kRmsBwdAdd = 7, kXent = 8, kAdamWMulti = 9 } kind;
  uint32_t first = 0, count = 0;
  uint32_t idx[8] = {0, 0, 0, 0, 0, 0, 0, 0};   // instruction indices of the group's members by role
  float alpha = 1.0f;
  float* bt = nullptr;                          // side buffer: alpha * B_lora^T, [N, r]
  bool da_last = false;                         // dA after the dgrad GEMM (slot reuse, see backend_fuse.inc)
  bool via_temp = false;                        // result lands in a dead slot first, then moves
  bool via_side = false;                        // result lands in the program's side buffer first, then moves
  bool residual = false;                        // kLoraFwd: the residual add that follows rides the GEMM's addend
  bool skip = false;                            // kSwigluBwd: ds is dead; kXent: probs is dead
  seeml_b200::k::AdamwDesc* descs = nullptr;    // kAdamWMulti: device descriptor table
  uint32_t ndesc = 0, blocks = 0;
};

struct Program {
  std::vector<Instr> instrs;
  std::vector<FusedStep> steps;
  std::vector<int32_t> step_at;                 // instruction index -> steps[] index, -1 = none
  uint32_t version = kSeeuVersion;
  uint32_t mode = SEEML_B200_MODE_CONTRACT;
  uint64_t last_launches = 0;
  float* side = nullptr;                        // fused groups whose output slot aliases a live input stage here
  // One CUDA graph per executed instruction range: the first run of a range executes directly
  // (lazy allocations and attribute calls happen there), the second is captured, later runs
  // replay the graph. The step scalars live in device memory and are written before each launch,
  // so a graph stays valid from step to step.
  struct RangeGraph {
    int runs = 0;
    bool disabled = false;
    cudaGraphExec_t exec = nullptr;
    uint64_t launches = 0;
  };
  std::map<std::pair<uint64_t, uint64_t>, RangeGraph> graphs;
};

}  // namespace seeml_b200

struct seeml_b200_ctx {
  int device = 0;
  cudaStream_t stream = nullptr, copy_stream = nullptr;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  // device staging double buffer for batches (feeder): H2D on copy_stream, D2D on stream
  struct Stage {
    uint8_t* dev = nullptr;
    uint64_t cap = 0, input_bytes = 0, label_bytes = 0;
    cudaEvent_t h2d_done = nullptr, consumed = nullptr;
    bool pending_consume = false;
  } stage[2];
  uint8_t* arena = nullptr;
  uint64_t arena_bytes = 0;
  bool owns_arena = true;
  uint8_t* rodata = nullptr;
  uint64_t rodata_bytes = 0;
  uint32_t gemm_kind = SEEML_B200_GEMM_TF32X3;
  bool timing = false, timed_valid = false;
  // SEEML_B200_UNIT_TIMES=1: device time per dispatched unit (graph replay off), keyed by opcode or
  // fused-group kind (GEMM-carrying units also by shape), printed when the context is destroyed.
  bool unit_times = false;
  std::vector<cudaEvent_t> unit_events;
  std::vector<std::string> unit_keys;
  std::map<std::string, std::pair<double, unsigned long long>> unit_acc;   // label -> device ms, count
  bool use_graphs = true;          // SEEML_B200_GRAPHS=0 turns graph replay off
  // serial number of the instruction / fused group being enqueued: consecutive units of one run
  // differ by one, separate runs by more (kernels use it to tell what may have changed in between)
  uint64_t exec_unit = 0;
  seeml_b200::DevScalars* scalars_dev = nullptr;
  double* loss_scratch = nullptr;
  uint64_t loss_scratch_doubles = 0;
  float* gemm_ws = nullptr;
  uint64_t gemm_ws_floats = 0;
  float* read_slot = nullptr;  // pinned
  // transposed copies of frozen weights, keyed by (rodata offset, rows K, cols N): [N][K]
  std::map<std::tuple<uint64_t, uint64_t, uint64_t>, float*> wt;
  // RoPE (cos,sin) tables keyed by (S, d, base bits)
  std::map<std::tuple<uint64_t, uint64_t, uint32_t>, float2*> rope;
  seeml_b200::k::Span* spans_dev = nullptr;
  uint64_t spans_cap = 0;
  std::vector<std::unique_ptr<seeml_b200::Program>> programs;
};
