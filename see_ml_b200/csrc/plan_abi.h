// Byte layout of the SEEU update plan as this backend reads it. The layout is
// the contract with the plan producer: 64-byte instruction words, a 280-byte
// header, 24-byte emit entries, all little-endian and packed (reference:
// source/plan/instruction.h:15-151, source/plan/schema.h:18-178).
#pragma once
#include <cstdint>

namespace seeml_b200 {

constexpr uint64_t kRodataBit = 1ull << 63;
constexpr uint64_t kNullRef = ~0ull;
constexpr uint32_t kSeeuMagic = 0x55454553u;
constexpr uint32_t kSeeuVersion = 7, kSeeuOldestReadable = 4;
constexpr uint32_t kFlagsVersion = 5, kTransformerVersion = 6, kTokenVersion = 7;

enum Opc : uint16_t {
  kNop = 0, kGemmNN = 1, kGemmNT = 2, kGemmTN = 3, kGemmAccNN = 4, kAddEW = 5,
  kAddBias = 6, kReluFwd = 7, kReluBwd = 8, kScale = 9, kReduceRows = 10,
  kXentFwd = 11, kXentBwd = 12, kMseFwd = 13, kMseBwd = 14, kKlFwd = 15,
  kKlBwd = 16, kSgd = 17, kAdamW = 18, kFill = 19, kCopy = 20, kMulEW = 21,
  kGeluFwd = 22, kGeluBwd = 23, kSiluFwd = 24, kSiluBwd = 25, kLayerNormFwd = 26,
  kLayerNormBwd = 27, kClipNorm = 28, kGemmNNQ8 = 29, kGemmNTQ8 = 30,
  kRmsNormFwd = 31, kRmsNormBwd = 32, kRopeFwd = 33, kRopeBwd = 34, kAttnFwd = 35,
  kAttnDP = 36, kAttnDV = 37, kSoftmaxRowsBwd = 38, kAttnDQ = 39, kAttnDK = 40,
  kEmbedFwd = 41, kOpcCount = 42
};

constexpr uint16_t kFlagBias = 1u, kFlagActShift = 1, kFlagActMask = 3u << 1;
constexpr uint16_t kKnownFlags = kFlagBias | kFlagActMask;

#pragma pack(push, 1)
struct Instr {
  uint16_t opcode;
  uint16_t flags;
  uint32_t pad;
  uint64_t in[4];
  uint64_t out[3];
};
struct PlanHeader {
  uint32_t magic, version;
  uint64_t arena_size, persistent_size;
  uint64_t input_ref, input_floats, label_ref, label_bytes;
  uint32_t label_kind, optimizer_kind;
  uint64_t loss_ref;
  uint64_t train_instr_offset, train_instr_count, merge_instr_offset, merge_instr_count;
  uint64_t rodata_offset, rodata_size, persist_init_offset, persist_init_size;
  uint64_t emit_table_offset, emit_count;
  float lr, beta1, beta2, eps, weight_decay;
  uint32_t pad2;
  uint64_t batch, default_steps;
  uint64_t eval_instr_offset, eval_instr_count;
  uint64_t source_model_hash, plan_hash;
  uint32_t lr_schedule, pad3;
  uint64_t warmup_steps;
  float min_lr_factor, clip_norm;
  uint32_t input_kind, pad4;
  uint64_t seq_len;
  uint64_t reserved[2];
};
struct EmitEntry {
  uint64_t smf_data_offset, byte_size, arena_offset;
};
#pragma pack(pop)
static_assert(sizeof(Instr) == 64, "instruction word is 64 bytes");
static_assert(sizeof(PlanHeader) == 280, "plan header is 280 bytes");
static_assert(sizeof(EmitEntry) == 24, "emit entry is 24 bytes");

inline bool is_rodata(uint64_t ref) { return (ref & kRodataBit) != 0; }
inline uint64_t ref_off(uint64_t ref) { return ref & ~kRodataBit; }

}  // namespace seeml_b200
