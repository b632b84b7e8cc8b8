// Plan types under the reference's names, for programs written against the reference
// runtime's headers (source/plan/update_types.h, schema.h:84-178, instruction.h:15-151).
// Layouts are the SEEU on-disk contract: packed, little-endian.
#ifndef SEEML_COMPAT_SOURCE_PLAN_UPDATE_TYPES_H_
#define SEEML_COMPAT_SOURCE_PLAN_UPDATE_TYPES_H_

#include <cstdint>

namespace seeml::update {

inline constexpr uint64_t kRodataBit = 1ull << 63;
inline constexpr uint64_t kNullRef = ~0ull;

#pragma pack(push, 1)
struct UpdateInstruction {
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
static_assert(sizeof(UpdateInstruction) == 64 && sizeof(PlanHeader) == 280 && sizeof(EmitEntry) == 24);

}  // namespace seeml::update

#endif  // SEEML_COMPAT_SOURCE_PLAN_UPDATE_TYPES_H_
