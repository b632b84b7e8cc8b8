// Host-side admission of a plan before any kernel launches: integrity hashes,
// header/section contract, and the per-instruction operand proof. After this the
// dispatcher launches blindly, as the reference's does. Error strings start with
// a unit name the reference registers ("UpdateEngine: " / "PlanValidator: ") so
// callers that route diagnostics by unit keep working (reference:
// runtime/engine/contract.cc:18-33).
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "backend.h"

namespace seeml_b200 {
namespace {

constexpr uint64_t kBasis = 0xcbf29ce484222325ull, kPrime = 0x100000001b3ull;

inline uint64_t mix_word(uint64_t st, uint64_t w) {
  for (int b = 0; b < 8; ++b) {
    st ^= (w >> (8 * b)) & 0xff;
    st *= kPrime;
  }
  return st;
}
// Eight interleaved FNV-1a lanes over one span; [zero_at, zero_at+zero_n) reads as 0
// (the sealed hash field). Reference: source/identity/hash.h:89-109.
uint64_t striped(const uint8_t* p, size_t n, size_t zero_at, size_t zero_n) {
  uint64_t lane[8];
  for (size_t l = 0; l < 8; ++l) lane[l] = kBasis ^ (0x9E3779B97F4A7C15ull * (l + 1));
  auto byte_at = [&](size_t i) -> uint8_t {
    return (i >= zero_at && i < zero_at + zero_n) ? 0 : p[i];
  };
  size_t i = 0;
  if (zero_n == 0) {
    for (; i + 8 <= n; i += 8)
      for (size_t l = 0; l < 8; ++l) lane[l] = (lane[l] ^ p[i + l]) * kPrime;
  } else {
    for (; i + 8 <= n; i += 8)
      for (size_t l = 0; l < 8; ++l) lane[l] = (lane[l] ^ byte_at(i + l)) * kPrime;
  }
  for (size_t l = 0; i < n; ++i, ++l) lane[l] = (lane[l] ^ byte_at(i)) * kPrime;
  uint64_t h = kBasis;
  for (size_t l = 0; l < 8; ++l) h = mix_word(h, lane[l]);
  return mix_word(h, n);
}
// Chunk size is a function of the buffer size only (1 MiB, raised so that at most
// 256 chunks exist), so the digest is the same however many threads compute it.
uint64_t chunked(const uint8_t* p, size_t n, size_t hash_off, bool seal) {
  size_t grain = size_t{1} << 20;
  const size_t cap = (n + 255) / 256;
  if (grain < cap) grain = cap;
  const size_t chunks = n == 0 ? 1 : (n + grain - 1) / grain;
  std::vector<uint64_t> part(chunks, 0);
  auto one = [&](size_t c) {
    const size_t b = c * grain, e = b + grain < n ? b + grain : n;
    size_t za = ~size_t{0}, zn = 0;
    if (seal && hash_off < e && hash_off + 8 > b) {
      const size_t lo = hash_off > b ? hash_off : b;
      const size_t hi = hash_off + 8 < e ? hash_off + 8 : e;
      za = lo - b;
      zn = hi - lo;
    }
    part[c] = striped(p + b, e - b, za, zn);
  };
  unsigned nt = std::thread::hardware_concurrency();
  if (nt > 16) nt = 16;
  if (chunks < 8 || nt < 2) {
    for (size_t c = 0; c < chunks; ++c) one(c);
  } else {
    std::vector<std::thread> pool;
    for (unsigned t = 0; t < nt; ++t)
      pool.emplace_back([&, t] {
        for (size_t c = t; c < chunks; c += nt) one(c);
      });
    for (auto& th : pool) th.join();
  }
  uint64_t h = kBasis;
  for (size_t c = 0; c < chunks; ++c) h = mix_word(h, part[c]);
  return mix_word(h, n);
}

inline bool mul_ok(uint64_t a, uint64_t b, uint64_t* out) {
  if (b != 0 && a > UINT64_MAX / b) return false;
  *out = a * b;
  return true;
}
inline bool range_ok(uint64_t off, uint64_t bytes, uint64_t space) {
  return off <= space && bytes <= space - off;
}

}  // namespace

uint64_t content_hash64(const uint8_t* p, uint64_t n) { return chunked(p, n, 0, false); }
uint64_t plan_self_hash(const uint8_t* p, uint64_t n, uint64_t hash_off) {
  return chunked(p, n, hash_off, true);
}

// Per-opcode operand extents (elements of 4 bytes; int8 B operands 1 byte), address
// spaces and aliasing. Reference: runtime/validator/plan_validator.cc:9-343.
std::string validate_instruction(const Instr& ins, uint64_t arena_size, uint64_t rodata_size,
                                 uint32_t version) {
  return validate_instruction_ranges(ins, arena_size, rodata_size, version, nullptr);
}

std::string validate_instruction_ranges(const Instr& ins, uint64_t arena_size, uint64_t rodata_size,
                                        uint32_t version, std::vector<OpRange>* ranges_out) {
  const std::string opc = std::to_string(ins.opcode);
  if (version < kFlagsVersion) {
    if (ins.flags != 0)
      return "PlanValidator: instruction carries flags in a pre-v5 plan (opcode " + opc + ")";
  } else {
    const uint16_t allowed = ins.opcode == kGemmNN ? kKnownFlags
                             : ins.opcode == kGemmNNQ8 ? kFlagActMask : uint16_t{0};
    if (ins.flags & static_cast<uint16_t>(~allowed))
      return "PlanValidator: unknown or misplaced instruction flags " + std::to_string(ins.flags) +
             " (opcode " + opc + ")";
  }
  if (ins.opcode >= kRmsNormFwd && ins.opcode <= kAttnDK && version < kTransformerVersion)
    return "PlanValidator: transformer opcode " + opc + " in a pre-v6 plan";
  if (ins.opcode == kEmbedFwd && version < kTokenVersion)
    return "PlanValidator: token opcode " + opc + " in a pre-v7 plan";

  struct Range { uint64_t off, bytes; bool write, ro; };
  Range rg[8];
  int nr = 0;
  bool bad = false;
  auto operand = [&](uint64_t ref, uint64_t elems, bool write, uint64_t esz = 4) {
    uint64_t bytes = 0;
    if (ref == kNullRef || (write && is_rodata(ref)) || elems == 0 || !mul_ok(elems, esz, &bytes) ||
        ref_off(ref) % esz != 0 ||
        !range_ok(ref_off(ref), bytes, is_rodata(ref) ? rodata_size : arena_size)) {
      bad = true;
      return;
    }
    if (nr < 8) rg[nr++] = {ref_off(ref), bytes, write, is_rodata(ref)};
  };
  const uint64_t d0 = ins.out[0], d1 = ins.out[1], d2 = ins.out[2];
  auto hi = [](uint64_t w) { return w >> 32; };
  auto lo = [](uint64_t w) { return w & 0xFFFFFFFFu; };
  auto prod = [&](uint64_t a, uint64_t b) {
    uint64_t r = 0;
    if (!mul_ok(a, b, &r)) bad = true;
    return r;
  };
  // [B*S, H*d] activation volume and [B*H*S, S] probability volume
  auto geometry = [&](uint64_t bs, uint64_t hd, uint64_t* td, uint64_t* pn) {
    const uint64_t B = hi(bs), S = lo(bs), H = hi(hd), d = lo(hd);
    if (B == 0 || S == 0 || H == 0 || d == 0) { bad = true; return; }
    const uint64_t t = prod(B, S), dm = prod(H, d);
    *td = prod(t, dm);
    *pn = prod(prod(t, H), S);
  };
  const uint64_t* in = ins.in;
  switch (ins.opcode) {
    case kNop: break;
    case kGemmNN: case kGemmNT: case kGemmTN: case kGemmAccNN: case kGemmNNQ8: case kGemmNTQ8: {
      const bool q8 = ins.opcode == kGemmNNQ8 || ins.opcode == kGemmNTQ8;
      const uint64_t mk = prod(d0, d2), kn = prod(d2, d1), mn = prod(d0, d1);
      if (q8 && !is_rodata(in[1])) bad = true;
      if (!bad) {
        operand(in[0], mk, false);
        operand(in[1], kn, false, q8 ? 1 : 4);
        operand(in[2], mn, true);
        if (ins.flags & kFlagBias) operand(in[3], d1, false);
      }
      break;
    }
    case kAddEW: case kMulEW: case kReluBwd: case kGeluBwd: case kSiluBwd:
      operand(in[0], d0, false); operand(in[1], d0, false); operand(in[2], d0, true); break;
    case kAddBias: {
      const uint64_t mn = prod(d0, d1);
      if (!bad) { operand(in[0], mn, false); operand(in[1], d1, false); operand(in[2], mn, true); }
      break;
    }
    case kReluFwd: case kGeluFwd: case kSiluFwd: case kScale: case kCopy:
      operand(in[0], d0, false); operand(in[1], d0, true); break;
    case kLayerNormFwd: {
      const uint64_t rows = hi(d0), cols = lo(d0), nc = prod(rows, cols);
      if (!bad) {
        operand(in[0], nc, false); operand(in[1], cols, false); operand(in[2], cols, false);
        operand(in[3], nc, true); operand(ins.out[1], rows, true); operand(ins.out[2], rows, true);
      }
      break;
    }
    case kLayerNormBwd: {
      const uint64_t rows = hi(d2), cols = lo(d2), nc = prod(rows, cols);
      if (!bad) {
        operand(in[0], nc, false); operand(in[1], nc, false); operand(in[2], cols, false);
        operand(in[3], nc, true); operand(ins.out[0], rows, false); operand(ins.out[1], rows, false);
      }
      break;
    }
    case kClipNorm: operand(in[0], d0, true); break;
    case kReduceRows: {
      const uint64_t mn = prod(d0, d1);
      if (!bad) { operand(in[0], mn, false); operand(in[1], d1, true); }
      break;
    }
    case kXentFwd: {
      const uint64_t nc = prod(d0, d1);
      if (!bad) {
        operand(in[0], nc, false); operand(in[1], d0, false); operand(in[2], 1, true);
        operand(in[3], nc, true);
      }
      break;
    }
    case kXentBwd: {
      const uint64_t nc = prod(d0, d1);
      if (!bad) {
        operand(in[0], nc, false); operand(in[1], d0, false); operand(in[2], 1, false);
        operand(in[3], nc, true);
      }
      break;
    }
    case kMseFwd:
      operand(in[0], d0, false); operand(in[1], d0, false); operand(in[2], 1, true); break;
    case kMseBwd:
      operand(in[0], d0, false); operand(in[1], d0, false); operand(in[2], 1, false);
      operand(in[3], d0, true); break;
    case kKlFwd: {
      const uint64_t nc = prod(hi(d1), lo(d1));
      if (!bad) {
        operand(in[0], nc, false); operand(in[1], nc, false); operand(in[2], 1, true);
        operand(in[3], nc, true); operand(ins.out[0], nc, true);
      }
      break;
    }
    case kKlBwd: {
      const uint64_t nc = prod(hi(d0), lo(d0));
      if (!bad) {
        operand(in[0], nc, false); operand(in[1], nc, false); operand(in[2], 1, false);
        operand(in[3], nc, true);
      }
      break;
    }
    case kSgd: operand(in[0], d0, true); operand(in[1], d0, false); break;
    case kAdamW:
      operand(in[0], d0, true); operand(in[1], d0, false); operand(in[2], d0, true);
      operand(in[3], d0, true); break;
    case kFill: operand(in[0], d0, true); break;
    case kRmsNormFwd: {
      const uint64_t rows = hi(d0), cols = lo(d0), nc = prod(rows, cols);
      if (!bad) {
        operand(in[0], nc, false); operand(in[1], cols, false); operand(in[2], nc, true);
        operand(in[3], rows, true);
      }
      break;
    }
    case kRmsNormBwd: {
      const uint64_t rows = hi(d1), cols = lo(d1), nc = prod(rows, cols);
      if (!bad) {
        operand(in[0], nc, false); operand(in[1], nc, false); operand(in[2], cols, false);
        operand(in[3], nc, true); operand(ins.out[0], rows, false);
      }
      break;
    }
    case kRopeFwd: case kRopeBwd: {
      uint64_t td = 0, pn = 0;
      geometry(d0, d1, &td, &pn);
      if (lo(d1) % 2 != 0) bad = true;  // rotation pairs need an even head width
      if (!bad) { operand(in[0], td, false); operand(in[1], td, true); }
      break;
    }
    case kAttnFwd: {
      uint64_t td = 0, pn = 0;
      geometry(d1, d2, &td, &pn);
      if (!bad) {
        operand(in[0], td, false); operand(in[1], td, false); operand(in[2], td, false);
        operand(in[3], td, true); operand(ins.out[0], pn, true);
      }
      break;
    }
    case kAttnDP: {
      uint64_t td = 0, pn = 0;
      geometry(d0, d1, &td, &pn);
      if (!bad) { operand(in[0], td, false); operand(in[1], td, false); operand(in[2], pn, true); }
      break;
    }
    case kAttnDV: case kAttnDQ: case kAttnDK: {
      uint64_t td = 0, pn = 0;
      geometry(d0, d1, &td, &pn);
      if (!bad) { operand(in[0], pn, false); operand(in[1], td, false); operand(in[2], td, true); }
      break;
    }
    case kSoftmaxRowsBwd: {
      const uint64_t nc = prod(hi(d0), lo(d0));
      if (!bad) { operand(in[0], nc, false); operand(in[1], nc, false); operand(in[2], nc, true); }
      break;
    }
    case kEmbedFwd: {
      const uint64_t vocab = hi(d1), dim = lo(d1);
      const uint64_t vd = prod(vocab, dim), td = prod(d0, dim);
      if (!is_rodata(in[1])) bad = true;
      if (!bad) { operand(in[0], d0, false); operand(in[1], vd, false); operand(in[2], td, true); }
      break;
    }
    default:
      return "PlanValidator: unknown opcode " + opc;
  }
  if (bad) return "PlanValidator: instruction operand out of bounds (opcode " + opc + ")";
  // a written range may not overlap any other operand of the same instruction
  for (int i = 0; i < nr; ++i)
    for (int j = i + 1; j < nr; ++j) {
      const Range& a = rg[i];
      const Range& b = rg[j];
      if (!(a.write || b.write) || a.ro != b.ro) continue;
      if (a.off < b.off + b.bytes && b.off < a.off + a.bytes)
        return "PlanValidator: instruction operands alias a written range (opcode " + opc + ")";
    }
  if (ranges_out) {
    ranges_out->clear();
    for (int i = 0; i < nr; ++i) ranges_out->push_back({rg[i].off, rg[i].bytes, rg[i].write, rg[i].ro});
  }
  return {};
}

// Whole-plan admission. Reference: runtime/engine/update_engine.cc:80-225,
// runtime/engine/contract.cc:35-168.
std::string verify_plan(const uint8_t* plan, uint64_t size, PlanHeader* out) {
  PlanHeader h{};
  if (!plan || size < sizeof(h)) return "UpdateEngine: plan smaller than its header";
  std::memcpy(&h, plan, sizeof(h));
  if (h.magic != kSeeuMagic) return "UpdateEngine: bad plan magic";
  if (h.version < kSeeuOldestReadable || h.version > kSeeuVersion)
    return "UpdateEngine: unsupported plan version " + std::to_string(h.version) +
           " (this runtime reads v" + std::to_string(kSeeuOldestReadable) + "..v" +
           std::to_string(kSeeuVersion) + ")";
  if (plan_self_hash(plan, size, offsetof(PlanHeader, plan_hash)) != h.plan_hash)
    return "UpdateEngine: plan hash mismatch — the .seeu blob is corrupt";

  uint64_t tb = 0, mb = 0, eb = 0, emb = 0;
  if (!mul_ok(h.train_instr_count, 64, &tb) || !mul_ok(h.merge_instr_count, 64, &mb) ||
      !mul_ok(h.eval_instr_count, 64, &eb) || !mul_ok(h.emit_count, 24, &emb))
    return "UpdateEngine: plan section size overflows";
  if (!range_ok(h.train_instr_offset, tb, size) || !range_ok(h.merge_instr_offset, mb, size) ||
      !range_ok(h.eval_instr_offset, eb, size) || !range_ok(h.rodata_offset, h.rodata_size, size) ||
      !range_ok(h.persist_init_offset, h.persist_init_size, size) ||
      !range_ok(h.emit_table_offset, emb, size))
    return "UpdateEngine: plan section out of bounds";
  if (h.batch == 0) return "UpdateEngine: plan batch size is zero";
  if (h.input_floats == 0) return "UpdateEngine: plan input width is zero";
  if (h.arena_size > UINT64_MAX - 63) return "UpdateEngine: arena size overflows";
  if (h.persist_init_size > h.arena_size || h.persistent_size > h.arena_size)
    return "UpdateEngine: persistent segment exceeds arena";
  uint64_t in_bytes = 0;
  if (is_rodata(h.input_ref) || ref_off(h.input_ref) % 4 != 0 || !mul_ok(h.input_floats, 4, &in_bytes) ||
      !range_ok(ref_off(h.input_ref), in_bytes, h.arena_size))
    return "UpdateEngine: plan input slot out of bounds";
  if (h.label_kind != 0 && (is_rodata(h.label_ref) || ref_off(h.label_ref) % 4 != 0 ||
                            !range_ok(ref_off(h.label_ref), h.label_bytes, h.arena_size)))
    return "UpdateEngine: plan label slot out of bounds";
  if (is_rodata(h.loss_ref) || ref_off(h.loss_ref) % 4 != 0 ||
      !range_ok(ref_off(h.loss_ref), 4, h.arena_size))
    return "UpdateEngine: plan loss slot out of bounds";

  uint64_t fwd_classes = 0;
  bool any_embed = false;
  struct Sec { uint64_t off, count; bool executable_labels; };
  const Sec secs[3] = {{h.train_instr_offset, h.train_instr_count, true},
                       {h.merge_instr_offset, h.merge_instr_count, false},
                       {h.eval_instr_offset, h.eval_instr_count, true}};
  for (const Sec& s : secs)
    for (uint64_t i = 0; i < s.count; ++i) {
      Instr ins;
      std::memcpy(&ins, plan + s.off + i * 64, 64);
      std::string err = validate_instruction(ins, h.arena_size, h.rodata_size, h.version);
      if (!err.empty()) return err;
      if (ins.opcode == kXentFwd || ins.opcode == kXentBwd) {
        // raw labels index probability rows: they must be the staged, validated slot
        if (h.label_kind != 1) return "UpdateEngine: softmax cross-entropy in a plan without class labels";
        if (ins.in[1] != h.label_ref)
          return "UpdateEngine: softmax labels are not the plan's staged label slot";
        if (ins.out[0] != h.batch) return "UpdateEngine: softmax row count disagrees with the plan batch";
      }
      if (ins.opcode == kXentFwd && s.executable_labels) {
        if (fwd_classes != 0 && fwd_classes != ins.out[1])
          return "UpdateEngine: plan softmax class widths disagree across programs";
        fwd_classes = ins.out[1];
      }
      if (ins.opcode == kEmbedFwd) {
        if (h.input_kind != 1) return "UpdateEngine: embedding gather in a plan without token input";
        if (ins.in[0] != h.input_ref)
          return "UpdateEngine: embedding tokens are not the plan's staged input slot";
        if (ins.out[0] != h.batch) return "UpdateEngine: embedding row count disagrees with the plan batch";
        if ((ins.out[1] >> 32) != 0) any_embed = true;
      }
    }
  if (h.label_kind == 1 && fwd_classes == 0)
    return "UpdateEngine: class-label plan carries no softmax cross-entropy — its labels could never "
           "be validated";
  if (h.input_kind > 1) return "UpdateEngine: unknown plan input kind " + std::to_string(h.input_kind);
  if (h.input_kind == 1) {
    if (!any_embed)
      return "UpdateEngine: token plan carries no embedding — its token ids could never be validated";
    if (h.seq_len == 0 || h.batch % h.seq_len != 0)
      return "UpdateEngine: token plan sequence length must be nonzero and divide the batch";
  }
  for (uint64_t i = 0; i < h.emit_count; ++i) {
    EmitEntry e;
    std::memcpy(&e, plan + h.emit_table_offset + i * 24, 24);
    if (!range_ok(e.arena_offset, e.byte_size, h.arena_size)) return "UpdateEngine: emit entry outside the arena";
    if (e.arena_offset % 4 != 0 || e.byte_size % 4 != 0) return "UpdateEngine: emit entry misaligned";
  }
  if (out) *out = h;
  return {};
}

}  // namespace seeml_b200

using namespace seeml_b200;
extern "C" {
uint64_t seeml_b200_plan_self_hash(const void* plan, uint64_t size, uint64_t hash_offset) {
  return plan_self_hash(static_cast<const uint8_t*>(plan), size, hash_offset);
}
uint64_t seeml_b200_content_hash64(const void* data, uint64_t size) {
  return content_hash64(static_cast<const uint8_t*>(data), size);
}
int seeml_b200_validate_instruction(const void* instr, uint64_t arena_size, uint64_t rodata_size,
                                    uint32_t version) {
  if (!instr) return fail("PlanValidator: null instruction");
  Instr ins;
  std::memcpy(&ins, instr, 64);
  const std::string err = validate_instruction(ins, arena_size, rodata_size, version);
  return err.empty() ? 0 : fail(err);
}
int seeml_b200_plan_verify(const void* plan, uint64_t size) {
  const std::string err = verify_plan(static_cast<const uint8_t*>(plan), size, nullptr);
  return err.empty() ? 0 : fail(err);
}
}
