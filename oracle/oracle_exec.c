/* TEST INFRASTRUCTURE — see oracle.h. Interpreter for the 64-byte update
 * instruction word (source/plan/instruction.h:27-151), dispatching with the
 * operand conventions of runtime/engine/update_engine.cc:306-509: which in[]
 * words are tensor refs (bit 63 = rodata) or f32-bit immediates, and which
 * out[] words are dims, packed hi<<32|lo pairs, or further refs. */
#include <string.h>

#include "oracle.h"

typedef struct {
  uint16_t opcode, flags;
  uint32_t pad;
  uint64_t in[4];
  uint64_t out[3];
} Ins;

static float bits_f32(uint64_t w) {
  uint32_t u = (uint32_t)w;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

int orc_execute(const uint8_t* program, size_t count, uint8_t* arena,
                const uint8_t* rodata, float lr, float b1, float b2, float eps,
                float wd, uint64_t step) {
  const uint64_t kRo = 1ULL << 63;
#define R(ref) ((const float*)((((ref) & kRo) ? rodata : arena) + ((ref) & ~kRo)))
#define W(ref) ((float*)(arena + ((ref) & ~kRo)))
#define I32(ref) ((const int32_t*)R(ref))
#define HI(w) ((size_t)((w) >> 32))
#define LO(w) ((size_t)((w) & 0xFFFFFFFFu))
  for (size_t idx = 0; idx < count; ++idx) {
    Ins s;
    memcpy(&s, program + idx * 64, 64);
    const uint64_t* in = s.in;
    const uint64_t* o = s.out;
    const int act = (s.flags >> 1) & 3;
    switch (s.opcode) {
      case 0: break;
      case 1: orc_gemm_nn(R(in[0]), R(in[1]), W(in[2]), o[0], o[1], o[2],
                          (s.flags & 1) ? R(in[3]) : NULL, act); break;
      case 2: orc_gemm_nt(R(in[0]), R(in[1]), W(in[2]), o[0], o[1], o[2]); break;
      case 3: orc_gemm_tn(R(in[0]), R(in[1]), W(in[2]), o[0], o[1], o[2]); break;
      case 4: orc_gemm_acc_nn(R(in[0]), R(in[1]), W(in[2]), o[0], o[1], o[2],
                              bits_f32(in[3])); break;
      case 5: orc_add(R(in[0]), R(in[1]), W(in[2]), o[0]); break;
      case 6: orc_add_bias(R(in[0]), R(in[1]), W(in[2]), o[0], o[1]); break;
      case 7: orc_relu_fwd(R(in[0]), W(in[1]), o[0]); break;
      case 8: orc_relu_bwd(R(in[0]), R(in[1]), W(in[2]), o[0]); break;
      case 9: orc_scale(R(in[0]), W(in[1]), bits_f32(in[2]), o[0]); break;
      case 10: orc_reduce_rows(R(in[0]), W(in[1]), o[0], o[1]); break;
      case 11: orc_xent_fwd(R(in[0]), I32(in[1]), W(in[2]), W(in[3]), o[0], o[1]); break;
      case 12: orc_xent_bwd(R(in[0]), I32(in[1]), R(in[2]), W(in[3]), o[0], o[1]); break;
      case 13: orc_mse_fwd(R(in[0]), R(in[1]), W(in[2]), o[0]); break;
      case 14: orc_mse_bwd(R(in[0]), R(in[1]), R(in[2]), W(in[3]), o[0]); break;
      case 15: orc_kl_fwd(R(in[0]), R(in[1]), W(in[2]), W(in[3]), W(o[0]), HI(o[1]),
                          LO(o[1]), bits_f32(o[2])); break;
      case 16: orc_kl_bwd(R(in[0]), R(in[1]), R(in[2]), W(in[3]), HI(o[0]), LO(o[0]),
                          bits_f32(o[1])); break;
      case 17: orc_sgd(W(in[0]), R(in[1]), o[0], lr, wd); break;
      case 18: orc_adamw(W(in[0]), R(in[1]), W(in[2]), W(in[3]), o[0], lr, b1, b2, eps,
                         wd, step); break;
      case 19: orc_fill(W(in[0]), bits_f32(in[1]), o[0]); break;
      case 20: orc_copy(R(in[0]), W(in[1]), o[0]); break;
      case 21: orc_mul(R(in[0]), R(in[1]), W(in[2]), o[0]); break;
      case 22: orc_gelu_fwd(R(in[0]), W(in[1]), o[0]); break;
      case 23: orc_gelu_bwd(R(in[0]), R(in[1]), W(in[2]), o[0]); break;
      case 24: orc_silu_fwd(R(in[0]), W(in[1]), o[0]); break;
      case 25: orc_silu_bwd(R(in[0]), R(in[1]), W(in[2]), o[0]); break;
      case 26: orc_layernorm_fwd(R(in[0]), R(in[1]), R(in[2]), W(in[3]), W(o[1]), W(o[2]),
                                 HI(o[0]), LO(o[0])); break;
      case 27: orc_layernorm_bwd(R(in[0]), R(in[1]), R(in[2]), R(o[0]), R(o[1]), W(in[3]),
                                 HI(o[2]), LO(o[2])); break;
      case 28: orc_clip_norm(W(in[0]), o[0], bits_f32(in[1])); break;
      case 29: orc_gemm_nn_q8(R(in[0]), (const int8_t*)R(in[1]), W(in[2]), o[0], o[1], o[2],
                              bits_f32(in[3]), act); break;
      case 30: orc_gemm_nt_q8(R(in[0]), (const int8_t*)R(in[1]), W(in[2]), o[0], o[1], o[2],
                              bits_f32(in[3])); break;
      case 31: orc_rmsnorm_fwd(R(in[0]), R(in[1]), W(in[2]), W(in[3]), HI(o[0]), LO(o[0])); break;
      case 32: orc_rmsnorm_bwd(R(in[0]), R(in[1]), R(in[2]), R(o[0]), W(in[3]), HI(o[1]),
                               LO(o[1])); break;
      case 33: orc_rope(R(in[0]), W(in[1]), HI(o[0]), LO(o[0]), HI(o[1]), LO(o[1]),
                        bits_f32(o[2]), 0); break;
      case 34: orc_rope(R(in[0]), W(in[1]), HI(o[0]), LO(o[0]), HI(o[1]), LO(o[1]),
                        bits_f32(o[2]), 1); break;
      case 35: orc_attn_fwd(R(in[0]), R(in[1]), R(in[2]), W(in[3]), W(o[0]), HI(o[1]),
                            LO(o[1]), HI(o[2]), LO(o[2])); break;
      case 36: orc_attn_dp(R(in[0]), R(in[1]), W(in[2]), HI(o[0]), LO(o[0]), HI(o[1]),
                           LO(o[1])); break;
      case 37: orc_attn_dv(R(in[0]), R(in[1]), W(in[2]), HI(o[0]), LO(o[0]), HI(o[1]),
                           LO(o[1])); break;
      case 38: orc_softmax_rows_bwd(R(in[0]), R(in[1]), W(in[2]), HI(o[0]), LO(o[0])); break;
      case 39: orc_attn_dq(R(in[0]), R(in[1]), W(in[2]), HI(o[0]), LO(o[0]), HI(o[1]),
                           LO(o[1])); break;
      case 40: orc_attn_dk(R(in[0]), R(in[1]), W(in[2]), HI(o[0]), LO(o[0]), HI(o[1]),
                           LO(o[1])); break;
      case 41: orc_embed(I32(in[0]), R(in[1]), W(in[2]), o[0], LO(o[1])); break;
      default: return (int)idx + 1;
    }
  }
  return 0;
}
