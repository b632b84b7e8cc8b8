// Device context, program decode and the per-instruction dispatcher: the CUDA
// counterpart of UpdateEngine::ExecuteRange (reference:
// runtime/engine/update_engine.cc:306-509). Operand conventions per opcode — which
// in[] words are tensor refs or f32-bit immediates, which out[] words are dims,
// packed hi<<32|lo pairs or further refs — follow that switch exactly.
#include "backend.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace seeml_b200 {

static thread_local std::string g_error;
void set_error(const std::string& msg) { g_error = msg; }
int fail(const std::string& msg) {
  g_error = msg;
  return 1;
}
int cuda_fail(cudaError_t e, const char* what) {
  g_error = std::string("UpdateEngine: CUDA error in ") + what + ": " + cudaGetErrorString(e);
  return 2;
}
#define CU(call, what)                                     \
  do {                                                     \
    cudaError_t e_ = (call);                               \
    if (e_ != cudaSuccess) return cuda_fail(e_, what);     \
  } while (0)

// Captured range graphs hold the addresses of the context's scratch buffers: whenever one of
// those buffers is replaced, every graph of the context is dropped (its range is captured again
// on a later run).
void drop_graphs(seeml_b200_ctx* c) {
  for (auto& p : c->programs)
    if (p) {
      for (auto& g : p->graphs) if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
      p->graphs.clear();
    }
}

namespace {

inline float bits_f32(uint64_t w) {
  const uint32_t u = static_cast<uint32_t>(w);
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint64_t hi32(uint64_t w) { return w >> 32; }
inline uint64_t lo32(uint64_t w) { return w & 0xFFFFFFFFu; }

struct Exec {
  seeml_b200_ctx* c;
  uint64_t launches = 0;
  const float* R(uint64_t ref) const {
    return reinterpret_cast<const float*>((is_rodata(ref) ? c->rodata : c->arena) + ref_off(ref));
  }
  float* W(uint64_t ref) const { return reinterpret_cast<float*>(c->arena + ref_off(ref)); }
  const int32_t* I(uint64_t ref) const { return reinterpret_cast<const int32_t*>(R(ref)); }
};

k::GemmDesc dense_desc(const float* A, const float* B, float* C, uint64_t M, uint64_t N, uint64_t K) {
  k::GemmDesc d{};
  d.A = A; d.B = B; d.C = C;
  d.M = (int)M; d.N = (int)N; d.K = (int)K;
  d.sCm = (long long)N;
  d.nb_inner = 1; d.batch = 1; d.alpha = 1.0f;
  return d;
}

// Per-(b,h) batched products of the attention primitives over [B*S, H*d] activations
// and the [B*H*S, S] probability matrix (attention.cc:94-242).
k::GemmDesc attn_desc(uint64_t B, uint64_t S, uint64_t H, uint64_t dh) {
  k::GemmDesc d{};
  d.nb_inner = (int)H;
  d.batch = (int)(B * H);
  d.alpha = 1.0f;
  (void)S; (void)dh;
  return d;
}

int ensure_rope(seeml_b200_ctx* c, uint64_t S, uint64_t dh, float base) {
  uint32_t bb;
  std::memcpy(&bb, &base, 4);
  const auto key = std::make_tuple(S, dh, bb);
  if (c->rope.count(key)) return 0;
  // angle(s, pair) with the reference's float recurrence (attention.cc:48-63):
  // step = powf(base, -2/d); freq starts at 1 and is multiplied per pair.
  const uint64_t half = dh / 2;
  std::vector<float2> tab(S * half);
  const float step = std::pow(base, -2.0f / static_cast<float>(dh));
  for (uint64_t s = 0; s < S; ++s) {
    float freq = 1.0f;
    for (uint64_t p = 0; p < half; ++p) {
      const float theta = static_cast<float>(s) * freq;
      tab[s * half + p] = make_float2(std::cos(theta), std::sin(theta));
      freq *= step;
    }
  }
  float2* dev = nullptr;
  CU(cudaMalloc(&dev, tab.size() * sizeof(float2) + 16), "rope table alloc");
  CU(cudaMemcpy(dev, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice), "rope table copy");
  c->rope[key] = dev;
  return 0;
}

int ensure_scratch(seeml_b200_ctx* c, uint64_t loss_doubles, uint64_t ws_floats) {
  if (loss_doubles > c->loss_scratch_doubles || ws_floats > c->gemm_ws_floats) {
    cudaStreamSynchronize(c->stream);     // nothing in flight may still use the old buffers
    drop_graphs(c);
  }
  if (loss_doubles > c->loss_scratch_doubles) {
    if (c->loss_scratch) cudaFree(c->loss_scratch);
    c->loss_scratch = nullptr;
    CU(cudaMalloc(&c->loss_scratch, loss_doubles * sizeof(double)), "loss scratch alloc");
    c->loss_scratch_doubles = loss_doubles;
  }
  if (ws_floats > c->gemm_ws_floats) {
    if (c->gemm_ws) cudaFree(c->gemm_ws);
    c->gemm_ws = nullptr;
    CU(cudaMalloc(&c->gemm_ws, ws_floats * sizeof(float)), "gemm workspace alloc");
    c->gemm_ws_floats = ws_floats;
  }
  return 0;
}

// The GEMM descriptor an instruction lowers to (CUDA-core path).
k::GemmDesc gemm_desc_of(const Exec& x, const Instr& ins) {
  const uint64_t M = ins.out[0], N = ins.out[1], K = ins.out[2];
  k::GemmDesc d = dense_desc(x.R(ins.in[0]), x.R(ins.in[1]), x.W(ins.in[2]), M, N, K);
  switch (ins.opcode) {
    case kGemmNN: case kGemmAccNN: case kGemmNNQ8:
      d.sAm = (long long)K; d.sAk = 1; d.sBk = (long long)N; d.sBn = 1; break;
    case kGemmNT: case kGemmNTQ8:
      d.sAm = (long long)K; d.sAk = 1; d.sBk = 1; d.sBn = (long long)K; break;
    case kGemmTN:
      d.sAm = 1; d.sAk = (long long)M; d.sBk = (long long)N; d.sBn = 1; break;
  }
  if (ins.opcode == kGemmAccNN) { d.accumulate = 1; d.alpha = bits_f32(ins.in[3]); }
  if (ins.opcode == kGemmNNQ8 || ins.opcode == kGemmNTQ8) {
    d.Bq8 = reinterpret_cast<const int8_t*>(d.B);
    d.alpha = bits_f32(ins.in[3]);
  }
  if (ins.opcode == kGemmNN && (ins.flags & kFlagBias)) d.bias = x.R(ins.in[3]);
  if (ins.opcode == kGemmNN || ins.opcode == kGemmNNQ8) d.act = (ins.flags & kFlagActMask) >> kFlagActShift;
  return d;
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Rank-r shapes go to the dedicated kernels. Returns the launch count, or 0 when the
// instruction is not one of those shapes.
// Rank-r products: the tensor-core kernels when the shape allows, else the CUDA-core ones.
// Both return the number of kernels launched.
int rank_n(seeml_b200_ctx* c, const float* A, const float* B, float* out, int M, int n, int K, int b_is_nk,
           float alpha) {
  const float* bnk = B;
  int extra = 0;
  if (!b_is_nk && n >= 16 && M >= 1024) {
    float* t = gemm_tc_rank_scratch(c, (uint64_t)n * K);
    if (t) {
      gemm_tc_transpose(c, B, t, K, n);
      bnk = t;
      extra = 1;
    } else {
      bnk = nullptr;
    }
  }
  if (bnk && gemm_tc_rank_n(c, A, bnk, out, M, n, K, alpha) == 1) return 1 + extra;
  if (!k::skinny_n_ok(M, n, K)) {               // wider than the CUDA-core rank kernels take: the any-shape GEMM
    k::GemmDesc d = dense_desc(A, B, out, (uint64_t)M, (uint64_t)n, (uint64_t)K);
    d.sAm = K; d.sAk = 1;
    if (b_is_nk) { d.sBk = 1; d.sBn = K; } else { d.sBk = n; d.sBn = 1; }
    d.alpha = alpha;
    return extra + k::gemm_simt(d, c->gemm_ws, c->stream);
  }
  return extra + k::skinny_n(A, B, out, M, n, K, b_is_nk, alpha, c->stream);
}

// Whether the rank-r kernels (tensor-core or CUDA-core) take these shapes; rank 64 only with the
// F16X2 arithmetic, whose fused GEMM carries a 64-wide tail.
bool rank_n_ok(const seeml_b200_ctx* c, uint64_t M, uint64_t n, uint64_t K) {
  if (k::skinny_n_ok((int)M, (int)n, (int)K)) return true;
  return n == 64 && c->gemm_kind == SEEML_B200_GEMM_F16X2 && M >= 1024 && K >= 128 && K % 8 == 0;
}
bool rank_tn_ok(const seeml_b200_ctx* c, uint64_t T, uint64_t big, uint64_t small) {
  if (k::skinny_tn_ok((int)T, (int)big, (int)small)) return true;
  return small == 64 && c->gemm_kind == SEEML_B200_GEMM_F16X2 && gemm_tc_rank_tn_chunk_rows(T, big, small) != 0;
}
// Floats of workspace the tensor-core split-T product writes its chunk partials into (0: not that path).
uint64_t rank_tn_partial_floats(uint64_t T, uint64_t big, uint64_t small) {
  const uint64_t rows = gemm_tc_rank_tn_chunk_rows(T, big, small);
  return rows ? (T / rows) * big * small : 0;
}
int rank_tn(seeml_b200_ctx* c, const float* W, const float* S, float* out, int T, int big, int small,
            int transposed, float alpha) {
  const uint64_t rows = gemm_tc_rank_tn_chunk_rows(T, big, small);
  if (rows && (uint64_t)(T / rows) * big * small <= c->gemm_ws_floats &&
      gemm_tc_rank_tn(c, W, S, c->gemm_ws, T, big, small, rows) == 1)
    return 1 + k::skinny_tn_reduce_bs(c->gemm_ws, out, (int)(T / rows), big, small, transposed, alpha, c->stream);
  if (!k::skinny_tn_ok(T, big, small)) {         // wider than the CUDA-core kernel takes: the any-shape GEMM
    // out = alpha * W^T S as [big, small] (transposed) or alpha * S^T W as [small, big]
    const int Mc = transposed ? big : small, Nc = transposed ? small : big;
    k::GemmDesc d = dense_desc(transposed ? W : S, transposed ? S : W, out, (uint64_t)Mc, (uint64_t)Nc, (uint64_t)T);
    d.sAm = 1; d.sAk = Mc; d.sBk = Nc; d.sBn = 1;
    d.alpha = alpha;
    return k::gemm_simt(d, c->gemm_ws, c->stream);
  }
  return k::skinny_tn(W, S, out, c->gemm_ws, T, big, small, transposed, alpha, c->stream);
}

int try_skinny(const Exec& x, const Instr& ins, bool launch, uint64_t* ws_need) {
  if (ins.opcode != kGemmNN && ins.opcode != kGemmNT && ins.opcode != kGemmTN) return 0;
  if (ins.flags != 0) return 0;
  const uint64_t M64 = ins.out[0], N64 = ins.out[1], K64 = ins.out[2];
  if (M64 > 0x7FFFFFFF || N64 > 0x7FFFFFFF || K64 > 0x7FFFFFFF) return 0;
  if (M64 * N64 > 0x7FFFFFFF) return 0;
  const int M = (int)M64, N = (int)N64, K = (int)K64;
  const float* A = x.R(ins.in[0]);
  const float* B = x.R(ins.in[1]);
  float* C = x.W(ins.in[2]);
  cudaStream_t st = x.c->stream;
  if (ins.opcode == kGemmTN) {
    // C[M,N] = A[K,M]^T B[K,N]; the reduction runs over the K rows
    if (N <= M && k::skinny_tn_ok(K, M, N)) {
      if (ws_need) *ws_need = k::skinny_tn_workspace_floats(K, M, N);
      return launch ? rank_tn(x.c, A, B, C, K, M, N, 1, 1.0f) : 2;
    }
    if (M < N && k::skinny_tn_ok(K, N, M)) {
      if (ws_need) *ws_need = k::skinny_tn_workspace_floats(K, N, M);
      return launch ? rank_tn(x.c, B, A, C, K, N, M, 0, 1.0f) : 2;
    }
    return 0;
  }
  const int b_is_nk = ins.opcode == kGemmNT;
  if (k::skinny_n_ok(M, N, K) && al16(A)) return launch ? rank_n(x.c, A, B, C, M, N, K, b_is_nk, 1.0f) : 1;
  if (k::skinny_k_ok(M, N, K) && al16(C)) return launch ? k::skinny_k(A, B, nullptr, C, M, N, K, b_is_nk, 1.0f, st) : 1;
  return 0;
}

uint64_t scratch_need_loss(const Instr& ins) {
  switch (ins.opcode) {
    case kXentFwd: return k::loss_scratch_doubles(ins.out[0]);
    case kKlFwd: return k::loss_scratch_doubles(hi32(ins.out[1]));
    case kMseFwd: case kClipNorm: return 512;
    default: return 0;
  }
}

// The six per-head products of attention on the tensor cores (0 when the shape is not
// eligible and the CUDA-core descriptors below run instead). which: 0 scores = alpha Q K^T
// (masked), 1 O = P V, 2 dP = dO V^T (masked), 3 dV/dK = alpha X^T Y (X = P or dS), 4 dQ =
// alpha dS K. Q/K/V/O-like operands are [B*S, H*dh]; P-like operands are [B*H*S, S].
static int attn_tc(seeml_b200_ctx* c, int which, const float* A, const float* Bm, float* C, uint64_t B, uint64_t S,
                   uint64_t H, uint64_t dh, float alpha) {
  if (S % 128 != 0 || dh % 64 != 0) return 0;
  const uint64_t T = B * S, D = H * dh;
  TcBatched g{};
  g.A = A; g.B = Bm; g.C = C;
  g.batch = (int)(B * H); g.H = (int)H; g.alpha = alpha;
  auto seq = [&](uint64_t& rows, uint64_t& cols, int* x, int* y) {   // [T, D] operand
    rows = T; cols = D; x[0] = 0; x[1] = (int)dh; y[0] = (int)S; y[1] = 0;
  };
  auto sq = [&](uint64_t& rows, uint64_t& cols, int* x, int* y) {    // [B*H*S, S] operand
    rows = B * H * S; cols = S; x[0] = 0; x[1] = 0; y[0] = (int)(H * S); y[1] = (int)S;
  };
  switch (which) {
    case 0: case 2:
      seq(g.a_rows, g.a_cols, g.ax, g.ay); seq(g.b_rows, g.b_cols, g.bx, g.by); sq(g.c_rows, g.c_cols, g.cx, g.cy);
      g.M = (int)S; g.N = (int)S; g.K = (int)dh; g.causal = 1;
      break;
    case 1: case 4:
      sq(g.a_rows, g.a_cols, g.ax, g.ay); seq(g.b_rows, g.b_cols, g.bx, g.by); seq(g.c_rows, g.c_cols, g.cx, g.cy);
      g.b_t = true; g.M = (int)S; g.N = (int)dh; g.K = (int)S; g.causal = 2;
      break;
    default:
      sq(g.a_rows, g.a_cols, g.ax, g.ay); seq(g.b_rows, g.b_cols, g.bx, g.by); seq(g.c_rows, g.c_cols, g.cx, g.cy);
      g.a_t = true; g.b_t = true; g.M = (int)S; g.N = (int)dh; g.K = (int)S; g.causal = 3;
      break;
  }
  return gemm_tc_batched(c, g);
}

int dispatch(Exec& x, const Instr& ins) {
  seeml_b200_ctx* c = x.c;
  cudaStream_t st = c->stream;
  const uint64_t* in = ins.in;
  const uint64_t* o = ins.out;
  int n = 0;
  switch (ins.opcode) {
    case kNop: break;
    case kGemmNN: case kGemmNT: case kGemmTN: case kGemmAccNN: case kGemmNNQ8: case kGemmNTQ8: {
      if ((n = try_skinny(x, ins, true, nullptr)) != 0) break;
      int tc = gemm_tensor_core(c, ins, &n);
      if (tc < 0) return 1;
      if (tc == 0) {
        k::GemmDesc d = gemm_desc_of(x, ins);
        n = k::gemm_simt(d, c->gemm_ws, st);
      }
      break;
    }
    case kAddEW: n = k::add(x.R(in[0]), x.R(in[1]), x.W(in[2]), o[0], st); break;
    case kMulEW: n = k::mul(x.R(in[0]), x.R(in[1]), x.W(in[2]), o[0], st); break;
    case kAddBias: n = k::add_bias(x.R(in[0]), x.R(in[1]), x.W(in[2]), o[0], o[1], st); break;
    case kReluFwd: n = k::act_fwd(1, x.R(in[0]), x.W(in[1]), o[0], st); break;
    case kGeluFwd: n = k::act_fwd(2, x.R(in[0]), x.W(in[1]), o[0], st); break;
    case kSiluFwd: n = k::act_fwd(3, x.R(in[0]), x.W(in[1]), o[0], st); break;
    case kReluBwd: n = k::act_bwd(1, x.R(in[0]), x.R(in[1]), x.W(in[2]), o[0], st); break;
    case kGeluBwd: n = k::act_bwd(2, x.R(in[0]), x.R(in[1]), x.W(in[2]), o[0], st); break;
    case kSiluBwd: n = k::act_bwd(3, x.R(in[0]), x.R(in[1]), x.W(in[2]), o[0], st); break;
    case kScale: n = k::scale(x.R(in[0]), x.W(in[1]), bits_f32(in[2]), o[0], st); break;
    case kReduceRows: n = k::reduce_rows(x.R(in[0]), x.W(in[1]), o[0], o[1], st); break;
    case kFill: n = k::fill(x.W(in[0]), bits_f32(in[1]), o[0], st); break;
    case kCopy: n = k::copy(x.R(in[0]), x.W(in[1]), o[0], st); break;
    case kEmbedFwd: n = k::embed(x.I(in[0]), x.R(in[1]), x.W(in[2]), o[0], lo32(o[1]), hi32(o[1]), st); break;
    case kLayerNormFwd:
      n = k::layernorm_fwd(x.R(in[0]), x.R(in[1]), x.R(in[2]), x.W(in[3]), x.W(o[1]), x.W(o[2]),
                           hi32(o[0]), lo32(o[0]), st);
      break;
    case kLayerNormBwd:
      n = k::layernorm_bwd(x.R(in[0]), x.R(in[1]), x.R(in[2]), x.R(o[0]), x.R(o[1]), x.W(in[3]),
                           hi32(o[2]), lo32(o[2]), st);
      break;
    case kRmsNormFwd:
      n = k::rmsnorm_fwd(x.R(in[0]), x.R(in[1]), x.W(in[2]), x.W(in[3]), hi32(o[0]), lo32(o[0]), st);
      break;
    case kRmsNormBwd:
      n = k::rmsnorm_bwd(x.R(in[0]), x.R(in[1]), x.R(in[2]), x.R(o[0]), x.W(in[3]), hi32(o[1]),
                         lo32(o[1]), st);
      break;
    case kRopeFwd: case kRopeBwd: {
      const uint64_t S = lo32(o[0]), dh = lo32(o[1]);
      uint32_t bb = (uint32_t)o[2];
      auto it = c->rope.find(std::make_tuple(S, dh, bb));
      if (it == c->rope.end()) return fail("UpdateEngine: RoPE table missing (program not built)");
      n = k::rope(x.R(in[0]), x.W(in[1]), it->second, hi32(o[0]), S, hi32(o[1]), dh,
                  ins.opcode == kRopeBwd, st);
      break;
    }
    case kAttnFwd: {
      const uint64_t B = hi32(o[1]), S = lo32(o[1]), H = hi32(o[2]), dh = lo32(o[2]);
      const long long D = (long long)(H * dh);
      float* P = x.W(o[0]);
      // raw scaled scores into P (rows j<=i), causal row softmax in place, then O = P V
      k::GemmDesc s = attn_desc(B, S, H, dh);
      s.A = x.R(in[0]); s.B = x.R(in[1]); s.C = P;
      s.M = (int)S; s.N = (int)S; s.K = (int)dh;
      s.sAm = D; s.sAk = 1; s.sBk = 1; s.sBn = D; s.sCm = (long long)S;
      s.sAb0 = (long long)S * D; s.sAb1 = (long long)dh; s.sBb0 = s.sAb0; s.sBb1 = s.sAb1;
      s.sCb0 = (long long)(H * S * S); s.sCb1 = (long long)(S * S);
      s.alpha = 1.0f / std::sqrt(static_cast<float>(dh));
      s.causal = 1;
      if (attn_scores_softmax_tc(c, s.A, s.B, P, B, S, H, dh, s.alpha) == 1) {
        n += 1;
      } else {
        if (attn_tc(c, 0, s.A, s.B, P, B, S, H, dh, s.alpha) == 1) n += 1;
        else n += k::gemm_simt(s, nullptr, st);
        n += k::causal_softmax_rows(P, B * H, S, st);
      }
      k::GemmDesc pv = attn_desc(B, S, H, dh);
      pv.A = P; pv.B = x.R(in[2]); pv.C = x.W(in[3]);
      pv.M = (int)S; pv.N = (int)dh; pv.K = (int)S;
      pv.sAm = (long long)S; pv.sAk = 1; pv.sBk = D; pv.sBn = 1; pv.sCm = D;
      pv.sAb0 = s.sCb0; pv.sAb1 = s.sCb1; pv.sBb0 = s.sAb0; pv.sBb1 = s.sAb1;
      pv.sCb0 = s.sAb0; pv.sCb1 = s.sAb1;
      pv.causal = 2;
      if (attn_tc(c, 1, P, pv.B, pv.C, B, S, H, dh, 1.0f) == 1) n += 1;
      else n += k::gemm_simt(pv, nullptr, st);
      break;
    }
    case kAttnDP: {  // dP = dO V^T, masked entries zero
      const uint64_t B = hi32(o[0]), S = lo32(o[0]), H = hi32(o[1]), dh = lo32(o[1]);
      const long long D = (long long)(H * dh);
      k::GemmDesc s = attn_desc(B, S, H, dh);
      s.A = x.R(in[0]); s.B = x.R(in[1]); s.C = x.W(in[2]);
      s.M = (int)S; s.N = (int)S; s.K = (int)dh;
      s.sAm = D; s.sAk = 1; s.sBk = 1; s.sBn = D; s.sCm = (long long)S;
      s.sAb0 = (long long)S * D; s.sAb1 = (long long)dh; s.sBb0 = s.sAb0; s.sBb1 = s.sAb1;
      s.sCb0 = (long long)(H * S * S); s.sCb1 = (long long)(S * S);
      s.causal = 1;
      if (attn_tc(c, 2, s.A, s.B, s.C, B, S, H, dh, 1.0f) == 1) n = 1;
      else n = k::gemm_simt(s, nullptr, st);
      break;
    }
    case kAttnDV: case kAttnDK: {  // dV = P^T dO ; dK = dS^T Q / sqrt(d)
      const uint64_t B = hi32(o[0]), S = lo32(o[0]), H = hi32(o[1]), dh = lo32(o[1]);
      const long long D = (long long)(H * dh);
      k::GemmDesc g = attn_desc(B, S, H, dh);
      g.A = x.R(in[0]); g.B = x.R(in[1]); g.C = x.W(in[2]);
      g.M = (int)S; g.N = (int)dh; g.K = (int)S;
      g.sAm = 1; g.sAk = (long long)S;              // A[m=j,k=i] = P[i,j]
      g.sBk = D; g.sBn = 1; g.sCm = D;
      g.sAb0 = (long long)(H * S * S); g.sAb1 = (long long)(S * S);
      g.sBb0 = (long long)S * D; g.sBb1 = (long long)dh; g.sCb0 = g.sBb0; g.sCb1 = g.sBb1;
      g.causal = 3;
      if (ins.opcode == kAttnDK) g.alpha = 1.0f / std::sqrt(static_cast<float>(dh));
      if (attn_tc(c, 3, g.A, g.B, g.C, B, S, H, dh, g.alpha) == 1) n = 1;
      else n = k::gemm_simt(g, nullptr, st);
      break;
    }
    case kAttnDQ: {  // dQ = dS K / sqrt(d)
      const uint64_t B = hi32(o[0]), S = lo32(o[0]), H = hi32(o[1]), dh = lo32(o[1]);
      const long long D = (long long)(H * dh);
      k::GemmDesc g = attn_desc(B, S, H, dh);
      g.A = x.R(in[0]); g.B = x.R(in[1]); g.C = x.W(in[2]);
      g.M = (int)S; g.N = (int)dh; g.K = (int)S;
      g.sAm = (long long)S; g.sAk = 1; g.sBk = D; g.sBn = 1; g.sCm = D;
      g.sAb0 = (long long)(H * S * S); g.sAb1 = (long long)(S * S);
      g.sBb0 = (long long)S * D; g.sBb1 = (long long)dh; g.sCb0 = g.sBb0; g.sCb1 = g.sBb1;
      g.causal = 2;
      g.alpha = 1.0f / std::sqrt(static_cast<float>(dh));
      if (attn_tc(c, 4, g.A, g.B, g.C, B, S, H, dh, g.alpha) == 1) n = 1;
      else n = k::gemm_simt(g, nullptr, st);
      break;
    }
    case kSoftmaxRowsBwd:
      n = k::softmax_rows_bwd(x.R(in[0]), x.R(in[1]), x.W(in[2]), hi32(o[0]), lo32(o[0]), st);
      break;
    case kXentFwd:
      n = k::xent_fwd(x.R(in[0]), x.I(in[1]), x.W(in[2]), x.W(in[3]), o[0], o[1], c->loss_scratch, st);
      break;
    case kXentBwd:
      n = k::xent_bwd(x.R(in[0]), x.I(in[1]), x.R(in[2]), x.W(in[3]), o[0], o[1], st);
      break;
    case kMseFwd: n = k::mse_fwd(x.R(in[0]), x.R(in[1]), x.W(in[2]), o[0], c->loss_scratch, st); break;
    case kMseBwd: n = k::mse_bwd(x.R(in[0]), x.R(in[1]), x.R(in[2]), x.W(in[3]), o[0], st); break;
    case kKlFwd:
      n = k::kl_fwd(x.R(in[0]), x.R(in[1]), x.W(in[2]), x.W(in[3]), x.W(o[0]), hi32(o[1]), lo32(o[1]),
                    bits_f32(o[2]), c->loss_scratch, st);
      break;
    case kKlBwd:
      n = k::kl_bwd(x.R(in[0]), x.R(in[1]), x.R(in[2]), x.W(in[3]), hi32(o[0]), lo32(o[0]),
                    bits_f32(o[1]), st);
      break;
    case kClipNorm: n = k::clip_norm(x.W(in[0]), o[0], bits_f32(in[1]), c->loss_scratch, st); break;
    case kSgd: n = k::sgd(x.W(in[0]), x.R(in[1]), o[0], c->scalars_dev, st); break;
    case kAdamW:
      n = k::adamw(x.W(in[0]), x.R(in[1]), x.W(in[2]), x.W(in[3]), o[0], c->scalars_dev, st);
      break;
    default:
      return fail("UpdateEngine: unknown opcode " + std::to_string(ins.opcode));
  }
  x.launches += (uint64_t)n;
  return 0;
}

#include "backend_fuse.inc"

__global__ void set_scalars_kernel(DevScalars* dst, DevScalars v) { *dst = v; }

int upload_scalars(seeml_b200_ctx* c, const seeml_b200_scalars* sc) {
  DevScalars d{};
  if (sc) {
    d.lr = sc->lr; d.beta1 = sc->beta1; d.beta2 = sc->beta2; d.eps = sc->eps; d.wd = sc->weight_decay;
    // 1/(1 - pow(beta, (float)step)), evaluated once per call in f32 (optimizer.cc:51-54)
    const float stepf = static_cast<float>(sc->step);
    d.inv_bc1 = 1.0f / (1.0f - std::pow(sc->beta1, stepf));
    d.inv_bc2 = 1.0f / (1.0f - std::pow(sc->beta2, stepf));
    d.om_b1 = 1.0f - sc->beta1;
    d.om_b2 = 1.0f - sc->beta2;
  }
  set_scalars_kernel<<<1, 1, 0, c->stream>>>(c->scalars_dev, d);
  return 0;
}

int prepare_instr(seeml_b200_ctx* c, const Instr& ins, uint64_t* loss_need, uint64_t* ws_need) {
  if (ins.opcode == kRopeFwd || ins.opcode == kRopeBwd) {
    if (int r = ensure_rope(c, lo32(ins.out[0]), lo32(ins.out[1]), bits_f32(ins.out[2]))) return r;
  }
  const uint64_t ln = scratch_need_loss(ins);
  if (ln > *loss_need) *loss_need = ln;
  if (ins.opcode >= kGemmNN && ins.opcode <= kGemmAccNN) {
    Exec x{c};
    const k::GemmDesc d = gemm_desc_of(x, ins);
    uint64_t w = k::gemm_simt_workspace_floats(d);
    uint64_t wsk = 0;
    if (try_skinny(x, ins, false, &wsk) != 0 && wsk > w) w = wsk;
    if (w > *ws_need) *ws_need = w;
    if (int r = gemm_tensor_core_prepare(c, ins)) return r;
  }
  return 0;
}

}  // namespace
}  // namespace seeml_b200

using namespace seeml_b200;

extern "C" {

uint32_t seeml_b200_abi_version(void) { return SEEML_B200_ABI_VERSION; }
const char* seeml_b200_last_error(void) { return g_error.c_str(); }

int seeml_b200_ctx_create(int device, uint64_t arena_bytes, const void* rodata, uint64_t rodata_bytes,
                          const void* persist_init, uint64_t persist_bytes, void* external_arena,
                          seeml_b200_ctx** out) {
  if (!out) return fail("UpdateEngine: null output pointer");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail("UpdateEngine: no CUDA device available — this backend has no CPU fallback");
  if (device < 0 || device >= count) return fail("UpdateEngine: device ordinal out of range");
  if (persist_bytes > arena_bytes) return fail("UpdateEngine: persistent segment exceeds arena");
  CU(cudaSetDevice(device), "cudaSetDevice");
  auto c = std::make_unique<seeml_b200_ctx>();
  c->device = device;
  CU(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking), "stream create");
  CU(cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking), "stream create");
  for (auto& sg : c->stage) {
    CU(cudaEventCreateWithFlags(&sg.h2d_done, cudaEventDisableTiming), "event create");
    CU(cudaEventCreateWithFlags(&sg.consumed, cudaEventDisableTiming), "event create");
  }
  CU(cudaEventCreate(&c->t0), "event create");
  CU(cudaEventCreate(&c->t1), "event create");
  const uint64_t ab = (arena_bytes + 63) & ~uint64_t{63};
  c->arena_bytes = ab;
  if (external_arena) {
    c->arena = static_cast<uint8_t*>(external_arena);
    c->owns_arena = false;
  } else {
    CU(cudaMalloc(&c->arena, ab ? ab : 64), "arena alloc");
  }
  CU(cudaMemsetAsync(c->arena, 0, ab, c->stream), "arena clear");
  if (persist_bytes)
    CU(cudaMemcpyAsync(c->arena, persist_init, persist_bytes, cudaMemcpyHostToDevice, c->stream),
       "persistent image upload");
  c->rodata_bytes = rodata_bytes;
  CU(cudaMalloc(&c->rodata, rodata_bytes ? rodata_bytes : 64), "rodata alloc");
  if (rodata_bytes)
    CU(cudaMemcpyAsync(c->rodata, rodata, rodata_bytes, cudaMemcpyHostToDevice, c->stream),
       "rodata upload");
  CU(cudaMalloc(&c->scalars_dev, sizeof(DevScalars)), "scalars alloc");
  CU(cudaMemsetAsync(c->scalars_dev, 0, sizeof(DevScalars), c->stream), "scalars clear");
  CU(cudaMallocHost(&c->read_slot, 64), "pinned alloc");
  CU(cudaStreamSynchronize(c->stream), "ctx init sync");
  *out = c.release();
  return 0;
}

void seeml_b200_ctx_destroy(seeml_b200_ctx* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  cudaStreamSynchronize(c->copy_stream);
  if (c->unit_times) {
    double tot = 0.0;
    for (const auto& kv : c->unit_acc) tot += kv.second.first;
    std::fprintf(stderr, "seeml_b200 unit times (device ms, all runs of this context; total %.3f):\n", tot);
    for (const auto& kv : c->unit_acc)
      std::fprintf(stderr, "  %-44s n=%8llu  %10.3f ms  %5.1f %%\n", kv.first.c_str(), kv.second.second, kv.second.first,
                   tot > 0 ? 100.0 * kv.second.first / tot : 0.0);
  }
  for (cudaEvent_t ev : c->unit_events) cudaEventDestroy(ev);
  for (auto& p : c->programs)
    if (p) {
      for (auto& g : p->graphs) if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
      for (auto& fs : p->steps) {
        cudaFree(fs.bt);
        cudaFree(fs.descs);
      }
      cudaFree(p->side);
    }
  gemm_tensor_core_release(c);
  for (auto& kv : c->wt) cudaFree(kv.second);
  for (auto& kv : c->rope) cudaFree(kv.second);
  if (c->owns_arena && c->arena) cudaFree(c->arena);
  cudaFree(c->rodata);
  cudaFree(c->scalars_dev);
  cudaFree(c->loss_scratch);
  cudaFree(c->gemm_ws);
  cudaFree(c->spans_dev);
  cudaFreeHost(c->read_slot);
  for (auto& sg : c->stage) {
    cudaFree(sg.dev);
    cudaEventDestroy(sg.h2d_done);
    cudaEventDestroy(sg.consumed);
  }
  cudaEventDestroy(c->t0);
  cudaEventDestroy(c->t1);
  cudaStreamDestroy(c->stream);
  cudaStreamDestroy(c->copy_stream);
  delete c;
}

void* seeml_b200_ctx_arena(seeml_b200_ctx* c) { return c ? c->arena : nullptr; }
uint64_t seeml_b200_ctx_arena_bytes(seeml_b200_ctx* c) { return c ? c->arena_bytes : 0; }
void* seeml_b200_ctx_stream(seeml_b200_ctx* c) { return c ? c->stream : nullptr; }
int seeml_b200_ctx_set_gemm(seeml_b200_ctx* c, uint32_t kind) {
  if (!c) return fail("UpdateEngine: null context");
  if (kind > SEEML_B200_GEMM_TF32) return fail("UpdateEngine: unknown GEMM kind");
  if (c->gemm_kind != kind) drop_graphs(c);     // captured graphs hold the previous kind's kernels
  c->gemm_kind = kind;
  return 0;
}

int seeml_b200_program_build(seeml_b200_ctx* c, const void* instrs, uint64_t count, uint32_t version,
                             uint32_t mode, int* program_id) {
  if (!c || !program_id) return fail("UpdateEngine: null argument");
  if (count && !instrs) return fail("UpdateEngine: null instruction stream");
  CU(cudaSetDevice(c->device), "cudaSetDevice");
  auto p = std::make_unique<Program>();
  p->instrs.resize(count);
  if (count) std::memcpy(p->instrs.data(), instrs, count * sizeof(Instr));
  p->version = version;
  p->mode = mode;
  uint64_t loss_need = 0, ws_need = 0;
  for (uint64_t i = 0; i < count; ++i) {
    const std::string err = validate_instruction(p->instrs[i], c->arena_bytes, c->rodata_bytes, version);
    if (!err.empty()) return fail(err);
    if (int r = prepare_instr(c, p->instrs[i], &loss_need, &ws_need)) return r;
  }
  if (int r = ensure_scratch(c, loss_need, ws_need)) return r;
  if (int r = build_fused_steps(c, *p)) return r;
  c->programs.push_back(std::move(p));
  *program_id = static_cast<int>(c->programs.size()) - 1;
  return 0;
}

uint64_t seeml_b200_program_size(seeml_b200_ctx* c, int id) {
  if (!c || id < 0 || (size_t)id >= c->programs.size()) return 0;
  return c->programs[id]->instrs.size();
}
uint64_t seeml_b200_program_launches(seeml_b200_ctx* c, int id) {
  if (!c || id < 0 || (size_t)id >= c->programs.size()) return 0;
  return c->programs[id]->last_launches;
}

int seeml_b200_program_run(seeml_b200_ctx* c, int id, uint64_t begin, uint64_t end,
                           const seeml_b200_scalars* scalars) {
  if (!c || id < 0 || (size_t)id >= c->programs.size()) return fail("UpdateEngine: bad program id");
  Program& p = *c->programs[id];
  if (begin > end || end > p.instrs.size()) return fail("UpdateEngine: instruction range out of bounds");
  CU(cudaSetDevice(c->device), "cudaSetDevice");
  if (c->timing) CU(cudaEventRecord(c->t0, c->stream), "event record");
  upload_scalars(c, scalars);
  static const bool graphs_off = [] { const char* e = std::getenv("SEEML_B200_GRAPHS"); return e && std::atoi(e) == 0; }();
  static const bool unit_times = [] { const char* e = std::getenv("SEEML_B200_UNIT_TIMES"); return e && std::atoi(e) != 0; }();
  c->unit_times = unit_times;
  Program::RangeGraph* rg = nullptr;
  if (c->use_graphs && !graphs_off && !unit_times && end - begin >= 8) rg = &p.graphs[std::make_pair(begin, end)];
  if (rg && rg->exec) {
    CU(cudaGraphLaunch(rg->exec, c->stream), "graph launch");
    p.last_launches = rg->launches;
    if (c->timing) {
      CU(cudaEventRecord(c->t1, c->stream), "event record");
      c->timed_valid = true;
    }
    return 0;
  }
  const bool capture = rg && !rg->disabled && rg->runs >= 1;
  if (rg) ++rg->runs;
  if (capture && cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    cudaGetLastError();
    rg->disabled = true;
    return seeml_b200_program_run(c, id, begin, end, scalars);
  }
  Exec x{c};
  x.launches = 1;
  int failed = 0;
  c->exec_unit += 2;
  size_t nmark = 0;
  auto mark = [&](const std::string& label) {     // an event ahead of every unit, one behind the last
    if (nmark == c->unit_events.size()) {
      cudaEvent_t ev = nullptr;
      if (cudaEventCreate(&ev) != cudaSuccess) return;
      c->unit_events.push_back(ev);
      c->unit_keys.emplace_back();
    }
    c->unit_keys[nmark] = label;
    cudaEventRecord(c->unit_events[nmark++], c->stream);
  };
  auto unit_label = [&](uint64_t i, int32_t si) {  // opcode or fused-group kind; GEMM-carrying units with their shape
    static const char* const kinds[] = {"", "lora forward group", "lora backward group", "dgrad + add", "attention dS",
                                        "swiglu forward", "swiglu backward", "rmsnorm backward + add", "xent group",
                                        "adamw run"};
    char buf[96];
    const Instr& ins = p.instrs[i];
    if (si >= 0) {
      const int kind = (int)p.steps[si].kind;
      const Instr& g = kind == FusedStep::kLoraBwd ? p.instrs[i + 1] : ins;
      if (kind <= FusedStep::kDgradAdd)
        std::snprintf(buf, sizeof buf, "%s %llux%llux%llu", kinds[kind], (unsigned long long)g.out[0],
                      (unsigned long long)g.out[1], (unsigned long long)g.out[2]);
      else std::snprintf(buf, sizeof buf, "%s", kind < 10 ? kinds[kind] : "fused group");
    } else if (ins.opcode >= kGemmNN && ins.opcode <= kGemmAccNN) {
      std::snprintf(buf, sizeof buf, "opcode %d %llux%llux%llu", (int)ins.opcode, (unsigned long long)ins.out[0],
                    (unsigned long long)ins.out[1], (unsigned long long)ins.out[2]);
    } else {
      std::snprintf(buf, sizeof buf, "opcode %d", (int)ins.opcode);
    }
    return std::string(buf);
  };
  for (uint64_t i = begin; i < end && !failed;) {
    ++c->exec_unit;
    const int32_t si = p.step_at.empty() ? -1 : p.step_at[i];
    if (unit_times) mark(unit_label(i, si >= 0 && i + p.steps[si].count <= end ? si : -1));
    if (si >= 0 && i + p.steps[si].count <= end) {
      const int fr = run_fused(x, p, p.steps[si]);
      if (fr < 0) { failed = 1; break; }
      if (fr == 1) { i += p.steps[si].count; continue; }
      for (uint32_t q = 0; q < p.steps[si].count && !failed; ++q) failed = dispatch(x, p.instrs[i + q]);
      i += p.steps[si].count;
      continue;
    }
    failed = dispatch(x, p.instrs[i]);
    ++i;
  }
  if (capture) {
    cudaGraph_t graph = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(c->stream, &graph);
    if (failed || ce != cudaSuccess || !graph ||
        cudaGraphInstantiate(&rg->exec, graph, 0) != cudaSuccess) {
      // something in this range cannot be captured: run it directly from now on
      cudaGetLastError();
      if (graph) cudaGraphDestroy(graph);
      rg->exec = nullptr;
      rg->disabled = true;
      if (failed) return failed;
      return seeml_b200_program_run(c, id, begin, end, scalars);
    }
    cudaGraphDestroy(graph);
    rg->launches = x.launches;
    CU(cudaGraphLaunch(rg->exec, c->stream), "graph launch");
  } else if (failed) {
    return failed;
  }
  p.last_launches = x.launches;
  if (unit_times && nmark) {
    mark(std::string());
    if (cudaEventSynchronize(c->unit_events[nmark - 1]) == cudaSuccess)
      for (size_t u = 0; u + 1 < nmark; ++u) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, c->unit_events[u], c->unit_events[u + 1]) == cudaSuccess) {
          auto& acc = c->unit_acc[c->unit_keys[u]];
          acc.first += ms;
          ++acc.second;
        }
      }
  }
  if (c->timing) {
    CU(cudaEventRecord(c->t1, c->stream), "event record");
    c->timed_valid = true;
  }
  CU(cudaGetLastError(), "kernel launch");
  return 0;
}

int seeml_b200_exec_one(seeml_b200_ctx* c, const void* instr, uint32_t version,
                        const seeml_b200_scalars* scalars) {
  if (!c || !instr) return fail("UpdateEngine: null argument");
  int id = -1;
  if (int r = seeml_b200_program_build(c, instr, 1, version, SEEML_B200_MODE_CONTRACT, &id)) return r;
  int r = seeml_b200_program_run(c, id, 0, 1, scalars);
  if (!r) r = seeml_b200_sync(c);
  c->programs.pop_back();
  return r;
}

static int range_ok(seeml_b200_ctx* c, uint64_t off, uint64_t bytes);
int seeml_b200_gemm_fused(seeml_b200_ctx* c, const seeml_b200_fused_gemm* f) {
  if (!c || !f) return fail("UpdateEngine: null argument");
  if (f->m == 0 || f->n == 0 || f->k == 0 || f->m > 0x7FFFFFFF || f->n > 0x7FFFFFFF || f->k > 0x7FFFFFFF ||
      f->k2 > 0x7FFFFFFF)
    return fail("UpdateEngine: fused GEMM dimension out of range");
  const bool has_add = f->addend_offset != ~0ull;
  if (range_ok(c, f->a_offset, f->m * f->k * 4) || range_ok(c, f->b_offset, f->n * f->k * 4) ||
      range_ok(c, f->c_offset, f->m * f->n * 4) ||
      (f->k2 && (range_ok(c, f->a2_offset, f->m * f->k2 * 4) || range_ok(c, f->b2_offset, f->n * f->k2 * 4))) ||
      (has_add && range_ok(c, f->addend_offset, f->m * f->n * 4)))
    return 1;
  if ((f->a_offset | f->b_offset | f->c_offset | (f->k2 ? f->a2_offset | f->b2_offset : 0) |
       (has_add ? f->addend_offset : 0)) & 3)
    return fail("UpdateEngine: fused GEMM operand misaligned");
  CU(cudaSetDevice(c->device), "cudaSetDevice");
  auto at = [&](uint64_t off) { return reinterpret_cast<float*>(c->arena + off); };
  uint64_t loss_need = 0, ws_need = 0;
  Instr probe{};
  probe.opcode = kGemmNT;
  if (int r = gemm_tensor_core_prepare(c, probe)) return r;   // makes sure the tensor-core state exists
  (void)loss_need; (void)ws_need;
  TcGemm g{};
  g.A = at(f->a_offset); g.Bt = at(f->b_offset); g.C = at(f->c_offset);
  g.M = f->m; g.N = f->n; g.K = f->k;
  if (f->k2) { g.A2 = at(f->a2_offset); g.B2t = at(f->b2_offset); g.K2 = f->k2; }
  if (has_add) g.addend = at(f->addend_offset);
  const int r = gemm_tc_launch(c, g);
  if (r < 0) return 1;
  if (r == 0) {
    // CUDA-core form: the main product (plus addend), then the low-rank product accumulated on top
    k::GemmDesc d = dense_desc(g.A, g.Bt, g.C, g.M, g.N, g.K);
    d.sAm = (long long)g.K; d.sAk = 1; d.sBk = 1; d.sBn = (long long)g.K;
    if (has_add) {
      if (g.addend != g.C) CU(cudaMemcpyAsync(g.C, g.addend, g.M * g.N * 4, cudaMemcpyDeviceToDevice, c->stream), "addend");
      d.accumulate = 1;
    }
    k::gemm_simt(d, nullptr, c->stream);
    if (g.K2) {
      k::GemmDesc e = dense_desc(g.A2, g.B2t, g.C, g.M, g.N, g.K2);
      e.sAm = (long long)g.K2; e.sAk = 1; e.sBk = 1; e.sBn = (long long)g.K2;
      e.accumulate = 1;
      k::gemm_simt(e, nullptr, c->stream);
    }
  }
  CU(cudaGetLastError(), "fused GEMM launch");
  return 0;
}

static int range_ok(seeml_b200_ctx* c, uint64_t off, uint64_t bytes) {
  if (!c) return fail("UpdateEngine: null context");
  if (off > c->arena_bytes || bytes > c->arena_bytes - off)
    return fail("UpdateEngine: arena range out of bounds");
  return 0;
}
int seeml_b200_h2d(seeml_b200_ctx* c, uint64_t off, const void* src, uint64_t bytes) {
  if (int r = range_ok(c, off, bytes)) return r;
  CU(cudaSetDevice(c->device), "cudaSetDevice");
  CU(cudaMemcpyAsync(c->arena + off, src, bytes, cudaMemcpyHostToDevice, c->stream), "h2d");
  CU(cudaStreamSynchronize(c->stream), "h2d sync");
  return 0;
}
int seeml_b200_d2h(seeml_b200_ctx* c, uint64_t off, void* dst, uint64_t bytes) {
  if (int r = range_ok(c, off, bytes)) return r;
  CU(cudaSetDevice(c->device), "cudaSetDevice");
  CU(cudaMemcpyAsync(dst, c->arena + off, bytes, cudaMemcpyDeviceToHost, c->stream), "d2h");
  CU(cudaStreamSynchronize(c->stream), "d2h sync");
  return 0;
}
int seeml_b200_d2d(seeml_b200_ctx* c, uint64_t off, const void* src, uint64_t bytes) {
  if (int r = range_ok(c, off, bytes)) return r;
  if (!src) return fail("UpdateEngine: null source");
  CU(cudaMemcpyAsync(c->arena + off, src, bytes, cudaMemcpyDeviceToDevice, c->stream), "d2d");
  return 0;
}
int seeml_b200_memset(seeml_b200_ctx* c, uint64_t off, int byte, uint64_t bytes) {
  if (int r = range_ok(c, off, bytes)) return r;
  CU(cudaMemsetAsync(c->arena + off, byte, bytes, c->stream), "memset");
  return 0;
}
int seeml_b200_stage_h2d(seeml_b200_ctx* c, int slot, const void* input, uint64_t in_bytes,
                         const void* label, uint64_t lab_bytes) {
  if (!c || slot < 0 || slot > 1 || !input) return fail("UpdateEngine: bad staging argument");
  CU(cudaSetDevice(c->device), "cudaSetDevice");
  seeml_b200_ctx::Stage& s = c->stage[slot];
  const uint64_t in_al = (in_bytes + 255) & ~uint64_t{255};
  const uint64_t need = in_al + lab_bytes + 256;
  if (need > s.cap) {
    if (s.dev) cudaFree(s.dev);
    s.dev = nullptr;
    CU(cudaMalloc(&s.dev, need), "staging alloc");
    s.cap = need;
  }
  // the slot's previous batch must have been moved into the arena first
  if (s.pending_consume) CU(cudaStreamWaitEvent(c->copy_stream, s.consumed, 0), "stream wait");
  CU(cudaMemcpyAsync(s.dev, input, in_bytes, cudaMemcpyHostToDevice, c->copy_stream), "stage input");
  if (label && lab_bytes)
    CU(cudaMemcpyAsync(s.dev + in_al, label, lab_bytes, cudaMemcpyHostToDevice, c->copy_stream),
       "stage labels");
  s.input_bytes = in_bytes;
  s.label_bytes = label ? lab_bytes : 0;
  CU(cudaEventRecord(s.h2d_done, c->copy_stream), "event record");
  return 0;
}
int seeml_b200_stage_wait(seeml_b200_ctx* c, int slot) {
  if (!c || slot < 0 || slot > 1) return fail("UpdateEngine: bad staging argument");
  CU(cudaEventSynchronize(c->stage[slot].h2d_done), "stage wait");
  return 0;
}
int seeml_b200_stage_commit(seeml_b200_ctx* c, int slot, uint64_t in_off, uint64_t lab_off) {
  if (!c || slot < 0 || slot > 1) return fail("UpdateEngine: bad staging argument");
  seeml_b200_ctx::Stage& s = c->stage[slot];
  if (!s.dev) return fail("UpdateEngine: staging slot is empty");
  if (int r = range_ok(c, in_off, s.input_bytes)) return r;
  if (s.label_bytes) if (int r = range_ok(c, lab_off, s.label_bytes)) return r;
  CU(cudaSetDevice(c->device), "cudaSetDevice");
  const uint64_t in_al = (s.input_bytes + 255) & ~uint64_t{255};
  CU(cudaStreamWaitEvent(c->stream, s.h2d_done, 0), "stream wait");
  CU(cudaMemcpyAsync(c->arena + in_off, s.dev, s.input_bytes, cudaMemcpyDeviceToDevice, c->stream),
     "commit input");
  if (s.label_bytes)
    CU(cudaMemcpyAsync(c->arena + lab_off, s.dev + in_al, s.label_bytes, cudaMemcpyDeviceToDevice,
                       c->stream), "commit labels");
  CU(cudaEventRecord(s.consumed, c->stream), "event record");
  s.pending_consume = true;
  return 0;
}
int seeml_b200_stage_io(seeml_b200_ctx* c, uint64_t in_off, const void* input, uint64_t in_bytes,
                        uint64_t lab_off, const void* label, uint64_t lab_bytes) {
  if (int r = seeml_b200_stage_h2d(c, 0, input, in_bytes, label, lab_bytes)) return r;
  return seeml_b200_stage_commit(c, 0, in_off, lab_off);
}
void* seeml_b200_pinned_alloc(uint64_t bytes) {
  void* p = nullptr;
  if (cudaMallocHost(&p, bytes ? bytes : 64) != cudaSuccess) {
    fail("UpdateEngine: pinned allocation failed");
    return nullptr;
  }
  return p;
}
void seeml_b200_pinned_free(void* p) {
  if (p) cudaFreeHost(p);
}
int seeml_b200_read_f32(seeml_b200_ctx* c, uint64_t off, float* out) {
  if (int r = range_ok(c, off, 4)) return r;
  CU(cudaSetDevice(c->device), "cudaSetDevice");
  CU(cudaMemcpyAsync(c->read_slot, c->arena + off, 4, cudaMemcpyDeviceToHost, c->stream), "loss read");
  CU(cudaStreamSynchronize(c->stream), "loss read sync");
  *out = *c->read_slot;
  return 0;
}
int seeml_b200_sync(seeml_b200_ctx* c) {
  if (!c) return fail("UpdateEngine: null context");
  CU(cudaSetDevice(c->device), "cudaSetDevice");
  CU(cudaStreamSynchronize(c->stream), "stream sync");
  CU(cudaGetLastError(), "kernel execution");
  if (const int code = gemm_tensor_core_error(c))
    return fail("UpdateEngine: tensor-core GEMM gave up on a bounded wait (code " + std::to_string(code) + ")");
  return 0;
}
int seeml_b200_ctx_enable_timing(seeml_b200_ctx* c, int on) {
  if (!c) return fail("UpdateEngine: null context");
  c->timing = on != 0;
  c->timed_valid = false;
  return 0;
}
int seeml_b200_last_run_ms(seeml_b200_ctx* c, float* ms) {
  if (!c || !ms) return fail("UpdateEngine: null argument");
  if (!c->timed_valid) return fail("UpdateEngine: no timed run");
  CU(cudaEventSynchronize(c->t1), "event sync");
  CU(cudaEventElapsedTime(ms, c->t0, c->t1), "event elapsed");
  return 0;
}

static int upload_spans(seeml_b200_ctx* c, const uint64_t* offs, const uint64_t* counts, uint64_t n,
                        uint64_t* total) {
  std::vector<k::Span> spans(n);
  uint64_t at = 0;
  for (uint64_t i = 0; i < n; ++i) {
    if (offs[i] % 4 || offs[i] > c->arena_bytes || counts[i] * 4 > c->arena_bytes - offs[i])
      return fail("UpdateEngine: gradient span out of bounds");
    spans[i] = {offs[i], counts[i], at};
    at += counts[i];
  }
  *total = at;
  if (n > c->spans_cap) {
    cudaFree(c->spans_dev);
    c->spans_dev = nullptr;
    CU(cudaMalloc(&c->spans_dev, n * sizeof(k::Span)), "span table alloc");
    c->spans_cap = n;
  }
  CU(cudaMemcpyAsync(c->spans_dev, spans.data(), n * sizeof(k::Span), cudaMemcpyHostToDevice, c->stream),
     "span table upload");
  CU(cudaStreamSynchronize(c->stream), "span table sync");
  return 0;
}
int seeml_b200_grads_pack(seeml_b200_ctx* c, const uint64_t* offs, const uint64_t* counts, uint64_t n,
                          void* dst) {
  if (!c || !dst) return fail("UpdateEngine: null argument");
  uint64_t total = 0;
  if (int r = upload_spans(c, offs, counts, n, &total)) return r;
  k::pack_spans(c->arena, c->spans_dev, n, static_cast<float*>(dst), 0, total, c->stream);
  CU(cudaGetLastError(), "pack launch");
  return 0;
}
int seeml_b200_grads_unpack(seeml_b200_ctx* c, const uint64_t* offs, const uint64_t* counts, uint64_t n,
                            const void* src) {
  if (!c || !src) return fail("UpdateEngine: null argument");
  uint64_t total = 0;
  if (int r = upload_spans(c, offs, counts, n, &total)) return r;
  k::pack_spans(c->arena, c->spans_dev, n, const_cast<float*>(static_cast<const float*>(src)), 1, total,
                c->stream);
  CU(cudaGetLastError(), "unpack launch");
  return 0;
}
int seeml_b200_tree_sum(seeml_b200_ctx* c, void* sets, uint64_t fps, uint64_t count, float scale) {
  if (!c || !sets) return fail("UpdateEngine: null argument");
  k::tree_sum(static_cast<float*>(sets), fps, count, scale, c->stream);
  CU(cudaGetLastError(), "tree sum launch");
  return 0;
}

}  // extern "C"
