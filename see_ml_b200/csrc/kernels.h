// Host-callable launchers of the sm_100a kernels. All pointers are device
// pointers; every launcher enqueues on `st` and returns without synchronising.
// Each launcher returns the number of kernels it enqueued.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace seeml_b200 {

// Per-step optimiser scalars as the kernels read them (device memory, so that a
// captured graph replays with new values). inv_bc* are computed on the host with
// the reference's expression 1/(1-powf(beta,(float)step)) (optimizer.cc:51-56).
struct DevScalars {
  float lr, beta1, beta2, eps, wd, inv_bc1, inv_bc2, om_b1, om_b2;
  float pad[7];
};

namespace k {

// ---- elementwise / broadcast (elementwise.cc:16-78, activation.cc:22-75) ------
int add(const float* x, const float* y, float* o, size_t n, cudaStream_t st);
int mul(const float* x, const float* y, float* o, size_t n, cudaStream_t st);
int scale(const float* x, float* o, float alpha, size_t n, cudaStream_t st);
int add_bias(const float* x, const float* b, float* o, size_t rows, size_t cols, cudaStream_t st);
int act_fwd(int act, const float* x, float* o, size_t n, cudaStream_t st);   // 1 relu 2 gelu 3 silu
int act_bwd(int act, const float* dy, const float* x, float* dx, size_t n, cudaStream_t st);
int fill(float* d, float v, size_t n, cudaStream_t st);
int copy(const float* s, float* d, size_t n, cudaStream_t st);
int embed(const int32_t* tok, const float* table, float* o, size_t rows, size_t dim, size_t vocab,
          cudaStream_t st);
int reduce_rows(const float* dy, float* db, size_t rows, size_t cols, cudaStream_t st);
// bias + activation over finished GEMM rows (gemm.cc:145-169)
int bias_act(float* c, const float* bias, size_t rows, size_t cols, int act, cudaStream_t st);

// ---- normalisation (normalization.cc:17-113) -------------------------------------
int layernorm_fwd(const float* x, const float* g, const float* b, float* y, float* mean,
                  float* rstd, size_t rows, size_t cols, cudaStream_t st);
int layernorm_bwd(const float* dy, const float* x, const float* g, const float* mean,
                  const float* rstd, float* dx, size_t rows, size_t cols, cudaStream_t st);
int rmsnorm_fwd(const float* x, const float* g, float* y, float* rstd, size_t rows, size_t cols,
                cudaStream_t st);
// addend (nullable): dx = addend + gradient (the residual sum that follows in the stream)
int rmsnorm_bwd(const float* dy, const float* x, const float* g, const float* rstd, float* dx,
                size_t rows, size_t cols, cudaStream_t st, const float* addend = nullptr);

// ---- rotary embedding (attention.cc:39-92). table = [S][d/2] (cos,sin) pairs
// computed on the host with the reference's float recurrence. ----------------------
int rope(const float* x, float* y, const float2* table, size_t B, size_t S, size_t H, size_t d,
         int backward, cudaStream_t st);

// ---- softmax pieces of attention (attention.cc:94-203) ----------------------------
// In place over P[(b,h,i), :]: entries j<=i hold raw scaled scores; writes the
// causal row softmax and exact zeros for j>i.
int causal_softmax_rows(float* P, size_t BH, size_t S, cudaStream_t st);
int softmax_rows_bwd(const float* P, const float* dP, float* dS, size_t rows, size_t cols,
                     cudaStream_t st);

// ---- losses (loss.cc:21-140). scratch: >= N doubles + 256 doubles ------------------
int xent_fwd(const float* logits, const int32_t* labels, float* loss, float* probs, size_t N,
             size_t C, double* scratch, cudaStream_t st);
int xent_bwd(const float* probs, const int32_t* labels, const float* seed, float* dlogits,
             size_t N, size_t C, cudaStream_t st);
int mse_fwd(const float* p, const float* t, float* loss, size_t n, double* scratch, cudaStream_t st);
int mse_bwd(const float* p, const float* t, const float* seed, float* dp, size_t n, cudaStream_t st);
int kl_fwd(const float* s, const float* t, float* loss, float* ps, float* pt, size_t N, size_t C,
           float T, double* scratch, cudaStream_t st);
int kl_bwd(const float* ps, const float* pt, const float* seed, float* d, size_t N, size_t C,
           float T, cudaStream_t st);
size_t loss_scratch_doubles(size_t rows_or_elems);

// ---- optimiser family (optimizer.cc:17-69) -------------------------------------------
int clip_norm(float* g, size_t n, float max_norm, double* scratch, cudaStream_t st);
int sgd(float* p, const float* g, size_t n, const DevScalars* sc, cudaStream_t st);
int adamw(float* p, const float* g, float* m, float* v, size_t n, const DevScalars* sc,
          cudaStream_t st);

// ---- gate metrics (update_engine.cc:612-638, 799-808) -------------------------------------
// counter += number of rows r < real whose first-maximum column equals labels[r].
int count_correct(const float* probs, const int32_t* labels, size_t real, size_t C,
                  unsigned long long* counter, cudaStream_t st);
// counter += number of non-finite floats in x[0..n).
int count_nonfinite(const float* x, size_t n, unsigned long long* counter, cudaStream_t st);

// ---- data-parallel gradient plumbing ---------------------------------------------------
// ---- groups of consecutive instructions run as one kernel (FUSED mode); n % 4 == 0 and
// 16-byte aligned operands are the caller's job ----------------------------------------------
int swiglu_fwd(const float* g, const float* u, float* s, float* m, size_t n, cudaStream_t st);
int swiglu_bwd(const float* dm, const float* u, const float* s, const float* g, float* ds, float* du, float* dg,
               size_t n, cudaStream_t st);
// loss, (probs when not null) and dlogits = (seed / N) (p - onehot) in one pass; scratch as xent_fwd
int xent_fused(const float* logits, const int32_t* labels, float* loss, float* probs, float* dlogits, float seed,
               size_t N, size_t C, double* scratch, cudaStream_t st);
struct AdamwDesc { float* p; const float* g; float* m; float* v; uint64_t n; uint32_t first_block; uint32_t pad; };   // pad: 1 = 128-bit accesses allowed
int adamw_multi(const AdamwDesc* descs_dev, int ndesc, unsigned total_blocks, const DevScalars* sc, cudaStream_t st);

struct Span { uint64_t arena_off; uint64_t count; uint64_t packed_off; };
int pack_spans(const uint8_t* arena, const Span* spans_dev, size_t nspans, float* packed,
               int unpack, size_t total, cudaStream_t st);
int tree_sum(float* sets, size_t floats_per_set, size_t count, float scale, cudaStream_t st);

// ---- GEMM, CUDA-core path: batched, arbitrary strides -------------------------------------
struct GemmDesc {
  const float* A; const float* B; float* C;
  int M, N, K;
  long long sAm, sAk, sBk, sBn, sCm;          // element strides (C columns contiguous)
  int nb_inner;                                // batch z -> (z / nb_inner, z % nb_inner)
  long long sAb0, sAb1, sBb0, sBb1, sCb0, sCb1;
  int batch;
  float alpha;
  int accumulate;    // C += alpha*A@B
  int causal;        // 0 dense | 1 mask n>m to zero | 2 k<=m (lower-tri A) | 3 k>=m (A = lower-tri^T)
  const float* bias; // fused epilogue (kGemmNN flags)
  int act;
  const int8_t* Bq8; // when set, B elements are int8 (alpha carries the dequant scale)
};
// workspace: >= gemm_simt_workspace_floats(desc) floats when it is nonzero.
size_t gemm_simt_workspace_floats(const GemmDesc& d);
int gemm_simt(const GemmDesc& d, float* workspace, cudaStream_t st);

// ---- GEMMs with one tiny dimension (the LoRA factors), kernels_skinny.cu -------------------
bool skinny_n_ok(int M, int n, int K);
bool skinny_k_ok(int M, int N, int k);
bool skinny_tn_ok(int T, int big, int small);
size_t skinny_tn_workspace_floats(int T, int big, int small);
// out[M,n] = alpha * A[M,K] . B, B given [K,n] (b_is_nk = 0) or [n,K] (b_is_nk = 1)
int skinny_n(const float* A, const float* B, float* out, int M, int n, int K, int b_is_nk, float alpha,
             cudaStream_t st);
// out[M,N] = alpha * A[M,k] . B (+ addend[M,N]), B given [k,N] or [N,k]
int skinny_k(const float* A, const float* B, const float* addend, float* out, int M, int N, int k, int b_is_nk,
             float alpha, cudaStream_t st);
// R[s,b] = alpha * sum_t S[t,s] * W[t,b]; stored [small,big], or [big,small] when transposed
int skinny_tn(const float* W, const float* S, float* out, float* workspace, int T, int big, int small,
              int transposed, float alpha, cudaStream_t st);
int skinny_tn_reduce_bs(const float* workspace, float* out, int chunks, int big, int small, int transposed,
                        float alpha, cudaStream_t st);

}  // namespace k
}  // namespace seeml_b200
