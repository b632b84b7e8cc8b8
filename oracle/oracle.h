/* TEST INFRASTRUCTURE — CPU restatement of the SeeML update-runtime kernels.
 *
 * This is the parity checker for the CUDA backend, not part of the product:
 * only tests, the smoke check and the bench's cpu_baseline leg may load it.
 * Every function restates, in plain scalar C, the arithmetic of one kernel of
 * the reference runtime (file:line cited per function, paths relative to the
 * reference checkout) in the same accumulation order, so that on the same
 * inputs it reproduces the reference's results (bit-for-bit where libm agrees;
 * verified against the reference itself by tests/golden/make_golden.py and
 * tests/test_oracle_vs_golden.py — parity is pinned, not assumed).
 */
#ifndef SEEML_ORACLE_H_
#define SEEML_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GEMM family — runtime/executor/gemm.cc:55-228. act: 0 none 1 relu 2 gelu 3 silu */
void orc_gemm_nn(const float* A, const float* B, float* C, size_t M, size_t N,
                 size_t K, const float* bias, int act);
void orc_gemm_nt(const float* A, const float* B, float* C, size_t M, size_t N, size_t K);
void orc_gemm_tn(const float* A, const float* B, float* C, size_t M, size_t N, size_t K);
void orc_gemm_acc_nn(const float* A, const float* B, float* C, size_t M, size_t N,
                     size_t K, float alpha);
void orc_gemm_nn_q8(const float* A, const int8_t* B, float* C, size_t M, size_t N,
                    size_t K, float scale, int act);
void orc_gemm_nt_q8(const float* A, const int8_t* B, float* C, size_t M, size_t N,
                    size_t K, float scale);

/* Elementwise — runtime/executor/elementwise.cc:16-78 */
void orc_add(const float* x, const float* y, float* o, size_t n);
void orc_mul(const float* x, const float* y, float* o, size_t n);
void orc_add_bias(const float* x, const float* b, float* o, size_t rows, size_t cols);
void orc_scale(const float* x, float* o, float alpha, size_t n);
void orc_reduce_rows(const float* dy, float* db, size_t rows, size_t cols);
void orc_fill(float* d, float v, size_t n);
void orc_copy(const float* s, float* d, size_t n);
void orc_embed(const int32_t* tok, const float* table, float* o, size_t rows, size_t dim);

/* Activations — runtime/executor/activation.cc:22-75, kernel_policy.h:53-67 */
void orc_relu_fwd(const float* x, float* o, size_t n);
void orc_relu_bwd(const float* dy, const float* x, float* dx, size_t n);
void orc_gelu_fwd(const float* x, float* o, size_t n);
void orc_gelu_bwd(const float* dy, const float* x, float* dx, size_t n);
void orc_silu_fwd(const float* x, float* o, size_t n);
void orc_silu_bwd(const float* dy, const float* x, float* dx, size_t n);

/* Normalisation — runtime/executor/normalization.cc:17-113 */
void orc_layernorm_fwd(const float* x, const float* g, const float* b, float* y,
                       float* mean, float* rstd, size_t rows, size_t cols);
void orc_layernorm_bwd(const float* dy, const float* x, const float* g,
                       const float* mean, const float* rstd, float* dx,
                       size_t rows, size_t cols);
void orc_rmsnorm_fwd(const float* x, const float* g, float* y, float* rstd,
                     size_t rows, size_t cols);
void orc_rmsnorm_bwd(const float* dy, const float* x, const float* g,
                     const float* rstd, float* dx, size_t rows, size_t cols);

/* Transformer family — runtime/executor/attention.cc:39-242 */
void orc_rope(const float* x, float* y, size_t B, size_t S, size_t H, size_t d,
              float base, int backward);
void orc_attn_fwd(const float* q, const float* k, const float* v, float* o,
                  float* P, size_t B, size_t S, size_t H, size_t d);
void orc_attn_dp(const float* dO, const float* v, float* dP, size_t B, size_t S,
                 size_t H, size_t d);
void orc_attn_dv(const float* P, const float* dO, float* dV, size_t B, size_t S,
                 size_t H, size_t d);
void orc_softmax_rows_bwd(const float* P, const float* dP, float* dS, size_t rows,
                          size_t cols);
void orc_attn_dq(const float* dS, const float* k, float* dQ, size_t B, size_t S,
                 size_t H, size_t d);
void orc_attn_dk(const float* dS, const float* q, float* dK, size_t B, size_t S,
                 size_t H, size_t d);

/* Losses — runtime/executor/loss.cc:21-140 */
void orc_xent_fwd(const float* logits, const int32_t* labels, float* loss,
                  float* probs, size_t N, size_t C);
void orc_xent_bwd(const float* probs, const int32_t* labels, const float* seed,
                  float* dlogits, size_t N, size_t C);
void orc_mse_fwd(const float* p, const float* t, float* loss, size_t n);
void orc_mse_bwd(const float* p, const float* t, const float* seed, float* dp, size_t n);
void orc_kl_fwd(const float* s, const float* t, float* loss, float* ps, float* pt,
                size_t N, size_t C, float T);
void orc_kl_bwd(const float* ps, const float* pt, const float* seed, float* d,
                size_t N, size_t C, float T);

/* Optimiser family — runtime/executor/optimizer.cc:17-69 */
void orc_clip_norm(float* g, size_t n, float max_norm);
void orc_sgd(float* p, const float* g, size_t n, float lr, float wd);
void orc_adamw(float* p, const float* g, float* m, float* v, size_t n, float lr,
               float b1, float b2, float eps, float wd, uint64_t step);

/* Learning-rate schedule — runtime/engine/update_engine.cc:515-534 */
float orc_effective_lr(float lr, uint32_t schedule, uint64_t warmup,
                       uint64_t default_steps, float min_lr_factor, uint64_t step);

/* Integrity hashes — source/identity/hash.h:36-161 */
uint64_t orc_content_hash64(const uint8_t* p, size_t n);
uint64_t orc_plan_self_hash(const uint8_t* p, size_t n, size_t hash_off);

/* Instruction interpreter over 64-byte UpdateInstruction words, same operand
 * conventions as runtime/engine/update_engine.cc:306-509. Returns 0, or the
 * 1-based index of the first instruction with an unknown opcode. */
int orc_execute(const uint8_t* program, size_t count, uint8_t* arena,
                const uint8_t* rodata, float lr, float b1, float b2, float eps,
                float wd, uint64_t step);

#ifdef __cplusplus
}
#endif
#endif
