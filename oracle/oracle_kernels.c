/* TEST INFRASTRUCTURE — see oracle.h. Scalar C restatement of the reference
 * kernels. Build with -ffp-contract=off -fno-fast-math: the reference's
 * arithmetic has no fused multiply-adds and no reassociation, and the
 * accumulation orders below are the reference's. */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* --- the determinism rule: chunk geometry is a function of the shape only ---
 * source/parallel/parallel_for.h:50-67 (ceiling of 256 chunks),
 * runtime/executor/kernel_policy.h:37-47 (grains). Reductions that the
 * reference combines "one partial per chunk, in chunk order" are restated with
 * the same chunk boundaries so the double-precision sums round identically. */
enum { kMaxChunks = 256, kGrainCheap = 32768, kGrainMath = 4096 };

static size_t chunk_grain(size_t n, size_t grain) {
  if (grain == 0) grain = 1;
  size_t cap = (n + kMaxChunks - 1) / kMaxChunks;
  return grain < cap ? cap : grain;
}
static size_t row_grain(size_t per_row, size_t budget) {
  if (per_row == 0) return budget;
  return budget / per_row > 0 ? budget / per_row : 1;
}

/* --- activation expressions: runtime/executor/kernel_policy.h:53-67 -------- */
static const float kGeluC = 0.7978845608028654f;
static const float kGeluA = 0.044715f;
static float sigmoid_e(float x) { return 1.0f / (1.0f + expf(-x)); }
static float relu_e(float x) { return x > 0.0f ? x : 0.0f; }
static float gelu_e(float x) {
  float t = tanhf(kGeluC * (x + kGeluA * x * x * x));
  return 0.5f * x * (1.0f + t);
}
static float silu_e(float x) { return x * sigmoid_e(x); }
static float act_e(float v, int act) {
  switch (act) {
    case 1: return relu_e(v);
    case 2: return gelu_e(v);
    case 3: return silu_e(v);
    default: return v;
  }
}

/* --- GEMM ------------------------------------------------------------------
 * runtime/executor/gemm.cc:55-93: C row accumulates k in groups of four,
 * c += a0*b0 + a1*b1 + a2*b2 + a3*b3 (left-to-right), tail one k at a time,
 * alpha folded into a. The K tile (64) is a multiple of four and the N tile
 * only changes traversal order, so an untiled loop yields the same bits. */
#define BLOCKED_NN(BT)                                                         \
  for (size_t m = 0; m < M; ++m) {                                             \
    float* c = C + m * N;                                                      \
    size_t k = 0;                                                              \
    for (; k + 4 <= K; k += 4) {                                               \
      const float a0 = alpha * (at ? A[(k + 0) * as + m] : A[m * as + k + 0]); \
      const float a1 = alpha * (at ? A[(k + 1) * as + m] : A[m * as + k + 1]); \
      const float a2 = alpha * (at ? A[(k + 2) * as + m] : A[m * as + k + 2]); \
      const float a3 = alpha * (at ? A[(k + 3) * as + m] : A[m * as + k + 3]); \
      const BT* b0 = B + (k + 0) * N;                                          \
      const BT* b1 = B + (k + 1) * N;                                          \
      const BT* b2 = B + (k + 2) * N;                                          \
      const BT* b3 = B + (k + 3) * N;                                          \
      for (size_t n = 0; n < N; ++n)                                           \
        c[n] += a0 * (float)b0[n] + a1 * (float)b1[n] + a2 * (float)b2[n] +    \
                a3 * (float)b3[n];                                             \
    }                                                                          \
    for (; k < K; ++k) {                                                       \
      const float a = alpha * (at ? A[k * as + m] : A[m * as + k]);            \
      const BT* b = B + k * N;                                                 \
      for (size_t n = 0; n < N; ++n) c[n] += a * (float)b[n];                  \
    }                                                                          \
  }

/* The tile over K restarts the 4-group at every multiple of 64, which matters
 * only when K is not a multiple of 4 inside a tile — it never is (64 % 4 == 0),
 * except for the final partial tile, whose tail is the global tail. */
static void nn_f32(const float* A, const float* B, float* C, size_t M, size_t N,
                   size_t K, float alpha, size_t as, int at) {
  BLOCKED_NN(float)
}
static void nn_q8(const float* A, const int8_t* B, float* C, size_t M, size_t N,
                  size_t K, float alpha, size_t as, int at) {
  BLOCKED_NN(int8_t)
}

/* runtime/executor/gemm.cc:145-169 */
static void epilogue(float* C, const float* bias, size_t M, size_t N, int act) {
  if (!bias && act == 0) return;
  for (size_t m = 0; m < M; ++m)
    for (size_t n = 0; n < N; ++n) {
      float v = bias ? C[m * N + n] + bias[n] : C[m * N + n];
      C[m * N + n] = act_e(v, act);
    }
}

void orc_gemm_nn(const float* A, const float* B, float* C, size_t M, size_t N,
                 size_t K, const float* bias, int act) { /* gemm.cc:173-182 */
  memset(C, 0, M * N * sizeof(float));
  nn_f32(A, B, C, M, N, K, 1.0f, K, 0);
  epilogue(C, bias, M, N, act);
}
void orc_gemm_tn(const float* A, const float* B, float* C, size_t M, size_t N,
                 size_t K) { /* gemm.cc:192-200 — A is [K,M] */
  memset(C, 0, M * N * sizeof(float));
  nn_f32(A, B, C, M, N, K, 1.0f, M, 1);
}
void orc_gemm_acc_nn(const float* A, const float* B, float* C, size_t M, size_t N,
                     size_t K, float alpha) { /* gemm.cc:202-209 */
  nn_f32(A, B, C, M, N, K, alpha, K, 0);
}
void orc_gemm_nn_q8(const float* A, const int8_t* B, float* C, size_t M, size_t N,
                    size_t K, float scale, int act) { /* gemm.cc:211-220 */
  memset(C, 0, M * N * sizeof(float));
  nn_q8(A, B, C, M, N, K, scale, K, 0);
  epilogue(C, NULL, M, N, act);
}

/* runtime/executor/gemm.cc:99-136: one f32 accumulator per output, k ascending,
 * alpha applied to the finished dot product. */
#define BLOCKED_NT(BT)                                   \
  for (size_t m = 0; m < M; ++m)                         \
    for (size_t n = 0; n < N; ++n) {                     \
      const float* a = A + m * K;                        \
      const BT* b = B + n * K;                           \
      float acc = 0.0f;                                  \
      for (size_t k = 0; k < K; ++k) acc += a[k] * (float)b[k]; \
      C[m * N + n] = alpha * acc;                        \
    }
void orc_gemm_nt(const float* A, const float* B, float* C, size_t M, size_t N,
                 size_t K) { /* gemm.cc:184-190 */
  const float alpha = 1.0f;
  BLOCKED_NT(float)
}
void orc_gemm_nt_q8(const float* A, const int8_t* B, float* C, size_t M, size_t N,
                    size_t K, float scale) { /* gemm.cc:222-228 */
  const float alpha = scale;
  BLOCKED_NT(int8_t)
}

/* --- elementwise: runtime/executor/elementwise.cc -------------------------- */
void orc_add(const float* x, const float* y, float* o, size_t n) { /* :16-20 */
  for (size_t i = 0; i < n; ++i) o[i] = x[i] + y[i];
}
void orc_mul(const float* x, const float* y, float* o, size_t n) { /* :22-26 */
  for (size_t i = 0; i < n; ++i) o[i] = x[i] * y[i];
}
void orc_add_bias(const float* x, const float* b, float* o, size_t rows,
                  size_t cols) { /* :28-36 */
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) o[r * cols + c] = x[r * cols + c] + b[c];
}
void orc_scale(const float* x, float* o, float alpha, size_t n) { /* :38-42 */
  for (size_t i = 0; i < n; ++i) o[i] = alpha * x[i];
}
void orc_embed(const int32_t* tok, const float* table, float* o, size_t rows,
               size_t dim) { /* :44-53 */
  for (size_t r = 0; r < rows; ++r)
    memcpy(o + r * dim, table + (size_t)tok[r] * dim, dim * sizeof(float));
}
void orc_reduce_rows(const float* dy, float* db, size_t rows, size_t cols) { /* :55-67 */
  for (size_t c = 0; c < cols; ++c) db[c] = 0.0f;
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) db[c] += dy[r * cols + c];
}
void orc_fill(float* d, float v, size_t n) { /* :72-74 */
  for (size_t i = 0; i < n; ++i) d[i] = v;
}
void orc_copy(const float* s, float* d, size_t n) { /* :76-78 */
  memcpy(d, s, n * sizeof(float));
}

/* --- activations: runtime/executor/activation.cc --------------------------- */
void orc_relu_fwd(const float* x, float* o, size_t n) { /* :22-26 */
  for (size_t i = 0; i < n; ++i) o[i] = relu_e(x[i]);
}
void orc_relu_bwd(const float* dy, const float* x, float* dx, size_t n) { /* :28-32 */
  for (size_t i = 0; i < n; ++i) dx[i] = x[i] > 0.0f ? dy[i] : 0.0f;
}
void orc_gelu_fwd(const float* x, float* o, size_t n) { /* :34-38 */
  for (size_t i = 0; i < n; ++i) o[i] = gelu_e(x[i]);
}
void orc_gelu_bwd(const float* dy, const float* x, float* dx, size_t n) { /* :40-60 */
  for (size_t i = 0; i < n; ++i) {
    const float v = x[i];
    const float u = kGeluC * (v + kGeluA * v * v * v);
    const float t = tanhf(u);
    const float sech2 = 1.0f - t * t;
    /* saturated tail: a true zero times a possibly infinite u' is dropped */
    const float tail = sech2 == 0.0f
                           ? 0.0f
                           : 0.5f * v * sech2 * (kGeluC * (1.0f + 3.0f * kGeluA * v * v));
    dx[i] = dy[i] * (0.5f * (1.0f + t) + tail);
  }
}
void orc_silu_fwd(const float* x, float* o, size_t n) { /* :62-66 */
  for (size_t i = 0; i < n; ++i) o[i] = silu_e(x[i]);
}
void orc_silu_bwd(const float* dy, const float* x, float* dx, size_t n) { /* :68-75 */
  for (size_t i = 0; i < n; ++i) {
    const float s = sigmoid_e(x[i]);
    dx[i] = dy[i] * (s * (1.0f + x[i] * (1.0f - s)));
  }
}

/* --- normalisation: runtime/executor/normalization.cc ---------------------- */
void orc_layernorm_fwd(const float* x, const float* g, const float* b, float* y,
                       float* mean, float* rstd, size_t rows, size_t cols) { /* :17-45 */
  const float eps = 1e-5f;
  for (size_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    double sum = 0.0;
    for (size_t c = 0; c < cols; ++c) sum += xr[c];
    const float mu = (float)(sum / (double)cols);
    double var = 0.0;
    for (size_t c = 0; c < cols; ++c) {
      const double d = (double)xr[c] - mu;
      var += d * d;
    }
    const float rs = 1.0f / sqrtf((float)(var / (double)cols) + eps);
    mean[r] = mu;
    rstd[r] = rs;
    for (size_t c = 0; c < cols; ++c) y[r * cols + c] = (xr[c] - mu) * rs * g[c] + b[c];
  }
}
void orc_layernorm_bwd(const float* dy, const float* x, const float* g,
                       const float* mean, const float* rstd, float* dx,
                       size_t rows, size_t cols) { /* :47-73 */
  const float inv_d = 1.0f / (float)cols;
  for (size_t r = 0; r < rows; ++r) {
    const float* dyr = dy + r * cols;
    const float* xr = x + r * cols;
    const float mu = mean[r], rs = rstd[r];
    double sg = 0.0, sgx = 0.0;
    for (size_t c = 0; c < cols; ++c) {
      const float xh = (xr[c] - mu) * rs;
      const float gg = dyr[c] * g[c];
      sg += gg;
      sgx += (double)gg * xh;
    }
    const float mg = (float)sg * inv_d;
    const float mgx = (float)sgx * inv_d;
    for (size_t c = 0; c < cols; ++c) {
      const float xh = (xr[c] - mu) * rs;
      const float gg = dyr[c] * g[c];
      dx[r * cols + c] = rs * (gg - mg - xh * mgx);
    }
  }
}
void orc_rmsnorm_fwd(const float* x, const float* g, float* y, float* rstd,
                     size_t rows, size_t cols) { /* :75-92 */
  const float eps = 1e-5f;
  for (size_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    double ss = 0.0;
    for (size_t c = 0; c < cols; ++c) ss += (double)xr[c] * xr[c];
    const float rs = 1.0f / sqrtf((float)(ss / (double)cols) + eps);
    rstd[r] = rs;
    for (size_t c = 0; c < cols; ++c) y[r * cols + c] = xr[c] * rs * g[c];
  }
}
void orc_rmsnorm_bwd(const float* dy, const float* x, const float* g,
                     const float* rstd, float* dx, size_t rows, size_t cols) { /* :94-113 */
  const float inv_d = 1.0f / (float)cols;
  for (size_t r = 0; r < rows; ++r) {
    const float* dyr = dy + r * cols;
    const float* xr = x + r * cols;
    const float rs = rstd[r];
    double sgx = 0.0;
    for (size_t c = 0; c < cols; ++c) sgx += (double)(dyr[c] * g[c]) * xr[c];
    const float mgx = (float)sgx * inv_d;
    for (size_t c = 0; c < cols; ++c)
      dx[r * cols + c] = rs * (dyr[c] * g[c] - xr[c] * rs * rs * mgx);
  }
}

/* --- transformer family: runtime/executor/attention.cc --------------------- */
void orc_rope(const float* x, float* y, size_t B, size_t S, size_t H, size_t d,
              float base, int backward) { /* :39-92 */
  const size_t D = H * d;
  const float step = powf(base, -2.0f / (float)d);
  for (size_t row = 0; row < B * S; ++row) {
    const size_t s = row % S;
    for (size_t h = 0; h < H; ++h) {
      const float* xr = x + row * D + h * d;
      float* yr = y + row * D + h * d;
      float freq = 1.0f; /* float recurrence: freq *= step per pair */
      for (size_t c = 0; c + 1 < d; c += 2) {
        const float th = (float)s * freq;
        const float cs = cosf(th), sn = sinf(th);
        const float a = xr[c], b = xr[c + 1];
        if (!backward) {
          yr[c] = a * cs - b * sn;
          yr[c + 1] = a * sn + b * cs;
        } else {
          yr[c] = a * cs + b * sn;
          yr[c + 1] = -a * sn + b * cs;
        }
        freq *= step;
      }
    }
  }
}

void orc_attn_fwd(const float* q, const float* k, const float* v, float* o,
                  float* P, size_t B, size_t S, size_t H, size_t d) { /* :94-136 */
  const size_t D = H * d;
  const float isd = 1.0f / sqrtf((float)d);
  for (size_t b = 0; b < B; ++b)
    for (size_t h = 0; h < H; ++h)
      for (size_t i = 0; i < S; ++i) {
        const float* qi = q + (b * S + i) * D + h * d;
        float* pr = P + ((b * H + h) * S + i) * S;
        float mx = -INFINITY;
        for (size_t j = 0; j <= i; ++j) {
          const float* kj = k + (b * S + j) * D + h * d;
          double dot = 0.0;
          for (size_t c = 0; c < d; ++c) dot += (double)qi[c] * kj[c];
          const float sc = (float)dot * isd;
          pr[j] = sc;
          if (sc > mx) mx = sc;
        }
        double den = 0.0;
        for (size_t j = 0; j <= i; ++j) {
          const float e = expf(pr[j] - mx);
          pr[j] = e;
          den += e;
        }
        const float inv = 1.0f / (float)den;
        for (size_t j = 0; j <= i; ++j) pr[j] *= inv;
        for (size_t j = i + 1; j < S; ++j) pr[j] = 0.0f;
        float* oi = o + (b * S + i) * D + h * d;
        for (size_t c = 0; c < d; ++c) oi[c] = 0.0f;
        for (size_t j = 0; j <= i; ++j) {
          const float p = pr[j];
          const float* vj = v + (b * S + j) * D + h * d;
          for (size_t c = 0; c < d; ++c) oi[c] += p * vj[c];
        }
      }
}
void orc_attn_dp(const float* dO, const float* v, float* dP, size_t B, size_t S,
                 size_t H, size_t d) { /* :138-164 */
  const size_t D = H * d;
  for (size_t b = 0; b < B; ++b)
    for (size_t h = 0; h < H; ++h)
      for (size_t i = 0; i < S; ++i) {
        const float* doi = dO + (b * S + i) * D + h * d;
        float* row = dP + ((b * H + h) * S + i) * S;
        for (size_t j = 0; j <= i; ++j) {
          const float* vj = v + (b * S + j) * D + h * d;
          double dot = 0.0;
          for (size_t c = 0; c < d; ++c) dot += (double)doi[c] * vj[c];
          row[j] = (float)dot;
        }
        for (size_t j = i + 1; j < S; ++j) row[j] = 0.0f;
      }
}
void orc_attn_dv(const float* P, const float* dO, float* dV, size_t B, size_t S,
                 size_t H, size_t d) { /* :166-184 */
  const size_t D = H * d;
  for (size_t b = 0; b < B; ++b)
    for (size_t h = 0; h < H; ++h)
      for (size_t j = 0; j < S; ++j) {
        float* dvj = dV + (b * S + j) * D + h * d;
        for (size_t c = 0; c < d; ++c) dvj[c] = 0.0f;
        for (size_t i = j; i < S; ++i) {
          const float p = P[((b * H + h) * S + i) * S + j];
          const float* doi = dO + (b * S + i) * D + h * d;
          for (size_t c = 0; c < d; ++c) dvj[c] += p * doi[c];
        }
      }
}
void orc_softmax_rows_bwd(const float* P, const float* dP, float* dS, size_t rows,
                          size_t cols) { /* :186-203 */
  for (size_t r = 0; r < rows; ++r) {
    const float* p = P + r * cols;
    const float* g = dP + r * cols;
    double dot = 0.0;
    for (size_t c = 0; c < cols; ++c) dot += (double)g[c] * p[c];
    const float sum = (float)dot;
    for (size_t c = 0; c < cols; ++c) dS[r * cols + c] = p[c] * (g[c] - sum);
  }
}
void orc_attn_dq(const float* dS, const float* k, float* dQ, size_t B, size_t S,
                 size_t H, size_t d) { /* :205-223 */
  const size_t D = H * d;
  const float isd = 1.0f / sqrtf((float)d);
  for (size_t b = 0; b < B; ++b)
    for (size_t h = 0; h < H; ++h)
      for (size_t i = 0; i < S; ++i) {
        const float* row = dS + ((b * H + h) * S + i) * S;
        float* dqi = dQ + (b * S + i) * D + h * d;
        for (size_t c = 0; c < d; ++c) dqi[c] = 0.0f;
        for (size_t j = 0; j <= i; ++j) {
          const float gsc = row[j] * isd;
          const float* kj = k + (b * S + j) * D + h * d;
          for (size_t c = 0; c < d; ++c) dqi[c] += gsc * kj[c];
        }
      }
}
void orc_attn_dk(const float* dS, const float* q, float* dK, size_t B, size_t S,
                 size_t H, size_t d) { /* :225-242 */
  const size_t D = H * d;
  const float isd = 1.0f / sqrtf((float)d);
  for (size_t b = 0; b < B; ++b)
    for (size_t h = 0; h < H; ++h)
      for (size_t j = 0; j < S; ++j) {
        float* dkj = dK + (b * S + j) * D + h * d;
        for (size_t c = 0; c < d; ++c) dkj[c] = 0.0f;
        for (size_t i = j; i < S; ++i) {
          const float gsc = dS[((b * H + h) * S + i) * S + j] * isd;
          const float* qi = q + (b * S + i) * D + h * d;
          for (size_t c = 0; c < d; ++c) dkj[c] += gsc * qi[c];
        }
      }
}

/* --- losses: runtime/executor/loss.cc -------------------------------------- */
static void row_softmax(const float* z, float* p, size_t C, float inv_T) { /* :21-31 */
  float mx = z[0] * inv_T;
  for (size_t c = 1; c < C; ++c) mx = fmaxf(mx, z[c] * inv_T);
  float sum = 0.0f;
  for (size_t c = 0; c < C; ++c) {
    p[c] = expf(z[c] * inv_T - mx);
    sum += p[c];
  }
  const float inv = 1.0f / sum;
  for (size_t c = 0; c < C; ++c) p[c] *= inv;
}
void orc_xent_fwd(const float* logits, const int32_t* labels, float* loss,
                  float* probs, size_t N, size_t C) { /* :35-58 */
  const size_t g = chunk_grain(N, row_grain(C, kGrainMath));
  double total = 0.0;
  for (size_t r0 = 0; r0 < N; r0 += g) { /* one partial per chunk, in order */
    const size_t r1 = r0 + g < N ? r0 + g : N;
    double part = 0.0;
    for (size_t n = r0; n < r1; ++n) {
      row_softmax(logits + n * C, probs + n * C, C, 1.0f);
      const float p = probs[n * C + (size_t)labels[n]];
      const double safe = isnan(p) ? (double)p : (double)fmaxf(p, 1e-12f);
      part -= log(safe);
    }
    total += part;
  }
  *loss = (float)(total / (double)N);
}
void orc_xent_bwd(const float* probs, const int32_t* labels, const float* seed,
                  float* dlogits, size_t N, size_t C) { /* :61-72 */
  const float scale = *seed / (float)N;
  for (size_t n = 0; n < N; ++n) {
    for (size_t c = 0; c < C; ++c) dlogits[n * C + c] = scale * probs[n * C + c];
    dlogits[n * C + (size_t)labels[n]] -= scale;
  }
}
void orc_mse_fwd(const float* p, const float* t, float* loss, size_t n) { /* :74-89 */
  const size_t g = chunk_grain(n, kGrainCheap);
  double total = 0.0;
  for (size_t b = 0; b < n; b += g) {
    const size_t e = b + g < n ? b + g : n;
    double part = 0.0;
    for (size_t i = b; i < e; ++i) {
      const double dd = (double)p[i] - t[i];
      part += dd * dd;
    }
    total += part;
  }
  *loss = (float)(total / (double)n);
}
void orc_mse_bwd(const float* p, const float* t, const float* seed, float* dp,
                 size_t n) { /* :91-97 */
  const float scale = 2.0f * *seed / (float)n;
  for (size_t i = 0; i < n; ++i) dp[i] = scale * (p[i] - t[i]);
}
void orc_kl_fwd(const float* s, const float* t, float* loss, float* ps, float* pt,
                size_t N, size_t C, float T) { /* :99-132 */
  const float inv_T = 1.0f / T;
  const size_t g = chunk_grain(N, row_grain(C, kGrainMath));
  double total = 0.0;
  for (size_t r0 = 0; r0 < N; r0 += g) {
    const size_t r1 = r0 + g < N ? r0 + g : N;
    double part = 0.0;
    for (size_t n = r0; n < r1; ++n) {
      row_softmax(s + n * C, ps + n * C, C, inv_T);
      row_softmax(t + n * C, pt + n * C, C, inv_T);
      for (size_t c = 0; c < C; ++c) {
        const float ptv = pt[n * C + c];
        if (ptv <= 0.0f) continue;
        const float raw = ps[n * C + c];
        const double psv = isnan(raw) ? (double)raw : (double)fmaxf(raw, 1e-12f);
        part += (double)ptv * (log((double)ptv) - log(psv));
      }
    }
    total += part;
  }
  *loss = (float)(total / (double)N);
}
void orc_kl_bwd(const float* ps, const float* pt, const float* seed, float* d,
                size_t N, size_t C, float T) { /* :134-140 */
  const float scale = *seed / ((float)N * T);
  for (size_t i = 0; i < N * C; ++i) d[i] = scale * (ps[i] - pt[i]);
}

/* --- optimiser family: runtime/executor/optimizer.cc ----------------------- */
void orc_clip_norm(float* g, size_t n, float max_norm) { /* :17-35 */
  const size_t gr = chunk_grain(n, kGrainCheap);
  double sq = 0.0;
  for (size_t b = 0; b < n; b += gr) {
    const size_t e = b + gr < n ? b + gr : n;
    double part = 0.0;
    for (size_t i = b; i < e; ++i) part += (double)g[i] * (double)g[i];
    sq += part;
  }
  const double norm = sqrt(sq);
  if (norm <= (double)max_norm || norm == 0.0) return;
  const float s = (float)((double)max_norm / norm);
  for (size_t i = 0; i < n; ++i) g[i] *= s;
}
void orc_sgd(float* p, const float* g, size_t n, float lr, float wd) { /* :37-42 */
  for (size_t i = 0; i < n; ++i) p[i] -= lr * (g[i] + wd * p[i]);
}
void orc_adamw(float* p, const float* g, float* m, float* v, size_t n, float lr,
               float b1, float b2, float eps, float wd, uint64_t step) { /* :44-69 */
  const float ibc1 = 1.0f / (1.0f - powf(b1, (float)step));
  const float ibc2 = 1.0f / (1.0f - powf(b2, (float)step));
  const float o1 = 1.0f - b1, o2 = 1.0f - b2;
  for (size_t i = 0; i < n; ++i) {
    const float gi = g[i];
    const float mi = b1 * m[i] + o1 * gi;
    const float vi = b2 * v[i] + o2 * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float mh = mi * ibc1, vh = vi * ibc2;
    p[i] -= lr * (mh / (sqrtf(vh) + eps) + wd * p[i]);
  }
}

/* --- LR schedule: runtime/engine/update_engine.cc:515-534 ------------------ */
float orc_effective_lr(float lr, uint32_t schedule, uint64_t warmup,
                       uint64_t default_steps, float min_lr_factor, uint64_t step) {
  if (schedule != 1) return lr;
  if (warmup > 0 && step <= warmup) return lr * (float)step / (float)warmup;
  const uint64_t horizon = default_steps > warmup ? default_steps - warmup : 0;
  const float floor_lr = lr * min_lr_factor;
  if (horizon == 0 || step - warmup >= horizon) return floor_lr;
  const float t = (float)(step - warmup) / (float)horizon;
  const float pi = 3.14159265358979323846f;
  return floor_lr + (lr - floor_lr) * 0.5f * (1.0f + cosf(pi * t));
}

/* --- hashes: source/identity/hash.h ---------------------------------------- */
static const uint64_t kBasis = 0xcbf29ce484222325ULL, kPrime = 0x100000001b3ULL;
static uint64_t mix_word(uint64_t st, uint64_t w) { /* :80-86 */
  for (int b = 0; b < 8; ++b) {
    st ^= (w >> (8 * b)) & 0xff;
    st *= kPrime;
  }
  return st;
}
/* :89-109 — 8 interleaved lanes; zero_at/zero_n blank the sealed hash field */
static uint64_t striped(const uint8_t* p, size_t n, size_t zero_at, size_t zero_n) {
  uint64_t lane[8];
  for (size_t l = 0; l < 8; ++l) lane[l] = kBasis ^ (0x9E3779B97F4A7C15ULL * (l + 1));
  size_t i = 0;
  for (; i + 8 <= n; i += 8)
    for (size_t l = 0; l < 8; ++l) {
      const size_t at = i + l;
      const uint8_t byte = (at >= zero_at && at < zero_at + zero_n) ? 0 : p[at];
      lane[l] ^= byte;
      lane[l] *= kPrime;
    }
  for (size_t l = 0; i < n; ++i, ++l) {
    const uint8_t byte = (i >= zero_at && i < zero_at + zero_n) ? 0 : p[i];
    lane[l] ^= byte;
    lane[l] *= kPrime;
  }
  uint64_t h = kBasis;
  for (size_t l = 0; l < 8; ++l) h = mix_word(h, lane[l]);
  return mix_word(h, n);
}
static uint64_t chunked(const uint8_t* p, size_t n, size_t hash_off, int seal) { /* :114-161 */
  const size_t g = chunk_grain(n, 1u << 20);
  uint64_t h = kBasis;
  if (n == 0) {
    h = mix_word(h, striped(p, 0, 0, 0));
    return mix_word(h, 0);
  }
  for (size_t b = 0; b < n; b += g) {
    const size_t e = b + g < n ? b + g : n;
    size_t za = (size_t)-1, zn = 0;
    if (seal && hash_off < e && hash_off + 8 > b) {
      const size_t lo = hash_off > b ? hash_off : b;
      const size_t hi = hash_off + 8 < e ? hash_off + 8 : e;
      za = lo - b;
      zn = hi - lo;
    }
    h = mix_word(h, striped(p + b, e - b, za, zn));
  }
  return mix_word(h, n);
}
uint64_t orc_content_hash64(const uint8_t* p, size_t n) { return chunked(p, n, 0, 0); }
uint64_t orc_plan_self_hash(const uint8_t* p, size_t n, size_t hash_off) {
  return chunked(p, n, hash_off, 1);
}
