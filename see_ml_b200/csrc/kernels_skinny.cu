// GEMMs with one tiny dimension — the rank-r factors of the LoRA adapters. All three
// forms are HBM-bound on their one large operand (intensity ~ r/2 FLOP per byte), so
// they run on the CUDA cores with f32 FMA and are built to touch the large operand
// exactly once with coalesced 128-bit accesses:
//
//   skinny_n   out[M,n]  = alpha * A[M,K] . B        n <= 64   (t = X.A, dt = ds.B^T)
//   skinny_k   out[M,N]  = alpha * A[M,k] . B (+ D)  k <= 32   (u = t.B, dx = dt.A^T)
//   skinny_tn  out       = alpha * U[T,p]^T . V[T,q]           (dA = X^T.dt, dB = t^T.ds)
//
// skinny_tn reduces over the T rows in chunks of a fixed 512 rows and sums the chunk
// partials in chunk order, so the result does not depend on how blocks are scheduled.
#include "kernels.h"

namespace seeml_b200 {
namespace k {
namespace {

// ---- skinny_n: 64 rows per block, K walked in chunks of 64 through shared memory ----
template <int NPT>   // outputs per thread; n = 4 * NPT
__global__ void __launch_bounds__(256) skinny_n_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                       float* __restrict__ out, int M, int K, int b_is_nk,
                                                       float alpha) {
  constexpr int n = 4 * NPT, KC = 64, ROWS = 64;
  __shared__ float As[ROWS][KC + 4];
  __shared__ float Bs[KC][n];
  const int tid = threadIdx.x, row = tid >> 2, cg = (tid & 3) * NPT;
  const int m0 = blockIdx.x * ROWS;
  float acc[NPT];
#pragma unroll
  for (int j = 0; j < NPT; ++j) acc[j] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += KC) {
    // A tile: 64 x 128, K fastest (coalesced); K is a multiple of 4 (checked by the launcher)
    for (int e = tid; e < ROWS * KC / 4; e += 256) {
      const int r = e / (KC / 4), c4 = (e % (KC / 4)) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m0 + r < M && k0 + c4 < K) v = *reinterpret_cast<const float4*>(A + (size_t)(m0 + r) * K + k0 + c4);
      *reinterpret_cast<float4*>(&As[r][c4]) = v;
    }
    for (int e = tid; e < KC * n; e += 256) {
      int kk, nn;
      if (b_is_nk) { kk = e % KC; nn = e / KC; } else { nn = e % n; kk = e / n; }
      float v = 0.0f;
      if (k0 + kk < K) v = b_is_nk ? B[(size_t)nn * K + k0 + kk] : B[(size_t)(k0 + kk) * n + nn];
      Bs[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < KC; ++kk) {
      const float a = As[row][kk];
#pragma unroll
      for (int j = 0; j < NPT; ++j) acc[j] = fmaf(a, Bs[kk][cg + j], acc[j]);
    }
    __syncthreads();
  }
  if (m0 + row < M) {
#pragma unroll
    for (int j = 0; j < NPT; ++j) out[(size_t)(m0 + row) * n + cg + j] = alpha * acc[j];
  }
}

// ---- skinny_k: 32 x 256 output tile, whole (tiny) reduction held in shared memory -----
template <int KK>
__global__ void __launch_bounds__(256) skinny_k_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                       const float* __restrict__ addend, float* __restrict__ out,
                                                       int M, int N, int k, int b_is_nk, float alpha) {
  constexpr int ROWS = 32, COLS = 256;
  __shared__ float As[ROWS][KK];
  __shared__ __align__(16) float Bs[KK][COLS];
  const int tid = threadIdx.x, tx = tid & 63, ty = tid >> 6;
  const int m0 = blockIdx.y * ROWS, n0 = blockIdx.x * COLS;
  for (int e = tid; e < ROWS * KK; e += 256) {
    const int r = e / KK, c = e % KK;
    As[r][c] = (m0 + r < M && c < k) ? A[(size_t)(m0 + r) * k + c] : 0.0f;
  }
  for (int e = tid; e < KK * COLS; e += 256) {
    int kk, nn;
    if (b_is_nk) { kk = e % KK; nn = e / KK; } else { nn = e % COLS; kk = e / COLS; }
    float v = 0.0f;
    if (kk < k && n0 + nn < N) v = b_is_nk ? B[(size_t)(n0 + nn) * k + kk] : B[(size_t)kk * N + n0 + nn];
    Bs[kk][nn] = v;
  }
  __syncthreads();
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
#pragma unroll
  for (int kk = 0; kk < KK; ++kk) {
    const float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = As[ty * 8 + i][kk];
      acc[i][0] = fmaf(a, b.x, acc[i][0]); acc[i][1] = fmaf(a, b.y, acc[i][1]);
      acc[i][2] = fmaf(a, b.z, acc[i][2]); acc[i][3] = fmaf(a, b.w, acc[i][3]);
    }
  }
  const int n = n0 + tx * 4;
  if (n >= N) return;               // N is a multiple of 4 (checked by the launcher)
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + ty * 8 + i;
    if (m >= M) break;
    float4 v = make_float4(alpha * acc[i][0], alpha * acc[i][1], alpha * acc[i][2], alpha * acc[i][3]);
    if (addend) {
      const float4 d = *reinterpret_cast<const float4*>(addend + (size_t)m * N + n);
      v.x = d.x + v.x; v.y = d.y + v.y; v.z = d.z + v.z; v.w = d.w + v.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)m * N + n) = v;
  }
}

// ---- skinny_tn: partial[chunk][s][b] = sum over the chunk's rows of S[t,s] * W[t,b] -------
constexpr int kTnRows = 512;       // rows per chunk: a function of nothing but this constant
template <int SH>                  // accumulators per thread; small = 2 * SH
__global__ void __launch_bounds__(256) skinny_tn_kernel(const float* __restrict__ Wb, const float* __restrict__ Ss,
                                                        float* __restrict__ partial, int T, int big, int small) {
  constexpr int COLS = 128, RT = 32;
  __shared__ float Wt[RT][COLS];
  __shared__ float St[RT][2 * SH];
  const int tid = threadIdx.x, c = tid & 127, h = tid >> 7;
  const int b0 = blockIdx.x * COLS, chunk = blockIdx.y;
  const int t_begin = chunk * kTnRows, t_end = min(T, t_begin + kTnRows);
  float acc[SH];
#pragma unroll
  for (int j = 0; j < SH; ++j) acc[j] = 0.0f;
  for (int t0 = t_begin; t0 < t_end; t0 += RT) {
    for (int e = tid; e < RT * COLS; e += 256) {
      const int r = e >> 7, cc = e & 127;
      Wt[r][cc] = (t0 + r < t_end && b0 + cc < big) ? Wb[(size_t)(t0 + r) * big + b0 + cc] : 0.0f;
    }
    for (int e = tid; e < RT * 2 * SH; e += 256) {
      const int r = e / (2 * SH), s = e % (2 * SH);
      St[r][s] = (t0 + r < t_end && s < small) ? Ss[(size_t)(t0 + r) * small + s] : 0.0f;
    }
    __syncthreads();
#pragma unroll 4
    for (int r = 0; r < RT; ++r) {
      const float w = Wt[r][c];
#pragma unroll
      for (int j = 0; j < SH; ++j) acc[j] = fmaf(St[r][h * SH + j], w, acc[j]);
    }
    __syncthreads();
  }
  if (b0 + c < big) {
#pragma unroll
    for (int j = 0; j < SH; ++j) {
      const int s = h * SH + j;
      if (s < small) partial[((size_t)chunk * small + s) * big + b0 + c] = acc[j];
    }
  }
}
// out = alpha * (partials summed in chunk order); out is [small,big] or, transposed, [big,small].
__global__ void __launch_bounds__(256) skinny_tn_reduce_kernel(const float* __restrict__ partial,
                                                               float* __restrict__ out, int chunks, int big,
                                                               int small, int transposed, float alpha) {
  const int total = big * small;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int s = i / big, b = i % big;
    float acc = 0.0f;
    for (int ch = 0; ch < chunks; ++ch) acc += partial[((size_t)ch * small + s) * big + b];
    out[transposed ? (size_t)b * small + s : (size_t)i] = alpha * acc;
  }
}

}  // namespace

bool skinny_n_ok(int M, int n, int K) { return n >= 4 && n <= 64 && (n & (n - 1)) == 0 && K % 4 == 0 && K >= 128 && M >= 64; }
bool skinny_k_ok(int M, int N, int k) { return k >= 1 && k <= 32 && N % 4 == 0 && N >= 64 && M >= 32; }
bool skinny_tn_ok(int T, int big, int small) { return small >= 1 && small <= 64 && big >= 64 && T >= 1024; }
size_t skinny_tn_workspace_floats(int T, int big, int small) {
  return (size_t)((T + kTnRows - 1) / kTnRows) * big * small;
}

int skinny_n(const float* A, const float* B, float* out, int M, int n, int K, int b_is_nk, float alpha,
             cudaStream_t st) {
  const dim3 grid((M + 63) / 64);
  switch (n) {
    case 4: skinny_n_kernel<1><<<grid, 256, 0, st>>>(A, B, out, M, K, b_is_nk, alpha); break;
    case 8: skinny_n_kernel<2><<<grid, 256, 0, st>>>(A, B, out, M, K, b_is_nk, alpha); break;
    case 16: skinny_n_kernel<4><<<grid, 256, 0, st>>>(A, B, out, M, K, b_is_nk, alpha); break;
    case 32: skinny_n_kernel<8><<<grid, 256, 0, st>>>(A, B, out, M, K, b_is_nk, alpha); break;
    default: skinny_n_kernel<16><<<grid, 256, 0, st>>>(A, B, out, M, K, b_is_nk, alpha); break;
  }
  return 1;
}
int skinny_k(const float* A, const float* B, const float* addend, float* out, int M, int N, int k, int b_is_nk,
             float alpha, cudaStream_t st) {
  const dim3 grid((N + 255) / 256, (M + 31) / 32);
  if (k <= 8) skinny_k_kernel<8><<<grid, 256, 0, st>>>(A, B, addend, out, M, N, k, b_is_nk, alpha);
  else if (k <= 16) skinny_k_kernel<16><<<grid, 256, 0, st>>>(A, B, addend, out, M, N, k, b_is_nk, alpha);
  else skinny_k_kernel<32><<<grid, 256, 0, st>>>(A, B, addend, out, M, N, k, b_is_nk, alpha);
  return 1;
}
int skinny_tn(const float* W, const float* S, float* out, float* workspace, int T, int big, int small,
              int transposed, float alpha, cudaStream_t st) {
  const int chunks = (T + kTnRows - 1) / kTnRows;
  const dim3 grid((big + 127) / 128, chunks);
  if (small <= 8) skinny_tn_kernel<4><<<grid, 256, 0, st>>>(W, S, workspace, T, big, small);
  else if (small <= 16) skinny_tn_kernel<8><<<grid, 256, 0, st>>>(W, S, workspace, T, big, small);
  else if (small <= 32) skinny_tn_kernel<16><<<grid, 256, 0, st>>>(W, S, workspace, T, big, small);
  else skinny_tn_kernel<32><<<grid, 256, 0, st>>>(W, S, workspace, T, big, small);
  int blocks = (big * small + 255) / 256;
  if (blocks > 1184) blocks = 1184;
  skinny_tn_reduce_kernel<<<blocks, 256, 0, st>>>(workspace, out, chunks, big, small, transposed, alpha);
  return 2;
}

}  // namespace k
}  // namespace seeml_b200
