// GEMMs with one tiny dimension — the rank-r factors of the LoRA adapters. All three
// forms are HBM-bound on their one large operand (intensity ~ r/2 FLOP per byte), so
// they run on the CUDA cores with f32 FMA and are built to touch the large operand
// exactly once with coalesced 128-bit accesses:
//
//   skinny_n   out[M,n]  = alpha * A[M,K] . B        n <= 64   (t = X.A, dt = ds.B^T)
//   skinny_k   out[M,N]  = alpha * A[M,k] . B (+ D)  k <= 32   (u = t.B, dx = dt.A^T)
//   skinny_tn  out       = alpha * U[T,p]^T . V[T,q]           (dA = X^T.dt, dB = t^T.ds)
//
// skinny_tn reduces over the T rows in chunks of a fixed 256 rows and sums the chunk
// partials in chunk order, so the result does not depend on how blocks are scheduled.
#include "kernels.h"

namespace seeml_b200 {
namespace k {
namespace {

// ---- skinny_n: one warp owns 4 rows (2 for n = 32); lanes stride the reduction dimension ---------------
// Each lane reads 16 bytes of each of its warp's 4 rows per 128-wide K step (coalesced,
// every byte of A touched once), multiplies with the matching slice of B held in shared
// memory as [n][k] (conflict-free 128-bit reads for both B layouts) and keeps 4 x n partial
// sums; one fixed shuffle tree per output at the end. The next step's A words and B slice
// are fetched into registers while the current one is multiplied (double-buffered B tile).
template <int N_>
__host__ __device__ constexpr int skinny_n_rows() { return N_ >= 32 ? 2 : 4; }      // rows per warp
template <int N_>
__global__ void __launch_bounds__(256, 2) skinny_n_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                       float* __restrict__ out, int M, int K, int b_is_nk,
                                                       float alpha) {
  constexpr int KC = 128, R = skinny_n_rows<N_>(), WARPS = 8, PER = N_ * KC / 256;
  __shared__ __align__(16) float Bs[2][N_][KC + 4];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = (blockIdx.x * WARPS + warp) * R;
  float acc[R][N_];
#pragma unroll
  for (int i = 0; i < R; ++i)
#pragma unroll
    for (int j = 0; j < N_; ++j) acc[i][j] = 0.0f;
  float4 a[R], a_next[R];
  float b_next[PER];
  auto fetch = [&](int k0, float4* av, float* bv) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      av[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      const int k = k0 + lane * 4;
      if (m0 + i < M && k < K) av[i] = *reinterpret_cast<const float4*>(A + (size_t)(m0 + i) * K + k);   // K % 4 == 0
    }
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int e = tid + u * 256;
      int kk, nn;
      if (b_is_nk) { kk = e % KC; nn = e / KC; } else { nn = e % N_; kk = e / N_; }
      bv[u] = 0.0f;
      if (k0 + kk < K) bv[u] = b_is_nk ? B[(size_t)nn * K + k0 + kk] : B[(size_t)(k0 + kk) * N_ + nn];
    }
  };
  auto stash = [&](int buf, const float* bv) {
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int e = tid + u * 256;
      int kk, nn;
      if (b_is_nk) { kk = e % KC; nn = e / KC; } else { nn = e % N_; kk = e / N_; }
      Bs[buf][nn][kk] = bv[u];
    }
  };
  fetch(0, a, b_next);
  stash(0, b_next);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += KC) {
    const bool more = k0 + KC < K;
    if (more) fetch(k0 + KC, a_next, b_next);
#pragma unroll
    for (int j = 0; j < N_; ++j) {
      const float4 b = *reinterpret_cast<const float4*>(&Bs[buf][j][lane * 4]);
#pragma unroll
      for (int i = 0; i < R; ++i)
        acc[i][j] = fmaf(a[i].w, b.w, fmaf(a[i].z, b.z, fmaf(a[i].y, b.y, fmaf(a[i].x, b.x, acc[i][j]))));
    }
    if (more) {
      stash(buf ^ 1, b_next);
#pragma unroll
      for (int i = 0; i < R; ++i) a[i] = a_next[i];
    }
    __syncthreads();
    buf ^= 1;
  }
#pragma unroll
  for (int i = 0; i < R; ++i)
#pragma unroll
    for (int j = 0; j < N_; ++j) {
      float v = acc[i][j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == (j & 31) && m0 + i < M) out[(size_t)(m0 + i) * N_ + j] = alpha * v;
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
// A thread owns 4 consecutive columns of the big operand (one coalesced 128-bit global load
// per row, every byte of W touched once) and all `small` outputs for them; the chunk's S
// rows sit in shared memory and are read as broadcasts. Four row groups of 64 threads share
// the chunk's rows (row r belongs to group r / 64) and are added in group order at the end.
constexpr int kTnRows = 256;       // rows per chunk: a constant, so the summation tree is a function of T only
template <int SMALL>
__global__ void __launch_bounds__(256) skinny_tn_kernel(const float* __restrict__ Wb, const float* __restrict__ Ss,
                                                        float* __restrict__ partial, int T, int big, int small) {
  __shared__ __align__(16) float St[kTnRows * SMALL];       // S rows; afterwards the group-reduction buffer
  const int tid = threadIdx.x, col = tid & 63, grp = tid >> 6;
  const int b0 = (blockIdx.x * 64 + col) * 4, chunk = blockIdx.y;
  const int t_begin = chunk * kTnRows, t_end = min(T, t_begin + kTnRows), rows = t_end - t_begin;
  for (int e = tid; e < kTnRows * SMALL; e += 256) {
    const int r = e / SMALL, sidx = e % SMALL;
    St[e] = (r < rows && sidx < small) ? Ss[(size_t)(t_begin + r) * small + sidx] : 0.0f;
  }
  __syncthreads();
  float acc[SMALL][4];
#pragma unroll
  for (int j = 0; j < SMALL; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
  const bool live = b0 < big;      // big % 4 == 0
  if (live) {
    const int r_begin = grp * (kTnRows / 4), r_end = min(rows, r_begin + kTnRows / 4);
    const float* wp = Wb + (size_t)t_begin * big + b0;
#pragma unroll 8
    for (int r = r_begin; r < r_end; ++r) {
      const float4 w = __ldg(reinterpret_cast<const float4*>(wp + (size_t)r * big));
#pragma unroll
      for (int j4 = 0; j4 < SMALL / 4; ++j4) {
        const float4 sv = *reinterpret_cast<const float4*>(&St[r * SMALL + j4 * 4]);
        const float sj[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float* a = acc[j4 * 4 + q];
          a[0] = fmaf(sj[q], w.x, a[0]); a[1] = fmaf(sj[q], w.y, a[1]);
          a[2] = fmaf(sj[q], w.z, a[2]); a[3] = fmaf(sj[q], w.w, a[3]);
        }
      }
    }
  }
  // groups 1..3 hand their sums to group 0 one after the other: ((g0 + g1) + g2) + g3
  float4* red = reinterpret_cast<float4*>(St);            // [SMALL][64] float4
  for (int g = 1; g < 4; ++g) {
    __syncthreads();
    if (grp == g) {
#pragma unroll
      for (int j = 0; j < SMALL; ++j) red[j * 64 + col] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
    }
    __syncthreads();
    if (grp == 0) {
#pragma unroll
      for (int j = 0; j < SMALL; ++j) {
        const float4 v = red[j * 64 + col];
        acc[j][0] += v.x; acc[j][1] += v.y; acc[j][2] += v.z; acc[j][3] += v.w;
      }
    }
  }
  if (grp == 0 && live) {
#pragma unroll
    for (int j = 0; j < SMALL; ++j)
      if (j < small)
        *reinterpret_cast<float4*>(partial + ((size_t)chunk * small + j) * big + b0) =
            make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
  }
}
// out = alpha * (partials summed in chunk order); out is [small,big] or, transposed, [big,small].
// The partials are [chunk][small][big], or [chunk][big][small] when ws_bs is set.
__global__ void __launch_bounds__(256) skinny_tn_reduce_kernel(const float* __restrict__ partial,
                                                               float* __restrict__ out, int chunks, int big,
                                                               int small, int transposed, float alpha, int ws_bs) {
  const int total = big * small;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    // walk the index space in the partials' own order so the reads coalesce
    const int s = ws_bs ? i % small : i / big, b = ws_bs ? i / small : i % big;
    float acc = 0.0f;
    for (int ch = 0; ch < chunks; ++ch) acc += partial[(size_t)ch * total + i];
    out[transposed ? (size_t)b * small + s : (size_t)s * big + b] = alpha * acc;
  }
}

}  // namespace

bool skinny_n_ok(int M, int n, int K) { return (n == 4 || n == 8 || n == 16 || n == 32) && K % 4 == 0 && K >= 128 && M >= 64; }
bool skinny_k_ok(int M, int N, int k) { return k >= 1 && k <= 32 && N % 4 == 0 && N >= 64 && M >= 32; }
bool skinny_tn_ok(int T, int big, int small) { return small >= 1 && small <= 32 && big >= 64 && big % 4 == 0 && T >= 1024; }
size_t skinny_tn_workspace_floats(int T, int big, int small) {
  return (size_t)((T + kTnRows - 1) / kTnRows) * big * small;
}

int skinny_n(const float* A, const float* B, float* out, int M, int n, int K, int b_is_nk, float alpha,
             cudaStream_t st) {
  auto grid = [&](int rows_per_warp) { return dim3((unsigned)((M + 8 * rows_per_warp - 1) / (8 * rows_per_warp))); };
  switch (n) {
    case 4: skinny_n_kernel<4><<<grid(skinny_n_rows<4>()), 256, 0, st>>>(A, B, out, M, K, b_is_nk, alpha); break;
    case 8: skinny_n_kernel<8><<<grid(skinny_n_rows<8>()), 256, 0, st>>>(A, B, out, M, K, b_is_nk, alpha); break;
    case 16: skinny_n_kernel<16><<<grid(skinny_n_rows<16>()), 256, 0, st>>>(A, B, out, M, K, b_is_nk, alpha); break;
    default: skinny_n_kernel<32><<<grid(skinny_n_rows<32>()), 256, 0, st>>>(A, B, out, M, K, b_is_nk, alpha); break;
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
  const dim3 grid((big + 255) / 256, chunks);
  if (small <= 8) skinny_tn_kernel<8><<<grid, 256, 0, st>>>(W, S, workspace, T, big, small);
  else if (small <= 16) skinny_tn_kernel<16><<<grid, 256, 0, st>>>(W, S, workspace, T, big, small);
  else skinny_tn_kernel<32><<<grid, 256, 0, st>>>(W, S, workspace, T, big, small);
  int blocks = (big * small + 255) / 256;
  if (blocks > 1184) blocks = 1184;
  skinny_tn_reduce_kernel<<<blocks, 256, 0, st>>>(workspace, out, chunks, big, small, transposed, alpha, 0);
  return 2;
}

// Ordered sum of per-chunk partials laid out [chunk][big][small] (the tensor-core producer).
int skinny_tn_reduce_bs(const float* workspace, float* out, int chunks, int big, int small, int transposed,
                        float alpha, cudaStream_t st) {
  int blocks = (big * small + 255) / 256;
  if (blocks > 1184) blocks = 1184;
  skinny_tn_reduce_kernel<<<blocks, 256, 0, st>>>(workspace, out, chunks, big, small, transposed, alpha, 1);
  return 1;
}

}  // namespace k
}  // namespace seeml_b200
