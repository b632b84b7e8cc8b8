// CUDA-core GEMM for the update ISA: C = alpha * op(A) @ op(B) (+C), batched, with
// arbitrary element strides, so one kernel serves GemmNN / NT / TN / AccNN, the
// int8-dequantising variants, ragged shapes (N = 10, rank-r factors) and the
// batched per-head products of the attention primitives with their causal
// structure. It is the always-correct path; the large frozen-weight GEMMs go to
// the tcgen05 kernel instead. 64x64x16 tiles, 256 threads, 4x4 outputs per thread,
// f32 FMA accumulation. Reductions too short on tiles and long on K are split
// over K in chunks whose size depends on the shape only, and the partials are
// summed in split order, so the result does not depend on scheduling.
#include "kernels.h"

namespace seeml_b200 {
namespace k {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

struct Split {
  int splits;   // number of K chunks
  int kchunk;   // K elements per chunk (multiple of BK)
};
inline Split plan_split(const GemmDesc& d) {
  Split s{1, d.K};
  if (d.causal != 0 || d.accumulate || d.K < 4096) return s;
  const long long tiles = (long long)((d.M + BM - 1) / BM) * ((d.N + BN - 1) / BN) * d.batch;
  if (tiles >= 128) return s;
  int want = (int)(296 / tiles);              // about two waves of the 148 SMs
  int kchunk = ((d.K + want - 1) / want + BK - 1) / BK * BK;
  if (kchunk < 512) kchunk = 512;
  s.kchunk = kchunk;
  s.splits = (d.K + kchunk - 1) / kchunk;
  return s;
}

template <bool Q8>
__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmDesc d, int splits, int kchunk,
                                                        float* __restrict__ ws) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, each TM x TN
  const int z = blockIdx.z / splits, sp = blockIdx.z % splits;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const long long b0 = z / d.nb_inner, b1 = z % d.nb_inner;
  const float* A = d.A + b0 * d.sAb0 + b1 * d.sAb1;
  const float* B = d.B + b0 * d.sBb0 + b1 * d.sBb1;
  const int8_t* Bq = Q8 ? d.Bq8 : nullptr;
  float* C = d.C + b0 * d.sCb0 + b1 * d.sCb1;

  int k_begin = sp * kchunk, k_end = min(d.K, k_begin + kchunk);
  if (d.causal == 1 && n0 > m0 + BM - 1) {
    // tile entirely above the diagonal: masked entries are exact zeros
    for (int i = tid; i < BM * BN; i += 256) {
      const int m = m0 + i / BN, n = n0 + i % BN;
      if (m < d.M && n < d.N) C[(long long)m * d.sCm + n] = 0.0f;
    }
    return;
  }
  if (d.causal == 2) k_end = min(k_end, m0 + BM);        // A[m,k] = 0 for k > m
  if (d.causal == 3) k_begin = max(k_begin, m0 / BK * BK);  // A[m,k] = 0 for k < m

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  const bool a_kfast = d.sAk == 1;   // consecutive threads along k
  const bool b_nfast = d.sBn == 1;
  for (int k0 = k_begin; k0 < k_end; k0 += BK) {
    // A tile: BM x BK
#pragma unroll
    for (int i = 0; i < (BM * BK) / 256; ++i) {
      const int e = tid + i * 256;
      int m, kk;
      if (a_kfast) { kk = e % BK; m = e / BK; } else { m = e % BM; kk = e / BM; }
      const int gm = m0 + m, gk = k0 + kk;
      float v = 0.0f;
      if (gm < d.M && gk < k_end) v = A[(long long)gm * d.sAm + (long long)gk * d.sAk];
      As[kk][m] = v;
    }
#pragma unroll
    for (int i = 0; i < (BN * BK) / 256; ++i) {
      const int e = tid + i * 256;
      int n, kk;
      if (b_nfast) { n = e % BN; kk = e / BN; } else { kk = e % BK; n = e / BK; }
      const int gn = n0 + n, gk = k0 + kk;
      float v = 0.0f;
      if (gn < d.N && gk < k_end) {
        const long long at = (long long)gk * d.sBk + (long long)gn * d.sBn;
        v = Q8 ? (float)Bq[at] : B[at];
      }
      Bs[kk][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= d.M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= d.N) continue;
      if (splits > 1) {
        ws[((long long)blockIdx.z * d.M + m) * d.N + n] = acc[i][j];
        continue;
      }
      float v = d.alpha * acc[i][j];
      if (d.causal == 1 && n > m) v = 0.0f;
      float* c = &C[(long long)m * d.sCm + n];
      if (d.accumulate) v = *c + v;
      if (d.bias) v = v + d.bias[n];
      if (d.act) {
        if (d.act == 1) v = v > 0.0f ? v : 0.0f;
        else if (d.act == 2) {
          const float t = tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v));
          v = 0.5f * v * (1.0f + t);
        } else v = v * (1.0f / (1.0f + expf(-v)));
      }
      *c = v;
    }
  }
}

// Ordered sum of the K-split partials, then the same epilogue as the direct path.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(GemmDesc d, int splits,
                                                            const float* __restrict__ ws) {
  const long long per = (long long)d.M * d.N;
  const long long total = per * d.batch;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long z = i / per, e = i % per;
    const int m = (int)(e / d.N), n = (int)(e % d.N);
    float s = 0.0f;
    for (int sp = 0; sp < splits; ++sp) s += ws[(z * splits + sp) * per + e];
    float v = d.alpha * s;
    const long long b0 = z / d.nb_inner, b1 = z % d.nb_inner;
    float* c = d.C + b0 * d.sCb0 + b1 * d.sCb1 + (long long)m * d.sCm + n;
    if (d.bias) v = v + d.bias[n];
    if (d.act) {
      if (d.act == 1) v = v > 0.0f ? v : 0.0f;
      else if (d.act == 2) {
        const float t = tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v));
        v = 0.5f * v * (1.0f + t);
      } else v = v * (1.0f / (1.0f + expf(-v)));
    }
    *c = v;
  }
}

}  // namespace

size_t gemm_simt_workspace_floats(const GemmDesc& d) {
  const Split s = plan_split(d);
  if (s.splits <= 1) return 0;
  return (size_t)s.splits * d.batch * d.M * d.N;
}

int gemm_simt(const GemmDesc& d, float* workspace, cudaStream_t st) {
  if (d.M <= 0 || d.N <= 0 || d.batch <= 0) return 0;
  const Split s = plan_split(d);
  dim3 grid((d.N + BN - 1) / BN, (d.M + BM - 1) / BM, d.batch * s.splits);
  if (d.Bq8)
    gemm_simt_kernel<true><<<grid, 256, 0, st>>>(d, s.splits, s.kchunk, workspace);
  else
    gemm_simt_kernel<false><<<grid, 256, 0, st>>>(d, s.splits, s.kchunk, workspace);
  if (s.splits <= 1) return 1;
  const long long total = (long long)d.M * d.N * d.batch;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  splitk_reduce_kernel<<<blocks, 256, 0, st>>>(d, s.splits, workspace);
  return 2;
}

}  // namespace k
}  // namespace seeml_b200
