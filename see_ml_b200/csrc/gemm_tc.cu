// Tensor-core GEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T (+ bias, activation), f32
// in / f32 out, both operands K-major in global memory. Hand-written tcgen05 path:
//
//   TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) -> shared-memory stages
//   -> tcgen05.mma kind::tf32, 128 x BN accumulator in TMEM -> tcgen05.ld -> swizzled
//   shared staging -> TMA store (which clips ragged M / N edges).
//
// Precision modes. TF32X3 keeps f32-class accuracy with three tensor-core products
// per tile step, a*b ~= hi(a)*hi(b) + lo(a)*hi(b) + hi(a)*lo(b), where hi(x) is x
// with the low 13 mantissa bits cleared (what a tf32 operand keeps of an f32 word)
// and lo(x) = x - hi(x) is exact in f32. Four "split" warps derive the lo tiles in
// shared memory from the TMA-loaded f32 tiles, so no extra global traffic is spent
// on the split. TF32 is the single-product mode.
//
// Warp roles (320 threads): warp 0 issues TMA loads, warp 1 owns TMEM and issues the
// MMAs, warps 2..9 split the operands, collect finished accumulation chunks into registers
// and run the epilogue (the batched attention kernel keeps 4 such warps).
// Every wait on an mbarrier is bounded: on expiry the kernel records an error code,
// drains, frees its TMEM and returns, so a protocol bug cannot hang the device.
//
// The frozen weight of a forward GemmNN is stored [K,N]; the context keeps a
// transposed [N,K] copy (made once, when the program is built) so forward and
// backward GEMMs through frozen weights both take this K-major form.
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <set>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "backend.h"
#include "tc_ptx.cuh"

namespace seeml_b200 {
namespace {

using namespace tc;

// f32-class accuracy requested (a split product): the kernels other than the CTA-pair GEMM run
// the three-product tf32 split in both of these modes.
inline bool kind_x3(const seeml_b200_ctx* c) {
  return c->gemm_kind == SEEML_B200_GEMM_TF32X3 || c->gemm_kind == SEEML_B200_GEMM_F16X2;
}
inline bool kind_tc(const seeml_b200_ctx* c) { return c->gemm_kind != SEEML_B200_GEMM_FP32_SIMT; }

constexpr int BM = 128;
constexpr int BK = 32;                 // f32 elements = one 128-byte swizzle row
constexpr int kBgWorkers = 256;          // batched kernel: 8 split warps, the first 4 also collect and store
constexpr int kThreadsTC = 64 + kBgWorkers;

struct TcParams {
  int M, N, K;
  int K2;                // reduction length of the optional second operand pair (0 = none)
  const float* bias;     // nullable, length N
  const float* addend;   // nullable, [M,N] row-major: C = addend + A.B^T (+ A2.B2^T)
  int act;               // 0 none 1 relu 2 gelu 3 silu
  float alpha;           // scales the product before addend / bias / activation
  int b_lo;              // the lo tiles of B (main pair) come from a precomputed copy through mapBlo
  int n_tiles, total_tiles;   // pair kernel: 256-wide N tiles, and 256 x 256 tiles in all
  int* err;              // device error word
};

__device__ __forceinline__ float epi_act(int act, float v) {
  if (act == 1) return v > 0.0f ? v : 0.0f;
  if (act == 2) {
    const float t = tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v));
    return 0.5f * v * (1.0f + t);
  }
  if (act == 3) return v * (1.0f / (1.0f + expf(-v)));
  return v;
}

// ------------------------------------------------------------------- the kernel
// The tensor core adds into its f32 accumulator with truncation, so a long reduction kept
// in TMEM alone drifts (error ~ steps * 2^-24 * |partial sum|). The reduction is therefore
// cut into chunks of kChunk k-blocks that alternate between two TMEM accumulators; the worker
// warps add every finished chunk into f32 registers (round-to-nearest) while the next chunk is
// being multiplied, and the output tile is stored from those registers.
constexpr int kChunk = 4;              // k-blocks (x 32 elements) per TMEM accumulation chunk
constexpr int kWorkers = 256;          // threads of the 8 split / accumulate / epilogue warps
constexpr int kThreadsV2 = 64 + kWorkers;

template <int BN, bool SPLIT, int STAGES, int KB>
struct Smem {
  static constexpr int kABytes = BM * KB * 4;             // 16 KiB at KB = 32
  static constexpr int kBBytes = BN * KB * 4;
  static constexpr int kRawBytes = kABytes + kBBytes;
  static constexpr int kStageBytes = kRawBytes * (SPLIT ? 2 : 1);
  static constexpr int kEpiBytes = BM * (BN < 32 ? 32 : BN) * 4;   // store staging, aliases the stage buffers
  static constexpr int kBarBytes = 256;
  static constexpr int kTotal = STAGES * kStageBytes + kBarBytes + 1024;  // + alignment slack
  static_assert(STAGES * kStageBytes >= kEpiBytes, "store staging must fit in the stage buffers");
};

template <int BN, bool SPLIT, int STAGES, int KB>
__global__ void __launch_bounds__(kThreadsV2, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapA2,
               const __grid_constant__ CUtensorMap mapB2, const __grid_constant__ CUtensorMap mapBlo, TcParams p) {
  using S = Smem<BN, SPLIT, STAGES, KB>;
  constexpr int kChunkBlocks = kChunk * (BK / KB);   // k-blocks per accumulation chunk (128 elements of K)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + STAGES * S::kStageBytes;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_split = [&](int s) { return bars + 8u * (STAGES + s); };
  auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };
  auto bar_acc_full = [&](int b) { return bars + 8u * (3 * STAGES + b); };
  auto bar_acc_empty = [&](int b) { return bars + 8u * (3 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (3 * STAGES + 4);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + STAGES * S::kStageBytes + 8 * (3 * STAGES + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  // k-blocks of the main pair, then of the low-rank pair (C += A2[M,K2] . B2[N,K2]^T): the
  // LoRA term rides the same accumulators as extra reduction steps
  const int nkb1 = (p.K + KB - 1) / KB;
  const int nkb = nkb1 + (p.K2 + KB - 1) / KB;
  const int nchunks = (nkb + kChunkBlocks - 1) / kChunkBlocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_split(s), kWorkers / 32);        // one arrival per worker warp
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), kWorkers / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Stage layout: [A raw][A lo][B raw][B lo] (the lo tiles only when SPLIT). Narrow tiles stack
  // B_hi and B_lo into one MMA of width 2*BN (see bgemm_tc_kernel): two MMAs per step, not three.
  constexpr bool STACK = SPLIT && BN <= 64;
  constexpr int kAccCols = STACK ? 2 * BN : BN;
  constexpr int kBOff = S::kABytes * (SPLIT ? 2 : 1);
  constexpr uint32_t kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ---- TMA producer -------------------------------------------------------------------
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % STAGES, r = kb / STAGES;
        if (r > 0) ok = mbar_wait(bar_empty(s), (r - 1) & 1, p.err, 1);
        if (!ok) break;
        const uint32_t a_dst = base + s * S::kStageBytes, b_dst = a_dst + kBOff;
        const bool lo_too = SPLIT && p.b_lo && kb < nkb1;     // frozen weight: its lo tile is loaded, not derived
        mbar_expect_tx(bar_full(s), S::kRawBytes + (lo_too ? S::kBBytes : 0));
        if (kb < nkb1) {
          tma_load_2d(a_dst, &mapA, bar_full(s), kb * KB, m0);
          tma_load_2d(b_dst, &mapB, bar_full(s), kb * KB, n0);
          if (lo_too) tma_load_2d(b_dst + S::kBBytes, &mapBlo, bar_full(s), kb * KB, n0);
        } else {
          tma_load_2d(a_dst, &mapA2, bar_full(s), (kb - nkb1) * KB, m0);
          tma_load_2d(b_dst, &mapB2, bar_full(s), (kb - nkb1) * KB, n0);
        }
        ++issued;
      }
      if (!ok) {  // drain: let the copies already in flight land before the CTA retires
        for (int kb = (issued > STAGES ? issued - STAGES : 0); kb < issued; ++kb)
          mbar_wait(bar_full(kb % STAGES), (kb / STAGES) & 1, p.err, 5);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ---------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_tf32(BM, BN), idesc2 = idesc_tf32(BM, STACK ? 2 * BN : BN);
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % STAGES, r = kb / STAGES;
        const int ci = kb / kChunkBlocks, buf = ci & 1;
        if (kb % kChunkBlocks == 0 && ci >= 2) {      // the accumulator's previous chunk must have been collected
          ok = mbar_wait(bar_acc_empty(buf), ((ci >> 1) - 1) & 1, p.err, 6);
          if (!ok) break;
          tc_fence_after();
        }
        ok = mbar_wait(SPLIT ? bar_split(s) : bar_full(s), r & 1, p.err, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kAccCols;
        const uint32_t a_raw = base + s * S::kStageBytes, b_raw = a_raw + kBOff;
        const uint32_t a_lo = a_raw + S::kABytes, b_lo = b_raw + S::kBBytes;
#pragma unroll
        for (int kk = 0; kk < KB / 8; ++kk) {
          const uint64_t da = smem_desc_k<KB>(a_raw + kk * 32), db = smem_desc_k<KB>(b_raw + kk * 32);
          if (STACK) {
            mma_tf32(tmem_d, da, db, idesc2, ((kb % kChunkBlocks) | kk) != 0);
            mma_tf32(tmem_d, smem_desc_k<KB>(a_lo + kk * 32), db, idesc, 1);
          } else {
            mma_tf32(tmem_d, da, db, idesc, ((kb % kChunkBlocks) | kk) != 0);
            if (SPLIT) {
              mma_tf32(tmem_d, smem_desc_k<KB>(a_lo + kk * 32), db, idesc, 1);
              mma_tf32(tmem_d, da, smem_desc_k<KB>(b_lo + kk * 32), idesc, 1);
            }
          }
        }
        mma_commit(bar_empty(s));
        if (kb % kChunkBlocks == kChunkBlocks - 1 || kb == nkb - 1) mma_commit(bar_acc_full(buf));
      }
    }
  } else {
    // ---- worker warps: split, collect finished chunks, epilogue ---------------------------
    const int t = threadIdx.x - 64;
    const int q = warp & 3;                     // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;           // which half of the tile's columns it owns
    const int row0 = q * 32;
    constexpr int NH = BN >= 64 ? BN / 2 : BN;  // columns per collecting warp (narrow tiles: warps 2..5 only)
    constexpr int LD = NH >= 32 ? 32 : 16;      // columns per TMEM load / store box
    const bool collector = half * NH < BN;
    float acc[NH];
#pragma unroll
    for (int j = 0; j < NH; ++j) acc[j] = 0.0f;
    bool ok = true;
    int collected = 0;
    auto collect = [&](int ci) {
      const int buf = ci & 1;
      if (!mbar_wait(bar_acc_full(buf), (ci >> 1) & 1, p.err, 4)) return false;
      tc_fence_after();
      if (collector) {
#pragma unroll
        for (int c = 0; c < NH / LD; ++c) {
          uint32_t r[32];
          tmem_ld_cols<LD>(tmem_base + ((uint32_t)row0 << 16) + buf * kAccCols + half * NH + c * LD, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < LD; ++j) acc[c * LD + j] += __uint_as_float(r[j]);
          if (STACK) {
            tmem_ld_cols<LD>(tmem_base + ((uint32_t)row0 << 16) + buf * kAccCols + BN + half * NH + c * LD, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < LD; ++j) acc[c * LD + j] += __uint_as_float(r[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(buf));
      return true;
    };
    for (int kb = 0; kb < nkb && ok; ++kb) {
      const int s = kb % STAGES, r = kb / STAGES;
      if (SPLIT) {
        ok = mbar_wait(bar_full(s), r & 1, p.err, 3);
        if (!ok) break;
        uint8_t* stg = base_ptr + s * S::kStageBytes;
        auto split_range = [&](uint8_t* raw, int bytes) {     // lo tile directly behind its raw tile
          const float4* rp = reinterpret_cast<const float4*>(raw);
          float4* lp = reinterpret_cast<float4*>(raw + bytes);
#pragma unroll 4
          for (int i = t; i < bytes / 16; i += kWorkers) {
            const float4 v = rp[i];
            float4 l;
            l.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
            l.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
            l.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
            l.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
            lp[i] = l;
          }
        };
        split_range(stg, S::kABytes);
        if (!(p.b_lo && kb < nkb1)) split_range(stg + kBOff, S::kBBytes);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_split(s));
      }
      // one k-block into chunk ci the previous chunk has been multiplied: collect it now, while
      // the tensor core works on the blocks already split
      if (kb % kChunkBlocks == 1 && kb > kChunkBlocks) {
        ok = collect(collected);
        ++collected;
      }
    }
    for (; ok && collected < nchunks; ++collected) ok = collect(collected);
    if (ok && collector && m0 + row0 < p.M) {
      // every product has retired (the last chunk was collected), so the stage buffers serve as
      // store staging: one 32x32 box per (warp, column chunk), all stores in flight together
#pragma unroll
      for (int c = 0; c < NH / LD; ++c) {
        const int ncol = n0 + half * NH + c * LD;
        if (ncol < p.N) {
          const uint32_t box = (uint32_t)(((warp - 2) * (NH / LD) + c) * 4096);
          uint8_t* stage_ptr = base_ptr + box;
          uint32_t r[32];
#pragma unroll
          for (int j = 0; j < LD; ++j) r[j] = __float_as_uint(p.alpha * acc[c * LD + j]);
          if (p.addend != nullptr && m0 + row0 + lane < p.M) {
            const float* arow = p.addend + (size_t)(m0 + row0 + lane) * p.N + ncol;
#pragma unroll
            for (int j4 = 0; j4 < LD / 4; ++j4) {
              if (ncol + 4 * j4 < p.N) {          // N is a multiple of 4
                const float4 d = *reinterpret_cast<const float4*>(arow + 4 * j4);
                r[4 * j4 + 0] = __float_as_uint(d.x + __uint_as_float(r[4 * j4 + 0]));
                r[4 * j4 + 1] = __float_as_uint(d.y + __uint_as_float(r[4 * j4 + 1]));
                r[4 * j4 + 2] = __float_as_uint(d.z + __uint_as_float(r[4 * j4 + 2]));
                r[4 * j4 + 3] = __float_as_uint(d.w + __uint_as_float(r[4 * j4 + 3]));
              }
            }
          }
          if (p.bias != nullptr || p.act != 0) {
#pragma unroll
            for (int j = 0; j < LD; ++j) {
              float v = __uint_as_float(r[j]);
              if (p.bias != nullptr && ncol + j < p.N) v = v + p.bias[ncol + j];
              r[j] = __float_as_uint(epi_act(p.act, v));
            }
          }
          // row = lane; 16-byte chunk j lands at (j ^ (row & 7)): the 128-byte swizzle the store expects
#pragma unroll
          for (int j = 0; j < LD / 4; ++j) {
            uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            *reinterpret_cast<uint4*>(stage_ptr + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&mapC, base + box, ncol, m0 + row0);
            tma_store_commit();
          }
        }
      }
      if (lane == 0) tma_store_wait_all();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------- batched per-head products (attention)
// C_z[M,N] = alpha * A_z[M,K] . B_z[K,N] for z = b * H + h, every operand a window of a 2-D
// row-major matrix addressed through TMA coordinates (x0 = b*xb + h*xh, y0 = b*yb + h*yh).
// An operand may be stored "transposed" for the tensor core (A as [K,M], B as [K,N], the
// reduction index on rows): its tile is loaded unswizzled and the split warps write the hi
// and lo tiles K-major with the 128-byte swizzle while they split it, so no transposed copy
// of P, dS or V ever goes through global memory. Causal structure: mode 1 masks outputs with
// n > m (tiles wholly above the diagonal skip the products and store zeros), mode 2 stops the
// reduction at the tile's last row (A[m,k] = 0 for k > m), mode 3 starts it at the tile's
// first row (A[m,k] = 0 for k < m). M % 128 == 0, N % BN == 0 and K % 32 == 0 are required
// (windows of neighbouring heads touch, so the TMA cannot clip ragged edges here).
// What bounds these small-tile kernels is the single thread that issues the products: measured on a
// B200, a tcgen05.mma costs its issuing thread about 50 cycles whatever its width up to N = 64 (a
// 128 x 256 x 8 tf32 product: 133, its arithmetic), a commit arrives about 160 cycles after it is
// issued, and a second issuing thread raises the aggregate rate only 1.4 times. With 8 products and
// 1.25 commits per 32-row k-block the handshakes and issues alone take ~0.45 us per k-block, at any
// ring depth. Measured and without effect on the step time: a ring of raw tiles of its own ahead of
// the re-laid ones (7 loads in flight), collecting warps that do nothing else, the reduction spread
// over four TMEM accumulators (independent chains), 16 split warps, spinning on test_wait.
struct BgParams {
  int nkb;                 // K / 32
  int causal;
  float alpha;
  int H;
  int ax[2], ay[2], bx[2], by[2], cx[2], cy[2];
  int x3;                  // three products (f32-class accuracy) or one
  int pair_m;              // 0, or the number of M tiles when each CTA takes tiles y and (tiles - 1 - y)
  int* err;
};

template <int BN, bool TA, bool TB, int STAGES>
struct BgSmem {
  static constexpr int kA = BM * BK * 4, kB = BN * BK * 4;
  static constexpr int kARegion = kA * (TA ? 3 : 2);       // raw [, hi], lo
  static constexpr int kBRegion = kB * (TB ? 3 : 2);
  static constexpr int kStage = kARegion + kBRegion;
  static constexpr int kBarBytes = 256;
  static constexpr int kTotal = STAGES * kStage + kBarBytes + 1024;
};

__device__ __forceinline__ float lo_part(float v) { return v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }

// raw: f32 tile in the swizzled K-major layout the MMA reads; lo gets the same layout.
__device__ __forceinline__ void split_plain(const uint8_t* raw, uint8_t* lo, int bytes, int t) {
  const float4* r = reinterpret_cast<const float4*>(raw);
  float4* l = reinterpret_cast<float4*>(lo);
#pragma unroll 4
  for (int i = t; i < bytes / 16; i += kBgWorkers) {
    const float4 v = r[i];
    l[i] = make_float4(lo_part(v.x), lo_part(v.y), lo_part(v.z), lo_part(v.w));
  }
}
// raw: [32][W] f32, reduction index on rows. hi / lo: W rows of 128 bytes (K-major), 16-byte
// chunk c of row n stored at chunk (c ^ (n & 7)) - the 128-byte swizzle. Lanes walk n, so the
// reads are conflict-free and each quarter-warp's 128-bit stores cover all 32 banks.
// NW threads share the tile; all of a thread's loads are issued before its first store (these warps are
// bound by the latency of their own instruction stream, not by shared-memory bandwidth).
template <int W, int NW = kBgWorkers>
__device__ __forceinline__ void split_transposed(const uint8_t* raw, uint8_t* hi, uint8_t* lo, int t) {
  const float* r = reinterpret_cast<const float*>(raw);
  constexpr int kIter = (W * 8 + NW - 1) / NW;
  float v[kIter][4];
#pragma unroll
  for (int u = 0; u < kIter; ++u) {
    const int i = t + u * NW, n = i % W, k4 = i / W;
    if (W * 8 % NW == 0 || i < W * 8) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[u][j] = r[(4 * k4 + j) * W + n];
    }
  }
#pragma unroll
  for (int u = 0; u < kIter; ++u) {
    const int i = t + u * NW, n = i % W, k4 = i / W;
    if (W * 8 % NW == 0 || i < W * 8) {
      const int off = n * 128 + ((k4 ^ (n & 7)) << 4);
      *reinterpret_cast<float4*>(hi + off) = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
      *reinterpret_cast<float4*>(lo + off) =
          make_float4(lo_part(v[u][0]), lo_part(v[u][1]), lo_part(v[u][2]), lo_part(v[u][3]));
    }
  }
}

template <int BN, bool TA, bool TB, int STAGES>
__global__ void __launch_bounds__(kThreadsTC)
bgemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                const __grid_constant__ CUtensorMap mapC, BgParams p) {
  using S = BgSmem<BN, TA, TB, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + STAGES * S::kStage;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_split = [&](int s) { return bars + 8u * (STAGES + s); };
  auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };
  auto bar_acc_full = [&](int b) { return bars + 8u * (3 * STAGES + b); };
  auto bar_acc_empty = [&](int b) { return bars + 8u * (3 * STAGES + 2 + b); };
  const uint32_t bar_epi = bars + 8u * (3 * STAGES + 4);       // first tile's store staging has been read
  const uint32_t tmem_slot = bars + 8u * (3 * STAGES + 5);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + STAGES * S::kStage + 8 * (3 * STAGES + 5));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int bi = blockIdx.z / p.H, hd = blockIdx.z % p.H;
  // A CTA owns one M tile, or - for the causal reductions, whose length grows with the tile index -
  // the tiles y and (tiles - 1 - y): equal work per CTA, and the second tile's loads run under the
  // first tile's epilogue. The stage ring and the chunk counter run on across the two tiles.
  const int ntile = p.pair_m ? 2 : 1;
  auto tile_of = [&](int ti, int& m0, int& kb_begin, int& nk) {
    const int mt = ti == 0 ? (int)blockIdx.y : p.pair_m - 1 - (int)blockIdx.y;
    m0 = mt * BM;
    kb_begin = 0;
    int kb_end = p.nkb;
    if (p.causal == 1 && n0 > m0 + BM - 1) kb_end = 0;
    if (p.causal == 2) kb_end = min(kb_end, (m0 + BM) / BK);
    if (p.causal == 3) kb_begin = min(kb_end, m0 / BK);
    nk = kb_end - kb_begin;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_split(s), kBgWorkers / 32);      // one arrival per split warp
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 4);
    }
    mbar_init(bar_epi, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // 3xTF32 with the hi and lo tiles of B adjacent in shared memory: one MMA of width 2*BN
  // multiplies A_hi with [B_hi; B_lo] (columns [0,BN) and [BN,2BN) of the accumulator), a second
  // of width BN adds A_lo.B_hi into the first half; the halves are summed when a chunk is
  // collected. Two MMAs per step instead of three - their cost does not depend on the width.
  constexpr int kAccCols = 2 * BN;                 // per accumulator
  constexpr uint32_t kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;   // two accumulators, chunks alternate
  constexpr int LD = BN >= 32 ? 32 : 16;       // columns per TMEM load / store box
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  auto a_raw = [&](int s) { return (uint32_t)(s * S::kStage); };
  auto a_hi = [&](int s) { return (uint32_t)(s * S::kStage + (TA ? S::kA : 0)); };
  auto a_lo = [&](int s) { return (uint32_t)(s * S::kStage + (TA ? 2 : 1) * S::kA); };
  auto b_raw = [&](int s) { return (uint32_t)(s * S::kStage + S::kARegion); };
  auto b_hi = [&](int s) { return (uint32_t)(s * S::kStage + S::kARegion + (TB ? S::kB : 0)); };
  auto b_lo = [&](int s) { return (uint32_t)(s * S::kStage + S::kARegion + (TB ? 2 : 1) * S::kB); };

  if (warp == 0) {
    if (lane == 0) {
      const int ax0 = bi * p.ax[0] + hd * p.ax[1], ay0 = bi * p.ay[0] + hd * p.ay[1];
      const int bx0 = bi * p.bx[0] + hd * p.bx[1], by0 = bi * p.by[0] + hd * p.by[1];
      int it = 0, epi_stage = -1;       // epi_stage: the stage the first tile's epilogue stages its stores in
      bool ok = true;
      for (int ti = 0; ti < ntile && ok; ++ti) {
        int m0, kb_begin, nk;
        tile_of(ti, m0, kb_begin, nk);
        for (int i = 0; i < nk && ok; ++i, ++it) {
          const int s = it % STAGES, r = it / STAGES, k0 = (kb_begin + i) * BK;
          if (r > 0) ok = mbar_wait(bar_empty(s), (r - 1) & 1, p.err, 11);
          if (ok && s == epi_stage) {
            ok = mbar_wait(bar_epi, 0, p.err, 17);
            epi_stage = -1;
          }
          if (!ok) break;
          mbar_expect_tx(bar_full(s), S::kA + S::kB);
          if (TA) tma_load_2d(base + a_raw(s), &mapA, bar_full(s), ax0 + m0, ay0 + k0);
          else tma_load_2d(base + a_raw(s), &mapA, bar_full(s), ax0 + k0, ay0 + m0);
          if (TB) tma_load_2d(base + b_raw(s), &mapB, bar_full(s), bx0 + n0, by0 + k0);
          else tma_load_2d(base + b_raw(s), &mapB, bar_full(s), bx0 + k0, by0 + n0);
        }
        if (ti == 0 && ntile == 2 && it > 0) epi_stage = (it - 1) % STAGES;
      }
      if (!ok) {
        for (int i = (it > STAGES ? it - STAGES : 0); i < it; ++i)
          mbar_wait(bar_full(i % STAGES), (i / STAGES) & 1, p.err, 15);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_tf32(BM, BN), idesc2 = idesc_tf32(BM, 2 * BN);
      bool ok = true;
      int it = 0, ci = 0;               // k-blocks and accumulation chunks issued so far, over both tiles
      for (int ti = 0; ti < ntile && ok; ++ti) {
      int m0, kb_begin, nk;
      tile_of(ti, m0, kb_begin, nk);
      for (int i = 0; i < nk; ++i, ++it) {
        const int s = it % STAGES, r = it / STAGES;
        const int buf = ci & 1;
        if (i % kChunk == 0 && ci >= 2) {
          ok = mbar_wait(bar_acc_empty(buf), ((ci >> 1) - 1) & 1, p.err, 16);
          if (!ok) break;
          tc_fence_after();
        }
        ok = mbar_wait(bar_split(s), r & 1, p.err, 12);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kAccCols;
#pragma unroll
        for (int kk = 0; kk < BK / 8; ++kk) {
          const uint64_t da = smem_desc_sw128(base + a_hi(s) + kk * 32), db = smem_desc_sw128(base + b_hi(s) + kk * 32);
          if (p.x3) {
            mma_tf32(tmem_d, da, db, idesc2, ((i % kChunk) | kk) != 0);      // b_lo follows b_hi in the stage
            mma_tf32(tmem_d, smem_desc_sw128(base + a_lo(s) + kk * 32), db, idesc, 1);
          } else {
            mma_tf32(tmem_d, da, db, idesc, ((i % kChunk) | kk) != 0);
          }
        }
        mma_commit(bar_empty(s));
        if (i % kChunk == kChunk - 1 || i == nk - 1) {
          mma_commit(bar_acc_full(buf));
          ++ci;
        }
      }
      }
    }
  } else {
    const int t = threadIdx.x - 64;
    const int q = warp & 3, row0 = q * 32;
    bool ok = true;
    // finished chunks are added into f32 registers while the next chunk is multiplied (the
    // tensor core's own accumulation truncates; see gemm_tc_kernel)
    float acc[BN];
    int it = 0, cg = 0;                             // k-blocks split / chunks collected so far, over both tiles
    const bool collector = warp < 6;               // warps 2..5: one per TMEM lane quadrant
    auto collect = [&](int ci) {
      if (!collector) return true;
      const int buf = ci & 1;
      if (!mbar_wait(bar_acc_full(buf), (ci >> 1) & 1, p.err, 14)) return false;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < BN / LD; ++c) {
        uint32_t r[32];
        tmem_ld_cols<LD>(tmem_base + ((uint32_t)row0 << 16) + buf * kAccCols + c * LD, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < LD; ++j) acc[c * LD + j] += __uint_as_float(r[j]);
        if (p.x3) {
          tmem_ld_cols<LD>(tmem_base + ((uint32_t)row0 << 16) + buf * kAccCols + BN + c * LD, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < LD; ++j) acc[c * LD + j] += __uint_as_float(r[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(buf));
      return true;
    };
    for (int ti = 0; ti < ntile && ok; ++ti) {
    int m0, kb_begin, nk;
    tile_of(ti, m0, kb_begin, nk);
    (void)kb_begin;
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.0f;
    const int nchunks = (nk + kChunk - 1) / kChunk;
    int collected = 0;
    for (int i = 0; i < nk && ok; ++i, ++it) {
      const int s = it % STAGES, r = it / STAGES;
      ok = mbar_wait(bar_full(s), r & 1, p.err, 13);
      if (!ok) break;
      if (TA) split_transposed<BM>(base_ptr + a_raw(s), base_ptr + a_hi(s), base_ptr + a_lo(s), t);
      else split_plain(base_ptr + a_raw(s), base_ptr + a_lo(s), S::kA, t);
      if (TB) split_transposed<BN>(base_ptr + b_raw(s), base_ptr + b_hi(s), base_ptr + b_lo(s), t);
      else split_plain(base_ptr + b_raw(s), base_ptr + b_lo(s), S::kB, t);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_split(s));
      if (i % kChunk == 1 && i > kChunk) {
        ok = collect(cg);
        ++cg;
        ++collected;
      }
    }
    for (; ok && collected < nchunks; ++collected, ++cg) ok = collect(cg);
    if (ok && collector) {
      // every product of this tile has retired: the stage of its last k-block is the one the
      // producer refills last, so it serves as store staging (the producer waits for bar_epi
      // before it loads into that stage again)
      const uint32_t soff = (uint32_t)((it > 0 ? (it - 1) % STAGES : 0) * S::kStage) + q * 4096;
      const uint32_t stage = base + soff;
      uint8_t* stage_ptr = base_ptr + soff;
      const int cx0 = bi * p.cx[0] + hd * p.cx[1], cy0 = bi * p.cy[0] + hd * p.cy[1];
      const int m = m0 + row0 + lane;
      for (int c = 0; c < BN / LD; ++c) {
        const int ncol = n0 + c * LD;
        uint32_t r[32];
#pragma unroll
        for (int j = 0; j < LD; ++j) {
          float v = p.alpha * acc[c * LD + j];          // empty reduction ranges leave exact zeros
          if (p.causal == 1 && ncol + j > m) v = 0.0f;
          r[j] = __float_as_uint(v);
        }
        if (c > 0) {
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
        }
#pragma unroll
        for (int j = 0; j < LD / 4; ++j) {
          uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          *reinterpret_cast<uint4*>(stage_ptr + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&mapC, stage, cx0 + ncol, cy0 + m0 + row0);
          tma_store_commit();
        }
      }
      if (lane == 0) {
        if (ti + 1 < ntile) {
          tma_store_wait_read();
          mbar_arrive(bar_epi);
        } else {
          tma_store_wait_all();
        }
      }
      __syncwarp();
    }
    }
    if (collector && lane == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------ CTA-pair GEMM (cta_group::2, 3xTF32 only)
// Two CTAs of a cluster (consecutive 128-row tiles of M) share one 256 x 256 output tile: each
// stages its own 128 rows of A and HALF of the B tile (128 of the 256 rows of B^T), and the
// even CTA issues tcgen05.mma.cta_group::2 with M = 256 - the hardware reads A and the B halves
// from both CTAs' shared memory and leaves 128 x 256 accumulators in each CTA's TMEM. Per SM
// that is 8 KB of operand reads per MMA instead of 12 KB and half the B staging, which lifts
// the shared-memory bound of the single-CTA kernel; the smaller stages also allow three.
//
// Protocol: loads complete on each CTA's own barrier; the worker warps of BOTH CTAs arrive on
// the even CTA's "split" barrier once their tiles are split; the even CTA's MMA thread waits on
// that, issues, and commits with a multicast arrive to both CTAs' "empty" (stage reusable) and
// "accumulator full" barriers; collectors of both CTAs arrive on the even CTA's "accumulator
// empty" barrier. TMEM is allocated / freed by warp 1 of both CTAs (cta_group::2 forms). A cluster
// barrier after the barrier initialisation and one before exit keep remote arrivals and the
// peer's operand reads inside the lifetime of both CTAs. Every mbarrier wait is bounded.
// Three 32-wide stages. Measured alternatives that were slower: six 16-wide stages (the per-stage
// signalling cost doubles), issuing the products that need no lo tile of A ahead of the split
// on a separate "landed" barrier (an extra cross-CTA wait per stage), and L2 prefetch of the
// tiles ahead of the ring (the load latency is not an L2-miss latency).
constexpr int kPairKB = 32;
constexpr int kPairStages = 3;
struct PairSmem {
  static constexpr int kA = BM * kPairKB * 4, kBh = 128 * kPairKB * 4;   // A tile, half B tile: 8 KiB each
  static constexpr int kStage = 2 * kA + 2 * kBh;                // [A raw][A lo][B raw][B lo]
  static constexpr int kTotal = kPairStages * kStage + 256 + 1024;
};

__global__ void __launch_bounds__(kThreadsV2, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                    const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapA2,
                    const __grid_constant__ CUtensorMap mapB2, const __grid_constant__ CUtensorMap mapBlo,
                    TcParams p) {
  using S = PairSmem;
  constexpr int STAGES = kPairStages, BN = 256, KB = kPairKB;
  constexpr int kChunkBlocks = kChunk * (BK / KB);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + STAGES * S::kStage;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_split = [&](int s) { return bars + 8u * (STAGES + s); };
  auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };
  auto bar_acc_full = [&](int b) { return bars + 8u * (3 * STAGES + b); };
  auto bar_acc_empty = [&](int b) { return bars + 8u * (3 * STAGES + 2 + b); };
  const uint32_t bar_epi = bars + 8u * (3 * STAGES + 4);     // this CTA's store staging of a tile has been read
  const uint32_t tmem_slot = bars + 8u * (3 * STAGES + 5);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + STAGES * S::kStage + 8 * (3 * STAGES + 5));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: issues the MMAs; 1: its peer
  // Persistent clusters (one per SM pair, laid along x): cluster c takes tiles c, c + clusters, ...
  // in an order with the N tile fastest, so the clusters in flight share their rows of A and walk
  // the (small, L2-resident) weight. The stage ring, the accumulation-chunk counter and the
  // barriers' phases run on across tiles: the next tile's loads are in flight, and its MMAs can
  // start, while the workers store the finished tile from registers.
  const int cid = (int)(blockIdx.x >> 1), ncl = (int)(gridDim.x >> 1);
  auto tile_of = [&](int t, int& m0, int& n0) {
    n0 = (t % p.n_tiles) * BN;
    m0 = (2 * (t / p.n_tiles) + (int)rank) * BM;
  };
  const int nkb1 = (p.K + KB - 1) / KB;
  const int nkb = nkb1 + (p.K2 + KB - 1) / KB;
  const int nchunks = (nkb + kChunkBlocks - 1) / kChunkBlocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_split(s), 2 * kWorkers / 32); // one arrival per worker warp of both CTAs (used in the even CTA)
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 2 * kWorkers / 32);  // one per collector warp of both CTAs (used in the even CTA)
    }
    mbar_init(bar_epi, kWorkers / 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                               // the peer's barriers exist before anyone arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ---- TMA producer (each CTA loads its own tiles onto its own barrier) -------------------
    if (lane == 0) {
      int it = 0, ti = 0, pend = -1, epi_stage = -1;   // pend: tile whose store staging may still be in use
      bool ok = true;
      for (int tl = cid; tl < p.total_tiles && ok; tl += ncl, ++ti) {
        int m0, n0;
        tile_of(tl, m0, n0);
        const int nb = n0 + (int)rank * 128;        // this CTA's half of the B tile
        for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
          const int s = it % STAGES, r = it / STAGES;
          if (r > 0) ok = mbar_wait(bar_empty(s), (r - 1) & 1, p.err, 31);
          if (ok && pend >= 0 && s == epi_stage) {  // the previous tile's epilogue staged its stores here
            ok = mbar_wait(bar_epi, pend & 1, p.err, 38);
            pend = -1;
          }
          if (!ok) break;
          const uint32_t a_dst = base + s * S::kStage, b_dst = a_dst + 2 * S::kA;
          const bool lo_too = p.b_lo && kb < nkb1;
          mbar_expect_tx(bar_full(s), S::kA + S::kBh + (lo_too ? S::kBh : 0));
          if (kb < nkb1) {
            tma_load_2d(a_dst, &mapA, bar_full(s), kb * KB, m0);
            tma_load_2d(b_dst, &mapB, bar_full(s), kb * KB, nb);
            if (lo_too) tma_load_2d(b_dst + S::kBh, &mapBlo, bar_full(s), kb * KB, nb);
          } else {
            tma_load_2d(a_dst, &mapA2, bar_full(s), (kb - nkb1) * KB, m0);
            tma_load_2d(b_dst, &mapB2, bar_full(s), (kb - nkb1) * KB, nb);
          }
        }
        if (ok && pend >= 0) {                      // short tiles: take the phase anyway, in order
          ok = mbar_wait(bar_epi, pend & 1, p.err, 38);
          pend = -1;
        }
        pend = ti;
        epi_stage = (it - 1) % STAGES;
      }
      if (!ok) {
        for (int kb = (it > STAGES ? it - STAGES : 0); kb < it; ++kb)
          mbar_wait(bar_full(kb % STAGES), (kb / STAGES) & 1, p.err, 35);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the even CTA only --------------------------------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_tf32(256, BN);
      bool ok = true;
      int it = 0, ci = 0;
      for (int tl = cid; tl < p.total_tiles && ok; tl += ncl)
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % STAGES, r = it / STAGES;
        const int buf = ci & 1;
        if (kb % kChunkBlocks == 0 && ci >= 2) {
          ok = mbar_wait(bar_acc_empty(buf), ((ci >> 1) - 1) & 1, p.err, 36);
          if (!ok) break;
          tc_fence_after();
        }
        ok = mbar_wait(bar_split(s), r & 1, p.err, 32);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        const uint32_t a_raw = base + s * S::kStage, a_lo = a_raw + S::kA;
        const uint32_t b_raw = a_raw + 2 * S::kA, b_lo = b_raw + S::kBh;
#pragma unroll
        for (int kk = 0; kk < KB / 8; ++kk) {
          const uint64_t da = smem_desc_k<KB>(a_raw + kk * 32), db = smem_desc_k<KB>(b_raw + kk * 32);
          mma_tf32_pair(tmem_d, da, db, idesc, ((kb % kChunkBlocks) | kk) != 0);
          mma_tf32_pair(tmem_d, smem_desc_k<KB>(a_lo + kk * 32), db, idesc, 1);
          mma_tf32_pair(tmem_d, da, smem_desc_k<KB>(b_lo + kk * 32), idesc, 1);
        }
        mma_commit_pair(bar_empty(s));
        if (kb % kChunkBlocks == kChunkBlocks - 1 || kb == nkb - 1) {
          mma_commit_pair(bar_acc_full(buf));
          ++ci;
        }
      }
    }
  } else {
    // ---- worker warps (both CTAs): split, collect finished chunks, epilogue -------------------
    const int t = threadIdx.x - 64;
    const int q = warp & 3, half = (warp - 2) >> 2, row0 = q * 32;
    constexpr int NH = BN / 2, LD = 32;
    float acc[NH];
    bool ok = true;
    int it = 0, cg = 0;
    auto collect = [&](int ci) {
      const int buf = ci & 1;
      if (!mbar_wait(bar_acc_full(buf), (ci >> 1) & 1, p.err, 34)) return false;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < NH / LD; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)row0 << 16) + buf * BN + half * NH + c * LD, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < LD; ++j) acc[c * LD + j] += __uint_as_float(r[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(bar_acc_empty(buf), 0);     // remote arrivals are slow: one per warp
      return true;
    };
    auto split_range = [&](uint8_t* raw, int bytes) {
      const float4* rp = reinterpret_cast<const float4*>(raw);
      float4* lp = reinterpret_cast<float4*>(raw + bytes);
#pragma unroll 4
      for (int i = t; i < bytes / 16; i += kWorkers) {
        const float4 v = rp[i];
        lp[i] = make_float4(lo_part(v.x), lo_part(v.y), lo_part(v.z), lo_part(v.w));
      }
    };
    for (int tl = cid; tl < p.total_tiles && ok; tl += ncl) {
    int m0, n0;
    tile_of(tl, m0, n0);
#pragma unroll
    for (int j = 0; j < NH; ++j) acc[j] = 0.0f;
    int collected = 0;
    for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
      const int s = it % STAGES, r = it / STAGES;
      ok = mbar_wait(bar_full(s), r & 1, p.err, 33);
      if (!ok) break;
      uint8_t* stg = base_ptr + s * S::kStage;
      split_range(stg, S::kA);
      if (!(p.b_lo && kb < nkb1)) split_range(stg + 2 * S::kA, S::kBh);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(bar_split(s), 0);
      if (kb % kChunkBlocks == 1 && kb > kChunkBlocks) {
        ok = collect(cg);
        ++cg;
        ++collected;
      }
    }
    for (; ok && collected < nchunks; ++collected, ++cg) ok = collect(cg);
    if (!ok) break;
    // every product of the tile has retired; the stage of its last k-block is the one the producer
    // refills last, so it holds the store staging (one 32x32 box per warp, reused chunk by chunk)
    const uint32_t box = (uint32_t)(((it - 1) % STAGES) * S::kStage + (warp - 2) * 4096);
    if (m0 + row0 < p.M) {
      bool stored = false;
#pragma unroll
      for (int c = 0; c < NH / LD; ++c) {
        const int ncol = n0 + half * NH + c * LD;
        if (ncol < p.N) {
          uint8_t* stage_ptr = base_ptr + box;
          if (stored) {
            if (lane == 0) tma_store_wait_read();
            __syncwarp();
          }
          stored = true;
          uint32_t r[32];
#pragma unroll
          for (int j = 0; j < LD; ++j) r[j] = __float_as_uint(p.alpha * acc[c * LD + j]);
          if (p.addend != nullptr && m0 + row0 + lane < p.M) {
            const float* arow = p.addend + (size_t)(m0 + row0 + lane) * p.N + ncol;
#pragma unroll
            for (int j4 = 0; j4 < LD / 4; ++j4) {
              if (ncol + 4 * j4 < p.N) {
                const float4 d = *reinterpret_cast<const float4*>(arow + 4 * j4);
                r[4 * j4 + 0] = __float_as_uint(d.x + __uint_as_float(r[4 * j4 + 0]));
                r[4 * j4 + 1] = __float_as_uint(d.y + __uint_as_float(r[4 * j4 + 1]));
                r[4 * j4 + 2] = __float_as_uint(d.z + __uint_as_float(r[4 * j4 + 2]));
                r[4 * j4 + 3] = __float_as_uint(d.w + __uint_as_float(r[4 * j4 + 3]));
              }
            }
          }
          if (p.bias != nullptr || p.act != 0) {
#pragma unroll
            for (int j = 0; j < LD; ++j) {
              float v = __uint_as_float(r[j]);
              if (p.bias != nullptr && ncol + j < p.N) v = v + p.bias[ncol + j];
              r[j] = __float_as_uint(epi_act(p.act, v));
            }
          }
#pragma unroll
          for (int j = 0; j < LD / 4; ++j) {
            uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            *reinterpret_cast<uint4*>(stage_ptr + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&mapC, base + box, ncol, m0 + row0);
            tma_store_commit();
          }
        }
      }
    }
    if (lane == 0) {
      tma_store_wait_read();                          // the staging may be overwritten by the next tile's loads
      mbar_arrive(bar_epi);
    }
    __syncwarp();
    }
    if (lane == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                               // nobody leaves while the peer may still touch this CTA
  if (warp == 1) tmem_dealloc2(tmem_base, 512);
}


// ----------------------------------------- CTA-pair GEMM, two-term fp16 split (F16X2)
// The same 256 x 256 cluster tile, stage ring, chunked accumulation and epilogue as
// gemm_tc_pair_kernel, with a different arithmetic: every f32 operand x is scaled by a power of
// two s (chosen per tensor so that max|x| * s lies in [2^13, 2^14)) and cut into two fp16 terms,
// hi = fp16(x s) and lo = fp16(x s - hi). a.b ~ (hi.hi + lo.hi + hi.lo) / (sa sb): the same 22
// significant bits as the three-product tf32 split (the dropped lo.lo term is 2^-22 relative), but
// kind::f16 multiplies at twice the tf32 rate and its tiles are half as wide in shared memory.
// The power-of-two scale keeps fp16's narrow exponent range out of the result: after scaling, an
// element is held to max(2^-22 |x s|, 2^-25), i.e. to 2^-39 of the tensor's largest magnitude at
// worst. The scale is undone (exactly) when a finished chunk is added into the f32 registers, so
// the main product and the low-rank tail - which have different scales - ride the same
// accumulators as separate chunks.
// A frozen B operand comes pre-split (fp16 hi / lo copies made when the program is built, loaded
// by TMA with the 64-byte swizzle); every other operand is loaded as f32 and converted by the
// worker warps. max|x| of the run-time operands is measured by absmax4_kernel just before.
constexpr int kF16Raw = BM * 32 * 4;       // a 128 x 32 f32 tile
constexpr int kF16Half = BM * 32 * 2;      // the same tile in fp16: 64-byte rows
constexpr int kF16Stages = 4;
struct PairF16Smem {
  static constexpr int kARaw = 0, kAHi = kF16Raw, kALo = kAHi + kF16Half, kBHi = kALo + kF16Half,
                       kBLo = kBHi + kF16Half;
  static constexpr int kStage = kBLo + kF16Half;                   // 48 KiB
  static constexpr int kTotal = kF16Stages * kStage + 256 + 1024;
};
struct F16Params {
  int M, N, K, K2;
  const float* bias;
  const float* addend;
  int act;
  float alpha;
  int eb_pre;               // scale exponent of the frozen B copies: they hold the split of w * 2^eb_pre
  const uint32_t* absmax;   // device: bit patterns of max|x| over A, -, A2, B2
  int dbg;                  // measurement switches (0 in production): 1 = workers skip the conversion, 2 = one product
  int n_tiles, total_tiles;
  int* err;
};

// Scale exponent e for a tensor whose largest magnitude has these bits: max * 2^e in [2^13, 2^14).
// Zero, subnormal and non-finite maxima get no scaling.
__host__ __device__ __forceinline__ int f16_scale_exp(uint32_t bits) {
  const int ex = (int)((bits >> 23) & 0xFFu);
  if (ex == 0 || ex == 0xFF) return 0;
  const int e = 13 - (ex - 127);
  return e < -120 ? -120 : (e > 120 ? 120 : e);
}
__device__ __forceinline__ float pow2i(int e) { return __int_as_float((e + 127) << 23); }

// hi = x rounded to 11 significant bits (what an fp16 keeps), by Veltkamp's splitting with plain
// f32 arithmetic, and lo = x - hi (exact). Both then convert to fp16 two at a time. For |x| below
// fp16's normal range (2^-14) the conversion of hi rounds once more, by at most 2^-25.
__device__ __forceinline__ void split11(float x, float& hi, float& lo) {
  const float t = __fmul_rn(x, 8193.0f);          // 2^13 + 1
  hi = __fsub_rn(t, __fsub_rn(t, x));
  lo = __fsub_rn(x, hi);
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// 128 rows x 32 f32 in the 128-byte swizzled layout of a TMA load -> the hi and lo fp16 tiles,
// 64-byte rows in the 64-byte swizzled K-major layout the MMA reads.
__device__ __forceinline__ void split_f16_tile(const uint8_t* raw, uint8_t* hi, uint8_t* lo, float sc, int t) {
#pragma unroll
  for (int i = t; i < kF16Raw / 16; i += kWorkers) {
    const int row = i >> 3, c = (i & 7) ^ (row & 7);          // logical 16-byte chunk: k = 4c .. 4c+3
    const float4 v = reinterpret_cast<const float4*>(raw)[i];
    // hi by truncation to 11 significant bits (two instructions; the one-time weight split rounds
    // instead): lo = x - hi is exact and below 2^-10 |x|, so hi + fp16(lo) still carries 21 bits
    const float x0 = v.x * sc, x1 = v.y * sc, x2 = v.z * sc, x3 = v.w * sc;
    const float h0 = __uint_as_float(__float_as_uint(x0) & 0xFFFFE000u), h1 = __uint_as_float(__float_as_uint(x1) & 0xFFFFE000u);
    const float h2 = __uint_as_float(__float_as_uint(x2) & 0xFFFFE000u), h3 = __uint_as_float(__float_as_uint(x3) & 0xFFFFE000u);
    const float l0 = x0 - h0, l1 = x1 - h1, l2 = x2 - h2, l3 = x3 - h3;
    const int off = row * 64 + ((((c >> 1) ^ (row >> 1)) & 3) << 4) + ((c & 1) << 3);
    *reinterpret_cast<uint2*>(hi + off) = make_uint2(pack_h2(h0, h1), pack_h2(h2, h3));
    *reinterpret_cast<uint2*>(lo + off) = make_uint2(pack_h2(l0, l1), pack_h2(l2, l3));
  }
}

__global__ void __launch_bounds__(kThreadsV2, 1)
gemm_tc_pair_f16_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapA2,
                        const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapBhi,
                        const __grid_constant__ CUtensorMap mapBlo, const __grid_constant__ CUtensorMap mapB2hi,
                        const __grid_constant__ CUtensorMap mapB2lo, F16Params p) {
  using S = PairF16Smem;
  constexpr int STAGES = kF16Stages, BN = 256, KB = 32;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + STAGES * S::kStage;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_split = [&](int s) { return bars + 8u * (STAGES + s); };
  auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };
  auto bar_acc_full = [&](int b) { return bars + 8u * (3 * STAGES + b); };
  auto bar_acc_empty = [&](int b) { return bars + 8u * (3 * STAGES + 2 + b); };
  const uint32_t bar_epi = bars + 8u * (3 * STAGES + 4);
  const uint32_t tmem_slot = bars + 8u * (3 * STAGES + 5);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + STAGES * S::kStage + 8 * (3 * STAGES + 5));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cid = (int)(blockIdx.x >> 1), ncl = (int)(gridDim.x >> 1);
  auto tile_of = [&](int t, int& m0, int& n0) {
    n0 = (t % p.n_tiles) * BN;
    m0 = (2 * (t / p.n_tiles) + (int)rank) * BM;
  };
  // k-blocks of the main pair, then of the low-rank pair; accumulation chunks of up to kChunk
  // blocks never straddle the two (their scales differ)
  const int nkb1 = (p.K + KB - 1) / KB;
  const int nkb = nkb1 + (p.K2 + KB - 1) / KB;
  const int nmain = (nkb1 + kChunk - 1) / kChunk;
  const int nchunks = nmain + (nkb - nkb1 + kChunk - 1) / kChunk;
  auto chunk_pos = [&](int kb, int& c, int& j, bool& last) {
    if (kb < nkb1) { c = kb / kChunk; j = kb % kChunk; last = j == kChunk - 1 || kb == nkb1 - 1; }
    else { const int q = kb - nkb1; c = nmain + q / kChunk; j = q % kChunk; last = j == kChunk - 1 || kb == nkb - 1; }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_split(s), 2 * kWorkers / 32);
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 2 * kWorkers / 32);
    }
    mbar_init(bar_epi, kWorkers / 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ---- TMA producer ---------------------------------------------------------------------
    if (lane == 0) {
      int it = 0, ti = 0, pend = -1, epi_stage = -1;
      bool ok = true;
      for (int tl = cid; tl < p.total_tiles && ok; tl += ncl, ++ti) {
        int m0, n0;
        tile_of(tl, m0, n0);
        const int nb = n0 + (int)rank * 128;
        for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
          const int s = it % STAGES, r = it / STAGES;
          if (r > 0) ok = mbar_wait(bar_empty(s), (r - 1) & 1, p.err, 41);
          if (ok && pend >= 0 && s == epi_stage) {
            ok = mbar_wait(bar_epi, pend & 1, p.err, 48);
            pend = -1;
          }
          if (!ok) break;
          const uint32_t stg = base + s * S::kStage;
          mbar_expect_tx(bar_full(s), kF16Raw + 2 * kF16Half);          // A raw + B hi + B lo
          if (kb < nkb1) {
            tma_load_2d(stg + S::kARaw, &mapA, bar_full(s), kb * KB, m0);
            tma_load_2d(stg + S::kBHi, &mapBhi, bar_full(s), kb * KB, nb);
            tma_load_2d(stg + S::kBLo, &mapBlo, bar_full(s), kb * KB, nb);
          } else {
            tma_load_2d(stg + S::kARaw, &mapA2, bar_full(s), (kb - nkb1) * KB, m0);
            tma_load_2d(stg + S::kBHi, &mapB2hi, bar_full(s), (kb - nkb1) * KB, nb);
            tma_load_2d(stg + S::kBLo, &mapB2lo, bar_full(s), (kb - nkb1) * KB, nb);
          }
        }
        if (ok && pend >= 0) {
          ok = mbar_wait(bar_epi, pend & 1, p.err, 48);
          pend = -1;
        }
        pend = ti;
        epi_stage = (it - 1) % STAGES;
      }
      if (!ok) {
        for (int kb = (it > STAGES ? it - STAGES : 0); kb < it; ++kb)
          mbar_wait(bar_full(kb % STAGES), (kb / STAGES) & 1, p.err, 45);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the even CTA only --------------------------------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_f16(256, BN);
      bool ok = true;
      int it = 0, ci = 0;
      for (int tl = cid; tl < p.total_tiles && ok; tl += ncl)
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % STAGES, r = it / STAGES;
        const int buf = ci & 1;
        int c, j;
        bool last;
        chunk_pos(kb, c, j, last);
        if (j == 0 && ci >= 2) {
          ok = mbar_wait(bar_acc_empty(buf), ((ci >> 1) - 1) & 1, p.err, 46);
          if (!ok) break;
          tc_fence_after();
        }
        ok = mbar_wait(bar_split(s), r & 1, p.err, 42);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        const uint32_t stg = base + s * S::kStage;
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {       // 16 fp16 of K (32 bytes) per instruction
          const uint64_t da = smem_desc_sw64(stg + S::kAHi + kk * 32), dal = smem_desc_sw64(stg + S::kALo + kk * 32);
          const uint64_t db = smem_desc_sw64(stg + S::kBHi + kk * 32), dbl = smem_desc_sw64(stg + S::kBLo + kk * 32);
          mma_f16_pair(tmem_d, da, db, idesc, (j | kk) != 0);
          if (!(p.dbg & 2)) {
            mma_f16_pair(tmem_d, dal, db, idesc, 1);
            mma_f16_pair(tmem_d, da, dbl, idesc, 1);
          }
        }
        mma_commit_pair(bar_empty(s));
        if (last) {
          mma_commit_pair(bar_acc_full(buf));
          ++ci;
        }
      }
    }
  } else {
    // ---- worker warps (both CTAs): convert, collect finished chunks, epilogue -----------------
    const int t = threadIdx.x - 64;
    const int q = warp & 3, half = (warp - 2) >> 2, row0 = q * 32;
    constexpr int NH = BN / 2, LD = 32;
    const int ea = f16_scale_exp(p.absmax[0]), eb = p.eb_pre;
    const int ea2 = f16_scale_exp(p.absmax[2]), eb2 = f16_scale_exp(p.absmax[3]);
    const float sa = pow2i(ea), sa2 = pow2i(ea2);
    const float cs_main = pow2i(-ea) * pow2i(-eb), cs_tail = pow2i(-ea2) * pow2i(-eb2);
    float acc[NH];
    bool ok = true;
    int it = 0, cg = 0;
    auto collect = [&](int ci, float cs) {
      const int buf = ci & 1;
      if (!mbar_wait(bar_acc_full(buf), (ci >> 1) & 1, p.err, 44)) return false;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < NH / LD; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)row0 << 16) + buf * BN + half * NH + c * LD, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < LD; ++j) acc[c * LD + j] += __uint_as_float(r[j]) * cs;   // cs is a power of two: exact
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(bar_acc_empty(buf), 0);
      return true;
    };
    for (int tl = cid; tl < p.total_tiles && ok; tl += ncl) {
    int m0, n0;
    tile_of(tl, m0, n0);
#pragma unroll
    for (int j = 0; j < NH; ++j) acc[j] = 0.0f;
    int collected = 0;
    auto collect_to = [&](int upto) {          // collect this tile's chunks [collected, upto)
      for (; ok && collected < upto; ++collected, ++cg) ok = collect(cg, collected < nmain ? cs_main : cs_tail);
    };
    for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
      const int s = it % STAGES, r = it / STAGES;
      int c, j;
      bool last;
      chunk_pos(kb, c, j, last);
      // the issuer cannot start chunk c before chunk c-2 has been collected, and this warp cannot
      // get block kb before the issuer has retired block kb - STAGES
      if (j == 0 && c >= 2) collect_to(c - 1);
      if (!ok) break;
      ok = mbar_wait(bar_full(s), r & 1, p.err, 43);
      if (!ok) break;
      uint8_t* stg = base_ptr + s * S::kStage;
      if (!(p.dbg & 1)) split_f16_tile(stg + S::kARaw, stg + S::kAHi, stg + S::kALo, kb < nkb1 ? sa : sa2, t);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(bar_split(s), 0);
      if (j == 1) collect_to(c);              // the previous chunk, while the tensor core works on this one
    }
    collect_to(nchunks);
    if (!ok) break;
    const uint32_t box = (uint32_t)(((it - 1) % STAGES) * S::kStage + (warp - 2) * 4096);
    if (m0 + row0 < p.M) {
      bool stored = false;
#pragma unroll
      for (int c = 0; c < NH / LD; ++c) {
        const int ncol = n0 + half * NH + c * LD;
        if (ncol < p.N) {
          uint8_t* stage_ptr = base_ptr + box;
          if (stored) {
            if (lane == 0) tma_store_wait_read();
            __syncwarp();
          }
          stored = true;
          uint32_t r[32];
#pragma unroll
          for (int j = 0; j < LD; ++j) r[j] = __float_as_uint(p.alpha * acc[c * LD + j]);
          if (p.addend != nullptr && m0 + row0 + lane < p.M) {
            const float* arow = p.addend + (size_t)(m0 + row0 + lane) * p.N + ncol;
#pragma unroll
            for (int j4 = 0; j4 < LD / 4; ++j4) {
              if (ncol + 4 * j4 < p.N) {
                const float4 d = *reinterpret_cast<const float4*>(arow + 4 * j4);
                r[4 * j4 + 0] = __float_as_uint(d.x + __uint_as_float(r[4 * j4 + 0]));
                r[4 * j4 + 1] = __float_as_uint(d.y + __uint_as_float(r[4 * j4 + 1]));
                r[4 * j4 + 2] = __float_as_uint(d.z + __uint_as_float(r[4 * j4 + 2]));
                r[4 * j4 + 3] = __float_as_uint(d.w + __uint_as_float(r[4 * j4 + 3]));
              }
            }
          }
          if (p.bias != nullptr || p.act != 0) {
#pragma unroll
            for (int j = 0; j < LD; ++j) {
              float v = __uint_as_float(r[j]);
              if (p.bias != nullptr && ncol + j < p.N) v = v + p.bias[ncol + j];
              r[j] = __float_as_uint(epi_act(p.act, v));
            }
          }
#pragma unroll
          for (int j = 0; j < LD / 4; ++j) {
            uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            *reinterpret_cast<uint4*>(stage_ptr + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&mapC, base + box, ncol, m0 + row0);
            tma_store_commit();
          }
        }
      }
    }
    if (lane == 0) {
      tma_store_wait_read();
      mbar_arrive(bar_epi);
    }
    __syncwarp();
    }
    if (lane == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc2(tmem_base, 512);
}


// ------------------------------------- CTA-pair GEMM, fp16 split, operands pre-split (F16X2)
// The arithmetic of gemm_tc_pair_f16_kernel with the conversion taken out of the GEMM: every
// A operand is cut into its fp16 hi / lo terms once, by split_rows_f16_kernel (one pass over
// the tensor: row maximum, power-of-two row scale, convert), instead of once per N tile inside
// the GEMM; B comes from the frozen weight's copies as before. Every operand tile is then a
// plain TMA load of fp16 (64 elements = one 128-byte swizzle row per k-block), the worker warps
// only collect accumulation chunks and store, and three 64 KiB stages are all load buffers.
// Scales are per ROW of A (exact powers of two, undone when a chunk is collected - the thread
// that collects a row owns it), which also removes the dependence of a row's accuracy on the
// largest magnitude anywhere else in the tensor.
// Pair protocol: the even CTA's MMAs read both CTAs' shared memory, so the odd CTA's idle MMA
// warp relays its "stage loaded" phases to the even CTA with one remote arrive per stage.
constexpr int kF16pKB = 64;                       // fp16 elements per k-block: one 128-byte row
constexpr int kF16pStages = 3;
constexpr int kF16pTile = BM * kF16pKB * 2;       // 16 KiB: 128 rows x 64 fp16
struct PairF16pSmem {
  static constexpr int kAHi = 0, kALo = kF16pTile, kBHi = 2 * kF16pTile, kBLo = 3 * kF16pTile;
  static constexpr int kStage = 4 * kF16pTile;    // 64 KiB
  static constexpr int kEpi = (kWorkers / 32) * 4096;           // store staging of its own: one 32 x 32 box per worker warp
  static constexpr int kTotal = kF16pStages * kStage + kEpi + 256 + 1024;
};
struct F16pParams {
  int M, N, K, K2;
  const float* bias;
  const float* addend;
  int act;
  float alpha;
  int eb_pre;                  // scale exponent of the frozen B copies
  const float* inv_a;          // [M]: 2^-e of each row of A (main pair)
  const float* inv_a2;         // [M]: the same for the tail's A2
  const float* inv_b2;         // [1]: and of the tail's B2 as a whole
  int n_tiles, total_tiles;
  int full_tiles;              // tiles [0, full_tiles) are 256 columns wide; the rest are halves of the leftover tiles
  int* err;
};

__global__ void __launch_bounds__(kThreadsV2, 1)
gemm_tc_pair_f16p_kernel(const __grid_constant__ CUtensorMap mapAhi, const __grid_constant__ CUtensorMap mapAlo,
                         const __grid_constant__ CUtensorMap mapA2hi, const __grid_constant__ CUtensorMap mapA2lo,
                         const __grid_constant__ CUtensorMap mapBhi, const __grid_constant__ CUtensorMap mapBlo,
                         const __grid_constant__ CUtensorMap mapB2hi, const __grid_constant__ CUtensorMap mapB2lo,
                         const __grid_constant__ CUtensorMap mapBhiH, const __grid_constant__ CUtensorMap mapBloH,
                         const __grid_constant__ CUtensorMap mapB2hiH, const __grid_constant__ CUtensorMap mapB2loH,
                         const __grid_constant__ CUtensorMap mapC, F16pParams p) {
  using S = PairF16pSmem;
  constexpr int STAGES = kF16pStages, BN = 256, KB = kF16pKB, CH = 2;   // CH k-blocks (128 elements of K) per chunk
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + STAGES * S::kStage + S::kEpi;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_peer = [&](int s) { return bars + 8u * (STAGES + s); };        // even CTA: the odd CTA's stage has landed
  auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };
  auto bar_acc_full = [&](int b) { return bars + 8u * (3 * STAGES + b); };
  auto bar_acc_empty = [&](int b) { return bars + 8u * (3 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (3 * STAGES + 5);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + STAGES * S::kStage + S::kEpi + 8 * (3 * STAGES + 5));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cid = (int)(blockIdx.x >> 1), ncl = (int)(gridDim.x >> 1);
  // The tiles of the last, partly filled wave are cut into two 128-column halves (the *H maps load
  // 64-row B boxes), so that wave costs half a tile time instead of a whole one.
  auto tile_of = [&](int t, int& m0, int& n0, int& bn) {
    int full = t;
    bn = BN;
    int shift = 0;
    if (t >= p.full_tiles) {
      const int h = t - p.full_tiles;
      full = p.full_tiles + (h >> 1);
      bn = BN / 2;
      shift = (h & 1) * (BN / 2);
    }
    n0 = (full % p.n_tiles) * BN + shift;
    m0 = (2 * (full / p.n_tiles) + (int)rank) * BM;
  };
  const int nkb1 = (p.K + KB - 1) / KB;
  const int nkb = nkb1 + (p.K2 + KB - 1) / KB;
  const int nmain = (nkb1 + CH - 1) / CH;
  const int nchunks = nmain + (nkb - nkb1 + CH - 1) / CH;
  auto chunk_pos = [&](int kb, int& c, int& j, bool& last) {
    if (kb < nkb1) { c = kb / CH; j = kb % CH; last = j == CH - 1 || kb == nkb1 - 1; }
    else { const int q = kb - nkb1; c = nmain + q / CH; j = q % CH; last = j == CH - 1 || kb == nkb - 1; }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_peer(s), 1);
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 2 * kWorkers / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ---- TMA producer: four fp16 tiles per stage ------------------------------------------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tl = cid; tl < p.total_tiles && ok; tl += ncl) {
        int m0, n0, bn;
        tile_of(tl, m0, n0, bn);
        const int nb = n0 + (int)rank * (bn / 2);
        const bool wide = bn == BN;
        for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
          const int s = it % STAGES, r = it / STAGES;
          if (r > 0) ok = mbar_wait(bar_empty(s), (r - 1) & 1, p.err, 51);
          if (!ok) break;
          const uint32_t stg = base + s * S::kStage;
          mbar_expect_tx(bar_full(s), 2 * kF16pTile + 2 * (bn / 2) * kF16pKB * 2);
          if (kb < nkb1) {
            tma_load_2d(stg + S::kAHi, &mapAhi, bar_full(s), kb * KB, m0);
            tma_load_2d(stg + S::kALo, &mapAlo, bar_full(s), kb * KB, m0);
            tma_load_2d(stg + S::kBHi, wide ? &mapBhi : &mapBhiH, bar_full(s), kb * KB, nb);
            tma_load_2d(stg + S::kBLo, wide ? &mapBlo : &mapBloH, bar_full(s), kb * KB, nb);
          } else {
            tma_load_2d(stg + S::kAHi, &mapA2hi, bar_full(s), (kb - nkb1) * KB, m0);
            tma_load_2d(stg + S::kALo, &mapA2lo, bar_full(s), (kb - nkb1) * KB, m0);
            tma_load_2d(stg + S::kBHi, wide ? &mapB2hi : &mapB2hiH, bar_full(s), (kb - nkb1) * KB, nb);
            tma_load_2d(stg + S::kBLo, wide ? &mapB2lo : &mapB2loH, bar_full(s), (kb - nkb1) * KB, nb);
          }
        }
      }
      if (!ok) {
        for (int kb = (it > STAGES ? it - STAGES : 0); kb < it; ++kb)
          mbar_wait(bar_full(kb % STAGES), (kb / STAGES) & 1, p.err, 55);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 1) {
      // ---- odd CTA: relay "this CTA's stage has landed" to the even CTA ------------------------
      bool ok = true;
      int it = 0;
      for (int tl = cid; tl < p.total_tiles && ok; tl += ncl)
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          ok = mbar_wait(bar_full(it % STAGES), (it / STAGES) & 1, p.err, 57);
          if (!ok) break;
          mbar_arrive_remote(bar_peer(it % STAGES), 0);
        }
    } else if (lane == 0) {
      // ---- even CTA: MMA issuer ---------------------------------------------------------------
      bool ok = true;
      int it = 0, ci = 0;
      for (int tl = cid; tl < p.total_tiles && ok; tl += ncl) {
      const uint32_t idesc = tl < p.full_tiles ? idesc_f16(256, BN) : idesc_f16(256, BN / 2);
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % STAGES, r = it / STAGES;
        const int buf = ci & 1;
        int c, j;
        bool last;
        chunk_pos(kb, c, j, last);
        if (j == 0 && ci >= 2) {
          ok = mbar_wait(bar_acc_empty(buf), ((ci >> 1) - 1) & 1, p.err, 56);
          if (!ok) break;
          tc_fence_after();
        }
        ok = mbar_wait(bar_full(s), r & 1, p.err, 52) && mbar_wait(bar_peer(s), r & 1, p.err, 59);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        const uint32_t stg = base + s * S::kStage;
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
          const uint64_t da = smem_desc_sw128(stg + S::kAHi + kk * 32), dal = smem_desc_sw128(stg + S::kALo + kk * 32);
          const uint64_t db = smem_desc_sw128(stg + S::kBHi + kk * 32), dbl = smem_desc_sw128(stg + S::kBLo + kk * 32);
          mma_f16_pair(tmem_d, da, db, idesc, (j | kk) != 0);
          mma_f16_pair(tmem_d, dal, db, idesc, 1);
          mma_f16_pair(tmem_d, da, dbl, idesc, 1);
        }
        mma_commit_pair(bar_empty(s));
        if (last) {
          mma_commit_pair(bar_acc_full(buf));
          ++ci;
        }
      }
      }
    }
  } else {
    // ---- worker warps (both CTAs): collect finished chunks, epilogue ----------------------------
    const int q = warp & 3, half = (warp - 2) >> 2, row0 = q * 32;
    constexpr int NH = BN / 2, LD = 32;
    const float inv_b = pow2i(-p.eb_pre);
    float acc[NH];
    bool ok = true;
    int cg = 0, tiles_done = 0;
    for (int tl = cid; tl < p.total_tiles && ok; tl += ncl, ++tiles_done) {
      int m0, n0, bn;
      tile_of(tl, m0, n0, bn);
      const int nh = bn / 2, boxes = nh / LD;      // this warp's share of the tile's columns
      const int m = m0 + row0 + lane;
      const float cs_main = (m < p.M ? p.inv_a[m] : 1.0f) * inv_b;
      const float cs_tail = p.K2 ? (m < p.M ? p.inv_a2[m] : 1.0f) * __ldg(p.inv_b2) : 1.0f;
#pragma unroll
      for (int j = 0; j < NH; ++j) acc[j] = 0.0f;
      for (int ci = 0; ci < nchunks && ok; ++ci, ++cg) {
        const int buf = cg & 1;
        ok = mbar_wait(bar_acc_full(buf), (cg >> 1) & 1, p.err, 54);
        if (!ok) break;
        tc_fence_after();
        const float cs = ci < nmain ? cs_main : cs_tail;
#pragma unroll
        for (int c = 0; c < NH / LD; ++c) {
          if (c < boxes) {
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)row0 << 16) + buf * BN + half * nh + c * LD, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < LD; ++j) acc[c * LD + j] += __uint_as_float(r[j]) * cs;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(bar_acc_empty(buf), 0);
      }
      if (!ok) break;
      // store staging lives behind the stage ring, so the loads of the next tile never wait for it
      const uint32_t box = (uint32_t)(STAGES * S::kStage + (warp - 2) * 4096);
      if (m0 + row0 < p.M) {
        bool stored = false;
#pragma unroll
        for (int c = 0; c < NH / LD; ++c) {
          const int ncol = n0 + half * nh + c * LD;
          if (c < boxes && ncol < p.N) {
            uint8_t* stage_ptr = base_ptr + box;
            if (stored || tiles_done > 0) {          // the box's previous store (this tile's or the last tile's) has been read
              if (lane == 0) tma_store_wait_read();
              __syncwarp();
            }
            stored = true;
            uint32_t r[32];
#pragma unroll
            for (int j = 0; j < LD; ++j) r[j] = __float_as_uint(p.alpha * acc[c * LD + j]);
            if (p.addend != nullptr && m < p.M) {
              const float* arow = p.addend + (size_t)m * p.N + ncol;
#pragma unroll
              for (int j4 = 0; j4 < LD / 4; ++j4) {
                if (ncol + 4 * j4 < p.N) {
                  const float4 d = *reinterpret_cast<const float4*>(arow + 4 * j4);
                  r[4 * j4 + 0] = __float_as_uint(d.x + __uint_as_float(r[4 * j4 + 0]));
                  r[4 * j4 + 1] = __float_as_uint(d.y + __uint_as_float(r[4 * j4 + 1]));
                  r[4 * j4 + 2] = __float_as_uint(d.z + __uint_as_float(r[4 * j4 + 2]));
                  r[4 * j4 + 3] = __float_as_uint(d.w + __uint_as_float(r[4 * j4 + 3]));
                }
              }
            }
            if (p.bias != nullptr || p.act != 0) {
#pragma unroll
              for (int j = 0; j < LD; ++j) {
                float v = __uint_as_float(r[j]);
                if (p.bias != nullptr && ncol + j < p.N) v = v + p.bias[ncol + j];
                r[j] = __float_as_uint(epi_act(p.act, v));
              }
            }
#pragma unroll
            for (int j = 0; j < LD / 4; ++j) {
              uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
              *reinterpret_cast<uint4*>(stage_ptr + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&mapC, base + box, ncol, m0 + row0);
              tma_store_commit();
            }
          }
        }
      }
    }
    if (lane == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc2(tmem_base, 512);
}


// ---------------------------------------- rank-r product on pre-split operands (F16X2)
// out[M, BN] = alpha * A[M, K] . B[BN, K]^T for the LoRA factors (BN = 16 / 32 / 64), one CTA per
// 128 rows, reading the fp16 hi / lo copies of A that the neighbouring frozen-weight GEMM uses
// (split once by split_rows_f16_kernel) and a row-scaled split of the small factor. The kernel
// only streams A: TMA -> tcgen05.mma kind::f16 -> chunked collection. B_hi and B_lo sit next to
// each other in a stage, so one MMA of width 2 BN multiplies A_hi with [B_hi; B_lo] and a second
// of width BN adds A_lo . B_hi: two instructions per 16 elements of K.
struct RankF16Params {
  int M, K;
  float alpha;
  const float* inv_a;      // [M]
  const float* inv_b;      // [BN]
  int* err;
};
template <int BN>
struct RankF16Smem {
  static constexpr int kA = kF16pTile, kB = BN * kF16pKB * 2;
  static constexpr int kStage = 2 * kA + 2 * kB;                 // [A hi][A lo][B hi][B lo]
  static constexpr int kStages = BN <= 32 ? 5 : 4;
  static constexpr int kTotal = kStages * kStage + 256 + 1024;
};
constexpr int kRankThreads = 64 + 128;

template <int BN>
__global__ void __launch_bounds__(kRankThreads, 1)
gemm_tc_rank_f16p_kernel(const __grid_constant__ CUtensorMap mapAhi, const __grid_constant__ CUtensorMap mapAlo,
                         const __grid_constant__ CUtensorMap mapBhi, const __grid_constant__ CUtensorMap mapBlo,
                         const __grid_constant__ CUtensorMap mapC, RankF16Params p) {
  using S = RankF16Smem<BN>;
  constexpr int STAGES = S::kStages, KB = kF16pKB, CH = 2;
  constexpr uint32_t kCols = 4 * BN < 32 ? 32 : 4 * BN;        // two accumulators of 2 BN columns
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + STAGES * S::kStage;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_empty = [&](int s) { return bars + 8u * (STAGES + s); };
  auto bar_acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto bar_acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + STAGES * S::kStage + 8 * (2 * STAGES + 4));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM;
  const int nkb = (p.K + KB - 1) / KB;
  const int nchunks = (nkb + CH - 1) / CH;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % STAGES, r = kb / STAGES;
        if (r > 0) ok = mbar_wait(bar_empty(s), (r - 1) & 1, p.err, 61);
        if (!ok) break;
        const uint32_t stg = base + s * S::kStage;
        mbar_expect_tx(bar_full(s), S::kStage);
        tma_load_2d(stg, &mapAhi, bar_full(s), kb * KB, m0);
        tma_load_2d(stg + S::kA, &mapAlo, bar_full(s), kb * KB, m0);
        tma_load_2d(stg + 2 * S::kA, &mapBhi, bar_full(s), kb * KB, 0);
        tma_load_2d(stg + 2 * S::kA + S::kB, &mapBlo, bar_full(s), kb * KB, 0);
        ++issued;
      }
      if (!ok)
        for (int kb = (issued > STAGES ? issued - STAGES : 0); kb < issued; ++kb)
          mbar_wait(bar_full(kb % STAGES), (kb / STAGES) & 1, p.err, 65);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc1 = idesc_f16(BM, BN), idesc2 = idesc_f16(BM, 2 * BN);
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % STAGES, r = kb / STAGES, ci = kb / CH, buf = ci & 1;
        if (kb % CH == 0 && ci >= 2) {
          ok = mbar_wait(bar_acc_empty(buf), ((ci >> 1) - 1) & 1, p.err, 66);
          if (!ok) break;
          tc_fence_after();
        }
        ok = mbar_wait(bar_full(s), r & 1, p.err, 62);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * 2 * BN;
        const uint32_t stg = base + s * S::kStage;
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
          const uint64_t da = smem_desc_sw128(stg + kk * 32), dal = smem_desc_sw128(stg + S::kA + kk * 32);
          const uint64_t db = smem_desc_sw128(stg + 2 * S::kA + kk * 32);      // B hi, with B lo right behind it
          mma_f16(tmem_d, da, db, idesc2, ((kb % CH) | kk) != 0);
          mma_f16(tmem_d, dal, db, idesc1, 1);
        }
        mma_commit(bar_empty(s));
        if (kb % CH == CH - 1 || kb == nkb - 1) mma_commit(bar_acc_full(buf));
      }
    }
  } else {
    const int q = warp & 3, row0 = q * 32, m = m0 + row0 + lane;
    const float cs_row = m < p.M ? p.inv_a[m] : 1.0f;
    float acc[BN], csc[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) {
      acc[j] = 0.0f;
      csc[j] = cs_row * __ldg(p.inv_b + j);
    }
    bool ok = true;
    for (int ci = 0; ci < nchunks && ok; ++ci) {
      const int buf = ci & 1;
      ok = mbar_wait(bar_acc_full(buf), (ci >> 1) & 1, p.err, 64);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < BN / 16; ++c) {
        uint32_t rh[16], rl[16];
        tmem_ld16(tmem_base + ((uint32_t)row0 << 16) + buf * 2 * BN + c * 16, rh);
        tmem_ld16(tmem_base + ((uint32_t)row0 << 16) + buf * 2 * BN + BN + c * 16, rl);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c * 16 + j] += (__uint_as_float(rh[j]) + __uint_as_float(rl[j])) * csc[c * 16 + j];
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(buf));
    }
    if (ok && m0 + row0 < p.M) {
      // every product has retired: stage 0 holds the store staging, one 32 x 32 box per warp, reused
      uint8_t* stage_ptr = base_ptr + q * 4096;
#pragma unroll
      for (int c = 0; c < (BN + 31) / 32; ++c) {
        if (c > 0) {
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
        }
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
          float v[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = c * 32 + j4 * 4 + e;
            v[e] = col < BN ? p.alpha * acc[col < BN ? col : 0] : 0.0f;
          }
          *reinterpret_cast<float4*>(stage_ptr + lane * 128 + ((j4 ^ (lane & 7)) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&mapC, base + q * 4096, c * 32, m0 + row0);
          tma_store_commit();
        }
      }
      if (lane == 0) tma_store_wait_all();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kCols);
}

// One pass over a row-major f32 tensor [M, K]: each row's largest magnitude picks its power-of-two
// scale 2^e (max * 2^e in [2^13, 2^14)), the row is cut into fp16 hi = fp16(x 2^e) and
// lo = fp16(x 2^e - hi), and 2^-e goes to inv[row]. One warp per row; the second sweep over the
// row comes from L1 / L2. K % 4 == 0. Up to two tensors per launch (the low-rank tail's two small
// operands go together): rows [0, a.M) are the first tensor's, the rest the second's.
struct SplitJob { const float* src; __half* hi; __half* lo; float* inv; int M, K; };
__device__ __forceinline__ void split_row_f16(const SplitJob& t, int row, int lane) {
  const int K4 = t.K >> 2;
  const float4* r4 = reinterpret_cast<const float4*>(t.src + (size_t)row * t.K);
  uint32_t mx = 0;
  for (int i = lane; i < K4; i += 32) {
    const float4 v = r4[i];
    mx = max(max(mx, __float_as_uint(v.x) & 0x7FFFFFFFu), max(max(__float_as_uint(v.y) & 0x7FFFFFFFu,
             __float_as_uint(v.z) & 0x7FFFFFFFu), __float_as_uint(v.w) & 0x7FFFFFFFu));
  }
  mx = __reduce_max_sync(0xFFFFFFFFu, mx);
  const int e = f16_scale_exp(mx);
  const float sc = pow2i(e);
  uint2* h2 = reinterpret_cast<uint2*>(t.hi + (size_t)row * t.K);
  uint2* l2 = reinterpret_cast<uint2*>(t.lo + (size_t)row * t.K);
  for (int i = lane; i < K4; i += 32) {
    const float4 v = r4[i];
    float h0, h1, h2f, h3, l0, l1, l2f, l3;
    split11(v.x * sc, h0, l0);
    split11(v.y * sc, h1, l1);
    split11(v.z * sc, h2f, l2f);
    split11(v.w * sc, h3, l3);
    h2[i] = make_uint2(pack_h2(h0, h1), pack_h2(h2f, h3));
    l2[i] = make_uint2(pack_h2(l0, l1), pack_h2(l2f, l3));
  }
  if (lane == 0) t.inv[row] = pow2i(-e);
}
// The row of NV * 128 floats held in registers between the maximum and the conversion: one read.
template <int NV>
__device__ __forceinline__ void split_row_f16_regs(const SplitJob& t, int row, int lane) {
  const float4* r4 = reinterpret_cast<const float4*>(t.src + (size_t)row * t.K);
  float4 v[NV];
  uint32_t mx = 0;
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = r4[lane + 32 * i];
#pragma unroll
  for (int i = 0; i < NV; ++i)
    mx = max(max(mx, __float_as_uint(v[i].x) & 0x7FFFFFFFu), max(max(__float_as_uint(v[i].y) & 0x7FFFFFFFu,
             __float_as_uint(v[i].z) & 0x7FFFFFFFu), __float_as_uint(v[i].w) & 0x7FFFFFFFu));
  mx = __reduce_max_sync(0xFFFFFFFFu, mx);
  const int e = f16_scale_exp(mx);
  const float sc = pow2i(e);
  uint2* h2 = reinterpret_cast<uint2*>(t.hi + (size_t)row * t.K);
  uint2* l2 = reinterpret_cast<uint2*>(t.lo + (size_t)row * t.K);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float h0, h1, h2f, h3, l0, l1, l2f, l3;
    split11(v[i].x * sc, h0, l0);
    split11(v[i].y * sc, h1, l1);
    split11(v[i].z * sc, h2f, l2f);
    split11(v[i].w * sc, h3, l3);
    h2[lane + 32 * i] = make_uint2(pack_h2(h0, h1), pack_h2(h2f, h3));
    l2[lane + 32 * i] = make_uint2(pack_h2(l0, l1), pack_h2(l2f, l3));
  }
  if (lane == 0) t.inv[row] = pow2i(-e);
}

// whole != 0: tensor b is small and gets ONE scale (inv[0]); the last kWholeBlocks blocks share it,
// each finding the maximum of all of b on its own (b is a few hundred KB in L2) and converting a slice.
constexpr int kWholeBlocks = 16;
template <int NV>
__global__ void __launch_bounds__(256) split_rows_f16_kernel(SplitJob a, SplitJob b, int whole) {
  const int lane = threadIdx.x & 31;
  const int nb = whole ? (int)gridDim.x - kWholeBlocks : (int)gridDim.x;
  if (whole && (int)blockIdx.x >= nb) {
    __shared__ uint32_t smax[8];
    const int n4 = (b.M * b.K) >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(b.src);
    uint32_t mx = 0;
#pragma unroll 8
    for (int i = threadIdx.x; i < n4; i += 256) {
      const float4 v = r4[i];
      mx = max(max(mx, __float_as_uint(v.x) & 0x7FFFFFFFu), max(max(__float_as_uint(v.y) & 0x7FFFFFFFu,
               __float_as_uint(v.z) & 0x7FFFFFFFu), __float_as_uint(v.w) & 0x7FFFFFFFu));
    }
    mx = __reduce_max_sync(0xFFFFFFFFu, mx);
    if (lane == 0) smax[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = smax[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = max(mx, smax[i]);
    const int e = f16_scale_exp(mx);
    const float sc = pow2i(e);
    uint2* h2 = reinterpret_cast<uint2*>(b.hi);
    uint2* l2 = reinterpret_cast<uint2*>(b.lo);
    const int part = (int)blockIdx.x - nb;
#pragma unroll 4
    for (int i = part * 256 + threadIdx.x; i < n4; i += kWholeBlocks * 256) {
      const float4 v = r4[i];
      float h0, h1, h2f, h3, l0, l1, l2f, l3;
      split11(v.x * sc, h0, l0);
      split11(v.y * sc, h1, l1);
      split11(v.z * sc, h2f, l2f);
      split11(v.w * sc, h3, l3);
      h2[i] = make_uint2(pack_h2(h0, h1), pack_h2(h2f, h3));
      l2[i] = make_uint2(pack_h2(l0, l1), pack_h2(l2f, l3));
    }
    if (part == 0 && threadIdx.x == 0) b.inv[0] = pow2i(-e);
    return;
  }
  const int total = a.M + (whole ? 0 : b.M);
  for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < total; row += nb * 8) {
    if (row < a.M) {
      if constexpr (NV > 0) split_row_f16_regs<NV>(a, row, lane);
      else split_row_f16(a, row, lane);
    } else {
      split_row_f16(b, row - a.M, lane);
    }
  }
}
// NV = a.K / 128 when the first tensor's rows fit the register variant, else 0
inline void launch_split_rows(unsigned blocks, cudaStream_t st, const SplitJob& a, const SplitJob& b, int whole) {
  const int nv = (a.K % 128 == 0) ? a.K / 128 : 0;
  if (nv == 8) split_rows_f16_kernel<8><<<blocks, 256, 0, st>>>(a, b, whole);
  else if (nv == 22) split_rows_f16_kernel<22><<<blocks, 256, 0, st>>>(a, b, whole);
  else if (nv == 32) split_rows_f16_kernel<32><<<blocks, 256, 0, st>>>(a, b, whole);
  else split_rows_f16_kernel<0><<<blocks, 256, 0, st>>>(a, b, whole);
}

// max|x| (as f32 bit patterns, which order like the magnitudes; a NaN sorts above every finite
// value) of up to four tensors in one launch: blockIdx.y selects the tensor. The slots must be
// zero beforehand. The maximum does not depend on the order of the atomic updates.
struct AbsmaxArgs { const float* ptr[4]; unsigned long long n[4]; };
__global__ void __launch_bounds__(256) absmax4_kernel(AbsmaxArgs a, uint32_t* __restrict__ slots) {
  const float* x = a.ptr[blockIdx.y];
  const size_t n = a.n[blockIdx.y];
  if (x == nullptr || n == 0) return;
  uint32_t m = 0;
  const size_t n4 = n >> 2;
  const uint4* x4 = reinterpret_cast<const uint4*>(x);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = x4[i];
    m = max(max(m, v.x & 0x7FFFFFFFu), max(max(v.y & 0x7FFFFFFFu, v.z & 0x7FFFFFFFu), v.w & 0x7FFFFFFFu));
  }
  if (blockIdx.x == 0)
    for (size_t i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) m = max(m, __float_as_uint(x[i]) & 0x7FFFFFFFu);
  m = __reduce_max_sync(0xFFFFFFFFu, m);
  if ((threadIdx.x & 31) == 0 && m != 0) atomicMax(slots + blockIdx.y, m);
}

// One-time fp16 split of a frozen weight: hi = fp16(w s), lo = fp16(w s - hi).
__global__ void split_f16_kernel(const float* __restrict__ w, __half* __restrict__ hi, __half* __restrict__ lo,
                                 size_t n, float s) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float h, l;
    split11(w[i] * s, h, l);
    hi[i] = __float2half_rn(h);
    lo[i] = __float2half_rn(l);
  }
}

// The low-rank tail's B operand ([N, K2] f32, K2 <= 32, rewritten every step) as fp16 hi / lo
// tiles [N, 32] (zero-padded along K), scaled by the power of two its measured max|x| asks for.
__global__ void split_f16_tail_kernel(const float* __restrict__ b, __half* __restrict__ hi, __half* __restrict__ lo,
                                      int N, int K2, const uint32_t* __restrict__ absmax_slot) {
  const float s = pow2i(f16_scale_exp(*absmax_slot));
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * 32) return;
  const int n = i >> 5, k = i & 31;
  float h = 0.0f, l = 0.0f;
  if (k < K2) split11(b[(size_t)n * K2 + k] * s, h, l);
  hi[i] = __float2half_rn(h);
  lo[i] = __float2half_rn(l);
}

// ------------------------------------------ attention forward: scores + causal softmax -> P
// One CTA owns 128 query rows of one (batch item, head): the scaled scores of those rows
// against every key up to the diagonal, (i + 1) * 128 columns, accumulate in TMEM (all 512
// columns at S = 512) and the causal row softmax runs on them in place, so the raw scores
// never touch global memory. Sixteen worker warps share the softmax: a warp can read only
// its own quarter of the TMEM lanes (32 query rows), so four warps serve each quarter and
// take every fourth 64-column chunk; per-row maxima and sums of exponentials are combined
// through shared memory in a fixed order (sums: f32 within a chunk, f64 across chunks).
// Needs head width 64 and S <= 512, S % 128 == 0.
struct AfParams {
  int S, H;
  float alpha;
  int qx[2], qy[2];        // TMA origin of Q / K windows per batch item and head (column, row)
  const float* pin;        // MODE 1: the probabilities P [B*H*S, S] saved by the forward pass
  int x3;
  int* err;
};
constexpr int kAfWorkers = 512;
constexpr int kAfThreads = 64 + kAfWorkers;

__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kAfWorkers) : "memory"); }

// MODE 0: A = Q, B = K, output P = causal softmax(alpha A B^T).
// MODE 1 (backward): A = dO, B = V, so TMEM holds dP = dO V^T; output dS = P * (dP - rowsum(dP * P))
// with P read from global memory - dP itself is never written.
template <int MODE>
__global__ void __launch_bounds__(kAfThreads, 1)
attn_scores_softmax_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                           const __grid_constant__ CUtensorMap mapP, AfParams p) {
  constexpr int kTile = BM * BK * 4;                 // one 128 x 32 f32 tile: 16 KiB
  constexpr int kQ = 4 * kTile;                      // raw[2], lo[2]
  constexpr int kStage = 4 * kTile;                  // a 128-key tile: raw[2], lo[2]
  constexpr int kRed = 4 * 128 * 12;                 // per (column group, row): max f32 + sum f64
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + kQ + 2 * kStage + kRed;
  const uint32_t q_full = bars, q_split = bars + 8, accum = bars + 16;
  auto k_full = [&](int s) { return bars + 24u + 8u * s; };
  auto k_split = [&](int s) { return bars + 40u + 8u * s; };
  auto k_empty = [&](int s) { return bars + 56u + 8u * s; };
  const uint32_t tmem_slot = bars + 72;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + kQ + 2 * kStage + kRed + 72);
  double* red_den = reinterpret_cast<double*>(base_ptr + kQ + 2 * kStage);          // [4][128]
  float* red_max = reinterpret_cast<float*>(base_ptr + kQ + 2 * kStage + 4 * 128 * 8);  // [4][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = blockIdx.x, m0 = mt * BM, z = blockIdx.y;
  const int bi = z / p.H, hd = z % p.H;
  const int ntiles = mt + 1;                         // key tiles up to and including the diagonal
  const int x0 = bi * p.qx[0] + hd * p.qx[1], y0 = bi * p.qy[0] + hd * p.qy[1];

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_split, kAfWorkers / 32);       // one arrival per split warp
    mbar_init(accum, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_split(s), kAfWorkers / 32);
      mbar_init(k_empty(s), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * kTile);
      tma_load_2d(base, &mapQ, q_full, x0, y0 + m0);
      tma_load_2d(base + kTile, &mapQ, q_full, x0 + BK, y0 + m0);
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j & 1, r = j >> 1;
        if (r > 0) ok = mbar_wait(k_empty(s), (r - 1) & 1, p.err, 21);
        if (!ok) break;
        const uint32_t dst = base + kQ + s * kStage;
        mbar_expect_tx(k_full(s), 2 * kTile);
        tma_load_2d(dst, &mapK, k_full(s), x0, y0 + j * BM);
        tma_load_2d(dst + kTile, &mapK, k_full(s), x0 + BK, y0 + j * BM);
        ++issued;
      }
      if (!ok) {
        mbar_wait(q_full, 0, p.err, 25);
        for (int j = (issued > 2 ? issued - 2 : 0); j < issued; ++j) mbar_wait(k_full(j & 1), (j >> 1) & 1, p.err, 25);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_tf32(BM, 128);
      bool ok = mbar_wait(q_split, 0, p.err, 22);
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j & 1, r = j >> 1;
        ok = mbar_wait(k_split(s), r & 1, p.err, 22);
        if (!ok) break;
        tc_fence_after();
        const uint32_t kb0 = base + kQ + s * kStage;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
          for (int kk = 0; kk < BK / 8; ++kk) {
            const uint64_t da = smem_desc_sw128(base + kb * kTile + kk * 32);
            const uint64_t db = smem_desc_sw128(kb0 + kb * kTile + kk * 32);
            mma_tf32(tmem_base + j * 128, da, db, idesc, (kb | kk) != 0);
            if (p.x3) {
              mma_tf32(tmem_base + j * 128, smem_desc_sw128(base + (2 + kb) * kTile + kk * 32), db, idesc, 1);
              mma_tf32(tmem_base + j * 128, da, smem_desc_sw128(kb0 + (2 + kb) * kTile + kk * 32), idesc, 1);
            }
          }
        }
        mma_commit(k_empty(s));
      }
      if (ok) mma_commit(accum);
    }
  } else {
    const int t = threadIdx.x - 64;
    auto split512 = [&](uint8_t* raw) {            // 32 KiB of f32 -> lo parts, 32 KiB further on
      const float4* r = reinterpret_cast<const float4*>(raw);
      float4* l = reinterpret_cast<float4*>(raw + 2 * kTile);
#pragma unroll
      for (int i = t; i < 2 * kTile / 16; i += kAfWorkers) {
        const float4 v = r[i];
        l[i] = make_float4(lo_part(v.x), lo_part(v.y), lo_part(v.z), lo_part(v.w));
      }
    };
    bool ok = mbar_wait(q_full, 0, p.err, 23);
    if (ok) {
      split512(base_ptr);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_split);
    }
    for (int j = 0; j < ntiles && ok; ++j) {
      const int s = j & 1, r = j >> 1;
      ok = mbar_wait(k_full(s), r & 1, p.err, 23);
      if (!ok) break;
      split512(base_ptr + kQ + s * kStage);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(k_split(s));
    }
    if (MODE == 1 && ok) {
      // while the last products run: pull this tile's block of P toward L2 (one 128-byte line per request)
      const int lines_per_row = ntiles * 4;
      const char* pbase = reinterpret_cast<const char*>(p.pin + ((size_t)z * p.S + m0) * p.S);
      for (int i = t; i < BM * lines_per_row; i += kAfWorkers) {
        const char* a = pbase + (size_t)(i / lines_per_row) * p.S * 4 + (size_t)(i % lines_per_row) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
      }
    }
    if (ok) ok = mbar_wait(accum, 0, p.err, 24);
    tc_fence_after();
    // a failed wait is failed for every worker (same barriers, same limit): no one is left at
    // the worker barrier below
    if (ok) {
      const int q = warp & 3, grp = (warp - 2) >> 2, row0 = q * 32;
      const int rl = row0 + lane;                     // row within the tile
      const int m = m0 + rl;                          // query row in the sequence; keys 0..m are visible
      const uint32_t trow = tmem_base + ((uint32_t)row0 << 16);
      const int nch = ntiles * 2;                     // 64-column chunks holding scores
      auto ld64 = [&](int c, uint32_t* r) {
        tmem_ld32(trow + c * 64, r);
        tmem_ld32(trow + c * 64 + 32, r + 32);
        tmem_ld_wait();
      };
      float mx = 0.0f, inv = 1.0f, rsum = 0.0f;
      // two 32x32 boxes per warp (one 64-column chunk of its 32 rows), in the layout of a TMA
      // store box: row * 128 bytes, 16-byte chunk k of a row at position k ^ (row & 7)
      const uint32_t ring = base + (warp - 2) * (2 * 4096);
      uint8_t* ring_ptr = base_ptr + (warp - 2) * (2 * 4096);
      const int prow0 = z * p.S + m0 + row0;          // first row of this warp's boxes in P [B*H*S, S]
      // MODE 1: bring the warp's 32 x 64 block of P into its boxes with row-wise coalesced loads
      // (every product has retired by now, so the operand buffers are free)
      auto load_p_chunk = [&](int c) {
        const float* src = p.pin + (size_t)prow0 * p.S + c * 64 + lane * 2;
        uint8_t* dst = ring_ptr + (lane >> 4) * 4096 + (lane & 1) * 8;
        const int ch = (lane & 15) >> 1;
#pragma unroll
        for (int half = 0; half < 2; ++half) {       // 16 row loads in flight at a time
          float2 v2[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            v2[i] = __ldg(reinterpret_cast<const float2*>(src + (size_t)(half * 16 + i) * p.S));
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int rr = half * 16 + i;
            *reinterpret_cast<float2*>(dst + rr * 128 + ((ch ^ (rr & 7)) << 4)) = v2[i];
          }
        }
        __syncwarp();
      };
      if constexpr (MODE == 0) {
      mx = -INFINITY;
      for (int c = grp; c < nch; c += 4) {
        uint32_t r[64];
        ld64(c, r);
        // value selects, not branches: the 64 elements stay independent for the scheduler
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float v = p.alpha * __uint_as_float(r[j]);
          m4[j & 3] = fmaxf(m4[j & 3], (c * 64 + j <= m) ? v : -INFINITY);
        }
        mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
      }
      red_max[grp * 128 + rl] = mx;
      worker_sync();
      mx = fmaxf(fmaxf(red_max[rl], red_max[128 + rl]), fmaxf(red_max[256 + rl], red_max[384 + rl]));
      double den = 0.0;
      for (int c = grp; c < nch; c += 4) {
        uint32_t r[64];
        ld64(c, r);
        float part = 0.0f;                            // 64 terms in f32, in column order
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float e = __expf(p.alpha * __uint_as_float(r[j]) - mx);
          part += (c * 64 + j <= m) ? e : 0.0f;
        }
        den += (double)part;
      }
      red_den[grp * 128 + rl] = den;
      worker_sync();
      den = ((red_den[rl] + red_den[128 + rl]) + red_den[256 + rl]) + red_den[384 + rl];
      inv = 1.0f / (float)den;
      } else {
        // rowsum(dP * P): P is zero beyond the diagonal, so no mask is needed here
        double dot = 0.0;
        for (int c = grp; c < nch; c += 4) {
          load_p_chunk(c);
          uint32_t r[64];
          ld64(c, r);
          float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int j4 = 0; j4 < 16; ++j4) {
            const float4 pv = *reinterpret_cast<const float4*>(ring_ptr + (j4 >> 3) * 4096 + lane * 128 +
                                                               (((j4 & 7) ^ (lane & 7)) << 4));
            d4[0] = fmaf(__uint_as_float(r[j4 * 4 + 0]), pv.x, d4[0]);
            d4[1] = fmaf(__uint_as_float(r[j4 * 4 + 1]), pv.y, d4[1]);
            d4[2] = fmaf(__uint_as_float(r[j4 * 4 + 2]), pv.z, d4[2]);
            d4[3] = fmaf(__uint_as_float(r[j4 * 4 + 3]), pv.w, d4[3]);
          }
          dot += (double)((d4[0] + d4[1]) + (d4[2] + d4[3]));
          __syncwarp();                                // the boxes are refilled by the next chunk
        }
        red_den[grp * 128 + rl] = dot;
        worker_sync();
        dot = ((red_den[rl] + red_den[128 + rl]) + red_den[256 + rl]) + red_den[384 + rl];
        rsum = (float)dot;
      }
      // every product has retired: the operand buffers serve as store staging, two 32x32 boxes
      // per warp, plus one box of zeros per row quarter for the masked tail of the rows
      bool first = true;
      for (int c = grp; c < nch; c += 4) {
        if (!first) {
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
        }
        first = false;
        if constexpr (MODE == 1) load_p_chunk(c);
        uint32_t r[64];
        ld64(c, r);
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          uint8_t* box = ring_ptr + hb * 4096;
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            float v[4];
            float pq[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (MODE == 1) {   // the dS values replace the P values they were made from
              const float4 pv = *reinterpret_cast<const float4*>(box + lane * 128 + ((j4 ^ (lane & 7)) << 4));
              pq[0] = pv.x; pq[1] = pv.y; pq[2] = pv.z; pq[3] = pv.w;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int col = c * 64 + hb * 32 + j4 * 4 + e;
              float pe;
              if constexpr (MODE == 0) pe = __expf(p.alpha * __uint_as_float(r[hb * 32 + j4 * 4 + e]) - mx) * inv;
              else pe = pq[e] * (__uint_as_float(r[hb * 32 + j4 * 4 + e]) - rsum);
              v[e] = col <= m ? pe : 0.0f;
            }
            *reinterpret_cast<float4*>(box + lane * 128 + ((j4 ^ (lane & 7)) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&mapP, ring, c * 64, prow0);
          tma_store_2d(&mapP, ring + 4096, c * 64 + 32, prow0);
          tma_store_commit();
        }
      }
      if (grp == 0 && nch * 64 < p.S) {
        const uint32_t zoff = 16 * 2 * 4096 + q * 4096;
        uint8_t* zbox = base_ptr + zoff;
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) *reinterpret_cast<float4*>(zbox + lane * 128 + (j4 << 4)) = make_float4(0.f, 0.f, 0.f, 0.f);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          for (int col = nch * 64; col < p.S; col += 32) tma_store_2d(&mapP, base + zoff, col, prow0);
          tma_store_commit();
        }
      }
      if (lane == 0) tma_store_wait_all();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// lo part of every element: x minus x with the low 13 mantissa bits cleared (one-time, frozen weights).
__global__ void lo_copy_kernel(const float* __restrict__ in, float* __restrict__ out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = lo_part(in[i]);
}

// [K,N] row-major -> [N,K] row-major (one-time copy of a frozen weight).
__global__ void transpose_kernel(const float* __restrict__ in, float* __restrict__ out, int K, int N) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int k = k0 + i, n = n0 + threadIdx.x;
    tile[i][threadIdx.x] = (k < K && n < N) ? in[(size_t)k * N + n] : 0.0f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int n = n0 + i, k = k0 + threadIdx.x;
    if (n < N && k < K) out[(size_t)n * K + k] = tile[threadIdx.x][i];
  }
}

// ------------------------------------------------------------------- host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// 2-D f32 row-major tensor [rows, cols] (cols contiguous), box [box_rows, box_cols], 128-byte swizzle
// (box_cols = 32) or none.
bool make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows,
              uint32_t box_cols, int swizzle_bytes, bool f16 = false) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * (f16 ? 2u : 4u)};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr),
            dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE,
            swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                 : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr uint64_t kRankKMax = 32768;       // longest reduction the rank-r F16X2 scratch holds
constexpr uint64_t kF16TailRows = 65536;    // widest N the F16X2 tail scratch holds
constexpr uint64_t kF16TailK = 64;          // widest low-rank tail (fp16 elements: one k-block of the pre-split kernel)
struct TcState {
  int* err_dev = nullptr;
  bool attrs_set = false;
  bool usable = true;
  float* rank_scratch = nullptr;
  int pair_clusters = 0;          // resident clusters of the pair kernel on this device (0 = not queried yet)
  int pair_f16_clusters = 0, pair_f16p_clusters = 0;
  std::map<const float*, float*> lo_copies;   // frozen B operand -> its precomputed lo part (x - tf32(x))
  struct F16Copy { __half* hi; __half* lo; int exp; };
  std::map<const float*, F16Copy> f16_copies; // frozen B operand -> fp16 split of w * 2^exp (F16X2 mode)
  uint32_t* absmax_dev = nullptr;             // four max|x| slots for the run-time operands of an F16X2 launch
  const float* absmax_src = nullptr;          // the A operand whose maximum slot 0 holds, and when it was measured
  uint64_t absmax_n = 0, absmax_unit = 0;
  // pre-split A operands of the F16X2 GEMM (sized when programs are built): the main pair's A, the tail's A2
  __half *a_hi = nullptr, *a_lo = nullptr, *a2_hi = nullptr, *a2_lo = nullptr;
  float *a_inv = nullptr, *a2_inv = nullptr;
  uint64_t a_cap = 0, a_rows_cap = 0;           // elements of a_hi / a_lo, rows of the inv arrays and of a2_*
  const float* split_src = nullptr;             // the A operand a_hi / a_lo currently hold, and when it was split
  uint64_t split_m = 0, split_k = 0, split_unit = 0;
  __half *tail_hi = nullptr, *tail_lo = nullptr;
  float* tail_inv = nullptr;                    // per-row 2^-e of the pre-split tail operand
  __half *rank_b_hi = nullptr, *rank_b_lo = nullptr;   // pre-split LoRA factor of the rank-r kernel, [64, kRankKMax]
  float* rank_b_inv = nullptr;   // fp16 copies of a rank-r product.s small operand
  std::map<std::tuple<const void*, uint64_t, uint64_t, uint32_t, uint32_t>, CUtensorMap> maps;
  std::set<const void*> smem_attr_done;   // kernels whose dynamic shared-memory limit was raised on this context's device
};
std::map<seeml_b200_ctx*, TcState>& states() {
  static std::map<seeml_b200_ctx*, TcState> s;
  return s;
}

// Default: a swizzled K-major tile 32 elements (128 bytes) wide; box_cols = 16 is the 64-byte
// swizzled half-width tile; any other box_cols asks for an unswizzled tile of that width
// (operands stored with the reduction index on rows) - pass unswizzled = true for those.
const CUtensorMap* cached_map(TcState& st, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows,
                              uint32_t box_cols = 0, bool unswizzled = false) {
  const uint32_t tag = unswizzled ? (box_cols | 0x10000u) : box_cols;
  const auto key = std::make_tuple(ptr, rows, cols, box_rows, tag);
  auto it = st.maps.find(key);
  if (it != st.maps.end()) return &it->second;
  CUtensorMap m;
  const int swz = unswizzled ? 0 : (box_cols == 16 ? 64 : 128);
  if (!make_map(&m, ptr, rows, cols, box_rows, box_cols ? box_cols : 32, swz)) return nullptr;
  return &st.maps.emplace(key, m).first->second;
}

// fp16 [rows, cols] row-major: box of box_rows x 32 elements (64-byte rows, 64-byte swizzle), or
// x 64 elements (128-byte rows, 128-byte swizzle) when wide.
const CUtensorMap* cached_map_f16(TcState& st, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows,
                                  bool wide = false) {
  const auto key = std::make_tuple(ptr, rows, cols, box_rows, wide ? 0x40000u : 0x20000u);
  auto it = st.maps.find(key);
  if (it != st.maps.end()) return &it->second;
  CUtensorMap m;
  if (!make_map(&m, ptr, rows, cols, box_rows, wide ? 64 : 32, wide ? 128 : 64, true)) return nullptr;
  return &st.maps.emplace(key, m).first->second;
}

// cudaFuncSetAttribute applies to the current device only, so the "already raised" note is kept
// per context (a process may hold contexts on several GPUs).
template <class K>
bool ensure_smem_attr(TcState& st, K kern, int bytes) {
  const void* fn = reinterpret_cast<const void*>(kern);
  if (st.smem_attr_done.count(fn)) return true;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  st.smem_attr_done.insert(fn);
  return true;
}

}  // namespace

bool gemm_tc_shape_ok(const seeml_b200_ctx* c, uint64_t M, uint64_t N, uint64_t K) {
  if (c->gemm_kind == SEEML_B200_GEMM_FP32_SIMT) return false;
  if (M < 128 || N < 64 || K < 32) return false;
  if (K % 4 != 0 || N % 4 != 0) return false;              // 16-byte global strides for TMA
  if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return false;
  if (2.0 * (double)M * (double)N * (double)K < 3.0e7) return false;   // too small to fill the machine
  return true;
}

namespace {

template <int BN, bool SPLIT, int STAGES, int KB = BK>
int launch_tc(seeml_b200_ctx* c, TcState& st, const TcGemm& g) {
  using S = Smem<BN, SPLIT, STAGES, KB>;
  auto kern = gemm_tc_kernel<BN, SPLIT, STAGES, KB>;
  if (!ensure_smem_attr(st, kern, S::kTotal)) return -1;
  constexpr uint32_t kw = KB == BK ? 0 : KB;
  const CUtensorMap* ma = cached_map(st, g.A, g.M, g.K, BM, kw);
  const CUtensorMap* mb = cached_map(st, g.Bt, g.N, g.K, BN, kw);
  const CUtensorMap* mc = cached_map(st, g.C, g.M, g.N, 32);
  const CUtensorMap* ma2 = g.K2 ? cached_map(st, g.A2, g.M, g.K2, BM, kw) : ma;
  const CUtensorMap* mb2 = g.K2 ? cached_map(st, g.B2t, g.N, g.K2, BN, kw) : mb;
  const float* blo = nullptr;
  if (SPLIT) {
    auto it = st.lo_copies.find(g.Bt);
    if (it != st.lo_copies.end()) blo = it->second;
  }
  const CUtensorMap* mblo = blo ? cached_map(st, blo, g.N, g.K, BN, kw) : mb;
  if (!ma || !mb || !mc || !ma2 || !mb2 || !mblo) return -1;
  TcParams p{(int)g.M, (int)g.N, (int)g.K, (int)g.K2, g.bias, g.addend, g.act, g.alpha == 0.0f ? 1.0f : g.alpha,
             blo != nullptr, 0, 0, st.err_dev};
  dim3 grid((unsigned)((g.N + BN - 1) / BN), (unsigned)((g.M + BM - 1) / BM));
  kern<<<grid, kThreadsV2, S::kTotal, c->stream>>>(*ma, *mb, *mc, *ma2, *mb2, *mblo, p);
  if (cudaGetLastError() != cudaSuccess) return -1;     // a refused launch leaves the CUDA-core path in charge
  return 1;
}

// The CTA-pair kernel for wide tiles: M tiles must pair up (an even number of 128-row tiles).
int launch_pair(seeml_b200_ctx* c, TcState& st, const TcGemm& g) {
  if (!ensure_smem_attr(st, gemm_tc_pair_kernel, PairSmem::kTotal)) return -1;
  constexpr uint32_t kw = kPairKB == BK ? 0 : kPairKB;
  const CUtensorMap* ma = cached_map(st, g.A, g.M, g.K, BM, kw);
  const CUtensorMap* mb = cached_map(st, g.Bt, g.N, g.K, 128, kw);
  const CUtensorMap* mc = cached_map(st, g.C, g.M, g.N, 32);
  const CUtensorMap* ma2 = g.K2 ? cached_map(st, g.A2, g.M, g.K2, BM, kw) : ma;
  const CUtensorMap* mb2 = g.K2 ? cached_map(st, g.B2t, g.N, g.K2, 128, kw) : mb;
  const float* blo = nullptr;
  auto it = st.lo_copies.find(g.Bt);
  if (it != st.lo_copies.end()) blo = it->second;
  const CUtensorMap* mblo = blo ? cached_map(st, blo, g.N, g.K, 128, kw) : mb;
  if (!ma || !mb || !mc || !ma2 || !mb2 || !mblo) return -1;
  TcParams p{(int)g.M, (int)g.N, (int)g.K, (int)g.K2, g.bias, g.addend, g.act, g.alpha == 0.0f ? 1.0f : g.alpha,
             blo != nullptr, 0, 0, st.err_dev};
  p.n_tiles = (int)((g.N + 255) / 256);
  p.total_tiles = p.n_tiles * (int)(((g.M + BM - 1) / BM) / 2);
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(kThreadsV2);
  cfg.dynamicSmemBytes = PairSmem::kTotal;
  cfg.stream = c->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (st.pair_clusters == 0) {       // one persistent cluster per SM pair the device can keep resident
    cfg.gridDim = dim3(2u * 1024u);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 74;
    }
    if (const char* e = std::getenv("SEEML_B200_PAIR_PERSIST"))
      if (std::atoi(e) == 0) n = 1 << 20;      // one tile per cluster (measurement aid)
    st.pair_clusters = n;
  }
  cfg.gridDim = dim3(2u * (unsigned)std::min(p.total_tiles, st.pair_clusters));
  const cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel, *ma, *mb, *mc, *ma2, *mb2, *mblo, p);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return 1;
}

// fp16 hi / lo tiles of the low-rank tail's B operand ([N, K2], K2 <= kF16TailK) and its scale.
bool ensure_tail_buffers(TcState& st) {
  if (st.tail_hi && st.tail_inv) return true;
  if ((!st.tail_hi && cudaMalloc(&st.tail_hi, 2 * kF16TailRows * kF16TailK * sizeof(__half)) != cudaSuccess) ||
      (!st.tail_inv && cudaMalloc(&st.tail_inv, kF16TailRows * sizeof(float)) != cudaSuccess)) {
    cudaGetLastError();
    return false;
  }
  st.tail_lo = st.tail_hi + kF16TailRows * kF16TailK;
  return true;
}

// The CTA-pair kernel with the two-term fp16 split. Same shape rule as launch_pair; the main
// pair's B must be a frozen operand with fp16 copies (made at build time) and the tail at most 32
// wide, otherwise the three-product tf32 kernel takes the launch.
int launch_pair_f16(seeml_b200_ctx* c, TcState& st, const TcGemm& g) {
  auto it = st.f16_copies.find(g.Bt);
  if (it == st.f16_copies.end() || g.K2 > 32 || g.N > kF16TailRows) return launch_pair(c, st, g);
  if (!ensure_smem_attr(st, gemm_tc_pair_f16_kernel, PairF16Smem::kTotal)) return -1;
  if (!st.absmax_dev && cudaMalloc(&st.absmax_dev, 64) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (!ensure_tail_buffers(st)) return -1;
  const CUtensorMap* ma = cached_map(st, g.A, g.M, g.K, BM);
  const CUtensorMap* mc = cached_map(st, g.C, g.M, g.N, 32);
  const CUtensorMap* ma2 = g.K2 ? cached_map(st, g.A2, g.M, g.K2, BM) : ma;
  const CUtensorMap* mbh = cached_map_f16(st, it->second.hi, g.N, g.K, 128);
  const CUtensorMap* mbl = cached_map_f16(st, it->second.lo, g.N, g.K, 128);
  const CUtensorMap* mb2h = g.K2 ? cached_map_f16(st, st.tail_hi, g.N, 32, 128) : mbh;
  const CUtensorMap* mb2l = g.K2 ? cached_map_f16(st, st.tail_lo, g.N, 32, 128) : mbl;
  if (!ma || !mc || !ma2 || !mbh || !mbl || !mb2h || !mb2l) return -1;
  static const int dbg = [] { const char* e = std::getenv("SEEML_B200_F16_DBG"); return e ? std::atoi(e) : 0; }();
  // max|x| of the operands converted at run time, then the tail's B as fp16 tiles
  AbsmaxArgs aa{};
  aa.ptr[0] = g.A; aa.n[0] = g.M * g.K;
  if (g.K2) { aa.ptr[2] = g.A2; aa.n[2] = g.M * g.K2; aa.ptr[3] = g.B2t; aa.n[3] = g.N * g.K2; }
  // The previous unit of the same run measured the same A (q / k / v, gate / up): nothing has
  // written it since, so its maximum is still in slot 0.
  const bool reuse_a = st.absmax_src == g.A && st.absmax_n == aa.n[0] &&
                       (c->exec_unit == st.absmax_unit || c->exec_unit == st.absmax_unit + 1) && !(dbg & 8);
  st.absmax_src = g.A; st.absmax_n = aa.n[0]; st.absmax_unit = c->exec_unit;
  if (reuse_a) { aa.ptr[0] = nullptr; aa.n[0] = 0; }
  if (!(dbg & 4) && (!reuse_a || g.K2)) {
    if (cudaMemsetAsync(st.absmax_dev + (reuse_a ? 1 : 0), 0, reuse_a ? 12 : 16, c->stream) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    const uint64_t big = std::max<uint64_t>(aa.n[0], aa.n[2]);
    const unsigned blocks = (unsigned)std::min<uint64_t>(592, (big / 4 + 1023) / 1024 + 1);
    absmax4_kernel<<<dim3(blocks, g.K2 ? 4 : 1), 256, 0, c->stream>>>(aa, st.absmax_dev);
  }
  if (g.K2)
    split_f16_tail_kernel<<<(unsigned)((g.N * 32 + 255) / 256), 256, 0, c->stream>>>(g.B2t, st.tail_hi, st.tail_lo, (int)g.N,
                                                                                  (int)g.K2, st.absmax_dev + 3);
  F16Params p{};
  p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K; p.K2 = (int)g.K2;
  p.bias = g.bias; p.addend = g.addend; p.act = g.act; p.alpha = g.alpha == 0.0f ? 1.0f : g.alpha;
  p.eb_pre = it->second.exp; p.absmax = st.absmax_dev; p.err = st.err_dev; p.dbg = dbg;
  p.n_tiles = (int)((g.N + 255) / 256);
  p.total_tiles = p.n_tiles * (int)(((g.M + BM - 1) / BM) / 2);
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(kThreadsV2);
  cfg.dynamicSmemBytes = PairF16Smem::kTotal;
  cfg.stream = c->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (st.pair_f16_clusters == 0) {
    cfg.gridDim = dim3(2u * 1024u);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_f16_kernel, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 74;
    }
    st.pair_f16_clusters = n;
  }
  cfg.gridDim = dim3(2u * (unsigned)std::min(p.total_tiles, st.pair_f16_clusters));
  const cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_tc_pair_f16_kernel, *ma, *ma2, *mc, *mbh, *mbl, *mb2h, *mb2l, p);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return 1;
}

// Makes a_hi / a_lo / a_inv hold the row-scaled fp16 split of A [M, K], unless the previous unit
// of the same run already split this very tensor (q / k / v, gate / up, a LoRA factor product and
// its GEMM): nothing has written it since. `extra` (optional) is a second, small tensor to split
// row by row in the same launch.
void split_a_rows(seeml_b200_ctx* c, TcState& st, const float* A, uint64_t M, uint64_t K, const SplitJob* extra = nullptr) {
  const bool reuse = st.split_src == A && st.split_m == M && st.split_k == K &&
                     (c->exec_unit == st.split_unit || c->exec_unit == st.split_unit + 1);
  st.split_src = A; st.split_m = M; st.split_k = K; st.split_unit = c->exec_unit;
  const SplitJob none{nullptr, nullptr, nullptr, nullptr, 0, 0};
  if (reuse) {
    if (extra) launch_split_rows((unsigned)((extra->M + 7) / 8), c->stream, *extra, none, 0);
    return;
  }
  if (extra) {
    const SplitJob ja2{A, st.a_hi, st.a_lo, st.a_inv, (int)M, (int)K};
    launch_split_rows((unsigned)std::min<uint64_t>((M + extra->M + 7) / 8, 148 * 16), c->stream, ja2, *extra, 0);
    return;
  }
  const SplitJob ja{A, st.a_hi, st.a_lo, st.a_inv, (int)M, (int)K};
  launch_split_rows((unsigned)std::min<uint64_t>((M + 7) / 8, 148 * 16), c->stream, ja, none, 0);
}

// F16X2 with pre-split operands (see gemm_tc_pair_f16p_kernel). Needs the A scratch sized at build
// time; anything it cannot take goes to launch_pair_f16. The low-rank tail may be up to 64 wide
// here (one k-block of 64 fp16 elements); the other kernels take 32, so a wider tail this launcher
// cannot serve is reported as not eligible (0) and the caller runs the group unfused.
int launch_pair_f16p(seeml_b200_ctx* c, TcState& st, const TcGemm& g) {
  auto it = st.f16_copies.find(g.Bt);
  if (it == st.f16_copies.end() || g.K2 > kF16TailK || (g.K2 % 8) != 0 || g.N > kF16TailRows || g.K % 8 != 0 ||
      g.M * g.K > st.a_cap || g.M > st.a_rows_cap || !st.a_hi)
    return g.K2 > 32 ? 0 : launch_pair_f16(c, st, g);      // the other kernels take tails up to 32 wide
  if (!ensure_smem_attr(st, gemm_tc_pair_f16p_kernel, PairF16pSmem::kTotal)) return -1;
  if (!ensure_tail_buffers(st)) return -1;
  const CUtensorMap* mah = cached_map_f16(st, st.a_hi, g.M, g.K, BM, true);
  const CUtensorMap* mal = cached_map_f16(st, st.a_lo, g.M, g.K, BM, true);
  const CUtensorMap* ma2h = g.K2 ? cached_map_f16(st, st.a2_hi, g.M, g.K2, BM, true) : mah;
  const CUtensorMap* ma2l = g.K2 ? cached_map_f16(st, st.a2_lo, g.M, g.K2, BM, true) : mal;
  const CUtensorMap* mbh = cached_map_f16(st, it->second.hi, g.N, g.K, 128, true);
  const CUtensorMap* mbl = cached_map_f16(st, it->second.lo, g.N, g.K, 128, true);
  const CUtensorMap* mb2h = g.K2 ? cached_map_f16(st, st.tail_hi, g.N, g.K2, 128, true) : mbh;
  const CUtensorMap* mb2l = g.K2 ? cached_map_f16(st, st.tail_lo, g.N, g.K2, 128, true) : mbl;
  const CUtensorMap* mc = cached_map(st, g.C, g.M, g.N, 32);
  const CUtensorMap* mbhH = cached_map_f16(st, it->second.hi, g.N, g.K, 64, true);      // 64-row boxes for half tiles
  const CUtensorMap* mblH = cached_map_f16(st, it->second.lo, g.N, g.K, 64, true);
  const CUtensorMap* mb2hH = g.K2 ? cached_map_f16(st, st.tail_hi, g.N, g.K2, 64, true) : mbhH;
  const CUtensorMap* mb2lH = g.K2 ? cached_map_f16(st, st.tail_lo, g.N, g.K2, 64, true) : mblH;
  if (!mah || !mal || !ma2h || !ma2l || !mbh || !mbl || !mb2h || !mb2l || !mc || !mbhH || !mblH || !mb2hH || !mb2lH) return -1;
  split_a_rows(c, st, g.A, g.M, g.K);
  auto row_blocks = [](uint64_t rows) { return (unsigned)std::min<uint64_t>((rows + 7) / 8, 148 * 16); };
  if (g.K2) {       // the tail's A2 [M, K2] and B2 [N, K2] in one launch
    const SplitJob j2{g.A2, st.a2_hi, st.a2_lo, st.a2_inv, (int)g.M, (int)g.K2};
    const SplitJob jb{g.B2t, st.tail_hi, st.tail_lo, st.tail_inv, (int)g.N, (int)g.K2};
    launch_split_rows(row_blocks(g.M) + kWholeBlocks, c->stream, j2, jb, 1);     // B2 is small: one scale, the last blocks
  }
  F16pParams p{};
  p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K; p.K2 = (int)g.K2;
  p.bias = g.bias; p.addend = g.addend; p.act = g.act; p.alpha = g.alpha == 0.0f ? 1.0f : g.alpha;
  p.eb_pre = it->second.exp; p.inv_a = st.a_inv; p.inv_a2 = st.a2_inv; p.inv_b2 = st.tail_inv; p.err = st.err_dev;
  p.n_tiles = (int)((g.N + 255) / 256);
  p.total_tiles = p.n_tiles * (int)(((g.M + BM - 1) / BM) / 2);
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(kThreadsV2);
  cfg.dynamicSmemBytes = PairF16pSmem::kTotal;
  cfg.stream = c->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (st.pair_f16p_clusters == 0) {
    cfg.gridDim = dim3(2u * 1024u);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_f16p_kernel, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 74;
    }
    st.pair_f16p_clusters = n;
  }
  // a partly filled last wave: its tiles are cut in two when the halves still fit one wave
  p.full_tiles = p.total_tiles;
  static const bool halves = [] { const char* e = std::getenv("SEEML_B200_F16_HALF_TILES"); return !e || std::atoi(e) != 0; }();
  const int ncl = st.pair_f16p_clusters;
  if (halves && p.total_tiles > ncl) {
    const int left = p.total_tiles % ncl;
    if (left > 0 && 2 * left <= ncl) {
      p.full_tiles = p.total_tiles - left;
      p.total_tiles = p.full_tiles + 2 * left;
    }
  }
  cfg.gridDim = dim3(2u * (unsigned)std::min(p.total_tiles, st.pair_f16p_clusters));
  const cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_tc_pair_f16p_kernel, *mah, *mal, *ma2h, *ma2l, *mbh, *mbl, *mb2h,
                                            *mb2l, *mbhH, *mblH, *mb2hH, *mb2lH, *mc, p);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return 1;
}

TcState* state_of(seeml_b200_ctx* c, bool create) {
  auto it = states().find(c);
  if (it == states().end()) {
    if (!create) return nullptr;
    it = states().emplace(c, TcState{}).first;
  }
  TcState& st = it->second;
  if (!st.err_dev && create) {
    if (cudaMalloc(&st.err_dev, 64) != cudaSuccess) return nullptr;
    cudaMemset(st.err_dev, 0, 64);
  }
  return &st;
}

}  // namespace

// Launches C = (addend +) A.Bt^T (+ A2.B2t^T) on the tensor cores. 1 = launched, 0 = not
// available for this context / shape (caller falls back), -1 = error.
int gemm_tc_launch(seeml_b200_ctx* c, const TcGemm& g) {
  if (!gemm_tc_shape_ok(c, g.M, g.N, g.K)) return 0;
  if (g.K2 && (g.K2 % 4 != 0)) return 0;
  if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.Bt) | reinterpret_cast<uintptr_t>(g.C) |
       reinterpret_cast<uintptr_t>(g.A2) | reinterpret_cast<uintptr_t>(g.B2t) |
       reinterpret_cast<uintptr_t>(g.addend)) & 15)
    return 0;
  TcState* st = state_of(c, false);
  if (!st || !st->usable || !st->err_dev) return 0;
  const bool split = kind_x3(c);
  int r;
  static const bool half_blocks = [] { const char* e = std::getenv("SEEML_B200_GEMM_KB"); return e && std::atoi(e) == 16; }();
  static const bool pairs = [] { const char* e = std::getenv("SEEML_B200_GEMM_PAIR"); return !e || std::atoi(e) != 0; }();
  const uint64_t m_tiles = (g.M + BM - 1) / BM;
  static const bool presplit = [] { const char* e = std::getenv("SEEML_B200_F16_PRESPLIT"); return !e || std::atoi(e) != 0; }();
  if (g.K2 > 32 && !(g.N >= 192 && pairs && presplit && m_tiles % 2 == 0 && c->gemm_kind == SEEML_B200_GEMM_F16X2))
    return 0;                                           // tails wider than 32: the pre-split pair kernel only
  if (g.N >= 192 && pairs && m_tiles % 2 == 0 && c->gemm_kind == SEEML_B200_GEMM_F16X2)
    r = presplit ? launch_pair_f16p(c, *st, g) : launch_pair_f16(c, *st, g);
  else if (g.N >= 192 && split && pairs && m_tiles % 2 == 0) r = launch_pair(c, *st, g);
  else if (g.N >= 192 && split && half_blocks) r = launch_tc<256, true, 4, 16>(c, *st, g);
  else if (g.N >= 192) r = split ? launch_tc<256, true, 2>(c, *st, g) : launch_tc<256, false, 4>(c, *st, g);
  else r = split ? launch_tc<128, true, 3>(c, *st, g) : launch_tc<128, false, 6>(c, *st, g);
  if (r < 0) {   // tensor maps / attributes unavailable: leave the CUDA-core path in charge
    st->usable = false;
    return 0;
  }
  return r;
}

namespace {
template <int BN, bool TA, bool TB, int STAGES>
int launch_bg(seeml_b200_ctx* c, TcState& st, const TcBatched& g) {
  using S = BgSmem<BN, TA, TB, STAGES>;
  auto kern = bgemm_tc_kernel<BN, TA, TB, STAGES>;
  if (!ensure_smem_attr(st, kern, S::kTotal)) return -1;
  const CUtensorMap* ma = TA ? cached_map(st, g.A, g.a_rows, g.a_cols, BK, BM, true) : cached_map(st, g.A, g.a_rows, g.a_cols, BM);
  const CUtensorMap* mb = TB ? cached_map(st, g.B, g.b_rows, g.b_cols, BK, BN, true) : cached_map(st, g.B, g.b_rows, g.b_cols, BN);
  const CUtensorMap* mc = cached_map(st, g.C, g.c_rows, g.c_cols, 32);
  if (!ma || !mb || !mc) return -1;
  BgParams p{};
  p.nkb = g.K / BK; p.causal = g.causal; p.alpha = g.alpha; p.H = g.H;
  for (int i = 0; i < 2; ++i) {
    p.ax[i] = g.ax[i]; p.ay[i] = g.ay[i]; p.bx[i] = g.bx[i]; p.by[i] = g.by[i]; p.cx[i] = g.cx[i]; p.cy[i] = g.cy[i];
  }
  p.x3 = kind_x3(c);
  p.err = st.err_dev;
  const int m_tiles = g.M / BM;
  p.pair_m = ((g.causal == 2 || g.causal == 3) && m_tiles % 2 == 0) ? m_tiles : 0;
  dim3 grid((unsigned)(g.N / BN), (unsigned)(p.pair_m ? m_tiles / 2 : m_tiles), (unsigned)g.batch);
  kern<<<grid, kThreadsTC, S::kTotal, c->stream>>>(*ma, *mb, *mc, p);
  if (cudaGetLastError() != cudaSuccess) return -1;
  return 1;
}

}  // namespace

// Batched per-head product on the tensor cores. 1 = launched, 0 = shape / context not
// eligible (the caller's CUDA-core path runs instead).
int gemm_tc_batched(seeml_b200_ctx* c, const TcBatched& g) {
  if (!kind_tc(c)) return 0;
  if (g.M % BM != 0 || g.N % 64 != 0 || g.K % BK != 0 || g.M <= 0 || g.N <= 0 || g.K <= 0) return 0;
  if (g.batch <= 0 || g.batch > 65535 || g.H <= 0) return 0;
  if ((g.a_cols | g.b_cols | g.c_cols) % 4 != 0) return 0;
  if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.B) | reinterpret_cast<uintptr_t>(g.C)) & 15)
    return 0;
  if ((g.a_rows | g.a_cols | g.b_rows | g.b_cols | g.c_rows | g.c_cols) >> 31) return 0;   // 32-bit TMA coordinates
  if (g.a_t && !g.b_t) return 0;
  TcState* st = state_of(c, false);
  if (!st || !st->usable || !st->err_dev) return 0;
  int r;
  if (g.a_t) r = launch_bg<64, true, true, 3>(c, *st, g);
  else if (g.b_t) r = launch_bg<64, false, true, 4>(c, *st, g);
  else r = launch_bg<64, false, false, 2>(c, *st, g);
  if (r < 0) {
    st->usable = false;
    return 0;
  }
  return 1;
}

namespace {
// The rank-r product on the pre-split copies (F16X2). 1 = launched, 0 = not eligible.
template <int BN>
int launch_rank_f16p(seeml_b200_ctx* c, TcState& st, const float* A, const float* Bnk, float* out, uint64_t M,
                     uint64_t K, float alpha) {
  using S = RankF16Smem<BN>;
  auto kern = gemm_tc_rank_f16p_kernel<BN>;
  if (!ensure_smem_attr(st, kern, S::kTotal)) return -1;
  if (!st.rank_b_hi) {
    if (cudaMalloc(&st.rank_b_hi, 2 * 64 * kRankKMax * sizeof(__half)) != cudaSuccess ||
        cudaMalloc(&st.rank_b_inv, 64 * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    st.rank_b_lo = st.rank_b_hi + 64 * kRankKMax;
  }
  const CUtensorMap* mah = cached_map_f16(st, st.a_hi, M, K, BM, true);
  const CUtensorMap* mal = cached_map_f16(st, st.a_lo, M, K, BM, true);
  const CUtensorMap* mbh = cached_map_f16(st, st.rank_b_hi, BN, K, BN, true);
  const CUtensorMap* mbl = cached_map_f16(st, st.rank_b_lo, BN, K, BN, true);
  const CUtensorMap* mc = cached_map(st, out, M, BN, 32);
  if (!mah || !mal || !mbh || !mbl || !mc) return -1;
  const SplitJob jb{Bnk, st.rank_b_hi, st.rank_b_lo, st.rank_b_inv, BN, (int)K};
  split_a_rows(c, st, A, M, K, &jb);
  RankF16Params p{(int)M, (int)K, alpha, st.a_inv, st.rank_b_inv, st.err_dev};
  kern<<<(unsigned)((M + BM - 1) / BM), kRankThreads, S::kTotal, c->stream>>>(*mah, *mal, *mbh, *mbl, *mc, p);
  if (cudaGetLastError() != cudaSuccess) return -1;
  return 1;
}
}  // namespace

// ---- rank-r (LoRA factor) products on the tensor cores -------------------------------------
// out[M,n] = alpha * A[M,K] . Bnk[n,K]^T for n in {16, 32, 64}: one CTA per 128 rows streams
// A once through a deep TMA ring (HBM-bound). 1 = launched, 0 = not eligible.
int gemm_tc_rank_n(seeml_b200_ctx* c, const float* A, const float* Bnk, float* out, uint64_t M, uint64_t n,
                   uint64_t K, float alpha) {
  if (!kind_tc(c)) return 0;
  if ((n != 16 && n != 32 && n != 64) || M < 1024 || K < 128 || K % 4 != 0) return 0;
  if (M > 0x7FFFFFFF || K > 0x7FFFFFFF) return 0;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Bnk) | reinterpret_cast<uintptr_t>(out)) & 15) return 0;
  TcState* st = state_of(c, false);
  if (!st || !st->usable || !st->err_dev) return 0;
  static const bool rank_f16 = [] { const char* e = std::getenv("SEEML_B200_F16_RANK"); return !e || std::atoi(e) != 0; }();
  if (rank_f16 && c->gemm_kind == SEEML_B200_GEMM_F16X2 && K % 8 == 0 && K <= kRankKMax && M * K <= st->a_cap &&
      M <= st->a_rows_cap && st->a_hi) {
    int rr = n == 16 ? launch_rank_f16p<16>(c, *st, A, Bnk, out, M, K, alpha)
                     : (n == 32 ? launch_rank_f16p<32>(c, *st, A, Bnk, out, M, K, alpha)
                                : launch_rank_f16p<64>(c, *st, A, Bnk, out, M, K, alpha));
    if (rr == 1) return 1;
  }
  TcGemm g{};
  g.A = A; g.Bt = Bnk; g.C = out; g.M = M; g.N = n; g.K = K; g.alpha = alpha;
  const bool split = kind_x3(c);
  int r;
  if (n == 16) r = split ? launch_tc<16, true, 6>(c, *st, g) : launch_tc<16, false, 8>(c, *st, g);
  else if (n == 32) r = split ? launch_tc<32, true, 5>(c, *st, g) : launch_tc<32, false, 8>(c, *st, g);
  else r = split ? launch_tc<64, true, 4>(c, *st, g) : launch_tc<64, false, 8>(c, *st, g);
  if (r < 0) {
    st->usable = false;
    return 0;
  }
  return 1;
}

// Scratch for the [n,K] copy of a rank-r factor stored [K,n] (at most kRankScratchFloats).
constexpr uint64_t kRankScratchFloats = 64 * 8192;
float* gemm_tc_rank_scratch(seeml_b200_ctx* c, uint64_t floats) {
  TcState* st = state_of(c, false);
  if (!st || floats > kRankScratchFloats) return nullptr;
  if (!st->rank_scratch && cudaMalloc(&st->rank_scratch, kRankScratchFloats * sizeof(float)) != cudaSuccess) {
    cudaGetLastError();
    st->rank_scratch = nullptr;
  }
  return st->rank_scratch;
}
void gemm_tc_transpose(seeml_b200_ctx* c, const float* in, float* out, uint64_t K, uint64_t N) {
  dim3 grid((unsigned)((N + 31) / 32), (unsigned)((K + 31) / 32)), block(32, 8);
  transpose_kernel<<<grid, block, 0, c->stream>>>(in, out, (int)K, (int)N);
}

// Rows per reduction chunk of the rank-r TN product: a function of the shape only (fills
// whole waves of 148 CTAs as far as the divisors of T allow), 0 when not eligible.
uint64_t gemm_tc_rank_tn_chunk_rows(uint64_t T, uint64_t big, uint64_t small) {
  // rank 64 has no CUDA-core kernel to fall back on, so it takes this path from 1024 rows on
  if ((small != 16 && small != 32 && small != 64) || big % BM != 0 || big < BM || T < (small == 64 ? 1024u : 4096u)) return 0;
  uint64_t best = 0;
  double best_eff = 0.0;
  for (uint64_t rows : {2048ull, 1024ull, 512ull}) {
    if (T % rows != 0) continue;
    const uint64_t ctas = (T / rows) * (big / BM), waves = (ctas + 147) / 148;
    const double eff = (double)ctas / (double)(waves * 148);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = rows; }
  }
  return best;
}

// partial[chunk][big][small] = sum over the chunk's rows t of W[t,big]^T S[t,small]; both
// operands are stored with the reduction index on rows and are re-laid K-major in shared
// memory. The caller sums the chunks in order. 1 = launched, 0 = not eligible.
int gemm_tc_rank_tn(seeml_b200_ctx* c, const float* W, const float* S, float* partial, uint64_t T, uint64_t big,
                    uint64_t small, uint64_t chunk_rows) {
  if (!kind_tc(c)) return 0;
  if (chunk_rows == 0 || T % chunk_rows != 0 || chunk_rows % BK != 0) return 0;
  const uint64_t chunks = T / chunk_rows;
  if (chunks > 65535 || chunks * big > 0x7FFFFFFF || T > 0x7FFFFFFF) return 0;
  if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(S) | reinterpret_cast<uintptr_t>(partial)) & 15) return 0;
  TcState* st = state_of(c, false);
  if (!st || !st->usable || !st->err_dev) return 0;
  TcBatched g{};
  g.A = W; g.B = S; g.C = partial;
  g.a_rows = T; g.a_cols = big; g.b_rows = T; g.b_cols = small; g.c_rows = chunks * big; g.c_cols = small;
  g.a_t = true; g.b_t = true;
  g.ay[0] = (int)chunk_rows; g.by[0] = (int)chunk_rows; g.cy[0] = (int)big;
  g.M = (int)big; g.N = (int)small; g.K = (int)chunk_rows; g.batch = (int)chunks; g.H = 1; g.causal = 0;
  g.alpha = 1.0f;
  int r;
  if (small == 16) r = launch_bg<16, true, true, 4>(c, *st, g);
  else if (small == 32) r = launch_bg<32, true, true, 3>(c, *st, g);
  else r = launch_bg<64, true, true, 3>(c, *st, g);
  if (r < 0) {
    st->usable = false;
    return 0;
  }
  return 1;
}

// Attention's score-shaped products with their row softmax in one kernel (head width 64,
// S <= 512, S % 128 == 0). mode 0: P[z,i,:] = softmax over the visible keys of alpha A_z[i].B_z[j]
// (A = Q, B = K). mode 1: out = Pin * (dP - rowsum(dP * Pin)) with dP = A B^T (A = dO, B = V).
// A and B are [B*S, H*64]; out / Pin are [B*H*S, S]. 1 = launched, 0 = not eligible.
static int attn_rows_launch(seeml_b200_ctx* c, int mode, const float* A, const float* Bm, const float* Pin, float* out,
                            uint64_t B, uint64_t S, uint64_t H, uint64_t dh, float alpha) {
  if (!kind_tc(c)) return 0;
  if (dh != 64 || S % BM != 0 || S > 512 || B * H == 0 || B * H > 65535) return 0;
  if ((B * S) >> 31 || (H * dh) >> 31 || (B * H * S) >> 31) return 0;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Bm) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(Pin)) & 15)
    return 0;
  TcState* st = state_of(c, false);
  if (!st || !st->usable || !st->err_dev) return 0;
  constexpr int kSmem = 12 * BM * BK * 4 + 4 * 128 * 12 + 256 + 1024;
  if (!ensure_smem_attr(*st, attn_scores_softmax_kernel<0>, kSmem) ||
      !ensure_smem_attr(*st, attn_scores_softmax_kernel<1>, kSmem)) {
    st->usable = false;
    return 0;
  }
  const CUtensorMap* mq = cached_map(*st, A, B * S, H * dh, BM);
  const CUtensorMap* mk = cached_map(*st, Bm, B * S, H * dh, BM);
  const CUtensorMap* mp = cached_map(*st, out, B * H * S, S, 32);
  if (!mq || !mk || !mp) return 0;
  AfParams p{};
  p.S = (int)S; p.H = (int)H; p.alpha = alpha;
  p.qx[0] = 0; p.qx[1] = (int)dh; p.qy[0] = (int)S; p.qy[1] = 0;
  p.pin = Pin;
  p.x3 = kind_x3(c); p.err = st->err_dev;
  dim3 grid((unsigned)(S / BM), (unsigned)(B * H));
  if (mode == 0) attn_scores_softmax_kernel<0><<<grid, kAfThreads, kSmem, c->stream>>>(*mq, *mk, *mp, p);
  else attn_scores_softmax_kernel<1><<<grid, kAfThreads, kSmem, c->stream>>>(*mq, *mk, *mp, p);
  if (cudaGetLastError() != cudaSuccess) {
    st->usable = false;
    return 0;
  }
  return 1;
}
int attn_scores_softmax_tc(seeml_b200_ctx* c, const float* Q, const float* K, float* P, uint64_t B, uint64_t S,
                           uint64_t H, uint64_t dh, float alpha) {
  return attn_rows_launch(c, 0, Q, K, nullptr, P, B, S, H, dh, alpha);
}
bool attn_rows_eligible(const seeml_b200_ctx* c, uint64_t B, uint64_t S, uint64_t H, uint64_t dh) {
  return kind_tc(c) && dh == 64 &&
         S % BM == 0 && S <= 512 && B * H > 0 && B * H <= 65535 && !((B * H * S) >> 31);
}
int attn_ds_tc(seeml_b200_ctx* c, const float* dO, const float* V, const float* P, float* dS, uint64_t B, uint64_t S,
               uint64_t H, uint64_t dh) {
  return attn_rows_launch(c, 1, dO, V, P, dS, B, S, H, dh, 1.0f);
}

// Transposed [N,K] copy of the frozen weight at `rodata_off` ([K,N]); made on first request.
const float* gemm_tc_transposed_weight(seeml_b200_ctx* c, uint64_t rodata_off, uint64_t K, uint64_t N, bool create) {
  const auto key = std::make_tuple(rodata_off, K, N);
  auto it = c->wt.find(key);
  if (it != c->wt.end()) return it->second;
  if (!create) return nullptr;
  float* t = nullptr;
  if (cudaMalloc(&t, K * N * sizeof(float)) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  const float* w = reinterpret_cast<const float*>(c->rodata + rodata_off);
  dim3 grid((unsigned)((N + 31) / 32), (unsigned)((K + 31) / 32)), block(32, 8);
  transpose_kernel<<<grid, block, 0, c->stream>>>(w, t, (int)K, (int)N);
  c->wt[key] = t;
  return t;
}

// Registers the precomputed split of a frozen B operand (device pointer `w`, [N, K] floats): the
// lo part x - tf32(x) for the three-product tf32 kernels, or - in F16X2 mode, for shapes the
// CTA-pair kernel takes - the fp16 hi / lo copies of w * 2^exp. Failure to allocate is not fatal:
// the kernels then split the operand themselves.
static int ensure_lo_copy(seeml_b200_ctx* c, const float* w, uint64_t N, uint64_t K) {
  TcState* st = state_of(c, false);
  if (!st || !kind_x3(c)) return 0;
  const uint64_t elems = N * K;
  if (c->gemm_kind == SEEML_B200_GEMM_F16X2 && N >= 192 && K % 8 == 0) {
    if (st->f16_copies.count(w)) return 0;
    if (!st->absmax_dev && cudaMalloc(&st->absmax_dev, 64) != cudaSuccess) {
      cudaGetLastError();
      st->absmax_dev = nullptr;
      return 0;
    }
    __half *hi = nullptr, *lo = nullptr;
    if (cudaMalloc(&hi, elems * sizeof(__half)) != cudaSuccess || cudaMalloc(&lo, elems * sizeof(__half)) != cudaSuccess) {
      cudaGetLastError();
      cudaFree(hi);
      return 0;
    }
    AbsmaxArgs aa{};
    aa.ptr[0] = w; aa.n[0] = elems;
    uint32_t bits = 0;
    cudaMemsetAsync(st->absmax_dev, 0, 16, c->stream);
    absmax4_kernel<<<dim3(592, 1), 256, 0, c->stream>>>(aa, st->absmax_dev);
    cudaMemcpyAsync(&bits, st->absmax_dev, 4, cudaMemcpyDeviceToHost, c->stream);
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) {
      cudaGetLastError();
      cudaFree(hi);
      cudaFree(lo);
      return 0;
    }
    const int e = f16_scale_exp(bits);
    split_f16_kernel<<<1184, 256, 0, c->stream>>>(w, hi, lo, (size_t)elems, std::ldexp(1.0f, e));
    st->f16_copies[w] = TcState::F16Copy{hi, lo, e};
    return 0;
  }
  if (st->lo_copies.count(w)) return 0;
  float* lo = nullptr;
  if (cudaMalloc(&lo, elems * sizeof(float)) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  lo_copy_kernel<<<1184, 256, 0, c->stream>>>(w, lo, (size_t)elems);
  st->lo_copies[w] = lo;
  return 0;
}

static bool tc_instr(const seeml_b200_ctx* c, const Instr& ins) {
  if (ins.opcode != kGemmNN && ins.opcode != kGemmNT) return false;
  if (ins.opcode == kGemmNN && !is_rodata(ins.in[1])) return false;   // only frozen weights have a transposed copy
  return gemm_tc_shape_ok(c, ins.out[0], ins.out[1], ins.out[2]);
}

// Scratch for the pre-split A operands of the F16X2 GEMM: grown when a program with a larger
// GEMM is built (never while running). Growing replaces buffers whose addresses captured graphs
// hold, so every graph of the context is dropped first.
static int ensure_a_split(seeml_b200_ctx* c, TcState& st, uint64_t M, uint64_t K) {
  if (M * K <= st.a_cap && M <= st.a_rows_cap) return 0;
  const uint64_t cap = std::max(st.a_cap, M * K), rows = std::max(st.a_rows_cap, M);
  cudaStreamSynchronize(c->stream);
  drop_graphs(c);
  st.maps.clear();                      // tensor maps of the old buffers
  st.split_src = nullptr;
  cudaFree(st.a_hi); cudaFree(st.a_lo); cudaFree(st.a2_hi); cudaFree(st.a2_lo); cudaFree(st.a_inv); cudaFree(st.a2_inv);
  st.a_hi = st.a_lo = st.a2_hi = st.a2_lo = nullptr;
  st.a_inv = st.a2_inv = nullptr;
  st.a_cap = st.a_rows_cap = 0;
  if (cudaMalloc(&st.a_hi, cap * 2) != cudaSuccess || cudaMalloc(&st.a_lo, cap * 2) != cudaSuccess ||
      cudaMalloc(&st.a2_hi, rows * kF16TailK * 2) != cudaSuccess || cudaMalloc(&st.a2_lo, rows * kF16TailK * 2) != cudaSuccess ||
      cudaMalloc(&st.a_inv, rows * 4) != cudaSuccess || cudaMalloc(&st.a2_inv, rows * 4) != cudaSuccess) {
    cudaGetLastError();                 // not fatal: the launcher falls back to the in-kernel split
    cudaFree(st.a_hi); cudaFree(st.a_lo); cudaFree(st.a2_hi); cudaFree(st.a2_lo); cudaFree(st.a_inv); cudaFree(st.a2_inv);
    st.a_hi = st.a_lo = st.a2_hi = st.a2_lo = nullptr;
    st.a_inv = st.a2_inv = nullptr;
    return 0;
  }
  st.a_cap = cap;
  st.a_rows_cap = rows;
  return 0;
}

int gemm_tensor_core_prepare(seeml_b200_ctx* c, const Instr& ins) {
  if (c->gemm_kind == SEEML_B200_GEMM_FP32_SIMT) return 0;
  TcState* stp = state_of(c, true);
  if (!stp) return cuda_fail(cudaGetLastError(), "tc error word");
  if (!tc_instr(c, ins)) return 0;
  if (c->gemm_kind == SEEML_B200_GEMM_F16X2 && ins.out[1] >= 192 && ((ins.out[0] + BM - 1) / BM) % 2 == 0)
    ensure_a_split(c, *stp, ins.out[0], ins.out[2]);
  if (ins.opcode == kGemmNN) {
    const float* wt = gemm_tc_transposed_weight(c, ref_off(ins.in[1]), ins.out[2], ins.out[1], true);
    if (!wt) return fail("UpdateEngine: transposed weight allocation failed");
    ensure_lo_copy(c, wt, ins.out[1], ins.out[2]);
  } else if (is_rodata(ins.in[1])) {
    ensure_lo_copy(c, reinterpret_cast<const float*>(c->rodata + ref_off(ins.in[1])), ins.out[1], ins.out[2]);
  }
  return 0;
}

int gemm_tensor_core(seeml_b200_ctx* c, const Instr& ins, int* launches) {
  if (!tc_instr(c, ins)) return 0;
  auto at = [&](uint64_t ref) {
    return reinterpret_cast<const float*>((is_rodata(ref) ? c->rodata : c->arena) + ref_off(ref));
  };
  TcGemm g{};
  g.A = at(ins.in[0]);
  g.M = ins.out[0]; g.N = ins.out[1]; g.K = ins.out[2];
  if (ins.opcode == kGemmNN) {
    g.Bt = gemm_tc_transposed_weight(c, ref_off(ins.in[1]), g.K, g.N, false);
    if (!g.Bt) return 0;
    if (ins.flags & kFlagBias) g.bias = at(ins.in[3]);
    g.act = (ins.flags & kFlagActMask) >> kFlagActShift;
  } else {
    g.Bt = at(ins.in[1]);
  }
  g.C = reinterpret_cast<float*>(c->arena + ref_off(ins.in[2]));
  const int r = gemm_tc_launch(c, g);
  if (r == 1) *launches = 1;
  return r;
}

// Nonzero when a tensor-core kernel of this context gave up on a bounded wait.
int gemm_tensor_core_error(seeml_b200_ctx* c) {
  TcState* st = state_of(c, false);
  if (!st || !st->err_dev) return 0;
  int v = 0;
  cudaMemcpyAsync(&v, st->err_dev, 4, cudaMemcpyDeviceToHost, c->stream);
  cudaStreamSynchronize(c->stream);
  return v;
}

void gemm_tensor_core_release(seeml_b200_ctx* c) {
  auto sit = states().find(c);
  if (sit == states().end()) return;
  cudaFree(sit->second.err_dev);
  cudaFree(sit->second.rank_scratch);
  for (auto& kv : sit->second.lo_copies) cudaFree(kv.second);
  for (auto& kv : sit->second.f16_copies) {
    cudaFree(kv.second.hi);
    cudaFree(kv.second.lo);
  }
  cudaFree(sit->second.absmax_dev);
  cudaFree(sit->second.tail_hi);
  cudaFree(sit->second.tail_inv);
  cudaFree(sit->second.rank_b_hi);
  cudaFree(sit->second.rank_b_inv);
  cudaFree(sit->second.a_hi); cudaFree(sit->second.a_lo); cudaFree(sit->second.a2_hi); cudaFree(sit->second.a2_lo);
  cudaFree(sit->second.a_inv); cudaFree(sit->second.a2_inv);
  states().erase(sit);
}

}  // namespace seeml_b200
