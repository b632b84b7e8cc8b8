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
// Warp roles (192 threads): warp 0 issues TMA loads, warp 1 owns TMEM and issues the
// MMAs, warps 2..5 split the operands during the main loop and run the epilogue.
// Every wait on an mbarrier is bounded: on expiry the kernel records an error code,
// drains, frees its TMEM and returns, so a protocol bug cannot hang the device.
//
// The frozen weight of a forward GemmNN is stored [K,N]; the context keeps a
// transposed [N,K] copy (made once, when the program is built) so forward and
// backward GEMMs through frozen weights both take this K-major form.
#include <cuda.h>

#include <cstring>

#include "backend.h"

namespace seeml_b200 {
namespace {

constexpr int BM = 128;
constexpr int BK = 32;                 // f32 elements = one 128-byte swizzle row
constexpr int kThreadsTC = 192;
constexpr uint32_t kSpinLimit = 1u << 21;

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false (and an error code left in *err) when the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err, int code) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try(bar, parity)) return true;
  atomicCAS(err, 0, code);
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: K-major tile whose rows are one 128-byte swizzle
// atom wide; 8-row groups are 1024 bytes apart. Fields (bit positions): start address
// >>4 [0,14), leading byte offset >>4 [16,30) (unused for swizzled K-major, 1),
// stride byte offset >>4 [32,46) = 64, descriptor version [46,48) = 1 on sm_100,
// layout type [61,64) = 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor, kind::tf32: D = f32 [4,6)=1, A = B = tf32 [7,10)=[10,13)=2,
// both operands K-major (bits 15, 16 = 0), N>>3 at [17,23), M>>4 at [24,29).
__host__ __device__ constexpr uint32_t idesc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct TcParams {
  int M, N, K;
  int K2;                // reduction length of the optional second operand pair (0 = none)
  const float* bias;     // nullable, length N
  const float* addend;   // nullable, [M,N] row-major: C = addend + A.B^T (+ A2.B2^T)
  int act;               // 0 none 1 relu 2 gelu 3 silu
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
template <int BN, bool SPLIT, int STAGES>
struct Smem {
  static constexpr int kABytes = BM * BK * 4;             // 16 KiB
  static constexpr int kBBytes = BN * BK * 4;
  static constexpr int kRawBytes = kABytes + kBBytes;
  static constexpr int kStageBytes = kRawBytes * (SPLIT ? 2 : 1);
  static constexpr int kEpiBytes = 4 * 32 * 128;          // one 32x32 f32 box per epilogue warp
  static constexpr int kBarBytes = 256;
  static constexpr int kTotal = STAGES * kStageBytes + kEpiBytes + kBarBytes + 1024;  // + alignment slack
};

template <int BN, bool SPLIT, int STAGES>
__global__ void __launch_bounds__(kThreadsTC, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapA2,
               const __grid_constant__ CUtensorMap mapB2, TcParams p) {
  using S = Smem<BN, SPLIT, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t epi = base + STAGES * S::kStageBytes;
  const uint32_t bars = epi + S::kEpiBytes;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_split = [&](int s) { return bars + 8u * (STAGES + s); };
  auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };
  const uint32_t bar_accum = bars + 8u * (3 * STAGES);
  const uint32_t tmem_slot = bars + 8u * (3 * STAGES + 1);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + STAGES * S::kStageBytes + S::kEpiBytes + 8 * (3 * STAGES + 1));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  // k-blocks of the main pair, then of the low-rank pair (C += A2[M,K2] . B2[N,K2]^T): the
  // LoRA term rides the same accumulator as extra reduction steps
  const int nkb1 = (p.K + BK - 1) / BK;
  const int nkb = nkb1 + (p.K2 + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_split(s), 128);
      mbar_init(bar_empty(s), 1);
    }
    mbar_init(bar_accum, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, BN);
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
        const uint32_t a_dst = base + s * S::kStageBytes, b_dst = a_dst + S::kABytes;
        mbar_expect_tx(bar_full(s), S::kRawBytes);
        if (kb < nkb1) {
          tma_load_2d(a_dst, &mapA, bar_full(s), kb * BK, m0);
          tma_load_2d(b_dst, &mapB, bar_full(s), kb * BK, n0);
        } else {
          tma_load_2d(a_dst, &mapA2, bar_full(s), (kb - nkb1) * BK, m0);
          tma_load_2d(b_dst, &mapB2, bar_full(s), (kb - nkb1) * BK, n0);
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
      constexpr uint32_t idesc = idesc_tf32(BM, BN);
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % STAGES, r = kb / STAGES;
        ok = mbar_wait(SPLIT ? bar_split(s) : bar_full(s), r & 1, p.err, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_raw = base + s * S::kStageBytes, b_raw = a_raw + S::kABytes;
        const uint32_t a_lo = a_raw + S::kRawBytes, b_lo = b_raw + S::kRawBytes;
#pragma unroll
        for (int kk = 0; kk < BK / 8; ++kk) {
          const uint64_t da = smem_desc_sw128(a_raw + kk * 32), db = smem_desc_sw128(b_raw + kk * 32);
          mma_tf32(tmem_base, da, db, idesc, (kb | kk) != 0);
          if (SPLIT) {
            mma_tf32(tmem_base, smem_desc_sw128(a_lo + kk * 32), db, idesc, 1);
            mma_tf32(tmem_base, da, smem_desc_sw128(b_lo + kk * 32), idesc, 1);
          }
        }
        mma_commit(bar_empty(s));
      }
      if (ok) mma_commit(bar_accum);
    }
  } else {
    // ---- split warps, then epilogue -----------------------------------------------------
    const int t = threadIdx.x - 64;
    bool ok = true;
    if (SPLIT) {
      constexpr int NV = S::kRawBytes / 16;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % STAGES, r = kb / STAGES;
        ok = mbar_wait(bar_full(s), r & 1, p.err, 3);
        if (!ok) break;
        const float4* raw = reinterpret_cast<const float4*>(base_ptr + s * S::kStageBytes);
        float4* lo = reinterpret_cast<float4*>(base_ptr + s * S::kStageBytes + S::kRawBytes);
#pragma unroll 4
        for (int i = t; i < NV; i += 128) {
          const float4 v = raw[i];
          float4 l;
          l.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
          l.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
          l.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
          l.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
          lo[i] = l;
        }
        fence_async_smem();
        mbar_arrive(bar_split(s));
      }
    }
    if (ok) ok = mbar_wait(bar_accum, 0, p.err, 4);
    tc_fence_after();
    const int q = warp & 3;                     // TMEM lane quadrant this warp may read
    const int row0 = q * 32;
    if (ok && m0 + row0 < p.M) {
      const uint32_t stage = epi + q * 4096;
      uint8_t* stage_ptr = base_ptr + STAGES * S::kStageBytes + q * 4096;
      for (int c = 0; c < BN / 32; ++c) {
        const int ncol = n0 + c * 32;
        if (ncol >= p.N) break;
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)row0 << 16) + c * 32, r);
        tmem_ld_wait();
        if (p.addend != nullptr && m0 + row0 + lane < p.M) {
          const float* arow = p.addend + (size_t)(m0 + row0 + lane) * p.N + ncol;
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
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
          for (int j = 0; j < 32; ++j) {
            float v = __uint_as_float(r[j]);
            if (p.bias != nullptr && ncol + j < p.N) v = v + p.bias[ncol + j];
            r[j] = __float_as_uint(epi_act(p.act, v));
          }
        }
        if (c > 0) {
          if (lane == 0) tma_store_wait_read();   // the staging box of the previous chunk is free
          __syncwarp();
        }
        // row = lane; 16-byte chunk j lands at (j ^ (row & 7)): the 128-byte swizzle the store expects
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          *reinterpret_cast<uint4*>(stage_ptr + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&mapC, stage, ncol, m0 + row0);
          tma_store_commit();
        }
      }
      if (lane == 0) tma_store_wait_all();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, BN);
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

// 2-D f32 row-major tensor [rows, cols] (cols contiguous), box [box_rows, box_cols], 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows,
              uint32_t box_cols) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 4};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct TcState {
  int* err_dev = nullptr;
  bool attrs_set = false;
  bool usable = true;
  std::map<std::tuple<const void*, uint64_t, uint64_t, uint32_t>, CUtensorMap> maps;
};
std::map<seeml_b200_ctx*, TcState>& states() {
  static std::map<seeml_b200_ctx*, TcState> s;
  return s;
}

const CUtensorMap* cached_map(TcState& st, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  const auto key = std::make_tuple(ptr, rows, cols, box_rows);
  auto it = st.maps.find(key);
  if (it != st.maps.end()) return &it->second;
  CUtensorMap m;
  if (!make_map(&m, ptr, rows, cols, box_rows, 32)) return nullptr;
  return &st.maps.emplace(key, m).first->second;
}

}  // namespace

bool gemm_tc_shape_ok(const seeml_b200_ctx* c, uint64_t M, uint64_t N, uint64_t K) {
  if (c->gemm_kind == SEEML_B200_GEMM_FP32_SIMT || c->gemm_kind == SEEML_B200_GEMM_BF16) return false;
  if (M < 128 || N < 64 || K < 32) return false;
  if (K % 4 != 0 || N % 4 != 0) return false;              // 16-byte global strides for TMA
  if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return false;
  if (2.0 * (double)M * (double)N * (double)K < 3.0e7) return false;   // too small to fill the machine
  return true;
}

namespace {

template <int BN, bool SPLIT, int STAGES>
int launch_tc(seeml_b200_ctx* c, TcState& st, const TcGemm& g) {
  using S = Smem<BN, SPLIT, STAGES>;
  auto kern = gemm_tc_kernel<BN, SPLIT, STAGES>;
  static bool attr_done = false;
  if (!attr_done) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    attr_done = true;
  }
  const CUtensorMap* ma = cached_map(st, g.A, g.M, g.K, BM);
  const CUtensorMap* mb = cached_map(st, g.Bt, g.N, g.K, BN);
  const CUtensorMap* mc = cached_map(st, g.C, g.M, g.N, 32);
  const CUtensorMap* ma2 = g.K2 ? cached_map(st, g.A2, g.M, g.K2, BM) : ma;
  const CUtensorMap* mb2 = g.K2 ? cached_map(st, g.B2t, g.N, g.K2, BN) : mb;
  if (!ma || !mb || !mc || !ma2 || !mb2) return -1;
  TcParams p{(int)g.M, (int)g.N, (int)g.K, (int)g.K2, g.bias, g.addend, g.act, st.err_dev};
  dim3 grid((unsigned)((g.N + BN - 1) / BN), (unsigned)((g.M + BM - 1) / BM));
  kern<<<grid, kThreadsTC, S::kTotal, c->stream>>>(*ma, *mb, *mc, *ma2, *mb2, p);
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
  const bool split = c->gemm_kind == SEEML_B200_GEMM_TF32X3;
  int r;
  if (g.N >= 192) r = split ? launch_tc<256, true, 2>(c, *st, g) : launch_tc<256, false, 4>(c, *st, g);
  else r = split ? launch_tc<128, true, 3>(c, *st, g) : launch_tc<128, false, 6>(c, *st, g);
  if (r < 0) {   // tensor maps / attributes unavailable: leave the CUDA-core path in charge
    st->usable = false;
    return 0;
  }
  return 1;
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

static bool tc_instr(const seeml_b200_ctx* c, const Instr& ins) {
  if (ins.opcode != kGemmNN && ins.opcode != kGemmNT) return false;
  if (ins.opcode == kGemmNN && !is_rodata(ins.in[1])) return false;   // only frozen weights have a transposed copy
  return gemm_tc_shape_ok(c, ins.out[0], ins.out[1], ins.out[2]);
}

int gemm_tensor_core_prepare(seeml_b200_ctx* c, const Instr& ins) {
  if (c->gemm_kind == SEEML_B200_GEMM_FP32_SIMT || c->gemm_kind == SEEML_B200_GEMM_BF16) return 0;
  if (!state_of(c, true)) return cuda_fail(cudaGetLastError(), "tc error word");
  if (!tc_instr(c, ins)) return 0;
  if (ins.opcode == kGemmNN &&
      !gemm_tc_transposed_weight(c, ref_off(ins.in[1]), ins.out[2], ins.out[1], true))
    return fail("UpdateEngine: transposed weight allocation failed");
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
  states().erase(sit);
}

}  // namespace seeml_b200
