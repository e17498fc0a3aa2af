// fp32 GEMM on the tensor cores: C[M,N] = A[M,K] * B[K,N] (+ bias[N]) (+ ReLU), all row-major fp32, with
// fp32-level accuracy from three tcgen05.mma.kind::tf32 products per k step ("3xTF32").
//
// linalg.matmul on f32 is nncv's SGEMM case (tests/MatMulOptimization/MatMulDeafult.mlir:6-9 1024^3,
// MatMulNv.mlir:6-9 8192^3); its own CUDA kernel for it is an unfinished SIMT stub
// (src/libnncv/kernel/sgemm.cu:13-100) and its GPU lowering aims at 16^3 wmma tiles
// (src/nncv/compiler/Conversion/MatMulOptimize/MatMul2NvMMA.cpp:37-90).
//
// A tf32 operand keeps 10 mantissa bits, so one product is good to about 1e-3.  Every operand x is
// split into hi = x rounded to the nearest tf32 value and lo = x - hi (exact in fp32, then rounded
// to tf32 as well); A*B ~= Ahi*Bhi + Ahi*Blo + Alo*Bhi with fp32 accumulation in TMEM, the dropped
// Alo*Blo term being about 2^-24 of the product.
// Data path: kind::tf32 takes K-major operands only (an MN-major B, which the 16-bit kinds accept,
// gives wrong products -- measured), so the row-major B[K,N] is transposed on the way in.  TMA lands
// 128 x 32 fp32 tiles of A with the 128-byte swizzle; two groups of four converter warps take
// alternate stages: a thread owns one column n of the 32 x 128 B tile, reads its 32 k values with
// coalesced global loads (a warp reads 128 contiguous bytes of a row of B per load), and writes them
// as row n of the K-major hi and lo tiles in the swizzled layout; the same group rewrites the A tile
// in place as hi and writes A's lo twin at the same offsets.  One thread issues 3 x 4 MMAs per stage;
// four epilogue warps drain the accumulator (double-buffered in TMEM) through a swizzled staging slab
// and TMA stores.  Out-of-range rows/columns read as zero and are clipped on store, so N and K need
// only be multiples of 4 (16-byte row pitches of A and C).
// Every wait is bounded and abortable; a timed-out wait sets the device status word.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include <mutex>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace {

constexpr int kBN = 128;                   // N tile
constexpr int kConvWarps = 4, kConvGroups = 2, kEpiWarps = 4;
constexpr int kConvThreads = kConvWarps * 32, kEpiThreads = kEpiWarps * 32;
constexpr int kThreads = 64 + kConvGroups * kConvThreads + kEpiThreads;
constexpr int kTile = 128 * 128;           // bytes of one operand tile: 128 rows (pixels of A / columns of B) x 32 fp32
constexpr int kStageBytes = 4 * kTile;     // A, A_lo, B, B_lo
constexpr int kStages = 3;
constexpr int kSlabBytes = 128 * 128;      // 128 rows x 32 fp32

// Nearest tf32 value (10 mantissa bits; ties away from zero): rounding, unlike cutting the low bits,
// leaves no error of one sign to pile up over a long k loop (cutting gave rel-L2 1.5e-5 at K = 2048).
__device__ __forceinline__ float tf32_round(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
}

struct GtParams {
  const float* bias;
  const float* B;
  int* error_flag;
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  int relu;
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_c, const GtParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_abort;
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t sRing = base;
  const uint32_t sStage = sRing + kStages * kStageBytes;
  const uint32_t bars = sStage + 2 * kSlabBytes;
  const uint32_t full = bars, conv = bars + 8 * kStages, empty = conv + 8 * kStages;
  const uint32_t acc_full = empty + 8 * kStages, acc_empty = acc_full + 16;
  const uint32_t tmem_slot = acc_empty + 16;
  {
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (tmem_slot + 4 > raw + dyn_bytes) {
      if (threadIdx.x == 0 && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrBounds);
      return;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(full + 8 * i, 1);
      ptx::mbar_init(conv + 8 * i, kConvThreads);
      ptx::mbar_init(empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(acc_full + 8 * i, 1);
      ptx::mbar_init(acc_empty + 8 * i, kEpiThreads);
    }
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&tm_a);
    ptx::prefetch_tensormap(&tm_c);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, 4 * kBN);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  volatile int* abort_flag = &s_abort;

  const int total = p.m_tiles * p.n_tiles;
  auto item_of = [&](int i, int& m0, int& n0) {
    const int w = (int)blockIdx.x + i * (int)gridDim.x;
    if (w >= total) return false;
    const int mt = w / p.n_tiles;
    m0 = mt * 128;
    n0 = (w - mt * p.n_tiles) * kBN;
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer ----
    if (lane == 0) {
      uint32_t cnt = 0;
      bool okw = true;
      for (int i = 0; okw; ++i) {
        int m0, n0;
        if (!item_of(i, m0, n0)) break;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++cnt) {
          const uint32_t st = cnt % kStages;
          if (!ptx::mbar_wait_abortable(empty + 8 * st, ((cnt / kStages) & 1u) ^ 1u, abort_flag)) { okw = false; break; }
          ptx::mbar_arrive_expect_tx(full + 8 * st, kTile);
          ptx::tma_load_2d(sRing + st * kStageBytes, &tm_a, kb * 32, m0, full + 8 * st);
        }
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitProducer);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer ------
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc(128, kBN, 2);   // kind::tf32, fp32 accumulate, both operands K-major
      uint32_t cnt = 0, acc_cnt = 0;
      bool okw = true;
      for (int i = 0; okw; ++i) {
        int m0, n0;
        if (!item_of(i, m0, n0)) break;
        const uint32_t ab = acc_cnt & 1u;
        if (!ptx::mbar_wait_abortable(acc_empty + 8 * ab, ((acc_cnt >> 1) & 1u) ^ 1u, abort_flag)) { okw = false; break; }
        ptx::tc_fence_after();
        // two accumulators per buffer: the hi*hi products, and the two small cross terms.  The tensor core
        // cuts (does not round) every accumulation into TMEM, an error of one sign per step: keeping the
        // large sum to one step per k block of 8 instead of three makes it three times smaller
        const uint32_t d = tmem_base + ab * (2 * kBN), dl = d + kBN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++cnt) {
          const uint32_t st = cnt % kStages;
          if (!ptx::mbar_wait_abortable(conv + 8 * st, (cnt / kStages) & 1u, abort_flag)) { okw = false; break; }
          ptx::tc_fence_after();
          const uint32_t s0 = sRing + st * kStageBytes;
          const uint32_t a_hi = ptx::smem_desc_k128_lo(s0), a_lo = ptx::smem_desc_k128_lo(s0 + kTile);
          const uint32_t b_hi = ptx::smem_desc_k128_lo(s0 + 2 * kTile), b_lo = ptx::smem_desc_k128_lo(s0 + 3 * kTile);
#pragma unroll
          for (uint32_t k4 = 0; k4 < 4; ++k4) {   // k step of 8 fp32 = 32 bytes along the rows of both operands
            const uint64_t ah = ptx::desc_from_halves(a_hi + k4 * 2, ptx::kSmemDescK128Hi);
            const uint64_t al = ptx::desc_from_halves(a_lo + k4 * 2, ptx::kSmemDescK128Hi);
            const uint64_t bh = ptx::desc_from_halves(b_hi + k4 * 2, ptx::kSmemDescK128Hi);
            const uint64_t bl = ptx::desc_from_halves(b_lo + k4 * 2, ptx::kSmemDescK128Hi);
            ptx::umma_tf32(dl, al, bh, idesc, (kb | (int)k4) != 0 ? 1u : 0u);
            ptx::umma_tf32(dl, ah, bl, idesc, 1u);
            ptx::umma_tf32(d, ah, bh, idesc, (kb | (int)k4) != 0 ? 1u : 0u);
          }
          ptx::tc_commit(empty + 8 * st);
        }
        if (!okw) break;
        ptx::tc_commit(acc_full + 8 * ab);
        ++acc_cnt;
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitMma);
    }
  } else if (warp < 2 + kConvGroups * kConvWarps) {
    // ------------------------------------------------------------------ transpose B, hi / lo split ----
    const int grp = (warp - 2) / kConvWarps;           // this group takes the stages with cnt % 2 == grp
    const int t = (threadIdx.x - 64) % kConvThreads;   // 0..127: column of the B tile / share of the A tile
    const uint32_t swz = (uint32_t)(t & 7);
    uint32_t cnt = 0;
    bool okw = true;
    for (int i = 0; okw; ++i) {
      int m0, n0;
      if (!item_of(i, m0, n0)) break;
      const int n = n0 + t;
      for (int kb = 0; kb < p.k_blocks; ++kb, ++cnt) {
        if ((cnt & 1u) != (uint32_t)grp) continue;
        const uint32_t st = cnt % kStages;
        // the MMAs that read this stage last have finished: its B and lo tiles may be rewritten
        bool got = ptx::mbar_wait_abortable(empty + 8 * st, ((cnt / kStages) & 1u) ^ 1u, abort_flag);
        float bv[32];
        const float* bp = p.B + (size_t)(kb * 32) * p.N + n;
#pragma unroll
        for (int k = 0; k < 32; ++k) bv[k] = (n < p.N && kb * 32 + k < p.K) ? __ldg(bp + (size_t)k * p.N) : 0.0f;
        got = got && ptx::mbar_wait_abortable(full + 8 * st, (cnt / kStages) & 1u, abort_flag);
        if (!ptx::named_bar_and(4 + grp, kConvThreads, got)) { okw = false; break; }
        const uint32_t s0 = sRing + st * kStageBytes;
        // A at s0 -> hi in place, lo at s0 + kTile at the same (swizzled) offsets
#pragma unroll 4
        for (int c = t; c < kTile / 16; c += kConvThreads) {
          const uint32_t src = s0 + (uint32_t)c * 16u;
          float4 v;
          asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(src));
          float hi[4], lo[4];
          const float in[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            hi[e] = tf32_round(in[e]);
            lo[e] = tf32_round(in[e] - hi[e]);
          }
          asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(src), "f"(hi[0]), "f"(hi[1]), "f"(hi[2]), "f"(hi[3]) : "memory");
          asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(src + kTile), "f"(lo[0]), "f"(lo[1]), "f"(lo[2]), "f"(lo[3]) : "memory");
        }
        // column n of B becomes row t of the K-major tiles: 8 chunks of 4 k values, chunk index XOR (row % 8)
        const uint32_t brow = s0 + 2 * kTile + (uint32_t)t * 128u;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float hi[4], lo[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            hi[e] = tf32_round(bv[4 * j + e]);
            lo[e] = tf32_round(bv[4 * j + e] - hi[e]);
          }
          const uint32_t dst = brow + (((uint32_t)j ^ swz) << 4);
          asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "f"(hi[0]), "f"(hi[1]), "f"(hi[2]), "f"(hi[3]) : "memory");
          asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(dst + kTile), "f"(lo[0]), "f"(lo[1]), "f"(lo[2]), "f"(lo[3]) : "memory");
        }
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(conv + 8 * st);
      }
    }
    if (!okw && p.error_flag && t == 0) atomicCAS(p.error_flag, 0, (int)kErrWaitLoader);
  } else {
    // ------------------------------------------------------------------ epilogue --------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const bool elected = threadIdx.x == 64 + kConvGroups * kConvThreads;
    const uint32_t sw = (uint32_t)(row & 7);
    uint32_t acc_cnt = 0;
    int jglob = 0;
    bool okw = true;
    for (int i = 0; okw; ++i) {
      int m0, n0;
      if (!item_of(i, m0, n0)) break;
      const uint32_t ab = acc_cnt & 1u;
      const bool got = ptx::mbar_wait_abortable(acc_full + 8 * ab, (acc_cnt >> 1) & 1u, abort_flag);
      if (!ptx::named_bar_and(3, kEpiThreads, got)) { okw = false; break; }
      ptx::tc_fence_after();
      for (int sl = 0; sl < kBN / 32; ++sl, ++jglob) {
        const uint32_t sb = (uint32_t)jglob & 1u;
        const int ncol = n0 + sl * 32;
        uint32_t acc[32], accl[32];
        __syncwarp();
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + ab * (2 * kBN) + (uint32_t)(sl * 32), acc);
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + ab * (2 * kBN) + kBN + (uint32_t)(sl * 32), accl);
        ptx::tmem_ld_wait();
        if (sl == kBN / 32 - 1) {
          ptx::tc_fence_before();
          ptx::mbar_arrive(acc_empty + 8 * ab);
        }
        const uint32_t srow = sStage + sb * kSlabBytes + (uint32_t)row * 128u;
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          float o[4];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const int n = ncol + c4 * 4 + h;
            float a = __uint_as_float(acc[c4 * 4 + h]) + __uint_as_float(accl[c4 * 4 + h]);
            if (p.bias && n < p.N) a += __ldg(p.bias + n);
            o[h] = p.relu ? (!(a <= 0.0f) ? a : 0.0f) : a;
          }
          asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(srow + (((uint32_t)c4 ^ sw) << 4)), "f"(o[0]), "f"(o[1]),
                       "f"(o[2]), "f"(o[3])
                       : "memory");
        }
        ptx::fence_proxy_async_smem();
        ptx::named_bar_sync(1, kEpiThreads);
        if (elected) {
          if (ncol < p.N) ptx::tma_store_2d(&tm_c, ncol, m0, sStage + sb * kSlabBytes);
          ptx::bulk_commit();
          ptx::bulk_wait_read<1>();
        }
        ptx::named_bar_sync(2, kEpiThreads);
      }
      ++acc_cnt;
    }
    if (elected) ptx::bulk_wait<0>();
    if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitEpilogue);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, 4 * kBN);
  }
}

PFN_cuTensorMapEncodeTiled_v12000 gt_get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

// 2-D map over a row-major fp32 [rows, cols] matrix, box 32 columns (128 bytes) x box_rows, 128-byte swizzle.
bool gt_map(CUtensorMap* m, const void* ptr, long long rows, long long cols, int box_rows) {
  auto enc = gt_get_encode();
  if (!enc) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstr[1] = {(cuuint64_t)cols * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool gemm_tf32x3_supported(int M, int N, int K) { return M > 0 && N >= 32 && K >= 32 && N % 4 == 0 && K % 4 == 0; }

cudaError_t launch_gemm_tf32x3(const float* A, const float* B, float* C, int M, int N, int K, const float* bias, int relu,
                               int sm_count, int* error_flag, cudaStream_t stream) {
  if (!gemm_tf32x3_supported(M, N, K)) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 3) || (reinterpret_cast<uintptr_t>(C) & 15))
    return cudaErrorMisalignedAddress;
  GtParams p;
  p.bias = bias; p.B = B; p.error_flag = error_flag; p.M = M; p.N = N; p.K = K; p.relu = relu;
  p.m_tiles = (M + 127) / 128; p.n_tiles = (N + kBN - 1) / kBN; p.k_blocks = (K + 31) / 32;
  if ((long long)p.m_tiles * p.n_tiles > 0x7fffffffLL) return cudaErrorInvalidValue;
  CUtensorMap tm_a, tm_c;
  if (!gt_map(&tm_a, A, M, K, 128) || !gt_map(&tm_c, C, M, N, 128)) return cudaErrorInvalidValue;
  const size_t smem = 1024 + (size_t)kStages * kStageBytes + 2 * kSlabBytes + 256;
  cudaError_t e = cudaFuncSetAttribute(gemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int sms = sm_count > 0 ? sm_count : 148;
  const int items = p.m_tiles * p.n_tiles;
  return launch_pdl(gemm_tf32x3_kernel, dim3(items < sms ? items : sms), dim3(kThreads), smem, stream, tm_a, tm_c, p);
}

}  // namespace nncv_b200
