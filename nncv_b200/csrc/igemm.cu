// Implicit-GEMM convolution / GEMM for sm_100a on tcgen05 tensor cores.
//
// Replaces what nncv's NV-GPU lowering aimed at with wmma tiles
// (src/nncv/compiler/Conversion/CodeGen/LlvmGpu/ModernTileGpu.cpp:427-525 for matmul;
// conv was never mapped to the GPU, :556-574) and its unfinished sgemm stub
// (src/libnncv/kernel/sgemm.cu:13-100).  Semantics: linalg.conv_2d_nchw_fchw
// (tests/Nets/Res18.mlir:125) and linalg.matmul (:623) followed by the folded batch-norm,
// residual add and ReLU generics (:127-143, :193-203), computed on NHWC data.
//
// GEMM view: D[M = N*OH*OW, Kout] = A[M, R*S*C] * B[Kout, R*S*C]^T, both operands K-major.
//   * A is never materialised: four producer warps gather each 128 x 64 tile straight from
//     the NHWC activation with 16-byte cp.async (zero fill for padding and ragged rows) into
//     the 128-byte-swizzled layout tcgen05.mma reads.
//   * B is pre-packed once at weight-upload time into that same shared-memory image, so one
//     bulk async copy per stage brings a whole BN x 64 tile.
//   * One thread issues tcgen05.mma (M=128, N=BN, K=16) with the fp32 accumulator in TMEM;
//     tcgen05.commit hands stages back to the producers through mbarriers.
//   * The producer warps then become the epilogue: tcgen05.ld the accumulator, apply
//     scale/shift (+ residual) (+ ReLU), store NHWC with 128-bit accesses.
// Every mbarrier wait is bounded; a timed-out wait records a KernelError and the CTA leaves
// through the common exit that frees its TMEM.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace {

constexpr int kBM = 128;        // rows (output pixels) per CTA tile
constexpr int kBK = 64;         // 16-bit elements per k-block = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kLag = 2;         // producers publish a stage two k-blocks after issuing it
constexpr int kProducerThreads = 128;
constexpr int kThreads = 192;   // warps 0-3 gather/epilogue, warp 4 MMA, warp 5 weight loader
constexpr int kABytes = kBM * 128;

struct IgemmParams {
  const uint16_t* in;
  const uint8_t* wpack;
  const float* scale;
  const float* shift;
  const uint16_t* residual;
  void* out;
  int* error_flag;
  long long ldo;
  int M, H, W, C, OH, OW, Kout, R, S, stride, pad;
  int k_blocks;
  int relu, out_f32, bf16;
  Layout il, ol;  // input / output(+residual) layouts
};

__device__ __forceinline__ void report(int* flag, int code) {
  if (flag) atomicCAS(flag, 0, code);
}

template <int BN>
__global__ void __launch_bounds__(kThreads) conv_igemm_kernel(const IgemmParams p) {
  constexpr int kBBytes = BN * 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t sA = base;
  const uint32_t sB = base + kStages * kABytes;
  const uint32_t bars = sB + kStages * kBBytes;  // 8-byte aligned
  const uint32_t full_a = bars;
  const uint32_t full_b = bars + 8 * kStages;
  const uint32_t empty = bars + 16 * kStages;
  const uint32_t accum = bars + 24 * kStages;
  const uint32_t tmem_slot = accum + 8;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_a + 8 * s, kProducerThreads);
      ptx::mbar_init(full_b + 8 * s, 1);
      ptx::mbar_init(empty + 8 * s, 1);
    }
    ptx::mbar_init(accum, 1);
    ptx::mbar_fence_init();
  }
  if (warp == 4) {
    ptx::tmem_alloc(tmem_slot, BN);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));

  const int m_tile = blockIdx.x;
  const int n_tile = blockIdx.y;
  const int KB = p.k_blocks;

  if (warp < 4) {
    // ------------------------------------------------------------- A producer ---------
    const int row = threadIdx.x;
    const long long m_log = (long long)m_tile * kBM + row;   // logical output pixel
    const bool valid = m_log < p.M;
    int iy0 = 0, ix0 = 0;
    long long m = 0;                                          // output slot
    const uint16_t* img = p.in;
    if (valid) {
      const int ohw = p.OH * p.OW;
      const int n_img = (int)(m_log / ohw);
      const int rem = (int)(m_log - (long long)n_img * ohw);
      const int oy = rem / p.OW;
      const int ox = rem - oy * p.OW;
      iy0 = oy * p.stride - p.pad + p.il.off;
      ix0 = ox * p.stride - p.pad + p.il.off;
      img = p.in + (size_t)n_img * p.il.img_rows * p.il.pitch * p.C;
      m = ((long long)n_img * p.ol.img_rows + oy + p.ol.off) * p.ol.pitch + ox + p.ol.off;
    }
    const int y_lo = p.il.off, y_hi = p.H + p.il.off, x_lo = p.il.off, x_hi = p.W + p.il.off;
    const uint32_t row_off = (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
    const uint32_t sw = (uint32_t)(row & 7);
    int r = 0, s = 0, c0 = 0;
    bool ok_wait = true;
    for (int kb = 0; kb < KB; ++kb) {
      const int stage = kb % kStages;
      const uint32_t u = (uint32_t)(kb / kStages);
      if (!ptx::mbar_wait(empty + 8 * stage, (u & 1u) ^ 1u)) {
        report(p.error_flag, kErrWaitProducer);
        ok_wait = false;
        break;
      }
      const uint32_t dst = sA + stage * kABytes + row_off;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int iy = iy0 + r, ix = ix0 + s;
        const bool ok = valid && r < p.R && iy >= y_lo && iy < y_hi && ix >= x_lo && ix < x_hi;
        const uint16_t* src = ok ? img + ((size_t)iy * p.il.pitch + ix) * p.C + c0 : p.in;
        ptx::cp_async_16(dst + (((uint32_t)j ^ sw) << 4), src, ok ? 16u : 0u);
        c0 += 8;
        if (c0 == p.C) {
          c0 = 0;
          if (++s == p.S) {
            s = 0;
            ++r;
          }
        }
      }
      ptx::cp_async_commit();
      if (kb >= kLag) {
        ptx::cp_async_wait<kLag>();
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(full_a + 8 * ((kb - kLag) % kStages));
      }
    }
    ptx::cp_async_wait<0>();
    ptx::fence_proxy_async_smem();
    if (ok_wait) {
      for (int kb = (KB > kLag ? KB - kLag : 0); kb < KB; ++kb)
        ptx::mbar_arrive(full_a + 8 * (kb % kStages));
    }

    // ------------------------------------------------------------- epilogue -----------
    if (!ptx::mbar_wait(accum, 0)) report(p.error_flag, kErrWaitEpilogue);
    ptx::tc_fence_after();
    const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16);
    const int n_base = n_tile * BN;
    const bool vec_ok = (p.ldo % 8 == 0);
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t acc[32];
      __syncwarp();  // tcgen05.ld is warp-collective: reconverge after the ragged paths below
      ptx::tmem_ld_32x32(t_row + (uint32_t)c, acc);
      ptx::tmem_ld_wait();
      const int n0 = n_base + c;
      if (!valid || n0 >= p.Kout) continue;
      const bool full = (n0 + 32 <= p.Kout) && vec_ok;
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]);
      if (full) {
        if (p.scale) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 sc = __ldg(reinterpret_cast<const float4*>(p.scale + n0 + i));
            v[i] *= sc.x; v[i + 1] *= sc.y; v[i + 2] *= sc.z; v[i + 3] *= sc.w;
          }
        }
        if (p.shift) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 sh = __ldg(reinterpret_cast<const float4*>(p.shift + n0 + i));
            v[i] += sh.x; v[i + 1] += sh.y; v[i + 2] += sh.z; v[i + 3] += sh.w;
          }
        }
        if (p.residual) {
          const uint4* rp = reinterpret_cast<const uint4*>(p.residual + (size_t)m * p.ldo + n0);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 rv = __ldg(rp + q);
            const uint32_t w4[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              float2 f;
              if (p.bf16)
                f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[h]));
              else
                f = __half22float2(*reinterpret_cast<const __half2*>(&w4[h]));
              v[q * 8 + h * 2] += f.x;
              v[q * 8 + h * 2 + 1] += f.y;
            }
          }
        }
        if (p.relu) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = !(v[i] <= 0.0f) ? v[i] : 0.0f;
        }
        if (p.out_f32) {
          float4* op = reinterpret_cast<float4*>(static_cast<float*>(p.out) + (size_t)m * p.ldo + n0);
#pragma unroll
          for (int q = 0; q < 8; ++q) op[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else {
          uint4* op = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + (size_t)m * p.ldo + n0);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w4[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              if (p.bf16) {
                __nv_bfloat162 b = __floats2bfloat162_rn(v[q * 8 + h * 2], v[q * 8 + h * 2 + 1]);
                w4[h] = *reinterpret_cast<uint32_t*>(&b);
              } else {
                w4[h] = ptx::pack_half2_sat(v[q * 8 + h * 2], v[q * 8 + h * 2 + 1]);
              }
            }
            op[q] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
        }
      } else {
        // ragged tail (Kout not a multiple of 32, or an unaligned row pitch): scalar path
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
          const int n = n0 + i;
          if (n >= p.Kout) break;
          float x = v[i];
          if (p.scale) x *= __ldg(p.scale + n);
          if (p.shift) x += __ldg(p.shift + n);
          if (p.residual) {
            const uint16_t rv = p.residual[(size_t)m * p.ldo + n];
            x += p.bf16 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&rv))
                        : __half2float(*reinterpret_cast<const __half*>(&rv));
          }
          if (p.relu) x = !(x <= 0.0f) ? x : 0.0f;
          if (p.out_f32) {
            static_cast<float*>(p.out)[(size_t)m * p.ldo + n] = x;
          } else if (p.bf16) {
            static_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(x);
          } else {
            static_cast<uint16_t*>(p.out)[(size_t)m * p.ldo + n] = (uint16_t)(ptx::pack_half2_sat(x, 0.f) & 0xffffu);
          }
        }
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------- MMA issuer ---------
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc(kBM, BN, p.bf16 ? 1 : 0);
      for (int kb = 0; kb < KB; ++kb) {
        const int stage = kb % kStages;
        const uint32_t u = (uint32_t)(kb / kStages);
        if (!ptx::mbar_wait(full_a + 8 * stage, u & 1u) ||
            !ptx::mbar_wait(full_b + 8 * stage, u & 1u)) {
          report(p.error_flag, kErrWaitMma);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t a_addr = sA + stage * kABytes;
        const uint32_t b_addr = sB + stage * kBBytes;
#pragma unroll
        for (int k4 = 0; k4 < kBK / 16; ++k4) {
          ptx::umma_f16(tmem_base, ptx::smem_desc_k128(a_addr + k4 * 32),
                        ptx::smem_desc_k128(b_addr + k4 * 32), idesc, (kb | k4) != 0 ? 1u : 0u);
        }
        ptx::tc_commit(empty + 8 * stage);
      }
      ptx::tc_commit(accum);
    }
  } else {
    // ------------------------------------------------------------- weight loader ------
    if (lane == 0) {
      const uint8_t* src = p.wpack + (size_t)n_tile * KB * kBBytes;
      for (int kb = 0; kb < KB; ++kb) {
        const int stage = kb % kStages;
        const uint32_t u = (uint32_t)(kb / kStages);
        if (!ptx::mbar_wait(empty + 8 * stage, (u & 1u) ^ 1u)) {
          report(p.error_flag, kErrWaitLoader);
          break;
        }
        ptx::mbar_arrive_expect_tx(full_b + 8 * stage, kBBytes);
        ptx::bulk_g2s(sB + stage * kBBytes, src + (size_t)kb * kBBytes, kBBytes,
                      full_b + 8 * stage);
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, BN);
  }
}

template <int BN>
constexpr size_t igemm_smem_bytes() {
  return 1024 + (size_t)kStages * (kABytes + BN * 128) + 24 * kStages + 16 + 16;
}

// One thread per 16-byte chunk of the packed image.
template <typename SrcT, typename DstT>
__global__ void pack_weights_kernel(const SrcT* __restrict__ src, long long sn, long long sc,
                                    long long stap, int Kout, int C, int Cpad, int taps, int bn,
                                    int k_blocks, int n_tiles, DstT* __restrict__ dst) {
  const long long total = (long long)n_tiles * k_blocks * bn * 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    // consecutive threads walk consecutive rows (n) so a [K,N] row-major source coalesces
    const int rr = (int)(i % bn);
    long long t = i / bn;
    const int j = (int)(t % 8);
    t /= 8;
    const int kb = (int)(t % k_blocks);
    const int nt = (int)(t / k_blocks);
    const int n = nt * bn + rr;
    alignas(16) DstT vals[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int kidx = kb * kBK + j * 8 + e;
      const int tap = kidx / Cpad;
      const int c = kidx - tap * Cpad;
      float f = 0.0f;
      if (n < Kout && tap < taps && c < C) f = (float)src[n * sn + c * sc + tap * stap];
      vals[e] = (DstT)f;
    }
    uint8_t* tile = reinterpret_cast<uint8_t*>(dst) + ((size_t)nt * k_blocks + kb) * bn * 128;
    const size_t off = (size_t)(rr >> 3) * 1024 + (size_t)(rr & 7) * 128 + (size_t)((j ^ (rr & 7)) << 4);
    *reinterpret_cast<uint4*>(tile + off) = *reinterpret_cast<const uint4*>(vals);
  }
}

template <typename SrcT>
cudaError_t pack_dispatch(const void* src, long long sn, long long sc, long long stap, int Kout,
                          int C, int Cpad, int taps, int bn, DType dst_dt, void* dst,
                          cudaStream_t stream) {
  const int k_blocks = (taps * Cpad + kBK - 1) / kBK;
  const int n_tiles = (Kout + bn - 1) / bn;
  const long long total = (long long)n_tiles * k_blocks * bn * 8;
  const int threads = 256;
  long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dst_dt == kBF16)
    pack_weights_kernel<SrcT, __nv_bfloat16><<<blocks, threads, 0, stream>>>(
        static_cast<const SrcT*>(src), sn, sc, stap, Kout, C, Cpad, taps, bn, k_blocks, n_tiles,
        static_cast<__nv_bfloat16*>(dst));
  else
    pack_weights_kernel<SrcT, __half><<<blocks, threads, 0, stream>>>(
        static_cast<const SrcT*>(src), sn, sc, stap, Kout, C, Cpad, taps, bn, k_blocks, n_tiles,
        static_cast<__half*>(dst));
  return cudaGetLastError();
}

template <int BN>
cudaError_t launch_bn(const IgemmParams& p, int m_tiles, int n_tiles, cudaStream_t stream) {
  const size_t smem = igemm_smem_bytes<BN>();
  cudaError_t e = cudaFuncSetAttribute(conv_igemm_kernel<BN>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  conv_igemm_kernel<BN><<<dim3(m_tiles, n_tiles), kThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

int igemm_k_blocks(int C, int R, int S) { return (R * S * C + kBK - 1) / kBK; }

size_t packed_weight_bytes(int Kout, int C, int R, int S, int bn) {
  const int n_tiles = (Kout + bn - 1) / bn;
  return (size_t)n_tiles * igemm_k_blocks(C, R, S) * bn * 128;
}

// N tile: as wide as Kout allows (fewer re-gathers of A), but narrow enough that the grid
// still fills the 148 SMs.
int igemm_pick_bn(long long M, int Kout) {
  const long long m_tiles = (M + kBM - 1) / kBM;
  int bn = Kout >= 256 ? 256 : (Kout > 64 ? 128 : 64);
  while (bn > 64 && m_tiles * ((Kout + bn - 1) / bn) < 2 * 148) bn >>= 1;
  return bn;
}

cudaError_t launch_pack_weights(const void* src, DType src_dt, long long sn, long long sc,
                                long long stap, int Kout, int C, int Cpad, int taps, int bn,
                                DType dst_dt, void* dst, cudaStream_t stream) {
  if (Cpad % 8 != 0 || (bn != 64 && bn != 128 && bn != 256) || dst_dt == kF32)
    return cudaErrorInvalidValue;
  switch (src_dt) {
    case kF32: return pack_dispatch<float>(src, sn, sc, stap, Kout, C, Cpad, taps, bn, dst_dt, dst, stream);
    case kF16: return pack_dispatch<__half>(src, sn, sc, stap, Kout, C, Cpad, taps, bn, dst_dt, dst, stream);
    case kBF16: return pack_dispatch<__nv_bfloat16>(src, sn, sc, stap, Kout, C, Cpad, taps, bn, dst_dt, dst, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_conv_igemm(const IgemmArgs& a, cudaStream_t stream) {
  if (a.C % 8 != 0 || a.ab == kF32 || (a.out_dtype != kF32 && a.out_dtype != a.ab))
    return cudaErrorInvalidValue;
  IgemmParams p;
  p.in = static_cast<const uint16_t*>(a.in);
  p.wpack = static_cast<const uint8_t*>(a.wpack);
  p.scale = a.scale;
  p.shift = a.shift;
  p.residual = static_cast<const uint16_t*>(a.residual);
  p.out = a.out;
  p.error_flag = a.error_flag;
  p.ldo = a.ldo;
  const long long M = (long long)a.N * a.OH * a.OW;
  if (M <= 0 || M > 0x7fffffffLL) return cudaErrorInvalidValue;
  p.M = (int)M;
  p.H = a.H; p.W = a.W; p.C = a.C; p.OH = a.OH; p.OW = a.OW; p.Kout = a.Kout;
  p.R = a.R; p.S = a.S; p.stride = a.stride; p.pad = a.pad;
  p.k_blocks = igemm_k_blocks(a.C, a.R, a.S);
  p.il = a.in_l.pitch ? a.in_l : dense_layout(a.H, a.W);
  p.ol = a.out_l.pitch ? a.out_l : dense_layout(a.OH, a.OW);
  p.relu = a.relu;
  p.out_f32 = a.out_dtype == kF32;
  p.bf16 = a.ab == kBF16;
  const int m_tiles = (int)((M + kBM - 1) / kBM);
  const int n_tiles = (a.Kout + a.bn - 1) / a.bn;
  // 16-byte epilogue accesses need 16-byte aligned rows; the kernel falls back to scalar
  // stores when the pitch is not a multiple of 8 elements, but the base must be aligned.
  if ((reinterpret_cast<uintptr_t>(a.out) & 15) || (reinterpret_cast<uintptr_t>(a.residual) & 15) ||
      (reinterpret_cast<uintptr_t>(a.in) & 15) || (reinterpret_cast<uintptr_t>(a.wpack) & 15))
    return cudaErrorMisalignedAddress;
  switch (a.bn) {
    case 64: return launch_bn<64>(p, m_tiles, n_tiles, stream);
    case 128: return launch_bn<128>(p, m_tiles, n_tiles, stream);
    case 256: return launch_bn<256>(p, m_tiles, n_tiles, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace nncv_b200
