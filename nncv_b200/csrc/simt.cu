// CUDA-core kernels of the forward pass: the fp32-accurate convolution / GEMM, and the
// memory-bound helpers (layout conversion, max-pool, global average pool, batch-norm folding).
//
// Reference semantics (nncv tree): tests/Nets/Res18.mlir:125 (conv), :127-137 (batch-norm,
// folded here into per-channel scale/shift), :138-143 (ReLU with unordered compare, NaN passes),
// :144-151 (max-pool over a -inf padded map), :606-614 (sum-pool / HW), :193-197 (residual add).
// All activations are NHWC; every helper moves 16 bytes per access.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cfloat>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace cg = cooperative_groups;

namespace {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
// finite values beyond the fp16 range saturate to +-65504 (NaN stays NaN), as in the conv epilogues
template <> __device__ __forceinline__ __half from_f<__half>(float v) {
  const unsigned short b = (unsigned short)(ptx::pack_half2_sat(v, 0.f) & 0xffffu);
  return __ushort_as_half(b);
}
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ------------------------------------------------------------------ fp32 conv ------------
// Implicit GEMM on CUDA cores: 64 x 64 output tile, k step 16, 256 threads, 4 x 4 per thread.
constexpr int kTM = 64, kTN = 64, kTK = 16;

struct SimtParams {
  const float* in;
  const float* w;
  const float* scale;
  const float* shift;
  const float* residual;
  float* out;
  long long ldo;
  int M, H, W, C, OH, OW, Kout, R, S, stride, pad, Kred;
  int relu;
  int splits;        // > 1: blockIdx.z takes one slice of the reduction and writes raw sums to `partial`
  int k_chunk;       // reduction elements per slice (a multiple of kTK)
  float* partial;    // [splits][M][Kout]
};

__global__ void __launch_bounds__(256) conv_simt_f32_kernel(const SimtParams p) {
  __shared__ float As[kTK][kTM + 4];
  __shared__ float Bs[kTK][kTN + 4];
  const int t = threadIdx.x;
  const int lrow = t >> 2;        // 0..63: tile row (A) / tile column (B) this thread loads
  const int lk = (t & 3) * 4;     // k offset of its float4
  const long long m = (long long)blockIdx.x * kTM + lrow;
  const bool mvalid = m < p.M;
  int iy0 = 0, ix0 = 0;
  const float* img = p.in;
  if (mvalid) {
    const int ohw = p.OH * p.OW;
    const int n_img = (int)(m / ohw);
    const int rem = (int)(m - (long long)n_img * ohw);
    const int oy = rem / p.OW, ox = rem - oy * p.OW;
    iy0 = oy * p.stride - p.pad;
    ix0 = ox * p.stride - p.pad;
    img = p.in + (size_t)n_img * p.H * p.W * p.C;
  }
  const int nb = blockIdx.y * kTN + lrow;
  const bool nvalid = nb < p.Kout;
  const int ty = t >> 4, tx = t & 15;
  float acc[4][4] = {};
  const int k_begin = p.splits > 1 ? (int)blockIdx.z * p.k_chunk : 0;
  const int k_end = p.splits > 1 ? min(p.Kred, k_begin + p.k_chunk) : p.Kred;
  for (int k0 = k_begin; k0 < k_end; k0 += kTK) {
    const int kidx = k0 + lk;
    float4 av = make_float4(0.f, 0.f, 0.f, 0.f), bv = av;
    if (kidx < k_end) {
      const int tap = kidx / p.C, c0 = kidx - tap * p.C;
      const int r = tap / p.S, s = tap - r * p.S;
      const int iy = iy0 + r, ix = ix0 + s;
      if (mvalid && (unsigned)iy < (unsigned)p.H && (unsigned)ix < (unsigned)p.W)
        av = __ldg(reinterpret_cast<const float4*>(img + ((size_t)iy * p.W + ix) * p.C + c0));
      if (nvalid) bv = __ldg(reinterpret_cast<const float4*>(p.w + (size_t)nb * p.Kred + kidx));
    }
    As[lk][lrow] = av.x; As[lk + 1][lrow] = av.y; As[lk + 2][lrow] = av.z; As[lk + 3][lrow] = av.w;
    Bs[lk][lrow] = bv.x; Bs[lk + 1][lrow] = bv.y; Bs[lk + 2][lrow] = bv.z; Bs[lk + 3][lrow] = bv.w;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float aa[4] = {a.x, a.y, a.z, a.w}, bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(aa[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long mo = (long long)blockIdx.x * kTM + ty * 4 + i;
    if (mo >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = blockIdx.y * kTN + tx * 4 + j;
      if (n >= p.Kout) continue;
      float v = acc[i][j];
      if (p.splits > 1) {   // the epilogue runs in conv_simt_reduce_kernel, over the slices in a fixed order
        p.partial[((size_t)blockIdx.z * p.M + mo) * p.Kout + n] = v;
        continue;
      }
      if (p.scale) v *= __ldg(p.scale + n);
      if (p.shift) v += __ldg(p.shift + n);
      if (p.residual) v += p.residual[(size_t)mo * p.ldo + n];
      if (p.relu) v = !(v <= 0.0f) ? v : 0.0f;
      p.out[(size_t)mo * p.ldo + n] = v;
    }
  }
}

// Second pass of a split reduction: out = epilogue(sum over the slices, in slice order).
__global__ void conv_simt_reduce_kernel(const SimtParams p) {
  const long long total = (long long)p.M * p.Kout;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long mo = i / p.Kout;
    const int n = (int)(i - mo * p.Kout);
    float v = 0.0f;
    for (int z = 0; z < p.splits; ++z) v += p.partial[(size_t)z * total + i];
    if (p.scale) v *= __ldg(p.scale + n);
    if (p.shift) v += __ldg(p.shift + n);
    if (p.residual) v += p.residual[(size_t)mo * p.ldo + n];
    if (p.relu) v = !(v <= 0.0f) ? v : 0.0f;
    p.out[(size_t)mo * p.ldo + n] = v;
  }
}

template <typename SrcT>
__global__ void repack_weights_f32_kernel(const SrcT* __restrict__ src, long long sn, long long sc,
                                          long long stap, int Kout, int C, int Cpad, int taps,
                                          float* __restrict__ dst) {
  const long long total = (long long)Kout * taps * Cpad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cpad);
    long long t = i / Cpad;
    const int tap = (int)(t % taps);
    const int n = (int)(t / taps);
    dst[i] = c < C ? to_f<SrcT>(src[n * sn + c * sc + tap * stap]) : 0.0f;
  }
}

// ------------------------------------------------------------------ layout ---------------
// NCHW -> NHWC with the channel count padded to Cpad (zeros); one thread per pixel.
template <typename SrcT, typename DstT>
__global__ void nchw_to_nhwc_kernel(const SrcT* __restrict__ src, DstT* __restrict__ dst, int N,
                                    int C, long long HW, int Cpad) {
  const long long total = (long long)N * HW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long n = i / HW, px = i - n * HW;
    const SrcT* s = src + (size_t)n * C * HW + px;
    DstT* d = dst + (size_t)i * Cpad;
    if (sizeof(DstT) == 2 && Cpad == 8) {
      alignas(16) DstT v[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) v[c] = from_f<DstT>(c < C ? to_f<SrcT>(s[(size_t)c * HW]) : 0.0f);
      *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(v);
    } else if (sizeof(DstT) == 4 && Cpad == 4) {
      alignas(16) DstT v[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) v[c] = from_f<DstT>(c < C ? to_f<SrcT>(s[(size_t)c * HW]) : 0.0f);
      *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(v);
    } else {
      for (int c = 0; c < Cpad; ++c) d[c] = from_f<DstT>(c < C ? to_f<SrcT>(s[(size_t)c * HW]) : 0.0f);
    }
  }
}

// ------------------------------------------------------------------ pooling --------------
template <typename T> struct Pair { using type = float2; };
template <> struct Pair<__half> {
  using type = __half2;
  static __device__ __forceinline__ __half2 neg_inf() { return __half2half2(__ushort_as_half((unsigned short)0xfc00)); }
};
template <> struct Pair<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ __nv_bfloat162 neg_inf() { return __bfloat162bfloat162(__ushort_as_bfloat16((unsigned short)0xff80)); }
};

// Max-pool over a -inf padded map; one thread per (output pixel, 16-byte channel vector).
template <typename T>
__global__ void maxpool_nhwc_kernel(const T* __restrict__ src, T* __restrict__ dst, int N, int H,
                                    int W, int C, int OH, int OW, int k, int stride, int pad,
                                    Layout il, Layout ol) {
  constexpr int V = 16 / sizeof(T);
  const int cv = C / V;
  // the launcher keeps the count of (output pixel, vector) items below 2^31: the index arithmetic is
  // 32-bit (four 64-bit divisions would cost more than the nine loads and maxima together)
  const unsigned total = (unsigned)N * OH * OW * cv;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    unsigned t = i / (unsigned)cv;
    const int c = (int)(i - t * cv) * V;
    const unsigned t2 = t / (unsigned)OW;
    const int ox = (int)(t - t2 * OW);
    const int n = (int)(t2 / (unsigned)OH);
    const int oy = (int)(t2 - (unsigned)n * OH);
    alignas(16) T o[V];
    if constexpr (sizeof(T) == 2) {
      // 16-bit types: the maximum is exact in the storage type, so it is taken on packed pairs
      // (NaN-propagating, like the scalar form below) without a round trip through fp32.
      using T2 = typename Pair<T>::type;
      T2 m2[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) m2[e] = Pair<T>::neg_inf();
      for (int r = 0; r < k; ++r) {
        const int iy = oy * stride - pad + r;
        if ((unsigned)iy >= (unsigned)H) continue;
        for (int s = 0; s < k; ++s) {
          const int ix = ox * stride - pad + s;
          if ((unsigned)ix >= (unsigned)W) continue;
          const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
              src + (((size_t)n * il.img_rows + iy + il.off) * il.pitch + ix + il.off) * C + c));
          const T2* v2 = reinterpret_cast<const T2*>(&raw);
#pragma unroll
          for (int e = 0; e < 4; ++e) m2[e] = __hmax2_nan(m2[e], v2[e]);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) reinterpret_cast<T2*>(o)[e] = m2[e];
    } else {
      float m[V];
#pragma unroll
      for (int e = 0; e < V; ++e) m[e] = -INFINITY;
      for (int r = 0; r < k; ++r) {
        const int iy = oy * stride - pad + r;
        if ((unsigned)iy >= (unsigned)H) continue;
        for (int s = 0; s < k; ++s) {
          const int ix = ox * stride - pad + s;
          if ((unsigned)ix >= (unsigned)W) continue;
          const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
              src + (((size_t)n * il.img_rows + iy + il.off) * il.pitch + ix + il.off) * C + c));
          const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int e = 0; e < V; ++e) {
            const float f = to_f<T>(v[e]);
            m[e] = (m[e] < f || f != f) ? f : m[e];  // maximumf: NaN propagates
          }
        }
      }
#pragma unroll
      for (int e = 0; e < V; ++e) o[e] = from_f<T>(m[e]);
    }
    *reinterpret_cast<uint4*>(dst + (((size_t)n * ol.img_rows + oy + ol.off) * ol.pitch + ox + ol.off) * C + c) =
        *reinterpret_cast<const uint4*>(o);
  }
}

// Global average pool: sum in fp32 over HW then divide by HW.  Eight adjacent lanes share one
// (image, 16-byte channel vector): each sums every eighth pixel, a shuffle tree adds the partial
// sums, the first lane stores.  (One thread per vector would walk the map as a chain of dependent
// loads and take ~15 us however small the tensor.)
template <typename T>
__global__ void avgpool_nhwc_kernel(const T* __restrict__ src, T* __restrict__ dst, int N, int H,
                                    int W, int C, Layout il) {
  const int HW = H * W;
  constexpr int V = 16 / sizeof(T);
  constexpr int kSlices = 8;
  const int cv = C / V;
  const long long total = (long long)N * cv * kSlices;   // a multiple of 8: whole groups of lanes
  for (long long i0 = blockIdx.x * (long long)blockDim.x; i0 < total; i0 += (long long)gridDim.x * blockDim.x) {
    const long long i = i0 + threadIdx.x;
    const bool live = i < total;
    const int slice = (int)(i % kSlices);
    const long long g = live ? i / kSlices : 0;
    const int c = (int)(g % cv) * V;
    const int n = (int)(g / cv);
    float s[V];
#pragma unroll
    for (int e = 0; e < V; ++e) s[e] = 0.0f;
    if (live) {
      for (int px = slice; px < HW; px += kSlices) {
        const int y = px / W, x = px - y * W;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
            src + (((size_t)n * il.img_rows + y + il.off) * il.pitch + x + il.off) * C + c));
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int e = 0; e < V; ++e) s[e] += to_f<T>(v[e]);
      }
    }
#pragma unroll
    for (int d = 1; d < kSlices; d <<= 1)
#pragma unroll
      for (int e = 0; e < V; ++e) s[e] += __shfl_xor_sync(0xffffffffu, s[e], d);
    if (live && slice == 0) {
      alignas(16) T o[V];
#pragma unroll
      for (int e = 0; e < V; ++e) o[e] = from_f<T>(s[e] / (float)HW);
      *reinterpret_cast<uint4*>(dst + (size_t)n * C + c) = *reinterpret_cast<const uint4*>(o);
    }
  }
}

// Global average pool of a large map (squeeze-and-excitation on early layers): a cluster of eight CTAs per
// (image, group of up to 256 channel vectors), each CTA summing one eighth of the pixels with
// threads laid out [pixel slice][channel vector] so that a warp reads whole pixels; the CTA's
// slices are added through shared memory, the eight CTA totals through distributed shared memory
// by the cluster's first CTA, in a fixed order.  No scratch memory, no atomics.
constexpr int kPoolCluster = 8;
template <typename T>
__global__ void __cluster_dims__(kPoolCluster, 1, 1) __launch_bounds__(256)
avgpool_cluster_kernel(const T* __restrict__ src, T* __restrict__ dst, int N, int H, int W, int C, Layout il) {
  constexpr int V = 16 / sizeof(T);
  __shared__ __align__(16) float part[256 * V];     // [slice][vector][V]
  __shared__ __align__(16) float tot[256 * V];      // [vector][V]: this CTA's sum
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int n = blockIdx.y;
  const int cv = C / V;
  const int v0 = blockIdx.z * 256;
  const int cvb = min(256, cv - v0);
  const int ps = 256 / cvb;
  const int slice = threadIdx.x / cvb, vc = threadIdx.x - slice * cvb;
  const int HW = H * W;
  const int lo = (int)((long long)HW * rank / kPoolCluster), hi = (int)((long long)HW * (rank + 1) / kPoolCluster);
  float s[V];
#pragma unroll
  for (int e = 0; e < V; ++e) s[e] = 0.0f;
  if (slice < ps) {
    if (il.off == 0 && il.pitch == W && il.img_rows == H) {
      // dense map: pixels are C elements apart, no row arithmetic
      const T* ptr = src + ((size_t)n * HW + lo + slice) * C + (size_t)(v0 + vc) * V;
      const size_t step = (size_t)ps * C;
#pragma unroll 4
      for (int px = lo + slice; px < hi; px += ps, ptr += step) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(ptr));
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int e = 0; e < V; ++e) s[e] += to_f<T>(v[e]);
      }
    } else {
#pragma unroll 4
      for (int px = lo + slice; px < hi; px += ps) {
        const int y = px / W, x = px - y * W;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
            src + (((size_t)n * il.img_rows + y + il.off) * il.pitch + x + il.off) * C + (size_t)(v0 + vc) * V));
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int e = 0; e < V; ++e) s[e] += to_f<T>(v[e]);
      }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) part[(slice * cvb + vc) * V + e] = s[e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < cvb * V; i += blockDim.x) {
    float a = 0.0f;
    for (int q = 0; q < ps; ++q) a += part[q * cvb * V + i];
    tot[i] = a;
  }
  cluster.sync();
  if (rank == 0) {
    for (int i = threadIdx.x; i < cvb * V; i += blockDim.x) {
      float a = 0.0f;
#pragma unroll
      for (int q = 0; q < kPoolCluster; ++q) a += *cluster.map_shared_rank(&tot[i], q);
      dst[(size_t)n * C + (size_t)v0 * V + i] = from_f<T>(a / (float)HW);
    }
  }
  cluster.sync();      // the other CTAs' shared memory stays alive until the first has read it
}

// Layout change, one thread per 16-byte vector of a destination slot; pads are written as zero.
__global__ void relayout_kernel(const uint4* __restrict__ src, Layout sl, uint4* __restrict__ dst,
                                Layout dl, int N, int H, int W, int cv) {
  const long long total = (long long)N * dl.img_rows * dl.pitch * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cv);
    long long t = i / cv;
    const int xs = (int)(t % dl.pitch);
    t /= dl.pitch;
    const int ys = (int)(t % dl.img_rows);
    const int n = (int)(t / dl.img_rows);
    const int y = ys - dl.off, x = xs - dl.off;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (y >= 0 && y < H && x >= 0 && x < W)
      v = __ldg(src + (((size_t)n * sl.img_rows + y + sl.off) * sl.pitch + x + sl.off) * cv + c);
    dst[i] = v;
  }
}

template <typename T>
__global__ void bn_fold_kernel(const T* gamma, const T* beta, const T* mean, const T* var, int C, float eps,
                               float* scale, float* shift) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  // eps: arith.truncf of the module's f64 constant (1e-5 in Res18.mlir:113,129; 1e-3 in MobileNetV3.mlir)
  const float rs = 1.0f / sqrtf(to_f<T>(var[c]) + eps);
  const float sc = to_f<T>(gamma[c]) * rs;
  scale[c] = sc;
  shift[c] = to_f<T>(beta[c]) - to_f<T>(mean[c]) * sc;
}

template <typename S, typename D>
__global__ void convert_kernel(const S* __restrict__ src, D* __restrict__ dst, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = from_f<D>(to_f<S>(src[i]));
}

inline int grid_for(long long total, int threads) {
  long long b = (total + threads - 1) / threads;
  const long long cap = 148LL * 32;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

template <typename F>
cudaError_t by_dtype(DType t, F&& f) {
  switch (t) {
    case kF32: return f(float{});
    case kF16: return f(__half{});
    case kBF16: return f(__nv_bfloat16{});
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_conv_simt_f32(const SimtConvArgs& a, cudaStream_t stream) {
  if (a.C % 4 != 0) return cudaErrorInvalidValue;
  SimtParams p;
  p.in = a.in; p.w = a.w; p.scale = a.scale; p.shift = a.shift; p.residual = a.residual; p.out = a.out;
  p.ldo = a.ldo;
  const long long M = (long long)a.N * a.OH * a.OW;
  if (M <= 0 || M > 0x7fffffffLL) return cudaErrorInvalidValue;
  p.M = (int)M; p.H = a.H; p.W = a.W; p.C = a.C; p.OH = a.OH; p.OW = a.OW; p.Kout = a.Kout;
  p.R = a.R; p.S = a.S; p.stride = a.stride; p.pad = a.pad; p.Kred = a.R * a.S * a.C; p.relu = a.relu;
  dim3 grid((unsigned)((M + kTM - 1) / kTM), (unsigned)((a.Kout + kTN - 1) / kTN));
  // Few output tiles and a long reduction (one image, late layers: 8 CTAs walking K = 4608): slice the reduction
  // over blockIdx.z so that the GPU is filled, raw sums to scratch, epilogue in a second pass.
  p.splits = 1; p.k_chunk = p.Kred; p.partial = nullptr;
  const long long ctas = (long long)grid.x * grid.y;
  const int sms = a.sm_count > 0 ? a.sm_count : 148;
  if (a.scratch && ctas < sms && p.Kred >= 8 * kTK) {
    int splits = (int)((2LL * sms + ctas - 1) / ctas);
    const int max_by_k = p.Kred / (4 * kTK);                 // at least four k steps per slice
    if (splits > max_by_k) splits = max_by_k;
    if (splits > 32) splits = 32;
    while (splits > 1 && (size_t)splits * M * a.Kout * sizeof(float) > a.scratch_bytes) --splits;
    if (splits > 1) {
      const int steps = (p.Kred + kTK - 1) / kTK;
      p.k_chunk = (steps + splits - 1) / splits * kTK;
      p.splits = (p.Kred + p.k_chunk - 1) / p.k_chunk;       // no empty slice
      p.partial = a.scratch;
      grid.z = (unsigned)p.splits;
    }
  }
  conv_simt_f32_kernel<<<grid, 256, 0, stream>>>(p);
  if (p.splits > 1) {
    const long long total = M * a.Kout;
    conv_simt_reduce_kernel<<<grid_for(total, 256), 256, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

cudaError_t launch_repack_weights_f32(const void* src, DType src_dt, long long sn, long long sc,
                                      long long stap, int Kout, int C, int Cpad, int taps,
                                      float* dst, cudaStream_t stream) {
  const long long total = (long long)Kout * taps * Cpad;
  return by_dtype(src_dt, [&](auto tag) {
    using S = decltype(tag);
    repack_weights_f32_kernel<S><<<grid_for(total, 256), 256, 0, stream>>>(
        static_cast<const S*>(src), sn, sc, stap, Kout, C, Cpad, taps, dst);
    return cudaGetLastError();
  });
}

cudaError_t launch_nchw_to_nhwc(const void* src, DType src_dt, void* dst, DType dst_dt, int N,
                                int C, int H, int W, int Cpad, cudaStream_t stream) {
  const long long HW = (long long)H * W;
  return by_dtype(src_dt, [&](auto stag) {
    using S = decltype(stag);
    return by_dtype(dst_dt, [&](auto dtag) {
      using D = decltype(dtag);
      nchw_to_nhwc_kernel<S, D><<<grid_for((long long)N * HW, 256), 256, 0, stream>>>(
          static_cast<const S*>(src), static_cast<D*>(dst), N, C, HW, Cpad);
      return cudaGetLastError();
    });
  });
}

cudaError_t launch_maxpool_nhwc(const void* src, void* dst, DType dt, int N, int H, int W, int C,
                                int k, int stride, int pad, Layout in_l, Layout out_l,
                                cudaStream_t stream) {
  const int OH = (H + 2 * pad - k) / stride + 1, OW = (W + 2 * pad - k) / stride + 1;
  if (in_l.pitch == 0) in_l = dense_layout(H, W);
  if (out_l.pitch == 0) out_l = dense_layout(OH, OW);
  return by_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int V = 16 / sizeof(T);
    if (C % V != 0) return cudaErrorInvalidValue;
    const long long total = (long long)N * OH * OW * (C / V);
    if (total >= (1LL << 31) - (1LL << 21)) return cudaErrorInvalidValue;   // 16 GiB of fp16 output: beyond any plan here
    maxpool_nhwc_kernel<T><<<grid_for(total, 256), 256, 0, stream>>>(
        static_cast<const T*>(src), static_cast<T*>(dst), N, H, W, C, OH, OW, k, stride, pad, in_l,
        out_l);
    return cudaGetLastError();
  });
}

cudaError_t launch_avgpool_nhwc(const void* src, void* dst, DType dt, int N, int H, int W, int C,
                                Layout in_l, cudaStream_t stream) {
  if (in_l.pitch == 0) in_l = dense_layout(H, W);
  return by_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int V = 16 / sizeof(T);
    if (C % V != 0) return cudaErrorInvalidValue;
    if ((long long)H * W >= 512 && N <= 65535) {
      const int cv = C / V;
      avgpool_cluster_kernel<T><<<dim3(kPoolCluster, N, (cv + 255) / 256), 256, 0, stream>>>(
          static_cast<const T*>(src), static_cast<T*>(dst), N, H, W, C, in_l);
      return cudaGetLastError();
    }
    const long long total = (long long)N * (C / V) * 8;
    avgpool_nhwc_kernel<T><<<grid_for(total, 256), 256, 0, stream>>>(
        static_cast<const T*>(src), static_cast<T*>(dst), N, H, W, C, in_l);
    return cudaGetLastError();
  });
}

cudaError_t launch_relayout(const void* src, Layout src_l, void* dst, Layout dst_l, DType dt, int N,
                            int H, int W, int C, cudaStream_t stream) {
  const int cv = (int)(C * dtype_size(dt) / 16);
  if ((size_t)cv * 16 != C * dtype_size(dt)) return cudaErrorInvalidValue;
  if (src_l.pitch == 0) src_l = dense_layout(H, W);
  if (dst_l.pitch == 0) dst_l = dense_layout(H, W);
  const long long total = layout_slots(dst_l, N) * cv;
  relayout_kernel<<<grid_for(total, 256), 256, 0, stream>>>(
      static_cast<const uint4*>(src), src_l, static_cast<uint4*>(dst), dst_l, N, H, W, cv);
  return cudaGetLastError();
}

cudaError_t launch_bn_fold(const void* gamma, const void* beta, const void* mean,
                           const void* var, DType dt, int C, float eps, float* scale, float* shift,
                           cudaStream_t stream) {
  return by_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    bn_fold_kernel<T><<<(C + 127) / 128, 128, 0, stream>>>(
        static_cast<const T*>(gamma), static_cast<const T*>(beta), static_cast<const T*>(mean),
        static_cast<const T*>(var), C, eps, scale, shift);
    return cudaGetLastError();
  });
}

cudaError_t launch_convert(const void* src, DType src_dt, void* dst, DType dst_dt, size_t n,
                           cudaStream_t stream) {
  return by_dtype(src_dt, [&](auto stag) {
    using S = decltype(stag);
    return by_dtype(dst_dt, [&](auto dtag) {
      using D = decltype(dtag);
      convert_kernel<S, D><<<grid_for((long long)n, 256), 256, 0, stream>>>(
          static_cast<const S*>(src), static_cast<D*>(dst), n);
      return cudaGetLastError();
    });
  });
}

}  // namespace nncv_b200
