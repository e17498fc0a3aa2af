// Winograd F(2x2,3x3) for 3x3 stride-1 pad-1 convolutions, in the three stages nncv's own
// Winograd rewrite has (src/nncv/compiler/Conversion/ConvOptimize/OptimizeConv2dUsingWinograd.cpp:
// 41-83 filter fold G g G^T, :173-284 input transform -> batched matmul -> output transform;
// decomposition in TileAndDecoWinogradPass.cpp:36-232).  nncv uses F(6x6,3x3) with 8x8 tiles and
// 64 GEMMs; here the tile is 4x4 with 16 GEMMs, whose constants (0, +-1, +-1/2) are exact in fp16:
//   B^T = [1 0 -1 0; 0 1 1 0; 0 -1 1 0; 0 1 0 -1]   G = [1 0 0; .5 .5 .5; .5 -.5 .5; 0 0 1]
//   A^T = [1 1 1 0; 0 1 -1 -1]
// Stage 1 and 3 are HBM-bound CUDA-core kernels with 16-byte accesses; stage 2 is sixteen
// [tiles x C] * [C x Kout] GEMMs on the tcgen05 kernels of this library (fp32 results, so the
// only extra rounding is V to 16 bits).  The transformed tensors V (4x the input) and M (4x the
// output, fp32) travel through HBM, which is why the network executor uses the direct
// shifted-view kernel instead; this path exists to measure that choice.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace {

template <typename T> __device__ __forceinline__ float wf(T v);
template <> __device__ __forceinline__ float wf<float>(float v) { return v; }
template <> __device__ __forceinline__ float wf<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float wf<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T wt(float v);
template <> __device__ __forceinline__ __half wt<__half>(float v) {
  return __ushort_as_half((unsigned short)(ptx::pack_half2_sat(v, 0.f) & 0xffffu));
}
template <> __device__ __forceinline__ __nv_bfloat16 wt<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// U[p][k][c] = (G g G^T)[p], one thread per (k, c).
template <typename S, typename D>
__global__ void wino_filter_kernel(const S* __restrict__ w, long long sn, long long sc, long long stap, int K,
                                   int C, D* __restrict__ U) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= (long long)K * C) return;
  const int c = (int)(i % C), k = (int)(i / C);
  float g[3][3];
#pragma unroll
  for (int r = 0; r < 3; ++r)
#pragma unroll
    for (int s = 0; s < 3; ++s) g[r][s] = wf<S>(w[k * sn + c * sc + (r * 3 + s) * stap]);
  float t[4][3];  // G g
#pragma unroll
  for (int s = 0; s < 3; ++s) {
    t[0][s] = g[0][s];
    t[1][s] = 0.5f * (g[0][s] + g[1][s] + g[2][s]);
    t[2][s] = 0.5f * (g[0][s] - g[1][s] + g[2][s]);
    t[3][s] = g[2][s];
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const float u0 = t[r][0], u1 = 0.5f * (t[r][0] + t[r][1] + t[r][2]), u2 = 0.5f * (t[r][0] - t[r][1] + t[r][2]),
                u3 = t[r][2];
    const size_t o = (size_t)k * C + c, ps = (size_t)K * C;
    U[(r * 4 + 0) * ps + o] = wt<D>(u0);
    U[(r * 4 + 1) * ps + o] = wt<D>(u1);
    U[(r * 4 + 2) * ps + o] = wt<D>(u2);
    U[(r * 4 + 3) * ps + o] = wt<D>(u3);
  }
}

// V[p][tile][c] = (B^T d B)[p]; one thread per (tile, 8-channel vector); dense NHWC input.
template <typename T>
__global__ void wino_input_kernel(const T* __restrict__ x, T* __restrict__ V, int N, int H, int W, int C, int ty_n,
                                  int tx_n) {
  const int cv = C / 8;
  const long long tiles = (long long)N * ty_n * tx_n, total = tiles * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cv) * 8;
    const long long tile = i / cv;
    const int tx = (int)(tile % tx_n);
    const int ty = (int)((tile / tx_n) % ty_n);
    const int n = (int)(tile / ((long long)tx_n * ty_n));
    float d[4][4][8];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int iy = 2 * ty - 1 + r;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const int ix = 2 * tx - 1 + s;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if ((unsigned)iy < (unsigned)H && (unsigned)ix < (unsigned)W)
          raw = __ldg(reinterpret_cast<const uint4*>(x + (((size_t)n * H + iy) * W + ix) * C + c));
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int e = 0; e < 8; ++e) d[r][s][e] = wf<T>(v[e]);
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float t[4][4];  // B^T d
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        t[0][s] = d[0][s][e] - d[2][s][e];
        t[1][s] = d[1][s][e] + d[2][s][e];
        t[2][s] = d[2][s][e] - d[1][s][e];
        t[3][s] = d[1][s][e] - d[3][s][e];
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        d[r][0][e] = t[r][0] - t[r][2];
        d[r][1][e] = t[r][1] + t[r][2];
        d[r][2][e] = t[r][2] - t[r][1];
        d[r][3][e] = t[r][1] - t[r][3];
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        alignas(16) T o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = wt<T>(d[r][s][e]);
        *reinterpret_cast<uint4*>(V + ((size_t)(r * 4 + s) * tiles + tile) * C + c) = *reinterpret_cast<const uint4*>(o);
      }
  }
}

// y = A^T m A per tile, then scale/shift (+ residual) (+ ReLU); one thread per (tile, 4 channels).
template <typename T>
__global__ void wino_output_kernel(const float* __restrict__ M, const float* __restrict__ scale,
                                   const float* __restrict__ shift, const T* __restrict__ res, T* __restrict__ y, int N,
                                   int H, int W, int K, int ty_n, int tx_n, int relu) {
  const int kv = K / 4;
  const long long tiles = (long long)N * ty_n * tx_n, total = tiles * kv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % kv) * 4;
    const long long tile = i / kv;
    const int tx = (int)(tile % tx_n);
    const int ty = (int)((tile / tx_n) % ty_n);
    const int n = (int)(tile / ((long long)tx_n * ty_n));
    float4 m[4][4];
#pragma unroll
    for (int p = 0; p < 16; ++p) m[p >> 2][p & 3] = __ldg(reinterpret_cast<const float4*>(M + ((size_t)p * tiles + tile) * K + k));
    const float4 sc = scale ? __ldg(reinterpret_cast<const float4*>(scale + k)) : make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 sh = shift ? __ldg(reinterpret_cast<const float4*>(shift + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float scv[4] = {sc.x, sc.y, sc.z, sc.w}, shv[4] = {sh.x, sh.y, sh.z, sh.w};
    float out[2][2][4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float t[2][4];  // A^T m
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const float a0 = reinterpret_cast<const float*>(&m[0][s])[e], a1 = reinterpret_cast<const float*>(&m[1][s])[e],
                    a2 = reinterpret_cast<const float*>(&m[2][s])[e], a3 = reinterpret_cast<const float*>(&m[3][s])[e];
        t[0][s] = a0 + a1 + a2;
        t[1][s] = a1 - a2 - a3;
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        out[r][0][e] = t[r][0] + t[r][1] + t[r][2];
        out[r][1][e] = t[r][1] - t[r][2] - t[r][3];
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int oy = 2 * ty + r, ox = 2 * tx + s;
        if (oy >= H || ox >= W) continue;
        const size_t o = (((size_t)n * H + oy) * W + ox) * K + k;
        alignas(8) T v[4];
        T rv[4];
        if (res) *reinterpret_cast<uint2*>(rv) = __ldg(reinterpret_cast<const uint2*>(res + o));
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float f = out[r][s][e] * scv[e] + shv[e];
          if (res) f += wf<T>(rv[e]);
          if (relu) f = !(f <= 0.0f) ? f : 0.0f;
          v[e] = wt<T>(f);
        }
        *reinterpret_cast<uint2*>(y + o) = *reinterpret_cast<const uint2*>(v);
      }
  }
}

inline int wgrid(long long total, int threads) {
  long long b = (total + threads - 1) / threads;
  return (int)(b < 1 ? 1 : (b > 148LL * 32 ? 148LL * 32 : b));
}

}  // namespace

cudaError_t launch_wino_filter(const void* w, DType w_dt, long long sn, long long sc, long long stap, int K, int C,
                               void* U, DType dt, cudaStream_t st) {
  const long long total = (long long)K * C;
  const int blocks = (int)((total + 255) / 256);
#define NNCV_WF(S, D) wino_filter_kernel<S, D><<<blocks, 256, 0, st>>>(static_cast<const S*>(w), sn, sc, stap, K, C, static_cast<D*>(U))
  if (dt == kF16) {
    if (w_dt == kF32) NNCV_WF(float, __half);
    else if (w_dt == kF16) NNCV_WF(__half, __half);
    else NNCV_WF(__nv_bfloat16, __half);
  } else if (dt == kBF16) {
    if (w_dt == kF32) NNCV_WF(float, __nv_bfloat16);
    else if (w_dt == kF16) NNCV_WF(__half, __nv_bfloat16);
    else NNCV_WF(__nv_bfloat16, __nv_bfloat16);
  } else {
    return cudaErrorInvalidValue;
  }
#undef NNCV_WF
  return cudaGetLastError();
}

cudaError_t launch_wino_input(const void* x, void* V, DType dt, int N, int H, int W, int C, cudaStream_t st) {
  if (C % 8 != 0) return cudaErrorInvalidValue;
  const int ty = (H + 1) / 2, tx = (W + 1) / 2;
  const long long total = (long long)N * ty * tx * (C / 8);
  if (dt == kF16)
    wino_input_kernel<__half><<<wgrid(total, 128), 128, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(V), N, H, W, C, ty, tx);
  else if (dt == kBF16)
    wino_input_kernel<__nv_bfloat16><<<wgrid(total, 128), 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                                     static_cast<__nv_bfloat16*>(V), N, H, W, C, ty, tx);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t launch_wino_output(const float* M, const float* scale, const float* shift, const void* res, void* y,
                               DType dt, int N, int H, int W, int K, int relu, cudaStream_t st) {
  if (K % 4 != 0) return cudaErrorInvalidValue;
  const int ty = (H + 1) / 2, tx = (W + 1) / 2;
  const long long total = (long long)N * ty * tx * (K / 4);
  if (dt == kF16)
    wino_output_kernel<__half><<<wgrid(total, 128), 128, 0, st>>>(M, scale, shift, static_cast<const __half*>(res),
                                                                  static_cast<__half*>(y), N, H, W, K, ty, tx, relu);
  else if (dt == kBF16)
    wino_output_kernel<__nv_bfloat16><<<wgrid(total, 128), 128, 0, st>>>(
        M, scale, shift, static_cast<const __nv_bfloat16*>(res), static_cast<__nv_bfloat16*>(y), N, H, W, K, ty, tx, relu);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace nncv_b200
