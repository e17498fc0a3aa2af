// Memory-bound operators of the mobile / detection networks among nncv's fixtures, NHWC with
// 16-byte accesses, each with its epilogue fused in (nothing here is GEMM-shaped: these kernels are
// bound by HBM bandwidth and are measured in GB/s):
//   depthwise convolution + folded batch-norm + activation
//       (linalg.depthwise_conv_2d_nchw_chw, tests/Nets/MobileNetV3.mlir:301,426,486 ...)
//   activations: ReLU, hard-sigmoid max(0, min(1, (x+3)/6)), hard-swish x * hard-sigmoid(x)
//       (MobileNetV3.mlir:345-383: addf 3, divf 6, olt/select against 1, ogt/select against 0, mulf),
//       sigmoid 1/(1+exp(-x)) and SiLU x * sigmoid(x) (tests/Nets/Yolov5s.mlir:158-169: negf, exp, addf 1, divf, mulf)
//   squeeze-and-excitation: gate = hard-sigmoid(W2 relu(W1 mean(x) + b1) + b2), y = x * gate
//       (MobileNetV3.mlir:319-383: pooling_nchw_sum/divf, two 1x1 convs on [N,C,1,1], broadcast mulf)
//   channel concatenation (tensor.concat dim(1), Yolov5s.mlir:276,445,837 ...)
//   nearest-neighbour 2x upsampling (tensor.extract at floordivsi(index, 2), Yolov5s.mlir:876-884)
// Comparisons keep the fixtures' NaN behaviour: `olt 1, x ? 1 : x` and `ogt 0, x ? 0 : x` pass a NaN on.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cooperative_groups.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace cg = cooperative_groups;

namespace {

template <typename T> __device__ __forceinline__ float ef(T v);
template <> __device__ __forceinline__ float ef<float>(float v) { return v; }
template <> __device__ __forceinline__ float ef<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float ef<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T et(float v);
template <> __device__ __forceinline__ float et<float>(float v) { return v; }
template <> __device__ __forceinline__ __half et<__half>(float v) {
  return __ushort_as_half((unsigned short)(ptx::pack_half2_sat(v, 0.f) & 0xffffu));   // saturating, NaN stays NaN
}
template <> __device__ __forceinline__ __nv_bfloat16 et<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float hard_sigmoid(float x) {
  float t = (x + 3.0f) / 6.0f;
  t = (1.0f < t) ? 1.0f : t;     // cmpf olt 1, t ; select
  t = (0.0f > t) ? 0.0f : t;     // cmpf ogt 0, t ; select
  return t;
}
__device__ __forceinline__ float sigmoid_ref(float x) { return 1.0f / (expf(-x) + 1.0f); }

// With a 16-bit result the last bits of an fp32 quotient or exponential are rounded away, so those types
// take a multiply by 1/6 and the hardware exponential / reciprocal (2 ulp of fp32) instead of IEEE division
// and expf; fp32 tensors keep the exact forms.  NaN and the clamp order are the same in both.
__device__ __forceinline__ float hard_sigmoid_fast(float x) {
  float t = (x + 3.0f) * 0.16666667f;
  t = (1.0f < t) ? 1.0f : t;
  t = (0.0f > t) ? 0.0f : t;
  return t;
}
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, __expf(-x) + 1.0f); }

template <bool FAST>
__device__ __forceinline__ float activate(float x, int act) {
  switch (act) {
    case kActRelu: return !(x <= 0.0f) ? x : 0.0f;        // cmpf ugt: NaN passes
    case kActHardSigmoid: return FAST ? hard_sigmoid_fast(x) : hard_sigmoid(x);
    case kActHardSwish: return x * (FAST ? hard_sigmoid_fast(x) : hard_sigmoid(x));
    case kActSigmoid: return FAST ? sigmoid_fast(x) : sigmoid_ref(x);
    case kActSilu: return x * (FAST ? sigmoid_fast(x) : sigmoid_ref(x));
    default: return x;
  }
}

// ---------------------------------------------------------------- depthwise convolution --
// The general form (any filter size and stride, a single channel vector): the 3x3 / 5x5 cases of the
// fixtures take the TMA-staged kernel of depthwise.cu instead.
// One thread per (output pixel, vector of V channels); weights [C][R*S] as in the fixture's
// collapsed filter tensor<Cx3x3>; per-channel scale/shift (folded batch-norm) and activation.
template <typename T, typename WT>
__global__ void depthwise_kernel(const T* __restrict__ x, const WT* __restrict__ w, const float* __restrict__ scale,
                                 const float* __restrict__ shift, T* __restrict__ y, int N, int H, int W, int C, int OH,
                                 int OW, int R, int S, int stride, int pad, int act, Layout il, Layout ol) {
  constexpr int V = 16 / sizeof(T);
  const int cv = C / V;
  const long long total = (long long)N * OH * OW * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cv) * V;
    long long t = i / cv;
    const int ox = (int)(t % OW);
    t /= OW;
    const int oy = (int)(t % OH);
    const int n = (int)(t / OH);
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = 0.0f;
    for (int r = 0; r < R; ++r) {
      const int iy = oy * stride - pad + r;
      if ((unsigned)iy >= (unsigned)H) continue;
      for (int s = 0; s < S; ++s) {
        const int ix = ox * stride - pad + s;
        if ((unsigned)ix >= (unsigned)W) continue;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + (((size_t)n * il.img_rows + iy + il.off) * il.pitch + ix + il.off) * C + c));
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = fmaf(ef<T>(v[e]), ef<WT>(__ldg(w + (size_t)(c + e) * R * S + r * S + s)), acc[e]);
      }
    }
    alignas(16) T o[V];
#pragma unroll
    for (int e = 0; e < V; ++e) {
      float a = acc[e];
      if (scale) a *= __ldg(scale + c + e);
      if (shift) a += __ldg(shift + c + e);
      o[e] = et<T>(activate<sizeof(T) == 2>(a, act));
    }
    *reinterpret_cast<uint4*>(y + (((size_t)n * ol.img_rows + oy + ol.off) * ol.pitch + ox + ol.off) * C + c) = *reinterpret_cast<const uint4*>(o);
  }
}

// ---------------------------------------------------------------- elementwise ------------
template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, T* __restrict__ y, size_t n_vec, int act) {
  constexpr int V = 16 / sizeof(T);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x) + i);
    const T* v = reinterpret_cast<const T*>(&raw);
    alignas(16) T o[V];
#pragma unroll
    for (int e = 0; e < V; ++e) o[e] = et<T>(activate<sizeof(T) == 2>(ef<T>(v[e]), act));
    reinterpret_cast<uint4*>(y)[i] = *reinterpret_cast<const uint4*>(o);
  }
}

// y[n, p, c] = x[n, p, c] * gate[n, c]
template <typename T>
__global__ void scale_channels_kernel(const T* __restrict__ x, const T* __restrict__ gate, T* __restrict__ y, int N,
                                      long long HW, int C) {
  constexpr int V = 16 / sizeof(T);
  const int cv = C / V;
  const long long total = (long long)N * HW * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cv);
    const int n = (int)(i / ((long long)cv * HW));
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x) + i);
    const uint4 graw = __ldg(reinterpret_cast<const uint4*>(gate) + (size_t)n * cv + c);
    const T* v = reinterpret_cast<const T*>(&raw);
    const T* g = reinterpret_cast<const T*>(&graw);
    alignas(16) T o[V];
#pragma unroll
    for (int e = 0; e < V; ++e) o[e] = et<T>(ef<T>(g[e]) * ef<T>(v[e]));   // mulf gate, x
    reinterpret_cast<uint4*>(y)[i] = *reinterpret_cast<const uint4*>(o);
  }
}

// Squeeze-and-excitation gate: hidden = relu(W1 p + b1), gate = hard-sigmoid(W2 hidden + b2).
// pooled [N,C] (type T), w1 [Cr,C], b1 [Cr], w2 [C,Cr], b2 [C] fp32.
// A cluster of kSeCluster CTAs serves kSeImages images: unit j of either layer belongs to CTA j % kSeCluster, one warp
// per unit reads the unit's weight row once (coalesced) for all images of the group; the hidden vector is
// exchanged through distributed shared memory.  (One CTA per image took 121 us for MobileNetV3's 576-channel
// gate at batch 256, four images per CTA 132 us: the time is the serial walk over the units, not the weight
// traffic, so the units are spread over more CTAs instead.)  Shared memory: kSeImages * (C + 2 Cr) floats.
constexpr int kSeImages = 4;
constexpr int kSeCluster = 8;
template <typename T>
__global__ void __cluster_dims__(kSeCluster, 1, 1) __launch_bounds__(256)
se_gate_kernel(const T* __restrict__ pooled, const float* __restrict__ w1, const float* __restrict__ b1,
               const float* __restrict__ w2, const float* __restrict__ b2, T* __restrict__ gate, int N, int C, int Cr) {
  extern __shared__ float sm[];
  float* p = sm;                          // [kSeImages][C]
  float* hid = sm + kSeImages * C;        // [kSeImages][Cr]: this CTA's units, read by the whole cluster
  float* hall = hid + kSeImages * Cr;     // [kSeImages][Cr]: every unit, gathered
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int n0 = blockIdx.y * kSeImages;
  const int imgs = min(kSeImages, N - n0);
  for (int i = threadIdx.x; i < kSeImages * C; i += blockDim.x) {
    const int im = i / C;
    p[i] = im < imgs ? ef<T>(pooled[(size_t)n0 * C + i]) : 0.0f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int j = rank + kSeCluster * warp; j < Cr; j += kSeCluster * warps) {
    float s[kSeImages];
#pragma unroll
    for (int im = 0; im < kSeImages; ++im) s[im] = 0.0f;
    for (int c = lane; c < C; c += 32) {
      const float w = __ldg(w1 + (size_t)j * C + c);
#pragma unroll
      for (int im = 0; im < kSeImages; ++im) s[im] = fmaf(p[im * C + c], w, s[im]);
    }
#pragma unroll
    for (int im = 0; im < kSeImages; ++im)
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) s[im] += __shfl_xor_sync(0xffffffffu, s[im], d);
    if (lane < kSeImages) {
      float v = s[0];
#pragma unroll
      for (int im = 1; im < kSeImages; ++im) v = lane == im ? s[im] : v;
      v += b1 ? __ldg(b1 + j) : 0.0f;
      hid[lane * Cr + j] = !(v <= 0.0f) ? v : 0.0f;
    }
  }
  cluster.sync();
  for (int i = threadIdx.x; i < kSeImages * Cr; i += blockDim.x) {
    const int j = i % Cr;
    hall[i] = *cluster.map_shared_rank(&hid[i], j % kSeCluster);
  }
  cluster.sync();      // nobody's `hid` is read after this point, so a CTA may finish while others still work
  for (int c = rank + kSeCluster * warp; c < C; c += kSeCluster * warps) {
    float s[kSeImages];
#pragma unroll
    for (int im = 0; im < kSeImages; ++im) s[im] = 0.0f;
    for (int j = lane; j < Cr; j += 32) {
      const float w = __ldg(w2 + (size_t)c * Cr + j);
#pragma unroll
      for (int im = 0; im < kSeImages; ++im) s[im] = fmaf(hall[im * Cr + j], w, s[im]);
    }
#pragma unroll
    for (int im = 0; im < kSeImages; ++im)
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) s[im] += __shfl_xor_sync(0xffffffffu, s[im], d);
    if (lane < imgs) {
      float v = s[0];
#pragma unroll
      for (int im = 1; im < kSeImages; ++im) v = lane == im ? s[im] : v;
      gate[(size_t)(n0 + lane) * C + c] = et<T>(hard_sigmoid(v + (b2 ? __ldg(b2 + c) : 0.0f)));
    }
  }
}

// Channel concatenation: out[p, off_i + c] = in_i[p, c]; 16-byte vectors (every C_i a multiple of V).
struct ConcatParams {
  const void* in[8];
  int cv[8];      // vectors per pixel of each input
  int off[8];     // vector offset inside an output pixel
  int n_in, cv_out;
};
__global__ void concat_kernel(const ConcatParams p, uint4* __restrict__ out, long long pixels) {
  const long long total = pixels * p.cv_out;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % p.cv_out);
    const long long px = i / p.cv_out;
    int k = 0;
#pragma unroll
    for (int j = 1; j < 8; ++j)
      if (j < p.n_in && v >= p.off[j]) k = j;
    out[i] = __ldg(reinterpret_cast<const uint4*>(p.in[k]) + px * p.cv[k] + (v - p.off[k]));
  }
}

// Nearest-neighbour 2x upsampling: out[n, y, x, :] = in[n, y / 2, x / 2, :].
// One thread per input vector: one load, four stores (the two copies along x are adjacent in memory).
__global__ void upsample2x_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int N, int H, int W, int cv) {
  const long long total = (long long)N * H * W * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cv);
    long long t = i / cv;
    const int x = (int)(t % W);
    t /= W;
    const int y = (int)(t % H);
    const int n = (int)(t / H);
    const uint4 v = __ldg(in + i);
    uint4* o = out + (((size_t)n * 2 * H + 2 * y) * (2 * W) + 2 * x) * cv + c;
    const size_t row = (size_t)2 * W * cv;
    o[0] = v;
    o[cv] = v;
    o[row] = v;
    o[row + cv] = v;
  }
}

int grid_for(long long work, int threads) {
  long long b = (work + threads - 1) / threads;
  const long long cap = 148LL * 16;   // a multiple of the SM count; the loops are grid-stride
  if (b > cap) b = cap;
  return b < 1 ? 1 : (int)b;
}

}  // namespace

cudaError_t launch_depthwise(const void* x, const void* w, DType w_dt, const float* scale, const float* shift, void* y, DType dt,
                             int N, int H, int W, int C, int R, int S, int stride, int pad, int act, Layout in_l, Layout out_l,
                             int sm_count, int* error_flag, cudaStream_t st) {
  const int V = 16 / (int)dtype_size(dt);
  if (C % V != 0 || w_dt == kBF16) return cudaErrorInvalidValue;
  if (dt != kF16 && w_dt != kF32) return cudaErrorInvalidValue;
  if (depthwise_tma_supported(dt, N, H, W, C, R, S, stride, pad) && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
    const cudaError_t e = launch_depthwise_tma(x, w, w_dt, scale, shift, y, dt, N, H, W, C, R, S, stride, pad, act, in_l, out_l, sm_count,
                                               error_flag, st);
    if (e == cudaSuccess) return e;
    cudaGetLastError();
  }
  const int OH = (H + 2 * pad - R) / stride + 1, OW = (W + 2 * pad - S) / stride + 1;
  if (OH <= 0 || OW <= 0) return cudaErrorInvalidValue;
  if (in_l.pitch == 0) in_l = dense_layout(H, W);
  if (out_l.pitch == 0) out_l = dense_layout(OH, OW);
  const long long work = (long long)N * OH * OW * (C / V);
  const int g = grid_for(work, 256);
#define NNCV_DW(T, WT)                                                                                                        \
  depthwise_kernel<T, WT><<<g, 256, 0, st>>>((const T*)x, (const WT*)w, scale, shift, (T*)y, N, H, W, C, OH, OW, R, S, stride, \
                                             pad, act, in_l, out_l)
  if (dt == kF32) { if (w_dt != kF32) return cudaErrorInvalidValue; NNCV_DW(float, float); }
  else if (dt == kF16) { if (w_dt == kF32) NNCV_DW(__half, float); else NNCV_DW(__half, __half); }
  else { if (w_dt != kF32) return cudaErrorInvalidValue; NNCV_DW(__nv_bfloat16, float); }
#undef NNCV_DW
  return cudaGetLastError();
}

cudaError_t launch_activation(const void* x, void* y, DType dt, size_t n, int act, cudaStream_t st) {
  const size_t V = 16 / dtype_size(dt);
  if (n % V != 0) return cudaErrorInvalidValue;
  const int g = grid_for((long long)(n / V), 256);
  if (dt == kF32) activation_kernel<float><<<g, 256, 0, st>>>((const float*)x, (float*)y, n / V, act);
  else if (dt == kF16) activation_kernel<__half><<<g, 256, 0, st>>>((const __half*)x, (__half*)y, n / V, act);
  else activation_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n / V, act);
  return cudaGetLastError();
}

cudaError_t launch_scale_channels(const void* x, const void* gate, void* y, DType dt, int N, long long HW, int C, cudaStream_t st) {
  const int V = 16 / (int)dtype_size(dt);
  if (C % V != 0) return cudaErrorInvalidValue;
  const int g = grid_for((long long)N * HW * (C / V), 256);
  if (dt == kF32) scale_channels_kernel<float><<<g, 256, 0, st>>>((const float*)x, (const float*)gate, (float*)y, N, HW, C);
  else if (dt == kF16) scale_channels_kernel<__half><<<g, 256, 0, st>>>((const __half*)x, (const __half*)gate, (__half*)y, N, HW, C);
  else scale_channels_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, (__nv_bfloat16*)y, N, HW, C);
  return cudaGetLastError();
}

cudaError_t launch_se_gate(const void* pooled, const float* w1, const float* b1, const float* w2, const float* b2, void* gate,
                           DType dt, int N, int C, int Cr, cudaStream_t st) {
  const size_t smem = (size_t)kSeImages * (C + 2 * Cr) * sizeof(float);
  if (smem > 160 * 1024 || N <= 0 || (N + kSeImages - 1) / kSeImages > 65535) return cudaErrorInvalidValue;
  const dim3 g(kSeCluster, (N + kSeImages - 1) / kSeImages);
  cudaError_t e = cudaSuccess;
#define NNCV_SE(T)                                                                                                   \
  do {                                                                                                               \
    auto kern = se_gate_kernel<T>;                                                                                   \
    if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    if (e == cudaSuccess) kern<<<g, 256, smem, st>>>((const T*)pooled, w1, b1, w2, b2, (T*)gate, N, C, Cr);          \
  } while (0)
  if (dt == kF32) NNCV_SE(float);
  else if (dt == kF16) NNCV_SE(__half);
  else NNCV_SE(__nv_bfloat16);
#undef NNCV_SE
  return e != cudaSuccess ? e : cudaGetLastError();
}

cudaError_t launch_concat(const void* const* in, const int* channels, int n_in, void* out, DType dt, long long pixels, cudaStream_t st) {
  const int V = 16 / (int)dtype_size(dt);
  if (n_in < 1 || n_in > 8) return cudaErrorInvalidValue;
  ConcatParams p{};
  int off = 0;
  for (int i = 0; i < n_in; ++i) {
    if (channels[i] <= 0 || channels[i] % V != 0 || (reinterpret_cast<uintptr_t>(in[i]) & 15)) return cudaErrorInvalidValue;
    p.in[i] = in[i]; p.cv[i] = channels[i] / V; p.off[i] = off;
    off += channels[i] / V;
  }
  p.n_in = n_in; p.cv_out = off;
  concat_kernel<<<grid_for(pixels * off, 256), 256, 0, st>>>(p, (uint4*)out, pixels);
  return cudaGetLastError();
}

cudaError_t launch_upsample2x(const void* in, void* out, DType dt, int N, int H, int W, int C, cudaStream_t st) {
  const int V = 16 / (int)dtype_size(dt);
  if (C % V != 0) return cudaErrorInvalidValue;
  upsample2x_kernel<<<grid_for((long long)N * H * W * (C / V), 256), 256, 0, st>>>((const uint4*)in, (uint4*)out, N, H, W, C / V);
  return cudaGetLastError();
}

}  // namespace nncv_b200
