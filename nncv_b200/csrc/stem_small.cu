// First convolution of a small-channel network: 3x3 (any stride) on the 3-channel NCHW network input,
// 16 .. 64 output channels, folded batch-norm / bias and activation, written as NHWC in the
// executor's layout (MobileNetV3's `conv 3 -> 16, 3x3 stride 2 + BN + hard-swish`,
// tests/Nets/MobileNetV3.mlir:240-295).
//
// With 27 multiply-adds per output value and 3 input channels this layer is bound by HBM (one read
// of the NCHW input, one write of the output), and it does not fit the tensor-core kernels: as an
// implicit GEMM its K of 27 would be padded to 9 x 64 and its N of 16 to 64 (measured on the TMA-fed
// kernel: 821 us at batch 256, plus 109 us for the NCHW -> NHWC conversion in front of it).  Here one
// thread computes 16 output channels of one pixel straight from the NCHW input (a warp reads
// consecutive columns of a row), filter / scale / shift in shared memory read as broadcast vectors,
// fp32 accumulation on register pairs, and the conversion pass disappears.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace {

constexpr int kCG = 16;   // output channels per thread

__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  unsigned long long ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}

template <typename T> __device__ __forceinline__ float ld(const T* p);
template <> __device__ __forceinline__ float ld<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld<__half>(const __half* p) { return __half2float(__ldg(p)); }

__device__ __forceinline__ float act16(float x, int act) {
  switch (act) {
    case kActRelu: return !(x <= 0.0f) ? x : 0.0f;
    case kActHardSwish: {
      float t = (x + 3.0f) * 0.16666667f;
      t = (1.0f < t) ? 1.0f : t;
      t = (0.0f > t) ? 0.0f : t;
      return x * t;
    }
    case kActSilu: return x * __fdividef(1.0f, __expf(-x) + 1.0f);
    default: return x;
  }
}

template <typename TI, bool BF16>
__global__ void __launch_bounds__(256) stem3x3_kernel(const TI* __restrict__ src, const float* __restrict__ w,
                                                      const float* __restrict__ scale, const float* __restrict__ shift,
                                                      void* __restrict__ dst, Layout ol, int N, int H, int W, int OH, int OW, int Cout,
                                                      int stride, int pad, int act) {
  extern __shared__ __align__(16) float sw[];     // [27][Cout] filter, [Cout] scale, [Cout] shift
  float* ssc = sw + 27 * Cout;
  float* ssh = ssc + Cout;
  for (int i = threadIdx.x; i < 27 * Cout; i += blockDim.x) {
    const int k = i / 27, t = i - k * 27;           // source [Cout][3][3][3]: t = (ci*3 + ky)*3 + kx
    sw[t * Cout + k] = w[i];
  }
  for (int c = threadIdx.x; c < Cout; c += blockDim.x) {
    ssc[c] = scale ? scale[c] : 1.0f;
    ssh[c] = shift ? shift[c] : 0.0f;
  }
  __syncthreads();
  const int groups = Cout / kCG;
  const unsigned total = (unsigned)N * OH * OW * groups;      // kept below 2^31 by the launcher
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    // the channel group is the slowest index: the threads of a warp share it and walk along a row
    const unsigned per = (unsigned)N * OH * OW;
    const int g = (int)(i / per);
    unsigned t = i - (unsigned)g * per;
    const unsigned t2 = t / (unsigned)OW;
    const int ox = (int)(t - t2 * OW);
    const int n = (int)(t2 / (unsigned)OH);
    const int oy = (int)(t2 - (unsigned)n * OH);
    float2 acc[kCG / 2];
#pragma unroll
    for (int e = 0; e < kCG / 2; ++e) acc[e] = make_float2(0.0f, 0.0f);
    const int ix0 = ox * stride - pad, iy0 = oy * stride - pad;
    // all 27 input values first (out-of-range taps read as zero without a branch), so that the loads are in
    // flight together; then the multiply-adds
    float in[27];
#pragma unroll
    for (int ci = 0; ci < 3; ++ci) {
      const TI* plane = src + ((size_t)n * 3 + ci) * H * W;
#pragma unroll
      for (int ky = 0; ky < 3; ++ky) {
        const int iy = iy0 + ky;
        const bool yin = (unsigned)iy < (unsigned)H;
        const TI* rowp = plane + (size_t)(yin ? iy : 0) * W;
#pragma unroll
        for (int kx = 0; kx < 3; ++kx) {
          const int ix = ix0 + kx;
          const bool inb = yin && (unsigned)ix < (unsigned)W;
          const float v = ld<TI>(rowp + (inb ? ix : 0));
          in[(ci * 3 + ky) * 3 + kx] = inb ? v : 0.0f;
        }
      }
    }
#pragma unroll
    for (int t9 = 0; t9 < 27; ++t9) {
      const float2 v2 = make_float2(in[t9], in[t9]);
      const float* wp = sw + t9 * Cout + g * kCG;
#pragma unroll
      for (int e = 0; e < kCG / 2; e += 2) {
        const float4 w4 = *reinterpret_cast<const float4*>(wp + 2 * e);
        acc[e] = fma2(v2, make_float2(w4.x, w4.y), acc[e]);
        acc[e + 1] = fma2(v2, make_float2(w4.z, w4.w), acc[e + 1]);
      }
    }
    uint32_t o[kCG / 2];
#pragma unroll
    for (int e = 0; e < kCG / 2; ++e) {
      const float2 sc = *reinterpret_cast<const float2*>(ssc + g * kCG + 2 * e);
      const float2 sh = *reinterpret_cast<const float2*>(ssh + g * kCG + 2 * e);
      const float2 a = fma2(acc[e], sc, sh);
      const float x = act16(a.x, act), y = act16(a.y, act);
      if (BF16) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(x, y);
        o[e] = *reinterpret_cast<const uint32_t*>(&b);
      } else {
        o[e] = ptx::pack_half2_sat(x, y);
      }
    }
    uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(dst) +
                                          (((size_t)n * ol.img_rows + oy + ol.off) * ol.pitch + ox + ol.off) * Cout + g * kCG);
    out[0] = make_uint4(o[0], o[1], o[2], o[3]);
    out[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

}  // namespace

bool stem3x3_supported(int Cin, int Cout, int R, int S, DType act_dt, int act) {
  return Cin == 3 && R == 3 && S == 3 && Cout % kCG == 0 && Cout >= kCG && Cout <= 64 && act_dt != kF32 &&
         (act == kActNone || act == kActRelu || act == kActHardSwish || act == kActSilu);
}

cudaError_t launch_stem3x3(const void* src, DType src_dt, const float* w, const float* scale, const float* shift, void* dst, DType dt,
                           Layout out_l, int N, int H, int W, int Cout, int stride, int pad, int act, cudaStream_t st) {
  if (!stem3x3_supported(3, Cout, 3, 3, dt, act) || src_dt == kBF16 || stride < 1 || pad < 0) return cudaErrorInvalidValue;
  const int OH = (H + 2 * pad - 3) / stride + 1, OW = (W + 2 * pad - 3) / stride + 1;
  if (OH <= 0 || OW <= 0) return cudaErrorInvalidValue;
  if (out_l.pitch == 0) out_l = dense_layout(OH, OW);
  const long long total = (long long)N * OH * OW * (Cout / kCG);
  if (total >= (1LL << 31) - (1LL << 21)) return cudaErrorInvalidValue;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const size_t smem = (size_t)29 * Cout * sizeof(float);
#define NNCV_ST(TI, BF) \
  stem3x3_kernel<TI, BF><<<(unsigned)blocks, 256, smem, st>>>((const TI*)src, w, scale, shift, dst, out_l, N, H, W, OH, OW, Cout, stride, pad, act)
  if (src_dt == kF32) { if (dt == kBF16) NNCV_ST(float, true); else NNCV_ST(float, false); }
  else { if (dt == kBF16) NNCV_ST(__half, true); else NNCV_ST(__half, false); }
#undef NNCV_ST
  return cudaGetLastError();
}

}  // namespace nncv_b200
