// 1x1 stride-1 convolution with few channels on CUDA cores (16-bit NHWC in the executor's layouts), folded
// batch-norm / bias, residual add and activation fused: MobileNetV3's first pointwise layer
// (tests/Nets/MobileNetV3.mlir: 16 -> 16 at 56 x 56 after the first squeeze-and-excitation block).
//
// With so few channels on either side the layer moves tens of bytes per pixel for a few hundred
// multiply-adds: it is bound by HBM, and on the tensor-core kernel it pays for tiles padded to 64 input
// channels and 64-column output slabs.  Here one thread computes 16 output channels of one pixel: the pixel's input vector comes from
// global memory in 16-byte loads, the weights of the thread's channel group sit in shared memory as fp32
// [c][k] and are read as broadcast vectors (a warp shares the group), accumulation is fp32 on register pairs.
// Measured at batch 256: 16 -> 16 at 112 x 112 takes 27 us here against 109 us on the tensor-core kernel; with more
// channels the tensor-core kernel wins (16 -> 72: 156 us here against 141 us), so the runtime sends only layers with
// at most 32 channels on both sides here.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace {

constexpr int kKG = 16;   // output channels per thread

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

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if (BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

struct PwParams {
  const uint16_t* in;
  const float* w;          // [Kout][C] fp32
  const float* scale;
  const float* shift;
  const uint16_t* residual;
  uint16_t* out;
  Layout il, ol;
  int N, H, W, C, Kout, Kp;   // Kp: Kout rounded up to a multiple of kKG
  int relu, act;
};

template <bool BF16>
__global__ void __launch_bounds__(256) pointwise_kernel(const PwParams p) {
  extern __shared__ __align__(16) float sw[];     // [C][Kp] weights, [Kp] scale, [Kp] shift
  float* ssc = sw + (size_t)p.C * p.Kp;
  float* ssh = ssc + p.Kp;
  for (int i = threadIdx.x; i < p.C * p.Kp; i += blockDim.x) {
    const int c = i / p.Kp, k = i - c * p.Kp;
    sw[i] = k < p.Kout ? p.w[(size_t)k * p.C + c] : 0.0f;
  }
  for (int k = threadIdx.x; k < p.Kp; k += blockDim.x) {
    ssc[k] = (k < p.Kout && p.scale) ? p.scale[k] : 1.0f;
    ssh[k] = (k < p.Kout && p.shift) ? p.shift[k] : 0.0f;
  }
  __syncthreads();
  const int groups = p.Kp / kKG;
  const unsigned per = (unsigned)p.N * p.H * p.W;
  const unsigned total = per * groups;                       // kept below 2^31 by the launcher
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int g = (int)(i / per);                            // slowest: a warp shares its channel group
    unsigned t = i - (unsigned)g * per;
    const unsigned t2 = t / (unsigned)p.W;
    const int x = (int)(t - t2 * p.W);
    const int n = (int)(t2 / (unsigned)p.H);
    const int y = (int)(t2 - (unsigned)n * p.H);
    const size_t slot_in = ((size_t)n * p.il.img_rows + y + p.il.off) * p.il.pitch + x + p.il.off;
    const size_t slot_out = ((size_t)n * p.ol.img_rows + y + p.ol.off) * p.ol.pitch + x + p.ol.off;
    const uint4* ip = reinterpret_cast<const uint4*>(p.in + slot_in * p.C);
    float2 acc[kKG / 2];
#pragma unroll
    for (int e = 0; e < kKG / 2; ++e) acc[e] = make_float2(0.0f, 0.0f);
    const float* wg = sw + g * kKG;
    for (int cv = 0; cv < p.C / 8; ++cv) {
      const uint4 raw = __ldg(ip + cv);
      const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float2 v = unpack2<BF16>(wds[h]);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const float xv = s ? v.y : v.x;
          const float2 x2 = make_float2(xv, xv);
          const float* wp = wg + (size_t)(cv * 8 + h * 2 + s) * p.Kp;
#pragma unroll
          for (int e = 0; e < kKG / 2; e += 2) {
            const float4 w4 = *reinterpret_cast<const float4*>(wp + 2 * e);
            acc[e] = fma2(x2, make_float2(w4.x, w4.y), acc[e]);
            acc[e + 1] = fma2(x2, make_float2(w4.z, w4.w), acc[e + 1]);
          }
        }
      }
    }
    const int k0 = g * kKG;
    const uint16_t* rp = p.residual ? p.residual + slot_out * p.Kout + k0 : nullptr;
    uint16_t* op = p.out + slot_out * p.Kout + k0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (k0 + half * 8 >= p.Kout) break;                    // Kout is a multiple of 8: whole vectors only
      uint4 rr = make_uint4(0, 0, 0, 0);
      if (rp) rr = __ldg(reinterpret_cast<const uint4*>(rp + half * 8));
      const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
      uint32_t o[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const int e = half * 4 + h;
        const float2 sc = *reinterpret_cast<const float2*>(ssc + k0 + 2 * e);
        const float2 sh = *reinterpret_cast<const float2*>(ssh + k0 + 2 * e);
        float2 a = fma2(acc[e], sc, sh);
        if (rp) {
          const float2 r = unpack2<BF16>(rw[h]);
          a.x += r.x; a.y += r.y;
        }
        if (p.act == kActHardSwish) {
          a.x *= fminf(fmaxf(fmaf(a.x, 0.16666667f, 0.5f), 0.0f), 1.0f);
          a.y *= fminf(fmaxf(fmaf(a.y, 0.16666667f, 0.5f), 0.0f), 1.0f);
        } else if (p.act == kActSilu) {
          a.x *= __fdividef(1.0f, __expf(-a.x) + 1.0f);
          a.y *= __fdividef(1.0f, __expf(-a.y) + 1.0f);
        }
        if (BF16) {
          __nv_bfloat162 b = __floats2bfloat162_rn(a.x, a.y);
          if (p.relu) b = __hmax2_nan(b, __floats2bfloat162_rn(0.f, 0.f));
          o[h] = *reinterpret_cast<const uint32_t*>(&b);
        } else {
          const uint32_t xs = ptx::pack_half2_sat(a.x, a.y);
          __half2 b = *reinterpret_cast<const __half2*>(&xs);
          if (p.relu) b = __hmax2_nan(b, __floats2half2_rn(0.f, 0.f));
          o[h] = *reinterpret_cast<const uint32_t*>(&b);
        }
      }
      *reinterpret_cast<uint4*>(op + half * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

}  // namespace

bool pointwise_supported(int C, int Kout, int R, int S, int stride, int pad, DType dt) {
  return dt != kF32 && R == 1 && S == 1 && stride == 1 && pad == 0 && C % 8 == 0 && Kout % 8 == 0 && C >= 8 && Kout >= 8 &&
         C <= 128 && Kout <= 128;
}

cudaError_t launch_pointwise(const PointwiseArgs& a, cudaStream_t st) {
  if (!pointwise_supported(a.C, a.Kout, 1, 1, 1, 0, a.ab) || (a.act != kActNone && a.act != kActHardSwish && a.act != kActSilu))
    return cudaErrorInvalidValue;
  PwParams p;
  p.in = static_cast<const uint16_t*>(a.in); p.w = a.w; p.scale = a.scale; p.shift = a.shift;
  p.residual = static_cast<const uint16_t*>(a.residual); p.out = static_cast<uint16_t*>(a.out);
  p.il = a.in_l.pitch ? a.in_l : dense_layout(a.H, a.W);
  p.ol = a.out_l.pitch ? a.out_l : dense_layout(a.H, a.W);
  p.N = a.N; p.H = a.H; p.W = a.W; p.C = a.C; p.Kout = a.Kout; p.Kp = (a.Kout + kKG - 1) / kKG * kKG;
  p.relu = a.relu; p.act = a.act;
  const long long total = (long long)a.N * a.H * a.W * (p.Kp / kKG);
  if (total <= 0 || total >= (1LL << 31) - (1LL << 21)) return cudaErrorInvalidValue;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)(a.sm_count > 0 ? a.sm_count : 148) * 8;
  if (blocks > cap) blocks = cap;
  const size_t smem = ((size_t)a.C + 2) * p.Kp * sizeof(float);
  cudaError_t e = cudaSuccess;
  if (a.ab == kBF16) {
    if (smem > 48 * 1024) e = cudaFuncSetAttribute(pointwise_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) pointwise_kernel<true><<<(unsigned)blocks, 256, smem, st>>>(p);
  } else {
    if (smem > 48 * 1024) e = cudaFuncSetAttribute(pointwise_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) pointwise_kernel<false><<<(unsigned)blocks, 256, smem, st>>>(p);
  }
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace nncv_b200
