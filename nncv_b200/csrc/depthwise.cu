// Depthwise convolution + folded batch-norm + activation, NHWC, staged through shared memory by TMA
// (linalg.depthwise_conv_2d_nchw_chw followed by the batch-norm and hard-swish / ReLU generics,
// tests/Nets/MobileNetV3.mlir:301,426,486 ...).
//
// The operator is bound by HBM: 2 bytes in and 2 bytes out per element, 9 or 25 multiply-adds.  A
// kernel that fetches its taps with per-thread global loads spends its time waiting for them (a
// few loads in flight per thread, bounds checks between them), so here a persistent CTA walks
// tiles of 8 output rows x TW output columns x CB channels and one thread issues, two tiles ahead,
// ONE tensor copy per tile: the input patch with its halo, out-of-range pixels filled with zeros by
// the copy engine (no bounds checks on the input side at all).  The 256 threads then read the
// patch from shared memory with 16-byte loads: thread = (channel vector, output column, half of
// the tile's rows) and computes a column strip of four output rows, so that each input value is
// loaded from shared memory once per filter column and reused down the strip, in fp32 pairs
// (fma.rn.f32x2).  The filter, scale and shift of the CTA's channel chunk sit in shared memory.
// Every wait on a copy is bounded; a wait that gives up sets the status word and the CTA leaves.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace {

constexpr int kThreads = 256;
constexpr int kP = 4;            // output rows per thread
constexpr int kTH = 2 * kP;      // output rows per tile
constexpr int kMaxStages = 3;

struct DwParams {
  const void* w;       // [C][KS*KS], fp32 or fp16
  int w_half;
  const float* scale;  // [C] or null
  const float* shift;  // [C] or null
  void* y;             // [N,OH,OW,C]
  int N, H, W, C, OH, OW, pad, act;
  Layout in_l, out_l;  // input coordinates and output pixels are shifted by the layouts' pad offsets
  int tw, cbv;         // output columns per tile, 16-byte channel vectors per chunk (tw * cbv == 128)
  int tiles_x, tiles_y, n_tiles;   // spatial tiles (n_tiles = N * tiles_y * tiles_x)
  int stages;
  uint32_t stage_bytes, stage_stride;
  int* error_flag;
};

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

__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  unsigned long long ra, rb, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}

template <typename T> __device__ __forceinline__ void unpack(const uint4& raw, float2* f);
template <> __device__ __forceinline__ void unpack<float>(const uint4& raw, float2* f) {
  f[0] = make_float2(__uint_as_float(raw.x), __uint_as_float(raw.y));
  f[1] = make_float2(__uint_as_float(raw.z), __uint_as_float(raw.w));
}
template <> __device__ __forceinline__ void unpack<__half>(const uint4& raw, float2* f) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) f[e] = __half22float2(h[e]);
}
template <> __device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& raw, float2* f) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw);   // a bf16 is the upper half of an fp32
#pragma unroll
  for (int e = 0; e < 4; ++e) f[e] = make_float2(__uint_as_float(u[e] << 16), __uint_as_float(u[e] & 0xffff0000u));
}
template <typename T> __device__ __forceinline__ uint4 pack(const float2* r);
template <> __device__ __forceinline__ uint4 pack<float>(const float2* r) {
  return make_uint4(__float_as_uint(r[0].x), __float_as_uint(r[0].y), __float_as_uint(r[1].x), __float_as_uint(r[1].y));
}
template <> __device__ __forceinline__ uint4 pack<__half>(const float2* r) {   // saturating, NaN stays NaN
  return make_uint4(ptx::pack_half2_sat(r[0].x, r[0].y), ptx::pack_half2_sat(r[1].x, r[1].y),
                    ptx::pack_half2_sat(r[2].x, r[2].y), ptx::pack_half2_sat(r[3].x, r[3].y));
}
template <> __device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float2* r) {
  uint4 o;
  uint32_t* u = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(r[e].x, r[e].y);
    u[e] = *reinterpret_cast<const uint32_t*>(&b);
  }
  return o;
}

// The activations of MobileNetV3.mlir:345-383 and Yolov5s.mlir:158-169.  EXACT (fp32 tensors) keeps
// IEEE division and expf; 16-bit results take the multiply by 1/6 and the hardware exponential.
// Compare-and-select clamps pass a NaN on, as the fixtures' cmpf/select pairs do.
template <bool EXACT>
__device__ __forceinline__ float act1(float x, int act) {
  switch (act) {
    case kActRelu: return !(x <= 0.0f) ? x : 0.0f;
    case kActHardSigmoid:
    case kActHardSwish: {
      float t = EXACT ? (x + 3.0f) / 6.0f : (x + 3.0f) * 0.16666667f;
      t = (1.0f < t) ? 1.0f : t;
      t = (0.0f > t) ? 0.0f : t;
      return act == kActHardSwish ? x * t : t;
    }
    case kActSigmoid:
    case kActSilu: {
      const float s = EXACT ? 1.0f / (expf(-x) + 1.0f) : __fdividef(1.0f, __expf(-x) + 1.0f);
      return act == kActSilu ? x * s : s;
    }
    default: return x;
  }
}

template <typename T, int KS, int STRIDE>
__global__ void __launch_bounds__(kThreads, KS == 3 ? 3 : 2) depthwise_tma_kernel(const __grid_constant__ CUtensorMap tm_in, const DwParams p) {
  constexpr int V = 16 / sizeof(T);
  constexpr int NR = (kP - 1) * STRIDE + KS;            // input rows under one strip of kP outputs
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long full_bar[kMaxStages];
  __shared__ int abort_flag;
  __shared__ int4 tile_info[kMaxStages];                 // (image, first output row, first output column) of the tile in a stage

  const int tid = threadIdx.x;
  const int cbv = p.cbv, tw = p.tw;
  const int CB = cbv * V;                                // channels per chunk
  const int IW = (tw - 1) * STRIDE + KS;
  const int c0 = blockIdx.y * CB;
  float* sw = reinterpret_cast<float*>(smem + (size_t)p.stages * p.stage_stride);   // [KS*KS][CB], scale[CB], shift[CB]
  float* ssc = sw + KS * KS * CB;
  float* ssh = ssc + CB;

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&tm_in);
  }
  for (int i = tid; i < KS * KS * CB; i += kThreads) {
    const int tap = i / CB, c = i - tap * CB;
    float v = 0.0f;
    if (c0 + c < p.C) {
      const size_t idx = (size_t)(c0 + c) * (KS * KS) + tap;
      v = p.w_half ? __half2float(reinterpret_cast<const __half*>(p.w)[idx]) : reinterpret_cast<const float*>(p.w)[idx];
    }
    sw[i] = v;
  }
  for (int c = tid; c < CB; c += kThreads) {
    const bool in = c0 + c < p.C;
    ssc[c] = (in && p.scale) ? p.scale[c0 + c] : 1.0f;
    ssh[c] = (in && p.shift) ? p.shift[c0 + c] : 0.0f;
  }
  __syncthreads();

  const int my_tiles = ((int)blockIdx.x < p.n_tiles) ? (p.n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  auto issue = [&](int k) {      // thread 0: the copy of this CTA's k-th tile into stage k % stages
    const int sp = blockIdx.x + k * gridDim.x;
    const int n = sp / (p.tiles_y * p.tiles_x);
    const int r = sp - n * (p.tiles_y * p.tiles_x);
    const int ty = r / p.tiles_x, tx = r - ty * p.tiles_x;
    const int s = k % p.stages;
    const uint32_t bar = ptx::smem_u32(&full_bar[s]);
    tile_info[s] = make_int4(n, ty * kTH, tx * tw, 0);   // read by the others after they have seen the barrier complete
    ptx::mbar_arrive_expect_tx(bar, p.stage_bytes);
    ptx::tma_load_4d(ptx::smem_u32(smem + (size_t)s * p.stage_stride), &tm_in, c0, tx * tw * STRIDE - p.pad + p.in_l.off,
                     ty * kTH * STRIDE - p.pad + p.in_l.off, n, bar);
  };
  int issued = 0;
  if (tid == 0)
    for (; issued < p.stages - 1 && issued < my_tiles; ++issued) issue(issued);

  const int cvec = tid % cbv;
  const int x = (tid / cbv) % tw;
  const int ys = tid / (cbv * tw);                       // 0 or 1
  int k = 0;
  for (; k < my_tiles; ++k) {
    const int s = k % p.stages;
    bool ok = ptx::mbar_wait_abortable(ptx::smem_u32(&full_bar[s]), (uint32_t)((k / p.stages) & 1), &abort_flag);
    // one barrier per tile: past it every thread has finished tile k - 1, whose stage the next copy overwrites
    if (__syncthreads_or(!ok)) break;
    if (tid == 0 && issued < my_tiles) { issue(issued); ++issued; }

    const unsigned char* st = smem + (size_t)s * p.stage_stride;
    float2 acc[kP][V / 2];
#pragma unroll
    for (int o = 0; o < kP; ++o)
#pragma unroll
      for (int e = 0; e < V / 2; ++e) acc[o][e] = make_float2(0.0f, 0.0f);
    const int row0 = ys * kP * STRIDE;
#pragma unroll
    for (int kx = 0; kx < KS; ++kx) {
      float2 wr[KS][V / 2];
#pragma unroll
      for (int q = 0; q < KS; ++q)
#pragma unroll
        for (int e = 0; e < V / 2; e += 2) {
          const float4 t4 = *reinterpret_cast<const float4*>(sw + (q * KS + kx) * CB + cvec * V + 2 * e);
          wr[q][e] = make_float2(t4.x, t4.y);
          wr[q][e + 1] = make_float2(t4.z, t4.w);
        }
      const unsigned char* col = st + ((size_t)(row0 * IW + x * STRIDE + kx) * cbv + cvec) * 16;
#pragma unroll
      for (int ry = 0; ry < NR; ++ry) {
        const uint4 raw = *reinterpret_cast<const uint4*>(col + (size_t)ry * IW * cbv * 16);
        float2 f[V / 2];
        unpack<T>(raw, f);
#pragma unroll
        for (int o = 0; o < kP; ++o) {
          const int q = ry - o * STRIDE;               // compile-time after unrolling
          if (q >= 0 && q < KS) {
#pragma unroll
            for (int e = 0; e < V / 2; ++e) acc[o][e] = fma2(f[e], wr[q][e], acc[o][e]);
          }
        }
      }
    }
    // epilogue: scale, shift, activation, store
    const int4 ti = tile_info[s];
    const int n = ti.x;
    const int ox = ti.z + x;
    const int c = c0 + cvec * V;
    if (ox < p.OW && c < p.C) {
      float2 sc[V / 2], sh[V / 2];
#pragma unroll
      for (int e = 0; e < V / 2; e += 2) {
        const float4 a4 = *reinterpret_cast<const float4*>(ssc + cvec * V + 2 * e);
        const float4 b4 = *reinterpret_cast<const float4*>(ssh + cvec * V + 2 * e);
        sc[e] = make_float2(a4.x, a4.y); sc[e + 1] = make_float2(a4.z, a4.w);
        sh[e] = make_float2(b4.x, b4.y); sh[e + 1] = make_float2(b4.z, b4.w);
      }
#pragma unroll
      for (int o = 0; o < kP; ++o) {
        const int oy = ti.y + ys * kP + o;
        if (oy >= p.OH) break;
        float2 r2[V / 2];
#pragma unroll
        for (int e = 0; e < V / 2; ++e) {
          // scale and shift default to 1 and 0 in shared memory, so one fused multiply-add serves every case
          const float2 a = fma2(acc[o][e], sc[e], sh[e]);
          if (sizeof(T) == 2 && p.act == kActHardSwish) {
            // min/max clamp: a NaN still comes out as NaN because the clamped factor multiplies x itself
            float2 t = fma2(a, make_float2(0.16666667f, 0.16666667f), make_float2(0.5f, 0.5f));
            t.x = fminf(fmaxf(t.x, 0.0f), 1.0f);
            t.y = fminf(fmaxf(t.y, 0.0f), 1.0f);
            r2[e] = mul2(a, t);
          } else {
            r2[e] = make_float2(act1<sizeof(T) == 4>(a.x, p.act), act1<sizeof(T) == 4>(a.y, p.act));
          }
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.y) +
                                  (((size_t)n * p.out_l.img_rows + oy + p.out_l.off) * p.out_l.pitch + ox + p.out_l.off) * p.C + c) =
            pack<T>(r2);
      }
    }
  }
  if (k < my_tiles && tid == 0) {
    // a wait gave up: record it, then give the copies still in flight a bounded time to land before
    // the CTA's shared memory is released
    if (p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitProducer);
    for (int j = k; j < issued; ++j)
      ptx::mbar_wait_limit(ptx::smem_u32(&full_bar[j % p.stages]), (uint32_t)((j / p.stages) & 1), 1LL << 24);
  }
}

PFN_cuTensorMapEncodeTiled_v12000 dw_get_encode() {
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

template <typename T, int KS, int STRIDE>
cudaError_t launch_one(const CUtensorMap& tm, const DwParams& p, dim3 grid, size_t smem, cudaStream_t st) {
  auto kern = depthwise_tma_kernel<T, KS, STRIDE>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, kThreads, smem, st>>>(tm, p);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_typed(const CUtensorMap& tm, const DwParams& p, int ks, int stride, dim3 grid, size_t smem, cudaStream_t st) {
  if (ks == 3 && stride == 1) return launch_one<T, 3, 1>(tm, p, grid, smem, st);
  if (ks == 3 && stride == 2) return launch_one<T, 3, 2>(tm, p, grid, smem, st);
  if (ks == 5 && stride == 1) return launch_one<T, 5, 1>(tm, p, grid, smem, st);
  return launch_one<T, 5, 2>(tm, p, grid, smem, st);
}

}  // namespace

bool depthwise_tma_supported(DType dt, int N, int H, int W, int C, int R, int S, int stride, int pad) {
  const int V = 16 / (int)dtype_size(dt);
  if (R != S || (R != 3 && R != 5) || (stride != 1 && stride != 2) || pad > R) return false;
  if (C % V != 0 || C / V < 2) return false;
  const int OH = (H + 2 * pad - R) / stride + 1, OW = (W + 2 * pad - S) / stride + 1;
  if (OH <= 0 || OW <= 0) return false;
  return (long long)N * ((OH + kTH - 1) / kTH) * ((OW + 7) / 8) < (1LL << 30);
}

cudaError_t launch_depthwise_tma(const void* x, const void* w, DType w_dt, const float* scale, const float* shift, void* y, DType dt,
                                 int N, int H, int W, int C, int R, int S, int stride, int pad, int act, Layout in_l, Layout out_l,
                                 int sm_count, int* error_flag, cudaStream_t st) {
  if (!depthwise_tma_supported(dt, N, H, W, C, R, S, stride, pad) || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(y) & 15))
    return cudaErrorInvalidValue;
  const int es = (int)dtype_size(dt), V = 16 / es, cv = C / V;
  const int OH = (H + 2 * pad - R) / stride + 1, OW = (W + 2 * pad - S) / stride + 1;
  DwParams p{};
  // 128 (column, vector) pairs per tile: wide tiles for wide maps, more channels per chunk for narrow ones;
  // a chunk never holds more vectors than the tensor has
  int cbv = 0, tw = 0;
  double best = 1e30;
  for (int cand = 16; cand >= 2; cand /= 2) {          // ties go to the wider chunk (longer contiguous runs in memory)
    if (cand > cv) continue;
    const int t = 128 / cand;
    if (t > 8 && t >= 2 * OW) continue;                // a tile more than twice as wide as the map
    const double waste = (double)((cv + cand - 1) / cand * cand) / cv * ((OW + t - 1) / t * t) / OW;
    if (waste < best - 1e-9) { best = waste; cbv = cand; tw = t; }
  }
  if (cbv == 0) return cudaErrorInvalidValue;
  p.tw = tw; p.cbv = cbv;
  const int IW = (tw - 1) * stride + R, IH = (kTH - 1) * stride + R;
  if (IW > 256 || IH > 256) return cudaErrorInvalidValue;
  p.stage_bytes = (uint32_t)IW * IH * cbv * 16;
  p.stage_stride = (p.stage_bytes + 127u) & ~127u;
  const size_t wbytes = (size_t)(R * S + 2) * cbv * V * sizeof(float);
  int stages = kMaxStages;
  while (stages > 2 && (size_t)stages * p.stage_stride + wbytes > 72 * 1024) --stages;   // three CTAs per SM when it fits
  const size_t smem = (size_t)stages * p.stage_stride + wbytes;
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  p.stages = stages;
  p.w = w; p.w_half = w_dt == kF16; p.scale = scale; p.shift = shift; p.y = y;
  p.N = N; p.H = H; p.W = W; p.C = C; p.OH = OH; p.OW = OW; p.pad = pad; p.act = act;
  if (in_l.pitch == 0) in_l = dense_layout(H, W);
  if (out_l.pitch == 0) out_l = dense_layout(OH, OW);
  // a padded layout's pad row / column is zero and everything beyond the map is out of the tensor map's range
  // (zero-filled), so the halo reads the same values as over a dense map
  if (in_l.off != 0 && (in_l.off != 1 || in_l.pitch != W + 1 || in_l.img_rows != H + 1)) return cudaErrorInvalidValue;
  p.in_l = in_l; p.out_l = out_l;
  p.tiles_x = (OW + tw - 1) / tw; p.tiles_y = (OH + kTH - 1) / kTH;
  p.n_tiles = N * p.tiles_y * p.tiles_x;
  p.error_flag = error_flag;

  auto enc = dw_get_encode();
  if (!enc) return cudaErrorNotSupported;
  CUtensorMap tm;
  const CUtensorMapDataType tdt = dt == kF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                  : dt == kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cuuint64_t gdim[4] = {(cuuint64_t)C, (cuuint64_t)in_l.pitch, (cuuint64_t)in_l.img_rows, (cuuint64_t)N};
  cuuint64_t gstr[3] = {(cuuint64_t)C * es, (cuuint64_t)in_l.pitch * C * es, (cuuint64_t)in_l.img_rows * in_l.pitch * C * es};
  cuuint32_t box[4] = {(cuuint32_t)(cbv * V), (cuuint32_t)IW, (cuuint32_t)IH, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (enc(&tm, tdt, 4, const_cast<void*>(x), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;

  const int chunks = (cv + cbv - 1) / cbv;
  const int per_sm = smem <= 72 * 1024 ? 3 : smem <= 110 * 1024 ? 2 : 1;
  int gx = (sm_count > 0 ? sm_count : 148) * per_sm / chunks;
  if (gx < 1) gx = 1;
  if (gx > p.n_tiles) gx = p.n_tiles;
  const dim3 grid((unsigned)gx, (unsigned)chunks);
  if (chunks > 65535) return cudaErrorInvalidValue;
  if (dt == kF32) return launch_typed<float>(tm, p, R, stride, grid, smem, st);
  if (dt == kF16) return launch_typed<__half>(tm, p, R, stride, grid, smem, st);
  return launch_typed<__nv_bfloat16>(tm, p, R, stride, grid, smem, st);
}

}  // namespace nncv_b200
