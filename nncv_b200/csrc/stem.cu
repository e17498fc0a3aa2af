// ResNet stem for sm_100a: 7x7 stride-2 pad-3 convolution (3 -> 64 channels) + folded batch-norm
// + ReLU + 3x3 stride-2 pad-1 max-pool in ONE kernel, on tcgen05 tensor cores.
//
// Reference semantics (nncv tree): tests/Nets/Res18.mlir:118-151 (tensor.pad 3, conv_2d_nchw_fchw
// with strides 2, the batch-norm and ReLU generics, tensor.pad -inf 1, pooling_nchw_max 3x3
// strides 2).  nncv tiles this conv with an extra {1,1} tile for strided ops
// (src/nncv/compiler/Conversion/CodeGen/LlvmCpu/ModernTile.cpp:201-209).
//
// Input format: the NCHW image is first rewritten (nchw_to_stem_rows) as fp16 rows of
// 4-channel pixels with 4 zero pixels on the left and >= 4 on the right:
//     row(n, y) = [0 0 0 0 | p(0) ... p(W-1) | 0 0 0 0 ...],   p = (c0, c1, c2, 0),  8 bytes each.
// With this layout the A operand of the implicit GEMM needs no im2col at all.  tcgen05.mma's
// un-swizzled K-major operand layout addresses element (row i, 16-byte chunk j) at
//     start + (i % 8) * 16 + (i / 8) * SBO + j * LBO .
// Choosing SBO = 128 and LBO = 16 makes that  start + 16 * (i + j):  row i (output column x0+i)
// reads the 16-byte chunks i, i+1, i+2, i+3 of the input row, i.e. the pixel pairs
// 2x-4 .. 2x+3 -- exactly the 7 taps (plus one zero-weight tap in front) of a stride-2 window.
// The rows of the operand overlap in memory; the tensor core only does address arithmetic.
// One filter row is therefore K = 32 (two MMAs of K = 16), a conv output row of up to 128
// pixels is 14 MMAs of 128 x 64 x 16, and every input row is brought into shared memory once
// (bulk async copies of row pairs into a ring) and reused by the seven filter rows of four
// output rows.
//
// Roles (11 warps, persistent over (image, band of pooled rows) items):
//   warp 0   bulk-copies input rows into the ring; weights (28 KB) are resident.
//   warps 1, 10  one thread each issues the MMAs of alternate conv rows into four TMEM accumulators.
//   warps 2-9  read the accumulator, apply scale/shift, keep the vertical maximum of the three
//            conv rows of a pooling window in registers, write one fp16 row per pooled row to
//            shared memory, take the horizontal maximum there (clamped window = -inf padding),
//            apply ReLU (it commutes with max) and store the pooled row, 16 bytes per thread,
//            fully coalesced.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace {

constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kIssuerBWarp = 2 + kEpiWarps;          // second MMA-issuing warp, after the epilogue warps
constexpr int kThreads = 64 + kEpiThreads + 32;
constexpr int kRingSlots = 8;       // input row PAIRS (rows 2k, 2k+1) resident in shared memory
constexpr int kAccBufs = 4;         // TMEM accumulators of 64 columns
constexpr int kConvRing = 2;        // rows of vertical maxima in shared memory (double buffer)
constexpr int kWBytes = 7 * 4096;   // packed weights: 7 filter rows x [64 x 32] fp16

// Optional clock64() trace of CTA 0 (built only with -DNNCV_B200_TRACE; a tuning aid).
#ifdef NNCV_B200_TRACE
unsigned long long* g_stem_trace = nullptr;  // device buffer [2 roles][64 rows][8 stamps]
#define ST_TRACE(role, idx, k)                                                            \
  do {                                                                                    \
    if (p.trace && blockIdx.x == 0 && (idx) < 64)                                          \
      p.trace[((role) * 64 + (idx)) * 8 + (k)] = (unsigned long long)clock64();            \
  } while (0)
#else
#define ST_TRACE(role, idx, k) \
  do {                         \
  } while (0)
#endif

struct StemParams {
  unsigned long long* trace;
  const uint8_t* in_rows;   // [N][H][RW] pixels of 8 bytes
  const uint8_t* wpack;     // kWBytes
  const float* scale;
  const float* shift;
  uint16_t* out;            // pooled [N, PH, PW, 64] in layout ol
  int* error_flag;
  Layout ol;
  int N, H, W, OH, OW, PH, PW;
  int row_bytes;            // RW * 8
  int slot_bytes;           // ring slot of one row pair (covers the junk rows of the last x tile)
  int x_tiles;              // ceil(OW / 128)
  int bands, band_rows;     // pooled rows per item
  int bf16;
};

// Un-swizzled K-major descriptor: LBO = byte step between 16-byte chunks along K, SBO = byte
// step between 8-row groups along M/N.
__device__ __forceinline__ uint64_t desc_noswz(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  const uint32_t lo = ((addr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16);
  const uint32_t hi = (sbo >> 4) | (1u << 14);
  return ptx::desc_from_halves(lo, hi);
}

template <int XT>   // x tiles of 128 output columns per conv row (1 or 2)
__global__ void __launch_bounds__(kThreads, 1) stem_pool_kernel(const StemParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_abort;
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  const int crow_bytes = p.x_tiles * 128 * 128;            // one fp16 conv row, 128 B per pixel
  const uint32_t sW = base;
  const uint32_t sRing = sW + kWBytes;
  const uint32_t sConv = sRing + (uint32_t)kRingSlots * p.slot_bytes + 256;
  const uint32_t bars = (sConv + (uint32_t)kConvRing * crow_bytes + 7u) & ~7u;
  const uint32_t full = bars, empty = bars + 8 * kRingSlots;
  const uint32_t acc_full = empty + 8 * kRingSlots, acc_empty = acc_full + 8 * kAccBufs;
  const uint32_t w_full = acc_empty + 8 * kAccBufs;
  const uint32_t tmem_slot = w_full + 8;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kRingSlots; ++i) {
      ptx::mbar_init(full + 8 * i, 1);
      ptx::mbar_init(empty + 8 * i, 1);
    }
    for (int i = 0; i < kAccBufs; ++i) {
      ptx::mbar_init(acc_full + 8 * i, 1);
      ptx::mbar_init(acc_empty + 8 * i, kEpiThreads);
    }
    ptx::mbar_init(w_full, 1);
    ptx::mbar_fence_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kAccBufs * 64);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  // The prologue above touched nothing the previous kernel of the stream writes; everything
  // below may, so wait for that kernel here and let the next one start its own prologue.
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  volatile int* abort_flag = &s_abort;

  const int total_items = p.N * p.bands;
  // item -> image, conv rows [y0, y1], input row pairs [ir0, ir1] (pair k = rows 2k, 2k+1)
  auto item_of = [&](int i, int& n, int& p0, int& p1, int& y0, int& y1, int& ir0, int& ir1) {
    const int w = (int)blockIdx.x + i * (int)gridDim.x;
    if (w >= total_items) return false;
    n = w / p.bands;
    const int b = w - n * p.bands;
    p0 = b * p.band_rows;
    p1 = min(p.PH, p0 + p.band_rows);
    y0 = max(0, 2 * p0 - 1);
    y1 = min(p.OH - 1, 2 * p1 - 1);
    ir0 = max(0, 2 * y0 - 3) >> 1;          // first and last input-row PAIR of the item
    ir1 = min(p.H - 1, 2 * y1 + 3) >> 1;
    return true;
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- input rows -------
    if (lane == 0) {
      ptx::mbar_arrive_expect_tx(w_full, kWBytes);
      ptx::bulk_g2s(sW, p.wpack, kWBytes, w_full);
      uint32_t seq = 0;
      bool okw = true;
      for (int i = 0; okw; ++i) {
        int n, p0, p1, y0, y1, ir0, ir1;
        if (!item_of(i, n, p0, p1, y0, y1, ir0, ir1)) break;
        const uint8_t* img = p.in_rows + (size_t)n * p.H * p.row_bytes;
        for (int pk = ir0; pk <= ir1; ++pk, ++seq) {
          const uint32_t slot = seq % kRingSlots;
          if (!ptx::mbar_wait_abortable(empty + 8 * slot, ((seq / kRingSlots) & 1u) ^ 1u, abort_flag)) { okw = false; break; }
          const uint32_t bytes = (uint32_t)p.row_bytes * (uint32_t)min(2, p.H - 2 * pk);   // rows are contiguous
          ptx::mbar_arrive_expect_tx(full + 8 * slot, bytes);
          ptx::bulk_g2s(sRing + slot * p.slot_bytes, img + (size_t)(2 * pk) * p.row_bytes, bytes, full + 8 * slot);
        }
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitProducer);
    }
  } else if (warp == 1 || warp == kIssuerBWarp) {
    // ---------------------------------------------------------------- MMA issuers ------
    // Two issuing threads take alternate accumulators (conv rows): while one waits on its
    // barriers and commits, the other keeps the tensor pipe fed.  Input row pairs are handed
    // back by the epilogue (it sees every row finish, in order), not by the issuers.
    if (lane == 0) {
      const uint32_t issuer = warp == 1 ? 0u : 1u;
      const uint32_t idesc = ptx::umma_idesc(128, 64, p.bf16 ? 1 : 0);
      bool okw = ptx::mbar_wait_abortable(w_full, 0, abort_flag);
      uint32_t seq_base = 0, acc_cnt = 0;
      for (int i = 0; okw; ++i) {
        int n, p0, p1, y0, y1, ir0, ir1;
        if (!item_of(i, n, p0, p1, y0, y1, ir0, ir1)) break;
        int waited_upto = ir0;     // pairs [ir0, waited_upto) are known to be in the ring
        for (int y = y0; y <= y1 && okw; ++y) {
          // does this issuer own any accumulator of row y?
          bool mine = false;
          for (int xt = 0; xt < p.x_tiles; ++xt) mine |= ((acc_cnt + xt) & 1u) == issuer;
          if (!mine) { acc_cnt += p.x_tiles; continue; }
          const int need = min(ir1, y + 1);            // conv row y reads pairs y-2 .. y+1
          for (; waited_upto <= need; ++waited_upto) {
            const uint32_t s = seq_base + (uint32_t)(waited_upto - ir0);
            if (!ptx::mbar_wait_abortable(full + 8 * (s % kRingSlots), (s / kRingSlots) & 1u, abort_flag)) { okw = false; break; }
          }
          if (!okw) break;
          ST_TRACE(0, acc_cnt, 5);
          ptx::tc_fence_after();
          // shared-memory address of each filter row's input row (0 = zero padding row, skipped)
          uint32_t row_addr[7];
#pragma unroll
          for (int r = 0; r < 7; ++r) {
            const int ir = 2 * y + r - 3;
            row_addr[r] = 0;
            if (ir >= 0 && ir < p.H) {
              const uint32_t s = seq_base + (uint32_t)((ir >> 1) - ir0);
              row_addr[r] = sRing + (s % kRingSlots) * p.slot_bytes + (uint32_t)(ir & 1) * p.row_bytes;
            }
          }
          for (int xt = 0; xt < p.x_tiles && okw; ++xt, ++acc_cnt) {
            if ((acc_cnt & 1u) != issuer) continue;
            const uint32_t ab = acc_cnt % kAccBufs;
            ST_TRACE(0, acc_cnt, 0);
            if (!ptx::mbar_wait_abortable(acc_empty + 8 * ab, ((acc_cnt / kAccBufs) & 1u) ^ 1u, abort_flag)) { okw = false; break; }
            ST_TRACE(0, acc_cnt, 1);
            ptx::tc_fence_after();
            uint32_t accumulate = 0;
#pragma unroll
            for (int r = 0; r < 7; ++r) {
              if (row_addr[r] == 0) continue;   // zero padding rows contribute nothing
              const uint32_t a_addr = row_addr[r] + (uint32_t)xt * 2048u;
              const uint32_t b_addr = sW + (uint32_t)r * 4096u;
#pragma unroll
              for (int k2 = 0; k2 < 2; ++k2) {
                ptx::umma_f16(tmem_base + ab * 64, desc_noswz(a_addr + k2 * 32, 16, 128),
                              desc_noswz(b_addr + k2 * 2048, 1024, 128), idesc, accumulate);
                accumulate = 1;
              }
            }
            ST_TRACE(0, acc_cnt, 2);
            ptx::tc_commit(acc_full + 8 * ab);
            ST_TRACE(0, acc_cnt, 3);
          }
        }
        seq_base += (uint32_t)(ir1 - ir0 + 1);
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitMma);
    }
  } else {
    // ---------------------------------------------------------------- epilogue ---------
    // Thread (quadrant, lane) owns output column x = xt*128 + row and 32 of the 64 channels of
    // every conv row, so the VERTICAL part of the 3x3 max-pool runs in its registers: `prev`
    // holds the last odd conv row (the top row of the next pooled row), `vm` the running
    // maximum.  Only one row per pooled row goes to shared memory; the horizontal part reads
    // three pixels of it.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;          // output column within the x tile
    const int et = threadIdx.x - 64;           // 0..255
    float4 sc[8], sh[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sc[i] = p.scale ? __ldg(reinterpret_cast<const float4*>(p.scale + half * 32) + i) : make_float4(1.f, 1.f, 1.f, 1.f);
      sh[i] = p.shift ? __ldg(reinterpret_cast<const float4*>(p.shift + half * 32) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    auto hmax = [&](uint32_t a, uint32_t b) -> uint32_t {
      if (p.bf16) {
        __nv_bfloat162 r = __hmax2_nan(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
      }
      __half2 r = __hmax2_nan(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
      return *reinterpret_cast<uint32_t*>(&r);
    };
    uint32_t acc_cnt = 0, epi_seq_base = 0;
    bool okw = true;
    for (int i = 0; okw; ++i) {
      int n, p0, p1, y0, y1, ir0, ir1;
      if (!item_of(i, n, p0, p1, y0, y1, ir0, ir1)) break;
      int next_pool = p0;
      int released_upto = ir0;   // input row pairs [ir0, released_upto) were handed back to the producer
      uint32_t prev[XT][16], vm[XT][16];
      bool has_prev = false;
      for (int y = y0; y <= y1 && okw; ++y) {
        const bool completes = next_pool < p1 && min(2 * next_pool + 1, p.OH - 1) == y;
        const bool top_only = (y & 1) && y == 2 * next_pool - 1;   // first row of a band: only the top of a window
        const uint32_t vrow = sConv + (uint32_t)(next_pool & 1) * crow_bytes;
#pragma unroll
        for (int xt = 0; xt < XT; ++xt) {
          if (xt >= p.x_tiles) break;
          const uint32_t ab = acc_cnt % kAccBufs;
          if (et == 0) ST_TRACE(1, acc_cnt, 0);
          const bool got = ptx::mbar_wait_abortable(acc_full + 8 * ab, (acc_cnt / kAccBufs) & 1u, abort_flag);
          if (et == 0) ST_TRACE(1, acc_cnt, 1);
          if (!ptx::named_bar_and(3, kEpiThreads, got)) { okw = false; break; }
          if (et == 0) ST_TRACE(1, acc_cnt, 2);
          ptx::tc_fence_after();
          uint32_t acc[32];
          __syncwarp();
          ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + ab * 64 + half * 32, acc);
          ptx::tmem_ld_wait();
          if (et == 0) ST_TRACE(1, acc_cnt, 3);
          ptx::tc_fence_before();
          ptx::mbar_arrive(acc_empty + 8 * ab);
          ++acc_cnt;
          uint32_t cur[16];
#pragma unroll
          for (int h = 0; h < 16; ++h) {
            const int e = 2 * h;
            const float4 s4 = sc[e >> 2], b4 = sh[e >> 2];
            const float sa = (e & 2) ? s4.z : s4.x, sb = (e & 2) ? s4.w : s4.y;
            const float ba = (e & 2) ? b4.z : b4.x, bb = (e & 2) ? b4.w : b4.y;
            const float a = fmaf(__uint_as_float(acc[e]), sa, ba);
            const float b = fmaf(__uint_as_float(acc[e + 1]), sb, bb);
            if (p.bf16) {
              __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
              cur[h] = *reinterpret_cast<uint32_t*>(&v);
            } else {
              __half2 v = __floats2half2_rn(a, b);
              cur[h] = *reinterpret_cast<uint32_t*>(&v);
            }
          }
          if ((y & 1) == 0) {          // middle row of window y/2
#pragma unroll
            for (int h = 0; h < 16; ++h) vm[xt][h] = has_prev ? hmax(prev[xt][h], cur[h]) : cur[h];
          } else {                     // bottom row of window (y-1)/2 and top row of the next one
            if (!top_only) {
#pragma unroll
              for (int h = 0; h < 16; ++h) vm[xt][h] = hmax(vm[xt][h], cur[h]);
            }
#pragma unroll
            for (int h = 0; h < 16; ++h) prev[xt][h] = cur[h];
          }
          if (completes) {
            const int x = xt * 128 + row;
            const uint32_t prow = vrow + (uint32_t)x * 128u;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              const uint32_t chunk = (uint32_t)(half * 4 + c4);
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(prow + ((chunk ^ (uint32_t)(x & 7)) << 4)),
                           "r"(vm[xt][c4 * 4]), "r"(vm[xt][c4 * 4 + 1]), "r"(vm[xt][c4 * 4 + 2]), "r"(vm[xt][c4 * 4 + 3])
                           : "memory");
            }
          }
        }
        if (!okw) break;
        if (y & 1) has_prev = true;
        if (et == 0) {
          // every MMA of rows <= y has finished (their accumulators were seen full, in order): the
          // pairs that only those rows read go back to the producer
          const int new_upto = (y == y1) ? ir1 + 1 : min(ir1 + 1, y - 1);
          for (; released_upto < new_upto; ++released_upto)
            ptx::mbar_arrive(empty + 8 * ((epi_seq_base + (uint32_t)(released_upto - ir0)) % kRingSlots));
        }
        if (!completes) continue;
        if (et == 0) ST_TRACE(1, acc_cnt - 1, 4);
        ptx::named_bar_sync(1, kEpiThreads);   // the vertical maxima of pooled row next_pool are in shared memory
        if (et == 0) ST_TRACE(1, acc_cnt - 1, 5);
        {
          const int pr = next_pool++;
          uint16_t* orow = p.out + ((size_t)((size_t)n * p.ol.img_rows + pr + p.ol.off) * p.ol.pitch + p.ol.off) * 64;
          for (int u = et; u < p.PW * 8; u += kEpiThreads) {
            const int px = u >> 3, c = u & 7;
            // clamped window: a tap outside the map is replaced by a neighbour already in the window
            const int xs[3] = {max(0, 2 * px - 1), 2 * px, min(p.OW - 1, 2 * px + 1)};
            uint32_t v[3][4];
#pragma unroll
            for (int j = 0; j < 3; ++j)
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(v[j][0]), "=r"(v[j][1]), "=r"(v[j][2]), "=r"(v[j][3])
                           : "r"(vrow + (uint32_t)xs[j] * 128u + (((uint32_t)c ^ (uint32_t)(xs[j] & 7)) << 4)));
            uint32_t m[4];
            const uint32_t zero = 0u;   // +0.0 in both halves, for fp16 and bf16
#pragma unroll
            for (int h = 0; h < 4; ++h) m[h] = hmax(hmax(hmax(v[0][h], v[1][h]), v[2][h]), zero);   // ReLU after the max
            *reinterpret_cast<uint4*>(orow + (size_t)px * 64 + c * 8) = make_uint4(m[0], m[1], m[2], m[3]);
          }
          if (et == 0) ST_TRACE(1, acc_cnt - 1, 6);
        }
      }
      epi_seq_base += (uint32_t)(ir1 - ir0 + 1);
      // the next item reuses the two shared-memory rows only after everyone has finished pooling
      ptx::named_bar_sync(2, kEpiThreads);
    }
    if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitEpilogue);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, kAccBufs * 64);
  }
}

// NCHW (any dtype) -> fp16/bf16 rows of 4-channel pixels with 4 zero pixels in front; one thread
// per output pixel slot (8-byte store), the tail of every row is zero.
template <typename SrcT, typename DstT>
__global__ void nchw_to_stem_rows_kernel(const SrcT* __restrict__ src, DstT* __restrict__ dst, int N,
                                         int H, int W, int RW) {
  const long long total = (long long)N * H * RW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int xs = (int)(i % RW);
    const long long t = i / RW;
    const int y = (int)(t % H);
    const int n = (int)(t / H);
    const int x = xs - 4;
    alignas(8) DstT v[4];
    if (x >= 0 && x < W) {
      const SrcT* s = src + ((size_t)n * 3 * H + y) * W + x;
      v[0] = (DstT)(float)s[0];
      v[1] = (DstT)(float)s[(size_t)H * W];
      v[2] = (DstT)(float)s[(size_t)2 * H * W];
      v[3] = (DstT)0.0f;
    } else {
      v[0] = v[1] = v[2] = v[3] = (DstT)0.0f;
    }
    *reinterpret_cast<uint2*>(dst + i * 4) = *reinterpret_cast<const uint2*>(v);
  }
}

// Fast variant for W % 8 == 0: one thread per 8 pixels (three 16- or 32-byte channel reads, one
// 64-byte write).  It writes only real pixels: the zero pixels in front of and behind every row
// must already be zero in dst (the executor clears the buffer once per shape).
template <typename SrcT, typename DstT>
__global__ void nchw_to_stem_rows8_kernel(const SrcT* __restrict__ src, DstT* __restrict__ dst, int N,
                                          int H, int W, int RW) {
  const int gw = W / 8;
  const long long total = (long long)N * H * gw;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int xg = (int)(i % gw);
    const long long t = i / gw;
    const int y = (int)(t % H);
    const int n = (int)(t / H);
    const SrcT* s = src + ((size_t)n * 3 * H + y) * W + xg * 8;
    alignas(16) SrcT c0[8], c1[8], c2[8];
    constexpr int kVec = (int)(8 * sizeof(SrcT) / 16);   // uint4 loads per channel
#pragma unroll
    for (int v = 0; v < kVec; ++v) {
      reinterpret_cast<uint4*>(c0)[v] = __ldg(reinterpret_cast<const uint4*>(s) + v);
      reinterpret_cast<uint4*>(c1)[v] = __ldg(reinterpret_cast<const uint4*>(s + (size_t)H * W) + v);
      reinterpret_cast<uint4*>(c2)[v] = __ldg(reinterpret_cast<const uint4*>(s + (size_t)2 * H * W) + v);
    }
    alignas(16) DstT o[32];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      o[4 * k] = (DstT)(float)c0[k];
      o[4 * k + 1] = (DstT)(float)c1[k];
      o[4 * k + 2] = (DstT)(float)c2[k];
      o[4 * k + 3] = (DstT)0.0f;
    }
    uint4* d = reinterpret_cast<uint4*>(dst + (((size_t)n * H + y) * RW + 4 + xg * 8) * 4);
#pragma unroll
    for (int v = 0; v < 4; ++v) d[v] = reinterpret_cast<const uint4*>(o)[v];
  }
}

// W[64][3][7][7] -> per filter row r a [64 x 32] K-major un-swizzled tile: element (n, k) at
// (k / 8) * 1024 + (n / 8) * 128 + (n % 8) * 16 + (k % 8) * 2; k = 4 * tap + channel, tap 0 is the
// zero-weight pixel in front of the window, channel 3 is the zero padding channel.
template <typename SrcT, typename DstT>
__global__ void pack_stem_weights_kernel(const SrcT* __restrict__ w, DstT* __restrict__ dst) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 7 * 64 * 32) return;
  const int k = i % 32, n = (i / 32) % 64, r = i / (32 * 64);
  const int tap = k / 4, ch = k % 4;
  float v = 0.0f;
  if (tap >= 1 && ch < 3) v = (float)w[((n * 3 + ch) * 7 + r) * 7 + (tap - 1)];
  const size_t off = (size_t)r * 4096 + (size_t)(k / 8) * 1024 + (size_t)(n / 8) * 128 + (size_t)(n % 8) * 16 + (size_t)(k % 8) * 2;
  *reinterpret_cast<DstT*>(reinterpret_cast<uint8_t*>(dst) + off) = (DstT)v;
}

template <typename F>
cudaError_t by_dt(DType t, F&& f) {
  switch (t) {
    case kF32: return f(float{});
    case kF16: return f(__half{});
    case kBF16: return f(__nv_bfloat16{});
  }
  return cudaErrorInvalidValue;
}

}  // namespace

#ifdef NNCV_B200_TRACE
extern "C" void nncv_b200_debug_set_stem_trace(unsigned long long* dev_buf) { g_stem_trace = dev_buf; }
#endif

int stem_row_pixels(int W) { return (4 + W + 4 + 1) & ~1; }
size_t stem_rows_bytes(int N, int H, int W) { return (size_t)N * H * stem_row_pixels(W) * 8; }
size_t stem_wpack_bytes() { return kWBytes; }

cudaError_t launch_nchw_to_stem_rows(const void* src, DType src_dt, void* dst, DType dst_dt, int N, int H,
                                     int W, bool pads_are_zero, cudaStream_t stream) {
  const int RW = stem_row_pixels(W);
  if (dst_dt == kF32) return cudaErrorInvalidValue;
  const bool fast = pads_are_zero && W % 8 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  const long long total = fast ? (long long)N * H * (W / 8) : (long long)N * H * RW;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  return by_dt(src_dt, [&](auto st) {
    using S = decltype(st);
    if (fast) {
      if (dst_dt == kBF16)
        nchw_to_stem_rows8_kernel<S, __nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
            static_cast<const S*>(src), static_cast<__nv_bfloat16*>(dst), N, H, W, RW);
      else
        nchw_to_stem_rows8_kernel<S, __half><<<(int)blocks, 256, 0, stream>>>(
            static_cast<const S*>(src), static_cast<__half*>(dst), N, H, W, RW);
    } else if (dst_dt == kBF16) {
      nchw_to_stem_rows_kernel<S, __nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
          static_cast<const S*>(src), static_cast<__nv_bfloat16*>(dst), N, H, W, RW);
    } else {
      nchw_to_stem_rows_kernel<S, __half><<<(int)blocks, 256, 0, stream>>>(
          static_cast<const S*>(src), static_cast<__half*>(dst), N, H, W, RW);
    }
    return cudaGetLastError();
  });
}

cudaError_t launch_pack_stem_weights(const void* w, DType w_dt, void* dst, DType dst_dt, cudaStream_t stream) {
  if (dst_dt == kF32) return cudaErrorInvalidValue;
  return by_dt(w_dt, [&](auto st) {
    using S = decltype(st);
    if (dst_dt == kBF16)
      pack_stem_weights_kernel<S, __nv_bfloat16><<<(7 * 64 * 32 + 255) / 256, 256, 0, stream>>>(
          static_cast<const S*>(w), static_cast<__nv_bfloat16*>(dst));
    else
      pack_stem_weights_kernel<S, __half><<<(7 * 64 * 32 + 255) / 256, 256, 0, stream>>>(
          static_cast<const S*>(w), static_cast<__half*>(dst));
    return cudaGetLastError();
  });
}

cudaError_t launch_stem_pool(const StemArgs& a, cudaStream_t stream) {
  if (a.ab == kF32 || a.N <= 0 || a.H < 7 || a.W < 7) return cudaErrorInvalidValue;
  StemParams p;
#ifdef NNCV_B200_TRACE
  p.trace = g_stem_trace;
#else
  p.trace = nullptr;
#endif
  p.in_rows = static_cast<const uint8_t*>(a.in_rows);
  p.wpack = static_cast<const uint8_t*>(a.wpack);
  p.scale = a.scale; p.shift = a.shift;
  p.out = static_cast<uint16_t*>(a.out);
  p.error_flag = a.error_flag;
  p.N = a.N; p.H = a.H; p.W = a.W;
  p.OH = (a.H + 6 - 7) / 2 + 1; p.OW = (a.W + 6 - 7) / 2 + 1;
  p.PH = (p.OH + 2 - 3) / 2 + 1; p.PW = (p.OW + 2 - 3) / 2 + 1;
  p.ol = a.out_l.pitch ? a.out_l : dense_layout(p.PH, p.PW);
  p.row_bytes = stem_row_pixels(a.W) * 8;
  p.x_tiles = (p.OW + 127) / 128;
  // a slot holds a pair of rows; the junk rows of the last x tile read up to byte
  // x_tiles * 2048 + 64 past the start of a row
  int slot = p.row_bytes + p.x_tiles * 2048 + 64;
  if (slot < 2 * p.row_bytes) slot = 2 * p.row_bytes;
  p.slot_bytes = (slot + 127) & ~127;
  p.bf16 = a.ab == kBF16;
  const int sms = a.sm_count > 0 ? a.sm_count : 148;
  // bands: enough items to fill the SMs several times over, at least 4 pooled rows each
  int band_rows = p.PH;
  while (band_rows > 4 && (long long)a.N * ((p.PH + band_rows - 1) / band_rows) < 6LL * sms) band_rows = (band_rows + 1) / 2;
  p.band_rows = band_rows;
  p.bands = (p.PH + band_rows - 1) / band_rows;
  const size_t smem = 128 + kWBytes + (size_t)kRingSlots * p.slot_bytes + 256 +
                      (size_t)kConvRing * p.x_tiles * 128 * 128 + 8 + 8 * (2 * kRingSlots + 2 * kAccBufs + 1) + 16;
  if (smem > 227 * 1024) return cudaErrorInvalidConfiguration;
  if (p.x_tiles > 2) return cudaErrorInvalidConfiguration;   // wider than 512 pixels: not covered by the fused kernel
  cudaError_t e = p.x_tiles == 1
                      ? cudaFuncSetAttribute(stem_pool_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                      : cudaFuncSetAttribute(stem_pool_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int items = a.N * p.bands;
  if (p.x_tiles == 1) return launch_pdl(stem_pool_kernel<1>, dim3(items < sms ? items : sms), dim3(kThreads), smem, stream, p);
  return launch_pdl(stem_pool_kernel<2>, dim3(items < sms ? items : sms), dim3(kThreads), smem, stream, p);
}

}  // namespace nncv_b200
