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
// With this layout the A operand of the implicit GEMM needs no im2col at all.  Two operand paths:
//
// Plain rows (SW = false; any shape up to 512 pixels wide).  tcgen05.mma's un-swizzled K-major
// layout addresses element (row i, 16-byte chunk j) at  start + (i % 8) * 16 + (i / 8) * SBO + j * LBO.
// Choosing SBO = 128 and LBO = 16 makes that  start + 16 * (i + j):  row i (output column x0+i)
// reads the chunks i .. i+3 of the input row, i.e. the pixels 2x-4 .. 2x+3 -- the 7 taps (plus one
// zero-weight tap in front) of a stride-2 window.  The operand rows overlap in memory; the tensor
// core only does address arithmetic.  One filter row is K = 32, a conv row 14 MMAs of
// 128 x 64 x 16; input rows are bulk-copied once, in pairs, into a ring and reused by the seven
// filter rows of four conv rows; two threads issue the MMAs of alternate conv rows.
//
// Swizzled pairs (SW = true; even H, conv row of at most 128 pixels).  Rows 2k and 2k+1 are stored
// interleaved in 16-byte chunks, one tiled TMA copy through a tensor map with overlapping strides
// lands each pair as a canonical swizzled [128 x 64] tile, and one thread multiplies it with the
// weight blocks of the four conv rows it feeds at once (see the kernel's comments).
//
// Roles (11 warps, persistent over (image, band of pooled rows) items):
//   warp 0   copies input rows / row pairs into the ring; the packed weights are resident.
//   warp 1   issues MMAs (plain rows: together with warp 10, on alternate conv rows).
//   warp 10  swizzled pairs: scout -- does the issuing lane's barrier waits up to four pairs ahead.
//   warps 2-9  per pooled row: read the accumulators of two conv rows, apply scale/shift, keep the
//            vertical maximum of the pooling window in registers, write one fp16 row to shared
//            memory, take the horizontal maximum there (clamped window = -inf padding), apply
//            ReLU (it commutes with max) and store the pooled row, 16 bytes per thread, coalesced.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cudaTypedefs.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace {

constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kIssuerBWarp = 2 + kEpiWarps;          // second MMA-issuing warp, after the epilogue warps
constexpr int kThreads = 64 + kEpiThreads + 32;
constexpr int kRingSlots = 8;       // input row PAIRS (rows 2k, 2k+1) resident in shared memory
constexpr int kAccBufs = 4;         // TMEM accumulators of 64 columns, per x tile
constexpr int kConvRing = 2;        // rows of vertical maxima in shared memory (double buffer)
constexpr int kWBytes = 7 * 4096;   // packed weights: 7 filter rows x [64 x 32] fp16
constexpr int kWBytesSw = 4 * 8192; // swizzled variant: 4 filter-row pairs x [64 x 64] fp16
constexpr int kSwSlot = 16384;      // swizzled variant: one row pair as a [128 pixels x 128 B] operand tile

struct StemParams {
  const uint8_t* in_rows;   // [N][H][RW] pixels of 8 bytes
  const uint8_t* wpack;     // kWBytes
  const float* scale;
  const float* shift;
  uint16_t* out;            // pooled [N, PH, PW, 64] in layout ol
  int* error_flag;
  Layout ol;
  int N, H, W, OH, OW, PH, PW;
  int row_bytes;            // RW * 8
  int w_bytes;              // bytes of packed weights the kernel keeps resident
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

// SW = true (one x tile, even H): the input rows are stored in PAIRS, interleaved in 16-byte
// chunks (chunk c of row 2k, chunk c of row 2k+1, chunk c+1 of row 2k, ...), so the 8-pixel
// windows of both rows that output pixel x reads are 128 contiguous bytes starting at byte 32x
// of the pair.  The producer fetches a pair with ONE tiled TMA copy whose tensor map has
// OVERLAPPING strides -- the "output pixel" dimension advances 32 bytes under a 128-byte
// innermost extent -- and shared memory receives a canonical [128 x 64] K-major tile in the
// 128-byte swizzle.  The tensor core reads a conflict-free operand (two filter rows per K
// block, 16 MMAs per conv row) instead of the overlapping un-swizzled one.
template <int XT, bool SW>   // x tiles of 128 output columns per conv row (1 or 2)
__global__ void __launch_bounds__(kThreads, 1) stem_pool_kernel(const __grid_constant__ CUtensorMap tm_in, const StemParams p) {
  // accumulators of 64 TMEM columns: a step of the epilogue drains 2 * XT of them; the pair kernel
  // keeps eight conv rows in flight
  constexpr uint32_t kAcc = SW ? 8u : (uint32_t)(kAccBufs * XT);
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_abort;
  __shared__ int s_consumed;   // pair kernel: newest pair the epilogue has finished waiting for
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const int crow_bytes = p.x_tiles * 128 * 128;            // one fp16 conv row, 128 B per pixel
  const uint32_t sW = base;
  const uint32_t sRing = sW + (uint32_t)p.w_bytes;
  const uint32_t sConv = sRing + (uint32_t)kRingSlots * p.slot_bytes + 256;
  const uint32_t bars = (sConv + (uint32_t)kConvRing * crow_bytes + 7u) & ~7u;
  const uint32_t full = bars, empty = bars + 8 * kRingSlots;
  const uint32_t acc_full = empty + 8 * kRingSlots, acc_empty = acc_full + 8 * kAcc;
  const uint32_t w_full = acc_empty + 8 * kAcc;
  const uint32_t go = w_full + 8;                 // pair kernel: "everything pair seq needs is there", 4 in flight
  const uint32_t tmem_slot = go + 8 * 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    s_abort = 0;
    s_consumed = -1;
    for (int i = 0; i < kRingSlots; ++i) {
      ptx::mbar_init(full + 8 * i, 1);
      ptx::mbar_init(empty + 8 * i, 1);
    }
    for (int i = 0; i < (int)kAcc; ++i) {
      ptx::mbar_init(acc_full + 8 * i, 1);
      ptx::mbar_init(acc_empty + 8 * i, kEpiWarps);
    }
    ptx::mbar_init(w_full, 1);
    for (int i = 0; i < 4; ++i) ptx::mbar_init(go + 8 * i, 1);
    ptx::mbar_fence_init();
  }
  if (SW && threadIdx.x == 32) ptx::prefetch_tensormap(&tm_in);
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kAcc * 64);
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
      ptx::mbar_arrive_expect_tx(w_full, (uint32_t)p.w_bytes);
      ptx::bulk_g2s(sW, p.wpack, (uint32_t)p.w_bytes, w_full);
      uint32_t seq = 0;
      bool okw = true;
      for (int i = 0; okw; ++i) {
        int n, p0, p1, y0, y1, ir0, ir1;
        if (!item_of(i, n, p0, p1, y0, y1, ir0, ir1)) break;
        const uint8_t* img = p.in_rows + (size_t)n * p.H * p.row_bytes;
        for (int pk = ir0; pk <= ir1; ++pk, ++seq) {
          const uint32_t slot = seq % kRingSlots;
          if (!ptx::mbar_wait_abortable(empty + 8 * slot, ((seq / kRingSlots) & 1u) ^ 1u, abort_flag)) { okw = false; break; }
          if (SW) {
            ptx::mbar_arrive_expect_tx(full + 8 * slot, (uint32_t)kSwSlot);
            ptx::tma_load_3d(sRing + slot * p.slot_bytes, &tm_in, 0, 0, n * (p.H >> 1) + pk, full + 8 * slot);
          } else {
            const uint32_t bytes = (uint32_t)p.row_bytes * (uint32_t)min(2, p.H - 2 * pk);   // rows are contiguous
            ptx::mbar_arrive_expect_tx(full + 8 * slot, bytes);
            ptx::bulk_g2s(sRing + slot * p.slot_bytes, img + (size_t)(2 * pk) * p.row_bytes, bytes, full + 8 * slot);
          }
        }
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitProducer);
    }
  } else if (SW && warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (pairs) --
    // A row pair p holds filter rows (2j-1, 2j) of the four conv rows y = p+2-j, j = 0..3.  The
    // packed weights are the four [64 x 64] blocks stacked by ascending conv row, so one MMA
    // multiplies the pair's [128 x 64] tile with several of them at once: conv row y lives in
    // TMEM columns 64 * (c % 8), c counting this CTA's conv rows, and the rows of a pair are
    // consecutive slots (two pieces where they wrap).  The pair's newest row has no partial
    // sum yet, so it takes MMAs of its own with the accumulate flag off at the first K step.
    // Compared with one N = 64 MMA per (row, filter-row pair) the A tile is read from shared
    // memory twice instead of four times and the issuing thread -- a single lane, ~10 clocks
    // per instruction, ~300 per tcgen05.commit -- has 8 MMAs and ONE commit per conv row: the
    // commit frees the pair's tile for the producer and tells the epilogue that every row
    // whose last pair this was is complete.
    if (lane == 0) {
      // instruction descriptor for N = 64 * k: the N field (N >> 3 at bit 17) grows by 8 per block
      const uint32_t idesc64 = ptx::umma_idesc(128, 64, p.bf16 ? 1 : 0);
      const uint32_t ring_lo = ptx::smem_desc_k128_lo(sRing), w_lo = ptx::smem_desc_k128_lo(sW);
      bool okw = ptx::mbar_wait_abortable(w_full, 0, abort_flag);
      uint32_t seq = 0, rc_base = 0;
      for (int i = 0; okw; ++i) {
        int n, p0, p1, y0, y1, ir0, ir1;
        if (!item_of(i, n, p0, p1, y0, y1, ir0, ir1)) break;
        for (int pk = ir0; pk <= ir1 && okw; ++pk, ++seq) {
          const uint32_t slot = seq % kRingSlots;
          // the scout warp has seen the pair's tile arrive, the epilogue move past pair seq - 8 and
          // the accumulator slots of the rows this pair starts come free
          if (!ptx::mbar_wait_abortable(go + 8 * (seq & 3u), (seq >> 2) & 1u, abort_flag)) { okw = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_lo = ring_lo + slot * (uint32_t)(kSwSlot >> 4);
          if (pk > ir0 && pk < ir1 && pk - 1 >= y0 && pk + 2 <= y1) {
            // Interior pair, straight-line: rows pk-1 .. pk+1 accumulate (N = 192, or two pieces
            // where the slots wrap), row pk+2 starts (N = 64, accumulate off at the first K step).
            const uint32_t c_lo = rc_base + (uint32_t)(pk - 1 - y0);
            const uint32_t cf = c_lo + 3;
            const uint32_t s0 = c_lo % kAcc;
            if (s0 + 3 <= kAcc) {
#pragma unroll
              for (uint32_t k4 = 0; k4 < 4; ++k4)
                ptx::umma_f16(tmem_base + s0 * 64, ptx::desc_from_halves(a_lo + k4 * 2, ptx::kSmemDescK128Hi),
                              ptx::desc_from_halves(w_lo + k4 * 2, ptx::kSmemDescK128Hi), idesc64 + (2u << 20), 1u);
            } else {
              const uint32_t n1 = kAcc - s0;   // 1 or 2 rows before the wrap
#pragma unroll
              for (uint32_t k4 = 0; k4 < 4; ++k4)
                ptx::umma_f16(tmem_base + s0 * 64, ptx::desc_from_halves(a_lo + k4 * 2, ptx::kSmemDescK128Hi),
                              ptx::desc_from_halves(w_lo + k4 * 2, ptx::kSmemDescK128Hi), idesc64 + ((n1 - 1) << 20), 1u);
#pragma unroll
              for (uint32_t k4 = 0; k4 < 4; ++k4)
                ptx::umma_f16(tmem_base, ptx::desc_from_halves(a_lo + k4 * 2, ptx::kSmemDescK128Hi),
                              ptx::desc_from_halves(w_lo + n1 * 512u + k4 * 2, ptx::kSmemDescK128Hi), idesc64 + ((2 - n1) << 20), 1u);
            }
#pragma unroll
            for (uint32_t k4 = 0; k4 < 4; ++k4)
              ptx::umma_f16(tmem_base + (cf % kAcc) * 64, ptx::desc_from_halves(a_lo + k4 * 2, ptx::kSmemDescK128Hi),
                            ptx::desc_from_halves(w_lo + 3u * 512u + k4 * 2, ptx::kSmemDescK128Hi), idesc64, k4 > 0 ? 1u : 0u);
            ptx::tc_commit(empty + 8 * slot);
            continue;
          }
          const int lo = max(y0, pk - 1), hi = min(y1, pk + 2);
          // rows that get their first partial sum from this pair: all of them for the first pair
          // of the item, else only row pk + 2
          const int fresh_lo = (pk == ir0) ? lo : (pk + 2 <= y1 ? pk + 2 : hi + 1);
          // rows [a, b] -> consecutive accumulator slots, in two pieces where the slot index wraps:
          // TMEM address, weight descriptor (low word) and instruction descriptor of each piece
          auto split = [&](int a, int b, uint32_t (&d)[2], uint32_t (&bl)[2], uint32_t (&id)[2]) -> int {
            if (a > b) return 0;
            const uint32_t s_a = (rc_base + (uint32_t)(a - y0)) % kAcc;
            const int nrow = b - a + 1;
            const int n1 = min(nrow, (int)(kAcc - s_a));
            const uint32_t brow = (uint32_t)(a - pk + 1);   // weight block of row a
            d[0] = tmem_base + s_a * 64; bl[0] = w_lo + brow * 512u; id[0] = idesc64 + ((uint32_t)(n1 - 1) << 20);
            if (nrow == n1) return 1;
            d[1] = tmem_base; bl[1] = w_lo + (brow + (uint32_t)n1) * 512u; id[1] = idesc64 + ((uint32_t)(nrow - n1 - 1) << 20);
            return 2;
          };
          uint32_t dA[2], bA[2], iA[2], dF[2], bF[2], iF[2];
          const int nA = split(lo, fresh_lo - 1, dA, bA, iA);
          const int nF = split(fresh_lo, hi, dF, bF, iF);
          // MMAs of one shape back to back
#pragma unroll
          for (int pc = 0; pc < 2; ++pc) {
            if (pc < nA) {
#pragma unroll
              for (uint32_t k4 = 0; k4 < 4; ++k4)
                ptx::umma_f16(dA[pc], ptx::desc_from_halves(a_lo + k4 * 2, ptx::kSmemDescK128Hi),
                              ptx::desc_from_halves(bA[pc] + k4 * 2, ptx::kSmemDescK128Hi), iA[pc], 1u);
            }
          }
#pragma unroll
          for (int pc = 0; pc < 2; ++pc) {
            if (pc < nF) {
#pragma unroll
              for (uint32_t k4 = 0; k4 < 4; ++k4)
                ptx::umma_f16(dF[pc], ptx::desc_from_halves(a_lo + k4 * 2, ptx::kSmemDescK128Hi),
                              ptx::desc_from_halves(bF[pc] + k4 * 2, ptx::kSmemDescK128Hi), iF[pc], k4 > 0 ? 1u : 0u);
            }
          }
          ptx::tc_commit(empty + 8 * slot);
        }
        rc_base += (uint32_t)(y1 - y0 + 1);
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitMma);
    }
  } else if (SW && warp == kIssuerBWarp) {
    // ---------------------------------------------------------------- scout (pairs) -------
    // Does the issuing lane's waiting for it, up to four pairs ahead: the issuer then tests one
    // barrier per pair and spends its instructions on MMAs (a lone lane runs ~10 clocks per
    // instruction, and the tensor pipe idles while it does anything else).
    if (lane == 0) {
      uint32_t seq = 0, rc_base = 0;
      bool okw = true;
      for (int i = 0; okw; ++i) {
        int n, p0, p1, y0, y1, ir0, ir1;
        if (!item_of(i, n, p0, p1, y0, y1, ir0, ir1)) break;
        for (int pk = ir0; pk <= ir1 && okw; ++pk, ++seq) {
          // go[seq & 3] is free again once the MMAs of pair seq - 4 are done (the issuer has long passed it)
          if (seq >= 4 && !ptx::mbar_wait_abortable(empty + 8 * ((seq - 4) % kRingSlots), ((seq - 4) / kRingSlots) & 1u, abort_flag)) { okw = false; break; }
          if (!ptx::mbar_wait_abortable(full + 8 * (seq % kRingSlots), (seq / kRingSlots) & 1u, abort_flag)) { okw = false; break; }
          // The issuer's commit completes a phase of empty[slot] that the epilogue may still have to
          // test for pair seq - 8 (it tests only the pairs that finish a pooling step), so the pair
          // is held back until the epilogue has moved past that one.  It is never more than a few
          // pairs behind the pair it waits for, so this cannot block for long.
          if ((int)seq - (int)kRingSlots > *(volatile int*)&s_consumed) {
            const long long t0 = clock64();
            while ((int)seq - (int)kRingSlots > *(volatile int*)&s_consumed) {
              if (*abort_flag) { okw = false; break; }
              if (clock64() - t0 > (1LL << 31)) { *abort_flag = 1; okw = false; break; }
            }
            if (!okw) break;
          }
          // accumulator slots of the rows that get their first partial sum from this pair
          const int lo = max(y0, pk - 1), hi = min(y1, pk + 2);
          const int fresh_lo = (pk == ir0) ? lo : (pk + 2 <= y1 ? pk + 2 : hi + 1);
          for (int y = fresh_lo; y <= hi && okw; ++y) {
            const uint32_t c = rc_base + (uint32_t)(y - y0);
            if (!ptx::mbar_wait_abortable(acc_empty + 8 * (c % kAcc), ((c / kAcc) & 1u) ^ 1u, abort_flag)) okw = false;
          }
          if (!okw) break;
          ptx::mbar_arrive(go + 8 * (seq & 3u));
        }
        rc_base += (uint32_t)(y1 - y0 + 1);
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitMma);
    }
  } else if (!SW && (warp == 1 || warp == kIssuerBWarp)) {
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
            const uint32_t ab = acc_cnt % kAcc;
            if (!ptx::mbar_wait_abortable(acc_empty + 8 * ab, ((acc_cnt / kAcc) & 1u) ^ 1u, abort_flag)) { okw = false; break; }
            ptx::tc_fence_after();
            uint32_t accumulate = 0;
            {
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
            }
            ptx::tc_commit(acc_full + 8 * ab);
          }
        }
        seq_base += (uint32_t)(ir1 - ir0 + 1);
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitMma);
    }
  } else if (warp >= 2 && warp < 2 + kEpiWarps) {
    // ---------------------------------------------------------------- epilogue ---------
    // Thread (quadrant, lane) owns output column x = xt*128 + row and 32 of the 64 channels of
    // every conv row, so the VERTICAL part of the 3x3 max-pool runs in its registers: `prev`
    // holds the last odd conv row (the top row of the next pooled row).  One step handles one
    // pooled row: it drains the accumulators of conv rows 2p and 2p+1 (all x tiles) behind a
    // single vote, writes one row of vertical maxima to shared memory, and takes the
    // horizontal maximum of three pixels there.  Per-row fixed costs (barrier waits, votes,
    // index arithmetic) are what bound this role, hence two rows per step.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;          // output column within the x tile
    const int et = threadIdx.x - 64;           // 0 .. kEpiThreads-1
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
    // wait until accumulators [acc_cnt, acc_cnt + n) are complete; one vote for all of them.
    // Pair kernel: they are complete when the MMAs of pair `last_pair_seq` (the last pair the
    // newest of these rows reads; pairs finish in order) have been committed.
    auto wait_accs = [&](int n, uint32_t last_pair_seq) -> bool {
      bool got = true;
      if (SW) {
        got = ptx::mbar_wait_abortable(empty + 8 * (last_pair_seq % kRingSlots), (last_pair_seq / kRingSlots) & 1u, abort_flag);
      } else {
        for (int k = 0; k < n && got; ++k) {
          const uint32_t c = acc_cnt + (uint32_t)k;
          got = ptx::mbar_wait_abortable(acc_full + 8 * (c % kAcc), (c / kAcc) & 1u, abort_flag);
        }
      }
      const bool all = ptx::named_bar_and(3, kEpiThreads, got);
      if (SW && et == 0 && all) *(volatile int*)&s_consumed = (int)last_pair_seq;   // every thread has tested the barrier
      ptx::tc_fence_after();
      return all;
    };
    // accumulator c -> scale/shift -> 16 packed pairs; the buffer goes back to the issuers
    auto drain = [&](uint32_t c, uint32_t (&cur)[16]) {
      uint32_t acc[32];
      __syncwarp();
      ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (c % kAcc) * 64 + half * 32, acc);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(acc_empty + 8 * (c % kAcc));   // one arrival per warp
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
          cur[h] = ptx::pack_half2_sat(a, b);
        }
      }
    };
    for (int i = 0; okw; ++i) {
      int n, p0, p1, y0, y1, ir0, ir1;
      if (!item_of(i, n, p0, p1, y0, y1, ir0, ir1)) break;
      int released_upto = ir0;   // input row pairs [ir0, released_upto) were handed back to the producer
      // every MMA of rows <= y has finished (their accumulators were seen full, in order): the
      // pairs that only those rows read go back to the producer -- at once, before the
      // accumulators are drained: a pair's TMA copy takes ~2700 clocks and sits on the loop
      // release -> copy -> MMA -> release that sets the pace of the kernel
      auto release_rows = [&](int y) {
        if (SW || et != 0) return;   // the pair kernel frees a tile with the commit of its MMAs
        const int new_upto = (y == y1) ? ir1 + 1 : min(ir1 + 1, y - 1);
        for (; released_upto < new_upto; ++released_upto)
          ptx::mbar_arrive(empty + 8 * ((epi_seq_base + (uint32_t)(released_upto - ir0)) % kRingSlots));
      };
      uint32_t prev[XT][16];
      bool has_prev = false;
      if (y0 & 1) {
        // the band starts with the bottom row of the previous band: only the top of a window
        if (!wait_accs(XT, epi_seq_base + (uint32_t)(min(ir1, y0 + 1) - ir0))) { okw = false; break; }
        release_rows(y0);
#pragma unroll
        for (int xt = 0; xt < XT; ++xt)
          if (xt < p.x_tiles) drain(acc_cnt + (uint32_t)xt, prev[xt]);
        acc_cnt += (uint32_t)p.x_tiles;
        has_prev = true;
      }
      for (int pr = p0; pr < p1; ++pr) {
        const int ym = 2 * pr;                         // middle row of the window
        const bool has_bot = ym + 1 <= p.OH - 1;
        const int nrows = has_bot ? 2 : 1;
        if (!wait_accs(nrows * p.x_tiles, epi_seq_base + (uint32_t)(min(ir1, ym + nrows) - ir0))) { okw = false; break; }
        release_rows(ym + nrows - 1);
        const uint32_t vrow = sConv + (uint32_t)(pr & 1) * crow_bytes;
#pragma unroll
        for (int xt = 0; xt < XT; ++xt) {
          if (xt >= p.x_tiles) break;
          uint32_t vm[16];
          drain(acc_cnt + (uint32_t)xt, vm);
          if (has_prev) {
#pragma unroll
            for (int h = 0; h < 16; ++h) vm[h] = hmax(vm[h], prev[xt][h]);
          }
          if (has_bot) {
            drain(acc_cnt + (uint32_t)(p.x_tiles + xt), prev[xt]);
#pragma unroll
            for (int h = 0; h < 16; ++h) vm[h] = hmax(vm[h], prev[xt][h]);
          }
          const int x = xt * 128 + row;
          const uint32_t prow = vrow + (uint32_t)x * 128u;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const uint32_t chunk = (uint32_t)(half * 4 + c4);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(prow + ((chunk ^ (uint32_t)(x & 7)) << 4)),
                         "r"(vm[c4 * 4]), "r"(vm[c4 * 4 + 1]), "r"(vm[c4 * 4 + 2]), "r"(vm[c4 * 4 + 3])
                         : "memory");
          }
        }
        acc_cnt += (uint32_t)(nrows * p.x_tiles);
        has_prev = has_bot;
        ptx::named_bar_sync(1, kEpiThreads);   // the vertical maxima of pooled row pr are in shared memory
        {
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
        }
        // the row of maxima two steps ahead reuses this buffer; every thread passes the barrier
        // of the next step (after its own pooling) before anyone writes it again
      }
      epi_seq_base += (uint32_t)(ir1 - ir0 + 1);
      // the next item reuses the shared-memory rows only after everyone has finished pooling
      ptx::named_bar_sync(2, kEpiThreads);
    }
    if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitEpilogue);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, kAcc * 64);
  }
}

// NCHW (any dtype) -> fp16/bf16 rows of 4-channel pixels with 4 zero pixels in front; one thread
// per output pixel slot (8-byte store), the tail of every row is zero.
template <typename SrcT, typename DstT>
__global__ void nchw_to_stem_rows_kernel(const SrcT* __restrict__ src, DstT* __restrict__ dst, int N,
                                         int H, int W, int RW, bool paired) {
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
    // paired: rows 2k and 2k+1 interleaved in 16-byte chunks (two pixels)
    const size_t o = paired ? ((size_t)n * H + (y & ~1)) * RW * 4 + (size_t)(xs >> 1) * 16 + (y & 1) * 8 + (xs & 1) * 4
                            : (size_t)i * 4;
    *reinterpret_cast<uint2*>(dst + o) = *reinterpret_cast<const uint2*>(v);
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

// Paired variant of the fast kernel (W even, H even): one thread per 16-byte chunk (two pixels of
// one row) of the interleaved pair layout, so consecutive threads write consecutive chunks (a
// warp stores 512 contiguous bytes) and read 64-byte runs of two rows of the three channel
// planes.  Pad chunks are written as zeros.
template <typename SrcT, typename DstT>
__global__ void nchw_to_stem_pairs2_kernel(const SrcT* __restrict__ src, DstT* __restrict__ dst, int N,
                                           int H, int W, int RW) {
  const int cw = RW;                       // chunks per row pair: RW / 2 per row, two rows
  const long long total = (long long)N * (H / 2) * cw;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % cw);
    const long long t = i / cw;
    const int yp = (int)(t % (H / 2));
    const int n = (int)(t / (H / 2));
    const int r = k & 1, x = (k >> 1) * 2 - 4;   // row of the pair, first pixel of the chunk
    alignas(16) DstT o[8];
    if (x >= 0 && x < W) {
      const SrcT* s = src + ((size_t)n * 3 * H + 2 * yp + r) * W + x;
      alignas(8) SrcT c0[2], c1[2], c2[2];
      if (sizeof(SrcT) == 2) {
        *reinterpret_cast<uint32_t*>(c0) = __ldg(reinterpret_cast<const uint32_t*>(s));
        *reinterpret_cast<uint32_t*>(c1) = __ldg(reinterpret_cast<const uint32_t*>(s + (size_t)H * W));
        *reinterpret_cast<uint32_t*>(c2) = __ldg(reinterpret_cast<const uint32_t*>(s + (size_t)2 * H * W));
      } else {
        *reinterpret_cast<uint2*>(c0) = __ldg(reinterpret_cast<const uint2*>(s));
        *reinterpret_cast<uint2*>(c1) = __ldg(reinterpret_cast<const uint2*>(s + (size_t)H * W));
        *reinterpret_cast<uint2*>(c2) = __ldg(reinterpret_cast<const uint2*>(s + (size_t)2 * H * W));
      }
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        o[4 * q] = (DstT)(float)c0[q];
        o[4 * q + 1] = (DstT)(float)c1[q];
        o[4 * q + 2] = (DstT)(float)c2[q];
        o[4 * q + 3] = (DstT)0.0f;
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) o[q] = (DstT)0.0f;
    }
    *reinterpret_cast<uint4*>(dst + (size_t)i * 8) = *reinterpret_cast<const uint4*>(o);
  }
}

// The same with four pixels per thread (W and the row length multiples of 4): chunks k and k + 2 of a
// pair are neighbouring pixel pairs of one row, so a thread reads 4 pixels of each channel plane in one
// load and writes two chunks.  Twice the bytes in flight per thread: with 4-byte loads the kernel is
// bound by the number of outstanding requests, not by HBM.
template <typename SrcT, typename DstT>
__global__ void nchw_to_stem_pairs4_kernel(const SrcT* __restrict__ src, DstT* __restrict__ dst, int N,
                                           int H, int W, int RW) {
  const int gw = RW / 2;                   // threads per row pair: RW / 4 per row, two rows
  const long long total = (long long)N * (H / 2) * gw;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % gw);
    const long long t = i / gw;
    const int yp = (int)(t % (H / 2));
    const int n = (int)(t / (H / 2));
    const int r = j & 1, g = j >> 1, x = 4 * g - 4;   // row of the pair, first of this thread's four pixels
    alignas(16) DstT o[16];
    if (x >= 0 && x < W) {
      const SrcT* s = src + ((size_t)n * 3 * H + 2 * yp + r) * W + x;
      alignas(16) SrcT c0[4], c1[4], c2[4];
      if (sizeof(SrcT) == 2) {
        *reinterpret_cast<uint2*>(c0) = __ldg(reinterpret_cast<const uint2*>(s));
        *reinterpret_cast<uint2*>(c1) = __ldg(reinterpret_cast<const uint2*>(s + (size_t)H * W));
        *reinterpret_cast<uint2*>(c2) = __ldg(reinterpret_cast<const uint2*>(s + (size_t)2 * H * W));
      } else {
        *reinterpret_cast<uint4*>(c0) = __ldg(reinterpret_cast<const uint4*>(s));
        *reinterpret_cast<uint4*>(c1) = __ldg(reinterpret_cast<const uint4*>(s + (size_t)H * W));
        *reinterpret_cast<uint4*>(c2) = __ldg(reinterpret_cast<const uint4*>(s + (size_t)2 * H * W));
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        o[4 * q] = (DstT)(float)c0[q];
        o[4 * q + 1] = (DstT)(float)c1[q];
        o[4 * q + 2] = (DstT)(float)c2[q];
        o[4 * q + 3] = (DstT)0.0f;
      }
    } else {
#pragma unroll
      for (int q = 0; q < 16; ++q) o[q] = (DstT)0.0f;
    }
    // chunk index inside the pair: pixel pair (x + 4) / 2 of row r -> 2 * pair + r
    DstT* d = dst + ((size_t)t * RW + (size_t)(4 * g + r)) * 8;
    *reinterpret_cast<uint4*>(d) = reinterpret_cast<const uint4*>(o)[0];
    *reinterpret_cast<uint4*>(d + 16) = reinterpret_cast<const uint4*>(o)[1];
  }
}

// W[64][3][7][7] -> per filter row r a [64 x 32] K-major un-swizzled tile: element (n, k) at
// (k / 8) * 1024 + (n / 8) * 128 + (n % 8) * 16 + (k % 8) * 2; k = 4 * tap + channel, tap 0 is the
// zero-weight pixel in front of the window, channel 3 is the zero padding channel.
//
// Behind those 28 KB follows the packing of the swizzled variant: per filter-row pair j a
// [64 x 64] K-major tile in the 128-byte swizzle, element (n, k) at
// (3 - j) * 8192 + n * 128 + (((k / 8) ^ (n % 8)) * 16) + (k % 8) * 2 (block j serves conv row
// p + 2 - j of pair p; the blocks are stacked by ascending conv row).  K follows the interleaved row
// pairs: 16-byte chunk c = k / 8 holds taps 2 * (c / 2) and 2 * (c / 2) + 1 (4 channels each)
// of filter row 2j - 1 + c % 2 (row -1, the upper row of block 0, is all zero).
template <typename SrcT, typename DstT>
__global__ void pack_stem_weights_kernel(const SrcT* __restrict__ w, DstT* __restrict__ dst) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 7 * 64 * 32 && i < 7 * 64 * 32 + 4 * 64 * 64) {
    const int e = i - 7 * 64 * 32;
    const int k = e % 64, n = (e / 64) % 64, j = e / (64 * 64);
    const int c = k / 8, ke = k % 8;
    const int r = 2 * j - 1 + (c & 1);
    const int tap = 2 * (c >> 1) + ke / 4, ch = ke % 4;
    float v = 0.0f;
    if (r >= 0 && tap >= 1 && ch < 3) v = (float)w[((n * 3 + ch) * 7 + r) * 7 + (tap - 1)];
    const size_t off = (size_t)kWBytes + (size_t)(3 - j) * 8192 + (size_t)n * 128 + (size_t)(((k / 8) ^ (n % 8)) * 16) + (size_t)(k % 8) * 2;
    *reinterpret_cast<DstT*>(reinterpret_cast<uint8_t*>(dst) + off) = (DstT)v;
    return;
  }
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


bool g_stem_force_plain = false;     // tests: keep the un-swizzled kernel
int g_stem_last_variant = 0;         // which variant the last launch used

namespace {
PFN_cuTensorMapEncodeTiled_v12000 stem_get_encode() {
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
}  // namespace

bool stem_paired_ok(int H, int W) { return !g_stem_force_plain && H % 2 == 0 && (W - 1) / 2 + 1 <= 128; }
int stem_row_pixels(int W) { return (4 + W + 4 + 1) & ~1; }
size_t stem_rows_bytes(int N, int H, int W) { return (size_t)N * H * stem_row_pixels(W) * 8; }
size_t stem_wpack_bytes() { return kWBytes + kWBytesSw; }

cudaError_t launch_nchw_to_stem_rows(const void* src, DType src_dt, void* dst, DType dst_dt, int N, int H,
                                     int W, bool pads_are_zero, bool paired, cudaStream_t stream) {
  const int RW = stem_row_pixels(W);
  if (dst_dt == kF32 || (paired && H % 2 != 0)) return cudaErrorInvalidValue;
  // the paired fast kernel writes the pads itself and needs 2-pixel alignment only
  const bool fast = paired ? (W % 2 == 0 && (reinterpret_cast<uintptr_t>(src) & 7) == 0)
                           : (pads_are_zero && W % 8 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0);
  const long long total = fast ? (paired ? (long long)N * (H / 2) * RW : (long long)N * H * (W / 8)) : (long long)N * H * RW;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  return by_dt(src_dt, [&](auto st) {
    using S = decltype(st);
    const bool four = fast && paired && W % 4 == 0 && RW % 4 == 0 &&
                      (reinterpret_cast<uintptr_t>(src) & (sizeof(S) == 2 ? 7 : 15)) == 0;
    if (four) {
      long long b4 = ((long long)N * (H / 2) * (RW / 2) + 255) / 256;
      if (b4 > 148LL * 32) b4 = 148LL * 32;
      if (dst_dt == kBF16)
        nchw_to_stem_pairs4_kernel<S, __nv_bfloat16><<<(int)b4, 256, 0, stream>>>(
            static_cast<const S*>(src), static_cast<__nv_bfloat16*>(dst), N, H, W, RW);
      else
        nchw_to_stem_pairs4_kernel<S, __half><<<(int)b4, 256, 0, stream>>>(
            static_cast<const S*>(src), static_cast<__half*>(dst), N, H, W, RW);
    } else if (fast && paired) {
      if (dst_dt == kBF16)
        nchw_to_stem_pairs2_kernel<S, __nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
            static_cast<const S*>(src), static_cast<__nv_bfloat16*>(dst), N, H, W, RW);
      else
        nchw_to_stem_pairs2_kernel<S, __half><<<(int)blocks, 256, 0, stream>>>(
            static_cast<const S*>(src), static_cast<__half*>(dst), N, H, W, RW);
    } else if (fast) {
      if (dst_dt == kBF16)
        nchw_to_stem_rows8_kernel<S, __nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
            static_cast<const S*>(src), static_cast<__nv_bfloat16*>(dst), N, H, W, RW);
      else
        nchw_to_stem_rows8_kernel<S, __half><<<(int)blocks, 256, 0, stream>>>(
            static_cast<const S*>(src), static_cast<__half*>(dst), N, H, W, RW);
    } else if (dst_dt == kBF16) {
      nchw_to_stem_rows_kernel<S, __nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
          static_cast<const S*>(src), static_cast<__nv_bfloat16*>(dst), N, H, W, RW, paired);
    } else {
      nchw_to_stem_rows_kernel<S, __half><<<(int)blocks, 256, 0, stream>>>(
          static_cast<const S*>(src), static_cast<__half*>(dst), N, H, W, RW, paired);
    }
    return cudaGetLastError();
  });
}

cudaError_t launch_pack_stem_weights(const void* w, DType w_dt, void* dst, DType dst_dt, cudaStream_t stream) {
  if (dst_dt == kF32) return cudaErrorInvalidValue;
  return by_dt(w_dt, [&](auto st) {
    using S = decltype(st);
    if (dst_dt == kBF16)
      pack_stem_weights_kernel<S, __nv_bfloat16><<<(7 * 64 * 32 + 4 * 64 * 64 + 255) / 256, 256, 0, stream>>>(
          static_cast<const S*>(w), static_cast<__nv_bfloat16*>(dst));
    else
      pack_stem_weights_kernel<S, __half><<<(7 * 64 * 32 + 4 * 64 * 64 + 255) / 256, 256, 0, stream>>>(
          static_cast<const S*>(w), static_cast<__half*>(dst));
    return cudaGetLastError();
  });
}

cudaError_t launch_stem_pool(const StemArgs& a, cudaStream_t stream) {
  if (a.ab == kF32 || a.N <= 0 || a.H < 7 || a.W < 7) return cudaErrorInvalidValue;
  StemParams p;
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
  p.w_bytes = kWBytes;
  // Swizzled variant: one x tile, even H (a row pair never straddles two images), and a tensor
  // map whose "output pixel" dimension advances 16 bytes under a 64-byte innermost extent.
  CUtensorMap tm_in;
  memset(&tm_in, 0, sizeof(tm_in));
  const bool sw = a.paired;
  if (sw) {
    if (!stem_paired_ok(a.H, a.W)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(a.in_rows) & 15) || (reinterpret_cast<uintptr_t>(a.wpack) & 15)) return cudaErrorMisalignedAddress;
    auto enc = stem_get_encode();
    // the innermost extent (128 B) equals the swizzle span; the pixel dimension advances 32 B
    cuuint64_t gdim[3] = {64, (cuuint64_t)p.OW, (cuuint64_t)a.N * (a.H / 2)};
    cuuint64_t gstr[2] = {32, 2 * (cuuint64_t)p.row_bytes};
    cuuint32_t box[3] = {64, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (!enc || enc(&tm_in, p.bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                    const_cast<void*>(a.in_rows), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
    p.w_bytes = kWBytesSw;
    p.wpack += kWBytes;
    p.slot_bytes = kSwSlot;
  }
  g_stem_last_variant = sw ? 2 : 1;
  const int sms = a.sm_count > 0 ? a.sm_count : 148;
  // bands: enough items to fill the SMs several times over, at least 4 pooled rows each
  int band_rows = p.PH;
  while (band_rows > 4 && (long long)a.N * ((p.PH + band_rows - 1) / band_rows) < 6LL * sms) band_rows = (band_rows + 1) / 2;
  p.band_rows = band_rows;
  p.bands = (p.PH + band_rows - 1) / band_rows;
  const size_t smem = 1024 + p.w_bytes + (size_t)kRingSlots * p.slot_bytes + 256 +
                      (size_t)kConvRing * p.x_tiles * 128 * 128 + 8 + 8 * (2 * kRingSlots + 4 * kAccBufs + 1 + 4) + 16;
  if (smem > 227 * 1024) return cudaErrorInvalidConfiguration;
  if (p.x_tiles > 2) return cudaErrorInvalidConfiguration;   // wider than 512 pixels: not covered by the fused kernel
  auto kern = sw ? stem_pool_kernel<1, true> : p.x_tiles == 1 ? stem_pool_kernel<1, false> : stem_pool_kernel<2, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int items = a.N * p.bands;
  return launch_pdl(kern, dim3(items < sms ? items : sms), dim3(kThreads), smem, stream, tm_in, p);
}

}  // namespace nncv_b200
