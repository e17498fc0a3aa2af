// 3x3 stride-1 pad-1 convolution on CTA PAIRS: the shifted-view kernel of conv3x3.cu with
// tcgen05.mma.cta_group::2.  Two CTAs of a cluster compute one 256-slot x 256-channel tile: each
// loads its own 128-slot halo tile and HALF of every weight tile (128 of the 256 rows) into its own
// shared memory, one thread of the leader CTA issues M=256, N=256 MMAs that read both CTAs'
// operands, and each CTA keeps the accumulator rows of its 128 slots in its own TMEM.  Per SM this
// halves the weight bytes fetched from L2 and the B bytes read from shared memory per FLOP, which
// is what bounds the single-CTA kernel on the wide layers (tests/Nets/Res18.mlir: the 256- and
// 512-channel 3x3 convolutions, :442-582).
//
// Synchronisation (all barriers live at the same shared-memory offsets in both CTAs):
//   in_full / w_full    local TMA completion in each CTA; the peer CTA's idle MMA warp relays each
//                       completion to the LEADER's in_full / w_full with a remote arrive (those expect
//                       two arrivals), so the issuing lane tests one barrier per stage.
//   in_empty / w_empty  the leader commits its MMAs to the local AND (mapped address) the peer's
//                       barrier, so both producers reuse the stage.
//   acc_full            committed to both CTAs; acc_empty (leader) collects one arrive per CTA.
// No cluster-multicast copies are used anywhere.  Every wait is bounded and abortable.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace {

constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kThreads = 64 + kEpiThreads;
constexpr int kSlabBytes = 128 * 128;
constexpr int kWGroup = 3;            // taps (one filter row) per weight stage: fewer barrier round trips per MMA
constexpr int kMaxIn = 4, kMaxW = 12;

struct PairParams {
  const uint8_t* wpack;      // packed for N tile max(64, BNP / 2); each CTA of the pair takes BNP / 2 rows
  const float* scale;
  const float* shift;
  const uint16_t* residual;
  int* error_flag;
  int T, P, Himg, CB, Kout, n_tiles, m_items;   // m_items of mt * 256 slots
  int mt;                    // sub-tiles of 256 slots per item: every weight stage feeds mt times the MMAs
  int box_rows, n_boxes;     // a CTA's halo tile (mt * 128 + 2P + 2 rows) arrives as n_boxes TMA boxes
  int in_stages, w_stages;
  int w_resident;            // all 3 * CB weight stages stay in shared memory (one Kout tile only)
  unsigned long long wpack_bytes;   // size of the packed weights (copies are range-checked against it)
  // Tail of the item list: the items of the last, partly filled round are split into tail_parts
  // column slices (BNP / tail_parts columns each) that run on different pairs at the same time.
  // Items [0, tail_start) are whole; tail_start is a multiple of the number of pairs.
  int tail_start, tail_parts;
  int relu, has_res, bf16;
};

template <int BNP, int MT>   // columns of the pair's tile (64, 128 or 256), sub-tiles of 256 slots per item
__global__ void __launch_bounds__(kThreads, 1)
conv3x3_pair_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_out,
                    const PairParams p) {
  constexpr int kBNPair = BNP;
  constexpr int kMT = MT;
  constexpr int kWTile = (BNP / 2) * 128;          // this CTA's half of a weight tile
  constexpr int kWStage = kWGroup * kWTile;
  constexpr int kPackBN = BNP / 2 < 64 ? 64 : BNP / 2;   // N tile of the packed weights
  constexpr int kPackTile = kPackBN * 128;
  // accumulator buffers in TMEM: two when they fit, else one (the MMAs of the next item then wait for the epilogue)
  constexpr uint32_t kAB = (2 * BNP * MT <= 512) ? 2u : 1u;
  constexpr uint32_t kAccCols = kAB * BNP * MT;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_abort;
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const int in_stage_bytes = p.box_rows * p.n_boxes * 128;
  const int kb_total = 9 * p.CB;
  const uint32_t sIn = base;
  const uint32_t sW = sIn + (uint32_t)p.in_stages * in_stage_bytes;
  const uint32_t sStage = sW + (uint32_t)p.w_stages * kWStage;
  const uint32_t bars = sStage + 2 * kSlabBytes;
  const uint32_t in_full = bars, in_empty = in_full + 8 * kMaxIn;
  const uint32_t w_full = in_empty + 8 * kMaxIn, w_empty = w_full + 8 * kMaxW;
  const uint32_t acc_full = w_empty + 8 * kMaxW, acc_empty = acc_full + 16;
  const uint32_t tmem_slot = acc_empty + 16;
  {
    // the carve-up above must fit the dynamic shared memory of this launch: refuse to run otherwise
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (tmem_slot + 4 > raw + dyn_bytes) {
      if (threadIdx.x == 0 && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrBounds);
      return;
    }
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();   // 0 = leader
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kMaxIn; ++i) {
      ptx::mbar_init(in_full + 8 * i, rank == 0 ? 2 : 1);   // leader: own copy + the peer's relay
      ptx::mbar_init(in_empty + 8 * i, 1);
    }
    for (int i = 0; i < kMaxW; ++i) {
      ptx::mbar_init(w_full + 8 * i, rank == 0 ? 2 : 1);
      ptx::mbar_init(w_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(acc_full + 8 * i, 1);
      ptx::mbar_init(acc_empty + 8 * i, 2);   // one arrive per CTA of the pair
    }
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&tm_in);
    ptx::prefetch_tensormap(&tm_out);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, kAccCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();   // both CTAs' barriers exist before anyone arrives remotely
  ptx::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  volatile int* abort_flag = &s_abort;
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  const int pairs = (int)gridDim.x >> 1, pair = (int)blockIdx.x >> 1;
  const int total_items = p.m_items * p.n_tiles;
  const int full_rounds = p.tail_start / pairs;   // whole items every pair processes before the tail
  // item i of this pair -> pixel tile, Kout tile, column slice `sub` of `parts`
  auto item_of = [&](int i, int& m_item, int& n_tile, int& sub, int& parts) {
    int w = pair + i * pairs;
    sub = 0; parts = 1;
    if (i >= full_rounds && p.tail_parts > 1) {
      if (i > full_rounds) return false;          // at most one slice per pair
      parts = p.tail_parts;                       // 2 or 4
      const int plog = parts == 2 ? 1 : 2;
      w = p.tail_start + (pair >> plog);
      sub = pair & (parts - 1);
    }
    if (p.n_tiles == 1) { m_item = w; n_tile = 0; }
    else { m_item = w / p.n_tiles; n_tile = w - m_item * p.n_tiles; }
    return w < total_items;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer ----
    if (lane == 0) {
      uint32_t in_cnt = 0, w_cnt = 0;
      bool okw = true;
      for (int i = 0; okw; ++i) {
        int m_item, n_tile, sub, parts;
        if (!item_of(i, m_item, n_tile, sub, parts)) break;
        // the leader owns the first mt * 128 slots of the item, the peer the rest: sub-tile t is rows
        // [t * 128, +128) of both CTAs' tiles
        const int row0 = (m_item * 2 + (int)rank) * 128 * MT - p.P - 1;
        // this CTA's half of the item's columns, as rows of the packed N tiles
        const int ncols = BNP / parts;
        const int wrow = n_tile * BNP + sub * ncols + (int)rank * (ncols / 2);
        const uint32_t wbytes = (uint32_t)(ncols / 2) * 128u;   // per tap
        const uint8_t* wsrc = p.wpack + (size_t)(wrow / kPackBN) * kb_total * kPackTile + (size_t)(wrow % kPackBN) * 128;
        for (int cb = 0; cb < p.CB && okw; ++cb) {
          const uint32_t st = in_cnt % (uint32_t)p.in_stages;
          if (!ptx::mbar_wait_cluster_abortable(in_empty + 8 * st, ((in_cnt / (uint32_t)p.in_stages) & 1u) ^ 1u, abort_flag)) { okw = false; break; }
          ptx::mbar_arrive_expect_tx(in_full + 8 * st, (uint32_t)in_stage_bytes);
          for (int bx = 0; bx < p.n_boxes; ++bx)
            ptx::tma_load_2d(sIn + st * in_stage_bytes + (uint32_t)(bx * p.box_rows) * 128u, &tm_in, cb * 64,
                             row0 + bx * p.box_rows, in_full + 8 * st);
          ++in_cnt;
          if (p.w_resident && i > 0) continue;       // resident weights were loaded with the first item
          for (int fr = 0; fr < 3; ++fr, ++w_cnt) {   // one filter row (three taps) per weight stage
            const uint32_t ws = w_cnt % (uint32_t)p.w_stages;
            if (!ptx::mbar_wait_cluster_abortable(w_empty + 8 * ws, ((w_cnt / (uint32_t)p.w_stages) & 1u) ^ 1u, abort_flag)) { okw = false; break; }
            ptx::mbar_arrive_expect_tx(w_full + 8 * ws, kWGroup * wbytes);
#pragma unroll
            for (int s3 = 0; s3 < kWGroup; ++s3) {
              const uint8_t* src = wsrc + ((size_t)(fr * 3 + s3) * p.CB + cb) * kPackTile;
              // never start a copy that would leave the packed weights: report and let the waits run out
              if ((size_t)(src - p.wpack) + wbytes > p.wpack_bytes || sW + ws * kWStage + (s3 + 1) * kWTile > sStage) {
                if (p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrBounds);
                *abort_flag = 1;
                okw = false;
                break;
              }
              ptx::bulk_g2s(sW + ws * kWStage + s3 * kWTile, src, wbytes, w_full + 8 * ws);
            }
            if (!okw) break;
          }
        }
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitProducer);
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---------------------------------------------------------------- MMA issuer (leader) --
      const uint32_t idesc_full = ptx::umma_idesc(256, kBNPair, p.bf16 ? 1 : 0);
      const uint32_t peer_in_empty = ptx::map_to_cta(in_empty, 1), peer_w_empty = ptx::map_to_cta(w_empty, 1);
      const uint32_t peer_acc_full = ptx::map_to_cta(acc_full, 1);
      uint32_t in_cnt = 0, w_cnt = 0, acc_cnt = 0;
      bool okw = true;
      for (int i = 0; okw; ++i) {
        int m_item, n_tile, sub, parts;
        if (!item_of(i, m_item, n_tile, sub, parts)) break;
        const uint32_t idesc = parts == 1 ? idesc_full : ptx::umma_idesc(256, kBNPair / parts, p.bf16 ? 1 : 0);
        const uint32_t ab = acc_cnt % kAB;
        if (!ptx::mbar_wait_cluster_abortable(acc_empty + 8 * ab, ((acc_cnt / kAB) & 1u) ^ 1u, abort_flag)) { okw = false; break; }
        ptx::tc_fence_after();
        const uint32_t d = tmem_base + ab * (uint32_t)(kBNPair * MT);
        for (int cb = 0; cb < p.CB && okw; ++cb) {
          const uint32_t st = in_cnt % (uint32_t)p.in_stages;
          const uint32_t ipar = (in_cnt / (uint32_t)p.in_stages) & 1u;
          if (!ptx::mbar_wait_cluster_abortable(in_full + 8 * st, ipar, abort_flag)) { okw = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_stage = sIn + st * in_stage_bytes;
          for (int fr = 0; fr < 3; ++fr, ++w_cnt) {
            // resident: stage cb * 3 + fr, filled once (phase 0)
            const uint32_t ws = p.w_resident ? (uint32_t)(cb * 3 + fr) : w_cnt % (uint32_t)p.w_stages;
            const uint32_t wpar = p.w_resident ? 0u : (w_cnt / (uint32_t)p.w_stages) & 1u;
            if (!p.w_resident || i == 0) {
              if (!ptx::mbar_wait_cluster_abortable(w_full + 8 * ws, wpar, abort_flag)) { okw = false; break; }
              ptx::tc_fence_after();
            }
#pragma unroll
            for (int t = 0; t < MT; ++t) {   // the stage's three weight tiles serve every sub-tile
#pragma unroll
              for (int s3 = 0; s3 < kWGroup; ++s3) {
                const uint32_t a_lo = ptx::smem_desc_k128_lo(a_stage + (uint32_t)(t * 128 + fr * p.P + s3) * 128u);
                const uint32_t b_lo = ptx::smem_desc_k128_lo(sW + ws * kWStage + s3 * kWTile);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4)
                  ptx::umma_f16_pair(d + (uint32_t)(t * kBNPair), ptx::desc_from_halves(a_lo + k4 * 2, ptx::kSmemDescK128Hi),
                                     ptx::desc_from_halves(b_lo + k4 * 2, ptx::kSmemDescK128Hi), idesc,
                                     (cb | fr | s3 | k4) != 0 ? 1u : 0u);
              }
            }
            if (!p.w_resident) {
              ptx::tc_commit_pair(w_empty + 8 * ws);
              ptx::tc_commit_pair(peer_w_empty + 8 * ws);
            }
          }
          if (!okw) break;
          ptx::tc_commit_pair(in_empty + 8 * st);
          ptx::tc_commit_pair(peer_in_empty + 8 * st);
          ++in_cnt;
        }
        if (!okw) break;
        ptx::tc_commit_pair(acc_full + 8 * ab);
        ptx::tc_commit_pair(peer_acc_full + 8 * ab);
        ++acc_cnt;
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitMma);
    } else if (lane == 0) {
      // ---------------------------------------------------------------- relay (peer CTA) ----
      // Tells the leader when this CTA's stages are full.
      const uint32_t lead_in_full = ptx::map_to_cta(in_full, 0), lead_w_full = ptx::map_to_cta(w_full, 0);
      uint32_t in_cnt = 0, w_cnt = 0;
      bool okw = true;
      for (int i = 0; okw; ++i) {
        int m_item, n_tile, sub, parts;
        if (!item_of(i, m_item, n_tile, sub, parts)) break;
        for (int cb = 0; cb < p.CB && okw; ++cb) {
          const uint32_t st = in_cnt % (uint32_t)p.in_stages;
          if (!ptx::mbar_wait_abortable(in_full + 8 * st, (in_cnt / (uint32_t)p.in_stages) & 1u, abort_flag)) { okw = false; break; }
          ptx::mbar_arrive_remote(lead_in_full + 8 * st);
          ++in_cnt;
          if (p.w_resident && i > 0) continue;
          for (int fr = 0; fr < 3; ++fr, ++w_cnt) {
            const uint32_t ws = w_cnt % (uint32_t)p.w_stages;
            if (!ptx::mbar_wait_abortable(w_full + 8 * ws, (w_cnt / (uint32_t)p.w_stages) & 1u, abort_flag)) { okw = false; break; }
            ptx::mbar_arrive_remote(lead_w_full + 8 * ws);
          }
        }
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitMma);
    }
  } else {
#include "conv3x3_pair_epilogue.inc"
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();   // the peer's shared memory and barriers stay valid until both are done
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc_pair(tmem_base, kAccCols);
  }
}

}  // namespace

#include "conv3x3_pair_host.inc"

}  // namespace nncv_b200
