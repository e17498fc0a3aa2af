// TMA-fed persistent implicit-GEMM convolution / GEMM for sm_100a (tcgen05 + TMEM).
//
// Covers the convolutions whose taps cannot share one halo tile -- 1x1 and 3x3 with stride 2
// (tests/Nets/Res18.mlir: the convs on %padded_107/111/115 and the 1x1 downsample convs on
// %cst_62/38/14), ResNet-50's 1x1 convs -- and plain linalg.matmul / the FC layer
// (Res18.mlir:617-628, tests/MatMulOptimization/MatMulNv.mlir:6-9).  nncv lowers strided convs
// with an extra {1,1} tile to near-scalar loops (ModernTile.cpp:201-209) and aims matmul at
// 16x16x16 wmma tiles (ModernTileGpu.cpp:427-525, PrepareModernVecGpu.cpp:43-48).
//
// GEMM view: D[pixels, Kout] = A[pixels, R*S*C] * W[Kout, R*S*C]^T.  The M tile is a block of
// tn images x th rows x tw columns of OUTPUT pixels (tn*th*tw = 128).  For every (tap, 64-channel
// block) ONE 4-D tiled TMA copy with element strides (1, stride, stride, 1) fetches exactly the
// input pixels that tile needs -- x = stride*ox + s - pad, y = stride*oy + r - pad -- as 128 rows
// of 128 bytes in the swizzled K-major layout tcgen05.mma reads; out-of-range pixels (padding,
// ragged tiles) arrive as zeros.  No thread touches the A operand.  A plain [M,K] matrix is the
// degenerate case tw = 128, th = tn = 1.
// Weights are the packed [Kout tile][k-block] images of launch_pack_weights(): resident in shared
// memory for the whole kernel when they fit, otherwise streamed with the A stage.
// Roles: warp 0 TMA producer, warp 1 MMA issuer (accumulator double-buffered in TMEM), warps 2-9
// epilogue (scale/shift, residual, ReLU, 128-byte-row slab in shared memory, 4-D TMA store, which
// clips ragged tiles and keeps the pads of shared-pad tensors untouched).
// Every wait is bounded and abortable; a timed-out wait sets the device status word.
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
constexpr int kABytes = 128 * 128;
constexpr int kSlabBytes = 128 * 128;
constexpr int kOutBufs = 2;     // staging buffers of the epilogue: kOutBufs - 1 stores may be reading shared memory at once
constexpr int kMaxStages = 8;

struct TcParams {
  const uint8_t* wpack;
  const float* scale;
  const float* shift;
  const uint8_t* residual;   // same layout / type as out, or null
  const uint8_t* wpack2;     // DUAL: packed 1x1 weights of the fused downsample branch
  const float* scale2;
  const float* shift2;
  int* error_flag;
  int Kout, CB, taps, S, stride, pad;
  int in_off;                // layout offset of the input (0 dense, 1 shared-pad)
  int out_off;
  int OH, OW, NB;            // logical output extent
  int out_pitch, out_rows;   // output layout: slots per row, rows per image
  int tw, th, tn;            // M tile shape
  int tiles_x, tiles_y, tiles_n, n_tiles, m_items;
  int stages;                // A (+ streamed weight) ring depth
  int relu, bf16, out_f32;
  int act;   // 0, or kActHardSwish / kActSilu applied after the residual add (16-bit outputs)
};

// DUAL: a ResNet block that changes resolution applies a 3x3 stride-2 pad-1 convolution and a 1x1
// stride-2 convolution to the SAME tensor (tests/Nets/Res18.mlir: the convs on %padded_107 and on
// %cst_62 both read the output of layer 1, and likewise for layers 3 and 4).  The 1x1 conv reads
// exactly the pixels of the 3x3 conv's centre tap, so it rides along as a tenth "tap" per channel
// block: the same A tile coordinates, its own weight tile, and a second accumulator beside the
// first.  Both results leave through the same epilogue (the second one with its own scale/shift,
// no ReLU, no residual) into a second output tensor.
// PAIR: two CTAs of a cluster work as one (tcgen05.mma.cta_group::2, M = 256): each loads the A tile
// of its own 128 output pixels and HALF of every weight tile (BN/2 rows), one lane of the leader
// issues MMAs that read both CTAs' shared memory, each CTA drains its own accumulator rows.  The
// streamed kernel is bound by the L2->SM path (one A tile and one weight tile per 128 x BN x 64
// block); halving the weight bytes per CTA is the point.  Barrier protocol as in conv3x3_pair.cu.
// BROW: the B operand is a plain row-major [K, N] matrix (linalg.matmul's right-hand side as it lies in
// memory): 64 x 64 boxes of it land by TMA as MN-major 128-byte-swizzled tiles -- k rows of 128 bytes,
// 8-row groups 1024 bytes apart, one box per 64 columns 8192 bytes apart -- and the instruction
// descriptor marks B as MN-major, so nothing is repacked; rows and columns past the matrix read as zero.
template <int BN, bool RESIDENT, bool DUAL, bool PAIR, bool BROW>
__global__ void __launch_bounds__(kThreads, 1)
tconv_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_out,
             const __grid_constant__ CUtensorMap tm_out2, const __grid_constant__ CUtensorMap tm_b, const TcParams p) {
  static_assert(!PAIR || !RESIDENT, "the pair kernel streams its weights");
  static_assert(!BROW || (!RESIDENT && !DUAL && !PAIR), "a row-major B is streamed by one CTA");
  constexpr int WTILE = (PAIR ? BN / 2 : BN) * 128;   // this CTA's part of a weight tile
  constexpr int ACC_W = DUAL ? 2 * BN : BN;   // columns of one accumulator buffer
  constexpr int ACC_COLS = 2 * ACC_W;         // two accumulator buffers
  const int taps_x = p.taps + (DUAL ? 1 : 0); // taps per channel block in the pipeline

  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_abort;
  __shared__ __align__(16) float s_scale[256], s_shift[256];   // per-channel scale / shift of the N tile in work (single-output kernels)
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const int KB = p.taps * p.CB;
  const int stage_bytes = RESIDENT ? kABytes : kABytes + WTILE;
  const uint32_t sRing = base;
  const uint32_t sW = sRing + (uint32_t)p.stages * stage_bytes;       // resident weights
  const uint32_t sStage = sW + (RESIDENT ? (uint32_t)(KB + (DUAL ? p.CB : 0)) * WTILE : 0u);   // resident: main tiles, then the branch's
  const uint32_t bars = sStage + kOutBufs * kSlabBytes;
  const uint32_t full = bars, empty = bars + 8 * kMaxStages;
  const uint32_t acc_full = empty + 8 * kMaxStages, acc_empty = acc_full + 16;
  const uint32_t w_full = acc_empty + 16;
  const uint32_t tmem_slot = w_full + 8;
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
  const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;   // 0 = leader
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kMaxStages; ++i) {
      ptx::mbar_init(full + 8 * i, (PAIR && rank == 0) ? 2 : 1);   // leader: own copies + the peer's relay
      ptx::mbar_init(empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(acc_full + 8 * i, 1);
      ptx::mbar_init(acc_empty + 8 * i, PAIR ? 2 : kEpiThreads);   // pair: one arrival per CTA
    }
    ptx::mbar_init(w_full, 1);
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&tm_in);
    ptx::prefetch_tensormap(&tm_out);
    if (DUAL) ptx::prefetch_tensormap(&tm_out2);
    if (BROW) ptx::prefetch_tensormap(&tm_b);
  }
  if (warp == 1) {
    if (PAIR) {
      ptx::tmem_alloc_pair(tmem_slot, ACC_COLS);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(tmem_slot, ACC_COLS);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (PAIR) ptx::cluster_sync_all();   // both CTAs' barriers exist before anyone arrives remotely
  ptx::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  // The prologue above touched nothing the previous kernel of the stream writes; everything
  // below may, so wait for that kernel here and let the next one start its own prologue.
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  volatile int* abort_flag = &s_abort;

  // Resident weights pin a CTA to one Kout tile (blockIdx.y); otherwise the CTA strides over
  // (pixel tile, Kout tile) pairs with the Kout tiles of a pixel tile adjacent.
  // Pair: a work item is two consecutive pixel tiles (one per CTA) times one Kout tile; a tile past
  // the end reads zeros and stores nothing.
  const int m_units = PAIR ? (p.m_items + 1) / 2 : p.m_items;
  const int total_items = RESIDENT ? m_units : m_units * p.n_tiles;
  const int worker = PAIR ? (int)blockIdx.x >> 1 : (int)blockIdx.x, workers = PAIR ? (int)gridDim.x >> 1 : (int)gridDim.x;
  auto item_of = [&](int i, int& n0, int& oy0, int& ox0, int& n_tile) {
    const int w = worker + i * workers;
    if (w >= total_items) return false;
    int m_item;
    if (RESIDENT) {
      m_item = w;
      n_tile = (int)blockIdx.y;
    } else {
      m_item = w / p.n_tiles;
      n_tile = w - m_item * p.n_tiles;
    }
    if (PAIR) m_item = 2 * m_item + (int)rank;
    const int tx = m_item % p.tiles_x;
    const int t2 = m_item / p.tiles_x;
    const int ty = t2 % p.tiles_y;
    n0 = (t2 / p.tiles_y) * p.tn;
    oy0 = ty * p.th;
    ox0 = tx * p.tw;
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer ----
    if (lane == 0) {
      if (RESIDENT) {
        const uint8_t* src = p.wpack + (size_t)blockIdx.y * KB * WTILE;
        ptx::mbar_arrive_expect_tx(w_full, (uint32_t)(KB + (DUAL ? p.CB : 0)) * WTILE);
        for (int i = 0; i < KB; ++i) ptx::bulk_g2s(sW + (uint32_t)i * WTILE, src + (size_t)i * WTILE, WTILE, w_full);
        if (DUAL) {
          const uint8_t* src2 = p.wpack2 + (size_t)blockIdx.y * p.CB * WTILE;
          for (int i = 0; i < p.CB; ++i)
            ptx::bulk_g2s(sW + (uint32_t)(KB + i) * WTILE, src2 + (size_t)i * WTILE, WTILE, w_full);
        }
      }
      uint32_t cnt = 0;
      bool okw = true;
      for (int i = 0; okw; ++i) {
        int n0, oy0, ox0, n_tile;
        if (!item_of(i, n0, oy0, ox0, n_tile)) break;
        const int xb = p.stride * ox0 - p.pad + p.in_off, yb = p.stride * oy0 - p.pad + p.in_off;
        // channel block outermost, taps innermost: the same accumulation order as the shifted-view
        // 3x3 kernel, so both kernels give bit-identical sums
        for (int cb = 0; cb < p.CB && okw; ++cb) {
          for (int tap = 0; tap < taps_x; ++tap, ++cnt) {
            const int gtap = tap < p.taps ? tap : p.taps / 2;   // the extra tap re-reads the centre tap's pixels
            const int r = gtap / p.S, s = gtap - r * p.S;
            const uint32_t st = cnt % (uint32_t)p.stages;
            const bool freed = PAIR ? ptx::mbar_wait_cluster_abortable(empty + 8 * st, ((cnt / (uint32_t)p.stages) & 1u) ^ 1u, abort_flag)
                                    : ptx::mbar_wait_abortable(empty + 8 * st, ((cnt / (uint32_t)p.stages) & 1u) ^ 1u, abort_flag);
            if (!freed) { okw = false; break; }
            ptx::mbar_arrive_expect_tx(full + 8 * st, (uint32_t)stage_bytes);
            const uint32_t dst = sRing + st * stage_bytes;
            ptx::tma_load_4d(dst, &tm_in, cb * 64, xb + s, yb + r, n0, full + 8 * st);
            if (BROW) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                ptx::tma_load_2d(dst + kABytes + (uint32_t)j * 8192u, &tm_b, n_tile * BN + j * 64, cb * 64, full + 8 * st);
            } else if (!RESIDENT) {
              // pair: the weights are packed for N tile BN/2; this CTA takes tile 2 * n_tile + rank
              const int wt = PAIR ? 2 * n_tile + (int)rank : n_tile;
              const uint8_t* wsrc = (DUAL && tap == p.taps) ? p.wpack2 + ((size_t)wt * p.CB + cb) * WTILE
                                                             : p.wpack + ((size_t)wt * KB + (size_t)tap * p.CB + cb) * WTILE;
              ptx::bulk_g2s(dst + kABytes, wsrc, WTILE, full + 8 * st);
            }
          }
        }
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitProducer);
    }
  } else if (warp == 1) {
    if (PAIR && rank != 0) {
      // ---------------------------------------------------------------- relay (peer CTA) ----
      // tells the leader when this CTA's stage is full
      if (lane == 0) {
        const uint32_t lead_full = ptx::map_to_cta(full, 0);
        uint32_t cnt = 0;
        bool okw = true;
        for (int i = 0; okw; ++i) {
          int n0, oy0, ox0, n_tile;
          if (!item_of(i, n0, oy0, ox0, n_tile)) break;
          const int KBX = taps_x * p.CB;
          for (int kb = 0; kb < KBX; ++kb, ++cnt) {
            const uint32_t st = cnt % (uint32_t)p.stages;
            if (!ptx::mbar_wait_abortable(full + 8 * st, (cnt / (uint32_t)p.stages) & 1u, abort_flag)) { okw = false; break; }
            ptx::mbar_arrive_remote(lead_full + 8 * st);
          }
        }
        if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitMma);
      }
    } else
    // ------------------------------------------------------------------ MMA issuer ------
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc(PAIR ? 256 : 128, BN, p.bf16 ? 1 : 0) | (BROW ? (1u << 16) : 0u);   // bit 16: B is MN-major
      const uint32_t peer_empty = PAIR ? ptx::map_to_cta(empty, 1) : 0u, peer_acc_full = PAIR ? ptx::map_to_cta(acc_full, 1) : 0u;
      bool okw = true;
      if (RESIDENT) okw = ptx::mbar_wait_abortable(w_full, 0, abort_flag);
      uint32_t cnt = 0, acc_cnt = 0;
      for (int i = 0; okw; ++i) {
        int n0, oy0, ox0, n_tile;
        if (!item_of(i, n0, oy0, ox0, n_tile)) break;
        const uint32_t ab = acc_cnt & 1u;
        const bool drained = PAIR ? ptx::mbar_wait_cluster_abortable(acc_empty + 8 * ab, ((acc_cnt >> 1) & 1u) ^ 1u, abort_flag)
                                  : ptx::mbar_wait_abortable(acc_empty + 8 * ab, ((acc_cnt >> 1) & 1u) ^ 1u, abort_flag);
        if (!drained) { okw = false; break; }
        ptx::tc_fence_after();
        const uint32_t d = tmem_base + ab * ACC_W;
        const int KBX = taps_x * p.CB;
        for (int kb = 0; kb < KBX; ++kb, ++cnt) {
          const int cb = kb / taps_x, tap = kb - cb * taps_x;   // producer order: cb outer, tap inner
          const bool second = DUAL && tap == p.taps;
          const uint32_t st = cnt % (uint32_t)p.stages;
          const bool landed = PAIR ? ptx::mbar_wait_cluster_abortable(full + 8 * st, (cnt / (uint32_t)p.stages) & 1u, abort_flag)
                                   : ptx::mbar_wait_abortable(full + 8 * st, (cnt / (uint32_t)p.stages) & 1u, abort_flag);
          if (!landed) { okw = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_addr = sRing + st * stage_bytes;
          const uint32_t a_lo = ptx::smem_desc_k128_lo(a_addr);
          // MN-major B: leading-dimension offset 8192 bytes (next 64 columns), one k step of 16 = two 8-row groups
          const uint32_t b_lo = BROW ? ((((a_addr + kABytes) & 0x3FFFFu) >> 4) | ((8192u >> 4) << 16))
                                     : ptx::smem_desc_k128_lo(
              RESIDENT ? sW + (uint32_t)(second ? KB + cb : tap * p.CB + cb) * WTILE : a_addr + kABytes);
          constexpr uint32_t kBStep = BROW ? (2048u >> 4) : 2u;
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            if (PAIR)
              ptx::umma_f16_pair(second ? d + BN : d, ptx::desc_from_halves(a_lo + k4 * 2, ptx::kSmemDescK128Hi),
                                 ptx::desc_from_halves(b_lo + k4 * 2, ptx::kSmemDescK128Hi), idesc,
                                 (second ? (cb | k4) : (cb | tap | k4)) != 0 ? 1u : 0u);
            else
              ptx::umma_f16(second ? d + BN : d, ptx::desc_from_halves(a_lo + k4 * 2, ptx::kSmemDescK128Hi),
                            ptx::desc_from_halves(b_lo + k4 * kBStep, ptx::kSmemDescK128Hi), idesc,
                            (second ? (cb | k4) : (cb | tap | k4)) != 0 ? 1u : 0u);
          }
          if (PAIR) {
            ptx::tc_commit_pair(empty + 8 * st);
            ptx::tc_commit_pair(peer_empty + 8 * st);
          } else {
            ptx::tc_commit(empty + 8 * st);
          }
        }
        if (!okw) break;
        if (PAIR) {
          ptx::tc_commit_pair(acc_full + 8 * ab);
          ptx::tc_commit_pair(peer_acc_full + 8 * ab);
        } else {
          ptx::tc_commit(acc_full + 8 * ab);
        }
        ++acc_cnt;
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitMma);
    }
  } else {
    // ------------------------------------------------------------------ epilogue --------
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const bool elected = threadIdx.x == 64;
    const uint32_t sw = (uint32_t)(row & 7);
    const int slab_cols = p.out_f32 ? 32 : 64;      // 128-byte rows either way
    const int slabs = BN / slab_cols;
    const int esz = p.out_f32 ? 4 : 2;
    // row of the tile -> pixel inside the tile
    const int tj = row % p.tw, ti = (row / p.tw) % p.th, tnn = row / (p.tw * p.th);
    uint32_t acc_cnt = 0;
    int jglob = 0;   // slab counter for the two staging buffers
    int cur_ntile = -1;
    bool okw = true;
    for (int i = 0; okw; ++i) {
      int n0, oy0, ox0, n_tile;
      if (!item_of(i, n0, oy0, ox0, n_tile)) break;
      const uint32_t ab = acc_cnt & 1u;
      const int nimg = n0 + tnn, oy = oy0 + ti, ox = ox0 + tj;
      const bool valid = nimg < p.NB && oy < p.OH && ox < p.OW;
      const size_t pix = ((size_t)nimg * p.out_rows + oy + p.out_off) * p.out_pitch + ox + p.out_off;
      if (p.residual != nullptr) {
        // pull the residual rows of the NEXT item from HBM into L2 while this item's accumulator is awaited
        // and drained, so that the epilogue's per-row loads of the next item do not start from DRAM
        int n0n, oy0n, ox0n, n_tile_n;
        if (item_of(i + 1, n0n, oy0n, ox0n, n_tile_n)) {
          const int nin = n0n + tnn, oyn = oy0n + ti, oxn = ox0n + tj;
          if (nin < p.NB && oyn < p.OH && oxn < p.OW) {
            const size_t pixn = ((size_t)nin * p.out_rows + oyn + p.out_off) * p.out_pitch + oxn + p.out_off;
            const int cfirst = n_tile_n * BN + (p.out_f32 ? 0 : half * 32);
            for (int sl = 0; sl < slabs; ++sl) {
              const int col = cfirst + sl * slab_cols;
              if (col < p.Kout)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(p.residual + (pixn * (size_t)p.Kout + col) * 2));
            }
          }
        }
      }
      if (!DUAL && n_tile != cur_ntile) {
        // scale / shift of this N tile into shared memory: the slabs read them as broadcast vectors instead of sixteen
        // global loads per thread and slab.  Every thread has passed the last slab's barrier of the previous item, so
        // nobody still reads the old values; the barrier below publishes the new ones.
        for (int c = (int)threadIdx.x - 64; c < BN; c += kEpiThreads) {
          const int col = n_tile * BN + c;
          s_scale[c] = (p.scale && col < p.Kout) ? __ldg(p.scale + col) : 1.0f;
          s_shift[c] = (p.shift && col < p.Kout) ? __ldg(p.shift + col) : 0.0f;
        }
        cur_ntile = n_tile;
      }
      const bool got = PAIR ? ptx::mbar_wait_cluster_abortable(acc_full + 8 * ab, (acc_cnt >> 1) & 1u, abort_flag)
                            : ptx::mbar_wait_abortable(acc_full + 8 * ab, (acc_cnt >> 1) & 1u, abort_flag);
      if (!ptx::named_bar_and(3, kEpiThreads, got)) { okw = false; break; }
      ptx::tc_fence_after();
      uint32_t res_next[2][8];   // residual of the next slab of this item, in flight one slab ahead
      bool have_next = false;
      for (int oi = 0; oi < (DUAL ? 2 : 1); ++oi)
      for (int sl = 0; sl < slabs; ++sl, ++jglob) {
        const float* scale_o = oi ? p.scale2 : p.scale;
        const float* shift_o = oi ? p.shift2 : p.shift;
        const uint8_t* residual_o = oi ? nullptr : p.residual;
        const bool relu_o = oi ? false : p.relu != 0;
        const uint32_t sb = (uint32_t)jglob % (uint32_t)kOutBufs;
        const int ncol = n_tile * BN + sl * slab_cols;     // first column of the slab
        // this warp's 32 accumulator columns inside the slab: 16-bit output -> columns
        // [half*32, +32) of a 64-column slab; fp32 output -> both halves share a 32-column
        // slab, so each warp takes 16 columns twice... keep it simple: for fp32 only half 0 works
        // on columns [0,32) and half 1 idles through the barriers.
        const bool active = p.out_f32 ? (half == 0) : true;
        const int c0 = p.out_f32 ? 0 : half * 32;
        const int n_first = ncol + c0;
        uint32_t acc[32];
        __syncwarp();
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + ab * ACC_W + (uint32_t)(oi * BN + sl * slab_cols + c0), acc);
        uint32_t res[2][8];
        // 32-byte loads need a pixel pitch that is a multiple of 32 bytes and a full group of 32 columns; other
        // widths (Kout a multiple of 8: column pairs never straddle the end) take guarded 4-byte loads
        const bool use_res = residual_o != nullptr && valid && active && n_first < p.Kout;
        if (use_res) {
          const uint8_t* rp = residual_o + (pix * (size_t)p.Kout + n_first) * 2;
          if (have_next) {   // fetched while the previous slab was converted and stored
#pragma unroll
            for (int e = 0; e < 8; ++e) { res[0][e] = res_next[0][e]; res[1][e] = res_next[1][e]; }
          } else if (n_first + 32 <= p.Kout && (p.Kout & 15) == 0) {
            ptx::ldg_256(rp, res[0]);
            ptx::ldg_256(rp + 32, res[1]);
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              res[e >> 3][e & 7] = (n_first + 2 * e < p.Kout) ? __ldg(reinterpret_cast<const uint32_t*>(rp + 4 * e)) : 0u;
          }
          // the next slab's residual of this row goes into flight now (the same item: the row stays, the columns move on)
          have_next = false;
          const int n_next = n_first + slab_cols;
          if (sl + 1 < slabs && n_next + 32 <= p.Kout && (p.Kout & 15) == 0) {
            ptx::ldg_256(rp + slab_cols * 2, res_next[0]);
            ptx::ldg_256(rp + slab_cols * 2 + 32, res_next[1]);
            have_next = true;
          }
        }
        __syncwarp();
        ptx::tmem_ld_wait();
        const bool last_slab = sl == slabs - 1 && oi == (DUAL ? 1 : 0);
        if (last_slab) {
          ptx::tc_fence_before();
          if (!PAIR) ptx::mbar_arrive(acc_empty + 8 * ab);   // pair: one arrival per CTA, after the barrier below
        }
        if (active) {
          float v[32];
          if constexpr (!DUAL) {
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              const float4 sc = *reinterpret_cast<const float4*>(&s_scale[sl * slab_cols + c0 + e]);
              const float4 sh = *reinterpret_cast<const float4*>(&s_shift[sl * slab_cols + c0 + e]);
              v[e] = fmaf(__uint_as_float(acc[e]), sc.x, sh.x);
              v[e + 1] = fmaf(__uint_as_float(acc[e + 1]), sc.y, sh.y);
              v[e + 2] = fmaf(__uint_as_float(acc[e + 2]), sc.z, sh.z);
              v[e + 3] = fmaf(__uint_as_float(acc[e + 3]), sc.w, sh.w);
            }
          } else if (n_first + 32 <= p.Kout) {
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              float4 sc = make_float4(1.f, 1.f, 1.f, 1.f), sh = make_float4(0.f, 0.f, 0.f, 0.f);
              if (scale_o) sc = __ldg(reinterpret_cast<const float4*>(scale_o + n_first + e));
              if (shift_o) sh = __ldg(reinterpret_cast<const float4*>(shift_o + n_first + e));
              v[e] = fmaf(__uint_as_float(acc[e]), sc.x, sh.x);
              v[e + 1] = fmaf(__uint_as_float(acc[e + 1]), sc.y, sh.y);
              v[e + 2] = fmaf(__uint_as_float(acc[e + 2]), sc.z, sh.z);
              v[e + 3] = fmaf(__uint_as_float(acc[e + 3]), sc.w, sh.w);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int n = n_first + e;
              float x = __uint_as_float(acc[e]);
              if (n < p.Kout) {
                if (scale_o) x *= __ldg(scale_o + n);
                if (shift_o) x += __ldg(shift_o + n);
              }
              v[e] = x;
            }
          }
          if (use_res) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const uint32_t w = res[e >> 3][e & 7];
              float2 f;
              if (p.bf16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
              else f = __half22float2(*reinterpret_cast<const __half2*>(&w));
              v[2 * e] += f.x;
              v[2 * e + 1] += f.y;
            }
          }
          if (p.act != 0 && oi == 0) {
            // hard-swish x * min(max(x + 3, 0), 6) / 6 or SiLU x / (1 + exp(-x)); a NaN stays NaN through the product with x
            if (p.act == kActHardSwish) {
#pragma unroll
              for (int e = 0; e < 32; ++e) v[e] *= fminf(fmaxf(fmaf(v[e], 0.16666667f, 0.5f), 0.0f), 1.0f);
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) v[e] *= __fdividef(1.0f, __expf(-v[e]) + 1.0f);
            }
          }
          const uint32_t srow = sStage + sb * kSlabBytes + (uint32_t)row * 128u;
          if (p.out_f32) {
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4) {
              float o[4];
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                const float a = v[c4 * 4 + h];
                o[h] = relu_o ? (!(a <= 0.0f) ? a : 0.0f) : a;
              }
              asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(srow + (((uint32_t)c4 ^ sw) << 4)), "f"(o[0]),
                           "f"(o[1]), "f"(o[2]), "f"(o[3])
                           : "memory");
            }
          } else {
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              uint32_t o[4];
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                const float a = v[c4 * 8 + h * 2], b = v[c4 * 8 + h * 2 + 1];
                // conversion and ReLU in one instruction (cvt.rn.relu: negative -> +0, NaN stays NaN)
                if (p.bf16) {
                  if (relu_o) {
                    o[h] = ptx::pack_bf162_relu(a, b);
                  } else {
                    const __nv_bfloat162 x = __floats2bfloat162_rn(a, b);
                    o[h] = *reinterpret_cast<const uint32_t*>(&x);
                  }
                } else {
                  o[h] = relu_o ? ptx::pack_half2_sat_relu(a, b) : ptx::pack_half2_sat(a, b);
                }
              }
              const uint32_t chunk = (uint32_t)(half * 4 + c4);
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(srow + ((chunk ^ sw) << 4)), "r"(o[0]), "r"(o[1]),
                           "r"(o[2]), "r"(o[3])
                           : "memory");
            }
          }
        }
        ptx::fence_proxy_async_smem();
        // One barrier per slab.  Before it the storing thread makes sure the previous slab's store has finished
        // reading its staging buffer: past the barrier every thread may fill that buffer for the next slab while
        // this slab's store (issued right after the barrier) reads the other one.  Nobody can run two slabs ahead,
        // because the next barrier needs the storing thread too.
        if (elected) ptx::bulk_wait_read<kOutBufs - 2>();
        ptx::named_bar_sync(1, kEpiThreads);
        if (elected) {
          if (PAIR && last_slab) {   // every thread of this CTA has read the accumulator: tell the leader
            if (rank == 0) ptx::mbar_arrive(acc_empty + 8 * ab);
            else ptx::mbar_arrive_remote(ptx::map_to_cta(acc_empty, 0) + 8 * ab);
          }
          if (ncol < p.Kout)
            ptx::tma_store_4d((DUAL && oi) ? &tm_out2 : &tm_out, ncol, ox0 + p.out_off, oy0 + p.out_off, n0, sStage + sb * kSlabBytes);
          ptx::bulk_commit();
        }
      }
      ++acc_cnt;
      (void)esz;
    }
    if (elected) ptx::bulk_wait<0>();
    if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitEpilogue);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (PAIR) ptx::cluster_sync_all();   // the peer's shared memory and barriers stay valid until both are done
  if (warp == 1) {
    __syncwarp();
    if (PAIR) ptx::tmem_dealloc_pair(tmem_base, ACC_COLS);
    else ptx::tmem_dealloc(tmem_base, ACC_COLS);
  }
}

PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
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

// 4-D map over an activation [NB][rows][pitch][C] (C innermost), box (box_c, bx, by, bn) with
// traversal strides (1, sx, sy, 1); 128-byte swizzle; out-of-range elements read as zero.
bool make_map4(CUtensorMap* m, const void* ptr, CUtensorMapDataType dt, int esz, int C, long long pitch,
               long long rows, long long NB, int box_c, int bx, int by, int bn, int sx, int sy) {
  auto enc = get_encode();
  if (!enc) return false;
  cuuint64_t gdim[4] = {(cuuint64_t)C, (cuuint64_t)pitch, (cuuint64_t)rows, (cuuint64_t)NB};
  cuuint64_t gstr[3] = {(cuuint64_t)C * esz, (cuuint64_t)pitch * C * esz, (cuuint64_t)rows * pitch * C * esz};
  cuuint32_t box[4] = {(cuuint32_t)box_c, (cuuint32_t)bx, (cuuint32_t)by, (cuuint32_t)bn};
  cuuint32_t estr[4] = {1, (cuuint32_t)sx, (cuuint32_t)sy, 1};
  return enc(m, dt, 4, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
         CUDA_SUCCESS;
}

constexpr size_t kSmemLimit = 225 * 1024;   // dynamic part: the kernel also holds 2 KB of static shared memory (scale / shift of an N tile)

// 2-D map over a row-major [K, N] 16-bit matrix, box 64 columns x 64 rows, 128-byte swizzle, zero fill.
bool make_map_b(CUtensorMap* m, const void* ptr, CUtensorMapDataType dt, long long K, long long N) {
  auto enc = get_encode();
  if (!enc) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)N, (cuuint64_t)K};
  cuuint64_t gstr[1] = {(cuuint64_t)N * 2};
  cuuint32_t box[2] = {64, 64};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, dt, 2, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool RESIDENT, bool DUAL = false, bool PAIR = false, bool BROW = false>
cudaError_t launch_cfg(const TconvArgs& a, TcParams p, cudaStream_t stream) {
  const size_t wtile = (size_t)(PAIR ? BN / 2 : BN) * 128;
  const int KB = p.taps * p.CB;
  const size_t fixed = 1024 + kOutBufs * kSlabBytes + 512;
  const size_t stage = RESIDENT ? kABytes : kABytes + wtile;
  const size_t wres = RESIDENT ? (size_t)(KB + (DUAL ? p.CB : 0)) * wtile : 0;
  if (fixed + wres + 2 * stage > kSmemLimit) return cudaErrorInvalidConfiguration;
  size_t st = (kSmemLimit - fixed - wres) / stage;
  if (st > kMaxStages) st = kMaxStages;
  p.stages = (int)st;
  const size_t smem = fixed + wres + st * stage;

  const Layout il = a.in_l, ol = a.out_l;
  const auto dt = p.bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tm_in, tm_out;
  if (!make_map4(&tm_in, a.in, dt, 2, a.C, il.pitch, il.img_rows, a.N, 64, p.tw * p.stride, p.th * p.stride, p.tn,
                 p.stride, p.stride))
    return cudaErrorInvalidValue;
  const bool f32 = p.out_f32 != 0;
  if (!make_map4(&tm_out, a.out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : dt, f32 ? 4 : 2, a.Kout, ol.pitch, ol.img_rows,
                 a.N, f32 ? 32 : 64, p.tw, p.th, p.tn, 1, 1))
    return cudaErrorInvalidValue;
  CUtensorMap tm_out2 = tm_out;
  if (DUAL && !make_map4(&tm_out2, a.out2, dt, 2, a.Kout, ol.pitch, ol.img_rows, a.N, 64, p.tw, p.th, p.tn, 1, 1))
    return cudaErrorInvalidValue;
  CUtensorMap tm_b = tm_out;
  if (BROW && !make_map_b(&tm_b, a.b_rowmajor, dt, a.b_rows, a.Kout)) return cudaErrorInvalidValue;
  auto kern = tconv_kernel<BN, RESIDENT, DUAL, PAIR, BROW>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int sms = a.sm_count > 0 ? a.sm_count : 148;
  dim3 grid;
  if (RESIDENT) {
    int gx = sms / p.n_tiles;
    if (gx < 1) gx = 1;
    if (gx > p.m_items) gx = p.m_items;
    grid = dim3(gx, p.n_tiles);
  } else if (PAIR) {
    const long long items = (long long)((p.m_items + 1) / 2) * p.n_tiles;
    const long long pairs = sms / 2;
    grid = dim3(2 * (unsigned)(items < pairs ? items : pairs), 1);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kern, tm_in, tm_out, tm_out2, tm_b, p);
  } else {
    const long long items = (long long)p.m_items * p.n_tiles;
    grid = dim3((unsigned)(items < sms ? items : sms), 1);
  }
  return launch_pdl(kern, grid, dim3(kThreads), smem, stream, tm_in, tm_out, tm_out2, tm_b, p);
}

}  // namespace

bool tconv_supported(int C, int Kout, DType out_dt, long long ldo) {
  // channels are read in blocks of 64 (a last block that reaches past C is zero-filled by the copy engine and
  // meets zero weights); pixel and output row pitches must be 16-byte aligned for the tensor maps
  return C % 8 == 0 && C >= 8 && ldo == Kout && (Kout * (out_dt == kF32 ? 4 : 2)) % 16 == 0;
}

// M-tile shape: tw covers the output row in as few pieces as possible.
void tconv_tile(int N, int OH, int OW, int* tw, int* th, int* tn) {
  int w = 128;
  if (OW <= 8) w = 8;
  else if (OW <= 16) w = 16;
  else if (OW <= 32) w = 32;
  else if (OW <= 64) w = 64;
  else if (OW < 112) w = 128;
  else {
    // pick the divisor-friendly width among 32/64/128 with the least ragged waste
    int best = 128, waste = (OW + 127) / 128 * 128 - OW;
    for (int c : {64, 32}) {
      const int ws = (OW + c - 1) / c * c - OW;
      if (ws < waste) { best = c; waste = ws; }
    }
    w = best;
  }
  int h = 128 / w;
  if (h > OH) {
    int hh = 1;
    while (hh * 2 <= h && hh < OH) hh *= 2;   // smallest power of two >= OH, capped at 128/w
    h = hh;
  }
  *tw = w; *th = h; *tn = 128 / (w * h);
  (void)N;
}

cudaError_t launch_tconv(const TconvArgs& a, cudaStream_t stream) {
  const bool brow = a.b_rowmajor != nullptr;
  if (brow) {   // plain GEMM with a row-major B: K and N multiples of 8 (16-byte row pitches), nothing else
    if (a.ab == kF32 || a.C % 8 != 0 || a.Kout % 8 != 0 || a.R != 1 || a.S != 1 || a.stride != 1 || a.pad != 0 || a.wpack2 ||
        a.pair || a.resident || a.b_rows != a.C || (reinterpret_cast<uintptr_t>(a.b_rowmajor) & 15))
      return cudaErrorInvalidValue;
  } else if (a.ab == kF32 || !tconv_supported(a.C, a.Kout, a.out_dtype, a.Kout)) {
    return cudaErrorInvalidValue;
  }
  if ((reinterpret_cast<uintptr_t>(a.in) & 15) || (reinterpret_cast<uintptr_t>(a.out) & 15) ||
      (reinterpret_cast<uintptr_t>(a.residual) & 31) || (!brow && (reinterpret_cast<uintptr_t>(a.wpack) & 15)))
    return cudaErrorMisalignedAddress;
  TcParams p;
  p.wpack = static_cast<const uint8_t*>(a.wpack);
  p.scale = a.scale; p.shift = a.shift; p.residual = static_cast<const uint8_t*>(a.residual);
  p.wpack2 = static_cast<const uint8_t*>(a.wpack2); p.scale2 = a.scale2; p.shift2 = a.shift2;
  p.error_flag = a.error_flag;
  p.Kout = a.Kout; p.CB = (a.C + 63) / 64; p.taps = a.R * a.S; p.S = a.S; p.stride = a.stride; p.pad = a.pad;
  p.in_off = a.in_l.off; p.out_off = a.out_l.off;
  p.OH = a.OH; p.OW = a.OW; p.NB = a.N;
  p.out_pitch = a.out_l.pitch; p.out_rows = a.out_l.img_rows;
  tconv_tile(a.N, a.OH, a.OW, &p.tw, &p.th, &p.tn);
  if (p.tw * a.stride > 256 || p.th * a.stride > 256) return cudaErrorInvalidConfiguration;
  p.tiles_x = (a.OW + p.tw - 1) / p.tw;
  p.tiles_y = (a.OH + p.th - 1) / p.th;
  p.tiles_n = (a.N + p.tn - 1) / p.tn;
  p.n_tiles = (a.Kout + a.bn - 1) / a.bn;
  const long long mi = (long long)p.tiles_x * p.tiles_y * p.tiles_n;
  if (mi <= 0 || mi * p.n_tiles > 0x7fffffffLL) return cudaErrorInvalidValue;
  p.m_items = (int)mi;
  p.relu = a.relu; p.bf16 = a.ab == kBF16; p.out_f32 = a.out_dtype == kF32;
  p.act = a.act;
  p.stages = 0;
  if (p.residual && p.out_f32) return cudaErrorInvalidValue;
  if (brow) {
    if (a.bn == 64) return launch_cfg<64, false, false, false, true>(a, p, stream);
    if (a.bn == 128) return launch_cfg<128, false, false, false, true>(a, p, stream);
    if (a.bn == 256) return launch_cfg<256, false, false, false, true>(a, p, stream);
    return cudaErrorInvalidConfiguration;
  }
  if (a.pair) {     // CTA pairs: a.wpack (and a.wpack2) packed for N tile bn / 2, streamed weights, 16-bit output
    if (a.resident || p.out_f32 || (a.bn != 128 && a.bn != 256) || a.Kout % a.bn != 0) return cudaErrorInvalidValue;
    if (a.wpack2) {
      if (!a.out2 || a.bn != 128 || a.R != a.S || a.R % 2 == 0 || a.pad != a.R / 2 ||
          (reinterpret_cast<uintptr_t>(a.wpack2) & 15) || (reinterpret_cast<uintptr_t>(a.out2) & 15))
        return cudaErrorInvalidValue;
      return launch_cfg<128, false, true, true>(a, p, stream);
    }
    return a.bn == 128 ? launch_cfg<128, false, false, true>(a, p, stream) : launch_cfg<256, false, false, true>(a, p, stream);
  }
  if (a.wpack2) {   // fused 1x1 stride-s branch on the centre tap: odd square filter, pad = R/2, N tile 128 streamed
    if (!a.out2 || a.bn != 128 || p.out_f32 || a.R != a.S || a.R % 2 == 0 || a.pad != a.R / 2 ||
        a.Kout % 128 != 0 || (reinterpret_cast<uintptr_t>(a.wpack2) & 15) || (reinterpret_cast<uintptr_t>(a.out2) & 15))
      return cudaErrorInvalidValue;
    return a.resident ? launch_cfg<128, true, true>(a, p, stream) : launch_cfg<128, false, true>(a, p, stream);
  }
#define NNCV_TC(BN_, RES_) \
  if (a.bn == BN_ && (a.resident != 0) == RES_) return launch_cfg<BN_, RES_>(a, p, stream);
  NNCV_TC(64, true)
  NNCV_TC(64, false)
  NNCV_TC(128, true)
  NNCV_TC(128, false)
  NNCV_TC(256, false)
#undef NNCV_TC
  return cudaErrorInvalidConfiguration;
}

// N tile and residency: keep all weights of one Kout tile in shared memory when they fit beside
// four A stages; otherwise stream them with the widest tile the grid can still fill.
void tconv_pick(long long m_items, int C, int Kout, int taps, int* bn, int* resident) {
  const size_t budget = kSmemLimit - (1024 + kOutBufs * kSlabBytes + 512) - 4 * (size_t)kABytes;
  const size_t kb = (size_t)taps * ((C + 63) / 64);
  for (int b : {128, 64}) {
    if (Kout >= b && kb * b * 128 <= budget) {
      *bn = b; *resident = 1;
      return;
    }
  }
  *resident = 0;
  int b = Kout >= 256 ? 256 : (Kout > 64 ? 128 : 64);
  while (b > 64 && m_items * ((Kout + b - 1) / b) < 148) b >>= 1;
  *bn = b;
}

}  // namespace nncv_b200
