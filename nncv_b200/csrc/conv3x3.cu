// 3x3 stride-1 pad-1 convolution for sm_100a: implicit GEMM on tcgen05 whose A operand is
// nine SHIFTED VIEWS of one shared-memory halo tile, so every input element crosses the
// L2->SM path once per tile instead of nine times.
//
// Replaces, for the thirteen 3x3 stride-1 convolutions of ResNet-18 (tests/Nets/Res18.mlir:157,
// 180, 208, 231 ... 582, each preceded by a zero tensor.pad, :152-156), what nncv lowers to
// tiled scf.for nests (src/nncv/compiler/Conversion/CodeGen/LlvmCpu/ModernTile.cpp:184-199).
//
// Activation layout ("shared-pad NHWC"): a logical [N,H,W,C] tensor is stored as
// [N, H+1, W+1, C]; row 0 of every image and column 0 of every row are zero.  With the row
// pitch P = W+1 the pad column of row y+1 doubles as the right neighbour of the last pixel of
// row y, and row 0 of image n+1 doubles as the bottom pad of image n.  Flattening
// (n, y, x) -> slot q = (n*(H+1) + y)*P + x turns the convolution into
//     out[q] = sum_{r,s in 0..2} W[r][s] * in[q + (r-1)*P + (s-1)]
// for every slot; slots that are pads are computed too (4-23 % extra MMA work, depending on W)
// and stored as zeros, which keeps the output in the same layout with its pads clean.
//
// Kernel (persistent, 10 warps):
//   warp 0  one thread: TMA loads.  Per (tile, 64-channel block) ONE tiled copy brings rows
//           [q0-P-1, q0+MT*128+P+1) x 64 channels into shared memory (128-byte swizzle; rows
//           before slot 0 / past the end are zero-filled by TMA).  Weights are pre-packed
//           [Kout tile][tap][channel block] images: either all of them stay resident in shared
//           memory for the whole kernel, or they stream through a ring, one BN x 64 tile per tap.
//   warp 1  one thread: tcgen05.mma.  For tap (r,s) the A descriptor simply starts
//           (r*P+s)*128 bytes into the halo tile: the 128-byte swizzle is a function of the
//           absolute shared-memory address, so a view shifted by whole rows reads consistently.
//           MT accumulators of 128 x BN fp32 live in TMEM, double-buffered when they fit.
//   warps 2-9  epilogue (two warps per TMEM lane quadrant, 32 columns each): tcgen05.ld, scale/shift (+ residual) (+ ReLU), zero the pad slots,
//           convert, write a swizzled 128 x 64 slab in shared memory, TMA store.  Each thread
//           fetches the residual of its own row one slab ahead, straight into registers.
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

constexpr int kEpiWarps = 8;               // two warps per TMEM lane quadrant, 32 columns each
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kThreads = 64 + kEpiThreads;  // warp 0 TMA, warp 1 MMA, warps 2.. epilogue
constexpr int kSlabBytes = 128 * 128;  // 128 rows x 64 fp16
constexpr int kResPrefetch = 5;  // slabs between the L2 prefetch of a residual row and its use
constexpr int kMaxInStages = 4;
constexpr int kMaxWStages = 8;

struct C3Params {
  const uint8_t* wpack;
  const float* scale;
  const float* shift;
  const uint16_t* residual;  // shared-pad [T, Kout] or null
  int Kout;
  int* error_flag;
  int T;          // total slots
  int P;          // row pitch in slots (W + 1)
  int Himg;       // rows per image (H + 1)
  int CB;         // channel blocks of 64
  int n_tiles;    // Kout / BN
  int m_items;    // ceil(T / (MT * 128))
  int box_rows;   // rows per TMA box of the input tile (multiple of 8)
  int in_boxes;   // boxes per input stage
  int in_stages;  // input ring depth
  int w_stages;   // weight ring depth (streamed mode)
  int relu, has_res, bf16;
};

template <int BN, int MT, bool RESIDENT>
__global__ void __launch_bounds__(kThreads, 1)
conv3x3_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_out,
               const C3Params p) {
  constexpr int AB = (2 * MT * BN <= 512) ? 2 : 1;  // accumulator buffers in TMEM
  constexpr int ACC_COLS = AB * MT * BN;
  constexpr int WTILE = BN * 128;
  constexpr int SLABS = BN / 64;       // 64-column slabs per 128-row sub-tile
  constexpr int SPI = MT * SLABS;      // slabs per work item

  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_abort;
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const int in_stage_bytes = p.in_boxes * p.box_rows * 128;  // multiple of 1024
  const int kb_total = 9 * p.CB;
  const uint32_t sIn = base;
  const uint32_t sW = sIn + (uint32_t)p.in_stages * in_stage_bytes;
  const uint32_t sStage = sW + (uint32_t)(RESIDENT ? kb_total : p.w_stages) * WTILE;
  const uint32_t bars = sStage + 2 * kSlabBytes;
  const uint32_t in_full = bars, in_empty = bars + 8 * kMaxInStages;
  const uint32_t w_full = in_empty + 8 * kMaxInStages, w_empty = w_full + 8 * kMaxWStages;
  const uint32_t acc_full = w_empty + 8 * kMaxWStages, acc_empty = acc_full + 16;
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

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kMaxInStages; ++i) {
      ptx::mbar_init(in_full + 8 * i, 1);
      ptx::mbar_init(in_empty + 8 * i, 1);
    }
    for (int i = 0; i < kMaxWStages; ++i) {
      ptx::mbar_init(w_full + 8 * i, 1);
      ptx::mbar_init(w_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(acc_full + 8 * i, 1);
      ptx::mbar_init(acc_empty + 8 * i, kEpiThreads);
    }
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&tm_in);
    ptx::prefetch_tensormap(&tm_out);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, ACC_COLS);
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

  // Work items of this CTA.  Resident weights pin the CTA to one Kout tile (blockIdx.y) and it
  // strides over the slot tiles; streamed mode strides over (slot tile, Kout tile) pairs with the
  // Kout tiles of one slot tile adjacent, so that they share the input tile in L2.
  const int total_items = RESIDENT ? p.m_items : p.m_items * p.n_tiles;
  auto item_of = [&](int i, int& m_item, int& n_tile) {
    const int w = (int)blockIdx.x + i * (int)gridDim.x;
    if (RESIDENT) {
      m_item = w;
      n_tile = (int)blockIdx.y;
    } else {
      m_item = w / p.n_tiles;
      n_tile = w - m_item * p.n_tiles;
    }
    return w < total_items;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer ----
    if (lane == 0) {
      if (RESIDENT) {
        const uint8_t* src = p.wpack + (size_t)blockIdx.y * kb_total * WTILE;
        ptx::mbar_arrive_expect_tx(w_full, (uint32_t)kb_total * WTILE);
        for (int i = 0; i < kb_total; ++i)
          ptx::bulk_g2s(sW + (uint32_t)i * WTILE, src + (size_t)i * WTILE, WTILE, w_full);
      }
      uint32_t in_cnt = 0, w_cnt = 0;
      bool okw = true;
      for (int i = 0; okw; ++i) {
        int m_item, n_tile;
        if (!item_of(i, m_item, n_tile)) break;
        const int row0 = m_item * (MT * 128) - p.P - 1;
        for (int cb = 0; cb < p.CB && okw; ++cb) {
          const uint32_t st = in_cnt % (uint32_t)p.in_stages;
          const uint32_t par = ((in_cnt / (uint32_t)p.in_stages) & 1u) ^ 1u;
          if (!ptx::mbar_wait_abortable(in_empty + 8 * st, par, abort_flag)) { okw = false; break; }
          ptx::mbar_arrive_expect_tx(in_full + 8 * st, (uint32_t)in_stage_bytes);
          for (int b = 0; b < p.in_boxes; ++b)
            ptx::tma_load_2d(sIn + st * in_stage_bytes + (uint32_t)b * p.box_rows * 128, &tm_in, cb * 64,
                             row0 + b * p.box_rows, in_full + 8 * st);
          ++in_cnt;
          if (!RESIDENT) {
            for (int tap = 0; tap < 9; ++tap) {
              const uint32_t ws = w_cnt % (uint32_t)p.w_stages;
              const uint32_t wpar = ((w_cnt / (uint32_t)p.w_stages) & 1u) ^ 1u;
              if (!ptx::mbar_wait_abortable(w_empty + 8 * ws, wpar, abort_flag)) { okw = false; break; }
              ptx::mbar_arrive_expect_tx(w_full + 8 * ws, WTILE);
              ptx::bulk_g2s(sW + ws * WTILE,
                            p.wpack + ((size_t)n_tile * kb_total + (size_t)tap * p.CB + cb) * WTILE, WTILE,
                            w_full + 8 * ws);
              ++w_cnt;
            }
          }
        }
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitProducer);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer ------
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc(128, BN, p.bf16 ? 1 : 0);
      bool okw = true;
      if (RESIDENT) okw = ptx::mbar_wait_abortable(w_full, 0, abort_flag);
      uint32_t in_cnt = 0, w_cnt = 0, acc_cnt = 0;
      for (int i = 0; okw; ++i) {
        int m_item, n_tile;
        if (!item_of(i, m_item, n_tile)) break;
        const uint32_t ab = acc_cnt % AB;
        if (!ptx::mbar_wait_abortable(acc_empty + 8 * ab, ((acc_cnt / AB) & 1u) ^ 1u, abort_flag)) { okw = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_base = tmem_base + ab * (MT * BN);
        for (int cb = 0; cb < p.CB && okw; ++cb) {
          const uint32_t st = in_cnt % (uint32_t)p.in_stages;
          if (!ptx::mbar_wait_abortable(in_full + 8 * st, (in_cnt / (uint32_t)p.in_stages) & 1u, abort_flag)) { okw = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_stage = sIn + st * in_stage_bytes;
          for (int tap = 0; tap < 9; ++tap) {
            uint32_t w_addr;
            uint32_t ws = 0;
            if (RESIDENT) {
              w_addr = sW + (uint32_t)(tap * p.CB + cb) * WTILE;
            } else {
              ws = w_cnt % (uint32_t)p.w_stages;
              if (!ptx::mbar_wait_abortable(w_full + 8 * ws, (w_cnt / (uint32_t)p.w_stages) & 1u, abort_flag)) { okw = false; break; }
              ptx::tc_fence_after();
              w_addr = sW + ws * WTILE;
            }
            const int r = tap / 3, s = tap - 3 * r;
            // descriptors differ only in the address bits of the low word: one add per MMA
            const uint32_t a_lo = ptx::smem_desc_k128_lo(a_stage + (uint32_t)(r * p.P + s) * 128u);
            const uint32_t b_lo = ptx::smem_desc_k128_lo(w_addr);
            const uint32_t first = (cb | tap) != 0 ? 1u : 0u;
#pragma unroll
            for (int t = 0; t < MT; ++t) {
#pragma unroll
              for (int k4 = 0; k4 < 4; ++k4) {
                ptx::umma_f16(d_base + t * BN,
                              ptx::desc_from_halves(a_lo + (uint32_t)(t * (128 * 128) + k4 * 32) / 16u, ptx::kSmemDescK128Hi),
                              ptx::desc_from_halves(b_lo + (uint32_t)(k4 * 32) / 16u, ptx::kSmemDescK128Hi), idesc,
                              k4 == 0 ? first : 1u);
              }
            }
            if (!RESIDENT) {
              ptx::tc_commit(w_empty + 8 * ws);
              ++w_cnt;
            }
          }
          ptx::tc_commit(in_empty + 8 * st);
          ++in_cnt;
        }
        ptx::tc_commit(acc_full + 8 * ab);
        ++acc_cnt;
      }
      if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitMma);
    }
  } else {
    // ------------------------------------------------------------------ epilogue --------
    const int quad = warp & 3;            // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;     // which 32 of the slab's 64 columns this warp handles
    const int row = quad * 32 + lane;     // row of the 128-row sub-tile
    const bool elected = threadIdx.x == 64;
    const uint32_t sw = (uint32_t)(row & 7);
    // slab j of this CTA -> (item, sub-tile, 64-column slab)
    auto slab_of = [&](int j, int& q_tile, int& ncol) {
      const int i = j / SPI, rem = j - i * SPI;
      int m_item, n_tile;
      if (!item_of(i, m_item, n_tile)) return false;
      const int t = rem / SLABS, sl = rem - t * SLABS;
      q_tile = m_item * (MT * 128) + t * 128;
      ncol = n_tile * BN + sl * 64;
      return true;
    };
    // residual of the first slab (later slabs are fetched one slab ahead inside the loop).  Two
    // register sets alternate between "in use" and "in flight": copying one into the other at the
    // end of a slab would make every slab wait for the loads it has just issued.
    uint32_t res_a[2][8], res_b[2][8];
    bool have_a = false, have_b = false;
    if (p.has_res) {
      int q_tile, ncol;
      if (slab_of(0, q_tile, ncol) && q_tile + row < p.T) {
        have_a = true;
        const uint16_t* rp = p.residual + ((size_t)(q_tile + row) * p.Kout + ncol + half * 32);
        ptx::ldg_256(rp, res_a[0]);
        ptx::ldg_256(rp + 16, res_a[1]);
      }
    }
    if (p.has_res) {
      for (int j = 1; j < kResPrefetch; ++j) {
        int qf, nf;
        if (slab_of(j, qf, nf) && qf + row < p.T)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.residual + ((size_t)(qf + row) * p.Kout + nf + half * 32)));
      }
    }
    uint32_t acc_cnt = 0;
    bool okw = true;
    // one slab; returns false when the loop is over (no more slabs, or a wait gave up: okw false)
    auto do_slab = [&](int j, uint32_t (&res_cur)[2][8], bool& have_cur, uint32_t (&res_next)[2][8], bool& have_next) -> bool {
      int q_tile, ncol;
      if (!slab_of(j, q_tile, ncol)) return false;
      const int rem = j % SPI;
      const int t = rem / SLABS, sl = rem - t * SLABS;
      const uint32_t sb = (uint32_t)j & 1u;
      const uint32_t ab = acc_cnt % AB;
      // Everything that does not depend on the accumulator is issued before the waits: pad test,
      // per-channel scale/shift, and (below) the residual of the NEXT slab.
      const int q = q_tile + row;
      bool valid = q < p.T;
      if (valid) {
        const int yrow = q / p.P;
        valid = (q - yrow * p.P != 0) && (yrow % p.Himg != 0);
      }
      const int n0 = ncol + half * 32;
      float4 sc[8], sh[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sc[i] = p.scale ? __ldg(reinterpret_cast<const float4*>(p.scale + n0) + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        sh[i] = p.shift ? __ldg(reinterpret_cast<const float4*>(p.shift + n0) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      bool got = true;
      if (rem == 0) got = ptx::mbar_wait_abortable(acc_full + 8 * ab, (acc_cnt / AB) & 1u, abort_flag);
      // all epilogue threads take the same exit: nobody is left alone at a named barrier
      if (!ptx::named_bar_and(3, kEpiThreads, got)) { okw = false; return false; }
      ptx::tc_fence_after();
      const uint32_t srow = sStage + sb * kSlabBytes + (uint32_t)row * 128u;
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + ab * (MT * BN) + t * BN + sl * 64;
      uint32_t acc[32];
      __syncwarp();
      ptx::tmem_ld_32x32(t_addr + half * 32, acc);
      // residual of the next slab: in flight while this slab is converted and stored
      have_next = false;
      if (p.has_res) {
        int qn, nn;
        if (slab_of(j + 1, qn, nn)) {
          const int qr = qn + row;
          if (qr < p.T) {
            have_next = true;
            const uint16_t* rp = p.residual + ((size_t)qr * p.Kout + nn + half * 32);
            ptx::ldg_256(rp, res_next[0]);
            ptx::ldg_256(rp + 16, res_next[1]);
          }
        }
      }
      __syncwarp();
      if (p.has_res) {  // and pull the residual rows of a later slab from HBM into L2
        int qf, nf;
        if (slab_of(j + kResPrefetch, qf, nf) && qf + row < p.T)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.residual + ((size_t)(qf + row) * p.Kout + nf + half * 32)));
      }
      ptx::tmem_ld_wait();
      if (rem == SPI - 1) {  // the accumulator is in registers: hand the TMEM buffer back
        ptx::tc_fence_before();
        ptx::mbar_arrive(acc_empty + 8 * ab);
        ++acc_cnt;
      }
      float v[32];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[4 * i] = fmaf(__uint_as_float(acc[4 * i]), sc[i].x, sh[i].x);
        v[4 * i + 1] = fmaf(__uint_as_float(acc[4 * i + 1]), sc[i].y, sh[i].y);
        v[4 * i + 2] = fmaf(__uint_as_float(acc[4 * i + 2]), sc[i].z, sh[i].z);
        v[4 * i + 3] = fmaf(__uint_as_float(acc[4 * i + 3]), sc[i].w, sh[i].w);
      }
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const uint32_t chunk = (uint32_t)(half * 4 + c4);
        const uint32_t addr = srow + ((chunk ^ sw) << 4);
        if (p.has_res && have_cur) {
          const uint32_t w4[4] = {res_cur[c4 >> 1][(c4 & 1) * 4], res_cur[c4 >> 1][(c4 & 1) * 4 + 1],
                                  res_cur[c4 >> 1][(c4 & 1) * 4 + 2], res_cur[c4 >> 1][(c4 & 1) * 4 + 3]};
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            float2 f;
            if (p.bf16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[h]));
            else f = __half22float2(*reinterpret_cast<const __half2*>(&w4[h]));
            v[c4 * 8 + h * 2] += f.x;
            v[c4 * 8 + h * 2 + 1] += f.y;
          }
        }
        uint32_t o[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float a = v[c4 * 8 + h * 2], b = v[c4 * 8 + h * 2 + 1];
          uint32_t packed;
          // conversion and ReLU in one instruction (cvt.rn.relu: negative -> +0, a NaN stays NaN, like cmpf ugt + select)
          if (p.bf16) {
            if (p.relu) {
              packed = ptx::pack_bf162_relu(a, b);
            } else {
              const __nv_bfloat162 x = __floats2bfloat162_rn(a, b);
              packed = *reinterpret_cast<const uint32_t*>(&x);
            }
          } else {
            packed = p.relu ? ptx::pack_half2_sat_relu(a, b) : ptx::pack_half2_sat(a, b);
          }
          o[h] = valid ? packed : 0u;
        }
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
      }
      ptx::fence_proxy_async_smem();
      ptx::named_bar_sync(1, kEpiThreads);
      if (elected) {
        ptx::tma_store_2d(&tm_out, ncol, q_tile, sStage + sb * kSlabBytes);
        ptx::bulk_commit();
        ptx::bulk_wait_read<1>();  // the store that last read the other buffer has finished
      }
      ptx::named_bar_sync(2, kEpiThreads);  // the other staging buffer is free for everyone
      return true;
    };
    for (int j = 0;; j += 2) {
      if (!do_slab(j, res_a, have_a, res_b, have_b)) break;
      if (!do_slab(j + 1, res_b, have_b, res_a, have_a)) break;
    }
    if (elected) ptx::bulk_wait<0>();
    if (!okw && p.error_flag) atomicCAS(p.error_flag, 0, (int)kErrWaitEpilogue);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, ACC_COLS);
  }
}

// ------------------------------------------------------------------------ host side -----
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

// 2-D map over a row-major [rows, cols] 16-bit tensor, box = 64 columns x box_rows rows,
// 128-byte swizzle, out-of-range elements read as zero.
bool make_map(CUtensorMap* m, const void* ptr, long long rows, int cols, int box_rows, bool bf16) {
  auto enc = get_encode();
  if (!enc) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstr[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
             const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr size_t kSmemLimit = 227 * 1024;

template <int BN, int MT, bool RESIDENT>
cudaError_t launch_cfg(const Conv3x3Args& a, cudaStream_t stream) {
  C3Params p;
  p.wpack = static_cast<const uint8_t*>(a.wpack);
  p.scale = a.scale; p.shift = a.shift; p.error_flag = a.error_flag;
  p.residual = static_cast<const uint16_t*>(a.residual); p.Kout = a.Kout;
  p.P = a.W + 1; p.Himg = a.H + 1;
  const long long T = (long long)a.N * p.Himg * p.P;
  if (T <= 0 || T > 0x7fffff00LL) return cudaErrorInvalidValue;
  p.T = (int)T;
  p.CB = a.C / 64;
  p.n_tiles = a.Kout / BN;
  p.m_items = (int)((T + MT * 128 - 1) / (MT * 128));
  const int rows_in = MT * 128 + 2 * p.P + 2;
  p.in_boxes = (rows_in + 255) / 256;
  p.box_rows = ((rows_in + p.in_boxes - 1) / p.in_boxes + 7) & ~7;
  if (p.box_rows > 256) return cudaErrorInvalidValue;
  const size_t in_stage = (size_t)p.in_boxes * p.box_rows * 128;
  const size_t fixed = 1024 + 2 * kSlabBytes + 512;
  const size_t wtile = (size_t)BN * 128;
  size_t wbytes;
  if (RESIDENT) {
    wbytes = (size_t)9 * p.CB * wtile;
    if (fixed + wbytes + 2 * in_stage > kSmemLimit) return cudaErrorInvalidConfiguration;
    p.w_stages = 0;
    size_t room = kSmemLimit - fixed - wbytes;
    p.in_stages = (int)(room / in_stage);
    if (p.in_stages > kMaxInStages) p.in_stages = kMaxInStages;
  } else {
    p.in_stages = 2;
    if (fixed + 2 * in_stage + 2 * wtile > kSmemLimit) return cudaErrorInvalidConfiguration;
    size_t room = kSmemLimit - fixed - 2 * in_stage;
    p.w_stages = (int)(room / wtile);
    if (p.w_stages > kMaxWStages) p.w_stages = kMaxWStages;
    // spare room beyond a deep weight ring goes to a third input stage
    if (p.w_stages >= 5 && fixed + 3 * in_stage + 4 * wtile <= kSmemLimit) {
      p.in_stages = 3;
      room = kSmemLimit - fixed - 3 * in_stage;
      p.w_stages = (int)(room / wtile);
      if (p.w_stages > kMaxWStages) p.w_stages = kMaxWStages;
    }
    wbytes = (size_t)p.w_stages * wtile;
  }
  const size_t smem = fixed + wbytes + (size_t)p.in_stages * in_stage;
  p.relu = a.relu; p.has_res = a.residual != nullptr; p.bf16 = a.ab == kBF16;

  CUtensorMap tm_in, tm_out;
  if (!make_map(&tm_in, a.in, T, a.C, p.box_rows, p.bf16) ||
      !make_map(&tm_out, a.out, T, a.Kout, 128, p.bf16))
    return cudaErrorInvalidValue;

  auto kern = conv3x3_kernel<BN, MT, RESIDENT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  int sms = a.sm_count > 0 ? a.sm_count : 148;
  dim3 grid;
  if (RESIDENT) {
    int gx = sms / p.n_tiles;
    if (gx < 1) gx = 1;
    if (gx > p.m_items) gx = p.m_items;
    grid = dim3(gx, p.n_tiles);
  } else {
    const int items = p.m_items * p.n_tiles;
    grid = dim3(items < sms ? items : sms, 1);
  }
  return launch_pdl(kern, grid, dim3(kThreads), smem, stream, tm_in, tm_out, p);
}

}  // namespace


bool conv3x3_supported(int C, int Kout, int R, int S, int stride, int pad) {
  return R == 3 && S == 3 && stride == 1 && pad == 1 && C % 64 == 0 && Kout % 64 == 0 && C >= 64;
}

// Tile configuration, from timing every variant on the four ResNet-18 layer shapes at batch 256.
// With 64 input channels all nine weight tiles of a 64-wide Kout tile stay resident in shared
// memory; wider layers stream weights and favour the widest N tile (fewer passes over the input,
// and tcgen05.mma runs closer to its peak rate as N grows).
Conv3x3Config conv3x3_pick(int N, int H, int W, int C, int Kout, int has_res) {
  Conv3x3Config c;
  (void)N; (void)H; (void)W;
  if (C <= 64) {
    c.bn = 64; c.resident = 1; c.mt = has_res ? 1 : 2;
  } else if (C <= 128 || Kout % 256 != 0) {
    c.resident = 0; c.bn = Kout % 128 == 0 ? 128 : 64; c.mt = 2;
  } else if (C <= 256) {
    c.resident = 0; c.bn = 256; c.mt = 1;
  } else {
    c.resident = 0; c.bn = 256; c.mt = 2;
  }
  // Small batches: shrink the tile until the persistent grid has an item for every SM.
  const long long T = (long long)N * (H + 1) * (W + 1);
  auto items = [&]() { return ((T + c.mt * 128 - 1) / (c.mt * 128)) * (c.resident ? 1 : Kout / c.bn); };
  while (items() < 148) {
    if (c.mt > 1) c.mt >>= 1;
    else if (!c.resident && c.bn > 64) c.bn >>= 1;
    else break;
  }
  return c;
}

cudaError_t launch_conv3x3(const Conv3x3Args& a, cudaStream_t stream) {
  if (!conv3x3_supported(a.C, a.Kout, 3, 3, 1, 1) || a.ab == kF32) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.in) & 15) || (reinterpret_cast<uintptr_t>(a.out) & 15) ||
      (reinterpret_cast<uintptr_t>(a.residual) & 15) || (reinterpret_cast<uintptr_t>(a.wpack) & 15))
    return cudaErrorMisalignedAddress;
  if (a.Kout % a.bn != 0) return cudaErrorInvalidValue;
#define NNCV_C3(BN_, MT_, RES_) \
  if (a.bn == BN_ && a.mt == MT_ && (a.resident != 0) == RES_) return launch_cfg<BN_, MT_, RES_>(a, stream);
  NNCV_C3(64, 1, true)
  NNCV_C3(64, 2, true)
  NNCV_C3(64, 1, false)
  NNCV_C3(64, 2, false)
  NNCV_C3(128, 1, false)
  NNCV_C3(128, 2, false)
  NNCV_C3(128, 4, false)
  NNCV_C3(256, 1, false)
  NNCV_C3(256, 2, false)
#undef NNCV_C3
  return cudaErrorInvalidConfiguration;
}

}  // namespace nncv_b200
