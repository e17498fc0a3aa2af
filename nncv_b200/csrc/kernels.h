// Internal launch interface between the host runtime and the CUDA kernels.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

#include <vector>

namespace nncv_b200 {

enum DType : int { kF32 = 0, kF16 = 1, kBF16 = 2 };

inline size_t dtype_size(DType t) { return t == kF32 ? 4 : 2; }

// Error words a kernel can leave in the device-side status flag.
enum KernelError : int {
  kErrNone = 0,
  kErrWaitProducer = 1,  // A-tile producer gave up waiting for a free stage
  kErrWaitLoader = 2,    // weight loader gave up waiting for a free stage
  kErrWaitMma = 3,       // MMA issuer gave up waiting for a full stage
  kErrWaitEpilogue = 4,  // epilogue gave up waiting for the accumulator
  kErrBounds = 5,        // a copy would have left its buffer and was not started
};

// Where pixel (n, y, x) of a logical [N,H,W,C] activation lives: slot
// (n*img_rows + y + off)*pitch + x + off, each slot holding C contiguous channels.
//   dense NHWC:      img_rows = H,   pitch = W,   off = 0
//   shared-pad NHWC: img_rows = H+1, pitch = W+1, off = 1 (row 0 / column 0 are zero pads)
struct Layout {
  int img_rows, pitch, off;
};
inline Layout dense_layout(int H, int W) { return Layout{H, W, 0}; }
inline Layout sp_layout(int H, int W) { return Layout{H + 1, W + 1, 1}; }
inline long long layout_slots(Layout l, int N) { return (long long)N * l.img_rows * l.pitch; }

// ---- implicit-GEMM convolution / GEMM on tcgen05 ---------------------------------------
// Activations NHWC with C a multiple of 8, weights packed by launch_pack_weights().
struct IgemmArgs {
  const void* in = nullptr;        // [N,H,W,C] fp16/bf16
  const void* wpack = nullptr;     // packed weight tiles
  const float* scale = nullptr;    // [Kout] or null (=1)
  const float* shift = nullptr;    // [Kout] or null (=0)
  const void* residual = nullptr;  // [M,ldo] same type as in, or null
  void* out = nullptr;             // [M,ldo] out_dtype
  int N = 0, H = 0, W = 0, C = 0, OH = 0, OW = 0, Kout = 0, R = 1, S = 1, stride = 1, pad = 0;
  long long ldo = 0;               // output row pitch in elements (>= Kout)
  Layout in_l{0, 0, 0};            // zero pitch = dense NHWC
  Layout out_l{0, 0, 0};           // layout of out and residual
  int bn = 64;                     // N tile the weights were packed for (64, 128 or 256)
  DType ab = kF16;                 // operand type (kF16 or kBF16)
  DType out_dtype = kF16;          // kF16/kBF16 (same as ab) or kF32
  int relu = 0;
  int* error_flag = nullptr;       // device int, receives a KernelError on a timed-out wait
};

int igemm_k_blocks(int C, int R, int S);
size_t packed_weight_bytes(int Kout, int C, int R, int S, int bn);
int igemm_pick_bn(long long M, int Kout);
cudaError_t launch_conv_igemm(const IgemmArgs& a, cudaStream_t stream);

// Packs weights W[n][c][tap] (element strides sn, sc, stap; type src_dt) into the tile image
// the kernel bulk-copies to shared memory: k index = tap * Cpad + c, zero padded.
cudaError_t launch_pack_weights(const void* src, DType src_dt, long long sn, long long sc,
                                long long stap, int Kout, int C, int Cpad, int taps, int bn,
                                DType dst_dt, void* dst, cudaStream_t stream);

// ---- 3x3 stride-1 pad-1 convolution with shared-memory halo reuse (tcgen05 + TMA) ----------
// in / out / residual are shared-pad NHWC; C and Kout multiples of 64.
struct Conv3x3Config {
  int bn = 64, mt = 1, resident = 0;
};
struct Conv3x3Args {
  const void* in = nullptr;
  const void* wpack = nullptr;     // packed by launch_pack_weights for N tile `bn`
  const float* scale = nullptr;
  const float* shift = nullptr;
  const void* residual = nullptr;
  void* out = nullptr;
  int N = 0, H = 0, W = 0, C = 0, Kout = 0;
  int bn = 64, mt = 1, resident = 0;
  int tail_split = 1;              // CTA-pair kernel: slice the items of a mostly empty last round by columns
  DType ab = kF16;
  int relu = 0;
  int sm_count = 0;
  int* error_flag = nullptr;
};
bool conv3x3_supported(int C, int Kout, int R, int S, int stride, int pad);
Conv3x3Config conv3x3_pick(int N, int H, int W, int C, int Kout, int has_res);
cudaError_t launch_conv3x3(const Conv3x3Args& a, cudaStream_t stream);
// CTA-pair variant (tcgen05.mma.cta_group::2, 256 slots x 256 channels per pair): Kout % 256 == 0,
// maps up to 62 pixels wide, weights packed for N tile 128.
cudaError_t launch_conv3x3_pair(const Conv3x3Args& a, cudaStream_t stream);

// ---- TMA-fed persistent implicit GEMM (1x1 / strided convs, GEMM): C % 64 == 0 -----------------
struct TconvArgs {
  const void* in = nullptr;        // activation in layout in_l, or A[M,K] as {1, M, 0}
  const void* wpack = nullptr;     // packed by launch_pack_weights for N tile `bn`
  const float* scale = nullptr;
  const float* shift = nullptr;
  const void* residual = nullptr;  // layout out_l, 16-bit
  void* out = nullptr;             // layout out_l, row pitch == Kout
  // fused 1x1 branch on the same input (same stride, pad 0, Kout outputs): weights packed for
  // N tile 128 as a 1-tap filter, its own scale/shift, no ReLU, written to out2 (layout out_l)
  const void* wpack2 = nullptr;
  const float* scale2 = nullptr;
  const float* shift2 = nullptr;
  void* out2 = nullptr;
  int N = 0, H = 0, W = 0, C = 0, OH = 0, OW = 0, Kout = 0, R = 1, S = 1, stride = 1, pad = 0;
  Layout in_l{0, 0, 0}, out_l{0, 0, 0};
  int bn = 64, resident = 0;
  int pair = 0;                    // CTA pairs (tcgen05.mma.cta_group::2): weights packed for N tile bn / 2
  // plain GEMM with B as it lies in memory: row-major [b_rows = C, Kout] 16-bit, read by TMA as an
  // MN-major operand; wpack is then unused.  C and Kout multiples of 8.
  const void* b_rowmajor = nullptr;
  int b_rows = 0;
  DType ab = kF16, out_dtype = kF16;
  int relu = 0;
  int act = 0;               // 0, or kActHardSwish / kActSilu fused into the epilogue (16-bit outputs only)
  int sm_count = 0;
  int* error_flag = nullptr;
};
bool tconv_supported(int C, int Kout, DType out_dt, long long ldo);
void tconv_tile(int N, int OH, int OW, int* tw, int* th, int* tn);
void tconv_pick(long long m_items, int C, int Kout, int taps, int* bn, int* resident);
cudaError_t launch_tconv(const TconvArgs& a, cudaStream_t stream);

// ---- Winograd F(2x2,3x3), three stages (filter transform once; input transform, 16 GEMMs, output
// transform per call); dense NHWC, 16-bit types ----------------------------------------------------
cudaError_t launch_wino_filter(const void* w, DType w_dt, long long sn, long long sc, long long stap, int K, int C,
                               void* U, DType dt, cudaStream_t st);
cudaError_t launch_wino_input(const void* x, void* V, DType dt, int N, int H, int W, int C, cudaStream_t st);
cudaError_t launch_wino_output(const float* M, const float* scale, const float* shift, const void* res, void* y,
                               DType dt, int N, int H, int W, int K, int relu, cudaStream_t st);

// ---- ResNet stem: 7x7 s2 p3 conv (3 -> 64) + scale/shift + ReLU + 3x3 s2 p1 max-pool, fused ---
struct StemArgs {
  const void* in_rows = nullptr;   // rows written by launch_nchw_to_stem_rows
  bool paired = false;             // in_rows holds interleaved row pairs (needs stem_paired_ok)
  const void* wpack = nullptr;     // written by launch_pack_stem_weights
  const float* scale = nullptr;
  const float* shift = nullptr;
  void* out = nullptr;             // pooled [N, PH, PW, 64]
  Layout out_l{0, 0, 0};
  int N = 0, H = 0, W = 0;
  DType ab = kF16;
  int sm_count = 0;
  int* error_flag = nullptr;
};
bool stem_paired_ok(int H, int W);   // may the rows be stored as interleaved pairs (swizzled-operand kernel)?
int stem_row_pixels(int W);
size_t stem_rows_bytes(int N, int H, int W);
size_t stem_wpack_bytes();
// pads_are_zero: the zero pixels around every row of dst are already zero (enables the wide variant);
// paired: rows 2k and 2k+1 interleaved in 16-byte chunks (H even)
cudaError_t launch_nchw_to_stem_rows(const void* src, DType src_dt, void* dst, DType dst_dt, int N, int H,
                                     int W, bool pads_are_zero, bool paired, cudaStream_t stream);
cudaError_t launch_pack_stem_weights(const void* w, DType w_dt, void* dst, DType dst_dt, cudaStream_t stream);
cudaError_t launch_stem_pool(const StemArgs& a, cudaStream_t stream);
extern bool g_stem_force_plain;   // keep the plain-row (un-swizzled operand) kernel
extern int g_stem_last_variant;   // 0 none yet, 1 plain rows, 2 swizzled operand

// ---- fp32 SIMT implicit-GEMM convolution (the fp32-accurate path) ------------------------
struct SimtConvArgs {
  const float* in = nullptr;        // [N,H,W,C] fp32, C % 4 == 0
  const float* w = nullptr;         // [Kout][R][S][C] fp32
  const float* scale = nullptr;
  const float* shift = nullptr;
  const float* residual = nullptr;  // [M,ldo]
  float* out = nullptr;             // [M,ldo]
  int N = 0, H = 0, W = 0, C = 0, OH = 0, OW = 0, Kout = 0, R = 1, S = 1, stride = 1, pad = 0;
  long long ldo = 0;
  int relu = 0;
  float* scratch = nullptr;         // optional: room for a split reduction's partial sums ([splits][M][Kout])
  size_t scratch_bytes = 0;
  int sm_count = 0;
};
cudaError_t launch_conv_simt_f32(const SimtConvArgs& a, cudaStream_t stream);
// W[n][c][tap] (strides) -> [Kout][taps][Cpad] fp32
cudaError_t launch_repack_weights_f32(const void* src, DType src_dt, long long sn, long long sc,
                                      long long stap, int Kout, int C, int Cpad, int taps,
                                      float* dst, cudaStream_t stream);

// ---- memory-bound helpers (NHWC, 128-bit accesses) ---------------------------------------
cudaError_t launch_nchw_to_nhwc(const void* src, DType src_dt, void* dst, DType dst_dt, int N,
                                int C, int H, int W, int Cpad, cudaStream_t stream);
cudaError_t launch_maxpool_nhwc(const void* src, void* dst, DType dt, int N, int H, int W, int C,
                                int k, int stride, int pad, Layout in_l, Layout out_l,
                                cudaStream_t stream);
cudaError_t launch_avgpool_nhwc(const void* src, void* dst, DType dt, int N, int H, int W, int C,
                                Layout in_l, cudaStream_t stream);
// Copies a [N,H,W,C] activation between layouts; every slot of dst that is a pad becomes zero.
cudaError_t launch_relayout(const void* src, Layout src_l, void* dst, Layout dst_l, DType dt, int N,
                            int H, int W, int C, cudaStream_t stream);
// scale = gamma * rsqrt(var + 1e-5f); shift = beta - mean * scale  (inputs of type dt)
cudaError_t launch_bn_fold(const void* gamma, const void* beta, const void* mean, const void* var, DType dt, int C, float eps,
                           float* scale, float* shift, cudaStream_t stream);
cudaError_t launch_convert(const void* src, DType src_dt, void* dst, DType dst_dt, size_t n,
                           cudaStream_t stream);

// ---- fp32 GEMM on tcgen05 with three tf32 products per k step (fp32-level accuracy) ---------------
bool gemm_tf32x3_supported(int M, int N, int K);
cudaError_t launch_gemm_tf32x3(const float* A, const float* B, float* C, int M, int N, int K, const float* bias, int relu,
                               int sm_count, int* error_flag, cudaStream_t stream);

// ---- memory-bound operators of the mobile / detection fixtures (NHWC, 16-byte accesses) --------
enum Activation : int { kActNone = 0, kActRelu = 1, kActHardSigmoid = 2, kActHardSwish = 3, kActSigmoid = 4, kActSilu = 5 };
// depthwise conv, weights [C][R*S] (fp32, or fp16 with fp16 activations), folded batch-norm, activation
// 3x3 / 5x5, stride 1 / 2 with at least two 16-byte channel vectors take the TMA-staged kernel (depthwise.cu), the rest a
// one-thread-per-output kernel; error_flag is the device status word for the staged kernel's bounded waits
// in_l / out_l: where the pixels live (pitch 0 = dense NHWC)
cudaError_t launch_depthwise(const void* x, const void* w, DType w_dt, const float* scale, const float* shift, void* y, DType dt,
                             int N, int H, int W, int C, int R, int S, int stride, int pad, int act, Layout in_l, Layout out_l,
                             int sm_count, int* error_flag, cudaStream_t st);
// 3x3 convolution on the 3-channel NCHW network input, 16 .. 64 output channels, scale / shift / activation, NHWC
// output in `out_l` (16-bit activations); w: fp32 [Cout][3][3][3]
bool stem3x3_supported(int Cin, int Cout, int R, int S, DType act_dt, int act);
cudaError_t launch_stem3x3(const void* src, DType src_dt, const float* w, const float* scale, const float* shift, void* dst, DType dt,
                           Layout out_l, int N, int H, int W, int Cout, int stride, int pad, int act, cudaStream_t st);
// 1x1 stride-1 convolution with at most 128 channels on either side, on CUDA cores (16-bit NHWC, any layout)
struct PointwiseArgs {
  const void* in = nullptr;
  const float* w = nullptr;          // [Kout][C] fp32
  const float* scale = nullptr;
  const float* shift = nullptr;
  const void* residual = nullptr;    // output layout
  void* out = nullptr;
  Layout in_l{0, 0, 0}, out_l{0, 0, 0};
  int N = 0, H = 0, W = 0, C = 0, Kout = 0;
  DType ab = kF16;
  int relu = 0, act = 0;             // act: 0, kActHardSwish or kActSilu (applied after the residual add)
  int sm_count = 0;
};
bool pointwise_supported(int C, int Kout, int R, int S, int stride, int pad, DType dt);
cudaError_t launch_pointwise(const PointwiseArgs& a, cudaStream_t st);
bool depthwise_tma_supported(DType dt, int N, int H, int W, int C, int R, int S, int stride, int pad);
cudaError_t launch_depthwise_tma(const void* x, const void* w, DType w_dt, const float* scale, const float* shift, void* y, DType dt,
                                 int N, int H, int W, int C, int R, int S, int stride, int pad, int act, Layout in_l, Layout out_l,
                                 int sm_count, int* error_flag, cudaStream_t st);
cudaError_t launch_activation(const void* x, void* y, DType dt, size_t n, int act, cudaStream_t st);
cudaError_t launch_scale_channels(const void* x, const void* gate, void* y, DType dt, int N, long long HW, int C, cudaStream_t st);
cudaError_t launch_se_gate(const void* pooled, const float* w1, const float* b1, const float* w2, const float* b2, void* gate,
                           DType dt, int N, int C, int Cr, cudaStream_t st);
cudaError_t launch_concat(const void* const* in, const int* channels, int n_in, void* out, DType dt, long long pixels, cudaStream_t st);
cudaError_t launch_upsample2x(const void* in, void* out, DType dt, int N, int H, int W, int C, cudaStream_t st);

// ---- activation arena planning (host only) ----------------------------------------------------
struct ArenaTensor {
  int first = 0, last = 0;   // ops that produce it / read it last, both included
  size_t size = 0;           // bytes
  size_t offset = 0;         // out: byte offset inside the arena
};
// Greedy by size for offset calculation; sizes are rounded up to `align`.  Returns the arena size.
size_t arena_plan(std::vector<ArenaTensor>& tensors, size_t align);

// ---- failure-path self-test: one bounded mbarrier wait that is left to run out ---------------
cudaError_t launch_wait_selftest(int* error_flag, long long limit_clocks, cudaStream_t stream);

}  // namespace nncv_b200
