/* C ABI of libnncv_b200.so: the sm_100a (B200) implementation of nncv's compiled vision-model
 * forward pass behind nncv's own runtime surface.
 *
 * Every entry point takes plain pointers and sizes.  Citations name the interface of the nncv
 * source tree that each declaration replaces or mirrors.
 *
 * Threading: calls are serialised by one library-wide mutex.  One model is loaded per process
 * and lives on the CUDA device that was current when it was loaded (one process per GPU).
 * There is no CPU fallback: every compute entry point fails with NNCV_B200_ENODEVICE when no
 * sm_100 device is usable.
 */
#ifndef NNCV_B200_H_
#define NNCV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- descriptors: nncv::rt::MemRefDescriptor<T,N>, include/libnncv/DataType.hpp:129-136.
 * Strides count elements.  T is float, or uint16_t carrying fp16 bits (DataType.hpp:124-127). */
typedef struct {
  void* allocated;
  void* aligned;
  intptr_t offset;
  intptr_t sizes[1];
  intptr_t strides[1];
} nncv_memref1;
typedef struct {
  void* allocated;
  void* aligned;
  intptr_t offset;
  intptr_t sizes[2];
  intptr_t strides[2];
} nncv_memref2;
typedef struct {
  void* allocated;
  void* aligned;
  intptr_t offset;
  intptr_t sizes[4];
  intptr_t strides[4];
} nncv_memref4;

/* ---- split-params container records, include/libnncv/DataType.hpp:144-162 (224 and 24 bytes). */
typedef struct {
  char name[128];
  size_t dims;
  size_t shape[8];
  size_t eleWidth;
  size_t aligned;
  size_t dataOffset;
} nncv_memref_indexer;
typedef struct {
  int64_t magicNumber; /* 0x42 */
  size_t memRefIndexStartOffset;
  size_t numMemRefIndex;
} nncv_memref_magic_head;

/* ---- status codes (the reference returns void / bool and exits on error,
 * src/nncv/compiler/Pipeline/DnnModelLowering.cpp:222-230, src/libnncv/DataType.cpp:55-59). */
enum {
  NNCV_B200_OK = 0,
  NNCV_B200_EINVAL = 1,     /* bad argument, shape, stride or dtype */
  NNCV_B200_EIO = 2,        /* file missing, truncated, bad magic */
  NNCV_B200_ENODEVICE = 3,  /* no usable sm_100 device / CUDA error at start-up */
  NNCV_B200_ECUDA = 4,      /* CUDA runtime error during a call */
  NNCV_B200_ENOMODEL = 5,   /* forward called with no model loaded and params unusable */
  NNCV_B200_ETIMEOUT = 6,   /* a bounded device-side wait ran out (kernel reported it) */
  NNCV_B200_ENOMEM = 7
};

enum { NNCV_B200_F32 = 0, NNCV_B200_F16 = 1, NNCV_B200_BF16 = 2 };

typedef struct {
  int compute_dtype; /* NNCV_B200_F32 (CUDA-core fp32 path), _F16 or _BF16 (tcgen05 path);
                        -1 = follow the params file: eleWidth 4 -> F32, 2 -> F16 */
  unsigned device_mask; /* 0: the model lives on the current CUDA device only.  Otherwise bit d set =
                        a replica of the weights on device d (the current device must be among them):
                        _mlir_ciface_forward then cuts a batch that lies in HOST memory into
                        contiguous slices, one per device, and every device writes its logits rows
                        straight into the caller's buffer (one host thread per extra device; no
                        exchange between devices).  Device-resident tensors are processed by the
                        current device alone. */
  int reserved[6];
} nncv_b200_opts;

/* ---- the drop-in boundary --------------------------------------------------------------
 * examples/Res18/main.cpp:18-23: the C-interface wrapper MLIR emits for @forward under
 * -wrap-c-interface (DnnModelLowering.cpp:769-771) with the split-params argument inserted as
 * function argument #1 (SplitParamsFlatArray.cpp:189-192).
 *   dst    [N,1000] logits (the output width of the loaded plan), written in place at dst->aligned + dst->offset (strides honoured).
 *          If dst->aligned is NULL the buffer is malloc'ed and the descriptor filled in.
 *   src    [N,3,H,W] dense NCHW.  N is taken from the descriptor at run time.
 *   params nncv_memref1* over the whole parameter blob (what MemRefFlatArray::get() returns,
 *          DataType.hpp:179, DataType.cpp:89-119).  If no model is loaded yet, a ResNet-18 (or
 *          ResNet-50, by element count) plan is built from this blob on first use.
 * dst / src may point to host memory (as in the reference) or to device memory of the model's
 * GPU; element type is float when the params are 4 bytes wide, fp16 bits when 2 bytes wide.
 * Returns void like the reference; the outcome is in nncv_b200_last_status(). */
void _mlir_ciface_forward(nncv_memref2* dst, nncv_memref4* src, void* params);

/* Weight loading: the counterpart of `nncv-c -split-params` + MemRefFlatArray::read
 * (src/nncv/compiler/main.cpp:102-103, src/libnncv/DataType.cpp:48-87): parses the container,
 * checks it against the network's layer plan, uploads the blob once, folds batch-norm into
 * per-channel scale/shift and packs the conv/FC weights for the kernels.
 * net names the layer plan: "resnet18" / "resnet50" (built in; tensor order of
 * tests/Nets/Res18.mlir:12-109), "plan:<text>", or the path of a plan file.  A plan is what nncv's
 * lowering pipeline would have baked into the compiled object (DnnModelLowering.cpp:614-797: the op
 * sequence of @forward; SplitParamsFlatArray.cpp:48-56: the element offset of every constant in
 * the blob); `python -m nncv_b200.mlir_import model.mlir model.plan` writes one from the
 * torch-mlir linalg module nncv-c takes as input.  Plan text, one node per line:
 *   nncv_b200_plan 1
 *   params <elements in the blob> out <output features>
 *   conv id= in= res= cin= cout= k= stride= pad= relu= w= gamma= beta= mean= var=
 *   maxpool id= in= k= stride= pad=        avgpool id= in=        fc id= in= cin= cout= w= b= [act=]
 *   dwconv id= in= c= k= stride= pad= act= w= gamma= beta= mean= var=      (depthwise conv + batch-norm + activation,
 *                                                  linalg.depthwise_conv_2d_nchw_chw of tests/Nets/MobileNetV3.mlir:301)
 *   se id= in= c= cr= w1= b1= w2= b2=       (squeeze-and-excitation, MobileNetV3.mlir:319-389: scales tensor `in` in place)
 * (tensor 0 is the input; res = tensor added before the activation or -1; w, gamma, ... are element
 * offsets into the blob; a conv may carry act=<NNCV_B200_ACT_* code> instead of relu=1, b=<bias> instead of
 * the batch-norm fields, and eps_bits=<fp32 bit pattern> when its batch-norm epsilon is not 1e-5; FC nodes
 * read the global average pool or another FC node, and the last node is an FC without activation). */
int nncv_b200_load(const char* net, const char* model_bin_path, const nncv_b200_opts* opts);
/* Same, from a blob already in host memory (tensors back to back in file order). */
int nncv_b200_load_blob(const char* net, const void* blob, size_t n_elements, size_t ele_width,
                        const nncv_b200_opts* opts);
/* Parses and validates a plan (same `net` argument as nncv_b200_load) without touching a device;
 * reports the blob size it expects, its node count and output width. */
int nncv_b200_plan_check(const char* net, size_t* n_params, int* n_nodes, int* out_features);
/* The plan `net` names, as canonical plan text (the built-in networks included): copies at most
 * cap - 1 bytes plus a terminator into buf and returns the full length, or -1 on error. */
long long nncv_b200_plan_text(const char* net, char* buf, size_t cap);
int nncv_b200_unload(void);
/* Forward with an explicit CUDA stream and device-resident src/dst; does not synchronise.
 * The same computation as _mlir_ciface_forward without the host copies. */
int nncv_b200_forward_device(nncv_memref2* dst, nncv_memref4* src, void* cuda_stream);
/* Makes _mlir_ciface_forward run on the caller's CUDA stream (enable != 0) instead of the
 * library's own; the call still synchronises that stream before it returns.  No counterpart in
 * the reference (it has no device). */
int nncv_b200_set_stream(void* cuda_stream, int enable);
int nncv_b200_last_status(void);
const char* nncv_b200_last_error(void);
/* Every wait inside the kernels is bounded; a wait that runs out (or a range check that refuses a
 * copy) leaves a code in a status word on the device and the kernel returns.  _mlir_ciface_forward
 * reads that word itself; after any of the calls that do not synchronise (nncv_b200_forward_device,
 * nncv_b200_matmul, nncv_b200_matmul_noalloc, nncv_b200_conv_run, ...) synchronise the stream and
 * call this: it reads and clears the word of the current device (and the one at the head of the
 * fixed array of nncv_b200_matmul_noalloc) and returns NNCV_B200_OK, NNCV_B200_ETIMEOUT (codes 1-4:
 * which role gave up is in the message) or NNCV_B200_ECUDA (code 5: refused copy).  The reference
 * has no device and no counterpart (its errors are exit(-1), DnnModelLowering.cpp:222-230). */
int nncv_b200_device_status(void);
/* The slice [lo, hi) of a batch of n images that part `rank` of `world` processes (the first
 * n % world parts get one image more): the rule of the multi-device fan-out. */
int nncv_b200_shard_range(int n, int rank, int world, int* lo, int* hi);
/* Host-side self-test of the fan-out machinery, needs no device: runs a stand-in job for every
 * part of [0, n) on the same worker threads and with the same join and error hand-over as the
 * multi-device forward, records each part's slice in lo_out/hi_out (parts entries), counts the
 * parts that ran on another thread than the caller's, and makes part `fail_rank` (or none: -1)
 * fail: the call must then return that part's status with its message, after all parts finished. */
int nncv_b200_selftest_fanout(int n, int parts, int fail_rank, int* lo_out, int* hi_out, int* thread_differs);
/* Failure-path self-test: launches one tiny kernel that waits on an mbarrier nobody arrives on,
 * with a limit of 2^log2_clocks clocks (at most 2^24, a few milliseconds), then reports the
 * time-out into the status word and returns; nothing faults and nothing hangs.  After a
 * synchronise, nncv_b200_device_status() must answer NNCV_B200_ETIMEOUT and later calls must work. */
int nncv_b200_selftest_wait_timeout(int log2_clocks, void* stream);
/* Number of kernels of this library launched since load (for benchmark accounting). */
long long nncv_b200_launch_count(void);

/* Activation memory planning.  nncv's MemSolver (include/nncv/compiler/Optimizer/MemSolver.hpp:55-70:
 * registerTensor(first op, last op, size) / solve() / getTotalConsumption(); known answer 124 in
 * tests/MemSolver/test.cpp:17-37) assigns every tensor an offset in one block with "greedy by size
 * for offset calculation".  nncv_b200_arena_plan is that planner: tensors whose [first_op, last_op]
 * intervals (both ends included) intersect never overlap in memory; sizes are rounded up to `align`
 * bytes (0 or 1: none).  Host only, needs no device.  The executor uses it for the activation
 * tensors of a forward; nncv_b200_activation_bytes reports, after a forward, the size of the arena
 * and what one private buffer per tensor would have taken. */
int nncv_b200_arena_plan(size_t n, const int* first_op, const int* last_op, const size_t* size, size_t align,
                         size_t* offset_out, size_t* total_out);
int nncv_b200_activation_bytes(size_t* arena_bytes, size_t* unshared_bytes);

/* Per-launch timing with CUDA events on the launching stream (off by default).  The reference
 * only has wall-clock timers around the whole forward (examples/Res18/main.cpp:95-99). */
typedef struct {
  int kind;      /* 0 tcgen05 implicit GEMM (gathered A), 1 fp32 CUDA-core conv, 2 tcgen05 3x3 shifted-view
                    conv, 3 memory-bound helper, 4 fused stem conv + max-pool, 5 tcgen05 implicit GEMM
                    (TMA-fed A), 6 Winograd F(2x2,3x3) (all three stages), 7 shifted-view conv on CTA pairs */
  int M, N, K;   /* GEMM view of the launch (helpers: elements, channels, 0) */
  int bn;        /* N tile (kind 0); helper id (kind 3) */
  double flops;  /* algorithmic: 2*M*N*K with K = C*R*S (direct-convolution count) */
  double bytes;  /* algorithmic: each operand and result once */
  float ms;      /* device time of the launch */
} nncv_b200_prof_rec;
int nncv_b200_profile(int enable); /* clears the records; enable != 0 starts recording */
long long nncv_b200_profile_count(void);
int nncv_b200_profile_get(long long i, nncv_b200_prof_rec* out);

/* ---- container reader / writer: MemRefFlatArray::read/write, DataType.cpp:9-87 ----------
 * read: returns a handle (NULL on error); tensors are addressed by index in file order. */
typedef struct nncv_flat_array nncv_flat_array;
nncv_flat_array* nncv_flat_array_read(const char* path);
void nncv_flat_array_free(nncv_flat_array* a);
size_t nncv_flat_array_count(const nncv_flat_array* a);
const nncv_memref_indexer* nncv_flat_array_indexer(const nncv_flat_array* a, size_t i);
const void* nncv_flat_array_data(const nncv_flat_array* a, size_t i);
/* The rank-1 descriptor over the whole blob (MemRefFlatArray::wrap, DataType.cpp:89-119). */
nncv_memref1* nncv_flat_array_wrapped(nncv_flat_array* a);
int nncv_flat_array_write(const char* path, size_t n, const nncv_memref_indexer* indexers,
                          const void* const* data);

/* ---- single kernels (device pointers; `stream` is a cudaStream_t; no synchronisation) ----
 * linalg.matmul C[M,N] = A[M,K] * B[K,N], row-major (tests/MatMulOptimization/MatMulNv.mlir:6-9),
 * optional bias[N] (fp32) and ReLU.  ab_dtype F16/BF16: tcgen05 with fp32 accumulate, K % 8 == 0;
 * ab_dtype F32: CUDA-core fp32.  c_dtype is F32 or ab_dtype.  B is repacked into a scratch
 * buffer owned by the library (grown with cudaMalloc on demand). */
int nncv_b200_matmul(const void* A, const void* B, void* C, int M, int N, int K, int ab_dtype,
                     int c_dtype, const float* bias, int relu, void* stream);

/* The same matmul for callers that must never allocate device memory: a server that gave all
 * device memory to its own pool, or a latency-bound loop that cannot take the device-wide
 * synchronisation a cudaMalloc implies.  The repacked B lives in a fixed array inside the library
 * image (NNCV_B200_NOALLOC_MAX_PACKED_BYTES plus a 256-byte header; every GPU that loads the
 * library holds it until the process exits), so this call makes no cudaMalloc, cudaFree or other
 * allocating call.  16-bit operands only (F16/BF16), K % 8 == 0.  Problems whose packed B
 * (about N*K*2 bytes, N and K rounded up to the tile) exceeds the array are rejected with
 * NNCV_B200_EINVAL and a message; use nncv_b200_matmul for those.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current) and loads the kernels; make that first call outside any stream capture.
 * All calls share the one array, which keeps the previous call's contents: the status word in it
 * is cleared and the packed image rewritten in full at the start of every call, and two calls
 * that overlap on the GPU (different streams, no dependency) race on it -- order them.
 * A bounded wait that runs out in this path is reported in the word at the head of the array:
 * synchronise and ask nncv_b200_device_status().
 * No counterpart in the reference, which never uses a device. */
#define NNCV_B200_NOALLOC_MAX_PACKED_BYTES (8u << 20)
int nncv_b200_matmul_noalloc(const void* A, const void* B, void* C, int M, int N, int K, int ab_dtype,
                             int c_dtype, const float* bias, int relu, void* stream);

/* linalg.conv_2d_nchw_fchw (tests/Nets/Res18.mlir:125) + folded batch-norm / residual / ReLU
 * epilogue, on NHWC activations.  Weights are prepared once into a plan. */
typedef struct nncv_b200_conv nncv_b200_conv;
/* weights: host or device [Kout,C,R,S] of w_dtype.  dtype: activation type (F16/BF16 -> tcgen05
 * implicit GEMM, F32 -> CUDA-core).  algo: 0 = implicit GEMM, A operand fetched by strided TMA
 * copies when C % 64 == 0 and by a cp.async gather otherwise (any shape), 3 = always the gather
 * kernel, 1 = Winograd F(2x2,3x3) in three stages (input transform, 16 tcgen05 GEMMs, output
 * transform; same shape limits as algo 2; the counterpart of nncv's disabled F(6x6,3x3) rewrite,
 * OptimizeConv2dUsingWinograd.cpp:173-284), 2 = 3x3 stride-1 pad-1 implicit GEMM whose nine taps are shifted views of one
 * shared-memory halo tile (16-bit types, C and Kout multiples of 64).  Activation channel count is C rounded up to 8 (F16/BF16) or 4 (F32). */
nncv_b200_conv* nncv_b200_conv_create(const void* weights, int w_dtype, int Kout, int C, int R,
                                      int S, int stride, int pad, int dtype, int algo);
void nncv_b200_conv_destroy(nncv_b200_conv* c);
/* in [N,H,W,Cpad], out/residual [N,OH,OW,Kout]; scale/shift fp32 [Kout] or NULL. */
int nncv_b200_conv_run(nncv_b200_conv* c, const void* in, void* out, int N, int H, int W,
                       const float* scale, const float* shift, const void* residual, int relu,
                       void* stream);

/* One launch for the two convolutions that open a ResNet BasicBlock which changes resolution
 * (tests/Nets/Res18.mlir: the 3x3 stride-2 conv on %padded_107 and the 1x1 stride-2 downsample
 * conv on %cst_62 read the same tensor; likewise in layers 3 and 4): `c` is an odd square filter
 * with pad = R/2, `branch` a 1x1 pad-0 filter of the same stride, input and output channels
 * (Kout a multiple of 128), both 16-bit plans made with algo 0.  The branch rides along as an
 * extra tap on the centre pixel; it gets its own scale/shift, no ReLU, and its own dense NHWC
 * output.  Results equal two separate nncv_b200_conv_run calls bit for bit. */
int nncv_b200_conv_run_fused(nncv_b200_conv* c, nncv_b200_conv* branch, const void* in, void* out,
                             void* out_branch, int N, int H, int W, const float* scale,
                             const float* shift, const float* scale_branch,
                             const float* shift_branch, int relu, void* stream);

/* Force the tile configuration (N tile 64/128/256; algo 2: sub-tiles per CTA 1/2/4; resident: 1 =
 * weights resident in shared memory, 0 = streamed; algo 2 with Kout a multiple of bn: 2 = the
 * CTA-pair kernel on tcgen05.mma.cta_group::2 (bn columns per pair), 3 = the same with the items of
 * a mostly empty last round sliced by columns; algo 0 with Kout a multiple of bn = 128 or 256:
 * 2 = the per-tap kernel on CTA pairs); bn = 0 restores the built-in choice.  A tuning
 * and test hook with no counterpart in the reference. */
int nncv_b200_conv_set_tile(nncv_b200_conv* c, int bn, int mt, int resident);

/* The ResNet stem in one kernel (tests/Nets/Res18.mlir:118-151): tensor.pad 3 + 7x7 stride-2
 * conv 3 -> 64 + per-channel scale/shift (folded batch-norm) + ReLU + tensor.pad(-inf) 1 +
 * 3x3 stride-2 max-pool.  in: NCHW [N,3,H,W] of in_dtype; weights: device [64,3,7,7] of w_dtype;
 * out: dense NHWC [N,PH,PW,64] of dtype (F16/BF16).  Uses the library's scratch buffer. */
int nncv_b200_stem_pool(const void* in_nchw, int in_dtype, const void* weights, int w_dtype,
                        const float* scale, const float* shift, void* out_nhwc, int dtype, int N, int H,
                        int W, void* stream);
/* The stem kernel has two operand paths: one tiled TMA copy per input row pair through a tensor
 * map with overlapping strides into a 128-byte-swizzled operand (used when the output row fits
 * 128 pixels and H is even), and bulk copies of plain rows read through an un-swizzled operand
 * (any shape up to 512 pixels wide).  policy 0 = automatic, 1 = always the plain-row path,
 * negative = leave unchanged.  Returns the path the last stem launch took (0 none yet, 1 plain
 * rows, 2 swizzled).  A test hook with no counterpart in the reference. */
int nncv_b200_stem_variant(int policy);

/* tensor.pad(-inf) + linalg.pooling_nchw_max (Res18.mlir:144-151), NHWC. */
int nncv_b200_maxpool_nhwc(const void* in, void* out, int dtype, int N, int H, int W, int C,
                           int k, int stride, int pad, void* stream);
/* linalg.pooling_nchw_sum over the map + divf (Res18.mlir:606-614), NHWC -> [N,C]. */
int nncv_b200_avgpool_nhwc(const void* in, void* out, int dtype, int N, int HW, int C,
                           void* stream);
/* NCHW -> NHWC with channels zero-padded to Cpad. */
int nncv_b200_nchw_to_nhwc(const void* in, int in_dtype, void* out, int out_dtype, int N, int C,
                           int H, int W, int Cpad, void* stream);
/* Batch-norm folding (Res18.mlir:127-137): scale = gamma*rsqrt(var+1e-5f), shift = beta-mean*scale. */
int nncv_b200_bn_fold(const void* gamma, const void* beta, const void* mean, const void* var,
                      int dtype, int C, float* scale, float* shift, void* stream);

/* ---- operators of nncv's mobile / detection fixtures (memory-bound; NHWC, device pointers) ----
 * Activations, as the fixtures spell them:
 *   RELU          cmpf ugt x, 0 ; select                         (tests/Nets/ReLU.mlir:8-13)
 *   HARD_SIGMOID  max(0, min(1, (x + 3) / 6))                    (tests/Nets/MobileNetV3.mlir:345-377)
 *   HARD_SWISH    x * hard_sigmoid(x)
 *   SIGMOID       1 / (1 + exp(-x))                              (tests/Nets/Yolov5s.mlir:158-164)
 *   SILU          x * sigmoid(x)                                 (Yolov5s.mlir:158-169)                  */
enum { NNCV_B200_ACT_NONE = 0, NNCV_B200_ACT_RELU = 1, NNCV_B200_ACT_HARD_SIGMOID = 2, NNCV_B200_ACT_HARD_SWISH = 3,
       NNCV_B200_ACT_SIGMOID = 4, NNCV_B200_ACT_SILU = 5 };
/* linalg.depthwise_conv_2d_nchw_chw (MobileNetV3.mlir:301,426,486) + folded batch-norm scale/shift
 * (fp32 [C] or NULL) + activation in one kernel.  in [N,H,W,C], weights [C,R,S] (the fixture's
 * collapsed tensor<CxRxS>; fp32, or fp16 when dtype is F16), out [N,OH,OW,C]; C a multiple of 8
 * (16-bit) or 4 (fp32). */
int nncv_b200_depthwise_conv_nhwc(const void* in, const void* weights, int w_dtype, const float* scale, const float* shift,
                                  void* out, int dtype, int N, int H, int W, int C, int R, int S, int stride, int pad, int act,
                                  void* stream);
/* Elementwise activation over n elements (n a multiple of 8 / 4); in == out allowed. */
int nncv_b200_activation(const void* in, void* out, int dtype, size_t n, int act, void* stream);
/* Squeeze-and-excitation (MobileNetV3.mlir:319-383): gate[N,C] = hard_sigmoid(w2 * relu(w1 * pooled + b1) + b2)
 * with pooled [N,C] (from nncv_b200_avgpool_nhwc), w1 [Cr,C], b1 [Cr], w2 [C,Cr], b2 [C] in fp32
 * (the two 1x1 convolutions on [N,C,1,1] of the fixture); then out = in * gate broadcast over pixels. */
int nncv_b200_se_gate(const void* pooled, const float* w1, const float* b1, const float* w2, const float* b2, void* gate,
                      int dtype, int N, int C, int Cr, void* stream);
int nncv_b200_scale_channels_nhwc(const void* in, const void* gate, void* out, int dtype, int N, int HW, int C, void* stream);
/* tensor.concat dim(1) (Yolov5s.mlir:276,445,837): out[p, :] = in_0[p, :] ++ in_1[p, :] ++ ... for
 * `pixels` = N*H*W pixels; up to 8 inputs, every channel count a multiple of 8 / 4. */
int nncv_b200_concat_channels_nhwc(const void* const* inputs, const int* channels, int n_inputs, void* out, int dtype,
                                   long long pixels, void* stream);
/* Nearest-neighbour 2x upsampling (Yolov5s.mlir:876-884: tensor.extract at floordivsi(index, 2)):
 * in [N,H,W,C] -> out [N,2H,2W,C]. */
int nncv_b200_upsample2x_nhwc(const void* in, void* out, int dtype, int N, int H, int W, int C, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NNCV_B200_H_ */
