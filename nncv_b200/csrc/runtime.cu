// Host runtime of libnncv_b200.so: the split-params container reader/writer, the params
// uploader (batch-norm folding, weight packing), the device executor that runs the ResNet
// forward as a sequence of kernels, and the C ABI declared in include/nncv_b200.h.
//
// It takes the place of nncv's libnncv runtime (src/libnncv/DataType.cpp, include/libnncv/
// DataType.hpp) plus the body MLIR would have generated for @forward (tests/Nets/Res18.mlir).
#include <cuda_runtime.h>

#include <algorithm>
#include <array>
#include <atomic>
#include <condition_variable>
#include <functional>
#include <thread>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "../../include/nncv_b200.h"
#include "kernels.h"

using namespace nncv_b200;

// =====================================================================================
// status
// =====================================================================================
namespace {

thread_local int g_status = NNCV_B200_OK;
thread_local char g_msg[512] = "";
std::mutex g_mutex;
std::atomic<long long> g_launches{0};

int fail(int code, const char* fmt, ...) {
  g_status = code;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_msg, sizeof(g_msg), fmt, ap);
  va_end(ap);
  return code;
}
int ok() {
  g_status = NNCV_B200_OK;
  g_msg[0] = 0;
  return NNCV_B200_OK;
}

#define CU(call)                                                                          \
  do {                                                                                    \
    cudaError_t e__ = (call);                                                             \
    if (e__ != cudaSuccess)                                                               \
      return fail(NNCV_B200_ECUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), \
                  __FILE__, __LINE__);                                                    \
  } while (0)
#define LAUNCH(call)                                                                      \
  do {                                                                                    \
    ++g_launches;                                                                         \
    CU(call);                                                                             \
  } while (0)

}  // namespace

// Status plumbing for the other translation units of the library.
namespace nncv_b200 {
int internal_fail(int code, const char* fmt, ...) {
  g_status = code;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_msg, sizeof(g_msg), fmt, ap);
  va_end(ap);
  return code;
}
int internal_ok() { return ok(); }
std::mutex& internal_mutex() { return g_mutex; }
int noalloc_read_status(int dev, int* flag);   // matmul_noalloc.cu
}  // namespace nncv_b200

namespace {

// =====================================================================================
// device contexts
// =====================================================================================
// One context per CUDA device, created the first time an entry point runs with that device
// current and kept until the process exits.  Every entry point works on the context of the
// calling thread's current device, so kernels always run on the GPU that owns their buffers.
struct Model;
struct Device {
  bool ready = false;
  int id = -1;
  cudaStream_t stream = nullptr;
  int* error_flag = nullptr;   // device
  cudaStream_t copy_stream = nullptr;  // host->device copies of a split batch
  cudaEvent_t copy_done[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};   // one per part + one ordering the copies after earlier work
  cudaStream_t user_stream = nullptr;  // stream _mlir_ciface_forward runs on when set
  bool user_stream_set = false;
  int sm_count = 148;
  void* scratch = nullptr;     // grow-only scratch (packed B of nncv_b200_matmul)
  size_t scratch_bytes = 0;
  Model* model = nullptr;      // the model replica living on this device
  std::vector<int> group;      // devices that hold a replica of this device's model (itself first), or empty
};
constexpr int kMaxDevices = 64;
Device* g_devices[kMaxDevices] = {};
thread_local Device* t_dev = nullptr;   // context of the device current on this thread (set by device_init)
#define g_dev (*t_dev)

int device_init() {
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(NNCV_B200_ENODEVICE, "no CUDA device: %s (this library has no CPU fallback)",
                cudaGetErrorString(e));
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(NNCV_B200_ENODEVICE, "cudaGetDevice failed");
  if (dev < 0 || dev >= kMaxDevices) return fail(NNCV_B200_ENODEVICE, "device index %d out of range", dev);
  if (g_devices[dev] && g_devices[dev]->ready) {
    t_dev = g_devices[dev];
    return NNCV_B200_OK;
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess)
    return fail(NNCV_B200_ENODEVICE, "cudaGetDeviceProperties failed");
  if (prop.major != 10)
    return fail(NNCV_B200_ENODEVICE, "device %d is sm_%d%d; the kernels are built for sm_100a only",
                dev, prop.major, prop.minor);
  if (!g_devices[dev]) g_devices[dev] = new Device();
  Device& d = *g_devices[dev];
  d.id = dev;
  d.sm_count = prop.multiProcessorCount;
  if (cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking) != cudaSuccess)
    return fail(NNCV_B200_ENODEVICE, "cudaStreamCreate failed");
  if (cudaMalloc(&d.error_flag, sizeof(int)) != cudaSuccess)
    return fail(NNCV_B200_ENOMEM, "cudaMalloc(error flag) failed");
  cudaMemset(d.error_flag, 0, sizeof(int));
  d.ready = true;
  t_dev = &d;
  return NNCV_B200_OK;
}

// Context of the calling thread's current device if one exists already (never creates one).
Device* current_device_or_null() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (dev < 0 || dev >= kMaxDevices || !g_devices[dev] || !g_devices[dev]->ready) return nullptr;
  return g_devices[dev];
}

int ensure_scratch(size_t bytes) {
  if (bytes <= g_dev.scratch_bytes) return NNCV_B200_OK;
  if (g_dev.scratch) {
    cudaDeviceSynchronize();
    cudaFree(g_dev.scratch);
    g_dev.scratch = nullptr;
    g_dev.scratch_bytes = 0;
  }
  const size_t want = (bytes + (1u << 20) - 1) & ~((size_t)(1u << 20) - 1);
  if (cudaMalloc(&g_dev.scratch, want) != cudaSuccess)
    return fail(NNCV_B200_ENOMEM, "cudaMalloc(%zu) for scratch failed", want);
  g_dev.scratch_bytes = want;
  return NNCV_B200_OK;
}

// ---- per-launch timing (off by default): CUDA events on the launching stream around each
// kernel of a forward, so a benchmark can attribute time to kernels without a profiler.
struct ProfRec {
  int kind;  // 0 tcgen05 igemm, 1 fp32 CUDA-core conv, 2 winograd, 3 memory-bound helper
  double flops, bytes;
  int M, N, K, bn;
  cudaEvent_t e0, e1;
  float ms;
};
bool g_autotune = getenv("NNCV_B200_AUTOTUNE") ? atoi(getenv("NNCV_B200_AUTOTUNE")) != 0 : true;
// NNCV_B200_LOG=1: one line to stderr per model load, activation plan and tuning decision (2: also every plan node of a
// forward).  NNCV_B200_NVTX=1: an NVTX range around every plan node of a forward, named after the node, for timeline
// tools.  Both are off by default and cost one branch when off.  (nncv's counterparts: its `-debug`-style LLVM options and
// the timers its fixtures carry, tests/Nets/Res18.mlir has none.)
int g_log_level = getenv("NNCV_B200_LOG") ? atoi(getenv("NNCV_B200_LOG")) : 0;
bool g_nvtx = getenv("NNCV_B200_NVTX") ? atoi(getenv("NNCV_B200_NVTX")) != 0 : false;
void log_line(int level, const char* fmt, ...) {
  if (g_log_level < level) return;
  va_list ap;
  va_start(ap, fmt);
  fputs("[nncv_b200] ", stderr);
  vfprintf(stderr, fmt, ap);
  fputc('\n', stderr);
  va_end(ap);
}
struct NvtxRange {   // RAII: pops on every exit path of the enclosing block
  bool on;
  explicit NvtxRange(const char* name) : on(g_nvtx) { if (on) nvtxRangePushA(name); }
  ~NvtxRange() { if (on) nvtxRangePop(); }
};
bool g_force_gather = false;  // tuning/test hook: route algo-0 convs through the gather kernel
bool g_prof_on = false;
int g_prof_dev = -1;            // records are taken on this device only (worker threads of a fan-out skip them)
std::vector<ProfRec> g_prof;

void prof_begin(int kind, double flops, double bytes, int M, int N, int K, int bn, cudaStream_t st) {
  if (!g_prof_on || !t_dev || t_dev->id != g_prof_dev) return;
  ProfRec r{kind, flops, bytes, M, N, K, bn, nullptr, nullptr, -1.0f};
  cudaEventCreate(&r.e0);
  cudaEventCreate(&r.e1);
  cudaEventRecord(r.e0, st);
  g_prof.push_back(r);
}
void prof_end(cudaStream_t st) {
  if (!g_prof_on || g_prof.empty() || !t_dev || t_dev->id != g_prof_dev) return;
  cudaEventRecord(g_prof.back().e1, st);
}
void prof_clear() {
  for (auto& r : g_prof) {
    if (r.e0) cudaEventDestroy(r.e0);
    if (r.e1) cudaEventDestroy(r.e1);
  }
  g_prof.clear();
}

// Turns a non-zero device status word into a status code and message.
int report_kernel_error(int flag, const char* where) {
  switch (flag) {
    case kErrWaitProducer:
      return fail(NNCV_B200_ETIMEOUT, "%s: the copy-issuing role of a kernel gave up a bounded wait for a free stage (code 1)", where);
    case kErrWaitLoader:
      return fail(NNCV_B200_ETIMEOUT, "%s: the weight loader of a kernel gave up a bounded wait for a free stage (code 2)", where);
    case kErrWaitMma:
      return fail(NNCV_B200_ETIMEOUT, "%s: the MMA-issuing role of a kernel gave up a bounded wait for a full stage (code 3)", where);
    case kErrWaitEpilogue:
      return fail(NNCV_B200_ETIMEOUT, "%s: the epilogue of a kernel gave up a bounded wait for its accumulator (code 4)", where);
    case kErrBounds:
      return fail(NNCV_B200_ECUDA, "%s: a kernel refused a copy that would have left its buffer (range check, code 5)", where);
    default:
      return fail(NNCV_B200_ECUDA, "%s: a kernel left the unknown status word %d", where, flag);
  }
}

// Reads (4-byte copy, cannot fault) and clears the device-side status word of the current
// device; call after the stream has been synchronised.  *flag_out receives the raw word.
int read_kernel_status(int* flag_out) {
  int flag = 0;
  CU(cudaMemcpy(&flag, g_dev.error_flag, sizeof(int), cudaMemcpyDeviceToHost));
  if (flag != 0) cudaMemset(g_dev.error_flag, 0, sizeof(int));
  *flag_out = flag;
  return NNCV_B200_OK;
}

int check_kernel_status() {
  int flag = 0;
  int rc = read_kernel_status(&flag);
  if (rc) return rc;
  return flag ? report_kernel_error(flag, "forward") : NNCV_B200_OK;
}

bool is_device_ptr(const void* p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  ~DevBuf() { if (p) cudaFree(p); }
  DevBuf() = default;
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
  int reserve(size_t n) {
    if (n <= bytes) return NNCV_B200_OK;
    if (p) { cudaFree(p); p = nullptr; bytes = 0; }
    if (cudaMalloc(&p, n) != cudaSuccess) return fail(NNCV_B200_ENOMEM, "cudaMalloc(%zu) failed", n);
    bytes = n;
    return NNCV_B200_OK;
  }
};

}  // namespace

// =====================================================================================
// convolution plan
// =====================================================================================
// NNCV_B200_FUSE_DS=0 runs the downsample 1x1 convs as their own launches
bool g_fuse_downsample = getenv("NNCV_B200_FUSE_DS") ? atoi(getenv("NNCV_B200_FUSE_DS")) != 0 : true;

// Optional on-disk memo of the timing decisions (NNCV_B200_TUNE_CACHE=<file>): one "key = value"
// line per decision, appended as they are made and read back at the first use, so that a later
// process -- a profiler run of the same command, a server restart -- launches exactly the kernels
// the first one settled on without timing anything.
struct TuneCache {
  bool loaded = false;
  std::string path;
  std::map<std::string, std::string> kv;
  void load() {
    if (loaded) return;
    loaded = true;
    const char* e = getenv("NNCV_B200_TUNE_CACHE");
    if (!e || !*e) return;
    path = e;
    if (FILE* f = fopen(path.c_str(), "r")) {
      char line[512];
      while (fgets(line, sizeof(line), f)) {
        char* eq = strstr(line, " = ");
        if (!eq) continue;
        *eq = 0;
        std::string v = eq + 3;
        while (!v.empty() && (v.back() == '\n' || v.back() == '\r')) v.pop_back();
        kv[line] = v;
      }
      fclose(f);
    }
  }
  std::mutex mu;   // the replicas of a multi-device model tune concurrently, each on its own thread
  // Entries are never erased or overwritten with another value, and std::map nodes do not move:
  // the returned pointer stays valid.
  const std::string* find(const std::string& k) {
    std::lock_guard<std::mutex> lk(mu);
    load();
    auto it = kv.find(k);
    return it == kv.end() ? nullptr : &it->second;
  }
  void put(const std::string& k, const std::string& v) {
    std::lock_guard<std::mutex> lk(mu);
    load();
    if (kv.count(k)) return;
    kv[k] = v;
    if (path.empty()) return;
    if (FILE* f = fopen(path.c_str(), "a")) {
      fprintf(f, "%s = %s\n", k.c_str(), v.c_str());
      fclose(f);
    }
  }
};
TuneCache g_tune_cache;

struct ConvChoice {
  int kernel = 5;  // 2 shifted-view conv3x3, 5 per-tap TMA kernel
  int bn = 64, mt = 1, resident = 0;
};

struct nncv_b200_conv {
  int Kout = 0, C = 0, R = 1, S = 1, stride = 1, pad = 0;
  int Cpad = 0;
  int device = -1;     // CUDA device the plan's buffers live on
  DType dtype = kF16;  // activation / operand type
  int algo = 0;
  // raw weights on the device, element strides for W[n][c][tap]
  const void* raw = nullptr;
  DType raw_dt = kF32;
  long long sn = 0, sc = 0, stap = 0;
  DevBuf raw_owned;                                // set when create() copied the weights
  DevBuf splitk;          // fp32 path: partial sums of a split reduction (small batches only)
  int want_act = 0;       // set by the plan executor: activation beyond ReLU it would like fused (hard-swish, SiLU)
  bool act_done = false;  // set by conv_run when the kernel it launched applied want_act
  std::map<int, std::unique_ptr<DevBuf>> packed;   // tcgen05 path: per N-tile width
  DevBuf w_f32;                                    // fp32 path: [Kout][R*S][Cpad]
  bool w_f32_ready = false;
  DevBuf sp_in, sp_out, sp_res;                    // standalone algo 2: shared-pad copies
  DevBuf wino_U, wino_V, wino_M;                   // algo 1: transformed filters / input / products
  std::vector<std::unique_ptr<DevBuf>> wino_w;     // algo 1: packed U per transform position
  int wino_bn = 0, wino_resident = 0;
  bool force_gather = false;                       // algo 3: the cp.async gather kernel even where TMA would do
  std::map<std::array<int, 5>, ConvChoice> tuned;  // measured best kernel/tile per (N, H, W, residual, out type)
  Conv3x3Config cfg3{0, 0, 0};                     // algo 2: forced tile configuration (bn 0 = auto)
  std::map<std::array<int, 3>, bool> fuse_tuned;   // per (N, H, W): is the launch fused with the 1x1 branch faster?
};

namespace {

// per_tap: the k blocks of 64 belong to one filter tap each (the TMA-fed kernels read 64 channels of one
// tap per block, so every tap's channels are padded to a multiple of 64 with zeros); otherwise the taps'
// channels are laid end to end (the gather kernel).  The two coincide when Cpad is a multiple of 64.
int conv_prepare(nncv_b200_conv* c, int bn, cudaStream_t st, const void** wpack, bool per_tap = false) {
  const int cpad = (per_tap && c->Cpad % 64 != 0) ? (c->Cpad + 63) / 64 * 64 : c->Cpad;
  const int key = bn + (cpad != c->Cpad ? (1 << 20) : 0);
  auto it = c->packed.find(key);
  if (it == c->packed.end()) {
    auto buf = std::make_unique<DevBuf>();
    int rc = buf->reserve(packed_weight_bytes(c->Kout, cpad, c->R, c->S, bn));
    if (rc) return rc;
    LAUNCH(launch_pack_weights(c->raw, c->raw_dt, c->sn, c->sc, c->stap, c->Kout, c->C, cpad,
                               c->R * c->S, bn, c->dtype, buf->p, st));
    it = c->packed.emplace(key, std::move(buf)).first;
  }
  *wpack = it->second->p;
  return NNCV_B200_OK;
}

// A 1x1 convolution of the same stride on the same input, fused into the per-tap kernel as an
// extra tap on the centre pixel (ResNet's downsample branch beside the block's first 3x3 conv).
struct FusedBranch {
  nncv_b200_conv* conv = nullptr;
  const float* scale = nullptr;
  const float* shift = nullptr;
  void* out = nullptr;   // layout and type of the main output
};

bool fused_branch_ok(const nncv_b200_conv& c, const nncv_b200_conv& b) {
  return !g_force_gather && g_fuse_downsample && c.dtype != kF32 && b.dtype == c.dtype && c.algo == 0 && b.algo == 0 &&
         !c.force_gather && c.R == c.S && (c.R & 1) && c.pad == c.R / 2 && b.R == 1 && b.S == 1 && b.pad == 0 &&
         b.stride == c.stride && b.Cpad == c.Cpad && b.Kout == c.Kout && c.Kout % 128 == 0 && c.Cpad % 64 == 0;
}

int conv_run(nncv_b200_conv* c, const void* in, Layout in_l, void* out, Layout out_l, int N, int H,
             int W, const float* scale, const float* shift, const void* residual, int relu,
             DType out_dt, long long ldo, cudaStream_t st, const FusedBranch* fb = nullptr) {
  const int OH = (H + 2 * c->pad - c->R) / c->stride + 1;
  const int OW = (W + 2 * c->pad - c->S) / c->stride + 1;
  if (N <= 0 || OH <= 0 || OW <= 0) return fail(NNCV_B200_EINVAL, "conv: empty output");
  if (in_l.pitch == 0) in_l = dense_layout(H, W);
  if (out_l.pitch == 0) out_l = dense_layout(OH, OW);
  if (c->dtype == kF32) {
    if (in_l.off != 0 || out_l.off != 0) return fail(NNCV_B200_EINVAL, "fp32 conv takes dense NHWC only");
    if (!c->w_f32_ready) {
      int rc = c->w_f32.reserve((size_t)c->Kout * c->R * c->S * c->Cpad * sizeof(float));
      if (rc) return rc;
      LAUNCH(launch_repack_weights_f32(c->raw, c->raw_dt, c->sn, c->sc, c->stap, c->Kout, c->C,
                                       c->Cpad, c->R * c->S, (float*)c->w_f32.p, st));
      c->w_f32_ready = true;
    }
    SimtConvArgs a;
    a.in = (const float*)in; a.w = (const float*)c->w_f32.p; a.scale = scale; a.shift = shift;
    a.residual = (const float*)residual; a.out = (float*)out;
    a.N = N; a.H = H; a.W = W; a.C = c->Cpad; a.OH = OH; a.OW = OW; a.Kout = c->Kout;
    a.R = c->R; a.S = c->S; a.stride = c->stride; a.pad = c->pad; a.ldo = ldo; a.relu = relu;
    a.sm_count = g_dev.sm_count;
    {
      // a small batch leaves few output tiles: room for the partial sums of a reduction split over more CTAs
      const long long tiles = (((long long)N * OH * OW + 63) / 64) * ((c->Kout + 63) / 64);
      if (tiles < g_dev.sm_count) {
        const size_t want = (size_t)32 * N * OH * OW * c->Kout * sizeof(float);
        const size_t cap = (size_t)16 << 20;
        int rc = c->splitk.reserve(want < cap ? want : cap);
        if (rc) return rc;
        a.scratch = (float*)c->splitk.p;
        a.scratch_bytes = c->splitk.bytes;
      }
    }
    const double Ms = (double)N * OH * OW;
    prof_begin(1, 2.0 * Ms * c->Kout * c->C * c->R * c->S,
               4.0 * ((double)N * H * W * c->C + (double)c->Kout * c->C * c->R * c->S +
                      Ms * c->Kout * (residual ? 2 : 1)),
               (int)Ms, c->Kout, c->C * c->R * c->S, 64, st);
    LAUNCH(launch_conv_simt_f32(a, st));
    prof_end(st);
    return NNCV_B200_OK;
  }
  const long long M = (long long)N * OH * OW;
  // Pointwise convolutions with up to 32 channels on both sides (MobileNetV3's 16 -> 16 at 112 x 112) are bound by HBM
  // and lose on tiles padded to 64 channels: they take the CUDA-core kernel (27 us against 109 us at batch 256; with
  // more channels the tensor-core kernel wins: 16 -> 72 measured 156 us against 141 us, 88 -> 24 64 against 43).  The
  // rule depends on the layer alone, never on the batch or on a timing, so a batch split over devices or into halves
  // gives the same bits as the whole batch.
  if (!fb && !g_force_gather && !c->force_gather && c->cfg3.bn == 0 && out_dt == c->dtype && ldo == c->Kout &&
      pointwise_supported(c->Cpad, c->Kout, c->R, c->S, c->stride, c->pad, c->dtype) && c->Cpad <= 32 && c->Kout <= 32) {
    if (!c->w_f32_ready) {
      int rc = c->w_f32.reserve((size_t)c->Kout * c->Cpad * sizeof(float));
      if (rc) return rc;
      LAUNCH(launch_repack_weights_f32(c->raw, c->raw_dt, c->sn, c->sc, c->stap, c->Kout, c->C, c->Cpad, 1, (float*)c->w_f32.p, st));
      c->w_f32_ready = true;
    }
    PointwiseArgs a;
    a.in = in; a.w = (const float*)c->w_f32.p; a.scale = scale; a.shift = shift; a.residual = residual; a.out = out;
    a.in_l = in_l; a.out_l = out_l; a.N = N; a.H = H; a.W = W; a.C = c->Cpad; a.Kout = c->Kout; a.ab = c->dtype; a.relu = relu;
    a.sm_count = g_dev.sm_count;
    if (c->want_act > kActRelu) { a.act = c->want_act; c->act_done = true; }
    prof_begin(9, 2.0 * (double)M * c->Kout * c->C, 2.0 * (double)M * (c->Cpad + c->Kout * (residual ? 2 : 1)), (int)M, c->Kout, c->C, 16, st);
    ++g_launches;
    LAUNCH(launch_pointwise(a, st));
    prof_end(st);
    return NNCV_B200_OK;
  }
  if (fb && (c->dtype == kF32 || out_dt != c->dtype || ldo != c->Kout || !fused_branch_ok(*c, *fb->conv)))
    return fail(NNCV_B200_EINVAL, "conv: the fused 1x1 branch does not fit this convolution");
  const double flops = 2.0 * (double)M * c->Kout * c->C * (c->R * c->S + (fb ? 1 : 0));
  const double bytes = 2.0 * ((double)N * H * W * c->C + (double)c->Kout * c->C * (c->R * c->S + (fb ? 1 : 0)) +
                              (double)M * c->Kout * ((residual ? 2 : 1) + (fb ? 1 : 0))) +
                       (out_dt == kF32 ? 2.0 * M * c->Kout : 0.0);
  // ---- tensor-core kernels fed by TMA: the shifted-view 3x3 kernel (needs shared-pad layouts) and
  // the per-tap kernel.  Which one, and with which tile, is timed once per (plan, shape).
  const bool sv_ok = c->algo == 2 && in_l.off == 1 && out_l.off == 1 && out_dt == c->dtype && ldo == c->Kout;
  if (c->algo == 2 && !sv_ok) return fail(NNCV_B200_EINVAL, "conv3x3: needs shared-pad NHWC input and output");
  const bool tc_ok = !g_force_gather && !c->force_gather && tconv_supported(c->Cpad, c->Kout, out_dt, ldo) && c->Kout >= 8;
  if (sv_ok || (c->algo == 0 && tc_ok)) {
    auto launch_choice = [&](const ConvChoice& ch, bool profile) -> int {
      const void* wpack = nullptr;
      // the CTA-pair kernels (7: shifted-view, 8: per-tap) read weights packed for half their N tile
      int rc = conv_prepare(c, (ch.kernel == 7 || ch.kernel == 8) ? (ch.bn / 2 < 64 ? 64 : ch.bn / 2) : ch.bn, st, &wpack, true);
      if (rc) return rc;
      if (ch.kernel == 7) {   // CTA-pair shifted-view kernel
        Conv3x3Args a;
        a.in = in; a.wpack = wpack; a.scale = scale; a.shift = shift; a.residual = residual; a.out = out;
        a.N = N; a.H = H; a.W = W; a.C = c->Cpad; a.Kout = c->Kout; a.ab = c->dtype; a.relu = relu; a.bn = ch.bn;
        a.mt = ch.mt;
        a.tail_split = ch.resident;   // for this kernel the field says whether the last round is sliced by columns
        a.sm_count = g_dev.sm_count; a.error_flag = g_dev.error_flag;
        if (profile) prof_begin(7, flops, bytes, (int)M, c->Kout, c->C * 9, ch.bn * 100 + ch.mt * 10 + ch.resident, st);
        ++g_launches;
        const cudaError_t e = launch_conv3x3_pair(a, st);
        if (profile) prof_end(st);
        return e == cudaSuccess ? 0 : -1;
      }
      if (ch.kernel == 2) {
        Conv3x3Args a;
        a.in = in; a.wpack = wpack; a.scale = scale; a.shift = shift; a.residual = residual; a.out = out;
        a.N = N; a.H = H; a.W = W; a.C = c->Cpad; a.Kout = c->Kout;
        a.bn = ch.bn; a.mt = ch.mt; a.resident = ch.resident; a.ab = c->dtype; a.relu = relu;
        a.sm_count = g_dev.sm_count; a.error_flag = g_dev.error_flag;
        if (profile) prof_begin(2, flops, bytes, (int)M, c->Kout, c->C * 9, ch.bn * 1000 + ch.mt * 10 + ch.resident, st);
        ++g_launches;
        const cudaError_t e = launch_conv3x3(a, st);
        if (profile) prof_end(st);
        return e == cudaSuccess ? 0 : -1;
      }
      TconvArgs a;
      a.in = in; a.wpack = wpack; a.scale = scale; a.shift = shift; a.residual = residual; a.out = out;
      a.pair = ch.kernel == 8;
      if (fb) {
        rc = conv_prepare(fb->conv, a.pair ? 64 : 128, st, &a.wpack2, true);
        if (rc) return rc;
        a.scale2 = fb->scale; a.shift2 = fb->shift; a.out2 = fb->out;
      }
      a.N = N; a.H = H; a.W = W; a.C = c->Cpad; a.OH = OH; a.OW = OW; a.Kout = c->Kout;
      a.R = c->R; a.S = c->S; a.stride = c->stride; a.pad = c->pad; a.in_l = in_l; a.out_l = out_l;
      a.bn = ch.bn; a.resident = ch.resident; a.ab = c->dtype; a.out_dtype = out_dt; a.relu = relu;
      if (c->want_act > kActRelu && out_dt != kF32 && !fb) { a.act = c->want_act; c->act_done = true; }
      a.sm_count = g_dev.sm_count; a.error_flag = g_dev.error_flag;
      if (profile) prof_begin(5, flops, bytes, (int)M, c->Kout, c->C * c->R * c->S, ch.bn * 10 + ch.resident + (a.pair ? 2 : 0), st);
      ++g_launches;
      const cudaError_t e = launch_tconv(a, st);
      if (profile) prof_end(st);
      return e == cudaSuccess ? 0 : -1;
    };
    // built-in choice
    ConvChoice ch;
    if (sv_ok) {
      const Conv3x3Config cfg = conv3x3_pick(N, H, W, c->Cpad, c->Kout, residual != nullptr);
      ch = ConvChoice{2, cfg.bn, cfg.mt, cfg.resident};
    } else {
      int tw, th, tn, bn, resident;
      tconv_tile(N, OH, OW, &tw, &th, &tn);
      const long long m_items = (long long)((OW + tw - 1) / tw) * ((OH + th - 1) / th) * ((N + tn - 1) / tn);
      tconv_pick(m_items, c->Cpad, c->Kout, c->R * c->S, &bn, &resident);
      ch = ConvChoice{5, bn, 1, resident};
    }
    if (fb) {
      // N tile 128, weights streamed with the A tiles: resident weights (160 KB for 64 channels) leave
      // room for two A stages only, too few copies in flight to cover the L2 latency (measured: 92 us
      // against 80 us on the 64 -> 128 channel block at batch 256)
      ch = ConvChoice{5, 128, 1, 0};
    }
    if (c->cfg3.bn) {
      if (fb) {
        if (c->cfg3.resident >= 2) ch.kernel = 8;   // forced: the fused launch on CTA pairs
      } else {
        ch.bn = c->cfg3.bn; ch.mt = c->cfg3.mt > 0 ? c->cfg3.mt : 1; ch.resident = c->cfg3.resident;
        if (c->cfg3.resident >= 2 && sv_ok) { ch.kernel = 7; ch.resident = c->cfg3.resident == 3; }   // forced CTA-pair kernel (3: sliced last round)
        if (c->cfg3.resident >= 2 && !sv_ok) { ch.kernel = 8; ch.resident = 0; }                      // per-tap kernel on CTA pairs
      }
    } else if (g_autotune) {
      const std::array<int, 5> key{N, H, W, (residual ? 1 : 0) + (fb ? 2 : 0), (int)out_dt};
      auto it = c->tuned.find(key);
      char ckey[192];
      snprintf(ckey, sizeof(ckey), "conv c%d k%d r%d s%d st%d p%d dt%d a%d n%d h%d w%d res%d o%d", c->Cpad, c->Kout, c->R, c->S,
               c->stride, c->pad, (int)c->dtype, c->algo, N, H, W, (residual ? 1 : 0) + (fb ? 2 : 0), (int)out_dt);
      if (it == c->tuned.end()) {
        if (const std::string* v = g_tune_cache.find(ckey)) {
          ConvChoice m;
          if (sscanf(v->c_str(), "%d %d %d %d", &m.kernel, &m.bn, &m.mt, &m.resident) == 4 &&
              (((m.kernel == 5 || m.kernel == 8) && tc_ok) || ((m.kernel == 2 || m.kernel == 7) && sv_ok)) &&
              (!fb || ((m.kernel == 5 || m.kernel == 8) && m.bn == 128 && !m.resident)))
            it = c->tuned.emplace(key, m).first;
        }
      }
      if (it == c->tuned.end()) {
        // time every candidate once per shape (results are identical, each run overwrites `out`)
        std::vector<ConvChoice> cand;
        if (sv_ok) {
          for (int mt : {1, 2}) cand.push_back(ConvChoice{2, 64, mt, 1});
          for (int bn : {64, 128, 256})
            for (int mt : {1, 2, 4})
              if (c->Kout % bn == 0 && bn * mt <= 512) cand.push_back(ConvChoice{2, bn, mt, 0});
          for (int bn : {64, 128, 256})
            if (c->Kout % bn == 0) {   // CTA pairs: sub-tiles per item, without and with the sliced last round
              for (int mt : {1, 2, 4}) {
                if (bn * mt > 512) continue;   // beyond 256 columns the accumulator is single-buffered
                cand.push_back(ConvChoice{7, bn, mt, 0});
                if (bn >= 128) cand.push_back(ConvChoice{7, bn, mt, 1});
              }
            }
        }
        if (fb) {   // the fused launch exists for N tile 128, streamed: one CTA or a pair
          cand.clear();
          cand.push_back(ConvChoice{5, 128, 1, 0});
          cand.push_back(ConvChoice{8, 128, 1, 0});
        } else if (tc_ok) {
          for (int bn : {64, 128}) cand.push_back(ConvChoice{5, bn, 1, 1});
          for (int bn : {64, 128, 256})
            if (bn <= c->Kout || bn == 64) cand.push_back(ConvChoice{5, bn, 1, 0});
          if (out_dt != kF32)
            for (int bn : {128, 256})
              if (c->Kout % bn == 0) cand.push_back(ConvChoice{8, bn, 1, 0});   // CTA pairs
        }
        cudaEvent_t e0, e1;
        CU(cudaEventCreate(&e0));
        CU(cudaEventCreate(&e1));
        float best = 1e30f;
        ConvChoice best_ch = ch;
        for (const ConvChoice& k : cand) {
          cudaGetLastError();
          if (launch_choice(k, false) != 0) { cudaGetLastError(); continue; }   // does not fit: skip
          // two groups of four launches, the faster group counts (one slow group -- another
          // tenant's burst, a clock dip -- must not decide)
          float ms = 1e30f;
          bool okl = true;
          for (int grp = 0; grp < 2 && okl; ++grp) {
            cudaEventRecord(e0, st);
            for (int rep = 0; rep < 4 && okl; ++rep) okl = launch_choice(k, false) == 0;
            cudaEventRecord(e1, st);
            if (cudaEventSynchronize(e1) != cudaSuccess) okl = false;
            float t = 0.f;
            if (okl) cudaEventElapsedTime(&t, e0, e1);
            if (okl && t < ms) ms = t;
          }
          if (!okl) { cudaGetLastError(); continue; }
          // A candidate that gave up (a bounded wait ran out, a range check refused a copy) leaves early
          // and would look fastest: read the status word and never choose, keep or persist such a one.
          int flag = 0;
          if (read_kernel_status(&flag) != NNCV_B200_OK || flag != 0) continue;
          if (ms < best) { best = ms; best_ch = k; }
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        it = c->tuned.emplace(key, best_ch).first;
        if (best < 1e30f) {   // only a choice that was measured without a complaint goes to the cache file
          char cval[64];
          snprintf(cval, sizeof(cval), "%d %d %d %d", best_ch.kernel, best_ch.bn, best_ch.mt, best_ch.resident);
          g_tune_cache.put(ckey, cval);
          log_line(1, "tuned %s -> kernel %d tile %d x%d mode %d (%.1f us, %zu candidates)", ckey, best_ch.kernel, best_ch.bn, best_ch.mt,
                   best_ch.resident, best * 250.0f, cand.size());
        }
      }
      ch = it->second;
    }
    c->act_done = false;   // candidates timed above may have set it; only the launch that stays counts
    if (launch_choice(ch, true) != 0)
      return fail(NNCV_B200_ECUDA, "conv launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return NNCV_B200_OK;
  }
  const int bn = igemm_pick_bn(M, c->Kout);
  const void* wpack = nullptr;
  int rc = conv_prepare(c, bn, st, &wpack);
  if (rc) return rc;
  IgemmArgs a;
  a.in = in; a.wpack = wpack; a.scale = scale; a.shift = shift; a.residual = residual; a.out = out;
  a.N = N; a.H = H; a.W = W; a.C = c->Cpad; a.OH = OH; a.OW = OW; a.Kout = c->Kout;
  a.R = c->R; a.S = c->S; a.stride = c->stride; a.pad = c->pad; a.ldo = ldo; a.bn = bn;
  a.in_l = in_l; a.out_l = out_l;
  a.ab = c->dtype; a.out_dtype = out_dt; a.relu = relu; a.error_flag = g_dev.error_flag;
  prof_begin(0, flops, bytes, (int)M, c->Kout, c->C * c->R * c->S, bn, st);
  LAUNCH(launch_conv_igemm(a, st));
  prof_end(st);
  return NNCV_B200_OK;
}

// =====================================================================================
// layer plans
// =====================================================================================
// A plan is the op sequence of @forward after the fusions nncv leaves to separate elementwise
// generics (tests/Nets/Res18.mlir:118-629): conv + batch-norm (+ residual add) (+ ReLU) is one
// node, then max-pool, global average pool and FC nodes.  Every parameter is named by its ELEMENT
// offset inside the params blob, i.e. the running sum of the element counts of the constants before
// it in module order, which is what -split-params bakes into the compiled object
// (SplitParamsFlatArray.cpp:48-56,84-92).  Tensor 0 is the network input; node i produces tensor
// `id`.  Built-in plans: ResNet-18 (constant order of Res18.mlir:12-109) and ResNet-50 (same rule,
// torchvision v1.5 topology); any other plan arrives as text from the .mlir importer.
struct PlanNode {
  enum Kind { kConv = 0, kMaxPool = 1, kAvgPool = 2, kFc = 3, kDwConv = 4, kSe = 5 };
  int kind = kConv;
  int id = 0, in = 0, res = -1;    // tensor ids; res: residual added before the activation (conv only)
  int cin = 0, cout = 0, k = 1, stride = 1, pad = 0, relu = 0;
  int act = 0;                     // activation code of the C ABI (0 none, 1 ReLU, 3 hard-swish, 5 SiLU); relu == (act == 1)
  int has_bn = 0, has_bias = 0;    // conv: batch-norm, or a plain bias (off_b)
  float eps = 1e-5f;               // batch-norm epsilon
  int cr = 0;                      // se: squeezed width; off_w/off_b = first 1x1 conv, off_w2/off_b2 = second
  size_t off_w = 0, off_gamma = 0, off_beta = 0, off_mean = 0, off_var = 0, off_b = 0, off_w2 = 0, off_b2 = 0;
  int aux_idx = -1;                // dwconv / se / fc: index into the model's per-kind tables
  // derived when the model is built
  int conv_idx = -1;      // index into Model::convs
  int branch = -1;        // node of a 1x1 conv on the same input that may ride along in this conv's launch
  int fused_into = -1;    // the reverse link
  int stem_pool = -1;     // conv: the max-pool node the fused stem kernel absorbs
  int absorbed = 0;       // max-pool node computed by the stem kernel
};
struct Plan {
  std::string name;
  std::vector<PlanNode> nodes;   // forward order
  size_t total = 0;              // elements in the params blob
  int out_features = 0;
};

Plan builtin_plan(int depth) {
  struct G { int cin, cout, k, stride, pad; size_t ob, og, ov, om, ow; };
  std::vector<G> groups;
  auto add = [&](int cin, int cout, int k, int stride, int pad) { groups.push_back(G{cin, cout, k, stride, pad, 0, 0, 0, 0, 0}); };
  add(3, 64, 7, 2, 3);
  const int widths[4] = {64, 128, 256, 512};
  const int blocks50[4] = {3, 4, 6, 3};
  int cin = 64;
  for (int l = 0; l < 4; ++l)
    for (int b = 0; b < (depth == 18 ? 2 : blocks50[l]); ++b) {
      const int stride = (b == 0 && l > 0) ? 2 : 1;
      if (depth == 18) {
        add(cin, widths[l], 3, stride, 1);
        add(widths[l], widths[l], 3, 1, 1);
        if (b == 0 && l > 0) add(cin, widths[l], 1, 2, 0);
        cin = widths[l];
      } else {
        add(cin, widths[l], 1, 1, 0);
        add(widths[l], widths[l], 3, stride, 1);
        add(widths[l], widths[l] * 4, 1, 1, 0);
        if (b == 0) add(cin, widths[l] * 4, 1, stride, 0);
        cin = widths[l] * 4;
      }
    }
  const int fc_in = depth == 18 ? 512 : 2048;
  Plan p;
  p.name = depth == 18 ? "resnet18" : "resnet50";
  size_t off = 0;
  const size_t off_fc_b = off; off += 1000;
  const size_t off_fc_w = off; off += (size_t)1000 * fc_in;
  for (int i = (int)groups.size() - 1; i >= 0; --i) {   // params order: last group first
    G& g = groups[i];
    g.ob = off; off += g.cout;
    g.og = off; off += g.cout;
    g.ov = off; off += g.cout;
    g.om = off; off += g.cout;
    g.ow = off; off += (size_t)g.cout * g.cin * g.k * g.k;
  }
  p.total = off;
  p.out_features = 1000;
  int next_id = 1;
  size_t gi = 0;
  auto conv = [&](int in, int res, int relu) {
    const G& g = groups[gi++];
    PlanNode n;
    n.kind = PlanNode::kConv; n.id = next_id++; n.in = in; n.res = res; n.relu = relu;
    n.cin = g.cin; n.cout = g.cout; n.k = g.k; n.stride = g.stride; n.pad = g.pad; n.has_bn = 1;
    n.off_w = g.ow; n.off_gamma = g.og; n.off_beta = g.ob; n.off_mean = g.om; n.off_var = g.ov;
    p.nodes.push_back(n);
    return n.id;
  };
  int x = conv(0, -1, 1);
  {
    PlanNode n;
    n.kind = PlanNode::kMaxPool; n.id = next_id++; n.in = x; n.k = 3; n.stride = 2; n.pad = 1; n.cin = n.cout = 64;
    p.nodes.push_back(n);
    x = n.id;
  }
  for (int l = 0; l < 4; ++l)
    for (int b = 0; b < (depth == 18 ? 2 : blocks50[l]); ++b) {
      const bool has_ds = depth == 18 ? (b == 0 && l > 0) : (b == 0);
      int t = conv(x, -1, 1);
      if (depth == 50) t = conv(t, -1, 1);
      // the last conv of the block comes before the downsample conv in the params order of the built-in
      // nets (conv2/conv3, then downsample), but it needs the downsample result: emit the node after it
      const size_t last_g = gi++;
      int idn = x;
      if (has_ds) idn = conv(x, -1, 0);
      const size_t after = gi;
      gi = last_g;
      x = conv(t, idn, 1);
      gi = after;
    }
  {
    PlanNode n;
    n.kind = PlanNode::kAvgPool; n.id = next_id++; n.in = x; n.cin = n.cout = fc_in;
    p.nodes.push_back(n);
    x = n.id;
    PlanNode f;
    f.kind = PlanNode::kFc; f.id = next_id++; f.in = x; f.cin = fc_in; f.cout = 1000; f.off_w = off_fc_w; f.off_b = off_fc_b;
    p.nodes.push_back(f);
  }
  return p;
}

// Plan text: one node per line, "key=value" fields after the kind; '#' starts a comment.
//   nncv_b200_plan 1
//   params <elements> out <features>
//   conv id=1 in=0 res=-1 cin=3 cout=64 k=7 stride=2 pad=3 relu=1 w=<off> gamma=<off> beta=<off> mean=<off> var=<off>
//   maxpool id=2 in=1 k=3 stride=2 pad=1
//   avgpool id=.. in=..
//   fc id=.. in=.. cin=512 cout=1000 w=<off> b=<off> [act=3]
// and, for the MobileNetV3 fixture: conv fields act=<code> (instead of relu=1), b=<off> (a bias instead of
// batch-norm), eps_bits=<fp32 bit pattern of the batch-norm epsilon when it is not 1e-5>;
//   dwconv id=.. in=.. c=.. k=.. stride=.. pad=.. act=.. w=<off> gamma=.. beta=.. mean=.. var=..   (depthwise conv + BN + act)
//   se id=.. in=.. c=.. cr=.. w1=<off> b1=<off> w2=<off> b2=<off>     (squeeze-and-excitation: scales its input)
int parse_plan(const std::string& text, Plan* out) {
  Plan p;
  p.name = "plan";
  size_t pos = 0;
  bool header = false;
  int line_no = 0;
  while (pos < text.size()) {
    size_t eol = text.find('\n', pos);
    if (eol == std::string::npos) eol = text.size();
    std::string line = text.substr(pos, eol - pos);
    pos = eol + 1;
    ++line_no;
    const size_t hash = line.find('#');
    if (hash != std::string::npos) line.resize(hash);
    std::vector<std::string> tok;
    {
      size_t i = 0;
      while (i < line.size()) {
        while (i < line.size() && isspace((unsigned char)line[i])) ++i;
        size_t j = i;
        while (j < line.size() && !isspace((unsigned char)line[j])) ++j;
        if (j > i) tok.push_back(line.substr(i, j - i));
        i = j;
      }
    }
    if (tok.empty()) continue;
    if (tok[0] == "nncv_b200_plan") {
      if (tok.size() < 2 || tok[1] != "1") return fail(NNCV_B200_EINVAL, "plan line %d: unknown plan version", line_no);
      header = true;
      continue;
    }
    if (!header) return fail(NNCV_B200_EINVAL, "plan line %d: the text does not start with \"nncv_b200_plan 1\"", line_no);
    if (tok[0] == "params") {
      if (tok.size() != 4 || tok[2] != "out") return fail(NNCV_B200_EINVAL, "plan line %d: expected \"params <n> out <features>\"", line_no);
      p.total = strtoull(tok[1].c_str(), nullptr, 10);
      p.out_features = atoi(tok[3].c_str());
      continue;
    }
    PlanNode n;
    if (tok[0] == "conv") n.kind = PlanNode::kConv;
    else if (tok[0] == "maxpool") n.kind = PlanNode::kMaxPool;
    else if (tok[0] == "avgpool") n.kind = PlanNode::kAvgPool;
    else if (tok[0] == "fc") n.kind = PlanNode::kFc;
    else if (tok[0] == "dwconv") n.kind = PlanNode::kDwConv;
    else if (tok[0] == "se") n.kind = PlanNode::kSe;
    else return fail(NNCV_B200_EINVAL, "plan line %d: unknown node kind \"%s\"", line_no, tok[0].c_str());
    for (size_t i = 1; i < tok.size(); ++i) {
      const size_t eq = tok[i].find('=');
      if (eq == std::string::npos) return fail(NNCV_B200_EINVAL, "plan line %d: field \"%s\" is not key=value", line_no, tok[i].c_str());
      const std::string k = tok[i].substr(0, eq);
      const long long v = strtoll(tok[i].c_str() + eq + 1, nullptr, 10);
      if (k == "id") n.id = (int)v;
      else if (k == "in") n.in = (int)v;
      else if (k == "res") n.res = (int)v;
      else if (k == "cin") n.cin = (int)v;
      else if (k == "cout") n.cout = (int)v;
      else if (k == "k") n.k = (int)v;
      else if (k == "stride") n.stride = (int)v;
      else if (k == "pad") n.pad = (int)v;
      else if (k == "relu") { n.relu = (int)v; if (v) n.act = kActRelu; }
      else if (k == "act") { n.act = (int)v; n.relu = v == kActRelu; }
      else if (k == "c") n.cin = n.cout = (int)v;
      else if (k == "cr") n.cr = (int)v;
      else if (k == "w" || k == "w1") n.off_w = (size_t)v;
      else if (k == "b" || k == "b1") { n.off_b = (size_t)v; n.has_bias = 1; }
      else if (k == "w2") n.off_w2 = (size_t)v;
      else if (k == "b2") n.off_b2 = (size_t)v;
      else if (k == "eps_bits") { const uint32_t bits = (uint32_t)v; memcpy(&n.eps, &bits, 4); }
      else if (k == "gamma") { n.off_gamma = (size_t)v; n.has_bn = 1; }
      else if (k == "beta") n.off_beta = (size_t)v;
      else if (k == "mean") n.off_mean = (size_t)v;
      else if (k == "var") n.off_var = (size_t)v;
      else return fail(NNCV_B200_EINVAL, "plan line %d: unknown field \"%s\"", line_no, k.c_str());
    }
    p.nodes.push_back(n);
  }
  if (!header || p.nodes.empty() || p.total == 0 || p.out_features <= 0)
    return fail(NNCV_B200_EINVAL, "plan: header, params line or nodes missing");
  *out = std::move(p);
  return NNCV_B200_OK;
}

// Checks ids, shapes and parameter ranges of a plan and derives the fusion links.  `act16`: the
// 16-bit tensor-core path (the fused stem and the fused downsample launch exist only there).
int finalize_plan(Plan& p, bool act16) {
  std::map<int, int> producer;   // tensor id -> node index
  std::map<int, int> channels;   // tensor id -> channels
  std::map<int, int> readers;    // tensor id -> number of reading nodes
  channels[0] = 3;
  for (size_t i = 0; i < p.nodes.size(); ++i) {
    PlanNode& n = p.nodes[i];
    if (n.id <= 0 || producer.count(n.id)) return fail(NNCV_B200_EINVAL, "plan: node %zu has a bad or repeated id %d", i, n.id);
    if (!channels.count(n.in)) return fail(NNCV_B200_EINVAL, "plan: node %zu reads tensor %d before it exists", i, n.in);
    ++readers[n.in];
    const int cin = channels[n.in];
    auto in_range = [&](size_t off, size_t cnt) { return off <= p.total && cnt <= p.total - off; };
    if (n.kind == PlanNode::kConv) {
      if (n.cin != cin || n.cout <= 0 || n.k <= 0 || n.stride <= 0 || n.pad < 0)
        return fail(NNCV_B200_EINVAL, "plan: conv node %zu has %d input channels, its input tensor has %d", i, n.cin, cin);
      if (!in_range(n.off_w, (size_t)n.cout * n.cin * n.k * n.k) ||
          (n.has_bn && (!in_range(n.off_gamma, n.cout) || !in_range(n.off_beta, n.cout) || !in_range(n.off_mean, n.cout) ||
                        !in_range(n.off_var, n.cout))) ||
          (!n.has_bn && n.has_bias && !in_range(n.off_b, n.cout)))
        return fail(NNCV_B200_EINVAL, "plan: conv node %zu names parameters outside the blob", i);
      if (n.act != kActNone && n.act != kActRelu && n.act != kActHardSwish && n.act != kActSilu)
        return fail(NNCV_B200_EINVAL, "plan: conv node %zu has activation %d; none, ReLU, hard-swish and SiLU can follow a convolution", i, n.act);
      if (!(n.eps > 0.f && n.eps < 1.f)) return fail(NNCV_B200_EINVAL, "plan: conv node %zu has a bad batch-norm epsilon", i);
      if (n.res >= 0) {
        if (!channels.count(n.res) || channels[n.res] != n.cout)
          return fail(NNCV_B200_EINVAL, "plan: conv node %zu adds tensor %d, which is missing or has other channels", i, n.res);
        ++readers[n.res];
      }
      channels[n.id] = n.cout;
    } else if (n.kind == PlanNode::kMaxPool) {
      if (n.k <= 0 || n.stride <= 0 || n.pad < 0 || n.in == 0) return fail(NNCV_B200_EINVAL, "plan: bad max-pool node %zu", i);
      n.cin = n.cout = cin;
      channels[n.id] = cin;
    } else if (n.kind == PlanNode::kAvgPool) {
      if (n.in == 0) return fail(NNCV_B200_EINVAL, "plan: bad average-pool node %zu", i);
      n.cin = n.cout = cin;
      channels[n.id] = cin;
    } else if (n.kind == PlanNode::kDwConv) {
      if (n.in == 0 || n.cin != cin || n.k <= 0 || n.stride <= 0 || n.pad < 0 || !n.has_bn || !(n.eps > 0.f && n.eps < 1.f))
        return fail(NNCV_B200_EINVAL, "plan: depthwise node %zu must read a %d-channel activation and carry a batch-norm", i, n.cin);
      if (!in_range(n.off_w, (size_t)n.cin * n.k * n.k) || !in_range(n.off_gamma, n.cin) || !in_range(n.off_beta, n.cin) ||
          !in_range(n.off_mean, n.cin) || !in_range(n.off_var, n.cin))
        return fail(NNCV_B200_EINVAL, "plan: depthwise node %zu names parameters outside the blob", i);
      if (n.act != kActNone && n.act != kActRelu && n.act != kActHardSwish && n.act != kActSilu)
        return fail(NNCV_B200_EINVAL, "plan: depthwise node %zu has activation %d", i, n.act);
      channels[n.id] = cin;
    } else if (n.kind == PlanNode::kSe) {
      if (n.in == 0 || n.cin != cin || n.cr <= 0 || (size_t)(n.cin + n.cr) * sizeof(float) > 48 * 1024)
        return fail(NNCV_B200_EINVAL, "plan: squeeze-and-excitation node %zu does not match its %d-channel input", i, cin);
      if (!in_range(n.off_w, (size_t)n.cr * n.cin) || !in_range(n.off_b, n.cr) || !in_range(n.off_w2, (size_t)n.cr * n.cin) ||
          !in_range(n.off_b2, n.cin))
        return fail(NNCV_B200_EINVAL, "plan: squeeze-and-excitation node %zu names parameters outside the blob", i);
      channels[n.id] = cin;
    } else {
      const int pk = producer.count(n.in) ? p.nodes[producer[n.in]].kind : -1;
      if (n.cin != cin || !in_range(n.off_w, (size_t)n.cout * n.cin) || !in_range(n.off_b, n.cout) ||
          (pk != PlanNode::kAvgPool && pk != PlanNode::kFc))
        return fail(NNCV_B200_EINVAL, "plan: FC node %zu must read a global average pool or another FC layer of %d features", i, n.cin);
      if (i + 1 == p.nodes.size() ? (n.cout != p.out_features || n.act != kActNone)
                                  : (n.act != kActNone && n.act != kActRelu && n.act != kActHardSwish))
        return fail(NNCV_B200_EINVAL, "plan: the last FC node must match the output size and have no activation");
      channels[n.id] = n.cout;
    }
    producer[n.id] = (int)i;
  }
  if (p.nodes.back().kind != PlanNode::kFc) return fail(NNCV_B200_EINVAL, "plan: the last node must be the FC layer");
  for (const PlanNode& n : p.nodes)
    if (n.kind == PlanNode::kSe && readers[n.in] != 1)
      return fail(NNCV_B200_EINVAL, "plan: tensor %d is scaled in place by squeeze-and-excitation node %d but has other readers", n.in, n.id);
  if (!act16) return NNCV_B200_OK;
  for (size_t i = 0; i < p.nodes.size(); ++i) {
    PlanNode& a = p.nodes[i];
    if (a.kind != PlanNode::kConv) continue;
    // ResNet stem: 7x7 stride-2 pad-3 conv 3 -> 64 + BN + ReLU on the network input, read only by a 3x3 stride-2 pad-1 max-pool
    if (a.in == 0 && a.cin == 3 && a.cout == 64 && a.k == 7 && a.stride == 2 && a.pad == 3 && a.relu && a.res < 0 && a.has_bn &&
        readers[a.id] == 1 && i + 1 < p.nodes.size()) {
      PlanNode& m = p.nodes[i + 1];
      if (m.kind == PlanNode::kMaxPool && m.in == a.id && m.k == 3 && m.stride == 2 && m.pad == 1) {
        a.stem_pool = (int)i + 1;
        m.absorbed = 1;
      }
    }
    // a 1x1 conv of the same stride on the same input may ride along as an extra tap (ResNet's downsample branch)
    if (a.in != 0 && a.res < 0 && a.relu && (a.k & 1) && a.pad == a.k / 2 && a.k >= 3 && a.cout % 128 == 0 && a.cin % 64 == 0)
      for (size_t j = i + 1; j < p.nodes.size() && j <= i + 3; ++j) {
        PlanNode& b = p.nodes[j];
        if (b.kind == PlanNode::kConv && b.in == a.in && b.k == 1 && b.pad == 0 && b.stride == a.stride && b.cout == a.cout &&
            b.res < 0 && !b.relu && b.fused_into < 0) {
          a.branch = (int)j;
          b.fused_into = (int)i;
          break;
        }
      }
  }
  return NNCV_B200_OK;
}

// =====================================================================================
// model + executor
// =====================================================================================
struct Model {
  Plan plan;
  size_t ele_width = 4;      // params / io element width
  DType io_dt = kF32;        // element type of src / dst
  DType act_dt = kF16;       // activation / compute type
  DevBuf blob;               // raw params on the device
  DevBuf folded;             // scale/shift for every group, fp32
  DevBuf aux;                // fp32 copies of the small tensors: biases, depthwise filters, squeeze-and-excitation weights
  std::vector<std::unique_ptr<nncv_b200_conv>> convs;
  std::vector<float*> scale, shift;
  std::vector<std::unique_ptr<nncv_b200_conv>> fcs;   // FC layers in plan order (PlanNode::aux_idx)
  std::vector<const float*> fc_bias;
  struct DwW { const float *w, *scale, *shift; };
  std::vector<DwW> dws;                                // depthwise nodes
  struct SeW { const float *w1, *b1, *w2, *b2; };
  std::vector<SeW> ses;                                // squeeze-and-excitation nodes
  int stem3_node = -1;                                 // 3x3 conv on the network input served by the direct kernel, or -1
  const float* stem3_w = nullptr;                      // its filter, fp32 [Cout][27]
  int stem_node = -1;        // conv node served by the fused stem + max-pool kernel, or -1
  const void* host_blob_id = nullptr;  // pointer identity of the blob the plan was built from
  // per-shape workspace
  int wsN = 0, wsH = 0, wsW = 0;
  DevBuf in_stage, in_nhwc, stem, pooled, logits32, logits_io;
  DevBuf stem_rows, stem_w;  // fused stem (16-bit path): reformatted input rows, packed weights
  bool fused_stem = false;
  int stem_rows_paired = -1;  // layout the zeroed pad pixels of stem_rows belong to (-1: none yet)
  // Activation tensors of one forward live in one arena.  The first forward of a shape walks the
  // network once without launching anything (planning = true) to record every tensor's size, layout
  // and usage interval in ops; offsets then come from arena_plan() (greedy by size, the scheme of
  // nncv's MemSolver), applied per layout class: tensors share memory only with tensors of the same
  // [rows, pitch, channels], so the zero pad slots of shared-pad tensors coincide and stay zero
  // whichever kernel writes the interior (the arena is zeroed once when it is created).
  struct ActRec {
    size_t bytes;
    std::array<int, 3> geom;   // rows per image, pitch, channels
    int first, last;           // ops that write it first / read it last
    size_t offset;
  };
  std::vector<ActRec> act_plan;
  bool planning = false, planned = false;
  int op_idx = 0;
  DevBuf arena;
  size_t act_bytes_unshared = 0;   // what one buffer per tensor would take
  size_t act_next = 0;
  static constexpr uintptr_t kFakeBase = (uintptr_t)0x7A00000000000000ull;   // planning pass: stand-in pointers
  void note_use(const void* p) {
    const uintptr_t v = (uintptr_t)p;
    if (!planning || v < kFakeBase) return;
    const size_t i = (size_t)((v - kFakeBase) >> 8);
    if (i < act_plan.size() && act_plan[i].last < op_idx) act_plan[i].last = op_idx;
  }
};
void model_reset() {
  if (t_dev && t_dev->model) {
    delete t_dev->model;
    t_dev->model = nullptr;
  }
}

DType dt_from_width(size_t w) { return w == 4 ? kF32 : kF16; }

int model_build(Plan plan, const void* host_blob, size_t n_elements, size_t ele_width,
                const nncv_b200_opts* opts) {
  int rc = device_init();
  if (rc) return rc;
  if (ele_width != 4 && ele_width != 2) return fail(NNCV_B200_EINVAL, "eleWidth must be 2 or 4");
  auto m = std::make_unique<Model>();
  if (n_elements != plan.total)
    return fail(NNCV_B200_EINVAL, "params hold %zu elements, %s needs %zu", n_elements, plan.name.c_str(), plan.total);
  m->ele_width = ele_width;
  m->io_dt = dt_from_width(ele_width);
  int cd = opts ? opts->compute_dtype : -1;
  if (cd < 0) cd = ele_width == 4 ? NNCV_B200_F32 : NNCV_B200_F16;
  if (cd != NNCV_B200_F32 && cd != NNCV_B200_F16 && cd != NNCV_B200_BF16)
    return fail(NNCV_B200_EINVAL, "bad compute_dtype %d", cd);
  m->act_dt = (DType)cd;
  if ((rc = finalize_plan(plan, m->act_dt != kF32))) return rc;
  m->plan = std::move(plan);
  cudaStream_t st = g_dev.stream;
  rc = m->blob.reserve(n_elements * ele_width);
  if (rc) return rc;
  CU(cudaMemcpyAsync(m->blob.p, host_blob, n_elements * ele_width, cudaMemcpyHostToDevice, st));
  const char* base = (const char*)m->blob.p;
  const DType pdt = dt_from_width(ele_width);
  auto at = [&](size_t off) { return (const void*)(base + off * ele_width); };

  size_t nfold = 0, naux = 0;
  for (auto& n : m->plan.nodes) {
    // every small tensor starts on a 16-byte boundary (the conv epilogues read scale / shift as vectors)
    if (n.kind == PlanNode::kConv) {
      nfold += 2 * (size_t)n.cout;
      if (!n.has_bn && n.has_bias) naux += n.cout + 4;
      if (n.in == 0) naux += (size_t)n.cout * 27 + 4;
    }
    else if (n.kind == PlanNode::kDwConv) { nfold += 2 * (size_t)n.cin; naux += (size_t)n.cin * n.k * n.k + 4; }
    else if (n.kind == PlanNode::kSe) naux += 2 * (size_t)n.cr * n.cin + n.cr + n.cin + 16;
    else if (n.kind == PlanNode::kFc) naux += n.cout + 4;
  }
  rc = m->folded.reserve(nfold * sizeof(float) + 16);
  if (rc) return rc;
  rc = m->aux.reserve(naux * sizeof(float) + 16);
  if (rc) return rc;
  float* fp = (float*)m->folded.p;
  float* ap = (float*)m->aux.p;
  auto to_f32 = [&](size_t off, size_t count) -> const float* {   // a small tensor of the blob as fp32
    float* dst = ap;
    ap += (count + 3) / 4 * 4;
    if (launch_convert(at(off), pdt, dst, kF32, count, st) != cudaSuccess) return nullptr;
    return dst;
  };
  for (size_t i = 0; i < m->plan.nodes.size(); ++i) {
    PlanNode& g = m->plan.nodes[i];
    if (g.kind == PlanNode::kFc) {
      // FC: weight [out, in] is already "[Kout][C]" (the forward's transpose generic,
      // Res18.mlir:617-620, is absorbed by reading it K-major); bias in fp32.
      if (g.cin % 8 != 0) return fail(NNCV_B200_EINVAL, "plan: FC input width %d must be a multiple of 8", g.cin);
      auto fc = std::make_unique<nncv_b200_conv>();
      fc->device = g_dev.id;
      fc->Kout = g.cout; fc->C = g.cin; fc->Cpad = g.cin; fc->dtype = m->act_dt;
      fc->raw = at(g.off_w); fc->raw_dt = pdt;
      fc->sn = g.cin; fc->sc = 1; fc->stap = 1;
      g.aux_idx = (int)m->fcs.size();
      m->fcs.push_back(std::move(fc));
      m->fc_bias.push_back(to_f32(g.off_b, (size_t)g.cout));
      if (!m->fc_bias.back()) return fail(NNCV_B200_ECUDA, "converting the FC bias failed");
      continue;
    }
    if (g.kind == PlanNode::kDwConv) {
      // depthwise filter [C,1,k,k] in fp32; batch-norm folded like a convolution's
      Model::DwW w{to_f32(g.off_w, (size_t)g.cin * g.k * g.k), fp, fp + g.cin};
      if (!w.w) return fail(NNCV_B200_ECUDA, "converting a depthwise filter failed");
      LAUNCH(launch_bn_fold(at(g.off_gamma), at(g.off_beta), at(g.off_mean), at(g.off_var), pdt, g.cin, g.eps, fp, fp + g.cin, st));
      fp += 2 * g.cin;
      g.aux_idx = (int)m->dws.size();
      m->dws.push_back(w);
      continue;
    }
    if (g.kind == PlanNode::kSe) {
      Model::SeW w{to_f32(g.off_w, (size_t)g.cr * g.cin), to_f32(g.off_b, (size_t)g.cr), to_f32(g.off_w2, (size_t)g.cr * g.cin),
                   to_f32(g.off_b2, (size_t)g.cin)};
      if (!w.w1 || !w.b1 || !w.w2 || !w.b2) return fail(NNCV_B200_ECUDA, "converting squeeze-and-excitation weights failed");
      g.aux_idx = (int)m->ses.size();
      m->ses.push_back(w);
      continue;
    }
    if (g.kind != PlanNode::kConv) continue;
    auto c = std::make_unique<nncv_b200_conv>();
    c->Kout = g.cout; c->C = g.cin; c->R = g.k; c->S = g.k; c->stride = g.stride; c->pad = g.pad;
    c->device = g_dev.id;
    c->dtype = m->act_dt;
    c->Cpad = m->act_dt == kF32 ? (g.cin + 3) / 4 * 4 : (g.cin + 7) / 8 * 8;
    if (m->act_dt != kF32 && g.in != 0 && conv3x3_supported(g.cin, g.cout, g.k, g.k, g.stride, g.pad)) c->algo = 2;
    c->raw = at(g.off_w); c->raw_dt = pdt;
    c->sn = (long long)g.cin * g.k * g.k; c->sc = (long long)g.k * g.k; c->stap = 1;
    g.conv_idx = (int)m->convs.size();
    m->convs.push_back(std::move(c));
    if (g.has_bn) {
      m->scale.push_back(fp);
      m->shift.push_back(fp + g.cout);
      LAUNCH(launch_bn_fold(at(g.off_gamma), at(g.off_beta), at(g.off_mean), at(g.off_var), pdt,
                            g.cout, g.eps, fp, fp + g.cout, st));
      fp += 2 * g.cout;
    } else if (g.has_bias) {
      const float* b = to_f32(g.off_b, (size_t)g.cout);
      if (!b) return fail(NNCV_B200_ECUDA, "converting a convolution bias failed");
      m->scale.push_back(nullptr);
      m->shift.push_back(const_cast<float*>(b));
    } else {
      m->scale.push_back(nullptr);
      m->shift.push_back(nullptr);
    }
    if (g.in == 0 && g.res < 0 && m->stem3_node < 0 && stem3x3_supported(g.cin, g.cout, g.k, g.k, m->act_dt, g.act) &&
        (g.has_bn || g.has_bias)) {
      m->stem3_w = to_f32(g.off_w, (size_t)g.cout * 27);
      if (!m->stem3_w) return fail(NNCV_B200_ECUDA, "converting the first convolution's filter failed");
      m->stem3_node = (int)i;
    }
    if (g.stem_pool >= 0 && m->stem_node < 0) {
      rc = m->stem_w.reserve(stem_wpack_bytes());
      if (rc) return rc;
      LAUNCH(launch_pack_stem_weights(at(g.off_w), pdt, m->stem_w.p, m->act_dt, st));
      m->fused_stem = true;
      m->stem_node = (int)i;
    }
  }
  CU(cudaStreamSynchronize(st));
  log_line(1, "loaded %s on device %d: %zu nodes, %zu parameters of %zu bytes, compute type %d", m->plan.name.c_str(), g_dev.id,
           m->plan.nodes.size(), m->plan.total, ele_width, (int)m->act_dt);
  m->host_blob_id = host_blob;
  model_reset();
  g_dev.model = m.release();
  return ok();
}

int ensure_workspace(Model& m, int N, int H, int W) {
  if (m.wsN == N && m.wsH == H && m.wsW == W) return NNCV_B200_OK;
  const size_t es = dtype_size(m.act_dt);
  if (H < 1 || W < 1) return fail(NNCV_B200_EINVAL, "input %dx%d too small", H, W);
  cudaDeviceSynchronize();
  m.act_plan.clear();
  m.planned = false;
  m.act_next = 0;
  int rc = 0;
  const int of = m.plan.out_features;
  if ((rc = m.in_stage.reserve((size_t)N * 3 * H * W * m.ele_width))) return rc;
  if (m.fused_stem && W <= 512 && H >= 7 && W >= 7) {
    if ((rc = m.stem_rows.reserve(stem_rows_bytes(N, H, W)))) return rc;
    CU(cudaMemset(m.stem_rows.p, 0, stem_rows_bytes(N, H, W)));   // the pad pixels of every row stay zero
    m.stem_rows_paired = (int)stem_paired_ok(H, W);
  } else {
    const int cpad0 = m.act_dt == kF32 ? 4 : 8;
    if ((rc = m.in_nhwc.reserve((size_t)N * H * W * cpad0 * es))) return rc;
  }
  if ((rc = m.logits32.reserve((size_t)N * of * sizeof(float)))) return rc;
  if ((rc = m.logits_io.reserve((size_t)N * of * m.ele_width))) return rc;
  m.wsN = N; m.wsH = H; m.wsW = W;
  return NNCV_B200_OK;
}

// Next activation tensor of the current forward ([N,h,w,c] in layout l).  Planning pass: records it
// and hands out a stand-in pointer; afterwards: its place in the arena.
int next_act(Model& m, int N, int h, int w, int c, Layout l, cudaStream_t st, void** out) {
  const size_t bytes = (size_t)layout_slots(l, N) * c * dtype_size(m.act_dt);
  (void)h; (void)w; (void)st;
  if (m.planning) {
    m.act_plan.push_back(Model::ActRec{bytes, {l.img_rows, l.pitch, c}, m.op_idx + 1, m.op_idx + 1, 0});
    *out = (void*)(Model::kFakeBase + ((uintptr_t)(m.act_plan.size() - 1) << 8));
    return NNCV_B200_OK;
  }
  if (m.act_next >= m.act_plan.size() || m.act_plan[m.act_next].bytes != bytes)
    return fail(NNCV_B200_ECUDA, "activation plan changed under a fixed shape");
  *out = (char*)m.arena.p + m.act_plan[m.act_next++].offset;
  return NNCV_B200_OK;
}

// Turns the tensors recorded by the planning pass into arena offsets and creates the arena.
int finish_act_plan(Model& m) {
  std::map<std::array<int, 3>, std::vector<size_t>> classes;
  for (size_t i = 0; i < m.act_plan.size(); ++i) classes[m.act_plan[i].geom].push_back(i);
  size_t base = 0, unshared = 0;
  for (auto& kv : classes) {
    std::vector<ArenaTensor> ts;
    for (size_t i : kv.second) {
      ArenaTensor t;
      t.first = m.act_plan[i].first; t.last = m.act_plan[i].last; t.size = m.act_plan[i].bytes;
      ts.push_back(t);
      unshared += m.act_plan[i].bytes;
    }
    const size_t total = arena_plan(ts, 1024);
    for (size_t k = 0; k < kv.second.size(); ++k) m.act_plan[kv.second[k]].offset = base + ts[k].offset;
    base += total;
  }
  m.act_bytes_unshared = unshared;
  if (base == 0) base = 1024;
  cudaDeviceSynchronize();   // nothing may still be reading an older arena
  int rc = m.arena.reserve(base);
  if (rc) return rc;
  CU(cudaMemset(m.arena.p, 0, m.arena.bytes));
  log_line(1, "activation arena: %zu tensors in %zu bytes (%zu bytes as private buffers)", m.act_plan.size(), base, unshared);
  m.planned = true;
  return NNCV_B200_OK;
}

// Runs the network on a dense NCHW device tensor; logits (io type) land in m.logits_io
// (or m.logits32 when io is fp32).  Asynchronous on `st`.
int model_forward_device(Model& m, const void* src_dev, int N, int H, int W, cudaStream_t st) {
  int rc = ensure_workspace(m, N, H, W);
  if (rc) return rc;
  if (!m.planned && !m.planning) {
    // first forward of this shape: one walk that launches nothing records the activation tensors
    m.planning = true;
    m.act_plan.clear();
    m.op_idx = 0;
    rc = model_forward_device(m, src_dev, N, H, W, st);
    m.planning = false;
    if (rc) return rc;
    if ((rc = finish_act_plan(m))) return rc;
  }
  m.act_next = 0;
  m.op_idx = 0;
  // every launch site is one op; in the planning pass it only notes which tensors the op reads
  auto begin_op = [&](std::initializer_list<const void*> reads) {
    ++m.op_idx;
    for (const void* q : reads) m.note_use(q);
    return !m.planning;
  };
  const DType adt = m.act_dt;
  const bool sp = adt != kF32;  // tensor-core path keeps block activations in shared-pad NHWC
  auto lay = [&](int h, int w) { return sp ? sp_layout(h, w) : dense_layout(h, w); };
  const double aes = (double)dtype_size(adt);
  struct Ten { void* p = nullptr; Layout l{0, 0, 0}; int h = 0, w = 0, c = 0; };
  std::map<int, Ten> tens;   // tensor id -> where it lives in this forward
  auto conv_of = [&](const PlanNode& n) -> nncv_b200_conv& { return *m.convs[n.conv_idx]; };
  auto run = [&](const PlanNode& n, const Ten& in, const Ten& out, const void* res) {
    nncv_b200_conv& c = conv_of(n);
    if (!begin_op({in.p, res})) return (int)NNCV_B200_OK;
    return conv_run(&c, in.p, in.l, out.p, out.l, N, in.h, in.w, m.scale[n.conv_idx], m.shift[n.conv_idx], res, n.relu, adt,
                    c.Kout, st);
  };
  const bool stem_fused_here = m.fused_stem && W <= 512 && H >= 7 && W >= 7;
  bool input_converted = false;
  const int cpad0 = adt == kF32 ? 4 : 8;
  static const char* const kKindName[] = {"conv", "maxpool", "avgpool", "fc", "dwconv", "se"};
  for (size_t ni = 0; ni < m.plan.nodes.size(); ++ni) {
    const PlanNode& n = m.plan.nodes[ni];
    char range_name[64] = "";
    if (g_nvtx || g_log_level >= 2) snprintf(range_name, sizeof(range_name), "%s id=%d in=%d c=%d->%d k=%d", kKindName[n.kind], n.id, n.in, n.cin, n.cout, n.k);
    NvtxRange range(range_name);
    if (!m.planning) log_line(2, "node %s", range_name);
    if (n.kind == PlanNode::kConv && n.in == 0 && stem_fused_here && (int)ni == m.stem_node) {
      // stem conv + BN + ReLU + max-pool in one kernel (Res18.mlir:118-151)
      const int oh = (H + 6 - 7) / 2 + 1, ow = (W + 6 - 7) / 2 + 1;
      const int ph = (oh + 2 - 3) / 2 + 1, pw = (ow + 2 - 3) / 2 + 1;
      if (ph <= 0 || pw <= 0) return fail(NNCV_B200_EINVAL, "input %dx%d too small", H, W);
      const bool paired = stem_paired_ok(H, W);
      if (begin_op({})) {
        prof_begin(3, 0, (double)N * H * (3.0 * W * m.ele_width + stem_row_pixels(W) * 8.0), N * H * W, 3, 0, 3, st);
        if (m.stem_rows_paired != (int)paired) {   // pad pixels sit elsewhere in the other layout
          CU(cudaMemsetAsync(m.stem_rows.p, 0, stem_rows_bytes(N, H, W), st));
          m.stem_rows_paired = (int)paired;
        }
        LAUNCH(launch_nchw_to_stem_rows(src_dev, m.io_dt, m.stem_rows.p, adt, N, H, W, true, paired, st));
        prof_end(st);
      }
      Ten o;
      o.l = lay(ph, pw); o.h = ph; o.w = pw; o.c = 64;
      if ((rc = next_act(m, N, ph, pw, 64, o.l, st, &o.p))) return rc;
      if (begin_op({})) {
        StemArgs a;
        a.in_rows = m.stem_rows.p; a.paired = paired; a.wpack = m.stem_w.p; a.scale = m.scale[n.conv_idx]; a.shift = m.shift[n.conv_idx];
        a.out = o.p; a.out_l = o.l; a.N = N; a.H = H; a.W = W; a.ab = adt;
        a.sm_count = g_dev.sm_count; a.error_flag = g_dev.error_flag;
        prof_begin(4, 2.0 * N * oh * ow * 64.0 * 147.0,
                   (double)N * H * stem_row_pixels(W) * 8.0 + 2.0 * N * ph * pw * 64.0, N * oh * ow, 64, 147, 64, st);
        LAUNCH(launch_stem_pool(a, st));
        prof_end(st);
      }
      tens[m.plan.nodes[n.stem_pool].id] = o;   // the pooled map; the conv's own output never exists
      continue;
    }
    if (n.kind == PlanNode::kMaxPool && n.absorbed && stem_fused_here) continue;
    if (n.kind == PlanNode::kConv && n.in == 0 && (int)ni == m.stem3_node) {
      // small-channel first layer straight from the NCHW input: no conversion pass, no padded GEMM (MobileNetV3.mlir:240-295)
      const int oh = (H + 2 * n.pad - 3) / n.stride + 1, ow = (W + 2 * n.pad - 3) / n.stride + 1;
      if (oh <= 0 || ow <= 0) return fail(NNCV_B200_EINVAL, "input %dx%d too small for the network", H, W);
      Ten o;
      o.l = lay(oh, ow); o.h = oh; o.w = ow; o.c = n.cout;
      if ((rc = next_act(m, N, oh, ow, n.cout, o.l, st, &o.p))) return rc;
      if (begin_op({})) {
        prof_begin(3, 2.0 * N * oh * ow * n.cout * 27.0, (double)N * (3.0 * H * W * m.ele_width + aes * oh * ow * n.cout), N * oh * ow,
                   n.cout, 27, 8, st);
        LAUNCH(launch_stem3x3(src_dev, m.io_dt, m.stem3_w, m.scale[n.conv_idx], m.shift[n.conv_idx], o.p, adt, o.l, N, H, W, n.cout,
                              n.stride, n.pad, n.act, st));
        ++g_launches;
        prof_end(st);
      }
      tens[n.id] = o;
      continue;
    }
    Ten in;
    if (n.in == 0) {
      // NCHW -> NHWC (channels padded), io type -> activation type; once per forward
      if (!input_converted) {
        if (!m.in_nhwc.p || m.in_nhwc.bytes < (size_t)N * H * W * cpad0 * dtype_size(adt)) {
          cudaDeviceSynchronize();
          if ((rc = m.in_nhwc.reserve((size_t)N * H * W * cpad0 * dtype_size(adt)))) return rc;
        }
        if (begin_op({})) {
          prof_begin(3, 0, (double)N * H * W * (3.0 * m.ele_width + cpad0 * aes), N * H * W, 3, 0, 0, st);
          LAUNCH(launch_nchw_to_nhwc(src_dev, m.io_dt, m.in_nhwc.p, adt, N, 3, H, W, cpad0, st));
          prof_end(st);
        }
        input_converted = true;
      }
      in.p = m.in_nhwc.p; in.l = dense_layout(H, W); in.h = H; in.w = W; in.c = 3;
    } else {
      auto it = tens.find(n.in);
      if (it == tens.end()) return fail(NNCV_B200_EINVAL, "plan: tensor %d is read before it is written", n.in);
      in = it->second;
    }
    if (n.kind == PlanNode::kConv) {
      if (n.fused_into >= 0 && tens.count(n.id) && tens[n.id].h < 0) {   // already computed beside its partner
        tens[n.id].h = -tens[n.id].h;
        continue;
      }
      nncv_b200_conv& c = conv_of(n);
      const int oh = (in.h + 2 * c.pad - c.R) / c.stride + 1, ow = (in.w + 2 * c.pad - c.S) / c.stride + 1;
      if (oh <= 0 || ow <= 0) return fail(NNCV_B200_EINVAL, "input %dx%d too small for the network", H, W);
      Ten o;
      if (n.fused_into >= 0 && tens.count(n.id)) {
        o = tens[n.id];   // allocated beside its partner, which ran alone
      } else {
        o.l = lay(oh, ow); o.h = oh; o.w = ow; o.c = c.Kout;
        if ((rc = next_act(m, N, oh, ow, c.Kout, o.l, st, &o.p))) return rc;
      }
      const void* res = nullptr;
      if (n.res >= 0) {
        auto it = tens.find(n.res);
        if (it == tens.end() || it->second.h != oh || it->second.w != ow)
          return fail(NNCV_B200_EINVAL, "plan: the residual of tensor %d does not have its shape", n.id);
        res = it->second.p;
      }
      bool done = false;
      if (n.branch >= 0 && sp && fused_branch_ok(c, conv_of(m.plan.nodes[n.branch]))) {
        // BasicBlock: the 3x3 stride-2 conv and the 1x1 stride-2 downsample conv read the same tensor
        const PlanNode& bn = m.plan.nodes[n.branch];
        Ten d;
        d.l = lay(oh, ow); d.h = oh; d.w = ow; d.c = c.Kout;
        if ((rc = next_act(m, N, oh, ow, c.Kout, d.l, st, &d.p))) return rc;
        FusedBranch fb{&conv_of(bn), m.scale[bn.conv_idx], m.shift[bn.conv_idx], d.p};
        bool fuse = c.Kout <= 128 && !m.planning;   // one Kout tile: the input is read once for both convolutions
        if (g_autotune && !m.planning) {
          // time both ways once per shape: one fused launch against the two tuned separate ones
          const std::array<int, 3> key{N, in.h, in.w};
          auto it = c.fuse_tuned.find(key);
          char fkey[128];
          snprintf(fkey, sizeof(fkey), "fuse c%d k%d r%d st%d dt%d n%d h%d w%d", c.Cpad, c.Kout, c.R, c.stride, (int)c.dtype, N, in.h, in.w);
          if (it == c.fuse_tuned.end()) {
            if (const std::string* v = g_tune_cache.find(fkey)) it = c.fuse_tuned.emplace(key, *v == "1").first;
          }
          if (it == c.fuse_tuned.end()) {
            cudaEvent_t e[3];
            for (auto& ev : e) CU(cudaEventCreate(&ev));
            const bool was = g_prof_on;
            g_prof_on = false;
            auto both = [&](bool fused) -> int {
              if (fused)
                return conv_run(&c, in.p, in.l, o.p, o.l, N, in.h, in.w, m.scale[n.conv_idx], m.shift[n.conv_idx], nullptr, 1,
                                adt, c.Kout, st, &fb);
              int r = run(n, in, o, nullptr);
              return r ? r : run(bn, in, d, nullptr);
            };
            rc = both(false);            // also lets each separate conv pick its own kernel
            if (!rc) rc = both(true);
            float ms_sep = 0.f, ms_fused = 0.f;
            if (!rc) {
              cudaEventRecord(e[0], st);
              for (int rep = 0; rep < 3 && !rc; ++rep) rc = both(false);
              cudaEventRecord(e[1], st);
              for (int rep = 0; rep < 3 && !rc; ++rep) rc = both(true);
              cudaEventRecord(e[2], st);
              if (!rc && cudaEventSynchronize(e[2]) == cudaSuccess) {
                cudaEventElapsedTime(&ms_sep, e[0], e[1]);
                cudaEventElapsedTime(&ms_fused, e[1], e[2]);
              }
              int flag = 0;
              if (!rc) rc = read_kernel_status(&flag);
              if (!rc && flag) rc = report_kernel_error(flag, "timing the fused downsample launch");
            }
            g_prof_on = was;
            for (auto& ev : e) cudaEventDestroy(ev);
            if (rc) return rc;
            it = c.fuse_tuned.emplace(key, ms_fused > 0.f && ms_fused < ms_sep).first;
            g_tune_cache.put(fkey, it->second ? "1" : "0");
          }
          fuse = it->second;
        }
        if (fuse) {
          begin_op({in.p});
          rc = conv_run(&c, in.p, in.l, o.p, o.l, N, in.h, in.w, m.scale[n.conv_idx], m.shift[n.conv_idx], nullptr, 1, adt,
                        c.Kout, st, &fb);
          if (rc) return rc;
          d.h = -d.h;   // marks the branch's tensor as already computed
          done = true;
        }
        tens[bn.id] = d;
      }
      c.want_act = n.act;
      c.act_done = false;
      if (!done && (rc = run(n, in, o, res))) return rc;
      c.want_act = 0;
      if (n.act > kActRelu && !(c.act_done && !m.planning) && begin_op({o.p})) {
        // hard-swish / SiLU: an elementwise pass over the tensor in place; both map 0 to 0, so the zero pads of a
        // padded layout stay zero
        const size_t elems = (size_t)layout_slots(o.l, N) * o.c;
        prof_begin(3, 0, 2.0 * aes * elems, (int)(elems / o.c), o.c, 0, 4, st);
        LAUNCH(launch_activation(o.p, o.p, adt, elems, n.act, st));
        prof_end(st);
      }
      tens[n.id] = o;
    } else if (n.kind == PlanNode::kDwConv) {
      // depthwise conv + folded batch-norm + activation in one kernel (MobileNetV3.mlir:296-318)
      const int oh = (in.h + 2 * n.pad - n.k) / n.stride + 1, ow = (in.w + 2 * n.pad - n.k) / n.stride + 1;
      if (oh <= 0 || ow <= 0) return fail(NNCV_B200_EINVAL, "input %dx%d too small for the network", H, W);
      Ten o;
      o.l = lay(oh, ow); o.h = oh; o.w = ow; o.c = in.c;
      if ((rc = next_act(m, N, oh, ow, in.c, o.l, st, &o.p))) return rc;
      if (begin_op({in.p})) {
        const Model::DwW& w = m.dws[n.aux_idx];
        prof_begin(3, 2.0 * N * oh * ow * in.c * n.k * n.k, aes * in.c * N * ((double)in.h * in.w + (double)oh * ow), N * oh * ow, in.c,
                   n.k * n.k, 5, st);
        if (launch_depthwise(in.p, w.w, kF32, w.scale, w.shift, o.p, adt, N, in.h, in.w, in.c, n.k, n.k, n.stride, n.pad, n.act, in.l,
                             o.l, g_dev.sm_count, g_dev.error_flag, st) != cudaSuccess) {
          cudaGetLastError();
          return fail(NNCV_B200_EINVAL, "depthwise node %d: %d channels are not a multiple of the 16-byte vector", n.id, in.c);
        }
        ++g_launches;
        prof_end(st);
      }
      tens[n.id] = o;
    } else if (n.kind == PlanNode::kSe) {
      // squeeze-and-excitation (MobileNetV3.mlir:319-389): pooled = mean(x); gate = hard-sigmoid(W2 relu(W1 pooled + b1) + b2);
      // x *= gate, in place (the plan checker has made sure nothing else reads the unscaled tensor)
      const Model::SeW& w = m.ses[n.aux_idx];
      Ten pooled, gate;
      pooled.l = gate.l = dense_layout(1, 1);
      pooled.h = pooled.w = gate.h = gate.w = 1;
      pooled.c = gate.c = in.c;
      if ((rc = next_act(m, N, 1, 1, in.c, pooled.l, st, &pooled.p))) return rc;
      if ((rc = next_act(m, N, 1, 1, in.c, gate.l, st, &gate.p))) return rc;
      if (begin_op({in.p})) {
        prof_begin(3, 0, aes * in.c * N * (in.h * in.w + 1.0), N * in.h * in.w, in.c, 0, 2, st);
        LAUNCH(launch_avgpool_nhwc(in.p, pooled.p, adt, N, in.h, in.w, in.c, in.l, st));
        prof_end(st);
      }
      if (begin_op({pooled.p})) {
        prof_begin(3, 4.0 * N * in.c * n.cr, 8.0 * in.c * n.cr, N, in.c, n.cr, 6, st);
        LAUNCH(launch_se_gate(pooled.p, w.w1, w.b1, w.w2, w.b2, gate.p, adt, N, in.c, n.cr, st));
        prof_end(st);
      }
      if (begin_op({in.p, gate.p})) {
        const long long slots = (long long)in.l.img_rows * in.l.pitch;
        prof_begin(3, 0, 2.0 * aes * in.c * N * slots, (int)(N * slots), in.c, 0, 7, st);
        LAUNCH(launch_scale_channels(in.p, gate.p, in.p, adt, N, slots, in.c, st));
        prof_end(st);
      }
      tens[n.id] = in;
    } else if (n.kind == PlanNode::kMaxPool) {
      const int oh = (in.h + 2 * n.pad - n.k) / n.stride + 1, ow = (in.w + 2 * n.pad - n.k) / n.stride + 1;
      if (oh <= 0 || ow <= 0) return fail(NNCV_B200_EINVAL, "input %dx%d too small for the network", H, W);
      Ten o;
      o.l = lay(oh, ow); o.h = oh; o.w = ow; o.c = in.c;
      if ((rc = next_act(m, N, oh, ow, in.c, o.l, st, &o.p))) return rc;
      if (begin_op({in.p})) {
        prof_begin(3, 0, aes * in.c * N * ((double)in.h * in.w + (double)oh * ow), N * in.h * in.w, in.c, 0, 1, st);
        LAUNCH(launch_maxpool_nhwc(in.p, o.p, adt, N, in.h, in.w, in.c, n.k, n.stride, n.pad, in.l, o.l, st));
        prof_end(st);
      }
      tens[n.id] = o;
    } else if (n.kind == PlanNode::kAvgPool) {
      // global average pool (Res18.mlir:606-614) -> dense [N, C]
      Ten o;
      o.l = dense_layout(1, 1); o.h = 1; o.w = 1; o.c = in.c;
      if ((rc = next_act(m, N, 1, 1, in.c, o.l, st, &o.p))) return rc;
      if (begin_op({in.p})) {
        prof_begin(3, 0, aes * in.c * N * (in.h * in.w + 1.0), N * in.h * in.w, in.c, 0, 2, st);
        LAUNCH(launch_avgpool_nhwc(in.p, o.p, adt, N, in.h, in.w, in.c, in.l, st));
        prof_end(st);
      }
      tens[n.id] = o;
    } else {
      // FC (Res18.mlir:617-628)
      nncv_b200_conv* fc = m.fcs[n.aux_idx].get();
      const float* bias = m.fc_bias[n.aux_idx];
      if (ni + 1 != m.plan.nodes.size()) {
        // a hidden FC layer (MobileNetV3.mlir:1784-1845): [N, cin] -> [N, cout] in the activation type, then its activation
        Ten o;
        o.l = dense_layout(1, 1); o.h = o.w = 1; o.c = n.cout;
        if ((rc = next_act(m, N, 1, 1, n.cout, o.l, st, &o.p))) return rc;
        if (begin_op({in.p}) &&
            (rc = conv_run(fc, in.p, dense_layout(1, 1), o.p, dense_layout(1, 1), N, 1, 1, nullptr, bias, nullptr, n.act == kActRelu, adt,
                           n.cout, st)))
          return rc;
        if (n.act > kActRelu && begin_op({o.p})) LAUNCH(launch_activation(o.p, o.p, adt, (size_t)N * n.cout, n.act, st));
        tens[n.id] = o;
        continue;
      }
      const int of = m.plan.out_features;
      if (!begin_op({in.p})) return NNCV_B200_OK;   // the planning pass ends with the last reader of an activation tensor
      if (m.io_dt == adt && adt != kF32) {
        // 16-bit logits wanted and computed in the same type: the FC epilogue rounds once, exactly as
        // the fp32 -> io conversion kernel would, and that kernel is not launched
        return conv_run(fc, in.p, dense_layout(1, 1), m.logits_io.p, dense_layout(1, 1), N, 1, 1, nullptr, bias, nullptr, 0, adt, of,
                        st);
      }
      rc = conv_run(fc, in.p, dense_layout(1, 1), m.logits32.p, dense_layout(1, 1), N, 1, 1, nullptr, bias, nullptr, 0, kF32, of, st);
      if (rc) return rc;
      if (m.io_dt != kF32)
        LAUNCH(launch_convert(m.logits32.p, kF32, m.logits_io.p, m.io_dt, (size_t)N * of, st));
      return NNCV_B200_OK;
    }
  }
  return fail(NNCV_B200_EINVAL, "plan: no FC node produced the output");
}

int check_src(const nncv_memref4* src, int* N, int* H, int* W) {
  if (!src || !src->aligned) return fail(NNCV_B200_EINVAL, "src descriptor or its pointer is null");
  const intptr_t n = src->sizes[0], c = src->sizes[1], h = src->sizes[2], w = src->sizes[3];
  if (n <= 0 || c != 3 || h <= 0 || w <= 0 || n > 65536 || h > 16384 || w > 16384)
    return fail(NNCV_B200_EINVAL, "src must be [N,3,H,W], got [%ld,%ld,%ld,%ld]", (long)n, (long)c, (long)h, (long)w);
  // dense NCHW.  The reference's example writes the row stride as H (examples/Res18/main.cpp:87-93),
  // which equals W only for square images; accept exactly that spelling too.
  const bool row_ok = src->strides[2] == w || (h == w && src->strides[2] == h);
  if (src->strides[3] != 1 || !row_ok || src->strides[1] != h * w || src->strides[0] != c * h * w)
    return fail(NNCV_B200_EINVAL, "src must be dense NCHW (strides %ld,%ld,%ld,%ld)", (long)src->strides[0],
                (long)src->strides[1], (long)src->strides[2], (long)src->strides[3]);
  *N = (int)n; *H = (int)h; *W = (int)w;
  return NNCV_B200_OK;
}

int check_dst(nncv_memref2* dst, int N, int of, size_t ele_width, bool* allocated_here) {
  *allocated_here = false;
  if (!dst) return fail(NNCV_B200_EINVAL, "dst descriptor is null");
  if (!dst->aligned) {
    // MLIR convention: the callee allocates the result memref.
    void* p = malloc((size_t)N * of * ele_width);
    if (!p) return fail(NNCV_B200_ENOMEM, "malloc of the result buffer failed");
    dst->allocated = dst->aligned = p;
    dst->offset = 0;
    dst->sizes[0] = N; dst->sizes[1] = of;
    dst->strides[0] = of; dst->strides[1] = 1;
    *allocated_here = true;
    return NNCV_B200_OK;
  }
  if (dst->sizes[0] != N || dst->sizes[1] != of)
    return fail(NNCV_B200_EINVAL, "dst must be [%d,%d], got [%ld,%ld]", N, of, (long)dst->sizes[0], (long)dst->sizes[1]);
  if (dst->strides[1] != 1 || dst->strides[0] < of)
    return fail(NNCV_B200_EINVAL, "dst rows must be contiguous (strides %ld,%ld)", (long)dst->strides[0], (long)dst->strides[1]);
  return NNCV_B200_OK;
}

// One device's share of a forward: images [sp, sp + N images) -> logits rows at dp (row pitch
// dst_stride elements).  Runs on the calling thread's current device (g_dev), on stream st;
// synchronises and reads the device status word unless device_only.
int forward_slice(Model& m, const char* sp, bool src_dev, char* dp, bool dst_dev, size_t dst_stride, int N, int H, int W,
                  cudaStream_t st, bool device_only) {
  int rc;
  const size_t ew = m.ele_width;
  const int of = m.plan.out_features;
  const size_t img_bytes = (size_t)3 * H * W * ew;
  // Host input, large batch: run the batch as two halves so that the host->device copy of the
  // second half overlaps the forward of the first (copies on their own stream, ordered by events).
  // Four parts were slower at batch 256 (2.48 ms against 2.27 ms): four forwards of 64 images take
  // longer than two of 128, and the kernels, not the copy, are then the longer leg.
  const int chunks = (!src_dev && !device_only && N >= 128 && N % 2 == 0) ? 2 : 1;
  const int Nc = N / chunks;
  if ((rc = ensure_workspace(m, Nc, H, W))) return rc;
  if (!src_dev && (rc = m.in_stage.reserve((size_t)N * img_bytes))) return rc;
  if (chunks > 1) {
    if (!g_dev.copy_stream) {
      CU(cudaStreamCreateWithFlags(&g_dev.copy_stream, cudaStreamNonBlocking));
      for (auto& e : g_dev.copy_done) CU(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    // the copy stream must not overwrite the staging buffer before earlier work on `st` has read it
    CU(cudaEventRecord(g_dev.copy_done[4], st));
    CU(cudaStreamWaitEvent(g_dev.copy_stream, g_dev.copy_done[4], 0));
    for (int c = 0; c < chunks; ++c) {
      CU(cudaMemcpyAsync((char*)m.in_stage.p + (size_t)c * Nc * img_bytes, sp + (size_t)c * Nc * img_bytes,
                         (size_t)Nc * img_bytes, cudaMemcpyHostToDevice, g_dev.copy_stream));
      CU(cudaEventRecord(g_dev.copy_done[c], g_dev.copy_stream));
    }
  } else if (!src_dev) {
    CU(cudaMemcpyAsync(m.in_stage.p, sp, (size_t)N * img_bytes, cudaMemcpyHostToDevice, st));
  }
  for (int c = 0; c < chunks; ++c) {
    const void* src_d = src_dev ? (const void*)sp : (const void*)((char*)m.in_stage.p + (size_t)c * Nc * img_bytes);
    if (chunks > 1) CU(cudaStreamWaitEvent(st, g_dev.copy_done[c], 0));
    if ((rc = model_forward_device(m, src_d, Nc, H, W, st))) return rc;
    const void* logits = m.io_dt == kF32 ? m.logits32.p : m.logits_io.p;
    CU(cudaMemcpy2DAsync(dp + (size_t)c * Nc * dst_stride * ew, dst_stride * ew, logits, (size_t)of * ew,
                         (size_t)of * ew, (size_t)Nc, dst_dev ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, st));
  }
  if (device_only) return ok();
  CU(cudaStreamSynchronize(st));
  if ((rc = check_kernel_status())) return rc;
  return ok();
}

int forward_fanout(const char* sp, char* dp, size_t dst_stride, int N, int H, int W);

int forward_impl(nncv_memref2* dst, nncv_memref4* src, void* params, cudaStream_t user_stream,
                 bool device_only) {
  int rc = device_init();
  if (rc) return rc;
  if (!g_dev.model) {
    // Lazy plan from the blob descriptor: element count selects the network; the element type of
    // a bare descriptor is float (the only type the reference's -split-params writes,
    // SplitParamsFlatArray.cpp:144-147).
    auto* pd = static_cast<nncv_memref1*>(params);
    if (!pd || !pd->aligned) return fail(NNCV_B200_ENOMODEL, "no model loaded and params is null");
    const size_t n = (size_t)pd->sizes[0];
    int depth = 0;
    if (n == builtin_plan(18).total) depth = 18;
    else if (n == builtin_plan(50).total) depth = 50;
    else return fail(NNCV_B200_ENOMODEL, "params hold %zu elements: neither resnet18 nor resnet50", n);
    rc = model_build(builtin_plan(depth), (const char*)pd->aligned + pd->offset * 4, n, 4, nullptr);
    if (rc) return rc;
  } else if (params) {
    auto* pd = static_cast<nncv_memref1*>(params);
    if ((size_t)pd->sizes[0] != g_dev.model->plan.total)
      return fail(NNCV_B200_EINVAL, "params hold %ld elements, the loaded model has %zu", (long)pd->sizes[0],
                  g_dev.model->plan.total);
  }
  Model& m = *g_dev.model;
  int N, H, W;
  if ((rc = check_src(src, &N, &H, &W))) return rc;
  bool allocated_here = false;
  const int of = m.plan.out_features;
  if ((rc = check_dst(dst, N, of, m.ele_width, &allocated_here))) return rc;
  const size_t ew = m.ele_width;
  const char* sp = (const char*)src->aligned + src->offset * (intptr_t)ew;
  char* dp = (char*)dst->aligned + dst->offset * (intptr_t)ew;
  const bool src_dev = is_device_ptr(sp), dst_dev = is_device_ptr(dp);
  if (device_only && (!src_dev || !dst_dev))
    return fail(NNCV_B200_EINVAL, "nncv_b200_forward_device needs device-resident src and dst");
  cudaStream_t st = device_only ? user_stream : (g_dev.user_stream_set ? g_dev.user_stream : g_dev.stream);
  // several devices hold a replica (nncv_b200_opts.device_mask at load) and the tensors are in host
  // memory: every device takes a contiguous slice of the batch
  if (!device_only && !src_dev && !dst_dev && g_dev.group.size() > 1 && N > 1)
    return forward_fanout(sp, dp, (size_t)dst->strides[0], N, H, W);
  return forward_slice(m, sp, src_dev, dp, dst_dev, (size_t)dst->strides[0], N, H, W, st, device_only);
}

// =====================================================================================
// batch fan-out over the devices of one process
// =====================================================================================
// Images are independent, so a batch in host memory is cut into contiguous slices, one per device
// that holds a replica of the model; each device copies its slice in, runs the forward and copies
// its logits rows straight into the caller's buffer -- there is no exchange between devices, hence
// no collective.  One persistent host thread per extra device issues that device's work (its launch
// sequence would otherwise queue behind the other devices' on one thread); the calling thread serves
// the first device of the group.  nncv itself is single-device (include/nncv/compiler/Utils/
// PlatformCtx.hpp:140-144 warns when the GPU count is not 1).

// Slice [lo, hi) of n items owned by part `rank` of `world`: the first n % world parts get one more.
void shard_range(int n, int rank, int world, int* lo, int* hi) {
  const int base = n / world, extra = n % world;
  *lo = rank * base + (rank < extra ? rank : extra);
  *hi = *lo + base + (rank < extra ? 1 : 0);
}

struct Worker {
  std::thread th;
  std::mutex mu;
  std::condition_variable cv;
  std::function<int()> job;
  bool has_job = false, done = false, quit = false;
  int rc = 0;
  std::string msg;
  void loop() {
    std::unique_lock<std::mutex> lk(mu);
    for (;;) {
      cv.wait(lk, [&] { return has_job || quit; });
      if (quit) return;
      std::function<int()> j = std::move(job);
      has_job = false;
      lk.unlock();
      const int r = j();
      lk.lock();
      rc = r;
      msg = r ? g_msg : "";    // the status text lives in this thread's own buffer: hand it over
      done = true;
      cv.notify_all();
    }
  }
  void submit(std::function<int()> j) {
    std::lock_guard<std::mutex> lk(mu);
    job = std::move(j);
    has_job = true;
    done = false;
    cv.notify_all();
  }
  int wait(std::string* m) {
    std::unique_lock<std::mutex> lk(mu);
    cv.wait(lk, [&] { return done; });
    *m = msg;
    return rc;
  }
};
// One worker per slot, created on first use and kept for the life of the process (threads parked
// on a condition variable); slot i serves the (i+1)-th device of a group.
// The workers are never destroyed: a parked thread must not see its mutex go away at process exit.
Worker& worker(size_t i) {
  static std::vector<Worker*>* workers = new std::vector<Worker*>();
  while (workers->size() <= i) {
    Worker* w = new Worker();
    workers->push_back(w);
    w->th = std::thread([w] { w->loop(); });
    w->th.detach();
  }
  return *(*workers)[i];
}

// Runs job(rank, lo, hi) for every part of [0, n): parts 1.. on worker threads, part 0 on the calling
// thread, then joins them all.  The first failure (lowest rank) becomes this thread's status; every
// part runs to its end either way, so no work is left in flight behind an error.
int run_parts(int n, int parts, const std::function<int(int, int, int)>& job) {
  if (parts > n) parts = n;
  if (parts < 1) parts = 1;
  for (int r = 1; r < parts; ++r) {
    int lo, hi;
    shard_range(n, r, parts, &lo, &hi);
    worker((size_t)r - 1).submit([=, &job] { return job(r, lo, hi); });
  }
  int lo0, hi0;
  shard_range(n, 0, parts, &lo0, &hi0);
  int rc0 = job(0, lo0, hi0);
  std::string msg0 = rc0 ? g_msg : "";
  int first_rc = rc0, first_rank = 0;
  std::string first_msg = msg0;
  for (int r = 1; r < parts; ++r) {
    std::string m;
    const int rc = worker((size_t)r - 1).wait(&m);
    if (rc && !first_rc) { first_rc = rc; first_rank = r; first_msg = m; }
  }
  if (first_rc) return fail(first_rc, "part %d of %d: %s", first_rank, parts, first_msg.c_str());
  return NNCV_B200_OK;
}

int forward_fanout(const char* sp, char* dp, size_t dst_stride, int N, int H, int W) {
  Device& primary = g_dev;
  const std::vector<int> group = primary.group;
  const size_t ew = primary.model->ele_width;
  const size_t img_bytes = (size_t)3 * H * W * ew;
  auto job = [&, sp, dp](int rank, int lo, int hi) -> int {
    if (hi <= lo) return (int)NNCV_B200_OK;
    if (cudaSetDevice(group[(size_t)rank]) != cudaSuccess) return fail(NNCV_B200_ECUDA, "cudaSetDevice(%d) failed", group[(size_t)rank]);
    int rc = device_init();
    if (rc) return rc;
    if (!g_dev.model) return fail(NNCV_B200_ENOMODEL, "device %d holds no replica of the model", g_dev.id);
    cudaStream_t st = (rank == 0 && g_dev.user_stream_set) ? g_dev.user_stream : g_dev.stream;
    return forward_slice(*g_dev.model, sp + (size_t)lo * img_bytes, false, dp + (size_t)lo * dst_stride * ew, false, dst_stride,
                         hi - lo, H, W, st, false);
  };
  const int rc = run_parts(N, (int)group.size(), job);
  cudaSetDevice(primary.id);
  t_dev = &primary;
  return rc;
}

// "resnet18" / "resnet50": the built-in plans; "plan:<text>": a plan given inline; anything else:
// the path of a plan file (what nncv_b200.mlir_import writes from a torch-mlir linalg module).
int plan_from_name(const char* net, Plan* out) {
  if (!net || !*net) return fail(NNCV_B200_EINVAL, "net is null or empty");
  if (!strcmp(net, "resnet18")) { *out = builtin_plan(18); return NNCV_B200_OK; }
  if (!strcmp(net, "resnet50")) { *out = builtin_plan(50); return NNCV_B200_OK; }
  std::string text;
  if (!strncmp(net, "plan:", 5)) {
    text = net + 5;
  } else {
    std::ifstream f(net, std::ifstream::binary);
    if (!f.good())
      return fail(NNCV_B200_EINVAL, "net must be \"resnet18\", \"resnet50\", \"plan:<text>\" or the path of a plan file (cannot open %s)", net);
    text.assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
  }
  return parse_plan(text, out);
}

// Builds the model on the current device, or -- opts->device_mask set -- a replica on every listed
// device (the current one must be among them and serves the first slice of every batch).
int load_group(const Plan& plan, const void* blob, size_t n_elements, size_t ew, const nncv_b200_opts* opts) {
  const unsigned mask = opts ? opts->device_mask : 0u;
  int rc = device_init();
  if (rc) return rc;
  Device* primary = t_dev;
  // replicas of an earlier multi-device load go away with the model they belong to
  for (int d : std::vector<int>(primary->group)) {
    if (d == primary->id || d < 0 || d >= kMaxDevices || !g_devices[d]) continue;
    if (cudaSetDevice(d) == cudaSuccess) {
      cudaDeviceSynchronize();
      t_dev = g_devices[d];
      model_reset();
    }
  }
  cudaSetDevice(primary->id);
  t_dev = primary;
  primary->group.clear();
  model_reset();
  if (mask == 0 || mask == (1u << primary->id)) return model_build(plan, blob, n_elements, ew, opts);
  if (!(mask & (1u << primary->id)))
    return fail(NNCV_B200_EINVAL, "device_mask 0x%x does not include the current device %d", mask, primary->id);
  int count = 0;
  cudaGetDeviceCount(&count);
  std::vector<int> group{primary->id};
  for (int d = 0; d < 32; ++d)
    if ((mask & (1u << d)) && d != primary->id) {
      if (d >= count) return fail(NNCV_B200_EINVAL, "device_mask 0x%x names device %d, this process sees %d", mask, d, count);
      group.push_back(d);
    }
  for (int d : group) {
    if (cudaSetDevice(d) != cudaSuccess) { rc = fail(NNCV_B200_ECUDA, "cudaSetDevice(%d) failed", d); break; }
    if ((rc = device_init())) break;
    model_reset();
    if ((rc = model_build(plan, blob, n_elements, ew, opts))) break;
  }
  cudaSetDevice(primary->id);
  t_dev = primary;
  if (rc) return rc;
  primary->group = group;
  return ok();
}

}  // namespace

// =====================================================================================
// container reader / writer
// =====================================================================================
struct nncv_flat_array {
  nncv_memref_magic_head head;
  std::vector<nncv_memref_indexer> idx;
  std::vector<char> data;
  std::vector<size_t> offs;  // byte offset of each tensor inside `data`
  nncv_memref1 wrapped;
};

namespace {
size_t indexer_elems(const nncv_memref_indexer& i) {
  size_t n = 1;
  for (size_t d = 0; d < i.dims && d < 8; ++d) n *= i.shape[d];
  return n;
}
}  // namespace

extern "C" {

nncv_flat_array* nncv_flat_array_read(const char* path) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if (!path) { fail(NNCV_B200_EINVAL, "path is null"); return nullptr; }
  std::ifstream f(path, std::ifstream::binary);
  if (!f.good()) { fail(NNCV_B200_EIO, "cannot open %s", path); return nullptr; }
  f.seekg(0, std::ios::end);
  const size_t fsize = (size_t)f.tellg();
  f.seekg(0);
  auto a = std::make_unique<nncv_flat_array>();
  if (fsize < sizeof(a->head) || !f.read((char*)&a->head, sizeof(a->head))) {
    fail(NNCV_B200_EIO, "%s: shorter than the magic head", path);
    return nullptr;
  }
  if (a->head.magicNumber != 0x42) { fail(NNCV_B200_EIO, "%s: bad magic number", path); return nullptr; }
  const size_t n = a->head.numMemRefIndex, start = a->head.memRefIndexStartOffset;
  if (start < sizeof(a->head) || start > fsize || n > (fsize - start) / sizeof(nncv_memref_indexer)) {
    fail(NNCV_B200_EIO, "%s: indexer table runs past the end of the file", path);
    return nullptr;
  }
  f.seekg((std::streamoff)start);
  a->idx.resize(n);
  if (n && !f.read((char*)a->idx.data(), (std::streamsize)(n * sizeof(nncv_memref_indexer)))) {
    fail(NNCV_B200_EIO, "%s: truncated indexer table", path);
    return nullptr;
  }
  size_t total = 0, elems = 0;
  const size_t budget = fsize - start - n * sizeof(nncv_memref_indexer);
  for (auto& i : a->idx) {
    if (i.dims > 8 || (i.eleWidth != 2 && i.eleWidth != 4) || i.eleWidth != a->idx[0].eleWidth) {
      fail(NNCV_B200_EIO, "%s: unsupported indexer (dims %zu, eleWidth %zu)", path, i.dims, i.eleWidth);
      return nullptr;
    }
    const size_t e = indexer_elems(i);
    if (e > budget || total + e * i.eleWidth > budget) {
      fail(NNCV_B200_EIO, "%s: tensor data runs past the end of the file", path);
      return nullptr;
    }
    a->offs.push_back(total);
    total += e * i.eleWidth;
    elems += e;
  }
  a->data.resize(total);
  if (total && !f.read(a->data.data(), (std::streamsize)total)) {
    fail(NNCV_B200_EIO, "%s: truncated tensor data", path);
    return nullptr;
  }
  a->wrapped.allocated = a->wrapped.aligned = a->data.data();
  a->wrapped.offset = 0;
  a->wrapped.sizes[0] = (intptr_t)elems;
  a->wrapped.strides[0] = 1;
  ok();
  return a.release();
}

void nncv_flat_array_free(nncv_flat_array* a) { delete a; }
size_t nncv_flat_array_count(const nncv_flat_array* a) { return a ? a->idx.size() : 0; }
const nncv_memref_indexer* nncv_flat_array_indexer(const nncv_flat_array* a, size_t i) {
  return (a && i < a->idx.size()) ? &a->idx[i] : nullptr;
}
const void* nncv_flat_array_data(const nncv_flat_array* a, size_t i) {
  return (a && i < a->idx.size()) ? a->data.data() + a->offs[i] : nullptr;
}
nncv_memref1* nncv_flat_array_wrapped(nncv_flat_array* a) { return a ? &a->wrapped : nullptr; }

int nncv_flat_array_write(const char* path, size_t n, const nncv_memref_indexer* indexers,
                          const void* const* data) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if (!path || (n && (!indexers || !data))) return fail(NNCV_B200_EINVAL, "null argument");
  std::ofstream out(path, std::ofstream::binary);
  if (!out.good()) return fail(NNCV_B200_EIO, "cannot create %s", path);
  nncv_memref_magic_head head;
  head.magicNumber = 0x42;
  head.memRefIndexStartOffset = sizeof(head);
  head.numMemRefIndex = n;
  out.write((const char*)&head, sizeof(head));
  size_t off = sizeof(head) + n * sizeof(nncv_memref_indexer);
  for (size_t i = 0; i < n; ++i) {
    nncv_memref_indexer idx = indexers[i];
    if (idx.dims > 8) return fail(NNCV_B200_EINVAL, "tensor %zu has rank %zu > 8", i, idx.dims);
    idx.dataOffset = off;
    out.write((const char*)&idx, sizeof(idx));
    off += indexer_elems(idx) * idx.eleWidth;
  }
  for (size_t i = 0; i < n; ++i)
    out.write((const char*)data[i], (std::streamsize)(indexer_elems(indexers[i]) * indexers[i].eleWidth));
  out.close();
  if (!out.good()) return fail(NNCV_B200_EIO, "write to %s failed", path);
  return ok();
}

// =====================================================================================
// model API
// =====================================================================================
int nncv_b200_load(const char* net, const char* model_bin_path, const nncv_b200_opts* opts) {
  Plan plan;
  {
    std::lock_guard<std::mutex> lk(g_mutex);
    int rc = plan_from_name(net, &plan);
    if (rc) return rc;
  }
  nncv_flat_array* a = nncv_flat_array_read(model_bin_path);
  if (!a) return g_status;
  std::lock_guard<std::mutex> lk(g_mutex);
  std::unique_ptr<nncv_flat_array> hold(a);
  // every parameter the plan names must start at a tensor of the file and have that tensor's size
  // (element offset of tensor i = sum of the element counts before it, SplitParamsFlatArray.cpp:48-56)
  std::map<size_t, size_t> at_off;   // element offset -> tensor index
  {
    size_t off = 0;
    for (size_t i = 0; i < a->idx.size(); ++i) {
      at_off.emplace(off, i);
      off += indexer_elems(a->idx[i]);
    }
    if (off != plan.total)
      return fail(NNCV_B200_EINVAL, "%s holds %zu elements, %s needs %zu", model_bin_path, off, plan.name.c_str(), plan.total);
  }
  auto tensor_at = [&](size_t off, size_t elems, const char* what, const PlanNode& n) -> const nncv_memref_indexer* {
    auto it = at_off.find(off);
    if (it == at_off.end() || indexer_elems(a->idx[it->second]) != elems) {
      fail(NNCV_B200_EINVAL, "the %s of node %d (offset %zu, %zu elements) is not a tensor of %s", what, n.id, off, elems,
           model_bin_path);
      return nullptr;
    }
    return &a->idx[it->second];
  };
  for (const PlanNode& n : plan.nodes) {
    if (n.kind == PlanNode::kConv) {
      const nncv_memref_indexer* w = tensor_at(n.off_w, (size_t)n.cout * n.cin * n.k * n.k, "conv weight", n);
      if (!w) return g_status;
      if (w->dims != 4 || (int)w->shape[0] != n.cout || (int)w->shape[1] != n.cin || (int)w->shape[2] != n.k || (int)w->shape[3] != n.k)
        return fail(NNCV_B200_EINVAL, "tensor %s is not the %dx%dx%dx%d conv weight the plan expects", w->name, n.cout, n.cin, n.k, n.k);
      if (n.has_bn)
        for (size_t off : {n.off_gamma, n.off_beta, n.off_mean, n.off_var})
          if (!tensor_at(off, (size_t)n.cout, "batch-norm vector", n)) return g_status;
    } else if (n.kind == PlanNode::kFc) {
      if (!tensor_at(n.off_w, (size_t)n.cout * n.cin, "FC weight", n) || !tensor_at(n.off_b, (size_t)n.cout, "FC bias", n))
        return g_status;
    }
  }
  const size_t ew = a->idx[0].eleWidth;
  return load_group(plan, a->data.data(), (size_t)a->wrapped.sizes[0], ew, opts);
}

long long nncv_b200_plan_text(const char* net, char* buf, size_t cap) {
  std::lock_guard<std::mutex> lk(g_mutex);
  Plan plan;
  if (plan_from_name(net, &plan)) return -1;
  std::string t = "nncv_b200_plan 1\nparams " + std::to_string(plan.total) + " out " + std::to_string(plan.out_features) + "\n";
  char line[512];
  for (const PlanNode& n : plan.nodes) {
    if (n.kind == PlanNode::kConv) {
      snprintf(line, sizeof(line), "conv id=%d in=%d res=%d cin=%d cout=%d k=%d stride=%d pad=%d relu=%d w=%zu", n.id, n.in, n.res,
               n.cin, n.cout, n.k, n.stride, n.pad, n.relu, n.off_w);
      t += line;
      if (n.act > kActRelu) {
        snprintf(line, sizeof(line), " act=%d", n.act);
        t += line;
      }
      if (n.has_bn) {
        snprintf(line, sizeof(line), " gamma=%zu beta=%zu mean=%zu var=%zu", n.off_gamma, n.off_beta, n.off_mean, n.off_var);
        t += line;
      } else if (n.has_bias) {
        snprintf(line, sizeof(line), " b=%zu", n.off_b);
        t += line;
      }
    } else if (n.kind == PlanNode::kDwConv) {
      snprintf(line, sizeof(line), "dwconv id=%d in=%d c=%d k=%d stride=%d pad=%d act=%d w=%zu gamma=%zu beta=%zu mean=%zu var=%zu",
               n.id, n.in, n.cin, n.k, n.stride, n.pad, n.act, n.off_w, n.off_gamma, n.off_beta, n.off_mean, n.off_var);
      t += line;
    } else if (n.kind == PlanNode::kSe) {
      snprintf(line, sizeof(line), "se id=%d in=%d c=%d cr=%d w1=%zu b1=%zu w2=%zu b2=%zu", n.id, n.in, n.cin, n.cr, n.off_w, n.off_b,
               n.off_w2, n.off_b2);
      t += line;
    } else if (n.kind == PlanNode::kMaxPool) {
      snprintf(line, sizeof(line), "maxpool id=%d in=%d k=%d stride=%d pad=%d", n.id, n.in, n.k, n.stride, n.pad);
      t += line;
    } else if (n.kind == PlanNode::kAvgPool) {
      snprintf(line, sizeof(line), "avgpool id=%d in=%d", n.id, n.in);
      t += line;
    } else {
      snprintf(line, sizeof(line), "fc id=%d in=%d cin=%d cout=%d w=%zu b=%zu", n.id, n.in, n.cin, n.cout, n.off_w, n.off_b);
      t += line;
      if (n.act) {
        snprintf(line, sizeof(line), " act=%d", n.act);
        t += line;
      }
    }
    if ((n.kind == PlanNode::kConv || n.kind == PlanNode::kDwConv) && n.has_bn && fabsf(n.eps - 1e-5f) > 1e-9f) {
      uint32_t bits;
      memcpy(&bits, &n.eps, 4);
      snprintf(line, sizeof(line), " eps_bits=%u", bits);
      t += line;
    }
    t += "\n";
  }
  if (buf && cap) {
    const size_t k = t.size() < cap - 1 ? t.size() : cap - 1;
    memcpy(buf, t.data(), k);
    buf[k] = 0;
  }
  ok();
  return (long long)t.size();
}

int nncv_b200_plan_check(const char* net, size_t* n_params, int* n_nodes, int* out_features) {
  std::lock_guard<std::mutex> lk(g_mutex);
  Plan plan;
  int rc = plan_from_name(net, &plan);
  if (rc) return rc;
  if ((rc = finalize_plan(plan, true))) return rc;
  if (n_params) *n_params = plan.total;
  if (n_nodes) *n_nodes = (int)plan.nodes.size();
  if (out_features) *out_features = plan.out_features;
  return ok();
}

int nncv_b200_load_blob(const char* net, const void* blob, size_t n_elements, size_t ele_width,
                        const nncv_b200_opts* opts) {
  std::lock_guard<std::mutex> lk(g_mutex);
  Plan plan;
  int rc = plan_from_name(net, &plan);
  if (rc) return rc;
  if (!blob) return fail(NNCV_B200_EINVAL, "blob is null");
  return load_group(plan, blob, n_elements, ele_width, opts);
}

int nncv_b200_unload(void) {
  std::lock_guard<std::mutex> lk(g_mutex);
  t_dev = current_device_or_null();
  if (t_dev) {
    Device* primary = t_dev;
    for (int d : std::vector<int>(primary->group)) {   // replicas on the other devices of a multi-device load
      if (d == primary->id || d < 0 || d >= kMaxDevices || !g_devices[d]) continue;
      if (cudaSetDevice(d) == cudaSuccess) {
        cudaDeviceSynchronize();
        t_dev = g_devices[d];
        model_reset();
      }
    }
    cudaSetDevice(primary->id);
    t_dev = primary;
    primary->group.clear();
    cudaDeviceSynchronize();
    model_reset();
  }
  return ok();
}

void _mlir_ciface_forward(nncv_memref2* dst, nncv_memref4* src, void* params) {
  std::lock_guard<std::mutex> lk(g_mutex);
  forward_impl(dst, src, params, nullptr, false);
}

int nncv_b200_forward_device(nncv_memref2* dst, nncv_memref4* src, void* cuda_stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!g_dev.model) return fail(NNCV_B200_ENOMODEL, "no model loaded on device %d", g_dev.id);
  return forward_impl(dst, src, nullptr, (cudaStream_t)cuda_stream, true);
}

int nncv_b200_set_stream(void* cuda_stream, int enable) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  g_dev.user_stream = (cudaStream_t)cuda_stream;
  g_dev.user_stream_set = enable != 0;
  return ok();
}

int nncv_b200_profile(int enable) {
  std::lock_guard<std::mutex> lk(g_mutex);
  Device* pd = current_device_or_null();
  if (pd) cudaDeviceSynchronize();
  prof_clear();
  g_prof_dev = pd ? pd->id : 0;
  g_prof_on = enable != 0;
  return ok();
}

long long nncv_b200_profile_count(void) {
  std::lock_guard<std::mutex> lk(g_mutex);
  return (long long)g_prof.size();
}

int nncv_b200_profile_get(long long i, nncv_b200_prof_rec* out) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if (!out || i < 0 || i >= (long long)g_prof.size()) return fail(NNCV_B200_EINVAL, "profile_get: bad index");
  ProfRec& r = g_prof[(size_t)i];
  if (r.ms < 0) {
    CU(cudaEventSynchronize(r.e1));
    CU(cudaEventElapsedTime(&r.ms, r.e0, r.e1));
  }
  out->kind = r.kind; out->M = r.M; out->N = r.N; out->K = r.K; out->bn = r.bn;
  out->flops = r.flops; out->bytes = r.bytes; out->ms = r.ms;
  return ok();
}

int nncv_b200_arena_plan(size_t n, const int* first_op, const int* last_op, const size_t* size, size_t align,
                         size_t* offset_out, size_t* total_out) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if ((n && (!first_op || !last_op || !size || !offset_out)) || !total_out)
    return fail(NNCV_B200_EINVAL, "arena_plan: null argument");
  std::vector<ArenaTensor> ts(n);
  for (size_t i = 0; i < n; ++i) {
    if (first_op[i] > last_op[i]) return fail(NNCV_B200_EINVAL, "arena_plan: tensor %zu ends before it starts", i);
    ts[i].first = first_op[i]; ts[i].last = last_op[i]; ts[i].size = size[i];
  }
  *total_out = arena_plan(ts, align);
  for (size_t i = 0; i < n; ++i) offset_out[i] = ts[i].offset;
  return ok();
}

int nncv_b200_activation_bytes(size_t* arena_bytes, size_t* unshared_bytes) {
  std::lock_guard<std::mutex> lk(g_mutex);
  Device* d = current_device_or_null();
  if (!d || !d->model || !d->model->planned) return fail(NNCV_B200_ENOMODEL, "no forward has run on this device yet");
  if (arena_bytes) *arena_bytes = d->model->arena.bytes;
  if (unshared_bytes) *unshared_bytes = d->model->act_bytes_unshared;
  return ok();
}

int nncv_b200_shard_range(int n, int rank, int world, int* lo, int* hi) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if (n < 0 || world <= 0 || rank < 0 || rank >= world || !lo || !hi) return fail(NNCV_B200_EINVAL, "shard_range: bad argument");
  shard_range(n, rank, world, lo, hi);
  return ok();
}

int nncv_b200_selftest_fanout(int n, int parts, int fail_rank, int* lo_out, int* hi_out, int* thread_differs) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if (n < 0 || parts < 1 || parts > 64 || !lo_out || !hi_out) return fail(NNCV_B200_EINVAL, "selftest_fanout: bad argument");
  for (int i = 0; i < parts; ++i) lo_out[i] = hi_out[i] = -1;
  const std::thread::id me = std::this_thread::get_id();
  std::atomic<int> others{0};
  auto job = [&](int rank, int lo, int hi) -> int {
    lo_out[rank] = lo;
    hi_out[rank] = hi;
    if (std::this_thread::get_id() != me) ++others;
    if (rank == fail_rank) return fail(NNCV_B200_ETIMEOUT, "injected failure on part %d", rank);
    return (int)NNCV_B200_OK;
  };
  const int rc = run_parts(n, parts, job);
  if (thread_differs) *thread_differs = others.load();
  return rc ? rc : ok();
}

int nncv_b200_device_status(void) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  int flag = 0;
  if ((rc = read_kernel_status(&flag))) return rc;
  if (flag) return report_kernel_error(flag, "device status");
  if (noalloc_read_status(g_dev.id, &flag) != 0)
    return fail(NNCV_B200_ECUDA, "device status: reading the status word of the fixed scratch array failed");
  if (flag) return report_kernel_error(flag, "device status (nncv_b200_matmul_noalloc)");
  return ok();
}

int nncv_b200_selftest_wait_timeout(int log2_clocks, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (log2_clocks < 0 || log2_clocks > 24) return fail(NNCV_B200_EINVAL, "selftest: log2_clocks must be in [0, 24]");
  LAUNCH(launch_wait_selftest(g_dev.error_flag, 1LL << log2_clocks, (cudaStream_t)stream));
  return ok();
}

int nncv_b200_last_status(void) { return g_status; }
const char* nncv_b200_last_error(void) { return g_msg; }
long long nncv_b200_launch_count(void) { return g_launches; }

// =====================================================================================
// single kernels
// =====================================================================================
int nncv_b200_matmul(const void* A, const void* B, void* C, int M, int N, int K, int ab_dtype,
                     int c_dtype, const float* bias, int relu, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return fail(NNCV_B200_EINVAL, "matmul: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  if (ab_dtype == NNCV_B200_F32) {
    if (c_dtype != NNCV_B200_F32 || K % 4 != 0) return fail(NNCV_B200_EINVAL, "fp32 matmul needs fp32 C and K %% 4 == 0");
    if (!g_force_gather && gemm_tf32x3_supported(M, N, K) && !(reinterpret_cast<uintptr_t>(A) & 15) &&
        !(reinterpret_cast<uintptr_t>(B) & 15) && !(reinterpret_cast<uintptr_t>(C) & 15)) {
      // tensor cores, three tf32 products per k step: fp32-level accuracy, no scratch
      LAUNCH(launch_gemm_tf32x3((const float*)A, (const float*)B, (float*)C, M, N, K, bias, relu, g_dev.sm_count, g_dev.error_flag, st));
      return ok();
    }
    if ((rc = ensure_scratch((size_t)N * K * sizeof(float)))) return rc;
    LAUNCH(launch_repack_weights_f32(B, kF32, 1, N, 0, N, K, K, 1, (float*)g_dev.scratch, st));
    SimtConvArgs a;
    a.in = (const float*)A; a.w = (const float*)g_dev.scratch; a.shift = bias; a.out = (float*)C;
    a.N = M; a.H = a.W = a.OH = a.OW = 1; a.C = K; a.Kout = N; a.ldo = N; a.relu = relu;
    LAUNCH(launch_conv_simt_f32(a, st));
    return ok();
  }
  if (ab_dtype != NNCV_B200_F16 && ab_dtype != NNCV_B200_BF16) return fail(NNCV_B200_EINVAL, "matmul: bad ab_dtype");
  if (c_dtype != NNCV_B200_F32 && c_dtype != ab_dtype) return fail(NNCV_B200_EINVAL, "matmul: c_dtype must be F32 or ab_dtype");
  if (K % 8 != 0) return fail(NNCV_B200_EINVAL, "matmul: the tcgen05 path needs K %% 8 == 0");
  if (N % 8 == 0 && N >= 64 && K >= 64 && !g_force_gather && !(reinterpret_cast<uintptr_t>(B) & 15) && !(reinterpret_cast<uintptr_t>(A) & 15) &&
      !(reinterpret_cast<uintptr_t>(C) & 15)) {
    // B as it lies in memory: 64 x 64 boxes of the row-major [K, N] matrix are MN-major operand tiles,
    // so the whole matmul is one kernel and needs no scratch
    int bn = N >= 256 ? 256 : (N > 64 ? 128 : 64);
    const long long mi = ((long long)M + 127) / 128;
    while (bn > 64 && mi * ((N + bn - 1) / bn) < g_dev.sm_count) bn >>= 1;
    TconvArgs a;
    a.in = A; a.b_rowmajor = B; a.b_rows = K; a.shift = bias; a.out = C;
    a.N = 1; a.H = 1; a.W = M; a.OH = 1; a.OW = M; a.C = K; a.Kout = N;
    a.in_l = Layout{1, M, 0}; a.out_l = Layout{1, M, 0};
    a.bn = bn; a.resident = 0; a.ab = (DType)ab_dtype; a.out_dtype = (DType)c_dtype; a.relu = relu;
    a.sm_count = g_dev.sm_count; a.error_flag = g_dev.error_flag;
    LAUNCH(launch_tconv(a, st));
    return ok();
  }
  if (K % 64 == 0 && tconv_supported(K, N, (DType)c_dtype, N) && N >= 64) {
    int bn, resident;
    tconv_pick((M + 127) / 128, K, N, 1, &bn, &resident);
    if ((rc = ensure_scratch(packed_weight_bytes(N, K, 1, 1, bn)))) return rc;
    LAUNCH(launch_pack_weights(B, (DType)ab_dtype, 1, N, 0, N, K, K, 1, bn, (DType)ab_dtype, g_dev.scratch, st));
    TconvArgs a;
    a.in = A; a.wpack = g_dev.scratch; a.shift = bias; a.out = C;
    a.N = 1; a.H = 1; a.W = M; a.OH = 1; a.OW = M; a.C = K; a.Kout = N;
    a.in_l = Layout{1, M, 0}; a.out_l = Layout{1, M, 0};
    a.bn = bn; a.resident = resident; a.ab = (DType)ab_dtype; a.out_dtype = (DType)c_dtype; a.relu = relu;
    a.sm_count = g_dev.sm_count; a.error_flag = g_dev.error_flag;
    LAUNCH(launch_tconv(a, st));
    return ok();
  }
  const int bn = igemm_pick_bn(M, N);
  if ((rc = ensure_scratch(packed_weight_bytes(N, K, 1, 1, bn)))) return rc;
  LAUNCH(launch_pack_weights(B, (DType)ab_dtype, 1, N, 0, N, K, K, 1, bn, (DType)ab_dtype, g_dev.scratch, st));
  IgemmArgs a;
  a.in = A; a.wpack = g_dev.scratch; a.shift = bias; a.out = C;
  a.N = M; a.H = a.W = a.OH = a.OW = 1; a.C = K; a.Kout = N; a.ldo = N; a.bn = bn;
  a.ab = (DType)ab_dtype; a.out_dtype = (DType)c_dtype; a.relu = relu; a.error_flag = g_dev.error_flag;
  LAUNCH(launch_conv_igemm(a, st));
  return ok();
}

nncv_b200_conv* nncv_b200_conv_create(const void* weights, int w_dtype, int Kout, int C, int R,
                                      int S, int stride, int pad, int dtype, int algo) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if (device_init()) return nullptr;
  if (!weights || Kout <= 0 || C <= 0 || R <= 0 || S <= 0 || stride <= 0 || pad < 0 || w_dtype < 0 ||
      w_dtype > 2 || dtype < 0 || dtype > 2) {
    fail(NNCV_B200_EINVAL, "conv_create: bad argument");
    return nullptr;
  }
  if (algo < 0 || algo > 3) {
    fail(NNCV_B200_EINVAL, "conv_create: algo %d is not available", algo);
    return nullptr;
  }
  if ((algo == 2 || algo == 1) && (dtype == NNCV_B200_F32 || !conv3x3_supported(C, Kout, R, S, stride, pad))) {
    fail(NNCV_B200_EINVAL, "conv_create: algo 1 and 2 need a 16-bit 3x3 stride-1 pad-1 conv with C, Kout %% 64 == 0");
    return nullptr;
  }
  auto c = std::make_unique<nncv_b200_conv>();
  c->Kout = Kout; c->C = C; c->R = R; c->S = S; c->stride = stride; c->pad = pad; c->device = g_dev.id;
  c->dtype = (DType)dtype; c->algo = algo == 3 ? 0 : algo; c->force_gather = algo == 3;
  c->Cpad = dtype == NNCV_B200_F32 ? (C + 3) / 4 * 4 : (C + 7) / 8 * 8;
  const size_t bytes = (size_t)Kout * C * R * S * dtype_size((DType)w_dtype);
  if (c->raw_owned.reserve(bytes)) return nullptr;
  if (cudaMemcpy(c->raw_owned.p, weights, bytes, cudaMemcpyDefault) != cudaSuccess) {
    fail(NNCV_B200_ECUDA, "conv_create: copying the weights failed");
    return nullptr;
  }
  c->raw = c->raw_owned.p; c->raw_dt = (DType)w_dtype;
  c->sn = (long long)C * R * S; c->sc = (long long)R * S; c->stap = 1;
  ok();
  return c.release();
}

void nncv_b200_conv_destroy(nncv_b200_conv* c) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if (c && current_device_or_null()) cudaDeviceSynchronize();
  delete c;
}

int nncv_b200_conv_run(nncv_b200_conv* c, const void* in, void* out, int N, int H, int W,
                       const float* scale, const float* shift, const void* residual, int relu,
                       void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if (!c || !in || !out) return fail(NNCV_B200_EINVAL, "conv_run: null argument");
  cudaStream_t st = (cudaStream_t)stream;
  int rc = device_init();
  if (rc) return rc;
  if (c->device != g_dev.id)
    return fail(NNCV_B200_EINVAL, "conv_run: the plan lives on device %d, the current device is %d", c->device, g_dev.id);
  if (c->algo == 2) {
    // The kernel works on shared-pad NHWC; this entry point takes dense NHWC, so convert on both
    // sides (the network executor keeps its activations in shared-pad form and skips this).
    const Layout dl = dense_layout(H, W), sl = sp_layout(H, W);
    const size_t es = dtype_size(c->dtype);
    const size_t slots = (size_t)layout_slots(sl, N);
    if ((rc = c->sp_in.reserve(slots * c->Cpad * es))) return rc;
    if ((rc = c->sp_out.reserve(slots * c->Kout * es))) return rc;
    LAUNCH(launch_relayout(in, dl, c->sp_in.p, sl, c->dtype, N, H, W, c->Cpad, st));
    const void* res = nullptr;
    if (residual) {
      if ((rc = c->sp_res.reserve(slots * c->Kout * es))) return rc;
      LAUNCH(launch_relayout(residual, dl, c->sp_res.p, sl, c->dtype, N, H, W, c->Kout, st));
      res = c->sp_res.p;
    }
    rc = conv_run(c, c->sp_in.p, sl, c->sp_out.p, sl, N, H, W, scale, shift, res, relu, c->dtype, c->Kout, st);
    if (rc) return rc;
    LAUNCH(launch_relayout(c->sp_out.p, sl, out, dl, c->dtype, N, H, W, c->Kout, st));
    return ok();
  }
  if (c->algo == 1) {
    // Winograd F(2x2,3x3): input transform -> 16 GEMMs [tiles x C] * [C x Kout] -> output transform
    const size_t es = dtype_size(c->dtype);
    const long long T = (long long)N * ((H + 1) / 2) * ((W + 1) / 2);
    if (T > 0x7fffffffLL) return fail(NNCV_B200_EINVAL, "winograd: too many tiles");
    if (c->wino_w.empty()) {
      if ((rc = c->wino_U.reserve((size_t)16 * c->Kout * c->Cpad * es))) return rc;
      LAUNCH(launch_wino_filter(c->raw, c->raw_dt, c->sn, c->sc, c->stap, c->Kout, c->C, c->wino_U.p, c->dtype, st));
      tconv_pick((T + 127) / 128, c->Cpad, c->Kout, 1, &c->wino_bn, &c->wino_resident);
      for (int p = 0; p < 16; ++p) {
        auto b = std::make_unique<DevBuf>();
        if ((rc = b->reserve(packed_weight_bytes(c->Kout, c->Cpad, 1, 1, c->wino_bn)))) return rc;
        LAUNCH(launch_pack_weights((const char*)c->wino_U.p + (size_t)p * c->Kout * c->Cpad * es, c->dtype, c->Cpad, 1, 0,
                                   c->Kout, c->Cpad, c->Cpad, 1, c->wino_bn, c->dtype, b->p, st));
        c->wino_w.push_back(std::move(b));
      }
    }
    if ((rc = c->wino_V.reserve((size_t)16 * T * c->Cpad * es))) return rc;
    if ((rc = c->wino_M.reserve((size_t)16 * T * c->Kout * sizeof(float)))) return rc;
    const double flops = 2.0 * N * H * W * (double)c->Kout * c->C * 9.0;
    prof_begin(6, flops, 2.0 * ((double)N * H * W * (c->C + c->Kout * (residual ? 2 : 1)) + 9.0 * c->Kout * c->C), (int)T,
               c->Kout, c->C, c->wino_bn, st);
    LAUNCH(launch_wino_input(in, c->wino_V.p, c->dtype, N, H, W, c->Cpad, st));
    for (int p = 0; p < 16; ++p) {
      TconvArgs a;
      a.in = (const char*)c->wino_V.p + (size_t)p * T * c->Cpad * es;
      a.wpack = c->wino_w[p]->p;
      a.out = (float*)c->wino_M.p + (size_t)p * T * c->Kout;
      a.N = 1; a.H = 1; a.W = (int)T; a.OH = 1; a.OW = (int)T; a.C = c->Cpad; a.Kout = c->Kout;
      a.in_l = Layout{1, (int)T, 0}; a.out_l = Layout{1, (int)T, 0};
      a.bn = c->wino_bn; a.resident = c->wino_resident; a.ab = c->dtype; a.out_dtype = kF32;
      a.sm_count = g_dev.sm_count; a.error_flag = g_dev.error_flag;
      LAUNCH(launch_tconv(a, st));
    }
    LAUNCH(launch_wino_output((const float*)c->wino_M.p, scale, shift, residual, out, c->dtype, N, H, W, c->Kout, relu, st));
    prof_end(st);
    return ok();
  }
  rc = conv_run(c, in, Layout{0, 0, 0}, out, Layout{0, 0, 0}, N, H, W, scale, shift, residual, relu, c->dtype,
                c->Kout, st);
  return rc ? rc : ok();
}

int nncv_b200_conv_run_fused(nncv_b200_conv* c, nncv_b200_conv* branch, const void* in, void* out, void* out_branch,
                             int N, int H, int W, const float* scale, const float* shift, const float* scale_branch,
                             const float* shift_branch, int relu, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!c || !branch || !in || !out || !out_branch) return fail(NNCV_B200_EINVAL, "conv_run_fused: null argument");
  if (N <= 0 || H <= 0 || W <= 0) return fail(NNCV_B200_EINVAL, "conv_run_fused: bad shape");
  if (c->device != g_dev.id || branch->device != g_dev.id)
    return fail(NNCV_B200_EINVAL, "conv_run_fused: the plans live on device %d / %d, the current device is %d", c->device,
                branch->device, g_dev.id);
  if (!fused_branch_ok(*c, *branch))
    return fail(NNCV_B200_EINVAL, "conv_run_fused: needs an odd square filter with pad = R/2 and a 1x1 pad-0 branch of the "
                                  "same stride, channels and (multiple of 128) output channels, 16-bit, algo 0");
  FusedBranch fb{branch, scale_branch, shift_branch, out_branch};
  rc = conv_run(c, in, Layout{0, 0, 0}, out, Layout{0, 0, 0}, N, H, W, scale, shift, nullptr, relu, c->dtype, c->Kout,
                (cudaStream_t)stream, &fb);
  return rc ? rc : ok();
}

int nncv_b200_conv_set_tile(nncv_b200_conv* c, int bn, int mt, int resident) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if (!c) return fail(NNCV_B200_EINVAL, "conv_set_tile: null plan");
  c->cfg3 = Conv3x3Config{bn, mt, resident};
  return ok();
}

int nncv_b200_stem_pool(const void* in_nchw, int in_dtype, const void* weights, int w_dtype,
                        const float* scale, const float* shift, void* out_nhwc, int dtype, int N, int H,
                        int W, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!in_nchw || !weights || !out_nhwc || N <= 0 || H < 7 || W < 7 || (dtype != NNCV_B200_F16 && dtype != NNCV_B200_BF16))
    return fail(NNCV_B200_EINVAL, "stem_pool: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t rows = (stem_rows_bytes(N, H, W) + 255) & ~(size_t)255;
  if ((rc = ensure_scratch(rows + stem_wpack_bytes()))) return rc;
  char* sp = (char*)g_dev.scratch;
  const bool paired = stem_paired_ok(H, W);
  LAUNCH(launch_nchw_to_stem_rows(in_nchw, (DType)in_dtype, sp, (DType)dtype, N, H, W, false, paired, st));
  LAUNCH(launch_pack_stem_weights(weights, (DType)w_dtype, sp + rows, (DType)dtype, st));
  StemArgs a;
  a.in_rows = sp; a.paired = paired; a.wpack = sp + rows; a.scale = scale; a.shift = shift; a.out = out_nhwc;
  a.N = N; a.H = H; a.W = W; a.ab = (DType)dtype; a.sm_count = g_dev.sm_count; a.error_flag = g_dev.error_flag;
  LAUNCH(launch_stem_pool(a, st));
  return ok();
}

int nncv_b200_stem_variant(int policy) {
  std::lock_guard<std::mutex> lk(g_mutex);
  if (policy >= 0) g_stem_force_plain = policy == 1;
  return g_stem_last_variant;
}

int nncv_b200_maxpool_nhwc(const void* in, void* out, int dtype, int N, int H, int W, int C,
                           int k, int stride, int pad, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!in || !out || N <= 0 || k <= 0 || stride <= 0 || dtype < 0 || dtype > 2) return fail(NNCV_B200_EINVAL, "maxpool: bad argument");
  LAUNCH(launch_maxpool_nhwc(in, out, (DType)dtype, N, H, W, C, k, stride, pad, Layout{0, 0, 0}, Layout{0, 0, 0},
                             (cudaStream_t)stream));
  return ok();
}

int nncv_b200_avgpool_nhwc(const void* in, void* out, int dtype, int N, int HW, int C, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!in || !out || N <= 0 || HW <= 0 || dtype < 0 || dtype > 2) return fail(NNCV_B200_EINVAL, "avgpool: bad argument");
  LAUNCH(launch_avgpool_nhwc(in, out, (DType)dtype, N, 1, HW, C, Layout{0, 0, 0}, (cudaStream_t)stream));
  return ok();
}

int nncv_b200_nchw_to_nhwc(const void* in, int in_dtype, void* out, int out_dtype, int N, int C,
                           int H, int W, int Cpad, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!in || !out || N <= 0 || C <= 0 || Cpad < C) return fail(NNCV_B200_EINVAL, "nchw_to_nhwc: bad argument");
  LAUNCH(launch_nchw_to_nhwc(in, (DType)in_dtype, out, (DType)out_dtype, N, C, H, W, Cpad, (cudaStream_t)stream));
  return ok();
}

int nncv_b200_depthwise_conv_nhwc(const void* in, const void* weights, int w_dtype, const float* scale, const float* shift,
                                  void* out, int dtype, int N, int H, int W, int C, int R, int S, int stride, int pad, int act,
                                  void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!in || !weights || !out || N <= 0 || H <= 0 || W <= 0 || C <= 0 || R <= 0 || S <= 0 || stride <= 0 || pad < 0 || dtype < 0 ||
      dtype > 2 || act < 0 || act > 5)
    return fail(NNCV_B200_EINVAL, "depthwise_conv: bad argument");
  if (launch_depthwise(in, weights, (DType)w_dtype, scale, shift, out, (DType)dtype, N, H, W, C, R, S, stride, pad, act,
                       Layout{0, 0, 0}, Layout{0, 0, 0}, g_dev.sm_count, g_dev.error_flag, (cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return fail(NNCV_B200_EINVAL, "depthwise_conv: C must be a multiple of %d, weights fp32 (or fp16 with fp16 activations), output not empty",
                16 / (int)dtype_size((DType)dtype));
  }
  ++g_launches;
  return ok();
}

int nncv_b200_activation(const void* in, void* out, int dtype, size_t n, int act, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!in || !out || dtype < 0 || dtype > 2 || act < 0 || act > 5) return fail(NNCV_B200_EINVAL, "activation: bad argument");
  if (n == 0) return ok();
  if (launch_activation(in, out, (DType)dtype, n, act, (cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return fail(NNCV_B200_EINVAL, "activation: the element count must be a multiple of %d", 16 / (int)dtype_size((DType)dtype));
  }
  ++g_launches;
  return ok();
}

int nncv_b200_se_gate(const void* pooled, const float* w1, const float* b1, const float* w2, const float* b2, void* gate,
                      int dtype, int N, int C, int Cr, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!pooled || !w1 || !w2 || !gate || N <= 0 || C <= 0 || Cr <= 0 || dtype < 0 || dtype > 2)
    return fail(NNCV_B200_EINVAL, "se_gate: bad argument");
  if (launch_se_gate(pooled, w1, b1, w2, b2, gate, (DType)dtype, N, C, Cr, (cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return fail(NNCV_B200_EINVAL, "se_gate: C + Cr must fit 48 KB of shared memory as floats");
  }
  ++g_launches;
  return ok();
}

int nncv_b200_scale_channels_nhwc(const void* in, const void* gate, void* out, int dtype, int N, int HW, int C, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!in || !gate || !out || N <= 0 || HW <= 0 || C <= 0 || dtype < 0 || dtype > 2)
    return fail(NNCV_B200_EINVAL, "scale_channels: bad argument");
  if (launch_scale_channels(in, gate, out, (DType)dtype, N, HW, C, (cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return fail(NNCV_B200_EINVAL, "scale_channels: C must be a multiple of %d", 16 / (int)dtype_size((DType)dtype));
  }
  ++g_launches;
  return ok();
}

int nncv_b200_concat_channels_nhwc(const void* const* inputs, const int* channels, int n_inputs, void* out, int dtype,
                                   long long pixels, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!inputs || !channels || !out || pixels <= 0 || dtype < 0 || dtype > 2) return fail(NNCV_B200_EINVAL, "concat: bad argument");
  if (launch_concat(inputs, channels, n_inputs, out, (DType)dtype, pixels, (cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return fail(NNCV_B200_EINVAL, "concat: 1 to 8 inputs, every channel count a multiple of %d, pointers 16-byte aligned",
                16 / (int)dtype_size((DType)dtype));
  }
  ++g_launches;
  return ok();
}

int nncv_b200_upsample2x_nhwc(const void* in, void* out, int dtype, int N, int H, int W, int C, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!in || !out || N <= 0 || H <= 0 || W <= 0 || C <= 0 || dtype < 0 || dtype > 2) return fail(NNCV_B200_EINVAL, "upsample2x: bad argument");
  if (launch_upsample2x(in, out, (DType)dtype, N, H, W, C, (cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return fail(NNCV_B200_EINVAL, "upsample2x: C must be a multiple of %d", 16 / (int)dtype_size((DType)dtype));
  }
  ++g_launches;
  return ok();
}

int nncv_b200_bn_fold(const void* gamma, const void* beta, const void* mean, const void* var,
                      int dtype, int C, float* scale, float* shift, void* stream) {
  std::lock_guard<std::mutex> lk(g_mutex);
  int rc = device_init();
  if (rc) return rc;
  if (!gamma || !beta || !mean || !var || !scale || !shift || C <= 0) return fail(NNCV_B200_EINVAL, "bn_fold: bad argument");
  LAUNCH(launch_bn_fold(gamma, beta, mean, var, (DType)dtype, C, 1e-5f, scale, shift, (cudaStream_t)stream));
  return ok();
}

}  // extern "C"
