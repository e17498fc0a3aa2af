// nncv_b200_matmul_noalloc: the tensor-core matmul for callers that must not allocate.
//
// nncv_b200_matmul repacks B into a scratch buffer that the library grows with cudaMalloc when a
// larger problem arrives.  Some callers cannot live with that: an inference server that has
// handed every byte of device memory to its own pool (so a later cudaMalloc fails or evicts),
// or a latency-bound loop in which cudaMalloc's implicit device-wide synchronisation would stall
// the other streams of the process.  For them this file keeps the scratch in a fixed array in
// device memory that comes with the library image: nothing is allocated or freed, ever, by this
// entry point.  The price is a size limit and one array per GPU for the life of the process.
//
// This entry point has no counterpart in nncv (the reference never touches a device).
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/nncv_b200.h"
#include "kernels.h"

namespace nncv_b200 {
int internal_fail(int code, const char* fmt, ...);
int internal_ok();
std::mutex& internal_mutex();
}  // namespace nncv_b200

using namespace nncv_b200;

namespace {

// First 256 bytes: the status word the kernels report bounded-wait time-outs into (cleared at the
// start of every call).  The rest: the packed image of B.
constexpr size_t kHeaderBytes = 256;
constexpr size_t kPackBytes = NNCV_B200_NOALLOC_MAX_PACKED_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kHeaderBytes + kPackBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the
// address each device gave its copy is looked up once per device and kept here.
constexpr int kMaxDevices = 64;
unsigned char* g_scratch_ptr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};

// Once per device, with that device current.  Returns 0 or a status code.
int setup_current_device(int* dev_out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return internal_fail(NNCV_B200_ENODEVICE, "matmul_noalloc: no current CUDA device (this library has no CPU fallback)");
  *dev_out = dev;
  if (g_scratch_ptr[dev]) return 0;
  int major = 0, sms = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
    return internal_fail(NNCV_B200_ENODEVICE, "matmul_noalloc: device %d is not sm_100; the kernels are built for sm_100a only", dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return internal_fail(NNCV_B200_ECUDA, "matmul_noalloc: cannot read the SM count of device %d", dev);
  void* ptr = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
  if (e != cudaSuccess || !ptr)
    return internal_fail(NNCV_B200_ECUDA, "matmul_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                         cudaGetErrorString(e));
  g_sm_count[dev] = sms;
  g_scratch_ptr[dev] = static_cast<unsigned char*>(ptr);
  return 0;
}

}  // namespace

namespace nncv_b200 {
// Status word at the head of the static array of device `dev` (0 when this path never ran
// there); read with a 4-byte copy and cleared when non-zero.  Allocates nothing.
int noalloc_read_status(int dev, int* flag) {
  *flag = 0;
  if (dev < 0 || dev >= kMaxDevices || !g_scratch_ptr[dev]) return 0;
  if (cudaMemcpy(flag, g_scratch_ptr[dev], sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (*flag != 0 && cudaMemset(g_scratch_ptr[dev], 0, sizeof(int)) != cudaSuccess) return -1;
  return 0;
}
}  // namespace nncv_b200

extern "C" int nncv_b200_matmul_noalloc(const void* A, const void* B, void* C, int M, int N, int K,
                                        int ab_dtype, int c_dtype, const float* bias, int relu,
                                        void* stream) {
  std::lock_guard<std::mutex> lk(internal_mutex());
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0)
    return internal_fail(NNCV_B200_EINVAL, "matmul_noalloc: bad argument");
  if (ab_dtype != NNCV_B200_F16 && ab_dtype != NNCV_B200_BF16)
    return internal_fail(NNCV_B200_EINVAL, "matmul_noalloc: operands must be F16 or BF16");
  if (c_dtype != NNCV_B200_F32 && c_dtype != ab_dtype)
    return internal_fail(NNCV_B200_EINVAL, "matmul_noalloc: c_dtype must be F32 or ab_dtype");
  if (K % 8 != 0) return internal_fail(NNCV_B200_EINVAL, "matmul_noalloc: K must be a multiple of 8");
  int dev = -1;
  int rc = setup_current_device(&dev);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* base = g_scratch_ptr[dev];
  int* status_word = reinterpret_cast<int*>(base);
  void* packed = base + kHeaderBytes;

  const bool tma = K % 64 == 0 && N >= 64 && tconv_supported(K, N, (DType)c_dtype, N);
  int bn = 64, resident = 0;
  if (tma) tconv_pick((M + 127) / 128, K, N, 1, &bn, &resident);
  else bn = igemm_pick_bn(M, N);
  const size_t need = packed_weight_bytes(N, K, 1, 1, bn);
  if (need > kPackBytes)
    return internal_fail(NNCV_B200_EINVAL,
                         "matmul_noalloc: B packs into %zu bytes, the fixed scratch holds %zu (about N*K <= %zu elements); "
                         "use nncv_b200_matmul for larger problems",
                         need, kPackBytes, kPackBytes / 2);
  // The array still holds whatever the previous call left: the status word must start at zero;
  // the packed image is rewritten in full (padding included) by the pack kernel.
  cudaError_t e = cudaMemsetAsync(status_word, 0, sizeof(int), st);
  if (e != cudaSuccess) return internal_fail(NNCV_B200_ECUDA, "matmul_noalloc: cudaMemsetAsync failed: %s", cudaGetErrorString(e));
  e = launch_pack_weights(B, (DType)ab_dtype, 1, N, 0, N, K, K, 1, bn, (DType)ab_dtype, packed, st);
  if (e != cudaSuccess) return internal_fail(NNCV_B200_ECUDA, "matmul_noalloc: packing B failed: %s", cudaGetErrorString(e));
  if (tma) {
    TconvArgs a;
    a.in = A; a.wpack = packed; a.shift = bias; a.out = C;
    a.N = 1; a.H = 1; a.W = M; a.OH = 1; a.OW = M; a.C = K; a.Kout = N;
    a.in_l = Layout{1, M, 0}; a.out_l = Layout{1, M, 0};
    a.bn = bn; a.resident = resident; a.ab = (DType)ab_dtype; a.out_dtype = (DType)c_dtype; a.relu = relu;
    a.sm_count = g_sm_count[dev]; a.error_flag = status_word;
    e = launch_tconv(a, st);
  } else {
    IgemmArgs a;
    a.in = A; a.wpack = packed; a.shift = bias; a.out = C;
    a.N = M; a.H = a.W = a.OH = a.OW = 1; a.C = K; a.Kout = N; a.ldo = N; a.bn = bn;
    a.ab = (DType)ab_dtype; a.out_dtype = (DType)c_dtype; a.relu = relu; a.error_flag = status_word;
    e = launch_conv_igemm(a, st);
  }
  if (e != cudaSuccess) return internal_fail(NNCV_B200_ECUDA, "matmul_noalloc: launch failed: %s", cudaGetErrorString(e));
  return internal_ok();
}
