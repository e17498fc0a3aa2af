// CPU oracle for the compiled vision-model forward pass of nncv.
//
// THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA path is compared against
// (and the CPU baseline that the benchmark times); nothing in the product library links,
// loads or calls it.
//
// It restates, op by op and in plain C++17, what nncv's linalg-on-tensors fixtures compute
// (paths are relative to the nncv source tree):
//   * tests/Nets/Res18.mlir:118-629          the ResNet-18 forward (fp32, NCHW)
//   * tests/Nets/BatchNorm2d.mlir:12-22      inference batch-norm generic
//   * tests/Nets/ReLU.mlir:8-13              ReLU as `cmpf ugt` + `select`
//   * tests/Nets/Pool2DMax.mlir:3-9          max-pool with -inf initial value
//   * tests/SplitParams/data.mlir:4-12       two chained convs (known-answer case)
//   * tests/MatMulOptimization/MatMulDeafult.mlir:6-9   linalg.matmul
//   * tests/Nets/MobileNetV3.mlir:301,345-383  depthwise conv, hard-sigmoid / hard-swish, squeeze-and-excitation
//   * tests/Nets/Yolov5s.mlir:158-169,276,876-884  sigmoid / SiLU, channel concat, nearest 2x upsampling
// The arithmetic of those ops lives in upstream MLIR/LLVM ("18git", not vendored in nncv and
// not pinned), so the semantics followed here are the linalg named-op definitions as the
// fixtures instantiate them; the accumulation order per output element is the one of nncv's
// CPU lowering (src/nncv/compiler/Conversion/ConvOptimize/ConvertOptimizedConv2dToAffine.cpp:87-140:
// a plain running sum over c, then kh, then kw, in the element type).
//
// Pinning: the oracle is checked against every known-answer case the reference's own tests
// contain for this path (SplitParams all-ones -> 15.0; the Winograd fixture's closed form 3.6;
// the batch-norm fixture's identity statistics) and against PyTorch's CPU operators on seeded
// tensors.  nncv records no logits for any network, so whole-network parity is pinned only
// through those single-op cases: beyond them it is "parity unpinned".
//
// Build: see oracle/Makefile (g++ -O3 -march=x86-64-v3 -fopenmp -shared).

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// tensor.pad with a constant (Res18.mlir:118-122 zero pad, :144-147 -inf pad).
std::vector<float> pad_nchw(const float* x, int N, int C, int H, int W, int p, float v) {
  const int Hp = H + 2 * p, Wp = W + 2 * p;
  std::vector<float> out((size_t)N * C * Hp * Wp, v);
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < (long)N * C; ++nc) {
    for (int y = 0; y < H; ++y) {
      std::memcpy(&out[((size_t)nc * Hp + y + p) * Wp + p], &x[((size_t)nc * H + y) * W],
                  sizeof(float) * W);
    }
  }
  return out;
}

template <typename Acc>
void conv_core(const float* xp, const float* w, float* y, int N, int C, int Hp, int Wp, int K,
               int R, int S, int stride, int OH, int OW) {
#pragma omp parallel
  {
    std::vector<Acc> acc((size_t)OH * OW);
#pragma omp for collapse(2) schedule(dynamic, 4)
    for (int n = 0; n < N; ++n) {
      for (int k = 0; k < K; ++k) {
        std::fill(acc.begin(), acc.end(), Acc(0));  // linalg.fill 0 (Res18.mlir:124)
        for (int c = 0; c < C; ++c) {
          const float* xc = xp + ((size_t)n * C + c) * Hp * Wp;
          for (int r = 0; r < R; ++r) {
            for (int s = 0; s < S; ++s) {
              const Acc wv = (Acc)w[(((size_t)k * C + c) * R + r) * S + s];
              for (int oy = 0; oy < OH; ++oy) {
                const float* xr = xc + (size_t)(oy * stride + r) * Wp + s;
                Acc* ar = acc.data() + (size_t)oy * OW;
                if (stride == 1) {
                  for (int ox = 0; ox < OW; ++ox) ar[ox] += (Acc)xr[ox] * wv;
                } else {
                  for (int ox = 0; ox < OW; ++ox) ar[ox] += (Acc)xr[(size_t)ox * stride] * wv;
                }
              }
            }
          }
        }
        float* yo = y + ((size_t)n * K + k) * OH * OW;
        for (size_t i = 0; i < (size_t)OH * OW; ++i) yo[i] = (float)acc[i];
      }
    }
  }
}

}  // namespace

extern "C" {

// Launchers such as torchrun export OMP_NUM_THREADS=1; the CPU baseline is meant to use every
// host core, so the thread count can be set explicitly.
void nncv_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int nncv_oracle_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// linalg.conv_2d_nchw_fchw over a zero-padded input (Res18.mlir:118-125).  y is [N,K,OH,OW].
// acc64 != 0 accumulates in double ("gold" mode, bounds summation-order noise).
void nncv_oracle_conv2d_nchw_fchw(const float* x, const float* w, float* y, int N, int C, int H,
                                  int W, int K, int R, int S, int stride, int pad, int acc64) {
  const int Hp = H + 2 * pad, Wp = W + 2 * pad;
  const int OH = (Hp - R) / stride + 1, OW = (Wp - S) / stride + 1;
  std::vector<float> padded;
  const float* xp = x;
  if (pad > 0) {
    padded = pad_nchw(x, N, C, H, W, pad, 0.0f);
    xp = padded.data();
  }
  if (acc64)
    conv_core<double>(xp, w, y, N, C, Hp, Wp, K, R, S, stride, OH, OW);
  else
    conv_core<float>(xp, w, y, N, C, Hp, Wp, K, R, S, stride, OH, OW);
}

// Inference batch-norm generic (Res18.mlir:127-137): operands (x, gamma, beta, mean, var);
// eps = truncf(1e-5 : f64); y = ((x - mean) * rsqrt(var + eps)) * gamma + beta, all in f32.
void nncv_oracle_batchnorm(const float* x, const float* gamma, const float* beta,
                           const float* mean, const float* var, float* y, int N, int C,
                           long HW) {
  const float eps = (float)1e-5;
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < (long)N * C; ++nc) {
    const int c = (int)(nc % C);
    const float rs = 1.0f / std::sqrt(var[c] + eps);
    const float* xi = x + (size_t)nc * HW;
    float* yo = y + (size_t)nc * HW;
    for (long i = 0; i < HW; ++i) yo[i] = ((xi[i] - mean[c]) * rs) * gamma[c] + beta[c];
  }
}

// ReLU generic (Res18.mlir:138-143): `cmpf ugt` is true for NaN, so NaN passes through.
void nncv_oracle_relu(float* x, size_t n) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)n; ++i) {
    const float v = x[i];
    x[i] = !(v <= 0.0f) ? v : 0.0f;
  }
}

// Residual add generic (Res18.mlir:193-197).
void nncv_oracle_add(float* y, const float* a, size_t n) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)n; ++i) y[i] = y[i] + a[i];
}

// tensor.pad(-inf) + linalg.pooling_nchw_max (Res18.mlir:144-151; Pool2DMax.mlir:3-9).
void nncv_oracle_maxpool_nchw(const float* x, float* y, int N, int C, int H, int W, int k,
                              int stride, int pad) {
  const float ninf = -std::numeric_limits<float>::infinity();
  const int OH = (H + 2 * pad - k) / stride + 1, OW = (W + 2 * pad - k) / stride + 1;
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < (long)N * C; ++nc) {
    const float* xi = x + (size_t)nc * H * W;
    float* yo = y + (size_t)nc * OH * OW;
    for (int oy = 0; oy < OH; ++oy)
      for (int ox = 0; ox < OW; ++ox) {
        float m = ninf;
        for (int r = 0; r < k; ++r) {
          const int iy = oy * stride - pad + r;
          if (iy < 0 || iy >= H) continue;
          for (int s = 0; s < k; ++s) {
            const int ix = ox * stride - pad + s;
            if (ix < 0 || ix >= W) continue;
            const float v = xi[(size_t)iy * W + ix];
            m = (m < v || v != v) ? v : m;  // arith.maximumf propagates NaN
          }
        }
        yo[(size_t)oy * OW + ox] = m;
      }
  }
}

// linalg.pooling_nchw_sum over the whole map + divf by H*W (Res18.mlir:606-614).
void nncv_oracle_avgpool_global(const float* x, float* y, int N, int C, long HW) {
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < (long)N * C; ++nc) {
    float s = 0.0f;
    const float* xi = x + (size_t)nc * HW;
    for (long i = 0; i < HW; ++i) s += xi[i];
    y[nc] = s / (float)HW;
  }
}

// linalg.matmul C[M,N] = A[M,K] * B[K,N], row-major (MatMulDeafult.mlir:6-9), optional
// bias[N] add and ReLU (the benchmark's fused-epilogue variant).
void nncv_oracle_matmul(const float* A, const float* B, float* Cm, int M, int N, int K,
                        const float* bias, int relu, int acc64) {
#pragma omp parallel
  {
    std::vector<double> accd(acc64 ? N : 0);
    std::vector<float> accf(acc64 ? 0 : N);
#pragma omp for schedule(static)
    for (int m = 0; m < M; ++m) {
      if (acc64) {
        std::fill(accd.begin(), accd.end(), 0.0);
        for (int k = 0; k < K; ++k) {
          const double a = A[(size_t)m * K + k];
          const float* b = B + (size_t)k * N;
          for (int n = 0; n < N; ++n) accd[n] += a * (double)b[n];
        }
      } else {
        std::fill(accf.begin(), accf.end(), 0.0f);
        for (int k = 0; k < K; ++k) {
          const float a = A[(size_t)m * K + k];
          const float* b = B + (size_t)k * N;
          for (int n = 0; n < N; ++n) accf[n] += a * b[n];
        }
      }
      for (int n = 0; n < N; ++n) {
        float v = acc64 ? (float)accd[n] : accf[n];
        if (bias) v += bias[n];
        if (relu) v = !(v <= 0.0f) ? v : 0.0f;
        Cm[(size_t)m * N + n] = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Whole networks.  `blob` is the concatenation of all parameter tensors in the order the
// split-params file stores them (SplitParamsFlatArray.cpp:48-56: tensor i sits at the element
// offset sum_{j<i} numel_j), which mirrors the constant order of Res18.mlir:12-109:
//   fc.bias, fc.weight, then conv groups from the LAST to the FIRST of the forward pass,
//   each group = bn.bias, bn.weight, bn.running_var, bn.running_mean, conv.weight.
// The forward order of groups inside a residual block is conv1, conv2, (conv3,) downsample.
// ---------------------------------------------------------------------------------------

struct Group {  // one conv + its batch-norm
  int cin, cout, k, stride, pad;
  size_t off_beta, off_gamma, off_var, off_mean, off_w;
};

struct Net {
  std::vector<Group> groups;  // forward order
  int fc_in;
  size_t off_fc_b, off_fc_w, total;
};

static Net build_net(int depth) {
  Net net;
  auto add = [&](int cin, int cout, int k, int stride, int pad) {
    Group g{cin, cout, k, stride, pad, 0, 0, 0, 0, 0};
    net.groups.push_back(g);
  };
  add(3, 64, 7, 2, 3);
  if (depth == 18) {
    const int widths[4] = {64, 128, 256, 512};
    int cin = 64;
    for (int l = 0; l < 4; ++l) {
      for (int b = 0; b < 2; ++b) {
        const int stride = (b == 0 && l > 0) ? 2 : 1;
        add(cin, widths[l], 3, stride, 1);
        add(widths[l], widths[l], 3, 1, 1);
        if (b == 0 && l > 0) add(cin, widths[l], 1, 2, 0);
        cin = widths[l];
      }
    }
    net.fc_in = 512;
  } else {  // ResNet-50, torchvision v1.5 topology (stride on the 3x3); nncv has no fixture.
    const int widths[4] = {64, 128, 256, 512};
    const int blocks[4] = {3, 4, 6, 3};
    int cin = 64;
    for (int l = 0; l < 4; ++l) {
      for (int b = 0; b < blocks[l]; ++b) {
        const int stride = (b == 0 && l > 0) ? 2 : 1;
        add(cin, widths[l], 1, 1, 0);
        add(widths[l], widths[l], 3, stride, 1);
        add(widths[l], widths[l] * 4, 1, 1, 0);
        if (b == 0) add(cin, widths[l] * 4, 1, stride, 0);
        cin = widths[l] * 4;
      }
    }
    net.fc_in = 2048;
  }
  size_t off = 0;
  net.off_fc_b = off;
  off += 1000;
  net.off_fc_w = off;
  off += (size_t)1000 * net.fc_in;
  for (int i = (int)net.groups.size() - 1; i >= 0; --i) {
    Group& g = net.groups[i];
    g.off_beta = off;
    off += g.cout;
    g.off_gamma = off;
    off += g.cout;
    g.off_var = off;
    off += g.cout;
    g.off_mean = off;
    off += g.cout;
    g.off_w = off;
    off += (size_t)g.cout * g.cin * g.k * g.k;
  }
  net.total = off;
  return net;
}

// linalg.depthwise_conv_2d_nchw_chw (MobileNetV3.mlir:301): y[n,c,oy,ox] = sum_{r,s} x[n,c,oy*st+r-p,ox*st+s-p] * w[c,r,s],
// zero padding (the tensor.pad before it, :292-296), running sum over r then s.
void nncv_oracle_depthwise_conv_nchw_chw(const float* x, const float* w, float* y, int N, int C, int H, int W, int R, int S,
                                         int stride, int pad, int acc64) {
  const int OH = (H + 2 * pad - R) / stride + 1, OW = (W + 2 * pad - S) / stride + 1;
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < (long)N * C; ++nc) {
    const int c = (int)(nc % C);
    const float* xi = x + (size_t)nc * H * W;
    const float* wc = w + (size_t)c * R * S;
    float* yo = y + (size_t)nc * OH * OW;
    for (int oy = 0; oy < OH; ++oy)
      for (int ox = 0; ox < OW; ++ox) {
        float a32 = 0.0f;
        double a64 = 0.0;
        for (int r = 0; r < R; ++r) {
          const int iy = oy * stride - pad + r;
          for (int q = 0; q < S; ++q) {
            const int ix = ox * stride - pad + q;
            const float v = (iy < 0 || iy >= H || ix < 0 || ix >= W) ? 0.0f : xi[(size_t)iy * W + ix];
            if (acc64) a64 += (double)v * (double)wc[r * S + q];
            else a32 += v * wc[r * S + q];
          }
        }
        yo[(size_t)oy * OW + ox] = acc64 ? (float)a64 : a32;
      }
  }
}

// Elementwise activations as the fixtures spell them.  kind: 1 ReLU (cmpf ugt, select), 2 hard-sigmoid
// (MobileNetV3.mlir:345-377: addf 3, divf 6, `olt 1, t ? 1 : t`, `ogt 0, t ? 0 : t`), 3 hard-swish (x times it),
// 4 sigmoid (Yolov5s.mlir:158-164: negf, exp, addf 1, divf 1 / .), 5 SiLU (:165-169: mulf sigmoid(x), x).
void nncv_oracle_activation(float* x, size_t n, int kind) {
  auto hsig = [](float v) {
    float t = (v + 3.0f) / 6.0f;
    t = (1.0f < t) ? 1.0f : t;
    t = (0.0f > t) ? 0.0f : t;
    return t;
  };
  auto sig = [](float v) { return 1.0f / (std::exp(-v) + 1.0f); };
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)n; ++i) {
    const float v = x[i];
    switch (kind) {
      case 1: x[i] = !(v <= 0.0f) ? v : 0.0f; break;
      case 2: x[i] = hsig(v); break;
      case 3: x[i] = v * hsig(v); break;
      case 4: x[i] = sig(v); break;
      case 5: x[i] = sig(v) * v; break;
      default: break;
    }
  }
}

// tensor.concat dim(1) of NCHW tensors (Yolov5s.mlir:276).
void nncv_oracle_concat_channels(const float* const* in, const int* channels, int n_in, float* y, int N, long HW) {
  long Ct = 0;
  for (int i = 0; i < n_in; ++i) Ct += channels[i];
  for (int n = 0; n < N; ++n) {
    long off = 0;
    for (int i = 0; i < n_in; ++i) {
      std::copy(in[i] + (size_t)n * channels[i] * HW, in[i] + (size_t)(n + 1) * channels[i] * HW, y + ((size_t)n * Ct + off) * HW);
      off += channels[i];
    }
  }
}

// Nearest 2x upsampling (Yolov5s.mlir:876-884): y[n,c,i,j] = x[n,c,i floordiv 2,j floordiv 2].
void nncv_oracle_upsample2x(const float* x, float* y, int N, int C, int H, int W) {
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < (long)N * C; ++nc)
    for (int i = 0; i < 2 * H; ++i)
      for (int j = 0; j < 2 * W; ++j)
        y[((size_t)nc * 2 * H + i) * 2 * W + j] = x[((size_t)nc * H + i / 2) * W + j / 2];
}


size_t nncv_oracle_resnet_param_count(int depth) {
  if (depth != 18 && depth != 50) return 0;
  return build_net(depth).total;
}

// conv -> BN (-> ReLU) with the ops above; returns the output tensor and its spatial size.
static std::vector<float> conv_bn(const Net&, const Group& g, const float* blob,
                                  const std::vector<float>& x, int N, int& H, int& W, bool relu,
                                  int acc64) {
  const int OH = (H + 2 * g.pad - g.k) / g.stride + 1, OW = (W + 2 * g.pad - g.k) / g.stride + 1;
  std::vector<float> y((size_t)N * g.cout * OH * OW);
  nncv_oracle_conv2d_nchw_fchw(x.data(), blob + g.off_w, y.data(), N, g.cin, H, W, g.cout, g.k,
                               g.k, g.stride, g.pad, acc64);
  nncv_oracle_batchnorm(y.data(), blob + g.off_gamma, blob + g.off_beta, blob + g.off_mean,
                        blob + g.off_var, y.data(), N, g.cout, (long)OH * OW);
  if (relu) nncv_oracle_relu(y.data(), y.size());
  H = OH;
  W = OW;
  return y;
}

// ResNet-18 (Res18.mlir:118-629) or ResNet-50 forward.  x: [N,3,H,W]; logits: [N,1000].
// Returns 0 on success, non-zero on a bad argument.
int nncv_oracle_resnet_forward(int depth, const float* x, int N, int H, int W, const float* blob,
                               size_t blob_elems, float* logits, int acc64) {
  if (depth != 18 && depth != 50) return 1;
  const Net net = build_net(depth);
  if (blob_elems != net.total) return 2;
  size_t gi = 0;
  int h = H, w = W;
  std::vector<float> cur(x, x + (size_t)N * 3 * H * W);
  // stem: pad 3, conv 7x7 s2, BN, ReLU (Res18.mlir:118-143)
  cur = conv_bn(net, net.groups[gi++], blob, cur, N, h, w, true, acc64);
  {  // pad(-inf,1) + max-pool 3x3 s2 (Res18.mlir:144-151)
    const int oh = (h + 2 - 3) / 2 + 1, ow = (w + 2 - 3) / 2 + 1;
    std::vector<float> y((size_t)N * 64 * oh * ow);
    nncv_oracle_maxpool_nchw(cur.data(), y.data(), N, 64, h, w, 3, 2, 1);
    cur.swap(y);
    h = oh;
    w = ow;
  }
  const int nblocks18[4] = {2, 2, 2, 2}, nblocks50[4] = {3, 4, 6, 3};
  const int* nb = depth == 18 ? nblocks18 : nblocks50;
  for (int l = 0; l < 4; ++l) {
    for (int b = 0; b < nb[l]; ++b) {
      const bool has_ds = depth == 18 ? (b == 0 && l > 0) : (b == 0);
      int h1 = h, w1 = w;
      std::vector<float> t = conv_bn(net, net.groups[gi++], blob, cur, N, h1, w1, true, acc64);
      if (depth == 18) {
        t = conv_bn(net, net.groups[gi++], blob, t, N, h1, w1, false, acc64);
      } else {
        t = conv_bn(net, net.groups[gi++], blob, t, N, h1, w1, true, acc64);
        t = conv_bn(net, net.groups[gi++], blob, t, N, h1, w1, false, acc64);
      }
      if (has_ds) {  // BN(conv1x1(identity)) (Res18.mlir:297-311)
        int h2 = h, w2 = w;
        std::vector<float> idn =
            conv_bn(net, net.groups[gi++], blob, cur, N, h2, w2, false, acc64);
        nncv_oracle_add(t.data(), idn.data(), t.size());
      } else {
        nncv_oracle_add(t.data(), cur.data(), t.size());
      }
      nncv_oracle_relu(t.data(), t.size());
      cur.swap(t);
      h = h1;
      w = w1;
    }
  }
  const int cfin = net.fc_in;
  std::vector<float> pooled((size_t)N * cfin);
  nncv_oracle_avgpool_global(cur.data(), pooled.data(), N, cfin, (long)h * w);
  // transpose generic + matmul + bias generic (Res18.mlir:617-628)
  std::vector<float> wt((size_t)cfin * 1000);
  for (int o = 0; o < 1000; ++o)
    for (int i = 0; i < cfin; ++i) wt[(size_t)i * 1000 + o] = blob[net.off_fc_w + (size_t)o * cfin + i];
  nncv_oracle_matmul(pooled.data(), wt.data(), logits, N, 1000, cfin, blob + net.off_fc_b, 0,
                     acc64);
  return 0;
}

}  // extern "C"
