// conv3d / conv2d (cross-correlation, zero padding, any kernel extent, stride and padding per axis) as an implicit GEMM
// on the CUDA cores, fp32, with bias, residual add and activation fused into the epilogue; plus the network driver for
// stacks of such layers.
//
// Replaces the reference's cuDNN lowerings fortis_conv2d / fortis_conv3d (runtime/fortis_rt.c:108-156: descriptors
// rebuilt every call, heuristic algorithm, workspace from the pool, bias / activation / residual as further kernels:
// compiler/FortisFuse.cpp:626-655, 687-760), its library-free direct kernels (runtime/fortis_fft.cu:91-201) and its
// cuFFT convolution for large kernels (runtime/fortis_fft.cu:15-79); a 2-D convolution is the D = KD = 1 case.
//
// GEMM view: rows = output voxels (n, d, h, w), columns = output channels, reduction = taps x input channels.
// A block owns 128 voxels x 64 channels; per (tap, 16 input channels) slice the activations (gathered with the
// padding applied) and the weights are staged in shared memory; each of the 256 threads accumulates 8 x 4 outputs.
// Element strides of x and y are parameters, so the same kernel serves NDHWC networks and the NCDHW single-layer
// entry of the memref ABI.
#include <cuda_runtime.h>

#include <cstring>
#include <string>
#include <vector>

#include "fortis_kernels.h"
#include "fortis_model.h"

namespace fortis {

namespace {

struct ConvGeom {
  int N, D, H, W, C, F;
  int KD, KH, KW, pd, ph, pw, sd, sh, sw;
  int dd, dh, dw;                             // input dilation (1 = none): tap positions that fall between input samples read zero
  int Do, Ho, Wo;
  long long xs_n, xs_d, xs_h, xs_w, xs_c;     // element strides of x
  long long ys_n, ys_d, ys_h, ys_w, ys_c;     // element strides of y (and of the residual)
};

constexpr int CBM = 128, CBN = 64, CBK = 16;

// Tile 128 voxels x 64 channels per block of 256 threads, 8 x 4 outputs per thread.  The reduction runs over slices of
// (one tap, 16 input channels); the next slice's global loads are issued into registers before the current slice is
// multiplied out of shared memory (double-buffered: one barrier per slice).  Per k step a thread reads three 16-byte
// words from shared memory for 32 FMAs.
__global__ void __launch_bounds__(256) conv3d_f32_kernel(const float* __restrict__ x, const float* __restrict__ wt,   // wt [tap][C][F]
                                                         const float* __restrict__ bias, const float* __restrict__ residual,
                                                         float* __restrict__ y, ConvGeom g, int act, float slope) {
  __shared__ __align__(16) float As[2][CBK][CBM + 4];
  __shared__ __align__(16) float Ws[2][CBK][CBN + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const long long nvox = (long long)g.N * g.Do * g.Ho * g.Wo;
  const long long m0 = (long long)blockIdx.x * CBM;
  const int f0 = blockIdx.y * CBN;
  // A tile: this thread loads one voxel, 8 input channels per slice
  const int lv = tid & 127, lc = (tid >> 7) * 8;
  const long long vox = m0 + lv;
  int on = 0, od = 0, oh = 0, ow = 0;
  const bool vlive = vox < nvox;
  if (vlive) {
    long long t = vox;
    ow = (int)(t % g.Wo); t /= g.Wo;
    oh = (int)(t % g.Ho); t /= g.Ho;
    od = (int)(t % g.Do); on = (int)(t / g.Do);
  }
  // W tile: 16 input-channel rows x 64 output channels, 4 consecutive output channels per thread
  const int wr = tid >> 4, wc = (tid & 15) * 4;
  const bool wvec = (g.F & 3) == 0 && f0 + wc + 3 < g.F;
  // channels-last input whose every (voxel, 16-channel block) starts on a 16-byte boundary: vector loads
  const bool avec = g.xs_c == 1 && (g.C % CBK) == 0 && ((g.xs_w | g.xs_h | g.xs_d | g.xs_n) & 3) == 0 &&
                    (reinterpret_cast<unsigned long long>(x) & 15ull) == 0;

  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  const int ntaps = g.KD * g.KH * g.KW, cblocks = (g.C + CBK - 1) / CBK, nslices = ntaps * cblocks;
  float pa[8], pw[4];
  auto fetch = [&](int slice) {
    const int tap = slice / cblocks, c0 = (slice - tap * cblocks) * CBK;
    const int kd = tap / (g.KH * g.KW), kh = (tap / g.KW) % g.KH, kw = tap % g.KW;
    int id = od * g.sd + kd - g.pd, ih = oh * g.sh + kh - g.ph, iw = ow * g.sw + kw - g.pw;
    bool inb = vlive && id >= 0 && ih >= 0 && iw >= 0;
    if (g.dd > 1) { inb = inb && id % g.dd == 0; id /= g.dd; }
    if (g.dh > 1) { inb = inb && ih % g.dh == 0; ih /= g.dh; }
    if (g.dw > 1) { inb = inb && iw % g.dw == 0; iw /= g.dw; }
    inb = inb && id < g.D && ih < g.H && iw < g.W;
    const float* xp = x + (long long)on * g.xs_n + (long long)id * g.xs_d + (long long)ih * g.xs_h + (long long)iw * g.xs_w;
    if (avec) {                                                // channels-last: the thread's 8 channels are 32 contiguous bytes
      float4 q0 = make_float4(0.f, 0.f, 0.f, 0.f), q1 = q0;
      if (inb) {
        q0 = __ldg(reinterpret_cast<const float4*>(xp + c0 + lc));
        q1 = __ldg(reinterpret_cast<const float4*>(xp + c0 + lc) + 1);
      }
      pa[0] = q0.x; pa[1] = q0.y; pa[2] = q0.z; pa[3] = q0.w; pa[4] = q1.x; pa[5] = q1.y; pa[6] = q1.z; pa[7] = q1.w;
    } else {
#pragma unroll
      for (int e = 0; e < 8; e++) {
        const int c = c0 + lc + e;
        pa[e] = (inb && c < g.C) ? __ldg(xp + (long long)c * g.xs_c) : 0.f;
      }
    }
    const int c = c0 + wr;
    const float* wp = wt + ((long long)tap * g.C + c) * g.F + f0 + wc;
    if (c < g.C && wvec) {
      const float4 q = __ldg(reinterpret_cast<const float4*>(wp));
      pw[0] = q.x; pw[1] = q.y; pw[2] = q.z; pw[3] = q.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; e++) pw[e] = (c < g.C && f0 + wc + e < g.F) ? __ldg(wp + e) : 0.f;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int e = 0; e < 8; e++) As[buf][lc + e][lv] = pa[e];
    *reinterpret_cast<float4*>(&Ws[buf][wr][wc]) = make_float4(pw[0], pw[1], pw[2], pw[3]);
  };
  fetch(0);
  stash(0);
  __syncthreads();
  for (int slice = 0; slice < nslices; slice++) {
    const int buf = slice & 1;
    if (slice + 1 < nslices) fetch(slice + 1);                 // in flight while this slice is multiplied
#pragma unroll
    for (int k = 0; k < CBK; k++) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 8]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 8 + 4]);
      const float4 w = *reinterpret_cast<const float4*>(&Ws[buf][k][tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    if (slice + 1 < nslices) stash(buf ^ 1);                   // the other buffer was last read before the previous barrier
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const long long v = m0 + ty * 8 + i;
    if (v >= nvox) continue;
    long long t = v;
    const int w_ = (int)(t % g.Wo); t /= g.Wo;
    const int h_ = (int)(t % g.Ho); t /= g.Ho;
    const int d_ = (int)(t % g.Do); const int n_ = (int)(t / g.Do);
    const long long yo = (long long)n_ * g.ys_n + (long long)d_ * g.ys_d + (long long)h_ * g.ys_h + (long long)w_ * g.ys_w;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int f = f0 + tx * 4 + j;
      if (f >= g.F) continue;
      float o = acc[i][j] + (bias ? bias[f] : 0.f);
      if (residual) o += residual[yo + (long long)f * g.ys_c];
      if (act == ACT_RELU) o = fmaxf(o, 0.f);
      else if (act == ACT_LEAKY) o = o > 0.f ? o : o * slope;
      y[yo + (long long)f * g.ys_c] = o;
    }
  }
}

void launch_conv(const float* x, const float* wt, const float* bias, const float* residual, float* y, const ConvGeom& g, int act,
                 float slope, cudaStream_t s) {
  const long long nvox = (long long)g.N * g.Do * g.Ho * g.Wo;
  if (nvox <= 0) return;
  dim3 grid((unsigned)((nvox + CBM - 1) / CBM), (unsigned)((g.F + CBN - 1) / CBN));
  conv3d_f32_kernel<<<grid, 256, 0, s>>>(x, wt, bias, residual, y, g, act, slope);
}

// the same repack on the device, for weights that only exist there (the memref entry)
__global__ void repack_weights_kernel(const float* __restrict__ w, float* __restrict__ out, int F, int C, int taps) {
  const size_t n = (size_t)F * C * taps;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;     // index into out: [tap][C][F]
  if (i >= n) return;
  const int f = (int)(i % F);
  const int c = (int)((i / F) % C);
  const int t = (int)(i / ((size_t)F * C));
  out[i] = w[((size_t)f * C + c) * taps + t];
}

// torch layout (F, C, taps...) -> [tap][C][F]
std::vector<float> repack_weights_taps(const float* w, int F, int C, int taps);
std::vector<float> repack_weights(const float* w, int F, int C, int K) { return repack_weights_taps(w, F, C, K * K * K); }
std::vector<float> repack_weights_taps(const float* w, int F, int C, int taps) {
  std::vector<float> out((size_t)taps * C * F);
  for (int f = 0; f < F; f++)
    for (int c = 0; c < C; c++)
      for (int t = 0; t < taps; t++) out[((size_t)t * C + c) * F + f] = w[((size_t)f * C + c) * taps + t];
  return out;
}

// ---- 2-D operator layers without weights (NCHW): the operator micro-suite's pooling and upsampling
__global__ void maxpool2d_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int H, int W, int KH, int KW,
                                 int sh, int sw, int Ho, int Wo) {
  const long long n = planes * Ho * Wo;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int ow = (int)(i % Wo), oh = (int)((i / Wo) % Ho);
    const long long pl = i / ((long long)Wo * Ho);
    const float* src = x + pl * H * W;
    float m = -INFINITY;
    for (int kh = 0; kh < KH; kh++)
      for (int kw = 0; kw < KW; kw++) m = fmaxf(m, __ldg(src + (long long)(oh * sh + kh) * W + ow * sw + kw));
    y[i] = m;
  }
}

__global__ void upsample_nearest2d_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int H, int W, int fh, int fw) {
  const int Ho = H * fh, Wo = W * fw;
  const long long n = planes * Ho * Wo;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int ow = (int)(i % Wo), oh = (int)((i / Wo) % Ho);
    const long long pl = i / ((long long)Wo * Ho);
    y[i] = __ldg(x + pl * H * W + (long long)(oh / fh) * W + ow / fw);
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// Networks of 2-D operator layers, NCHW fp32: Conv2d (any kernel, stride, padding; transposed convolutions as the
// convolution of the dilated input; BatchNorm, explicit padding and channel concatenation of parallel convolutions are
// folded into the weights by the exporter), MaxPool2d, nearest Upsample.  The counterpart of what the reference's
// compiler generates for the operator micro-suite (tests/optest.py; compiler/FortisFuse.cpp:309-356 for the pad folding).
// ---------------------------------------------------------------------------------------------------------------
struct OpNet {
  std::vector<LayerHost> meta;
  std::vector<float*> wt, bias;           // per layer (null for layers without weights)
  float* buf[2] = {nullptr, nullptr};
  long long cap = 0;
};

void opnet_destroy(OpNet* m) {
  if (!m) return;
  for (float* p : m->wt) cudaFree(p);
  for (float* p : m->bias) cudaFree(p);
  for (float* p : m->buf) cudaFree(p);
  delete m;
}

// output extent of one layer; false when the layer does not fit the input
static bool opnet_layer_shape(const LayerHost& L, int H, int W, int* Ho, int* Wo) {
  if (L.kind == LAYER_UPSAMPLE2D) { *Ho = H * L.sh; *Wo = W * L.sw; return true; }
  const int He = (H - 1) * L.dil + 1 + 2 * L.ph + L.eh, We = (W - 1) * L.dil + 1 + 2 * L.pw + L.ew;
  if (He < L.kh || We < L.kw) return false;
  *Ho = (He - L.kh) / L.sh + 1; *Wo = (We - L.kw) / L.sw + 1;
  return true;
}

bool opnet_shape(const ModelHost& M, int H, int W, int* C, int* Ho, int* Wo, long long* max_elems_per_image) {
  long long mx = 0;
  int c = M.n_in();
  for (auto& L : M.layers) {
    int h2, w2;
    if (!opnet_layer_shape(L, H, W, &h2, &w2)) return false;
    H = h2; W = w2; c = L.cout;
    const long long e = (long long)c * H * W;
    mx = e > mx ? e : mx;
  }
  *C = c; *Ho = H; *Wo = W;
  if (max_elems_per_image) *max_elems_per_image = mx;
  return true;
}

OpNet* opnet_create(const ModelHost& M, std::string* err) {
  for (auto& L : M.layers)
    if (L.kind != LAYER_CONV2D && (L.ph || L.pw || L.dil != 1 || L.eh || L.ew)) {
      if (err) *err = "pooling and upsampling layers take no padding or dilation";
      return nullptr;
    }
  OpNet* m = new OpNet();
  for (auto& L : M.layers) {
    LayerHost meta = L; meta.W.clear(); meta.b.clear();
    m->meta.push_back(meta);
    float *dw = nullptr, *db = nullptr;
    if (L.kind == LAYER_CONV2D) {
      const std::vector<float> wt = repack_weights_taps(L.W.data(), L.cout, L.cin, L.kh * L.kw);
      if (cudaMalloc(&dw, wt.size() * 4) != cudaSuccess || cudaMalloc(&db, L.b.size() * 4) != cudaSuccess) {
        if (err) *err = "out of device memory for conv weights";
        cudaFree(dw); opnet_destroy(m);
        return nullptr;
      }
      cudaMemcpy(dw, wt.data(), wt.size() * 4, cudaMemcpyHostToDevice);
      cudaMemcpy(db, L.b.data(), L.b.size() * 4, cudaMemcpyHostToDevice);
    }
    m->wt.push_back(dw); m->bias.push_back(db);
  }
  return m;
}

// x (N, Cin, H, W) -> y (N, Cout, Ho, Wo)
bool opnet_forward(OpNet* m, const float* x, float* y, int N, int H, int W, cudaStream_t s, std::string* err) {
  if ((long long)N * H * W <= 0) { if (err) *err = "2-D network: set the input extent (option conv_shape = N,1,H,W)"; return false; }
  // intermediate extents
  long long mx = 0;
  {
    int h = H, w = W;
    for (size_t l = 0; l + 1 < m->meta.size(); l++) {
      int h2, w2;
      if (!opnet_layer_shape(m->meta[l], h, w, &h2, &w2)) { if (err) *err = "2-D network: a layer's kernel is larger than its input"; return false; }
      h = h2; w = w2;
      const long long e = (long long)N * m->meta[l].cout * h * w;
      mx = e > mx ? e : mx;
    }
  }
  if (m->cap < mx) {
    for (float*& p : m->buf) { cudaFree(p); p = nullptr; }
    for (float*& p : m->buf)
      if (cudaMalloc(&p, (size_t)mx * 4) != cudaSuccess) { if (err) *err = "out of device memory for 2-D network activations"; return false; }
    m->cap = mx;
  }
  const float* src = x;
  int h = H, w = W;
  const int nl = (int)m->meta.size();
  for (int l = 0; l < nl; l++) {
    const LayerHost& L = m->meta[l];
    float* dst = l == nl - 1 ? y : (src == m->buf[0] ? m->buf[1] : m->buf[0]);
    int h2, w2;
    if (!opnet_layer_shape(L, h, w, &h2, &w2)) { if (err) *err = "2-D network: a layer's kernel is larger than its input"; return false; }
    const long long planes = (long long)N * L.cin, nout = (long long)N * L.cout * h2 * w2;
    const unsigned blocks = (unsigned)((nout + 255) / 256 < 148 * 16 ? (nout + 255) / 256 : 148 * 16);
    if (L.kind == LAYER_CONV2D) {
      ConvGeom g;
      g.N = N; g.D = 1; g.H = h; g.W = w; g.C = L.cin; g.F = L.cout;
      g.KD = 1; g.KH = L.kh; g.KW = L.kw; g.pd = 0; g.ph = L.ph; g.pw = L.pw; g.sd = 1; g.sh = L.sh; g.sw = L.sw;
      g.dd = 1; g.dh = g.dw = L.dil;
      g.Do = 1; g.Ho = h2; g.Wo = w2;
      g.xs_w = 1; g.xs_h = w; g.xs_d = (long long)h * w; g.xs_c = (long long)h * w; g.xs_n = (long long)L.cin * h * w;
      g.ys_w = 1; g.ys_h = w2; g.ys_d = (long long)h2 * w2; g.ys_c = (long long)h2 * w2; g.ys_n = (long long)L.cout * h2 * w2;
      launch_conv(src, m->wt[l], m->bias[l], nullptr, dst, g, L.act, L.slope, s);
    } else if (L.kind == LAYER_MAXPOOL2D) {
      maxpool2d_kernel<<<blocks, 256, 0, s>>>(src, dst, planes, h, w, L.kh, L.kw, L.sh, L.sw, h2, w2);
    } else {
      upsample_nearest2d_kernel<<<blocks, 256, 0, s>>>(src, dst, planes, h, w, L.sh, L.sw);
    }
    src = dst; h = h2; w = w2;
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { if (err) *err = std::string("2-D network launch: ") + cudaGetErrorString(e); return false; }
  return true;
}

struct ConvModel {
  ConvTcModel* tcm = nullptr;           // bf16 tensor-core network (precision bf16); the fields below serve fp32
  std::vector<LayerHost> meta;          // shapes and flags (weights dropped after upload)
  std::vector<float*> wt, bias;
  float *buf[3] = {nullptr, nullptr, nullptr};
  long long buf_elems = 0;
};

void conv_model_destroy(ConvModel* m) {
  if (!m) return;
  conv_tc_destroy(m->tcm);
  for (float* p : m->wt) cudaFree(p);
  for (float* p : m->bias) cudaFree(p);
  for (float* p : m->buf) cudaFree(p);
  delete m;
}

int conv_model_status(ConvModel* m) { return m && m->tcm ? conv_tc_status(m->tcm) : 0; }
void conv_model_clear_status(ConvModel* m) { if (m && m->tcm) conv_tc_clear_status(m->tcm); }

ConvModel* conv_model_create(const ModelHost& M, int precision, cudaStream_t s, std::string* err) {
  (void)s;
  if (precision == PREC_FP8W) { if (err) *err = "conv3d networks run in fp32, bf16 or fp16"; return nullptr; }
  ConvModel* m = new ConvModel();
  if (precision == PREC_BF16 || precision == PREC_FP16) {
    std::string why;
    m->tcm = conv_tc_create(M, precision == PREC_FP16, &why);
    if (!m->tcm) { if (err) *err = "precision bf16 / fp16 needs the tensor-core conv kernel, which cannot take this model: " + why; delete m; return nullptr; }
    return m;
  }
  for (auto& L : M.layers) {
    LayerHost meta = L;
    meta.W.clear(); meta.b.clear();
    m->meta.push_back(meta);
    std::vector<float> wt = repack_weights(L.W.data(), L.cout, L.cin, L.ksize);
    float *dw = nullptr, *db = nullptr;
    if (cudaMalloc(&dw, wt.size() * 4) != cudaSuccess || cudaMalloc(&db, L.b.size() * 4) != cudaSuccess) {
      if (err) *err = "out of device memory for conv weights";
      conv_model_destroy(m);
      return nullptr;
    }
    cudaMemcpy(dw, wt.data(), wt.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(db, L.b.data(), L.b.size() * 4, cudaMemcpyHostToDevice);
    m->wt.push_back(dw); m->bias.push_back(db);
  }
  return m;
}

// x (N, D, H, W, Cin) -> y (N, D, H, W, Cout); every layer keeps the spatial extent (pad = K / 2)
bool conv_forward(ConvModel* m, const float* x, float* y, int N, int D, int H, int W, cudaStream_t s, std::string* err) {
  if (m->tcm) return conv_tc_forward(m->tcm, x, y, N, D, H, W, s, err);
  const long long nvox = (long long)N * D * H * W;
  if (nvox <= 0) { if (err) *err = "conv3d model: set the input extent (option conv_shape = N,D,H,W)"; return false; }
  int cmax = 1;
  for (auto& L : m->meta) {
    if (L.pad * 2 + 1 != L.ksize) { if (err) *err = "conv3d model layers must keep the spatial extent (pad = K / 2)"; return false; }
    cmax = L.cout > cmax ? L.cout : cmax;
  }
  if (m->buf_elems < nvox * cmax) {
    for (float*& p : m->buf) { cudaFree(p); p = nullptr; }
    for (float*& p : m->buf)
      if (cudaMalloc(&p, (size_t)nvox * cmax * 4) != cudaSuccess) { if (err) *err = "out of device memory for conv activations"; return false; }
    m->buf_elems = nvox * cmax;
  }
  const float* src = x;
  const float* skip = nullptr;
  int skip_buf = -1;
  const int nl = (int)m->meta.size();
  for (int l = 0; l < nl; l++) {
    const LayerHost& L = m->meta[l];
    float* dst = y;
    int dst_buf = -1;
    if (l != nl - 1) {
      for (int b = 0; b < 3; b++)
        if (m->buf[b] != src && b != skip_buf) { dst = m->buf[b]; dst_buf = b; break; }
    }
    ConvGeom g;
    g.N = N; g.D = D; g.H = H; g.W = W; g.C = L.cin; g.F = L.cout;
    g.KD = g.KH = g.KW = L.ksize; g.pd = g.ph = g.pw = L.pad; g.sd = g.sh = g.sw = 1; g.dd = g.dh = g.dw = 1;
    g.Do = D; g.Ho = H; g.Wo = W;
    g.xs_c = 1; g.xs_w = L.cin; g.xs_h = (long long)W * L.cin; g.xs_d = (long long)H * W * L.cin; g.xs_n = (long long)D * H * W * L.cin;
    g.ys_c = 1; g.ys_w = L.cout; g.ys_h = (long long)W * L.cout; g.ys_d = (long long)H * W * L.cout; g.ys_n = (long long)D * H * W * L.cout;
    const float* res = (L.flags & LFLAG_ADD_SKIP) ? skip : nullptr;
    if ((L.flags & LFLAG_ADD_SKIP) && !skip) { if (err) *err = "conv3d model: a layer adds a skip that was never saved"; return false; }
    launch_conv(src, m->wt[l], m->bias[l], res, dst, g, L.act, L.slope, s);
    if (L.flags & LFLAG_SAVE_SKIP) { skip = dst; skip_buf = dst_buf; }
    src = dst;
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { if (err) *err = std::string("conv3d launch: ") + cudaGetErrorString(e); return false; }
  return true;
}

// single layer, NCDHW fp32, weights in the torch layout on the device (memref ABI of runtime/fortis_rt.c:128-131)
bool conv3d_ncdhw(const float* x, const float* w, float* y, int N, int C, int D, int H, int W, int F, const int K[3],
                  const int stride[3], const int pad[3], cudaStream_t s, std::string* err) {
  // weights are constants of the caller: repack each distinct (pointer, shape) once, as the reference caches its
  // transposed GEMM weights (runtime/fortis_rt.c:55-66)
  // The repack runs as a kernel on the caller's stream (no synchronisation, no host round trip).  The cache holds 64
  // entries; when it is full the oldest entry is replaced and its buffer reused or freed.  A weight seen for the
  // first time needs a buffer: that cannot happen while the stream is being captured into a graph, so such a call
  // is refused (the reference captures on the second call for the same reason: the first call allocates).
  struct Cached { const float* w; int F, C, taps; float* wt; size_t cap; };
  static std::vector<Cached> cache;
  static size_t victim = 0;
  float* wt = nullptr;
  const int taps = K[0] * K[1] * K[2];
  for (auto& c : cache) if (c.w == w && c.F == F && c.C == C && c.taps == taps) wt = c.wt;
  if (!wt) {
    const size_t n = (size_t)F * C * taps;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(s, &cs);
    if (cs != cudaStreamCaptureStatusNone) { if (err) *err = "conv weights seen for the first time during graph capture; run one eager call first"; return false; }
    Cached* slot = nullptr;
    if (cache.size() < 64) { cache.push_back({nullptr, 0, 0, 0, nullptr, 0}); slot = &cache.back(); }
    else { slot = &cache[victim]; victim = (victim + 1) % cache.size(); }
    if (slot->cap < n) {
      if (slot->wt) { cudaStreamSynchronize(s); cudaFree(slot->wt); slot->wt = nullptr; slot->cap = 0; }
      if (cudaMalloc(&slot->wt, n * 4) != cudaSuccess) { slot->w = nullptr; if (err) *err = "out of device memory for conv weights"; return false; }
      slot->cap = n;
    }
    slot->w = w; slot->F = F; slot->C = C; slot->taps = taps;
    wt = slot->wt;
    repack_weights_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(w, wt, F, C, taps);
  }
  ConvGeom g;
  g.N = N; g.D = D; g.H = H; g.W = W; g.C = C; g.F = F;
  g.KD = K[0]; g.KH = K[1]; g.KW = K[2]; g.sd = stride[0]; g.sh = stride[1]; g.sw = stride[2]; g.pd = pad[0]; g.ph = pad[1]; g.pw = pad[2];
  g.dd = g.dh = g.dw = 1;
  g.Do = (D + 2 * pad[0] - K[0]) / stride[0] + 1; g.Ho = (H + 2 * pad[1] - K[1]) / stride[1] + 1; g.Wo = (W + 2 * pad[2] - K[2]) / stride[2] + 1;
  g.xs_w = 1; g.xs_h = W; g.xs_d = (long long)H * W; g.xs_c = (long long)D * H * W; g.xs_n = (long long)C * D * H * W;
  g.ys_w = 1; g.ys_h = g.Wo; g.ys_d = (long long)g.Ho * g.Wo; g.ys_c = (long long)g.Do * g.Ho * g.Wo; g.ys_n = (long long)F * g.Do * g.Ho * g.Wo;
  launch_conv(x, wt, nullptr, nullptr, y, g, ACT_NONE, 0.f, s);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { if (err) *err = std::string("conv3d launch: ") + cudaGetErrorString(e); return false; }
  return true;
}

}  // namespace fortis
