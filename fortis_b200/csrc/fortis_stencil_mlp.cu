// Fused gather -> small MLP -> scatter for 3x3-stencil hosts (ocean eddy parameterisations: 3 fields x 9 taps = 27
// inputs, two or three narrow layers, a few outputs per gridpoint), fp32, one thread per gridpoint.
//
// Replaces, for such hosts, the reference's generated fortis_gather_k (27 separate global loads per row, each input
// re-read nine times, X written with 108-byte-strided stores: driver/fortis_gather_emit.py:52-62), the per-layer
// matvec / GEMM kernels behind it and fortis_scatter_k (compiler/FortisFuse.cpp:587-655).  Loop order per layer is the
// shipped native forward's: inputs outer, outputs inner, bias, activation (mom6_zb/fwd_native_zb.f90:36-47).
//
// The step is bound by fp32 multiply-add issue, not by HBM (1000 MACs per 24 bytes), so the kernel is built to spend
// its issue slots on nothing else:
//   * packed fp32 FMAs (fma.rn.f32x2): one instruction updates two output neurons, the weight PAIR comes straight from
//     the constant bank (weights are stored as (w[i][j], w[i][j+1]) pairs), the input is duplicated once per input;
//   * a block stages its (32+2) x (4+2) halo tile of every field in shared memory with coalesced loads, so a point's 27
//     inputs are shared-memory reads at immediate offsets (no address arithmetic) and each input is read from L2 once;
//   * accumulators start at the bias; ReLU is one instruction per value; outputs are stored coalesced along i.
// Widths are template parameters (that is what makes every weight an immediate-address operand): hidden widths are
// padded to 16, 20 or 32, outputs to 4.  Other stencil nets take the generic small-MLP kernel.
#include <cuda_runtime.h>

#include <cstring>

#include "fortis_kernels.h"

namespace fortis {

namespace {

#ifndef FORTIS_STENCIL_MINBLOCKS
#define FORTIS_STENCIL_MINBLOCKS 8
#endif
constexpr int kTI = 32, kTJ = 4, kPitch = 36;       // points per tile, shared-memory row pitch (34 used)
constexpr int kRows = kTJ + 2;
constexpr int kNF = 3;                               // fields
constexpr int kD0 = 9 * kNF;
constexpr int kPairs = 2048;                         // constant-bank budget: float2 weight pairs

__constant__ float2 c_pair[kPairs];
__constant__ float c_in_div[kD0];
__constant__ float c_out_mul[4];

__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
      "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}

template <bool RELU> __device__ __forceinline__ float act1(float v, float slope) {
  if constexpr (RELU) return fmaxf(v, 0.f);
  else return fmaxf(v, v * slope);                   // none: slope 1, LeakyReLU: its slope
}

// y[N] (as N/2 pairs) = act(b + x[K] . W), weights at c_pair[OFF + k * N/2 + jp], biases behind them
template <int K, int N, int OFF, bool RELU>
__device__ __forceinline__ void layer2(const float (&x)[K], float (&y)[N], float slope) {
  float2 acc[N / 2];
#pragma unroll
  for (int jp = 0; jp < N / 2; jp++) acc[jp] = c_pair[OFF + K * (N / 2) + jp];
#pragma unroll
  for (int k = 0; k < K; k++) {
    const float2 xx = make_float2(x[k], x[k]);
#pragma unroll
    for (int jp = 0; jp < N / 2; jp++) acc[jp] = fma2(xx, c_pair[OFF + k * (N / 2) + jp], acc[jp]);
  }
#pragma unroll
  for (int jp = 0; jp < N / 2; jp++) { y[2 * jp] = act1<RELU>(acc[jp].x, slope); y[2 * jp + 1] = act1<RELU>(acc[jp].y, slope); }
}

template <int P1, int P2>
struct StencilLayout {   // offsets in float2 units; P2 == 0: two layers
  static constexpr int w1 = 0, w2 = w1 + kD0 * (P1 / 2) + P1 / 2;
  static constexpr int w3 = P2 ? w2 + P1 * (P2 / 2) + P2 / 2 : w2;
  static constexpr int total = P2 ? w3 + P2 * 2 + 2 : w2 + P1 * 2 + 2;
};

template <int P1, int P2, bool RELU>
__global__ void __launch_bounds__(128, FORTIS_STENCIL_MINBLOCKS) stencil_mlp_kernel(StencilLaunch S) {
  using LY = StencilLayout<P1, P2>;
  __shared__ float tile[kNF][kRows][kPitch];
  const int ti = threadIdx.x & 31, tj = threadIdx.x >> 5;
  const int tiles_i = (S.ni + kTI - 1) / kTI, tiles_j = (S.nj + kTJ - 1) / kTJ;
  const long long ntiles = (long long)tiles_i * tiles_j * S.nk;
  double csum = 0.0;
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int kk = (int)(t / ((long long)tiles_i * tiles_j));
    const int rem = (int)(t - (long long)kk * tiles_i * tiles_j);
    const int ci0 = (rem % tiles_i) * kTI, cj0 = (rem / tiles_i) * kTJ;
    __syncthreads();                                   // the previous tile has been consumed
    // halo tile of every field: rows cj0-1 .. cj0+kTJ, columns ci0-1 .. ci0+kTI, lanes along i (coalesced)
    // warp tj takes rows tj and tj + 4 of every field; lane = column, lanes 0 and 1 also fetch columns 32 and 33
#pragma unroll
    for (int f = 0; f < kNF; f++) {
      const float* fb = S.in[f] + (long long)kk * S.sk_in + (ci0 - 1);
#pragma unroll
      for (int rr = 0; rr < 2; rr++) {
        const int r = tj + 4 * rr;
        if (r < kRows) {
          const int gj = cj0 - 1 + r;
          const float* rowp = fb + (long long)gj * S.sj_in;
          const bool rok = gj <= S.nj;
          tile[f][r][ti] = (rok && ci0 - 1 + ti <= S.ni) ? __ldg(rowp + ti) : 0.f;
          if (ti < 2) tile[f][r][kTI + ti] = (rok && ci0 - 1 + kTI + ti <= S.ni) ? __ldg(rowp + kTI + ti) : 0.f;
        }
      }
    }
    __syncthreads();
    const int ci = ci0 + ti, cj = cj0 + tj;
    if (ci >= S.ni || cj >= S.nj) continue;
    float x[kD0];
#pragma unroll
    for (int f = 0; f < kNF; f++)
#pragma unroll
      for (int dj = 0; dj < 3; dj++)
#pragma unroll
        for (int di = 0; di < 3; di++) x[f * 9 + dj * 3 + di] = tile[f][tj + dj][ti + di];
    if (S.has_in_div) {
#pragma unroll
      for (int q = 0; q < kD0; q++) x[q] = __fdiv_rn(x[q], c_in_div[q]);
    }
    float h1[P1];
    layer2<kD0, P1, LY::w1, RELU>(x, h1, S.slope[0]);
    float y[4];
    if constexpr (P2 == 0) {
      layer2<P1, 4, LY::w2, false>(h1, y, S.slope[1]);
    } else {
      float h2[P2];
      layer2<P1, P2, LY::w2, RELU>(h1, h2, S.slope[1]);
      layer2<P2, 4, LY::w3, false>(h2, y, S.slope[2]);
    }
    if (S.has_out_mul) {
#pragma unroll
      for (int j = 0; j < 4; j++) y[j] *= c_out_mul[j];
    }
    const long long opos = ci + (long long)cj * S.sj_out + (long long)kk * S.sk_out;
#pragma unroll
    for (int s = 0; s < 4; s++) {
      if (s < S.nstores) {
        float v = y[0];
#pragma unroll
        for (int j = 1; j < 4; j++) if (S.out_slot[s] == j) v = y[j];
        S.out[s][opos] = v;
        csum += (double)v;
      }
    }
  }
  if (S.partials) {
    // deterministic per-block partial, then the last block folds all partials into the step checksum in block order
    __shared__ double wsum[4];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) csum += __shfl_down_sync(0xffffffffu, csum, o);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = csum;
    __syncthreads();
    if (threadIdx.x == 0) {
      S.partials[blockIdx.x] = (wsum[0] + wsum[1]) + (wsum[2] + wsum[3]);
      if (S.sum) {
        __threadfence();
        if (atomicAdd(S.done, 1u) == gridDim.x - 1) {
          __threadfence();
          double total = *S.sum;
          for (unsigned i = 0; i < gridDim.x; i++) total += __ldcg(S.partials + i);
          *S.sum = total;
          *S.done = 0u;
        }
      }
    }
  }
}

int pad_width(int d) { return d <= 16 ? 16 : d <= 20 ? 20 : d <= 32 ? 32 : 0; }

}  // namespace

bool stencil_mlp_supported(int nlayers, const int* dims) {
  if (nlayers != 2 && nlayers != 3) return false;
  if (dims[0] != kD0 || dims[nlayers] > 4 || dims[nlayers] < 1) return false;
  for (int l = 1; l < nlayers; l++) if (pad_width(dims[l]) == 0) return false;
  if (nlayers == 3 && pad_width(dims[1]) != pad_width(dims[2])) return false;      // instantiated for equal hidden widths
  return true;
}

// Writes the constant-bank image: weight pairs (w[i][j], w[i][j+1]) per layer, [in][out/2], biases behind each layer,
// zero where a width is padded.  W[l] is (out, in) row-major (torch layout).
cudaError_t stencil_mlp_upload(int nlayers, const int* dims, const float* const* W, const float* const* b, const float* in_div,
                               const float* out_mul, cudaStream_t s) {
  int pd[4];
  pd[0] = dims[0];
  for (int l = 1; l < nlayers; l++) pd[l] = pad_width(dims[l]);
  pd[nlayers] = 4;
  static float2 img[kPairs];
  std::memset(img, 0, sizeof img);
  int o = 0;
  for (int l = 0; l < nlayers; l++) {
    const int K = pd[l], N = pd[l + 1], Kr = dims[l], Nr = dims[l + 1];
    if (o + K * (N / 2) + N / 2 > kPairs) return cudaErrorInvalidValue;
    for (int k = 0; k < Kr; k++)
      for (int j = 0; j < Nr; j++) {
        float* dst = reinterpret_cast<float*>(&img[o + k * (N / 2) + j / 2]);
        dst[j & 1] = W[l][(size_t)j * Kr + k];
      }
    o += K * (N / 2);
    for (int j = 0; j < Nr; j++) reinterpret_cast<float*>(&img[o + j / 2])[j & 1] = b[l] ? b[l][j] : 0.f;
    o += N / 2;
  }
  cudaError_t e = cudaMemcpyToSymbolAsync(c_pair, img, sizeof(float2) * o, 0, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return e;
  float idv[kD0], om[4] = {1.f, 1.f, 1.f, 1.f};
  for (int q = 0; q < kD0; q++) idv[q] = in_div ? in_div[q] : 1.f;
  for (int j = 0; j < dims[nlayers]; j++) om[j] = out_mul ? out_mul[j] : 1.f;
  e = cudaMemcpyToSymbolAsync(c_in_div, idv, sizeof idv, 0, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyToSymbolAsync(c_out_mul, om, sizeof om, 0, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(s);                   // the staging image is a static buffer
}

int stencil_mlp_grid(const StencilLaunch& S) {
  const long long tiles = (long long)((S.ni + kTI - 1) / kTI) * ((S.nj + kTJ - 1) / kTJ) * S.nk;
  const long long cap = 148LL * 16;                  // 16 resident 128-thread blocks per SM
  return (int)(tiles < cap ? (tiles > 0 ? tiles : 1) : cap);
}

bool launch_stencil_mlp(int nlayers, const int* dims, bool relu_only, const StencilLaunch& S, cudaStream_t st) {
  const int p1 = pad_width(dims[1]), p2 = nlayers == 3 ? pad_width(dims[2]) : 0;
  const int grid = stencil_mlp_grid(S);
#define FORTIS_STENCIL_CASE(A, B)                                                                      \
  if (p1 == A && p2 == B) {                                                                            \
    if (relu_only) stencil_mlp_kernel<A, B, true><<<grid, 128, 0, st>>>(S);                            \
    else stencil_mlp_kernel<A, B, false><<<grid, 128, 0, st>>>(S);                                     \
    return true;                                                                                       \
  }
  FORTIS_STENCIL_CASE(20, 20)
  FORTIS_STENCIL_CASE(20, 0)
  FORTIS_STENCIL_CASE(16, 16)
  FORTIS_STENCIL_CASE(16, 0)
  FORTIS_STENCIL_CASE(32, 32)
  FORTIS_STENCIL_CASE(32, 0)
#undef FORTIS_STENCIL_CASE
  return false;                                      // mixed hidden widths: the caller takes the generic kernel
}

}  // namespace fortis
