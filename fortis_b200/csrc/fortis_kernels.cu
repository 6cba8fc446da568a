// CUDA-core kernels of the step: descriptor-driven gather and scatter (coalesced through a shared-memory
// transpose), the fp32 layer kernel (FFMA, bias + activation fused), the fused small-MLP kernel for stencil hosts
// (gather -> all layers in registers -> scatter in ONE launch, weights as constant-bank FFMA operands), and the
// deterministic fp64 checksum.
//
// Reference counterparts: fortis_gather_k / fortis_scatter_k (driver/fortis_gather_emit.py:52-62, 75-83),
// fortis_gemm + the bias/activation epilogue kernel (runtime/fortis_rt.c:45-75, compiler/FortisFuse.cpp:687-760).
#include "fortis_kernels.h"

#include <cstdio>

#include "fortis_device.cuh"

namespace fortis {

// ---------------------------------------------------------------------------------------------------------------
// gather: X[row, q] for a tile of 32 rows per block iteration.  Lanes run along rows (the host arrays' fastest
// index), so every slot is one coalesced 128-byte read; the tile is transposed through shared memory and written
// to X as contiguous rows.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_kernel(const IoPlanDev* __restrict__ P, const Access* __restrict__ slots,
                                                     ArrayTable T, RowGeom g, float* __restrict__ X) {
  extern __shared__ float tile[];                 // [32][n + 1]
  const int n = P->n, ld = n + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long nrows = g.count * g.nk;
  for (long long r0 = (long long)blockIdx.x * 32; r0 < nrows; r0 += (long long)gridDim.x * 32) {
    const long long row = r0 + lane;
    if (row < nrows) {
      long long ci, cj, kk;
      row_to_pos(g, row, &ci, &cj, &kk);
      double sc[kMaxScalars];
      if (P->nscalars) load_scalars(*P, T, ci, cj, kk, sc);
      for (int q = warp; q < n; q += 8) tile[lane * ld + q] = gather_value(*P, slots[q], T, q, ci, cj, kk, sc);
    }
    __syncthreads();
    const long long rows_here = min((long long)32, nrows - r0);
    const long long total = rows_here * n;
    float* dst = X + r0 * n;
    for (long long e = threadIdx.x; e < total; e += 256) dst[e] = tile[(e / n) * ld + (e % n)];
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------------------------
// scatter: one plane's worth of columns (or all planes when g.nk > 1).  Y tile read coalesced, stores issued with
// lanes along columns so that each store instruction writes 32 neighbouring host-array elements.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) scatter_kernel(const IoPlanDev* __restrict__ P, const StoreTarget* __restrict__ stores,
                                                      ArrayTable T, RowGeom g, const float* __restrict__ Y,
                                                      double* __restrict__ partials) {
  extern __shared__ float tile[];                 // [32][nout + 1]
  const int n = P->n, ld = n + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long nrows = g.count * g.nk;
  double csum = 0.0;
  for (long long r0 = (long long)blockIdx.x * 32; r0 < nrows; r0 += (long long)gridDim.x * 32) {
    const long long rows_here = min((long long)32, nrows - r0);
    const long long total = rows_here * n;
    const float* src = Y + r0 * n;
    for (long long e = threadIdx.x; e < total; e += 256) tile[(e / n) * ld + (e % n)] = src[e];
    __syncthreads();
    const long long row = r0 + lane;
    if (row < nrows) {
      long long ci, cj, kk;
      row_to_pos(g, row, &ci, &cj, &kk);
      double sc[kMaxScalars];
      if (P->nscalars) load_scalars(*P, T, ci, cj, kk, sc);
      for (int s = warp; s < P->nstores; s += 8) {
        const StoreTarget st = stores[s];
        const double v = scatter_value(*P, T, st.slot, tile[lane * ld + st.slot], sc);
        store_elem(T, st.a, access_offset(st.a, ci, cj, kk), v);
        csum += st.a.elt == 0 ? (double)(float)v : v;
      }
    }
    __syncthreads();
  }
  if (partials) {
    // deterministic per-block partial: shuffle tree per warp, then the warp results in index order
    __shared__ double wsum[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) csum += __shfl_down_sync(0xffffffffu, csum, o);
    if (lane == 0) wsum[warp] = csum;
    __syncthreads();
    if (threadIdx.x == 0) {
      double t = 0.0;
      for (int w = 0; w < 8; w++) t += wsum[w];
      partials[blockIdx.x] = t;
    }
  }
}

void launch_gather(const IoPlanDev* P, const Access* slots, int n, const ArrayTable& T, const RowGeom& g, float* X,
                   cudaStream_t s) {
  const long long nrows = g.count * g.nk;
  if (nrows <= 0) return;
  const size_t smem = (size_t)32 * (n + 1) * sizeof(float);
  static size_t gather_smem_set = 0;
  if (smem > 48 * 1024 && smem > gather_smem_set) {
    cudaFuncSetAttribute(gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gather_smem_set = smem;
  }
  const long long tiles = (nrows + 31) / 32;
  const int grid = (int)(tiles < 148 * 8 ? tiles : 148 * 8);
  gather_kernel<<<grid, 256, smem, s>>>(P, slots, T, g, X);
}

int scatter_grid(long long nrows) {
  const long long tiles = (nrows + 31) / 32;
  return (int)(tiles < 148 * 8 ? (tiles > 0 ? tiles : 1) : 148 * 8);
}

void launch_scatter(const IoPlanDev* P, const StoreTarget* stores, int nout, const ArrayTable& T, const RowGeom& g,
                    const float* Y, cudaStream_t s, double* partials) {
  const long long nrows = g.count * g.nk;
  if (nrows <= 0) return;
  const size_t smem = (size_t)32 * (nout + 1) * sizeof(float);
  static size_t scatter_smem_set = 0;
  if (smem > 48 * 1024 && smem > scatter_smem_set) {
    cudaFuncSetAttribute(scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    scatter_smem_set = smem;
  }
  scatter_kernel<<<scatter_grid(nrows), 256, smem, s>>>(P, stores, T, g, Y, partials);
}

// ---------------------------------------------------------------------------------------------------------------
// fp32 layer: C[M,N] = act(A[M,K] . W[N,K]^T + b), optional per-column input divide / output multiply (the ZB
// network's norms) and a final ReLU on masked outputs.  128x64 block tile, 16-deep k slices, 8x4 outputs per
// thread, both operands staged k-major in shared memory.
// ---------------------------------------------------------------------------------------------------------------
constexpr int LBM = 128, LBN = 64, LBK = 16;

__device__ __forceinline__ float act_apply(float v, int act, float slope) {
  if (act == ACT_RELU) return fmaxf(v, 0.f);
  if (act == ACT_LEAKY) return v > 0.f ? v : v * slope;
  return v;
}

__global__ void __launch_bounds__(256) linear_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                                                         const float* __restrict__ bias, float* __restrict__ C,
                                                         long long M, int N, int K, int act, float slope,
                                                         const float* __restrict__ in_div,
                                                         const float* __restrict__ out_mul,
                                                         const float* __restrict__ relu_mask) {
  __shared__ float As[LBK][LBM + 4];
  __shared__ float Ws[LBK][LBN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;            // 16 x 16 threads; thread owns rows ty*8.., cols tx*4..
  const long long m0 = (long long)blockIdx.x * LBM;
  const int n0 = blockIdx.y * LBN;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += LBK) {
    // A tile: 128 rows x 16 k.  Thread loads 8 elements: row = tid / 2 (+0), k = (tid % 2) * 8 + e
    {
      const int r = tid >> 1, kb = (tid & 1) * 8;
      const long long row = m0 + r;
#pragma unroll
      for (int e = 0; e < 8; e++) {
        const int k = k0 + kb + e;
        float v = 0.f;
        if (row < M && k < K) {
          v = A[row * K + k];
          if (in_div) v = __fdiv_rn(v, in_div[k]);
        }
        As[kb + e][r] = v;
      }
    }
    // W tile: 64 rows(n) x 16 k.  Thread loads 4 elements: n = tid / 4, k = (tid % 4) * 4 + e
    {
      const int r = tid >> 2, kb = (tid & 3) * 4;
      const int nn = n0 + r;
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int k = k0 + kb + e;
        Ws[kb + e][r] = (nn < N && k < K) ? W[(long long)nn * K + k] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < LBK; k++) {
      float a[8], w[4];
      const float4 a0 = *(const float4*)&As[k][ty * 8], a1 = *(const float4*)&As[k][ty * 8 + 4];
      const float4 w0 = *(const float4*)&Ws[k][tx * 4];
      a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w; a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
      w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w;
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const long long row = m0 + ty * 8 + i;
    if (row >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int nn = n0 + tx * 4 + j;
      if (nn >= N) continue;
      float v = acc[i][j] + (bias ? bias[nn] : 0.f);
      v = act_apply(v, act, slope);
      if (out_mul) v = v * out_mul[nn];
      if (relu_mask && relu_mask[nn] != 0.f) v = fmaxf(v, 0.f);
      C[row * N + nn] = v;
    }
  }
}

void launch_linear_f32(const float* A, const float* W, const float* bias, float* C, long long M, int N, int K, int act,
                       float slope, const float* in_div, const float* out_mul, const float* relu_mask, cudaStream_t s) {
  if (M <= 0) return;
  dim3 grid((unsigned)((M + LBM - 1) / LBM), (unsigned)((N + LBN - 1) / LBN));
  linear_f32_kernel<<<grid, 256, 0, s>>>(A, W, bias, C, M, N, K, act, slope, in_div, out_mul, relu_mask);
}

// ---------------------------------------------------------------------------------------------------------------
// fused small MLP (stencil hosts): one thread per gridpoint.  The thread gathers its own NIN inputs straight from
// the host arrays (lanes along i: coalesced, neighbours' halo reads hit L1), runs every layer with activations in
// registers and the weights as constant-bank operands of the FFMAs, and stores its outputs straight into the host
// arrays.  No X, no Y, no intermediate ever touches HBM: 4*(NIN_distinct + NOUT) bytes per point.
// Loop order per layer is the shipped native forward's (inputs outer, outputs inner, then bias, then activation:
// mom6_zb/fwd_native_zb.f90:36-47).
// ---------------------------------------------------------------------------------------------------------------
__constant__ float c_small[kSmallConstFloats];

// Constant-bank layout (floats), fixed by the layer widths so that every weight is an immediate-address operand:
//   W0 [D0][D1] | b0 [D1] | W1 [D1][D2] | b1 [D2] | (W2 [D2][D3] | b2 [D3]) | in_div [D0] | out_mul [NOUT]
template <int D0, int D1, int D2, int D3>
struct SmallLayout {
  static constexpr int NOUT = D3 ? D3 : D2;
  static constexpr int w0 = 0, b0 = w0 + D0 * D1, w1 = b0 + D1, b1 = w1 + D1 * D2, w2 = b1 + D2, b2 = w2 + D2 * D3,
                       in_div = b2 + D3, out_mul = in_div + D0, total = out_mul + NOUT;
};

struct SmallMlpMeta {
  int act[4];
  float slope[4];
  int has_in_div, has_out_mul;
};

template <int K, int N, int OFF_W, int OFF_B>
__device__ __forceinline__ void small_layer(const float (&x)[K], float (&y)[N], int act, float slope) {
#pragma unroll
  for (int j = 0; j < N; j++) y[j] = 0.f;
#pragma unroll
  for (int i = 0; i < K; i++) {
#pragma unroll
    for (int j = 0; j < N; j++) y[j] = fmaf(x[i], c_small[OFF_W + i * N + j], y[j]);
  }
#pragma unroll
  for (int j = 0; j < N; j++) y[j] = act_apply(y[j] + c_small[OFF_B + j], act, slope);
}

template <int D0, int D1, int D2, int D3>      // D3 == 0: two layers D0 -> D1 -> D2
__global__ void __launch_bounds__(128) small_mlp_fused_kernel(const IoPlanDev* __restrict__ GP, const Access* __restrict__ slots,
                                                              const IoPlanDev* __restrict__ SP, const StoreTarget* __restrict__ stores,
                                                              ArrayTable TG, ArrayTable TS, RowGeom g, SmallMlpMeta meta,
                                                              float* __restrict__ Yout, double* __restrict__ partials) {
  using LY = SmallLayout<D0, D1, D2, D3>;
  constexpr int NOUT = LY::NOUT;
  const long long nrows = g.count * g.nk;
  double csum = 0.0;
  for (long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x; row < nrows; row += (long long)gridDim.x * blockDim.x) {
    long long ci, cj, kk;
    row_to_pos(g, row, &ci, &cj, &kk);
    float x[D0];
    {
      double sc[kMaxScalars];
      if (GP->nscalars) load_scalars(*GP, TG, ci, cj, kk, sc);
#pragma unroll
      for (int q = 0; q < D0; q++) {
        float v = gather_value(*GP, slots[q], TG, q, ci, cj, kk, sc);
        if (meta.has_in_div) v = __fdiv_rn(v, c_small[LY::in_div + q]);
        x[q] = v;
      }
    }
    float h1[D1];
    small_layer<D0, D1, LY::w0, LY::b0>(x, h1, meta.act[0], meta.slope[0]);
    float y[NOUT];
    if constexpr (D3 == 0) {
      small_layer<D1, D2, LY::w1, LY::b1>(h1, y, meta.act[1], meta.slope[1]);
    } else {
      float h2[D2];
      small_layer<D1, D2, LY::w1, LY::b1>(h1, h2, meta.act[1], meta.slope[1]);
      small_layer<D2, D3, LY::w2, LY::b2>(h2, y, meta.act[2], meta.slope[2]);
    }
    if (meta.has_out_mul) {
#pragma unroll
      for (int j = 0; j < NOUT; j++) y[j] = y[j] * c_small[LY::out_mul + j];
    }
    if (Yout) {
#pragma unroll
      for (int j = 0; j < NOUT; j++) Yout[row * NOUT + j] = y[j];
    }
    if (SP) {
      double sc[kMaxScalars];
      if (SP->nscalars) load_scalars(*SP, TS, ci, cj, kk, sc);
      for (int s = 0; s < SP->nstores; s++) {
        const StoreTarget st = stores[s];
        float yv = 0.f;
#pragma unroll
        for (int j = 0; j < NOUT; j++) if (st.slot == j) yv = y[j];
        const double v = scatter_value(*SP, TS, st.slot, yv, sc);
        store_elem(TS, st.a, access_offset(st.a, ci, cj, kk), v);
        csum += st.a.elt == 0 ? (double)(float)v : v;
      }
    }
  }
  if (partials) {
    // deterministic per-block partial: warp shuffle tree then a fixed-order sum of the warp results
    __shared__ double wsum[4];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) csum += __shfl_down_sync(0xffffffffu, csum, o);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = csum;
    __syncthreads();
    if (threadIdx.x == 0) partials[blockIdx.x] = (wsum[0] + wsum[1]) + (wsum[2] + wsum[3]);
  }
}

// Fast-addressing variant: when every input slot shares one (si, sj, sk) stride triple and every array is fp32, the
// per-slot base pointers travel as kernel parameters (constant bank, immediate addresses) and a point's 27 loads
// are `ptr[q][pos]` with ONE position computed per point in 32-bit arithmetic.  Same arithmetic as the generic
// kernel; only the address computation differs.
template <int D0, int D1, int D2, int D3, bool PROG>
__global__ void __launch_bounds__(128) small_mlp_fast_kernel(SmallFast F, const IoPlanDev* __restrict__ GP,
                                                             const IoPlanDev* __restrict__ SP, ArrayTable TG, ArrayTable TS,
                                                             SmallMlpMeta meta, float* __restrict__ Yout,
                                                             double* __restrict__ partials) {
  using LY = SmallLayout<D0, D1, D2, D3>;
  constexpr int NOUT = LY::NOUT;
  const unsigned nrows = F.nrows, count = F.count, ni = F.ni;
  double csum = 0.0;
  for (unsigned row = blockIdx.x * blockDim.x + threadIdx.x; row < nrows; row += gridDim.x * blockDim.x) {
    const unsigned kk = row / count, col = row - kk * count, cj = col / ni, ci = col - cj * ni;
    const int pos = (int)ci * F.si + (int)cj * F.sj + (int)kk * F.sk;
    float x[D0];
#pragma unroll
    for (int q = 0; q < D0; q++) x[q] = __ldg(F.in_ptr[q] + pos);
    if (PROG && F.in_prog) {
      double sc[kMaxScalars];
      if (GP->nscalars) load_scalars(*GP, TG, ci, cj, kk, sc);
#pragma unroll
      for (int q = 0; q < D0; q++) x[q] = (float)eval_prog(GP->prog, (double)x[q], sc, TG, q);
    }
    if (meta.has_in_div) {
#pragma unroll
      for (int q = 0; q < D0; q++) x[q] = __fdiv_rn(x[q], c_small[LY::in_div + q]);
    }
    float h1[D1];
    small_layer<D0, D1, LY::w0, LY::b0>(x, h1, meta.act[0], meta.slope[0]);
    float y[NOUT];
    if constexpr (D3 == 0) {
      small_layer<D1, D2, LY::w1, LY::b1>(h1, y, meta.act[1], meta.slope[1]);
    } else {
      float h2[D2];
      small_layer<D1, D2, LY::w1, LY::b1>(h1, h2, meta.act[1], meta.slope[1]);
      small_layer<D2, D3, LY::w2, LY::b2>(h2, y, meta.act[2], meta.slope[2]);
    }
    if (meta.has_out_mul) {
#pragma unroll
      for (int j = 0; j < NOUT; j++) y[j] = y[j] * c_small[LY::out_mul + j];
    }
    if (Yout) {
#pragma unroll
      for (int j = 0; j < NOUT; j++) Yout[(size_t)row * NOUT + j] = y[j];
    }
    if (F.nstores) {
      double sc[kMaxScalars];
      if (PROG && F.out_prog && SP->nscalars) load_scalars(*SP, TS, ci, cj, kk, sc);
      const int opos = (int)ci * F.oi + (int)cj * F.oj + (int)kk * F.ok;
#pragma unroll
      for (int s = 0; s < 8; s++) {
        if (s < F.nstores) {
          float yv = 0.f;
#pragma unroll
          for (int j = 0; j < NOUT; j++) if (F.out_slot[s] == j) yv = y[j];
          if (PROG && F.out_prog) yv = (float)eval_prog(SP->prog, (double)yv, sc, TS, F.out_slot[s]);
          F.out_ptr[s][opos] = yv;
          csum += (double)yv;
        }
      }
    }
  }
  if (partials) {
    __shared__ double wsum[4];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) csum += __shfl_down_sync(0xffffffffu, csum, o);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = csum;
    __syncthreads();
    if (threadIdx.x == 0) partials[blockIdx.x] = (wsum[0] + wsum[1]) + (wsum[2] + wsum[3]);
  }
}

bool small_mlp_supported(int nlayers, const int* dims) {
  if (nlayers == 2) return dims[0] == 27 && dims[1] == 20 && dims[2] == 3;
  if (nlayers == 3) return dims[0] == 27 && dims[1] == 20 && dims[2] == 20 && dims[3] == 3;
  return false;
}

int small_mlp_grid(long long nrows) {
  const long long blocks = (nrows + 127) / 128;
  const long long cap = 148LL * 16;             // 16 resident 128-thread CTAs per SM cover the machine once
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

int small_mlp_pack(int nlayers, const int* dims, const float* const* W, const float* const* b, const float* in_div,
                   const float* out_mul, float* dst) {
  // dst receives the constant-bank image described at SmallLayout; W[l] is (out, in) row-major (torch layout)
  int o = 0;
  for (int l = 0; l < nlayers; l++) {
    const int K = dims[l], N = dims[l + 1];
    for (int i = 0; i < K; i++)
      for (int j = 0; j < N; j++) dst[o + i * N + j] = W[l][(size_t)j * K + i];
    o += K * N;
    for (int j = 0; j < N; j++) dst[o + j] = b[l] ? b[l][j] : 0.f;
    o += N;
  }
  for (int i = 0; i < dims[0]; i++) dst[o + i] = in_div ? in_div[i] : 1.f;
  o += dims[0];
  for (int j = 0; j < dims[nlayers]; j++) dst[o + j] = out_mul ? out_mul[j] : 1.f;
  o += dims[nlayers];
  return o;
}

cudaError_t small_mlp_upload(const float* host, int nfloats, cudaStream_t s) {
  if (nfloats > kSmallConstFloats) return cudaErrorInvalidValue;
  return cudaMemcpyToSymbolAsync(c_small, host, sizeof(float) * nfloats, 0, cudaMemcpyHostToDevice, s);
}

void launch_small_mlp(int nlayers, const int* dims, const SmallMlpLaunch& L, cudaStream_t s) {
  const long long nrows = L.g.count * L.g.nk;
  if (nrows <= 0) return;
  SmallMlpMeta m;
  for (int l = 0; l < 4; l++) { m.act[l] = L.act[l]; m.slope[l] = L.slope[l]; }
  m.has_in_div = L.has_in_div; m.has_out_mul = L.has_out_mul;
  const int grid = L.grid > 0 ? L.grid : small_mlp_grid(nrows);
  if (L.use_fast) {
    const bool prog = L.fast.in_prog || L.fast.out_prog;
    if (nlayers == 2 && prog)
      small_mlp_fast_kernel<27, 20, 3, 0, true><<<grid, 128, 0, s>>>(L.fast, L.GP, L.SP, L.TG, L.TS, m, L.Yout, L.partials);
    else if (nlayers == 2)
      small_mlp_fast_kernel<27, 20, 3, 0, false><<<grid, 128, 0, s>>>(L.fast, L.GP, L.SP, L.TG, L.TS, m, L.Yout, L.partials);
    else if (prog)
      small_mlp_fast_kernel<27, 20, 20, 3, true><<<grid, 128, 0, s>>>(L.fast, L.GP, L.SP, L.TG, L.TS, m, L.Yout, L.partials);
    else
      small_mlp_fast_kernel<27, 20, 20, 3, false><<<grid, 128, 0, s>>>(L.fast, L.GP, L.SP, L.TG, L.TS, m, L.Yout, L.partials);
    return;
  }
  if (nlayers == 2)
    small_mlp_fused_kernel<27, 20, 3, 0><<<grid, 128, 0, s>>>(L.GP, L.slots, L.SP, L.stores, L.TG, L.TS, L.g, m, L.Yout, L.partials);
  else
    small_mlp_fused_kernel<27, 20, 20, 3><<<grid, 128, 0, s>>>(L.GP, L.slots, L.SP, L.stores, L.TG, L.TS, L.g, m, L.Yout, L.partials);
}

// ---------------------------------------------------------------------------------------------------------------
// checksum: fp64 sum of an array in a fixed order (so that 1, 2, 4 or 8 ranks and repeated runs agree bit for
// bit): kChecksumBlocks blocks each sum a contiguous chunk into partials[block]; a second launch folds the
// partials in index order.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) checksum_partial_kernel(const void* __restrict__ data, long long n, int elt,
                                                               double* __restrict__ partials) {
  const long long per = (n + gridDim.x - 1) / gridDim.x;
  const long long b = (long long)blockIdx.x * per, e = min(n, b + per);
  double acc = 0.0;
  for (long long i = b + threadIdx.x; i < e; i += 256)
    acc += elt == 0 ? (double)((const float*)data)[i] : ((const double*)data)[i];
  __shared__ double wsum[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < 8; w++) t += wsum[w];
    partials[blockIdx.x] = t;
  }
}

__global__ void checksum_fold_kernel(const double* __restrict__ partials, int n, double* __restrict__ out, int accumulate) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double t = accumulate ? *out : 0.0;
    for (int i = 0; i < n; i++) t += partials[i];
    *out = t;
  }
}

void launch_checksum(const void* data, long long n, int elt, double* partials, double* out, int accumulate, cudaStream_t s) {
  checksum_partial_kernel<<<kChecksumBlocks, 256, 0, s>>>(data, n, elt, partials);
  checksum_fold_kernel<<<1, 32, 0, s>>>(partials, kChecksumBlocks, out, accumulate);
}

void launch_fold(const double* partials, int n, double* out, int accumulate, cudaStream_t s) {
  checksum_fold_kernel<<<1, 32, 0, s>>>(partials, n, out, accumulate);
}

}  // namespace fortis
