/* CPU restatement, in C, of the reference's native (Fortran) forward and of the host's own gather / scatter loops.
 * TEST INFRASTRUCTURE ONLY: the parity checker and the timed CPU baseline.  Nothing in the product links it.
 *
 *   Layer_apply loop order (inputs outer, outputs inner, then bias, then activation):
 *       mom6_zb/fwd_native_zb.f90:30-48   and its batched driver   mom6_zb/fwd_native_zb_batched.f90:11-20
 *   host gather of a stencil / column into x(:), and the stores of y(:) back into the host arrays:
 *       mom6_zb/zb_host.f90:77-100
 *   conv3d as cross-correlation with zero padding (what cuDNN is asked for):  runtime/fortis_rt.c:139-147
 *
 * The reference's CPU path is Fortran and this image has no Fortran compiler, so this is a port ("kind": "port").
 * Threads: OpenMP over columns, which is how a host would run independent columns on all its cores.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { ACT_NONE = 0, ACT_RELU = 1, ACT_LEAKY = 2 };

static inline float act_f(float v, int act, float slope) {
  if (act == ACT_RELU) return v > 0.f ? v : 0.f;
  if (act == ACT_LEAKY) return v > 0.f ? v : v * slope;
  return v;
}

/* y(out) = act(A(out,in) x + b) with the shipped loop order.  W is (out,in) row-major (torch layout), which is
 * the Fortran A(j,i) read with stride `in`; Wt is the same matrix stored (in,out) so the inner loop is unit
 * stride, as it is for the Fortran column-major A(j,i). */
static void layer_apply(const float* x, float* y, const float* Wt, const float* b, int nin, int nout, int act, float slope) {
  for (int j = 0; j < nout; j++) y[j] = 0.f;
  for (int i = 0; i < nin; i++) {
    const float xi = x[i];
    const float* w = Wt + (size_t)i * nout;
    for (int j = 0; j < nout; j++) y[j] = y[j] + xi * w[j];
  }
  for (int j = 0; j < nout; j++) y[j] = act_f(y[j] + b[j], act, slope);
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* X (ncols, dims[0]) row-major -> Y (ncols, dims[nlayers]).  Wt[l] is (dims[l], dims[l+1]) = W^T.
 * in_norms / out_norms may be NULL (mom6_zb/fwd_native_zb.f90:58-60, 74-76). */
void oracle_mlp_forward(const float* X, float* Y, long ncols, int nlayers, const int* dims,
                        const float* const* Wt, const float* const* b, const int* act, const float* slope,
                        const float* in_norms, const float* out_norms, int nthreads) {
  int wmax = 0;
  for (int l = 0; l <= nlayers; l++) if (dims[l] > wmax) wmax = dims[l];
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
#pragma omp parallel
  {
    float* h0 = (float*)malloc(sizeof(float) * wmax);
    float* h1 = (float*)malloc(sizeof(float) * wmax);
#pragma omp for schedule(static)
    for (long c = 0; c < ncols; c++) {
      const float* x = X + (size_t)c * dims[0];
      for (int i = 0; i < dims[0]; i++) h0[i] = in_norms ? x[i] / in_norms[i] : x[i];
      float *src = h0, *dst = h1;
      for (int l = 0; l < nlayers; l++) {
        layer_apply(src, dst, Wt[l], b[l], dims[l], dims[l + 1], act[l], slope[l]);
        float* t = src; src = dst; dst = t;
      }
      float* y = Y + (size_t)c * dims[nlayers];
      for (int j = 0; j < dims[nlayers]; j++) y[j] = out_norms ? src[j] * out_norms[j] : src[j];
    }
    free(h0); free(h1);
  }
}

/* The whole host step on the CPU for descriptor sets without expressions: per column, pick the inputs out of the
 * Fortran arrays, run the forward, store the outputs.  A column `c` of plane `kk` reads input slot q at
 *   in_arr[in_slot_arr[q]][ in_slot_off[q] + (c % ni) * in_si[a] + (c / ni) * in_sj[a] + kk * in_sk[a] ]
 * and writes output slot q likewise (offsets are 0-based element offsets precomputed from the descriptors). */
void oracle_step(long count, int nk, int ni,
                 int nin, const float* const* in_arr, const int* in_slot_arr, const long* in_slot_off,
                 const long* in_si, const long* in_sj, const long* in_sk,
                 int nout, float* const* out_arr, const int* out_slot_arr, const long* out_slot_off,
                 const long* out_si, const long* out_sj, const long* out_sk,
                 int nlayers, const int* dims, const float* const* Wt, const float* const* b, const int* act,
                 const float* slope, int nthreads, double* checksum) {
  int wmax = 0;
  for (int l = 0; l <= nlayers; l++) if (dims[l] > wmax) wmax = dims[l];
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
  double total = 0.0;
#pragma omp parallel reduction(+ : total)
  {
    float* h0 = (float*)malloc(sizeof(float) * wmax);
    float* h1 = (float*)malloc(sizeof(float) * wmax);
#pragma omp for schedule(static)
    for (long r = 0; r < count * nk; r++) {
      const long c = r % count, kk = r / count, ci = c % ni, cj = c / ni;
      for (int q = 0; q < nin; q++) {
        const int a = in_slot_arr[q];
        h0[q] = in_arr[a][in_slot_off[q] + ci * in_si[a] + cj * in_sj[a] + kk * in_sk[a]];
      }
      float *src = h0, *dst = h1;
      for (int l = 0; l < nlayers; l++) {
        layer_apply(src, dst, Wt[l], b[l], dims[l], dims[l + 1], act[l], slope[l]);
        float* t = src; src = dst; dst = t;
      }
      for (int q = 0; q < nout; q++) {
        const int a = out_slot_arr[q];
        out_arr[a][out_slot_off[q] + ci * out_si[a] + cj * out_sj[a] + kk * out_sk[a]] = src[q];
        total += (double)src[q];
      }
    }
    free(h0); free(h1);
  }
  if (checksum) *checksum = total;
}

/* NDHWC conv3d, K^3 cross-correlation, stride 1, zero padding `pad`, optional residual add, then activation.
 * x (N,D,H,W,C), w (F,C,K,K,K) torch layout, y (N,D,H,W,F). */
void oracle_conv3d_ndhwc(const float* x, const float* w, const float* bias, const float* residual, float* y,
                         int N, int D, int H, int W, int C, int F, int K, int pad, int act, float slope, int nthreads) {
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
  const long nvox = (long)N * D * H * W;
#pragma omp parallel for schedule(static)
  for (long v = 0; v < nvox; v++) {
    const int xw = (int)(v % W), xh = (int)((v / W) % H), xd = (int)((v / ((long)W * H)) % D), n = (int)(v / ((long)W * H * D));
    for (int f = 0; f < F; f++) {
      float acc = 0.f;
      for (int kd = 0; kd < K; kd++) {
        const int id = xd + kd - pad; if (id < 0 || id >= D) continue;
        for (int kh = 0; kh < K; kh++) {
          const int ih = xh + kh - pad; if (ih < 0 || ih >= H) continue;
          for (int kw = 0; kw < K; kw++) {
            const int iw = xw + kw - pad; if (iw < 0 || iw >= W) continue;
            const float* xp = x + ((((size_t)n * D + id) * H + ih) * W + iw) * C;
            const float* wp = w + (size_t)f * C * K * K * K + ((size_t)kd * K + kh) * K + kw;
            for (int c = 0; c < C; c++) acc += xp[c] * wp[(size_t)c * K * K * K];
          }
        }
      }
      float o = acc + (bias ? bias[f] : 0.f);
      if (residual) o += residual[(size_t)v * F + f];
      y[(size_t)v * F + f] = act_f(o, act, slope);
    }
  }
}
