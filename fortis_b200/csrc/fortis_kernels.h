// Launch interface of the CUDA-core kernels (fortis_kernels.cu) and of the tensor-core kernels (fortis_mlp_tc.cu).
#pragma once
#include <cuda_runtime.h>

#include <string>

#include "fortis_plan.h"

namespace fortis {

struct IoPlanDev;

enum { ACT_NONE = 0, ACT_RELU = 1, ACT_LEAKY = 2 };

constexpr int kSmallConstFloats = 8192;     // constant-bank budget of the fused small-MLP kernel
constexpr int kChecksumBlocks = 592;        // 4 x 148 SMs

void launch_gather(const IoPlanDev* P, const Access* slots, int n, const ArrayTable& T, const RowGeom& g, float* X, cudaStream_t s);
// `partials` (optional, scatter_grid(rows) doubles): per-block fp64 sums of the stored values in a fixed order
void launch_scatter(const IoPlanDev* P, const StoreTarget* stores, int nout, const ArrayTable& T, const RowGeom& g,
                    const float* Y, cudaStream_t s, double* partials = nullptr);
int scatter_grid(long long nrows);
void launch_linear_f32(const float* A, const float* W, const float* bias, float* C, long long M, int N, int K, int act,
                       float slope, const float* in_div, const float* out_mul, const float* relu_mask, cudaStream_t s);

// Immediate-address operands of the fast small-MLP kernel (see small_mlp_fast_kernel)
struct SmallFast {
  const float* in_ptr[32];        // per model input: array base + constant part of the offset
  float* out_ptr[8];              // per store
  int out_slot[8];
  int nstores;
  int si, sj, sk, oi, oj, ok;     // element strides of (ci, cj, kk) for inputs / stores
  int in_prog, out_prog;          // lifted expressions present
  unsigned nrows, count, ni;
};

struct SmallMlpLaunch {
  int use_fast; SmallFast fast;
  const IoPlanDev* GP; const Access* slots;          // gather plan (required)
  const IoPlanDev* SP; const StoreTarget* stores;    // scatter plan (null: only Yout is written)
  ArrayTable TG, TS;
  RowGeom g;
  int act[4]; float slope[4];
  int has_in_div, has_out_mul;
  float* Yout;                                       // optional (rows, nout) model output
  double* partials;                                  // optional per-block checksum partials [grid]
  int grid;                                          // 0: pick
};
bool small_mlp_supported(int nlayers, const int* dims);
int small_mlp_grid(long long nrows);
int small_mlp_pack(int nlayers, const int* dims, const float* const* W, const float* const* b, const float* in_div,
                   const float* out_mul, float* dst);
cudaError_t small_mlp_upload(const float* host, int nfloats, cudaStream_t s);
void launch_small_mlp(int nlayers, const int* dims, const SmallMlpLaunch& L, cudaStream_t s);

// ---- 3x3-stencil hosts: packed-FMA fused kernel (fortis_stencil_mlp.cu) ---------------------------------------
struct StencilLaunch {
  const float* in[3];             // per field: the element the CENTRE tap of point (0, 0) of plane 0 reads
  float* out[4]; int out_slot[4]; int nstores;      // per store: the element point (0, 0, 0) writes, and which model output
  long long sj_in, sk_in, sj_out, sk_out;           // element strides of the j index and of the plane (i has stride 1)
  int ni, nj, nk;                 // interior extent
  int has_in_div, has_out_mul;
  float slope[3];                 // act(v) = max(v, v * slope) per layer (ignored for hidden layers of an all-ReLU net)
  double* partials; double* sum; unsigned int* done;   // optional checksum (partials: stencil_mlp_grid() doubles)
};
bool stencil_mlp_supported(int nlayers, const int* dims);     // 27 inputs, hidden widths <= 32 (equal after padding), <= 4 outputs
cudaError_t stencil_mlp_upload(int nlayers, const int* dims, const float* const* W, const float* const* b, const float* in_div,
                               const float* out_mul, cudaStream_t s);
int stencil_mlp_grid(const StencilLaunch& S);
bool launch_stencil_mlp(int nlayers, const int* dims, bool relu_only, const StencilLaunch& S, cudaStream_t st);

// the same step on the tensor cores (fortis_stencil_tc.cu): three TF32 MMAs per product, rows in tensor memory
struct StencilTcModel;
bool stencil_tc_supported(int nlayers, const int* dims);      // 27 inputs, hidden widths <= 32, <= 4 outputs
StencilTcModel* stencil_tc_create(int nlayers, const int* dims, const float* const* W, const float* const* b, const float* in_div,
                                  const float* out_mul);
void stencil_tc_destroy(StencilTcModel* m);
int stencil_tc_grid(const StencilLaunch& S);
bool launch_stencil_tc(StencilTcModel* m, const StencilLaunch& S, int* status, cudaStream_t st);

// Test knobs of the tensor-core kernels (set through fortis_set_option "test_wait_limit" / "test_skip_stage"; both 0
// in normal operation): a short poll limit for the bounded barrier waits, and "the first CTA's TMA warp does not load
// its first stage", which makes a wait run out so that the give-up path can be exercised without hanging anything.
struct TcTestKnobs { unsigned int wait_limit; int skip_stage; int no_stage; };   // no_stage: fused MLP kernel, move every tile's inputs and outputs element by element
extern TcTestKnobs g_tc_test;

// ---- tensor-core fused MLP (fortis_mlp_tc.cu) ----------------------------------------------------------------
struct ModelHost;
struct TcModel;                                        // packed bf16 weights, TMA tensor maps, biases, scales
enum { PREC_F32 = 0, PREC_BF16 = 1, PREC_FP8W = 2, PREC_FP16 = 3 };
bool tc_model_supported(const ModelHost& M, std::string* why);
TcModel* tc_model_create(const ModelHost& M, int precision, cudaStream_t s, std::string* err);
int tc_debug_pack_layer(const float* W, const float* b, int cout, int cin, int last, int precision, uint16_t* image, float* bias,
                        float* scale, int* K, int* N);
void tc_model_destroy(TcModel* m);
struct TcLaunch {
  const IoPlanDev* GP; const Access* slots;          // gather plan, or null with X set
  const IoPlanDev* SP; const StoreTarget* stores;    // scatter plan, or null with Y set
  const int* slot_head; const int* store_next;       // per model output: first store (-1: none) and the chain
  // fast I/O (all accesses fp32, no lifted expressions, at most two stride classes): see fortis_mlp_tc.cu
  int fast_in, fast_out;
  long long cin[2][3], cout[2][3];                   // (si, sj, sk) per class
  const Access* store_by_slot;                       // [n_out], array < 0 where an output is not stored
  ArrayTable TG, TS;
  RowGeom g;
  const float* X;                                    // (rows, n_in) when there is no gather plan
  float* Y;                                          // (rows, n_out) when there is no scatter plan (may be set with SP too)
  double* partials;                                  // per-CTA checksum partials (size >= tc_grid())
  double* sum; unsigned int* done;                   // optional: fold the partials into *sum inside the kernel (done: zeroed counter)
  int* status;                                       // device word: 0 ok, else the code of the wait that gave up
};
int tc_grid(const TcModel* m, long long nrows);
void tc_set_pair_mode(int on);                      // 1 / 0: two-CTA clusters or one CTA per SM for models created from now on; -1: the default (clusters)
bool tc_forward(TcModel* m, const TcLaunch& L, cudaStream_t s, std::string* err);

// ---- fp32-class Linear layers on the tensor cores, three TF32 MMAs per product (fortis_mlp_f32tc.cu) ----------------
struct F32TcModel;                                     // split weights (W_hi, W_lo), TMA tensor maps, biases
bool f32tc_supported(const ModelHost& M, std::string* why);
F32TcModel* f32tc_create(const ModelHost& M, std::string* err);
void f32tc_destroy(F32TcModel* m);
struct F32TcLaunch {
  int fast_in; const Access* slots; ArrayTable TG; long long cin[2][3];   // gather fused into layer 0 (table-driven) ...
  const float* X;                                                          // ... or a materialised (rows, n_in) input
  int fast_out; const Access* store_by_slot; ArrayTable TS; long long cout[2][3];   // scatter fused into the last epilogue ...
  float* Y;                                                                // ... or a (rows, n_out) output
  RowGeom g;
  float* act[2]; long long act_ld;                   // two feature-major activation buffers [max width][act_ld], act_ld >= rows
  double* partials; double* sum; unsigned int* done; // optional checksum of the fused scatter (partials: f32tc_grid() doubles)
  int* status;
};
int f32tc_grid(long long nrows);
bool f32tc_forward(F32TcModel* m, const F32TcLaunch& L, cudaStream_t s, std::string* err);
// C[M][N] = A[M][K] . W[N][K]^T, row-major device operands (the memref entry fortis_gemm)
bool f32tc_gemm(const float* A, const float* W, float* C, long long M, int N, int K, int* status, cudaStream_t s, std::string* err);

// ---- conv3d network (fortis_conv3d.cu) -------------------------------------------------------------------------
struct ConvModel;
ConvModel* conv_model_create(const ModelHost& M, int precision, cudaStream_t s, std::string* err);
void conv_model_destroy(ConvModel* m);
int conv_model_status(ConvModel* m);
void conv_model_clear_status(ConvModel* m);        // 0, or the code of a bounded wait that gave up in the tensor-core conv kernel
// x (N,D,H,W,Cin) fp32 NDHWC on the device -> y (N,D,H,W,Cout)
bool conv_forward(ConvModel* m, const float* x, float* y, int N, int D, int H, int W, cudaStream_t s, std::string* err);
// single layer, NCDHW fp32 (the memref ABI of runtime/fortis_rt.c:128-131)
// networks of 2-D operator layers (NCHW fp32)
struct OpNet;
OpNet* opnet_create(const ModelHost& M, std::string* err);
void opnet_destroy(OpNet* m);
bool opnet_shape(const ModelHost& M, int H, int W, int* C, int* Ho, int* Wo, long long* max_elems_per_image);
bool opnet_forward(OpNet* m, const float* x, float* y, int N, int H, int W, cudaStream_t s, std::string* err);
bool conv3d_ncdhw(const float* x, const float* w, float* y, int N, int C, int D, int H, int W, int F, const int K[3],
                  const int stride[3], const int pad[3], cudaStream_t s, std::string* err);

// tensor-core conv network (fortis_conv3d_tc.cu): bf16 activations in a zero-padded channels-last volume
struct ConvTcModel;
bool conv_tc_supported(const ModelHost& M, std::string* why);
ConvTcModel* conv_tc_create(const ModelHost& M, bool f16, std::string* err);
void conv_tc_destroy(ConvTcModel* m);
bool conv_tc_forward(ConvTcModel* m, const float* x, float* y, int N, int D, int H, int W, cudaStream_t s, std::string* err);
int conv_tc_status(ConvTcModel* m);
void conv_tc_clear_status(ConvTcModel* m);

void launch_checksum(const void* data, long long n, int elt, double* partials, double* out, int accumulate, cudaStream_t s);
void launch_fold(const double* partials, int n, double* out, int accumulate, cudaStream_t s);

}  // namespace fortis
