// Fused gather -> small MLP -> scatter for 3x3-stencil hosts on the tensor cores, fp32-exact (<= 1e-5): the
// tensor-core form of fortis_stencil_mlp.cu (same operands, same host interface: StencilLaunch).
//
// Replaces the same reference code (driver/fortis_gather_emit.py:52-62 gather, the per-layer kernels of
// compiler/FortisFuse.cpp:587-655, fortis_scatter_k); layer semantics as mom6_zb/fwd_native_zb.f90:30-78.
//
// One thread per gridpoint, 128 gridpoints (a 32 x 4 tile) per group of four warps, four groups per CTA.  A layer
// y = act(W x + b) of 128 points is D[128 x N] = A[128 x 32] . B[N x 32]^T with N = 32 (hidden) or 16 (outputs):
//   * A lives in TENSOR MEMORY, lane = gridpoint, column = input: each thread writes ITS OWN row (tcgen05.st), reads its
//     own row of D (tcgen05.ld), applies bias and activation and writes the next layer's A row.  Thread = row = TMEM
//     lane end to end, so no operand ever crosses threads and nothing is staged or swizzled in shared memory.
//   * fp32 accuracy from TF32 MMAs: x = x_hi + x_lo, w = w_hi + w_lo (hi = nearest TF32, lo = the remainder), and
//     x.w ~ x_hi w_hi + x_lo w_hi + x_hi w_lo: three kind::tf32 MMAs per 8-wide k step, 12 per layer.  K = 32, so the
//     truncating fp32 accumulation of the tensor core costs ~2e-7; measured error against the fp64 oracle ~5e-7.
//   * B: all weights (hi and lo, 24 KB) sit in shared memory for the whole kernel, K-major, 128-byte swizzled.
//   * The 3 x 3 x 3 stencil inputs come from a (32+2) x (4+2) halo tile per group in shared memory (coalesced loads,
//     every input read from L2 once); outputs are stored coalesced along i; the checksum is folded in the launch.
//   * A group's four warps run gather -> MMA -> epilogue -> MMA -> ... for one tile at a time; the four groups of a CTA
//     are independent (own tile, own TMEM columns, own barrier) and hide each other's MMA round trips.
// Every mbarrier wait is bounded; on expiry the kernel records a code, leaves its loops and frees its tensor memory.
//
// MEASURED, and the reason this kernel is an option (fortis_set_option "stencil_tc" = "1") and not the default: on the
// 1440 x 1080 x 4 configuration it takes 0.59 - 0.61 ms against 0.365 ms for the packed-FMA kernel.  With layers this narrow
// the per-element work that stays on the CUDA cores (tensor-memory load, bias, activation, the TF32 split, tensor-memory
// store: 8-10 instructions per element of a 32-wide padded row) costs as much as computing the element with K / 2
// packed FMAs (10-14 instructions for K = 20-27): 1354 instructions per gridpoint against 1150, tensor pipe 12 % busy.
// The form pays from K of about 64 upwards, which is where fortis_mlp_f32tc.cu takes over.
#include <cuda_runtime.h>

#include <cstring>
#include <vector>

#include "fortis_kernels.h"
#include "fortis_tc.cuh"

namespace fortis {

using namespace tc;

namespace {

constexpr int kG = 4;                                  // groups of 128 threads per CTA
constexpr int kThreadsS = 128 * kG;
constexpr int kTI = 32, kTJ = 4, kPitch = 36, kRows = kTJ + 2, kNF = 3, kD0 = 9 * kNF;
constexpr int kKP = 32;                                // padded width of inputs and hidden layers (one 128-byte row of TF32)
constexpr int kNOut = 16;                              // padded width of the output layer (the smallest MMA N)
constexpr int kMatBytes = kKP * 128;                   // one 32-row K-major matrix: 4 KB
constexpr int kWBytes = 3 * 2 * kMatBytes;             // three layers x (hi, lo)
constexpr int kColsPerGroup = 128;                     // TMEM columns per group: A_hi 0-31, A_lo 32-63, D 64-95
enum { SST_MMA = 21, SST_ALIGN = 22 };

struct StencilTcParams {
  StencilLaunch S;
  const uint8_t* wimg;          // kWBytes: per layer hi then lo, rows = outputs, 128-byte swizzled
  const float* bias;            // [3][32]
  const float* in_div;          // [32] (ones where unused)
  const float* out_mul;         // [4]
  int nlayers;                  // 2 or 3; the output layer always uses weight slot 2
  int ksteps[3];                // 8-wide k steps per weight slot: ceil(inputs of that layer / 8)
  int* status;
  unsigned int wait_limit;
};

// kind::tf32, D = f32, A (tensor memory) and B (shared memory) K-major, M = 128
__device__ __forceinline__ constexpr uint32_t idesc_tf32_n(int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\telect.sync _|p, 0xffffffff;\n\tsetp.ne.b32 q, %4, 0;\n\t"
      "@p tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, q;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// rounds v[0..31] to TF32 in place and returns the remainders (exact in fp32; the MMA truncates them to TF32)
__device__ __forceinline__ void split_row(uint32_t (&hi)[kKP], uint32_t (&lo)[kKP]) {
#pragma unroll
  for (int j = 0; j < kKP; j++) {
    const float x = __uint_as_float(hi[j]);
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi[j] = h;
    lo[j] = __float_as_uint(x - __uint_as_float(h));
  }
}

__global__ void __launch_bounds__(kThreadsS, 1) stencil_mlp_tc_kernel(const __grid_constant__ StencilTcParams P) {
  __shared__ __align__(1024) uint8_t w_s[kWBytes];
  __shared__ float tile[kG][kNF][kRows][kPitch];
  __shared__ float bias_s[3][kKP];
  __shared__ float in_div_s[kKP];
  __shared__ __align__(8) unsigned long long bar_s[kG];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_s;
  __shared__ double wsum[kThreadsS / 32];
  const StencilLaunch& S = P.S;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = warp >> 2, quad = warp & 3;              // group; TMEM lane quadrant of this warp
  const int ti = lane, tj = quad;                        // position inside the group's 32 x 4 tile
  volatile int* abort_flag = &abort_s;
  const uint32_t wbase = smem_u32(w_s);
  if (wbase & 1023u) {
    if (threadIdx.x == 0) atomicCAS(P.status, 0, SST_ALIGN);
    return;
  }
  // weights, biases, input scales -> shared memory (generic-proxy writes, made visible to the MMA's async proxy below)
  for (int i = threadIdx.x; i < kWBytes / 16; i += kThreadsS)
    reinterpret_cast<uint4*>(w_s)[i] = __ldg(reinterpret_cast<const uint4*>(P.wimg) + i);
  for (int i = threadIdx.x; i < 3 * kKP; i += kThreadsS) (&bias_s[0][0])[i] = __ldg(P.bias + i);
  if (threadIdx.x < kKP) in_div_s[threadIdx.x] = __ldg(P.in_div + threadIdx.x);
  if (threadIdx.x == 0) {
    for (int i = 0; i < kG; i++) mbar_init(smem_u32(&bar_s[i]), 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t row_addr = tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(g * kColsPerGroup);   // this thread's lane, this group's columns
  const uint32_t grp_addr = tmem + (uint32_t)(g * kColsPerGroup);
  const uint32_t bar = smem_u32(&bar_s[g]);
  const uint64_t desc0 = make_kmajor_sw128_desc(0) & 0xFFFFFFFF00000000ull;
  auto bdesc = [&](int layer, int part) { return desc0 | (uint64_t)(((wbase + (layer * 2 + part) * kMatBytes) >> 4) & 0x3FFF); };
  // the 12 MMAs of one layer: hi.hi, lo.hi, hi.lo over four 8-wide k steps (one warp, one elected lane issues)
  // (Two accumulators with interleaved k steps, to shorten the chain of MMAs retiring into one accumulator, were
  // measured slower: the second accumulator costs a second tensor-memory load and 32 adds per row.)
  auto issue_layer = [&](int layer, uint32_t idesc) {
    const uint32_t d = grp_addr + 64, a_hi = grp_addr, a_lo = grp_addr + 32;
    const uint64_t bh = bdesc(layer, 0), bl = bdesc(layer, 1);
    const int nk = P.ksteps[layer];
    for (int k = 0; k < nk; k++) {
      mma_tf32_ts(d, a_hi + 8 * k, bh + (uint64_t)(2 * k), idesc, (uint32_t)k);
      mma_tf32_ts(d, a_lo + 8 * k, bh + (uint64_t)(2 * k), idesc, 1u);
      mma_tf32_ts(d, a_hi + 8 * k, bl + (uint64_t)(2 * k), idesc, 1u);
    }
    tc_commit(bar);
  };
  auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(1 + g) : "memory"); };
  // this thread's A row (32 fp32 values in `a`) -> A_hi / A_lo, then the group's warp 0 issues the layer
  auto run_layer = [&](uint32_t (&a)[kKP], int layer, uint32_t idesc) {
    uint32_t lo[kKP];
    split_row(a, lo);
    tmem_st32(row_addr, a);
    tmem_st32(row_addr + 32, lo);
    tmem_st_wait();
    tc_fence_before();
    group_sync();
    if (quad == 0) { tc_fence_after(); issue_layer(layer, idesc); }
  };

  const int tiles_i = (S.ni + kTI - 1) / kTI, tiles_j = (S.nj + kTJ - 1) / kTJ;
  const long long ntiles = (long long)tiles_i * tiles_j * S.nk;
  uint32_t par = 0;
  double csum = 0.0;
  for (long long t = (long long)blockIdx.x * kG + g; t < ntiles; t += (long long)gridDim.x * kG) {
    const int kk = (int)(t / ((long long)tiles_i * tiles_j));
    const int rem = (int)(t - (long long)kk * tiles_i * tiles_j);
    const int ci0 = (rem % tiles_i) * kTI, cj0 = (rem / tiles_i) * kTJ;
    group_sync();                                      // the group's previous tile has been read out of shared memory
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
          tile[g][f][r][ti] = (rok && ci0 - 1 + ti <= S.ni) ? __ldg(rowp + ti) : 0.f;
          if (ti < 2) tile[g][f][r][kTI + ti] = (rok && ci0 - 1 + kTI + ti <= S.ni) ? __ldg(rowp + kTI + ti) : 0.f;
        }
      }
    }
    group_sync();
    const int ci = ci0 + ti, cj = cj0 + tj;
    const bool live = ci < S.ni && cj < S.nj;            // rows outside the domain run through the MMAs as zeros
    uint32_t a[kKP];
#pragma unroll
    for (int f = 0; f < kNF; f++)
#pragma unroll
      for (int dj = 0; dj < 3; dj++)
#pragma unroll
        for (int di = 0; di < 3; di++) {
          float v = live ? tile[g][f][tj + dj][ti + di] : 0.f;
          if (S.has_in_div) v = __fdiv_rn(v, in_div_s[f * 9 + dj * 3 + di]);
          a[f * 9 + dj * 3 + di] = __float_as_uint(v);
        }
#pragma unroll
    for (int q = kD0; q < kKP; q++) a[q] = 0u;
    run_layer(a, 0, idesc_tf32_n(kKP));
    // ---- hidden layers: D -> bias, activation -> next A
    for (int l = 0; l + 1 < P.nlayers; l++) {
      if (!mbar_wait(bar, par, abort_flag, P.status, SST_MMA, P.wait_limit)) goto done;
      par ^= 1;
      tc_fence_after();
      tmem_ld32(row_addr + 64, a);
      tmem_ld_wait();
      const float slope = S.slope[l];
#pragma unroll
      for (int j = 0; j < kKP; j++) {
        const float v = __uint_as_float(a[j]) + bias_s[l][j];
        a[j] = __float_as_uint(fmaxf(v, v * slope));
      }
      const bool last_hidden = l + 2 == P.nlayers;
      run_layer(a, last_hidden ? 2 : 1, last_hidden ? idesc_tf32_n(kNOut) : idesc_tf32_n(kKP));
    }
    // ---- output layer: D (16 columns) -> bias, activation, output scale -> the host arrays
    {
      if (!mbar_wait(bar, par, abort_flag, P.status, SST_MMA, P.wait_limit)) goto done;
      par ^= 1;
      tc_fence_after();
      uint32_t d[kNOut];
      tmem_ld16(row_addr + 64, d);
      tmem_ld_wait();
      tc_fence_before();
      if (live) {
        const float slope = S.slope[P.nlayers - 1];
        float y[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const float v = __uint_as_float(d[j]) + bias_s[2][j];
          y[j] = fmaxf(v, v * slope);
          if (S.has_out_mul) y[j] *= __ldg(P.out_mul + j);
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
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
  if (S.partials) {
    // deterministic per-block partial, then the last block folds all partials into the step checksum in block order
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) csum += __shfl_down_sync(0xffffffffu, csum, o);
    if (lane == 0) wsum[warp] = csum;
    __syncthreads();
    if (threadIdx.x == 0) {
      double tsum = 0.0;
      for (int w = 0; w < kThreadsS / 32; w++) tsum += wsum[w];
      S.partials[blockIdx.x] = tsum;
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

// nearest TF32 value, ties away from zero (what cvt.rna.tf32.f32 does)
float tf32_round(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;
  u = (u + 0x1000u) & 0xffffe000u;
  float r;
  std::memcpy(&r, &u, 4);
  return r;
}

}  // namespace

struct StencilTcModel {
  uint8_t* wimg = nullptr;
  float *bias = nullptr, *in_div = nullptr, *out_mul = nullptr;
  int nlayers = 0;
  int ksteps[3] = {4, 4, 4};
};

bool stencil_tc_supported(int nlayers, const int* dims) {
  if (nlayers != 2 && nlayers != 3) return false;
  if (dims[0] != kD0 || dims[nlayers] < 1 || dims[nlayers] > 4) return false;
  for (int l = 1; l < nlayers; l++) if (dims[l] < 1 || dims[l] > kKP) return false;
  return true;
}

void stencil_tc_destroy(StencilTcModel* m) {
  if (!m) return;
  cudaFree(m->wimg); cudaFree(m->bias); cudaFree(m->in_div); cudaFree(m->out_mul);
  delete m;
}

// W[l] is (out, in) row-major (torch layout).  Weight slot 0 = first layer, 1 = second hidden layer (three-layer
// nets), 2 = output layer.  Row n of a matrix is 128 bytes (32 TF32 values, zero where padded); its 16-byte piece j
// is stored at piece j ^ (n & 7) (the 128-byte swizzle the K-major descriptor expects).
StencilTcModel* stencil_tc_create(int nlayers, const int* dims, const float* const* W, const float* const* b, const float* in_div,
                                  const float* out_mul) {
  if (!stencil_tc_supported(nlayers, dims)) return nullptr;
  std::vector<uint8_t> img(kWBytes, 0);
  std::vector<float> bias(3 * kKP, 0.f), idv(kKP, 1.f), om(4, 1.f);
  for (int l = 0; l < nlayers; l++) {
    const int slot = l == nlayers - 1 ? 2 : l, K = dims[l], N = dims[l + 1];
    float* hi = reinterpret_cast<float*>(img.data() + (slot * 2 + 0) * kMatBytes);
    float* lo = reinterpret_cast<float*>(img.data() + (slot * 2 + 1) * kMatBytes);
    for (int n = 0; n < N; n++) {
      for (int k = 0; k < K; k++) {
        const float w = W[l][(size_t)n * K + k], h = tf32_round(w);
        const int off = n * 32 + ((((k >> 2) ^ (n & 7)) << 2) | (k & 3));
        hi[off] = h;
        lo[off] = tf32_round(w - h);
      }
      bias[slot * kKP + n] = b[l] ? b[l][n] : 0.f;
    }
  }
  for (int q = 0; q < kD0; q++) idv[q] = in_div ? in_div[q] : 1.f;
  for (int j = 0; j < dims[nlayers]; j++) om[j] = out_mul ? out_mul[j] : 1.f;
  StencilTcModel* m = new StencilTcModel();
  m->nlayers = nlayers;
  for (int l = 0; l < nlayers; l++) m->ksteps[l == nlayers - 1 ? 2 : l] = (dims[l] + 7) / 8;
  if (cudaMalloc(&m->wimg, kWBytes) != cudaSuccess || cudaMalloc(&m->bias, bias.size() * 4) != cudaSuccess ||
      cudaMalloc(&m->in_div, idv.size() * 4) != cudaSuccess || cudaMalloc(&m->out_mul, om.size() * 4) != cudaSuccess) {
    cudaGetLastError();
    stencil_tc_destroy(m);
    return nullptr;
  }
  cudaMemcpy(m->wimg, img.data(), kWBytes, cudaMemcpyHostToDevice);
  cudaMemcpy(m->bias, bias.data(), bias.size() * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(m->in_div, idv.data(), idv.size() * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(m->out_mul, om.data(), om.size() * 4, cudaMemcpyHostToDevice);
  return m;
}

int stencil_tc_grid(const StencilLaunch& S) {
  const long long tiles = (long long)((S.ni + kTI - 1) / kTI) * ((S.nj + kTJ - 1) / kTJ) * S.nk;
  const long long ctas = (tiles + kG - 1) / kG;
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return (int)(ctas < sms ? (ctas > 0 ? ctas : 1) : sms);
}

bool launch_stencil_tc(StencilTcModel* m, const StencilLaunch& S, int* status, cudaStream_t st) {
  if (!m) return false;
  StencilTcParams P;
  P.S = S;
  P.wimg = m->wimg; P.bias = m->bias; P.in_div = m->in_div; P.out_mul = m->out_mul;
  P.nlayers = m->nlayers;
  for (int i = 0; i < 3; i++) P.ksteps[i] = m->ksteps[i];
  P.status = status;
  P.wait_limit = g_tc_test.wait_limit ? g_tc_test.wait_limit : kWaitLimit;
  stencil_mlp_tc_kernel<<<stencil_tc_grid(S), kThreadsS, 0, st>>>(P);
  return cudaGetLastError() == cudaSuccess;
}

}  // namespace fortis
