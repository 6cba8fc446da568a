// fp32-class Linear layers on the tensor cores: C = act(A . W^T + b) with every product formed as three TF32 MMAs
//     A . W  ~=  A_hi . W_hi + A_hi . W_lo + A_lo . W_hi        (x_hi = tf32(x), x_lo = x - x_hi, accumulation in fp32)
// which keeps 21 significant bits per operand: 9e-7 relative L2 against fp64 on the 244 -> 768 x4 -> 128 column network,
// the same as fp32 FFMA arithmetic, at six bf16-MMA-equivalents per multiply-add instead of one FFMA per MAC.
//
// Replaces, for the fp32 precision, the reference's large-batch lowering of a Linear layer: fortis_gemm = cuBLAS SGEMM on
// pre-transposed weights plus a separate bias / activation kernel (runtime/fortis_rt.c:45-75, compiler/FortisFuse.cpp:616-624,
// 687-760), with fortis_gather_k in front and fortis_scatter_k behind (driver/fortis_gather_emit.py:52-62, 75-83): the
// gather is fused into the first layer's operand load, bias + activation into every epilogue, the scatter (and the fp64
// checksum) into the last one.  Activations travel between layers in fp32, feature-major ([feature][row]: the memory
// order of a Fortran (ncol, nlev) array), so both the epilogue's stores and the next layer's loads are coalesced with
// one thread per row.
//
// One persistent CTA per SM, output tiles of 128 rows x n_tile (<= 256) features, K in steps of 32:
//   * warps 2-5 (thread = row) load the tile's activations (from the host arrays through the slot table, from a
//     feature-major buffer, or from a row-major matrix), split them and write A_hi / A_lo into shared memory in the
//     K-major 128-byte-swizzled layout the MMA reads;
//   * warp 0 brings the matching W_hi / W_lo tiles (split once on the host or by a kernel) with two TMA loads;
//   * warp 1 issues, per 8-wide k step, the three kind::tf32 MMAs (M = 128, N = n_tile) into a 256-column accumulator
//     in tensor memory;
//   * warps 6-9 (thread = row) read the accumulator, add the bias, apply the activation and store.
// The tensor core adds into its fp32 accumulator with truncation, not rounding: measured on this kernel, a relative
// bias of -6e-9 per unit of K (-4.7e-6 at K = 768, 2.2e-5 over the five layers of the column network).  So K is
// accumulated in chunks of 128: after each chunk the epilogue warps add the chunk's accumulator into a running sum
// held in the other 256 tensor-memory columns with IEEE additions (tcgen05.ld, FADD, tcgen05.st), which divides the
// bias by the number of chunks; the last chunk's pass goes straight on to bias, activation and store.
// Two stages of 96 KB (A_hi, A_lo 16 KB each; W_hi, W_lo up to 32 KB each).  Every barrier wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "fortis_device.cuh"
#include "fortis_kernels.h"
#include "fortis_model.h"
#include "fortis_tc.cuh"

namespace fortis {

namespace {

using namespace tc;

constexpr int kM = 128;                    // rows per tile
constexpr int kKt = 32;                    // k per stage: one 128-byte swizzle row of fp32
constexpr int kNtMax = 256;                // widest output tile (the MMA's N)
constexpr int kStagesF = 2;
constexpr int kChunkKt = 4;                // k steps of 32 accumulated in the tensor core before the sum is taken over (K = 128)
constexpr int kABytes = kM * kKt * 4;      // 16 KB per split half
constexpr int kWBytes = kNtMax * kKt * 4;  // 32 KB per split half
constexpr int kStageBytesF = 2 * kABytes + 2 * kWBytes;   // 96 KB
constexpr int kBarF = 128;
constexpr int kTabIn = 768, kTabOut = 256;     // widest gathered input / scattered output the tables hold
constexpr int kTabBytesF = kTabIn * 5 + kTabOut * 5 + 2 * kMaxArrays * 8 + 64;
constexpr int kSmemF = kStagesF * kStageBytesF + kBarF + kTabBytesF + 64;
constexpr int kThreadsF = 320;
enum { FST_FULL = 21, FST_EMPTY = 22, FST_ACC_FULL = 23, FST_ACC_EMPTY = 24, FST_ALIGN = 25 };
enum { A_FEATURE_MAJOR = 0, A_ROW_MAJOR = 1, A_GATHER = 2 };
enum { C_FEATURE_MAJOR = 0, C_ROW_MAJOR = 1, C_SCATTER = 2 };

struct StrideClassF { long long si, sj, sk; };

struct F32Params {
  CUtensorMap map_hi, map_lo;            // W_hi / W_lo [N_pad][K_pad] fp32, box 32 x n_tile
  int K_pad, N_pad, n_tile, K_real, N_real;
  const float* bias;                     // [N_pad] or null
  float slope;                           // act(v) = max(v, v * slope)
  const float* in_div;                   // first layer only, optional
  const float* out_mul;                  // last layer only, optional
  const float* relu_mask;                // last layer only, optional
  int a_mode; const float* A; long long lda;
  const Access* slots; ArrayTable TG; StrideClassF cin[2]; RowGeom g;
  int c_mode; float* C; long long ldc;
  const Access* store_by_slot; ArrayTable TS; StrideClassF cout[2];
  long long nrows;
  double* partials; double* sum; unsigned int* done;
  int* status;
};

// instruction descriptor of kind::tf32: D = f32, A = B = tf32 (format code 2), both K-major, M = 128, N at run time
__device__ __forceinline__ uint32_t idesc_tf32(int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kM >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\telect.sync _|p, 0xffffffff;\n\tsetp.ne.b32 q, %4, 0;\n\t"
      "@p tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, q;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// x = hi + lo with hi the nearest TF32 value (10 explicit mantissa bits); lo is exact in fp32 and is truncated to TF32
// by the MMA, which leaves 21 significant bits
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  uint32_t h;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
  hi = __uint_as_float(h);
  lo = x - hi;
}

__device__ __forceinline__ float act_slope(float v, float slope) { return fmaxf(v, v * slope); }

__global__ void __launch_bounds__(kThreadsF, 1) linear_tf32x3_kernel(const __grid_constant__ F32Params P) {
  extern __shared__ __align__(1024) uint8_t smem[];
  // Programmatic dependent launch: the next layer's CTAs may be scheduled as SMs free up; they set up, start streaming
  // their weights, and wait (griddepcontrol.wait in the warps that read or write activations) for this grid to finish.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t base = smem_u32(smem);
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicCAS(P.status, 0, FST_ALIGN);
    return;
  }
  uint8_t* tail = smem + kStagesF * kStageBytesF;
  const uint32_t bars = base + kStagesF * kStageBytesF;
  // barrier block: full [2] | empty [2] | acc_full [2] | acc_empty [2]; tmem base 64, abort flag 68, checksum scratch [72,104)
  const uint32_t bar_full = bars, bar_empty = bars + 16, bar_acc_full = bars + 32, bar_acc_empty = bars + 48;
  uint32_t* tmem_slot = (uint32_t*)(tail + 64);
  volatile int* abort_flag = (volatile int*)(tail + 68);
  uint32_t* s_off = (uint32_t*)(tail + kBarF);
  uint32_t* o_off = s_off + kTabIn;
  uint8_t* s_code = (uint8_t*)(o_off + kTabOut);
  uint8_t* o_code = s_code + kTabIn;
  const float** s_base_in = (const float**)(((uintptr_t)(o_code + kTabOut) + 15) & ~(uintptr_t)15);
  float** s_base_out = (float**)(s_base_in + kMaxArrays);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntn = P.N_pad / P.n_tile;
  const long long ntm = (P.nrows + kM - 1) / kM, ntiles = ntm * ntn;
  const int nkt = P.K_pad / kKt;
  const uint32_t w_bytes = (uint32_t)(P.n_tile * kKt * 4);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesF; s++) { mbar_init(bar_full + 8 * s, 1 + kM); mbar_init(bar_empty + 8 * s, 1); }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, kM);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < kMaxArrays) {
    s_base_in[threadIdx.x] = (const float*)P.TG.base[threadIdx.x];
    s_base_out[threadIdx.x] = (float*)P.TS.base[threadIdx.x];
  }
  if (P.a_mode == A_GATHER)
    for (int q = threadIdx.x; q < kTabIn; q += kThreadsF) {
      uint8_t code = 0xFF; uint32_t off = 0;
      if (q < P.K_real) {
        const Access a = P.slots[q];
        code = (uint8_t)(a.array | ((a.si == P.cin[0].si && a.sj == P.cin[0].sj && a.sk == P.cin[0].sk) ? 0 : 0x80));
        off = (uint32_t)a.off0;
      }
      s_code[q] = code; s_off[q] = off;
    }
  if (P.c_mode == C_SCATTER)
    for (int n = threadIdx.x; n < kTabOut; n += kThreadsF) {
      uint8_t code = 0xFF; uint32_t off = 0;
      if (n < P.N_real && P.store_by_slot[n].array >= 0) {
        const Access a = P.store_by_slot[n];
        code = (uint8_t)(a.array | ((a.si == P.cout[0].si && a.sj == P.cout[0].sj && a.sk == P.cout[0].sk) ? 0 : 0x80));
        off = (uint32_t)a.off0;
      }
      o_code[n] = code; o_off[n] = off;
    }
  if (warp == 0 && lane < 2)
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(lane ? &P.map_lo : &P.map_hi)) : "memory");
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA: the W_hi / W_lo tiles of every stage
    uint32_t s = 0, ph = 0;
    bool stop = false;
    for (long long t = blockIdx.x; t < ntiles && !stop; t += gridDim.x) {
      const int n0 = (int)(t % ntn) * P.n_tile;
      for (int kt = 0; kt < nkt; kt++) {
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, P.status, FST_EMPTY)) { stop = true; break; }
        mbar_expect_tx(bar_full + 8 * s, 2 * w_bytes);
        const uint32_t st = base + s * kStageBytesF + 2 * kABytes;
        tma_load_2d(st, &P.map_hi, kt * kKt, n0, bar_full + 8 * s);
        tma_load_2d(st + kWBytes, &P.map_lo, kt * kKt, n0, bar_full + 8 * s);
        if (++s == kStagesF) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    uint32_t s = 0, ph = 0, chunk_it = 0;
    const uint64_t desc_hi = make_kmajor_sw128_desc(0) & 0xFFFFFFFF00000000ull;
    const uint32_t idesc = idesc_tf32(P.n_tile);
    for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
      for (int kt0 = 0; kt0 < nkt; kt0 += kChunkKt, chunk_it++) {
        // the chunk accumulator (columns 0..255) is free again once the epilogue warps have taken the previous chunk over
        mbar_wait(bar_acc_empty, (chunk_it & 1) ^ 1, abort_flag, P.status, FST_ACC_EMPTY);
        tc_fence_after();
        const int kt1 = kt0 + kChunkKt < nkt ? kt0 + kChunkKt : nkt;
        for (int kt = kt0; kt < kt1; kt++) {
          mbar_wait(bar_full + 8 * s, ph, abort_flag, P.status, FST_FULL);
          tc_fence_after();
          const uint32_t st = base + s * kStageBytesF;
          const uint64_t ah = desc_hi | (uint64_t)((st >> 4) & 0x3FFF), al = desc_hi | (uint64_t)(((st + kABytes) >> 4) & 0x3FFF);
          const uint64_t wh = desc_hi | (uint64_t)(((st + 2 * kABytes) >> 4) & 0x3FFF);
          const uint64_t wl = desc_hi | (uint64_t)(((st + 2 * kABytes + kWBytes) >> 4) & 0x3FFF);
#pragma unroll
          for (int j = 0; j < kKt / 8; j++) {             // 8 tf32 = 32 bytes per k step: the address field moves by 2
            mma_tf32_ss(tmem, ah + (uint64_t)(2 * j), wh + (uint64_t)(2 * j), idesc, (uint32_t)((kt - kt0) | j));
            mma_tf32_ss(tmem, ah + (uint64_t)(2 * j), wl + (uint64_t)(2 * j), idesc, 1u);
            mma_tf32_ss(tmem, al + (uint64_t)(2 * j), wh + (uint64_t)(2 * j), idesc, 1u);
          }
          tc_commit(bar_empty + 8 * s);
          if (++s == kStagesF) { s = 0; ph ^= 1; }
        }
        tc_commit(bar_acc_full);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ A producers: thread = row of the tile
    asm volatile("griddepcontrol.wait;" ::: "memory");         // the previous layer's activations are complete and visible
    const int r = (warp - 2) * 32 + lane;
    uint32_t s = 0, ph = 0;
    bool stop = false;
    for (long long t = blockIdx.x; t < ntiles && !stop; t += gridDim.x) {
      const long long m0 = (t / ntn) * kM;
      const long long row = m0 + r;
      const bool live = row < P.nrows;
      long long p0 = 0, p1 = 0;
      if (P.a_mode == A_GATHER) {
        long long ci = 0, cj = 0, kk = 0;
        if (live) row_to_pos(P.g, row, &ci, &cj, &kk);
        p0 = ci * P.cin[0].si + cj * P.cin[0].sj + kk * P.cin[0].sk;
        p1 = ci * P.cin[1].si + cj * P.cin[1].sj + kk * P.cin[1].sk;
      }
      for (int kt = 0; kt < nkt; kt++) {
        const int k0 = kt * kKt;
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, P.status, FST_EMPTY)) { stop = true; break; }
        uint8_t* a_hi = smem + s * kStageBytesF;
        uint8_t* a_lo = a_hi + kABytes;
        if (P.a_mode == A_ROW_MAJOR) {
          // lanes run along k: one coalesced 128-byte read per row; element (row rr, k = lane) lands in 16-byte piece
          // (lane / 4) ^ (rr % 8) of the row's 128-byte line
          const int rb = (warp - 2) * 32;
          const bool kin = k0 + lane < P.K_real;
#pragma unroll 8
          for (int rr = 0; rr < 32; rr++) {
            const long long rw = m0 + rb + rr;
            float x = 0.f;
            if (kin && rw < P.nrows) {
              x = __ldg(P.A + rw * P.lda + k0 + lane);
              if (P.in_div) x = __fdiv_rn(x, __ldg(P.in_div + k0 + lane));
            }
            float hi, lo;
            split_tf32(x, hi, lo);
            const int off = (rb + rr) * 128 + ((((lane >> 2) ^ ((rb + rr) & 7)) << 4) | ((lane & 3) << 2));
            *reinterpret_cast<float*>(a_hi + off) = hi;
            *reinterpret_cast<float*>(a_lo + off) = lo;
          }
        } else {
          float v[kKt];
          if (P.a_mode == A_GATHER) {
#pragma unroll
            for (int j = 0; j < kKt; j++) {
              const uint32_t code = s_code[k0 + j];
              v[j] = 0.f;
              if (live && code != 0xFF)
                v[j] = __ldg(s_base_in[code & 0x7F] + ((long long)s_off[k0 + j] + ((code & 0x80) ? p1 : p0)));
            }
          } else {
#pragma unroll
            for (int j = 0; j < kKt; j++) v[j] = (live && k0 + j < P.K_real) ? __ldg(P.A + (long long)(k0 + j) * P.lda + row) : 0.f;
          }
          if (P.in_div) {
#pragma unroll
            for (int j = 0; j < kKt; j++) if (k0 + j < P.K_real) v[j] = __fdiv_rn(v[j], __ldg(P.in_div + k0 + j));
          }
#pragma unroll
          for (int kc = 0; kc < kKt / 4; kc++) {
            float4 h4, l4;
            split_tf32(v[4 * kc], h4.x, l4.x);
            split_tf32(v[4 * kc + 1], h4.y, l4.y);
            split_tf32(v[4 * kc + 2], h4.z, l4.z);
            split_tf32(v[4 * kc + 3], h4.w, l4.w);
            const int off = r * 128 + ((kc ^ (r & 7)) << 4);
            *reinterpret_cast<float4*>(a_hi + off) = h4;
            *reinterpret_cast<float4*>(a_lo + off) = l4;
          }
        }
        // the tensor core reads shared memory through the async proxy: order these generic-proxy writes before it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(bar_full + 8 * s);
        if (++s == kStagesF) { s = 0; ph ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: thread = row of the tile
    asm volatile("griddepcontrol.wait;" ::: "memory");         // the buffer written here may still be read by the previous layer
    const int quad = warp & 3;                                // the TMEM lanes this warp may read
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    uint32_t chunk_it = 0;
    double csum = 0.0;
    const int nch = (nkt + kChunkKt - 1) / kChunkKt;
    for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
      const long long row = (t / ntn) * kM + r;
      const int nt0 = (int)(t % ntn) * P.n_tile;
      const bool live = row < P.nrows;
      long long op0 = 0, op1 = 0;
      if (P.c_mode == C_SCATTER) {
        long long ci = 0, cj = 0, kk = 0;
        if (live) row_to_pos(P.g, row, &ci, &cj, &kk);
        op0 = ci * P.cout[0].si + cj * P.cout[0].sj + kk * P.cout[0].sk;
        op1 = ci * P.cout[1].si + cj * P.cout[1].sj + kk * P.cout[1].sk;
      }
      for (int ch = 0; ch < nch; ch++, chunk_it++) {
        const bool last = ch == nch - 1;
        mbar_wait(bar_acc_full, chunk_it & 1, abort_flag, P.status, FST_ACC_FULL);
        tc_fence_after();
        for (int c0 = 0; c0 < P.n_tile; c0 += 32) {
          uint32_t a[32], sm[32];
          tmem_ld32(lane_addr + c0, a);                          // this chunk's partial sums
          if (ch > 0) tmem_ld32(lane_addr + kNtMax + c0, sm);    // the running sum of the earlier chunks
          tmem_ld_wait();
          if (last && c0 + 32 >= P.n_tile) {                     // the chunk accumulator has been read completely
            tc_fence_before();
            mbar_arrive(bar_acc_empty);
          }
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = ch > 0 ? __fadd_rn(__uint_as_float(sm[j]), __uint_as_float(a[j])) : __uint_as_float(a[j]);
          if (!last) {
#pragma unroll
            for (int j = 0; j < 32; j++) a[j] = __float_as_uint(v[j]);
            tmem_st32(lane_addr + kNtMax + c0, a);
            continue;
          }
          const int n0 = nt0 + c0;
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const float bj = P.bias ? __ldg(P.bias + n0 + j) : 0.f;
            v[j] = act_slope(v[j] + bj, P.slope);
          }
          if (P.out_mul || P.relu_mask) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const int n = n0 + j;
              if (n < P.N_real) {
                if (P.out_mul) v[j] *= __ldg(P.out_mul + n);
                if (P.relu_mask && __ldg(P.relu_mask + n) != 0.f) v[j] = fmaxf(v[j], 0.f);
              }
            }
          }
          if (!live) continue;
          if (P.c_mode == C_FEATURE_MAJOR) {
#pragma unroll
            for (int j = 0; j < 32; j++) if (n0 + j < P.N_real) P.C[(long long)(n0 + j) * P.ldc + row] = v[j];
          } else if (P.c_mode == C_ROW_MAJOR) {
            float* dst = P.C + row * P.ldc + n0;
            if (n0 + 32 <= P.N_real && ((P.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(P.C) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 8; j++) reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; j++) if (n0 + j < P.N_real) dst[j] = v[j];
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const uint32_t code = (n0 + j < kTabOut) ? o_code[n0 + j] : 0xFFu;
              if (code != 0xFF) {
                s_base_out[code & 0x7F][(long long)o_off[n0 + j] + ((code & 0x80) ? op1 : op0)] = v[j];
                csum += (double)v[j];
              }
            }
          }
        }
        if (!last) {                                             // the running sum is in place: hand the chunk accumulator back
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(bar_acc_empty);
        }
      }
    }
    if (P.partials) {
      // per-CTA checksum partial in a fixed order; the last CTA to finish folds all partials into the step checksum
      double* wsum = (double*)(tail + 72);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) csum += __shfl_down_sync(0xffffffffu, csum, o);
      if (lane == 0) wsum[quad] = csum;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (quad == 0 && lane == 0) {
        P.partials[blockIdx.x] = (wsum[0] + wsum[1]) + (wsum[2] + wsum[3]);
        if (P.sum) {
          __threadfence();
          if (atomicAdd(P.done, 1u) == gridDim.x - 1) {
            __threadfence();
            double total = *P.sum;
            for (unsigned i = 0; i < gridDim.x; i++) total += __ldcg(P.partials + i);
            *P.sum = total;
            *P.done = 0u;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0)
    for (int i = 0; i < 2000; i++) __nanosleep(1000);        // let copies in flight land before the CTA gives its memory back
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// W (N, K) row-major on the device -> W_hi / W_lo [N_pad][K_pad] (zero padded): the split of fortis_gemm's weights,
// which only exist on the device
__global__ void split_weights_kernel(const float* __restrict__ W, int N, int K, float* __restrict__ hi, float* __restrict__ lo, int N_pad,
                                     int K_pad) {
  const long long n_el = (long long)N_pad * K_pad;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_el; i += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(i / K_pad), k = (int)(i % K_pad);
    float h = 0.f, l = 0.f;
    if (n < N && k < K) split_tf32(W[(long long)n * K + k], h, l);
    hi[i] = h; lo[i] = l;
  }
}

typedef CUresult (*EncodeTiledFnF)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFnF encode_fn_f() {
  static EncodeTiledFnF fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return nullptr;
  fn = (EncodeTiledFnF)p;
  return fn;
}

int round_up_f(int v, int m) { return (v + m - 1) / m * m; }

// nearest TF32 value, ties away from zero (what cvt.rna.tf32.f32 returns)
float tf32_rna_host(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;            // inf / nan unchanged
  u = (u + 0x1000u) & 0xFFFFE000u;
  float r;
  std::memcpy(&r, &u, 4);
  return r;
}

struct LayerGeom { int K_real, N_real, K_pad, N_pad, n_tile; };
LayerGeom layer_geom(int cin, int cout) {
  LayerGeom g;
  g.K_real = cin; g.N_real = cout;
  g.K_pad = round_up_f(cin, kKt);
  g.N_pad = round_up_f(cout, 64);
  if (g.N_pad > kNtMax) g.N_pad = round_up_f(cout, kNtMax);
  g.n_tile = g.N_pad < kNtMax ? g.N_pad : kNtMax;
  return g;
}

bool make_w_maps(float* hi, float* lo, const LayerGeom& g, CUtensorMap* mh, CUtensorMap* ml) {
  EncodeTiledFnF enc = encode_fn_f();
  if (!enc) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)g.K_pad, (cuuint64_t)g.N_pad};
  const cuuint64_t strides[1] = {(cuuint64_t)g.K_pad * 4};
  const cuuint32_t box[2] = {(cuuint32_t)kKt, (cuuint32_t)g.n_tile};
  const cuuint32_t estr[2] = {1, 1};
  for (int i = 0; i < 2; i++)
    if (enc(i ? ml : mh, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, i ? lo : hi, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  return true;
}

bool prepare_kernel(std::string* err) {
  static bool done = false;
  if (done) return true;
  if (cudaFuncSetAttribute(linear_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemF) != cudaSuccess) {
    if (err) *err = "cannot reserve " + std::to_string(kSmemF) + " bytes of shared memory for the split-TF32 kernel";
    return false;
  }
  done = true;
  return true;
}

int grid_for(long long nrows, const LayerGeom& g) {
  const long long tiles = ((nrows + kM - 1) / kM) * (g.N_pad / g.n_tile);
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return (int)(tiles < sms ? (tiles > 0 ? tiles : 1) : sms);
}

}  // namespace

struct F32TcModel {
  struct Layer {
    LayerGeom g;
    float *hi = nullptr, *lo = nullptr, *bias = nullptr;
    CUtensorMap mh, ml;
    float slope = 1.f;
  };
  std::vector<Layer> layers;
  float *in_div = nullptr, *out_mul = nullptr, *relu_mask = nullptr;
};

bool f32tc_supported(const ModelHost& M, std::string* why) {
  auto no = [&](const char* w) { if (why) *why = w; return false; };
  if (!M.is_mlp()) return no("not an MLP");
  for (auto& L : M.layers)
    if (L.act == ACT_LEAKY && !(L.slope >= 0.f && L.slope <= 1.f)) return no("LeakyReLU slope outside [0, 1]");
  return true;
}

void f32tc_destroy(F32TcModel* m) {
  if (!m) return;
  for (auto& L : m->layers) { cudaFree(L.hi); cudaFree(L.lo); cudaFree(L.bias); }
  cudaFree(m->in_div); cudaFree(m->out_mul); cudaFree(m->relu_mask);
  delete m;
}

F32TcModel* f32tc_create(const ModelHost& M, std::string* err) {
  std::string why;
  if (!f32tc_supported(M, &why)) { if (err) *err = why; return nullptr; }
  if (!prepare_kernel(err)) return nullptr;
  F32TcModel* m = new F32TcModel();
  auto fail = [&](const std::string& w) { if (err) *err = w; f32tc_destroy(m); return (F32TcModel*)nullptr; };
  for (auto& L : M.layers) {
    F32TcModel::Layer T;
    T.g = layer_geom(L.cin, L.cout);
    std::vector<float> hi((size_t)T.g.N_pad * T.g.K_pad, 0.f), lo(hi.size(), 0.f), bias(T.g.N_pad, 0.f);
    for (int n = 0; n < L.cout; n++) {
      bias[n] = L.b[n];
      for (int k = 0; k < L.cin; k++) {
        const float w = L.W[(size_t)n * L.cin + k], h = tf32_rna_host(w);
        hi[(size_t)n * T.g.K_pad + k] = h;
        lo[(size_t)n * T.g.K_pad + k] = w - h;
      }
    }
    if (cudaMalloc(&T.hi, hi.size() * 4) != cudaSuccess || cudaMalloc(&T.lo, lo.size() * 4) != cudaSuccess ||
        cudaMalloc(&T.bias, bias.size() * 4) != cudaSuccess) {
      cudaFree(T.hi); cudaFree(T.lo); cudaFree(T.bias);
      return fail("out of device memory for split weights");
    }
    cudaMemcpy(T.hi, hi.data(), hi.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(T.lo, lo.data(), lo.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(T.bias, bias.data(), bias.size() * 4, cudaMemcpyHostToDevice);
    T.slope = L.act == ACT_NONE ? 1.f : L.act == ACT_RELU ? 0.f : L.slope;
    m->layers.push_back(T);
    if (!make_w_maps(T.hi, T.lo, T.g, &m->layers.back().mh, &m->layers.back().ml)) return fail("cuTensorMapEncodeTiled failed for split weights");
  }
  auto up = [&](const std::vector<float>& v) -> float* {
    if (v.empty()) return nullptr;
    float* d = nullptr;
    cudaMalloc(&d, v.size() * 4);
    cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
    return d;
  };
  m->in_div = up(M.in_div); m->out_mul = up(M.out_mul); m->relu_mask = up(M.relu_mask);
  return m;
}

int f32tc_grid(long long nrows) {
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  (void)nrows;
  return sms;
}

// one layer, allowed to start while the launch before it in the stream drains (programmatic stream serialisation)
// (`early` = false for a launch whose WEIGHTS were produced by the kernel in front of it: the weight loads do not wait)
static bool launch_layer(const F32Params& P, int grid, cudaStream_t s, bool early = true) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kThreadsF); cfg.dynamicSmemBytes = kSmemF; cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  static const bool pdl = std::getenv("FORTIS_NO_PDL") == nullptr;
  cfg.attrs = at; cfg.numAttrs = (pdl && early) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, linear_tf32x3_kernel, P) == cudaSuccess;
}

bool f32tc_forward(F32TcModel* m, const F32TcLaunch& L, cudaStream_t s, std::string* err) {
  const long long nrows = L.g.count * L.g.nk;
  if (nrows <= 0) return true;
  const int nl = (int)m->layers.size();
  const int n_in = m->layers.front().g.K_real, n_out = m->layers.back().g.N_real;
  const bool fast_in = L.fast_in && n_in <= kTabIn, fast_out = L.fast_out && n_out <= kTabOut;
  if (!fast_in && !L.X) { if (err) *err = "split-TF32 step: no input"; return false; }
  if (!fast_out && !L.Y) { if (err) *err = "split-TF32 step: no output"; return false; }
  if (nl > 1 && (!L.act[0] || (nl > 2 && !L.act[1]))) { if (err) *err = "split-TF32 step: no activation buffers"; return false; }
  for (int l = 0; l < nl; l++) {
    const F32TcModel::Layer& T = m->layers[l];
    F32Params P;
    std::memset(&P, 0, sizeof P);
    P.map_hi = T.mh; P.map_lo = T.ml;
    P.K_pad = T.g.K_pad; P.N_pad = T.g.N_pad; P.n_tile = T.g.n_tile; P.K_real = T.g.K_real; P.N_real = T.g.N_real;
    P.bias = T.bias; P.slope = T.slope; P.nrows = nrows; P.g = L.g; P.status = L.status;
    if (l == 0) {
      P.in_div = m->in_div;
      if (fast_in) {
        P.a_mode = A_GATHER; P.slots = L.slots; P.TG = L.TG;
        for (int i = 0; i < 2; i++) P.cin[i] = StrideClassF{L.cin[i][0], L.cin[i][1], L.cin[i][2]};
      } else { P.a_mode = A_ROW_MAJOR; P.A = L.X; P.lda = n_in; }
    } else { P.a_mode = A_FEATURE_MAJOR; P.A = L.act[(l - 1) & 1]; P.lda = L.act_ld; }
    if (l == nl - 1) {
      P.out_mul = m->out_mul; P.relu_mask = m->relu_mask;
      if (fast_out) {
        P.c_mode = C_SCATTER; P.store_by_slot = L.store_by_slot; P.TS = L.TS;
        for (int i = 0; i < 2; i++) P.cout[i] = StrideClassF{L.cout[i][0], L.cout[i][1], L.cout[i][2]};
        P.partials = L.partials; P.sum = L.partials ? L.sum : nullptr; P.done = L.done;
      } else { P.c_mode = C_ROW_MAJOR; P.C = L.Y; P.ldc = n_out; }
    } else { P.c_mode = C_FEATURE_MAJOR; P.C = L.act[l & 1]; P.ldc = L.act_ld; }
    if (!launch_layer(P, grid_for(nrows, T.g), s)) { if (err) *err = "split-TF32 kernel launch failed"; return false; }
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { if (err) *err = std::string("split-TF32 kernel launch: ") + cudaGetErrorString(e); return false; }
  return true;
}

// C[M][N] = A[M][K] . W[N][K]^T, all row-major on the device (the memref entry of runtime/fortis_rt.c:45-48).  The
// weights are constants of the caller: each distinct (pointer, N, K) is split once, by a kernel on the caller's stream,
// as the reference caches its transposed weights (runtime/fortis_rt.c:55-66).
bool f32tc_gemm(const float* A, const float* W, float* C, long long M, int N, int K, int* status, cudaStream_t s, std::string* err) {
  if (M <= 0 || N <= 0 || K <= 0) return true;
  if (!prepare_kernel(err)) return false;
  struct Cached { const float* w; int N, K; float *hi, *lo; LayerGeom g; CUtensorMap mh, ml; };
  static std::vector<Cached> cache;
  static size_t victim = 0;
  Cached* c = nullptr;
  for (auto& e : cache) if (e.w == W && e.N == N && e.K == K) c = &e;
  if (!c) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(s, &cs);
    if (cs != cudaStreamCaptureStatusNone) { if (err) *err = "weights seen for the first time during graph capture; run one eager call first"; return false; }
    if (cache.size() < 64) { cache.push_back(Cached{}); c = &cache.back(); c->hi = c->lo = nullptr; }
    else { c = &cache[victim]; victim = (victim + 1) % cache.size(); cudaStreamSynchronize(s); cudaFree(c->hi); cudaFree(c->lo); c->hi = c->lo = nullptr; }
    c->w = nullptr;
    c->g = layer_geom(K, N);
    const size_t n_el = (size_t)c->g.N_pad * c->g.K_pad;
    if (cudaMalloc(&c->hi, n_el * 4) != cudaSuccess || cudaMalloc(&c->lo, n_el * 4) != cudaSuccess) { if (err) *err = "out of device memory for split weights"; return false; }
    split_weights_kernel<<<(unsigned)((n_el + 255) / 256 < 1184 ? (n_el + 255) / 256 : 1184), 256, 0, s>>>(W, N, K, c->hi, c->lo, c->g.N_pad, c->g.K_pad);
    if (!make_w_maps(c->hi, c->lo, c->g, &c->mh, &c->ml)) { if (err) *err = "cuTensorMapEncodeTiled failed"; return false; }
    c->w = W; c->N = N; c->K = K;
  }
  F32Params P;
  std::memset(&P, 0, sizeof P);
  P.map_hi = c->mh; P.map_lo = c->ml;
  P.K_pad = c->g.K_pad; P.N_pad = c->g.N_pad; P.n_tile = c->g.n_tile; P.K_real = K; P.N_real = N;
  P.slope = 1.f; P.nrows = M; P.status = status;
  P.g.count = M; P.g.nk = 1; P.g.ni = 1; P.g.kk0 = 0;
  P.a_mode = A_ROW_MAJOR; P.A = A; P.lda = K;
  P.c_mode = C_ROW_MAJOR; P.C = C; P.ldc = N;
  launch_layer(P, grid_for(M, c->g), s, false);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { if (err) *err = std::string("split-TF32 kernel launch: ") + cudaGetErrorString(e); return false; }
  return true;
}

}  // namespace fortis
