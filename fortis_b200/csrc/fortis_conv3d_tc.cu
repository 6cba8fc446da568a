// conv3d 3x3x3, stride 1, pad 1 as an implicit GEMM on tcgen05 tensor cores (bf16 operands, fp32 accumulation in
// tensor memory), with bias + residual add + LeakyReLU fused into the epilogue, and the bf16 network driver.  Three
// instantiations of one kernel: 64 -> 64 channels (the body of the network), few -> 64 (first layer: only the first
// 16-wide k step of every tap is issued) and 64 -> few (last layer: N = 16 MMAs, fp32 NDHWC output straight from the
// accumulator).
//
// Replaces fortis_conv3d -> cudnnConvolutionForward and the separate bias / activation / residual kernels the
// reference chains behind it (runtime/fortis_rt.c:128-156, compiler/FortisFuse.cpp:626-655, 687-760).
//
// Layout: activations are bf16, channels-last, ZERO-PADDED in memory: [N][D+2][H+2][W+2][64], viewed as a matrix
// [P rows][64 channels] (one 128-byte row per voxel), with further zero rows in front of and behind the volume inside
// its allocation.  With the border stored explicitly, the input rows the taps (kd, kh, *) need for output rows
// p.. are simply rows p+shift.. with shift = (kd-1)(H+2)(W+2) + (kh-1)(W+2): no im2col, no masks, and no copy ever
// leaves the allocation.  Border rows of the output are computed and then written as zeros, which keeps the padding
// intact for the next layer; that costs ((D+2)(H+2)(W+2))/(DHW) = 1.19x the useful work at 33^3.
//
// The kernel runs as clusters of two CTAs (cta_group::2), one cluster per SM pair, each CTA owning a 128-row tile:
//  * MMA: per (kd, kh) KSTEPS MMAs of M = 256 (both CTAs' rows), N = 3 * 64, K = 16: the three kw taps are the three
//    64-column blocks of the accumulator, computed from the SAME (unshifted) rows, and the kw shift is applied once
//    per tile in the epilogue: out[row] = acc_kw0[row-1] + acc_kw1[row] + acc_kw2[row+1] (a tile writes 126 rows).
//    (With one N = 64 MMA per tap both operands stream from shared memory at 128 B/clk and the MMA runs at 2/3
//    rate; N = 192 reads the activation slice once for three taps.)
//  * weights: each CTA holds its half (96 of a group's 192 rows) of ALL 27 weight tiles in shared memory for the
//    whole kernel (108 KB); cta_group::2 MMAs take half of B from each CTA.  Only activations stream.
//  * activations: ONE stage per kd holds rows q - (W+2) .. q + 127 + (W+2), which serve all three kh taps through
//    descriptors whose start address moves by (W+2) rows (the 128-byte swizzle is a function of the shared-memory
//    address, so shifted views match what TMA wrote).  Ring of kRingBytes / stage size stages (4 x 25 KB at W = 33).
//    No multicast loads anywhere: every copy goes to the issuing CTA's own shared memory, its completion counted on
//    the leader's barrier.
//  * two accumulators (2 x 192 TMEM columns) so that the epilogue of a tile overlaps the MMAs of the next.
//  * warp 0: TMA (both CTAs), warp 1: MMA (leader only), warps 2-9: epilogue, two warps per lane quadrant (thread =
//    one voxel row x 32 channels): row neighbours by warp shuffle, the rows on either side of a warp boundary through
//    shared memory; bias + residual row (prefetched one tile ahead) + LeakyReLU -> bf16 -> row store.  The
//    accumulator is handed back with a RELAXED cluster-scope arrive: a release would first drain the thread's
//    outstanding global stores (measured ~1700 cycles per tile).
//
// First layer: the fp32 NDHWC input is packed into its own padded bf16 volume with channels >= Cin zero, and the
// weights are padded the same way, so the layer is the same GEMM with one k step per group instead of four.
// Last layer: the weights are padded to 16 output channels (N = 48); the epilogue adds the bias, applies the
// activation and writes the real channels of interior voxels as fp32.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "fortis_kernels.h"
#include "fortis_model.h"
#include "fortis_tc.cuh"

namespace fortis {

using namespace tc;

namespace {

// How the kw taps are applied.  0 (default): one MMA of N = 3 NOUT per (kd, kh) group on unshifted rows, the shift
// applied in the epilogue (three accumulator loads, 64 shuffles and a shared-memory exchange per row).  1: one MMA of
// N = NOUT per tap, the kw shift taken on the A side (the descriptor's start address moves by kw rows, exactly as it
// moves by kh (W+2) rows), so a tile's accumulator IS the output tile and the epilogue is one accumulator load per
// row.  Bit-compatible tests pass for both; measured on the 8 x 33^3 network 1 is slower (0.895 vs 0.844 ms): three
// N = 64 MMAs read the activation slice three times and the kernel becomes bound by shared-memory operand reads.
#ifndef FORTIS_CONV_SHIFT_A
#define FORTIS_CONV_SHIFT_A 0
#endif
constexpr bool kShiftA = FORTIS_CONV_SHIFT_A != 0;
constexpr int kC = 64;                       // channels of the tensor-core layers
constexpr int kTile = 128;                   // rows computed per tile (the MMA's M)
constexpr int kTileOut = kShiftA ? kTile : kTile - 2;   // rows written per tile (epilogue-side shift: the first and last computed rows only feed their neighbours)
constexpr int kHalo = kShiftA ? 1 : 0;       // rows in front of and behind a stage's 128 + 2 (W+2) rows, for the kw shift
constexpr int kRingBytes = 108 * 1024;       // activation ring: nstages stages of (128 + 2 (W+2)) rows each
constexpr int kMaxStages = 7;
constexpr int kXchBytes = 2 * 2 * 4 * kC * 4; // rows exchanged between epilogue warps: [tile parity][up | down][quadrant][channel] floats
constexpr int kResW = 9 * 96 * kC * 2;       // 108 KB: this CTA's half of all 27 weight tiles, resident for the whole kernel
constexpr int kConvThreads = 320;           // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quadrant)
constexpr int kConvSmem = kResW + kRingBytes + 256 + kXchBytes;
constexpr int kAccStride = 256;              // TMEM columns between the two accumulators (each 3 * NOUT wide)
// the pair's M = 256; operand format code 1 = bf16, 0 = IEEE half (bits 7-9 for A, 10-12 for B)
template <int NOUT, bool F16> struct ConvIdesc {
  static constexpr uint32_t value = idesc_bf16(2 * kTile, kShiftA ? NOUT : 3 * NOUT) & ~(F16 ? ((1u << 7) | (1u << 10)) : 0u);
};
// the 16-bit storage format of activations and weights: bf16 (range of fp32, 8 significant bits) or IEEE half (11
// significant bits, values beyond 65504 overflow)
template <bool F16> __device__ __forceinline__ uint32_t cpack16(float lo, float hi) {
  if constexpr (F16) { const __half2 v = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t*>(&v); }
  else return pack_bf16(lo, hi);
}
template <bool F16> __device__ __forceinline__ float2 cunpack16(uint32_t u) {
  if constexpr (F16) return __half22float2(*reinterpret_cast<const __half2*>(&u));
  else return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
}
constexpr int kEdgeC = 16;                   // first layer: input channels kept; last layer: output channels computed
enum { CST_FULL = 11, CST_EMPTY = 12, CST_ACC_FULL = 13, CST_ACC_EMPTY = 14, CST_WEIGHTS = 15, CST_ALIGN = 16 };

struct ConvTcParams {
  CUtensorMap amap;            // the activation allocation [rows][64] bf16, box 64 x box_rows
  int stage_bytes, nstages;    // activation ring geometry: one stage holds the 128 + 2 (W+2) rows one kd needs
  int box_rows, nbox;          // a stage is loaded as nbox boxes of box_rows rows
  int front;                   // zero rows in front of row 0 of the volume inside the allocation
  CUtensorMap wmap;            // weights [27 * NOUT (tap, cout)][64 cin] bf16, box 64 x 3 NOUT
  const float* bias;           // [64] (zero beyond the layer's real outputs)
  const __nv_bfloat16* skip;   // [P][64] or null
  __nv_bfloat16* out;          // [P][64]
  float* y;                    // last layer: fp32 [N*D*H*W][F]
  int F;                       // last layer: real output channels (<= 16)
  int D, H, W;                 // unpadded extent
  long long P;                 // padded rows
  float slope;                 // act(v) = max(v, v * slope)
  int* status;
  unsigned int wait_limit;     // polls before a barrier wait gives up
  int test_skip_stage;         // test only: the first pair's leader never loads its first activation stage
  long long* prof;             // optional cycle counters of CTA 0 (diagnostics; null in normal runs)
};

// cycle accounting for diagnostics: adds the time since *t to prof[slot] (CTA 0, one lane) and restarts the clock
__device__ __forceinline__ void cprof_add(long long* prof, int slot, long long* t, bool who) {
  if (prof && who) { const long long n = clock64(); atomicAdd((unsigned long long*)&prof[slot], (unsigned long long)(n - *t)); *t = n; }
}

// KSTEPS: 16-wide k steps issued per (kd, kh) group (4 = all 64 input channels, 1 = only the first 16);  NOUT: output
// channels (weight rows per tap);  LAST: write fp32 NDHWC instead of the padded bf16 volume.
// Launched as clusters of two CTAs (cta_group::2): the leader's MMA warp issues for both.
template <int KSTEPS, int NOUT, bool LAST, bool F16>
__global__ void __launch_bounds__(kConvThreads, 1) conv3d_tc_kernel(const __grid_constant__ ConvTcParams P) {
  constexpr uint32_t kIdescN = ConvIdesc<NOUT, F16>::value;            // M = 256 (128 rows per CTA), N = NOUT per tap (or 3 * NOUT per group)
  constexpr int kWLoads = kShiftA ? 27 : 9;                       // weight tiles: one per tap, or one per (kd, kh) group
  constexpr int kHalfRows = (kShiftA ? NOUT : 3 * NOUT) / 2;      // weight rows of one tile held by each CTA
  constexpr int kHalfBytes = kHalfRows * kC * 2;                  // 4 KB per tap (12 KB per group)
  extern __shared__ __align__(1024) uint8_t smem[];
  // Programmatic dependent launch: the next layer's CTAs may be scheduled as soon as SMs free up.  They set up their
  // barriers and tensor memory and load their weights while this layer's last tiles finish, and wait (griddep_wait below)
  // for this grid to complete before they touch an activation buffer.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t base = smem_u32(smem);                           // resident weights at offset 0
  if (base & 1023u) {                                             // same in both CTAs of a pair: both leave
    if (threadIdx.x == 0) atomicCAS(P.status, 0, CST_ALIGN);
    return;
  }
  const uint32_t ring = base + kResW;
  const uint32_t bars = ring + kRingBytes;
  // barrier block (256 B): full [0,56) empty [56,112) acc_full [112,128) acc_empty [128,144) weights [144,152)
  // tmem base 160, abort flag 164
  const uint32_t bar_full = bars, bar_empty = bars + 56, bar_acc_full = bars + 112, bar_acc_empty = bars + 128, bar_w = bars + 144;
  uint8_t* barp = smem + kResW + kRingBytes;
  uint32_t* tmem_slot = (uint32_t*)(barp + 160);
  volatile int* abort_flag = (volatile int*)(barp + 164);
  float* xch = (float*)(barp + 256);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();
  const long long ntiles = (P.P + kTileOut - 1) / kTileOut;
  const long long npairs = (ntiles + 1) / 2;                       // a pair works on tiles 2 t and 2 t + 1
  const long long pair0 = blockIdx.x >> 1, pair_step = gridDim.x >> 1;
  const int Wp = P.W + 2, Hp = P.H + 2, Dp = P.D + 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int b = 0; b < 2; b++) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, 16); }   // 8 epilogue warps per CTA
    mbar_init(bar_w, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0 && lane < 2)
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(lane ? &P.wmap : &P.amap)) : "memory");
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                      // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer (one per CTA): this CTA's half of the weights once, then per tile 9 activation tiles.
    //      Completion of both CTAs' copies is counted on the LEADER's barriers, which the leader arms for both.
    const uint32_t full0 = map_to_cta(bar_full, 0), w0 = map_to_cta(bar_w, 0);
    if (crank == 0) mbar_expect_tx(bar_w, 2 * kWLoads * kHalfBytes);
#pragma unroll 1
    for (int g = 0; g < kWLoads; g++)
      tma_load_2d_pair(base + g * kHalfBytes, &P.wmap, 0, g * 2 * kHalfRows + (int)crank * kHalfRows, w0);
    asm volatile("griddepcontrol.wait;" ::: "memory");           // the previous layer's output is complete and visible
    uint32_t s = 0, ph = 0;
    bool stop = false;
    const bool pw = blockIdx.x == 0 && lane == 0;
    long long pt = clock64();
    for (long long tp = pair0; tp < npairs && !stop; tp += pair_step) {
      const long long q0 = (2 * tp + crank) * kTileOut - (kShiftA ? 0 : 1);       // first computed row of this CTA's tile
      for (int kd = 0; kd < 3; kd++) {
        // rows q0 + (kd-1) Hp Wp - Wp ... + 127 + Wp serve the three kh taps of this kd.  The allocation carries zero
        // rows on both sides, so every coordinate is in bounds.
        const int y0 = (int)(q0 + (long long)(kd - 1) * Hp * Wp - Wp - kHalo) + P.front;
        cprof_add(P.prof, 7, &pt, pw);
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, P.status, CST_EMPTY, P.wait_limit)) { stop = true; break; }
        cprof_add(P.prof, 6, &pt, pw);
        if (crank == 0) mbar_expect_tx(bar_full + 8 * s, 2 * P.nbox * P.box_rows * kC * 2);
        const bool skip = P.test_skip_stage && blockIdx.x == 0 && tp == pair0 && kd == 0;     // test only: the stage never completes
        for (int bx = 0; bx < P.nbox && !skip; bx++)
          tma_load_2d_pair(ring + s * P.stage_bytes + bx * P.box_rows * kC * 2, &P.amap, 0, y0 + bx * P.box_rows, full0 + 8 * s);
        if (++s == (uint32_t)P.nstages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (crank == 0) {
      // ---- MMA issuer (leader only): per (kd, kh) group KSTEPS MMAs of M = 256, N = 3 * NOUT; accumulator column
      //      block kw holds sum over groups of X[row + shift(kd, kh)] . W(kd, kh, kw), still to be shifted by kw - 1 rows
      uint32_t s = 0, ph = 0, acc_it = 0;
      const uint64_t desc_hi = make_kmajor_sw128_desc(0) & 0xFFFFFFFF00000000ull;
      const bool pw = blockIdx.x == 0 && lane == 0;
      long long pt = clock64();
      mbar_wait(bar_w, 0, abort_flag, P.status, CST_WEIGHTS, P.wait_limit);
      cprof_add(P.prof, 3, &pt, pw);
      for (long long tp = pair0; tp < npairs; tp += pair_step, acc_it++) {
        const uint32_t b = acc_it & 1, aph = (acc_it >> 1) & 1;
        cprof_add(P.prof, 2, &pt, pw);
        mbar_wait(bar_acc_empty + 8 * b, aph ^ 1, abort_flag, P.status, CST_ACC_EMPTY, P.wait_limit);
        cprof_add(P.prof, 0, &pt, pw);
        tc_fence_after();
        const uint32_t d_tmem = tmem + b * kAccStride;
        for (int kd = 0; kd < 3; kd++) {
          cprof_add(P.prof, 2, &pt, pw);
          mbar_wait(bar_full + 8 * s, ph, abort_flag, P.status, CST_FULL, P.wait_limit);
          cprof_add(P.prof, 1, &pt, pw);
          tc_fence_after();
          const uint32_t sa = ring + s * P.stage_bytes;
#pragma unroll
          for (int kh = 0; kh < 3; kh++) {
            // tap row kh reads the stage kh * Wp rows further down: the descriptor's start address moves; the 128-byte
            // swizzle is a function of the shared-memory address, so the shifted view matches what TMA wrote
            if constexpr (kShiftA) {
#pragma unroll
              for (int kw = 0; kw < 3; kw++) {
                // stage row 0 is input row q0 - (W+2) - 1 of this kd: output row r under tap (kh, kw) reads stage row r + kh (W+2) + kw
                const uint64_t ad = desc_hi | (uint64_t)(((sa + (kh * Wp + kw) * (kC * 2)) >> 4) & 0x3FFF);
                const uint64_t bd = desc_hi | (uint64_t)(((base + ((kd * 3 + kh) * 3 + kw) * kHalfBytes) >> 4) & 0x3FFF);
#pragma unroll
                for (int j = 0; j < KSTEPS; j++)
                  tc_mma_ss_pair<kIdescN>(d_tmem, ad + (uint64_t)(j * 2), bd + (uint64_t)(j * 2), (uint32_t)(kd | kh | kw | j));
              }
            } else {
              const uint64_t ad = desc_hi | (uint64_t)(((sa + kh * Wp * (kC * 2)) >> 4) & 0x3FFF);
              const uint64_t bd = desc_hi | (uint64_t)(((base + (kd * 3 + kh) * kHalfBytes) >> 4) & 0x3FFF);
#pragma unroll
              for (int j = 0; j < KSTEPS; j++)
                tc_mma_ss_pair<kIdescN>(d_tmem, ad + (uint64_t)(j * 2), bd + (uint64_t)(j * 2), (uint32_t)(kd | kh | j));
            }
          }
          tc_commit_pair(bar_empty + 8 * s);                      // frees this stage in both CTAs
          if (++s == (uint32_t)P.nstages) { s = 0; ph ^= 1; }
        }
        tc_commit_pair(bar_acc_full + 8 * b);                     // both CTAs' epilogues
      }
    }
  } else {
    // ---- epilogue: thread = one computed row (voxel of the padded volume);
    //      out[row] = acc_kw0[row - 1] + acc_kw1[row] + acc_kw2[row + 1], the neighbours by warp shuffle: each warp's 32
    //      computed rows overlap the next warp's by two, so lanes 1..30 have both neighbours in their own warp
    const int quad = warp & 3, half = (warp - 2) >> 2;            // TMEM lane quadrant; which half of the channels
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    constexpr int CW = NOUT == kC ? kC / 2 : NOUT;                 // channels per warp: two warps share a row of 64
    const bool active = NOUT == kC || half == 0;                   // a 16-channel layer needs one warp per quadrant
    const int c0 = NOUT == kC ? CW * half : 0;
    float bias[CW];
#pragma unroll
    for (int j = 0; j < CW / 4; j++) {
      const float4 q = __ldg(reinterpret_cast<const float4*>(P.bias + c0) + j);
      bias[4 * j] = q.x; bias[4 * j + 1] = q.y; bias[4 * j + 2] = q.z; bias[4 * j + 3] = q.w;
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");           // before the first read of the residual volume and the first store
    const uint32_t arr_acc_empty = map_to_cta(bar_acc_empty, 0);   // the leader's barrier
    const bool pw = blockIdx.x == 0 && threadIdx.x == 64;
    long long pt = clock64();
    const uint32_t uW = (uint32_t)Wp, uH = (uint32_t)Hp, uD = (uint32_t)Dp;
    // row of this thread in tile pair tp_ and whether it is written / an interior voxel (P < 2^31: 32-bit arithmetic).
    // (Advancing the coordinates from tile to tile by additions with carries instead of dividing was measured 6 %
    // SLOWER over the whole kernel: the divisions sit in front of the accumulator wait, where the warp would idle.)
    auto locate = [&](long long tp_, uint32_t& p_, bool& writes_, bool& interior_, uint32_t& wp_, uint32_t& hp_, uint32_t& dp_, uint32_t& n_) {
      const int r = quad * 32 + lane;                              // epilogue-side shift: rows 0 and 127 are computed for their neighbours only
      const long long pl = (2 * tp_ + crank) * kTileOut + r - (kShiftA ? 0 : 1);
      writes_ = active && tp_ < npairs && (kShiftA || (r >= 1 && r <= kTileOut)) && pl < P.P;
      p_ = writes_ ? (uint32_t)pl : 0u;
      const uint32_t t1 = p_ / uW, t2 = t1 / uH;
      wp_ = p_ - t1 * uW; hp_ = t1 - t2 * uH; n_ = t2 / uD; dp_ = t2 - n_ * uD;
      interior_ = writes_ && wp_ >= 1 && wp_ <= (uint32_t)P.W && hp_ >= 1 && hp_ <= (uint32_t)P.H && dp_ >= 1 && dp_ <= (uint32_t)P.D;
    };
    uint32_t p, wp, hp, dp, n_;
    bool writes, interior;
    locate(pair0, p, writes, interior, wp, hp, dp, n_);
    // this warp's half of the residual row of the thread's voxel, always fetched one tile ahead
    uint4 sk[CW / 8];
    bool use_skip = !LAST && P.skip != nullptr && interior;
    if (use_skip) {
#pragma unroll
      for (int j = 0; j < CW / 8; j++) sk[j] = __ldg(reinterpret_cast<const uint4*>(P.skip + (size_t)p * kC + c0) + j);
    }
    uint32_t acc_it = 0;
    for (long long tp = pair0; tp < npairs; tp += pair_step, acc_it++) {
      const uint32_t b = acc_it & 1, aph = (acc_it >> 1) & 1;
      uint32_t np, nwp, nhp, ndp, nn;
      bool nwrites, ninterior;
      locate(tp + pair_step, np, nwrites, ninterior, nwp, nhp, ndp, nn);
      const bool nuse_skip = !LAST && P.skip != nullptr && ninterior;
      cprof_add(P.prof, 10, &pt, pw);
      mbar_wait(bar_acc_full + 8 * b, aph, abort_flag, P.status, CST_ACC_FULL, P.wait_limit);
      cprof_add(P.prof, 8, &pt, pw);
      tc_fence_after();
      const uint32_t accb = lane_addr + b * kAccStride + c0;
      float v[CW];
      if constexpr (kShiftA) {
        uint32_t a1[CW];
        if (active) { tmem_ldn(accb, a1); tmem_ld_wait(); }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(arr_acc_empty + 8 * b);   // one arrival per warp: the leader may refill this accumulator
        if (!active) continue;
#pragma unroll
        for (int i = 0; i < CW; i++) v[i] = __uint_as_float(a1[i]) + bias[i];
      } else {
        uint32_t a0[CW], a1[CW], a2[CW];
        if (active) {
          tmem_ldn(accb, a0);
          tmem_ldn(accb + NOUT, a1);
          tmem_ldn(accb + 2 * NOUT, a2);
          tmem_ld_wait();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(arr_acc_empty + 8 * b);   // one arrival per warp: the leader may refill this accumulator
        if (!active) continue;
        // rows on either side of a warp boundary go through shared memory (the buffer alternates per tile, so one
        // barrier per tile among the four warps that hold the same channels is enough)
        float* xu = xch + (acc_it & 1) * (2 * 4 * kC);               // kw = 0 partials of each quadrant's last row
        float* xd = xu + 4 * kC;                                     // kw = 2 partials of each quadrant's first row
        if (lane == 31) {
#pragma unroll
          for (int i = 0; i < CW; i++) xu[quad * kC + c0 + i] = __uint_as_float(a0[i]);
        }
        if (lane == 0) {
#pragma unroll
          for (int i = 0; i < CW; i++) xd[quad * kC + c0 + i] = __uint_as_float(a2[i]);
        }
        if (half == 0) asm volatile("bar.sync 1, 128;" ::: "memory"); else asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
        for (int i = 0; i < CW; i++) {
          float up = __shfl_up_sync(0xffffffffu, __uint_as_float(a0[i]), 1);
          float dn = __shfl_down_sync(0xffffffffu, __uint_as_float(a2[i]), 1);
          if (lane == 0 && quad > 0) up = xu[(quad - 1) * kC + c0 + i];
          if (lane == 31 && quad < 3) dn = xd[(quad + 1) * kC + c0 + i];
          v[i] = (__uint_as_float(a1[i]) + up) + (dn + bias[i]);
        }
      }
      if (LAST) {
        if (interior) {
          float* dst = P.y + ((((size_t)n_ * P.D + dp - 1) * P.H + hp - 1) * P.W + wp - 1) * P.F;
#pragma unroll
          for (int f = 0; f < CW; f++)
            if (f < P.F) dst[f] = fmaxf(v[f], v[f] * P.slope);
        }
      } else {
        if (use_skip) {
#pragma unroll
          for (int h = 0; h < CW / 8; h++) {
            const uint32_t* s2 = reinterpret_cast<const uint32_t*>(&sk[h]);
#pragma unroll
            for (int e = 0; e < 4; e++) { const float2 f = cunpack16<F16>(s2[e]); v[8 * h + 2 * e] += f.x; v[8 * h + 2 * e + 1] += f.y; }
          }
        }
        if (nuse_skip) {                                           // these registers are free again: next tile's residual row
#pragma unroll
          for (int h = 0; h < CW / 8; h++) sk[h] = __ldg(reinterpret_cast<const uint4*>(P.skip + (size_t)np * kC + c0) + h);
        }
        if (writes) {
          uint4* dst = reinterpret_cast<uint4*>(P.out + (size_t)p * kC + c0);
#pragma unroll
          for (int h = 0; h < CW / 8; h++) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const float x0 = interior ? fmaxf(v[8 * h + 2 * e], v[8 * h + 2 * e] * P.slope) : 0.f;
              const float x1 = interior ? fmaxf(v[8 * h + 2 * e + 1], v[8 * h + 2 * e + 1] * P.slope) : 0.f;
              pk[e] = cpack16<F16>(x0, x1);
            }
            dst[h] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      }
      p = np; writes = nwrites; interior = ninterior; wp = nwp; hp = nhp; dp = ndp; n_ = nn; use_skip = nuse_skip;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0)
    for (int i = 0; i < 2000; i++) __nanosleep(1000);        // let copies in flight land before the CTA gives its memory back
  __syncthreads();
  cluster_sync_all();                      // neither CTA leaves while its partner can still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// ---- network input: fp32 NDHWC with C <= 16 channels -> the first 16 channels (32 bytes) of the padded bf16 rows; the
// border rows and the channels beyond 16 of this buffer are never written (zero from allocation; the first layer's
// MMAs read only the first 16 channels)
template <bool F16>
__global__ void __launch_bounds__(256) conv_pack_input_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                              int N, int D, int H, int W, int C) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the first layer may set up while this kernel runs
  const long long nvox = (long long)N * D * H * W;
  for (long long v = (long long)blockIdx.x * 256 + threadIdx.x; v < nvox; v += (long long)gridDim.x * 256) {
    const int w_ = (int)(v % W), h_ = (int)((v / W) % H), d_ = (int)((v / ((long long)W * H)) % D), n_ = (int)(v / ((long long)W * H * D));
    const long long p = (((long long)n_ * (D + 2) + d_ + 1) * (H + 2) + h_ + 1) * (W + 2) + w_ + 1;
    float f[16];
#pragma unroll
    for (int c = 0; c < 16; c++) f[c] = c < C ? __ldg(x + v * C + c) : 0.f;
    uint32_t pk[8];
#pragma unroll
    for (int e = 0; e < 8; e++) pk[e] = cpack16<F16>(f[2 * e], f[2 * e + 1]);
    uint4* dst = reinterpret_cast<uint4*>(out + p * kC);
    dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn conv_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return nullptr;
  fn = (EncodeTiledFn)p;
  return fn;
}

bool make_map(CUtensorMap* m, void* base, long long rows, int box_rows) {
  EncodeTiledFn enc = conv_encode_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)kC, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)kC * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kC, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// geometry of the activation ring for a volume whose padded W extent is Wp: a stage holds 128 + 2 Wp rows, loaded as
// nbox boxes of box_rows (<= 256, multiple of 8) rows
struct RingGeom { int stage_bytes, nstages, box_rows, nbox; };
bool ring_geometry(int Wp, RingGeom* g) {
  const int R = kTile + 2 * Wp + 2 * kHalo;
  g->nbox = (R + 255) / 256;
  g->box_rows = (((R + g->nbox - 1) / g->nbox) + 7) / 8 * 8;
  g->stage_bytes = ((g->nbox * g->box_rows * kC * 2) + 1023) / 1024 * 1024;
  g->nstages = kRingBytes / g->stage_bytes;
  if (g->nstages > kMaxStages) g->nstages = kMaxStages;
  return g->nstages >= 2;
}

uint16_t to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

uint16_t to_f16(float f) {
  const __half h = __float2half_rn(f);
  uint16_t u;
  std::memcpy(&u, &h, 2);
  return u;
}

float slope_of(const LayerHost& L) { return L.act == ACT_NONE ? 1.f : L.act == ACT_RELU ? 0.f : L.slope; }

}  // namespace

struct ConvTcModel {
  std::vector<LayerHost> meta;
  std::vector<void*> w; std::vector<float*> b;             // per layer: bf16 [27 * rows][64] (rows = 64, last layer 16), fp32 bias [64]
  std::vector<CUtensorMap> wmaps;
  __nv_bfloat16* buf[4] = {nullptr, nullptr, nullptr, nullptr};   // three rotating activation volumes + the packed input (allocations)
  long long front = 0;                                            // zero rows in front of each volume inside its allocation
  CUtensorMap amaps[4];
  long long P = 0;
  int shape[4] = {0, 0, 0, 0};
  int* status = nullptr;
  bool f16 = false;                                               // operands and stored activations are IEEE half instead of bf16
};

bool conv_tc_supported(const ModelHost& M, std::string* why) {
  auto no = [&](const char* w) { if (why) *why = w; return false; };
  const int nl = (int)M.layers.size();
  if (nl < 3) return no("the tensor-core conv path needs a first, at least one 64->64 and a last layer");
  for (int l = 0; l < nl; l++) {
    const LayerHost& L = M.layers[l];
    if (L.kind != LAYER_CONV3D || L.ksize != 3 || L.pad != 1) return no("only 3x3x3 pad-1 convolutions");
    if (L.act == ACT_LEAKY && !(L.slope >= 0.f && L.slope <= 1.f)) return no("LeakyReLU slope outside [0, 1]");
    if (l == 0 && (L.cout != kC || L.cin < 1 || L.cin > kEdgeC || (L.flags & LFLAG_ADD_SKIP))) return no("first layer must be 1..16 channels -> 64");
    if (l == nl - 1 && (L.cin != kC || L.cout < 1 || L.cout > kEdgeC || (L.flags & (LFLAG_ADD_SKIP | LFLAG_SAVE_SKIP))))
      return no("last layer must be 64 -> 1..16 channels");
    if (l > 0 && l < nl - 1 && (L.cin != kC || L.cout != kC)) return no("middle layers must be 64 -> 64");
  }
  return true;
}

void conv_tc_destroy(ConvTcModel* m) {
  if (!m) return;
  for (void* p : m->w) cudaFree(p);
  for (float* p : m->b) cudaFree(p);
  for (auto& p : m->buf) cudaFree(p);
  cudaFree(m->status);
  delete m;
}

ConvTcModel* conv_tc_create(const ModelHost& M, bool f16, std::string* err) {
  std::string why;
  if (!conv_tc_supported(M, &why)) { if (err) *err = why; return nullptr; }
  ConvTcModel* m = new ConvTcModel();
  m->f16 = f16;
  auto fail = [&](const std::string& w) { if (err) *err = w; conv_tc_destroy(m); return (ConvTcModel*)nullptr; };
  const int nl = (int)M.layers.size();
  auto upload = [&](const void* h, size_t bytes) -> void* {
    void* d = nullptr;
    if (cudaMalloc(&d, bytes) != cudaSuccess) return nullptr;
    cudaMemcpy(d, h, bytes, cudaMemcpyHostToDevice);
    return d;
  };
  for (int l = 0; l < nl; l++) {
    const LayerHost& L = M.layers[l];
    LayerHost meta = L; meta.W.clear(); meta.b.clear();
    m->meta.push_back(meta);
    // [tap][cout][cin] with cin contiguous (K-major B operand), zero where the layer has no channel
    const int rows = l == nl - 1 ? kEdgeC : kC;
    std::vector<uint16_t> wb((size_t)27 * rows * kC, 0);
    for (int f = 0; f < L.cout; f++)
      for (int c = 0; c < L.cin; c++)
        for (int t = 0; t < 27; t++) wb[((size_t)t * rows + f) * kC + c] = f16 ? to_f16(L.W[((size_t)f * L.cin + c) * 27 + t]) : to_bf16(L.W[((size_t)f * L.cin + c) * 27 + t]);
    std::vector<float> bias(kC, 0.f);
    for (int f = 0; f < L.cout; f++) bias[f] = L.b[f];
    void* dw = upload(wb.data(), wb.size() * 2);
    float* db = (float*)upload(bias.data(), bias.size() * 4);
    if (!dw || !db) return fail("out of device memory for conv weights");
    m->w.push_back(dw); m->b.push_back(db);
    CUtensorMap map;
    if (!make_map(&map, dw, 27 * rows, (kShiftA ? rows : 3 * rows) / 2)) return fail("cuTensorMapEncodeTiled failed for conv weights");
    m->wmaps.push_back(map);
  }
  if (cudaMalloc(&m->status, sizeof(int)) != cudaSuccess) return fail("out of device memory");
  cudaMemset(m->status, 0, sizeof(int));
  const cudaFuncAttribute att = cudaFuncAttributeMaxDynamicSharedMemorySize;
  if (cudaFuncSetAttribute(conv3d_tc_kernel<4, kC, false, false>, att, kConvSmem) != cudaSuccess ||
      cudaFuncSetAttribute(conv3d_tc_kernel<1, kC, false, false>, att, kConvSmem) != cudaSuccess ||
      cudaFuncSetAttribute(conv3d_tc_kernel<4, kEdgeC, true, false>, att, kConvSmem) != cudaSuccess ||
      cudaFuncSetAttribute(conv3d_tc_kernel<4, kC, false, true>, att, kConvSmem) != cudaSuccess ||
      cudaFuncSetAttribute(conv3d_tc_kernel<1, kC, false, true>, att, kConvSmem) != cudaSuccess ||
      cudaFuncSetAttribute(conv3d_tc_kernel<4, kEdgeC, true, true>, att, kConvSmem) != cudaSuccess)
    return fail("cannot reserve shared memory for the tensor-core conv kernel");
  return m;
}

bool conv_tc_forward(ConvTcModel* m, const float* x, float* y, int N, int D, int H, int W, cudaStream_t s, std::string* err) {
  const long long nvox = (long long)N * D * H * W;
  if (nvox <= 0) { if (err) *err = "conv3d model: set the input extent (option conv_shape = N,D,H,W)"; return false; }
  const long long P = (long long)N * (D + 2) * (H + 2) * (W + 2);
  if (P >= (1LL << 31) - 4096) { if (err) *err = "conv3d model: volume too large for 32-bit TMA row coordinates"; return false; }
  if (m->P != P || m->shape[0] != N || m->shape[1] != D || m->shape[2] != H || m->shape[3] != W) {
    for (auto& p : m->buf) { cudaFree(p); p = nullptr; }
    for (int b = 0; b < 4; b++) {
      // zero rows on both sides of the volume cover every tap shift and the last (partial) pair of tiles, so the
      // kernel's copies never leave the allocation
      const long long front = (((long long)(H + 2) * (W + 2) + (W + 2) + 2 + 7) / 8) * 8, rows = front + P + front + 512;
      m->front = front;
      if (cudaMalloc(&m->buf[b], (size_t)rows * kC * 2) != cudaSuccess) { if (err) *err = "out of device memory for conv activations"; return false; }
      cudaMemsetAsync(m->buf[b], 0, (size_t)rows * kC * 2, s);     // padding and border must be zero before the first layer writes the interior
      RingGeom g;
      if (!ring_geometry(W + 2, &g)) { if (err) *err = "conv3d bf16 path: W too large for the shared-memory activation ring (use precision=fp32)"; return false; }
      if (!make_map(&m->amaps[b], m->buf[b], rows, g.box_rows)) { if (err) *err = "cuTensorMapEncodeTiled failed for conv activations"; return false; }
    }
    m->P = P; m->shape[0] = N; m->shape[1] = D; m->shape[2] = H; m->shape[3] = W;
  }
  RingGeom geom;
  ring_geometry(W + 2, &geom);
  const int nl = (int)m->meta.size();
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  {
    const long long blocks = (nvox + 255) / 256;
    const unsigned pg = (unsigned)(blocks < sms * 8 ? blocks : sms * 8);
    if (m->f16) conv_pack_input_kernel<true><<<pg, 256, 0, s>>>(x, m->buf[3] + m->front * kC, N, D, H, W, m->meta[0].cin);
    else conv_pack_input_kernel<false><<<pg, 256, 0, s>>>(x, m->buf[3] + m->front * kC, N, D, H, W, m->meta[0].cin);
  }
  const long long ntiles = (P + kTileOut - 1) / kTileOut, npairs = (ntiles + 1) / 2;
  const int max_pairs = sms / 2 > 0 ? sms / 2 : 1;
  const int grid = 2 * (int)(npairs < max_pairs ? npairs : max_pairs);          // clusters of two CTAs
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kConvThreads); cfg.dynamicSmemBytes = kConvSmem; cfg.stream = s;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;    // a layer may start while the one before it drains
  at[1].val.programmaticStreamSerializationAllowed = 1;
  static const bool pdl = std::getenv("FORTIS_NO_PDL") == nullptr;
  cfg.attrs = at; cfg.numAttrs = pdl ? 2 : 1;
  static const bool want_prof = std::getenv("FORTIS_TC_PROF") != nullptr;
  static long long* dprof = nullptr;
  if (want_prof && !dprof) cudaMalloc(&dprof, 16 * sizeof(long long));
  if (want_prof) cudaMemsetAsync(dprof, 0, 16 * sizeof(long long), s);
  int cur = 3, skip = -1;
  for (int l = 0; l < nl; l++) {
    const LayerHost& L = m->meta[l];
    int dst = -1;
    for (int b = 0; b < 3; b++) if (b != cur && b != skip) { dst = b; break; }
    if ((L.flags & LFLAG_ADD_SKIP) && skip < 0) { if (err) *err = "conv3d model: a layer adds a skip that was never saved"; return false; }
    ConvTcParams P_;
    std::memset(&P_, 0, sizeof P_);
    P_.amap = m->amaps[cur]; P_.wmap = m->wmaps[l]; P_.bias = m->b[l];
    P_.skip = (L.flags & LFLAG_ADD_SKIP) ? m->buf[skip] + m->front * kC : nullptr;
    P_.out = m->buf[dst] + m->front * kC; P_.y = y; P_.F = L.cout; P_.front = (int)m->front;
    P_.stage_bytes = geom.stage_bytes; P_.nstages = geom.nstages; P_.box_rows = geom.box_rows; P_.nbox = geom.nbox;
    P_.wait_limit = g_tc_test.wait_limit ? g_tc_test.wait_limit : kWaitLimit;
    P_.test_skip_stage = g_tc_test.skip_stage;
    P_.D = D; P_.H = H; P_.W = W; P_.P = P; P_.slope = slope_of(L); P_.status = m->status; P_.prof = (want_prof && l == 2) ? dprof : nullptr;
    const cudaError_t le = m->f16 ? (l == nl - 1 ? cudaLaunchKernelEx(&cfg, conv3d_tc_kernel<4, kEdgeC, true, true>, P_)
                                     : l == 0    ? cudaLaunchKernelEx(&cfg, conv3d_tc_kernel<1, kC, false, true>, P_)
                                                 : cudaLaunchKernelEx(&cfg, conv3d_tc_kernel<4, kC, false, true>, P_))
                                  : (l == nl - 1 ? cudaLaunchKernelEx(&cfg, conv3d_tc_kernel<4, kEdgeC, true, false>, P_)
                                     : l == 0    ? cudaLaunchKernelEx(&cfg, conv3d_tc_kernel<1, kC, false, false>, P_)
                                                 : cudaLaunchKernelEx(&cfg, conv3d_tc_kernel<4, kC, false, false>, P_));
    if (le != cudaSuccess) { if (err) *err = std::string("tensor-core conv launch: ") + cudaGetErrorString(le); return false; }
    if (L.flags & LFLAG_SAVE_SKIP) skip = dst;
    cur = dst;
  }
  if (want_prof) {
    long long h[16];
    cudaStreamSynchronize(s);
    cudaMemcpy(h, dprof, sizeof h, cudaMemcpyDeviceToHost);
    std::fprintf(stderr, "conv prof, layer 2 (cycles, CTA 0): mma wait acc_empty %lld full %lld weights %lld issue %lld | tma wait empty %lld issue %lld | "
                 "epilogue wait acc_full %lld boundary %lld rows %lld\n", h[0], h[1], h[3], h[2], h[6], h[7], h[8], h[9], h[10]);
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { if (err) *err = std::string("tensor-core conv launch: ") + cudaGetErrorString(e); return false; }
  return true;
}

void conv_tc_clear_status(ConvTcModel* m) {
  if (m && m->status) cudaMemset(m->status, 0, sizeof(int));
}

int conv_tc_status(ConvTcModel* m) {
  int v = 0;
  if (m && m->status) cudaMemcpy(&v, m->status, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

}  // namespace fortis
