// Fused gather -> MLP -> scatter on the 5th-generation tensor cores (tcgen05, sm_100a), bf16 operands, fp32
// accumulation in tensor memory, activations never leaving the SM between layers.
//
// Replaces, for wide column MLPs, the reference's per-layer lowering: fortis_gemm (cuBLAS SGEMM) + a separate
// bias/activation epilogue kernel per layer (runtime/fortis_rt.c:45-75, compiler/FortisFuse.cpp:616-624, 687-760),
// with fortis_gather_k in front and fortis_scatter_k behind (driver/fortis_gather_emit.py:52-62, 75-83).
//
// One persistent CTA per SM processes tiles of 128 columns (rows of the model batch).  Per tile and layer
//     D[128 x N] = A[128 x K] . W[N x K]^T,  N processed in chunks of 64 output features.
//   * A (the layer's input activations, bf16) lives in TENSOR MEMORY: lane = row, two K values per 32-bit column
//     (K <= 768 -> 384 columns).  The MMAs take A from TMEM and B from shared memory, so shared-memory read
//     bandwidth is spent on the weights only.
//   * W streams from L2 through a ring of 32 KB TMA stages (64 features x 256 k, 128-byte swizzle, one 3-D tile
//     load per stage, no multicast).
//   * D: two 64-column fp32 accumulators in TMEM; the epilogue of chunk c overlaps the MMAs of chunk c+1.
//   * The epilogue (8 warps; thread = one row x 32 features) adds bias, applies the activation, rounds to bf16 and
//     parks the chunk: chunks 0-7 in shared memory, chunks 8-11 in registers (A is still being read by later
//     chunks, so the output cannot overwrite it).  When the layer's last MMA has retired, the parked chunks are
//     written into the A columns with tcgen05.st and the next layer starts.
//   * Layer 0's A is produced by the same threads straight from the host's Fortran arrays (thread = row, so every
//     slot is a coalesced load); the last layer's epilogue stores straight into the host arrays and accumulates
//     the fp64 checksum.  This fusion is table-driven and covers fp32 arrays without lifted expressions; any other
//     descriptor is served by the standalone gather / scatter kernels writing X / reading Y around this kernel.
// TMEM: 384 (A) + 2 x 64 (D) = 512 columns.  Shared memory: 128 KB parked chunks + 3 x 32 KB weight ring.
//
// Every wait on an mbarrier is bounded; a wait that gives up records a code in the status word, raises a CTA-wide
// abort flag that turns all later waits into no-ops, and the CTA still frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "fortis_device.cuh"
#include "fortis_kernels.h"
#include "fortis_model.h"
#include "fortis_tc.cuh"

namespace fortis {

namespace {

constexpr int kTileM = 128;
constexpr int kChunkN = 64;                 // output features per accumulator
constexpr int kStageK = 256;                // k extent of one weight stage: four 64-wide swizzled sub-tiles, ONE TMA
constexpr int kStageBytes = kChunkN * kStageK * 2;   // 32 KB
constexpr int kSubBytes = kChunkN * 64 * 2;          // one 64 x 64 sub-tile, 8 KB
constexpr int kStages = 3;
constexpr int kSmemChunks = 8;              // parked chunks held in shared memory; the rest in registers
constexpr int kMaxChunks = 12;              // 768 / 64
constexpr int kMaxK = 768;
constexpr int kMaxLayers = 8;
constexpr int kEpiThreads = 256;
constexpr int kThreads = kEpiThreads + 64;  // + TMA warp + MMA warp
constexpr int kParkBytes = kSmemChunks * kTileM * kChunkN * 2;      // 128 KB
constexpr int kRingBytes = kStages * kStageBytes;                   // 96 KB
constexpr int kBarBytes = 256;
constexpr int kFastIn = 256, kFastOut = 128;          // widest model input / output the fast I/O tables hold
constexpr int kTabBytes = kFastIn * 5 + kFastOut * 5 + 2 * kMaxArrays * 8;   // uint32 offset + uint8 code per slot / store, array bases
constexpr int kSmemBytes = kParkBytes + kRingBytes + kBarBytes + kTabBytes;   // the base must be 1024-byte aligned
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCol0 = 384;

// status codes (which wait gave up)
enum { ST_OK = 0, ST_FULL = 1, ST_EMPTY = 2, ST_ACC_FULL = 3, ST_ACC_EMPTY = 4, ST_A_READY = 5, ST_SMEM_ALIGN = 6 };

struct TcLayer {
  int K, N;                // padded: K multiple of 256, N multiple of 64 (hidden: multiple of 256)
  int n_real;              // unpadded output width
  int act;
  float slope;             // branch-free activation: act(v) = max(v, v * slope); none -> 1, ReLU -> 0, LeakyReLU -> slope
  const float* bias;       // [N] padded with zeros
  const float* scale;      // [N] per-output-channel dequantisation scale (fp8 weights) or null
};

// Stride class of a fast gather / scatter: element offset of a row = ci*si + cj*sj + kk*sk
struct StrideClass { long long si, sj, sk; };

struct TcParams {
  CUtensorMap maps[kMaxLayers];
  TcLayer layer[kMaxLayers];
  int nlayers;
  int n_in, n_out;                       // unpadded model widths
  const float* in_div;                   // optional
  const float* out_mul;                  // optional
  const float* relu_mask;                // optional
  // gather side
  const IoPlanDev* GP; const Access* slots; ArrayTable TG;
  const float* X;                        // (rows, n_in) when GP is null
  // scatter side
  const IoPlanDev* SP; const StoreTarget* stores; ArrayTable TS;
  const int* slot_head; const int* store_next;   // per output: first store index (-1: none), chain
  float* Y;                              // optional (rows, n_out)
  RowGeom g;
  long long nrows;
  double* partials;
  int* status;
  long long* prof;                       // optional cycle counters of CTA 0 (diagnostics; null in normal runs)
  // fast I/O: every access is fp32 without lifted expressions and uses one of two stride classes; the per-slot
  // (array, class, constant offset) triples are unpacked into shared memory once per CTA
  int fast_in, fast_out;
  StrideClass cin[2], cout[2];
  const Access* store_by_slot;           // [n_out] store target per model output (array < 0: none), fast_out only
};

using namespace tc;

// shared-memory matrix descriptor: K-major, 128-byte swizzle, rows 128 B apart, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t make_b_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);            // start address
  d |= (uint64_t)0 << 16;                            // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset
  d |= (uint64_t)1 << 46;                            // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
  return d;
}

// instruction descriptor: D = f32, A and B both bf16 (format code 1) or both IEEE half (code 0), both K-major,
// N = 64, M = 128
template <bool F16> struct MlpIdesc {
  static constexpr uint32_t value = (1u << 4) | (F16 ? 0u : ((1u << 7) | (1u << 10))) | ((uint32_t)(kChunkN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
};
// two consecutive k values as one 32-bit tensor-memory column, in the kernel's 16-bit operand format
template <bool F16> __device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (F16) { const __half2 v = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t*>(&v); }
  else return pack_bf16(lo, hi);
}

__device__ __forceinline__ float act_f(float v, float slope) { return fmaxf(v, v * slope); }

// cycle accounting for diagnostics: adds the time since *t to prof[slot] (CTA 0, one lane) and restarts the clock
__device__ __forceinline__ void prof_add(long long* prof, int slot, long long* t, bool who) {
  // always compiled (one well-predicted branch per call when prof is null): compiling it out makes the optimiser
  // restructure the role loops and nvcc's front end then runs for tens of minutes on this kernel
  if (prof && who) { const long long n = clock64(); atomicAdd((unsigned long long*)&prof[slot], (unsigned long long)(n - *t)); *t = n; }
}

// ---------------------------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------------------------
template <bool HAS_SCALE, bool F16>
__global__ void __launch_bounds__(kThreads, 1) mlp_tc_fused_kernel(const __grid_constant__ TcParams P) {
  constexpr uint32_t kIdesc = MlpIdesc<F16>::value;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = smem_u32(smem);                         // parked chunks: 8 x 16 KB at offset 0
  if (base & 1023u) {                                           // the swizzled weight stages need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(P.status, 0, ST_SMEM_ALIGN);
    return;
  }
  const uint32_t ring = base + kParkBytes;                      // kStages x 16 KB
  const uint32_t bars = ring + kRingBytes;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kStages;            // [kStages] each
  const uint32_t bar_acc_full = bars + 16 * kStages, bar_acc_empty = bar_acc_full + 16;   // [2] each
  const uint32_t bar_a_ready = bar_acc_empty + 16;
  // barrier block (256 B): full [0,48) empty [48,96) acc_full [96,112) acc_empty [112,128) a_ready [128,136)
  // tmem base 144, abort flag 148, checksum scratch [160,224)
  uint32_t* tmem_slot = (uint32_t*)(smem + kParkBytes + kRingBytes + 144);
  volatile int* abort_flag = (volatile int*)(smem + kParkBytes + kRingBytes + 148);
  uint32_t* s_off = (uint32_t*)(smem + kParkBytes + kRingBytes + kBarBytes);          // [kFastIn] input slot offsets
  uint32_t* o_off = s_off + kFastIn;                                                  // [kFastOut] store offsets
  uint8_t* s_code = (uint8_t*)(o_off + kFastOut);                                     // array | class << 7, 0xFF: none
  uint8_t* o_code = s_code + kFastIn;
  // array base pointers of the fast paths, copied out of the kernel parameters so that the unrolled load / store
  // loops index shared memory (indexing the parameter block dynamically makes nvcc's front end crawl)
  const float** s_base_in = (const float**)(o_code + kFastOut);
  float** s_base_out = (float**)(s_base_in + kMaxArrays);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long ntiles = (P.nrows + kTileM - 1) / kTileM;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int b = 0; b < 2; b++) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, kEpiThreads); }
    mbar_init(bar_a_ready, kEpiThreads);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < kMaxArrays) {
    s_base_in[threadIdx.x] = (const float*)P.TG.base[threadIdx.x];
    s_base_out[threadIdx.x] = (float*)P.TS.base[threadIdx.x];
  }
  if (P.fast_in)
    for (int q = threadIdx.x; q < kFastIn; q += kThreads) {
      uint8_t code = 0xFF; uint32_t off = 0;
      if (q < P.n_in) {
        const Access a = P.slots[q];
        code = (uint8_t)(a.array | ((a.si == P.cin[0].si && a.sj == P.cin[0].sj && a.sk == P.cin[0].sk) ? 0 : 0x80));
        off = (uint32_t)a.off0;
      }
      s_code[q] = code; s_off[q] = off;
    }
  if (P.fast_out)
    for (int n = threadIdx.x; n < kFastOut; n += kThreads) {
      uint8_t code = 0xFF; uint32_t off = 0;
      if (n < P.n_out && P.store_by_slot[n].array >= 0) {
        const Access a = P.store_by_slot[n];
        code = (uint8_t)(a.array | ((a.si == P.cout[0].si && a.sj == P.cout[0].sj && a.sk == P.cout[0].sk) ? 0 : 0x80));
        off = (uint32_t)a.off0;
      }
      o_code[n] = code; o_off[n] = off;
    }
  if (warp == 8 && lane < P.nlayers)
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&P.maps[lane])) : "memory");
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer (whole warp, one lane issues)
    uint32_t s = 0, ph = 0;
    const bool pw = blockIdx.x == 0 && lane == 0;
    long long pt = clock64();
    bool stop = false;
    for (long long tile = blockIdx.x; tile < ntiles && !stop; tile += gridDim.x)
      for (int l = 0; l < P.nlayers && !stop; l++) {
        const int nchunks = P.layer[l].N / kChunkN, nkb = P.layer[l].K / kStageK;
        const CUtensorMap* map = &P.maps[l];
        for (int c = 0; c < nchunks && !stop; c++)
          for (int kb = 0; kb < nkb; kb++) {
            prof_add(P.prof, 17, &pt, pw);
            if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, P.status, ST_EMPTY)) { stop = true; break; }
            prof_add(P.prof, 16, &pt, pw);
            mbar_expect_tx(bar_full + 8 * s, kStageBytes);
            const uint32_t dst = ring + s * kStageBytes;
            tma_load_3d(dst, map, 0, c * kChunkN, kb * (kStageK / 64), bar_full + 8 * s);
            if (++s == kStages) { s = 0; ph ^= 1; }
          }
      }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
    uint32_t s = 0, ph = 0, acc_it = 0, a_it = 0;
    const uint64_t desc_hi = make_b_desc(0) & 0xFFFFFFFF00000000ull;
    const bool pw = blockIdx.x == 0 && lane == 0;
    long long pt = clock64();
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x)
      for (int l = 0; l < P.nlayers; l++, a_it++) {
        const int nchunks = P.layer[l].N / kChunkN, nkb = P.layer[l].K / kStageK;
        prof_add(P.prof, 0, &pt, pw);
        mbar_wait(bar_a_ready, a_it & 1, abort_flag, P.status, ST_A_READY);      // A of this layer is in TMEM
        prof_add(P.prof, 1, &pt, pw);
        tc_fence_after();
        for (int c = 0; c < nchunks; c++, acc_it++) {
          const uint32_t b = acc_it & 1, aph = (acc_it >> 1) & 1;
          prof_add(P.prof, 0, &pt, pw);
          mbar_wait(bar_acc_empty + 8 * b, aph ^ 1, abort_flag, P.status, ST_ACC_EMPTY);
          prof_add(P.prof, 2, &pt, pw);
          tc_fence_after();
          const uint32_t d_tmem = tmem + kAccCol0 + b * kChunkN;
          for (int kb = 0; kb < nkb; kb++) {
            prof_add(P.prof, 0, &pt, pw);
            mbar_wait(bar_full + 8 * s, ph, abort_flag, P.status, ST_FULL);
            prof_add(P.prof, 3, &pt, pw);
            tc_fence_after();
            // descriptor of the stage's first 64-wide k sub-tile; the next sub-tile starts kSubBytes further, and
            // stepping k by 16 inside a 128-byte swizzle row adds 32 bytes (the address field is in 16-byte units)
            const uint32_t sb = ring + s * kStageBytes;
            const uint64_t bd0 = desc_hi | (uint64_t)((sb >> 4) & 0x3FFF);
            const uint32_t a0 = tmem + kb * (kStageK / 2);
            tc_mma_ts_first<kIdesc>(d_tmem, a0, bd0, (uint32_t)kb);
#pragma unroll
            for (int j = 1; j < kStageK / 16; j++)
              tc_mma_ts_acc<kIdesc>(d_tmem, a0 + j * 8, bd0 + (uint64_t)((j >> 2) * (kSubBytes >> 4) + (j & 3) * 2));
            tc_commit(bar_empty + 8 * s);                   // stage reusable once these MMAs have read it
            if (++s == kStages) { s = 0; ph ^= 1; }
          }
          tc_commit(bar_acc_full + 8 * b);                  // accumulator complete
        }
      }
  } else {
    // ------------------------------------------------------------------ row warps: gather, epilogues, scatter
    const int quad = warp & 3, half = warp >> 2;              // TMEM lane quadrant, which 32 of a chunk's 64 features
    const int r = quad * 32 + lane;                           // row of the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    uint32_t acc_it = 0;
    double csum = 0.0;
    const bool pw = blockIdx.x == 0 && threadIdx.x == 0;
    long long pt = clock64();
    uint32_t kept[(kMaxChunks - kSmemChunks) * 16];           // parked chunks 8..11 of this thread (bf16 pairs)
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
      const long long row = tile * kTileM + r;
      const bool live = row < P.nrows;
      long long ci = 0, cj = 0, kk = 0;
      if (live) row_to_pos(P.g, row, &ci, &cj, &kk);
      // ---- layer 0 input: this thread's half of the row, 32 features (16 packed columns) at a time
      {
        const int K0 = P.layer[0].K, per = K0 / 2;            // features per half
        if (P.fast_in) {
          // one position per stride class, then 32 independent loads per step: base[array] + offset + position
          const long long pos0 = ci * P.cin[0].si + cj * P.cin[0].sj + kk * P.cin[0].sk;
          const long long pos1 = ci * P.cin[1].si + cj * P.cin[1].sj + kk * P.cin[1].sk;
          for (int q0 = half * per; q0 < (half + 1) * per; q0 += 32) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const uint32_t code = s_code[q0 + j];
              v[j] = 0.f;
              if (live && code != 0xFF)
                v[j] = __ldg(s_base_in[code & 0x7F] + ((long long)s_off[q0 + j] + ((code & 0x80) ? pos1 : pos0)));
            }
            if (P.in_div) {
#pragma unroll
              for (int j = 0; j < 32; j++) if (q0 + j < P.n_in) v[j] = __fdiv_rn(v[j], __ldg(P.in_div + q0 + j));
            }
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; j++) pk[j] = pack16<F16>(v[2 * j], v[2 * j + 1]);
            tmem_st16(lane_addr + (uint32_t)(q0 >> 1), pk);
          }
        } else {
          // input already materialised as X (rows, n_in): array-form calls, and descriptors the fast tables cannot
          // express (lifted expressions, f64 arrays, scalars), for which the standalone gather kernel ran first
          for (int q0 = half * per; q0 < (half + 1) * per; q0 += 32) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = (live && q0 + j < P.n_in) ? __ldg(P.X + row * P.n_in + q0 + j) : 0.f;
            if (P.in_div) {
#pragma unroll
              for (int j = 0; j < 32; j++) if (q0 + j < P.n_in) v[j] = __fdiv_rn(v[j], __ldg(P.in_div + q0 + j));
            }
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; j++) pk[j] = pack16<F16>(v[2 * j], v[2 * j + 1]);
            tmem_st16(lane_addr + (uint32_t)(q0 >> 1), pk);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(bar_a_ready);
        prof_add(P.prof, 9, &pt, pw);
      }
      for (int l = 0; l < P.nlayers; l++) {
        const TcLayer& L = P.layer[l];
        const int nchunks = L.N / kChunkN;
        const bool last = l == P.nlayers - 1;
        const float slope = L.slope;
        if (!last) {
          // epilogue of one chunk: accumulator -> (x scale) + bias -> activation -> 16 packed bf16 pairs
          auto chunk_epilogue = [&](int c, uint32_t (&pk)[16]) {
            const uint32_t b = acc_it & 1, aph = (acc_it >> 1) & 1;
            acc_it++;
            const int n0 = c * kChunkN + half * 32;
            // the 32 biases of this thread's features: warp-uniform 16-byte loads issued before the wait
            float4 bq[8];
#pragma unroll
            for (int j = 0; j < 8; j++) bq[j] = __ldg(reinterpret_cast<const float4*>(L.bias + n0) + j);
            prof_add(P.prof, 11, &pt, pw);
            mbar_wait(bar_acc_full + 8 * b, aph, abort_flag, P.status, ST_ACC_FULL);
            prof_add(P.prof, 10, &pt, pw);
            tc_fence_after();
            uint32_t a[32];
            tmem_ld32(lane_addr + kAccCol0 + b * kChunkN + half * 32, a);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(bar_acc_empty + 8 * b);             // the MMA warp may refill this accumulator
            if (HAS_SCALE) {
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const float4 sq = __ldg(reinterpret_cast<const float4*>(L.scale + n0) + j);
                a[4 * j] = __float_as_uint(__uint_as_float(a[4 * j]) * sq.x);
                a[4 * j + 1] = __float_as_uint(__uint_as_float(a[4 * j + 1]) * sq.y);
                a[4 * j + 2] = __float_as_uint(__uint_as_float(a[4 * j + 2]) * sq.z);
                a[4 * j + 3] = __float_as_uint(__uint_as_float(a[4 * j + 3]) * sq.w);
              }
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const float v0 = act_f(__uint_as_float(a[4 * j]) + bq[j].x, slope);
              const float v1 = act_f(__uint_as_float(a[4 * j + 1]) + bq[j].y, slope);
              const float v2 = act_f(__uint_as_float(a[4 * j + 2]) + bq[j].z, slope);
              const float v3 = act_f(__uint_as_float(a[4 * j + 3]) + bq[j].w, slope);
              pk[2 * j] = pack16<F16>(v0, v1);
              pk[2 * j + 1] = pack16<F16>(v2, v3);
            }
          };
          // chunks parked in shared memory: a rolled loop (the address depends on c only arithmetically)
          const int nsm = nchunks < kSmemChunks ? nchunks : kSmemChunks;
#pragma unroll 1
          for (int c = 0; c < nsm; c++) {
            uint32_t pk[16];
            chunk_epilogue(c, pk);
            // [chunk][half][16-byte piece][row]: lanes are rows, so every store is conflict-free
            uint8_t* dst = smem + c * (kTileM * kChunkN * 2) + half * (kTileM * 64) + r * 16;
#pragma unroll
            for (int p = 0; p < 4; p++)
              *reinterpret_cast<uint4*>(dst + p * (kTileM * 16)) = make_uint4(pk[4 * p], pk[4 * p + 1], pk[4 * p + 2], pk[4 * p + 3]);
          }
          // chunks parked in registers: unrolled so that `kept` is indexed statically
#pragma unroll
          for (int c = kSmemChunks; c < kMaxChunks; c++) {
            if (c < nchunks) {
              uint32_t pk[16];
              chunk_epilogue(c, pk);
#pragma unroll
              for (int j = 0; j < 16; j++) kept[(c - kSmemChunks) * 16 + j] = pk[j];
            }
          }
          // every MMA of this layer has retired (its last accumulator was complete), so A may be overwritten:
          // move the parked chunks into the A columns and release the next layer
          prof_add(P.prof, 11, &pt, pw);
#pragma unroll 1
          for (int c = 0; c < nsm; c++) {
            uint32_t pk[16];
            const uint8_t* src = smem + c * (kTileM * kChunkN * 2) + half * (kTileM * 64) + r * 16;
#pragma unroll
            for (int p = 0; p < 4; p++) {
              const uint4 q = *reinterpret_cast<const uint4*>(src + p * (kTileM * 16));
              pk[4 * p] = q.x; pk[4 * p + 1] = q.y; pk[4 * p + 2] = q.z; pk[4 * p + 3] = q.w;
            }
            tmem_st16(lane_addr + (uint32_t)(c * (kChunkN / 2) + half * 16), pk);
          }
#pragma unroll
          for (int c = kSmemChunks; c < kMaxChunks; c++) {
            if (c < nchunks) {
              uint32_t pk[16];
#pragma unroll
              for (int j = 0; j < 16; j++) pk[j] = kept[(c - kSmemChunks) * 16 + j];
              tmem_st16(lane_addr + (uint32_t)(c * (kChunkN / 2) + half * 16), pk);
            }
          }
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(bar_a_ready);
          prof_add(P.prof, 12, &pt, pw);
        } else {
          // ---- last layer: bias, output scaling / masks, then straight into the host arrays
          const long long opos0 = ci * P.cout[0].si + cj * P.cout[0].sj + kk * P.cout[0].sk;
          const long long opos1 = ci * P.cout[1].si + cj * P.cout[1].sj + kk * P.cout[1].sk;
          for (int c = 0; c < nchunks; c++) {
            const uint32_t b = acc_it & 1, aph = (acc_it >> 1) & 1;
            acc_it++;
            const int n0 = c * kChunkN + half * 32;
            float4 bq[8];
#pragma unroll
            for (int j = 0; j < 8; j++) bq[j] = __ldg(reinterpret_cast<const float4*>(L.bias + n0) + j);
            prof_add(P.prof, 13, &pt, pw);
            mbar_wait(bar_acc_full + 8 * b, aph, abort_flag, P.status, ST_ACC_FULL);
            prof_add(P.prof, 14, &pt, pw);
            tc_fence_after();
            uint32_t a[32];
            tmem_ld32(lane_addr + kAccCol0 + b * kChunkN + half * 32, a);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(bar_acc_empty + 8 * b);
            float v[32];
#pragma unroll
            for (int j = 0; j < 8; j++) {
              float4 sq = make_float4(1.f, 1.f, 1.f, 1.f);
              if (HAS_SCALE) sq = __ldg(reinterpret_cast<const float4*>(L.scale + n0) + j);
              v[4 * j] = act_f(__uint_as_float(a[4 * j]) * sq.x + bq[j].x, slope);
              v[4 * j + 1] = act_f(__uint_as_float(a[4 * j + 1]) * sq.y + bq[j].y, slope);
              v[4 * j + 2] = act_f(__uint_as_float(a[4 * j + 2]) * sq.z + bq[j].z, slope);
              v[4 * j + 3] = act_f(__uint_as_float(a[4 * j + 3]) * sq.w + bq[j].w, slope);
            }
            if (P.out_mul || P.relu_mask) {
#pragma unroll
              for (int j = 0; j < 32; j++) {
                const int n = n0 + j;
                if (n < P.n_out) {
                  if (P.out_mul) v[j] *= __ldg(P.out_mul + n);
                  if (P.relu_mask && __ldg(P.relu_mask + n) != 0.f) v[j] = fmaxf(v[j], 0.f);
                }
              }
            }
            if (live) {
              if (P.Y) {
#pragma unroll
                for (int j = 0; j < 32; j++) if (n0 + j < P.n_out) P.Y[row * P.n_out + n0 + j] = v[j];
              }
              if (P.fast_out) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                  const uint32_t code = (n0 + j < kFastOut) ? o_code[n0 + j] : 0xFFu;
                  if (code != 0xFF) {
                    s_base_out[code & 0x7F][(long long)o_off[n0 + j] + ((code & 0x80) ? opos1 : opos0)] = v[j];
                    csum += (double)v[j];
                  }
                }
              }
            }
          }
          prof_add(P.prof, 13, &pt, pw);
        }
      }
    }
    if (P.partials) {
      // per-CTA checksum partial in a fixed order: shuffle tree per warp, then warp results in index order
      double* wsum = (double*)(smem + kParkBytes + kRingBytes + 160);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) csum += __shfl_down_sync(0xffffffffu, csum, o);
      if (lane == 0) wsum[warp] = csum;
      asm volatile("bar.sync 1, %0;" ::"r"(kEpiThreads) : "memory");
      if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < 8; w++) t += wsum[w];
        P.partials[blockIdx.x] = t;
      }
    }
  }
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // a wait gave up: copies of this CTA may still be in flight; give them time to land before the shared memory
    // is handed back (bounded)
    for (int i = 0; i < 2000; i++) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return nullptr;
  fn = (EncodeTiledFn)p;
  return fn;
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);   // NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

uint16_t f32_to_f16(float f) {
  const __half h = __float2half_rn(f);
  uint16_t u;
  std::memcpy(&u, &h, 2);
  return u;
}

// nearest (ties-to-even) E4M3 value, saturating at +-448: 4 exponent bits (bias 7), 3 mantissa bits, subnormal
// step 2^-9
float e4m3_round(float v) {
  double a = std::fabs((double)v);
  if (a > 448.0) a = 448.0;
  int e = (int)std::floor(std::log2(a > 9.5367431640625e-07 ? a : 9.5367431640625e-07));
  if (e < -6) e = -6;
  if (e > 8) e = 8;
  const double step = std::ldexp(1.0, e - 3);
  double q = std::nearbyint(a / step) * step;
  if (q > 448.0) q = 448.0;
  return (float)(v < 0 ? -q : q);
}

}  // namespace

struct TcModel {
  int nlayers = 0, n_in = 0, n_out = 0;
  std::vector<void*> w;            // bf16 [N][K] padded
  std::vector<float*> bias, scale;
  float *in_div = nullptr, *out_mul = nullptr, *relu_mask = nullptr;
  TcLayer layer[kMaxLayers];
  CUtensorMap maps[kMaxLayers];
  bool has_scale = false, f16 = false;
};

bool tc_model_supported(const ModelHost& M, std::string* why) {
  auto no = [&](const char* w) { if (why) *why = w; return false; };
  if (!M.is_mlp()) return no("not an MLP");
  if ((int)M.layers.size() > kMaxLayers) return no("more than 8 layers");
  for (size_t l = 0; l < M.layers.size(); l++) {
    const LayerHost& L = M.layers[l];
    if (round_up(L.cin, kStageK) > kMaxK) return no("a layer input is wider than 768");
    if (L.act == ACT_LEAKY && !(L.slope >= 0.f && L.slope <= 1.f)) return no("LeakyReLU slope outside [0, 1]");
    const int npad = l + 1 < M.layers.size() ? round_up(L.cout, kStageK) : round_up(L.cout, kChunkN);
    if (npad > kMaxK) return no("a layer output is wider than 768");
  }
  return true;
}

int tc_grid(long long nrows) {
  const long long tiles = (nrows + kTileM - 1) / kTileM;
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return (int)(tiles < sms ? (tiles > 0 ? tiles : 1) : sms);
}

void tc_model_destroy(TcModel* m) {
  if (!m) return;
  for (void* p : m->w) cudaFree(p);
  for (float* p : m->bias) cudaFree(p);
  for (float* p : m->scale) cudaFree(p);
  cudaFree(m->in_div); cudaFree(m->out_mul); cudaFree(m->relu_mask);
  delete m;
}

TcModel* tc_model_create(const ModelHost& M, int precision, cudaStream_t s, std::string* err) {
  (void)s;
  std::string why;
  if (!tc_model_supported(M, &why)) { if (err) *err = why; return nullptr; }
  EncodeTiledFn enc = encode_fn();
  if (!enc) { if (err) *err = "cuTensorMapEncodeTiled is not available from the driver"; return nullptr; }
  TcModel* m = new TcModel();
  m->nlayers = (int)M.layers.size(); m->n_in = M.n_in(); m->n_out = M.n_out();
  auto fail = [&](const std::string& w) { if (err) *err = w; tc_model_destroy(m); return (TcModel*)nullptr; };
  for (int l = 0; l < m->nlayers; l++) {
    const LayerHost& L = M.layers[l];
    const int K = round_up(L.cin, kStageK);
    const int N = l + 1 < m->nlayers ? round_up(L.cout, kStageK) : round_up(L.cout, kChunkN);
    std::vector<uint16_t> wb((size_t)N * K, 0);
    std::vector<float> bias(N, 0.f), scale(N, 1.f);
    for (int n = 0; n < L.cout; n++) {
      bias[n] = L.b[n];
      float sc = 1.f;
      if (precision == PREC_FP8W) {
        float amax = 0.f;
        for (int k = 0; k < L.cin; k++) amax = std::fmax(amax, std::fabs(L.W[(size_t)n * L.cin + k]));
        sc = amax > 0.f ? amax / 448.0f : 1.0f;
        scale[n] = sc;
      }
      for (int k = 0; k < L.cin; k++) {
        float w = L.W[(size_t)n * L.cin + k];
        if (precision == PREC_FP8W) w = e4m3_round(w / sc);       // E4M3 codes are exact in bf16
        wb[(size_t)n * K + k] = precision == PREC_FP16 ? f32_to_f16(w) : f32_to_bf16(w);
      }
    }
    void* dw = nullptr; float *db = nullptr, *ds = nullptr;
    if (cudaMalloc(&dw, wb.size() * 2) != cudaSuccess || cudaMalloc(&db, N * 4) != cudaSuccess) return fail("out of device memory for packed weights");
    m->w.push_back(dw); m->bias.push_back(db);
    cudaMemcpy(dw, wb.data(), wb.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(db, bias.data(), N * 4, cudaMemcpyHostToDevice);
    if (precision == PREC_FP8W) {
      if (cudaMalloc(&ds, N * 4) != cudaSuccess) return fail("out of device memory for weight scales");
      cudaMemcpy(ds, scale.data(), N * 4, cudaMemcpyHostToDevice);
    }
    m->scale.push_back(ds);
    TcLayer& T = m->layer[l];
    T.K = K; T.N = N; T.n_real = L.cout; T.act = L.act; T.bias = db; T.scale = ds;
    T.slope = L.act == ACT_NONE ? 1.f : L.act == ACT_RELU ? 0.f : L.slope;      // act(v) = max(v, v * slope)
    // W[N][K] viewed as [K/64][N][64]: one box of {64 k, 64 rows, 4 k-blocks} lands in shared memory as four
    // consecutive 64 x 64 sub-tiles, each in the 128-byte-swizzled K-major layout the MMA descriptor expects
    const cuuint64_t dims[3] = {64, (cuuint64_t)N, (cuuint64_t)(K / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
    const cuuint32_t box[3] = {64, (cuuint32_t)kChunkN, (cuuint32_t)(kStageK / 64)};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(&m->maps[l], precision == PREC_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dw, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  }
  auto up = [&](const std::vector<float>& v) -> float* {
    if (v.empty()) return nullptr;
    float* d = nullptr;
    cudaMalloc(&d, v.size() * 4);
    cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
    return d;
  };
  m->in_div = up(M.in_div); m->out_mul = up(M.out_mul); m->relu_mask = up(M.relu_mask);
  if (cudaFuncSetAttribute(mlp_tc_fused_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(mlp_tc_fused_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(mlp_tc_fused_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
    return fail("cannot reserve " + std::to_string(kSmemBytes) + " bytes of shared memory for the tensor-core kernel");
  m->has_scale = precision == PREC_FP8W;
  m->f16 = precision == PREC_FP16;
  return m;
}

bool tc_forward(TcModel* m, const TcLaunch& L, cudaStream_t s, std::string* err) {
  const long long nrows = L.g.count * L.g.nk;
  if (nrows <= 0) return true;
  TcParams P;
  std::memset(&P, 0, sizeof P);
  for (int l = 0; l < m->nlayers; l++) { P.maps[l] = m->maps[l]; P.layer[l] = m->layer[l]; }
  P.nlayers = m->nlayers; P.n_in = m->n_in; P.n_out = m->n_out;
  P.in_div = m->in_div; P.out_mul = m->out_mul; P.relu_mask = m->relu_mask;
  P.GP = L.GP; P.slots = L.slots; P.TG = L.TG; P.X = L.X;
  P.SP = L.SP; P.stores = L.stores; P.TS = L.TS; P.Y = L.Y;
  P.slot_head = L.slot_head; P.store_next = L.store_next;
  P.g = L.g; P.nrows = nrows; P.partials = L.partials; P.status = L.status;
  P.fast_in = L.fast_in && m->n_in <= kFastIn; P.fast_out = L.fast_out && m->n_out <= kFastOut;
  for (int i = 0; i < 2; i++) {
    P.cin[i] = StrideClass{L.cin[i][0], L.cin[i][1], L.cin[i][2]};
    P.cout[i] = StrideClass{L.cout[i][0], L.cout[i][1], L.cout[i][2]};
  }
  P.store_by_slot = L.store_by_slot;
  if (!P.fast_in && !P.X) { if (err) *err = "tensor-core step: no input"; return false; }
  if (!P.fast_out && !P.Y) { if (err) *err = "tensor-core step: no output"; return false; }
  const int grid = tc_grid(nrows);
  static const bool want_prof = std::getenv("FORTIS_TC_PROF") != nullptr;
  static long long* dprof = nullptr;
  if (want_prof) {
    if (!dprof) cudaMalloc(&dprof, 32 * sizeof(long long));
    cudaMemsetAsync(dprof, 0, 32 * sizeof(long long), s);
    P.prof = dprof;
  }
  if (m->has_scale) mlp_tc_fused_kernel<true, false><<<grid, kThreads, kSmemBytes, s>>>(P);
  else if (m->f16) mlp_tc_fused_kernel<false, true><<<grid, kThreads, kSmemBytes, s>>>(P);
  else mlp_tc_fused_kernel<false, false><<<grid, kThreads, kSmemBytes, s>>>(P);
  if (want_prof) {
    long long h[32];
    cudaStreamSynchronize(s);
    cudaMemcpy(h, dprof, sizeof h, cudaMemcpyDeviceToHost);
    std::fprintf(stderr, "tc prof (cycles, CTA 0): mma issue %lld | wait a_ready %lld acc_empty %lld full %lld || rows: gather %lld | hidden wait %lld work %lld "
                 "transfer %lld | last wait %lld work %lld || tma wait-empty %lld issue %lld\n",
                 h[0], h[1], h[2], h[3], h[9], h[10], h[11], h[12], h[14], h[13], h[16], h[17]);
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { if (err) *err = std::string("tensor-core kernel launch: ") + cudaGetErrorString(e); return false; }
  return true;
}

}  // namespace fortis
