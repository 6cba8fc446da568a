// Fused gather -> MLP -> scatter on the 5th-generation tensor cores (tcgen05, sm_100a), bf16 operands, fp32
// accumulation in tensor memory, activations never leaving the SM between layers.
//
// Replaces, for wide column MLPs, the reference's per-layer lowering: fortis_gemm (cuBLAS SGEMM) + a separate
// bias/activation epilogue kernel per layer (runtime/fortis_rt.c:45-75, compiler/FortisFuse.cpp:616-624, 687-760),
// with fortis_gather_k in front and fortis_scatter_k behind (driver/fortis_gather_emit.py:52-62, 75-83).
//
// One persistent CTA per SM processes tiles of 128 columns (rows of the model batch); by default the CTAs run as
// clusters of two (cta_group::2) whose leader issues every MMA over both CTAs' tiles, each CTA streaming half of the
// weights (see the kernel's template parameter PAIR).  Per tile and layer
//     D[128 x N] = A[128 x K] . W[N x K]^T,  N processed in chunks of 64 output features.
//   * A (the layer's input activations, bf16) lives in TENSOR MEMORY: lane = row, two K values per 32-bit column
//     (K <= 768 -> 384 columns).  The MMAs take A from TMEM and B from shared memory, so shared-memory read
//     bandwidth is spent on the weights only.
//   * W streams from L2 through a ring of 32 KB TMA stages (64 features x 256 k, 128-byte swizzle, one 3-D tile
//     load per stage, no multicast).
//   * D: two 64-column fp32 accumulators in TMEM; the epilogue of chunk c overlaps the MMAs of chunk c+1.
//   * The epilogue (8 warps; thread = one row x 32 features) adds bias, applies the activation, rounds to bf16 and
//     parks the chunk: chunks 0-9 in shared memory, chunks 10-11 in registers (0-7 and 8-11 with one CTA per SM; A
//     is still being read by later chunks, so the output cannot overwrite it).  When the layer's last MMA has retired, the parked chunks are
//     written into the A columns with tcgen05.st and the next layer starts.
//   * Layer 0's A is produced by the same threads straight from the host's Fortran arrays, and the last layer's
//     epilogue stores straight into them and accumulates the fp64 checksum.  A tile of 128 whole rows along the
//     fastest loop index moves as bulk copies (one 512-byte run per model input / output through an fp32 staging area
//     in the park), any other tile element by element (thread = row, so every access is coalesced).  This fusion is
//     table-driven and covers fp32 arrays without lifted expressions; any other descriptor is served by the
//     standalone gather / scatter kernels writing X / reading Y around this kernel.
// TMEM: 384 (A) + 2 x 64 (D) = 512 columns.  Shared memory: 128 KB parked chunks + 3 x 32 KB weight ring (one CTA per
// SM), 160 KB parked chunks + 4 x 16 KB ring (CTA of a pair).
//
// Every wait on an mbarrier is bounded; a wait that gives up records a code in the status word, raises a CTA-wide
// abort flag that turns all later waits into no-ops, and the CTA still frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <type_traits>
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
constexpr int kBlockK = 256;                // K-block: granularity of the layer hand-off and of the padding of K
#ifndef FORTIS_TC_STAGE_K
#define FORTIS_TC_STAGE_K 256
#endif
constexpr int kStageK = FORTIS_TC_STAGE_K;  // k extent of one weight stage (256 or 128): 64-wide swizzled sub-tiles, ONE copy per stage
constexpr int kSubStages = kBlockK / kStageK;        // stages per K-block (16 KB stages, -DFORTIS_TC_STAGE_K=128, measured 3-4 % slower)
constexpr int kStageBytes = kChunkN * kStageK * 2;   // 32 KB
constexpr int kSubBytes = kChunkN * 64 * 2;          // one 64 x 64 sub-tile, 8 KB
// Two builds of the same kernel.  Shallow ring (default): 3 weight stages, 8 output chunks parked in shared memory and
// up to 4 in registers, 320 threads, 168 registers.  Deep ring (-DFORTIS_TC_DEEP_RING=1): 4 stages, 6 + 6 parked
// chunks, which needs the row warps' register budget raised (setmaxnreg; 384 threads so that the producer warps form a
// warpgroup of their own) and, because a function call stops the compiler from allocating per budget, the barrier waits
// inlined.  Measured: the inlined waits cost 10 % by themselves (whatever the polling loop looks like), more than
// the fourth stage returns, so the deep ring is not the default.
// Weight stages as linear bulk copies of pre-tiled stage images (1, default) or as 3-D tensor copies of the row-major
// weights (0).
#ifndef FORTIS_TC_TILED_W
#define FORTIS_TC_TILED_W 1
#endif
#ifndef FORTIS_TC_GATHER64
#define FORTIS_TC_GATHER64 1
#endif
#ifndef FORTIS_TC_DEEP_RING
#define FORTIS_TC_DEEP_RING 0
#endif
constexpr bool kRegRealloc = FORTIS_TC_DEEP_RING != 0;
#ifdef FORTIS_TC_INLINE_WAIT
constexpr bool kInlineWait = true;
#else
constexpr bool kInlineWait = false;
#endif
constexpr int kStages = (kRegRealloc ? 4 : 3) * kSubStages;
constexpr int kSmemChunks = kRegRealloc ? 6 : 8;   // parked chunks held in shared memory; the rest in registers
constexpr int kRegsProducer = 40, kRegsRow = 232;  // 168 at launch; 2 x 128 x 232 + 128 x 40 = 64 K registers
constexpr int kMaxKBlocks = 3;                     // 768 / 256: K-blocks of a layer's A, each with its own hand-off barriers
constexpr int kMaxChunks = 12;              // 768 / 64
constexpr int kMaxK = 768;
constexpr int kMaxLayers = 8;
constexpr int kEpiThreads = 256;
constexpr int kIssuers = 2;                 // MMA-issuing warps: issuer w owns accumulator w and every chunk that lands in it
constexpr int kThreads = kEpiThreads + (kRegRealloc ? 128 : 96);   // + TMA warp + two MMA warps (+ an idle warp: register re-allocation works per warpgroup)
constexpr int kParkBytes = kSmemChunks * kTileM * kChunkN * 2;      // 128 KB
constexpr int kRingBytes = kStages * kStageBytes;                   // 96 KB
#ifndef FORTIS_TC_PAIR_PARK
#define FORTIS_TC_PAIR_PARK 10
#endif
constexpr int kPairParkChunks = FORTIS_TC_PAIR_PARK;                // two-CTA form: parked chunks in shared memory (8 or 10) ...
constexpr int kPairStages = (kParkBytes + kRingBytes) / (kStageBytes / 2) - kPairParkChunks;   // ... and the 16 KB stages that fit beside them (6 or 4)
static_assert(kPairStages >= 3 && kPairStages <= 6 && kPairParkChunks <= 12, "two-CTA form: ring depth");
constexpr int kBarBytes = 384;             // barriers in the first 256 bytes, then the tensor-memory base, the abort flag and the checksum scratch
constexpr int kFastIn = 256, kFastOut = 128;          // widest model input / output the fast I/O tables hold
constexpr int kTabBytes = kFastIn * 5 + kFastOut * 5 + 2 * kMaxArrays * 8;   // uint32 offset + uint8 code per slot / store, array bases
constexpr int kSmemBytes = kParkBytes + kRingBytes + kBarBytes + kTabBytes;   // the base must be 1024-byte aligned
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCol0 = 384;

// status codes (which wait gave up)
enum { ST_OK = 0, ST_FULL = 1, ST_EMPTY = 2, ST_ACC_FULL = 3, ST_ACC_EMPTY = 4, ST_A_READY = 5, ST_SMEM_ALIGN = 6, ST_A_DEAD = 7, ST_IN = 8 };

struct TcLayer {
  int K, N;                // padded: K multiple of 256, N multiple of 64 (hidden: multiple of 256)
  int n_real;              // unpadded output width
  int act;
  float slope;             // branch-free activation: act(v) = max(v, v * slope); none -> 1, ReLU -> 0, LeakyReLU -> slope
  const float* bias;       // [N] padded with zeros
  const float* scale;      // [N] per-output-channel dequantisation scale (fp8 weights) or null
  const uint8_t* wtiled;   // the weights as consecutive 32 KB stage images, [chunk of 64 features][256-wide K-block]
  const uint8_t* wdev;     // whichever form of the 16-bit weights the kernel streams (N x K x 2 bytes), for the L2 prefetch
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
  double* sum;                           // with partials: the last CTA to finish folds them into *sum (accumulating), in index order
  unsigned int* done;                    // CTA completion counter for that fold (zero between launches)
  int* status;
  unsigned int wait_limit;               // polls before a barrier wait gives up
  int test_skip_stage;                   // test only: CTA 0 never loads its first weight stage
  int no_l2_prefetch;                    // FORTIS_TC_NO_L2_PREFETCH: do not ask for the weights to be brought into L2 at kernel start
  int no_stage_inputs;                   // FORTIS_TC_NO_STAGE_INPUTS: fetch the next tile's inputs element by element
  int no_stage_outputs;                  // FORTIS_TC_NO_STAGE_OUTPUTS: store a tile's outputs element by element
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
template <bool F16, bool PAIR = false> struct MlpIdesc {
  static constexpr uint32_t value = (1u << 4) | (F16 ? 0u : ((1u << 7) | (1u << 10))) | ((uint32_t)(kChunkN >> 3) << 17) |
                                    ((uint32_t)((PAIR ? 2 * kTileM : kTileM) >> 4) << 24);
};
// two consecutive k values as one 32-bit tensor-memory column, in the kernel's 16-bit operand format
template <bool F16> __device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (F16) { const __half2 v = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t*>(&v); }
  else return pack_bf16(lo, hi);
}

__device__ __forceinline__ float act_f(float v, float slope) { return fmaxf(v, v * slope); }


// A model input is read once per step: keep it out of L1, which is small beside 224 KB of shared memory and has to hold
// the bias and scale vectors every chunk epilogue reads (measured in one call against the plain load: 0.2253 -> 0.2232 ms
// on the 49,152-column configuration).
__device__ __forceinline__ float ldg_stream(const float* p) {
  float v;
  asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// Cycle accounting of the three roles (CTA 0, one lane each), compiled in with -DFORTIS_TC_PROF only: PROF_ADD(slot) adds
// the time since the previous call to prof[slot].
#ifdef FORTIS_TC_PROF
#define PROF_DECL(who) const bool prof_who = P.prof && (who); long long prof_t = clock64()
#define PROF_ADD(slot) do { if (prof_who) { const long long n_ = clock64(); atomicAdd((unsigned long long*)&P.prof[slot], (unsigned long long)(n_ - prof_t)); prof_t = n_; } } while (0)
// the same, also broken down by layer: prof[32 + 8 * slot + layer] for slots 0 .. 3 (the issuer's)
#define PROF_ADDL(slot, l) do { if (prof_who) { const long long n_ = clock64(); atomicAdd((unsigned long long*)&P.prof[slot], (unsigned long long)(n_ - prof_t)); \
    atomicAdd((unsigned long long*)&P.prof[32 + 8 * (slot) + (l)], (unsigned long long)(n_ - prof_t)); prof_t = n_; } } while (0)
#else
#define PROF_ADDL(slot, l) do { } while (0)
#define PROF_DECL(who) do { } while (0)
#define PROF_ADD(slot) do { } while (0)
#endif

// the kernel's bounded barrier wait: inlined where warpgroups get different register budgets (a call would stop that)
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code, uint32_t limit) {
  if constexpr (kRegRealloc || kInlineWait) return mbar_wait_inline(bar, parity, abort_flag, status, code);
  else return mbar_wait(bar, parity, abort_flag, status, code, limit);
}

// ---------------------------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------------------------
//
// PAIR: the same kernel as clusters of two CTAs (cta_group::2).  Each CTA owns a 128-row tile with its own A, accumulators,
// epilogue and parked chunks; the leader (cluster rank 0) issues every MMA over both CTAs' rows (M = 256), and a chunk's
// 64 weight rows come half from each CTA's shared memory, so each SM streams HALF of the weights (16 KB stages, six of
// them).  Copies are plain tensor copies whose completion is counted on the leader's barriers; the leader's commits
// arrive on the barriers of both CTAs; the row warps of both CTAs hand accumulators and A blocks back on the leader's
// barriers, one arrival per warp.
template <bool HAS_SCALE, bool F16, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1) mlp_tc_fused_kernel(const __grid_constant__ TcParams P) {
  constexpr uint32_t kIdesc = MlpIdesc<F16, PAIR>::value;
  // Ring and park: one CTA per SM keeps 3 stages of 32 KB and parks 8 output chunks in shared memory (4 in registers).
  // A CTA of a pair streams half the bytes, so 4 stages of 16 KB cover the same time; the 32 KB saved park two more
  // chunks in shared memory (2 in registers), which takes the epilogue out of register spilling.
  constexpr int kStg = PAIR ? kPairStages : kStages;                 // ring depth in stages
  constexpr int kPark = PAIR ? kPairParkChunks : kSmemChunks;        // parked chunks held in shared memory; the rest in registers
  constexpr int kParkB = kPark * kTileM * kChunkN * 2, kRingB = kStg * (PAIR ? kStageBytes / 2 : kStageBytes);
  static_assert(kParkB + kRingB <= kParkBytes + kRingBytes, "the pair form must fit the same shared memory");
  constexpr int kStgBytes = PAIR ? kStageBytes / 2 : kStageBytes;    // this CTA's part of a stage
  constexpr int kSubB = PAIR ? kSubBytes / 2 : kSubBytes;            // one 64-wide k sub-tile of it
  constexpr int kRowArrivals = PAIR ? 16 : kEpiThreads;              // arrivals that hand an accumulator / an A block back
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = smem_u32(smem);                         // parked chunks: kPark x 16 KB at offset 0
  if (base & 1023u) {                                           // the swizzled weight stages need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(P.status, 0, ST_SMEM_ALIGN);
    return;
  }
  const uint32_t ring = base + kParkB;                      // kStages x 32 KB
  const uint32_t bars = ring + kRingB;
  // barrier block: full [kIssuers][kStages] | empty [kStages] | acc_full [2] | acc_empty [2] | a_ready [3] | a_dead [2]
  // within the first 256 bytes; tmem base 256, abort flag 260, checksum scratch [272,336).
  // Every stage has one "full" barrier PER ISSUER: a parity wait can only tell a barrier's current phase from the
  // previous one, so each barrier needs a single waiter that sees every one of its phases; the TMA warp arms the
  // barrier of the issuer that will consume the stage.
  static_assert(8 * ((kIssuers + 1) * kStg + 9) <= 256, "the barriers must fit the first 256 bytes of the barrier block");
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kIssuers * kStg;
  const uint32_t bar_acc_full = bar_empty + 8 * kStg, bar_acc_empty = bar_acc_full + 16;
  const uint32_t bar_a_ready = bar_acc_empty + 16, bar_a_dead = bar_a_ready + 24;
  const uint32_t bar_park = bars + 240;                           // every row thread has read its parked chunks 0-7 of the last hidden layer
  const uint32_t bar_in = bars + 248;                             // the staged inputs of the next tile have landed (one phase per staged tile)
  uint32_t* tmem_slot = (uint32_t*)(smem + kParkB + kRingB + 256);
  volatile int* abort_flag = (volatile int*)(smem + kParkB + kRingB + 260);
  uint32_t* s_off = (uint32_t*)(smem + kParkB + kRingB + kBarBytes);          // [kFastIn] input slot offsets
  uint32_t* o_off = s_off + kFastIn;                                                  // [kFastOut] store offsets
  uint8_t* s_code = (uint8_t*)(o_off + kFastOut);                                     // array | class << 7, 0xFF: none
  uint8_t* o_code = s_code + kFastIn;
  // array base pointers of the fast paths, copied out of the kernel parameters so that the unrolled load / store
  // loops index shared memory (indexing the parameter block dynamically makes nvcc's front end crawl)
  const float** s_base_in = (const float**)(o_code + kFastOut);
  float** s_base_out = (float**)(s_base_in + kMaxArrays);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long ntiles = (P.nrows + kTileM - 1) / kTileM;
  // work units: tiles, or (PAIR) pairs of tiles 2 u and 2 u + 1, one per CTA of the cluster
  uint32_t crank = 0;
  if constexpr (PAIR) crank = cluster_ctarank();
  const long long nunits = PAIR ? (ntiles + 1) / 2 : ntiles;
  const long long unit0 = PAIR ? (long long)(blockIdx.x >> 1) : (long long)blockIdx.x;
  const long long ustep = PAIR ? (long long)(gridDim.x >> 1) : (long long)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kIssuers * kStg; s++) mbar_init(bar_full + 8 * s, 1);
    for (int s = 0; s < kStg; s++) mbar_init(bar_empty + 8 * s, 1);
    for (int b = 0; b < 2; b++) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, kRowArrivals); }
    for (int k = 0; k < kMaxKBlocks; k++) mbar_init(bar_a_ready + 8 * k, kRowArrivals);
    for (int k = 0; k < kMaxKBlocks - 1; k++) mbar_init(bar_a_dead + 8 * k, kIssuers);
    mbar_init(bar_in, kEpiThreads);
    mbar_init(bar_park, kEpiThreads);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < kMaxArrays) {
    s_base_in[threadIdx.x] = (const float*)P.TG.base[threadIdx.x];
    s_base_out[threadIdx.x] = (float*)P.TS.base[threadIdx.x];
  }
  // can a tile's inputs be staged by 16-byte asynchronous copies?  Every slot must run along the fastest loop index with
  // unit stride and start 16-byte aligned wherever a tile starts on a multiple of four of that index.
  int stage_bad = 0;
  if (P.fast_in)
    for (int q = threadIdx.x; q < kFastIn; q += kThreads) {
      uint8_t code = 0xFF; uint32_t off = 0;
      if (q < P.n_in) {
        const Access a = P.slots[q];
        code = (uint8_t)(a.array | ((a.si == P.cin[0].si && a.sj == P.cin[0].sj && a.sk == P.cin[0].sk) ? 0 : 0x80));
        off = (uint32_t)a.off0;
        const unsigned long long b0 = reinterpret_cast<unsigned long long>(P.TG.base[a.array]) + 4ull * (unsigned long long)a.off0;
        if (a.si != 1 || (a.sj & 3) || (a.sk & 3) || (b0 & 15ull)) stage_bad = 1;
      }
      s_code[q] = code; s_off[q] = off;
    }
  int stage_out_bad = 0;                      // the same question for the stores of a tile's outputs
  if (P.fast_out)
    for (int n = threadIdx.x; n < kFastOut; n += kThreads) {
      uint8_t code = 0xFF; uint32_t off = 0;
      if (n < P.n_out && P.store_by_slot[n].array >= 0) {
        const Access a = P.store_by_slot[n];
        code = (uint8_t)(a.array | ((a.si == P.cout[0].si && a.sj == P.cout[0].sj && a.sk == P.cout[0].sk) ? 0 : 0x80));
        off = (uint32_t)a.off0;
        const unsigned long long b0 = reinterpret_cast<unsigned long long>(P.TS.base[a.array]) + 4ull * (unsigned long long)a.off0;
        if (a.si != 1 || (a.sj & 3) || (a.sk & 3) || (b0 & 15ull)) stage_out_bad = 1;
      }
      o_code[n] = code; o_off[n] = off;
    }
  if (warp == 8 && lane < P.nlayers)
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&P.maps[lane])) : "memory");
  if (warp == 9) {
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  const int any_stage_bad = __syncthreads_or(stage_bad);                    // also the CTA's setup barrier
  const bool can_stage = P.fast_in && !P.no_stage_inputs && any_stage_bad == 0;
  const bool can_stage_out = (__syncthreads_or(stage_out_bad) == 0) && P.fast_out && !P.no_stage_outputs && !P.Y;
  if constexpr (PAIR) cluster_sync_all();      // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp >= 8) {
    // Register re-allocation between warpgroups (deep-ring build): the producer warpgroup (TMA warp, MMA warp, two idle
    // warps) keeps kRegsProducer registers per thread and hands the rest to the two row warpgroups, whose threads park
    // six output chunks (96 registers) next to the epilogue's working set.
    if constexpr (kRegRealloc) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsProducer));
    if (warp == 9 + kIssuers - 1 && !P.no_l2_prefetch) {
      // A step usually starts with the weights out of L2 (the host's arrays have streamed through it since the last
      // step), and every CTA then asks for the same stage at the same moment, one memory latency per stage.  Each CTA
      // asks for its 1/gridDim slice of every layer's weights to be brought into L2 now, while the first inputs are
      // gathered.
      for (int l = 0; l < P.nlayers; l++) {
        const unsigned long long bytes = (unsigned long long)P.layer[l].N * P.layer[l].K * 2;
        const unsigned long long per = ((bytes + gridDim.x - 1) / gridDim.x + 127ull) & ~127ull;
        const unsigned long long off = per * blockIdx.x;
        if (off < bytes) l2_prefetch(P.layer[l].wdev + off, (uint32_t)(bytes - off < per ? bytes - off : per));
      }
    }
    if (warp == 8) {
      // ---------------------------------------------------------------- TMA producer (whole warp, one lane issues)
      uint32_t s = 0, ph = 0, acc_it = 0;
      PROF_DECL(blockIdx.x == 0 && lane == 0);
      bool stop = false;
      uint32_t full_leader = bar_full;           // PAIR: the leader's barriers collect both CTAs' copies
      if constexpr (PAIR) full_leader = map_to_cta(bar_full, 0);
      for (long long u = unit0; u < nunits && !stop; u += ustep)
        for (int l = 0; l < P.nlayers && !stop; l++) {
          const int nchunks = P.layer[l].N / kChunkN, nkb = P.layer[l].K / kBlockK;
          const CUtensorMap* map = &P.maps[l];
          const uint8_t* wtiled = P.layer[l].wtiled;
          (void)map; (void)wtiled;
          for (int c = 0; c < nchunks && !stop; c++, acc_it++) {
            const uint32_t full_off = 8 * kStg * (acc_it & 1);      // the barriers of the issuer that owns this chunk
            for (int ks = 0; ks < nkb * kSubStages; ks++) {
              PROF_ADD(17);
              if (!wait_bar(bar_empty + 8 * s, ph ^ 1, abort_flag, P.status, ST_EMPTY, P.wait_limit)) { stop = true; break; }
              PROF_ADD(16);
              const bool skip = P.test_skip_stage && blockIdx.x == 0 && u == unit0 && l == 0 && c == 0 && ks == 0;   // test only
              if constexpr (PAIR) {
                // the leader arms its barrier for both halves; each CTA copies its 32 of the chunk's 64 weight rows
                if (crank == 0) mbar_expect_tx(bar_full + full_off + 8 * s, 2 * kStgBytes);
                if (!skip)
                  tma_load_3d_pair(ring + s * kStgBytes, map, 0, c * kChunkN + (int)crank * (kChunkN / 2), ks * (kStageK / 64),
                                   full_leader + full_off + 8 * s);
              } else if (!skip) {
                mbar_expect_tx(bar_full + full_off + 8 * s, kStageBytes);
#if FORTIS_TC_TILED_W
                bulk_load(ring + s * kStageBytes, wtiled + (size_t)(c * (nkb * kSubStages) + ks) * kStageBytes, kStageBytes, bar_full + full_off + 8 * s);
#else
                tma_load_3d(ring + s * kStageBytes, map, 0, c * kChunkN, ks * (kStageK / 64), bar_full + full_off + 8 * s);
#endif
              }
              if (++s == kStg) { s = 0; ph ^= 1; }
            }
          }
        }
    } else if (warp < 9 + kIssuers && crank == 0) {
      // ---------------------------------------------------------------- MMA issuers (whole warps, one lane issues; PAIR: the leader's only)
      // Two warps issue: a 128 x 64 x 16 MMA keeps the tensor pipe busy for 32 cycles, less than one warp needs to wait
      // for a stage, issue sixteen MMAs and commit.  Chunks alternate between the two accumulators, so issuer w simply
      // owns accumulator w and all chunks that land in it; the pipe sees one in-order stream.  Both walk the same
      // chunk / stage sequence and skip what is not theirs.
      const uint32_t me = (uint32_t)(warp - 9);
      const uint32_t my_full = bar_full + 8 * kStg * me;
      uint32_t s = 0, full_par = 0, acc_it = 0, lay_it = 0;     // full_par: bit s = parity of this issuer's next phase of stage s
      const uint64_t desc_hi = make_b_desc(0) & 0xFFFFFFFF00000000ull;
      PROF_DECL(blockIdx.x == 0 && lane == 0 && me == 0);
      // commits arrive on this CTA's barrier or (PAIR) on the barrier at the same offset in both CTAs
      auto commit = [&](uint32_t bar) { if constexpr (PAIR) tc_commit_pair(bar); else tc_commit(bar); };
      for (long long u = unit0; u < nunits; u += ustep)
        for (int l = 0; l < P.nlayers; l++, lay_it++) {
          const int nchunks = P.layer[l].N / kChunkN, nkb = P.layer[l].K / kBlockK;
          const uint32_t lph = lay_it & 1;
          bool first = true, any = false;
          for (int c = 0; c < nchunks; c++, acc_it++) {
            const uint32_t b = acc_it & 1, aph = (acc_it >> 1) & 1;
            if (b != me) {                                    // the other issuer's chunk: step over its stages
              s = (s + (uint32_t)(nkb * kSubStages)) % kStg;
              continue;
            }
            any = true;
            // this issuer's last chunk of the layer: no later chunk lands in accumulator `me`
            const bool mine_last = c + kIssuers >= nchunks;
            PROF_ADDL(0, l);
            wait_bar(bar_acc_empty + 8 * b, aph ^ 1, abort_flag, P.status, ST_ACC_EMPTY, P.wait_limit);
            PROF_ADDL(2, l);
            tc_fence_after();
            const uint32_t d_tmem = tmem + kAccCol0 + b * kChunkN;
            for (int kb = 0; kb < nkb; kb++) {
              if (first) {                                    // K-block kb of this layer's A is in tensor memory
                PROF_ADDL(0, l);
                wait_bar(bar_a_ready + 8 * kb, lph, abort_flag, P.status, ST_A_READY, P.wait_limit);
                PROF_ADDL(1, l);
              }
#pragma unroll
              for (int sub = 0; sub < kSubStages; sub++) {
                PROF_ADDL(0, l);
                wait_bar(my_full + 8 * s, (full_par >> s) & 1u, abort_flag, P.status, ST_FULL, P.wait_limit);
                full_par ^= 1u << s;
                PROF_ADDL(3, l);
                tc_fence_after();
                // descriptor of the stage's first 64-wide k sub-tile; the next sub-tile starts kSubBytes further, and
                // stepping k by 16 inside a 128-byte swizzle row adds 32 bytes (the address field is in 16-byte units)
                const uint32_t sb = ring + s * kStgBytes;
                const uint64_t bd0 = desc_hi | (uint64_t)((sb >> 4) & 0x3FFF);
                const uint32_t a0 = tmem + kb * (kBlockK / 2) + sub * (kStageK / 2);
                if constexpr (PAIR) {
                  tc_mma_ts_first_pair<kIdesc>(d_tmem, a0, bd0, (uint32_t)(kb | sub));
#pragma unroll
                  for (int j = 1; j < kStageK / 16; j++)
                    tc_mma_ts_acc_pair<kIdesc>(d_tmem, a0 + j * 8, bd0 + (uint64_t)((j >> 2) * (kSubB >> 4) + (j & 3) * 2));
                } else {
                  tc_mma_ts_first<kIdesc>(d_tmem, a0, bd0, (uint32_t)(kb | sub));
#pragma unroll
                  for (int j = 1; j < kStageK / 16; j++)
                    tc_mma_ts_acc<kIdesc>(d_tmem, a0 + j * 8, bd0 + (uint64_t)((j >> 2) * (kSubBytes >> 4) + (j & 3) * 2));
                }
                commit(bar_empty + 8 * s);                    // stage reusable once these MMAs have read it
                if (++s == kStg) s = 0;
              }
              if (mine_last) {
                // this issuer's last MMAs on K-block kb in this layer: once both issuers' have retired, those columns
                // of A may be overwritten with the next layer's input.  Blocks the layer does not have are signalled
                // with the last one, which keeps every barrier at one phase per layer.
                // (a one-chunk layer has one working issuer, which then signals for both)
                for (int rep = 0; rep < (nchunks < kIssuers ? kIssuers : 1); rep++) {
                  if (kb < kMaxKBlocks - 1) commit(bar_a_dead + 8 * kb);
                  if (kb == nkb - 1)
                    for (int k2 = kb + 1; k2 < kMaxKBlocks - 1; k2++) commit(bar_a_dead + 8 * k2);
                }
              }
            }
            first = false;
            commit(bar_acc_full + 8 * b);                     // accumulator complete
          }
          if (!any)                                           // a one-chunk layer: the idle issuer still sees the layer's phases complete
            for (int kb = 0; kb < nkb; kb++) wait_bar(bar_a_ready + 8 * kb, lph, abort_flag, P.status, ST_A_READY, P.wait_limit);
        }
    }
  } else {
    if constexpr (kRegRealloc) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsRow));
    // ------------------------------------------------------------------ row warps: gather, epilogues, scatter
    const int quad = warp & 3, half = warp >> 2;              // TMEM lane quadrant, which 32 of a chunk's 64 features
    const int r = quad * 32 + lane;                           // row of the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    uint32_t acc_it = 0, lay_it = 0;
    double csum = 0.0;
    PROF_DECL(blockIdx.x == 0 && threadIdx.x == 0);
    const int per0 = P.layer[0].K / 2;                        // model inputs per half row (padded)
    const bool can_prefetch = P.layer[0].K == kBlockK;        // one K-block of inputs: 64 packed registers per thread
    // Hands an accumulator or a block of A back to the issuers.  One CTA: every row thread arrives on the CTA's barrier.
    // PAIR: the issuers are the leader's, so the arrival goes to the leader's barrier, one per warp; it publishes no
    // generic-memory writes (the thread has completed its tensor-memory accesses: tcgen05.wait + fence), so it is relaxed.
    auto signal = [&](uint32_t bar) {
      if constexpr (PAIR) {
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(map_to_cta(bar, 0));
      } else {
        mbar_arrive(bar);
      }
    };

    // position of row `row_` in the host arrays, once per stride class of the gather
    auto locate_in = [&](long long row_, bool& live_, long long& p0, long long& p1) {
      live_ = row_ < P.nrows;
      long long ci = 0, cj = 0, kk = 0;
      if (live_) row_to_pos(P.g, row_, &ci, &cj, &kk);
      p0 = ci * P.cin[0].si + cj * P.cin[0].sj + kk * P.cin[0].sk;
      p1 = ci * P.cin[1].si + cj * P.cin[1].sj + kk * P.cin[1].sk;
    };
    // model inputs q0 .. q0 + 31 of one row as 16 packed 16-bit pairs: 32 independent loads, each coalesced across the
    // warp (thread = row).  Either straight from the host arrays through the per-CTA slot table, or from a
    // materialised X (array-form calls, and descriptors the table cannot express: lifted expressions, f64 arrays,
    // scalars, for which the standalone gather kernel ran first).
    auto gather_group = [&](long long row_, bool live_, long long p0, long long p1, int q0, uint32_t (&pk)[16]) {
      float v[32];
      if (P.fast_in) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
          const uint32_t code = s_code[q0 + j];
          v[j] = 0.f;
          if (live_ && code != 0xFF)
            v[j] = ldg_stream(s_base_in[code & 0x7F] + ((long long)s_off[q0 + j] + ((code & 0x80) ? p1 : p0)));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = (live_ && q0 + j < P.n_in) ? ldg_stream(P.X + row_ * P.n_in + q0 + j) : 0.f;
      }
      if (P.in_div) {
#pragma unroll
        for (int j = 0; j < 32; j++) if (q0 + j < P.n_in) v[j] = __fdiv_rn(v[j], __ldg(P.in_div + q0 + j));
      }
#pragma unroll
      for (int j = 0; j < 16; j++) pk[j] = pack16<F16>(v[2 * j], v[2 * j + 1]);
    };
    // the same for inputs q0 .. q0 + 63 with all 64 loads issued before the first is used
    auto gather_two_groups = [&](long long row_, bool live_, long long p0, long long p1, int q0, uint32_t (&pka)[16], uint32_t (&pkb)[16]) {
      float v[64];
      if (P.fast_in) {
#pragma unroll
        for (int j = 0; j < 64; j++) {
          const uint32_t code = s_code[q0 + j];
          v[j] = 0.f;
          if (live_ && code != 0xFF)
            v[j] = ldg_stream(s_base_in[code & 0x7F] + ((long long)s_off[q0 + j] + ((code & 0x80) ? p1 : p0)));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 64; j++) v[j] = (live_ && q0 + j < P.n_in) ? ldg_stream(P.X + row_ * P.n_in + q0 + j) : 0.f;
      }
      if (P.in_div) {
#pragma unroll
        for (int j = 0; j < 64; j++) if (q0 + j < P.n_in) v[j] = __fdiv_rn(v[j], __ldg(P.in_div + q0 + j));
      }
#pragma unroll
      for (int j = 0; j < 16; j++) { pka[j] = pack16<F16>(v[2 * j], v[2 * j + 1]); pkb[j] = pack16<F16>(v[32 + 2 * j], v[33 + 2 * j]); }
    };
    // layer 0's A is complete: release all K-block barriers (blocks the layer does not have stay in step)
    auto release_layer0 = [&]() {
      tmem_st_wait();
      tc_fence_before();
      // block 0 last: a waiter that has seen block 0's phase complete has thereby seen the others'
#pragma unroll
      for (int k = kMaxKBlocks - 1; k >= 0; k--) signal(bar_a_ready + 8 * k);
    };

    uint32_t in_ph = 0, park_ph = 0;                          // parities of the next phases of bar_in and bar_park
    // Staged fetch of a tile's inputs.  A tile qualifies when it is 128 whole rows that run along the fastest loop index
    // (and the per-CTA conditions of can_stage hold): every model input is then one aligned 512-byte run.
    auto stage_issue = [&](long long first) -> bool {
      if (first + kTileM > P.nrows) return false;
      long long ci, cj, kk, ci2, cj2, kk2;
      row_to_pos(P.g, first, &ci, &cj, &kk);
      row_to_pos(P.g, first + kTileM - 1, &ci2, &cj2, &kk2);
      if (cj2 != cj || kk2 != kk || ci2 - ci != kTileM - 1 || (ci & 3) != 0) return false;
      const long long pf0 = ci + cj * P.cin[0].sj + kk * P.cin[0].sk, pf1 = ci + cj * P.cin[1].sj + kk * P.cin[1].sk;
      // thread q (0 .. 255: the row warps) copies input q's run into fp32 [input][row]; all of them arrive on the barrier
      const int q = (int)threadIdx.x;
      const uint32_t code = s_code[q];
      if (code != 0xFF) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the copy writes what generic reads have just left
        mbar_arrive_expect_tx_thread(bar_in, kTileM * 4);
        bulk_load_thread(base + (uint32_t)(q * (kTileM * 4)),
                         s_base_in[code & 0x7F] + ((long long)s_off[q] + ((code & 0x80) ? pf1 : pf0)), kTileM * 4, bar_in);
      } else {
        mbar_arrive(bar_in);
      }
      return true;
    };
    // the staged inputs, converted, into the A columns of K-block 0 (one K-block of inputs: can_prefetch)
    auto stage_consume = [&]() {
      wait_bar(bar_in, in_ph, abort_flag, P.status, ST_IN, P.wait_limit);   // every thread's copy has landed
      in_ph ^= 1;
#pragma unroll 1
      for (int g = 0; g < 4; g++) {
        uint32_t pk[16];
        const int q0 = half * per0 + 32 * g;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; j++)
          v[j] = s_code[q0 + j] != 0xFF ? *reinterpret_cast<const float*>(smem + (q0 + j) * (kTileM * 4) + r * 4) : 0.f;
        if (P.in_div) {
#pragma unroll
          for (int j = 0; j < 32; j++) if (q0 + j < P.n_in) v[j] = __fdiv_rn(v[j], __ldg(P.in_div + q0 + j));
        }
#pragma unroll
        for (int j = 0; j < 16; j++) pk[j] = pack16<F16>(v[2 * j], v[2 * j + 1]);
        tmem_st16(lane_addr + (uint32_t)(q0 >> 1), pk);
      }
      asm volatile("bar.sync 1, %0;" ::"r"(kEpiThreads) : "memory");       // all have read the staging area: it may be parked into again
    };
    // Staged stores of a tile's outputs: fp32 [output][row] in the last 64 KB of the park area, then one bulk store per
    // model output.  The area is parked into again from chunk kOutSlot of the next tile's hidden layers on, and the
    // next tile's staged inputs reach into it: before either, the stores must have read it.
    constexpr int kOutSlot = kPark - 4;
    constexpr uint32_t kOutStage = (uint32_t)kOutSlot * (kTileM * kChunkN * 2);
    bool out_pending = false;
    auto out_stage_drain = [&]() {
      if (out_pending) {
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync 1, %0;" ::"r"(kEpiThreads) : "memory");
        out_pending = false;
      }
    };
    bool prefetched = false;
    for (long long u = unit0; u < nunits; u += ustep) {
      const long long tile = PAIR ? 2 * u + crank : u;
      const long long row = tile * kTileM + r;
      const bool live = row < P.nrows;
      if (!prefetched) {
        // ---- layer 0 input straight into A: the CTA's first tile, or inputs wider than one K-block.  The previous
        //      tile's MMAs have all retired (its last accumulator was read), so A may be overwritten.
        bool lv; long long p0, p1;
        locate_in(row, lv, p0, p1);
        if (can_stage && can_prefetch && stage_issue(tile * kTileM)) stage_consume();      // (the park area is not in use)
        else
#if FORTIS_TC_GATHER64
        for (int q0 = half * per0; q0 < (half + 1) * per0; q0 += 64) {     // K is a multiple of 256, so per0 of 128
          uint32_t pka[16], pkb[16];
          gather_two_groups(row, lv, p0, p1, q0, pka, pkb);
          tmem_st16(lane_addr + (uint32_t)(q0 >> 1), pka);
          tmem_st16(lane_addr + (uint32_t)((q0 >> 1) + 16), pkb);
        }
#else
        for (int q0 = half * per0; q0 < (half + 1) * per0; q0 += 32) {
          uint32_t pk[16];
          gather_group(row, lv, p0, p1, q0, pk);
          tmem_st16(lane_addr + (uint32_t)(q0 >> 1), pk);
        }
#endif
        release_layer0();
        PROF_ADD(9);
      }
      prefetched = false;
      for (int l = 0; l < P.nlayers; l++, lay_it++) {
        const TcLayer& L = P.layer[l];
        const int nchunks = L.N / kChunkN, nkb = L.K / kBlockK;
        const bool last = l == P.nlayers - 1;
        const float slope = L.slope;
        const uint32_t lph = lay_it & 1;
        if (!last) {
          uint32_t kept[(kMaxChunks - kPark) * 16];     // this thread's parked chunks beyond those in shared memory (16-bit pairs)
          // epilogue of one chunk: accumulator -> (x scale) + bias -> activation -> 16 packed 16-bit pairs
          auto chunk_epilogue = [&](int c, uint32_t (&pk)[16]) {
            const uint32_t b = acc_it & 1, aph = (acc_it >> 1) & 1;
            acc_it++;
            const int n0 = c * kChunkN + half * 32;
            // the 32 biases of this thread's features: warp-uniform 16-byte loads issued before the wait
            float4 bq[8];
#pragma unroll
            for (int j = 0; j < 8; j++) bq[j] = __ldg(reinterpret_cast<const float4*>(L.bias + n0) + j);
            PROF_ADD(11);
            wait_bar(bar_acc_full + 8 * b, aph, abort_flag, P.status, ST_ACC_FULL, P.wait_limit);
            PROF_ADD(10);
            tc_fence_after();
            uint32_t a[32];
            tmem_ld32(lane_addr + kAccCol0 + b * kChunkN + half * 32, a);
            tmem_ld_wait();
            tc_fence_before();
            signal(bar_acc_empty + 8 * b);                    // the MMA warp may refill this accumulator
#pragma unroll
            for (int j = 0; j < 8; j++) {
              // FP8 weights: acc * scale + bias as one fused multiply-add (the last layer's epilogue does the same)
              float4 sq = make_float4(1.f, 1.f, 1.f, 1.f);
              if (HAS_SCALE) sq = __ldg(reinterpret_cast<const float4*>(L.scale + n0) + j);
              const float v0 = act_f(HAS_SCALE ? fmaf(__uint_as_float(a[4 * j]), sq.x, bq[j].x) : __uint_as_float(a[4 * j]) + bq[j].x, slope);
              const float v1 = act_f(HAS_SCALE ? fmaf(__uint_as_float(a[4 * j + 1]), sq.y, bq[j].y) : __uint_as_float(a[4 * j + 1]) + bq[j].y, slope);
              const float v2 = act_f(HAS_SCALE ? fmaf(__uint_as_float(a[4 * j + 2]), sq.z, bq[j].z) : __uint_as_float(a[4 * j + 2]) + bq[j].z, slope);
              const float v3 = act_f(HAS_SCALE ? fmaf(__uint_as_float(a[4 * j + 3]), sq.w, bq[j].w) : __uint_as_float(a[4 * j + 3]) + bq[j].w, slope);
              pk[2 * j] = pack16<F16>(v0, v1);
              pk[2 * j + 1] = pack16<F16>(v2, v3);
            }
          };
          // shared-memory park: [chunk][half][16-byte piece][row]: lanes are rows, so every access is conflict-free
          auto park_smem = [&](int c, const uint32_t (&pk)[16]) {
            uint8_t* dst = smem + c * (kTileM * kChunkN * 2) + half * (kTileM * 64) + r * 16;
#pragma unroll
            for (int p = 0; p < 4; p++)
              *reinterpret_cast<uint4*>(dst + p * (kTileM * 16)) = make_uint4(pk[4 * p], pk[4 * p + 1], pk[4 * p + 2], pk[4 * p + 3]);
          };
          const int lastc = nchunks - 1;
          // all chunks but the last: those parked in shared memory in a rolled loop (the address depends on c only
          // arithmetically), those parked in registers unrolled so that `kept` is indexed statically
          const int nsm = lastc < kPark ? lastc : kPark;
#pragma unroll 1
          for (int c = 0; c < nsm; c++) {
            uint32_t pk[16];
            chunk_epilogue(c, pk);
            if (c == kOutSlot) out_stage_drain();
            park_smem(c, pk);
          }
#pragma unroll
          for (int c = kPark; c < kMaxChunks; c++) {
            if (c < lastc) {
              uint32_t pk[16];
              chunk_epilogue(c, pk);
#pragma unroll
              for (int j = 0; j < 16; j++) kept[(c - kPark) * 16 + j] = pk[j];
            }
          }
          // The next layer's A, K-block by K-block (four output chunks each).  A block of A may be overwritten once
          // this layer's last MMAs on it have retired: the MMA warp signals that per block while the last chunk is
          // still being computed, so blocks 0 and 1 are moved during the last chunk's MMAs and the next layer's first
          // MMAs run while the last chunk's epilogue and block are finished.
          const int nkb2 = L.N / kBlockK;
          // blocks before `wall` only need this layer's MMAs on the same block retired; from `wall` on a block holds
          // the last chunk or columns the layer reads to its end, so everything has to have retired
          const int wall = (nkb2 < nkb ? nkb2 : nkb) - 1;
          // move output chunks 4 kb2 .. 4 kb2 + 3 into the A columns of K-block kb2 and release the block
          auto move_block = [&](auto KB2) {
            constexpr int kb2 = decltype(KB2)::value;
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
              const int c = 4 * kb2 + c4;                     // compile-time after unrolling
              uint32_t pk[16];
              if (c < kPark) {
                const uint8_t* src = smem + c * (kTileM * kChunkN * 2) + half * (kTileM * 64) + r * 16;
#pragma unroll
                for (int p = 0; p < 4; p++) {
                  const uint4 q = *reinterpret_cast<const uint4*>(src + p * (kTileM * 16));
                  pk[4 * p] = q.x; pk[4 * p + 1] = q.y; pk[4 * p + 2] = q.z; pk[4 * p + 3] = q.w;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; j++) pk[j] = kept[(c - kPark) * 16 + j];
              }
              tmem_st16(lane_addr + (uint32_t)(c * (kChunkN / 2) + half * 16), pk);
            }
            tmem_st_wait();
            tc_fence_before();
            signal(bar_a_ready + 8 * kb2);
          };
          PROF_ADD(11);
          if (0 < wall) { wait_bar(bar_a_dead + 0, lph, abort_flag, P.status, ST_A_DEAD, P.wait_limit); tc_fence_after(); move_block(std::integral_constant<int, 0>{}); }
          if (1 < wall) { wait_bar(bar_a_dead + 8, lph, abort_flag, P.status, ST_A_DEAD, P.wait_limit); tc_fence_after(); move_block(std::integral_constant<int, 1>{}); }
          {
            uint32_t pk[16];
            chunk_epilogue(lastc, pk);                        // waits for the layer's last accumulator: every MMA has retired
            if (lastc < kPark) { if (lastc >= kOutSlot) out_stage_drain(); park_smem(lastc, pk); }
            else {
#pragma unroll
              for (int cc = kPark; cc < kMaxChunks; cc++)
                if (lastc == cc) {
#pragma unroll
                  for (int j = 0; j < 16; j++) kept[(cc - kPark) * 16 + j] = pk[j];
                }
            }
          }
          if (wall <= 0 && 0 < nkb2) move_block(std::integral_constant<int, 0>{}); else if (nkb2 <= 0) signal(bar_a_ready + 0);
          if (wall <= 1 && 1 < nkb2) move_block(std::integral_constant<int, 1>{}); else if (nkb2 <= 1) signal(bar_a_ready + 8);
          // Chunks 0-7 have left the park (what block 2 still reads lies behind them): the first 128 KB may take the next
          // tile's staged inputs.  An arrive here and a wait before the copies, instead of a rendezvous there.
          if (can_stage && l == P.nlayers - 2) mbar_arrive(bar_park);
          if (2 < nkb2) move_block(std::integral_constant<int, 2>{}); else signal(bar_a_ready + 16);   // blocks the next layer does not have stay in step
          PROF_ADD(12);
        } else {
          // ---- last layer: bias, output scaling / masks, then into the host arrays.  While its MMAs run, the next
          //      tile's inputs are fetched into the park area; they go into A as soon as the layer's last MMAs on
          //      K-block 0 have retired, so that the next tile's first layer runs under this tile's scatter.
          long long ci = 0, cj = 0, kk = 0;
          if (live) row_to_pos(P.g, row, &ci, &cj, &kk);
          const long long opos0 = ci * P.cout[0].si + cj * P.cout[0].sj + kk * P.cout[0].sk;
          const long long opos1 = ci * P.cout[1].si + cj * P.cout[1].sj + kk * P.cout[1].sk;
          const bool do_pre = can_prefetch && u + ustep < nunits;
          out_stage_drain();
          // this tile's outputs by bulk stores: 128 whole rows along the fastest loop index (as for the inputs)
          bool out_staged = false;
          long long of0 = 0, of1 = 0;
          if (can_stage_out && tile * kTileM + kTileM <= P.nrows) {
            long long c0, j0, k0, c2, j2, k2;
            row_to_pos(P.g, tile * kTileM, &c0, &j0, &k0);
            row_to_pos(P.g, tile * kTileM + kTileM - 1, &c2, &j2, &k2);
            if (j2 == j0 && k2 == k0 && c2 - c0 == kTileM - 1 && (c0 & 3) == 0) {
              out_staged = true;
              of0 = c0 + j0 * P.cout[0].sj + k0 * P.cout[0].sk;
              of1 = c0 + j0 * P.cout[1].sj + k0 * P.cout[1].sk;
            }
          }
          // Fetched element by element, the inputs wait in the park area (free during the last layer: every parked
          // chunk has been moved) in the park's thread-private layout, so no other thread ever touches them.
          static_assert(kBlockK / 2 / 32 == 4 && kPark >= 4, "the prefetch uses four park slots of 32 inputs per half row");
          // Staged form of that fetch: when the next tile is 128 whole rows that run along the fastest loop index, its
          // inputs come as fp32 [input][row] into the park area by bulk copies, one 512-byte run per model input (the
          // copy engine keeps far more bytes in flight than 128 loads per thread can, and nothing passes through
          // registers), and are converted when they go into A.  Otherwise the row threads load them one element each
          // as in the first tile.
          bool staged = false;
          if (do_pre && can_stage && P.nlayers >= 2) {
            wait_bar(bar_park, park_ph, abort_flag, P.status, ST_IN, P.wait_limit);
            park_ph ^= 1;
          }
          if (do_pre && can_stage) staged = stage_issue((PAIR ? 2 * (u + ustep) + crank : u + ustep) * kTileM);
          if (do_pre && !staged) {
            const long long nrow = (PAIR ? 2 * (u + ustep) + crank : u + ustep) * kTileM + r;
            bool lv; long long p0, p1;
            locate_in(nrow, lv, p0, p1);
            // 64 loads in flight per thread (no parked chunk is live in registers here), two batches per tile
#if !FORTIS_TC_GATHER64
#pragma unroll 1
            for (int g = 0; g < 4; g++) {
              uint32_t pk[16];
              gather_group(nrow, lv, p0, p1, half * per0 + 32 * g, pk);
              uint8_t* dst = smem + g * (kTileM * kChunkN * 2) + half * (kTileM * 64) + r * 16;
#pragma unroll
              for (int p = 0; p < 4; p++)
                *reinterpret_cast<uint4*>(dst + p * (kTileM * 16)) = make_uint4(pk[4 * p], pk[4 * p + 1], pk[4 * p + 2], pk[4 * p + 3]);
            }
#else
#pragma unroll 1
            for (int g2 = 0; g2 < 2; g2++) {
              uint32_t pk[2][16];
              gather_two_groups(nrow, lv, p0, p1, half * per0 + 64 * g2, pk[0], pk[1]);
#pragma unroll
              for (int h = 0; h < 2; h++) {
                uint8_t* dst = smem + (2 * g2 + h) * (kTileM * kChunkN * 2) + half * (kTileM * 64) + r * 16;
#pragma unroll
                for (int p = 0; p < 4; p++)
                  *reinterpret_cast<uint4*>(dst + p * (kTileM * 16)) = make_uint4(pk[h][4 * p], pk[h][4 * p + 1], pk[h][4 * p + 2], pk[h][4 * p + 3]);
              }
            }
#endif
          }
          PROF_ADD(20);
          for (int c = 0; c < nchunks; c++) {
            // From the epilogue of chunk n - 2 on, both issuers' last chunks can run (their accumulators were read by
            // the epilogues before), so the layer's last MMAs on K-block 0 retire without this thread's help.
            if (c == (nchunks < 2 ? nchunks - 1 : nchunks - 2) && do_pre) {
              wait_bar(bar_a_dead, lph, abort_flag, P.status, ST_A_DEAD, P.wait_limit);
              tc_fence_after();
              if (staged) {
                stage_consume();
              } else
#pragma unroll 1
              for (int g = 0; g < 4; g++) {
                uint32_t pk[16];
                const uint8_t* src = smem + g * (kTileM * kChunkN * 2) + half * (kTileM * 64) + r * 16;
#pragma unroll
                for (int p = 0; p < 4; p++) {
                  const uint4 q = *reinterpret_cast<const uint4*>(src + p * (kTileM * 16));
                  pk[4 * p] = q.x; pk[4 * p + 1] = q.y; pk[4 * p + 2] = q.z; pk[4 * p + 3] = q.w;
                }
                tmem_st16(lane_addr + (uint32_t)((half * per0 + 32 * g) >> 1), pk);
              }
              release_layer0();
              prefetched = true;
              PROF_ADD(21);
            }
            const uint32_t b = acc_it & 1, aph = (acc_it >> 1) & 1;
            acc_it++;
            const int n0 = c * kChunkN + half * 32;
            float4 bq[8];
#pragma unroll
            for (int j = 0; j < 8; j++) bq[j] = __ldg(reinterpret_cast<const float4*>(L.bias + n0) + j);
            PROF_ADD(13);
            wait_bar(bar_acc_full + 8 * b, aph, abort_flag, P.status, ST_ACC_FULL, P.wait_limit);
            PROF_ADD(14);
            tc_fence_after();
            uint32_t a[32];
            tmem_ld32(lane_addr + kAccCol0 + b * kChunkN + half * 32, a);
            tmem_ld_wait();
            tc_fence_before();
            signal(bar_acc_empty + 8 * b);
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
              if (out_staged) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                  const uint32_t code = (n0 + j < kFastOut) ? o_code[n0 + j] : 0xFFu;
                  if (code != 0xFF) {
                    *reinterpret_cast<float*>(smem + kOutStage + (n0 + j) * (kTileM * 4) + r * 4) = v[j];
                    csum += (double)v[j];
                  }
                }
              } else if (P.fast_out) {
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
          if (out_staged) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");          // this thread's values, for the copy engine
            asm volatile("bar.sync 1, %0;" ::"r"(kEpiThreads) : "memory");        // every row of every output is there
            const int n = (int)threadIdx.x;
            if (n < kFastOut) {
              const uint32_t code = o_code[n];
              if (code != 0xFF)
                bulk_store_thread(s_base_out[code & 0x7F] + ((long long)o_off[n] + ((code & 0x80) ? of1 : of0)),
                                  base + kOutStage + (uint32_t)(n * (kTileM * 4)), kTileM * 4);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            out_pending = true;
          }
          PROF_ADD(13);
        }
      }
    }
    if (out_pending) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");     // the last tile's output stores are complete
    if (P.partials) {
      // per-CTA checksum partial in a fixed order: shuffle tree per warp, then warp results in index order
      double* wsum = (double*)(smem + kParkB + kRingB + 272);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) csum += __shfl_down_sync(0xffffffffu, csum, o);
      if (lane == 0) wsum[warp] = csum;
      asm volatile("bar.sync 1, %0;" ::"r"(kEpiThreads) : "memory");
      if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < 8; w++) t += wsum[w];
        P.partials[blockIdx.x] = t;
        if (P.sum) {
          // the last CTA to get here adds all partials to the step checksum, in CTA order (so the result does not
          // depend on which CTA was last); it also re-arms the counter for the next launch
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
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // a wait gave up: copies of this CTA may still be in flight; give them time to land before the shared memory
    // is handed back (bounded)
    for (int i = 0; i < 2000; i++) __nanosleep(1000);
  }
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();      // neither CTA leaves while its partner can still signal its barriers
  if (warp == 9) {
    tc_fence_after();
    if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
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

TcTestKnobs g_tc_test = {0u, 0, 0};

// One Linear layer converted for the tensor-core kernel: padded, rounded to the 16-bit operand type (FP8 weights: the
// nearest E4M3 code of w / scale, which bf16 represents exactly), as row-major [N][K] (`rowmajor`, optional) and as
// the stage images the kernel streams: per chunk of 64 features and per 256-wide K-block one contiguous 32 KB block
// holding four 64 x 64 sub-tiles in the 128-byte-swizzled K-major layout the MMA descriptor expects (16-byte piece j of
// row r sits at piece j ^ (r & 7)), so that a stage is ONE linear bulk copy.
void pack_layer_host(const LayerHost& L, bool last, int precision, PackedLayer* Q, std::vector<uint16_t>* rowmajor) {
  const int K = round_up(L.cin, kBlockK);
  const int N = last ? round_up(L.cout, kChunkN) : round_up(L.cout, kBlockK);
  std::vector<uint16_t> wb((size_t)N * K, 0);
  Q->K = K; Q->N = N;
  Q->bias.assign(N, 0.f); Q->scale.assign(N, 1.f);
  for (int n = 0; n < L.cout; n++) {
    Q->bias[n] = L.b[n];
    float sc = 1.f;
    if (precision == PREC_FP8W) {
      float amax = 0.f;
      for (int k = 0; k < L.cin; k++) amax = std::fmax(amax, std::fabs(L.W[(size_t)n * L.cin + k]));
      sc = amax > 0.f ? amax / 448.0f : 1.0f;
      Q->scale[n] = sc;
    }
    for (int k = 0; k < L.cin; k++) {
      float w = L.W[(size_t)n * L.cin + k];
      if (precision == PREC_FP8W) w = e4m3_round(w / sc);
      wb[(size_t)n * K + k] = precision == PREC_FP16 ? f32_to_f16(w) : f32_to_bf16(w);
    }
  }
  Q->image.assign((size_t)N * K, 0);
  const int nks = K / kStageK;
  for (int c = 0; c < N / kChunkN; c++)
    for (int ks = 0; ks < nks; ks++) {
      uint16_t* blk = Q->image.data() + ((size_t)c * nks + ks) * (kStageBytes / 2);
      for (int t = 0; t < kStageK / 64; t++)
        for (int r = 0; r < kChunkN; r++)
          for (int j = 0; j < 8; j++) {
            const uint16_t* src = wb.data() + (size_t)(c * kChunkN + r) * K + ks * kStageK + t * 64 + j * 8;
            uint16_t* dst = blk + (size_t)t * (kChunkN * 64) + r * 64 + ((j ^ (r & 7)) * 8);
            std::memcpy(dst, src, 16);
          }
    }
  if (rowmajor) rowmajor->swap(wb);
}

// host-only: the stage images of one layer, for tests that compare them with the exporter's
int tc_debug_pack_layer(const float* W, const float* b, int cout, int cin, int last, int precision, uint16_t* image, float* bias,
                        float* scale, int* K, int* N) {
  LayerHost L;
  L.cin = cin; L.cout = cout;
  L.W.assign(W, W + (size_t)cout * cin);
  L.b.assign(b, b + cout);
  PackedLayer Q;
  pack_layer_host(L, last != 0, precision, &Q, nullptr);
  *K = Q.K; *N = Q.N;
  if (image) std::memcpy(image, Q.image.data(), Q.image.size() * 2);
  if (bias) std::memcpy(bias, Q.bias.data(), Q.bias.size() * 4);
  if (scale) std::memcpy(scale, Q.scale.data(), Q.scale.size() * 4);
  return 0;
}

struct TcModel {
  int nlayers = 0, n_in = 0, n_out = 0;
  std::vector<void*> w;            // bf16 [N][K] padded
  std::vector<float*> bias, scale;
  float *in_div = nullptr, *out_mul = nullptr, *relu_mask = nullptr;
  TcLayer layer[kMaxLayers];
  CUtensorMap maps[kMaxLayers];
  bool has_scale = false, f16 = false;
  bool pair = false;               // run as two-CTA clusters (row-major weights + tensor maps are on the device as well)
};

// Two-CTA clusters (each SM streams half of the weights; the default) or one CTA per SM: option "tc_pair", else
// FORTIS_TC_PAIR=0|1.  Measured on the 244-768x4-128 net, 49,152 to 2^20 columns: the cluster form is 9-16 % faster in
// bf16 / fp16 and 8-9 % faster with FP8 weights.
static int g_tc_pair = -1;
void tc_set_pair_mode(int on) { g_tc_pair = on; }
bool tc_pair_mode(int precision) {
  static const int env = [] { const char* e = std::getenv("FORTIS_TC_PAIR"); return e ? (std::atoi(e) != 0 ? 1 : 0) : -1; }();
  if (g_tc_pair >= 0) return g_tc_pair != 0;
  if (env >= 0) return env != 0;
  (void)precision;
  return true;
}

bool tc_model_supported(const ModelHost& M, std::string* why) {
  auto no = [&](const char* w) { if (why) *why = w; return false; };
  if (!M.is_mlp()) return no("not an MLP");
  if ((int)M.layers.size() > kMaxLayers) return no("more than 8 layers");
  for (size_t l = 0; l < M.layers.size(); l++) {
    const LayerHost& L = M.layers[l];
    if (round_up(L.cin, kBlockK) > kMaxK) return no("a layer input is wider than 768");
    if (L.act == ACT_LEAKY && !(L.slope >= 0.f && L.slope <= 1.f)) return no("LeakyReLU slope outside [0, 1]");
    const int npad = l + 1 < M.layers.size() ? round_up(L.cout, kBlockK) : round_up(L.cout, kChunkN);
    if (npad > kMaxK) return no("a layer output is wider than 768");
  }
  return true;
}

// how many two-CTA clusters of the kernel the device holds at once (the SMs of a cluster share a GPC, so this can be
// fewer than half the SM count); 0 when the query fails
int tc_max_clusters() {
  static int cached[16] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return 0;
  if (cached[dev]) return cached[dev] > 0 ? cached[dev] : 0;
  cudaFuncSetAttribute(mlp_tc_fused_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 148); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kSmemBytes;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, mlp_tc_fused_kernel<false, false, true>, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = -1; }
  cached[dev] = n;
  if (std::getenv("FORTIS_TC_DEBUG")) std::fprintf(stderr, "fortis: %d two-CTA clusters of the fused MLP kernel fit the device\n", n);
  return n > 0 ? n : 0;
}

int tc_grid(const TcModel* m, long long nrows) {
  const long long tiles = (nrows + kTileM - 1) / kTileM;
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (m && m->pair) {
    // clusters of two CTAs, a pair of tiles per cluster and wave; the same evening-out over the clusters
    const int fit = tc_max_clusters();
    const long long units = (tiles + 1) / 2, slots = fit > 0 ? fit : (sms / 2 > 0 ? sms / 2 : 1);
    if (units <= slots) return (int)(2 * (units > 0 ? units : 1));
    const long long waves = (units + slots - 1) / slots;
    return (int)(2 * ((units + waves - 1) / waves));
  }
  if (tiles <= sms) return (int)(tiles > 0 ? tiles : 1);
  // The launch lasts as long as the CTA with the most tiles: waves = ceil(tiles / SMs).  With that fixed, use only as
  // many CTAs as give every one of them `waves` tiles (384 tiles: 128 CTAs x 3 instead of 88 x 3 + 60 x 2): the idle SMs
  // draw no power and put no load on L2, and the part holds a higher clock for the others.
  static const bool even = std::getenv("FORTIS_TC_FULL_GRID") == nullptr;
  const long long waves = (tiles + sms - 1) / sms;
  return even ? (int)((tiles + waves - 1) / waves) : sms;
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
  const bool pair = tc_pair_mode(precision);
  const bool want_maps = pair || !FORTIS_TC_TILED_W;
  EncodeTiledFn enc = want_maps ? encode_fn() : nullptr;
  if (want_maps && !enc) { if (err) *err = "cuTensorMapEncodeTiled is not available from the driver"; return nullptr; }
  TcModel* m = new TcModel();
  m->pair = pair;
  m->nlayers = (int)M.layers.size(); m->n_in = M.n_in(); m->n_out = M.n_out();
  auto fail = [&](const std::string& w) { if (err) *err = w; tc_model_destroy(m); return (TcModel*)nullptr; };
  for (int l = 0; l < m->nlayers; l++) {
    const LayerHost& L = M.layers[l];
    PackedLayer Q;
    std::vector<uint16_t> wb;
    const bool prepacked = FORTIS_TC_TILED_W && !pair && M.packed_precision == precision && l < (int)M.packed.size() &&
                           M.packed[l].K == round_up(L.cin, kBlockK) &&
                           M.packed[l].N == (l + 1 < m->nlayers ? round_up(L.cout, kBlockK) : round_up(L.cout, kChunkN));
    if (prepacked) Q = M.packed[l];                        // the blob carries this precision's stage images
    else pack_layer_host(L, l + 1 == m->nlayers, precision, &Q, &wb);
    const int K = Q.K, N = Q.N;
    const std::vector<uint16_t>& wt = Q.image;
    const std::vector<float>&bias = Q.bias, &scale = Q.scale;
    // only the form this build streams goes to the device: the stage images, or (tensor copies: the two-CTA form) the
    // row-major weights
    void *dw = nullptr, *dwt = nullptr; float *db = nullptr, *ds = nullptr;
    const bool tiled = FORTIS_TC_TILED_W && !pair;
    const std::vector<uint16_t>& image = tiled ? wt : wb;
    void** slot = tiled ? &dwt : &dw;
    if (cudaMalloc(slot, image.size() * 2) != cudaSuccess || cudaMalloc(&db, N * 4) != cudaSuccess)
      return fail("out of device memory for packed weights");
    m->w.push_back(*slot); m->bias.push_back(db);
    cudaMemcpy(*slot, image.data(), image.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(db, bias.data(), N * 4, cudaMemcpyHostToDevice);
    if (precision == PREC_FP8W) {
      if (cudaMalloc(&ds, N * 4) != cudaSuccess) return fail("out of device memory for weight scales");
      cudaMemcpy(ds, scale.data(), N * 4, cudaMemcpyHostToDevice);
    }
    m->scale.push_back(ds);
    TcLayer& T = m->layer[l];
    T.K = K; T.N = N; T.n_real = L.cout; T.act = L.act; T.bias = db; T.scale = ds; T.wtiled = (const uint8_t*)dwt;
    T.wdev = (const uint8_t*)*slot;
    T.slope = L.act == ACT_NONE ? 1.f : L.act == ACT_RELU ? 0.f : L.slope;      // act(v) = max(v, v * slope)
    if (!tiled) {
      // W[N][K] viewed as [K/64][N][64]: one box of {64 k, 64 rows (32: a CTA's half in the two-CTA form), 4 k-blocks}
      // lands in shared memory as four consecutive sub-tiles, each in the 128-byte-swizzled K-major layout the MMA
      // descriptor expects
      const cuuint64_t dims[3] = {64, (cuuint64_t)N, (cuuint64_t)(K / 64)};
      const cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
      const cuuint32_t box[3] = {64, (cuuint32_t)(pair ? kChunkN / 2 : kChunkN), (cuuint32_t)(kStageK / 64)};
      const cuuint32_t estr[3] = {1, 1, 1};
      const CUresult r = enc(&m->maps[l], precision == PREC_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dw, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    }
  }
  auto up = [&](const std::vector<float>& v) -> float* {
    if (v.empty()) return nullptr;
    float* d = nullptr;
    cudaMalloc(&d, v.size() * 4);
    cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
    return d;
  };
  m->in_div = up(M.in_div); m->out_mul = up(M.out_mul); m->relu_mask = up(M.relu_mask);
  if (cudaFuncSetAttribute(mlp_tc_fused_kernel<false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(mlp_tc_fused_kernel<true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(mlp_tc_fused_kernel<false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(mlp_tc_fused_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(mlp_tc_fused_kernel<true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(mlp_tc_fused_kernel<false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
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
  P.g = L.g; P.nrows = nrows; P.partials = L.partials; P.sum = L.sum; P.done = L.done; P.status = L.status;
  P.fast_in = L.fast_in && m->n_in <= kFastIn; P.fast_out = L.fast_out && m->n_out <= kFastOut;
  for (int i = 0; i < 2; i++) {
    P.cin[i] = StrideClass{L.cin[i][0], L.cin[i][1], L.cin[i][2]};
    P.cout[i] = StrideClass{L.cout[i][0], L.cout[i][1], L.cout[i][2]};
  }
  P.store_by_slot = L.store_by_slot;
  P.wait_limit = g_tc_test.wait_limit ? g_tc_test.wait_limit : kWaitLimit;
  P.test_skip_stage = g_tc_test.skip_stage;
  static const bool no_prefetch = std::getenv("FORTIS_TC_NO_L2_PREFETCH") != nullptr;
  P.no_l2_prefetch = no_prefetch;
  static const bool no_stage_inputs = std::getenv("FORTIS_TC_NO_STAGE_INPUTS") != nullptr;
  // (mapped host pages are staged the same way: bulk copies read them at 33 GB/s, the threads' own loads at 24)
  P.no_stage_inputs = no_stage_inputs || g_tc_test.no_stage;
  static const bool no_stage_outputs = std::getenv("FORTIS_TC_NO_STAGE_OUTPUTS") != nullptr;
  P.no_stage_outputs = no_stage_outputs || g_tc_test.no_stage;
  if (!P.fast_in && !P.X) { if (err) *err = "tensor-core step: no input"; return false; }
  if (!P.fast_out && !P.Y) { if (err) *err = "tensor-core step: no output"; return false; }
  const int grid = tc_grid(m, nrows);
#ifdef FORTIS_TC_PROF
  static const bool want_prof = std::getenv("FORTIS_TC_PROF") != nullptr;
#else
  static const bool want_prof = false;
#endif
  static long long* dprof = nullptr;
  if (want_prof) {
    if (!dprof) cudaMalloc(&dprof, 64 * sizeof(long long));
    cudaMemsetAsync(dprof, 0, 64 * sizeof(long long), s);
    P.prof = dprof;
  }
  if (m->pair) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kSmemBytes; cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    if (m->has_scale) cudaLaunchKernelEx(&cfg, mlp_tc_fused_kernel<true, false, true>, P);
    else if (m->f16) cudaLaunchKernelEx(&cfg, mlp_tc_fused_kernel<false, true, true>, P);
    else cudaLaunchKernelEx(&cfg, mlp_tc_fused_kernel<false, false, true>, P);
  } else if (m->has_scale) mlp_tc_fused_kernel<true, false, false><<<grid, kThreads, kSmemBytes, s>>>(P);
  else if (m->f16) mlp_tc_fused_kernel<false, true, false><<<grid, kThreads, kSmemBytes, s>>>(P);
  else mlp_tc_fused_kernel<false, false, false><<<grid, kThreads, kSmemBytes, s>>>(P);
  if (want_prof) {
    long long h[64];
    cudaStreamSynchronize(s);
    cudaMemcpy(h, dprof, sizeof h, cudaMemcpyDeviceToHost);
    std::fprintf(stderr, "tc prof (cycles, CTA 0): mma issue %lld | wait a_ready %lld acc_empty %lld full %lld || rows: gather %lld | hidden wait %lld work %lld "
                 "transfer %lld | last wait %lld work %lld || tma wait-empty %lld issue %lld\n",
                 h[0], h[1], h[2], h[3], h[9], h[10], h[11], h[12], h[14], h[13], h[16], h[17]);
    std::fprintf(stderr, "tc prof last layer: next tile's gather %lld, its move into tensor memory %lld\n", h[20], h[21]);
    for (int l = 0; l < m->nlayers && l < 8; l++)
      std::fprintf(stderr, "tc prof layer %d: issue %lld | wait a_ready %lld acc_empty %lld full %lld\n", l, h[32 + l], h[40 + l], h[48 + l], h[56 + l]);
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { if (err) *err = std::string("tensor-core kernel launch: ") + cudaGetErrorString(e); return false; }
  return true;
}

}  // namespace fortis
