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
// [P rows][64 channels] (one 128-byte row per voxel).  With the border stored explicitly, the input rows a tap
// (kd, kh, kw) needs for output rows p0..p0+127 are simply rows p0+shift..p0+shift+127 with
// shift = (kd-1)(H+2)(W+2) + (kh-1)(W+2) + (kw-1): every tap is ONE plain 2-D TMA tile load, no im2col, no masks
// (rows outside [0, P) are zero-filled by TMA).  Border rows of the output are computed and then written as zeros,
// which keeps the padding intact for the next layer; that costs ((D+2)(H+2)(W+2))/(DHW) = 1.19x the useful work
// at 33^3.
//
// Per 128-row tile: D[128 x 64] = sum over 27 taps of A_tap[128 x 64] . W_tap[64 x 64]^T, 4 MMAs (K = 16) per tap.
// The three kw taps of one (kd, kh) read the same activation rows shifted by one, so ONE 130-row tile is staged per
// (kd, kh) and the three taps address it through descriptors whose start moves by 128 bytes (the kernel is bound
// by the L2 -> shared-memory stream, and this cuts it from 648 KB to 366 KB per tile).  Ring of 5 stages of 41 KB
// (activation tile + the three weight tiles, 128-byte swizzle); two accumulators so that the epilogue of a tile
// overlaps the MMAs of the next.  Warp 0: TMA, warp 1: MMA, warps 2-5:
// epilogue (thread = one voxel row, 64 channels).
//
// First layer: the fp32 NDHWC input is packed into its own padded bf16 volume with channels >= Cin zero, and the
// weights are padded the same way, so the layer is the same shifted-tile GEMM with one k step per tap instead of
// four.  Last layer: the weights are padded to 16 output channels; the epilogue adds the bias, applies the
// activation and writes the real channels of interior voxels as fp32.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "fortis_kernels.h"
#include "fortis_model.h"
#include "fortis_tc.cuh"

namespace fortis {

using namespace tc;

namespace {

constexpr int kC = 64;                       // channels of the tensor-core layers
constexpr int kTile = 128;                   // output rows per tile
constexpr int kRowsA = kTile + 2;            // the three kw taps of one (kd, kh) read rows p0-1 .. p0+128 of the same tile
constexpr int kBytesA = kRowsA * kC * 2;     // 16,640 B landed by TMA
constexpr int kStageA = 17 * 1024;           // region reserved for it (1024-byte multiple keeps the weights aligned)
constexpr int kStageW = 3 * kC * kC * 2;     // 24 KB: the three kw weight tiles, consecutive rows of the weight matrix
constexpr int kStage = kStageA + kStageW;    // 41 KB
constexpr int kStagesC = 5;
constexpr int kConvThreads = 192;
constexpr int kConvSmem = kStagesC * kStage + 256;
template <int NOUT> struct ConvIdesc { static constexpr uint32_t value = idesc_bf16(kTile, NOUT); };
constexpr int kEdgeC = 16;                   // first layer: input channels kept; last layer: output channels computed
enum { CST_FULL = 11, CST_EMPTY = 12, CST_ACC_FULL = 13, CST_ACC_EMPTY = 14, CST_ALIGN = 16 };

struct ConvTcParams {
  CUtensorMap amap;            // input activations [P][64] bf16, box 64 x 130
  CUtensorMap wmap;            // weights [27 * 64 (tap, cout)][64 cin] bf16, box 64 x 192
  const float* bias;           // [64] (zero beyond the layer's real outputs)
  const __nv_bfloat16* skip;   // [P][64] or null
  __nv_bfloat16* out;          // [P][64]
  float* y;                    // last layer: fp32 [N*D*H*W][F]
  int F;                       // last layer: real output channels (<= 16)
  int D, H, W;                 // unpadded extent
  long long P;                 // padded rows
  float slope;                 // act(v) = max(v, v * slope)
  int* status;
};

// KSTEPS: 16-wide k steps issued per tap (4 = all 64 input channels, 1 = only the first 16);  NOUT: output channels
// of the MMA (weight rows staged per tap);  LAST: write fp32 NDHWC instead of the padded bf16 volume
template <int KSTEPS, int NOUT, bool LAST>
__global__ void __launch_bounds__(kConvThreads, 1) conv3d_tc_kernel(const __grid_constant__ ConvTcParams P) {
  constexpr uint32_t kIdescN = ConvIdesc<NOUT>::value;
  constexpr int kBytesW = 3 * NOUT * kC * 2;                      // the three kw weight tiles of one (kd, kh)
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = smem_u32(smem);
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicCAS(P.status, 0, CST_ALIGN);
    return;
  }
  const uint32_t bars = base + kStagesC * kStage;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kStagesC, bar_acc_full = bars + 16 * kStagesC, bar_acc_empty = bar_acc_full + 16;
  uint32_t* tmem_slot = (uint32_t*)(smem + kStagesC * kStage + 16 * kStagesC + 32);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long ntiles = (P.P + kTile - 1) / kTile;
  const int Wp = P.W + 2, Hp = P.H + 2, Dp = P.D + 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesC; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int b = 0; b < 2; b++) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, 128); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0 && lane < 2)
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(lane ? &P.wmap : &P.amap)) : "memory");
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(128u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer: per tile 27 stages, each the shifted activation tile and that tap's weight tile
    uint32_t s = 0, ph = 0;
    bool stop = false;
    for (long long tile = blockIdx.x; tile < ntiles && !stop; tile += gridDim.x) {
      const long long p0 = tile * kTile;
      for (int g = 0; g < 9; g++) {                               // (kd, kh) groups: one activation tile serves kw = 0, 1, 2
        const int kd = g / 3, kh = g % 3;
        const long long shift = (long long)(kd - 1) * Hp * Wp + (long long)(kh - 1) * Wp - 1;
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, P.status, CST_EMPTY)) { stop = true; break; }
        mbar_expect_tx(bar_full + 8 * s, kBytesA + kBytesW);
        const uint32_t dst = base + s * kStage;
        tma_load_2d(dst, &P.amap, 0, (int)(p0 + shift), bar_full + 8 * s);
        tma_load_2d(dst + kStageA, &P.wmap, 0, g * 3 * NOUT, bar_full + 8 * s);
        if (++s == kStagesC) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    uint32_t s = 0, ph = 0, acc_it = 0;
    const uint64_t desc_hi = make_kmajor_sw128_desc(0) & 0xFFFFFFFF00000000ull;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, acc_it++) {
      const uint32_t b = acc_it & 1, aph = (acc_it >> 1) & 1;
      mbar_wait(bar_acc_empty + 8 * b, aph ^ 1, abort_flag, P.status, CST_ACC_EMPTY);
      tc_fence_after();
      const uint32_t d_tmem = tmem + b * kC;
      for (int g = 0; g < 9; g++) {
        mbar_wait(bar_full + 8 * s, ph, abort_flag, P.status, CST_FULL);
        tc_fence_after();
        const uint32_t sb = base + s * kStage;
        const uint64_t ad = desc_hi | (uint64_t)((sb >> 4) & 0x3FFF);
        const uint64_t bd = desc_hi | (uint64_t)(((sb + kStageA) >> 4) & 0x3FFF);
#pragma unroll
        for (int kw = 0; kw < 3; kw++) {
          // tap kw reads the tile shifted down by kw rows: the start address moves by kw * 128 bytes; the 128-byte
          // swizzle is a function of the shared-memory address itself, so the shifted view stays consistent with
          // what TMA wrote
          const uint64_t adk = ad + (uint64_t)(kw * 8);
          const uint64_t bdk = bd + (uint64_t)(kw * (NOUT * kC * 2 >> 4));
#pragma unroll
          for (int j = 0; j < KSTEPS; j++)
            tc_mma_ss<kIdescN>(d_tmem, adk + (uint64_t)(j * 2), bdk + (uint64_t)(j * 2), (uint32_t)(g | kw | j));
        }
        tc_commit(bar_empty + 8 * s);
        if (++s == kStagesC) { s = 0; ph ^= 1; }
      }
      tc_commit(bar_acc_full + 8 * b);
    }
  } else {
    // ---- epilogue: thread = one output row (voxel of the padded volume), 64 channels
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    float bias[kC];
#pragma unroll
    for (int j = 0; j < kC / 4; j++) {
      const float4 q = __ldg(reinterpret_cast<const float4*>(P.bias) + j);
      bias[4 * j] = q.x; bias[4 * j + 1] = q.y; bias[4 * j + 2] = q.z; bias[4 * j + 3] = q.w;
    }
    uint32_t acc_it = 0;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, acc_it++) {
      const uint32_t b = acc_it & 1, aph = (acc_it >> 1) & 1;
      const long long p = tile * kTile + r;
      bool interior = false;
      if (p < P.P) {
        const int wp = (int)(p % Wp), hp = (int)((p / Wp) % Hp), dp = (int)((p / ((long long)Wp * Hp)) % Dp);
        interior = wp >= 1 && wp <= P.W && hp >= 1 && hp <= P.H && dp >= 1 && dp <= P.D;
      }
      // residual row, fetched while the MMAs of this tile are still running
      uint4 sk[8];
      const bool use_skip = !LAST && P.skip != nullptr && interior;
      if (use_skip) {
#pragma unroll
        for (int j = 0; j < 8; j++) sk[j] = __ldg(reinterpret_cast<const uint4*>(P.skip + p * kC) + j);
      }
      mbar_wait(bar_acc_full + 8 * b, aph, abort_flag, P.status, CST_ACC_FULL);
      tc_fence_after();
      if (LAST) {
        uint32_t a[32];                                            // columns >= NOUT are not part of this layer
        tmem_ld32(lane_addr + b * kC, a);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(bar_acc_empty + 8 * b);
        if (interior) {
          const long long n_ = p / ((long long)Wp * Hp * Dp);
          const int wp = (int)(p % Wp), hp = (int)((p / Wp) % Hp), dp = (int)((p / ((long long)Wp * Hp)) % Dp);
          float* dst = P.y + ((((n_ * P.D + dp - 1) * P.H + hp - 1) * P.W) + wp - 1) * P.F;
#pragma unroll
          for (int f = 0; f < NOUT; f++)
            if (f < P.F) { const float v = __uint_as_float(a[f]) + bias[f]; dst[f] = fmaxf(v, v * P.slope); }
        }
        continue;
      }
      uint32_t a0[32], a1[32];
      tmem_ld32(lane_addr + b * kC, a0);
      tmem_ld32(lane_addr + b * kC + 32, a1);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(bar_acc_empty + 8 * b);
      if (p < P.P) {
        uint4 o[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; e++) {
            const int c = 8 * j + e;
            v[e] = __uint_as_float(c < 32 ? a0[c] : a1[c - 32]) + bias[c];
          }
          if (use_skip) {
            const __nv_bfloat162* s2 = reinterpret_cast<const __nv_bfloat162*>(&sk[j]);
#pragma unroll
            for (int e = 0; e < 4; e++) { const float2 f = __bfloat1622float2(s2[e]); v[2 * e] += f.x; v[2 * e + 1] += f.y; }
          }
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const float x0 = interior ? fmaxf(v[2 * e], v[2 * e] * P.slope) : 0.f;
            const float x1 = interior ? fmaxf(v[2 * e + 1], v[2 * e + 1] * P.slope) : 0.f;
            pk[e] = pack_bf16(x0, x1);
          }
          o[j] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        uint4* dst = reinterpret_cast<uint4*>(P.out + p * kC);
#pragma unroll
        for (int j = 0; j < 8; j++) dst[j] = o[j];
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
  }
}

// ---- network input: fp32 NDHWC with C <= 16 channels -> the first 16 channels (32 bytes) of the padded bf16 rows; the
// border rows and the channels beyond 16 of this buffer are never written (zero from allocation; the first layer's
// MMAs read only the first 16 channels)
__global__ void __launch_bounds__(256) conv_pack_input_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                              int N, int D, int H, int W, int C) {
  const long long nvox = (long long)N * D * H * W;
  for (long long v = (long long)blockIdx.x * 256 + threadIdx.x; v < nvox; v += (long long)gridDim.x * 256) {
    const int w_ = (int)(v % W), h_ = (int)((v / W) % H), d_ = (int)((v / ((long long)W * H)) % D), n_ = (int)(v / ((long long)W * H * D));
    const long long p = (((long long)n_ * (D + 2) + d_ + 1) * (H + 2) + h_ + 1) * (W + 2) + w_ + 1;
    float f[16];
#pragma unroll
    for (int c = 0; c < 16; c++) f[c] = c < C ? __ldg(x + v * C + c) : 0.f;
    uint32_t pk[8];
#pragma unroll
    for (int e = 0; e < 8; e++) pk[e] = pack_bf16(f[2 * e], f[2 * e + 1]);
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

uint16_t to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

float slope_of(const LayerHost& L) { return L.act == ACT_NONE ? 1.f : L.act == ACT_RELU ? 0.f : L.slope; }

}  // namespace

struct ConvTcModel {
  std::vector<LayerHost> meta;
  std::vector<void*> w; std::vector<float*> b;             // per layer: bf16 [27 * rows][64] (rows = 64, last layer 16), fp32 bias [64]
  std::vector<CUtensorMap> wmaps;
  __nv_bfloat16* buf[4] = {nullptr, nullptr, nullptr, nullptr};   // three rotating activation volumes + the packed input
  CUtensorMap amaps[4];
  long long P = 0;
  int shape[4] = {0, 0, 0, 0};
  int* status = nullptr;
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

ConvTcModel* conv_tc_create(const ModelHost& M, std::string* err) {
  std::string why;
  if (!conv_tc_supported(M, &why)) { if (err) *err = why; return nullptr; }
  ConvTcModel* m = new ConvTcModel();
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
        for (int t = 0; t < 27; t++) wb[((size_t)t * rows + f) * kC + c] = to_bf16(L.W[((size_t)f * L.cin + c) * 27 + t]);
    std::vector<float> bias(kC, 0.f);
    for (int f = 0; f < L.cout; f++) bias[f] = L.b[f];
    void* dw = upload(wb.data(), wb.size() * 2);
    float* db = (float*)upload(bias.data(), bias.size() * 4);
    if (!dw || !db) return fail("out of device memory for conv weights");
    m->w.push_back(dw); m->b.push_back(db);
    CUtensorMap map;
    if (!make_map(&map, dw, 27 * rows, 3 * rows)) return fail("cuTensorMapEncodeTiled failed for conv weights");
    m->wmaps.push_back(map);
  }
  if (cudaMalloc(&m->status, sizeof(int)) != cudaSuccess) return fail("out of device memory");
  cudaMemset(m->status, 0, sizeof(int));
  if (cudaFuncSetAttribute(conv3d_tc_kernel<4, kC, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kConvSmem) != cudaSuccess ||
      cudaFuncSetAttribute(conv3d_tc_kernel<1, kC, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kConvSmem) != cudaSuccess ||
      cudaFuncSetAttribute(conv3d_tc_kernel<4, kEdgeC, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kConvSmem) != cudaSuccess)
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
      if (cudaMalloc(&m->buf[b], (size_t)P * kC * 2) != cudaSuccess) { if (err) *err = "out of device memory for conv activations"; return false; }
      cudaMemsetAsync(m->buf[b], 0, (size_t)P * kC * 2, s);        // the border must be zero before the first layer writes the interior
      if (!make_map(&m->amaps[b], m->buf[b], P, kRowsA)) { if (err) *err = "cuTensorMapEncodeTiled failed for conv activations"; return false; }
    }
    m->P = P; m->shape[0] = N; m->shape[1] = D; m->shape[2] = H; m->shape[3] = W;
  }
  const int nl = (int)m->meta.size();
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  {
    const long long blocks = (nvox + 255) / 256;
    conv_pack_input_kernel<<<(unsigned)(blocks < sms * 8 ? blocks : sms * 8), 256, 0, s>>>(x, m->buf[3], N, D, H, W, m->meta[0].cin);
  }
  const long long ntiles = (P + kTile - 1) / kTile;
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  int cur = 3, skip = -1;
  for (int l = 0; l < nl; l++) {
    const LayerHost& L = m->meta[l];
    int dst = -1;
    for (int b = 0; b < 3; b++) if (b != cur && b != skip) { dst = b; break; }
    if ((L.flags & LFLAG_ADD_SKIP) && skip < 0) { if (err) *err = "conv3d model: a layer adds a skip that was never saved"; return false; }
    ConvTcParams P_;
    std::memset(&P_, 0, sizeof P_);
    P_.amap = m->amaps[cur]; P_.wmap = m->wmaps[l]; P_.bias = m->b[l];
    P_.skip = (L.flags & LFLAG_ADD_SKIP) ? m->buf[skip] : nullptr;
    P_.out = m->buf[dst]; P_.y = y; P_.F = L.cout;
    P_.D = D; P_.H = H; P_.W = W; P_.P = P; P_.slope = slope_of(L); P_.status = m->status;
    if (l == nl - 1) conv3d_tc_kernel<4, kEdgeC, true><<<grid, kConvThreads, kConvSmem, s>>>(P_);
    else if (l == 0) conv3d_tc_kernel<1, kC, false><<<grid, kConvThreads, kConvSmem, s>>>(P_);
    else conv3d_tc_kernel<4, kC, false><<<grid, kConvThreads, kConvSmem, s>>>(P_);
    if (L.flags & LFLAG_SAVE_SKIP) skip = dst;
    cur = dst;
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { if (err) *err = std::string("tensor-core conv launch: ") + cudaGetErrorString(e); return false; }
  return true;
}

int conv_tc_status(ConvTcModel* m) {
  int v = 0;
  if (m && m->status) cudaMemcpy(&v, m->status, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

}  // namespace fortis
