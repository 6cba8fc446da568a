// fortis_checksum_noalloc: the fp64 checksum of a device array for callers that must not allocate.
//
// Who cannot allocate: a simulation that sizes its own device pools at start-up and hands the rest of the GPU to
// them (an OpenACC / CUDA Fortran host with a fixed memory budget), and code that runs between two time-critical
// launches, where cudaMalloc's implicit device synchronisation would stall the step.  For them the block partials of the two-pass sum live in a fixed array that is part of
// the library image instead of in memory obtained at run time.
//
// The scratch is the file-scope array below: kNoAllocSlots doubles (32 KB).  Every GPU that loads the library
// holds it from load to exit.  Each block sums one contiguous span of kNoAllocSpan elements into its own slot, so
// the largest array that can be summed is kNoAllocSlots * kNoAllocSpan = 2^28 elements; larger requests are refused.
// Every slot that the second pass reads was written by the first pass of the same call, so nothing has to be cleared
// between calls, although the array does keep the previous call's partials.  All calls share the one array: two
// calls whose kernels can overlap on the GPU (different streams, no dependency between them) race on it.
#include <cuda_runtime.h>

#include <cstdio>

#include "../../include/fortis_b200.h"

namespace {

constexpr int kNoAllocSlots = 4096;
constexpr long kNoAllocSpan = 65536;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) double g_noalloc_partials[kNoAllocSlots];

// Device address of the array per device.  In host code the symbol's name is only a handle: the address a kernel
// can use has to be asked for, once per device, with that device current.  The address is cached per device ordinal
// for the life of the process: a host that destroys the device's primary context (cudaDeviceReset) and goes on must
// not call this entry again, the cached address would belong to the old context.
double* g_scratch_addr[kMaxDevices] = {};

__global__ void __launch_bounds__(256) noalloc_partial_kernel(const void* __restrict__ data, long n, int elt, double* __restrict__ partials) {
  const long b = (long)blockIdx.x * kNoAllocSpan;
  const long e = b + kNoAllocSpan < n ? b + kNoAllocSpan : n;
  double acc = 0.0;
  for (long i = b + threadIdx.x; i < e; i += 256)
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

__global__ void noalloc_fold_kernel(const double* __restrict__ partials, int nslots, double* __restrict__ out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < nslots; i++) t += partials[i];
    *out = t;
  }
}

}  // namespace

extern "C" int fortis_checksum_noalloc(const void* dev_data, long n, int elt, double* dev_out, void* stream) {
  if (!dev_data || !dev_out || n < 0 || (elt != 0 && elt != 1)) {
    std::fprintf(stderr, "fortis_checksum_noalloc: bad arguments\n");
    return -1;
  }
  if (n > (long)kNoAllocSlots * kNoAllocSpan) {
    std::fprintf(stderr, "fortis_checksum_noalloc: %ld elements exceed the fixed scratch (at most %ld); use fortis_checksum\n", n,
                 (long)kNoAllocSlots * kNoAllocSpan);
    return -2;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    std::fprintf(stderr, "fortis_checksum_noalloc: cannot identify the current device (%s)\n", cudaGetErrorString(e));
    return -3;
  }
  if (!g_scratch_addr[dev]) {
    // set-up, once per device: resolve the array's device address while that device is current
    double* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_partials);
    if (e != cudaSuccess || !p) {
      std::fprintf(stderr, "fortis_checksum_noalloc: cudaGetSymbolAddress failed (%s)\n", cudaGetErrorString(e));
      return -4;
    }
    g_scratch_addr[dev] = p;
  }
  double* scratch = g_scratch_addr[dev];
  cudaStream_t s = (cudaStream_t)stream;
  const int blocks = n == 0 ? 0 : (int)((n + kNoAllocSpan - 1) / kNoAllocSpan);
  if (blocks) noalloc_partial_kernel<<<blocks, 256, 0, s>>>(dev_data, n, elt, scratch);
  noalloc_fold_kernel<<<1, 32, 0, s>>>(scratch, blocks, dev_out);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    std::fprintf(stderr, "fortis_checksum_noalloc: launch failed (%s)\n", cudaGetErrorString(e));
    return -5;
  }
  return 0;
}
