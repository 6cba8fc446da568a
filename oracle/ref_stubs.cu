// Stand-ins for the three symbols the reference's generated gather.cu expects from the rest of a fortisc build
// (driver/fortis_gather_emit.py:14-15).  TEST INFRASTRUCTURE ONLY: linked with the reference's own
// mom6_zb/gather.cu into oracle/_ref/ so that GPU tests can run the reference's kernels as a second checker.
#include <cuda_runtime.h>
#include <stdio.h>

static cudaStream_t ref_stream = 0;
static float *ref_din = 0, *ref_dout = 0;
static const long REF_ROWS = 71040, REF_NIN = 27, REF_NOUT = 3;   // 15 planes x 4736 cells (mom6_zb/gather.cu:56)

extern "C" void* mgpuStreamCreate(void) {
  if (!ref_stream) cudaStreamCreate(&ref_stream);
  return (void*)ref_stream;
}
extern "C" void* fortis_model_input(void) {
  if (!ref_din) cudaMalloc(&ref_din, REF_ROWS * REF_NIN * sizeof(float));
  return ref_din;
}
extern "C" void* fortis_model_output(void) {
  if (!ref_dout) cudaMalloc(&ref_dout, REF_ROWS * REF_NOUT * sizeof(float));
  return ref_dout;
}
// test access to the two model-side buffers
extern "C" int ref_download_input(float* host) {
  cudaStreamSynchronize((cudaStream_t)mgpuStreamCreate());
  return (int)cudaMemcpy(host, fortis_model_input(), REF_ROWS * REF_NIN * sizeof(float), cudaMemcpyDeviceToHost);
}
extern "C" int ref_upload_output(const float* host) {
  return (int)cudaMemcpy(fortis_model_output(), host, REF_ROWS * REF_NOUT * sizeof(float), cudaMemcpyHostToDevice);
}
