/* fortis_b200: C ABI of the gather -> NN forward -> scatter step for B200 (sm_100a).
 *
 * The first block is the operator surface a fortisc-built executable links against; every entry keeps the
 * reference's name, argument meaning and error behaviour (messages on stderr, no status codes, nothing thrown).
 * The reference generates these entries per host with the descriptors baked in; this library reads the same
 * descriptors at run time (second block), so one prebuilt .so serves every host.
 *
 * Pointers named "host array" may be HOST pointers (staged over PCIe exactly as the reference does: pinned once,
 * H2D planes, D2H rectangles) or DEVICE pointers (used in place, nothing is copied).
 */
#ifndef FORTIS_B200_H
#define FORTIS_B200_H
#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------------------------------------------------------
 * 1. The reference's operator surface
 * ------------------------------------------------------------------------------------------------------------- */

/* Replaces the generated fortis_gather (driver/fortis_gather_emit.py:63-70; sample mom6_zb/gather.cu:50-57).
 * Arguments, as the descriptor dictates: [int a_v by value for every entry of gather.json "args", unless the
 * enclosing loop is k-distributed], then one pointer per entry of gather.json "arrays".  Stages the arrays and
 * marks the model input as "to be gathered"; the gather itself runs fused into the first layer of the next
 * mlp_forward_batched() (or as its own kernel when fusing is off or fortis_model_input() is used). */
void fortis_gather(long a0, ...);

/* Replaces the generated fortis_scatter (driver/fortis_gather_emit.py:84-97; mom6_zb/gather.cu:82-91).
 * Arguments: [int a_v by value per scatter.json "args" entry; a0 is the 1-based enclosing-loop index], then one
 * pointer per scatter.json "arrays" entry.  Applies the lifted expressions to the model outputs of that plane,
 * stores them, copies the visited rectangle back to host arrays and synchronises (device arrays: in place). */
void fortis_scatter(long a0, ...);

/* Replaces mlp_forward_batched of the generated shim (driver/fortis_shim.py:113, 115, 117-121): with a gather /
 * pack pending the arguments are ignored (the lifted and packed forms take none); otherwise (in, out) are whole
 * row-major (batch, n_in) / (batch, n_out) arrays. */
void mlp_forward_batched(void* in, void* out);

/* Replaces mlp_forward (driver/fortis_shim.py:122, 127-133): whole-array call; under a lift2d boundary `in` and
 * `out` are the host's own column-major arrays in their own element type, pinned once; with a batched loop
 * verdict it is the single-row entry. */
void mlp_forward(void* in, void* out);

/* driver/fortis_shim.py:82-93: upload the model input, run the step on the device (CUDA-graph replay from the
 * second call on when FORTIS_GRAPH is set), download the output. */
void mlp_upload(void* in);
void mlp_forward_dev(void);
void mlp_download(void* out);

/* driver/fortis_shim.py:103-106: copy one row into / out of the pinned batch buffers; col is 0-based. */
void fortis_pack(void* f, int col);
void fortis_unpack(void* o, int col);

/* driver/fortis_shim.py:109-110: borrowed device pointers to the model input (rows, n_in) and output
 * (rows, n_out).  Asking for the input makes a pending gather run as its own kernel so that the buffer is valid. */
void* fortis_model_input(void);
void* fortis_model_output(void);

/* Replaces the run-time-extent stub (driver/fortis_stub.c:12-31): sets the number of rows of the next steps.
 * Kernels take the extent as an argument, so nothing is specialised or loaded. */
void fortis_begin(int count);

/* runtime/fortis_rt.c:5-12: the one persistent stream; Destroy / Synchronize are no-ops as in the reference. */
void* mgpuStreamCreate(void);
void mgpuStreamDestroy(void* s);
void mgpuStreamSynchronize(void* s);
extern int fortis_capturing;

/* runtime/fortis_rt.c:14-40: device buffer pool (best fit among released buffers, release-all-and-retry under
 * pressure, returns 0 and prints on failure). */
void* fortis_alloc(long nbytes);
void fortis_free(void* p);

/* runtime/fortis_rt.c:45-48: C[B][N] = A[B][K] . W[N][K]^T on the persistent stream, memref ABI
 * (allocated, aligned, offset, sizes[2], strides[2]) per operand. */
void fortis_gemm(float* Aa, float* A, long Ao, long As0, long As1, long At0, long At1,
                 float* Wa, float* W, long Wo, long Ws0, long Ws1, long Wt0, long Wt1,
                 float* Ca, float* C, long Co, long Cs0, long Cs1, long Ct0, long Ct1, long B, long N, long K);

/* runtime/fortis_rt.c:128-131, runtime/fortis_fft.cu:131-135 and runtime/fortis_fft.cu:66-70: NCDHW fp32
 * cross-correlation with zero padding, memref ABI (allocated, aligned, offset, sizes[5], strides[5]) per operand, then
 * 18 longs.  Operands must be dense; a shape an entry does not take prints "<entry>: unsupported shape" on stderr and
 * leaves y untouched, as in the reference.
 *   fortis_conv3d         any kernel extent, stride and padding per axis (the reference's cuDNN lowering)
 *   fortis_conv3d_direct  stride 1, kernel extents up to 5 (the reference's direct kernels; here N > 1 is taken too)
 *   fortis_conv3d_fft     stride 1, no padding (the entry the compiler picks for kernels of 5^3 taps and more; the
 *                         result is computed directly in fp32, without a transform) */
void fortis_conv3d(float* xa, float* x, long xo, long x0, long x1, long x2, long x3, long x4, long xt0, long xt1, long xt2, long xt3, long xt4,
                   float* wa, float* w, long wo, long w0, long w1, long w2, long w3, long w4, long wt0, long wt1, long wt2, long wt3, long wt4,
                   float* ya, float* y, long yo, long y0, long y1, long y2, long y3, long y4, long yt0, long yt1, long yt2, long yt3, long yt4,
                   long N, long C, long Din, long Hin, long Win, long F, long KD, long KH, long KW, long Dout, long Hout, long Wout,
                   long sd, long sh, long sw, long pd, long ph, long pw);
void fortis_conv3d_direct(float* xa, float* x, long xo, long x0, long x1, long x2, long x3, long x4, long xt0, long xt1, long xt2, long xt3, long xt4,
                   float* wa, float* w, long wo, long w0, long w1, long w2, long w3, long w4, long wt0, long wt1, long wt2, long wt3, long wt4,
                   float* ya, float* y, long yo, long y0, long y1, long y2, long y3, long y4, long yt0, long yt1, long yt2, long yt3, long yt4,
                   long N, long C, long Din, long Hin, long Win, long F, long KD, long KH, long KW, long Dout, long Hout, long Wout,
                   long sd, long sh, long sw, long pd, long ph, long pw);

void fortis_conv3d_fft(float* xa, float* x, long xo, long x0, long x1, long x2, long x3, long x4, long xt0, long xt1, long xt2, long xt3, long xt4,
                   float* wa, float* w, long wo, long w0, long w1, long w2, long w3, long w4, long wt0, long wt1, long wt2, long wt3, long wt4,
                   float* ya, float* y, long yo, long y0, long y1, long y2, long y3, long y4, long yt0, long yt1, long yt2, long yt3, long yt4,
                   long N, long C, long Din, long Hin, long Win, long F, long KD, long KH, long KW, long Dout, long Hout, long Wout,
                   long sd, long sh, long sw, long pd, long ph, long pw);
/* runtime/fortis_rt.c:108-111: NCHW fp32 cross-correlation, memref ABI (allocated, aligned, offset, sizes[4],
 * strides[4]) per operand, then 13 longs; any kernel extent, stride and padding per axis. */
void fortis_conv2d(float* xa, float* x, long xo, long x0, long x1, long x2, long x3, long xt0, long xt1, long xt2, long xt3,
                   float* wa, float* w, long wo, long w0, long w1, long w2, long w3, long wt0, long wt1, long wt2, long wt3,
                   float* ya, float* y, long yo, long y0, long y1, long y2, long y3, long yt0, long yt1, long yt2, long yt3,
                   long N, long C, long Hin, long Win, long F, long KH, long KW, long Hout, long Wout, long sh, long sw, long ph, long pw);

/* ---------------------------------------------------------------------------------------------------------------
 * 2. Run-time configuration (what fortisc bakes in at build time)
 * ------------------------------------------------------------------------------------------------------------- */

/* key: "gather" | "scatter" | "loop" | "kdist" | "lift2d"; text: the JSON document.  Returns 0, or -1 with the
 * reason in fortis_last_error_message().  The files named by the environment variables FORTIS_GATHER_JSON,
 * FORTIS_SCATTER_JSON, FORTIS_LOOP_JSON, FORTIS_KDIST_JSON, FORTIS_LIFT2D_JSON and FORTIS_MODEL are loaded at the
 * first call of any step entry when nothing was configured. */
int fortis_configure(const char* key, const char* json_text);
int fortis_configure_file(const char* key, const char* path);
/* per-feature vectors a lift2d boundary names (the host's own globals in a fortisc build:
 * driver/fortis_boundary_trt.py:22-24).  elt: 0 = float, 1 = double, must match the side's element type. */
int fortis_set_vector(const char* name, const void* host_data, long n, int elt);
/* the model blob (layout in fortis_b200/csrc/fortis_model.h; written by fortis_b200.model.write_blob) */
int fortis_load_model(const char* path);
int fortis_load_model_mem(const void* blob, long nbytes);
/* options:
 *   "precision"   "fp32" (default; large layers run as three TF32 tensor-core products per fp32 product with IEEE
 *                 running sums, <= 1e-5) | "bf16" | "fp16" (16-bit operands, fp32 accumulation) | "fp8w" (FP8-E4M3
 *                 weights with per-channel scales, bf16 activations; MLP models only)
 *   "fuse"        "0" | "1"   one launch per step where the descriptors allow it (default 1)
 *   "graph"       "0" | "1"   replay a step as a CUDA graph from its second call (FORTIS_GRAPH)
 *   "async"       "0" | "1"   return from a step without waiting for the stream (fortis_sync() waits)
 *   "checksum"    "0" | "1"   accumulate the fp64 sum of everything a fused step scatters
 *   "host_access" "copy" (default: host arrays are staged by copies; column layouts in chunks, uploads, kernels and
 *                 downloads overlapped) | "mapped_out" (kernels store into the pinned host pages) | "mapped" (they
 *                 load from them as well); also FORTIS_HOST_ACCESS
 *   "stencil_tc"  "0" | "1"   3x3-stencil hosts with narrow MLPs: run the layers as TF32x3 tensor-core products instead
 *                 of packed FMAs (same <= 1e-5; measured slower for 27-20-20-3, default 0); also FORTIS_STENCIL_TC
 *   "tc_pair"     "1" (default) | "0" | "default"   wide MLPs in 16-bit / FP8-weight precision: run the fused
 *                 tensor-core kernel as clusters of two CTAs that share one stream of weights, or one CTA per SM (same
 *                 results bit for bit; the cluster form is 9-16 % faster); also FORTIS_TC_PAIR
 *   "conv_shape"  "N,D,H,W"   input extent of a conv3d model (NDHWC arrays); "N,1,H,W" for a network of 2-D operator
 *                 layers (Conv2d / transposed / pooling / upsampling; NCHW arrays in and out of mlp_forward)
 * The keys "test_wait_limit" and "test_skip_stage" exist for the tests of the bounded waits, "test_no_stage" for the test
 * of the staged input fetch (fortis_b200_test.h). */
int fortis_set_option(const char* key, const char* value);
/* drop every descriptor, model, buffer registration and captured graph (device pool buffers stay pooled) */
void fortis_reset(void);
int fortis_last_error(void);
const char* fortis_last_error_message(void);
void fortis_sync(void);

/* ---------------------------------------------------------------------------------------------------------------
 * 3. Fused and array-argument forms (no counterpart in the reference's generated code; they are what a maintainer
 *    would have the host rewriter, driver/fortis_fission_hlfir.py:76-109, emit instead of the three calls)
 * ------------------------------------------------------------------------------------------------------------- */

/* One launch for the whole step: gather -> forward -> scatter.  Arguments: [the gather entry's integer arguments,
 * by value, unless the enclosing loop is k-distributed], the gather entry's arrays, then the scatter entry's arrays.
 * A k-distributed loop processes all its planes; otherwise the integers select the plane as they do for
 * fortis_gather / fortis_scatter.  Refused (message, nothing run) when a stored array has no plane dimension while
 * nk > 1, because the host consumes such an array between the per-plane scatters, and when a plane-selecting
 * integer is missing.  When a device-resident gather array shares memory with a device-resident stored array the
 * step runs as separate gather, forward and scatter kernels, so that no input is read after it was overwritten. */
void fortis_step(long a0, ...);
/* the same three entries with arguments in arrays, for bindings that cannot call C variadics */
void fortis_gatherv(const int* iargs, int nint, const void* const* arrays, int narrays);
void fortis_scatterv(const int* iargs, int nint, void* const* arrays, int narrays);
void fortis_stepv(const void* const* gather_arrays, int ngather, void* const* scatter_arrays, int nscatter);
void fortis_stepvi(const int* iargs, int nint, const void* const* gather_arrays, int ngather, void* const* scatter_arrays,
                   int nscatter);

/* synchronous copies between host memory and buffers of this library (fortis_alloc, fortis_model_input/output);
 * the first waits for the persistent stream */
int fortis_copy_to_host(void* dst, const void* dev, long nbytes);
int fortis_copy_to_device(void* dev, const void* src, long nbytes);

/* fp64 sum of n elements (elt 0 = float, 1 = double) of a device or host array, summed in a fixed order */
int fortis_checksum(const void* data, long n, int elt, double* out);
/* No counterpart in the reference.  The same fp64 sum for callers that cannot allocate device memory: hosts that
 * give their whole GPU memory budget to pools sized at start-up, and code between latency-critical launches, where
 * cudaMalloc's device synchronisation would stall the step.  dev_data and dev_out are DEVICE pointers supplied by the
 * caller, `stream` is the caller's cudaStream_t (0 = default stream); the result is written to *dev_out in stream
 * order and nothing is synchronised.  The block partials live in a 32 KB array inside the library image, so n is
 * limited to 2^28 elements (return -2 and a message beyond that) and the call performs no cudaMalloc / cudaFree and
 * uses no pool.  The first call on each device resolves the array's device address (a set-up step: make that call
 * before any stream capture).  The address is remembered per device ordinal for the life of the process: a host that
 * destroys the device's primary context (cudaDeviceReset) must not call this entry afterwards.  All calls share the
 * array: calls that can overlap on the GPU race on it.  Returns 0, or a negative code with a message on stderr. */
int fortis_checksum_noalloc(const void* dev_data, long n, int elt, double* dev_out, void* stream);

/* fp64 sum of everything the fused steps scattered since the last call (needs option "checksum" = "1") */
int fortis_step_checksum(double* out);
/* device status word of the tensor-core kernel: 0, or the code of a bounded wait that gave up */
int fortis_device_status(void);

#ifdef __cplusplus
}
#endif
#endif
