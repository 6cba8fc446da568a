/* fortis_b200: test-only entries of libfortis_b200.so.  Not part of the operator surface: nothing a host program
 * links against is declared here. */
#ifndef FORTIS_B200_TEST_H
#define FORTIS_B200_TEST_H
#ifdef __cplusplus
extern "C" {
#endif

/* Host-only introspection of the expression compiler and the descriptor planner (no CUDA call is made):
 * evaluate the expression list `exprs_json` (a JSON array of strings) on one value; list the element offsets one
 * row touches.  Used by the CPU test-suite; no counterpart in the reference. */
int fortis_debug_eval_expr(const char* exprs_json, int tv_double, double tv, const double* scalars, const int* scalar_elt,
                           int nscalars, double* out);
int fortis_debug_plan(const char* desc_json, const char* loop_json, const char* kdist_json, int is_scatter, long row,
                      const int* args, int nargs, long long* offsets, int* arrays, int* slots, int cap, long long* geom);

/* Host-only: one Linear layer (W (cout, cin) row-major fp32, b) converted as the tensor-core kernel wants it for
 * `precision` (1 = bf16, 2 = FP8-E4M3 weights, 3 = fp16): the padded extents in *K / *N and, into the buffers that are
 * not null, the stage images (N x K 16-bit values), the padded bias and the per-channel scales.  `last` != 0 pads the
 * output width to 64 instead of 256.  Call once with null buffers to learn K and N.  Used to check that the exporter's
 * pre-packed blobs (fortis_b200.model.write_blob(prepack=...)) are bit-identical to what the loader would compute. */
int fortis_debug_pack_layer(const float* W, const float* b, int cout, int cin, int last, int precision, unsigned short* image,
                            float* bias, float* scale, int* K, int* N);

/* Test-only keys of fortis_set_option (cleared by fortis_reset):
 *   "test_wait_limit"  N      polls before a bounded barrier wait of the tensor-core kernels gives up (0: the default)
 *   "test_skip_stage"  0 | 1  the first CTA's copy warp leaves out its first stage, so that a wait runs out: the
 *                             kernel returns, fortis_device_status() reports which wait gave up
 *   "test_no_stage"    0 | 1  fused MLP kernel: fetch every tile's inputs and store its outputs element by element
 *                             instead of staging whole tiles by bulk copies (same bits; for the comparison of the paths) */

#ifdef __cplusplus
}
#endif
#endif
