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

#ifdef __cplusplus
}
#endif
#endif
