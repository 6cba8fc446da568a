// Device-side plan interpretation shared by every kernel: element loads / stores through an Access, and the
// typed postfix evaluator for lifted expressions.  Expression arithmetic uses the explicit round-to-nearest
// intrinsics so that the compiler can never contract a multiply and an add into an FMA; this is what keeps
// gather / scatter bit-exact with the reference's `-fmad=false` kernels (driver/fortisc.sh:136).
#pragma once
#include <cuda_runtime.h>

#include "fortis_plan.h"

namespace fortis {

struct IoPlanDev {
  int n;                         // model inputs (gather) / outputs (scatter)
  int nscalars;
  int nstores;
  int has_prog;
  int scalar_ids[kMaxScalars];
  Access scalars[kMaxScalars];
  ExprProg prog;
};

__device__ __forceinline__ double load_elem(const ArrayTable& T, const Access& a, long long off) {
  if (a.elt == 0) return (double)__ldg((const float*)T.base[a.array] + off);
  return __ldg((const double*)T.base[a.array] + off);
}

__device__ __forceinline__ void store_elem(const ArrayTable& T, const Access& a, long long off, double v) {
  if (a.elt == 0) ((float*)T.base[a.array])[off] = (float)v;
  else ((double*)T.base[a.array])[off] = v;
}

__device__ __forceinline__ void load_scalars(const IoPlanDev& P, const ArrayTable& T, long long ci, long long cj,
                                             long long kk, double* sc) {
  for (int s = 0; s < P.nscalars; s++)
    sc[P.scalar_ids[s]] = load_elem(T, P.scalars[s], access_offset(P.scalars[s], ci, cj, kk));
}

// tv in, tv out.  `q` selects the element of per-feature vectors (lift2d).  Values travel as double; a float value
// is exactly representable, so float operations round-trip through (float) casts without loss.
static __device__ __noinline__ double eval_prog(const ExprProg& P, double tv, const double* sc, const ArrayTable& T, int q) {
  double st[kMaxStack];
  int sp = 0;
  for (int k = 0; k < P.nops; k++) {
    const int a = P.arg[k];
    switch (P.op[k]) {
      case OP_TV: st[sp++] = tv; break;
      case OP_SCALAR: st[sp++] = sc[a]; break;
      case OP_CONST: st[sp++] = P.cst[a]; break;
      case OP_VEC:
        st[sp++] = P.tv_double ? __ldg((const double*)T.vec[a] + q) : (double)__ldg((const float*)T.vec[a] + q);
        break;
      case OP_ADD_F: sp--; st[sp - 1] = (double)__fadd_rn((float)st[sp - 1], (float)st[sp]); break;
      case OP_SUB_F: sp--; st[sp - 1] = (double)__fsub_rn((float)st[sp - 1], (float)st[sp]); break;
      case OP_MUL_F: sp--; st[sp - 1] = (double)__fmul_rn((float)st[sp - 1], (float)st[sp]); break;
      case OP_DIV_F: sp--; st[sp - 1] = (double)__fdiv_rn((float)st[sp - 1], (float)st[sp]); break;
      case OP_ADD_D: sp--; st[sp - 1] = __dadd_rn(st[sp - 1], st[sp]); break;
      case OP_SUB_D: sp--; st[sp - 1] = __dsub_rn(st[sp - 1], st[sp]); break;
      case OP_MUL_D: sp--; st[sp - 1] = __dmul_rn(st[sp - 1], st[sp]); break;
      case OP_DIV_D: sp--; st[sp - 1] = __ddiv_rn(st[sp - 1], st[sp]); break;
      case OP_NEG: st[sp - 1] = -st[sp - 1]; break;
      case OP_TO_F: st[sp - 1] = (double)(float)st[sp - 1]; break;
      case OP_SQRT_F: st[sp - 1] = (double)__fsqrt_rn((float)st[sp - 1]); break;
      case OP_EXP_F: st[sp - 1] = (double)expf((float)st[sp - 1]); break;
      case OP_LOG_F: st[sp - 1] = (double)logf((float)st[sp - 1]); break;
      case OP_TANH_F: st[sp - 1] = (double)tanhf((float)st[sp - 1]); break;
      case OP_MAX_F: sp--; st[sp - 1] = (double)fmaxf((float)st[sp - 1], (float)st[sp]); break;
      case OP_MIN_F: sp--; st[sp - 1] = (double)fminf((float)st[sp - 1], (float)st[sp]); break;
      case OP_END_EXPR: tv = st[--sp]; break;
    }
  }
  return tv;
}

// One model input: load the host element, narrow to float (`float tv = A[...]`) unless the plan keeps the host
// type, run the lifted expressions, narrow to the model's float.
__device__ __forceinline__ float gather_value(const IoPlanDev& P, const Access& a, const ArrayTable& T, int q,
                                              long long ci, long long cj, long long kk, const double* sc) {
  double v = load_elem(T, a, access_offset(a, ci, cj, kk));
  if (!P.has_prog) return (float)v;
  if (!P.prog.tv_double) v = (double)(float)v;
  return (float)eval_prog(P.prog, v, sc, T, q);
}

// One model output on its way to the host array: expressions in float (scatter.json) or in the host's type after
// widening (lift2d), then the store converts to the array's element type.
__device__ __forceinline__ double scatter_value(const IoPlanDev& P, const ArrayTable& T, int q, float y, const double* sc) {
  if (!P.has_prog) return (double)y;
  return eval_prog(P.prog, (double)y, sc, T, q);
}

__device__ __forceinline__ void row_to_pos(const RowGeom& g, long long row, long long* ci, long long* cj, long long* kk) {
  if (((unsigned long long)row | (unsigned long long)g.count | (unsigned long long)g.ni) >> 31 == 0) {
    // everything fits 32 bits (the usual case): four 32-bit divisions instead of four 64-bit ones
    const unsigned r = (unsigned)row, cnt = (unsigned)g.count, ni = (unsigned)g.ni;
    const unsigned k = r / cnt, col = r - k * cnt, j = col / ni;
    *kk = g.kk0 + k;
    *ci = col - j * ni;
    *cj = j;
    return;
  }
  const long long col = row % g.count;
  *kk = g.kk0 + row / g.count;
  *ci = col % g.ni;
  *cj = col / g.ni;
}

}  // namespace fortis
