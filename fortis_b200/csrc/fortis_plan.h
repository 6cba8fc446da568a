// Layout plans: the run-time form of gather.json / scatter.json / loop.json / kdist.json / lift2d.json.
//
// The reference bakes these descriptors into generated CUDA text at build time (driver/fortis_gather_emit.py).
// Here they are parsed once into a small plan that every kernel (standalone gather / scatter and the fused
// gather->forward->scatter kernels) interprets: per input slot an element offset that is affine in the column
// position, per output a store target, plus a typed postfix program for the lifted expressions.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "fortis_json.h"

namespace fortis {

constexpr int kMaxArrays = 24;    // host arrays named by one descriptor
constexpr int kMaxScalars = 8;    // S0..S7
constexpr int kMaxOps = 160;      // postfix program length (all expressions of one descriptor)
constexpr int kMaxConsts = 32;
constexpr int kMaxVecs = 8;       // per-feature vectors of a lift2d boundary (mean, max, min, scale ...)
constexpr int kMaxStack = 12;

enum ExprOp : uint8_t {
  OP_TV = 0, OP_SCALAR, OP_CONST, OP_VEC,
  OP_ADD_F, OP_SUB_F, OP_MUL_F, OP_DIV_F,       // float operands, one IEEE rounding, never contracted
  OP_ADD_D, OP_SUB_D, OP_MUL_D, OP_DIV_D,       // double operands
  OP_NEG, OP_TO_F,                              // negation is exact in either type; TO_F narrows double -> float
  OP_SQRT_F, OP_EXP_F, OP_LOG_F, OP_TANH_F, OP_MAX_F, OP_MIN_F,
  OP_END_EXPR                                   // tv = top of stack (narrowed to float unless tv_double)
};

struct ExprProg {
  int nops;
  int tv_double;                 // 1: tv keeps the host's f64 (lift2d boundary); 0: tv is float (gather/scatter.json)
  uint8_t op[kMaxOps];
  int16_t arg[kMaxOps];
  double cst[kMaxConsts];
};

// Element offset of one access for column position (ci, cj) in plane kk:  off0 + ci*si + cj*sj + kk*sk  (elements)
struct Access {
  int array;                     // index into ArrayTable::base
  int elt;                       // 0 = f32, 1 = f64
  long long off0, si, sj, sk;
};

struct StoreTarget {
  Access a;
  int slot;                      // which model output goes there
  int pad;
};

// Call-time operands (kernel parameter, passed by value): effective base pointer of every array for this call.
struct ArrayTable {
  void* base[kMaxArrays];
  const void* vec[kMaxVecs];
};

struct RowGeom {
  long long count;               // columns per plane
  int nk;                        // planes handled by this launch
  int ni;                        // inner-loop extent: ci = col % ni, cj = col / ni
  int kk0;                       // first plane (row r of the launch is plane kk0 + r / count)
};

#ifndef __CUDACC__
#define FORTIS_HD
#else
#define FORTIS_HD __host__ __device__
#endif

FORTIS_HD inline long long access_offset(const Access& a, long long ci, long long cj, long long kk) {
  return a.off0 + ci * a.si + cj * a.sj + kk * a.sk;
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
struct ArrayInfo {
  std::string name;
  int elt = 0;                       // 0 f32, 1 f64
  std::vector<long long> shape, strides;
  std::vector<int> vdims;            // trailing plane-selector dims
  std::vector<std::pair<int, long long>> vterms;   // (argument index, stride) for plane selection by argument
  long long plane = 1, total = 1;
  bool used = false;
};

struct LoopInfo {
  long long batch = 0, count = 0;
  int ilo = 1, ni = 1, jlo = 0, nj = 1, nk = 1, klo = 1;
  bool kdist = false, has_outer = false;
};

struct IoPlanHost {
  bool ok = false;
  bool is_scatter = false;
  int n = 0;                         // model inputs (gather) or outputs (scatter)
  int nargs = 0;                     // leading by-value integer arguments of the entry point
  std::vector<ArrayInfo> arrays;
  std::vector<Access> slots;         // gather: one per model input
  std::vector<StoreTarget> stores;   // scatter
  std::vector<Access> scalars;       // S0..
  std::vector<int> scalar_ids;       // the k of S<k> for scalars[i]
  ExprProg prog{};
  std::vector<std::string> vec_names;  // lift2d per-feature vectors referenced by the program
  std::vector<bool> written;         // scatter: array is a store target (not uploaded)
};

LoopInfo make_loop(const JValue* loop, const JValue* kdist);
IoPlanHost make_io_plan(const JValue& J, const LoopInfo& L, bool is_scatter);
// lift2d.json -> the same plan form: one (NI, NK) host array read transposed, per-feature vectors, host-typed tv
void make_lift2d_plans(const JValue& J, IoPlanHost* pre, IoPlanHost* post, LoopInfo* L);
// compile one C-syntax expression string and append it to `prog` (throws on unknown syntax)
void compile_expr(const std::string& text, const std::vector<int>& scalar_elt_by_id, ExprProg* prog);
// host-side evaluation of a compiled program (used by unit tests of the compiler through the C ABI)
double eval_prog_host(const ExprProg& P, double tv, const double* scalars, const double* vecvals);

}  // namespace fortis
