// Descriptor -> plan.  Semantics follow the reference's emitter (driver/fortis_gather_emit.py:9-36, 52-62, 75-83)
// and its boundary generator (driver/fortis_boundary_trt.py:12-38); the expression grammar is the one
// driver/fortis_gather.py:92-120 produces.
#include "fortis_plan.h"

#include <cctype>
#include <cmath>
#include <cstring>
#include <stdexcept>

namespace fortis {

// ---------------------------------------------------------------------------------------------------------------
// expression compiler: C text -> typed postfix.  C's usual arithmetic conversions are applied per node: an
// operation is done in double iff one operand is double (an f64 array scalar or an unsuffixed literal); the
// *f functions always take and return float.
// ---------------------------------------------------------------------------------------------------------------
namespace {

struct ExprCompiler {
  const std::string& s;
  const std::vector<int>& scalar_elt;
  ExprProg* P;
  size_t p = 0;

  [[noreturn]] void fail(const std::string& what) const {
    throw std::runtime_error("expression \"" + s + "\": " + what);
  }
  void ws() { while (p < s.size() && std::isspace((unsigned char)s[p])) p++; }
  bool peek(char c) { ws(); return p < s.size() && s[p] == c; }
  void expect(char c) { if (!peek(c)) fail(std::string("expected '") + c + "'"); p++; }
  void emit(uint8_t op, int arg = 0) {
    if (P->nops >= kMaxOps) fail("program too long");
    P->op[P->nops] = op; P->arg[P->nops] = (int16_t)arg; P->nops++;
  }
  int add_const(double v) {
    for (int i = 0; i < kMaxConsts; i++) {
      // slot 0..n-1 in use are those referenced so far; find an equal one or the first never used
      bool used = false;
      for (int k = 0; k < P->nops; k++) if (P->op[k] == OP_CONST && P->arg[k] == i) used = true;
      if (used && std::memcmp(&P->cst[i], &v, sizeof v) == 0) return i;
      if (!used) { P->cst[i] = v; return i; }
    }
    fail("too many constants");
  }
  // each parse function returns true when the value's C type is double
  bool primary() {
    ws();
    if (p >= s.size()) fail("unexpected end");
    char c = s[p];
    if (c == '(') {
      p++;
      ws();
      if (p < s.size() && s[p] == '-') {           // "(-x)"
        size_t save = p; int save_n = P->nops;
        p++;
        bool d = expr();
        if (peek(')')) { p++; emit(OP_NEG); return d; }
        p = save; P->nops = save_n;
      }
      bool d = expr();
      expect(')');
      return d;
    }
    if (c == '-') { p++; bool d = primary(); emit(OP_NEG); return d; }
    if (std::isdigit((unsigned char)c) || c == '.') {
      size_t b = p;
      while (p < s.size() && (std::isdigit((unsigned char)s[p]) || s[p] == '.')) p++;
      if (p < s.size() && (s[p] == 'e' || s[p] == 'E')) {
        p++;
        if (p < s.size() && (s[p] == '+' || s[p] == '-')) p++;
        while (p < s.size() && std::isdigit((unsigned char)s[p])) p++;
      }
      std::string num = s.substr(b, p - b);
      bool is_f = p < s.size() && (s[p] == 'f' || s[p] == 'F');
      if (is_f) p++;
      double v = is_f ? (double)std::strtof(num.c_str(), nullptr) : std::strtod(num.c_str(), nullptr);
      emit(OP_CONST, add_const(v));
      return !is_f;
    }
    if (std::isalpha((unsigned char)c) || c == '_') {
      size_t b = p;
      while (p < s.size() && (std::isalnum((unsigned char)s[p]) || s[p] == '_')) p++;
      std::string id = s.substr(b, p - b);
      if (id == "tv") { emit(OP_TV); return P->tv_double != 0; }
      if (id.size() >= 2 && id[0] == 'S' && std::isdigit((unsigned char)id[1])) {
        int k = std::atoi(id.c_str() + 1);
        if (k < 0 || k >= (int)scalar_elt.size() || scalar_elt[k] < 0) fail("scalar " + id + " is not declared");
        emit(OP_SCALAR, k);
        return scalar_elt[k] == 1;
      }
      static const struct { const char* name; uint8_t op; int nargs; } F[] = {
          {"sqrtf", OP_SQRT_F, 1}, {"expf", OP_EXP_F, 1}, {"logf", OP_LOG_F, 1}, {"tanhf", OP_TANH_F, 1},
          {"fmaxf", OP_MAX_F, 2}, {"fminf", OP_MIN_F, 2}};
      for (auto& f : F)
        if (id == f.name) {
          expect('(');
          if (expr()) emit(OP_TO_F);
          if (f.nargs == 2) { expect(','); if (expr()) emit(OP_TO_F); }
          expect(')');
          emit(f.op);
          return false;
        }
      fail("unknown identifier " + id);
    }
    fail(std::string("unexpected '") + c + "'");
  }
  bool term() {
    bool d = primary();
    for (;;) {
      ws();
      if (p < s.size() && (s[p] == '*' || s[p] == '/')) {
        char o = s[p++];
        bool d2 = primary();
        d = d || d2;
        emit(o == '*' ? (d ? OP_MUL_D : OP_MUL_F) : (d ? OP_DIV_D : OP_DIV_F));
      } else {
        return d;
      }
    }
  }
  bool expr() {
    bool d = term();
    for (;;) {
      ws();
      if (p < s.size() && (s[p] == '+' || s[p] == '-')) {
        char o = s[p++];
        bool d2 = term();
        d = d || d2;
        emit(o == '+' ? (d ? OP_ADD_D : OP_ADD_F) : (d ? OP_SUB_D : OP_SUB_F));
      } else {
        return d;
      }
    }
  }
};

}  // namespace

void compile_expr(const std::string& text, const std::vector<int>& scalar_elt_by_id, ExprProg* prog) {
  ExprCompiler C{text, scalar_elt_by_id, prog};
  bool d = C.expr();
  C.ws();
  if (C.p != text.size()) C.fail("trailing input");
  if (d && !prog->tv_double) C.emit(OP_TO_F);
  C.emit(OP_END_EXPR);
}

double eval_prog_host(const ExprProg& P, double tv, const double* sc, const double* vecvals) {
  double st[kMaxStack];
  int sp = 0;
  for (int k = 0; k < P.nops; k++) {
    const int a = P.arg[k];
    switch (P.op[k]) {
      case OP_TV: st[sp++] = tv; break;
      case OP_SCALAR: st[sp++] = sc[a]; break;
      case OP_CONST: st[sp++] = P.cst[a]; break;
      case OP_VEC: st[sp++] = vecvals[a]; break;
      case OP_ADD_F: sp--; st[sp - 1] = (double)((float)st[sp - 1] + (float)st[sp]); break;
      case OP_SUB_F: sp--; st[sp - 1] = (double)((float)st[sp - 1] - (float)st[sp]); break;
      case OP_MUL_F: sp--; st[sp - 1] = (double)((float)st[sp - 1] * (float)st[sp]); break;
      case OP_DIV_F: sp--; st[sp - 1] = (double)((float)st[sp - 1] / (float)st[sp]); break;
      case OP_ADD_D: sp--; st[sp - 1] = st[sp - 1] + st[sp]; break;
      case OP_SUB_D: sp--; st[sp - 1] = st[sp - 1] - st[sp]; break;
      case OP_MUL_D: sp--; st[sp - 1] = st[sp - 1] * st[sp]; break;
      case OP_DIV_D: sp--; st[sp - 1] = st[sp - 1] / st[sp]; break;
      case OP_NEG: st[sp - 1] = -st[sp - 1]; break;
      case OP_TO_F: st[sp - 1] = (double)(float)st[sp - 1]; break;
      case OP_SQRT_F: st[sp - 1] = (double)std::sqrt((float)st[sp - 1]); break;
      case OP_EXP_F: st[sp - 1] = (double)std::exp((float)st[sp - 1]); break;
      case OP_LOG_F: st[sp - 1] = (double)std::log((float)st[sp - 1]); break;
      case OP_TANH_F: st[sp - 1] = (double)std::tanh((float)st[sp - 1]); break;
      // as the device computes them: +0 > -0 (PTX max.f32 / min.f32), where the host's fmax may return either zero
      case OP_MAX_F: {
        sp--;
        const float a = (float)st[sp - 1], b = (float)st[sp];
        st[sp - 1] = (a == 0.f && b == 0.f) ? ((std::signbit(a) && std::signbit(b)) ? -0.0 : 0.0) : (double)std::fmax(a, b);
        break;
      }
      case OP_MIN_F: {
        sp--;
        const float a = (float)st[sp - 1], b = (float)st[sp];
        st[sp - 1] = (a == 0.f && b == 0.f) ? ((std::signbit(a) || std::signbit(b)) ? -0.0 : 0.0) : (double)std::fmin(a, b);
        break;
      }
      case OP_END_EXPR: tv = st[--sp]; break;
    }
  }
  return tv;
}

// ---------------------------------------------------------------------------------------------------------------
// loop geometry  (driver/fortis_gather_emit.py:9-12)
// ---------------------------------------------------------------------------------------------------------------
LoopInfo make_loop(const JValue* loop, const JValue* kdist) {
  LoopInfo L;
  if (!loop) throw std::runtime_error("loop.json is not configured");
  if (kdist && kdist->find("ok") && kdist->at("ok").truthy()) {
    L.kdist = true;
    L.nk = (int)kdist->at("nk").as_long();
    L.klo = (int)kdist->at("loop").at("lo").as_long();
    if (L.nk <= 0) throw std::runtime_error("kdist.json: nk must be positive");
  }
  L.batch = loop->at("batch").as_long();
  L.count = L.batch / L.nk;
  const JValue& in = loop->at("inner");
  L.ilo = (int)in.at("lo").as_long();
  L.ni = (int)in.at("n").as_long();
  if (L.ni <= 0) throw std::runtime_error("loop.json: inner.n must be positive");
  const JValue* out = loop->find("outer");
  if (out && !out->is_null()) {
    L.has_outer = true;
    L.jlo = (int)out->at("lo").as_long();
    L.nj = (int)(L.count / L.ni);
  }
  return L;
}

// ---------------------------------------------------------------------------------------------------------------
// gather.json / scatter.json -> plan  (driver/fortis_gather_emit.py:16-36)
// ---------------------------------------------------------------------------------------------------------------
namespace {

int elt_code(const std::string& e) {
  if (e == "f32") return 0;
  if (e == "f64") return 1;
  throw std::runtime_error("descriptor: unsupported element type " + e);
}

Access make_access(const std::vector<ArrayInfo>& A, int ai, const JValue& idx, const LoopInfo& L) {
  if (ai < 0 || ai >= (int)A.size()) throw std::runtime_error("descriptor: array index out of range");
  const ArrayInfo& a = A[ai];
  if (idx.size() != a.shape.size()) throw std::runtime_error("descriptor: subscript rank differs from array rank (" + a.name + ")");
  Access x{};
  x.array = ai; x.elt = a.elt;
  for (size_t d = 0; d < idx.size(); d++) {
    const std::string& kind = idx.at(d).at(0).as_str();
    const long long v = idx.at(d).at(1).as_long(), st = a.strides[d];
    if (kind == "i") { x.off0 += (L.ilo + v - 1) * st; x.si += st; }
    else if (kind == "j") { x.off0 += (L.jlo + v - 1) * st; x.sj += st; }
    else if (kind == "c") { x.off0 += (v - 1) * st; }
    else if (kind == "v") { /* plane selector: call-time base or kk * plane */ }
    else throw std::runtime_error("descriptor: unknown subscript kind \"" + kind + "\"");
  }
  x.sk = a.vdims.empty() ? 0 : a.plane;
  return x;
}

}  // namespace

IoPlanHost make_io_plan(const JValue& J, const LoopInfo& L, bool is_scatter) {
  IoPlanHost P;
  P.is_scatter = is_scatter;
  if (!J.find("ok") || !J.at("ok").truthy()) return P;
  P.n = (int)J.at("n").as_long();
  P.nargs = J.find("args") ? (int)J.at("args").size() : 0;
  const JValue& arrs = J.at("arrays");
  if ((int)arrs.size() > kMaxArrays) throw std::runtime_error("descriptor: too many arrays");
  const char* use_key = is_scatter ? "stores" : "slots";
  for (size_t ai = 0; ai < arrs.size(); ai++) {
    ArrayInfo a;
    a.name = arrs.at(ai).find("name") ? arrs.at(ai).at("name").as_str() : std::string("array") + std::to_string(ai);
    a.elt = elt_code(arrs.at(ai).at("elt").as_str());
    for (size_t d = 0; d < arrs.at(ai).at("shape").size(); d++) a.shape.push_back(arrs.at(ai).at("shape").at(d).as_long());
    a.strides.push_back(1);
    for (size_t d = 0; d + 1 < a.shape.size(); d++) a.strides.push_back(a.strides.back() * a.shape[d]);
    // plane dims = the dims any use marks "v"; they must be exactly the trailing dims (emit :21-22)
    std::vector<bool> isv(a.shape.size(), false);
    const JValue* first_use = nullptr;
    auto scan = [&](const JValue& list) {
      for (size_t k = 0; k < list.size(); k++)
        if (list.at(k).at("array").as_long() == (long)ai) {
          const JValue& idx = list.at(k).at("idx");
          if (!first_use) first_use = &idx;
          for (size_t d = 0; d < idx.size() && d < isv.size(); d++)
            if (idx.at(d).at(0).as_str() == "v") isv[d] = true;
        }
    };
    scan(J.at(use_key));
    if (J.find("scalars")) scan(J.at("scalars"));
    a.used = first_use != nullptr;
    for (size_t d = 0; d < isv.size(); d++) if (isv[d]) a.vdims.push_back((int)d);
    for (size_t k = 0; k < a.vdims.size(); k++)
      if (a.vdims[k] != (int)(a.shape.size() - a.vdims.size() + k))
        throw std::runtime_error("descriptor: plane dims must be the trailing dims (" + a.name + ")");
    a.plane = 1;
    for (size_t d = 0; d + a.vdims.size() < a.shape.size(); d++) a.plane *= a.shape[d];
    a.total = a.plane;
    for (int v : a.vdims) a.total *= a.shape[v];
    if (first_use)
      for (size_t d = 0; d < first_use->size(); d++)
        if (first_use->at(d).at(0).as_str() == "v") a.vterms.emplace_back((int)first_use->at(d).at(1).as_long(), a.strides[d]);
    P.arrays.push_back(a);
  }
  // scalars
  std::vector<int> scalar_elt(kMaxScalars, -1);
  if (J.find("scalars")) {
    const JValue& sc = J.at("scalars");
    if ((int)sc.size() > kMaxScalars) throw std::runtime_error("descriptor: too many scalars");
    for (size_t k = 0; k < sc.size(); k++) {
      const std::string& nm = sc.at(k).at("name").as_str();
      if (nm.size() < 2 || nm[0] != 'S') throw std::runtime_error("descriptor: scalar name must be S<k>");
      int id = std::atoi(nm.c_str() + 1);
      if (id < 0 || id >= kMaxScalars) throw std::runtime_error("descriptor: scalar id out of range");
      Access x = make_access(P.arrays, (int)sc.at(k).at("array").as_long(), sc.at(k).at("idx"), L);
      P.scalars.push_back(x);
      P.scalar_ids.push_back(id);
      scalar_elt[id] = x.elt;
    }
  }
  // expressions, applied in list order to every slot / output
  P.prog.nops = 0;
  P.prog.tv_double = 0;
  if (J.find("exprs"))
    for (size_t k = 0; k < J.at("exprs").size(); k++) compile_expr(J.at("exprs").at(k).as_str(), scalar_elt, &P.prog);
  if (!is_scatter) {
    const JValue& sl = J.at("slots");
    if ((int)sl.size() != P.n) throw std::runtime_error("gather.json: len(slots) != n");
    for (size_t q = 0; q < sl.size(); q++)
      P.slots.push_back(make_access(P.arrays, (int)sl.at(q).at("array").as_long(), sl.at(q).at("idx"), L));
  } else {
    const JValue& st = J.at("stores");
    P.written.assign(P.arrays.size(), false);
    for (size_t q = 0; q < st.size(); q++) {
      StoreTarget t{};
      t.a = make_access(P.arrays, (int)st.at(q).at("array").as_long(), st.at(q).at("idx"), L);
      t.slot = (int)st.at(q).at("slot").as_long();
      if (t.slot < 0 || t.slot >= P.n) throw std::runtime_error("scatter.json: store slot out of range");
      P.stores.push_back(t);
      P.written[t.a.array] = true;
    }
  }
  P.ok = true;
  return P;
}

// ---------------------------------------------------------------------------------------------------------------
// lift2d.json (whole-array boundary): host array A(NI, NK) column-major, model input x[i, k] = pre(A[i + NI*k]);
// model output y[i, k] -> B[i + NI*k] = post(y)            (driver/fortis_boundary_trt.py:12-38)
// ---------------------------------------------------------------------------------------------------------------
namespace {

void compile_tree(const JValue& e, int host_elt, IoPlanHost* P) {
  ExprProg* G = &P->prog;
  auto emit = [&](uint8_t op, int arg = 0) {
    if (G->nops >= kMaxOps) throw std::runtime_error("lift2d: expression too long");
    G->op[G->nops] = op; G->arg[G->nops] = (int16_t)arg; G->nops++;
  };
  const std::string& k = e.at(0).as_str();
  if (k == "A") { emit(OP_TV); return; }
  if (k == "V") {
    const std::string& nm = e.at(1).as_str();
    int id = -1;
    for (size_t i = 0; i < P->vec_names.size(); i++) if (P->vec_names[i] == nm) id = (int)i;
    if (id < 0) {
      if ((int)P->vec_names.size() >= kMaxVecs) throw std::runtime_error("lift2d: too many vectors");
      id = (int)P->vec_names.size();
      P->vec_names.push_back(nm);
    }
    emit(OP_VEC, id);
    return;
  }
  if (k == "C") {
    const JValue& c = e.at(1);
    double v = c.kind == JValue::Num ? c.num : std::strtod(c.as_str().c_str(), nullptr);
    if (host_elt == 0) v = (double)(float)v;
    int slot = -1;
    for (int i = 0; i < kMaxConsts && slot < 0; i++) {
      bool used = false;
      for (int t = 0; t < G->nops; t++) if (G->op[t] == OP_CONST && G->arg[t] == i) used = true;
      if (!used) { G->cst[i] = v; slot = i; }
      else if (std::memcmp(&G->cst[i], &v, sizeof v) == 0) slot = i;
    }
    if (slot < 0) throw std::runtime_error("lift2d: too many constants");
    emit(OP_CONST, slot);
    return;
  }
  compile_tree(e.at(1), host_elt, P);
  compile_tree(e.at(2), host_elt, P);
  const bool d = host_elt == 1;
  if (k == "arith.addf") emit(d ? OP_ADD_D : OP_ADD_F);
  else if (k == "arith.subf") emit(d ? OP_SUB_D : OP_SUB_F);
  else if (k == "arith.mulf") emit(d ? OP_MUL_D : OP_MUL_F);
  else if (k == "arith.divf") emit(d ? OP_DIV_D : OP_DIV_F);
  else throw std::runtime_error("lift2d: unsupported operation " + k);
}

}  // namespace

void make_lift2d_plans(const JValue& J, IoPlanHost* pre, IoPlanHost* post, LoopInfo* L) {
  const JValue& lin = J.at("layout").at("in");
  const JValue& lout = J.at("layout").at("out");
  const long long NI = lin.at("from_shape").at(0).as_long(), NK = lin.at("from_shape").at(1).as_long();
  const long long NO = lout.at("to_shape").at(1).as_long();
  if (lout.at("to_shape").at(0).as_long() != NI) throw std::runtime_error("lift2d: input and output column counts differ");
  *L = LoopInfo{};
  L->batch = L->count = NI; L->ilo = 1; L->ni = (int)NI; L->nk = 1;
  auto build = [&](IoPlanHost* P, bool scatter, long long nfeat, const std::string& elt, const JValue* side) {
    *P = IoPlanHost{};
    P->is_scatter = scatter; P->n = (int)nfeat; P->nargs = 0;
    ArrayInfo a; a.name = scatter ? "out" : "in"; a.elt = elt_code(elt);
    a.shape = {NI, nfeat}; a.strides = {1, NI}; a.plane = a.total = NI * nfeat; a.used = true;
    P->arrays.push_back(a);
    P->prog.nops = 0; P->prog.tv_double = a.elt;
    if (side && !side->is_null() && side->find("expr")) { compile_tree(side->at("expr"), a.elt, P);
      if (P->prog.nops >= kMaxOps) throw std::runtime_error("lift2d: expression too long");
      P->prog.op[P->prog.nops] = OP_END_EXPR; P->prog.arg[P->prog.nops] = 0; P->prog.nops++; }
    for (long long k = 0; k < nfeat; k++) {
      Access x{}; x.array = 0; x.elt = a.elt; x.off0 = k * NI; x.si = 1;
      if (!scatter) P->slots.push_back(x);
      else { StoreTarget t{}; t.a = x; t.slot = (int)k; P->stores.push_back(t); }
    }
    if (scatter) P->written.assign(1, true);
    P->ok = true;
  };
  build(pre, false, NK, lin.at("from_elt").as_str(), J.find("pre"));
  build(post, true, NO, lout.at("to_elt").as_str(), J.find("post"));
}

}  // namespace fortis
