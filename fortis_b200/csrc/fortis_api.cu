// The C ABI (include/fortis_b200.h): process-wide session state, run-time configuration, host-array staging, the
// step driver (which kernels run for which model / precision / fusion mode) and CUDA-graph replay.
//
// Mirrors, entry by entry, the generated shim (driver/fortis_shim.py:61-133), the generated gather/scatter host
// entries (driver/fortis_gather_emit.py:37-48, 63-70, 84-97), the run-time-extent stub (driver/fortis_stub.c) and
// the runtime (runtime/fortis_rt.c:5-75).  Like the reference it is single-threaded by contract: one host thread,
// file-scope state, one stream.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/fortis_b200.h"
#include "../../include/fortis_b200_test.h"
#include "fortis_device.cuh"
#include "fortis_kernels.h"
#include "fortis_model.h"
#include "fortis_plan.h"

using namespace fortis;

int fortis_capturing = 0;

namespace {

// ---------------------------------------------------------------------------------------------------------------
// errors: the reference prints and carries on; so do we, and additionally keep the last message
// ---------------------------------------------------------------------------------------------------------------
int g_err = 0;
std::string g_errmsg;
void set_error(const std::string& msg) {
  g_err = -1;
  g_errmsg = msg;
  std::fprintf(stderr, "fortis: %s\n", msg.c_str());
}
bool cuda_ok(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  set_error(std::string(what) + ": " + cudaGetErrorString(e));
  return false;
}

// ---------------------------------------------------------------------------------------------------------------
// stream and pool  (runtime/fortis_rt.c:5-40)
// ---------------------------------------------------------------------------------------------------------------
cudaStream_t g_stream = nullptr;
cudaStream_t stream() {
  if (!g_stream) cuda_ok(cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking), "cudaStreamCreate");
  return g_stream;
}

// Copy streams of the overlapped staging path: column chunks travel host -> device on one, device -> host on the other,
// while the step kernels run on the persistent stream.
constexpr int kMaxChunks = 16;
cudaStream_t g_h2d = nullptr, g_d2h = nullptr;
cudaEvent_t g_ev_in[kMaxChunks] = {}, g_ev_k[kMaxChunks] = {}, g_ev_fork = nullptr, g_ev_join_in = nullptr, g_ev_join_out = nullptr;
bool ensure_copy_streams() {
  if (g_h2d) return true;
  if (cudaStreamCreateWithFlags(&g_h2d, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&g_d2h, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); g_h2d = g_d2h = nullptr; return false; }
  for (int i = 0; i < kMaxChunks; i++) {
    cudaEventCreateWithFlags(&g_ev_in[i], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&g_ev_k[i], cudaEventDisableTiming);
  }
  cudaEventCreateWithFlags(&g_ev_fork, cudaEventDisableTiming);
  cudaEventCreateWithFlags(&g_ev_join_in, cudaEventDisableTiming);
  cudaEventCreateWithFlags(&g_ev_join_out, cudaEventDisableTiming);
  return true;
}

// The policy restates runtime/fortis_rt.c:14-40 (it IS the contract of fortis_alloc / fortis_free): 256 slots, best
// fit among released buffers, cudaMalloc on a miss, release every unused buffer and retry once, 0 + message on failure.
constexpr int kPool = 256;
struct PoolSlot { long n; void* p; int used; } g_pool[kPool];

void* pool_alloc(long n) {
  if (n <= 0) n = 1;
  int best = -1;
  for (int i = 0; i < kPool; i++)
    if (g_pool[i].p && !g_pool[i].used && g_pool[i].n >= n && (best < 0 || g_pool[i].n < g_pool[best].n)) best = i;
  if (best >= 0) { g_pool[best].used = 1; return g_pool[best].p; }
  for (int attempt = 0; attempt < 2; attempt++) {
    for (int i = 0; i < kPool; i++)
      if (!g_pool[i].p) {
        if (cudaMalloc(&g_pool[i].p, (size_t)n) == cudaSuccess) { g_pool[i].n = n; g_pool[i].used = 1; return g_pool[i].p; }
        g_pool[i].p = nullptr;
        break;
      }
    cudaGetLastError();
    for (int i = 0; i < kPool; i++)
      if (g_pool[i].p && !g_pool[i].used) { cudaFree(g_pool[i].p); g_pool[i].p = nullptr; g_pool[i].n = 0; }
  }
  std::fprintf(stderr, "fortis_alloc: cudaMalloc(%ld) failed\n", n);
  return nullptr;
}
void pool_free(void* p) {
  if (!p) return;
  for (int i = 0; i < kPool; i++) if (g_pool[i].p == p) { g_pool[i].used = 0; return; }
  cudaFree(p);
}

// ---------------------------------------------------------------------------------------------------------------
// session
// ---------------------------------------------------------------------------------------------------------------
struct PlanDev {
  IoPlanHost h;
  IoPlanDev* hdr = nullptr;
  void* items = nullptr;                     // Access[n] (gather) or StoreTarget[nstores] (scatter)
  std::vector<void*> stage;                  // device staging buffer per array (host-resident arrays only)
  std::vector<long long> stage_elems;
  std::vector<const void*> reg;              // pinned registration: nullptr = none yet, (void*)1 = never again
  std::vector<const void*> cur;              // this call's pointers
  std::vector<char> on_dev;
  void* vec_dev[kMaxVecs] = {};
  int *slot_head = nullptr, *store_next = nullptr;   // scatter: stores indexed by model output
  Access* store_by_slot = nullptr;                   // scatter: one store target per model output (fast path)
  bool fast = false;                                 // fp32 only, no expressions / scalars, <= 2 stride classes
  long long cls[2][3] = {{0, 0, 0}, {0, 0, 0}};
};

struct Session {
  JValue jg, js, jl, jk, jl2;
  bool have_g = false, have_s = false, have_l = false, have_k = false, have_l2 = false;
  bool planned = false, env_loaded = false;
  LoopInfo loop;
  PlanDev G, S;
  std::map<std::string, std::pair<std::vector<char>, int>> vectors;   // name -> (bytes, elt)

  bool have_model = false, model_on_dev = false;
  ModelHost model;
  std::vector<float*> dW, dB;
  float *d_in_div = nullptr, *d_out_mul = nullptr, *d_relu_mask = nullptr;
  bool small_ok = false, stencil_ok = false;
  TcModel* tc = nullptr;
  F32TcModel* f32 = nullptr;                   // fp32 precision on the tensor cores (split TF32), large batches
  ConvModel* conv = nullptr;
  OpNet* opnet = nullptr;
  StencilTcModel* stencil_tc = nullptr;
  bool use_stencil_tc = false;                // option "stencil_tc" / FORTIS_STENCIL_TC
  int conv_shape[4] = {0, 0, 0, 0};

  int precision = PREC_F32;
  bool fuse = true, graph = false, async = false, want_checksum = false;
  long long begin_count = -1;

  long long buf_rows = 0;
  float *din = nullptr, *dout = nullptr, *act0 = nullptr, *act1 = nullptr;
  float *X_pinned = nullptr, *Y_pinned = nullptr;
  long long pinned_rows = 0;
  bool pack_pending = false, gather_pending = false, gather_done = false;
  int gather_args[8] = {};
  const void *reg_in = nullptr, *reg_out = nullptr;
  bool nopin = false;
  int host_access = 0;                        // host arrays of a step: 0 staged by copies, 1 outputs written by the kernels
                                              // into the mapped host pages, 2 inputs read from them as well

  double *d_partials = nullptr, *d_sum = nullptr;
  unsigned int* d_done = nullptr;             // CTA completion counter of the in-kernel checksum fold
  int* d_status = nullptr;
  long long partials_cap = 0;

  cudaGraphExec_t gexec = nullptr;
  std::string gkey;
  int ncalls = 0;
  cudaGraphExec_t ov_gexec = nullptr;        // the chunked staging pipeline of a step over host arrays, as one graph
  std::string ov_key;
  int ov_calls = 0;
};
Session* g_S = nullptr;
Session& S() {
  if (!g_S) {
    g_S = new Session();
    // option environment variables apply however the descriptors and the model arrive
    if (std::getenv("FORTIS_GRAPH")) g_S->graph = true;                              // driver/fortis_shim.py:84
    if (std::getenv("FORTIS_STENCIL_TC")) g_S->use_stencil_tc = true;
    if (const char* m = std::getenv("FORTIS_HOST_ACCESS")) {
      const std::string v(m);
      g_S->host_access = v == "mapped" ? 2 : v == "mapped_out" ? 1 : 0;
    }
  }
  return *g_S;
}

std::string read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

void free_plan(PlanDev& P) {
  for (size_t i = 0; i < P.reg.size(); i++)
    if (P.reg[i] && P.reg[i] != (const void*)1) { cudaHostUnregister((void*)P.reg[i]); cudaGetLastError(); }
  for (void* p : P.stage) pool_free(p);
  for (void*& v : P.vec_dev) { pool_free(v); v = nullptr; }
  pool_free(P.hdr); pool_free(P.items); pool_free(P.slot_head); pool_free(P.store_next); pool_free(P.store_by_slot);
  P = PlanDev();
}

void drop_graph() {
  Session& s = S();
  if (s.gexec) { cudaGraphExecDestroy(s.gexec); s.gexec = nullptr; }
  s.gkey.clear();
  s.ncalls = 0;
  if (s.ov_gexec) { cudaGraphExecDestroy(s.ov_gexec); s.ov_gexec = nullptr; }
  s.ov_key.clear();
  s.ov_calls = 0;
}

void free_model_dev() {
  Session& s = S();
  for (float* p : s.dW) pool_free(p);
  for (float* p : s.dB) pool_free(p);
  s.dW.clear(); s.dB.clear();
  pool_free(s.d_in_div); pool_free(s.d_out_mul); pool_free(s.d_relu_mask);
  s.d_in_div = s.d_out_mul = s.d_relu_mask = nullptr;
  if (s.tc) { tc_model_destroy(s.tc); s.tc = nullptr; }
  if (s.f32) { f32tc_destroy(s.f32); s.f32 = nullptr; }
  if (s.conv) { conv_model_destroy(s.conv); s.conv = nullptr; }
  if (s.opnet) { opnet_destroy(s.opnet); s.opnet = nullptr; }
  if (s.stencil_tc) { stencil_tc_destroy(s.stencil_tc); s.stencil_tc = nullptr; }
  s.model_on_dev = false;
  s.small_ok = false; s.stencil_ok = false;
}

void upload_plan(PlanDev& P) {
  IoPlanDev hd;
  std::memset(&hd, 0, sizeof hd);
  hd.n = P.h.n;
  hd.nscalars = (int)P.h.scalars.size();
  hd.nstores = (int)P.h.stores.size();
  hd.has_prog = P.h.prog.nops > 0;
  for (size_t i = 0; i < P.h.scalars.size(); i++) { hd.scalars[i] = P.h.scalars[i]; hd.scalar_ids[i] = P.h.scalar_ids[i]; }
  hd.prog = P.h.prog;
  P.hdr = (IoPlanDev*)pool_alloc(sizeof hd);
  if (!P.hdr) throw std::runtime_error("out of device memory for a layout plan");
  cudaMemcpy(P.hdr, &hd, sizeof hd, cudaMemcpyHostToDevice);
  if (!P.h.is_scatter) {
    const size_t nb = sizeof(Access) * P.h.slots.size();
    P.items = pool_alloc((long)nb);
    if (nb) cudaMemcpy(P.items, P.h.slots.data(), nb, cudaMemcpyHostToDevice);
  } else {
    const size_t nb = sizeof(StoreTarget) * P.h.stores.size();
    P.items = pool_alloc((long)nb);
    if (nb) cudaMemcpy(P.items, P.h.stores.data(), nb, cudaMemcpyHostToDevice);
    std::vector<int> head(P.h.n > 0 ? P.h.n : 1, -1), next(P.h.stores.size() ? P.h.stores.size() : 1, -1);
    for (int q = (int)P.h.stores.size() - 1; q >= 0; q--) { next[q] = head[P.h.stores[q].slot]; head[P.h.stores[q].slot] = q; }
    P.slot_head = (int*)pool_alloc((long)(head.size() * 4));
    P.store_next = (int*)pool_alloc((long)(next.size() * 4));
    cudaMemcpy(P.slot_head, head.data(), head.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(P.store_next, next.data(), next.size() * 4, cudaMemcpyHostToDevice);
  }
  // fast-path eligibility and stride classes
  {
    std::vector<Access> acc;
    if (!P.h.is_scatter) acc = P.h.slots; else for (auto& t : P.h.stores) acc.push_back(t.a);
    bool ok = P.h.prog.nops == 0 && P.h.scalars.empty() && !acc.empty() && P.h.arrays.size() < 0x7F;
    int ncls = 0;
    for (auto& a : acc) {
      if (a.elt != 0 || a.off0 < 0 || a.off0 >= (1LL << 32)) { ok = false; break; }
      int c = -1;
      for (int i = 0; i < ncls; i++) if (P.cls[i][0] == a.si && P.cls[i][1] == a.sj && P.cls[i][2] == a.sk) c = i;
      if (c < 0) { if (ncls == 2) { ok = false; break; } P.cls[ncls][0] = a.si; P.cls[ncls][1] = a.sj; P.cls[ncls][2] = a.sk; ncls++; }
    }
    if (P.h.is_scatter && ok) {
      std::vector<Access> by(P.h.n > 0 ? P.h.n : 1);
      for (auto& b : by) { std::memset(&b, 0, sizeof b); b.array = -1; }
      for (auto& t : P.h.stores) { if (by[t.slot].array >= 0) ok = false; by[t.slot] = t.a; }
      P.store_by_slot = (Access*)pool_alloc((long)(by.size() * sizeof(Access)));
      cudaMemcpy(P.store_by_slot, by.data(), by.size() * sizeof(Access), cudaMemcpyHostToDevice);
    }
    P.fast = ok;
  }
  const size_t na = P.h.arrays.size();
  P.stage.assign(na, nullptr); P.stage_elems.assign(na, 0); P.reg.assign(na, nullptr); P.cur.assign(na, nullptr);
  P.on_dev.assign(na, 0);
}

void load_env_config() {
  Session& s = S();
  if (s.env_loaded) return;
  s.env_loaded = true;
  const struct { const char* env; const char* key; } E[] = {{"FORTIS_GATHER_JSON", "gather"}, {"FORTIS_SCATTER_JSON", "scatter"},
      {"FORTIS_LOOP_JSON", "loop"}, {"FORTIS_KDIST_JSON", "kdist"}, {"FORTIS_LIFT2D_JSON", "lift2d"}};
  for (auto& e : E) {
    const char* v = std::getenv(e.env);
    if (v && *v) fortis_configure_file(e.key, v);
  }
  if (!s.have_model) { const char* m = std::getenv("FORTIS_MODEL"); if (m && *m) fortis_load_model(m); }
  if (const char* p = std::getenv("FORTIS_PRECISION")) fortis_set_option("precision", p);
  if (const char* b = std::getenv("FORTIS_BATCH")) if (s.begin_count < 0) s.begin_count = std::atoll(b);
}

void ensure_plans() {
  Session& s = S();
  if (!s.have_g && !s.have_s && !s.have_l && !s.have_l2) load_env_config();
  if (s.planned) return;
  free_plan(s.G); free_plan(s.S);
  if (s.have_l2) {
    make_lift2d_plans(s.jl2, &s.G.h, &s.S.h, &s.loop);
  } else {
    if (s.have_l) s.loop = make_loop(&s.jl, s.have_k ? &s.jk : nullptr);
    if (s.have_g) { if (!s.have_l) throw std::runtime_error("gather.json needs loop.json"); s.G.h = make_io_plan(s.jg, s.loop, false); }
    if (s.have_s) { if (!s.have_l) throw std::runtime_error("scatter.json needs loop.json"); s.S.h = make_io_plan(s.js, s.loop, true); }
  }
  if (s.G.h.ok) upload_plan(s.G);
  if (s.S.h.ok) upload_plan(s.S);
  // per-feature vectors of a boundary
  for (PlanDev* P : {&s.G, &s.S})
    for (size_t v = 0; v < P->h.vec_names.size(); v++) {
      auto it = s.vectors.find(P->h.vec_names[v]);
      if (it == s.vectors.end()) throw std::runtime_error("lift2d vector \"" + P->h.vec_names[v] + "\" was not set (fortis_set_vector)");
      if (it->second.second != P->h.prog.tv_double) throw std::runtime_error("lift2d vector \"" + P->h.vec_names[v] + "\" has the wrong element type");
      P->vec_dev[v] = pool_alloc((long)it->second.first.size());
      cudaMemcpy(P->vec_dev[v], it->second.first.data(), it->second.first.size(), cudaMemcpyHostToDevice);
    }
  s.planned = true;
  drop_graph();
}

void ensure_model() {
  Session& s = S();
  if (!s.have_model) { load_env_config(); }
  if (!s.have_model) throw std::runtime_error("no model loaded (fortis_load_model or FORTIS_MODEL)");
  if (s.model_on_dev) return;
  cudaStream_t st = stream();
  for (auto& L : s.model.layers) {
    float* w = (float*)pool_alloc((long)(L.W.size() * 4));
    float* b = (float*)pool_alloc((long)(L.b.size() * 4));
    if (!w || !b) throw std::runtime_error("out of device memory for weights");
    cudaMemcpy(w, L.W.data(), L.W.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(b, L.b.data(), L.b.size() * 4, cudaMemcpyHostToDevice);
    s.dW.push_back(w); s.dB.push_back(b);
  }
  auto up = [&](const std::vector<float>& v) -> float* {
    if (v.empty()) return nullptr;
    float* d = (float*)pool_alloc((long)(v.size() * 4));
    cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
    return d;
  };
  s.d_in_div = up(s.model.in_div); s.d_out_mul = up(s.model.out_mul); s.d_relu_mask = up(s.model.relu_mask);
  if (s.model.is_mlp()) {
    std::vector<int> dims{s.model.n_in()};
    for (auto& L : s.model.layers) dims.push_back(L.cout);
    const int nl = (int)s.model.layers.size();
    if (small_mlp_supported(nl, dims.data()) && s.model.relu_mask.empty()) {
      std::vector<float> img(kSmallConstFloats, 0.f);
      std::vector<const float*> W, B;
      for (auto& L : s.model.layers) { W.push_back(L.W.data()); B.push_back(L.b.data()); }
      const int nf = small_mlp_pack(nl, dims.data(), W.data(), B.data(), s.model.in_div.empty() ? nullptr : s.model.in_div.data(),
                                    s.model.out_mul.empty() ? nullptr : s.model.out_mul.data(), img.data());
      if (cuda_ok(small_mlp_upload(img.data(), nf, st), "small-MLP constant upload")) s.small_ok = true;
      cudaStreamSynchronize(st);
    }
    if (s.precision == PREC_F32 && stencil_mlp_supported(nl, dims.data()) && s.model.relu_mask.empty()) {
      std::vector<const float*> W, B;
      for (auto& L : s.model.layers) { W.push_back(L.W.data()); B.push_back(L.b.data()); }
      if (cuda_ok(stencil_mlp_upload(nl, dims.data(), W.data(), B.data(), s.model.in_div.empty() ? nullptr : s.model.in_div.data(),
                                     s.model.out_mul.empty() ? nullptr : s.model.out_mul.data(), st), "stencil-MLP constant upload"))
        s.stencil_ok = true;
    }
    // the tensor-core form of the same step: an option (measured slower than the packed-FMA kernel for nets this narrow)
    if (s.precision == PREC_F32 && stencil_tc_supported(nl, dims.data()) && s.model.relu_mask.empty()) {
      std::vector<const float*> W, B;
      for (auto& L : s.model.layers) { W.push_back(L.W.data()); B.push_back(L.b.data()); }
      s.stencil_tc = stencil_tc_create(nl, dims.data(), W.data(), B.data(), s.model.in_div.empty() ? nullptr : s.model.in_div.data(),
                                       s.model.out_mul.empty() ? nullptr : s.model.out_mul.data());
    }
    if (s.precision == PREC_F32) {
      std::string err;
      s.f32 = f32tc_create(s.model, &err);                       // optional: without it every batch takes the FFMA kernels
      if (!s.f32) std::fprintf(stderr, "fortis: fp32 layers stay on the FFMA kernels (%s)\n", err.c_str());
    }
    if (s.precision != PREC_F32) {
      std::string err;
      s.tc = tc_model_create(s.model, s.precision, st, &err);
      if (!s.tc) {
        // Layers wider than the fused kernel holds on chip (the reference's width sweep goes to 2048) run layer by layer
        // on the fp32 tensor-core kernel instead: slower than a 16-bit GEMM would be, and more accurate than asked for.
        std::string err32;
        const bool shape = err.find("wider than") != std::string::npos || err.find("layers") != std::string::npos;
        if (shape) s.f32 = f32tc_create(s.model, &err32);
        if (!s.f32)
          throw std::runtime_error("precision " + std::string(s.precision == PREC_BF16 ? "bf16" : s.precision == PREC_FP16 ? "fp16" : "fp8w") +
                                   " needs the tensor-core kernel, which cannot take this model: " + err);
        std::fprintf(stderr, "fortis: %s; the layers run one by one on the fp32 (TF32x3) tensor-core kernel\n", err.c_str());
      }
    }
  } else if (s.model.is_conv()) {
    std::string err;
    s.conv = conv_model_create(s.model, s.precision, st, &err);
    if (!s.conv) throw std::runtime_error("conv3d model: " + err);
  } else if (s.model.is_opnet()) {
    if (s.precision != PREC_F32) throw std::runtime_error("networks of 2-D operator layers run in fp32");
    std::string err;
    s.opnet = opnet_create(s.model, &err);
    if (!s.opnet) throw std::runtime_error("2-D network: " + err);
  } else {
    throw std::runtime_error("a model must be all Linear, all Conv3d or all 2-D operator layers");
  }
  s.model_on_dev = true;
  drop_graph();
}

long long model_rows() {
  Session& s = S();
  if (s.model.is_conv() || s.model.is_opnet()) return (long long)s.conv_shape[0] * s.conv_shape[1] * s.conv_shape[2] * s.conv_shape[3];
  if (s.planned && (s.G.h.ok || s.S.h.ok || s.have_l)) {
    if (s.begin_count >= 0 && s.have_l && !s.have_l2) return s.begin_count * s.loop.nk;   // run-time extent
    return s.loop.count * s.loop.nk;
  }
  return s.begin_count > 0 ? s.begin_count : 1;
}

// floats of the model output for `rows` input rows (a 2-D operator network changes the spatial extent)
long long out_floats(long long rows) {
  Session& s = S();
  if (!s.model.is_opnet()) return rows * s.model.n_out();
  int C = 0, Ho = 0, Wo = 0;
  if (s.conv_shape[1] != 1) throw std::runtime_error("2-D network: option conv_shape must be N,1,H,W");
  if (!opnet_shape(s.model, s.conv_shape[2], s.conv_shape[3], &C, &Ho, &Wo, nullptr))
    throw std::runtime_error("2-D network: a layer's kernel is larger than its input");
  return (long long)s.conv_shape[0] * C * Ho * Wo;
}

void ensure_buffers(long long rows) {
  Session& s = S();
  if (rows <= s.buf_rows && s.din) return;
  pool_free(s.din); pool_free(s.dout); pool_free(s.act0); pool_free(s.act1);
  int wmax = 1;
  for (auto& L : s.model.layers) wmax = L.cout > wmax ? L.cout : wmax;
  const long long nin = s.model.n_in(), nout = s.model.n_out();
  s.din = (float*)pool_alloc(rows * nin * 4);
  s.dout = (float*)pool_alloc(out_floats(rows) * 4);
  (void)nout;
  const bool need_act = s.model.is_mlp() && s.model.layers.size() > 1;
  s.act0 = need_act ? (float*)pool_alloc(rows * wmax * 4) : nullptr;
  s.act1 = need_act && s.model.layers.size() > 2 ? (float*)pool_alloc(rows * wmax * 4) : nullptr;
  if (!s.din || !s.dout || (need_act && !s.act0)) throw std::runtime_error("out of device memory for the model buffers");
  s.buf_rows = rows;
  drop_graph();
}

void ensure_aux(long long npartials) {
  Session& s = S();
  if (!s.d_sum) {
    s.d_sum = (double*)pool_alloc(sizeof(double));
    s.d_status = (int*)pool_alloc(sizeof(int));
    s.d_done = (unsigned int*)pool_alloc(sizeof(unsigned int));
    cudaMemset(s.d_done, 0, sizeof(unsigned int));
    cudaMemset(s.d_sum, 0, sizeof(double));
    cudaMemset(s.d_status, 0, sizeof(int));
  }
  if (npartials > s.partials_cap) {
    pool_free(s.d_partials);
    s.d_partials = (double*)pool_alloc(npartials * (long long)sizeof(double));
    s.partials_cap = npartials;
    drop_graph();
  }
}

// ---------------------------------------------------------------------------------------------------------------
// host-array staging  (driver/fortis_gather_emit.py:37-48, 66-68, 86-97)
// ---------------------------------------------------------------------------------------------------------------
bool is_device_ptr(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// pin once; an array whose address moves between calls is a temporary: unpin it and never pin it again
void pin_policy(PlanDev& P, int ai, const void* H, size_t bytes) {
  if (P.reg[ai] == (const void*)1 || P.reg[ai] == H) return;
  if (P.reg[ai]) { cudaHostUnregister((void*)P.reg[ai]); cudaGetLastError(); P.reg[ai] = (const void*)1; return; }
  if (std::getenv("FORTIS_NO_PIN")) { P.reg[ai] = (const void*)1; return; }
  if (cudaHostRegister((void*)H, bytes, cudaHostRegisterDefault) == cudaSuccess) P.reg[ai] = H;
  else { cudaGetLastError(); P.reg[ai] = (const void*)1; }
}

size_t elt_size(int elt) { return elt ? 8 : 4; }

// does this plan's side of a step address pinned host arrays in place (option host_access)?
bool maps_host(const PlanDev& P) {
  const int m = S().host_access;
  return m == 2 || (m == 1 && P.h.is_scatter);
}

long long plane_off_args(const ArrayInfo& a, const int* args, int nargs) {
  long long off = 0;
  for (auto& t : a.vterms) {
    const int av = t.first < nargs ? args[t.first] : 1;
    off += (long long)(av - 1) * t.second;
  }
  return off;
}

// Bind this call's arrays into an ArrayTable.  `multi_plane`: all planes klo..klo+nk-1 are addressed through kk
// (k-distributed gather, fused step); otherwise the plane chosen by the integer arguments.
void bind_arrays(PlanDev& P, void* const* ptrs, const int* args, int nargs, bool multi_plane, bool upload_readonly,
                 ArrayTable* T) {
  Session& s = S();
  cudaStream_t st = stream();
  std::memset(T, 0, sizeof *T);
  for (size_t ai = 0; ai < P.h.arrays.size(); ai++) {
    const ArrayInfo& a = P.h.arrays[ai];
    const size_t es = elt_size(a.elt);
    char* H = (char*)ptrs[ai];
    P.cur[ai] = H;
    const bool planes = multi_plane && !a.vdims.empty();
    const long long first = planes ? (long long)(s.loop.klo - 1) * a.plane : (multi_plane ? 0 : plane_off_args(a, args, nargs));
    P.on_dev[ai] = is_device_ptr(H);
    if (P.on_dev[ai]) { T->base[ai] = H + first * es; continue; }
    const long long need = planes ? a.plane * s.loop.nk : a.plane;
    pin_policy(P, (int)ai, H, (size_t)a.total * es);
    if (maps_host(P) && P.reg[ai] == H) {
      // The kernels address the pinned host pages themselves: loads and stores cross the bus inside the launch, no
      // staging copy on either side.
      void* dp = nullptr;
      if (cudaHostGetDevicePointer(&dp, H, 0) == cudaSuccess && dp) { P.on_dev[ai] = true; T->base[ai] = (char*)dp + first * es; continue; }
      cudaGetLastError();
    }
    if (P.stage_elems[ai] < need) {
      pool_free(P.stage[ai]);
      P.stage[ai] = pool_alloc(need * (long long)es);
      if (!P.stage[ai]) throw std::runtime_error("out of device memory staging array " + a.name);
      P.stage_elems[ai] = need;
    }
    const bool written = P.h.is_scatter && ai < P.h.written.size() && P.h.written[ai];
    if (a.used && (!written) && upload_readonly)
      cuda_ok(cudaMemcpyAsync(P.stage[ai], H + first * es, (size_t)need * es, cudaMemcpyHostToDevice, st), "H2D of a host array");
    T->base[ai] = P.stage[ai];
  }
  for (int v = 0; v < kMaxVecs; v++) T->vec[v] = P.vec_dev[v];
}

// copy the visited cells of every stored array back to the host (the reference's cudaMemcpy2DAsync rectangles);
// stores that form one contiguous run in an array (column physics: level after level) are merged into one copy
void download_stores(PlanDev& P, const int* args, int nargs, bool multi_plane, cudaStream_t on = nullptr, int kk_begin = 0, int kk_end = -1) {
  Session& s = S();
  cudaStream_t st = on ? on : stream();
  const long long ni = s.loop.ni, nj = s.loop.count / (s.loop.ni > 0 ? s.loop.ni : 1);
  struct Run { int array; long long off, len; };
  std::vector<Run> runs;
  // Stores that walk a strided column (the column index is not the array's fastest dimension): when the stores of
  // one array interleave densely (offsets off, off+1, ..., off+si-1 with stride si) their union is one contiguous
  // range; otherwise each is copied as a 1-element-wide 2-D copy.
  std::map<std::pair<int, long long>, std::vector<long long>> columns;
  for (auto& t : P.h.stores)
    if (!P.on_dev[t.a.array] && t.a.si != 1 && (t.a.sj == 0 || nj == 1)) columns[{t.a.array, t.a.si}].push_back(t.a.off0);
  std::map<std::pair<int, long long>, bool> dense;
  for (auto& kv : columns) {
    std::vector<long long>& o = kv.second;
    std::sort(o.begin(), o.end());
    bool ok = (long long)o.size() == kv.first.second;
    for (size_t i = 1; ok && i < o.size(); i++) ok = o[i] == o[i - 1] + 1;
    dense[kv.first] = ok;
    if (ok) runs.push_back({kv.first.first, o[0], ni * kv.first.second});
  }
  for (auto& t : P.h.stores) {
    const int ai = t.a.array;
    if (P.on_dev[ai]) continue;
    const ArrayInfo& a = P.h.arrays[ai];
    const size_t es = elt_size(a.elt);
    if (t.a.si == 1 && (t.a.sj == 0 || nj == 1)) { runs.push_back({ai, t.a.off0, ni}); continue; }
    if (t.a.si != 1 && (t.a.sj == 0 || nj == 1) && dense[{ai, t.a.si}]) continue;
    const bool planes = multi_plane && !a.vdims.empty();
    const int nplanes = planes ? s.loop.nk : 1;
    for (int kk = planes ? kk_begin : 0; kk < (planes && kk_end >= 0 ? kk_end : nplanes); kk++) {
      const long long hoff = planes ? (long long)(s.loop.klo - 1 + kk) * a.plane : (multi_plane ? 0 : plane_off_args(a, args, nargs));
      char* dsrc = (char*)P.stage[ai] + ((long long)kk * a.plane + t.a.off0) * es;
      char* hdst = (char*)P.cur[ai] + (hoff + t.a.off0) * es;
      // a 2-D copy is validated over pitch x height, which would reach past the end of the array on the last
      // row: copy all rows but the last as 2-D, the last one as 1-D
      if (t.a.si == 1) {
        if (nj > 1) cuda_ok(cudaMemcpy2DAsync(hdst, (size_t)t.a.sj * es, dsrc, (size_t)t.a.sj * es, (size_t)ni * es, (size_t)(nj - 1),
                                              cudaMemcpyDeviceToHost, st), "D2H of a stored rectangle");
        cuda_ok(cudaMemcpyAsync(hdst + (nj - 1) * t.a.sj * es, dsrc + (nj - 1) * t.a.sj * es, (size_t)ni * es, cudaMemcpyDeviceToHost, st),
                "D2H of a stored rectangle (last row)");
      } else if (t.a.sj == 0 || nj == 1) {
        if (ni > 1) cuda_ok(cudaMemcpy2DAsync(hdst, (size_t)t.a.si * es, dsrc, (size_t)t.a.si * es, es, (size_t)(ni - 1),
                                              cudaMemcpyDeviceToHost, st), "D2H of a stored column");
        cuda_ok(cudaMemcpyAsync(hdst + (ni - 1) * t.a.si * es, dsrc + (ni - 1) * t.a.si * es, es, cudaMemcpyDeviceToHost, st),
                "D2H of a stored column (last element)");
      } else {
        throw std::runtime_error("store into host-resident " + a.name + " has a stride pattern that is not a rectangle; pass a device array");
      }
    }
  }
  std::sort(runs.begin(), runs.end(), [](const Run& x, const Run& y) { return x.array != y.array ? x.array < y.array : x.off < y.off; });
  for (size_t i = 0; i < runs.size();) {
    Run r = runs[i++];
    while (i < runs.size() && runs[i].array == r.array && runs[i].off <= r.off + r.len) {
      const long long e = runs[i].off + runs[i].len;
      if (e > r.off + r.len) r.len = e - r.off;
      i++;
    }
    const ArrayInfo& a = P.h.arrays[r.array];
    const size_t es = elt_size(a.elt);
    const bool planes = multi_plane && !a.vdims.empty();
    const int nplanes = planes ? s.loop.nk : 1;
    for (int kk = planes ? kk_begin : 0; kk < (planes && kk_end >= 0 ? kk_end : nplanes); kk++) {
      const long long hoff = planes ? (long long)(s.loop.klo - 1 + kk) * a.plane : (multi_plane ? 0 : plane_off_args(a, args, nargs));
      cuda_ok(cudaMemcpyAsync((char*)P.cur[r.array] + (hoff + r.off) * es, (char*)P.stage[r.array] + ((long long)kk * a.plane + r.off) * es,
                              (size_t)r.len * es, cudaMemcpyDeviceToHost, st), "D2H of a stored run");
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// the step
// ---------------------------------------------------------------------------------------------------------------
constexpr long long kF32TcMinRows = 512;     // below this the per-layer FFMA kernels win on latency

struct StepArgs {
  bool use_gather = false;      // model input comes from the gather plan (else din)
  bool fuse_scatter = false;    // outputs go straight to the host arrays (all planes)
  bool unfused = false;         // run gather, forward and scatter as separate kernels (gather and scatter share memory)
  ArrayTable TG{}, TS{};
  long long rows = 0;
};

RowGeom geom_all(long long rows) {
  Session& s = S();
  RowGeom g;
  g.nk = s.loop.nk > 0 ? s.loop.nk : 1;
  g.count = rows / g.nk;
  g.ni = s.loop.ni > 0 ? s.loop.ni : 1;
  g.kk0 = 0;
  return g;
}

// Operands of the fast small-MLP kernel: possible when all input slots (and all stores) are fp32 and share one
// stride triple, and every index fits 32 bits.
bool small_fast_operands(const StepArgs& A, const RowGeom& g, SmallFast* F) {
  Session& s = S();
  std::memset(F, 0, sizeof *F);
  const long long nrows = g.count * g.nk;
  if (nrows >= (1LL << 31) || s.G.h.slots.size() > 32) return false;
  const Access& a0 = s.G.h.slots[0];
  for (size_t q = 0; q < s.G.h.slots.size(); q++) {
    const Access& a = s.G.h.slots[q];
    const ArrayInfo& ai = s.G.h.arrays[a.array];
    if (a.elt != 0 || a.si != a0.si || a.sj != a0.sj || a.sk != a0.sk || ai.total >= (1LL << 31)) return false;
    F->in_ptr[q] = (const float*)A.TG.base[a.array] + a.off0;
  }
  F->si = (int)a0.si; F->sj = (int)a0.sj; F->sk = (int)a0.sk;
  F->in_prog = s.G.h.prog.nops > 0;
  if (A.fuse_scatter) {
    if (s.S.h.stores.size() > 8 || s.S.h.stores.empty()) return false;
    const Access& b0 = s.S.h.stores[0].a;
    for (size_t q = 0; q < s.S.h.stores.size(); q++) {
      const Access& a = s.S.h.stores[q].a;
      const ArrayInfo& ai = s.S.h.arrays[a.array];
      if (a.elt != 0 || a.si != b0.si || a.sj != b0.sj || a.sk != b0.sk || ai.total >= (1LL << 31)) return false;
      F->out_ptr[q] = (float*)A.TS.base[a.array] + a.off0;
      F->out_slot[q] = s.S.h.stores[q].slot;
    }
    F->nstores = (int)s.S.h.stores.size();
    F->oi = (int)b0.si; F->oj = (int)b0.sj; F->ok = (int)b0.sk;
    F->out_prog = s.S.h.prog.nops > 0;
  }
  F->nrows = (unsigned)nrows; F->count = (unsigned)g.count; F->ni = (unsigned)g.ni;
  return true;
}

// the standalone scatter of a step; with option "checksum" its stores are summed like those of the fused kernels
void scatter_with_checksum(const StepArgs& A, const RowGeom& g) {
  Session& s = S();
  cudaStream_t st = stream();
  double* partials = nullptr;
  const int grid = scatter_grid(g.count * g.nk);
  if (s.want_checksum) { ensure_aux(grid); partials = s.d_partials; }
  launch_scatter(s.S.hdr, (const StoreTarget*)s.S.items, s.S.h.n, A.TS, g, s.dout, st, partials);
  if (partials) launch_fold(s.d_partials, grid, s.d_sum, 1, st);
}

// Operands of the packed-FMA stencil kernel: a fused step whose gather is the 3x3 stencil of three fp32 fields in
// field-major, j-major, i-fastest slot order with unit i stride, without lifted expressions, and whose stores are fp32
// with unit i stride.
bool stencil_operands(const StepArgs& A, const RowGeom& g, StencilLaunch* L) {
  Session& s = S();
  std::memset(L, 0, sizeof *L);
  const IoPlanHost& G = s.G.h;
  const IoPlanHost& Sc = s.S.h;
  if (G.prog.nops || !G.scalars.empty() || Sc.prog.nops || !Sc.scalars.empty() || G.slots.size() != 27 || g.kk0 != 0) return false;
  if (Sc.stores.empty() || Sc.stores.size() > 4) return false;
  const Access& c0 = G.slots[4];
  for (int f = 0; f < 3; f++) {
    const Access& c = G.slots[f * 9 + 4];
    if (c.elt != 0 || c.si != 1 || c.sj != c0.sj || c.sk != c0.sk) return false;
    for (int dj = 0; dj < 3; dj++)
      for (int di = 0; di < 3; di++) {
        const Access& a = G.slots[f * 9 + dj * 3 + di];
        if (a.array != c.array || a.elt != 0 || a.si != 1 || a.sj != c.sj || a.sk != c.sk || a.off0 - c.off0 != (di - 1) + (dj - 1) * c.sj) return false;
      }
    L->in[f] = (const float*)A.TG.base[c.array] + c.off0;
  }
  const Access& o0 = Sc.stores[0].a;
  for (size_t q = 0; q < Sc.stores.size(); q++) {
    const Access& a = Sc.stores[q].a;
    if (a.elt != 0 || a.si != 1 || a.sj != o0.sj || a.sk != o0.sk || Sc.stores[q].slot > 3) return false;
    L->out[q] = (float*)A.TS.base[a.array] + a.off0;
    L->out_slot[q] = Sc.stores[q].slot;
  }
  L->nstores = (int)Sc.stores.size();
  L->sj_in = c0.sj; L->sk_in = c0.sk; L->sj_out = o0.sj; L->sk_out = o0.sk;
  L->ni = g.ni; L->nj = (int)(g.count / g.ni); L->nk = g.nk;
  if ((long long)L->ni * L->nj != g.count) return false;
  return true;
}

void run_step_kernels(const StepArgs& A) {
  Session& s = S();
  cudaStream_t st = stream();
  const long long rows = A.rows;
  const RowGeom g = geom_all(rows);
  const int nl = (int)s.model.layers.size();
  if (s.model.is_conv()) {
    std::string err;
    if (!conv_forward(s.conv, s.din, s.dout, s.conv_shape[0], s.conv_shape[1], s.conv_shape[2], s.conv_shape[3], st, &err))
      throw std::runtime_error(err);
    return;
  }
  if (s.model.is_opnet()) {
    std::string err;
    if (!opnet_forward(s.opnet, s.din, s.dout, s.conv_shape[0], s.conv_shape[2], s.conv_shape[3], st, &err)) throw std::runtime_error(err);
    return;
  }
  const bool fuse = s.fuse && !A.unfused;
  const bool fused_gather = A.use_gather && fuse;
  if (s.tc) {
    // The tensor-core kernel fuses the gather / scatter when the descriptor is in its table-driven class (fp32
    // arrays, no lifted expressions or scalars, at most two stride classes, <= 256 inputs / <= 128 outputs);
    // other descriptors run the bit-exact standalone gather / scatter kernels around it.
    TcLaunch L{};
    const bool fuse_in = A.use_gather && fuse && s.G.fast && s.model.n_in() <= 256;
    const bool fuse_out = A.fuse_scatter && fuse && s.S.fast && s.model.n_out() <= 128;
    if (fuse_in) { L.GP = s.G.hdr; L.slots = (const Access*)s.G.items; L.TG = A.TG; L.fast_in = 1; std::memcpy(L.cin, s.G.cls, sizeof L.cin); }
    else {
      if (A.use_gather) launch_gather(s.G.hdr, (const Access*)s.G.items, s.G.h.n, A.TG, g, s.din, st);
      L.X = s.din;
    }
    if (fuse_out) { L.SP = s.S.hdr; L.stores = (const StoreTarget*)s.S.items; L.TS = A.TS; L.fast_out = 1;
                    L.store_by_slot = s.S.store_by_slot; std::memcpy(L.cout, s.S.cls, sizeof L.cout); }
    L.Y = fuse_out ? nullptr : s.dout;
    L.g = g;
    ensure_aux(tc_grid(s.tc, rows));
    L.partials = (fuse_out && s.want_checksum) ? s.d_partials : nullptr;
    L.sum = L.partials ? s.d_sum : nullptr; L.done = s.d_done;
    L.status = s.d_status;
    std::string err;
    if (!tc_forward(s.tc, L, st, &err)) throw std::runtime_error(err);
    if (A.fuse_scatter && !fuse_out) scatter_with_checksum(A, g);
    return;
  }
  if (fused_gather && A.fuse_scatter && (s.stencil_ok || (s.use_stencil_tc && s.stencil_tc))) {
    StencilLaunch SL;
    if (stencil_operands(A, g, &SL)) {
      std::vector<int> dims{s.model.n_in()};
      bool relu_only = true;
      for (int l = 0; l < nl; l++) {
        const LayerHost& L = s.model.layers[l];
        dims.push_back(L.cout);
        SL.slope[l] = L.act == ACT_NONE ? 1.f : L.act == ACT_RELU ? 0.f : L.slope;
        if (l < nl - 1 && L.act != ACT_RELU) relu_only = false;
      }
      SL.has_in_div = !s.model.in_div.empty(); SL.has_out_mul = !s.model.out_mul.empty();
      const int gmax = stencil_mlp_grid(SL) > stencil_tc_grid(SL) ? stencil_mlp_grid(SL) : stencil_tc_grid(SL);
      ensure_aux(s.want_checksum ? gmax : 1);
      if (s.want_checksum) { SL.partials = s.d_partials; SL.sum = s.d_sum; SL.done = s.d_done; }
      if (s.use_stencil_tc && s.stencil_tc && launch_stencil_tc(s.stencil_tc, SL, s.d_status, st)) return;
      if (s.stencil_ok && launch_stencil_mlp(nl, dims.data(), relu_only, SL, st)) return;
    }
  }
  if (fused_gather && s.small_ok) {
    std::vector<int> dims{s.model.n_in()};
    SmallMlpLaunch L{};
    for (int l = 0; l < nl; l++) { dims.push_back(s.model.layers[l].cout); L.act[l] = s.model.layers[l].act; L.slope[l] = s.model.layers[l].slope; }
    L.GP = s.G.hdr; L.slots = (const Access*)s.G.items; L.TG = A.TG;
    if (A.fuse_scatter) { L.SP = s.S.hdr; L.stores = (const StoreTarget*)s.S.items; L.TS = A.TS; }
    L.g = g;
    L.use_fast = small_fast_operands(A, g, &L.fast) ? 1 : 0;
    L.has_in_div = !s.model.in_div.empty(); L.has_out_mul = !s.model.out_mul.empty();
    L.Yout = A.fuse_scatter ? nullptr : s.dout;
    L.grid = small_mlp_grid(rows);
    if (A.fuse_scatter && s.want_checksum) { ensure_aux(L.grid); L.partials = s.d_partials; }
    launch_small_mlp(nl, dims.data(), L, st);
    if (L.partials) launch_fold(s.d_partials, L.grid, s.d_sum, 1, st);
    return;
  }
  if (s.f32 && rows >= kF32TcMinRows) {
    // fp32 on the tensor cores: one split-TF32 kernel per layer, gather fused into the first layer's operand load and
    // scatter (+ checksum) into the last epilogue when the descriptors are table-driven, activations feature-major
    F32TcLaunch L{};
    const bool fuse_in = A.use_gather && fuse && s.G.fast && s.model.n_in() <= 768;
    const bool fuse_out = A.fuse_scatter && fuse && s.S.fast && s.model.n_out() <= 256;
    if (fuse_in) { L.fast_in = 1; L.slots = (const Access*)s.G.items; L.TG = A.TG; std::memcpy(L.cin, s.G.cls, sizeof L.cin); }
    else {
      if (A.use_gather) launch_gather(s.G.hdr, (const Access*)s.G.items, s.G.h.n, A.TG, g, s.din, st);
      L.X = s.din;
    }
    if (fuse_out) { L.fast_out = 1; L.store_by_slot = s.S.store_by_slot; L.TS = A.TS; std::memcpy(L.cout, s.S.cls, sizeof L.cout); }
    else L.Y = s.dout;
    L.g = g;
    L.act[0] = s.act0; L.act[1] = s.act1; L.act_ld = s.buf_rows;
    ensure_aux(f32tc_grid(rows));
    if (fuse_out && s.want_checksum) { L.partials = s.d_partials; L.sum = s.d_sum; L.done = s.d_done; }
    L.status = s.d_status;
    std::string err;
    if (!f32tc_forward(s.f32, L, st, &err)) throw std::runtime_error(err);
    if (A.fuse_scatter && !fuse_out) scatter_with_checksum(A, g);
    return;
  }
  // generic fp32 path: gather kernel -> one FFMA kernel per layer -> scatter kernel
  if (A.use_gather) launch_gather(s.G.hdr, (const Access*)s.G.items, s.G.h.n, A.TG, g, s.din, st);
  const float* src = s.din;
  for (int l = 0; l < nl; l++) {
    const LayerHost& L = s.model.layers[l];
    float* dst = l == nl - 1 ? s.dout : ((l & 1) ? s.act1 : s.act0);
    launch_linear_f32(src, s.dW[l], s.dB[l], dst, rows, L.cout, L.cin, L.act, L.slope, l == 0 ? s.d_in_div : nullptr,
                      l == nl - 1 ? s.d_out_mul : nullptr, l == nl - 1 ? s.d_relu_mask : nullptr, st);
    src = dst;
  }
  if (A.fuse_scatter) scatter_with_checksum(A, g);
}

std::string step_key(const StepArgs& A) {
  std::string k((const char*)&A.use_gather, sizeof(bool));
  k.append((const char*)&A.fuse_scatter, sizeof(bool));
  k.append((const char*)&A.unfused, sizeof(bool));
  k.append((const char*)&A.rows, sizeof A.rows);
  if (A.use_gather) k.append((const char*)&A.TG, sizeof A.TG);
  if (A.fuse_scatter) k.append((const char*)&A.TS, sizeof A.TS);
  return k;
}

// driver/fortis_shim.py:82-90: replay if captured; capture on the second call when asked; eager on failure
void run_step(const StepArgs& A) {
  Session& s = S();
  cudaStream_t st = stream();
  if (!s.graph) { run_step_kernels(A); return; }
  const std::string key = step_key(A);
  if (s.gexec && key == s.gkey) { cuda_ok(cudaGraphLaunch(s.gexec, st), "cudaGraphLaunch"); return; }
  if (key != s.gkey) { drop_graph(); s.gkey = key; }
  const bool cap = (++s.ncalls == 2);
  if (!cap) { run_step_kernels(A); return; }
  fortis_capturing = 1;
  if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    cudaGetLastError(); fortis_capturing = 0; run_step_kernels(A); return;
  }
  bool threw = false; std::string what;
  try { run_step_kernels(A); } catch (const std::exception& e) { threw = true; what = e.what(); }
  cudaGraph_t gr = nullptr;
  fortis_capturing = 0;
  const bool ok = cudaStreamEndCapture(st, &gr) == cudaSuccess && !threw &&
                  cudaGraphInstantiate(&s.gexec, gr, 0) == cudaSuccess;
  if (gr) cudaGraphDestroy(gr);
  if (ok) { cuda_ok(cudaGraphLaunch(s.gexec, st), "cudaGraphLaunch"); return; }
  std::fprintf(stderr, "fortis: graph capture failed, running eagerly\n");
  s.gexec = nullptr; cudaGetLastError();
  if (threw) throw std::runtime_error(what);
  run_step_kernels(A);
}

void prepare(long long* rows_out) {
  ensure_plans();
  ensure_model();
  Session& s0 = S();
  if (s0.model.is_mlp()) {
    // descriptors and model arrive independently: a pair that does not fit would index past the model's buffers
    if (s0.G.h.ok && s0.G.h.n != s0.model.n_in())
      throw std::runtime_error("the gather descriptor produces " + std::to_string(s0.G.h.n) + " inputs per row, the model takes " +
                               std::to_string(s0.model.n_in()));
    if (s0.S.h.ok && s0.S.h.n != s0.model.n_out())
      throw std::runtime_error("the scatter descriptor consumes " + std::to_string(s0.S.h.n) + " outputs per row, the model produces " +
                               std::to_string(s0.model.n_out()));
  }
  const long long rows = model_rows();
  ensure_buffers(rows);
  *rows_out = rows;
}

void collect_args(PlanDev& P, bool skip_ints, long first, va_list ap, bool first_is_named, std::vector<int>* ints,
                  std::vector<void*>* ptrs) {
  const int nint = skip_ints ? 0 : P.h.nargs;
  const int narr = (int)P.h.arrays.size();
  bool used_first = !first_is_named;
  for (int i = 0; i < nint; i++) {
    if (!used_first) { ints->push_back((int)first); used_first = true; }
    else ints->push_back(va_arg(ap, int));
  }
  for (int i = 0; i < narr; i++) {
    if (!used_first) { ptrs->push_back((void*)first); used_first = true; }
    else ptrs->push_back(va_arg(ap, void*));
  }
}

void do_gather(const int* iargs, int nint, void* const* ptrs, int narr) {
  Session& s = S();
  ensure_plans();
  if (!s.G.h.ok) throw std::runtime_error("fortis_gather: no gather descriptor is configured");
  if (narr != (int)s.G.h.arrays.size()) throw std::runtime_error("fortis_gather: wrong number of arrays");
  ensure_model();
  for (int i = 0; i < 8; i++) s.gather_args[i] = i < nint ? iargs[i] : 1;
  // staging happens now (the host may change its arrays after this call returns); the gather itself is deferred
  ArrayTable T;
  bind_arrays(s.G, ptrs, s.gather_args, nint, s.loop.kdist, true, &T);
  s.gather_pending = true;
}

ArrayTable current_gather_table() {
  Session& s = S();
  ArrayTable T;
  std::memset(&T, 0, sizeof T);
  for (size_t ai = 0; ai < s.G.h.arrays.size(); ai++) {
    const ArrayInfo& a = s.G.h.arrays[ai];
    if (!s.G.on_dev[ai]) { T.base[ai] = s.G.stage[ai]; continue; }
    const bool planes = s.loop.kdist && !a.vdims.empty();
    const long long first = planes ? (long long)(s.loop.klo - 1) * a.plane : (s.loop.kdist ? 0 : plane_off_args(a, s.gather_args, 8));
    T.base[ai] = (char*)s.G.cur[ai] + first * elt_size(a.elt);
  }
  for (int v = 0; v < kMaxVecs; v++) T.vec[v] = s.G.vec_dev[v];
  return T;
}

void do_forward_batched(void* in, void* out) {
  Session& s = S();
  long long rows;
  prepare(&rows);
  cudaStream_t st = stream();
  const long long nin = s.model.n_in(), nout = s.model.n_out();
  StepArgs A;
  A.rows = rows;
  if (s.gather_pending) {
    A.use_gather = true;
    A.TG = current_gather_table();
    run_step(A);
    s.gather_pending = false;
    if (!s.S.h.ok && s.Y_pinned) {    // gather lifted but outputs unpacked on the host (FORTIS_GATHER only: shim :111-113)
      cuda_ok(cudaMemcpyAsync(s.Y_pinned, s.dout, rows * nout * 4, cudaMemcpyDeviceToHost, st), "D2H of Y");
      cudaStreamSynchronize(st);
    }
    return;
  }
  if (s.gather_done) {               // the gather already ran as its own kernel (fortis_model_input was asked for)
    run_step(A);
    s.gather_done = false;
    return;
  }
  if (s.pack_pending) {              // packed form: X -> din, step, dout -> Y   (driver/fortis_shim.py:115)
    cuda_ok(cudaMemcpyAsync(s.din, s.X_pinned, rows * nin * 4, cudaMemcpyHostToDevice, st), "H2D of X");
    run_step(A);
    if (!s.S.h.ok) {
      cuda_ok(cudaMemcpyAsync(s.Y_pinned, s.dout, rows * nout * 4, cudaMemcpyDeviceToHost, st), "D2H of Y");
      cudaStreamSynchronize(st);
    }
    s.pack_pending = false;
    return;
  }
  // a run-time extent of zero (driver/fortis_stub.c: fortis_begin(0), a loop that packs nothing): nothing to do
  if (s.begin_count == 0 && !in && !out) return;
  // array form  (driver/fortis_shim.py:117-121)
  if (!in || !out) throw std::runtime_error("mlp_forward_batched: no gather or pack is pending and no arrays were given");
  if (is_device_ptr(in)) cuda_ok(cudaMemcpyAsync(s.din, in, rows * nin * 4, cudaMemcpyDeviceToDevice, st), "D2D of the input");
  else cuda_ok(cudaMemcpyAsync(s.din, in, rows * nin * 4, cudaMemcpyHostToDevice, st), "H2D of the input");
  run_step(A);
  cuda_ok(cudaMemcpyAsync(out, s.dout, rows * nout * 4, is_device_ptr(out) ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, st),
          "copy of the output");
  cudaStreamSynchronize(st);
}

void do_scatter(const int* iargs, int nint, void* const* ptrs, int narr) {
  Session& s = S();
  long long rows;
  prepare(&rows);
  if (!s.S.h.ok) throw std::runtime_error("fortis_scatter: no scatter descriptor is configured");
  if (narr != (int)s.S.h.arrays.size()) throw std::runtime_error("fortis_scatter: wrong number of arrays");
  cudaStream_t st = stream();
  int args[8];
  for (int i = 0; i < 8; i++) args[i] = i < nint ? iargs[i] : 1;
  ArrayTable T;
  bind_arrays(s.S, ptrs, args, nint, false, true, &T);
  RowGeom g = geom_all(rows);
  const long long count = g.count;
  g.nk = 1; g.kk0 = 0;
  const long long yoff = s.loop.kdist ? (long long)(args[0] - s.loop.klo) * count * s.model.n_out() : 0;
  if (s.loop.kdist && (args[0] < s.loop.klo || args[0] >= s.loop.klo + s.loop.nk))
    throw std::runtime_error("fortis_scatter: enclosing-loop index outside the distributed range");
  launch_scatter(s.S.hdr, (const StoreTarget*)s.S.items, s.S.h.n, T, g, s.dout + yoff, st);
  download_stores(s.S, args, nint, false);
  if (!s.async) cudaStreamSynchronize(st);
}

// byte ranges [lo, hi) of two arrays of a call overlap
bool ranges_overlap(const void* a, size_t na, const void* b, size_t nb) {
  const char *a0 = (const char*)a, *b0 = (const char*)b;
  return a0 < b0 + nb && b0 < a0 + na;
}

// Overlapped staging of a fused step over HOST arrays (the reference's per-call H2D of every plane and D2H of every
// visited rectangle, driver/fortis_gather_emit.py:66-68, 91-96, serialises copies and kernels on one stream).  For
// column layouts (one loop over the arrays' first, unit-stride dimension, no plane loop) the column range is cut into
// chunks: chunk c's slices of the input arrays go up on the H2D stream, the step kernels run on chunk c as soon as they
// have landed, and chunk c's slices of the stored arrays come back on the D2H stream while chunk c+1 computes and
// chunk c+2 uploads.  Returns false when the call is not of that shape (the caller then takes the serial path).
bool overlapped_step(void* const* gptrs, void* const* sptrs, long long rows) {
  Session& s = S();
  if (s.loop.kdist || s.loop.has_outer || s.loop.nk != 1 || !s.fuse || rows < 4096 || std::getenv("FORTIS_NO_OVERLAP")) return false;
  const long long ncol = rows;
  bool any_host = false;
  auto column_array = [&](const ArrayInfo& a) { return a.vdims.empty() && !a.shape.empty() && a.shape[0] == ncol && a.total % ncol == 0; };
  for (size_t ai = 0; ai < s.G.h.arrays.size(); ai++) {
    const ArrayInfo& a = s.G.h.arrays[ai];
    if (!a.used) continue;
    if (!column_array(a)) return false;
    if (!is_device_ptr(gptrs[ai]) && !maps_host(s.G)) any_host = true;
  }
  for (auto& x : s.G.h.slots) if (x.si != 1) return false;
  for (auto& x : s.G.h.scalars) if (x.si != 1) return false;
  for (size_t ai = 0; ai < s.S.h.arrays.size(); ai++) {
    const ArrayInfo& a = s.S.h.arrays[ai];
    if (!a.used) continue;
    if (!column_array(a) || !s.S.h.written[ai]) return false;       // arrays a scatter only reads would need a whole upload
    if (!is_device_ptr(sptrs[ai]) && !maps_host(s.S)) any_host = true;
  }
  for (auto& t : s.S.h.stores) if (t.a.si != 1) return false;
  if (!any_host || !ensure_copy_streams()) return false;

  cudaStream_t st = stream();
  // The pipeline is a fixed sequence of copies, kernels and event edges for a given set of array addresses: from the
  // second call on it is replayed as one CUDA graph (some 150 API calls per step otherwise, which would leave the GPU
  // waiting for the host).  Call 1 runs eagerly (it pins the arrays and sizes every buffer), call 2 is captured.
  std::string key((const char*)&rows, sizeof rows);
  key.append((const char*)gptrs, sizeof(void*) * s.G.h.arrays.size());
  key.append((const char*)sptrs, sizeof(void*) * s.S.h.arrays.size());
  if (s.ov_gexec && key == s.ov_key) {
    cuda_ok(cudaGraphLaunch(s.ov_gexec, st), "cudaGraphLaunch");
    if (!s.async) cudaStreamSynchronize(st);
    return true;
  }
  if (key != s.ov_key) {
    if (s.ov_gexec) { cudaGraphExecDestroy(s.ov_gexec); s.ov_gexec = nullptr; }
    s.ov_key = key; s.ov_calls = 0;
  }
  int args[8] = {1, 1, 1, 1, 1, 1, 1, 1};
  StepArgs A;
  A.use_gather = true; A.fuse_scatter = true;
  // pins the arrays, sizes the staging buffers; the copies themselves are issued per chunk below
  bind_arrays(s.G, gptrs, args, 0, false, false, &A.TG);
  bind_arrays(s.S, sptrs, args, 0, false, false, &A.TS);
  // Per-column vectors (one element per column) are not staged at all: a copy of a few hundred KB costs a copy's
  // latency (7-10 us each, and copies of one direction run one after another whatever their stream), which for a dozen
  // vectors is a tenth of the step.  The kernels load and store them through the pinned host pages instead; their
  // bytes cross the bus inside the launches, beside the chunk copies.
  auto map_vectors = [&](PlanDev& P, void* const* ptrs, ArrayTable& T) {
    for (size_t ai = 0; ai < P.h.arrays.size(); ai++) {
      const ArrayInfo& a = P.h.arrays[ai];
      if (!a.used || P.on_dev[ai] || a.total != ncol || P.reg[ai] != ptrs[ai]) continue;
      void* dp = nullptr;
      if (cudaHostGetDevicePointer(&dp, ptrs[ai], 0) == cudaSuccess && dp) { P.on_dev[ai] = true; T.base[ai] = dp; }
      else cudaGetLastError();
    }
  };
  if (!std::getenv("FORTIS_STAGE_VECTORS")) { map_vectors(s.G, gptrs, A.TG); map_vectors(s.S, sptrs, A.TS); }
  const ArrayTable TG0 = A.TG, TS0 = A.TS;
  // Chunk schedule: large chunks first, small ones last, so that what is left after the last upload (one forward
  // and one download) is short.  FORTIS_STAGING_CHUNKS overrides it with a list of relative weights ("2,2,2,1,1").
  std::vector<long long> weights;
  if (const char* e = std::getenv("FORTIS_STAGING_CHUNKS")) {
    for (const char* q = e; *q;) {
      char* end = nullptr;
      const long long w = std::strtoll(q, &end, 10);
      if (end == q) break;
      if (w > 0 && (int)weights.size() < kMaxChunks) weights.push_back(w);
      q = *end == ',' ? end + 1 : end;
    }
  }
  if (weights.empty()) {
    // measured on a PCIe 5 x16 link: a few large chunks (a copy of under 1 MB pays mostly latency) and a short tail
    if (ncol >= 40960) weights = {4, 4, 4, 2, 1, 1};
    else if (ncol >= 16384) weights = {2, 2, 1, 1};
    else weights = {1, 1};
  }
  long long wsum = 0;
  for (long long w : weights) wsum += w;
  std::vector<long long> cuts;                 // first column of every chunk, whole 128-row tiles
  {
    long long acc = 0;
    for (long long w : weights) {
      const long long c0 = (ncol * acc / wsum) / 128 * 128;
      if (cuts.empty() || c0 > cuts.back()) cuts.push_back(c0);
      acc += w;
    }
  }
  const int nchunks = (int)cuts.size();
  cuts.push_back(ncol);

  bool capturing = (++s.ov_calls == 2) && !std::getenv("FORTIS_NO_STAGING_GRAPH");
  if (capturing && cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); capturing = false; }
  if (capturing) fortis_capturing = 1;
  bool threw = false; std::string what;
  try {
    // fork: both copy streams start behind everything already on the persistent stream (the previous step included)
    cudaEventRecord(g_ev_fork, st);
    cudaStreamWaitEvent(g_h2d, g_ev_fork, 0);
    cudaStreamWaitEvent(g_d2h, g_ev_fork, 0);
    // per-column vectors that could not be mapped travel whole, ahead of the first chunk
    for (size_t ai = 0; ai < s.G.h.arrays.size(); ai++) {
      const ArrayInfo& a = s.G.h.arrays[ai];
      if (a.used && !s.G.on_dev[ai] && a.total == ncol)
        cuda_ok(cudaMemcpyAsync(s.G.stage[ai], gptrs[ai], (size_t)ncol * elt_size(a.elt), cudaMemcpyHostToDevice, g_h2d), "H2D of a column vector");
    }
    for (int c = 0; c < nchunks; c++) {
      const long long c0 = cuts[c], n = cuts[c + 1] - cuts[c];
      for (size_t ai = 0; ai < s.G.h.arrays.size(); ai++) {
        const ArrayInfo& a = s.G.h.arrays[ai];
        if (!a.used) continue;
        const size_t es = elt_size(a.elt);
        if (!s.G.on_dev[ai] && a.total != ncol)
          cuda_ok(cudaMemcpy2DAsync((char*)s.G.stage[ai] + c0 * es, (size_t)ncol * es, (const char*)gptrs[ai] + c0 * es, (size_t)ncol * es,
                                    (size_t)n * es, (size_t)(a.total / ncol), cudaMemcpyHostToDevice, g_h2d), "H2D of a column chunk");
        A.TG.base[ai] = (char*)TG0.base[ai] + c0 * es;
      }
      cudaEventRecord(g_ev_in[c], g_h2d);
      cudaStreamWaitEvent(st, g_ev_in[c], 0);
      for (size_t ai = 0; ai < s.S.h.arrays.size(); ai++)
        if (s.S.h.arrays[ai].used) A.TS.base[ai] = (char*)TS0.base[ai] + c0 * elt_size(s.S.h.arrays[ai].elt);
      A.rows = n;
      run_step_kernels(A);
      cudaEventRecord(g_ev_k[c], st);
      cudaStreamWaitEvent(g_d2h, g_ev_k[c], 0);
      for (size_t ai = 0; ai < s.S.h.arrays.size(); ai++) {
        const ArrayInfo& a = s.S.h.arrays[ai];
        if (!a.used || s.S.on_dev[ai]) continue;
        const size_t es = elt_size(a.elt);
        if (a.total != ncol)
          cuda_ok(cudaMemcpy2DAsync((char*)sptrs[ai] + c0 * es, (size_t)ncol * es, (const char*)s.S.stage[ai] + c0 * es, (size_t)ncol * es,
                                    (size_t)n * es, (size_t)(a.total / ncol), cudaMemcpyDeviceToHost, g_d2h), "D2H of a column chunk");
      }
    }
    // unmapped vectors come back whole behind the last chunk
    for (size_t ai = 0; ai < s.S.h.arrays.size(); ai++) {
      const ArrayInfo& a = s.S.h.arrays[ai];
      if (a.used && !s.S.on_dev[ai] && a.total == ncol)
        cuda_ok(cudaMemcpyAsync(sptrs[ai], s.S.stage[ai], (size_t)ncol * elt_size(a.elt), cudaMemcpyDeviceToHost, g_d2h), "D2H of a column vector");
    }
    // join: the persistent stream continues behind the last upload and the last download
    cudaEventRecord(g_ev_join_in, g_h2d);
    cudaStreamWaitEvent(st, g_ev_join_in, 0);
    cudaEventRecord(g_ev_join_out, g_d2h);
    cudaStreamWaitEvent(st, g_ev_join_out, 0);
  } catch (const std::exception& e) { threw = true; what = e.what(); }
  if (capturing) {
    fortis_capturing = 0;
    cudaGraph_t gr = nullptr;
    const bool ok = cudaStreamEndCapture(st, &gr) == cudaSuccess && !threw && cudaGraphInstantiate(&s.ov_gexec, gr, 0) == cudaSuccess;
    if (gr) cudaGraphDestroy(gr);
    if (ok) cuda_ok(cudaGraphLaunch(s.ov_gexec, st), "cudaGraphLaunch");
    else {
      s.ov_gexec = nullptr; cudaGetLastError();
      if (threw) throw std::runtime_error(what);
      std::fprintf(stderr, "fortis: capture of the staging pipeline failed, running eagerly\n");
      s.ov_calls = 2;                                   // do not try again for this set of arrays
      return overlapped_step(gptrs, sptrs, rows);
    }
  } else if (threw) throw std::runtime_error(what);
  if (!s.async) cudaStreamSynchronize(st);
  return true;
}

// The same pipelining for k-distributed loops over HOST arrays (stencil hosts: every array carries the distributed
// loop's plane dimension): plane k+1 goes up while plane k is computed and the visited rectangle of plane k-1 comes
// back (driver/fortis_gather_emit.py:66-68, 91-96 moves all planes up, then computes, then copies back rectangle by
// rectangle on one stream).  A plane is contiguous, so the uploads are plain 1-D copies; planes are independent (the
// stencil is within a plane), so a plane is a step of its own with nk = 1.  Replayed as one graph from the second call.
bool overlapped_planes_step(void* const* gptrs, void* const* sptrs) {
  Session& s = S();
  if (!s.loop.kdist || s.loop.nk < 2 || s.loop.nk > kMaxChunks || !s.fuse || std::getenv("FORTIS_NO_OVERLAP")) return false;
  bool any_host = false;
  for (size_t ai = 0; ai < s.G.h.arrays.size(); ai++) {
    const ArrayInfo& a = s.G.h.arrays[ai];
    if (!a.used) continue;
    if (a.vdims.empty()) return false;
    if (!is_device_ptr(gptrs[ai]) && !maps_host(s.G)) any_host = true;
  }
  for (size_t ai = 0; ai < s.S.h.arrays.size(); ai++) {
    const ArrayInfo& a = s.S.h.arrays[ai];
    if (!a.used) continue;
    if (a.vdims.empty() || !s.S.h.written[ai]) return false;
    if (!is_device_ptr(sptrs[ai]) && !maps_host(s.S)) any_host = true;
  }
  if (!any_host || !ensure_copy_streams()) return false;
  cudaStream_t st = stream();
  const int nk = s.loop.nk;
  std::string key("planes");
  key.append((const char*)gptrs, sizeof(void*) * s.G.h.arrays.size());
  key.append((const char*)sptrs, sizeof(void*) * s.S.h.arrays.size());
  if (s.ov_gexec && key == s.ov_key) {
    cuda_ok(cudaGraphLaunch(s.ov_gexec, st), "cudaGraphLaunch");
    if (!s.async) cudaStreamSynchronize(st);
    return true;
  }
  if (key != s.ov_key) {
    if (s.ov_gexec) { cudaGraphExecDestroy(s.ov_gexec); s.ov_gexec = nullptr; }
    s.ov_key = key; s.ov_calls = 0;
  }
  int args[8] = {1, 1, 1, 1, 1, 1, 1, 1};
  StepArgs A;
  A.use_gather = true; A.fuse_scatter = true;
  bind_arrays(s.G, gptrs, args, 0, true, false, &A.TG);          // pins, sizes the staging of all planes; no copies
  bind_arrays(s.S, sptrs, args, 0, true, false, &A.TS);
  const ArrayTable TG0 = A.TG, TS0 = A.TS;
  const LoopInfo saved = s.loop;
  bool capturing = (++s.ov_calls == 2) && !std::getenv("FORTIS_NO_STAGING_GRAPH");
  if (capturing && cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); capturing = false; }
  if (capturing) fortis_capturing = 1;
  bool threw = false; std::string what;
  try {
    cudaEventRecord(g_ev_fork, st);
    cudaStreamWaitEvent(g_h2d, g_ev_fork, 0);
    cudaStreamWaitEvent(g_d2h, g_ev_fork, 0);
    for (int kk = 0; kk < nk; kk++) {
      for (size_t ai = 0; ai < s.G.h.arrays.size(); ai++) {
        const ArrayInfo& a = s.G.h.arrays[ai];
        if (!a.used) continue;
        const size_t es = elt_size(a.elt);
        const long long off = (long long)kk * a.plane;
        if (!s.G.on_dev[ai])
          cuda_ok(cudaMemcpyAsync((char*)s.G.stage[ai] + off * es, (const char*)gptrs[ai] + ((long long)(saved.klo - 1) * a.plane + off) * es,
                                  (size_t)a.plane * es, cudaMemcpyHostToDevice, g_h2d), "H2D of a plane");
        A.TG.base[ai] = (char*)TG0.base[ai] + off * es;
      }
      cudaEventRecord(g_ev_in[kk], g_h2d);
      cudaStreamWaitEvent(st, g_ev_in[kk], 0);
      for (size_t ai = 0; ai < s.S.h.arrays.size(); ai++)
        if (s.S.h.arrays[ai].used) A.TS.base[ai] = (char*)TS0.base[ai] + (long long)kk * s.S.h.arrays[ai].plane * elt_size(s.S.h.arrays[ai].elt);
      A.rows = saved.count;
      s.loop.nk = 1;                                   // one plane is a step of its own
      run_step_kernels(A);
      s.loop = saved;
      cudaEventRecord(g_ev_k[kk], st);
      cudaStreamWaitEvent(g_d2h, g_ev_k[kk], 0);
      download_stores(s.S, args, 0, true, g_d2h, kk, kk + 1);
    }
    cudaEventRecord(g_ev_join_in, g_h2d);
    cudaStreamWaitEvent(st, g_ev_join_in, 0);
    cudaEventRecord(g_ev_join_out, g_d2h);
    cudaStreamWaitEvent(st, g_ev_join_out, 0);
  } catch (const std::exception& e) { threw = true; what = e.what(); s.loop = saved; }
  if (capturing) {
    fortis_capturing = 0;
    cudaGraph_t gr = nullptr;
    const bool ok = cudaStreamEndCapture(st, &gr) == cudaSuccess && !threw && cudaGraphInstantiate(&s.ov_gexec, gr, 0) == cudaSuccess;
    if (gr) cudaGraphDestroy(gr);
    if (ok) cuda_ok(cudaGraphLaunch(s.ov_gexec, st), "cudaGraphLaunch");
    else {
      s.ov_gexec = nullptr; cudaGetLastError();
      if (threw) throw std::runtime_error(what);
      std::fprintf(stderr, "fortis: capture of the staging pipeline failed, running eagerly\n");
      s.ov_calls = 2;
      return overlapped_planes_step(gptrs, sptrs);
    }
  } else if (threw) throw std::runtime_error(what);
  if (!s.async) cudaStreamSynchronize(st);
  return true;
}

// The fused step: gather -> forward -> scatter of every plane in one launch.  `iargs` are the enclosing-loop
// indices (1-based) that select the plane of arrays with "v" subscripts when the loop is NOT k-distributed; a
// k-distributed loop takes none (all planes klo .. klo+nk-1 are processed).
void do_step(const int* iargs, int nint, void* const* gptrs, int ng, void* const* sptrs, int ns) {
  Session& s = S();
  long long rows;
  prepare(&rows);
  if (!s.G.h.ok || !s.S.h.ok) throw std::runtime_error("fortis_step: needs both a gather and a scatter descriptor");
  if (ng != (int)s.G.h.arrays.size() || ns != (int)s.S.h.arrays.size()) throw std::runtime_error("fortis_step: wrong number of arrays");
  if (s.loop.nk > 1)
    for (auto& t : s.S.h.stores)
      if (s.S.h.arrays[t.a.array].vdims.empty())
        throw std::runtime_error("fortis_step: stored array " + s.S.h.arrays[t.a.array].name +
                                 " has no plane dimension; the host consumes it between planes, use fortis_scatter per plane");
  const bool multi = s.loop.kdist;
  if (!multi) {
    // planes are chosen by the integer arguments, as in fortis_gather / fortis_scatter: every argument a used
    // array's "v" subscript names must be there, else the plane would be a guess
    int need = 0;
    for (PlanDev* P : {&s.G, &s.S})
      for (auto& a : P->h.arrays)
        if (a.used) for (auto& t : a.vterms) need = t.first + 1 > need ? t.first + 1 : need;
    if (nint < need)
      throw std::runtime_error("fortis_step: the descriptors select a plane by " + std::to_string(need) +
                               " enclosing-loop index argument(s) and the loop is not k-distributed; pass them first");
  }
  // a device-resident gather array that shares memory with a device-resident stored array forces the unfused sequence
  // below; the pipelined staging paths run fused kernels, so they are not taken then
  bool dev_overlap = false;
  for (size_t gi = 0; gi < s.G.h.arrays.size() && !dev_overlap; gi++) {
    if (!s.G.h.arrays[gi].used || !is_device_ptr(gptrs[gi])) continue;
    const ArrayInfo& ga = s.G.h.arrays[gi];
    for (size_t si = 0; si < s.S.h.arrays.size(); si++) {
      if (!s.S.h.written[si] || !is_device_ptr(sptrs[si])) continue;
      const ArrayInfo& sa = s.S.h.arrays[si];
      if (ranges_overlap(gptrs[gi], (size_t)ga.total * elt_size(ga.elt), sptrs[si], (size_t)sa.total * elt_size(sa.elt))) { dev_overlap = true; break; }
    }
  }
  if (!dev_overlap && (overlapped_step(gptrs, sptrs, rows) || overlapped_planes_step(gptrs, sptrs))) return;
  cudaStream_t st = stream();
  int args[8];
  for (int i = 0; i < 8; i++) args[i] = i < nint ? iargs[i] : 1;
  StepArgs A;
  A.rows = rows; A.use_gather = true; A.fuse_scatter = true;
  bind_arrays(s.G, gptrs, args, nint, multi, true, &A.TG);
  bind_arrays(s.S, sptrs, args, nint, multi, true, &A.TS);
  // A fused kernel reads its inputs and writes its outputs in the same launch.  When a device-resident gather array
  // shares memory with a device-resident stored array, a stencil would read neighbours another thread is
  // overwriting; the reference is well-defined there because gather and scatter work on separate staging copies.
  // Such a call runs as separate gather, forward and scatter kernels (host-resident arrays are staged separately
  // anyway).
  for (size_t gi = 0; gi < s.G.h.arrays.size() && !A.unfused; gi++) {
    if (!s.G.on_dev[gi] || !s.G.h.arrays[gi].used) continue;
    const ArrayInfo& ga = s.G.h.arrays[gi];
    for (size_t si = 0; si < s.S.h.arrays.size(); si++) {
      if (!s.S.on_dev[si] || !s.S.h.written[si]) continue;
      const ArrayInfo& sa = s.S.h.arrays[si];
      if (ranges_overlap(gptrs[gi], (size_t)ga.total * elt_size(ga.elt), sptrs[si], (size_t)sa.total * elt_size(sa.elt))) { A.unfused = true; break; }
    }
  }
  run_step(A);
  download_stores(s.S, args, nint, multi);
  if (!s.async) cudaStreamSynchronize(st);
}

#define FORTIS_TRY try {
#define FORTIS_CATCH(ret) } catch (const std::exception& e) { set_error(e.what()); ret; }

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// exported entries
// ---------------------------------------------------------------------------------------------------------------
extern "C" {

void* mgpuStreamCreate(void) { return (void*)stream(); }
void mgpuStreamDestroy(void*) {}
void mgpuStreamSynchronize(void*) {}

void* fortis_alloc(long n) { return pool_alloc(n); }
void fortis_free(void* p) { pool_free(p); }

int fortis_last_error(void) { return g_err; }
const char* fortis_last_error_message(void) { return g_errmsg.c_str(); }
void fortis_sync(void) { cudaStreamSynchronize(stream()); }

int fortis_configure(const char* key, const char* text) {
  FORTIS_TRY
  Session& s = S();
  const std::string k = key ? key : "";
  JValue v = parse_json(text ? text : "");
  if (k == "gather") { s.jg = v; s.have_g = true; }
  else if (k == "scatter") { s.js = v; s.have_s = true; }
  else if (k == "loop") { s.jl = v; s.have_l = true; }
  else if (k == "kdist") { s.jk = v; s.have_k = true; }
  else if (k == "lift2d") { s.jl2 = v; s.have_l2 = true; }
  else throw std::runtime_error("fortis_configure: unknown key \"" + k + "\"");
  s.planned = false;
  g_err = 0;
  return 0;
  FORTIS_CATCH(return -1)
}

int fortis_configure_file(const char* key, const char* path) {
  FORTIS_TRY
  const std::string text = read_file(path ? path : "");
  return fortis_configure(key, text.c_str());
  FORTIS_CATCH(return -1)
}

int fortis_set_vector(const char* name, const void* data, long n, int elt) {
  FORTIS_TRY
  if (!name || !data || n <= 0) throw std::runtime_error("fortis_set_vector: bad arguments");
  std::vector<char> bytes((size_t)n * elt_size(elt));
  std::memcpy(bytes.data(), data, bytes.size());
  S().vectors[name] = std::make_pair(std::move(bytes), elt);
  S().planned = false;
  return 0;
  FORTIS_CATCH(return -1)
}

int fortis_load_model_mem(const void* blob, long nbytes) {
  FORTIS_TRY
  Session& s = S();
  ModelHost M = parse_model_blob(blob, (size_t)nbytes);
  free_model_dev();
  s.model = std::move(M);
  s.have_model = true;
  pool_free(s.din); pool_free(s.dout); pool_free(s.act0); pool_free(s.act1);
  s.din = s.dout = s.act0 = s.act1 = nullptr; s.buf_rows = 0;
  g_err = 0;
  return 0;
  FORTIS_CATCH(return -1)
}

int fortis_load_model(const char* path) {
  FORTIS_TRY
  const std::string b = read_file(path ? path : "");
  return fortis_load_model_mem(b.data(), (long)b.size());
  FORTIS_CATCH(return -1)
}

int fortis_set_option(const char* key, const char* value) {
  FORTIS_TRY
  Session& s = S();
  const std::string k = key ? key : "", v = value ? value : "";
  if (k == "precision") {
    int p;
    if (v == "fp32" || v == "f32") p = PREC_F32;
    else if (v == "bf16") p = PREC_BF16;
    else if (v == "fp8w") p = PREC_FP8W;
    else if (v == "fp16" || v == "f16") p = PREC_FP16;
    else throw std::runtime_error("precision must be fp32, bf16, fp16 or fp8w");
    if (p != s.precision) { s.precision = p; free_model_dev(); }
  } else if (k == "fuse") { s.fuse = v != "0"; drop_graph(); }
  else if (k == "graph") { s.graph = v != "0"; drop_graph(); }
  else if (k == "async") { s.async = v != "0"; }
  else if (k == "stencil_tc") { s.use_stencil_tc = v != "0"; drop_graph(); }
  else if (k == "tc_pair") { tc_set_pair_mode(v == "default" ? -1 : (v != "0")); free_model_dev(); drop_graph(); }
  else if (k == "host_access") {
    if (v == "copy") s.host_access = 0;
    else if (v == "mapped_out") s.host_access = 1;
    else if (v == "mapped") s.host_access = 2;
    else throw std::runtime_error("host_access must be copy, mapped_out or mapped");
    drop_graph();
  }
  else if (k == "checksum") { s.want_checksum = v != "0"; drop_graph(); }
  else if (k == "test_wait_limit") { g_tc_test.wait_limit = (unsigned int)std::strtoul(v.c_str(), nullptr, 10); drop_graph(); }
  else if (k == "test_skip_stage") { g_tc_test.skip_stage = v != "0"; drop_graph(); }
  else if (k == "test_no_stage") { g_tc_test.no_stage = v != "0"; drop_graph(); }
  else if (k == "conv_shape") {
    if (std::sscanf(v.c_str(), "%d,%d,%d,%d", &s.conv_shape[0], &s.conv_shape[1], &s.conv_shape[2], &s.conv_shape[3]) != 4)
      throw std::runtime_error("conv_shape must be N,D,H,W");
    s.buf_rows = 0;
  } else throw std::runtime_error("fortis_set_option: unknown option \"" + k + "\"");
  return 0;
  FORTIS_CATCH(return -1)
}

void fortis_reset(void) {
  g_tc_test = TcTestKnobs{0u, 0, 0};
  tc_set_pair_mode(-1);
  if (!g_S) return;
  if (g_stream) cudaStreamSynchronize(g_stream);
  Session& s = S();
  drop_graph();
  free_plan(s.G); free_plan(s.S);
  free_model_dev();
  pool_free(s.din); pool_free(s.dout); pool_free(s.act0); pool_free(s.act1);
  pool_free(s.d_partials); pool_free(s.d_sum); pool_free(s.d_status); pool_free(s.d_done);
  if (s.X_pinned) cudaFreeHost(s.X_pinned);
  if (s.Y_pinned) cudaFreeHost(s.Y_pinned);
  if (s.reg_in) cudaHostUnregister((void*)s.reg_in);
  if (s.reg_out) cudaHostUnregister((void*)s.reg_out);
  cudaGetLastError();
  delete g_S;
  g_S = nullptr;
  g_err = 0;
  g_errmsg.clear();
}

void fortis_begin(int count) {
  Session& s = S();
  if (s.begin_count != count) { s.begin_count = count; drop_graph(); }
}

void* fortis_model_input(void) {
  FORTIS_TRY
  Session& s = S();
  long long rows;
  prepare(&rows);
  if (s.gather_pending) {     // make the buffer valid for a caller that consumes X itself
    launch_gather(s.G.hdr, (const Access*)s.G.items, s.G.h.n, current_gather_table(), geom_all(rows), s.din, stream());
    s.gather_pending = false;
    s.gather_done = true;       // the model input is materialised; the next mlp_forward_batched() consumes it
  }
  return s.din;
  FORTIS_CATCH(return nullptr)
}

void* fortis_model_output(void) {
  FORTIS_TRY
  long long rows;
  prepare(&rows);
  return S().dout;
  FORTIS_CATCH(return nullptr)
}

void fortis_gatherv(const int* iargs, int nint, const void* const* arrays, int narrays) {
  FORTIS_TRY
  do_gather(iargs, nint, (void* const*)arrays, narrays);
  FORTIS_CATCH(return)
}

void fortis_scatterv(const int* iargs, int nint, void* const* arrays, int narrays) {
  FORTIS_TRY
  do_scatter(iargs, nint, arrays, narrays);
  FORTIS_CATCH(return)
}

void fortis_stepv(const void* const* ga, int ng, void* const* sa, int ns) {
  FORTIS_TRY
  do_step(nullptr, 0, (void* const*)ga, ng, sa, ns);
  FORTIS_CATCH(return)
}

void fortis_stepvi(const int* iargs, int nint, const void* const* ga, int ng, void* const* sa, int ns) {
  FORTIS_TRY
  do_step(iargs, nint, (void* const*)ga, ng, sa, ns);
  FORTIS_CATCH(return)
}

void fortis_gather(long a0, ...) {
  FORTIS_TRY
  ensure_plans();
  Session& s = S();
  if (!s.G.h.ok) throw std::runtime_error("fortis_gather: no gather descriptor is configured");
  std::vector<int> ints; std::vector<void*> ptrs;
  va_list ap; va_start(ap, a0);
  collect_args(s.G, s.loop.kdist, a0, ap, true, &ints, &ptrs);   // no integer arguments under kdist (emit :63)
  va_end(ap);
  do_gather(ints.data(), (int)ints.size(), ptrs.data(), (int)ptrs.size());
  FORTIS_CATCH(return)
}

void fortis_scatter(long a0, ...) {
  FORTIS_TRY
  ensure_plans();
  Session& s = S();
  if (!s.S.h.ok) throw std::runtime_error("fortis_scatter: no scatter descriptor is configured");
  std::vector<int> ints; std::vector<void*> ptrs;
  va_list ap; va_start(ap, a0);
  collect_args(s.S, false, a0, ap, true, &ints, &ptrs);
  va_end(ap);
  do_scatter(ints.data(), (int)ints.size(), ptrs.data(), (int)ptrs.size());
  FORTIS_CATCH(return)
}

void fortis_step(long a0, ...) {
  FORTIS_TRY
  ensure_plans();
  Session& s = S();
  if (!s.G.h.ok || !s.S.h.ok) throw std::runtime_error("fortis_step: needs both a gather and a scatter descriptor");
  // [the gather entry's integer arguments unless the loop is k-distributed], gather arrays, scatter arrays
  std::vector<int> ints; std::vector<void*> g, sc;
  va_list ap; va_start(ap, a0);
  collect_args(s.G, s.loop.kdist, a0, ap, true, &ints, &g);
  for (size_t i = 0; i < s.S.h.arrays.size(); i++) sc.push_back(va_arg(ap, void*));
  va_end(ap);
  do_step(ints.data(), (int)ints.size(), g.data(), (int)g.size(), sc.data(), (int)sc.size());
  FORTIS_CATCH(return)
}

void mlp_forward_batched(void* in, void* out) {
  FORTIS_TRY
  do_forward_batched(in, out);
  FORTIS_CATCH(return)
}

void mlp_upload(void* in) {
  FORTIS_TRY
  Session& s = S();
  long long rows;
  prepare(&rows);
  cuda_ok(cudaMemcpy(s.din, in, rows * s.model.n_in() * 4, is_device_ptr(in) ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice), "mlp_upload");
  FORTIS_CATCH(return)
}

void mlp_forward_dev(void) {
  FORTIS_TRY
  long long rows;
  prepare(&rows);
  StepArgs A;
  A.rows = rows;
  run_step(A);
  FORTIS_CATCH(return)
}

void mlp_download(void* out) {
  FORTIS_TRY
  Session& s = S();
  long long rows;
  prepare(&rows);
  cudaStreamSynchronize(stream());
  cuda_ok(cudaMemcpy(out, s.dout, out_floats(rows) * 4, is_device_ptr(out) ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost), "mlp_download");
  FORTIS_CATCH(return)
}

void mlp_forward(void* in, void* out) {
  FORTIS_TRY
  Session& s = S();
  ensure_plans();
  if (s.have_l2) {
    // boundary verdict: the host's own arrays, their element type and memory order; pinned once
    // (driver/fortis_shim.py:123-133); transpose + cast + lifted expressions run fused around the model
    void* gp[1] = {in};
    void* sp[1] = {out};
    do_step(nullptr, 0, gp, 1, sp, 1);
    cudaStreamSynchronize(stream());
    return;
  }
  ensure_model();
  const long long nin = s.model.n_in(), nout = s.model.n_out();
  cudaStream_t st = stream();
  if (s.have_l) {
    // batched verdict: single-row entry for calls outside the loop (driver/fortis_shim.py:122)
    const long long keep = s.begin_count; const bool had_l = s.have_l;
    ensure_buffers(model_rows());
    cuda_ok(cudaMemcpyAsync(s.din, in, nin * 4, cudaMemcpyDefault, st), "H2D of one row");
    StepArgs A; A.rows = 1;
    const LoopInfo saved = s.loop;
    s.loop.nk = 1; s.loop.count = 1; s.loop.ni = 1;
    try { run_step_kernels(A); } catch (...) { s.loop = saved; throw; }
    s.loop = saved; (void)keep; (void)had_l;
    cuda_ok(cudaMemcpyAsync(out, s.dout, nout * 4, cudaMemcpyDefault, st), "D2H of one row");
    cudaStreamSynchronize(st);
    return;
  }
  // whole-array call without a boundary: row-major (batch, n_in) -> (batch, n_out), pinned once
  long long rows;
  prepare(&rows);
  auto pin = [&](const void** reg, void* p, size_t n) {
    if (s.nopin || *reg == p || std::getenv("FORTIS_NO_PIN") || is_device_ptr(p)) return;
    if (*reg) { cudaHostUnregister((void*)*reg); *reg = nullptr; s.nopin = true; cudaGetLastError(); return; }
    *reg = cudaHostRegister(p, n, cudaHostRegisterDefault) == cudaSuccess ? p : nullptr;
    if (!*reg) cudaGetLastError();
  };
  pin(&s.reg_in, in, (size_t)rows * nin * 4);
  pin(&s.reg_out, out, (size_t)out_floats(rows) * 4);
  cuda_ok(cudaMemcpyAsync(s.din, in, rows * nin * 4, cudaMemcpyDefault, st), "H2D of the input");
  StepArgs A; A.rows = rows;
  run_step(A);
  cuda_ok(cudaMemcpyAsync(out, s.dout, out_floats(rows) * 4, cudaMemcpyDefault, st), "D2H of the output");
  cudaStreamSynchronize(st);
  FORTIS_CATCH(return)
}

static void ensure_pinned(long long rows) {
  Session& s = S();
  if (s.X_pinned && s.pinned_rows >= rows) return;
  if (s.X_pinned) cudaFreeHost(s.X_pinned);
  if (s.Y_pinned) cudaFreeHost(s.Y_pinned);
  cuda_ok(cudaHostAlloc((void**)&s.X_pinned, (size_t)rows * s.model.n_in() * 4, cudaHostAllocDefault), "cudaHostAlloc X");
  cuda_ok(cudaHostAlloc((void**)&s.Y_pinned, (size_t)rows * s.model.n_out() * 4, cudaHostAllocDefault), "cudaHostAlloc Y");
  s.pinned_rows = rows;
}

void fortis_pack(void* f, int col) {
  FORTIS_TRY
  Session& s = S();
  long long rows;
  prepare(&rows);
  ensure_pinned(rows);
  if (col < 0 || col >= rows) throw std::runtime_error("fortis_pack: column out of range");
  std::memcpy(s.X_pinned + (size_t)col * s.model.n_in(), f, (size_t)s.model.n_in() * 4);
  s.pack_pending = true;
  FORTIS_CATCH(return)
}

void fortis_unpack(void* o, int col) {
  FORTIS_TRY
  Session& s = S();
  long long rows;
  prepare(&rows);
  ensure_pinned(rows);
  if (col < 0 || col >= rows) throw std::runtime_error("fortis_unpack: column out of range");
  std::memcpy(o, s.Y_pinned + (size_t)col * s.model.n_out(), (size_t)s.model.n_out() * 4);
  FORTIS_CATCH(return)
}

void fortis_gemm(float* Aa, float* A, long Ao, long As0, long As1, long At0, long At1,
                 float* Wa, float* W, long Wo, long Ws0, long Ws1, long Wt0, long Wt1,
                 float* Ca, float* C, long Co, long Cs0, long Cs1, long Ct0, long Ct1, long B, long N, long K) {
  (void)Aa; (void)As0; (void)As1; (void)Wa; (void)Ws0; (void)Ws1; (void)Ca; (void)Cs0; (void)Cs1;
  // The kernels (like the reference's cuBLAS call) address dense row-major operands; a strided memref would be
  // computed wrong without a word, so it is refused instead and C is left untouched.
  auto dense = [](long t0, long t1, long rows, long cols) { return (cols <= 1 || t1 == 1) && (rows <= 1 || t0 == cols); };
  if (!dense(At0, At1, B, K) || !dense(Wt0, Wt1, N, K) || !dense(Ct0, Ct1, B, N)) {
    std::fprintf(stderr, "fortis_gemm: operands must be dense row-major (A %ldx%ld strides %ld,%ld; W %ldx%ld strides %ld,%ld; C %ldx%ld strides %ld,%ld)\n",
                 B, K, At0, At1, N, K, Wt0, Wt1, B, N, Ct0, Ct1);
    return;
  }
  if (B >= kF32TcMinRows) {
    // large batch: the tensor-core kernel (three TF32 MMAs per product, fp32-class accuracy)
    S();
    ensure_aux(1);
    std::string err;
    if (f32tc_gemm(A + Ao, W + Wo, C + Co, B, (int)N, (int)K, S().d_status, stream(), &err)) return;
    std::fprintf(stderr, "fortis_gemm: %s; using the FFMA kernel\n", err.c_str());
  }
  launch_linear_f32(A + Ao, W + Wo, nullptr, C + Co, B, (int)N, (int)K, ACT_NONE, 0.f, nullptr, nullptr, nullptr, stream());
}

// dense NCDHW-style strides of a rank-5 memref (dimensions of extent 1 may carry any stride)
static bool dense5(const long* t, long n0, long n1, long n2, long n3, long n4) {
  const long want[5] = {n1 * n2 * n3 * n4, n2 * n3 * n4, n3 * n4, n4, 1}, ext[5] = {n0, n1, n2, n3, n4};
  for (int d = 0; d < 5; d++) if (ext[d] > 1 && t[d] != want[d]) return false;
  return true;
}

// One convolution layer through the memref ABI.  `max_k` > 0 and `unit_stride` reproduce the refusals of the
// reference entry being replaced (message on stderr, y untouched).
static void conv3d_entry(const char* who, float* x, long xo, float* w, long wo, float* y, long yo, long N, long C, long Din, long Hin,
                         long Win, long F, long KD, long KH, long KW, long Dout, long Hout, long Wout, long sd, long sh, long sw,
                         long pd, long ph, long pw, const long* xt, const long* wt, const long* yt, bool unit_stride, long max_k,
                         bool no_pad) {
  if (!dense5(xt, N, C, Din, Hin, Win) || !dense5(wt, F, C, KD, KH, KW) || !dense5(yt, N, F, Dout, Hout, Wout)) {
    std::fprintf(stderr, "%s: operands must be dense NCDHW / FCKKK memrefs\n", who);
    return;
  }
  const bool sane = N > 0 && C > 0 && F > 0 && KD > 0 && KH > 0 && KW > 0 && sd > 0 && sh > 0 && sw > 0 && pd >= 0 && ph >= 0 && pw >= 0 &&
                    Din + 2 * pd >= KD && Hin + 2 * ph >= KH && Win + 2 * pw >= KW &&
                    Dout == (Din + 2 * pd - KD) / sd + 1 && Hout == (Hin + 2 * ph - KH) / sh + 1 && Wout == (Win + 2 * pw - KW) / sw + 1;
  if (!sane || (unit_stride && (sd != 1 || sh != 1 || sw != 1)) || (max_k > 0 && (KD > max_k || KH > max_k || KW > max_k)) ||
      (no_pad && (pd || ph || pw))) {
    std::fprintf(stderr, "%s: unsupported shape\n", who);
    return;
  }
  const int K[3] = {(int)KD, (int)KH, (int)KW}, st[3] = {(int)sd, (int)sh, (int)sw}, pad[3] = {(int)pd, (int)ph, (int)pw};
  std::string err;
  if (!conv3d_ncdhw(x + xo, w + wo, y + yo, (int)N, (int)C, (int)Din, (int)Hin, (int)Win, (int)F, K, st, pad, stream(), &err))
    std::fprintf(stderr, "%s: %s\n", who, err.c_str());
}

#define FORTIS_MEMREF5_UNUSED \
  (void)xa; (void)x0; (void)x1; (void)x2; (void)x3; (void)x4; (void)wa; (void)w0; (void)w1; (void)w2; (void)w3; (void)w4; \
  (void)ya; (void)y0; (void)y1; (void)y2; (void)y3; (void)y4; \
  const long xt[5] = {xt0, xt1, xt2, xt3, xt4}, wt[5] = {wt0, wt1, wt2, wt3, wt4}, yt[5] = {yt0, yt1, yt2, yt3, yt4}

// any kernel extent, stride and padding (the reference hands these to cuDNN)
void fortis_conv3d(float* xa, float* x, long xo, long x0, long x1, long x2, long x3, long x4, long xt0, long xt1, long xt2, long xt3, long xt4,
                   float* wa, float* w, long wo, long w0, long w1, long w2, long w3, long w4, long wt0, long wt1, long wt2, long wt3, long wt4,
                   float* ya, float* y, long yo, long y0, long y1, long y2, long y3, long y4, long yt0, long yt1, long yt2, long yt3, long yt4,
                   long N, long C, long Din, long Hin, long Win, long F, long KD, long KH, long KW, long Dout, long Hout, long Wout,
                   long sd, long sh, long sw, long pd, long ph, long pw) {
  FORTIS_MEMREF5_UNUSED;
  conv3d_entry("fortis_conv3d", x, xo, w, wo, y, yo, N, C, Din, Hin, Win, F, KD, KH, KW, Dout, Hout, Wout, sd, sh, sw, pd, ph, pw, xt, wt, yt,
               false, 0, false);
}

// stride 1 and kernels up to 5 per axis only, as the reference's direct kernels (runtime/fortis_fft.cu:135); N > 1 is taken
void fortis_conv3d_direct(float* xa, float* x, long xo, long x0, long x1, long x2, long x3, long x4, long xt0, long xt1, long xt2, long xt3, long xt4,
                   float* wa, float* w, long wo, long w0, long w1, long w2, long w3, long w4, long wt0, long wt1, long wt2, long wt3, long wt4,
                   float* ya, float* y, long yo, long y0, long y1, long y2, long y3, long y4, long yt0, long yt1, long yt2, long yt3, long yt4,
                   long N, long C, long Din, long Hin, long Win, long F, long KD, long KH, long KW, long Dout, long Hout, long Wout,
                   long sd, long sh, long sw, long pd, long ph, long pw) {
  FORTIS_MEMREF5_UNUSED;
  conv3d_entry("fortis_conv3d_direct", x, xo, w, wo, y, yo, N, C, Din, Hin, Win, F, KD, KH, KW, Dout, Hout, Wout, sd, sh, sw, pd, ph, pw, xt,
               wt, yt, true, 5, false);
}

// The entry the compiler picks for kernels of 5^3 taps and more (compiler/FortisFuse.cpp, runtime/fortis_fft.cu:66-79:
// stride 1, no padding).  The result is the same convolution; here it is computed directly, in fp32, by the implicit
// GEMM (no transform, no spectrum buffers, no round-off of a forward and an inverse FFT).
void fortis_conv3d_fft(float* xa, float* x, long xo, long x0, long x1, long x2, long x3, long x4, long xt0, long xt1, long xt2, long xt3, long xt4,
                   float* wa, float* w, long wo, long w0, long w1, long w2, long w3, long w4, long wt0, long wt1, long wt2, long wt3, long wt4,
                   float* ya, float* y, long yo, long y0, long y1, long y2, long y3, long y4, long yt0, long yt1, long yt2, long yt3, long yt4,
                   long N, long C, long Din, long Hin, long Win, long F, long KD, long KH, long KW, long Dout, long Hout, long Wout,
                   long sd, long sh, long sw, long pd, long ph, long pw) {
  FORTIS_MEMREF5_UNUSED;
  conv3d_entry("fortis_conv3d_fft", x, xo, w, wo, y, yo, N, C, Din, Hin, Win, F, KD, KH, KW, Dout, Hout, Wout, sd, sh, sw, pd, ph, pw, xt, wt,
               yt, true, 0, true);
}

// NCHW convolution (runtime/fortis_rt.c:108-127): the D = KD = 1 case of the same kernel
void fortis_conv2d(float* xa, float* x, long xo, long x0, long x1, long x2, long x3, long xt0, long xt1, long xt2, long xt3,
                   float* wa, float* w, long wo, long w0, long w1, long w2, long w3, long wt0, long wt1, long wt2, long wt3,
                   float* ya, float* y, long yo, long y0, long y1, long y2, long y3, long yt0, long yt1, long yt2, long yt3,
                   long N, long C, long Hin, long Win, long F, long KH, long KW, long Hout, long Wout, long sh, long sw, long ph, long pw) {
  (void)xa; (void)x0; (void)x1; (void)x2; (void)x3; (void)wa; (void)w0; (void)w1; (void)w2; (void)w3; (void)ya; (void)y0; (void)y1; (void)y2; (void)y3;
  // a dense 4-d memref is a dense 5-d one with a unit depth axis (its stride never multiplies anything but 0)
  const long xt[5] = {xt0, xt1, Hin * Win, xt2, xt3}, wt[5] = {wt0, wt1, KH * KW, wt2, wt3}, yt[5] = {yt0, yt1, Hout * Wout, yt2, yt3};
  conv3d_entry("fortis_conv2d", x, xo, w, wo, y, yo, N, C, 1, Hin, Win, F, 1, KH, KW, 1, Hout, Wout, 1, sh, sw, 0, ph, pw, xt, wt, yt, false, 0,
               false);
}

int fortis_copy_to_host(void* dst, const void* dev, long nbytes) {
  cudaStreamSynchronize(stream());
  return cuda_ok(cudaMemcpy(dst, dev, (size_t)nbytes, cudaMemcpyDeviceToHost), "fortis_copy_to_host") ? 0 : -1;
}
int fortis_copy_to_device(void* dev, const void* src, long nbytes) {
  return cuda_ok(cudaMemcpy(dev, src, (size_t)nbytes, cudaMemcpyHostToDevice), "fortis_copy_to_device") ? 0 : -1;
}

int fortis_checksum(const void* data, long n, int elt, double* out) {
  FORTIS_TRY
  Session& s = S();
  cudaStream_t st = stream();
  ensure_aux(kChecksumBlocks);
  const void* d = data;
  void* tmp = nullptr;
  if (!is_device_ptr(data)) {
    tmp = pool_alloc((long)(n * (long)elt_size(elt)));
    if (!tmp) throw std::runtime_error("fortis_checksum: out of device memory");
    cuda_ok(cudaMemcpyAsync(tmp, data, (size_t)n * elt_size(elt), cudaMemcpyHostToDevice, st), "H2D for checksum");
    d = tmp;
  }
  double* dres = (double*)pool_alloc(sizeof(double));
  launch_checksum(d, n, elt, s.d_partials, dres, 0, st);
  cuda_ok(cudaMemcpyAsync(out, dres, sizeof(double), cudaMemcpyDeviceToHost, st), "D2H of the checksum");
  cudaStreamSynchronize(st);
  pool_free(dres); pool_free(tmp);
  return cuda_ok(cudaGetLastError(), "checksum kernels") ? 0 : -1;
  FORTIS_CATCH(return -1)
}

int fortis_step_checksum(double* out) {
  FORTIS_TRY
  Session& s = S();
  ensure_aux(1);
  cudaStream_t st = stream();
  cuda_ok(cudaMemcpyAsync(out, s.d_sum, sizeof(double), cudaMemcpyDeviceToHost, st), "D2H of the step checksum");
  cudaMemsetAsync(s.d_sum, 0, sizeof(double), st);
  cudaStreamSynchronize(st);
  return 0;
  FORTIS_CATCH(return -1)
}

// ---- host-only introspection (no CUDA call): lets the CPU test-suite check the descriptor planner and the
// expression compiler against the oracle
int fortis_debug_pack_layer(const float* W, const float* b, int cout, int cin, int last, int precision, unsigned short* image,
                            float* bias, float* scale, int* K, int* N) {
  FORTIS_TRY
  if (!W || !b || cout <= 0 || cin <= 0 || cin > 768 || !K || !N) throw std::runtime_error("fortis_debug_pack_layer: bad arguments");
  if (precision != PREC_BF16 && precision != PREC_FP8W && precision != PREC_FP16) throw std::runtime_error("fortis_debug_pack_layer: precision");
  return tc_debug_pack_layer(W, b, cout, cin, last, precision, image, bias, scale, K, N);
  FORTIS_CATCH(return -1)
}

int fortis_debug_eval_expr(const char* exprs_json, int tv_double, double tv, const double* scalars, const int* scalar_elt,
                           int nscalars, double* out) {
  FORTIS_TRY
  JValue v = parse_json(exprs_json ? exprs_json : "[]");
  std::vector<int> elt(kMaxScalars, -1);
  double sc[kMaxScalars] = {};
  for (int i = 0; i < nscalars && i < kMaxScalars; i++) { elt[i] = scalar_elt[i]; sc[i] = scalars[i]; }
  ExprProg P{};
  P.tv_double = tv_double;
  for (size_t k = 0; k < v.size(); k++) compile_expr(v.at(k).as_str(), elt, &P);
  *out = eval_prog_host(P, tv, sc, nullptr);
  return P.nops;
  FORTIS_CATCH(return -1)
}

// Element offsets (relative to each host array's first element) that `row` of a gather (is_scatter = 0: one per
// slot) or scatter (is_scatter = 1: one per store) touches, with the enclosing-loop arguments `args`.
int fortis_debug_plan(const char* desc_json, const char* loop_json, const char* kdist_json, int is_scatter, long row,
                      const int* args, int nargs, long long* offsets, int* arrays, int* slots, int cap, long long* geom) {
  FORTIS_TRY
  JValue jd = parse_json(desc_json), jl = parse_json(loop_json);
  JValue jk;
  const bool hk = kdist_json && *kdist_json;
  if (hk) jk = parse_json(kdist_json);
  LoopInfo L = make_loop(&jl, hk ? &jk : nullptr);
  IoPlanHost P = make_io_plan(jd, L, is_scatter != 0);
  if (geom) { geom[0] = L.count; geom[1] = L.nk; geom[2] = L.ni; geom[3] = L.klo; geom[4] = L.ilo; geom[5] = L.jlo; geom[6] = P.nargs; }
  if (!P.ok) return 0;
  const long long col = row % L.count, kk = row / L.count, ci = col % L.ni, cj = col / L.ni;
  const int n = is_scatter ? (int)P.stores.size() : (int)P.slots.size();
  for (int q = 0; q < n && q < cap; q++) {
    const Access& a = is_scatter ? P.stores[q].a : P.slots[q];
    const ArrayInfo& ai = P.arrays[a.array];
    long long base;
    if (L.kdist && !is_scatter) base = ai.vdims.empty() ? 0 : (long long)(L.klo - 1 + kk) * ai.plane;
    else base = plane_off_args(ai, args, nargs);
    offsets[q] = base + a.off0 + ci * a.si + cj * a.sj;
    arrays[q] = a.array;
    if (slots) slots[q] = is_scatter ? P.stores[q].slot : q;
  }
  return n;
  FORTIS_CATCH(return -1)
}

int fortis_device_status(void) {
  FORTIS_TRY
  Session& s = S();
  ensure_aux(1);
  int v = 0;
  cudaStreamSynchronize(stream());
  cudaMemcpy(&v, s.d_status, sizeof(int), cudaMemcpyDeviceToHost);
  if (v == 0 && s.conv) v = conv_model_status(s.conv);
  if (v != 0) {
    // reading a failure clears it (and re-arms the in-kernel checksum fold, which an aborted launch may have left
    // half way), so that the next step starts clean
    cudaMemset(s.d_status, 0, sizeof(int));
    if (s.d_done) cudaMemset(s.d_done, 0, sizeof(unsigned int));
    if (s.conv) conv_model_clear_status(s.conv);
  }
  return v;
  FORTIS_CATCH(return -1)
}

}  // extern "C"
