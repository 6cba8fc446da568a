// Model blob: the layer list and weights the runtime loads at start-up.  It replaces the weights that a fortisc
// build links in as `w0..wN` globals next to outline.json (driver/fortis_outline.py:13-35).
//
// Layout (little-endian):
//   char  magic[8] = "FORTISM1"
//   u32   nlayers, n_in_div, n_out_mul, n_relu_mask
//   per layer:  u32 kind (1 = Linear, 2 = Conv3d), cin, cout, ksize, pad, act (0 none, 1 ReLU, 2 LeakyReLU),
//               u32 flags (bit0: remember this layer's output as the skip, bit1: add the skip before the activation)
//               f32 slope
//               f32 W[cout * cin * ksize^3]   (torch layout: Linear (out,in); Conv3d (F,C,KD,KH,KW))
//               f32 b[cout]
//   f32 in_div[n_in_div]        input is divided by it      (mom6_zb/export_zb.py:13)
//   f32 out_mul[n_out_mul]      output is multiplied by it  (mom6_zb/export_zb.py:14)
//   f32 relu_mask[n_relu_mask]  outputs with mask != 0 get a final ReLU (benchmarks/climsim/export_wide.py:24-27)
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace fortis {

enum { LAYER_LINEAR = 1, LAYER_CONV3D = 2 };
enum { LFLAG_SAVE_SKIP = 1, LFLAG_ADD_SKIP = 2 };

struct LayerHost {
  int kind = LAYER_LINEAR, cin = 0, cout = 0, ksize = 1, pad = 0, act = 0, flags = 0;
  float slope = 0.f;
  std::vector<float> W, b;
};

struct ModelHost {
  std::vector<LayerHost> layers;
  std::vector<float> in_div, out_mul, relu_mask;
  bool is_mlp() const {
    for (auto& l : layers) if (l.kind != LAYER_LINEAR) return false;
    return !layers.empty();
  }
  bool is_conv() const {
    for (auto& l : layers) if (l.kind != LAYER_CONV3D) return false;
    return !layers.empty();
  }
  int n_in() const { return layers.empty() ? 0 : layers.front().cin; }
  int n_out() const { return layers.empty() ? 0 : layers.back().cout; }
};

inline ModelHost parse_model_blob(const void* data, size_t nbytes) {
  const uint8_t* p = (const uint8_t*)data;
  const uint8_t* end = p + nbytes;
  auto need = [&](size_t n) { if ((size_t)(end - p) < n) throw std::runtime_error("model blob: truncated"); };
  auto u32 = [&]() { need(4); uint32_t v; std::memcpy(&v, p, 4); p += 4; return v; };
  auto f32 = [&]() { need(4); float v; std::memcpy(&v, p, 4); p += 4; return v; };
  auto floats = [&](std::vector<float>& dst, size_t n) { need(n * 4); dst.resize(n); if (n) std::memcpy(dst.data(), p, n * 4); p += n * 4; };
  need(8);
  if (std::memcmp(p, "FORTISM1", 8) != 0) throw std::runtime_error("model blob: bad magic");
  p += 8;
  ModelHost M;
  const uint32_t nl = u32(), nid = u32(), nom = u32(), nrm = u32();
  if (nl == 0 || nl > 64) throw std::runtime_error("model blob: layer count out of range");
  for (uint32_t l = 0; l < nl; l++) {
    LayerHost L;
    L.kind = (int)u32(); L.cin = (int)u32(); L.cout = (int)u32(); L.ksize = (int)u32(); L.pad = (int)u32();
    L.act = (int)u32(); L.flags = (int)u32(); L.slope = f32();
    if (L.kind != LAYER_LINEAR && L.kind != LAYER_CONV3D) throw std::runtime_error("model blob: unknown layer kind");
    if (L.cin <= 0 || L.cout <= 0 || L.ksize <= 0 || L.ksize > 7) throw std::runtime_error("model blob: bad layer shape");
    const size_t kvol = L.kind == LAYER_CONV3D ? (size_t)L.ksize * L.ksize * L.ksize : 1;
    floats(L.W, (size_t)L.cout * L.cin * kvol);
    floats(L.b, (size_t)L.cout);
    if (l && M.layers.back().cout != L.cin) throw std::runtime_error("model blob: layer widths do not chain");
    M.layers.push_back(std::move(L));
  }
  floats(M.in_div, nid); floats(M.out_mul, nom); floats(M.relu_mask, nrm);
  if (nid && (int)nid != M.n_in()) throw std::runtime_error("model blob: in_div length != model inputs");
  if (nom && (int)nom != M.n_out()) throw std::runtime_error("model blob: out_mul length != model outputs");
  if (nrm && (int)nrm != M.n_out()) throw std::runtime_error("model blob: relu_mask length != model outputs");
  return M;
}

}  // namespace fortis
