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
//   2-D operator layers (kind >= 3; NCHW fp32 networks: the operator micro-suite of tests/optest.py) use this record:
//               u32 kind (3 = Conv2d, 4 = MaxPool2d, 5 = nearest Upsample), cin, cout, kh, kw, sh, sw, ph, pw,
//               u32 dil (input dilation: a transposed convolution of stride s is the convolution of the s-dilated
//                   input with the flipped kernel), eh, ew (extra zero rows / columns behind the input: output_padding),
//               u32 act;  f32 slope;  Conv2d only: f32 W[cout * cin * kh * kw] (F, C, KH, KW), f32 b[cout]
//   f32 in_div[n_in_div]        input is divided by it      (mom6_zb/export_zb.py:13)
//   f32 out_mul[n_out_mul]      output is multiplied by it  (mom6_zb/export_zb.py:14)
//   f32 relu_mask[n_relu_mask]  outputs with mask != 0 get a final ReLU (benchmarks/climsim/export_wide.py:24-27)
//
// Optional pre-packed section behind it (MLP models): the weights already converted for one tensor-core precision and
// laid out as the 32 KB stage images the fused kernel streams, so that loading is a copy.
//   char  tag[8] = "FORTISP1"
//   u32   precision (1 = bf16, 2 = FP8-E4M3 weights as bf16 codes + per-channel scales, 3 = fp16), nlayers
//   u64   FNV-1a 64 of every byte in front of the tag: the section belongs to exactly these fp32 weights
//   per layer:  u32 K_pad, N_pad;  u16 image[N_pad * K_pad];  f32 bias[N_pad];  f32 scale[N_pad]
//               image: [chunk of 64 features][256-wide K-block] blocks of four 64 x 64 sub-tiles, K-major rows of 128
//               bytes, 16-byte piece j of row r stored at piece j ^ (r & 7)
//   u64   FNV-1a 64 of the section from its tag up to here
// A section whose hashes do not match is an error, one for another precision than the session's is ignored.
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace fortis {

enum { LAYER_LINEAR = 1, LAYER_CONV3D = 2, LAYER_CONV2D = 3, LAYER_MAXPOOL2D = 4, LAYER_UPSAMPLE2D = 5 };
enum { LFLAG_SAVE_SKIP = 1, LFLAG_ADD_SKIP = 2 };

struct LayerHost {
  int kind = LAYER_LINEAR, cin = 0, cout = 0, ksize = 1, pad = 0, act = 0, flags = 0;
  float slope = 0.f;
  int kh = 1, kw = 1, sh = 1, sw = 1, ph = 0, pw = 0, dil = 1, eh = 0, ew = 0;      // 2-D operator layers
  std::vector<float> W, b;
};

struct PackedLayer {
  int K = 0, N = 0;                      // padded extents
  std::vector<uint16_t> image;           // stage images
  std::vector<float> bias, scale;        // padded; scale is all ones unless the weights are FP8 codes
};

struct ModelHost {
  std::vector<LayerHost> layers;
  std::vector<float> in_div, out_mul, relu_mask;
  int packed_precision = -1;             // precision of the pre-packed section, -1 = none
  std::vector<PackedLayer> packed;
  bool is_mlp() const {
    for (auto& l : layers) if (l.kind != LAYER_LINEAR) return false;
    return !layers.empty();
  }
  bool is_conv() const {
    for (auto& l : layers) if (l.kind != LAYER_CONV3D) return false;
    return !layers.empty();
  }
  bool is_opnet() const {                 // a network of 2-D operator layers (NCHW)
    for (auto& l : layers) if (l.kind < LAYER_CONV2D) return false;
    return !layers.empty();
  }
  int n_in() const { return layers.empty() ? 0 : layers.front().cin; }
  int n_out() const { return layers.empty() ? 0 : layers.back().cout; }
};

inline uint64_t fnv1a64(const uint8_t* p, size_t n) {
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < n; i++) { h ^= p[i]; h *= 1099511628211ull; }
  return h;
}

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
    L.kind = (int)u32();
    if (L.kind >= LAYER_CONV2D && L.kind <= LAYER_UPSAMPLE2D) {
      L.cin = (int)u32(); L.cout = (int)u32(); L.kh = (int)u32(); L.kw = (int)u32(); L.sh = (int)u32(); L.sw = (int)u32();
      L.ph = (int)u32(); L.pw = (int)u32(); L.dil = (int)u32(); L.eh = (int)u32(); L.ew = (int)u32(); L.act = (int)u32(); L.slope = f32();
      auto bad = [&](int v, int lo, int hi) { return v < lo || v > hi; };
      if (bad(L.cin, 1, 1 << 16) || bad(L.cout, 1, 1 << 16) || bad(L.kh, 1, 31) || bad(L.kw, 1, 31) || bad(L.sh, 1, 16) || bad(L.sw, 1, 16) ||
          bad(L.ph, 0, 64) || bad(L.pw, 0, 64) || bad(L.dil, 1, 16) || bad(L.eh, 0, 16) || bad(L.ew, 0, 16) || bad(L.act, 0, 2))
        throw std::runtime_error("model blob: bad 2-D layer shape");
      if (L.kind == LAYER_CONV2D) {
        floats(L.W, (size_t)L.cout * L.cin * L.kh * L.kw);
        floats(L.b, (size_t)L.cout);
      } else if (L.cin != L.cout || L.act != 0) {
        throw std::runtime_error("model blob: pooling / upsampling layers keep the channel count and have no activation");
      }
      if (l && M.layers.back().cout != L.cin) throw std::runtime_error("model blob: layer widths do not chain");
      M.layers.push_back(std::move(L));
      continue;
    }
    L.cin = (int)u32(); L.cout = (int)u32(); L.ksize = (int)u32(); L.pad = (int)u32();
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
  if (p == end) return M;
  // ---- pre-packed section
  const uint8_t* sec = p;
  need(8);
  if (std::memcmp(p, "FORTISP1", 8) != 0) throw std::runtime_error("model blob: unknown data behind the layers");
  p += 8;
  auto u64 = [&]() { need(8); uint64_t v; std::memcpy(&v, p, 8); p += 8; return v; };
  const uint32_t prec = u32(), npl = u32();
  if (u64() != fnv1a64((const uint8_t*)data, (size_t)(sec - (const uint8_t*)data)))
    throw std::runtime_error("model blob: the pre-packed section does not belong to these weights (hash mismatch)");
  if (npl != nl || !M.is_mlp()) throw std::runtime_error("model blob: pre-packed section does not match the layer list");
  for (uint32_t l = 0; l < npl; l++) {
    PackedLayer Q;
    Q.K = (int)u32(); Q.N = (int)u32();
    if (Q.K < M.layers[l].cin || Q.N < M.layers[l].cout || Q.K % 256 || Q.N % 64 || Q.K > 4096 || Q.N > 4096)
      throw std::runtime_error("model blob: bad pre-packed layer shape");
    const size_t n = (size_t)Q.K * Q.N;
    need(n * 2); Q.image.resize(n); std::memcpy(Q.image.data(), p, n * 2); p += n * 2;
    floats(Q.bias, (size_t)Q.N); floats(Q.scale, (size_t)Q.N);
    M.packed.push_back(std::move(Q));
  }
  const uint64_t want = fnv1a64(sec, (size_t)(p - sec));
  if (u64() != want) throw std::runtime_error("model blob: pre-packed section is corrupt (hash mismatch)");
  if (p != end) throw std::runtime_error("model blob: unknown data behind the pre-packed section");
  M.packed_precision = (int)prec;
  return M;
}

}  // namespace fortis
