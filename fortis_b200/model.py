"""Writer of the model blob the runtime loads (layout: fortis_b200/csrc/fortis_model.h).

It plays the role of the reference's export scripts + weight outlining (frontend/export_*.py,
driver/fortis_outline.py:13-35): a layer list with torch-layout weights goes in, one binary blob comes out.
"""
import struct

import numpy as np

_ACT = {"none": 0, "relu": 1, "leaky": 2}
LINEAR, CONV3D, CONV2D, MAXPOOL2D, UPSAMPLE2D = 1, 2, 3, 4, 5
SAVE_SKIP, ADD_SKIP = 1, 2


PRECISIONS = {"bf16": 1, "fp8w": 2, "fp16": 3}
_BLOCK_K, _CHUNK_N, _STAGE_K = 256, 64, 256


def fnv1a64(data: bytes) -> int:
    """FNV-1a, 64 bit (the hash the loader checks: fortis_b200/csrc/fortis_model.h).  The hash is sequential by
    construction; the loop runs over 64 KB slices with local-variable integer arithmetic (~10 MB/s)."""
    h, prime, mask = 1469598103934665603, 1099511628211, 0xFFFFFFFFFFFFFFFF
    mv = memoryview(data)
    for i in range(0, len(mv), 1 << 16):
        for b in mv[i:i + (1 << 16)].tobytes():
            h = ((h ^ b) * prime) & mask
    return h


def round_bf16_bits(x):
    """fp32 -> bf16 bit patterns, round to nearest even, NaN kept quiet (as the loader's f32_to_bf16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    r = np.where(nan, (u >> 16) | 0x40, r)
    return (r & 0xFFFF).astype(np.uint16)


def round_e4m3(v):
    """Nearest (ties to even) E4M3 value, saturating at +-448 (as the loader's e4m3_round: computed in double)."""
    v = np.asarray(v, dtype=np.float32).astype(np.float64)
    a = np.minimum(np.abs(v), 448.0)
    e = np.floor(np.log2(np.maximum(a, 9.5367431640625e-07))).astype(np.int64)
    e = np.clip(e, -6, 8)
    step = np.ldexp(1.0, (e - 3).astype(np.int32))
    q = np.minimum(np.rint(a / step) * step, 448.0)
    return np.where(v < 0, -q, q).astype(np.float32)


def pack_layer(W, b, last, precision):
    """One Linear layer as the fused tensor-core kernel streams it: (K_pad, N_pad, image uint16[N_pad*K_pad],
    bias float32[N_pad], scale float32[N_pad]).  Same arithmetic, padding and tiling as the loader
    (fortis_b200/csrc/fortis_mlp_tc.cu: pack_layer_host), so a pre-packed blob loads bit-identically."""
    W = np.ascontiguousarray(W, dtype=np.float32)
    cout, cin = W.shape
    up = lambda v, m: (v + m - 1) // m * m
    K, N = up(cin, _BLOCK_K), up(cout, _CHUNK_N if last else _BLOCK_K)
    scale = np.ones(N, np.float32)
    if precision == "fp8w":
        amax = np.abs(W).max(axis=1)
        sc = np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
        scale[:cout] = sc
        Wq = round_e4m3((W / sc[:, None]).astype(np.float32))
    else:
        Wq = W
    bits = np.zeros((N, K), np.uint16)
    bits[:cout, :cin] = Wq.astype(np.float16).view(np.uint16) if precision == "fp16" else round_bf16_bits(Wq)
    bias = np.zeros(N, np.float32)
    bias[:cout] = np.asarray(b, dtype=np.float32)
    # [chunk c][K-block ks][sub-tile t][row r][16-byte piece j ^ (r & 7)][8 values]
    nks = K // _STAGE_K
    v = bits.reshape(N // _CHUNK_N, _CHUNK_N, nks, _STAGE_K // 64, 8, 8)          # c, r, ks, t, j, e
    v = v.transpose(0, 2, 3, 1, 4, 5)                                              # c, ks, t, r, j, e
    img = np.empty_like(v)
    r = np.arange(_CHUNK_N)
    for j in range(8):
        img[:, :, :, r, j ^ (r & 7), :] = v[:, :, :, r, j, :]
    return K, N, np.ascontiguousarray(img).reshape(-1), bias, scale


def _pair(v):
    return (int(v), int(v)) if np.isscalar(v) else (int(v[0]), int(v[1]))


def _op2d_record(L) -> bytes:
    """One 2-D operator layer (NCHW networks): dict(op='conv2d', W (F,C,KH,KW), b, stride, pad, dil (input dilation),
    extra (zero rows / columns behind the input), act, slope) | dict(op='maxpool2d', channels, k, stride) |
    dict(op='upsample2d', channels, scale)."""
    op = L["op"]
    if op == "conv2d":
        W = np.ascontiguousarray(L["W"], dtype=np.float32)
        if W.ndim != 4:
            raise ValueError("conv2d weights are (F, C, KH, KW)")
        cout, cin, kh, kw = W.shape
        b = np.ascontiguousarray(L["b"] if L.get("b") is not None else np.zeros(cout), dtype=np.float32)
        (sh, sw), (ph, pw), (eh, ew) = _pair(L.get("stride", 1)), _pair(L.get("pad", 0)), _pair(L.get("extra", 0))
        head = struct.pack("<13If", CONV2D, cin, cout, kh, kw, sh, sw, ph, pw, int(L.get("dil", 1)), eh, ew,
                           _ACT[L.get("act", "none")], float(L.get("slope", 0.0)))
        return head + W.tobytes() + b.tobytes()
    c = int(L["channels"])
    if op == "maxpool2d":
        (kh, kw) = _pair(L["k"])
        (sh, sw) = _pair(L.get("stride", L["k"]))
        return struct.pack("<13If", MAXPOOL2D, c, c, kh, kw, sh, sw, 0, 0, 1, 0, 0, 0, 0.0)
    (fh, fw) = _pair(L["scale"])
    return struct.pack("<13If", UPSAMPLE2D, c, c, 1, 1, fh, fw, 0, 0, 1, 0, 0, 0, 0.0)


def write_blob(layers, in_div=None, out_mul=None, relu_mask=None, prepack=None) -> bytes:
    """layers: dicts with W ((out,in) or (F,C,K,K,K)), b, act ('none'|'relu'|'leaky'), slope, and for conv layers
    pad, save (remember output as skip), add (add skip before the activation).  prepack = 'bf16' | 'fp16' | 'fp8w'
    (MLP models) appends the weights already converted and tiled for that precision, with hashes that tie the section
    to these fp32 weights; a session running that precision then loads by copying."""
    def vec(v):
        return np.zeros(0, np.float32) if v is None else np.ascontiguousarray(v, dtype=np.float32).ravel()
    ind, outm, rm = vec(in_div), vec(out_mul), vec(relu_mask)
    out = [b"FORTISM1", struct.pack("<4I", len(layers), ind.size, outm.size, rm.size)]
    for L in layers:
        if L.get("op") in ("conv2d", "maxpool2d", "upsample2d"):
            out.append(_op2d_record(L))
            continue
        W = np.ascontiguousarray(L["W"], dtype=np.float32)
        kind = CONV3D if W.ndim == 5 else LINEAR
        cout, cin = W.shape[0], W.shape[1]
        k = W.shape[2] if kind == CONV3D else 1
        b = np.ascontiguousarray(L["b"] if L.get("b") is not None else np.zeros(cout), dtype=np.float32)
        flags = (SAVE_SKIP if L.get("save") else 0) | (ADD_SKIP if L.get("add") else 0)
        out.append(struct.pack("<7If", kind, cin, cout, k, int(L.get("pad", 1 if kind == CONV3D else 0)),
                               _ACT[L.get("act", "none")], flags, float(L.get("slope", 0.0))))
        out.append(W.tobytes())
        out.append(b.tobytes())
    out += [ind.tobytes(), outm.tobytes(), rm.tobytes()]
    base = b"".join(out)
    if prepack is None:
        return base
    if prepack not in PRECISIONS:
        raise ValueError("prepack must be one of %s" % sorted(PRECISIONS))
    if any(L.get("op") or np.asarray(L["W"]).ndim != 2 for L in layers):
        raise ValueError("only MLP models carry a pre-packed section")
    sec = [b"FORTISP1", struct.pack("<2I", PRECISIONS[prepack], len(layers)), struct.pack("<Q", fnv1a64(base))]
    for l, L in enumerate(layers):
        cout = np.asarray(L["W"]).shape[0]
        b = L["b"] if L.get("b") is not None else np.zeros(cout)
        K, N, img, bias, scale = pack_layer(L["W"], b, l == len(layers) - 1, prepack)
        sec += [struct.pack("<2I", K, N), img.tobytes(), bias.tobytes(), scale.tobytes()]
    body = b"".join(sec)
    return base + body + struct.pack("<Q", fnv1a64(body))


def mlp_layers(dims, seed, init="kaiming_normal", act="leaky", slope=0.15, bias="zero", last_act="none", scale=0.3):
    """Seeded random MLP weights as layer dicts.  init: 'kaiming_normal' (std = sqrt(2/fan_in), the reference's
    export_wide.py:17-19), 'kaiming_uniform' (bound = sqrt(6/fan_in)), or 'uniform' (U(-scale, scale))."""
    rng = np.random.default_rng(seed)
    layers = []
    for l in range(len(dims) - 1):
        fan_in, fan_out = dims[l], dims[l + 1]
        if init == "kaiming_normal":
            W = rng.normal(0.0, np.sqrt(2.0 / fan_in), size=(fan_out, fan_in))
        elif init == "kaiming_uniform":
            bound = np.sqrt(6.0 / fan_in)
            W = rng.uniform(-bound, bound, size=(fan_out, fan_in))
        else:
            W = rng.uniform(-scale, scale, size=(fan_out, fan_in))
        b = rng.uniform(-scale, scale, size=fan_out) if bias == "uniform" else np.zeros(fan_out)
        layers.append(dict(W=W.astype(np.float32), b=b.astype(np.float32),
                           act=(act if l < len(dims) - 2 else last_act), slope=slope))
    return layers


def conv_layers(cin, width, cout, nblocks, seed, slope=0.2, k=3):
    """Super-resolution style conv3d net: conv cin->width + LeakyReLU; nblocks x [conv, LeakyReLU, conv, +skip];
    conv width->cout.  He-normal weights std = sqrt(2 / (k^3 * Cin)), zero bias."""
    rng = np.random.default_rng(seed)

    def conv(ci, co):
        return rng.normal(0.0, np.sqrt(2.0 / (k ** 3 * ci)), size=(co, ci, k, k, k)).astype(np.float32)
    layers = [dict(W=conv(cin, width), b=np.zeros(width, np.float32), act="leaky", slope=slope, pad=k // 2, save=True)]
    for _ in range(nblocks):
        layers.append(dict(W=conv(width, width), b=np.zeros(width, np.float32), act="leaky", slope=slope, pad=k // 2))
        layers.append(dict(W=conv(width, width), b=np.zeros(width, np.float32), act="none", pad=k // 2, add=True, save=True))
    layers.append(dict(W=conv(width, cout), b=np.zeros(cout, np.float32), act="none", pad=k // 2))
    return layers
