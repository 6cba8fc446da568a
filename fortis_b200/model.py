"""Writer of the model blob the runtime loads (layout: fortis_b200/csrc/fortis_model.h).

It plays the role of the reference's export scripts + weight outlining (frontend/export_*.py,
driver/fortis_outline.py:13-35): a layer list with torch-layout weights goes in, one binary blob comes out.
"""
import struct

import numpy as np

_ACT = {"none": 0, "relu": 1, "leaky": 2}
LINEAR, CONV3D = 1, 2
SAVE_SKIP, ADD_SKIP = 1, 2


def write_blob(layers, in_div=None, out_mul=None, relu_mask=None) -> bytes:
    """layers: dicts with W ((out,in) or (F,C,K,K,K)), b, act ('none'|'relu'|'leaky'), slope, and for conv layers
    pad, save (remember output as skip), add (add skip before the activation)."""
    def vec(v):
        return np.zeros(0, np.float32) if v is None else np.ascontiguousarray(v, dtype=np.float32).ravel()
    ind, outm, rm = vec(in_div), vec(out_mul), vec(relu_mask)
    out = [b"FORTISM1", struct.pack("<4I", len(layers), ind.size, outm.size, rm.size)]
    for L in layers:
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
    return b"".join(out)


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
