"""ctypes front end of oracle/native_forward.c.  TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline)."""
import ctypes

import numpy as np

_ACT = {"none": 0, "relu": 1, "leaky": 2}


def _fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def pack_layers(layers):
    n = len(layers)
    dims = (ctypes.c_int * (n + 1))(*([int(layers[0]["W"].shape[1])] + [int(L["W"].shape[0]) for L in layers]))
    Wt = [np.ascontiguousarray(np.asarray(L["W"], dtype=np.float32).T) for L in layers]
    b = [np.ascontiguousarray(np.asarray(L["b"], dtype=np.float32)) for L in layers]
    Wp = (ctypes.POINTER(ctypes.c_float) * n)(*[_fp(w) for w in Wt])
    bp = (ctypes.POINTER(ctypes.c_float) * n)(*[_fp(x) for x in b])
    act = (ctypes.c_int * n)(*[_ACT[L.get("act", "none")] for L in layers])
    slope = (ctypes.c_float * n)(*[float(L.get("slope", 0.0)) for L in layers])
    return dict(n=n, dims=dims, Wp=Wp, bp=bp, act=act, slope=slope, keep=(Wt, b))


def mlp_forward_c(lib, layers, X, in_norms=None, out_norms=None, nthreads=0):
    P = pack_layers(layers)
    X = np.ascontiguousarray(X, dtype=np.float32)
    Y = np.empty((X.shape[0], int(P["dims"][P["n"]])), dtype=np.float32)
    inn = np.ascontiguousarray(in_norms, dtype=np.float32) if in_norms is not None else None
    outn = np.ascontiguousarray(out_norms, dtype=np.float32) if out_norms is not None else None
    lib.oracle_mlp_forward(_fp(X), _fp(Y), ctypes.c_long(X.shape[0]), P["n"], P["dims"], P["Wp"], P["bp"], P["act"],
                           P["slope"], _fp(inn) if inn is not None else None, _fp(outn) if outn is not None else None,
                           int(nthreads))
    return Y
