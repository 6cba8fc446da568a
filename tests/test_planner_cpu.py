"""Host logic of the library (descriptor planner, expression compiler) against the oracle, on the CPU."""
import ctypes
import json
import os

import numpy as np
import pytest

import fortis_b200
from fortis_b200 import build as fb
from oracle import fortis_oracle as fo


@pytest.fixture(scope="module")
def lib():
    fb.build()
    return fortis_b200.load()


def lib_offsets(lib, J, Lp, K, is_scatter, row, args):
    cap = 2048
    offs = (ctypes.c_longlong * cap)()
    arrs = (ctypes.c_int * cap)()
    slots = (ctypes.c_int * cap)()
    geom = (ctypes.c_longlong * 8)()
    a = (ctypes.c_int * max(1, len(args)))(*args)
    n = lib.fortis_debug_plan(json.dumps(J).encode(), json.dumps(Lp).encode(), json.dumps(K).encode() if K else b"",
                              int(is_scatter), row, a, len(args), offs, arrs, slots, cap, geom)
    assert n >= 0, lib.fortis_last_error_message()
    return [(arrs[q], offs[q], slots[q]) for q in range(n)], list(geom)


def oracle_offsets(J, Lp, K, is_scatter, row, args):
    P = fo.loop_params(Lp, K)
    uses = [(s["array"], s["idx"]) for s in J["stores" if is_scatter else "slots"]] + [(s["array"], s["idx"]) for s in J["scalars"]]
    A = fo.plan_arrays(J, uses)
    col, kk = row % P["count"], row // P["count"]
    i, j = P["ilo"] + col % P["ni"], P["jlo"] + col // P["ni"]
    out = []
    for q, s in enumerate(J["stores" if is_scatter else "slots"]):
        ai = s["array"]
        if P["kdist"] and not is_scatter:
            base = ((P["klo"] - 1) + kk) * A[ai]["plane"] if A[ai]["vdims"] else 0
        else:
            base = fo._plane_off(A, ai, A[ai]["idx"], args)
        out.append((ai, base + fo._elem(A, ai, s["idx"], i, j), s["slot"] if is_scatter else q))
    return out


def all_cases(golden_dir):
    G = json.load(open(os.path.join(golden_dir, "gather_scatter_golden.json")))
    zb = tuple(json.load(open(os.path.join(golden_dir, f))) for f in ("zb_gather.json", "zb_scatter.json", "zb_loop.json", "zb_kdist.json"))
    cases = {"zb": zb + ([3],)}
    for name in ("f64_kdist", "arg_plane", "inner_only"):
        g = G[name]
        cases[name] = (g["gather"], g["scatter"], g["loop"], g["kdist"], g["a0s"][:1] or [1])
    cases["column"] = fo.column_descriptors(96, 5) + ([],)
    cases["stencil"] = fo.stencil_descriptors(17, 9, 3) + ([2],)
    cases["toy"] = fo.identity_descriptors(6, 4, 33) + ([],)
    return cases


def test_planner_offsets_match_oracle(lib, golden_dir):
    for name, (G, S, Lp, K, args) in all_cases(golden_dir).items():
        P = fo.loop_params(Lp, K)
        nrows = P["count"] * P["nk"]
        for row in sorted({0, 1, P["ni"] - 1, P["ni"], nrows // 2, nrows - 1}):
            if row < 0 or row >= nrows:
                continue
            got, geom = lib_offsets(lib, G, Lp, K, False, row, [] if P["kdist"] else args)
            assert geom[0] == P["count"] and geom[1] == P["nk"] and geom[2] == P["ni"], name
            assert got == oracle_offsets(G, Lp, K, False, row, [] if P["kdist"] else args), (name, row)
        for col in sorted({0, P["ni"] - 1, P["count"] - 1}):
            got, _ = lib_offsets(lib, S, Lp, K, True, col, args)
            assert got == oracle_offsets(S, Lp, K, True, col, args), (name, col)


EXPRS = [
    (["(tv / (S0 + 1.000000e-30f))"], [0]),
    (["(((tv * S0) * S0) * S1)"], [0, 0]),
    (["(((tv * S1) - 1.100000e+00f) / (S0 + 1.000000e-30f))", "fmaxf(sqrtf((tv * tv)), 2.500000e-01f)",
      "((tv * 3.300000e-01) + (S1 * 7.000000e-01f))"], [1, 0]),
    (["(-tv)", "fminf((tv + 2.000000e+00f), (S0 * 1.500000e+00))"], [1]),
    (["((tv - S0) * (tv + S0))", "(tv / 3.000000e+00f)"], [0]),
]


@pytest.mark.parametrize("exprs,elts", EXPRS)
def test_expression_compiler_is_bit_exact_with_oracle(lib, exprs, elts):
    rng = np.random.default_rng(3)
    asts = [fo.parse_expr(e) for e in exprs]
    for _ in range(200):
        tv = np.float32(rng.normal() * 3)
        scal = {k: (np.float64(rng.random() + 0.5) if e else np.float32(rng.random() + 0.5)) for k, e in enumerate(elts)}
        want = np.float32(tv)
        for a in asts:
            want = fo._eval_c(a, want, scal)
        sc = (ctypes.c_double * len(elts))(*[float(scal[k]) for k in range(len(elts))])
        se = (ctypes.c_int * len(elts))(*elts)
        out = ctypes.c_double()
        n = lib.fortis_debug_eval_expr(json.dumps(exprs).encode(), 0, float(tv), sc, se, len(elts), ctypes.byref(out))
        assert n > 0, lib.fortis_last_error_message()
        assert np.float32(out.value).tobytes() == np.float32(want).tobytes(), (exprs, tv, scal)


def test_expression_compiler_rejects_unknown_syntax(lib):
    out = ctypes.c_double()
    sc = (ctypes.c_double * 1)(1.0)
    se = (ctypes.c_int * 1)(0)
    for bad in (["(tv + q7)"], ["(tv + S3)"], ["(tv +"], ["powf(tv, 2.0f)"]):
        assert lib.fortis_debug_eval_expr(json.dumps(bad).encode(), 0, 1.0, sc, se, 1, ctypes.byref(out)) == -1


def test_model_blob_roundtrip_shapes():
    layers = fortis_b200.mlp_layers([27, 20, 20, 3], seed=4, init="uniform", act="relu", bias="uniform")
    blob = fortis_b200.write_blob(layers, in_div=np.ones(27), out_mul=np.ones(3))
    assert blob[:8] == b"FORTISM1"
    nfloats = sum(L["W"].size + L["b"].size for L in layers) + 27 + 3
    assert len(blob) == 8 + 16 + 3 * 32 + 4 * nfloats
    conv = fortis_b200.conv_layers(3, 8, 3, nblocks=1, seed=1)
    assert len(conv) == 4 and conv[2]["add"] and conv[0]["save"]
