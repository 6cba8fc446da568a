"""Generators of the layout descriptors the library consumes: gather.json, scatter.json, loop.json, kdist.json and
lift2d.json, in the schema the reference's analyses emit (driver/fortis_gather.py:201-206 for gather / scatter,
driver/fortis_kdist.py for kdist, driver/fortis_lift2d.py:163-243 for a whole-array boundary).

In a fortisc build these files come out of the Flang/MLIR analyses of a host program.  A host that is wired by hand
(or a test, or a benchmark) builds them here from a description of its arrays and loops instead:

    stencil(nx, ny, nz)          3x3 stencil over (nx+2, ny+2, nz) fields, k loop distributed
    column(ncol, nlev)           column physics: (ncol, nlev) fields + (ncol) scalars -> feature vector per column
    identity(nin, nout, ncol)    A(nin, ncol) read column by column
    boundary(NI, NK, NO, ...)    lift2d.json of a whole-array host (transpose + cast + per-feature affine maps)
    random_case(rng)             a random but valid descriptor set (differential testing)

Subscript kinds: ["i", d] inner loop variable + d, ["j", d] outer loop variable + d, ["v", a] the enclosing-loop
variable a (plane selector, trailing dimensions only), ["c", n] the constant 1-based subscript n (an extension over
the reference's schema, needed for (ncol, nlev) column layouts).
"""
import numpy as np


def _array(name, shape, elt="f32"):
    return {"ssa": "%" + name, "name": name, "shape": [int(s) for s in shape], "elt": elt}


def _loop(batch, ilo, ni, outer, nin, nout):
    return {"verdict": "batched", "batch": int(batch), "inner": {"lo": int(ilo), "hi": int(ilo + ni - 1), "n": int(ni)},
            "outer": None if outer is None else {"lo": int(outer[0]), "hi": int(outer[1])},
            "in_shape": [int(nin)], "out_shape": [int(nout)], "in_elt": "f32", "out_elt": "f32"}


def stencil(nx, ny, nz, nfields=3, nout=3, halo=1, elt="f32", radius=1):
    """(2*radius+1)^2 stencil of `nfields` fields of extent (nx+2*halo, ny+2*halo, nz) around every interior point;
    slot order is field-major, then the i offset fastest, then the j offset (the RESHAPE order of
    mom6_zb/zb_host.f90:79-87).  `nout` outputs are stored at (i, j, k) of separate arrays.  The k loop is
    distributed: one gather and one forward serve all nz planes."""
    if radius > halo:
        raise ValueError("the stencil radius needs a halo at least as wide")
    sx, sy = nx + 2 * halo, ny + 2 * halo
    offs = range(-radius, radius + 1)
    slots = [{"array": f, "idx": [["i", di], ["j", dj], ["v", 0]]} for f in range(nfields) for dj in offs for di in offs]
    karg = [{"alloca": "%k", "name": "k"}]
    G = {"ok": True, "n": len(slots), "args": karg, "arrays": [_array("in%d" % f, (sx, sy, nz), elt) for f in range(nfields)],
         "scalars": [], "exprs": [], "slots": slots}
    S = {"ok": True, "n": nout, "args": karg, "arrays": [_array("out%d" % q, (sx, sy, nz), elt) for q in range(nout)],
         "scalars": [], "exprs": [],
         "stores": [{"slot": q, "array": q, "idx": [["i", 0], ["j", 0], ["v", 0]]} for q in range(nout)]}
    Lp = _loop(nx * ny * nz, halo + 1, nx, (halo + 1, halo + ny), len(slots), nout)
    K = {"ok": True, "loop": {"lo": 1, "hi": int(nz)}, "nk": int(nz)}
    return G, S, Lp, K


def column(ncol, nlev, nfields=4, nscal=4, nout_fields=2, nout_scal=8, elt="f32"):
    """Column physics.  Features per column: field 0 levels 1..nlev, field 1 levels 1..nlev, ..., then the per-column
    scalars (the packing order of benchmarks/cam/cam_host.f90:34-39).  Outputs: `nout_fields` (ncol, nlev) arrays
    level by level, then `nout_scal` (ncol) vectors."""
    arrays = [_array("f%d" % f, (ncol, nlev), elt) for f in range(nfields)] + [_array("s%d" % s, (ncol,), elt) for s in range(nscal)]
    slots = [{"array": f, "idx": [["i", 0], ["c", l + 1]]} for f in range(nfields) for l in range(nlev)]
    slots += [{"array": nfields + s, "idx": [["i", 0]]} for s in range(nscal)]
    G = {"ok": True, "n": len(slots), "args": [], "arrays": arrays, "scalars": [], "exprs": [], "slots": slots}
    oarr = [_array("o%d" % f, (ncol, nlev), elt) for f in range(nout_fields)] + [_array("t%d" % s, (ncol,), elt) for s in range(nout_scal)]
    stores = [{"slot": f * nlev + l, "array": f, "idx": [["i", 0], ["c", l + 1]]} for f in range(nout_fields) for l in range(nlev)]
    stores += [{"slot": nout_fields * nlev + s, "array": nout_fields + s, "idx": [["i", 0]]} for s in range(nout_scal)]
    S = {"ok": True, "n": len(stores), "args": [], "arrays": oarr, "scalars": [], "exprs": [], "stores": stores}
    return G, S, _loop(ncol, 1, ncol, None, len(slots), len(stores)), None


def identity(nin, nout, ncol, elt="f32"):
    """Host array A(nin, ncol), column-major, one model row per column; output into B(nout, ncol)."""
    G = {"ok": True, "n": nin, "args": [], "arrays": [_array("a", (nin, ncol), elt)], "scalars": [], "exprs": [],
         "slots": [{"array": 0, "idx": [["c", f + 1], ["i", 0]]} for f in range(nin)]}
    S = {"ok": True, "n": nout, "args": [], "arrays": [_array("b", (nout, ncol), elt)], "scalars": [], "exprs": [],
         "stores": [{"slot": f, "array": 0, "idx": [["c", f + 1], ["i", 0]]} for f in range(nout)]}
    return G, S, _loop(ncol, 1, ncol, None, nin, nout), None


def boundary(NI, NK, NO, in_elt="f64", out_elt="f64", pre=None, post=None):
    """lift2d.json of a whole-array host: A(NI, NK) column-major in the host's element type -> model rows
    x[i, k] = pre(A[i + NI*k]); model output y[i, k] -> B[i + NI*k] = post(y[i, k]).  `pre` / `post` are expression
    trees over ["A"], ["V", name, len] (per-feature vector) and ["C", value] with arith.addf / subf / mulf / divf
    nodes (driver/fortis_lift2d.py:98-115, 182-195), or None."""
    side = lambda e, elt: None if e is None else {"expr": e, "elt": elt}
    return {"layout": {"in": {"from": "col", "to": "row", "from_shape": [int(NI), int(NK)], "to_shape": [int(NI), int(NK)],
                              "from_elt": in_elt, "to_elt": "f32"},
                       "out": {"from": "row", "to": "col", "from_shape": [int(NI), int(NO)], "to_shape": [int(NI), int(NO)],
                               "from_elt": "f32", "to_elt": out_elt}},
            "pre": side(pre, in_elt), "post": side(post, out_elt), "drop": [], "new_args": []}


# -----------------------------------------------------------------------------------------------------------------
# random descriptor sets (differential testing: every case is valid by construction, sizes stay small)
# -----------------------------------------------------------------------------------------------------------------
def _random_expr(rng, scalars, depth=0):
    """A fully parenthesised C expression over tv, declared scalars and literals, safe for any finite tv in
    (-4, 4): divisions have denominators bounded away from zero, sqrt sees a non-negative operand."""
    leaves = ["tv"] + ["S%d" % k for k in scalars]
    r = rng.random()
    if depth >= 2 or r < 0.25:
        if rng.random() < 0.3:
            v = float(rng.uniform(0.25, 3.0))
            return ("%.6e" % v) + ("f" if rng.random() < 0.7 else "")
        return leaves[int(rng.integers(len(leaves)))]
    a = _random_expr(rng, scalars, depth + 1)
    b = _random_expr(rng, scalars, depth + 1)
    kind = int(rng.integers(7))
    if kind == 0:
        return "(%s + %s)" % (a, b)
    if kind == 1:
        return "(%s - %s)" % (a, b)
    if kind == 2:
        return "(%s * %s)" % (a, b)
    if kind == 3:
        return "(%s / ((%s * %s) + 1.500000e+00f))" % (a, b, b)
    if kind == 4:
        return "sqrtf(((%s * %s) + 1.000000e-03f))" % (a, a)
    if kind == 5:
        return "fmaxf(%s, fminf(%s, 2.000000e+00f))" % (a, b)
    return "(-%s)" % a


def random_case(rng, max_arrays=4, max_slots=24, max_out=6):
    """A random gather / scatter / loop / kdist set plus array shapes.  Returns (G, S, Lp, K, nargs, planes): nargs is the
    number of enclosing-loop integer arguments the non-distributed form takes (0 or 1), planes the extent of the plane
    dimension those arguments index."""
    two_d = rng.random() < 0.7
    ni = int(rng.integers(3, 40))
    nj = int(rng.integers(2, 12)) if two_d else 1
    halo = int(rng.integers(0, 3))
    planes = int(rng.integers(1, 5))
    kdist = planes > 1 and rng.random() < 0.6
    has_v = planes > 1
    sx, sy = ni + 2 * halo + int(rng.integers(0, 3)), nj + 2 * halo + int(rng.integers(0, 3))

    def shape(with_plane):
        s = [sx] + ([sy] if two_d else [])
        return s + ([planes] if with_plane else [])

    def index(with_plane, di=0, dj=0):
        idx = [["i", int(di)]] + ([["j", int(dj)]] if two_d else [])
        return idx + ([["v", 0]] if with_plane else [])

    nin_arr = int(rng.integers(1, max_arrays + 1))
    garr, gplane = [], []
    for a in range(nin_arr):
        wp = has_v and rng.random() < 0.8
        garr.append(_array("g%d" % a, shape(wp), "f64" if rng.random() < 0.3 else "f32"))
        gplane.append(wp)
    n = int(rng.integers(1, max_slots + 1))
    slots = []
    for _ in range(n):
        a = int(rng.integers(nin_arr))
        di = int(rng.integers(-halo, halo + 1)) if halo else 0
        dj = int(rng.integers(-halo, halo + 1)) if (halo and two_d) else 0
        slots.append({"array": a, "idx": index(gplane[a], di, dj)})
    nsc = int(rng.integers(0, 3))
    scalars = [{"name": "S%d" % k, "array": int(rng.integers(nin_arr)), "idx": None} for k in range(nsc)]
    for sc in scalars:
        sc["idx"] = index(gplane[sc["array"]])
    # scalars feed divisions and square roots: the generator keeps denominators away from zero by construction
    exprs = [_random_expr(rng, range(nsc)) for _ in range(int(rng.integers(0, 3)))]
    args = [{"alloca": "%k", "name": "k"}] if has_v else []
    G = {"ok": True, "n": n, "args": args, "arrays": garr, "scalars": scalars, "exprs": exprs, "slots": slots}

    nout = int(rng.integers(1, max_out + 1))
    # every stored array carries the plane dimension when the loop is distributed (a fused step requires it)
    sarr = [_array("s%d" % q, shape(has_v), "f64" if rng.random() < 0.3 else "f32") for q in range(nout)]
    stores = [{"slot": q, "array": q, "idx": index(has_v)} for q in range(nout)]
    sexprs = [_random_expr(rng, ()) for _ in range(int(rng.integers(0, 2)))]
    S = {"ok": True, "n": nout, "args": args, "arrays": sarr, "scalars": [], "exprs": sexprs, "stores": stores}
    nk = planes if kdist else 1
    Lp = _loop(ni * nj * nk, halo + 1, ni, (halo + 1, halo + nj) if two_d else None, n, nout)
    K = {"ok": True, "loop": {"lo": 1, "hi": planes}, "nk": planes} if kdist else None
    return G, S, Lp, K, (1 if (has_v and not kdist) else 0), planes
