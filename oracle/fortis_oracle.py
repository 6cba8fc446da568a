"""CPU restatement of the FORTIS gather -> NN forward -> scatter step.  TEST INFRASTRUCTURE ONLY.

This module is the parity checker.  Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline /
--impl reference legs may import it; the product (fortis_b200 and its CUDA library) never does.

What it restates, and where the reference defines it:
  * descriptor planning (strides, planes, "v" dims)      driver/fortis_gather_emit.py:16-36
  * gather row semantics (row -> col,kk -> i,j, exprs)   driver/fortis_gather_emit.py:52-62
  * scatter semantics (exprs on every output, stores)    driver/fortis_gather_emit.py:75-83, 91-96
  * boundary pre/post (transpose + cast + affine)        driver/fortis_boundary_trt.py:27-38
  * MLP forward conventions C[B,N] = A[B,K] . W[N,K]^T   runtime/fortis_rt.c:42-48
  * shipped native forward loop order                    mom6_zb/fwd_native_zb.f90:30-78
  * conv3d = cross-correlation, zero padding             runtime/fortis_rt.c:139-147
  * single convolution layers (2-D, strided, 'valid')    runtime/fortis_rt.c:108-156, runtime/fortis_fft.cu:66-79
  * 2-D operators of the micro-suite, by definition     tests/optest.py:6-32

Parity pins (see tests/test_oracle_golden.py): the ZB network's x_test -> y_test vector, the README checksum
stamps for the toy MLP and the conv probe, and gather/scatter outputs produced by compiling the reference's own
generated kernels for the CPU (tests/golden/make_golden.py); single convolution layers and 2-D operator networks
against outputs of torch's CPU operators (tests/golden/make_conv_golden.py, make_opnet_golden.py).

All float32 arithmetic is done op by op in numpy float32 (round-to-nearest, no fused multiply-add), which is what
the reference's `-fmad=false` gather/scatter kernels compute.
"""
from __future__ import annotations

import math
import re
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

# --------------------------------------------------------------------------------------------------------------
# expression strings of gather.json / scatter.json  (grammar: driver/fortis_gather.py:92-120)
# --------------------------------------------------------------------------------------------------------------
_TOK = re.compile(r"\s*(?:(\d+\.?\d*(?:[eE][-+]?\d+)?f?|\.\d+(?:[eE][-+]?\d+)?f?)|([A-Za-z_]\w*)|(.))")
_FUNCS1 = {"sqrtf": "sqrt", "expf": "exp", "logf": "log", "tanhf": "tanh",
           "sqrt": "sqrt", "exp": "exp", "log": "log", "tanh": "tanh"}
_FUNCS2 = {"fmaxf": "max", "fminf": "min", "fmax": "max", "fmin": "min"}


def parse_expr(text: str):
    """Parse a fully parenthesised C expression over tv, S<k>, literals, + - * /, unary minus and the
    sqrtf/expf/logf/tanhf/fmaxf/fminf calls into a nested tuple AST."""
    toks: List[Tuple[str, str]] = []
    pos = 0
    while pos < len(text):
        m = _TOK.match(text, pos)
        if not m:
            break
        pos = m.end()
        if m.group(1):
            toks.append(("num", m.group(1)))
        elif m.group(2):
            toks.append(("id", m.group(2)))
        elif m.group(3).strip():
            toks.append(("op", m.group(3)))
    idx = [0]

    def peek():
        return toks[idx[0]] if idx[0] < len(toks) else ("eof", "")

    def take(kind=None, val=None):
        t = peek()
        if (kind and t[0] != kind) or (val and t[1] != val):
            raise ValueError("expression %r: unexpected %r" % (text, t))
        idx[0] += 1
        return t

    def primary():
        t = peek()
        if t == ("op", "("):
            take()
            if peek() == ("op", "-"):           # unary minus is always written "(-x)"
                save = idx[0]
                take()
                inner = expr()
                if peek() == ("op", ")"):
                    take()
                    return ("neg", inner)
                idx[0] = save
            e = expr()
            take("op", ")")
            return e
        if t == ("op", "-"):
            take()
            return ("neg", primary())
        if t[0] == "num":
            take()
            s = t[1]
            is_f32 = s.endswith("f")
            return ("const", float(s[:-1] if is_f32 else s), is_f32)
        if t[0] == "id":
            take()
            if t[1] in _FUNCS1:
                take("op", "(")
                a = expr()
                take("op", ")")
                return (_FUNCS1[t[1]], a)
            if t[1] in _FUNCS2:
                take("op", "(")
                a = expr()
                take("op", ",")
                b = expr()
                take("op", ")")
                return (_FUNCS2[t[1]], a, b)
            if t[1] == "tv":
                return ("tv",)
            m = re.fullmatch(r"S(\d+)", t[1])
            if m:
                return ("scalar", int(m.group(1)))
            raise ValueError("expression %r: unknown identifier %s" % (text, t[1]))
        raise ValueError("expression %r: unexpected %r" % (text, t))

    def term():
        e = primary()
        while peek() in (("op", "*"), ("op", "/")):
            op = take()[1]
            e = ("mul" if op == "*" else "div", e, primary())
        return e

    def expr():
        e = term()
        while peek() in (("op", "+"), ("op", "-")):
            op = take()[1]
            e = ("add" if op == "+" else "sub", e, term())
        return e

    out = expr()
    if peek()[0] != "eof":
        raise ValueError("expression %r: trailing input" % text)
    return out


def fmax_cuda(a, b):
    """fmaxf as the GPU computes it (the reference's expressions run in its generated CUDA kernels): the number when
    one operand is NaN, and +0 > -0 (PTX max.f32), where C's fmax may return either zero."""
    a, b = np.asarray(a), np.asarray(b)
    r = np.fmax(a, b)
    zeros = (a == 0) & (b == 0)
    return np.where(zeros, np.where(np.signbit(a) & np.signbit(b), -0.0, 0.0).astype(r.dtype), r)


def fmin_cuda(a, b):
    """fminf as the GPU computes it: -0 < +0 (PTX min.f32)."""
    a, b = np.asarray(a), np.asarray(b)
    r = np.fmin(a, b)
    zeros = (a == 0) & (b == 0)
    return np.where(zeros, np.where(np.signbit(a) | np.signbit(b), -0.0, 0.0).astype(r.dtype), r)


def eval_expr(ast, tv, scalars: Dict[int, Any], dtype=np.float32):
    """Evaluate an AST in `dtype`, one IEEE operation per node (numpy never contracts a*b+c)."""
    k = ast[0]
    if k == "tv":
        return tv
    if k == "scalar":
        return scalars[ast[1]]
    if k == "const":
        return dtype(ast[1])
    if k == "neg":
        return -eval_expr(ast[1], tv, scalars, dtype)
    if k in ("sqrt", "exp", "log", "tanh"):
        a = eval_expr(ast[1], tv, scalars, dtype)
        return getattr(np, k)(a).astype(dtype) if isinstance(a, np.ndarray) else dtype(getattr(np, k)(a))
    a = eval_expr(ast[1], tv, scalars, dtype)
    b = eval_expr(ast[2], tv, scalars, dtype)
    if k == "add":
        return a + b
    if k == "sub":
        return a - b
    if k == "mul":
        return a * b
    if k == "div":
        with np.errstate(divide="ignore", invalid="ignore"):
            return a / b
    if k == "max":
        return fmax_cuda(a, b)
    if k == "min":
        return fmin_cuda(a, b)
    raise ValueError(k)


# --------------------------------------------------------------------------------------------------------------
# descriptor planning  (driver/fortis_gather_emit.py:9-36)
# --------------------------------------------------------------------------------------------------------------
_NP = {"f32": np.float32, "f64": np.float64}


def loop_params(Lp: Dict, K: Optional[Dict]):
    """count, ilo, ni, jlo, nj, nk, klo as the emitter derives them (fortis_gather_emit.py:9-12)."""
    nk, klo = (K["nk"], K["loop"]["lo"]) if (K and K.get("ok")) else (1, 0)
    count, ilo, ni = Lp["batch"] // nk, Lp["inner"]["lo"], Lp["inner"]["n"]
    jlo, nj = (Lp["outer"]["lo"], count // ni) if Lp.get("outer") else (0, 1)
    return dict(count=count, ilo=ilo, ni=ni, jlo=jlo, nj=nj, nk=nk, klo=klo, kdist=bool(K and K.get("ok")))


def plan_arrays(J: Dict, uses: Sequence[Tuple[int, list]]):
    """Per array: column-major strides, the trailing "v" (plane-selector) dims, plane and total sizes.
    `["c", n]` (constant 1-based subscript) is accepted beside the reference's i/j/v kinds."""
    out = []
    for ai, a in enumerate(J["arrays"]):
        shape = a["shape"]
        strides = [1]
        for nn in shape[:-1]:
            strides.append(strides[-1] * nn)
        mine = [idx for (aj, idx) in uses if aj == ai]
        vdims = sorted({di for idx in mine for di, c in enumerate(idx) if c[0] == "v"})
        if vdims != list(range(len(shape) - len(vdims), len(shape))):
            raise ValueError("plane dims must be the trailing dims (array %d)" % ai)
        plane = 1
        for di in range(len(shape) - len(vdims)):
            plane *= shape[di]
        total = plane
        for v in vdims:
            total *= shape[v]
        out.append(dict(dtype=_NP[a["elt"]], strides=strides, plane=plane, shape=shape, total=total, vdims=vdims,
                        idx=mine[0] if mine else None))
    return out


def _elem(A, ai, idx, i, j):
    """Offset inside one plane: sum over non-"v" dims of (var + off - 1) * stride (fortis_gather_emit.py:28-34)."""
    off = 0
    for di, c in enumerate(idx):
        st = A[ai]["strides"][di]
        if c[0] == "v":
            continue
        if c[0] == "i":
            off = off + (i + c[1] - 1) * st
        elif c[0] == "j":
            off = off + (j + c[1] - 1) * st
        elif c[0] == "c":
            off = off + (c[1] - 1) * st
        else:
            raise ValueError("unknown subscript kind %r" % (c[0],))
    return off


def _plane_off(A, ai, idx, args):
    """Element offset of the plane chosen by the enclosing-loop variables (fortis_gather_emit.py:35-36)."""
    return sum((int(args[c[1]]) - 1) * A[ai]["strides"][di] for di, c in enumerate(idx) if c[0] == "v")


def _flat(arr, dtype):
    a = np.asarray(arr)
    if a.dtype != dtype:
        raise TypeError("host array has dtype %s, descriptor says %s" % (a.dtype, np.dtype(dtype)))
    return a.reshape(-1, order="F") if a.ndim > 1 else a


# --------------------------------------------------------------------------------------------------------------
# gather / scatter  (driver/fortis_gather_emit.py:49-97)
# --------------------------------------------------------------------------------------------------------------
def gather(G: Dict, Lp: Dict, K: Optional[Dict], arrays: Sequence[np.ndarray], args: Sequence[int] = ()):
    """X[row, q] for row in [0, count*nk): the model input the reference's fortis_gather_k writes.
    `arrays` are the host's Fortran arrays (any ndim, Fortran order or flat); `args` the enclosing-loop
    variables (1-based) when there is no k-distribution."""
    P = loop_params(Lp, K)
    uses = [(s["array"], s["idx"]) for s in G["slots"]] + [(s["array"], s["idx"]) for s in G["scalars"]]
    A = plan_arrays(G, uses)
    flat = [_flat(arrays[ai], A[ai]["dtype"]) for ai in range(len(A))]
    n, count, nk = G["n"], P["count"], P["nk"]
    rows = np.arange(count * nk, dtype=np.int64)
    col, kk = rows % count, rows // count
    i = P["ilo"] + col % P["ni"]
    j = P["jlo"] + col // P["ni"]
    base = []
    for ai in range(len(A)):
        if P["kdist"]:
            # device buffer holds planes klo..klo+nk-1; row's plane is kk      (emit :55-56, :66).
            # An array without a plane dimension is the same for every kk (the reference would step past its
            # end there, so no reference host has one; the well-defined reading is used).
            base.append(((P["klo"] - 1) + kk) * A[ai]["plane"] if A[ai]["vdims"] else np.zeros_like(rows))
        else:
            base.append(np.full_like(rows, _plane_off(A, ai, A[ai]["idx"], args) if A[ai]["idx"] else 0))
    exprs = [parse_expr(e) for e in G["exprs"]]
    scal = {}
    for s in G["scalars"]:
        ai = s["array"]
        k = int(re.fullmatch(r"S(\d+)", s["name"]).group(1))
        v = flat[ai][base[ai] + _elem(A, ai, s["idx"], i, j)]
        scal[k] = v  # kept in the array's own type, as `const T S = A[...]` does
    X = np.empty((count * nk, n), dtype=np.float32)
    for q, s in enumerate(G["slots"]):
        ai = s["array"]
        tv = flat[ai][base[ai] + _elem(A, ai, s["idx"], i, j)].astype(np.float32)  # `float tv = A[...]`
        for e in exprs:
            tv = _eval_c(e, tv, scal)
        X[:, q] = tv
    return X


def _eval_c(ast, tv, scal):
    """`tv = <expr>;` with C's usual arithmetic conversions applied PER OPERATION: an operation is done in double
    iff one of its operands is double (an f64 array scalar or an unsuffixed literal), the *f functions take and
    return float, and the assignment narrows the result to float."""
    v, _ = _eval_typed(ast, np.asarray(tv, dtype=np.float32), scal)
    return np.asarray(v).astype(np.float32)


def _eval_typed(ast, tv, scal):
    k = ast[0]
    if k == "tv":
        return tv, False
    if k == "scalar":
        v = scal[ast[1]]
        return v, np.asarray(v).dtype == np.float64
    if k == "const":
        return (np.float32(ast[1]), False) if ast[2] else (np.float64(ast[1]), True)
    if k == "neg":
        v, d = _eval_typed(ast[1], tv, scal)
        return -v, d
    if k in ("sqrt", "exp", "log", "tanh"):
        v, _ = _eval_typed(ast[1], tv, scal)
        return getattr(np, k)(np.asarray(v).astype(np.float32)).astype(np.float32), False
    a, da = _eval_typed(ast[1], tv, scal)
    b, db = _eval_typed(ast[2], tv, scal)
    if k in ("max", "min"):
        f = fmax_cuda if k == "max" else fmin_cuda
        return f(np.asarray(a).astype(np.float32), np.asarray(b).astype(np.float32)).astype(np.float32), False
    d = da or db
    dt = np.float64 if d else np.float32
    a, b = np.asarray(a).astype(dt), np.asarray(b).astype(dt)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        r = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide}[k](a, b)
    return r, d


def scatter(S: Dict, Lp: Dict, K: Optional[Dict], Y: np.ndarray, arrays: Sequence[np.ndarray],
            args: Sequence[int] = ()):
    """One fortis_scatter(a0, ...) call: applies the exprs to every output of every column and stores into the
    host arrays IN PLACE (arrays must be Fortran-ordered or flat so that reshape(-1, order='F') is a view).
    `Y` is the whole model output (count*nk, nout); with k-distribution args[0] = a0 picks the row block."""
    P = loop_params(Lp, K)
    uses = [(s["array"], s["idx"]) for s in S["stores"]] + [(s["array"], s["idx"]) for s in S["scalars"]]
    A = plan_arrays(S, uses)
    flat = []
    for ai in range(len(A)):
        f = _flat(arrays[ai], A[ai]["dtype"])
        if not np.shares_memory(f, np.asarray(arrays[ai])):
            raise ValueError("array %d is not Fortran-contiguous; scatter could not write in place" % ai)
        flat.append(f)
    nout, count = S["n"], P["count"]
    cols = np.arange(count, dtype=np.int64)
    i = P["ilo"] + cols % P["ni"]
    j = P["jlo"] + cols // P["ni"]
    Y = np.asarray(Y, dtype=np.float32).reshape(-1, nout)
    yoff = (int(args[0]) - P["klo"]) * count if P["kdist"] else 0
    yv = [Y[yoff:yoff + count, q].copy() for q in range(nout)]
    poff = [(_plane_off(A, ai, A[ai]["idx"], args) if A[ai]["idx"] else 0) for ai in range(len(A))]
    scal = {}
    for s in S["scalars"]:
        ai = s["array"]
        k = int(re.fullmatch(r"S(\d+)", s["name"]).group(1))
        scal[k] = flat[ai][poff[ai] + _elem(A, ai, s["idx"], i, j)]
    for e in [parse_expr(e) for e in S["exprs"]]:
        for q in range(nout):
            yv[q] = _eval_c(e, yv[q], scal)
    for s in S["stores"]:
        ai = s["array"]
        flat[ai][poff[ai] + _elem(A, ai, s["idx"], i, j)] = yv[s["slot"]].astype(A[ai]["dtype"])


# --------------------------------------------------------------------------------------------------------------
# whole-array boundary (lift2d.json)  (driver/fortis_boundary_trt.py:27-38, driver/fortis_emit2d.py:20-52)
# --------------------------------------------------------------------------------------------------------------
def _tree(e, a, vecs, dt):
    if e[0] == "A":
        return a
    if e[0] == "V":
        return np.asarray(vecs[e[1]], dtype=dt)[None, :]
    if e[0] == "C":
        return dt(float(e[1]))
    x, y = _tree(e[1], a, vecs, dt), _tree(e[2], a, vecs, dt)
    op = e[0]
    with np.errstate(divide="ignore", invalid="ignore"):
        return {"arith.addf": np.add, "arith.subf": np.subtract, "arith.mulf": np.multiply,
                "arith.divf": np.divide}[op](x, y)


def boundary_pre(L2: Dict, A_host: np.ndarray, vecs: Dict[str, np.ndarray]) -> np.ndarray:
    """x[i,k] = (float) pre(A[i + NI*k], vec[k]) evaluated in the host's element type."""
    lin = L2["layout"]["in"]
    NI, NK = lin["from_shape"]
    dt = _NP[lin["from_elt"]]
    a = _flat(A_host, dt).reshape(NK, NI).T            # a[i,k] = A[i + NI*k]
    if L2.get("pre"):
        a = _tree(L2["pre"]["expr"], a, vecs, dt)
    return np.ascontiguousarray(a.astype(np.float32))


def boundary_post(L2: Dict, Y: np.ndarray, B_host: np.ndarray, vecs: Dict[str, np.ndarray]) -> None:
    """B[i + NI*k] = post((OT) y[i,k], vec[k]) written in place into the host array."""
    lout = L2["layout"]["out"]
    NI, NO = lout["to_shape"]
    dt = _NP[lout["to_elt"]]
    b = np.asarray(Y, dtype=np.float32).reshape(NI, NO).astype(dt)
    if L2.get("post"):
        b = _tree(L2["post"]["expr"], b, vecs, dt)
    f = _flat(B_host, dt)
    f[:NI * NO] = np.asarray(b, dtype=dt).T.reshape(-1)


# --------------------------------------------------------------------------------------------------------------
# model forward
# --------------------------------------------------------------------------------------------------------------
def act_apply(y, act: str, slope: float = 0.0):
    if act == "relu":
        return np.maximum(y, y.dtype.type(0))
    if act == "leaky":
        return np.where(y > 0, y, y * y.dtype.type(slope))
    return y


def mlp_forward(layers: Sequence[Dict], X: np.ndarray, dtype=np.float32, in_norms=None, out_norms=None,
                relu_mask=None) -> np.ndarray:
    """y = act(x . W^T + b) per layer; W is (out, in) as torch.nn.Linear stores it (runtime/fortis_rt.c:42).
    in_norms divides the input, out_norms multiplies the output (mom6_zb/export_zb.py:6-14); relu_mask marks
    outputs that get a final ReLU (benchmarks/climsim/export_wide.py:24-27)."""
    h = np.asarray(X, dtype=dtype)
    if in_norms is not None:
        h = h / np.asarray(in_norms, dtype=dtype)
    for L in layers:
        W = np.asarray(L["W"], dtype=dtype)
        h = h @ W.T + np.asarray(L["b"], dtype=dtype)
        h = act_apply(h, L.get("act", "none"), L.get("slope", 0.0)).astype(dtype)
    if out_norms is not None:
        h = h * np.asarray(out_norms, dtype=dtype)
    if relu_mask is not None:
        m = np.asarray(relu_mask) != 0
        h = np.where(m[None, :], np.maximum(h, dtype(0)), h)
    return h


def mlp_forward_native(layers, X, in_norms=None, out_norms=None) -> np.ndarray:
    """The shipped CPU forward's loop order (mom6_zb/fwd_native_zb.f90:36-47): y = 0; for each input i, for
    each output j: y(j) += x(i)*A(j,i); then + bias, then activation.  float32, one rounding per operation."""
    h = np.asarray(X, dtype=np.float32)
    if in_norms is not None:
        h = h / np.asarray(in_norms, dtype=np.float32)
    for L in layers:
        W = np.asarray(L["W"], dtype=np.float32)
        y = np.zeros((h.shape[0], W.shape[0]), dtype=np.float32)
        for i in range(W.shape[1]):
            y = y + h[:, i:i + 1] * W[None, :, i]
        y = y + np.asarray(L["b"], dtype=np.float32)
        h = act_apply(y, L.get("act", "none"), L.get("slope", 0.0)).astype(np.float32)
    if out_norms is not None:
        h = h * np.asarray(out_norms, dtype=np.float32)
    return h


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 -> float32."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = r.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), x, out).astype(np.float32)


def round_fp16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> IEEE half -> float32 (overflow goes to infinity, as the conversion
    instruction does)."""
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def quant_e4m3(W: np.ndarray):
    """Per-output-channel FP8-E4M3 weights: scale[n] = max_k |W[n,k]| / 448; Wq = e4m3(W / scale)
    (round-to-nearest-even, saturating).  Returns (dequantised-code values as float32, scale)."""
    W = np.asarray(W, dtype=np.float32)
    amax = np.abs(W).max(axis=1)
    scale = np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
    v = (W / scale[:, None]).astype(np.float32)
    return e4m3_round(v), scale


def e4m3_round(v: np.ndarray) -> np.ndarray:
    """Nearest (ties-to-even) E4M3 value of each float32, saturating at +-448.  E4M3: 4 exponent bits (bias 7),
    3 mantissa bits, subnormal step 2^-9."""
    v = np.asarray(v, dtype=np.float32)
    a = np.minimum(np.abs(v).astype(np.float64), 448.0)
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -20)))
    e = np.clip(e, -6, 8)
    step = 2.0 ** (e - 3)
    q = np.round(a / step) * step          # np.round is ties-to-even
    q = np.minimum(q, 448.0)
    return (np.sign(v) * q).astype(np.float32)


def mlp_forward_lowp(layers, X, mode: str) -> np.ndarray:
    """Model of the tensor-core path: activations rounded to bf16 (mode 'fp16': to IEEE half) at every layer input,
    weights bf16 (mode 'bf16'), half (mode 'fp16') or E4M3 codes with a per-channel fp32 scale applied after
    accumulation (mode 'fp8w'), products accumulated in high precision, bias + activation in fp32."""
    h = np.asarray(X, dtype=np.float32)
    rnd = round_fp16 if mode == "fp16" else round_bf16
    for L in layers:
        a = rnd(h).astype(np.float64)
        W = np.asarray(L["W"], dtype=np.float32)
        if mode == "fp8w":
            Wq, sc = quant_e4m3(W)
            y = (a @ Wq.astype(np.float64).T) * sc.astype(np.float64)[None, :]
        else:
            y = a @ rnd(W).astype(np.float64).T
        y = y.astype(np.float32) + np.asarray(L["b"], dtype=np.float32)
        h = act_apply(y, L.get("act", "none"), L.get("slope", 0.0)).astype(np.float32)
    return h


def conv3d_ndhwc(x: np.ndarray, W: np.ndarray, b: Optional[np.ndarray], pad: int = 1, dtype=np.float32):
    """Cross-correlation, stride 1, zero padding.  x (N,D,H,W,C); W (F,C,KD,KH,KW) as torch stores it;
    returns (N,D',H',W',F)."""
    x = np.asarray(x, dtype=dtype)
    W = np.asarray(W, dtype=dtype)
    N, D, H, Wd, C = x.shape
    F, _, KD, KH, KW = W.shape
    xp = np.pad(x, ((0, 0), (pad, pad), (pad, pad), (pad, pad), (0, 0)))
    Do, Ho, Wo = D + 2 * pad - KD + 1, H + 2 * pad - KH + 1, Wd + 2 * pad - KW + 1
    y = np.zeros((N, Do, Ho, Wo, F), dtype=dtype)
    for kd in range(KD):
        for kh in range(KH):
            for kw in range(KW):
                y += xp[:, kd:kd + Do, kh:kh + Ho, kw:kw + Wo, :] @ W[:, :, kd, kh, kw].T
    if b is not None:
        y = y + np.asarray(b, dtype=dtype)
    return y


def conv_ncdhw(x: np.ndarray, W: np.ndarray, stride=(1, 1, 1), pad=(0, 0, 0), dtype=np.float32):
    """The single-layer library rules fortis_conv2d / fortis_conv3d / fortis_conv3d_fft (runtime/fortis_rt.c:108-156,
    runtime/fortis_fft.cu:66-79): cross-correlation with zero padding, x (N,C,D,H,W), W (F,C,KD,KH,KW), any stride and
    padding per axis; returns (N,F,D',H',W').  A 2-D convolution is D = KD = 1."""
    x = np.asarray(x, dtype=dtype)
    W = np.asarray(W, dtype=dtype)
    N, C, D, H, Wd = x.shape
    F, _, KD, KH, KW = W.shape
    (sd, sh, sw), (pd, ph, pw) = stride, pad
    xp = np.pad(x, ((0, 0), (0, 0), (pd, pd), (ph, ph), (pw, pw)))
    Do, Ho, Wo = (D + 2 * pd - KD) // sd + 1, (H + 2 * ph - KH) // sh + 1, (Wd + 2 * pw - KW) // sw + 1
    y = np.zeros((N, F, Do, Ho, Wo), dtype=dtype)
    for kd in range(KD):
        for kh in range(KH):
            for kw in range(KW):
                win = xp[:, :, kd:kd + (Do - 1) * sd + 1:sd, kh:kh + (Ho - 1) * sh + 1:sh, kw:kw + (Wo - 1) * sw + 1:sw]
                y += np.einsum("ncdhw,fc->nfdhw", win, W[:, :, kd, kh, kw])
    return y


# ---------------------------------------------------------------------------------------------------------------
# 2-D operators of the reference's micro-suite (tests/optest.py:6-32), NCHW, each by its definition
# ---------------------------------------------------------------------------------------------------------------
def conv2d_nchw(x, W, b=None, stride=(1, 1), pad=(0, 0), dil=1, extra=(0, 0), dtype=np.float64):
    """Cross-correlation (runtime/fortis_rt.c:108-127) of the input dilated by `dil` (zeros between samples), zero-padded
    by `pad` on both sides and by `extra` more rows / columns behind."""
    x = np.asarray(x, dtype=dtype)
    N, C, H, Wd = x.shape
    xd = np.zeros((N, C, (H - 1) * dil + 1, (Wd - 1) * dil + 1), dtype=dtype)
    xd[:, :, ::dil, ::dil] = x
    xd = np.pad(xd, ((0, 0), (0, 0), (pad[0], pad[0] + extra[0]), (pad[1], pad[1] + extra[1])))
    y = conv_ncdhw(xd[:, :, None], np.asarray(W, dtype=dtype)[:, :, None], stride=(1, stride[0], stride[1]), dtype=dtype)[:, :, 0]
    return y if b is None else y + np.asarray(b, dtype=dtype)[None, :, None, None]


def conv_transpose2d(x, W, b=None, stride=1, pad=(0, 0), opad=(0, 0), dtype=np.float64):
    """Transposed convolution by its definition: every input sample adds its value times the kernel into the output
    at stride * position - pad.  W is (Cin, Cout, KH, KW)."""
    x, W = np.asarray(x, dtype=dtype), np.asarray(W, dtype=dtype)
    N, C, H, Wd = x.shape
    _, F, KH, KW = W.shape
    Ho, Wo = (H - 1) * stride - 2 * pad[0] + KH + opad[0], (Wd - 1) * stride - 2 * pad[1] + KW + opad[1]
    full = np.zeros((N, F, (H - 1) * stride + KH + opad[0], (Wd - 1) * stride + KW + opad[1]), dtype=dtype)
    for kh in range(KH):
        for kw in range(KW):
            full[:, :, kh:kh + (H - 1) * stride + 1:stride, kw:kw + (Wd - 1) * stride + 1:stride] += np.einsum("nchw,cf->nfhw", x, W[:, :, kh, kw])
    y = full[:, :, pad[0]:pad[0] + Ho, pad[1]:pad[1] + Wo]
    return y if b is None else y + np.asarray(b, dtype=dtype)[None, :, None, None]


def maxpool2d(x, k, stride=None):
    k = (k, k) if np.isscalar(k) else k
    stride = k if stride is None else ((stride, stride) if np.isscalar(stride) else stride)
    N, C, H, Wd = x.shape
    Ho, Wo = (H - k[0]) // stride[0] + 1, (Wd - k[1]) // stride[1] + 1
    y = np.full((N, C, Ho, Wo), -np.inf, dtype=x.dtype)
    for i in range(k[0]):
        for j in range(k[1]):
            y = np.maximum(y, x[:, :, i:i + (Ho - 1) * stride[0] + 1:stride[0], j:j + (Wo - 1) * stride[1] + 1:stride[1]])
    return y


def upsample_nearest2d(x, scale):
    scale = (scale, scale) if np.isscalar(scale) else scale
    return np.repeat(np.repeat(x, scale[0], axis=2), scale[1], axis=3)


def batchnorm2d(x, gamma, beta, mean, var, eps):
    sh = (1, -1, 1, 1)
    return (x - np.reshape(mean, sh)) / np.sqrt(np.reshape(var, sh) + eps) * np.reshape(gamma, sh) + np.reshape(beta, sh)


def ops2d_forward(spec, x, dtype=np.float64):
    """A 2-D network given op by op, unfused: ('conv', W, b, stride, pad) | ('convT', W, b, stride, pad, opad) |
    ('bn', gamma, beta, mean, var, eps) | ('relu',) | ('leaky', slope) | ('maxpool', k) | ('upsample', scale) |
    ('pad', p) | ('cat', [spec, spec, ...]) (channel concatenation of sub-networks applied to the same input)."""
    h = np.asarray(x, dtype=dtype)
    for op in spec:
        kind = op[0]
        if kind == "conv":
            h = conv2d_nchw(h, op[1], op[2], stride=op[3], pad=op[4], dtype=dtype)
        elif kind == "convT":
            h = conv_transpose2d(h, op[1], op[2], stride=op[3], pad=op[4], opad=op[5], dtype=dtype)
        elif kind == "bn":
            h = batchnorm2d(h, *op[1:])
        elif kind == "relu":
            h = np.maximum(h, 0)
        elif kind == "leaky":
            h = np.where(h > 0, h, h * op[1])
        elif kind == "maxpool":
            h = maxpool2d(h, op[1])
        elif kind == "upsample":
            h = upsample_nearest2d(h, op[1])
        elif kind == "pad":
            h = np.pad(h, ((0, 0), (0, 0), (op[1], op[1]), (op[1], op[1])))
        elif kind == "cat":
            h = np.concatenate([ops2d_forward(sub, h, dtype) for sub in op[1]], axis=1)
        else:
            raise ValueError(kind)
    return h


def opnet_forward(layers, x, dtype=np.float32):
    """The exported form of such a network (fortis_b200.model.write_blob layer dicts: conv2d with folded BatchNorm /
    padding / concatenation and dilated-input transposed convolutions, maxpool2d, upsample2d), layer by layer."""
    h = np.asarray(x, dtype=dtype)
    for L in layers:
        if L["op"] == "conv2d":
            h = conv2d_nchw(h, L["W"], L["b"], stride=L.get("stride", (1, 1)), pad=L.get("pad", (0, 0)), dil=L.get("dil", 1),
                            extra=L.get("extra", (0, 0)), dtype=dtype)
            h = act_apply(h, L.get("act", "none"), L.get("slope", 0.0)).astype(dtype)
        elif L["op"] == "maxpool2d":
            h = maxpool2d(h, L["k"], L.get("stride"))
        else:
            h = upsample_nearest2d(h, L["scale"])
    return h


def convnet_forward(layers: Sequence[Dict], x: np.ndarray, dtype=np.float32) -> np.ndarray:
    """Sequence of conv3d layers with fused activation and optional residual.  Each layer dict: W, b, act,
    slope, and `save` (remember this layer's output as the skip) / `add` (add the remembered skip after the conv,
    before the activation)."""
    h = np.asarray(x, dtype=dtype)
    skip = None
    for L in layers:
        y = conv3d_ndhwc(h, L["W"], L.get("b"), L.get("pad", 1), dtype)
        if L.get("add"):
            y = y + skip
        y = act_apply(y, L.get("act", "none"), L.get("slope", 0.0)).astype(dtype)
        if L.get("save"):
            skip = y
        h = y
    return h


def convnet_forward_lowp(layers: Sequence[Dict], x: np.ndarray, mode: str = "bf16") -> np.ndarray:
    """Model of the 16-bit tensor-core conv network: the input and every layer's weights are rounded to bf16 (mode
    'fp16': IEEE half), products are accumulated wide, bias / skip / activation are applied in fp32, and every
    intermediate activation (including the remembered skip) is stored in the 16-bit format; the last layer's output
    stays fp32."""
    n = len(layers)
    round_bf16 = globals()["round_fp16"] if mode == "fp16" else globals()["round_bf16"]      # noqa: F841 (shadows on purpose)
    h = round_bf16(np.asarray(x, dtype=np.float32))
    skip = None
    for l, L in enumerate(layers):
        y = conv3d_ndhwc(h.astype(np.float64), round_bf16(L["W"]).astype(np.float64), None, L.get("pad", 1), np.float64)
        y = y.astype(np.float32) + np.asarray(L["b"], np.float32)
        if L.get("add"):
            y = y + skip
        y = act_apply(y, L.get("act", "none"), L.get("slope", 0.0)).astype(np.float32)
        if l < n - 1:
            y = round_bf16(y)
        if L.get("save"):
            skip = y
        h = y
    return h


def rel_l2(y, ref) -> float:
    y = np.asarray(y, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    d = np.linalg.norm(ref)
    return float(np.linalg.norm(y - ref) / (d if d > 0 else 1.0))


# --------------------------------------------------------------------------------------------------------------
# the ZB host's synthetic fields  (mom6_zb/zb_host.f90:37-40, 128-138)
# --------------------------------------------------------------------------------------------------------------
class ZbLcg:
    """seed = mod(seed*1103515245 + 12345, 2^31), shared across the three make_field calls."""

    def __init__(self, seed=12345):
        self.seed = seed

    def field(self, szi, szj, nz, a, b, c):
        n = szi * szj * nz
        r = np.empty(n, dtype=np.float64)
        s = self.seed
        for t in range(n):
            s = (s * 1103515245 + 12345) % 2147483648
            r[t] = s / 2147483648.0 - 0.5
        self.seed = s
        r = r.reshape((szi, szj, nz), order="F")
        i = np.arange(1, szi + 1, dtype=np.float64)[:, None, None]
        j = np.arange(1, szj + 1, dtype=np.float64)[None, :, None]
        k = np.arange(1, nz + 1, dtype=np.float64)[None, None, :]
        return np.asfortranarray(1e-5 * (0.6 * np.sin(a * i + b * j + c * k) * np.cos(b * i - a * j) + 0.4 * r))


# --------------------------------------------------------------------------------------------------------------
# descriptor builders for the benchmark configurations (the schema producers emit: driver/fortis_gather.py:201-206)
# --------------------------------------------------------------------------------------------------------------
def stencil_descriptors(nx: int, ny: int, nz: int, nfields: int = 3, nout: int = 3, halo: int = 1, elt="f32"):
    """3x3 stencil of `nfields` (nx+2h, ny+2h, nz) fields per interior point, field-major then i fastest then j
    (the RESHAPE order of mom6_zb/zb_host.f90:79-87); `nout` outputs stored at (i,j,k) of separate arrays;
    the k loop is distributed (kdist)."""
    sx, sy = nx + 2 * halo, ny + 2 * halo
    arr = lambda name: {"ssa": "%" + name, "name": name, "shape": [sx, sy, nz], "elt": elt}
    slots = [{"array": f, "idx": [["i", di], ["j", dj], ["v", 0]]}
             for f in range(nfields) for dj in (-1, 0, 1) for di in (-1, 0, 1)]
    G = {"ok": True, "n": 9 * nfields, "args": [{"alloca": "%k", "name": "k"}],
         "arrays": [arr("in%d" % f) for f in range(nfields)], "scalars": [], "exprs": [], "slots": slots}
    S = {"ok": True, "n": nout, "args": [{"alloca": "%k", "name": "k"}],
         "arrays": [arr("out%d" % q) for q in range(nout)], "scalars": [], "exprs": [],
         "stores": [{"slot": q, "array": q, "idx": [["i", 0], ["j", 0], ["v", 0]]} for q in range(nout)]}
    Lp = {"verdict": "batched", "batch": nx * ny * nz, "inner": {"lo": halo + 1, "hi": halo + nx, "n": nx},
          "outer": {"lo": halo + 1, "hi": halo + ny}, "in_shape": [9 * nfields], "out_shape": [nout],
          "in_elt": "f32", "out_elt": "f32"}
    K = {"ok": True, "loop": {"lo": 1, "hi": nz}, "nk": nz}
    return G, S, Lp, K


def column_descriptors(ncol: int, nlev: int, nfields: int = 4, nscal: int = 4, nout_fields: int = 2,
                       nout_scal: int = 8, elt="f32"):
    """Column physics: features [F0(1:nlev), F1(1:nlev), ..., s0, s1, ...] gathered from (ncol,nlev) fields and
    (ncol) vectors with constant level subscripts; outputs to `nout_fields` (ncol,nlev) arrays and `nout_scal`
    (ncol) vectors."""
    arrays = [{"ssa": "%%f%d" % f, "name": "f%d" % f, "shape": [ncol, nlev], "elt": elt} for f in range(nfields)]
    arrays += [{"ssa": "%%s%d" % s, "name": "s%d" % s, "shape": [ncol], "elt": elt} for s in range(nscal)]
    slots = [{"array": f, "idx": [["i", 0], ["c", l + 1]]} for f in range(nfields) for l in range(nlev)]
    slots += [{"array": nfields + s, "idx": [["i", 0]]} for s in range(nscal)]
    G = {"ok": True, "n": len(slots), "args": [], "arrays": arrays, "scalars": [], "exprs": [], "slots": slots}
    oarr = [{"ssa": "%%o%d" % f, "name": "o%d" % f, "shape": [ncol, nlev], "elt": elt} for f in range(nout_fields)]
    oarr += [{"ssa": "%%t%d" % s, "name": "t%d" % s, "shape": [ncol], "elt": elt} for s in range(nout_scal)]
    stores = [{"slot": f * nlev + l, "array": f, "idx": [["i", 0], ["c", l + 1]]}
              for f in range(nout_fields) for l in range(nlev)]
    stores += [{"slot": nout_fields * nlev + s, "array": nout_fields + s, "idx": [["i", 0]]}
               for s in range(nout_scal)]
    S = {"ok": True, "n": len(stores), "args": [], "arrays": oarr, "scalars": [], "exprs": [], "stores": stores}
    Lp = {"verdict": "batched", "batch": ncol, "inner": {"lo": 1, "hi": ncol, "n": ncol}, "outer": None,
          "in_shape": [len(slots)], "out_shape": [len(stores)], "in_elt": "f32", "out_elt": "f32"}
    return G, S, Lp, None


def identity_descriptors(nfeat_in: int, nfeat_out: int, ncol: int, elt="f32"):
    """Toy config: host array A(nfeat_in, ncol) column-major read column by column, output into B(nfeat_out, ncol).
    The column index is the second dimension, so it is the 'j'-free inner variable on dim 1 with stride nfeat."""
    G = {"ok": True, "n": nfeat_in, "args": [],
         "arrays": [{"ssa": "%a", "name": "a", "shape": [nfeat_in, ncol], "elt": elt}], "scalars": [], "exprs": [],
         "slots": [{"array": 0, "idx": [["c", f + 1], ["i", 0]]} for f in range(nfeat_in)]}
    S = {"ok": True, "n": nfeat_out, "args": [],
         "arrays": [{"ssa": "%b", "name": "b", "shape": [nfeat_out, ncol], "elt": elt}], "scalars": [], "exprs": [],
         "stores": [{"slot": f, "array": 0, "idx": [["c", f + 1], ["i", 0]]} for f in range(nfeat_out)]}
    Lp = {"verdict": "batched", "batch": ncol, "inner": {"lo": 1, "hi": ncol, "n": ncol}, "outer": None,
          "in_shape": [nfeat_in], "out_shape": [nfeat_out], "in_elt": "f32", "out_elt": "f32"}
    return G, S, Lp, None


def checksum(arrays: Sequence[np.ndarray]) -> float:
    """fp64 sum of all scattered outputs."""
    return float(sum(np.asarray(a, dtype=np.float64).sum() for a in arrays))


def full_step(G, S, Lp, K, layers, in_arrays, out_arrays, forward=None, **fw):
    """gather -> forward -> scatter(every k) on the CPU; writes out_arrays in place, returns (X, Y)."""
    P = loop_params(Lp, K)
    X = gather(G, Lp, K, in_arrays, args=(1,))
    Y = (forward or mlp_forward)(layers, X, **fw)
    if P["kdist"]:
        for a0 in range(P["klo"], P["klo"] + P["nk"]):
            scatter(S, Lp, K, Y, out_arrays, args=(a0,))
    else:
        scatter(S, Lp, K, Y, out_arrays, args=(1,))
    return X, Y
