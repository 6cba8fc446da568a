#!/usr/bin/env python3
"""Generate the golden fixtures under tests/golden/ from the reference checkout.

Run where a checkout of the reference (sanatgp/Fortis) is available (it is NOT needed to run the tests):

    python tests/golden/make_golden.py [path-to-reference-checkout]

What it does
  1. Copies the reference's checked-in layout descriptors for the MOM6 Zanna-Bolton host (data, not code):
     mom6_zb/{gather,scatter,kdist}.json and mom6_zb/zb_loop_verdict.json  ->  tests/golden/zb_*.json
     (zb_loop.json with `batch` multiplied by nk, the step driver/fortisc.sh:44 applies before emission)
  2. Copies the ZB network weights and its known-answer vector (mom6_zb/zb_nn.npz) -> tests/golden/zb_nn.npz
  3. Runs the reference's OWN kernel emitter (driver/fortis_gather_emit.py) on descriptor sets, extracts the two
     generated `__global__` kernels, compiles them for the CPU behind a tiny shim that supplies blockIdx /
     threadIdx (g++ -O1 -ffp-contract=off, i.e. the same no-FMA arithmetic as the reference's -fmad=false), runs
     them on seeded inputs and records SHA-256 digests plus sampled rows of what they produce
     -> tests/golden/gather_scatter_golden.json.  Inputs are regenerated from the recorded seeds by the tests.
  4. Records the reference's correctness stamps that are reproducible with torch on the CPU: the toy MLP checksum
     (frontend/export_mlp.py model, benchmarks/toy/bench_fortis.f90 input; README stamp 7.775037) and the conv
     probe checksum (frontend/export_conv.py; README stamp 9617.28), together with the seeded weights so that the
     tests need neither torch's RNG stream nor the reference -> tests/golden/stamps.npz
"""
import ctypes
import hashlib
import json
import os
import re
import shutil
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import fortis_oracle as fo  # noqa: E402

REF = sys.argv[1] if len(sys.argv) > 1 else (os.environ.get("FORTIS_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference"))

SHIM = r"""
#include <math.h>
#include <stddef.h>
struct idx3 { int x, y, z; };
static idx3 blockIdx, blockDim, threadIdx;
#define __global__
"""


def emit_kernels(G, S, Lp, K, workdir):
    """Run the reference emitter and return the text of fortis_gather_k / fortis_scatter_k."""
    paths = []
    for name, obj in (("gather", G), ("scatter", S), ("loop", Lp), ("kdist", K)):
        if obj is None:
            continue
        p = os.path.join(workdir, name + ".json")
        json.dump(obj, open(p, "w"))
        paths.append(p)
    src = subprocess.run([sys.executable, os.path.join(REF, "driver", "fortis_gather_emit.py")] + paths,
                         check=True, capture_output=True, text=True).stdout
    kernels = re.findall(r"^__global__ void fortis_(?:gather|scatter)_k\(.*?^\}$", src, flags=re.S | re.M)
    return src, kernels


def build_cpu(G, S, Lp, K):
    """Compile the emitted kernels for the CPU; returns (gather_fn, scatter_fn) taking numpy arrays."""
    work = tempfile.mkdtemp(prefix="fortis_golden_")
    src, kernels = emit_kernels(G, S, Lp, K, work)
    P = fo.loop_params(Lp, K)
    cty = {"f32": "float", "f64": "double"}
    code = [SHIM] + kernels
    ga = [cty[a["elt"]] for a in G["arrays"]]
    sa = [cty[a["elt"]] for a in S["arrays"]]
    nrows = P["count"] * P["nk"]
    code.append('extern "C" void run_gather(void** A, float* X) {\n  blockDim.x = 256;\n'
                '  for (int b = 0; b < (%d + 255) / 256; b++) for (int t = 0; t < 256; t++) { blockIdx.x = b; threadIdx.x = t;\n'
                '    fortis_gather_k(%s, X, %d, %d, %d, %d); }\n}\n'
                % (nrows, ", ".join("(const %s*)A[%d]" % (t, i) for i, t in enumerate(ga)),
                   P["count"], P["ilo"], P["jlo"], P["ni"]))
    code.append('extern "C" void run_scatter(const float* Yd, void** A) {\n  blockDim.x = 256;\n'
                '  for (int b = 0; b < (%d + 255) / 256; b++) for (int t = 0; t < 256; t++) { blockIdx.x = b; threadIdx.x = t;\n'
                '    fortis_scatter_k(Yd, %s, %d, %d, %d, %d); }\n}\n'
                % (P["count"], ", ".join("(%s*)A[%d]" % (t, i) for i, t in enumerate(sa)),
                   P["count"], P["ilo"], P["jlo"], P["ni"]))
    cpp = os.path.join(work, "k.cpp")
    open(cpp, "w").write("\n".join(code))
    so = os.path.join(work, "k.so")
    subprocess.run(["g++", "-O1", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC", cpp, "-o", so], check=True)
    lib = ctypes.CDLL(so)

    def ptrs(arrs):
        return (ctypes.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])

    def gather(dev_arrays):
        """dev_arrays: what the reference's device buffers hold (planes klo..klo+nk-1 under kdist, else the
        selected plane)."""
        X = np.zeros((nrows, G["n"]), dtype=np.float32)
        lib.run_gather(ptrs(dev_arrays), X.ctypes.data_as(ctypes.c_void_p))
        return X

    def scatter(Yblock, dev_arrays):
        Yblock = np.ascontiguousarray(Yblock, dtype=np.float32)
        lib.run_scatter(Yblock.ctypes.data_as(ctypes.c_void_p), ptrs(dev_arrays))

    return gather, scatter, work


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def zb_inputs():
    """The ZB host's fields (LCG seed 12345) and a positive norm field, as float32 Fortran arrays (68,78,15)."""
    g = fo.ZbLcg(12345)
    sh_xy = g.field(68, 78, 15, 0.31, 0.23, 0.17).astype(np.float32)
    sh_xx = g.field(68, 78, 15, 0.27, 0.19, 0.13).astype(np.float32)
    vort = g.field(68, 78, 15, 0.29, 0.21, 0.11).astype(np.float32)
    norm = np.sqrt(sh_xy.astype(np.float32) ** 2 + sh_xx ** 2 + vort ** 2).astype(np.float32)
    return [np.asfortranarray(x) for x in (sh_xy, sh_xx, vort, norm)]


def case_inputs(J, seed):
    """Seeded arrays for a descriptor's `arrays`: values in (0.5, 1.5) so divisions and sqrt stay finite."""
    rng = np.random.default_rng(seed)
    out = []
    for a in J["arrays"]:
        v = rng.random(int(np.prod(a["shape"]))) + 0.5
        out.append(np.asfortranarray(v.astype(fo._NP[a["elt"]]).reshape(a["shape"], order="F")))
    return out


def extra_cases():
    """Descriptor sets in the reference's own schema (i/j/v subscripts only) covering: f64 arrays, several
    expressions, sqrtf/fmaxf, no k-distribution with an enclosing-loop argument, 1-D inner loop only."""
    cases = {}
    # (a) f64 arrays, two exprs, scalar from a 2-D array, kdist over 3 planes
    arr = lambda n, shp, e: {"ssa": "%" + n, "name": n, "shape": shp, "elt": e}
    G = {"ok": True, "n": 5, "args": [{"alloca": "%k", "name": "k"}],
         "arrays": [arr("p", [13, 9, 3], "f64"), arr("q", [13, 9, 3], "f32"), arr("w", [13, 9, 3], "f64")],
         "scalars": [{"name": "S0", "array": 2, "idx": [["i", 0], ["j", 0], ["v", 0]]},
                     {"name": "S1", "array": 1, "idx": [["i", 1], ["j", -1], ["v", 0]]}],
         "exprs": ["(((tv * S1) - 1.100000e+00f) / (S0 + 1.000000e-30f))", "fmaxf(sqrtf((tv * tv)), 2.500000e-01f)",
                   "((tv * 3.300000e-01) + (S1 * 7.000000e-01f))"],
         "slots": [{"array": 0, "idx": [["i", -1], ["j", 0], ["v", 0]]},
                   {"array": 0, "idx": [["i", 1], ["j", 1], ["v", 0]]},
                   {"array": 1, "idx": [["i", 0], ["j", -1], ["v", 0]]},
                   {"array": 1, "idx": [["i", 0], ["j", 0], ["v", 0]]},
                   {"array": 0, "idx": [["i", 0], ["j", 0], ["v", 0]]}]}
    S = {"ok": True, "n": 2, "args": [{"alloca": "%k", "name": "k"}],
         "arrays": [arr("w", [13, 9], "f64"), arr("r0", [13, 9, 3], "f64"), arr("r1", [13, 9], "f32")],
         "scalars": [{"name": "S0", "array": 0, "idx": [["i", 0], ["j", 0]]}],
         "exprs": ["(((tv * 1.700000e+00f) * S0) + 1.250000e-01f)", "(-tv)"],
         "stores": [{"slot": 1, "array": 1, "idx": [["i", 0], ["j", 0], ["v", 0]]},
                    {"slot": 0, "array": 2, "idx": [["i", 0], ["j", 0]]}]}
    Lp = {"batch": 11 * 7 * 3, "inner": {"lo": 2, "hi": 12, "n": 11}, "outer": {"lo": 2, "hi": 8}}
    K = {"ok": True, "loop": {"lo": 1, "hi": 3}, "nk": 3}
    cases["f64_kdist"] = (G, S, Lp, K, [1, 2, 3])
    # (b) no kdist: the enclosing-loop variable arrives as an argument and selects the plane
    G2 = {"ok": True, "n": 3, "args": [{"alloca": "%k", "name": "k"}],
          "arrays": [arr("u", [10, 6, 4], "f32"), arr("m", [10, 6], "f32")],
          "scalars": [{"name": "S0", "array": 1, "idx": [["i", 0], ["j", 0]]}],
          "exprs": ["(tv * (S0 - 5.000000e-01f))"],
          "slots": [{"array": 0, "idx": [["i", -1], ["j", 0], ["v", 0]]},
                    {"array": 0, "idx": [["i", 0], ["j", 0], ["v", 0]]},
                    {"array": 0, "idx": [["i", 1], ["j", 0], ["v", 0]]}]}
    S2 = {"ok": True, "n": 1, "args": [{"alloca": "%k", "name": "k"}],
          "arrays": [arr("o", [10, 6, 4], "f32")], "scalars": [], "exprs": [],
          "stores": [{"slot": 0, "array": 0, "idx": [["i", 0], ["j", 0], ["v", 0]]}]}
    Lp2 = {"batch": 8 * 6, "inner": {"lo": 2, "hi": 9, "n": 8}, "outer": {"lo": 1, "hi": 6}}
    cases["arg_plane"] = (G2, S2, Lp2, None, [3])
    # (c) inner loop only (1-D arrays)
    G3 = {"ok": True, "n": 2, "args": [], "arrays": [arr("a", [37], "f32")], "scalars": [], "exprs": [],
          "slots": [{"array": 0, "idx": [["i", 0]]}, {"array": 0, "idx": [["i", 1]]}]}
    S3 = {"ok": True, "n": 2, "args": [], "arrays": [arr("b", [37], "f32"), arr("c", [37], "f64")], "scalars": [],
          "exprs": ["(tv / 3.000000e+00f)"],
          "stores": [{"slot": 0, "array": 0, "idx": [["i", 0]]}, {"slot": 1, "array": 1, "idx": [["i", 1]]}]}
    Lp3 = {"batch": 33, "inner": {"lo": 2, "hi": 34, "n": 33}, "outer": None}
    cases["inner_only"] = (G3, S3, Lp3, None, [])
    return cases


def dev_view(J, A, arrays, P, args, for_scatter):
    """Reproduce what the reference's device buffers hold: the nk planes from klo (gather under kdist) or the one
    plane chosen by the arguments (fortis_gather_emit.py:66-68, 86-88)."""
    out = []
    for ai, a in enumerate(arrays):
        f = a.reshape(-1, order="F")
        pl = A[ai]["plane"]
        if P["kdist"] and not for_scatter:
            # every gather buffer holds plane*nk elements filled from H + (klo-1)*plane
            assert A[ai]["vdims"], "reference gather under kdist needs a plane dimension on every array"
            out.append(np.ascontiguousarray(f[(P["klo"] - 1) * pl:(P["klo"] - 1) * pl + pl * P["nk"]].copy()))
        else:
            off = fo._plane_off(A, ai, A[ai]["idx"], args) if A[ai]["idx"] else 0
            out.append(np.ascontiguousarray(f[off:off + pl].copy()))
    return out


def run_case(name, G, S, Lp, K, a0s, gin, sin, record):
    P = fo.loop_params(Lp, K)
    gather, scatter, work = build_cpu(G, S, Lp, K)
    Ag = fo.plan_arrays(G, [(s["array"], s["idx"]) for s in G["slots"]] + [(s["array"], s["idx"]) for s in G["scalars"]])
    As = fo.plan_arrays(S, [(s["array"], s["idx"]) for s in S["stores"]] + [(s["array"], s["idx"]) for s in S["scalars"]])
    gargs = a0s[:1] if not P["kdist"] else []
    X = gather(dev_view(G, Ag, gin, P, gargs, False))
    Xo = fo.gather(G, Lp, K, gin, args=gargs)
    assert X.tobytes() == Xo.tobytes(), "%s: oracle gather differs from the reference's generated kernel" % name
    rng = np.random.default_rng(99)
    Y = (rng.random((P["count"] * P["nk"], S["n"])) - 0.5).astype(np.float32)
    ref_out = [a.copy(order="F") for a in sin]
    ora_out = [a.copy(order="F") for a in sin]
    for a0 in (a0s if a0s else [1]):
        dv = dev_view(S, As, ref_out, P, [a0], True)
        yoff = (a0 - P["klo"]) * P["count"] if P["kdist"] else 0
        scatter(Y[yoff:yoff + P["count"]], dv)
        # copy the visited rectangle back (fortis_gather_emit.py:91-96): the kernel only wrote visited cells, so
        # copying every written plane back whole is equivalent for a CPU replay
        for s in S["stores"]:
            ai = s["array"]
            off = fo._plane_off(As, ai, s["idx"], [a0])
            ref_out[ai].reshape(-1, order="F")[off:off + As[ai]["plane"]] = dv[ai]
        fo.scatter(S, Lp, K, Y, ora_out, args=[a0])
    for ai in range(len(sin)):
        assert ref_out[ai].tobytes(order="F") == ora_out[ai].tobytes(order="F"), \
            "%s: oracle scatter differs from the reference's generated kernel (array %d)" % (name, ai)
    record[name] = {"gather": G, "scatter": S, "loop": Lp, "kdist": K, "a0s": a0s,
                    "X_sha256": digest(X), "X_rows": X[:: max(1, X.shape[0] // 7)][:8].astype(np.float64).tolist(),
                    "out_sha256": [digest(a.reshape(-1, order="F")) for a in ref_out]}
    shutil.rmtree(work, ignore_errors=True)
    print("golden case %-12s rows %6d  X sha %s" % (name, X.shape[0], record[name]["X_sha256"][:12]))


def stamps():
    import torch
    out = {}
    torch.manual_seed(42)
    net = torch.nn.Sequential(torch.nn.Linear(1024, 256), torch.nn.ReLU(), torch.nn.Linear(256, 1024)).eval()
    y = torch.arange(1, 1025, dtype=torch.float32) / 1024
    y = (y - y.sum() / 1024) / torch.sqrt(((y - y.sum() / 1024) ** 2).sum() / 1024)
    with torch.no_grad():
        z = net(y.view(1, -1))
    out.update(toy_W0=net[0].weight.detach().numpy(), toy_b0=net[0].bias.detach().numpy(),
               toy_W1=net[2].weight.detach().numpy(), toy_b1=net[2].bias.detach().numpy(),
               toy_x=y.numpy(), toy_checksum_torch=np.float64(z.sum().item()), toy_checksum_readme=np.float64(7.775037))
    torch.manual_seed(3)
    m = torch.nn.Sequential(torch.nn.Conv3d(3, 8, 3, padding=1), torch.nn.LeakyReLU(0.1)).eval()
    n = 3 * 16 * 16 * 16
    x = torch.arange(1, n + 1, dtype=torch.float32) / n
    x = (x - x.mean()) / x.std(unbiased=False)
    with torch.no_grad():
        yc = m(x.view(1, 3, 16, 16, 16))
    out.update(conv_W=m[0].weight.detach().numpy(), conv_b=m[0].bias.detach().numpy(), conv_x=x.numpy(),
               conv_checksum_torch=np.float64(yc.sum().item()), conv_checksum_readme=np.float64(9617.28),
               conv_y4=yc.flatten()[:4].numpy())
    np.savez_compressed(os.path.join(HERE, "stamps.npz"), **out)
    print("stamps: toy %.6f (README 7.775037)  conv %.2f (README 9617.28)" % (out["toy_checksum_torch"], out["conv_checksum_torch"]))


def main():
    zb = os.path.join(REF, "mom6_zb")
    for src, dst in (("gather.json", "zb_gather.json"), ("scatter.json", "zb_scatter.json"),
                     ("kdist.json", "zb_kdist.json"), ("zb_loop_verdict.json", "zb_loop.json")):
        shutil.copyfile(os.path.join(zb, src), os.path.join(HERE, dst))
    shutil.copyfile(os.path.join(zb, "zb_nn.npz"), os.path.join(HERE, "zb_nn.npz"))
    # the checked-in verdict is the analysis output; the driver multiplies `batch` by nk once the enclosing loop
    # is distributed (driver/fortisc.sh:44) and THAT file is what the emitter and the runtime consume
    lp = json.load(open(os.path.join(HERE, "zb_loop.json")))
    lp["batch"] *= json.load(open(os.path.join(HERE, "zb_kdist.json")))["nk"]
    lp.pop("statements", None)
    json.dump(lp, open(os.path.join(HERE, "zb_loop.json"), "w"), indent=1)
    record = {}
    G, S, Lp, K = (json.load(open(os.path.join(HERE, f))) for f in ("zb_gather.json", "zb_scatter.json", "zb_loop.json", "zb_kdist.json"))
    gin = zb_inputs()
    rng = np.random.default_rng(7)
    sin = [gin[3], np.asfortranarray((rng.random((68, 78)) + 0.5).astype(np.float32)),
           np.zeros((68, 78), np.float32, order="F"), np.zeros((68, 78, 15), np.float32, order="F"),
           np.zeros((68, 78, 15), np.float32, order="F")]
    run_case("zb", G, S, Lp, K, list(range(1, 16)), gin, sin, record)
    for name, (G, S, Lp, K, a0s) in extra_cases().items():
        run_case(name, G, S, Lp, K, a0s, case_inputs(G, 11), case_inputs(S, 12), record)
    # the ZB descriptors are stored once as files; drop the duplicate copy from the record
    for k in ("gather", "scatter", "loop", "kdist"):
        record["zb"].pop(k)
    json.dump(record, open(os.path.join(HERE, "gather_scatter_golden.json"), "w"), indent=1)
    stamps()


if __name__ == "__main__":
    main()
