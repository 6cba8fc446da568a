"""The real boundary: a compiled C program that declares the library's gather / scatter / step entries with fixed
argument lists (as the reference's generated code does per host, mom6_zb/gather.cu:50,82) and calls them the way
Flang-compiled bind(C) code does: integers by value first, then one address per array, no variadic prototype in
scope.  The library's entries are C variadics whose first named parameter is an integer OR a pointer depending on
the descriptor, so this is the call sequence that has to be proven with a compiler, not with ctypes.

Also: the variadic entries called through ctypes, and the configuration through FORTIS_*_JSON / FORTIS_MODEL
environment variables as a rewritten host is run.
"""
import ctypes
import hashlib
import json
import os
import subprocess

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import fortis_b200
from fortis_b200 import descriptors as D
from oracle import fortis_oracle as fo
from tests.golden.make_golden import case_inputs, zb_inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "fortis_b200")


def build_host(tmp_path, scenario):
    exe = str(tmp_path / ("host%d" % scenario))
    cmd = ["gcc", "-O1", "-Wall", "-Werror", "-DSCENARIO=%d" % scenario, os.path.join(ROOT, "tests", "c_host", "host.c"), "-o", exe,
           "-L" + LIBDIR, "-lfortis_b200", "-Wl,-rpath," + LIBDIR]
    subprocess.run(cmd, check=True)
    return exe


def write_case(tmp_path, gin, sin, files):
    for i, a in enumerate(gin):
        (tmp_path / ("g%d.bin" % i)).write_bytes(a.tobytes(order="F"))
    for i, a in enumerate(sin):
        (tmp_path / ("s%d.bin" % i)).write_bytes(a.tobytes(order="F"))
    env = dict(os.environ)
    for key, obj in files.items():
        p = tmp_path / (key + ".json")
        p.write_text(json.dumps(obj))
        env["FORTIS_%s_JSON" % key.upper()] = str(p)
    return env


def read_out(tmp_path, sin):
    return [np.frombuffer((tmp_path / ("s%d.out" % i)).read_bytes(), dtype=a.dtype).reshape(a.shape, order="F") for i, a in enumerate(sin)]


def test_compiled_c_host_three_call_step_kdist(tmp_path, golden_dir):
    """Scenario 1: the MOM6-ZB host.  X bit-exact against the golden digest of the reference's own generated kernel;
    scattered arrays bit-exact against the oracle's scatter of the library's own forward output is not available from
    a separate process, so the arrays are compared with the oracle's full step at the fp32 bar and the gather by
    digest."""
    G, S, Lp, K = (json.load(open(os.path.join(golden_dir, f))) for f in ("zb_gather.json", "zb_scatter.json", "zb_loop.json", "zb_kdist.json"))
    Wz = np.load(os.path.join(golden_dir, "zb_nn.npz"))
    layers = [dict(W=Wz["A0"], b=Wz["b0"], act="relu"), dict(W=Wz["A1"], b=Wz["b1"], act="none")]
    gin = zb_inputs()
    rng = np.random.default_rng(7)
    sin = [gin[3], np.asfortranarray((rng.random((68, 78)) + 0.5).astype(np.float32)), np.zeros((68, 78), np.float32, order="F"),
           np.zeros((68, 78, 15), np.float32, order="F"), np.zeros((68, 78, 15), np.float32, order="F")]
    env = write_case(tmp_path, gin, sin, dict(gather=G, scatter=S, loop=Lp, kdist=K))
    model = tmp_path / "model.bin"
    model.write_bytes(fortis_b200.write_blob(layers, in_div=Wz["in_norms"], out_mul=Wz["out_norms"]))
    env["FORTIS_MODEL"] = str(model)
    exe = build_host(tmp_path, 1)
    subprocess.run([exe, str(tmp_path), "15", str(71040 * 27 * 4)], check=True, env=env)
    X = np.frombuffer((tmp_path / "X.bin").read_bytes(), np.float32).reshape(71040, 27)
    golden = json.load(open(os.path.join(golden_dir, "gather_scatter_golden.json")))["zb"]
    assert hashlib.sha256(X.tobytes()).hexdigest() == golden["X_sha256"]
    ref = [a.copy(order="F") for a in sin]
    Y = fo.mlp_forward(layers, X, in_norms=Wz["in_norms"], out_norms=Wz["out_norms"])
    for k in range(1, 16):
        fo.scatter(S, Lp, K, Y, ref, args=(k,))
    got = read_out(tmp_path, sin)
    for a, b in zip(got[2:], ref[2:]):
        assert fo.rel_l2(a, b) < 1e-5
    for a, b in zip(got[:2], ref[:2]):          # arrays the scatter only reads come back untouched
        assert a.tobytes(order="F") == b.tobytes(order="F")


def test_compiled_c_host_integer_first_arguments(tmp_path, golden_dir):
    """Scenario 2: fortis_gather(k, u, m) and fortis_scatter(k, o): an int by value where scenario 1 passes a pointer."""
    g = json.load(open(os.path.join(golden_dir, "gather_scatter_golden.json")))["arg_plane"]
    G, S, Lp, K, a0s = g["gather"], g["scatter"], g["loop"], g["kdist"], g["a0s"]
    rng = np.random.default_rng(21)
    layers = [dict(W=rng.normal(size=(S["n"], G["n"])).astype(np.float32), b=rng.normal(size=S["n"]).astype(np.float32), act="none")]
    gin, sin = case_inputs(G, 11), case_inputs(S, 12)
    env = write_case(tmp_path, gin, sin, dict(gather=G, scatter=S, loop=Lp))
    model = tmp_path / "model.bin"
    model.write_bytes(fortis_b200.write_blob(layers))
    env["FORTIS_MODEL"] = str(model)
    rows = fo.loop_params(Lp, K)["count"]
    exe = build_host(tmp_path, 2)
    subprocess.run([exe, str(tmp_path), str(a0s[0]), str(rows * G["n"] * 4)], check=True, env=env)
    X = np.frombuffer((tmp_path / "X.bin").read_bytes(), np.float32).reshape(rows, G["n"])
    assert hashlib.sha256(X.tobytes()).hexdigest() == g["X_sha256"]
    assert X.tobytes() == fo.gather(G, Lp, K, gin, args=a0s[:1]).tobytes()
    ref = [a.copy(order="F") for a in sin]
    fo.scatter(S, Lp, K, fo.mlp_forward(layers, X), ref, args=(a0s[0],))
    got = read_out(tmp_path, sin)
    for a, b in zip(got, ref):
        assert fo.rel_l2(a, b) < 1e-5


def test_compiled_c_host_fused_step(tmp_path):
    """Scenario 3: fortis_step(g0, g1, g2, s0, s1, s2) with pointer-only arguments."""
    nx, ny, nz = 37, 21, 3
    G, S, Lp, K = D.stencil(nx, ny, nz)
    layers = fortis_b200.mlp_layers([27, 20, 20, 3], seed=4, init="uniform", act="relu", bias="uniform")
    rng = np.random.default_rng(3)
    gin = [np.asfortranarray(rng.standard_normal((nx + 2, ny + 2, nz)).astype(np.float32)) for _ in range(3)]
    sin = [np.full((nx + 2, ny + 2, nz), -7.0, np.float32, order="F") for _ in range(3)]
    env = write_case(tmp_path, gin, sin, dict(gather=G, scatter=S, loop=Lp, kdist=K))
    model = tmp_path / "model.bin"
    model.write_bytes(fortis_b200.write_blob(layers))
    env["FORTIS_MODEL"] = str(model)
    exe = build_host(tmp_path, 3)
    subprocess.run([exe, str(tmp_path)], check=True, env=env)
    ref = [a.copy(order="F") for a in sin]
    fo.full_step(G, S, Lp, K, layers, gin, ref)
    for a, b in zip(read_out(tmp_path, sin), ref):
        assert fo.rel_l2(a, b) < 1e-5
        assert (a[0, :, :] == -7.0).all() and (a[:, -1, :] == -7.0).all()     # halo untouched


def test_variadic_entries_through_ctypes(golden_dir):
    """fortis_gather / fortis_scatter / fortis_step called as variadics (ctypes passes the same registers a C caller
    does on x86-64 and AArch64)."""
    h = fortis_b200.Host()
    h.reset()
    L = h.L
    vp = ctypes.c_void_p
    g = json.load(open(os.path.join(golden_dir, "gather_scatter_golden.json")))["arg_plane"]
    G, S, Lp, K, a0s = g["gather"], g["scatter"], g["loop"], g["kdist"], g["a0s"]
    rng = np.random.default_rng(21)
    layers = [dict(W=rng.normal(size=(S["n"], G["n"])).astype(np.float32), b=rng.normal(size=S["n"]).astype(np.float32), act="none")]
    h.configure(gather=G, scatter=S, loop=Lp)
    h.load_model(fortis_b200.write_blob(layers))
    gin, sin = case_inputs(G, 11), case_inputs(S, 12)
    ref = [a.copy(order="F") for a in sin]
    k = a0s[0]
    L.fortis_gather.restype = None
    L.fortis_scatter.restype = None
    L.fortis_step.restype = None
    L.fortis_gather(ctypes.c_int(k), vp(gin[0].ctypes.data), vp(gin[1].ctypes.data))
    h.check()
    rows = fo.loop_params(Lp, K)["count"]
    X = h.model_input(rows, G["n"])
    assert X.tobytes() == fo.gather(G, Lp, K, gin, args=(k,)).tobytes()
    h.forward_batched()
    Y = h.model_output(rows, S["n"])
    L.fortis_scatter(ctypes.c_int(k), vp(sin[0].ctypes.data))
    h.check()
    fo.scatter(S, Lp, K, Y, ref, args=(k,))
    assert sin[0].tobytes(order="F") == ref[0].tobytes(order="F")
    # the fused step of the same descriptors: the plane index travels first
    sin2 = case_inputs(S, 12)
    L.fortis_step(ctypes.c_int(k), vp(gin[0].ctypes.data), vp(gin[1].ctypes.data), vp(sin2[0].ctypes.data))
    h.check()
    h.sync()
    assert fo.rel_l2(sin2[0], ref[0]) < 1e-5
    # ... and it is refused, with nothing written, when the plane index is missing
    sin3 = case_inputs(S, 12)
    keep = sin3[0].copy(order="F")
    h.L.fortis_stepv((vp * 2)(gin[0].ctypes.data, gin[1].ctypes.data), 2, (vp * 1)(sin3[0].ctypes.data), 1)
    assert L.fortis_last_error() != 0 and b"plane" in L.fortis_last_error_message()
    assert sin3[0].tobytes(order="F") == keep.tobytes(order="F")
    h.reset()
