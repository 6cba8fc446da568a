"""Parity of the CUDA path with the oracle, through the C ABI, on a B200.

Bars: gather / scatter bit-exact; fp32 forward <= 1e-5 relative L2 (the tolerances the benchmark definition states).
"""
import ctypes
import json
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import fortis_b200
from oracle import fortis_oracle as fo
from tests.golden.make_golden import case_inputs, zb_inputs

FP32_TOL = 1e-5


@pytest.fixture()
def host():
    h = fortis_b200.Host()
    h.reset()
    yield h
    h.reset()


def zb_desc(golden_dir):
    return tuple(json.load(open(os.path.join(golden_dir, f))) for f in
                 ("zb_gather.json", "zb_scatter.json", "zb_loop.json", "zb_kdist.json"))


def zb_model(golden_dir):
    W = np.load(os.path.join(golden_dir, "zb_nn.npz"))
    layers = [dict(W=W["A0"], b=W["b0"], act="relu"), dict(W=W["A1"], b=W["b1"], act="none")]
    return layers, W


def zb_scatter_arrays(gin):
    rng = np.random.default_rng(7)
    return [gin[3], np.asfortranarray((rng.random((68, 78)) + 0.5).astype(np.float32)),
            np.zeros((68, 78), np.float32, order="F"), np.zeros((68, 78, 15), np.float32, order="F"),
            np.zeros((68, 78, 15), np.float32, order="F")]


def dev(a):
    """Device copy of a Fortran array with the same memory order (flat, column-major)."""
    return torch.from_numpy(np.ascontiguousarray(a.reshape(-1, order="F"))).cuda()


def back(t, like):
    return t.cpu().numpy().reshape(like.shape, order="F")


# ---------------------------------------------------------------------------------------------------------------
# gather / scatter: bit-exact
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("resident", [False, True])
def test_zb_gather_is_bit_exact(host, golden_dir, resident):
    G, S, Lp, K = zb_desc(golden_dir)
    layers, W = zb_model(golden_dir)
    host.configure(gather=G, scatter=S, loop=Lp, kdist=K)
    host.load_model(fortis_b200.write_blob(layers, in_div=W["in_norms"], out_mul=W["out_norms"]))
    gin = zb_inputs()
    arrays = [dev(a) for a in gin] if resident else gin
    host.gather(arrays)
    X = host.model_input(71040, 27)
    want = fo.gather(G, Lp, K, gin)
    assert X.tobytes() == want.tobytes()


@pytest.mark.parametrize("resident", [False, True])
def test_zb_three_call_step_matches_oracle(host, golden_dir, resident):
    """fortis_gather ; mlp_forward_batched ; do k: fortis_scatter(k)   (mom6_zb/host_fissioned.fir:732-740)"""
    G, S, Lp, K = zb_desc(golden_dir)
    layers, W = zb_model(golden_dir)
    host.configure(gather=G, scatter=S, loop=Lp, kdist=K)
    host.load_model(fortis_b200.write_blob(layers, in_div=W["in_norms"], out_mul=W["out_norms"]))
    gin = zb_inputs()
    sin = zb_scatter_arrays(gin)
    ref = [a.copy(order="F") for a in sin]
    Xo = fo.gather(G, Lp, K, gin)
    Yo = fo.mlp_forward(layers, Xo, in_norms=W["in_norms"], out_norms=W["out_norms"])
    g_arr = [dev(a) for a in gin] if resident else gin
    s_arr = [dev(a) for a in sin] if resident else sin
    host.gather(g_arr)
    host.forward_batched()
    Y = host.model_output(71040, 3)
    assert fo.rel_l2(Y, Yo) < FP32_TOL
    for k in range(1, 16):
        host.scatter(s_arr, args=(k,))
        fo.scatter(S, Lp, K, Y, ref, args=(k,))        # scatter of the SAME Y must be bit-exact
    got = [back(t, a) for t, a in zip(s_arr, sin)] if resident else sin
    for a, b in zip(got, ref):
        assert a.tobytes(order="F") == b.tobytes(order="F")


@pytest.mark.parametrize("name", ["f64_kdist", "arg_plane", "inner_only"])
@pytest.mark.parametrize("resident", [False, True])
def test_descriptor_cases_bit_exact(host, golden_dir, name, resident):
    g = json.load(open(os.path.join(golden_dir, "gather_scatter_golden.json")))[name]
    G, S, Lp, K, a0s = g["gather"], g["scatter"], g["loop"], g["kdist"], g["a0s"]
    P = fo.loop_params(Lp, K)
    nin, nout = G["n"], S["n"]
    rng = np.random.default_rng(21)
    layers = [dict(W=rng.normal(size=(nout, nin)).astype(np.float32), b=rng.normal(size=nout).astype(np.float32), act="none")]
    host.configure(gather=G, scatter=S, loop=Lp, kdist=K)
    host.load_model(fortis_b200.write_blob(layers))
    host.option("fuse", 0)
    gin, sin = case_inputs(G, 11), case_inputs(S, 12)
    ref = [a.copy(order="F") for a in sin]
    gargs = [] if P["kdist"] else a0s[:1]
    g_arr = [dev(a) for a in gin] if resident else gin
    s_arr = [dev(a) for a in sin] if resident else sin
    host.gather(g_arr, args=gargs)
    rows = P["count"] * P["nk"]
    X = host.model_input(rows, nin)
    assert X.tobytes() == fo.gather(G, Lp, K, gin, args=gargs).tobytes()
    host.forward_batched()
    Y = host.model_output(rows, nout)
    assert fo.rel_l2(Y, fo.mlp_forward(layers, X)) < FP32_TOL
    for a0 in (a0s or [1]):
        host.scatter(s_arr, args=(a0,))
        fo.scatter(S, Lp, K, Y, ref, args=(a0,))
    got = [back(t, a) for t, a in zip(s_arr, sin)] if resident else sin
    for a, b in zip(got, ref):
        assert a.tobytes(order="F") == b.tobytes(order="F")


_REF_PINNED = []   # the reference's gsetup pins its arrays for the life of the process and never unpins them


def test_reference_generated_kernels_agree(host, golden_dir):
    """Second checker: the reference's own generated ZB gather / scatter kernels (oracle/_ref), run on this GPU."""
    so = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libfortis_ref_zb.so")
    if not os.path.exists(so):
        pytest.skip("oracle/_ref was not built (needs the reference checkout at build time)")
    ref = ctypes.CDLL(so, mode=ctypes.RTLD_LOCAL | os.RTLD_DEEPBIND)   # its entry names equal ours: keep both private
    G, S, Lp, K = zb_desc(golden_dir)
    gin = zb_inputs()
    p = lambda a: ctypes.c_void_p(a.ctypes.data)
    ref.fortis_gather(p(gin[0]), p(gin[1]), p(gin[2]), p(gin[3]))
    Xr = np.empty((71040, 27), np.float32)
    assert ref.ref_download_input(p(Xr)) == 0
    Xo = fo.gather(G, Lp, K, gin)
    assert Xr.tobytes() == Xo.tobytes()
    Y = (np.random.default_rng(99).random((71040, 3)) - 0.5).astype(np.float32)
    assert ref.ref_upload_output(p(Y)) == 0
    sin = zb_scatter_arrays(gin)
    _REF_PINNED.extend(gin + sin)          # keep the pinned addresses from being reused by later allocations
    ora = [a.copy(order="F") for a in sin]
    for k in range(1, 16):
        ref.fortis_scatter(ctypes.c_int(k), *[p(a) for a in sin])
        fo.scatter(S, Lp, K, Y, ora, args=(k,))
    for a, b in zip(sin, ora):
        assert a.tobytes(order="F") == b.tobytes(order="F")


# ---------------------------------------------------------------------------------------------------------------
# forward paths
# ---------------------------------------------------------------------------------------------------------------
def toy_config(ncol=4096):
    G, S, Lp, K = fo.identity_descriptors(64, 64, ncol)
    rng = np.random.default_rng(0)
    A = np.asfortranarray((2 * rng.random((64, ncol)) - 1).astype(np.float32))
    layers = fortis_b200.mlp_layers([64, 256, 256, 64], seed=1, init="kaiming_uniform", act="relu")
    return G, S, Lp, K, A, layers


@pytest.mark.parametrize("resident", [False, True])
def test_toy_mlp_config(host, resident):
    """benchmark configuration 1: (64,4096) Fortran array -> 64-256-256-64 ReLU MLP -> (64,4096) array + checksum."""
    G, S, Lp, K, A, layers = toy_config()
    B = np.zeros((64, 4096), np.float32, order="F")
    Bo = B.copy(order="F")
    fo.full_step(G, S, Lp, K, layers, [A], [Bo])
    host.configure(gather=G, scatter=S, loop=Lp)
    host.load_model(fortis_b200.write_blob(layers))
    a, b = (dev(A), dev(B)) if resident else (A, B)
    host.step([a], [b])
    got = back(b, B) if resident else B
    assert fo.rel_l2(got, Bo) < FP32_TOL
    cs = host.checksum(b)
    assert abs(cs - fo.checksum([Bo])) <= 1e-5 * max(1.0, np.abs(Bo).sum())
    # the same through the three-call form
    B2 = np.zeros((64, 4096), np.float32, order="F")
    b2 = dev(B2) if resident else B2
    host.gather([a]); host.forward_batched(); host.scatter([b2])
    assert fo.rel_l2(back(b2, B2) if resident else B2, Bo) < FP32_TOL


def test_stamp_models_through_mlp_forward(host, golden_dir):
    """The reference's toy stamp (README.md:25: checksum 7.775037) through the whole-array mlp_forward entry."""
    Z = np.load(os.path.join(golden_dir, "stamps.npz"))
    layers = [dict(W=Z["toy_W0"], b=Z["toy_b0"], act="relu"), dict(W=Z["toy_W1"], b=Z["toy_b1"], act="none")]
    host.load_model(fortis_b200.write_blob(layers))
    x = np.ascontiguousarray(Z["toy_x"], dtype=np.float32)
    y = np.zeros(1024, np.float32)
    host.forward(x, y)
    assert abs(float(y.astype(np.float64).sum()) - 7.775037) / 7.775037 < 1e-5
    # resident / graph-replay variant (benchmarks/toy/bench_dev.f90): upload once, step, download
    host.option("graph", 1)
    host.L.mlp_upload(x.ctypes.data)
    for _ in range(4):
        host.L.mlp_forward_dev()
    y2 = np.zeros(1024, np.float32)
    host.L.mlp_download(y2.ctypes.data)
    host.check()
    assert y2.tobytes() == y.tobytes()


def test_zb_known_answer_vector(host, golden_dir):
    layers, W = zb_model(golden_dir)
    host.load_model(fortis_b200.write_blob(layers, in_div=W["in_norms"], out_mul=W["out_norms"]))
    x = np.ascontiguousarray(W["x_test"], dtype=np.float32)
    y = np.zeros(3, np.float32)
    host.forward(x, y)
    assert np.abs(y - W["y_test"]).max() / np.abs(W["y_test"]).max() < 1e-6


def test_packed_path_and_runtime_extent(host):
    """fortis_begin(count) ; fortis_pack per column ; mlp_forward_batched() ; fortis_unpack (driver/fortis_stub.c,
    driver/fortis_shim.py:103-115), including a ragged count that is no multiple of any tile."""
    layers = fortis_b200.mlp_layers([12, 40, 7], seed=3, act="leaky", slope=0.15)
    host.load_model(fortis_b200.write_blob(layers))
    rng = np.random.default_rng(1)
    for count in (1, 33, 200):
        host.L.fortis_begin(count)
        X = rng.normal(size=(count, 12)).astype(np.float32)
        for c in range(count):
            host.L.fortis_pack(X[c].ctypes.data, c)
        host.forward_batched()
        Y = np.zeros((count, 7), np.float32)
        for c in range(count):
            host.L.fortis_unpack(Y[c].ctypes.data, c)
        host.check()
        assert fo.rel_l2(Y, fo.mlp_forward(layers, X)) < FP32_TOL


def test_column_config_fp32_small(host):
    """benchmark configuration 2's layout at a reduced column count: four (ncol,60) fields + 4 vectors -> 244 features,
    244-768x4-128 LeakyReLU(0.15), outputs into two (ncol,60) arrays and eight vectors.  Ragged ncol."""
    ncol = 1000
    G, S, Lp, K = fo.column_descriptors(ncol, 60)
    rng = np.random.default_rng(2)
    gin = [np.asfortranarray((250 + 20 * rng.normal(size=(ncol, 60))).astype(np.float32)),
           np.asfortranarray(np.exp(-6 + rng.normal(size=(ncol, 60))).astype(np.float32)),
           np.asfortranarray((10 * rng.normal(size=(ncol, 60))).astype(np.float32)),
           np.asfortranarray((10 * rng.normal(size=(ncol, 60))).astype(np.float32))]
    gin += [rng.normal(size=ncol).astype(np.float32) for _ in range(4)]
    sout = [np.zeros((ncol, 60), np.float32, order="F") for _ in range(2)] + [np.zeros(ncol, np.float32) for _ in range(8)]
    ref = [a.copy(order="F") for a in sout]
    layers = fortis_b200.mlp_layers([244, 768, 768, 768, 768, 128], seed=0)
    fo.full_step(G, S, Lp, K, layers, gin, ref)
    host.configure(gather=G, scatter=S, loop=Lp)
    host.load_model(fortis_b200.write_blob(layers))
    host.step(gin, sout)
    assert fo.rel_l2(np.concatenate([a.ravel() for a in sout]), np.concatenate([a.ravel() for a in ref])) < FP32_TOL


@pytest.mark.parametrize("nx,ny,nz", [(64, 48, 2), (37, 5, 3)])
def test_stencil_config_fused(host, nx, ny, nz):
    """benchmark configuration 3's layout at reduced extent: 3 fields with a 1-cell halo, 27 -> 20 -> 20 -> 3, in place."""
    G, S, Lp, K = fo.stencil_descriptors(nx, ny, nz)
    rng = np.random.default_rng(3)
    gin = [np.asfortranarray(rng.normal(size=(nx + 2, ny + 2, nz)).astype(np.float32)) for _ in range(3)]
    sout = [np.full((nx + 2, ny + 2, nz), -999.0, np.float32, order="F") for _ in range(3)]
    ref = [a.copy(order="F") for a in sout]
    layers = fortis_b200.mlp_layers([27, 20, 20, 3], seed=4, init="uniform", act="relu", bias="uniform")
    fo.full_step(G, S, Lp, K, layers, gin, ref)
    host.configure(gather=G, scatter=S, loop=Lp, kdist=K)
    host.load_model(fortis_b200.write_blob(layers))
    host.option("checksum", 1)
    d_in, d_out = [dev(a) for a in gin], [dev(a) for a in sout]
    host.step(d_in, d_out)
    got = [back(t, a) for t, a in zip(d_out, sout)]
    for a, b in zip(got, ref):
        assert np.array_equal(a == -999.0, b == -999.0)          # halo cells untouched
        assert fo.rel_l2(a, b) < FP32_TOL
    want_cs = sum(float(b[b != -999.0].astype(np.float64).sum()) for b in ref)
    assert abs(host.step_checksum() - want_cs) < 1e-4 * (1 + abs(want_cs))
    # host-resident arrays through the same entry (staged planes in, visited rectangles out)
    host.step(gin, sout)
    for a, b in zip(sout, ref):
        assert np.array_equal(a == -999.0, b == -999.0)
        assert fo.rel_l2(a, b) < FP32_TOL
    # unfused path must give the same numbers as the fused one up to fp32 summation order
    host.option("fuse", 0)
    d_out2 = [dev(np.full((nx + 2, ny + 2, nz), -999.0, np.float32, order="F")) for _ in range(3)]
    host.step(d_in, d_out2)
    for t, b in zip(d_out2, ref):
        assert fo.rel_l2(back(t, b), b) < FP32_TOL


def test_lift2d_boundary_f64(host):
    """E3SM-style whole-array boundary (driver/fortis_boundary_trt.py:27-38): f64 (NI,NK) host array, pre =
    (a - mean[k]) / (max[k] - min[k]), model in fp32, post = y / scale[k] into an f64 (NI,NO) array."""
    NI, NK, NO = 384, 124, 128
    L2 = {"ok": True, "layout": {"in": {"from_shape": [NI, NK], "to_shape": [NK, NI], "from_elt": "f64", "to_elt": "f32"},
                                 "out": {"from_shape": [NO, NI], "to_shape": [NI, NO], "from_elt": "f32", "to_elt": "f64"}},
          "pre": {"expr": ["arith.divf", ["arith.subf", ["A"], ["V", "in_mean", NK]],
                           ["arith.subf", ["V", "in_max", NK], ["V", "in_min", NK]]],
                  "globals": ["in_mean", "in_max", "in_min"], "sizes": {"in_mean": NK, "in_max": NK, "in_min": NK}, "elt": "f64"},
          "post": {"expr": ["arith.divf", ["A"], ["V", "out_scale", NO]], "globals": ["out_scale"],
                   "sizes": {"out_scale": NO}, "elt": "f64"}}
    rng = np.random.default_rng(8)
    vecs = {"in_mean": rng.normal(size=NK), "in_min": rng.normal(size=NK) - 3.0, "in_max": rng.normal(size=NK) + 3.0,
            "out_scale": rng.random(NO) + 0.5}
    A = np.asfortranarray(rng.normal(size=(NI, NK)) * 2.0)
    B = np.zeros((NI, NO), np.float64, order="F")
    layers = fortis_b200.mlp_layers([NK, 256, 256, NO], seed=5)
    X = fo.boundary_pre(L2, A, vecs)
    Yo = fo.mlp_forward(layers, X)
    Bo = np.zeros((NI, NO), np.float64, order="F")
    fo.boundary_post(L2, Yo, Bo, vecs)
    host.configure(lift2d=L2)
    for k, v in vecs.items():
        host.set_vector(k, v)
    host.load_model(fortis_b200.write_blob(layers))
    host.forward(A, B)
    assert fo.rel_l2(B, Bo) < FP32_TOL
    # the boundary arithmetic itself is exact: feed the device's own Y back through the oracle's post
    Y = host.model_output(NI, NO)
    Bx = np.zeros((NI, NO), np.float64, order="F")
    fo.boundary_post(L2, Y, Bx, vecs)
    assert B.tobytes(order="F") == Bx.tobytes(order="F")


def test_gemm_entry_memref_abi(host):
    """fortis_gemm(A, W, C, B, N, K): C[B][N] = A[B][K] . W[N][K]^T  (runtime/fortis_rt.c:42-48)."""
    Bn, N, K = 77, 50, 33
    rng = np.random.default_rng(4)
    A = torch.from_numpy(rng.normal(size=(Bn, K)).astype(np.float32)).cuda()
    W = torch.from_numpy(rng.normal(size=(N, K)).astype(np.float32)).cuda()
    C = torch.zeros((Bn, N), dtype=torch.float32, device="cuda")
    L = host.L
    vp, cl = ctypes.c_void_p, ctypes.c_long
    L.fortis_gemm.argtypes = [vp, vp, cl, cl, cl, cl, cl] * 3 + [cl, cl, cl]
    L.fortis_gemm(A.data_ptr(), A.data_ptr(), 0, Bn, K, K, 1, W.data_ptr(), W.data_ptr(), 0, N, K, K, 1,
                  C.data_ptr(), C.data_ptr(), 0, Bn, N, N, 1, Bn, N, K)
    host.sync()
    want = A.cpu().numpy().astype(np.float64) @ W.cpu().numpy().astype(np.float64).T
    assert fo.rel_l2(C.cpu().numpy(), want) < FP32_TOL


def test_pool_reuses_released_buffers(host):
    L = host.L
    big = (37 << 20) + 4096                # larger than anything the other tests left in the pool
    a = L.fortis_alloc(big)
    L.fortis_free(a)
    b = L.fortis_alloc(big - 12345)        # best fit among released buffers: the same one comes back
    assert a == b
    c = L.fortis_alloc(big)                # b is in use, so this is a fresh allocation
    assert c != b
    L.fortis_free(b); L.fortis_free(c)


def test_errors_are_messages_not_crashes(host):
    G, S, Lp, K = fo.identity_descriptors(4, 2, 8)
    host.configure(gather=G, scatter=S, loop=Lp)
    host.load_model(fortis_b200.write_blob(fortis_b200.mlp_layers([4, 2], seed=0)))
    A = np.zeros((4, 8), np.float32, order="F")
    with pytest.raises(fortis_b200.FortisError):
        host.gather([A, A])                         # wrong number of arrays
    # an activation the 16-bit tensor-core kernel cannot express (its branch-free form needs a slope in [0, 1]): refused
    # with a message, not run some other way
    host.load_model(fortis_b200.write_blob(fortis_b200.mlp_layers([4, 16, 2], seed=0, act="leaky", slope=1.5)))
    host.option("precision", "bf16")
    with pytest.raises(fortis_b200.FortisError):
        host.step([A], [np.zeros((2, 8), np.float32, order="F")])


# ---------------------------------------------------------------------------------------------------------------
# the fused step outside its simplest form
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("resident", [False, True])
def test_fused_step_with_plane_chosen_by_argument(host, golden_dir, resident):
    """Descriptors whose arrays carry a "v" subscript while the loop is NOT k-distributed: the fused step takes the
    enclosing-loop index like fortis_gather / fortis_scatter do, and touches that plane only."""
    g = json.load(open(os.path.join(golden_dir, "gather_scatter_golden.json")))["arg_plane"]
    G, S, Lp, K, a0s = g["gather"], g["scatter"], g["loop"], g["kdist"], g["a0s"]
    rng = np.random.default_rng(21)
    layers = [dict(W=rng.normal(size=(S["n"], G["n"])).astype(np.float32), b=rng.normal(size=S["n"]).astype(np.float32), act="none")]
    host.configure(gather=G, scatter=S, loop=Lp)
    host.load_model(fortis_b200.write_blob(layers))
    gin, sin = case_inputs(G, 11), case_inputs(S, 12)
    for k in (1, a0s[0], 4):
        ref = [a.copy(order="F") for a in sin]
        X = fo.gather(G, Lp, K, gin, args=(k,))
        fo.scatter(S, Lp, K, fo.mlp_forward(layers, X), ref, args=(k,))
        work = [a.copy(order="F") for a in sin]
        g_arr = [dev(a) for a in gin] if resident else gin
        s_arr = [dev(a) for a in work] if resident else work
        host.step(g_arr, s_arr, args=(k,))
        host.sync()
        got = [back(t, a) for t, a in zip(s_arr, work)] if resident else work
        for a, b, orig in zip(got, ref, sin):
            assert fo.rel_l2(a, b) < FP32_TOL
            assert np.array_equal(a != orig, b != orig)        # exactly the cells of plane k's rectangle changed
    # without the index the call is refused and nothing is written
    work = [a.copy(order="F") for a in sin]
    with pytest.raises(fortis_b200.FortisError, match="plane"):
        host.step(gin, work)
    assert all(a.tobytes(order="F") == b.tobytes(order="F") for a, b in zip(work, sin))


def test_descriptor_and_model_that_do_not_fit_are_refused(host):
    G, S, Lp, K = fo.identity_descriptors(6, 3, 16)
    host.configure(gather=G, scatter=S, loop=Lp)
    A, B = np.zeros((6, 16), np.float32, order="F"), np.zeros((3, 16), np.float32, order="F")
    host.load_model(fortis_b200.write_blob(fortis_b200.mlp_layers([5, 8, 3], seed=0)))      # 5 inputs, the gather makes 6
    with pytest.raises(fortis_b200.FortisError, match="inputs per row"):
        host.step([A], [B])
    host.load_model(fortis_b200.write_blob(fortis_b200.mlp_layers([6, 8, 4], seed=0)))      # 4 outputs, the scatter takes 3
    with pytest.raises(fortis_b200.FortisError, match="outputs per row"):
        host.step([A], [B])
    # a 27-20-3 shaped model with a descriptor of another width must not reach the stencil kernel either
    host.load_model(fortis_b200.write_blob(fortis_b200.mlp_layers([27, 20, 3], seed=0)))
    with pytest.raises(fortis_b200.FortisError):
        host.step([A], [B])


def test_in_place_stencil_on_one_device_array_matches_the_staged_semantics(host):
    """The host passes the SAME device array as gather input and as scatter target (an in-place update with a halo
    stencil).  The reference is well-defined here (gather and scatter work on separate staging copies: every input is
    read before any output is written); the fused kernels would read neighbours that other threads are overwriting,
    so such a call has to run unfused."""
    nx, ny, nz = 70, 33, 2
    G, S, Lp, K = fo.stencil_descriptors(nx, ny, nz, nfields=3, nout=3)
    rng = np.random.default_rng(31)
    fields = [np.asfortranarray(rng.normal(size=(nx + 2, ny + 2, nz)).astype(np.float32)) for _ in range(3)]
    layers = fortis_b200.mlp_layers([27, 20, 20, 3], seed=4, init="uniform", act="relu", bias="uniform")
    ref = [a.copy(order="F") for a in fields]
    fo.full_step(G, S, Lp, K, layers, fields, ref)            # gathers from `fields`, scatters into copies
    host.configure(gather=G, scatter=S, loop=Lp, kdist=K)
    host.load_model(fortis_b200.write_blob(layers))
    d = [dev(a) for a in fields]
    host.step(d, d)
    host.sync()
    for t, a, b in zip(d, fields, ref):
        assert fo.rel_l2(back(t, a), b) < FP32_TOL


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_step_checksum_on_the_unfused_paths(host, precision):
    """Option checksum = 1 must give the sum of what was scattered whichever kernels ran the step."""
    ncol = 333
    G, S, Lp, K = fo.column_descriptors(ncol, 7, nfields=2, nscal=2, nout_fields=1, nout_scal=3)
    rng = np.random.default_rng(5)
    gin = [np.asfortranarray(rng.normal(size=(ncol, 7)).astype(np.float32)) for _ in range(2)] + [rng.normal(size=ncol).astype(np.float32) for _ in range(2)]
    sout = [np.zeros((ncol, 7), np.float32, order="F")] + [np.zeros(ncol, np.float32) for _ in range(3)]
    host.configure(gather=G, scatter=S, loop=Lp)
    host.load_model(fortis_b200.write_blob(fortis_b200.mlp_layers([16, 64, 10], seed=2)))
    host.option("precision", precision)
    host.option("checksum", 1)
    host.option("fuse", 0)
    d_in, d_out = [dev(a) for a in gin], [dev(a) for a in sout]
    host.step(d_in, d_out)
    host.sync()
    total = float(sum(t.double().sum().item() for t in d_out))
    assert abs(host.step_checksum() - total) <= 1e-9 * max(1.0, float(sum(t.double().abs().sum().item() for t in d_out)))


def test_gemm_entry_refuses_strided_operands(host):
    Bn, N, K = 16, 8, 12
    A = torch.randn(Bn, 2 * K, device="cuda")[:, :K]            # row stride 2K: not dense
    W = torch.randn(N, K, device="cuda")
    C = torch.full((Bn, N), -3.0, device="cuda")
    L = host.L
    vp, cl = ctypes.c_void_p, ctypes.c_long
    L.fortis_gemm.argtypes = [vp, vp, cl, cl, cl, cl, cl] * 3 + [cl, cl, cl]
    L.fortis_gemm(A.data_ptr(), A.data_ptr(), 0, Bn, K, 2 * K, 1, W.data_ptr(), W.data_ptr(), 0, N, K, K, 1,
                  C.data_ptr(), C.data_ptr(), 0, Bn, N, N, 1, Bn, N, K)
    host.sync()
    assert float(C.min()) == -3.0 and float(C.max()) == -3.0


# ---------------------------------------------------------------------------------------------------------------
# fp32 on the tensor cores (three TF32 MMAs per product): batches of 512 rows and more
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("Bn,N,K", [(4096, 300, 200), (777, 64, 33), (513, 768, 768)])
def test_gemm_entry_large_batch(host, Bn, N, K):
    """fortis_gemm at batch sizes the split-TF32 kernel takes, shapes that are multiples of no tile; against fp64."""
    rng = np.random.default_rng(14)
    A = torch.from_numpy(rng.normal(size=(Bn, K)).astype(np.float32)).cuda()
    W = torch.from_numpy(rng.normal(size=(N, K)).astype(np.float32)).cuda()
    C = torch.full((Bn, N), float("nan"), dtype=torch.float32, device="cuda")
    L = host.L
    vp, cl = ctypes.c_void_p, ctypes.c_long
    L.fortis_gemm.argtypes = [vp, vp, cl, cl, cl, cl, cl] * 3 + [cl, cl, cl]
    for _ in range(2):                      # the second call takes the cached split of W
        L.fortis_gemm(A.data_ptr(), A.data_ptr(), 0, Bn, K, K, 1, W.data_ptr(), W.data_ptr(), 0, N, K, K, 1,
                      C.data_ptr(), C.data_ptr(), 0, Bn, N, N, 1, Bn, N, K)
        host.sync()
        want = A.cpu().numpy().astype(np.float64) @ W.cpu().numpy().astype(np.float64).T
        got = C.cpu().numpy()
        assert np.isfinite(got).all()
        assert fo.rel_l2(got, want) < 2e-6
    assert L.fortis_device_status() == 0


def test_array_form_fp32_large_batch_with_norms_and_mask(host):
    """mlp_forward_batched(in, out) on 3,000 rows in fp32: row-major input and output around the tensor-core layers,
    with the input divide, the output multiply and the masked final ReLU."""
    rows, dims = 3000, [30, 100, 50, 7]
    layers = fortis_b200.mlp_layers(dims, seed=21, act="leaky", slope=0.15, bias="uniform", scale=0.2)
    rng = np.random.default_rng(22)
    in_div, out_mul = (rng.random(30) + 0.5).astype(np.float32), (rng.random(7) + 0.5).astype(np.float32)
    mask = np.array([0, 1, 0, 0, 1, 1, 0], np.float32)
    X = rng.normal(size=(rows, 30)).astype(np.float32)
    host.load_model(fortis_b200.write_blob(layers, in_div=in_div, out_mul=out_mul, relu_mask=mask))
    host.L.fortis_begin(rows)
    Y = np.zeros((rows, 7), np.float32)
    host.forward_batched(X, Y)
    want = fo.mlp_forward(layers, X, in_norms=in_div, out_norms=out_mul)
    want[:, mask != 0] = np.maximum(want[:, mask != 0], 0)
    assert fo.rel_l2(Y, want) < FP32_TOL
    assert host.L.fortis_device_status() == 0


def test_reference_runtime_gemm_agrees(host):
    """Second checker for fortis_gemm: the reference's own runtime (runtime/fortis_rt.c compiled unchanged under
    oracle/_ref: cuBLAS SGEMM on pre-transposed weights) on the same operands."""
    so = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libfortis_ref_rt.so")
    if not os.path.exists(so):
        pytest.skip("oracle/_ref/libfortis_ref_rt.so was not built (needs the reference checkout at build time)")
    ref = ctypes.CDLL(so, mode=ctypes.RTLD_LOCAL | os.RTLD_DEEPBIND)
    vp, cl = ctypes.c_void_p, ctypes.c_long
    for fn in (ref.fortis_gemm, host.L.fortis_gemm):
        fn.argtypes = [vp, vp, cl, cl, cl, cl, cl] * 3 + [cl, cl, cl]
        fn.restype = None
    rng = np.random.default_rng(33)
    for (Bn, N, K) in [(64, 40, 24), (2048, 768, 244)]:
        A = torch.from_numpy(rng.normal(size=(Bn, K)).astype(np.float32)).cuda()
        W = torch.from_numpy(rng.normal(size=(N, K)).astype(np.float32)).cuda()
        C0, C1 = torch.zeros((Bn, N), device="cuda"), torch.zeros((Bn, N), device="cuda")
        for fn, C in ((ref.fortis_gemm, C0), (host.L.fortis_gemm, C1)):
            fn(A.data_ptr(), A.data_ptr(), 0, Bn, K, K, 1, W.data_ptr(), W.data_ptr(), 0, N, K, K, 1, C.data_ptr(), C.data_ptr(), 0, Bn, N, N, 1, Bn, N, K)
        torch.cuda.synchronize()
        host.sync()
        assert fo.rel_l2(C1.cpu().numpy(), C0.cpu().numpy()) < 2e-6


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_empty_and_single_row_batches(host, precision):
    """A run-time extent of zero (a rank that owns no columns, an empty loop) is a step that does nothing and reports
    nothing; the next non-empty extent works, down to one row."""
    layers = fortis_b200.mlp_layers([12, 40, 7], seed=3, act="leaky", slope=0.15)
    host.load_model(fortis_b200.write_blob(layers))
    host.option("precision", precision)
    host.L.fortis_begin(0)
    host.forward_batched()
    host.check()
    assert host.L.fortis_device_status() == 0
    rng = np.random.default_rng(5)
    for count in (1, 0, 3):
        host.L.fortis_begin(count)
        X = rng.normal(size=(max(count, 1), 12)).astype(np.float32)
        for c in range(count):
            host.L.fortis_pack(X[c].ctypes.data, c)
        host.forward_batched()
        Y = np.zeros((max(count, 1), 7), np.float32)
        for c in range(count):
            host.L.fortis_unpack(Y[c].ctypes.data, c)
        host.check()
        if count:
            assert fo.rel_l2(Y[:count], fo.mlp_forward(layers, X[:count])) < (FP32_TOL if precision == "fp32" else 5e-3)


@pytest.mark.parametrize("tc", [0, 1])
def test_stencil_step_with_input_and_output_scales(host, tc):
    """The stencil step of a model that divides its inputs and multiplies its outputs by per-feature scales (what the
    ocean nets do: mom6_zb/export_zb.py:13-14), on the packed-FMA kernel and on the tensor-core option."""
    nx, ny, nz = 45, 23, 2
    G, S, Lp, K = fo.stencil_descriptors(nx, ny, nz)
    rng = np.random.default_rng(12)
    gin = [np.asfortranarray(rng.normal(size=(nx + 2, ny + 2, nz)).astype(np.float32)) for _ in range(3)]
    layers = fortis_b200.mlp_layers([27, 20, 20, 3], seed=6, init="uniform", act="relu", bias="uniform")
    in_div = (rng.random(27) + 0.5).astype(np.float32)
    out_mul = (rng.random(3) + 0.5).astype(np.float32)
    ref = [np.zeros((nx + 2, ny + 2, nz), np.float32, order="F") for _ in range(3)]
    fo.full_step(G, S, Lp, K, layers, gin, ref, in_norms=in_div, out_norms=out_mul)
    host.configure(gather=G, scatter=S, loop=Lp, kdist=K)
    host.load_model(fortis_b200.write_blob(layers, in_div=in_div, out_mul=out_mul))
    host.option("stencil_tc", tc)
    out = [np.zeros((nx + 2, ny + 2, nz), np.float32, order="F") for _ in range(3)]
    host.step(gin, out)
    host.sync()
    assert host.L.fortis_device_status() == 0
    cat = lambda L: np.concatenate([a.ravel() for a in L])
    assert fo.rel_l2(cat(out), cat(ref)) <= FP32_TOL


@pytest.mark.parametrize("dims", [[27, 20, 20, 3], [27, 32, 4], [27, 9, 17, 1]])
def test_stencil_step_on_tensor_cores_option(host, dims):
    """Option stencil_tc: the 3x3-stencil step with its layers as TF32x3 tensor-core products (rows in tensor memory,
    thread = gridpoint end to end).  Same bar as the packed-FMA kernel (<= 1e-5 against the oracle), ragged extents,
    hidden widths that differ, checksum folded in the launch."""
    nx, ny, nz = 70, 37, 3
    G, S, Lp, K = fo.stencil_descriptors(nx, ny, nz, nout=dims[-1])
    rng = np.random.default_rng(11)
    gin = [np.asfortranarray(rng.normal(size=(nx + 2, ny + 2, nz)).astype(np.float32)) for _ in range(3)]
    layers = fortis_b200.mlp_layers(dims, seed=4, init="uniform", act="relu", bias="uniform")
    ref = [np.zeros((nx + 2, ny + 2, nz), np.float32, order="F") for _ in range(dims[-1])]
    fo.full_step(G, S, Lp, K, layers, gin, ref)
    host.configure(gather=G, scatter=S, loop=Lp, kdist=K)
    host.load_model(fortis_b200.write_blob(layers))
    host.option("stencil_tc", 1)
    host.option("checksum", 1)
    d_in = [torch.from_numpy(np.ascontiguousarray(a.reshape(-1, order="F"))).cuda() for a in gin]
    d_out = [torch.zeros(a.size, dtype=torch.float32, device="cuda") for a in ref]
    host.step_checksum()
    host.step(d_in, d_out)
    host.sync()
    assert host.L.fortis_device_status() == 0
    got = np.concatenate([t.cpu().numpy() for t in d_out])
    want = np.concatenate([a.reshape(-1, order="F") for a in ref])
    assert fo.rel_l2(got, want) <= FP32_TOL
    assert abs(host.step_checksum() - float(got.astype(np.float64).sum())) <= 1e-9 * float(np.abs(got).astype(np.float64).sum())
