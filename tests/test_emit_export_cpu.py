"""The driver-side pieces a maintainer of the reference would switch to: the emitter that turns one host's descriptor
files into a link-ready configuration object + bind(C) interface (the role of driver/fortis_gather_emit.py and
driver/fortis_emit2d.py when nothing has to be compiled per host), the torch exporter (the role of frontend/export_*.py +
driver/fortis_outline.py) and the descriptor generators."""
import ctypes
import json
import os
import re
import subprocess

import numpy as np
import pytest

import fortis_b200
from fortis_b200 import build as fb
from fortis_b200 import descriptors as D
from fortis_b200 import emit, export
from oracle import fortis_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "fortis_b200")


def zb_docs(golden_dir):
    return [open(os.path.join(golden_dir, n)).read() for n in ("zb_gather.json", "zb_scatter.json", "zb_loop.json", "zb_kdist.json")]


def test_emitted_configuration_links_and_configures_the_library(tmp_path, golden_dir):
    fb.build()
    g, s, l, k = zb_docs(golden_dir)
    c_path, f_path = emit.emit(str(tmp_path), g, s, l, k, options={"graph": "1"})
    main = tmp_path / "main.c"
    main.write_text('int fortis_last_error(void);\nint main(void) { return fortis_last_error() != 0; }\n')
    exe = str(tmp_path / "host")
    subprocess.run(["gcc", "-Wall", "-Werror", str(main), c_path, "-o", exe, "-L" + LIBDIR, "-lfortis_b200", "-Wl,-rpath," + LIBDIR], check=True)
    subprocess.run([exe], check=True)            # the constructor parsed every descriptor; nothing needed a GPU
    # a descriptor that does not parse is refused at emission time
    with pytest.raises(json.JSONDecodeError):
        emit.emit(str(tmp_path), "{not json", s, l, k)


def test_emitted_interface_has_the_hosts_argument_lists(tmp_path, golden_dir):
    g, s, l, k = zb_docs(golden_dir)
    _, f_path = emit.emit(str(tmp_path), g, s, l, k)
    text = open(f_path).read()
    # k-distributed: fortis_gather takes the four arrays only; fortis_scatter the plane index by value + five arrays
    assert re.search(r"subroutine fortis_gather\(g0, g1, g2, g3\) bind\(c", text)
    assert re.search(r"subroutine fortis_scatter\(k0, s0, s1, s2, s3, s4\) bind\(c", text)
    assert "integer(c_int), value :: k0" in text
    # without k distribution the plane index also goes in front of fortis_gather's arrays
    golden = json.load(open(os.path.join(golden_dir, "gather_scatter_golden.json")))["arg_plane"]
    _, f2 = emit.emit(str(tmp_path / "b"), json.dumps(golden["gather"]), json.dumps(golden["scatter"]), json.dumps(golden["loop"]))
    t2 = open(f2).read()
    assert re.search(r"subroutine fortis_gather\(k0, g0, g1\) bind\(c", t2)
    assert re.search(r"subroutine fortis_step\(k0, g0, g1, s0\) bind\(c", t2)
    # a boundary host gets mlp_forward in its own element kinds
    _, f3 = emit.emit(str(tmp_path / "c"), lift2d=json.dumps(D.boundary(16, 8, 4, "f64", "f32")))
    t3 = open(f3).read()
    assert "real(c_double) :: x(*)" in t3 and "real(c_float) :: y(*)" in t3


def test_descriptor_generators_agree_with_the_oracles_builders():
    assert json.dumps(D.column(100, 60)) == json.dumps(fo.column_descriptors(100, 60))
    assert json.dumps(D.stencil(10, 8, 3)) == json.dumps(fo.stencil_descriptors(10, 8, 3))
    assert json.dumps(D.identity(5, 4, 9)) == json.dumps(fo.identity_descriptors(5, 4, 9))


def test_torch_exporter_round_trips_through_the_blob():
    torch = pytest.importorskip("torch")
    nn = torch.nn
    torch.manual_seed(3)
    net = nn.Sequential(nn.Linear(6, 10), nn.LeakyReLU(0.15), nn.Sequential(nn.Linear(10, 8), nn.ReLU()), nn.Linear(8, 3))
    layers = export.layers_from_torch(net)
    assert [(L["act"], round(L["slope"], 3)) for L in layers] == [("leaky", 0.15), ("relu", 0.0), ("none", 0.0)]
    x = torch.randn(17, 6)
    want = net(x).detach().numpy()
    assert fo.rel_l2(fo.mlp_forward(layers, x.numpy()), want) < 1e-6
    blob = export.blob_from_torch(net)
    assert blob == fortis_b200.write_blob(layers)
    sd = {("%d.%s" % (i, k)): v for i, m in enumerate([net[0], net[2][0], net[3]]) for k, v in m.state_dict().items()}
    blob2 = export.blob_from_state_dict(sd, ["leaky", "leaky", "none"], slope=0.15)
    assert len(blob2) == len(blob)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.body = nn.Sequential(nn.Conv3d(4, 4, 3, padding=1), nn.LeakyReLU(0.2), nn.Conv3d(4, 4, 3, padding=1))

        def forward(self, x):
            return x + self.body(x)
    cnet = nn.Sequential(nn.Conv3d(2, 4, 3, padding=1), nn.LeakyReLU(0.2), Block(), Block(), nn.Conv3d(4, 1, 3, padding=1))
    cl = export.layers_from_torch(cnet)
    assert [bool(L.get("save")) for L in cl] == [True, False, True, False, True, False]
    assert [bool(L.get("add")) for L in cl] == [False, False, True, False, True, False]
    xc = torch.randn(1, 2, 5, 6, 7)
    want = cnet(xc).detach().numpy().transpose(0, 2, 3, 4, 1)          # NCDHW -> NDHWC
    got = fo.convnet_forward(cl, xc.numpy().transpose(0, 2, 3, 4, 1))
    assert fo.rel_l2(got, want) < 1e-5
    with pytest.raises(ValueError):
        export.layers_from_torch(nn.Sequential(nn.Linear(3, 3), nn.Tanh()))


def test_random_descriptor_cases_are_valid_for_planner_and_oracle():
    """Every generated case plans in the library and gathers in the oracle; the planner's element offsets agree."""
    fb.build()
    lib = fortis_b200.load()
    rng = np.random.default_rng(2024)
    for case in range(40):
        G, S, Lp, K, nargs, planes = D.random_case(rng)
        P = fo.loop_params(Lp, K)
        arrays = [np.asfortranarray(rng.uniform(-2, 2, size=a["shape"]).astype(fo._NP[a["elt"]])) for a in G["arrays"]]
        args = (int(rng.integers(1, planes + 1)),) if nargs else ()
        X = fo.gather(G, Lp, K, arrays, args=args)
        assert X.shape == (P["count"] * P["nk"], G["n"]) and np.isfinite(X).all(), case
        geom = (ctypes.c_longlong * 8)()
        offs, arrs, slots = (ctypes.c_longlong * 64)(), (ctypes.c_int * 64)(), (ctypes.c_int * 64)()
        a = (ctypes.c_int * 8)(*(list(args) + [1] * (8 - len(args))))
        n = lib.fortis_debug_plan(json.dumps(G).encode(), json.dumps(Lp).encode(), json.dumps(K).encode() if K else b"", 0, 0, a,
                                  len(args), offs, arrs, slots, 64, geom)
        assert n == G["n"], (case, lib.fortis_last_error_message())
        assert geom[0] == P["count"] and geom[1] == P["nk"]


def test_prepacked_blob_matches_the_loaders_own_packing_and_is_hash_checked():
    """write_blob(prepack=...) carries the weights already converted and tiled for one tensor-core precision.  The
    exporter's arithmetic (bf16 / fp16 rounding, E4M3 codes and per-channel scales, padding, 128-byte swizzle of the
    stage images) must equal the loader's bit for bit, and a section that does not belong to the weights in front of
    it, or that is damaged, must be refused."""
    import ctypes
    import fortis_b200
    from fortis_b200 import model as M
    L = fortis_b200.load()
    fp, ci = ctypes.POINTER(ctypes.c_float), ctypes.c_int
    L.fortis_debug_pack_layer.argtypes = [fp, fp, ci, ci, ci, ci, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.POINTER(ci), ctypes.POINTER(ci)]
    rng = np.random.default_rng(0)
    for prec in ("bf16", "fp16", "fp8w"):
        for cout, cin, last in ((768, 244, 0), (128, 768, 1), (20, 27, 0), (3, 20, 1)):
            W = rng.normal(0, 0.1, size=(cout, cin)).astype(np.float32)
            b = rng.normal(size=cout).astype(np.float32)
            W[0, :] = 0                                               # a dead channel: scale 1
            W[1, :5] = [1.0, 2.0, 0.5, 448.0, -448.0]
            W[2, :4] = [1.9999999, 2.0000002, 0.99999994, 1e-9]       # either side of a binade, and a flush to zero
            K, N, img, bias, scale = M.pack_layer(W, b, bool(last), prec)
            k, n = ci(), ci()
            im2, b2, s2 = np.zeros(K * N, np.uint16), np.zeros(N, np.float32), np.zeros(N, np.float32)
            rc = L.fortis_debug_pack_layer(W.ctypes.data_as(fp), b.ctypes.data_as(fp), cout, cin, last, M.PRECISIONS[prec],
                                           im2.ctypes.data, b2.ctypes.data, s2.ctypes.data, ctypes.byref(k), ctypes.byref(n))
            assert rc == 0 and (k.value, n.value) == (K, N)
            assert np.array_equal(im2, img) and np.array_equal(b2, bias) and np.array_equal(s2, scale), (prec, cout, cin)
    layers = M.mlp_layers([27, 20, 20, 3], seed=4, init="uniform", act="relu", bias="uniform")
    plain, packed = M.write_blob(layers), M.write_blob(layers, prepack="bf16")
    assert packed.startswith(plain) and packed[len(plain):len(plain) + 8] == b"FORTISP1"
    load = lambda blob: L.fortis_load_model_mem(ctypes.c_char_p(blob), len(blob))
    assert load(packed) == 0
    damaged = bytearray(packed); damaged[len(plain) + 40] ^= 1                      # inside the first stage image
    assert load(bytes(damaged)) == -1 and b"corrupt" in L.fortis_last_error_message()
    other = M.write_blob(M.mlp_layers([27, 20, 20, 3], seed=5, init="uniform", act="relu", bias="uniform"))
    assert load(other + packed[len(plain):]) == -1 and b"does not belong" in L.fortis_last_error_message()
    assert load(plain + b"junkjunk") == -1
    L.fortis_reset()


def test_2d_operator_networks_oracle_and_exporter_against_torch_vectors(golden_dir):
    """The operator types of the reference's micro-suite as 2-D networks (tests/golden/opnet_models.py): the oracle's
    unfused definitions must reproduce torch's outputs, and so must the EXPORTED form interpreted by the oracle: that
    checks the exporter's algebra (BatchNorm, padding and concatenation folded into weights, transposed convolutions
    as convolutions of the dilated input).  The blobs must load."""
    import ctypes
    import fortis_b200
    from fortis_b200 import export as E
    from fortis_b200 import model as M
    from oracle import fortis_oracle as fo
    from tests.golden import opnet_models as OM
    Z = np.load(os.path.join(golden_dir, "opnet_golden.npz"))
    L = fortis_b200.load()
    for name in OM.NAMES:
        m, spec, x = OM.build(name)
        want = Z[name + "_y"]
        assert fo.rel_l2(fo.ops2d_forward(spec, x), want) < 1e-6, name
        layers = E.layers2d_from_torch(m)
        got = fo.opnet_forward(layers, x, dtype=np.float64)
        assert got.shape == want.shape and fo.rel_l2(got, want) < 1e-6, name
        blob = M.write_blob(layers)
        assert L.fortis_load_model_mem(ctypes.c_char_p(blob), len(blob)) == 0, L.fortis_last_error_message()
    L.fortis_reset()
    # what has no kernel is refused by the exporter, not dropped
    import torch.nn as nn
    for bad in (nn.Sequential(nn.Conv2d(1, 2, 3, dilation=2)), nn.Sequential(nn.Conv2d(1, 2, 3), nn.MaxPool2d(2, padding=1)),
                nn.Sequential(nn.Conv2d(1, 2, 3), nn.Upsample(scale_factor=2, mode="bilinear")), nn.Sequential(nn.ZeroPad2d(1), nn.MaxPool2d(2)),
                nn.Sequential(nn.Conv2d(1, 2, 3), nn.Sigmoid())):
        with pytest.raises(ValueError):
            E.layers2d_from_torch(bad.eval(), in_channels=1)
