"""The oracle against every known answer the reference holds for this path (CPU only).

Pins: the ZB network's x_test -> y_test vector (mom6_zb/zb_nn.npz, checked by mom6_zb/make_zb_weights.py:18-20),
the README checksum stamps 7.775037 (toy MLP) and 9617.28 (conv probe) (README.md:24-26), and gather / scatter
outputs of the reference's own generated kernels compiled for the CPU (tests/golden/make_golden.py).
"""
import hashlib
import json
import os

import numpy as np
import pytest

from oracle import fortis_oracle as fo
from tests.golden.make_golden import case_inputs, zb_inputs  # input generators only; needs no reference checkout


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def zb_layers(W):
    return [dict(W=W["A0"], b=W["b0"], act="relu"), dict(W=W["A1"], b=W["b1"], act="none")]


def test_zb_known_answer(golden_dir):
    W = np.load(os.path.join(golden_dir, "zb_nn.npz"))
    y = fo.mlp_forward(zb_layers(W), W["x_test"][None, :], in_norms=W["in_norms"], out_norms=W["out_norms"])[0]
    assert np.abs(y - W["y_test"]).max() / np.abs(W["y_test"]).max() < 1e-6
    yn = fo.mlp_forward_native(zb_layers(W), W["x_test"][None, :], in_norms=W["in_norms"], out_norms=W["out_norms"])[0]
    assert np.abs(yn - W["y_test"]).max() / np.abs(W["y_test"]).max() < 1e-6


def test_toy_checksum_stamp(golden_dir):
    Z = np.load(os.path.join(golden_dir, "stamps.npz"))
    layers = [dict(W=Z["toy_W0"], b=Z["toy_b0"], act="relu"), dict(W=Z["toy_W1"], b=Z["toy_b1"], act="none")]
    y = fo.mlp_forward(layers, Z["toy_x"][None, :])
    cs = float(y.astype(np.float64).sum())
    assert abs(cs - float(Z["toy_checksum_readme"])) / 7.775037 < 1e-5      # the reference's stamps are to ~1e-5
    assert abs(cs - float(Z["toy_checksum_torch"])) / 7.775037 < 2e-6


def test_conv_probe_stamp(golden_dir):
    Z = np.load(os.path.join(golden_dir, "stamps.npz"))
    x = Z["conv_x"].reshape(1, 3, 16, 16, 16).transpose(0, 2, 3, 4, 1)        # NCDHW -> NDHWC
    y = fo.conv3d_ndhwc(x, Z["conv_W"], Z["conv_b"], pad=1)
    y = fo.act_apply(y, "leaky", 0.1)
    cs = float(y.astype(np.float64).sum())
    assert abs(cs - float(Z["conv_checksum_readme"])) / 9617.28 < 3e-5
    assert abs(cs - float(Z["conv_checksum_torch"])) / 9617.28 < 1e-5
    ncdhw = y.transpose(0, 4, 1, 2, 3).ravel()
    assert np.allclose(ncdhw[:4], Z["conv_y4"], rtol=1e-5, atol=1e-6)


@pytest.fixture(scope="module")
def golden(golden_dir):
    return json.load(open(os.path.join(golden_dir, "gather_scatter_golden.json")))


def _zb_desc(golden_dir):
    return tuple(json.load(open(os.path.join(golden_dir, f))) for f in
                 ("zb_gather.json", "zb_scatter.json", "zb_loop.json", "zb_kdist.json"))


def test_zb_gather_scatter_matches_reference_kernels(golden, golden_dir):
    G, S, Lp, K = _zb_desc(golden_dir)
    gin = zb_inputs()
    X = fo.gather(G, Lp, K, gin)
    assert X.shape == (71040, 27)
    assert _sha(X) == golden["zb"]["X_sha256"]
    rng = np.random.default_rng(7)
    sin = [gin[3], np.asfortranarray((rng.random((68, 78)) + 0.5).astype(np.float32)),
           np.zeros((68, 78), np.float32, order="F"), np.zeros((68, 78, 15), np.float32, order="F"),
           np.zeros((68, 78, 15), np.float32, order="F")]
    Y = (np.random.default_rng(99).random((71040, 3)) - 0.5).astype(np.float32)
    for a0 in golden["zb"]["a0s"]:
        fo.scatter(S, Lp, K, Y, sin, args=[a0])
    assert [_sha(a.reshape(-1, order="F")) for a in sin] == golden["zb"]["out_sha256"]


@pytest.mark.parametrize("name", ["f64_kdist", "arg_plane", "inner_only"])
def test_descriptor_cases_match_reference_kernels(golden, name):
    g = golden[name]
    G, S, Lp, K, a0s = g["gather"], g["scatter"], g["loop"], g["kdist"], g["a0s"]
    P = fo.loop_params(Lp, K)
    gin, sin = case_inputs(G, 11), case_inputs(S, 12)
    X = fo.gather(G, Lp, K, gin, args=a0s[:1] if not P["kdist"] else [])
    assert _sha(X) == g["X_sha256"]
    Y = (np.random.default_rng(99).random((P["count"] * P["nk"], S["n"])) - 0.5).astype(np.float32)
    for a0 in (a0s or [1]):
        fo.scatter(S, Lp, K, Y, sin, args=[a0])
    assert [_sha(a.reshape(-1, order="F")) for a in sin] == g["out_sha256"]


def test_expression_grammar():
    e = fo.parse_expr("(((tv * S0) * S0) * S1)")
    v = fo.eval_expr(e, np.float32(2.0), {0: np.float32(3.0), 1: np.float32(0.5)})
    assert v == np.float32(9.0)
    e = fo.parse_expr("fminf(expf((-tv)), (tv / (S0 + 1.000000e-30f)))")
    assert e[0] == "min" and e[1][0] == "exp" and e[1][1][0] == "neg"
    with pytest.raises(ValueError):
        fo.parse_expr("(tv + q7)")


def test_lowp_models():
    x = np.array([1.0, 1.00390625, 3.140625, -2.5e-3, 447.9, 1e-9], dtype=np.float32)
    b = fo.round_bf16(x)
    assert b[0] == 1.0 and b[1] in (np.float32(1.0), np.float32(1.0078125))
    q = fo.e4m3_round(np.array([0.0, 1.0, 1.0625, 448.0, 500.0, -0.001953125, 0.0009765625], np.float32))
    assert list(q) == [0.0, 1.0, 1.0, 448.0, 448.0, -0.001953125, 0.0]
    W = np.random.default_rng(0).normal(size=(8, 16)).astype(np.float32)
    Wq, sc = fo.quant_e4m3(W)
    assert fo.rel_l2(Wq * sc[:, None], W) < 0.05


def test_c_port_matches_numpy_native(golden_dir):
    """The C port (the timed CPU baseline) against the numpy restatement of the same loop order: bit-exact."""
    import ctypes
    from oracle import build as ob
    lib = ctypes.CDLL(ob.build_port(verbose=False))
    W = np.load(os.path.join(golden_dir, "zb_nn.npz"))
    rng = np.random.default_rng(5)
    X = (rng.normal(size=(257, 27)) * W["in_norms"]).astype(np.float32)
    ref = fo.mlp_forward_native(zb_layers(W), X, in_norms=W["in_norms"], out_norms=W["out_norms"])
    from oracle.cport import mlp_forward_c
    got = mlp_forward_c(lib, zb_layers(W), X, in_norms=W["in_norms"], out_norms=W["out_norms"], nthreads=2)
    assert got.tobytes() == ref.tobytes()


def test_oracle_single_conv_layers_match_torch_vectors(golden_dir):
    """conv_ncdhw (the oracle of fortis_conv2d / fortis_conv3d / fortis_conv3d_fft) against outputs torch's CPU
    convolution wrote for 2-D, strided, non-cubic and 5^3 / 7^3 'valid' layers (tests/golden/make_conv_golden.py)."""
    Z = np.load(os.path.join(golden_dir, "conv_general.npz"))
    names = sorted(k[:-2] for k in Z.files if k.endswith("_y"))
    assert len(names) == 7
    for name in names:
        sp = [int(v) for v in Z[name + "_sp"]]
        y = fo.conv_ncdhw(Z[name + "_x"], Z[name + "_w"], stride=sp[:3], pad=sp[3:], dtype=np.float64)
        assert y.shape == Z[name + "_y"].shape, name
        assert fo.rel_l2(y, Z[name + "_y"]) < 2e-7, name
