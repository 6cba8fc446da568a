"""Parity at the FULL sizes of the benchmark configurations, through the C ABI, device-resident arrays.

The oracle cannot run a whole configuration in seconds, but columns / gridpoints / batch entries are independent, so
it is run on a fixed sample of them (spread over the first, middle and last tiles, so that every persistent CTA's
second and third tile and the last, ragged tile are covered) and compared with the same elements of the GPU result.
Bars are the stated tolerances themselves: fp32 <= 1e-5, 16-bit tensor-core variants <= 5e-3, FP8-E4M3 weights <= 2e-2
relative L2 against the fp32 oracle; the comparison with the oracle's model of the reduced-precision arithmetic is an
additional, tight check that isolates indexing mistakes from rounding.  Where exact arithmetic in the named format
cannot meet a bar the case is an expected failure with the measured value, never a widened bar.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import fortis_b200
from fortis_b200 import descriptors as D
from fortis_b200 import workloads as W
from oracle import fortis_oracle as fo

FP32_TOL, HALF_TOL, FP8W_TOL, MODEL_TOL = 1e-5, 5e-3, 2e-2, 2e-3


@pytest.fixture()
def host():
    h = fortis_b200.Host()
    h.reset()
    yield h
    assert h.L.fortis_device_status() == 0, "a bounded wait in a tensor-core kernel gave up"
    h.reset()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a.reshape(-1, order="F"))).cuda()


def back(t, like):
    return t.cpu().numpy().reshape(like.shape, order="F")


def cat(arrs):
    return np.concatenate([np.asarray(a).ravel() for a in arrs])


def sample_columns(ncol, n=4096, tile=128, seed=1):
    """First and last 8 tiles whole, the rest spread over the middle."""
    edge = 8 * tile
    rng = np.random.default_rng(seed)
    mid = rng.choice(np.arange(edge, ncol - edge), size=n - 2 * edge, replace=False)
    return np.unique(np.concatenate([np.arange(edge), mid, np.arange(ncol - edge, ncol)]))


def column_step(host, wl, precision):
    host.configure(gather=wl["G"], scatter=wl["S"], loop=wl["Lp"])
    host.load_model(fortis_b200.write_blob(wl["layers"]))
    host.option("precision", precision)
    host.option("checksum", 1)
    d_in, d_out = [dev(a) for a in wl["gin"]], [dev(a) for a in wl["sout"]]
    host.step(d_in, d_out)
    host.sync()
    got = [back(t, a) for t, a in zip(d_out, wl["sout"])]
    cs = host.step_checksum()
    total = float(sum(t.double().sum().item() for t in d_out))
    scale = float(sum(t.double().abs().sum().item() for t in d_out))
    assert abs(cs - total) <= 1e-9 * max(1.0, scale), "step checksum %r vs sum of the scattered arrays %r" % (cs, total)
    return got


def column_oracle(wl, idx, forward=None):
    """The oracle's step on the sampled columns only (a column problem of len(idx) columns with the same layout)."""
    G, S, Lp, K = D.column(len(idx), 60)
    gin = [np.asfortranarray(a[idx]) for a in wl["gin"]]
    out = W.column_outputs(len(idx))
    fo.full_step(G, S, Lp, K, wl["layers"], gin, out, forward=forward)
    return out


def compare_columns(got, wl, idx, precision):
    sub = [a[idx] for a in got]
    exact = column_oracle(wl, idx)
    e_exact = fo.rel_l2(cat(sub), cat(exact))
    e_model = None
    if precision != "fp32":
        model = column_oracle(wl, idx, forward=lambda L, X: fo.mlp_forward_lowp(L, X, precision))
        e_model = fo.rel_l2(cat(sub), cat(model))
    print("%s sample of %d columns: vs fp32 oracle %.3e, vs %s model %s, sample checksum %.9e"
          % (wl["label"], len(idx), e_exact, precision, "%.3e" % e_model if e_model is not None else "-", float(cat(sub).astype(np.float64).sum())))
    return e_exact, e_model


@pytest.mark.parametrize("precision,tol", [("fp32", FP32_TOL), ("bf16", HALF_TOL), ("fp16", HALF_TOL)])
def test_column_config_full_size(host, precision, tol):
    """49,152 columns x 60 levels: 384 tiles on 148 persistent CTAs."""
    wl = W.column(49152)
    got = column_step(host, wl, precision)
    idx = sample_columns(49152)
    e_exact, e_model = compare_columns(got, wl, idx, precision)
    assert e_exact <= tol
    assert e_model is None or e_model <= MODEL_TOL


def test_sharded_block_fp8_weights_full_size(host):
    """One rank's block of the sharded configuration: 2^20 columns, FP8-E4M3 weights.  The kernel must reproduce the
    oracle's model of E4M3 weights with per-output-channel absmax scales and add nothing on top of it."""
    wl = W.sharded_block(0)
    got = column_step(host, wl, "fp8w")
    idx = sample_columns(1 << 20)
    e_exact, e_model = compare_columns(got, wl, idx, "fp8w")
    assert e_model <= MODEL_TOL
    model_vs_exact = fo.rel_l2(cat(column_oracle(wl, idx[:512], forward=lambda L, X: fo.mlp_forward_lowp(L, X, "fp8w"))),
                               cat(column_oracle(wl, idx[:512])))
    assert e_exact <= 1.05 * model_vs_exact + 1e-4


@pytest.mark.xfail(strict=True, reason="stated bar unmet: exact E4M3 weights with per-output-channel absmax scales are "
                                       "6e-2 from fp32 on this network (3 mantissa bits = 3.6 % RMS weight error), bar 2e-2")
def test_fp8_weights_stated_bar(host):
    wl = W.column(4096)
    got = column_step(host, wl, "fp8w")
    e_exact, _ = compare_columns(got, wl, np.arange(4096), "fp8w")
    assert e_exact <= FP8W_TOL


def test_stencil_config_full_size(host):
    """1440 x 1080 x 4 gridpoints, fp32: windows at the corners, edges and centre of several planes against the oracle
    run on each window as its own small stencil problem; halo untouched; fp64 checksum."""
    wl = W.stencil()
    nx, ny, nz = wl["shape"]
    host.configure(gather=wl["G"], scatter=wl["S"], loop=wl["Lp"], kdist=wl["K"])
    host.load_model(fortis_b200.write_blob(wl["layers"]))
    host.option("checksum", 1)
    sentinel = -123.0
    outs = [np.full_like(a, sentinel) for a in wl["sout"]]
    d_in, d_out = [dev(a) for a in wl["gin"]], [dev(a) for a in outs]
    host.step(d_in, d_out)
    host.sync()
    got = [back(t, a) for t, a in zip(d_out, outs)]
    cs = host.step_checksum()
    wn = 32
    worst, npts = 0.0, 0
    for (i0, j0, k) in [(0, 0, 0), (nx - wn, ny - wn, nz - 1), (nx - wn, 0, 1), (0, ny - wn, 2), (nx // 2 - 7, ny // 2 + 3, 1),
                        (705, 3, 3), (1, ny - wn - 1, 0), (nx - wn - 1, 517, 2)]:
        G, S, Lp, K = D.stencil(wn, wn, 1)
        gin = [np.asfortranarray(a[i0:i0 + wn + 2, j0:j0 + wn + 2, k:k + 1]) for a in wl["gin"]]
        ref = [np.zeros((wn + 2, wn + 2, 1), np.float32, order="F") for _ in range(3)]
        fo.full_step(G, S, Lp, K, wl["layers"], gin, ref)
        for a, b in zip(got, ref):
            worst = max(worst, fo.rel_l2(a[i0 + 1:i0 + wn + 1, j0 + 1:j0 + wn + 1, k], b[1:-1, 1:-1, 0]))
        npts += wn * wn
    print("stencil full size: %d sampled points, worst window rel-L2 %.3e" % (npts, worst))
    assert worst <= FP32_TOL
    for a in got:
        assert (a[0] == sentinel).all() and (a[-1] == sentinel).all() and (a[:, 0] == sentinel).all() and (a[:, -1] == sentinel).all()
        assert (a[1:-1, 1:-1] != sentinel).all()
    total = float(sum(a[1:-1, 1:-1].astype(np.float64).sum() for a in got))
    scale = float(sum(np.abs(a[1:-1, 1:-1]).astype(np.float64).sum() for a in got))
    assert abs(cs - total) <= 1e-9 * scale


def test_stencil_config_full_size_host_arrays_plane_pipeline(host, monkeypatch):
    """The stencil step with HOST arrays: plane k+1 goes up while plane k is computed and the visited rectangle of plane
    k-1 comes back.  Bit-identical to the device-resident step call after call (eager, captured, replayed), halo of the
    host's arrays untouched, and identical to the serial staging path."""
    wl = W.stencil()
    host.configure(gather=wl["G"], scatter=wl["S"], loop=wl["Lp"], kdist=wl["K"])
    host.load_model(fortis_b200.write_blob(wl["layers"]))
    host.option("checksum", 1)
    sentinel = -123.0
    d_in, d_out = [dev(a) for a in wl["gin"]], [dev(np.full_like(a, sentinel)) for a in wl["sout"]]
    host.step(d_in, d_out)
    host.sync()
    want = [back(t, a) for t, a in zip(d_out, wl["sout"])]
    host.step_checksum()
    outs = [np.full_like(a, sentinel) for a in wl["sout"]]
    for call in range(4):
        host.step(wl["gin"], outs)
        host.sync()
        for a, b in zip(outs, want):
            assert a.tobytes(order="F") == b.tobytes(order="F"), "call %d" % call
        cs = host.step_checksum()
        total = float(sum(a[1:-1, 1:-1].astype(np.float64).sum() for a in outs))
        assert abs(cs - total) <= 1e-9 * float(sum(np.abs(a[1:-1, 1:-1]).astype(np.float64).sum() for a in outs))
        for a in outs:
            a.fill(sentinel)
    monkeypatch.setenv("FORTIS_NO_OVERLAP", "1")
    outs2 = [np.full_like(a, sentinel) for a in wl["sout"]]
    host.step(wl["gin"], outs2)
    host.sync()
    for a, b in zip(outs2, want):
        assert a.tobytes(order="F") == b.tobytes(order="F")


@pytest.mark.parametrize("precision,tol", [("fp32", FP32_TOL), ("fp16", HALF_TOL)])
def test_conv_config_full_size(host, precision, tol):
    """8 x 33^3 x 3, six residual blocks: whole batch entries 0 and 7 against the oracle."""
    wl = W.conv()
    x = wl["gin"][0]
    host.load_model(fortis_b200.write_blob(wl["layers"]))
    host.option("precision", precision)
    host.option("conv_shape", "%d,%d,%d,%d" % wl["shape"])
    y = np.zeros_like(wl["sout"][0])
    host.forward(x, y)
    for n in (0, 7):
        want = fo.convnet_forward(wl["layers"], x[n:n + 1])
        e = fo.rel_l2(y[n:n + 1], want)
        print("conv full size, precision %s, batch entry %d: rel-L2 vs fp32 oracle %.3e, checksum %.9e" % (precision, n, e, float(y[n].astype(np.float64).sum())))
        assert e <= tol


def conv_bf16_full(host):
    wl = W.conv()
    x = wl["gin"][0]
    host.load_model(fortis_b200.write_blob(wl["layers"]))
    host.option("precision", "bf16")
    host.option("conv_shape", "%d,%d,%d,%d" % wl["shape"])
    y = np.zeros_like(wl["sout"][0])
    host.forward(x, y)
    want = fo.convnet_forward(wl["layers"], x[:1])
    model = fo.convnet_forward_lowp(wl["layers"], x[:1])
    e, em = fo.rel_l2(y[:1], want), fo.rel_l2(model, want)
    print("conv full size bf16: vs fp32 %.3e; the oracle's bf16 model vs fp32 %.3e" % (e, em))
    return e, em


def test_conv_config_full_size_bf16_adds_nothing_to_bf16_arithmetic(host):
    e, em = conv_bf16_full(host)
    assert e <= 1.15 * em


@pytest.mark.xfail(strict=True, reason="stated bar unmet in bf16: a 14-layer residual stack with bf16 operands is 8e-3 "
                                       "from fp32 in exact arithmetic (the oracle's own bf16 model); precision=fp16 meets 5e-3")
def test_conv_config_full_size_bf16_bar(host):
    e, _ = conv_bf16_full(host)
    assert e <= HALF_TOL


@pytest.mark.parametrize("precision", ["bf16", "fp32"])
def test_column_config_full_size_host_arrays_chunked_staging(host, precision, monkeypatch):
    """The same step with HOST arrays: column chunks go up, compute and come back on three streams.  The result must be
    bit-identical to the device-resident step (the chunks are whole tiles of the same kernels), call after call, and
    identical to the serial staging path."""
    wl = W.column(49152)
    want = column_step(host, wl, precision)              # device-resident
    outs = [np.full_like(a, np.nan) for a in wl["sout"]]
    for _ in range(4):                                   # call 1 eager, call 2 captured, calls 3 and 4 replay the graph
        host.step(wl["gin"], outs)
        host.sync()
        for a, b in zip(outs, want):
            assert a.tobytes(order="F") == b.tobytes(order="F")
        for a in outs:
            a.fill(np.nan)
    host.step_checksum()
    host.step(wl["gin"], outs)
    cs = host.step_checksum()
    total = float(sum(a.astype(np.float64).sum() for a in outs))
    assert abs(cs - total) <= 1e-9 * float(sum(np.abs(a).astype(np.float64).sum() for a in outs))
    monkeypatch.setenv("FORTIS_NO_OVERLAP", "1")         # the serial path: whole arrays up, step, whole arrays back
    outs2 = [np.full_like(a, np.nan) for a in wl["sout"]]
    host.step(wl["gin"], outs2)
    host.sync()
    for a, b in zip(outs2, want):
        assert a.tobytes(order="F") == b.tobytes(order="F")


@pytest.mark.parametrize("mode", ["mapped_out", "mapped"])
def test_column_config_full_size_mapped_host_arrays(host, mode):
    """host_access = mapped_out / mapped: the kernels store into (and load from) the pinned host pages themselves
    instead of staging copies.  Same kernels, same tiles: bit-identical to the device-resident step."""
    wl = W.column(49152)
    want = column_step(host, wl, "bf16")
    host.reset()
    host.configure(gather=wl["G"], scatter=wl["S"], loop=wl["Lp"])
    host.load_model(fortis_b200.write_blob(wl["layers"]))
    host.option("precision", "bf16")
    host.option("host_access", mode)
    outs = [np.full_like(a, np.nan) for a in wl["sout"]]
    for _ in range(3):
        host.step(wl["gin"], outs)
        host.sync()
        for a, b in zip(outs, want):
            assert a.tobytes(order="F") == b.tobytes(order="F")
        for a in outs:
            a.fill(np.nan)
    with pytest.raises(fortis_b200.FortisError):
        host.option("host_access", "peer")
