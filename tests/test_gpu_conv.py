"""conv3d path (benchmark configuration 4's layer types) against the oracle, through the C ABI."""
import ctypes
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import fortis_b200
from oracle import fortis_oracle as fo

FP32_TOL = 1e-5


@pytest.fixture()
def host():
    h = fortis_b200.Host()
    h.reset()
    yield h
    h.reset()


@pytest.mark.parametrize("shape", [(2, 9, 7, 5), (1, 33, 33, 33)])
def test_superres_net_small(host, shape):
    """Conv3d 3->W k3 p1 + LeakyReLU(0.2); residual blocks [conv, LeakyReLU, conv, +skip]; Conv3d W->3 (NDHWC)."""
    N, D, H, W = shape
    width, blocks = (16, 2) if shape[1] < 20 else (64, 1)
    layers = fortis_b200.conv_layers(3, width, 3, nblocks=blocks, seed=6)
    for L in layers:                       # non-zero biases so that the bias path is exercised
        L["b"] = (np.random.default_rng(1).normal(size=L["b"].shape) * 0.05).astype(np.float32)
    x = np.random.default_rng(5).normal(size=(N, D, H, W, 3)).astype(np.float32)
    want = fo.convnet_forward(layers, x)
    host.load_model(fortis_b200.write_blob(layers))
    host.option("conv_shape", "%d,%d,%d,%d" % shape)
    y = np.zeros((N, D, H, W, 3), np.float32)
    host.forward(x, y)
    assert fo.rel_l2(y, want) < FP32_TOL


@pytest.mark.parametrize("shape,blocks", [((2, 9, 7, 5), 2), ((1, 33, 33, 33), 1), ((2, 16, 12, 20), 6)])
def test_superres_net_bf16_tensor_cores(host, shape, blocks):
    """The same network on the tcgen05 implicit-GEMM kernel (64 -> 64 layers) with bf16 activations.  Checked against
    the oracle's model of that arithmetic (tight) and against the fp32 oracle (the stated bf16 bar, 5e-3, or what
    bf16 storage of 2 * blocks + 1 activations costs by itself if that is more)."""
    N, D, H, W = shape
    layers = fortis_b200.conv_layers(3, 64, 3, nblocks=blocks, seed=6)
    for L in layers:
        L["b"] = (np.random.default_rng(1).normal(size=L["b"].shape) * 0.05).astype(np.float32)
    x = np.random.default_rng(5).normal(size=(N, D, H, W, 3)).astype(np.float32)
    model = fo.convnet_forward_lowp(layers, x)
    exact = fo.convnet_forward(layers, x)
    host.load_model(fortis_b200.write_blob(layers))
    host.option("precision", "bf16")
    host.option("conv_shape", "%d,%d,%d,%d" % shape)
    y = np.zeros((N, D, H, W, 3), np.float32)
    host.forward(x, y)
    y2 = np.zeros_like(y)
    host.forward(x, y2)                                      # second call reuses the padded buffers
    assert y2.tobytes() == y.tobytes()
    e_model, e_exact, m_exact = fo.rel_l2(y, model), fo.rel_l2(y, exact), fo.rel_l2(model, exact)
    print("conv bf16 %s, %d blocks: vs bf16 model %.3e, vs fp32 %.3e (the model itself: %.3e)" % (shape, blocks, e_model, e_exact, m_exact))
    if blocks <= 2:
        # shallow stacks: the stated bf16 bar itself, and a tight check against the model of the arithmetic
        assert e_model < 2e-3 and e_exact < 5e-3
    else:
        # A deep residual stack amplifies rounding decorrelation (merely accumulating the MODEL in fp32 instead of
        # fp64 moves its 6-block output by 5e-3), so the kernel is held to bf16 arithmetic's own distance from fp32:
        # it may add nothing on top.  The 5e-3 bar itself is asserted (and expected to fail in bf16) at full size in
        # test_gpu_fullsize.py; the layer-by-layer and boundary-row checks below are the tight ones.
        assert e_exact < 1.15 * m_exact
    assert host.L.fortis_device_status() == 0


def test_conv_net_bf16_other_edge_widths(host):
    """First / last layers with other channel counts (5 in, 7 out) and an extent whose row count is not a multiple of
    the tile: the padded channels of the packed input and of the last layer's weights must stay out of the result."""
    N, D, H, W = 1, 6, 9, 11
    layers = fortis_b200.conv_layers(5, 64, 7, nblocks=1, seed=11)
    for L in layers:
        L["b"] = (np.random.default_rng(2).normal(size=L["b"].shape) * 0.05).astype(np.float32)
    x = np.random.default_rng(12).normal(size=(N, D, H, W, 5)).astype(np.float32)
    model = fo.convnet_forward_lowp(layers, x)
    host.load_model(fortis_b200.write_blob(layers))
    host.option("precision", "bf16")
    host.option("conv_shape", "%d,%d,%d,%d" % (N, D, H, W))
    y = np.full((N, D, H, W, 7), np.nan, np.float32)
    host.forward(x, y)
    assert np.isfinite(y).all()
    assert fo.rel_l2(y, model) < 2e-3
    assert host.L.fortis_device_status() == 0


def test_conv_probe_stamp_through_memref_entry(host, golden_dir):
    """The reference's conv probe (frontend/export_conv.py; README stamp 9617.28) through fortis_conv3d's memref ABI:
    NCDHW fp32, the bias and LeakyReLU(0.1) applied afterwards as the compiled program does in its epilogue kernel."""
    Z = np.load(os.path.join(golden_dir, "stamps.npz"))
    x = torch.from_numpy(Z["conv_x"].reshape(1, 3, 16, 16, 16).copy()).cuda()
    w = torch.from_numpy(Z["conv_W"].copy()).cuda()
    y = torch.zeros((1, 8, 16, 16, 16), dtype=torch.float32, device="cuda")
    L = host.L
    vp, cl = ctypes.c_void_p, ctypes.c_long
    for fn in (L.fortis_conv3d, L.fortis_conv3d_direct):
        fn.argtypes = [vp, vp, cl] + [cl] * 10 + [vp, vp, cl] + [cl] * 10 + [vp, vp, cl] + [cl] * 10 + [cl] * 18
        fn.restype = None
        y.zero_()
        fn(x.data_ptr(), x.data_ptr(), 0, 1, 3, 16, 16, 16, 3 * 4096, 4096, 256, 16, 1,
           w.data_ptr(), w.data_ptr(), 0, 8, 3, 3, 3, 3, 81, 27, 9, 3, 1,
           y.data_ptr(), y.data_ptr(), 0, 1, 8, 16, 16, 16, 8 * 4096, 4096, 256, 16, 1,
           1, 3, 16, 16, 16, 8, 3, 3, 3, 16, 16, 16, 1, 1, 1, 1, 1, 1)
        host.sync()
        out = y.cpu().numpy() + Z["conv_b"].reshape(1, 8, 1, 1, 1)
        out = np.where(out > 0, out, out * np.float32(0.1))
        cs = float(out.astype(np.float64).sum())
        assert abs(cs - 9617.28) / 9617.28 < 3e-5
        assert np.allclose(out.ravel()[:4], Z["conv_y4"], rtol=1e-5, atol=1e-6)
    # stride 2 is refused with a message and leaves y untouched (runtime/fortis_fft.cu:135)
    y.fill_(-7.0)
    L.fortis_conv3d_direct(x.data_ptr(), x.data_ptr(), 0, 1, 3, 16, 16, 16, 3 * 4096, 4096, 256, 16, 1,
                           w.data_ptr(), w.data_ptr(), 0, 8, 3, 3, 3, 3, 81, 27, 9, 3, 1,
                           y.data_ptr(), y.data_ptr(), 0, 1, 8, 16, 16, 16, 8 * 4096, 4096, 256, 16, 1,
                           1, 3, 16, 16, 16, 8, 3, 3, 3, 16, 16, 16, 2, 2, 2, 1, 1, 1)
    host.sync()
    assert float(y.min()) == -7.0 and float(y.max()) == -7.0


@pytest.mark.parametrize("W", [6, 7, 8, 9, 10, 11, 12, 13])
def test_conv_bf16_every_row_pitch_residue(host, W):
    """The three kh taps of a kd read ONE staged activation tile through shared-memory descriptors whose start moves
    by (W+2) rows of 128 bytes, i.e. to every residue of the 8-row (1024-byte) swizzle period as W varies.  One
    64 -> 64 layer stack per residue, checked against the oracle's bf16 model per layer (no amplification)."""
    N, D, H = 1, 4, 5
    layers = fortis_b200.conv_layers(3, 64, 3, nblocks=1, seed=20 + W)
    for L in layers:
        L["b"] = (np.random.default_rng(3).normal(size=L["b"].shape) * 0.05).astype(np.float32)
    x = np.random.default_rng(W).normal(size=(N, D, H, W, 3)).astype(np.float32)
    host.load_model(fortis_b200.write_blob(layers))
    host.option("precision", "bf16")
    host.option("conv_shape", "%d,%d,%d,%d" % (N, D, H, W))
    y = np.zeros((N, D, H, W, 3), np.float32)
    host.forward(x, y)
    assert fo.rel_l2(y, fo.convnet_forward_lowp(layers, x)) < 2e-3, "W + 2 = %d (residue %d)" % (W + 2, (W + 2) % 8)
    assert host.L.fortis_device_status() == 0


def test_conv_bf16_layer_by_layer_at_tile_and_quadrant_boundaries(host):
    """Per-layer check without amplification: each tensor-core layer is fed the oracle's own bf16 activations (a
    one-layer-deep network per layer type) and compared at 1e-3, with the rows at tile and lane-quadrant boundaries
    (padded rows 1, 31/32, 63/64, 95/96, 126/127 of every tile of 126 written rows) compared explicitly."""
    N, D, H, W = 1, 10, 9, 12
    rng = np.random.default_rng(41)
    full = fortis_b200.conv_layers(3, 64, 3, nblocks=1, seed=9)
    for L in full:
        L["b"] = (rng.normal(size=L["b"].shape) * 0.05).astype(np.float32)
    x = rng.normal(size=(N, D, H, W, 3)).astype(np.float32)
    host.load_model(fortis_b200.write_blob(full))
    host.option("precision", "bf16")
    host.option("conv_shape", "%d,%d,%d,%d" % (N, D, H, W))
    y = np.zeros((N, D, H, W, 3), np.float32)
    host.forward(x, y)
    want = fo.convnet_forward_lowp(full, x)
    assert fo.rel_l2(y, want) < 1e-3
    # rows of the padded volume -> interior voxels; tile t writes padded rows 126 t .. 126 t + 125
    Dp, Hp, Wp = D + 2, H + 2, W + 2
    p = np.arange(N * Dp * Hp * Wp)
    wp, hp, dp = p % Wp, (p // Wp) % Hp, (p // (Wp * Hp)) % Dp
    interior = (wp >= 1) & (wp <= W) & (hp >= 1) & (hp <= H) & (dp >= 1) & (dp <= D)
    r = p % 126
    edge = interior & np.isin(r, [0, 1, 30, 31, 32, 62, 63, 64, 94, 95, 96, 124, 125])
    assert edge.sum() > 50
    ye = y[0, dp[edge] - 1, hp[edge] - 1, wp[edge] - 1]
    we = want[0, dp[edge] - 1, hp[edge] - 1, wp[edge] - 1]
    assert fo.rel_l2(ye, we) < 1e-3


def _memref(t):
    """(allocated, aligned, offset, sizes..., strides...) of a dense torch tensor."""
    return [t.data_ptr(), t.data_ptr(), 0] + list(t.shape) + list(t.stride())


def _conv_entry(L, name, nd):
    vp, cl = ctypes.c_void_p, ctypes.c_long
    fn = getattr(L, name)
    one = [vp, vp, cl] + [cl] * (2 * nd)
    fn.argtypes = one * 3 + [cl] * (18 if nd == 5 else 13)
    fn.restype = None
    return fn


def test_single_conv_layers_any_kernel_stride_padding(host, golden_dir):
    """fortis_conv3d (any kernel extent / stride / padding), fortis_conv2d (the NCHW form) and fortis_conv3d_fft (the
    entry the compiler picks for 5^3 taps and more: stride 1, no padding) against torch-made vectors and the oracle,
    fp32 <= 1e-5."""
    Z = np.load(os.path.join(golden_dir, "conv_general.npz"))
    L = host.L
    c3, c2, cf = _conv_entry(L, "fortis_conv3d", 5), _conv_entry(L, "fortis_conv2d", 4), _conv_entry(L, "fortis_conv3d_fft", 5)
    for name in sorted(k[:-2] for k in Z.files if k.endswith("_y")):
        x, w, want = Z[name + "_x"], Z[name + "_w"], Z[name + "_y"]
        sd, sh, sw, pd, ph, pw = [int(v) for v in Z[name + "_sp"]]
        N, C, D, H, W = x.shape
        F, _, KD, KH, KW = w.shape
        _, _, Do, Ho, Wo = want.shape
        oracle = fo.conv_ncdhw(x, w, (sd, sh, sw), (pd, ph, pw))
        dx, dw = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
        entries = [("fortis_conv3d", c3)]
        if name.startswith("c3d_valid"):
            entries.append(("fortis_conv3d_fft", cf))
        for label, fn in entries:
            y = torch.full((N, F, Do, Ho, Wo), float("nan"), device="cuda")
            fn(*_memref(dx), *_memref(dw), *_memref(y), N, C, D, H, W, F, KD, KH, KW, Do, Ho, Wo, sd, sh, sw, pd, ph, pw)
            host.sync()
            got = y.cpu().numpy()
            assert fo.rel_l2(got, want) <= 1e-5, (label, name, fo.rel_l2(got, want))
            assert fo.rel_l2(got, oracle) <= 1e-5, (label, name)
        if D == 1 and KD == 1:
            x4, w4 = dx.view(N, C, H, W), dw.view(F, C, KH, KW)
            y4 = torch.full((N, F, Ho, Wo), float("nan"), device="cuda")
            c2(*_memref(x4), *_memref(w4), *_memref(y4), N, C, H, W, F, KH, KW, Ho, Wo, sh, sw, ph, pw)
            host.sync()
            assert fo.rel_l2(y4.cpu().numpy().reshape(want.shape), want) <= 1e-5, ("fortis_conv2d", name)
    # refusals leave y untouched: padding through the transform entry, a strided (non-dense) input view
    x = torch.randn(1, 2, 8, 8, 8, device="cuda")
    w = torch.randn(3, 2, 5, 5, 5, device="cuda")
    y = torch.full((1, 3, 8, 8, 8), -7.0, device="cuda")
    cf(*_memref(x), *_memref(w), *_memref(y), 1, 2, 8, 8, 8, 3, 5, 5, 5, 8, 8, 8, 1, 1, 1, 2, 2, 2)
    xs = torch.randn(1, 2, 8, 8, 16, device="cuda")[..., ::2]
    y2 = torch.full((1, 3, 4, 4, 4), -7.0, device="cuda")
    c3(*_memref(xs), *_memref(w), *_memref(y2), 1, 2, 8, 8, 8, 3, 5, 5, 5, 4, 4, 4, 1, 1, 1, 0, 0, 0)
    host.sync()
    assert float(y.min()) == -7.0 == float(y.max()) and float(y2.min()) == -7.0 == float(y2.max())


def test_2d_operator_networks_through_the_whole_array_entry(host, golden_dir):
    """Conv2d chains, pooling, nearest upsampling, transposed convolutions (stride 1 and 2), BatchNorm (inference),
    concatenated parallel convolutions and explicit padding, exported from torch modules and run through mlp_forward on
    NCHW arrays: <= 1e-5 against torch-made vectors and against the oracle's interpretation of the exported layers."""
    from fortis_b200 import export as E
    from tests.golden import opnet_models as OM
    Z = np.load(os.path.join(golden_dir, "opnet_golden.npz"))
    for name in OM.NAMES:
        m, _, x = OM.build(name)
        want = Z[name + "_y"]
        layers = E.layers2d_from_torch(m)
        host.reset()
        host.load_model(fortis_b200.write_blob(layers))
        N, C, H, W = x.shape
        host.option("conv_shape", "%d,1,%d,%d" % (N, H, W))
        y = np.full(want.shape, np.nan, np.float32)
        host.forward(np.ascontiguousarray(x), y)
        assert fo.rel_l2(y, want) <= 1e-5, (name, fo.rel_l2(y, want))
        assert fo.rel_l2(y, fo.opnet_forward(layers, x)) <= 1e-5, name
        # device-resident in and out, twice (the second call reuses every buffer)
        dx, dy = torch.from_numpy(x).cuda(), torch.full(want.shape, float("nan"), device="cuda")
        for _ in range(2):
            host.forward(dx, dy)
            host.sync()
            assert np.array_equal(dy.cpu().numpy(), y), name
    host.reset()
    host.load_model(fortis_b200.write_blob(E.layers2d_from_torch(OM.build("pool")[0])))
    host.option("conv_shape", "2,1,12,10")
    with pytest.raises(fortis_b200.FortisError):
        host.option("precision", "bf16")
        host.forward(np.zeros((2, 2, 12, 10), np.float32), np.zeros((2, 5, 6, 5), np.float32))


@pytest.mark.parametrize("seed", range(int(os.environ.get("FORTIS_CONV_SWEEP", "6"))))
def test_conv_net_random_extents_against_the_low_precision_model(host, seed):
    """Random batch and spatial extents (every residue of the padded row pitch, volumes smaller than one tile pair and
    larger than a round of tiles), channel counts of the edge layers, depth and 16-bit format: the tensor-core network
    against the oracle's model of its arithmetic; a second call must reproduce the first bit for bit."""
    rng = np.random.default_rng(5100 + seed)
    shape = (int(rng.integers(1, 4)), int(rng.integers(1, 11)), int(rng.integers(1, 13)), int(rng.integers(1, 41)))
    cin, cout, blocks = int(rng.integers(1, 17)), int(rng.integers(1, 17)), int(rng.integers(1, 3))
    mode = str(rng.choice(["bf16", "fp16"]))
    layers = fortis_b200.conv_layers(cin, 64, cout, nblocks=blocks, seed=int(rng.integers(1 << 30)))
    for L in layers:
        L["b"] = (rng.normal(size=L["b"].shape) * 0.05).astype(np.float32)
    x = rng.normal(size=shape + (cin,)).astype(np.float32)
    model = fo.convnet_forward_lowp(layers, x, mode=mode)
    host.load_model(fortis_b200.write_blob(layers))
    host.option("precision", mode)
    host.option("conv_shape", "%d,%d,%d,%d" % shape)
    y, y2 = np.zeros(shape + (cout,), np.float32), np.zeros(shape + (cout,), np.float32)
    host.forward(x, y)
    host.forward(x, y2)
    tag = "seed %d shape %s cin %d cout %d blocks %d %s" % (seed, shape, cin, cout, blocks, mode)
    assert y2.tobytes() == y.tobytes(), tag
    # close to the model of the arithmetic, or (a single small output channel can decorrelate further) no further from
    # the fp32 result than that model is
    e_model = fo.rel_l2(y, model)
    if e_model >= 2e-3:
        exact = fo.convnet_forward(layers, x)
        assert fo.rel_l2(y, exact) < 1.15 * fo.rel_l2(model, exact), tag + " %.3e" % e_model
    assert host.L.fortis_device_status() == 0, tag
