"""The give-up path of the bounded barrier waits in the tensor-core kernels, exercised without hanging anything: a
test option makes the first CTA's TMA warp leave out one stage (a barrier that nothing completes) and shortens the poll
limit; the kernel must return, the host must be able to read which wait gave up, and the next ordinary step must be
bit-identical to the one before."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import fortis_b200
from fortis_b200 import workloads as W


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a.reshape(-1, order="F"))).cuda()


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("precision", ["bf16", "fp8w"])
def test_mlp_kernel_wait_gives_up_and_the_context_stays_usable(precision, pair):
    """Both forms of the kernel: one CTA per SM, and two-CTA clusters (where the leader's wait runs out first and the
    partner's waits follow)."""
    h = fortis_b200.Host()
    h.reset()
    h.option("tc_pair", pair)
    wl = W.column(3000)                                  # 24 tiles: several CTAs keep working while CTA 0 gives up
    h.configure(gather=wl["G"], scatter=wl["S"], loop=wl["Lp"])
    h.load_model(fortis_b200.write_blob(wl["layers"]))
    h.option("precision", precision)
    d_in, d_out = [dev(a) for a in wl["gin"]], [dev(a) for a in wl["sout"]]
    h.step(d_in, d_out)
    h.sync()
    assert h.L.fortis_device_status() == 0
    before = [t.clone() for t in d_out]
    h.option("test_wait_limit", 4096)
    h.option("test_skip_stage", 1)
    h.step(d_in, d_out)                                  # CTA 0 never gets its first weight stage
    h.sync()
    status = h.L.fortis_device_status()
    assert status in (1, 2, 3), "expected a wait on the weight ring (full: 1, empty: 2) or, in the partner CTA, for an accumulator (3) to give up, got %d" % status
    assert h.L.fortis_device_status() == 0               # reading the failure cleared it
    h.option("test_skip_stage", 0)
    h.option("test_wait_limit", 0)
    for t in d_out:
        t.zero_()
    h.step(d_in, d_out)
    h.sync()
    assert h.L.fortis_device_status() == 0
    for a, b in zip(d_out, before):
        assert torch.equal(a, b)
    h.reset()


def test_conv_pair_kernel_wait_gives_up_in_both_ctas_of_the_pair():
    h = fortis_b200.Host()
    h.reset()
    shape = (1, 6, 9, 11)
    layers = fortis_b200.conv_layers(3, 64, 3, nblocks=1, seed=11)
    x = np.random.default_rng(12).normal(size=shape + (3,)).astype(np.float32)
    h.load_model(fortis_b200.write_blob(layers))
    h.option("precision", "bf16")
    h.option("conv_shape", "%d,%d,%d,%d" % shape)
    y0 = np.zeros(shape + (3,), np.float32)
    h.forward(x, y0)
    assert h.L.fortis_device_status() == 0
    h.option("test_wait_limit", 4096)
    h.option("test_skip_stage", 1)
    y1 = np.zeros_like(y0)
    h.forward(x, y1)                                     # the leader of the first pair never completes its first stage
    status = h.L.fortis_device_status()
    assert status in (11, 12, 13, 14), "expected a conv kernel wait code, got %d" % status
    h.option("test_skip_stage", 0)
    h.option("test_wait_limit", 0)
    y2 = np.zeros_like(y0)
    h.forward(x, y2)
    assert h.L.fortis_device_status() == 0
    assert y2.tobytes() == y0.tobytes()
    h.reset()
