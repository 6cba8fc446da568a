"""Small 2-D operator networks covering the op types of the reference's operator micro-suite (tests/optest.py:
convolution chains, pooling, nearest upsampling, transposed convolutions with and without stride, BatchNorm in
inference mode, channel concatenation of parallel convolutions, explicit zero padding), with shapes of their own.
`build(name)` returns (torch module in eval mode, unfused op list for oracle.ops2d_forward, input array): used by the
fixture generator and by the tests, so that both talk about the same weights.
"""
import numpy as np
import torch
import torch.nn as nn

NAMES = ["pool", "upsample", "convT_s2", "bn", "convT_s1", "two_convs", "concat", "cat_only", "pad"]


def _np(t):
    return t.detach().numpy().astype(np.float64)


def _conv(m):
    return ("conv", _np(m.weight), _np(m.bias), m.stride, m.padding)


def _convT(m):
    return ("convT", _np(m.weight), _np(m.bias), m.stride[0], m.padding, m.output_padding)


class _Cat(nn.Module):
    def __init__(self, tail):
        super().__init__()
        self.a = nn.Conv2d(2, 3, 3, padding=1)
        self.b = nn.Conv2d(2, 5, 3, padding=1)
        self.c = nn.Conv2d(8, 4, 1) if tail else nn.Identity()

    def forward(self, x):
        return self.c(torch.cat([self.a(x), self.b(x)], dim=1))


def build(name):
    torch.manual_seed(31 + NAMES.index(name))
    cin = 2
    if name == "pool":
        m = nn.Sequential(nn.Conv2d(2, 5, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2))
        spec = [_conv(m[0]), ("relu",), ("maxpool", 2)]
    elif name == "upsample":
        m = nn.Sequential(nn.Conv2d(2, 3, 3, padding=1), nn.Upsample(scale_factor=2, mode="nearest"))
        spec = [_conv(m[0]), ("upsample", 2)]
    elif name == "convT_s2":
        m = nn.Sequential(nn.Conv2d(2, 4, 3, padding=1), nn.ConvTranspose2d(4, 3, 3, stride=2, padding=1, output_padding=1))
        spec = [_conv(m[0]), _convT(m[1])]
    elif name == "bn":
        m = nn.Sequential(nn.Conv2d(2, 6, 3, padding=1), nn.BatchNorm2d(6), nn.LeakyReLU(0.1))
        bn = m[1]
        with torch.no_grad():
            bn.running_mean.uniform_(-1, 1); bn.running_var.uniform_(0.5, 2); bn.weight.uniform_(0.5, 1.5); bn.bias.uniform_(-1, 1)
        spec = [_conv(m[0]), ("bn", _np(bn.weight), _np(bn.bias), _np(bn.running_mean), _np(bn.running_var), bn.eps), ("leaky", 0.1)]
    elif name == "convT_s1":
        m = nn.Sequential(nn.ConvTranspose2d(2, 4, 3, padding=1))
        spec = [_convT(m[0])]
    elif name == "two_convs":
        m = nn.Sequential(nn.Conv2d(2, 4, 3, padding=1), nn.Conv2d(4, 70, (3, 5), stride=(1, 2), padding=(1, 2)))
        spec = [_conv(m[0]), _conv(m[1])]
    elif name in ("concat", "cat_only"):
        m = _Cat(tail=name == "concat")
        spec = [("cat", [[_conv(m.a)], [_conv(m.b)]])] + ([_conv(m.c)] if name == "concat" else [])
    elif name == "pad":
        m = nn.Sequential(nn.ZeroPad2d(2), nn.Conv2d(2, 3, 5))
        spec = [("pad", 2), _conv(m[1])]
    else:
        raise ValueError(name)
    g = torch.Generator().manual_seed(97)
    x = torch.randn(2, cin, 12, 10, generator=g)
    return m.eval(), spec, x.numpy()
