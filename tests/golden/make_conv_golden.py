"""Writes conv_general.npz: inputs, weights and outputs of single convolution layers computed by torch's CPU
convolutions (an implementation independent of this repository), for the shapes the library rules fortis_conv2d /
fortis_conv3d / fortis_conv3d_fft have to cover: the 2-D probe of the reference's operator micro-suite
(tests/optest.py: Conv2d(1, 4, 3, padding=1) on a 16 x 16 ramp), per-axis strides and paddings, non-cubic kernels,
5^3 and 7^3 'valid' kernels (the transform path of runtime/fortis_fft.cu:66-79) and a strided 3-D layer.

    python tests/golden/make_conv_golden.py
"""
import os

import numpy as np
import torch

CASES = {
    # name: (N, C, D, H, W, F, (KD, KH, KW), stride, pad)
    "c2d_probe": (1, 1, 1, 16, 16, 4, (1, 3, 3), (1, 1, 1), (0, 1, 1)),
    "c2d_strided": (2, 3, 1, 13, 17, 5, (1, 3, 5), (1, 2, 1), (0, 1, 2)),
    "c2d_1x1": (1, 8, 1, 9, 9, 4, (1, 1, 1), (1, 1, 1), (0, 0, 0)),
    "c3d_valid5": (1, 2, 12, 12, 12, 3, (5, 5, 5), (1, 1, 1), (0, 0, 0)),
    "c3d_valid7": (1, 1, 10, 11, 12, 2, (7, 7, 7), (1, 1, 1), (0, 0, 0)),
    "c3d_strided": (2, 4, 9, 10, 11, 6, (3, 3, 3), (2, 2, 2), (1, 1, 1)),
    "c3d_mixed": (1, 3, 6, 9, 20, 70, (1, 3, 2), (1, 2, 3), (0, 2, 1)),
}


def main():
    g = torch.Generator().manual_seed(11)
    out = {}
    for name, (N, C, D, H, W, F, K, st, pad) in CASES.items():
        if name == "c2d_probe":
            n = H * W
            x = torch.arange(1, n + 1, dtype=torch.float32) / n
            x = ((x - x.mean()) / x.std(unbiased=False)).view(1, 1, 1, H, W)
        else:
            x = torch.randn(N, C, D, H, W, generator=g)
        w = torch.randn(F, C, *K, generator=g) / float(np.sqrt(C * K[0] * K[1] * K[2]))
        with torch.no_grad():
            y = torch.nn.functional.conv3d(x.double(), w.double(), stride=st, padding=pad).float()
        out[name + "_x"], out[name + "_w"], out[name + "_y"] = x.numpy(), w.numpy(), y.numpy()
        out[name + "_sp"] = np.array(list(st) + list(pad), dtype=np.int64)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "conv_general.npz"), **out)
    print({k: v.shape for k, v in out.items() if k.endswith("_y")})


if __name__ == "__main__":
    main()
