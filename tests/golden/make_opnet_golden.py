"""Writes opnet_golden.npz: the outputs torch's CPU operators give for the networks of tests/golden/opnet_models.py
(an implementation independent of this repository and of its oracle).

    python tests/golden/make_opnet_golden.py
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from tests.golden import opnet_models as OM  # noqa: E402


def main():
    out = {}
    for name in OM.NAMES:
        m, _, x = OM.build(name)
        with torch.no_grad():
            y = m.double()(torch.from_numpy(x).double()).float().numpy()
        out[name + "_y"] = y
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "opnet_golden.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
