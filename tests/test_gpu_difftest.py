"""Differential test at the descriptor level: random but valid gather / scatter / loop / kdist sets (stencil offsets,
1-D and 2-D loops, plane dimensions chosen by argument or distributed, f32 / f64 arrays, scalars, lifted expression
lists) with a small random MLP behind them, run through the library and through the CPU interpreter of the oracle.
The reference tests its compiler the same way, fused against unfused on random programs
(tests/difftest/gen_difftest.py:35-120, bar 5e-6); here gather and scatter have to be bit-exact and the forward within
the fp32 bar, in the three-call form and in the fused step, with host arrays and with device arrays."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import fortis_b200
from fortis_b200 import descriptors as D
from oracle import fortis_oracle as fo

# a longer sweep with other seeds: FORTIS_DIFFTEST_CASES=400 FORTIS_DIFFTEST_SEED=1 python -m pytest tests/test_gpu_difftest.py -m gpu
NCASES = int(os.environ.get("FORTIS_DIFFTEST_CASES", "200"))
SEED0 = 9000 + 1000 * int(os.environ.get("FORTIS_DIFFTEST_SEED", "0"))


def dev(a):
    t = torch.from_numpy(np.ascontiguousarray(a.reshape(-1, order="F")))
    return t.cuda()


def back(t, like):
    return t.cpu().numpy().reshape(like.shape, order="F")


def make_arrays(J, rng, lo=-2.0, hi=2.0):
    return [np.asfortranarray(rng.uniform(lo, hi, size=a["shape"]).astype(fo._NP[a["elt"]])) for a in J["arrays"]]


@pytest.mark.parametrize("block", range(4))
def test_random_descriptors_against_the_interpreter(block):
    rng = np.random.default_rng(SEED0 + block)
    h = fortis_b200.Host()
    for case in range(NCASES // 4):
        G, S, Lp, K, nargs, planes = D.random_case(rng)
        P = fo.loop_params(Lp, K)
        nin, nout = G["n"], S["n"]
        layers = fortis_b200.mlp_layers([nin, 12, nout], seed=int(rng.integers(1 << 30)), init="uniform", act="relu", bias="uniform")
        gin, sin = make_arrays(G, rng), make_arrays(S, rng)
        a0 = (int(rng.integers(1, planes + 1)),) if nargs else ()
        tag = "block %d case %d (%s, %s)" % (block, case, "kdist" if P["kdist"] else "arg plane" if nargs else "flat", G["exprs"])
        h.reset()
        h.configure(gather=G, scatter=S, loop=Lp, kdist=K)
        h.load_model(fortis_b200.write_blob(layers))
        rows = P["count"] * P["nk"]
        # ---- three calls: gather bit-exact, forward within the fp32 bar, scatter of the same Y bit-exact
        h.gather(gin, args=a0)
        X = h.model_input(rows, nin)
        Xo = fo.gather(G, Lp, K, gin, args=a0)
        assert X.tobytes() == Xo.tobytes(), tag
        h.forward_batched()
        Y = h.model_output(rows, nout)
        # the fp32 bar; where the outputs nearly cancel (constant inputs, tiny norms) a relative error means little, and
        # the library only has to be about as close to an fp64 forward as the fp32 oracle itself is
        Y64 = fo.mlp_forward(layers, X, dtype=np.float64)
        e_lib, e_ora = fo.rel_l2(Y, Y64), fo.rel_l2(fo.mlp_forward(layers, X), Y64)
        assert e_lib < 1e-5 or e_lib < 8 * e_ora + 1e-6, tag
        work, ref = [a.copy(order="F") for a in sin], [a.copy(order="F") for a in sin]
        for k in (range(P["klo"], P["klo"] + P["nk"]) if P["kdist"] else [a0[0] if a0 else 1]):
            h.scatter(work, args=(k,) if (P["kdist"] or a0) else ())
            fo.scatter(S, Lp, K, Y, ref, args=(k,))
        for a, b in zip(work, ref):
            assert a.tobytes(order="F") == b.tobytes(order="F"), tag
        # ---- fused step, host arrays then device arrays: the whole chain against the interpreter
        full = [a.copy(order="F") for a in sin]
        Yo = fo.mlp_forward(layers, Xo)
        full64 = [a.copy(order="F") for a in sin]
        Yo64 = fo.mlp_forward(layers, Xo, dtype=np.float64).astype(np.float32)
        for k in (range(P["klo"], P["klo"] + P["nk"]) if P["kdist"] else [a0[0] if a0 else 1]):
            fo.scatter(S, Lp, K, Yo, full, args=(k,))
            fo.scatter(S, Lp, K, Yo64, full64, args=(k,))
        for resident in (False, True):
            w2 = [a.copy(order="F") for a in sin]
            g_arr = [dev(a) for a in gin] if resident else gin
            s_arr = [dev(a) for a in w2] if resident else w2
            h.step(g_arr, s_arr, args=a0)
            h.sync()
            got = [back(t, a) for t, a in zip(s_arr, w2)] if resident else w2
            for a, b, c, orig in zip(got, full, full64, sin):
                assert np.array_equal(a != orig, b != orig) or fo.rel_l2(a, b) < 1e-6, tag      # the same cells were written
                assert fo.rel_l2(a, b) < 1e-5 or fo.rel_l2(a, c) < 8 * fo.rel_l2(b, c) + 1e-6, tag
    h.reset()
