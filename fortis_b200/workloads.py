"""Seeded synthetic workloads with the shapes and value distributions of the five benchmark configurations.  They
stand in for the climate / ocean / turbulence data sets and trained weights the reference measured on, which are not
redistributable.  Draws come from numpy's PCG64 generator (`np.random.default_rng(seed)`, draws in the order listed),
so a given (configuration, seed) is the same arrays everywhere.

Every workload is a dict:
    kind      "column" | "stencil" | "toy" | "conv"
    G, S, Lp, K   the descriptors (None for conv)
    gin, sout     host arrays in Fortran order (inputs, outputs), numpy float32
    layers        the model as layer dicts (fortis_b200.model.write_blob)
    units         rows of the model batch (columns, gridpoints, voxels)
    flop_per_unit, bytes_per_unit   algorithmic work: 2 x MACs, and host-array bytes read + written once
"""
import numpy as np

from . import descriptors as D
from .model import conv_layers, mlp_layers

COLUMN_DIMS = [244, 768, 768, 768, 768, 128]
STENCIL_DIMS = [27, 20, 20, 3]
TOY_DIMS = [64, 256, 256, 64]
F32 = np.float32


def _macs(dims):
    return sum(a * b for a, b in zip(dims[:-1], dims[1:]))


def column_inputs(ncol, seed, nlev=60):
    """T ~ N(250, 20), q ~ LogNormal(-6, 1), u, v ~ N(0, 10) as (ncol, nlev) Fortran arrays, then 4 per-column scalars
    ~ N(0, 1)."""
    rng = np.random.default_rng(seed)
    gin = [np.asfortranarray(250 + 20 * rng.standard_normal((ncol, nlev), dtype=F32)),
           np.asfortranarray(np.exp(-6 + rng.standard_normal((ncol, nlev), dtype=F32))),
           np.asfortranarray(10 * rng.standard_normal((ncol, nlev), dtype=F32)),
           np.asfortranarray(10 * rng.standard_normal((ncol, nlev), dtype=F32))]
    gin += [rng.standard_normal(ncol, dtype=F32) for _ in range(4)]
    return gin


def column_outputs(ncol, nlev=60):
    return [np.zeros((ncol, nlev), F32, order="F") for _ in range(2)] + [np.zeros(ncol, F32) for _ in range(8)]


def column_weights(seed=0):
    """Kaiming-normal (std = sqrt(2 / fan_in), benchmarks/climsim/export_wide.py:17-19) weights, zero biases,
    LeakyReLU(0.15) on the hidden layers."""
    return mlp_layers(COLUMN_DIMS, seed=seed)


def column(ncol=49152, seed=2, nlev=60, weight_seed=0):
    """Climate column-physics MLP: 244 features gathered from four (ncol, 60) fields and 4 scalars; 244 -> 768 x4 ->
    128; outputs scattered into two (ncol, 60) arrays and eight (ncol) vectors."""
    G, S, Lp, K = D.column(ncol, nlev)
    return dict(kind="column", G=G, S=S, Lp=Lp, K=K, gin=column_inputs(ncol, seed, nlev), sout=column_outputs(ncol, nlev),
                layers=column_weights(weight_seed), units=ncol, flop_per_unit=2 * _macs(COLUMN_DIMS), bytes_per_unit=4 * (244 + 128),
                label="climate column MLP, %d columns x %d levels, 244->768x4->128" % (ncol, nlev))


def stencil(nx=1440, ny=1080, nz=4, seed=3, weight_seed=4):
    """Ocean eddy-parameterisation stencil MLP: u, v, h ~ N(0, 1) on (nx+2, ny+2, nz) with a 1-cell halo; 27 -> 20 ->
    20 -> 3 with ReLU; weights and biases U(-0.3, 0.3)."""
    rng = np.random.default_rng(seed)
    gin = [np.asfortranarray(rng.standard_normal((nx + 2, ny + 2, nz), dtype=F32)) for _ in range(3)]
    sout = [np.zeros((nx + 2, ny + 2, nz), F32, order="F") for _ in range(3)]
    layers = mlp_layers(STENCIL_DIMS, seed=weight_seed, init="uniform", act="relu", bias="uniform")
    G, S, Lp, K = D.stencil(nx, ny, nz)
    return dict(kind="stencil", G=G, S=S, Lp=Lp, K=K, gin=gin, sout=sout, layers=layers, units=nx * ny * nz,
                flop_per_unit=2 * _macs(STENCIL_DIMS), bytes_per_unit=24, shape=(nx, ny, nz),
                label="ocean stencil MLP, %dx%dx%d points, 27->20->20->3" % (nx, ny, nz))


def toy(ncol=4096, seed=0, weight_seed=1):
    """Toy MLP: A(64, ncol) ~ U(-1, 1); 64 -> 256 -> 256 -> 64 with ReLU; Kaiming-uniform weights, zero biases."""
    rng = np.random.default_rng(seed)
    gin = [np.asfortranarray((2 * rng.random((64, ncol)) - 1).astype(F32))]
    sout = [np.zeros((64, ncol), F32, order="F")]
    layers = mlp_layers(TOY_DIMS, seed=weight_seed, init="kaiming_uniform", act="relu")
    G, S, Lp, K = D.identity(64, 64, ncol)
    return dict(kind="toy", G=G, S=S, Lp=Lp, K=K, gin=gin, sout=sout, layers=layers, units=ncol, flop_per_unit=2 * _macs(TOY_DIMS),
                bytes_per_unit=4 * 128, label="toy MLP, %d columns" % ncol)


def conv(shape=(8, 33, 33, 33), seed=5, weight_seed=6, nblocks=6):
    """3-D conv super-resolution net on an NDHWC fp32 batch ~ N(0, 1): conv 3->64 + LeakyReLU(0.2), `nblocks` residual
    blocks [conv, LeakyReLU, conv, + skip], conv 64->3; He-normal weights, zero biases."""
    shape = tuple(shape)
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(shape + (3,), dtype=F32)
    macs = 27 * (3 * 64 + 2 * nblocks * 64 * 64 + 64 * 3)
    return dict(kind="conv", G=None, S=None, Lp=None, K=None, gin=[x], sout=[np.zeros(shape + (3,), F32)],
                layers=conv_layers(3, 64, 3, nblocks=nblocks, seed=weight_seed), units=int(np.prod(shape)), shape=shape,
                flop_per_unit=2 * macs, bytes_per_unit=24,
                label="conv3d super-resolution net, %d x %dx%dx%d x 3 NDHWC, 3->64, %d residual blocks, 64->3" % (shape + (nblocks,)))


def sharded_block(block, ncol=1 << 20):
    """Block `block` of the sharded column problem: ncol columns drawn with seed 7000 + block.  The global problem of B
    blocks is their concatenation along the column index; rank r of R owns blocks [r*B/R, (r+1)*B/R)."""
    return column(ncol=ncol, seed=7000 + block)


def make(name, rank=0, ncol=0):
    if name == "column":
        return column(ncol or 49152, seed=2 + rank)
    if name == "column_c5":
        return sharded_block(rank, ncol or (1 << 20))
    if name == "stencil":
        return stencil(seed=3 + rank)
    if name == "conv":
        return conv(seed=5 + rank)
    if name == "toy":
        return toy(ncol or 4096, seed=rank)
    raise ValueError("unknown workload " + name)
