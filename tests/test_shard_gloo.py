"""The N > 1 host logic on the CPU: rank partitioning and the checksum all-reduce, world_size 2 over gloo."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fortis_b200 import shard
from oracle import fortis_oracle as fo
import fortis_b200


def test_column_blocks_tile_the_range():
    for ncol in (0, 1, 7, 49152, 1000003):
        for world in (1, 2, 3, 8):
            blocks = [shard.column_block(r, world, ncol) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == ncol
            assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in blocks]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.column_block(2, 2, 10)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ncol, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # the same seeded global problem on every rank; each computes only its own column block with the oracle
        nlev = 3
        rng = np.random.default_rng(0)
        gin = [np.asfortranarray(rng.normal(size=(ncol, nlev)).astype(np.float32)) for _ in range(2)]
        gin += [rng.normal(size=ncol).astype(np.float32)]
        layers = fortis_b200.mlp_layers([2 * nlev + 1, 16, nlev + 1], seed=1)
        lo, hi = shard.column_block(rank, world, ncol)
        G, S, Lp, K = fo.column_descriptors(hi - lo, nlev, nfields=2, nscal=1, nout_fields=1, nout_scal=1)
        mine = shard.shard_arrays(gin, lo, hi)
        outs = [np.zeros((hi - lo, nlev), np.float32, order="F"), np.zeros(hi - lo, np.float32)]
        fo.full_step(G, S, Lp, K, layers, mine, outs)
        total = shard.allreduce_checksum(fo.checksum(outs))
        if rank == 0:
            Gf, Sf, Lf, Kf = fo.column_descriptors(ncol, nlev, nfields=2, nscal=1, nout_fields=1, nout_scal=1)
            full = [np.zeros((ncol, nlev), np.float32, order="F"), np.zeros(ncol, np.float32)]
            fo.full_step(Gf, Sf, Lf, Kf, layers, gin, full)
            # per-column outputs identical to the unsharded run, and the reduced checksum equal to the global one
            assert np.array_equal(full[0][lo:hi], outs[0]) and np.array_equal(full[1][lo:hi], outs[1])
            out.put((total, fo.checksum(full)))
    finally:
        dist.destroy_process_group()


def test_two_rank_checksum_allreduce_matches_unsharded():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 101, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    total, want = out.get(timeout=10)
    assert abs(total - want) <= 1e-9 * max(1.0, abs(want))
