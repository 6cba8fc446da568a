"""Column sharding across ranks: each rank owns one contiguous block of the column index (the fastest index of the
(ncol, nlev) host arrays), holds that block resident in its own GPU, and runs the unchanged single-GPU step on it.
Columns are independent (that independence is what the reference's loop analysis proves before batching:
driver/fortis_units.py:1-11), so the only communication is the sum of the per-rank fp64 checksums.
"""
from typing import List, Tuple


def column_block(rank: int, world: int, ncol: int) -> Tuple[int, int]:
    """[lo, hi) of the columns rank `rank` owns: contiguous, sizes differ by at most one, earlier ranks take the
    remainder."""
    if not (0 <= rank < world) or ncol < 0:
        raise ValueError("bad rank / world / ncol")
    base, rem = divmod(ncol, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_arrays(arrays: List, lo: int, hi: int) -> List:
    """The rank's block of every (ncol, ...) Fortran array, as Fortran-contiguous copies."""
    import numpy as np
    return [np.asfortranarray(a[lo:hi]) for a in arrays]


def allreduce_checksum(local: float, group=None, device=None) -> float:
    """Sum of the per-rank checksums over the process group (NCCL on GPUs, gloo on CPUs); identity without one."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(local)
    t = torch.tensor([local], dtype=torch.float64, device=device or ("cuda" if dist.get_backend(group) == "nccl" else "cpu"))
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return float(t.item())
