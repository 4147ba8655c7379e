"""Splitting a batch of examples over the GPUs of one box.

Examples are independent in every operation of the path (the reference loops over them,
include/libmolgrid/grid_maker.h:197-200,288-300), so a batch is cut into contiguous slices, one per
rank, and each rank grids its slice on its own GPU.  No tensor is exchanged: the grids stay on the
GPU whose network replica consumes them.  The only thing ranks have to agree on is the cut, which
every rank computes from the same atom counts.
"""
import numpy as np


def shard_bounds(n_atoms, world_size, per_example_cost=1200.0):
    """Contiguous [start, end) slices of the batch, one per rank, balancing estimated work.

    The work of an example is its atom count plus a constant for writing/reading its grid
    (``per_example_cost`` atom-equivalents; one 28x48^3 grid costs about as much as 1200 atoms on a
    B200).  Deterministic and identical on every rank for the same ``n_atoms``.
    """
    n_atoms = np.asarray(n_atoms, dtype=np.float64)
    batch = int(n_atoms.shape[0])
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    cost = np.cumsum(n_atoms + per_example_cost)
    total = cost[-1] if batch else 0.0
    cuts = [0]
    for r in range(1, world_size):
        target = total * r / world_size
        k = int(np.searchsorted(cost, target, side="left")) + 1 if batch else 0
        # choose the boundary whose prefix cost is nearest the target
        if 1 < k <= batch and abs(cost[k - 2] - target) <= abs(cost[k - 1] - target):
            k -= 1
        cuts.append(min(max(k, cuts[-1]), batch))
    cuts.append(batch)
    return [(cuts[r], cuts[r + 1]) for r in range(world_size)]


def my_slice(n_atoms, rank, world_size):
    """The [start, end) slice of rank ``rank``."""
    return shard_bounds(n_atoms, world_size)[rank]
