"""Batch split across GPUs: one process per GPU, weights replicated, no collective.

Every image is an independent unit of the convolution, and the blocked layout
``[N][C/cb][H][W][cb]`` is batch-major, so a rank's share is one contiguous
slice of the input and of the output: no repack and no exchange step.
"""
from __future__ import annotations

from typing import Tuple


def batch_slice(total: int, rank: int, world: int) -> Tuple[int, int]:
    """[start, stop) of the images rank ``rank`` of ``world`` processes owns.

    The first ``total % world`` ranks take one image more, so any batch size
    splits over any number of ranks; ranks past the batch get an empty slice.
    """
    if world < 1 or not 0 <= rank < world or total < 0:
        raise ValueError('bad rank / world / total')
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard(tensor, rank: int, world: int):
    """The rank's batch slice of a batch-major tensor (a view, no copy)."""
    a, b = batch_slice(int(tensor.shape[0]), rank, world)
    return tensor[a:b]
