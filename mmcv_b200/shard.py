"""Batch sharding of the forward across ranks (the only way this path partitions)."""


def batch_shard(n_total: int, rank: int, world: int):
    """Contiguous shard [n0, n1) of the batch for `rank`; samples are independent, weights
    are replicated, and no exchange is needed (reference loop over samples:
    mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:108-130)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f'bad rank {rank} of {world}')
    per = (n_total + world - 1) // world
    n0 = min(n_total, rank * per)
    n1 = min(n_total, (rank + 1) * per)
    return n0, n1
