"""N-sharding of one projection across the GPUs of a node: every rank holds a contiguous block of weight rows
(codes and scale atoms), quantises the (tiny, replicated) activation itself and computes its block of output
columns; no reduction is needed, and the only collective is one all-gather of the bf16 output.

Shard boundaries are multiples of 128 weight rows so that scale atoms split cleanly; for the interleaved
gate | up matrix 128 rows are the gate and the up rows of the same 64 outputs, so a rank owns whole outputs.
"""

from __future__ import annotations

import torch


def shard_rows(n_rows: int, world: int, rank: int, glu: bool = False) -> tuple[int, int]:
    """Weight rows [begin, end) of `rank`: tiles of 128 rows dealt out as evenly as possible, in order."""
    assert n_rows % 128 == 0 and 0 <= rank < world
    tiles = n_rows // 128
    assert tiles >= world, "fewer 128-row tiles than ranks"
    base, extra = divmod(tiles, world)
    begin = rank * base + min(rank, extra)
    return begin * 128, (begin + base + (1 if rank < extra else 0)) * 128


def output_columns(n_rows: int, world: int, rank: int, glu: bool = False) -> tuple[int, int]:
    b, e = shard_rows(n_rows, world, rank, glu)
    return (b // 2, e // 2) if glu else (b, e)


def gathered_to_row_major(gathered: torch.Tensor) -> torch.Tensor:
    """[world][M][n_local] (what all_gather_into_tensor yields for equal shards) -> row-major [M][world * n_local]."""
    world, M, n_local = gathered.shape
    return gathered.permute(1, 0, 2).reshape(M, world * n_local)


def all_gather_output(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gathers equal-width local outputs [M][n_local] into row-major [M][world * n_local] on every rank."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if world == 1:
        return local
    M, n_local = local.shape
    # rank blocks concatenated along dim 0 (the form every backend accepts), viewed as [world][M][n_local]
    buf = torch.empty(world * M, n_local, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, local.contiguous(), group=group)
    return gathered_to_row_major(buf.view(world, M, n_local))
