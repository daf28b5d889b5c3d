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


def check_even_shards(n_rows: int, world: int) -> None:
    """The gather of the outputs is one collective with equal contributions: every rank must hold the same number of
    128-row tiles. Raises before anything is launched when they do not divide (a collective with mismatched sizes can
    hang the ranks)."""
    assert n_rows % 128 == 0, "weight rows must be a multiple of 128"
    if (n_rows // 128) % world != 0:
        raise ValueError(f"{n_rows} weight rows are {n_rows // 128} tiles of 128, which {world} ranks cannot share equally; "
                         "use a rank count that divides the tile count (or pad the weight)")


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
    # equal widths on every rank, checked on the host before the collective (mismatched sizes can hang it)
    widths = [None] * world
    dist.all_gather_object(widths, (M, n_local), group=group)
    if any(w != (M, n_local) for w in widths):
        raise ValueError(f"all_gather_output needs equal local shapes on every rank, got {widths}")
    # rank blocks concatenated along dim 0 (the form every backend accepts), viewed as [world][M][n_local]
    buf = torch.empty(world * M, n_local, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, local.contiguous(), group=group)
    return gathered_to_row_major(buf.view(world, M, n_local))
