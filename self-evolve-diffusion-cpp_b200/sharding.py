"""Host-side row / column partitioning of one quantized linear across GPUs.

Rows of A are independent in sd::qgemm (each row has its own activation scale,
reference src/core/qgemm.cpp:84-96) and so are the columns of the output (each
weight row has its own scale), so both splits reproduce the single-GPU result
bit for bit with no exchange inside the GEMM.
"""

TILE_M = 256  # rows of one CTA-pair tile of the large-problem GEMM: shard boundaries sit on it


def row_shard(M, world, rank, tile=TILE_M):
    """Contiguous [begin, end) rows of rank `rank`, balanced in whole tiles.

    The ceil(M / tile) row tiles are dealt out as evenly as whole tiles allow: every rank gets
    floor(tiles / world) of them and the first (tiles mod world) ranks one more, so no rank
    carries more than ceil(tiles / world) tiles and every tile but the ragged last one is full
    (a rank's time is set by its tile count, a partly filled tile costing as much as a full
    one).  M = 27280 over 8 ranks: 107 tiles -> 14, 14, 14, 13, 13, 13, 13, 13 (the last rank's
    13th tile holds the 144 remaining rows)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    tiles = (M + tile - 1) // tile
    base, extra = divmod(tiles, world)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    b = min(M, first * tile)
    e = min(M, (first + count) * tile)
    return b, e


def col_shard(N, world, rank, align=32):
    """Contiguous [begin, end) output columns (weight rows) of rank `rank`."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    per = (N + world - 1) // world
    per = (per + align - 1) // align * align
    b = min(N, rank * per)
    e = min(N, b + per)
    return b, e
