"""Host-side row / column partitioning of one quantized linear across GPUs.

Rows of A are independent in sd::qgemm (each row has its own activation scale,
reference src/core/qgemm.cpp:84-96) and so are the columns of the output (each
weight row has its own scale), so both splits reproduce the single-GPU result
bit for bit with no exchange inside the GEMM.
"""

TILE_M = 128  # the GEMM kernel's M tile: shard boundaries are kept on it


def row_shard(M, world, rank, tile=TILE_M):
    """Contiguous [begin, end) rows of rank `rank`: ceil(M/world) rounded up to the tile."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    per = (M + world - 1) // world
    per = (per + tile - 1) // tile * tile
    b = min(M, rank * per)
    e = min(M, b + per)
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
