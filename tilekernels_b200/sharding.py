"""Token-dimension sharding for multi-GPU runs.

Every cast on the hot path is independent per token (per 128-token band for the per-block and
per-channel casts), so k ranks each take a contiguous band of rows and run the same kernel on it;
no rank ever reads another rank's rows and there is no collective on the data path.  Concatenating
the ranks' outputs in rank order gives the single-GPU result byte for byte; each rank's
column-major scale tensor has its own pitch align(rows_of_rank, 4) (the global column-major tensor
is not materialised).
"""
from typing import Tuple


def shard_rows(num_tokens: int, rank: int, world_size: int, alignment: int = 128) -> Tuple[int, int]:
    """Rows [start, stop) of `rank`: bands of `alignment` rows dealt out as evenly as possible, the
    first `extra` ranks taking one band more; the last rank also takes the ragged tail."""
    assert 0 <= rank < world_size and num_tokens >= 0 and alignment > 0
    bands = num_tokens // alignment
    base, extra = divmod(bands, world_size)
    start_band = rank * base + min(rank, extra)
    stop_band = start_band + base + (1 if rank < extra else 0)
    start, stop = start_band * alignment, stop_band * alignment
    if rank == world_size - 1:
        stop = num_tokens
    return start, stop
