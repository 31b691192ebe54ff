"""Shapes and seeded inputs.

generate_num_tokens / generate_hidden_sizes / generate_e5m6_inputs follow the reference's
tile_kernels/testing/generator.py:10-23,76-89.  make_config_input builds the five benchmark
workloads; inputs are always drawn on the CPU generator (the CUDA generator produces different
numbers) and then moved."""
import os
from typing import Iterable

import torch

from ..utils import align


def generate_num_tokens(alignment: int = 1, is_benchmark: bool = False) -> list[int]:
    full = os.getenv('TK_FULL_TEST') in ('1', 'true', 'True')
    tokens = ([0] if full and not is_benchmark else []) + [4001, 8001]
    return [align(t, alignment) for t in tokens]


def generate_hidden_sizes(align: int = 64) -> list[int]:
    return [h for h in (576, 2048, 2560, 3072, 4096, 6144, 7168) if h % align == 0]


# E5M6 corner values: smallest subnormal 2^-20, largest subnormal, smallest normal 2^-14
_E5M6_SPECIAL_VALUES = (2.0 ** -20, 2.0 ** -14 * 63 / 64, 2.0 ** -14)


def generate_e5m6_inputs(num_tokens: int, hidden: int, dtype: torch.dtype, device='cuda',
                         generator: torch.Generator = None) -> Iterable[tuple[torch.Tensor, bool]]:
    """One random tensor, then one tensor per special value with the last column at the format maximum."""
    yield torch.randn((num_tokens, hidden), dtype=torch.float32, generator=generator).to(dtype).to(device), False
    for value in _E5M6_SPECIAL_VALUES:
        x = torch.full((num_tokens, hidden), value, dtype=dtype, device=device)
        x[:, -1] = 65024.0
        yield x, True


def make_config_input(name: str, num_tokens: int = None, first_row: int = 0, chunk_rows: int = 4096,
                      out: torch.Tensor = None) -> torch.Tensor:
    """Seeded CPU bf16 input of a benchmark workload: rows [first_row, first_row + num_tokens) of

    cfg1  [4096, 7168]   N(0,1), 0.1% of entries x100, rows 0/1023/2048/4095 zero          seed 0
    cfg2  [7168, 2048]   N(0, 0.02), block rows 384:512 x cols 640:768 x1000                seed 2
    cfg3  [16384, 4096]  N(0,1) (gate | up halves)                                          seed 1
    cfg4  [32768, 7168]  Student-t(4) * 0.5                                                 seed 4
    cfg5  [262144, 7168] as cfg1 without zero rows                                          seed 5

    The tensor is defined chunk by chunk (4096 rows, generator seeded with seed * 1000003 + chunk index), so any
    row range can be produced without drawing the rows before it: ranks generate their own shards.
    `first_row` must be a multiple of `chunk_rows`.  `out` may be a preallocated (e.g. pinned) destination."""
    shapes = {'cfg1': (4096, 7168), 'cfg2': (7168, 2048), 'cfg3': (16384, 4096), 'cfg4': (32768, 7168),
              'cfg5': (262144, 7168)}
    seeds = {'cfg1': 0, 'cfg2': 2, 'cfg3': 1, 'cfg4': 4, 'cfg5': 5}
    total_rows, cols = shapes[name]
    rows = total_rows - first_row if num_tokens is None else num_tokens
    assert first_row % chunk_rows == 0
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.bfloat16)
    assert out.shape == (rows, cols) and out.dtype == torch.bfloat16
    for r0 in range(0, rows, chunk_rows):
        n = min(chunk_rows, rows - r0)
        g0 = first_row + r0  # global row of the chunk start
        g = torch.Generator().manual_seed(seeds[name] * 1000003 + g0 // chunk_rows)
        if name in ('cfg1', 'cfg5'):
            x = torch.randn((n, cols), generator=g)
            mask = torch.rand((n, cols), generator=g) < 1e-3
            x = torch.where(mask, x * 100, x)
            if name == 'cfg1':
                for r in (0, 1023, 2048, 4095):
                    if g0 <= r < g0 + n:
                        x[r - g0] = 0
        elif name == 'cfg2':
            x = torch.randn((n, cols), generator=g) * 0.02
            lo, hi = max(384, g0), min(512, g0 + n)
            if lo < hi:
                x[lo - g0:hi - g0, 640:768] *= 1000
        elif name == 'cfg3':
            x = torch.randn((n, cols), generator=g)
        else:
            z = torch.randn((5, n, cols), generator=g)
            x = z[0] / torch.sqrt((z[1:] ** 2).mean(dim=0)) * 0.5
        out[r0:r0 + n] = x.to(torch.bfloat16)
    return out
