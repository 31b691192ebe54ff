"""Integer helpers (same names as the reference's tile_kernels/utils.py:1-10)."""


def ceil_div(x: int, y: int) -> int:
    return -(-x // y)


def align(x: int, y: int) -> int:
    return ceil_div(x, y) * y


def is_power_of_two(x: int) -> bool:
    return x > 0 and x & (x - 1) == 0
