"""Integer helpers under the names of the reference's tile_kernels/utils.py:1-10."""


def ceil_div(x: int, y: int) -> int:
    """Quotient of x / y rounded towards plus infinity."""
    quotient, remainder = divmod(x, y)
    return quotient + (1 if remainder else 0)


def align(x: int, y: int) -> int:
    """Smallest multiple of y that is not below x."""
    remainder = x % y
    return x if remainder == 0 else x + y - remainder


def is_power_of_two(x: int) -> bool:
    """True for 1, 2, 4, 8, ..."""
    return x >= 1 and bin(x).count('1') == 1
