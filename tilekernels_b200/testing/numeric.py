"""Bit-exact comparison, bias check and byte counting
(same conventions as the reference's tile_kernels/testing/numeric.py:5-65)."""
import math

import torch


def _raw_bytes(t: torch.Tensor) -> torch.Tensor:
    dense = torch.empty(t.shape, dtype=t.dtype, device=t.device)
    dense.copy_(t)
    return dense.flatten().view(torch.uint8)


def _strides_match(x: torch.Tensor, y: torch.Tensor) -> bool:
    # the stride of a dimension of extent 1 carries no information (torch itself normalises it at will)
    return all(sx == sy for sx, sy, n in zip(x.stride(), y.stride(), x.shape) if n > 1)


def assert_equal(x: torch.Tensor, y: torch.Tensor, check_dtype: bool = True, check_shape: bool = True,
                 check_stride: bool = True) -> None:
    """dtype, shape, strides and every byte must agree."""
    assert not check_dtype or x.dtype == y.dtype, f'Tensor dtypes are not equal: {x.dtype} vs {y.dtype}'
    assert not check_shape or x.shape == y.shape, f'Tensor shapes are not equal: {x.shape} vs {y.shape}'
    assert not check_stride or x.numel() == 0 or _strides_match(x, y), \
        f'Tensor strides are not equal: {x.stride()} vs {y.stride()}'
    assert x.device == y.device, f'Tensor devices are not equal: {x.device} vs {y.device}'
    bx, by = _raw_bytes(x), _raw_bytes(y)
    if not torch.equal(bx, by):
        bad = torch.nonzero(bx != by).flatten()
        raise AssertionError(f'Tensor values are not equal: shape {tuple(x.shape)}, {bad.numel()} differing bytes, '
                             f'first at byte offsets {bad[:8].tolist()}')


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """1 - cosine-like similarity, in float64."""
    x, y = x.double(), y.double()
    denominator = (x * x + y * y).sum()
    return 1 - 2 * (x * y).sum() / denominator if denominator != 0 else torch.zeros(())


def check_bias(x: torch.Tensor, ref_x: torch.Tensor) -> None:
    """Rounding must be unbiased: the share of dequantised values below the original stays within
    10 / sqrt(n) of one half (a binomial argument; ties count half)."""
    count = x.numel()
    if count == 0:
        return
    less = (x < ref_x).sum().item()
    equal = (x == ref_x).sum().item()
    ratio = (less + equal / 2) / count
    assert abs(ratio - 0.5) < 10 / math.sqrt(count), f'rounding looks biased: less-than ratio {ratio:.4f} over {count} values'


def count_bytes(*tensors) -> int:
    """Bytes of all tensors (nested tuples allowed, None ignored): the byte count behind every GB/s figure."""
    total = 0
    for t in tensors:
        if isinstance(t, (tuple, list)):
            total += count_bytes(*t)
        elif t is not None:
            total += t.numel() * t.element_size()
    return total
