"""per_channel_cast_and_transpose (reference: tile_kernels/quant/per_channel_cast_and_transpose_kernel.py:85-123)."""
import torch

from .. import _lib
from .common import current_stream_ptr, device_guard
from .types import QuantTensor


def per_channel_cast_and_transpose(x: torch.Tensor, fmt: str, num_per_tokens: int, round_sf: bool = False) -> QuantTensor:
    """Cast a contiguous bfloat16 matrix to FP8 e4m3 with one scale per (num_per_tokens tokens x 1 channel) and
    write the data transposed.

    Returns:
        (out, out_sf): float8_e4m3fn (hidden, num_tokens) and float32 (num_tokens / num_per_tokens, hidden).
    """
    assert x.dim() == 2 and x.is_contiguous() and x.is_cuda
    assert x.dtype == torch.bfloat16
    num_tokens, hidden = x.shape
    assert fmt == 'e4m3'
    assert num_tokens % 128 == 0 and hidden % 64 == 0
    assert num_per_tokens in [32, 128]

    out = torch.empty((hidden, num_tokens), dtype=torch.float8_e4m3fn, device=x.device)
    out_sf = torch.empty((num_tokens // num_per_tokens, hidden), dtype=torch.float32, device=x.device)
    if num_tokens > 0:
        with device_guard(x.device):
            rc = _lib.lib().tkq_per_channel_cast_and_transpose(x.data_ptr(), num_tokens, hidden, num_per_tokens,
                                                               _lib.ROUND_SF if round_sf else 0, out.data_ptr(), out_sf.data_ptr(),
                                                               current_stream_ptr(x.device))
        _lib.check(rc, 'tkq_per_channel_cast_and_transpose')
    return out, out_sf
