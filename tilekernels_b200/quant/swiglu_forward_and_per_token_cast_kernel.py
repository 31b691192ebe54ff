"""swiglu_forward_and_per_token_cast
(reference: tile_kernels/quant/swiglu_forward_and_per_token_cast_kernel.py:175-260)."""
from typing import Optional

import torch

from .. import _lib
from ..config import get_exact_swiglu_codes, get_num_sms
from .common import DTYPE_TO_ENUM, alloc_scaling_factors, cast_epilogue, current_stream_ptr, get_cast_output_config, device_guard
from .types import QuantTensor


def swiglu_forward_and_per_token_cast(
    x: torch.Tensor,
    fmt: str,
    num_per_channels: int,
    pos_to_token_topk: Optional[torch.Tensor] = None,
    topk_weights: Optional[torch.Tensor] = None,
    pos_to_expert: Optional[torch.Tensor] = None,
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
    swiglu_clamp_value: Optional[float] = None,
    clamped_count: Optional[torch.Tensor] = None,
    sf_clamp_min: Optional[float] = None,
) -> QuantTensor:
    """silu(x[:, :hidden]) * x[:, hidden:] in fp32 (optionally clamped and weighted per row), then the
    per-token FP8 e4m3 cast of that activation, in one kernel.

    Args:
        x: contiguous CUDA tensor (num_expanded_tokens, 2 * hidden), bfloat16 or float32; hidden % 128 == 0.
        fmt: 'e4m3'.
        num_per_channels: 128 or hidden.
        pos_to_token_topk, topk_weights: optional row weights, weight = topk_weights.flatten()[pos].
        pos_to_expert: optional int32 per row; rows with a negative entry are skipped (outputs untouched).
        swiglu_clamp_value: gate clamped to <= c, up to [-c, c] before the activation.
        clamped_count: int64[3], incremented by the numbers of gate > c, up > c, up < -c.
        sf_clamp_min: lower clamp of the group maximum (default 1e-4).

    Returns:
        (out, out_sf): float8_e4m3fn (num_expanded_tokens, hidden) and the scales.
    """
    assert x.dim() == 2 and x.is_contiguous() and x.is_cuda
    assert x.dtype in (torch.bfloat16, torch.float32)
    num_expanded_tokens, hidden = x.shape
    hidden = hidden // 2

    if pos_to_token_topk is not None:
        assert pos_to_token_topk.dim() == 1 and pos_to_token_topk.shape[0] == num_expanded_tokens
        assert pos_to_token_topk.dtype == torch.int32 and pos_to_token_topk.is_contiguous()
        assert topk_weights is not None
        assert topk_weights.dim() == 2 and topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()
    if pos_to_expert is not None:
        assert pos_to_expert.dim() == 1 and pos_to_expert.shape[0] == num_expanded_tokens
        assert pos_to_expert.dtype == torch.int32 and pos_to_expert.is_contiguous()
    if clamped_count is not None:
        assert swiglu_clamp_value is not None
        assert clamped_count.dim() == 1 and clamped_count.shape[0] == 3
        assert clamped_count.dtype == torch.int64 and clamped_count.is_contiguous()

    assert hidden % 128 == 0
    assert num_per_channels == 128 or num_per_channels == hidden
    assert num_per_channels == 128 or (not use_tma_aligned_col_major_sf)
    assert fmt == 'e4m3'

    out_config = get_cast_output_config(fmt, (1, num_per_channels), use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0,
                                        custom_clamp_min_value=sf_clamp_min)
    out = torch.empty((num_expanded_tokens, hidden), dtype=torch.float8_e4m3fn, device=x.device)
    out_sf = alloc_scaling_factors((num_expanded_tokens, hidden), out_config, device=x.device)
    if num_expanded_tokens > 0:
        with device_guard(x.device):
            rc = _lib.lib().tkq_swiglu_forward_and_per_token_cast(
                x.data_ptr(), DTYPE_TO_ENUM[x.dtype], num_expanded_tokens, hidden, num_per_channels,
                None if pos_to_token_topk is None else pos_to_token_topk.data_ptr(),
                None if topk_weights is None else topk_weights.data_ptr(),
                None if pos_to_expert is None else pos_to_expert.data_ptr(),
                -1.0 if swiglu_clamp_value is None else float(swiglu_clamp_value),
                None if clamped_count is None else clamped_count.data_ptr(),
                -1.0 if sf_clamp_min is None else float(sf_clamp_min),
                get_num_sms() if clamped_count is not None else 0,
                out_config.flags | (_lib.EXACT_CODES if get_exact_swiglu_codes() else 0), out.data_ptr(), out_sf.data_ptr(), out_sf.stride(0), current_stream_ptr(x.device))
        _lib.check(rc, 'tkq_swiglu_forward_and_per_token_cast')

    out_sf = cast_epilogue(out_sf, num_expanded_tokens, hidden, out_config)
    return out, out_sf
