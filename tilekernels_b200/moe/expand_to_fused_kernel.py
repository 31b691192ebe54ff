"""expand_to_fused, expand_to_fused_with_sf (reference: tile_kernels/moe/expand_to_fused_kernel.py:97-202)."""
import torch

from .. import _lib
from ..quant.common import current_stream_ptr, device_guard
from ..quant.types import QuantTensor
from ..utils import align, ceil_div


def _check_maps(token_topk_to_pos: torch.Tensor, pos_to_expert: torch.Tensor) -> None:
    assert token_topk_to_pos.dtype == torch.int32 and pos_to_expert.dtype == torch.int32
    assert token_topk_to_pos.is_cuda and pos_to_expert.is_cuda


def expand_to_fused(x: torch.Tensor, token_topk_to_pos: torch.Tensor, pos_to_expert: torch.Tensor) -> torch.Tensor:
    """Copy token t to every expanded position token_topk_to_pos[t, k] >= 0; positions with
    pos_to_expert < 0 are zero-filled.

    Args:
        x: (num_tokens, hidden), contiguous CUDA tensor of any element type; a row must be a multiple of 16 bytes.
        token_topk_to_pos: int32 (num_tokens, num_topk).
        pos_to_expert: int32 (num_expanded_tokens,).

    Returns: (num_expanded_tokens, hidden) tensor of x's dtype.
    """
    assert x.is_contiguous() and token_topk_to_pos.is_contiguous()
    assert x.dim() == 2 and token_topk_to_pos.dim() == 2
    assert x.is_cuda
    _check_maps(token_topk_to_pos, pos_to_expert)

    num_tokens, hidden = x.shape
    num_tokens_, num_topk = token_topk_to_pos.shape
    num_expanded_tokens = pos_to_expert.shape[0]
    assert num_tokens == num_tokens_

    out = torch.empty((num_expanded_tokens, hidden), dtype=x.dtype, device=x.device)
    if num_tokens > 0:
        with device_guard(x.device):
            _lib.check(_lib.lib().tkq_expand_to_fused(
                x.data_ptr(), num_tokens, hidden * x.element_size(), None, 0, token_topk_to_pos.data_ptr(), num_topk,
                pos_to_expert.data_ptr(), num_expanded_tokens, 0, out.data_ptr(), None, 0, current_stream_ptr(x.device)),
                'expand_to_fused')
    return out


def expand_to_fused_with_sf(
    x: QuantTensor,
    num_per_channels: int,
    token_topk_to_pos: torch.Tensor,
    pos_to_expert: torch.Tensor,
    use_tma_aligned_col_major_sf: bool = False,
) -> tuple[torch.Tensor, torch.Tensor]:
    """expand_to_fused for quantized rows: the scale factors of a token travel with its data.

    Args:
        x: (data, sf): data (num_tokens, hidden); sf (num_tokens, hidden_sf) contiguous, float32 (one scale per
            num_per_channels channels) or int32 (four ue8m0 exponents per word; needs the column-major output).
        num_per_channels: 32 or 128.
        token_topk_to_pos, pos_to_expert: as in expand_to_fused.
        use_tma_aligned_col_major_sf: return the scales column-major with a pitch of align(num_expanded_tokens, 4)
            (shape (num_expanded_tokens, hidden_sf), strides (1, pitch)).

    Returns: (out, out_sf).
    """
    x, x_sf = x
    assert x.is_contiguous() and x_sf.is_contiguous() and token_topk_to_pos.is_contiguous() and pos_to_expert.is_contiguous()
    assert x.dim() == 2 and token_topk_to_pos.dim() == 2 and pos_to_expert.dim() == 1
    assert x_sf.dtype in (torch.float32, torch.int32)
    assert num_per_channels in [32, 128]
    assert x.is_cuda and x_sf.is_cuda
    _check_maps(token_topk_to_pos, pos_to_expert)

    num_tokens, hidden = x.shape
    num_topk = token_topk_to_pos.shape[1]
    num_expanded_tokens = pos_to_expert.shape[0]
    assert num_tokens == token_topk_to_pos.shape[0]
    assert num_tokens == x_sf.shape[0]

    num_expanded_sf_tokens = align(num_expanded_tokens, 4) if use_tma_aligned_col_major_sf else num_expanded_tokens
    hidden_sf = ceil_div(hidden, num_per_channels)
    if x_sf.dtype == torch.int32:
        hidden_sf = ceil_div(hidden_sf, 4)
        assert use_tma_aligned_col_major_sf
    assert hidden_sf == x_sf.shape[1]

    out = torch.empty((num_expanded_tokens, hidden), dtype=x.dtype, device=x.device)
    sf_shape = (hidden_sf, num_expanded_sf_tokens) if use_tma_aligned_col_major_sf else (num_expanded_tokens, hidden_sf)
    out_sf = torch.empty(sf_shape, dtype=x_sf.dtype, device=x.device)
    if num_tokens > 0:
        with device_guard(x.device):
            _lib.check(_lib.lib().tkq_expand_to_fused(
                x.data_ptr(), num_tokens, hidden * x.element_size(), x_sf.data_ptr(), hidden_sf, token_topk_to_pos.data_ptr(),
                num_topk, pos_to_expert.data_ptr(), num_expanded_tokens, _lib.SF_COL_MAJOR if use_tma_aligned_col_major_sf else 0,
                out.data_ptr(), out_sf.data_ptr(), out_sf.stride(0), current_stream_ptr(x.device)), 'expand_to_fused_with_sf')
    out_sf = out_sf[:, :num_expanded_tokens].T if use_tma_aligned_col_major_sf else out_sf
    return out, out_sf
