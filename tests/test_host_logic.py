"""Host-side logic of the entry points that needs no GPU: scale-factor geometry (the reference's
tile_kernels/quant/common.py:130-193 contract), flag encoding, clamp defaults, the FP4 unpacker."""
import pytest
import torch

from tilekernels_b200 import _lib
from tilekernels_b200.quant import common


def _sf(shape, block, col, ue):
    cfg = common.get_cast_output_config('e4m3', block, col, True, ue)
    storage = common.alloc_scaling_factors(shape, cfg, device='cpu')
    return cfg, storage, common.cast_epilogue(storage, shape[0], shape[1], cfg)


def test_row_major_scales():
    cfg, storage, sf = _sf((4001, 7168), (1, 128), False, False)
    assert storage.shape == (4001, 56) and storage.dtype == torch.float32
    assert sf.shape == (4001, 56) and sf.stride() == (56, 1)
    assert cfg.flags == _lib.ROUND_SF


def test_col_major_scales_are_padded_to_16_bytes():
    cfg, storage, sf = _sf((4001, 7168), (1, 128), True, False)
    assert storage.shape == (56, 4001) and storage.stride() == (4004, 1)
    assert sf.shape == (4001, 56) and sf.stride() == (1, 4004)
    assert cfg.flags == _lib.ROUND_SF | _lib.SF_COL_MAJOR


def test_packed_ue8m0_scales():
    cfg, storage, sf = _sf((4001, 7168), (1, 128), True, True)
    assert storage.dtype == torch.uint8 and storage.shape == (14, 16004) and storage.stride() == (16016, 1)
    assert sf.dtype == torch.int32 and sf.shape == (4001, 14) and sf.stride() == (1, 4004)
    assert cfg.flags == _lib.ROUND_SF | _lib.SF_COL_MAJOR | _lib.SF_UE8M0
    # 224 groups of 32 -> 56 words per token (cfg4), 9 groups -> 3 words with 3 padding bytes
    _, _, sf = _sf((32768, 7168), (1, 32), True, True)
    assert sf.shape == (32768, 56) and sf.stride() == (1, 32768)
    _, _, sf = _sf((6, 288), (1, 32), True, True)
    assert sf.shape == (6, 3) and sf.stride() == (1, 8)


def test_block_scales_and_empty_input():
    _, _, sf = _sf((7168, 2048), (128, 128), False, False)
    assert sf.shape == (56, 16)
    _, _, sf = _sf((4001, 576), (32, 32), True, True)
    assert sf.shape == (126, 5) and sf.dtype == torch.int32 and sf.stride() == (1, 128)
    _, _, sf = _sf((0, 256), (1, 128), True, True)
    assert sf.shape == (0, 1) and sf.dtype == torch.int32
    _, _, sf = _sf((0, 256), (1, 128), False, False)
    assert sf.shape == (0, 2)


def test_config_rules():
    assert common.get_cast_output_config('e4m3', (1, 128)).clamp_min_value == 1e-4
    assert common.get_cast_output_config('e2m1', (1, 32)).clamp_min_value == 6.0 * 2.0 ** -126
    assert common.get_cast_output_config('e4m3', (1, 128), custom_clamp_min_value=0.5).clamp_min_value == 0.5
    with pytest.raises(AssertionError):
        common.get_cast_output_config('e3m4', (1, 128))
    with pytest.raises(AssertionError):  # packed exponent bytes exist only in the column-major layout
        common.get_cast_output_config('e4m3', (1, 128), use_packed_ue8m0=True)
    with pytest.raises(AssertionError):
        common.get_cast_input_and_config(torch.zeros(2, 2, dtype=torch.float16), None)
    # already quantized inputs: the scale layout is recognised from strides and dtype
    q = torch.zeros(8, 64, dtype=torch.int8)
    _, sf, cfg = common.get_cast_input_and_config((q, torch.zeros(8, 4)), (1, 32))
    assert cfg.with_sf and cfg.flags == 0 and sf.shape == (8, 4)
    _, sf, cfg = common.get_cast_input_and_config((q, torch.zeros(4, 8).T), (1, 32))
    assert cfg.flags == _lib.SF_COL_MAJOR and sf.shape == (4, 8)
    _, sf, cfg = common.get_cast_input_and_config((q, torch.zeros(1, 8, dtype=torch.int32).T), (1, 32))
    assert cfg.flags == _lib.SF_COL_MAJOR | _lib.SF_UE8M0 and sf.dtype == torch.uint8 and sf.shape == (1, 32)
    with pytest.raises(AssertionError):
        common.get_cast_input_and_config((torch.zeros(2, 2, dtype=torch.int32), torch.zeros(2, 1)), (1, 32))
    assert common.get_logical_hidden(64, torch.int8) == 128 and common.get_physical_hidden(128, torch.int8) == 64


def test_unpack_from_e2m1fn_x2():
    x = torch.tensor([[0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]], dtype=torch.uint8)
    want = torch.tensor([[0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]])
    got = common.unpack_from_e2m1fn_x2(x)
    assert torch.equal(got, want) and torch.equal(torch.signbit(got), torch.signbit(want))
    assert common.unpack_from_e2m1fn_x2(x.view(torch.int8), torch.bfloat16).dtype == torch.bfloat16


def test_entry_points_assert_before_any_launch():
    # the reference's wrappers validate with assert; a CPU tensor never reaches the library
    from tilekernels_b200 import quant
    x = torch.zeros((128, 256), dtype=torch.bfloat16)
    for call in (lambda: quant.per_token_cast(x, 'e4m3', 128), lambda: quant.per_block_cast(x, 'e4m3', (128, 128)),
                 lambda: quant.per_channel_cast(x, 'e4m3', 128), lambda: quant.swiglu_forward_and_per_token_cast(x, 'e4m3', 128),
                 lambda: quant.per_token_cast(x, 'e5m6', 256)):
        with pytest.raises(AssertionError):
            call()


def test_neighbour_entry_points_assert_before_any_launch():
    from tilekernels_b200 import moe, quant
    q = torch.zeros((8, 512), dtype=torch.float8_e4m3fn)
    sf = torch.ones((8, 4), dtype=torch.float32)
    grad = torch.zeros((8, 256), dtype=torch.bfloat16)
    weight = torch.ones((4, 2), dtype=torch.float32)
    pos = torch.arange(8, dtype=torch.int32)
    t2p = torch.arange(8, dtype=torch.int32).view(4, 2)
    calls = (
        lambda: quant.swiglu_backward_and_per_token_cast((q, sf), grad, weight, pos, t2p, 128),       # CPU tensors
        lambda: quant.swiglu_backward_and_per_token_cast((q, sf), grad, weight, pos, t2p, 64),        # group size
        lambda: quant.cast_back((q, sf), 'bf16', (1, 128)),
        lambda: quant.per_channel_cast_and_transpose(grad, 'e4m3', 128),
        lambda: moe.expand_to_fused(grad, t2p, pos),
        lambda: moe.expand_to_fused_with_sf((q, sf), 64, t2p, pos),                                   # group size
        lambda: moe.expand_to_fused_with_sf((q, sf.to(torch.int32)), 128, t2p, pos, False),          # packed needs column-major
    )
    for call in calls:
        with pytest.raises(AssertionError):
            call()
