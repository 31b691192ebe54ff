"""per_token_cast on the GPU against the CPU oracle, bit for bit.

Parametrisation follows the reference's tests/quant/test_per_token_cast.py:50-141 (token counts with
ragged tails, its hidden sizes, both tested flag sets, strided input, sf-only and precomputed-sf modes)
and adds the API-default flags (no rounding), which the reference never tests."""
import pytest
import torch

from helpers import flags_id, to_host
from tilekernels_b200.testing import assert_equal, check_bias

pytestmark = pytest.mark.gpu

FLAGS = [(False, True, False), (True, True, True), (False, False, False), (True, False, False)]
_inputs = {}


def make_input(num_tokens, hidden, dtype):
    key = (num_tokens, hidden, dtype)
    if key not in _inputs:
        g = torch.Generator().manual_seed(num_tokens * 131 + hidden)
        x = torch.randn((num_tokens, hidden), generator=g)
        if num_tokens > 4:
            x[1] = 0               # all-zero row -> clamped scale
            x[2] *= 100            # outlier row
            x[3, ::7] = -0.0
        _inputs.clear()            # keep one input alive at a time
        _inputs[key] = x.to(dtype)
    return _inputs[key]


def _params():
    for num_tokens, hiddens in ((4001, (576, 2048, 7168)), (129, (2560, 3072, 4096, 6144)), (1, (64,)), (3, (576,))):
        for hidden in hiddens:
            for dtype in (torch.bfloat16, torch.float32):
                for g in (32, 64, 128, hidden):
                    for fmt in ('e4m3', 'e2m1'):
                        for flags in FLAGS:
                            if num_tokens == 129 and flags == (True, False, False):
                                continue
                            yield pytest.param(num_tokens, hidden, dtype, g, fmt, flags,
                                               id=f'{num_tokens}x{hidden}-{str(dtype)[6:]}-g{g}-{fmt}-{flags_id(flags)}')
    yield pytest.param(257, 1024, torch.bfloat16, 16, 'e4m3', (False, True, False), id='257x1024-bfloat16-g16-e4m3-010')
    yield pytest.param(257, 1024, torch.float32, 16, 'e2m1', (True, True, True), id='257x1024-float32-g16-e2m1-111')


@pytest.mark.parametrize('num_tokens,hidden,dtype,g,fmt,flags', list(_params()))
def test_per_token_cast(oracle, cuda_device, num_tokens, hidden, dtype, g, fmt, flags):
    from tilekernels_b200 import quant
    col, rnd, ue = flags
    x_cpu = make_input(num_tokens, hidden, dtype)
    x = x_cpu.to(cuda_device)
    kw = dict(use_tma_aligned_col_major_sf=col, round_sf=rnd, use_packed_ue8m0=ue)

    out, sf = quant.per_token_cast(x, fmt, g, **kw)
    out_ref, sf_ref = oracle.cast(x_cpu, fmt, (1, g), **kw)
    assert_equal(to_host(out), out_ref)
    assert_equal(to_host(sf), sf_ref)

    if rnd and not col:
        check_bias(oracle.cast_back((out_ref, sf_ref), 'fp32', (1, g)), x_cpu.float())

    # rows strided by twice the hidden size (reference test: test_per_token_cast.py:115-125)
    if fmt == 'e4m3' and not ue:
        wide = torch.randn((num_tokens, hidden * 2), device=cuda_device).to(dtype)
        view = wide[:, :hidden]
        view.copy_(x)
        out2, sf2 = quant.per_token_cast(view, fmt, g, **kw)
        assert_equal(out2, out)
        assert_equal(to_host(sf2), to_host(sf))

    if g != hidden:
        if not col:
            pre = quant.per_token_cast_with_precomputed_sf(x, fmt, g, sf=sf, **kw)
            assert_equal(to_host(pre), oracle.cast(x_cpu, fmt, (1, g), sf=sf_ref))
        only = quant.per_token_cast_with_sf_only(x, fmt, g, **kw)
        assert_equal(to_host(only), sf_ref)


def test_per_token_cast_empty(cuda_device):
    # zero tokens: no launch, correctly shaped outputs (reference: per_token_cast_kernel.py:208, common.py:187-188)
    from tilekernels_b200 import quant
    x = torch.empty((0, 256), dtype=torch.bfloat16, device=cuda_device)
    out, sf = quant.per_token_cast(x, 'e4m3', 128)
    assert out.shape == (0, 256) and out.dtype == torch.float8_e4m3fn and sf.shape == (0, 2) and sf.dtype == torch.float32
    out, sf = quant.per_token_cast(x, 'e2m1', 32, use_tma_aligned_col_major_sf=True, round_sf=True, use_packed_ue8m0=True)
    assert out.shape == (0, 128) and out.dtype == torch.int8 and sf.shape == (0, 2) and sf.dtype == torch.int32
    out, sf = quant.per_token_cast(x, 'e5m6', 256)
    assert out.shape == (0, 384) and out.dtype == torch.uint8


def test_per_token_cast_rejects_bad_arguments(cuda_device):
    # argument errors surface as AssertionError before any launch, as in the reference's wrappers
    from tilekernels_b200 import quant
    x = torch.zeros((4, 256), dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(AssertionError):
        quant.per_token_cast(x, 'e4m3', 48)
    with pytest.raises(AssertionError):
        quant.per_token_cast(x.half(), 'e4m3', 128)
    with pytest.raises(AssertionError):
        quant.per_token_cast(x, 'e3m4', 128)
    with pytest.raises(AssertionError):
        quant.per_token_cast(x, 'e4m3', 128, use_packed_ue8m0=True)  # packed scales exist only column-major
    with pytest.raises(AssertionError):
        quant.per_token_cast(x, 'e5m6', 128)


def test_misaligned_view_uses_narrow_loads(oracle, cuda_device):
    # a view that starts 16 bytes into a row is only 16-byte aligned: the 128-bit load path must give the same bytes
    from tilekernels_b200 import quant
    g = torch.Generator().manual_seed(5)
    base = torch.randn((65, 1024 + 8), generator=g).to(torch.bfloat16)
    x_cpu = base[:, 8:]
    x = base.to(cuda_device)[:, 8:]
    out, sf = quant.per_token_cast(x, 'e4m3', 128, round_sf=True)
    out_ref, sf_ref = oracle.cast(x_cpu, 'e4m3', (1, 128), round_sf=True)
    assert_equal(to_host(out), out_ref)
    assert_equal(to_host(sf), sf_ref)


@pytest.mark.gpu
@pytest.mark.parametrize('xb', [(128, 128), (32, 32)], ids=lambda b: f'b{b[0]}')
def test_requantising_cast_of_tiny_codes(oracle, cuda_device, xb):
    """The f16 route of the production re-quantising cast (e4m3 + ue8m0 in, e4m3 g128 + ue8m0 out, hidden % 1024 == 0)
    at its edges: one large value per input block leaves the other groups of the block with subnormal codes only, so
    that 2^(e_in - e_out) exceeds f16's range and those pieces take the fp32 route; rows of zeros; a block of zeros."""
    from tilekernels_b200 import quant
    kw = dict(use_tma_aligned_col_major_sf=True, round_sf=True, use_packed_ue8m0=True)
    g = torch.Generator().manual_seed(77)
    x = torch.randn((384, 2048), generator=g) * 2.0 ** -8.5
    x[::xb[0], ::xb[1]] = 400.0          # one large value per input block
    x[5] = 0                             # a row of zeros next to it
    x[128:256, 1024:1152] = 0            # a whole 128 x 128 block of zeros
    x[300:, :] *= 2.0 ** 9               # ordinary magnitudes in the last rows
    x_cpu = x.to(torch.bfloat16)
    q_ref, qsf_ref = oracle.cast(x_cpu, 'e4m3', xb, **kw)
    q, qsf = quant.per_block_cast(x_cpu.to(cuda_device), 'e4m3', xb, **kw)
    assert_equal(to_host(q), q_ref)
    out, sf = quant.per_token_cast((q, qsf), 'e4m3', 128, x_block_size=xb, **kw)
    out_ref, sf_ref = oracle.cast((q_ref, qsf_ref), 'e4m3', (1, 128), x_block_size=xb, **kw)
    assert_equal(to_host(sf), sf_ref)
    assert_equal(to_host(out), out_ref)
    assert (to_host(out).view(torch.uint8) & 0x7F).max() > 0x40  # the tiny groups were scaled up, not flushed


def _requant_params():
    for num_tokens, hidden in ((4001, 576), (4001, 7168), (129, 2048), (33, 4096), (65, 1536)):
        for in_fmt in ('e4m3', 'e2m1'):
            for xb in ((128, 128), (32, 32)):
                for g in (32, 128):
                    for fmt in ('e4m3', 'e2m1'):
                        for flags in ((False, True, False), (True, True, True)):
                            yield pytest.param(num_tokens, hidden, in_fmt, xb, g, fmt, flags,
                                               id=f'{num_tokens}x{hidden}-{in_fmt}-b{xb[0]}-g{g}-{fmt}-{flags_id(flags)}')


@pytest.mark.parametrize('num_tokens,hidden,in_fmt,xb,g,fmt,flags', list(_requant_params()))
def test_per_token_cast_of_quantized_input(oracle, cuda_device, num_tokens, hidden, in_fmt, xb, g, fmt, flags):
    """Already quantized input (reference test: tests/quant/test_per_token_cast.py:27-38,62-66: FP8 / FP4 data with
    (128,128) or (32,32) block scales in the same layout as the requested output scales)."""
    from tilekernels_b200 import quant
    col, rnd, ue = flags
    kw = dict(use_tma_aligned_col_major_sf=col, round_sf=rnd, use_packed_ue8m0=ue)
    x_cpu = make_input(num_tokens, hidden, torch.bfloat16)
    q_ref, qsf_ref = oracle.cast(x_cpu, in_fmt, xb, **kw)
    # quantize on the GPU as well, so that the scale tensor has the strides a real producer hands over
    q, qsf = quant.per_block_cast(x_cpu.to(cuda_device), in_fmt, xb, **kw)
    assert_equal(to_host(q), q_ref)
    assert_equal(to_host(qsf), qsf_ref)
    out, sf = quant.per_token_cast((q, qsf), fmt, g, x_block_size=xb, **kw)
    out_ref, sf_ref = oracle.cast((q_ref, qsf_ref), fmt, (1, g), x_block_size=xb, **kw)
    assert_equal(to_host(out), out_ref)
    assert_equal(to_host(sf), sf_ref)
    if rnd and not col and num_tokens > 1000:
        check_bias(oracle.cast_back((out_ref, sf_ref), 'fp32', (1, g)), x_cpu.float())
