"""Dequantisation: the oracle against the reference's fixtures (CPU) and the CUDA kernels against the oracle and
the fixtures (GPU).  Parametrised after the reference's tests/quant/test_cast_back.py and test_cast_back_e5m6.py."""
import pytest
import torch

from helpers import FLAG_SETS, flags_id, golden, golden_tensor, to_host
from tilekernels_b200.testing import assert_equal, calc_diff

BLOCKS = [(1, 32), (1, 128), (128, 128), (32, 32)]


def _fixture_cases():
    for fmt in ('e4m3', 'e2m1'):
        for bs in BLOCKS:
            for flags in ((False, True, False), (True, True, True)):
                yield pytest.param(fmt, bs, flags, id=f'{fmt}-{bs[0]}x{bs[1]}-{flags_id(flags)}')
    for flags in FLAG_SETS:
        yield pytest.param('e5m6', (1, 128), flags, id=f'e5m6-{flags_id(flags)}')


def _key(fmt, bs, flags):
    return f'e5m6/{flags_id(flags)}' if fmt == 'e5m6' else f'{fmt}/{bs[0]}x{bs[1]}/{flags_id(flags)}'


@pytest.mark.parametrize('fmt,bs,flags', list(_fixture_cases()))
def test_oracle_cast_back_matches_reference(oracle, fmt, bs, flags):
    store = golden('cast_back')
    key = _key(fmt, bs, flags)
    q, qsf, want = (golden_tensor(store, f'{key}/{n}') for n in ('q', 'qsf', 'back'))
    fn = oracle.cast_back_from_e5m6 if fmt == 'e5m6' else oracle.cast_back
    assert_equal(fn((q, qsf), 'fp32', bs), want)
    assert_equal(fn((q, qsf), 'bf16', bs), want.bfloat16())


def _strided_to(device, t):
    span = 1 + sum((n - 1) * s for n, s in zip(t.shape, t.stride()))
    out = torch.zeros(span, dtype=t.dtype, device=device).as_strided(t.shape, t.stride())
    out.copy_(t)
    return out


@pytest.mark.gpu
@pytest.mark.parametrize('fmt,bs,flags', list(_fixture_cases()))
def test_cast_back_fixture(cuda_device, fmt, bs, flags):
    from tilekernels_b200 import quant
    store = golden('cast_back')
    key = _key(fmt, bs, flags)
    q, qsf, want = (golden_tensor(store, f'{key}/{n}') for n in ('q', 'qsf', 'back'))
    pair = (q.to(cuda_device), _strided_to(cuda_device, qsf))
    special = 'e5m6' if fmt == 'e5m6' else None
    assert_equal(to_host(quant.cast_back(pair, 'fp32', bs, x_special_fmt=special)), want)
    assert_equal(to_host(quant.cast_back(pair, 'bf16', bs, x_special_fmt=special)), want.bfloat16())


@pytest.mark.gpu
@pytest.mark.parametrize('out_fmt', ['fp32', 'bf16'])
@pytest.mark.parametrize('flags', [(False, True, False), (True, True, True), (False, False, False)], ids=flags_id)
@pytest.mark.parametrize('fmt', ['e4m3', 'e2m1'])
@pytest.mark.parametrize('num_tokens,hidden,g', [(4001, 576, 64), (4001, 7168, 128), (4001, 2048, 2048), (257, 4096, 32), (8001, 2560, 2560)])
def test_per_token_cast_back(oracle, cuda_device, num_tokens, hidden, g, fmt, flags, out_fmt):
    from tilekernels_b200 import quant
    col, rnd, ue = flags
    gen = torch.Generator().manual_seed(num_tokens + hidden)
    x = torch.randn((num_tokens, hidden), generator=gen).to(torch.bfloat16)
    kw = dict(use_tma_aligned_col_major_sf=col, round_sf=rnd, use_packed_ue8m0=ue)
    q, sf = quant.per_token_cast(x.to(cuda_device), fmt, g, **kw)
    back = quant.per_token_cast_back((q, sf), out_fmt, g)
    q_ref, sf_ref = oracle.cast(x, fmt, (1, g), **kw)
    assert_equal(to_host(back), oracle.cast_back((q_ref, sf_ref), out_fmt, (1, g)))
    # the error bounds of the reference's test (tests/quant/test_cast_back.py:108-109)
    assert calc_diff(to_host(back).float(), x.float()).item() < (2e-2 if fmt == 'e2m1' else 1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize('out_fmt', ['fp32', 'bf16'])
@pytest.mark.parametrize('block', [(128, 128), (32, 32)], ids=lambda b: f'{b[0]}x{b[1]}')
@pytest.mark.parametrize('fmt', ['e4m3', 'e2m1'])
@pytest.mark.parametrize('num_tokens,hidden', [(4001, 576), (1025, 7168), (129, 3072)])
def test_block_cast_back(oracle, cuda_device, num_tokens, hidden, fmt, block, out_fmt):
    from tilekernels_b200 import quant
    gen = torch.Generator().manual_seed(num_tokens * 3 + hidden)
    x = torch.randn((num_tokens, hidden), generator=gen).to(torch.bfloat16)
    for col, rnd, ue in ((False, True, False), (True, True, True)):
        kw = dict(use_tma_aligned_col_major_sf=col, round_sf=rnd, use_packed_ue8m0=ue)
        q, sf = quant.per_block_cast(x.to(cuda_device), fmt, block, **kw)
        q_ref, sf_ref = oracle.cast(x, fmt, block, **kw)
        assert_equal(to_host(quant.cast_back((q, sf), out_fmt, block)), oracle.cast_back((q_ref, sf_ref), out_fmt, block))


@pytest.mark.gpu
@pytest.mark.parametrize('out_fmt', ['fp32', 'bf16'])
@pytest.mark.parametrize('flags', FLAG_SETS, ids=flags_id)
@pytest.mark.parametrize('num_tokens,hidden', [(4001, 576), (4001, 7168), (130, 2560)])
def test_cast_back_e5m6(oracle, cuda_device, num_tokens, hidden, flags, out_fmt):
    from tilekernels_b200 import quant
    col, rnd, ue = flags
    gen = torch.Generator().manual_seed(num_tokens + 7 * hidden)
    x = torch.randn((num_tokens, hidden), generator=gen).to(torch.bfloat16)
    q, sf = quant.per_token_cast(x.to(cuda_device), 'e5m6', hidden, None, col, rnd, ue)
    back = quant.per_token_cast_back((q, sf), out_fmt, hidden, x_special_fmt='e5m6')
    q_ref, sf_ref = oracle.cast_to_e5m6(x, hidden, col, rnd, ue)
    assert_equal(to_host(back), oracle.cast_back_from_e5m6((q_ref, sf_ref), out_fmt, (1, hidden)))
    assert calc_diff(to_host(back).float(), x.float()).item() < 1e-4
