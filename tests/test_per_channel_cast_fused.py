"""per_channel_cast_fused on the GPU against the oracle: plain / FP8+scales input, with and without the
pos_to_token gather (parametrised after the reference's tests/quant/test_per_channel_cast_fused.py)."""
import pytest
import torch

from helpers import golden, golden_tensor, to_host
from tilekernels_b200.testing import assert_equal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('round_sf', [False, True])
@pytest.mark.parametrize('gather', [None, 'dense', 'padded'])
@pytest.mark.parametrize('src', ['bf16', 'fp32', 'fp8'])
@pytest.mark.parametrize('num_tokens,hidden', [(4096, 2048), (1024, 7168), (384, 576 * 0 + 640), (128, 128)])
def test_per_channel_cast_fused(oracle, cuda_device, num_tokens, hidden, src, gather, round_sf):
    from tilekernels_b200 import quant
    g = torch.Generator().manual_seed(num_tokens + hidden)
    x_cpu = torch.randn((num_tokens, hidden), generator=g)
    x_cpu[5] *= 40
    if src == 'fp8':
        q, s = oracle.cast(x_cpu.bfloat16(), 'e4m3', (1, 128))  # non-power-of-two input scales on purpose
        x_in_cpu, x_in = (q, s), (q.to(cuda_device), s.to(cuda_device))
        npc = 128
    else:
        xt = x_cpu.to(torch.bfloat16 if src == 'bf16' else torch.float32)
        x_in_cpu, x_in, npc = xt, xt.to(cuda_device), None
    pos = None
    if gather is not None:
        n_out = (num_tokens * 3 // 2) // 16 * 16 + 16  # a multiple of 16 that is usually not a multiple of 128
        pos = torch.randint(0, num_tokens, (n_out,), generator=g, dtype=torch.int32)
        if gather == 'padded':
            pos[torch.rand(n_out, generator=g) < 0.2] = -1
            pos[-16:] = -1
    out, sf = quant.per_channel_cast_fused(x_in, 'e4m3', 128, round_sf, npc, None if pos is None else pos.to(cuda_device))
    out_ref, sf_ref = oracle.per_channel_cast_fused(x_in_cpu, 128, npc, round_sf, pos)
    assert_equal(to_host(out), out_ref)
    assert_equal(to_host(sf), sf_ref)


@pytest.mark.parametrize('gather', [False, True])
@pytest.mark.parametrize('src', ['bf16', 'fp8'])
@pytest.mark.parametrize('rnd', [False, True])
def test_per_channel_cast_fused_fixture(cuda_device, rnd, src, gather):
    from tilekernels_b200 import quant
    store = golden('requant')
    if src == 'bf16':
        x, npc = golden_tensor(store, 'pc/x').to(cuda_device), None
    else:
        x, npc = (golden_tensor(store, 'pc/q8').to(cuda_device), golden_tensor(store, 'pc/s8').to(cuda_device)), 128
    pos = golden_tensor(store, 'pc/pos').to(cuda_device) if gather else None
    out, sf = quant.per_channel_cast_fused(x, 'e4m3', 128, rnd, npc, pos)
    assert_equal(to_host(out), golden_tensor(store, f'pc/{src}/r{int(rnd)}/g{int(gather)}/out'))
    assert_equal(to_host(sf), golden_tensor(store, f'pc/{src}/r{int(rnd)}/g{int(gather)}/sf'))


@pytest.mark.parametrize('round_sf', [False, True])
@pytest.mark.parametrize('num_per_tokens', [32, 128])
@pytest.mark.parametrize('num_tokens,hidden', [(4096, 576), (4096, 2048), (8064, 7168), (128, 64), (1024, 2560)])
def test_per_channel_cast_and_transpose(oracle, cuda_device, num_tokens, hidden, num_per_tokens, round_sf):
    """As the reference's tests/quant/test_per_channel_cast_and_transpose.py:41-52: the (n x 1)-block cast, data transposed."""
    from tilekernels_b200 import quant
    g = torch.Generator().manual_seed(num_tokens + hidden + num_per_tokens)
    x = torch.randn((num_tokens, hidden), generator=g).to(torch.bfloat16)
    x[3] *= 30
    x[:, 5] = 0
    out, sf = quant.per_channel_cast_and_transpose(x.to(cuda_device), 'e4m3', num_per_tokens, round_sf)
    out_ref, sf_ref = oracle.cast(x, 'e4m3', (num_per_tokens, 1), round_sf=round_sf)
    assert_equal(to_host(out), out_ref.view(torch.uint8).T.contiguous().view(torch.float8_e4m3fn))
    assert_equal(to_host(sf), sf_ref)
