"""expand_to_fused / expand_to_fused_with_sf: the oracle against reference fixtures (CPU) and the CUDA kernel against
the oracle (GPU), following the reference's tests/moe/test_expand_to_fused.py:35-124."""
import pytest
import torch

from helpers import golden, golden_tensor, to_host
from tilekernels_b200.testing import assert_equal

SF_MODES = ((False, True, False), (True, True, False), (True, True, True))  # (col_major, round_sf, ue8m0)


def _id(mode) -> str:
    return ''.join(str(int(f)) for f in mode)


def test_oracle_plain_matches_reference(oracle):
    store = golden('expand')
    out = oracle.expand_to_fused(golden_tensor(store, 'x'), golden_tensor(store, 'token_topk_to_pos'), golden_tensor(store, 'pos_to_expert'))
    assert_equal(out, golden_tensor(store, 'plain'))


@pytest.mark.parametrize('G', (32, 128))
@pytest.mark.parametrize('mode', SF_MODES, ids=_id)
def test_oracle_with_sf_matches_reference(oracle, G, mode):
    store = golden('expand')
    key = f'g{G}/{_id(mode)}'
    x = (golden_tensor(store, key + '/q'), golden_tensor(store, key + '/qsf'))
    out, out_sf = oracle.expand_to_fused_with_sf(x, G, golden_tensor(store, 'token_topk_to_pos'), golden_tensor(store, 'pos_to_expert'), mode[0])
    assert_equal(out, golden_tensor(store, key + '/out'))
    assert_equal(out_sf, golden_tensor(store, key + '/out_sf'))


def _routing(num_tokens: int, num_topk: int, num_pad: int, gen: torch.Generator):
    """Maps as tile_kernels.moe.get_fused_mapping produces them: routed (token, k) pairs at distinct positions, the
    remaining num_pad positions are padding (expert -1)."""
    entries = num_tokens * num_topk
    routed = torch.rand(entries, generator=gen) > 0.2
    num_routed = int(routed.sum().item())
    num_expanded = num_routed + num_pad
    positions = torch.randperm(num_expanded, generator=gen)[:num_routed].to(torch.int32)
    token_topk_to_pos = torch.full((entries,), -1, dtype=torch.int32)
    token_topk_to_pos[routed] = positions
    pos_to_expert = torch.full((num_expanded,), -1, dtype=torch.int32)
    pos_to_expert[positions.long()] = torch.randint(0, 8, (num_routed,), generator=gen, dtype=torch.int32)
    return token_topk_to_pos.view(num_tokens, num_topk), pos_to_expert


SHAPES = ((1, 1, 3), (33, 2, 7), (257, 6, 40), (1000, 8, 129), (64, 40, 5))
HIDDENS = (256, 576, 2048, 7168)


@pytest.mark.gpu
@pytest.mark.parametrize('num_tokens,num_topk,num_pad', SHAPES)
@pytest.mark.parametrize('hidden', HIDDENS)
@pytest.mark.parametrize('dtype', (torch.bfloat16, torch.float32, torch.float8_e4m3fn), ids=('bf16', 'fp32', 'fp8'))
def test_expand_to_fused(oracle, cuda_device, num_tokens, num_topk, num_pad, hidden, dtype):
    from tilekernels_b200 import moe
    gen = torch.Generator().manual_seed(num_tokens + hidden)
    t2p, p2e = _routing(num_tokens, num_topk, num_pad, gen)
    x = torch.randn((num_tokens, hidden), generator=gen).to(dtype)
    out = moe.expand_to_fused(x.to(cuda_device), t2p.to(cuda_device), p2e.to(cuda_device))
    assert_equal(to_host(out), oracle.expand_to_fused(x, t2p, p2e))


@pytest.mark.gpu
@pytest.mark.parametrize('num_tokens,num_topk,num_pad', SHAPES)
@pytest.mark.parametrize('hidden', HIDDENS)
@pytest.mark.parametrize('G', (32, 128))
@pytest.mark.parametrize('mode', SF_MODES, ids=_id)
def test_expand_to_fused_with_sf(oracle, cuda_device, num_tokens, num_topk, num_pad, hidden, G, mode):
    from tilekernels_b200 import moe
    col, rnd, ue = mode
    gen = torch.Generator().manual_seed(num_tokens * 3 + hidden + G)
    t2p, p2e = _routing(num_tokens, num_topk, num_pad, gen)
    x = torch.randn((num_tokens, hidden), generator=gen).to(torch.bfloat16)
    q, qsf = oracle.cast(x, 'e4m3', (1, G), round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
    qsf = qsf.contiguous()
    out, out_sf = moe.expand_to_fused_with_sf((q.to(cuda_device), qsf.to(cuda_device)), G, t2p.to(cuda_device), p2e.to(cuda_device), col)
    out_ref, out_sf_ref = oracle.expand_to_fused_with_sf((q, qsf), G, t2p, p2e, col)
    assert_equal(to_host(out), out_ref)
    # rows that are neither routed nor padding do not exist in consistent maps, so every scale is defined; the
    # padding columns of the column-major buffer (beyond the last position) are outside the returned view
    assert_equal(to_host(out_sf), out_sf_ref)


@pytest.mark.gpu
def test_expand_golden_and_empty(oracle, cuda_device):
    from tilekernels_b200 import moe
    store = golden('expand')
    t2p, p2e = golden_tensor(store, 'token_topk_to_pos').to(cuda_device), golden_tensor(store, 'pos_to_expert').to(cuda_device)
    assert_equal(to_host(moe.expand_to_fused(golden_tensor(store, 'x').to(cuda_device), t2p, p2e)), golden_tensor(store, 'plain'))
    for G in (32, 128):
        for mode in SF_MODES:
            key = f'g{G}/{_id(mode)}'
            x = (golden_tensor(store, key + '/q').to(cuda_device), golden_tensor(store, key + '/qsf').to(cuda_device))
            out, out_sf = moe.expand_to_fused_with_sf(x, G, t2p, p2e, mode[0])
            assert_equal(to_host(out), golden_tensor(store, key + '/out'))
            assert_equal(to_host(out_sf), golden_tensor(store, key + '/out_sf'))
    # no tokens: nothing is launched, shapes are still right
    out = moe.expand_to_fused(torch.empty((0, 256), dtype=torch.bfloat16, device=cuda_device),
                              torch.empty((0, 2), dtype=torch.int32, device=cuda_device), p2e)
    assert out.shape == (p2e.numel(), 256)
